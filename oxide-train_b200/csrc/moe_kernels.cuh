// Mixture-of-experts routing beside the grouped expert GEMM: top-k selection,
// deterministic slot assignment, expert offsets, the token permutation
// (dispatch) and the gate-weighted combine.  Integer outputs follow the
// reference's CPU router bit for bit (crates/nn/src/moe.rs:205-254); these are
// latency/HBM-bound kernels, not tensor-core work.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace b200 {

constexpr uint32_t kMoeDropped = 0xFFFFFFFFu;   // u32::MAX marks a dropped assignment
constexpr int kMoeMaxExperts = 256;
constexpr int kMoeMaxTopK = 16;

// f32::total_cmp as an integer key (crates/nn/src/moe.rs:217-219 sorts with it).
__device__ __forceinline__ int total_order_key(float f) {
  int b = __float_as_int(f);
  return b ^ static_cast<int>(static_cast<unsigned>(b >> 31) >> 1);
}

// One warp per token.  Picks the top_k experts by descending score, ties to the
// lower expert index (moe.rs:215-220), and the renormalised gate weights.
//   scores_are_logits == 0: scores are probabilities; gate = p / sum_topk(p) with
//       the denominator summed in f64 in rank order and rounded to f32 (moe.rs:222-225)
//   scores_are_logits != 0: gate = softmax over the selected logits (the same
//       quantity, computed without forming the full softmax)
__global__ void __launch_bounds__(256) moe_topk_kernel(const float* __restrict__ scores,
                                                       int scores_are_logits, long long tokens,
                                                       int experts, int top_k,
                                                       uint32_t* __restrict__ selected,
                                                       float* __restrict__ gates) {
  const int lane = threadIdx.x & 31;
  const long long token = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (token >= tokens) return;
  const float* row = scores + token * experts;
  constexpr int kPerLane = kMoeMaxExperts / 32;
  float val[kPerLane];
  int key[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    val[i] = e < experts ? row[e] : 0.f;
    key[i] = e < experts ? total_order_key(val[i]) : INT_MIN;
  }
  unsigned taken = 0;   // bit i: this lane's i-th expert was already selected
  float sel_val[kMoeMaxTopK];
  int sel_idx[kMoeMaxTopK];
  for (int rank = 0; rank < top_k; ++rank) {
    // best of this lane: highest key, then lowest index
    long long best = LLONG_MIN;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && !((taken >> i) & 1u)) {
        const long long cand = (static_cast<long long>(key[i]) << 32) |
                               static_cast<long long>(0xFFFFFFFFu - static_cast<unsigned>(e));
        best = cand > best ? cand : best;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const long long other = __shfl_xor_sync(0xffffffffu, best, off);
      best = other > best ? other : best;
    }
    const int e = static_cast<int>(0xFFFFFFFFu - static_cast<unsigned>(best & 0xFFFFFFFFll));
    if ((e & 31) == lane) taken |= 1u << (e >> 5);
    // the owner lane broadcasts the value
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (i == (e >> 5)) v = val[i];
    v = __shfl_sync(0xffffffffu, v, e & 31);
    sel_val[rank] = v;
    sel_idx[rank] = e;
  }
  if (lane == 0) {
    const long long base = token * top_k;
    if (!scores_are_logits) {
      double denom = 0.0;
      for (int r = 0; r < top_k; ++r) denom += static_cast<double>(sel_val[r]);
      const float d = static_cast<float>(denom);
      for (int r = 0; r < top_k; ++r) {
        selected[base + r] = static_cast<uint32_t>(sel_idx[r]);
        gates[base + r] = sel_val[r] / d;
      }
    } else {
      const float mx = sel_val[0];   // rank 0 is the largest
      float ex[kMoeMaxTopK];
      float sum = 0.f;
      for (int r = 0; r < top_k; ++r) {
        ex[r] = expf(sel_val[r] - mx);
        sum += ex[r];
      }
      for (int r = 0; r < top_k; ++r) {
        selected[base + r] = static_cast<uint32_t>(sel_idx[r]);
        gates[base + r] = ex[r] / sum;
      }
    }
  }
}

// Slot assignment (moe.rs:228-236): slot = number of earlier (token, rank) pairs,
// in flattened order, routed to the same expert; pairs beyond `capacity` are
// dropped.  Three passes over segments of kMoeSegment consecutive pairs, one warp
// per segment; no atomic ever decides an order, so the result is deterministic.
constexpr int kMoeSegment = 256;   // pairs per warp

// Pass 1: per-segment histogram over experts -> seg_counts[segment][experts].
__global__ void __launch_bounds__(256) moe_hist_kernel(const uint32_t* __restrict__ selected,
                                                       long long pairs, int experts,
                                                       uint32_t* __restrict__ seg_counts) {
  __shared__ unsigned hist[8][kMoeMaxExperts];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long seg = static_cast<long long>(blockIdx.x) * 8 + warp;
  for (int e = lane; e < experts; e += 32) hist[warp][e] = 0;
  __syncwarp();
  const long long base = seg * kMoeSegment;
  for (int i = lane; i < kMoeSegment; i += 32)
    if (base + i < pairs) atomicAdd(&hist[warp][selected[base + i]], 1u);
  __syncwarp();
  if (base < pairs)
    for (int e = lane; e < experts; e += 32) seg_counts[seg * experts + e] = hist[warp][e];
}

// Pass 2: one block per expert turns its column of seg_counts into exclusive
// prefix sums (in place) and writes the expert's totals.
__global__ void __launch_bounds__(256) moe_scan_kernel(uint32_t* __restrict__ seg_counts,
                                                       long long segments, int experts,
                                                       long long capacity,
                                                       uint32_t* __restrict__ assignment_counts,
                                                       uint32_t* __restrict__ accepted_counts) {
  __shared__ unsigned warp_totals[8];
  const int expert = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long running = 0;
  for (long long base = 0; base < segments; base += 256) {
    const long long i = base + threadIdx.x;
    const unsigned mine = i < segments ? seg_counts[i * experts + expert] : 0u;
    unsigned incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) warp_totals[warp] = incl;
    __syncthreads();
    unsigned warp_base = 0, tile_total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) warp_base += warp_totals[w];
      tile_total += warp_totals[w];
    }
    if (i < segments) seg_counts[i * experts + expert] = static_cast<uint32_t>(running + warp_base + incl - mine);
    running += tile_total;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    assignment_counts[expert] = static_cast<uint32_t>(running);
    accepted_counts[expert] = static_cast<uint32_t>(
        running < static_cast<unsigned long long>(capacity) ? running : capacity);
  }
}

// Pass 3: each warp walks its segment in order, 32 pairs at a time; lanes routed
// to the same expert rank themselves by lane index (match.any), on top of the
// expert's running count for this segment.
__global__ void __launch_bounds__(256) moe_assign_kernel(const uint32_t* __restrict__ selected,
                                                         const uint32_t* __restrict__ seg_base,
                                                         long long pairs, int experts,
                                                         long long capacity,
                                                         uint32_t* __restrict__ slots) {
  __shared__ unsigned counter[8][kMoeMaxExperts];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long seg = static_cast<long long>(blockIdx.x) * 8 + warp;
  const long long base = seg * kMoeSegment;
  if (base >= pairs) return;
  for (int e = lane; e < experts; e += 32) counter[warp][e] = seg_base[seg * experts + e];
  __syncwarp();
  for (int i = 0; i < kMoeSegment; i += 32) {
    const long long q = base + i + lane;
    const bool live = q < pairs;
    const uint32_t e = live ? selected[q] : 0xFFFFFFFFu;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const unsigned rank = __popc(peers & ((1u << lane) - 1u));
    unsigned slot = 0;
    if (live) slot = counter[warp][e] + rank;
    __syncwarp();
    if (live && rank == 0) counter[warp][e] += __popc(peers);
    __syncwarp();
    if (live) slots[q] = slot < static_cast<unsigned long long>(capacity) ? slot : kMoeDropped;
  }
}

// offsets[e] = number of accepted rows of experts before e; offsets[experts] = total.
__global__ void moe_offsets_kernel(const uint32_t* __restrict__ accepted_counts, int experts,
                                   int* __restrict__ offsets) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      run += static_cast<int>(accepted_counts[e]);
    }
    offsets[experts] = run;
  }
}

// dest_row[pair] = offsets[selected] + slot, or kMoeDropped.
__global__ void __launch_bounds__(256) moe_dest_kernel(const uint32_t* __restrict__ selected,
                                                       const uint32_t* __restrict__ slots,
                                                       const int* __restrict__ offsets,
                                                       long long pairs,
                                                       uint32_t* __restrict__ dest_row) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long q = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; q < pairs; q += stride) {
    const uint32_t s = slots[q];
    dest_row[q] = s == kMoeDropped ? kMoeDropped : static_cast<uint32_t>(offsets[selected[q]]) + s;
  }
}

// Dispatch: x_permuted[dest_row[token * top_k + rank], :] = x[token, :].  One warp
// per token: the row is read once, 16 bytes per lane per step, and written to
// each of its top_k destinations (d is a multiple of 8 bf16).
__global__ void __launch_bounds__(256) moe_scatter_kernel(const uint16_t* __restrict__ x,
                                                          const uint32_t* __restrict__ dest_row,
                                                          long long tokens, int top_k, long long d,
                                                          uint16_t* __restrict__ x_permuted) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long vecs = d / 8;
  for (long long token = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; token < tokens; token += warps) {
    const uint4* src = reinterpret_cast<const uint4*>(x + token * d);
    uint32_t dst = lane < top_k ? dest_row[token * top_k + lane] : kMoeDropped;
    for (long long v0 = 0; v0 < vecs; v0 += 128) {          // four 16-byte loads in flight per lane
      uint4 val[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long v = v0 + u * 32 + lane;
        if (v < vecs) val[u] = src[v];
      }
      for (int r = 0; r < top_k; ++r) {
        const uint32_t row = __shfl_sync(0xffffffffu, dst, r);
        if (row == kMoeDropped) continue;
        uint4* out = reinterpret_cast<uint4*>(x_permuted + static_cast<long long>(row) * d);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const long long v = v0 + u * 32 + lane;
          if (v < vecs) out[v] = val[u];
        }
      }
    }
  }
}

// Combine: out[token, :] = residual[token, :] + sum over ranks (in rank order) of
// gate * y_permuted[dest_row, :], accumulated in fp32 (moe.rs:292-306).  One
// warp per token; each lane owns 8 consecutive columns at a time.  The (row,
// gate) pairs of the token are read once and broadcast; the gathered rows of
// four ranks are loaded together before they are added.
template <bool kOutBf16>
__global__ void __launch_bounds__(256) moe_combine_kernel(const uint16_t* __restrict__ y_permuted,
                                                          const uint32_t* __restrict__ dest_row,
                                                          const float* __restrict__ gates,
                                                          const uint16_t* __restrict__ residual,
                                                          long long tokens, int top_k, long long d,
                                                          void* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long vecs = d / 8;
  for (long long token = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; token < tokens; token += warps) {
    const uint32_t my_row = lane < top_k ? dest_row[token * top_k + lane] : kMoeDropped;
    const float my_gate = lane < top_k ? (gates ? gates[token * top_k + lane] : 1.f) : 0.f;
    uint32_t rows[kMoeMaxTopK];
    float gs[kMoeMaxTopK];
#pragma unroll
    for (int r = 0; r < kMoeMaxTopK; ++r) {     // lanes at or beyond top_k hold "dropped"
      rows[r] = __shfl_sync(0xffffffffu, my_row, r);
      gs[r] = __shfl_sync(0xffffffffu, my_gate, r);
    }
    for (long long v = lane; v < vecs; v += 32) {
      float acc[8];
      if (residual) {
        const uint4 r = reinterpret_cast<const uint4*>(residual + token * d)[v];
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] = __uint_as_float(w[j] << 16);
          acc[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      }
#pragma unroll
      for (int r0 = 0; r0 < kMoeMaxTopK; r0 += 4) {
        if (r0 >= top_k) break;
        uint4 y[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (rows[r0 + u] != kMoeDropped)
            y[u] = reinterpret_cast<const uint4*>(y_permuted + static_cast<long long>(rows[r0 + u]) * d)[v];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (rows[r0 + u] == kMoeDropped) continue;
          const float g = gs[r0 + u];
          const uint32_t w[4] = {y[u].x, y[u].y, y[u].z, y[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(g, __uint_as_float(w[j] << 16)));
            acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(g, __uint_as_float(w[j] & 0xffff0000u)));
          }
        }
      }
      if (kOutBf16) {
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(ow[j]) : "f"(acc[2 * j + 1]), "f"(acc[2 * j]));
        reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + token * d)[v] = o;
      } else {
        float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + token * d) + 2 * v;
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
  }
}

// ------------------------------------------------------------------ backward of the expert path
// (crates/nn/src/moe.rs:354-445 MoeFfn::backward; crates/nn/src/swiglu.rs:30-47)

__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(w[j] << 16);
    f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 o;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(ow[j]) : "f"(f[2 * j + 1]), "f"(f[2 * j]));
  return o;
}

// Backward of the combine (moe.rs:360-381): for every accepted (token, rank) pair
//   dy_permuted[dest_row, :] = gate * dy[token, :]                      (bf16)
//   gate_grad[pair]          = sum_d y_permuted[dest_row, d] * dy[token, d]   (0 for a dropped pair)
// One warp per token; dy is read once.  `y_permuted` / `gate_grad` may be null together.
template <bool kDyBf16>
__global__ void __launch_bounds__(256) moe_combine_backward_kernel(
    const void* __restrict__ dy, const uint16_t* __restrict__ y_permuted, const uint32_t* __restrict__ dest_row,
    const float* __restrict__ gates, long long tokens, int top_k, long long d,
    uint16_t* __restrict__ dy_permuted, float* __restrict__ gate_grad) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long vecs = d / 8;
  for (long long token = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; token < tokens; token += warps) {
    const uint32_t my_row = lane < top_k ? dest_row[token * top_k + lane] : kMoeDropped;
    const float my_gate = lane < top_k ? gates[token * top_k + lane] : 0.f;
    // Every lane gets every rank's (row, gate) BEFORE the column loop: lanes leave that loop at
    // different trip counts when d / 8 is not a multiple of 32, and a warp shuffle is only
    // defined while all the lanes its mask names are executing it.
    uint32_t rows[kMoeMaxTopK];
    float gs[kMoeMaxTopK];
    float dots[kMoeMaxTopK];
#pragma unroll
    for (int r = 0; r < kMoeMaxTopK; ++r) {
      rows[r] = __shfl_sync(0xffffffffu, my_row, r);
      gs[r] = __shfl_sync(0xffffffffu, my_gate, r);
      dots[r] = 0.f;
    }
    for (long long v = lane; v < vecs; v += 32) {
      float g[8];
      if (kDyBf16) {
        unpack_bf16x8(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(dy) + token * d)[v], g);
      } else {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(dy) + token * d) + 2 * v;
        const float4 lo = src[0], hi = src[1];
        g[0] = lo.x; g[1] = lo.y; g[2] = lo.z; g[3] = lo.w;
        g[4] = hi.x; g[5] = hi.y; g[6] = hi.z; g[7] = hi.w;
      }
#pragma unroll
      for (int r = 0; r < kMoeMaxTopK; ++r) {
        if (r >= top_k) break;
        const uint32_t row = rows[r];
        const float gate = gs[r];
        if (row == kMoeDropped) continue;
        float scaled[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) scaled[j] = __fmul_rn(gate, g[j]);
        reinterpret_cast<uint4*>(dy_permuted + static_cast<long long>(row) * d)[v] = pack_bf16x8(scaled);
        if (gate_grad) {
          float y[8];
          unpack_bf16x8(reinterpret_cast<const uint4*>(y_permuted + static_cast<long long>(row) * d)[v], y);
#pragma unroll
          for (int j = 0; j < 8; ++j) dots[r] = fmaf(y[j], g[j], dots[r]);
        }
      }
    }
    if (gate_grad) {
#pragma unroll
      for (int r = 0; r < kMoeMaxTopK; ++r) {
        if (r >= top_k) break;
        float sum = dots[r];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (lane == 0) gate_grad[token * top_k + r] = sum;
      }
    }
  }
}

// Backward of the expert's activation, elementwise over the routed rows.
//   kGlu == false (SiLU, y = silu(a)):        d_a = d_y * s * (1 + a * (1 - s)),  s = sigmoid(a)
//   kGlu == true  (SwiGLU, y = silu(g) * u):  d_g = d_y * u * s * (1 + g * (1 - s)),  d_u = d_y * g * s
//     with `saved` and `d_saved` the [rows, 2, ff] gate/up panel and its gradient
//     (gpu/ops/src/lib.rs:1453 swiglu_backward_interleaved_packed).
// All operands bf16; eight elements per thread per step; ff a multiple of 8.  Row strides in elements.
template <bool kGlu>
__global__ void __launch_bounds__(256) activation_backward_kernel(
    const uint16_t* __restrict__ saved, long long ld_saved, const uint16_t* __restrict__ d_y, long long ld_dy,
    long long rows, long long ff, uint16_t* __restrict__ d_saved, long long ld_dsaved) {
  const long long vecs_per_row = ff / 8;
  const long long total = rows * vecs_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long row = i / vecs_per_row, v = i - row * vecs_per_row;
    float g[8], u[8], dy[8], dg[8], du[8];
    unpack_bf16x8(reinterpret_cast<const uint4*>(saved + row * ld_saved)[v], g);
    if (kGlu) unpack_bf16x8(reinterpret_cast<const uint4*>(saved + row * ld_saved + ff)[v], u);
    unpack_bf16x8(reinterpret_cast<const uint4*>(d_y + row * ld_dy)[v], dy);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + expf(-g[j]));
      const float dsilu = s * (1.f + g[j] * (1.f - s));
      if (kGlu) {
        dg[j] = dy[j] * u[j] * dsilu;
        du[j] = dy[j] * (g[j] * s);
      } else {
        dg[j] = dy[j] * dsilu;
      }
    }
    reinterpret_cast<uint4*>(d_saved + row * ld_dsaved)[v] = pack_bf16x8(dg);
    if (kGlu) reinterpret_cast<uint4*>(d_saved + row * ld_dsaved + ff)[v] = pack_bf16x8(du);
  }
}

// Backward of the routing (moe.rs:397-445): from the gradients of the combine weights to the
// gradient of the router's logits.  One warp per token.
//   weighted = sum_r gate_grad[r] * gate[r]          (f64)
//   psum     = sum_r probs[selected_r]               (f64)
//   dprob[selected_r] += (gate_grad[r] - weighted) / psum
//   dprob[e] += aux_coefficient * experts * fraction[e] / tokens,  fraction[e] = assignment_counts[e] / (tokens * top_k)
//   dlogits[e] = probs[e] * (dprob[e] - sum_e' probs[e'] * dprob[e'])
__global__ void __launch_bounds__(256) moe_route_backward_kernel(
    const float* __restrict__ probs, const uint32_t* __restrict__ selected, const float* __restrict__ gates,
    const float* __restrict__ gate_grad, const uint32_t* __restrict__ assignment_counts, float aux_coefficient,
    long long tokens, int experts, int top_k, float* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31;
  const long long token = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (token >= tokens) return;
  const float* prow = probs + token * experts;
  constexpr int kPerLane = kMoeMaxExperts / 32;
  float p[kPerLane], dp[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < experts ? prow[e] : 0.f;
    const float fraction = e < experts ? static_cast<float>(assignment_counts[e]) / static_cast<float>(tokens * top_k) : 0.f;
    dp[i] = e < experts ? aux_coefficient * static_cast<float>(experts) * fraction / static_cast<float>(tokens) : 0.f;
  }
  // lane r holds pair r
  const uint32_t my_e = lane < top_k ? selected[token * top_k + lane] : 0u;
  const float my_gg = lane < top_k ? gate_grad[token * top_k + lane] : 0.f;
  const float my_gate = lane < top_k ? gates[token * top_k + lane] : 0.f;
  double weighted = 0.0, psum = 0.0;
  for (int r = 0; r < top_k; ++r) {
    const float gg = __shfl_sync(0xffffffffu, my_gg, r);
    const float gt = __shfl_sync(0xffffffffu, my_gate, r);
    const uint32_t e = __shfl_sync(0xffffffffu, my_e, r);
    weighted += static_cast<double>(gg) * static_cast<double>(gt);
    psum += static_cast<double>(prow[e]);
  }
  const float wf = static_cast<float>(weighted), pf = static_cast<float>(psum);
  // The routing term is added first and the auxiliary term on top of it, as the reference does.
  float routed[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) routed[i] = 0.f;
  for (int r = 0; r < top_k; ++r) {
    const float gg = __shfl_sync(0xffffffffu, my_gg, r);
    const uint32_t e = __shfl_sync(0xffffffffu, my_e, r);
    if ((e & 31u) == static_cast<uint32_t>(lane)) {
#pragma unroll
      for (int i = 0; i < kPerLane; ++i)
        if (i == static_cast<int>(e >> 5)) routed[i] += (gg - wf) / pf;
    }
  }
  double dot = 0.0;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    dp[i] = routed[i] + dp[i];
    dot += static_cast<double>(p[i]) * static_cast<double>(dp[i]);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
  const float df = static_cast<float>(dot);
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = lane + 32 * i;
    if (e < experts) dlogits[token * experts + e] = p[i] * (dp[i] - df);
  }
}

// Router logits (gpu/ops/src/lib.rs:2319-2429 router_logits_bf16, which stops at 8 experts):
// logits[tokens, experts] = x[tokens, d] (bf16) . w[d, experts] (fp32), fp32 arithmetic on
// CUDA cores with products rounded and added in ascending k, i.e. the CPU router's
// `Linear::forward` (crates/tensor-cpu/src/ops.rs:87-104) bit for bit, so the expert
// selection downstream cannot differ from the reference's.  64-token x 64-expert tile per
// block, 16-deep slices, 4 x 4 outputs per thread.
__global__ void __launch_bounds__(256) router_logits_kernel(const uint16_t* __restrict__ x,
                                                            const float* __restrict__ w, long long tokens,
                                                            int d, int experts, float* __restrict__ logits) {
  constexpr int kT = 64, kK = 16;
  __shared__ float xs[kK][kT + 4];
  __shared__ float ws[kK][kT + 4];
  const int tid = threadIdx.x;
  const long long row0 = static_cast<long long>(blockIdx.x) * kT;
  const int col0 = blockIdx.y * kT;
  const int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < d; k0 += kK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      {
        const int kk = idx % kK, r = idx / kK;
        const long long gr = row0 + r;
        const int gk = k0 + kk;
        xs[kk][r] = (gr < tokens && gk < d) ? __uint_as_float(static_cast<uint32_t>(x[gr * d + gk]) << 16) : 0.f;
      }
      {
        const int cc = idx % kT, kk = idx / kT;
        const int gc = col0 + cc, gk = k0 + kk;
        ws[kk][cc] = (gc < experts && gk < d) ? w[static_cast<size_t>(gk) * experts + gc] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = xs[kk][tr + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = ws[kk][tc + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long gr = row0 + tr + i;
    if (gr >= tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = col0 + tc + j;
      if (gc < experts) logits[gr * experts + gc] = acc[i][j];
    }
  }
}

// ------------------------------------------------------------------ expert parallelism over peer memory
// Device-driven dispatch for experts spread over the GPUs of one box (contiguous
// blocks: expert e lives on rank e / (experts / world)).  Every rank owns an
// "inbox" that its peers can address (peer-mapped device memory); a routed row is
// written straight into the owner's inbox by the rank that holds the token, and
// read back from the owner's result buffer by the same rank.  Row layout of an
// inbox: blocks by source rank, inside a block sorted by local expert, inside an
// expert by slot -- so the owner multiplies what arrived as (source, expert)
// groups without moving it.  All offsets come from the all-gathered per-expert
// counts on the device; the host never sees a count.
constexpr int kMoeMaxPeers = 8;

struct PeerPointers {
  uint16_t* ptr[kMoeMaxPeers];
};

// One block.  all_counts[src * experts + e] = rows rank `src` routes to expert e.
//   dst_base[e]      row of owner(e)'s inbox where MY rows for expert e begin
//   group_offsets[g] first inbox row of group g = (src, local expert) of MY inbox; g in [0, experts]
//   group_b_index[g] local expert of group g
__global__ void moe_ep_plan_kernel(const int* __restrict__ all_counts, int world, int rank,
                                   int experts, int* __restrict__ dst_base,
                                   int* __restrict__ group_offsets, int* __restrict__ group_b_index) {
  const int local = experts / world;
  if (threadIdx.x == 0) {
    // my rows in each owner's inbox
    for (int owner = 0; owner < world; ++owner) {
      int base = 0;
      for (int s = 0; s < rank; ++s)
        for (int e = 0; e < local; ++e) base += all_counts[s * experts + owner * local + e];
      for (int e = 0; e < local; ++e) {
        dst_base[owner * local + e] = base;
        base += all_counts[rank * experts + owner * local + e];
      }
    }
    // groups of my own inbox
    int run = 0;
    for (int s = 0; s < world; ++s)
      for (int e = 0; e < local; ++e) {
        group_offsets[s * local + e] = run;
        group_b_index[s * local + e] = e;
        run += all_counts[s * experts + rank * local + e];
      }
    group_offsets[experts] = run;
  }
}

// Where the results of MY inbox's groups go when the owner sends them back itself (the
// grouped GEMM with peer stores in its epilogue): group g = (source rank s, local expert e)
// returns to rank s, whose own permutation holds the rows of expert E = rank * local + e from
// row sum over E' < E of all_counts[s][E'] on, in slot order -- the order they sit in my inbox.
__global__ void moe_ep_return_plan_kernel(const int* __restrict__ all_counts, int world, int rank,
                                          int experts, int* __restrict__ group_dst_rank,
                                          int* __restrict__ group_dst_row) {
  const int local = experts / world;
  for (int g = threadIdx.x; g < experts; g += blockDim.x) {
    const int s = g / local, e = g - s * local;
    int base = 0;
    for (int other = 0; other < rank * local + e; ++other) base += all_counts[s * experts + other];
    group_dst_rank[g] = s;
    group_dst_row[g] = base;
  }
}

// Dispatch: one warp per token reads the token's row once and stores it into the
// inbox of each selected expert's owner (a plain peer store over NVLink, or a
// local store when this rank owns the expert).
__global__ void __launch_bounds__(256) moe_ep_push_kernel(const uint16_t* __restrict__ x,
                                                          const uint32_t* __restrict__ selected,
                                                          const uint32_t* __restrict__ slots,
                                                          const int* __restrict__ dst_base,
                                                          PeerPointers inbox, int experts_per_rank,
                                                          long long tokens, int top_k, long long d,
                                                          long long inbox_rows, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long vecs = d / 8;
  for (long long token = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; token < tokens; token += warps) {
    const uint4* src = reinterpret_cast<const uint4*>(x + token * d);
    int my_owner = -1;
    long long my_row = 0;
    if (lane < top_k) {
      const uint32_t e = selected[token * top_k + lane];
      const uint32_t s = slots[token * top_k + lane];
      if (s != kMoeDropped) {
        my_owner = static_cast<int>(e) / experts_per_rank;
        my_row = static_cast<long long>(dst_base[e]) + s;
        if (my_row >= inbox_rows) {          // the owner's inbox is too small: drop the row, report it
          my_owner = -1;
          atomicCAS(status, 0, 105);
        }
      }
    }
    for (long long v0 = 0; v0 < vecs; v0 += 128) {
      uint4 val[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long v = v0 + u * 32 + lane;
        if (v < vecs) val[u] = src[v];
      }
      for (int r = 0; r < top_k; ++r) {
        const int owner = __shfl_sync(0xffffffffu, my_owner, r);
        const long long row = __shfl_sync(0xffffffffu, my_row, r);
        if (owner < 0) continue;
        uint4* out = reinterpret_cast<uint4*>(inbox.ptr[owner] + row * d);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const long long v = v0 + u * 32 + lane;
          if (v < vecs) out[v] = val[u];
        }
      }
    }
  }
}

// Combine: out[token, :] = residual + sum over ranks (in order) of gate * result row,
// each result row read from its expert owner's result buffer (plain peer loads).
template <bool kOutBf16>
__global__ void __launch_bounds__(256) moe_ep_pull_combine_kernel(PeerPointers results,
                                                                  const uint32_t* __restrict__ selected,
                                                                  const uint32_t* __restrict__ slots,
                                                                  const int* __restrict__ dst_base,
                                                                  const float* __restrict__ gates,
                                                                  const uint16_t* __restrict__ residual,
                                                                  int experts_per_rank, long long tokens,
                                                                  int top_k, long long d,
                                                                  long long result_rows, int* status,
                                                                  void* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long vecs = d / 8;
  for (long long token = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; token < tokens; token += warps) {
    const uint16_t* my_ptr = nullptr;
    float my_gate = 0.f;
    if (lane < top_k) {
      const uint32_t e = selected[token * top_k + lane];
      const uint32_t s = slots[token * top_k + lane];
      if (s != kMoeDropped) {
        const long long row = static_cast<long long>(dst_base[e]) + s;
        if (row < result_rows) {
          my_ptr = results.ptr[static_cast<int>(e) / experts_per_rank] + row * d;
          my_gate = gates[token * top_k + lane];
        } else {
          atomicCAS(status, 0, 105);       // outside the owner's buffer: skip the row, report it
        }
      }
    }
    const uint16_t* rows[kMoeMaxTopK];
    float gs[kMoeMaxTopK];
#pragma unroll
    for (int r = 0; r < kMoeMaxTopK; ++r) {
      rows[r] = reinterpret_cast<const uint16_t*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_ptr), r));
      gs[r] = __shfl_sync(0xffffffffu, my_gate, r);
    }
    for (long long v = lane; v < vecs; v += 32) {
      float acc[8];
      if (residual) {
        const uint4 r = reinterpret_cast<const uint4*>(residual + token * d)[v];
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] = __uint_as_float(w[j] << 16);
          acc[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      }
#pragma unroll
      for (int r0 = 0; r0 < kMoeMaxTopK; r0 += 4) {
        if (r0 >= top_k) break;
        uint4 y[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (rows[r0 + u]) y[u] = reinterpret_cast<const uint4*>(rows[r0 + u])[v];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (!rows[r0 + u]) continue;
          const float g = gs[r0 + u];
          const uint32_t w[4] = {y[u].x, y[u].y, y[u].z, y[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(g, __uint_as_float(w[j] << 16)));
            acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(g, __uint_as_float(w[j] & 0xffff0000u)));
          }
        }
      }
      if (kOutBf16) {
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(ow[j]) : "f"(acc[2 * j + 1]), "f"(acc[2 * j]));
        reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + token * d)[v] = o;
      } else {
        float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + token * d) + 2 * v;
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
  }
}

// Combine, the form for a few SMs: the same sums in the same order as
// moe_ep_pull_combine_kernel, but the result rows are fetched by bulk asynchronous copies
// (cp.async.bulk, global or peer memory -> shared memory, completion on an mbarrier)
// instead of by loads.  A load-driven combine needs some thousand warps resident to keep
// the links between the GPUs busy -- warps that share SMs, issue slots and load/store units
// with the expert GEMM running at the same time.  Here one producer warp per block keeps
// `stages` tokens (top_k rows each) in flight, so a dozen blocks on SMs the GEMM left free
// move the same bytes per second.
//   warp `stages`         producer: per token, the row addresses and gates, one bulk copy per row
//   warps 0..stages-1     consumers: warp w owns stage w; gate-weighted sum from shared memory
// Shared memory: [stages][top_k][d] bf16 rows | [stages][16] gates | [stages] row masks |
// full / empty barriers | dst_base table.
struct PullBulkSmem {
  unsigned long long full[8];
  unsigned long long empty[8];
  float gates[8][kMoeMaxTopK];
  uint32_t mask[8];
  int abort_flag;
};

__device__ __forceinline__ void bulk_load_row(uint32_t smem_dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

template <bool kOutBf16>
__global__ void __launch_bounds__(288) moe_ep_pull_bulk_kernel(PeerPointers results,
                                                               const uint32_t* __restrict__ selected,
                                                               const uint32_t* __restrict__ slots,
                                                               const int* __restrict__ dst_base,
                                                               const float* __restrict__ gates,
                                                               const uint16_t* __restrict__ residual,
                                                               int experts, int experts_per_rank, long long tokens,
                                                               int top_k, int top_k_pad, long long d,
                                                               long long result_rows, int stages, int* status,
                                                               void* __restrict__ out) {
  extern __shared__ __align__(128) unsigned char pull_smem[];
  const uint32_t row_bytes = static_cast<uint32_t>(d * 2);
  const uint32_t stage_bytes = row_bytes * top_k;
  PullBulkSmem* ctl = reinterpret_cast<PullBulkSmem*>(pull_smem + static_cast<size_t>(stages) * stage_bytes);
  int* base_tab = reinterpret_cast<int*>(ctl + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  for (int e = threadIdx.x; e < experts; e += blockDim.x) base_tab[e] = dst_base[e];
  __syncthreads();
  volatile int* abort_flag = &ctl->abort_flag;
  // this block's tokens: blockIdx.x, blockIdx.x + gridDim.x, ...; the i-th of them uses stage i % stages
  const long long mine = tokens > blockIdx.x ? (tokens - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (warp == stages) {
    // ---------------------------------------------------------------- producer
    // tokens whose rows one pass of the warp fetches (never two that share a stage)
    const int per_batch = (32 / top_k_pad) < stages ? (32 / top_k_pad) : stages;
    const int sub = lane / top_k_pad, r = lane % top_k_pad;
    // the routing of the batch after the current one is loaded while the current one's copies
    // are issued: the producer never waits for global memory between two tokens
    uint32_t next_e = 0, next_sl = kMoeDropped;
    float next_g = 0.f;
    if (sub < per_batch && sub < mine && r < top_k) {
      const long long q = (blockIdx.x + static_cast<long long>(sub) * gridDim.x) * top_k + r;
      next_e = selected[q];
      next_sl = slots[q];
      next_g = gates[q];
    }
    for (long long i0 = 0; i0 < mine && !*abort_flag; i0 += per_batch) {
      const long long i = i0 + sub;
      const bool live = sub < per_batch && i < mine;
      const uint32_t e = next_e, sl = next_sl;
      const float g_loaded = next_g;
      next_sl = kMoeDropped;
      if (sub < per_batch && i + per_batch < mine && r < top_k) {
        const long long q = (blockIdx.x + (i + per_batch) * gridDim.x) * top_k + r;
        next_e = selected[q];
        next_sl = slots[q];
        next_g = gates[q];
      }
      const uint16_t* src = nullptr;
      float g = 0.f;
      if (live && r < top_k && sl != kMoeDropped) {
        const long long row = static_cast<long long>(base_tab[e]) + sl;
        if (row < result_rows) {
          src = results.ptr[static_cast<int>(e) / experts_per_rank] + row * d;
          g = g_loaded;
        } else {
          atomicCAS(status, 0, 105);           // outside the owner's buffer: skip the row, report it
        }
      }
      const int stage = static_cast<int>(i % stages);
      const uint32_t phase = static_cast<uint32_t>((i / stages) & 1);
      const uint32_t votes = __ballot_sync(0xffffffffu, src != nullptr);
      const uint32_t my_mask = (votes >> (sub * top_k_pad)) & ((1u << top_k_pad) - 1u);   // top_k_pad <= 16
      bool ok = true;
      if (live && r == 0) {
        // the stage is free once its consumer has read the token that used it before
        ok = mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, status, kDevTimeoutProducer, abort_flag);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (live && r < top_k) ctl->gates[stage][r] = g;
      if (live && r == 0) ctl->mask[stage] = my_mask;
      __syncwarp();
      if (live && r == 0) mbar_arrive_expect_tx(smem_u32(&ctl->full[stage]), __popc(my_mask) * row_bytes);
      __syncwarp();
      if (src != nullptr)
        bulk_load_row(smem_u32(pull_smem + static_cast<size_t>(stage) * stage_bytes + static_cast<size_t>(r) * row_bytes),
                      src, row_bytes, smem_u32(&ctl->full[stage]));
    }
  } else {
    // ---------------------------------------------------------------- consumers
    const long long vecs = d / 8;
    for (long long i = warp; i < mine; i += stages) {
      const uint32_t phase = static_cast<uint32_t>((i / stages) & 1);
      if (!mbar_wait(smem_u32(&ctl->full[warp]), phase, status, kDevTimeoutEpilogue, abort_flag)) break;
      const long long token = blockIdx.x + i * gridDim.x;
      const uint32_t mask = ctl->mask[warp];
      const unsigned char* rows = pull_smem + static_cast<size_t>(warp) * stage_bytes;
      for (long long v = lane; v < vecs; v += 32) {
        float acc[8];
        if (residual) {
          const uint4 rr = reinterpret_cast<const uint4*>(residual + token * d)[v];
          const uint32_t w[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] = __uint_as_float(w[j] << 16);
            acc[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        }
        for (int r = 0; r < top_k; ++r) {
          if (!((mask >> r) & 1u)) continue;
          const float g = ctl->gates[warp][r];
          const uint4 y = reinterpret_cast<const uint4*>(rows + static_cast<size_t>(r) * row_bytes)[v];
          const uint32_t w[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(g, __uint_as_float(w[j] << 16)));
            acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(g, __uint_as_float(w[j] & 0xffff0000u)));
          }
        }
        if (kOutBf16) {
          uint4 o;
          uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(ow[j]) : "f"(acc[2 * j + 1]), "f"(acc[2 * j]));
          reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + token * d)[v] = o;
        } else {
          float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + token * d) + 2 * v;
          o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
          o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->empty[warp]));
    }
  }
  __syncthreads();
  // After a wait gave up, copies may still be on their way into this block's shared memory:
  // give each stage's barrier a last bounded chance to complete before the block ends.
  if (*abort_flag && threadIdx.x < stages) {
    const long long issued = mine;   // upper bound of what the producer may have armed
    if (issued > threadIdx.x) {
      const long long last = ((issued - 1 - threadIdx.x) / stages);
      int ignored = 0;
      mbar_wait(smem_u32(&ctl->full[threadIdx.x]), static_cast<uint32_t>(last & 1), status, kDevTimeoutDrain, &ignored,
                100000000ull);
    }
  }
}

// Dispatch, the form for a few SMs: every token's row is fetched once into a shared-memory
// ring (bulk asynchronous copy) and stored from there into the inbox of each selected
// expert's owner by bulk asynchronous copies, shared memory -> global or peer memory.  Two
// warps per block keep tens of rows in flight, where the store-driven kernel above needs
// hundreds of warps to fill the links.
//   warp 0, one lane   loader: one bulk load per token
//   warp 1             storer: lane (token of the batch, r) issues the store of pair r
// Shared memory: [stages][d] bf16 rows | full / empty barriers | dst_base table.
constexpr int kPushMaxStages = 64;
constexpr int kPushPendingBatches = 2;     // batches of stores in flight per lane
struct PushBulkSmem {
  unsigned long long full[kPushMaxStages];
  unsigned long long empty[kPushMaxStages];
  int abort_flag;
};

__device__ __forceinline__ void bulk_store_row(void* dst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_src), "r"(bytes)
               : "memory");
}

__global__ void __launch_bounds__(64) moe_ep_push_bulk_kernel(const uint16_t* __restrict__ x,
                                                              const uint32_t* __restrict__ selected,
                                                              const uint32_t* __restrict__ slots,
                                                              const int* __restrict__ dst_base, PeerPointers inbox,
                                                              int experts, int experts_per_rank, long long tokens,
                                                              int top_k, int top_k_pad, long long d,
                                                              long long inbox_rows, int stages, int* status) {
  extern __shared__ __align__(128) unsigned char push_smem[];
  const uint32_t row_bytes = static_cast<uint32_t>(d * 2);
  PushBulkSmem* ctl = reinterpret_cast<PushBulkSmem*>(push_smem + static_cast<size_t>(stages) * row_bytes);
  int* base_tab = reinterpret_cast<int*>(ctl + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    ctl->abort_flag = 0;
    fence_mbar_init();
  }
  for (int e = threadIdx.x; e < experts; e += blockDim.x) base_tab[e] = dst_base[e];
  __syncthreads();
  volatile int* abort_flag = &ctl->abort_flag;
  const long long mine = tokens > blockIdx.x ? (tokens - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (warp == 0) {
    // ---------------------------------------------------------------- loader
    if (lane == 0) {
      for (long long i = 0; i < mine; ++i) {
        const int stage = static_cast<int>(i % stages);
        const uint32_t phase = static_cast<uint32_t>((i / stages) & 1);
        if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, status, kDevTimeoutProducer, abort_flag)) break;
        const long long token = blockIdx.x + i * gridDim.x;
        mbar_arrive_expect_tx(smem_u32(&ctl->full[stage]), row_bytes);
        bulk_load_row(smem_u32(push_smem + static_cast<size_t>(stage) * row_bytes), x + token * d, row_bytes,
                      smem_u32(&ctl->full[stage]));
      }
    }
  } else {
    // ---------------------------------------------------------------- storer
    const int per_batch = 32 / top_k_pad;
    const int sub = lane / top_k_pad, r = lane % top_k_pad;
    uint32_t next_e = 0, next_sl = kMoeDropped;
    if (sub < mine && r < top_k) {
      const long long q = (blockIdx.x + static_cast<long long>(sub) * gridDim.x) * top_k + r;
      next_e = selected[q];
      next_sl = slots[q];
    }
    bool ok = true;
    for (long long i0 = 0; i0 < mine; i0 += per_batch) {
      const long long i = i0 + sub;
      const bool live = i < mine;
      const uint32_t e = next_e, sl = next_sl;
      next_sl = kMoeDropped;
      if (i + per_batch < mine && r < top_k) {
        const long long q = (blockIdx.x + (i + per_batch) * gridDim.x) * top_k + r;
        next_e = selected[q];
        next_sl = slots[q];
      }
      uint16_t* dst = nullptr;
      if (live && r < top_k && sl != kMoeDropped) {
        const long long row = static_cast<long long>(base_tab[e]) + sl;
        if (row < inbox_rows)
          dst = inbox.ptr[static_cast<int>(e) / experts_per_rank] + row * d;
        else
          atomicCAS(status, 0, 105);           // the owner's inbox is too small: drop the row, report it
      }
      const int stage = static_cast<int>(i % stages);
      const uint32_t phase = static_cast<uint32_t>((i / stages) & 1);
      bool landed = true;
      if (live && r == 0) landed = mbar_wait(smem_u32(&ctl->full[stage]), phase, status, kDevTimeoutEpilogue, abort_flag);
      ok = __all_sync(0xffffffffu, landed);
      if (!ok) break;
      fence_proxy_async_smem();
      if (dst != nullptr) bulk_store_row(dst, smem_u32(push_smem + static_cast<size_t>(stage) * row_bytes), row_bytes);
      tma_commit_group();
      // the stores of the batch issued kPushPendingBatches ago have read their rows: free them
      tma_wait_group_read<kPushPendingBatches>();
      __syncwarp();
      const long long freed = i - static_cast<long long>(kPushPendingBatches) * per_batch;
      if (r == 0 && freed >= 0 && freed < mine) mbar_arrive(smem_u32(&ctl->empty[static_cast<int>(freed % stages)]));
    }
    // every store of this lane has been written before the kernel ends
    tma_wait_group<0>();
  }
  __syncthreads();
  if (*abort_flag && threadIdx.x < stages) {
    // copies may still be on their way into this block's shared memory: a last bounded wait
    if (mine > threadIdx.x) {
      const long long last = (mine - 1 - threadIdx.x) / stages;
      int ignored = 0;
      mbar_wait(smem_u32(&ctl->full[threadIdx.x]), static_cast<uint32_t>(last & 1), status, kDevTimeoutDrain, &ignored,
                100000000ull);
    }
  }
}

// ------------------------------------------------------------------ barrier between the GPUs of one box
// Every rank owns a small array of 64-bit arrival words that its peers can address (peer-mapped
// memory), one word per source rank.  A barrier = "write my epoch into my word of every peer's
// array, then wait until every word of my own array has reached the epoch".  One block, no
// shared memory: it fits on an SM next to a persistent GEMM CTA, which a collective library's
// kernel does not, so it neither waits for the GEMM to end nor needs SMs set aside for it.
// Optionally the ranks exchange a few integers on the way (an all-gather of `count` int32 per
// rank: the expert-parallel exchange's per-expert counts), written before the arrival word.
// A table has two halves used by odd and even epochs in turn, so that a rank that is already
// at the next barrier does not overwrite integers a slower peer is still reading.
// The wait is bounded: after `limit_ns` the kernel records kDevTimeoutPeer and returns.
struct PeerWords {
  unsigned long long* ptr[kMoeMaxPeers];
};
struct PeerTables {
  int* ptr[kMoeMaxPeers];
};

__global__ void __launch_bounds__(256) peer_barrier_kernel(PeerWords words, int world, int rank,
                                                           unsigned long long epoch, const int* __restrict__ payload,
                                                           int count, PeerTables tables, int* status,
                                                           unsigned long long limit_ns) {
  // 1. my integers into row `rank` of every peer's table
  if (payload) {
    for (int i = threadIdx.x; i < world * count; i += blockDim.x) {
      const int peer = i / count, j = i - peer * count;
      tables.ptr[peer][((epoch & 1) * world + rank) * count + j] = payload[j];
    }
  }
  // everything this rank wrote into peer memory before this kernel, and the integers above,
  // are visible system-wide before the arrival words are
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) {
    volatile unsigned long long* theirs = words.ptr[threadIdx.x] + rank;
    *theirs = epoch;
    // 2. wait for peer `threadIdx.x`'s word in my own array
    volatile unsigned long long* mine = words.ptr[rank] + threadIdx.x;
    unsigned long long start = 0;
    for (unsigned spin = 1;; ++spin) {
      if (*mine >= epoch) break;
      __nanosleep(100);
      if ((spin & 0xff) == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (start == 0) {
          start = now;
        } else if (now - start > limit_ns) {
          atomicCAS(status, 0, kDevTimeoutPeer);
          break;
        }
      }
    }
  }
  __threadfence_system();
}

}  // namespace b200
