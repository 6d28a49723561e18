// Small kernels beside the fused lm-head + cross-entropy GEMM: merging the
// per-chunk softmax statistics into a log-sum-exp per row and the mean loss.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace b200 {

// Accumulator block at the head of the cross-entropy workspace.
struct CeAccum {
  double loss_sum;
  unsigned int blocks_done;
  unsigned int pad;
};

// One thread per row: merge `chunks` (max, sum-exp) pairs, write
// lse = max + ln(sum) and row_loss = lse - logit[target]; the mean over rows
// follows the reference's formula (crates/nn/src/cross_entropy.rs:36-58,
// gpu/ops/src/lib.rs:2852-2904) with the row sum carried in f64.
//
// A target outside [0, classes) has no logit: no chunk wrote target_logit[row], which still
// holds whatever an earlier call left there.  Such a row gets a NaN loss (so the mean is NaN
// too) and the status word is raised, instead of a plausible number built on a stale value
// (the reference asserts target < classes, crates/nn/src/cross_entropy.rs:38).
__global__ void __launch_bounds__(256) ce_combine_kernel(const float2* __restrict__ partials,
                                                         const float* __restrict__ target_logit,
                                                         const int* __restrict__ targets, int classes,
                                                         int m, int chunks, float* __restrict__ lse,
                                                         float* __restrict__ row_loss,
                                                         float* __restrict__ loss_mean,
                                                         CeAccum* accum, int* status) {
  __shared__ double warp_sums[8];
  double local = 0.0;
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < m; row += gridDim.x * blockDim.x) {
    float mx = -INFINITY;
    for (int c = 0; c < chunks; ++c) mx = fmaxf(mx, partials[static_cast<size_t>(c) * m + row].x);
    float sum = 0.f;
    for (int c = 0; c < chunks; ++c) {
      const float2 ps = partials[static_cast<size_t>(c) * m + row];
      sum += ps.y * expf(ps.x - mx);
    }
    const float l = mx + logf(sum);
    float loss = l - target_logit[row];
    if (static_cast<unsigned>(targets[row]) >= static_cast<unsigned>(classes)) {
      loss = __int_as_float(0x7fc00000);
      atomicCAS(status, 0, kDevBadTarget);
    }
    if (lse) lse[row] = l;
    if (row_loss) row_loss[row] = loss;
    local += static_cast<double>(loss);
  }
  for (int off = 16; off > 0; off >>= 1) local += __shfl_down_sync(0xffffffffu, local, off);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double block = 0.0;
    for (int w = 0; w < 8; ++w) block += warp_sums[w];
    atomicAdd(&accum->loss_sum, block);
    __threadfence();
    const unsigned int done = atomicAdd(&accum->blocks_done, 1u) + 1u;
    if (done == gridDim.x) {
      // Last block: publish the mean and leave the accumulator zeroed for the next call.
      const double total = atomicAdd(&accum->loss_sum, 0.0);
      if (loss_mean) *loss_mean = static_cast<float>(total / static_cast<double>(m));
      accum->loss_sum = 0.0;
      accum->blocks_done = 0u;
      __threadfence();
    }
  }
}

// Vocabulary-sharded form: merge the chunks of THIS shard only and hand back the
// shard's (max, sum-exp relative to that max, target logit) per row; the caller
// combines shards (max-reduce, rescaled sum-reduce, sum of target logits).
__global__ void __launch_bounds__(256) ce_partial_kernel(const float2* __restrict__ partials,
                                                         const float* __restrict__ target_logit,
                                                         int m, int chunks, float* __restrict__ row_max,
                                                         float* __restrict__ row_sum,
                                                         float* __restrict__ row_target_logit) {
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < m; row += gridDim.x * blockDim.x) {
    float mx = -INFINITY;
    for (int c = 0; c < chunks; ++c) mx = fmaxf(mx, partials[static_cast<size_t>(c) * m + row].x);
    float sum = 0.f;
    for (int c = 0; c < chunks; ++c) {
      const float2 ps = partials[static_cast<size_t>(c) * m + row];
      sum += ps.y * expf(ps.x - mx);
    }
    row_max[row] = mx;
    row_sum[row] = sum;
    row_target_logit[row] = target_logit[row];
  }
}

// Merge of the vocabulary shards' statistics (one thread per row): stats is
// [world][3][m] -- every shard's row_max, row_sum and row_target_logit as
// b200gemm_lmhead_ce_forward_shard wrote them, gathered from all ranks.
//   M = max_s row_max;  S = sum_s row_sum * exp(row_max - M);  lse = M + ln S
//   row_loss = lse - sum_s row_target_logit        (exactly one shard owns the target)
// A shard without real columns has row_max = -inf and row_sum = 0 and drops out.
__global__ void __launch_bounds__(256) ce_merge_shards_kernel(const float* __restrict__ stats, int world,
                                                              long long m, float* __restrict__ lse,
                                                              float* __restrict__ row_loss) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long row = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; row < m; row += stride) {
    float mx = -INFINITY;
    for (int s = 0; s < world; ++s) mx = fmaxf(mx, stats[(3ll * s) * m + row]);
    float sum = 0.f, target = 0.f;
    for (int s = 0; s < world; ++s) {
      const float smax = stats[(3ll * s) * m + row];
      const float ssum = stats[(3ll * s + 1) * m + row];
      if (ssum > 0.f) sum += ssum * expf(smax - mx);
      target += stats[(3ll * s + 2) * m + row];
    }
    const float l = mx + logf(sum);
    lse[row] = l;
    if (row_loss) row_loss[row] = l - target;
  }
}

// The scalar training loss (gpu/ops/src/lib.rs:2852-2904 loss_mean_with_aux): mean of the
// per-token losses plus coefficient * sum of the auxiliary terms (one per MoE layer), the
// terms added in index order.  One block; the token sum is carried in f64
// (crates/nn/src/cross_entropy.rs:36-58 sums rows in f64).
constexpr int kLossTailThreads = 1024;
__global__ void __launch_bounds__(kLossTailThreads) loss_mean_with_aux_kernel(
    const float* __restrict__ losses, long long tokens, const float* __restrict__ aux_terms, int aux_count,
    float coefficient, float* __restrict__ loss) {
  __shared__ double warp_sums[kLossTailThreads / 32];
  double local = 0.0;
  for (long long t = threadIdx.x; t < tokens; t += kLossTailThreads) local += static_cast<double>(losses[t]);
  for (int off = 16; off > 0; off >>= 1) local += __shfl_down_sync(0xffffffffu, local, off);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int w = 0; w < kLossTailThreads / 32; ++w) total += warp_sums[w];
    float auxiliary = 0.f;
    for (int i = 0; i < aux_count; ++i) auxiliary += aux_terms[i];
    *loss = static_cast<float>(total / static_cast<double>(tokens)) + coefficient * auxiliary;
  }
}

}  // namespace b200
