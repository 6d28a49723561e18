// Kernels beside the tcgen05 GEMM: the fp32 CUDA-core GEMM family for fp32
// operands and arbitrary shapes, the bf16 staging converts and the bf16
// transpose.  The converts and the transpose are pure HBM traffic: 16-byte
// accesses, grid-stride loops sized to the SM count.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace b200 {

// ------------------------------------------------------------------ fp32 GEMM
// 64x64 output tile, 16-deep K slices, 256 threads, 4x4 outputs per thread.
// Products are rounded to fp32 and added in ascending k per output element
// (no fused multiply-add), which is the arithmetic of the reference's CPU
// loops (crates/tensor-cpu/src/ops.rs:95-145), so results match them bit for
// bit.

constexpr int kSgTile = 64;
constexpr int kSgK = 16;

// op: 0 = NN (A[m,k], B[k,n]), 1 = NT (A[m,k], B[n,k]), 2 = TN (A[k,m], B[k,n]).
template <int kOp>
__global__ void __launch_bounds__(256) sgemm_kernel(const float* __restrict__ a,
                                                    const float* __restrict__ b,
                                                    float* __restrict__ c, int m, int n, int k,
                                                    int accumulate) {
  __shared__ float as[kSgK][kSgTile + 4];   // [k][row]
  __shared__ float bs[kSgK][kSgTile + 4];   // [k][col]
  const int tid = threadIdx.x;
  const int row0 = blockIdx.y * kSgTile, col0 = blockIdx.x * kSgTile;
  const int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += kSgK) {
    // 64 x 16 elements per operand, 256 threads: 4 each.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      {
        int r, kk;
        if (kOp == 2) { r = idx % kSgTile; kk = idx / kSgTile; }   // A[k,m]: rows contiguous
        else { kk = idx % kSgK; r = idx / kSgK; }                  // A[m,k]: k contiguous
        const int gr = row0 + r, gk = k0 + kk;
        float v = 0.f;
        if (gr < m && gk < k) v = kOp == 2 ? a[static_cast<size_t>(gk) * m + gr] : a[static_cast<size_t>(gr) * k + gk];
        as[kk][r] = v;
      }
      {
        int cc, kk;
        if (kOp == 1) { kk = idx % kSgK; cc = idx / kSgK; }        // B[n,k]: k contiguous
        else { cc = idx % kSgTile; kk = idx / kSgTile; }           // B[k,n]: cols contiguous
        const int gc = col0 + cc, gk = k0 + kk;
        float v = 0.f;
        if (gc < n && gk < k) v = kOp == 1 ? b[static_cast<size_t>(gc) * k + gk] : b[static_cast<size_t>(gk) * n + gc];
        bs[kk][cc] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSgK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[kk][tr + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = bs[kk][tc + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + tr + i;
    if (gr >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = col0 + tc + j;
      if (gc >= n) continue;
      float* dst = c + static_cast<size_t>(gr) * n + gc;
      *dst = accumulate ? __fadd_rn(*dst, acc[i][j]) : acc[i][j];
    }
  }
}

inline cudaError_t launch_sgemm(cudaStream_t stream, int op, bool accumulate, const float* a,
                                const float* b, float* c, int m, int n, int k) {
  dim3 grid((n + kSgTile - 1) / kSgTile, (m + kSgTile - 1) / kSgTile);
  if (grid.y > 65535) return cudaErrorInvalidValue;
  switch (op) {
    case 0: sgemm_kernel<0><<<grid, 256, 0, stream>>>(a, b, c, m, n, k, accumulate); break;
    case 1: sgemm_kernel<1><<<grid, 256, 0, stream>>>(a, b, c, m, n, k, accumulate); break;
    default: sgemm_kernel<2><<<grid, 256, 0, stream>>>(a, b, c, m, n, k, accumulate); break;
  }
  return cudaGetLastError();
}

// ------------------------------------------------------------------ converts

__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// 8 elements per thread per step: two 16-byte loads, one 16-byte store.
__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ src,
                                                          uint16_t* __restrict__ dst,
                                                          long long count) {
  const long long vecs = count / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs; v += stride) {
    const float4 x = reinterpret_cast<const float4*>(src)[2 * v];
    const float4 y = reinterpret_cast<const float4*>(src)[2 * v + 1];
    uint4 o;
    o.x = f32x2_to_bf16x2(x.x, x.y);
    o.y = f32x2_to_bf16x2(x.z, x.w);
    o.z = f32x2_to_bf16x2(y.x, y.y);
    o.w = f32x2_to_bf16x2(y.z, y.w);
    reinterpret_cast<uint4*>(dst)[v] = o;
  }
  if (blockIdx.x == 0) {
    for (long long i = vecs * 8 + threadIdx.x; i < count; i += blockDim.x)
      dst[i] = static_cast<uint16_t>(f32x2_to_bf16x2(src[i], 0.f) & 0xffffu);
  }
}

__global__ void __launch_bounds__(256) bf16_to_f32_kernel(const uint16_t* __restrict__ src,
                                                          float* __restrict__ dst,
                                                          long long count) {
  const long long vecs = count / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs; v += stride) {
    const uint4 x = reinterpret_cast<const uint4*>(src)[v];
    float4 lo, hi;
    lo.x = __uint_as_float(x.x << 16); lo.y = __uint_as_float(x.x & 0xffff0000u);
    lo.z = __uint_as_float(x.y << 16); lo.w = __uint_as_float(x.y & 0xffff0000u);
    hi.x = __uint_as_float(x.z << 16); hi.y = __uint_as_float(x.z & 0xffff0000u);
    hi.z = __uint_as_float(x.w << 16); hi.w = __uint_as_float(x.w & 0xffff0000u);
    reinterpret_cast<float4*>(dst)[2 * v] = lo;
    reinterpret_cast<float4*>(dst)[2 * v + 1] = hi;
  }
  if (blockIdx.x == 0) {
    for (long long i = vecs * 8 + threadIdx.x; i < count; i += blockDim.x)
      dst[i] = __uint_as_float(static_cast<uint32_t>(src[i]) << 16);
  }
}

inline int stream_grid(long long work_items, int sm_count) {
  long long blocks = (work_items + 255) / 256;
  long long cap = static_cast<long long>(sm_count) * 8;   // 8 resident 256-thread CTAs per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

inline cudaError_t launch_f32_to_bf16(cudaStream_t stream, const float* src, uint16_t* dst,
                                      long long count, int sm_count) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  if (!aligned) return cudaErrorMisalignedAddress;
  f32_to_bf16_kernel<<<stream_grid(count / 8 + 1, sm_count), 256, 0, stream>>>(src, dst, count);
  return cudaGetLastError();
}

inline cudaError_t launch_bf16_to_f32(cudaStream_t stream, const uint16_t* src, float* dst,
                                      long long count, int sm_count) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  if (!aligned) return cudaErrorMisalignedAddress;
  bf16_to_f32_kernel<<<stream_grid(count / 8 + 1, sm_count), 256, 0, stream>>>(src, dst, count);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ transpose
// 64x64 bf16 tile through shared memory (padded to dodge bank conflicts);
// reads and writes are both row-contiguous.
__global__ void __launch_bounds__(256) transpose_bf16_kernel(const uint16_t* __restrict__ src,
                                                             uint16_t* __restrict__ dst, int rows,
                                                             int cols) {
  __shared__ uint16_t tile[64][64 + 2];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int r = i / 64, c = i % 64;
    if (r0 + r < rows && c0 + c < cols) tile[r][c] = src[static_cast<size_t>(r0 + r) * cols + c0 + c];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int c = i / 64, r = i % 64;
    if (r0 + r < rows && c0 + c < cols) dst[static_cast<size_t>(c0 + c) * rows + r0 + r] = tile[r][c];
  }
}

inline cudaError_t launch_transpose_bf16(cudaStream_t stream, const uint16_t* src, uint16_t* dst,
                                         int rows, int cols) {
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  if (grid.y > 65535) return cudaErrorInvalidValue;
  transpose_bf16_kernel<<<grid, 256, 0, stream>>>(src, dst, rows, cols);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ wait self-test
// Waits, with the same bounded-wait helper the GEMM kernels use, on a barrier
// that nothing will ever complete; the wait gives up after `limit_ns`, records
// kDevTimeoutDrain in the status word and the kernel returns normally.
__global__ void wait_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, status, kDevTimeoutDrain, &abort_flag, limit_ns);
  __syncthreads();
}

// ------------------------------------------------------------------ sum of parts
// dst[i] = sum over p (ascending) of src[p * part_stride + i], added in fp32; the tail of a
// reduce-scatter whose parts were delivered by copies (one part per rank).  bf16 or fp32 in
// and out; eight elements per thread per step, count a multiple of 8.
template <bool kInBf16, bool kOutBf16>
__global__ void __launch_bounds__(256) sum_parts_kernel(const void* __restrict__ src, long long part_stride,
                                                        int parts, long long count, void* __restrict__ dst) {
  const long long vecs = count / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs; v += stride) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int p = 0; p < parts; ++p) {
      if (kInBf16) {
        const uint4 w = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(src) + p * part_stride)[v];
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] = __fadd_rn(acc[2 * j], __uint_as_float(u[j] << 16));
          acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __uint_as_float(u[j] & 0xffff0000u));
        }
      } else {
        const float4* s4 = reinterpret_cast<const float4*>(static_cast<const float*>(src) + p * part_stride) + 2 * v;
        const float4 lo = s4[0], hi = s4[1];
        acc[0] = __fadd_rn(acc[0], lo.x); acc[1] = __fadd_rn(acc[1], lo.y);
        acc[2] = __fadd_rn(acc[2], lo.z); acc[3] = __fadd_rn(acc[3], lo.w);
        acc[4] = __fadd_rn(acc[4], hi.x); acc[5] = __fadd_rn(acc[5], hi.y);
        acc[6] = __fadd_rn(acc[6], hi.z); acc[7] = __fadd_rn(acc[7], hi.w);
      }
    }
    if (kOutBf16) {
      uint4 o;
      o.x = f32x2_to_bf16x2(acc[0], acc[1]);
      o.y = f32x2_to_bf16x2(acc[2], acc[3]);
      o.z = f32x2_to_bf16x2(acc[4], acc[5]);
      o.w = f32x2_to_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(dst)[v] = o;
    } else {
      float4* o = reinterpret_cast<float4*>(dst) + 2 * v;
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

inline cudaError_t launch_sum_parts(cudaStream_t stream, const void* src, long long part_stride, int parts,
                                    long long count, void* dst, bool in_bf16, bool out_bf16, int blocks) {
  if (in_bf16 && out_bf16) sum_parts_kernel<true, true><<<blocks, 256, 0, stream>>>(src, part_stride, parts, count, dst);
  else if (in_bf16) sum_parts_kernel<true, false><<<blocks, 256, 0, stream>>>(src, part_stride, parts, count, dst);
  else if (out_bf16) sum_parts_kernel<false, true><<<blocks, 256, 0, stream>>>(src, part_stride, parts, count, dst);
  else sum_parts_kernel<false, false><<<blocks, 256, 0, stream>>>(src, part_stride, parts, count, dst);
  return cudaGetLastError();
}

}  // namespace b200
