// Small kernels beside the fused lm-head + cross-entropy GEMM: merging the
// per-chunk softmax statistics into a log-sum-exp per row and the mean loss.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

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
__global__ void __launch_bounds__(256) ce_combine_kernel(const float2* __restrict__ partials,
                                                         const float* __restrict__ target_logit,
                                                         int m, int chunks, float* __restrict__ lse,
                                                         float* __restrict__ row_loss,
                                                         float* __restrict__ loss_mean,
                                                         CeAccum* accum) {
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
    const float loss = l - target_logit[row];
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

}  // namespace b200
