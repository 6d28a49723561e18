// Host side of the C ABI declared in include/b200gemm.h: argument checking,
// tensor-map encoding, launch planning (tile shape, CTA pairing, split-K) and
// the launches themselves.  No cuBLAS, no CPU fallback: on a device that is not
// sm_100 every entry point fails with B200GEMM_ERR_UNSUPPORTED.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <new>

#include "../../include/b200gemm.h"
#include "aux_kernels.cuh"
#include "ce_kernels.cuh"
#include "gemm_kernel.cuh"
#include "moe_kernels.cuh"

#ifndef B200_L2_PROMOTION
#define B200_L2_PROMOTION CU_TENSOR_MAP_L2_PROMOTION_L2_256B
#endif

namespace {

using namespace b200;

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

#define CUDA_TRY(expr)                                                                         \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    if (e_ != cudaSuccess)                                                                     \
      return fail(B200GEMM_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_),  \
                  __FILE__, __LINE__);                                                         \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

struct b200gemm_context {
  int device = 0;
  int sm_count = 0;          // SMs the persistent kernels spread over (b200gemm_set_sm_limit)
  int sm_total = 0;          // SMs of the device
  bool push_bulk_opt_in = false;               // ... and for the bulk-copy dispatch
  bool pull_bulk_opt_in[2] = {false, false};   // large dynamic shared memory enabled for the bulk-copy combine (f32, bf16 out)
  bool exchange_bulk = false;   // the bulk-copy forms of those kernels
  int exchange_ctas = 0;     // thread blocks of the expert exchange's kernels (b200gemm_set_exchange_ctas); 0 = two per SM
  int* status = nullptr;        // device status word
  EncodeTiledFn encode = nullptr;
  // staging for b200gemm_gemm_host
  void* stage[3] = {nullptr, nullptr, nullptr};
  size_t stage_bytes[3] = {0, 0, 0};
  bool smem_opt_in[3][12][4] = {};   // [cta_group - 1, or 2 = wide CTA-pair tiles][epilogue kind][schedule kind]: one per kernel instantiation
  // per-segment expert counts of b200gemm_moe_route: one buffer per stream, so that routing
  // calls issued on different streams can overlap on the GPU without sharing scratch
  struct Scratch {
    void* ptr = nullptr;
    size_t bytes = 0;
  };
  std::map<cudaStream_t, Scratch> moe_scratch;
  // Dynamic tile scheduling (b200gemm_set_scheduler): two int32 counters per stream, zero
  // between launches.  Launches on one stream run one after another and so can share a
  // pair; launches on different streams may overlap and must not.
  int scheduler = 1;         // 0 = static round-robin, 1 = dynamic (the default)
  std::map<cudaStream_t, int*> sched_counters;
  std::mutex sched_mu;       // guards sched_counters only: taken inside launches that may hold `mu`
  std::mutex mu;
};

namespace {

// ---------------------------------------------------------------- tensor maps

// A 3-D tiled, 128-byte-swizzled map over a row-major [batch][rows][inner]
// array.  `row_stride` and `batch_stride` are in elements.
int encode_map(const b200gemm_context* ctx, CUtensorMap* map, CUtensorMapDataType dtype,
               int elem_bytes, const void* base, uint64_t inner, uint64_t rows, uint64_t batch,
               uint64_t row_stride, uint64_t batch_stride, uint32_t box_inner, uint32_t box_rows,
               const char* what) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(B200GEMM_ERR_SHAPE, "%s: base address must be 16-byte aligned", what);
  if ((row_stride * elem_bytes) % 16 != 0 || (batch > 1 && (batch_stride * elem_bytes) % 16 != 0))
    return fail(B200GEMM_ERR_SHAPE, "%s: row/batch strides must be multiples of 16 bytes", what);
  if (box_inner * elem_bytes != 128)
    return fail(B200GEMM_ERR_INVALID, "%s: inner box must span 128 bytes", what);
  cuuint64_t dims[3] = {inner, rows, batch};
  cuuint64_t strides[2] = {row_stride * elem_bytes,
                           (batch > 1 ? batch_stride : rows * row_stride) * elem_bytes};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = ctx->encode(map, dtype, 3, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           B200_L2_PROMOTION, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200GEMM_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what,
                static_cast<int>(r));
  return B200GEMM_OK;
}

// ---------------------------------------------------------------- planning

struct Plan {
  int cta_group = 1;
  int tile_m = 128;
  int tiles_m = 0, tiles_n = 0;
  int k_blocks = 0, split_k = 1, kb_per_split = 0;
  int grid = 0;
  int smem = 0;
  int epi = kEpiF32Tma;
  int reduce = 0;
  int wide = 0;              // 256 x 512 tiles per CTA pair (deep reductions, fp32 output)
  int64_t lda = 0, ldb = 0, ldc = 0, bsa = 0, bsb = 0, bsc = 0;
};

int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

int choose_split_k(int64_t items, int k_blocks, int units) {
  // Efficiency of the last wave when `items * s` work items are dealt to
  // `units` persistent CTAs/clusters.  Splitting costs one extra pass of
  // reduce-add traffic over C per slice, so the smallest split that fills the
  // machine wins, and none is used when the plain launch already does.
  auto eff = [&](int s) {
    double total = static_cast<double>(items) * s;
    double waves = static_cast<double>((static_cast<int64_t>(total) + units - 1) / units);
    return total / (waves * units);
  };
  if (eff(1) >= 0.88) return 1;
  int best = 1;
  double best_eff = eff(1);
  for (int s = 2; s <= 32; ++s) {
    int per = (k_blocks + s - 1) / s;
    if (per < 8) break;                                    // keep slices deep enough to pipeline
    if (static_cast<int64_t>(s - 1) * per >= k_blocks) continue;  // would leave an empty slice
    double e = eff(s);
    if (e > best_eff + 0.02) {
      best_eff = e;
      best = s;
      if (e >= 0.95) break;
    }
  }
  return best;
}

int make_plan(const b200gemm_context* ctx, const b200gemm_desc_t* d, Plan* p) {
  if (!d) return fail(B200GEMM_ERR_INVALID, "null descriptor");
  if (!d->a || !d->b || !d->c) return fail(B200GEMM_ERR_INVALID, "null matrix pointer");
  if (d->m <= 0 || d->n <= 0 || d->k <= 0 || d->batch < 1)
    return fail(B200GEMM_ERR_SHAPE, "m, n, k must be positive and batch >= 1");
  if (d->m > (1ll << 30) || d->n > (1ll << 30) || d->k > (1ll << 30))
    return fail(B200GEMM_ERR_SHAPE, "extent too large");
  if (d->a_layout < 0 || d->a_layout > 1 || d->b_layout < 0 || d->b_layout > 1)
    return fail(B200GEMM_ERR_INVALID, "bad operand layout");
  if (d->out_type < 0 || d->out_type > 1 || d->mode < 0 || d->mode > 1)
    return fail(B200GEMM_ERR_INVALID, "bad output type or mode");
  if (d->split_k < 0) return fail(B200GEMM_ERR_INVALID, "negative split_k");
  const bool a_mn = d->a_layout == B200GEMM_MN_MAJOR, b_mn = d->b_layout == B200GEMM_MN_MAJOR;
  p->lda = d->lda ? d->lda : (a_mn ? d->m : d->k);
  p->ldb = d->ldb ? d->ldb : (b_mn ? d->n : d->k);
  p->ldc = d->ldc ? d->ldc : d->n;
  if (p->lda < (a_mn ? d->m : d->k) || p->ldb < (b_mn ? d->n : d->k) || p->ldc < d->n)
    return fail(B200GEMM_ERR_SHAPE, "leading dimension smaller than the row it strides");
  p->bsa = d->batch_stride_a ? d->batch_stride_a : p->lda * (a_mn ? d->k : d->m);
  p->bsb = d->batch_stride_b ? d->batch_stride_b : p->ldb * (b_mn ? d->k : d->n);
  p->bsc = d->batch_stride_c ? d->batch_stride_c : p->ldc * d->m;

  const bool want2 = (d->flags & B200GEMM_FLAG_CTA_GROUP_2) != 0;
  const bool want1 = (d->flags & B200GEMM_FLAG_CTA_GROUP_1) != 0;
  if (want1 && want2) return fail(B200GEMM_ERR_INVALID, "both CTA-group flags set");
  p->cta_group = want2 ? 2 : (want1 ? 1 : (d->m > 128 ? 2 : 1));
  p->tile_m = kTileMCta * p->cta_group;
  p->tiles_m = ceil_div(d->m, p->tile_m);
  p->k_blocks = ceil_div(d->k, kBlockK);
  const bool f32 = d->out_type == B200GEMM_OUT_F32;
  const int units = std::max(1, ctx->sm_count / p->cta_group);
  // Wide tiles: one 512-column accumulator per CTA pair, a third less operand traffic per FLOP,
  // no overlap of a tile's drain with the next tile's MMAs -- so only where a tile's reduction is
  // so deep that the drain does not matter (weight gradients over the tokens, K >= 8192 per item)
  // and the columns fill whole wide tiles well.
  const bool want_wide = (d->flags & B200GEMM_FLAG_WIDE_TILE) != 0;
  const bool no_wide = (d->flags & B200GEMM_FLAG_NARROW_TILE) != 0;
  if (want_wide && (p->cta_group != 2 || !f32)) return fail(B200GEMM_ERR_UNSUPPORTED, "wide tiles need CTA pairs and fp32 output");
  p->wide = 0;
  if (p->cta_group == 2 && f32 && !no_wide) {
    // What the wide plan would look like: its tiles, the K split that fills the machine with
    // them, and how deep one item's reduction then is.  Measured on the step's weight gradients:
    // 171 K blocks per item win 10 % (4096 x 1536), 128 lose 1 % (1536 x 4608, where 54 wide
    // tiles need a 4-way split).
    const int64_t wide_tiles = static_cast<int64_t>(d->batch) * p->tiles_m * ceil_div(d->n, 2 * kTileN);
    const int wide_split = d->split_k ? d->split_k : choose_split_k(wide_tiles, p->k_blocks, units);
    const bool deep = p->k_blocks / std::max(1, wide_split) >= 160;
    const bool fills = d->n % (2 * kTileN) == 0 || d->n >= 8 * kTileN;
    // A store that has to be split pays a clearing pass and a read-modify-write of C per slice:
    // wide tiles halve the tile count, hence split sooner, so a store only goes wide unsplit.
    const bool cheap_split = d->mode == B200GEMM_ACCUMULATE || wide_split == 1;
    p->wide = want_wide || (deep && fills && cheap_split) ? 1 : 0;
  }
  const int tile_n = p->wide ? 2 * kTileN : kTileN;
  p->tiles_n = ceil_div(d->n, tile_n);
  const int64_t items = static_cast<int64_t>(d->batch) * p->tiles_m * p->tiles_n;
  if (items > (1ll << 30)) return fail(B200GEMM_ERR_SHAPE, "too many tiles");

  p->split_k = 1;
  if (f32) {
    if (d->split_k == 0) p->split_k = choose_split_k(items, p->k_blocks, units);
    else p->split_k = d->split_k;
  } else if (d->split_k > 1) {
    return fail(B200GEMM_ERR_UNSUPPORTED, "split-K needs fp32 output");
  }
  if (p->split_k > p->k_blocks) p->split_k = p->k_blocks;
  p->kb_per_split = ceil_div(p->k_blocks, p->split_k);
  p->split_k = ceil_div(p->k_blocks, p->kb_per_split);   // drop slices that would be empty

  if (f32) {
    p->epi = kEpiF32Tma;
    p->reduce = (d->mode == B200GEMM_ACCUMULATE || p->split_k > 1) ? 1 : 0;
  } else {
    p->epi = d->mode == B200GEMM_ACCUMULATE ? kEpiBf16Rmw : kEpiBf16Tma;
    if (p->epi == kEpiBf16Rmw && ((p->ldc % 8) != 0 || (p->bsc % 8) != 0))
      return fail(B200GEMM_ERR_SHAPE, "bf16 accumulate needs ldc and batch stride multiples of 8");
  }
  const int64_t work = items * p->split_k;
  p->grid = static_cast<int>(std::min<int64_t>(work, units)) * p->cta_group;
  p->smem = p->cta_group == 2 ? (p->wide ? GemmCfg<2, true>::kSmemBytes : GemmCfg<2>::kSmemBytes) : GemmCfg<1>::kSmemBytes;
  return B200GEMM_OK;
}

// GemmParams::sched_counter value a caller sets to keep a launch on the static schedule
// whatever the handle's mode is (the entry point that must not allocate).
int* const kStaticScheduleOnly = reinterpret_cast<int*>(1);

// The stream's counter pair, created on first use (null: static schedule).
int sched_counters_for(b200gemm_context* ctx, cudaStream_t stream, int** out) {
  std::lock_guard<std::mutex> lock(ctx->sched_mu);
  auto it = ctx->sched_counters.find(stream);
  if (it == ctx->sched_counters.end()) {
    int* ptr = nullptr;
    CUDA_TRY(cudaMalloc(&ptr, 2 * sizeof(int)));
    CUDA_TRY(cudaMemset(ptr, 0, 2 * sizeof(int)));
    it = ctx->sched_counters.emplace(stream, ptr).first;
  }
  *out = it->second;
  return B200GEMM_OK;
}

template <int CG, int EPI, int SCHED, bool WIDE = false>
int launch_kernel(b200gemm_context* ctx, const GemmParams& params_in, int grid, cudaStream_t stream) {
  auto kernel = gemm_tcgen05_kernel<CG, EPI, SCHED, WIDE>;
  GemmParams params = params_in;
  const bool static_only = params.sched_counter == kStaticScheduleOnly;
  params.sched_counter = nullptr;
  if (CG == 2 && ctx->scheduler == 1 && !static_only) {
    int rc = sched_counters_for(ctx, stream, &params.sched_counter);
    if (rc) return rc;
  }
  // Per-device opt-in to > 48 KiB dynamic shared memory, once per kernel
  // (the reference's opt_in_dynamic_smem, host.rs:485-505).
  bool& ready = ctx->smem_opt_in[CG - 1 + (WIDE ? 2 : 0)][EPI][SCHED];
  if (!ready) {
    CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  GemmCfg<CG, WIDE>::kSmemBytes));
    ready = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = GemmCfg<CG, WIDE>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, params));
  return B200GEMM_OK;
}

template <int CG, int EPI>
int launch_one(b200gemm_context* ctx, const GemmParams& params, const Plan& plan,
               cudaStream_t stream) {
  return launch_kernel<CG, EPI, kSchedDense>(ctx, params, plan.grid, stream);
}

int launch_gemm(b200gemm_context* ctx, cudaStream_t stream, const b200gemm_desc_t* d,
                void* dual_bf16 = nullptr, int64_t ld_dual = 0, int64_t batch_stride_dual = 0) {
  Plan plan;
  int rc = make_plan(ctx, d, &plan);
  if (rc) return rc;
  const bool a_mn = d->a_layout == B200GEMM_MN_MAJOR, b_mn = d->b_layout == B200GEMM_MN_MAJOR;

  GemmParams params;
  memset(&params, 0, sizeof(params));
  const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!a_mn) rc = encode_map(ctx, &params.map_a, bf16, 2, d->a, d->k, d->m, d->batch, plan.lda, plan.bsa, 64, kTileMCta, "A");
  else rc = encode_map(ctx, &params.map_a, bf16, 2, d->a, d->m, d->k, d->batch, plan.lda, plan.bsa, 64, 64, "A");
  if (rc) return rc;
  if (!b_mn) rc = encode_map(ctx, &params.map_b, bf16, 2, d->b, d->k, d->n, d->batch, plan.ldb, plan.bsb, 64, kTileN / plan.cta_group, "B");
  else rc = encode_map(ctx, &params.map_b, bf16, 2, d->b, d->n, d->k, d->batch, plan.ldb, plan.bsb, 64, 64, "B");
  if (rc) return rc;
  if (plan.epi == kEpiF32Tma)
    rc = encode_map(ctx, &params.map_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, d->c, d->n, d->m, d->batch, plan.ldc, plan.bsc, 32, 32, "C");
  else if (plan.epi == kEpiBf16Tma)
    rc = encode_map(ctx, &params.map_c, bf16, 2, d->c, d->n, d->m, d->batch, plan.ldc, plan.bsc, 64, 32, "C");
  if (rc) return rc;

  if (dual_bf16 && plan.wide) return fail(B200GEMM_ERR_UNSUPPORTED, "the dual-output form does not use wide tiles");
  if (dual_bf16) {
    rc = encode_map(ctx, &params.map_d, bf16, 2, dual_bf16, d->n, d->m, d->batch, ld_dual, batch_stride_dual, 64, 32,
                    "bf16 copy of C");
    if (rc) return rc;
  }

  params.status = ctx->status;
  params.c_bf16 = static_cast<uint16_t*>(d->c);
  params.ldc = plan.ldc;
  params.batch_stride_c = plan.bsc;
  params.m = static_cast<int>(d->m);
  params.n = static_cast<int>(d->n);
  params.tiles_m = plan.tiles_m;
  params.tiles_n = plan.tiles_n;
  params.batch = d->batch;
  params.k_blocks = plan.k_blocks;
  params.split_k = plan.split_k;
  params.kb_per_split = plan.kb_per_split;
  params.a_mn = a_mn;
  params.b_mn = b_mn;
  params.reduce = plan.reduce;

  if (plan.epi == kEpiF32Tma && d->mode == B200GEMM_STORE && plan.split_k > 1) {
    // K slices all reduce-add into C, so a store starts from zeros.
    for (int e = 0; e < d->batch; ++e) {
      float* ce = static_cast<float*>(d->c) + static_cast<int64_t>(e) * plan.bsc;
      CUDA_TRY(cudaMemset2DAsync(ce, plan.ldc * sizeof(float), 0, d->n * sizeof(float), d->m, stream));
    }
  }

  if (dual_bf16) {
    if (plan.cta_group == 1) return launch_one<1, kEpiF32DualBf16>(ctx, params, plan, stream);
    return launch_one<2, kEpiF32DualBf16>(ctx, params, plan, stream);
  }
  if (plan.cta_group == 1) {
    switch (plan.epi) {
      case kEpiF32Tma: return launch_one<1, kEpiF32Tma>(ctx, params, plan, stream);
      case kEpiBf16Tma: return launch_one<1, kEpiBf16Tma>(ctx, params, plan, stream);
      default: return launch_one<1, kEpiBf16Rmw>(ctx, params, plan, stream);
    }
  }
  switch (plan.epi) {
    case kEpiF32Tma:
      if (plan.wide) return launch_kernel<2, kEpiF32Tma, kSchedDense, true>(ctx, params, plan.grid, stream);
      return launch_one<2, kEpiF32Tma>(ctx, params, plan, stream);
    case kEpiBf16Tma: return launch_one<2, kEpiBf16Tma>(ctx, params, plan, stream);
    default: return launch_one<2, kEpiBf16Rmw>(ctx, params, plan, stream);
  }
}


// ---------------------------------------------------------------- lm-head + cross entropy

constexpr int kCeMaxChunks = 8;

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct CeWorkspace {
  CeAccum* accum;
  float* target_logit;
  float2* partials;
};

size_t ce_workspace_bytes(int64_t m) {
  return 256 + align_up(static_cast<size_t>(m) * sizeof(float), 256) +
         static_cast<size_t>(kCeMaxChunks) * m * sizeof(float2);
}

CeWorkspace ce_carve(void* ws, int64_t m) {
  uint8_t* p = static_cast<uint8_t*>(ws);
  CeWorkspace w;
  w.accum = reinterpret_cast<CeAccum*>(p);
  w.target_logit = reinterpret_cast<float*>(p + 256);
  w.partials = reinterpret_cast<float2*>(p + 256 + align_up(static_cast<size_t>(m) * sizeof(float), 256));
  return w;
}

int ce_check(const void* hidden, const void* weight, int32_t w_layout, const int32_t* targets,
             int64_t m, int64_t k, int64_t v, int64_t classes) {
  if (!hidden || !weight || !targets) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (w_layout < 0 || w_layout > 1) return fail(B200GEMM_ERR_INVALID, "bad weight layout");
  if (m <= 0 || k <= 0 || v <= 0 || classes <= 0 || classes > v)
    return fail(B200GEMM_ERR_SHAPE, "need m, k, v > 0 and 0 < classes <= v");
  if (m > (1ll << 30) || k > (1ll << 30) || v > (1ll << 30)) return fail(B200GEMM_ERR_SHAPE, "extent too large");
  if ((k % 8) != 0 || (v % 8) != 0)
    return fail(B200GEMM_ERR_SHAPE, "k and v must be multiples of 8 (16-byte rows)");
  return B200GEMM_OK;
}

// Operand maps of logits = hidden . W for a CTA-pair launch.
int ce_encode_operands(b200gemm_context* ctx, GemmParams* params, const void* hidden,
                       const void* weight, int32_t w_layout, int64_t m, int64_t k, int64_t v) {
  const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int rc = encode_map(ctx, &params->map_a, bf16, 2, hidden, k, m, 1, k, 0, 64, kTileMCta, "hidden");
  if (rc) return rc;
  if (w_layout == B200GEMM_MN_MAJOR)   // stored [k, v]
    rc = encode_map(ctx, &params->map_b, bf16, 2, weight, v, k, 1, v, 0, 64, 64, "weight");
  else                                  // stored [v, k]
    rc = encode_map(ctx, &params->map_b, bf16, 2, weight, k, v, 1, k, 0, 64, kTileN / 2, "weight");
  params->a_mn = 0;
  params->b_mn = w_layout == B200GEMM_MN_MAJOR;
  return rc;
}

// With `shard` set the launch is one vocabulary shard's: it hands back the
// shard's per-row (max, sum-exp, target logit) instead of lse and the loss.
struct CeShardOut {
  float* row_max;
  float* row_sum;
  float* row_target_logit;
};

int ce_forward(b200gemm_context* ctx, cudaStream_t stream, const void* hidden, const void* weight,
               int32_t w_layout, const int32_t* targets, int64_t m, int64_t k, int64_t v,
               int64_t classes, float* lse, float* row_loss, float* loss, void* workspace,
               size_t workspace_bytes, const CeShardOut* shard = nullptr, bool may_allocate = true) {
  int rc = ce_check(hidden, weight, w_layout, targets, m, k, v, classes);
  if (rc) return rc;
  if (!shard && !lse) return fail(B200GEMM_ERR_INVALID, "lse output is required");
  if (shard && (!shard->row_max || !shard->row_sum || !shard->row_target_logit))
    return fail(B200GEMM_ERR_INVALID, "null shard output");
  if (!workspace || workspace_bytes < ce_workspace_bytes(m) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return fail(B200GEMM_ERR_INVALID, "workspace missing, too small (%zu needed) or not 256-byte aligned",
                ce_workspace_bytes(m));
  const CeWorkspace ws = ce_carve(workspace, m);
  GemmParams params;
  memset(&params, 0, sizeof(params));
  rc = ce_encode_operands(ctx, &params, hidden, weight, w_layout, m, k, v);
  if (rc) return rc;
  params.status = ctx->status;
  params.m = static_cast<int>(m);
  params.n = static_cast<int>(v);
  params.tiles_m = ceil_div(m, 2 * kTileMCta);
  params.tiles_n = ceil_div(classes, kTileN);    // tiles that are all padding are never computed
  params.batch = 1;
  params.k_blocks = ceil_div(k, kBlockK);
  params.split_k = 1;
  params.kb_per_split = params.k_blocks;
  params.targets = targets;
  params.ce_partials = ws.partials;
  params.ce_target_logit = ws.target_logit;
  params.ce_classes = static_cast<int>(classes);
  // Vocabulary chunks: enough (row block, chunk) items to fill the last wave
  // of the persistent clusters, few enough that the merge stays negligible.
  const int units = std::max(1, ctx->sm_count / 2);
  int best = 1;
  double best_eff = 0.0;
  for (int c = 1; c <= std::min(kCeMaxChunks, params.tiles_n); ++c) {
    const int64_t items = static_cast<int64_t>(params.tiles_m) * c;
    const double eff = static_cast<double>(items) / (static_cast<double>((items + units - 1) / units) * units);
    if (eff > best_eff + 0.01) {
      best_eff = eff;
      best = c;
    }
  }
  params.ce_chunks = best;
  const int64_t items = static_cast<int64_t>(params.tiles_m) * params.ce_chunks;
  const int grid = static_cast<int>(std::min<int64_t>(items, units)) * 2;
  CUDA_TRY(cudaMemsetAsync(ws.accum, 0, sizeof(CeAccum), stream));
  // A row whose target lies in another shard gets no target logit from this one.
  if (shard) CUDA_TRY(cudaMemsetAsync(ws.target_logit, 0, static_cast<size_t>(m) * sizeof(float), stream));
  if (!may_allocate) params.sched_counter = kStaticScheduleOnly;
  rc = launch_kernel<2, kEpiCeForward, kSchedCeForward>(ctx, params, grid, stream);
  if (rc) return rc;
  const int blocks = static_cast<int>(std::min<int64_t>((m + 255) / 256, ctx->sm_count * 4));
  if (shard) {
    ce_partial_kernel<<<blocks, 256, 0, stream>>>(ws.partials, ws.target_logit, static_cast<int>(m),
                                                  params.ce_chunks, shard->row_max, shard->row_sum,
                                                  shard->row_target_logit);
    CUDA_TRY(cudaGetLastError());
    return B200GEMM_OK;
  }
  ce_combine_kernel<<<blocks, 256, 0, stream>>>(ws.partials, ws.target_logit, targets, static_cast<int>(classes),
                                                static_cast<int>(m), params.ce_chunks, lse, row_loss, loss,
                                                ws.accum, ctx->status);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int ce_backward(b200gemm_context* ctx, cudaStream_t stream, const void* hidden, const void* weight,
                int32_t w_layout, const int32_t* targets, const float* lse, float dy, int64_t m,
                int64_t k, int64_t v, int64_t classes, void* dlogits, float* d_hidden,
                float* d_weight, int32_t accumulate_dw) {
  int rc = ce_check(hidden, weight, w_layout, targets, m, k, v, classes);
  if (rc) return rc;
  if (!lse || !dlogits) return fail(B200GEMM_ERR_INVALID, "lse and dlogits are required");
  // 1. recompute the logits tile by tile; the epilogue writes dlogits (bf16).
  GemmParams params;
  memset(&params, 0, sizeof(params));
  rc = ce_encode_operands(ctx, &params, hidden, weight, w_layout, m, k, v);
  if (rc) return rc;
  rc = encode_map(ctx, &params.map_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dlogits, v, m, 1, v, 0, 64, 32, "dlogits");
  if (rc) return rc;
  params.status = ctx->status;
  params.m = static_cast<int>(m);
  params.n = static_cast<int>(v);
  params.tiles_m = ceil_div(m, 2 * kTileMCta);
  params.tiles_n = ceil_div(v, kTileN);           // padded columns are written as zeros
  params.batch = 1;
  params.k_blocks = ceil_div(k, kBlockK);
  params.split_k = 1;
  params.kb_per_split = params.k_blocks;
  params.targets = targets;
  params.ce_lse = lse;
  params.ce_scale = dy / static_cast<float>(m);
  params.ce_classes = static_cast<int>(classes);
  const int units = std::max(1, ctx->sm_count / 2);
  const int64_t items = static_cast<int64_t>(params.tiles_m) * params.tiles_n;
  const int grid = static_cast<int>(std::min<int64_t>(items, units)) * 2;
  rc = launch_kernel<2, kEpiCeBackward, kSchedDense>(ctx, params, grid, stream);
  if (rc) return rc;
  // 2. d_hidden[m, k] = dlogits[m, v] . W^T
  if (d_hidden) {
    b200gemm_desc_t d;
    memset(&d, 0, sizeof(d));
    d.a = dlogits; d.b = weight; d.c = d_hidden;
    d.m = m; d.n = k; d.k = v;
    d.a_layout = B200GEMM_K_MAJOR;
    // W stored [k, v] is B[n = k, K = v] K-major; stored [v, k] it is MN-major.
    d.b_layout = w_layout == B200GEMM_MN_MAJOR ? B200GEMM_K_MAJOR : B200GEMM_MN_MAJOR;
    d.out_type = B200GEMM_OUT_F32; d.mode = B200GEMM_STORE; d.batch = 1;
    rc = launch_gemm(ctx, stream, &d);
    if (rc) return rc;
  }
  // 3. d_weight (=|+=) hidden^T . dlogits, in the weight's own orientation
  if (d_weight) {
    b200gemm_desc_t d;
    memset(&d, 0, sizeof(d));
    d.a_layout = d.b_layout = B200GEMM_MN_MAJOR;   // both operands are [K = m rows, ...]
    d.k = m;
    if (w_layout == B200GEMM_MN_MAJOR) { d.a = hidden; d.b = dlogits; d.m = k; d.n = v; }
    else { d.a = dlogits; d.b = hidden; d.m = v; d.n = k; }
    d.c = d_weight;
    d.out_type = B200GEMM_OUT_F32;
    d.mode = accumulate_dw ? B200GEMM_ACCUMULATE : B200GEMM_STORE;
    d.batch = 1;
    rc = launch_gemm(ctx, stream, &d);
    if (rc) return rc;
  }
  return B200GEMM_OK;
}


// ---------------------------------------------------------------- grouped expert GEMM

int grouped_gemm(b200gemm_context* ctx, cudaStream_t stream, const void* a, int64_t lda,
                 const void* b, int32_t b_layout, int64_t ldb, int64_t batch_stride_b, void* c,
                 int64_t ldc, const int32_t* offsets, int32_t groups, int64_t total_rows, int64_t n,
                 int64_t k, int32_t activation, const int32_t* group_b_index = nullptr,
                 int32_t b_count = 0, void* panel = nullptr, int64_t ld_panel = 0,
                 const void* saved = nullptr, int64_t ld_saved = 0, const PeerBuffers* peer_out = nullptr,
                 const int32_t* group_dst_rank = nullptr, const int32_t* group_dst_row = nullptr,
                 int64_t peer_rows = 0) {
  // activation 2 (SwiGLU): B is [gate | up], 2 * n columns; C = silu(gate) * up has n.
  // activation 3 / 4: the backward of SiLU / SwiGLU applied to the product (an input gradient)
  // from `saved`; with 4, C is the [rows, 2, n] gradient panel.
  const bool glu = activation == 2;
  const bool act_bwd = activation == 3 || activation == 4;
  const int64_t bn = glu ? 2 * n : n;                      // B's extent along N
  const int64_t c_cols = activation == 4 ? 2 * n : n;      // C's row length
  if (act_bwd) {
    if (!saved) return fail(B200GEMM_ERR_INVALID, "null saved activations");
    if ((n % 8) != 0 || (activation == 4 && (n % 64) != 0))
      return fail(B200GEMM_ERR_SHAPE, "the fused activation backward needs n %% 8 == 0 (SiLU) / n %% 64 == 0 (SwiGLU)");
    ld_saved = ld_saved ? ld_saved : c_cols;
    if (ld_saved < c_cols || (ld_saved % 8) != 0 || (reinterpret_cast<uintptr_t>(saved) & 15u) != 0)
      return fail(B200GEMM_ERR_SHAPE, "saved activations: row stride must cover the row and be a multiple of 8, base 16-byte aligned");
  }
  if (!a || !b || (!c && !peer_out) || !offsets) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (peer_out && (!group_dst_rank || !group_dst_row || activation != 0 || (n % 8) != 0 || peer_rows <= 0))
    return fail(B200GEMM_ERR_INVALID, "the peer-store form needs its group tables, no activation, n %% 8 == 0 and a row limit");
  if (group_b_index && b_count < 1) return fail(B200GEMM_ERR_SHAPE, "b_count must be positive with a group index");
  const int32_t b_mats = group_b_index ? b_count : groups;
  if (b_layout < 0 || b_layout > 1 || activation < 0 || activation > 4)
    return fail(B200GEMM_ERR_INVALID, "bad layout or activation");
  if (panel && activation == 0) return fail(B200GEMM_ERR_INVALID, "a second output is written only with an activation");
  if (glu && (n % 8) != 0) return fail(B200GEMM_ERR_SHAPE, "SwiGLU needs ff to be a multiple of 8");
  if (panel && glu && (n % 64) != 0) return fail(B200GEMM_ERR_SHAPE, "the gate/up panel needs ff to be a multiple of 64");
  if (groups < 1 || groups > kMaxGroups) return fail(B200GEMM_ERR_SHAPE, "groups must be in [1, %d]", kMaxGroups);
  if (total_rows <= 0 || n <= 0 || k <= 0 || total_rows > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30))
    return fail(B200GEMM_ERR_SHAPE, "bad extent");
  const bool b_mn = b_layout == B200GEMM_MN_MAJOR;
  lda = lda ? lda : k;
  ldb = ldb ? ldb : (b_mn ? bn : k);
  ldc = ldc ? ldc : c_cols;
  const int64_t panel_cols = glu ? 2 * n : n;            // SiLU keeps the [rows, n] values before the activation
  ld_panel = ld_panel ? ld_panel : panel_cols;
  if (lda < k || ldb < (b_mn ? bn : k) || ldc < c_cols) return fail(B200GEMM_ERR_SHAPE, "leading dimension too small");
  if ((ldc % 8) != 0) return fail(B200GEMM_ERR_SHAPE, "ldc must be a multiple of 8");
  if (panel && (ld_panel < panel_cols || (ld_panel % 8) != 0))
    return fail(B200GEMM_ERR_SHAPE, "second output's row stride must cover its row and be a multiple of 8");
  const int64_t bsb = batch_stride_b ? batch_stride_b : ldb * (b_mn ? k : bn);
  GemmParams params;
  memset(&params, 0, sizeof(params));
  const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int rc = encode_map(ctx, &params.map_a, bf16, 2, a, k, total_rows, 1, lda, 0, 64, kTileMCta, "A");
  if (rc) return rc;
  if (!b_mn) rc = encode_map(ctx, &params.map_b, bf16, 2, b, k, bn, b_mats, ldb, bsb, 64, kTileN / 2, "B");
  else rc = encode_map(ctx, &params.map_b, bf16, 2, b, bn, k, b_mats, ldb, bsb, 64, 64, "B");
  if (rc) return rc;
  if (!peer_out) {
    rc = encode_map(ctx, &params.map_c, bf16, 2, c, c_cols, total_rows, 1, ldc, 0, 64, 32, "C");
    if (rc) return rc;
  } else {
    params.peer_out = *peer_out;
    params.group_dst_rank = group_dst_rank;
    params.group_dst_row = group_dst_row;
    params.peer_rows = peer_rows;
  }
  if (panel) {
    rc = encode_map(ctx, &params.map_d, bf16, 2, panel, panel_cols, total_rows, 1, ld_panel, 0, 64, 32, "panel");
    if (rc) return rc;
    params.d_bf16 = static_cast<uint16_t*>(panel);
    params.ldd = ld_panel;
  }
  params.status = ctx->status;
  params.c_bf16 = static_cast<uint16_t*>(c);
  params.ldc = ldc;
  params.m = static_cast<int>(total_rows);
  params.n = static_cast<int>(n);
  params.tiles_n = ceil_div(n, glu ? kTileN / 2 : kTileN);
  params.tiles_m = 0;
  params.batch = groups;
  params.k_blocks = ceil_div(k, kBlockK);
  params.split_k = 1;
  params.kb_per_split = params.k_blocks;
  params.b_mn = b_mn;
  params.group_offsets = offsets;
  params.group_b_index = group_b_index;
  params.groups = groups;
  params.act_silu = activation == 1 ? 1 : (activation == 3 ? 2 : (activation == 4 ? 3 : 0));
  params.saved = static_cast<const uint16_t*>(saved);
  params.ld_saved = ld_saved;
  params.glu_cols = glu ? static_cast<int>(n) : 0;
  // The tile count depends on the device-side offsets; bound it from above
  // (each group wastes at most one partial tile) and let surplus clusters exit.
  const int units = std::max(1, ctx->sm_count / 2);
  const int64_t max_items = (ceil_div(total_rows, 2 * kTileMCta) + static_cast<int64_t>(groups)) * params.tiles_n;
  const int grid = static_cast<int>(std::min<int64_t>(max_items, units)) * 2;
  if (glu) return launch_kernel<2, kEpiBf16GroupedGlu, kSchedGrouped>(ctx, params, grid, stream);
  if (act_bwd) return launch_kernel<2, kEpiBf16GroupedActBwd, kSchedGrouped>(ctx, params, grid, stream);
  if (peer_out) return launch_kernel<2, kEpiBf16GroupedPeer, kSchedGrouped>(ctx, params, grid, stream);
  return launch_kernel<2, kEpiBf16Grouped, kSchedGrouped>(ctx, params, grid, stream);
}

// Weight gradients of the grouped GEMM: the row groups are the reduction axis.
int grouped_wgrad(b200gemm_context* ctx, cudaStream_t stream, const void* a, int64_t lda, const void* b,
                  int64_t ldb, float* c, int64_t ldc, int64_t batch_stride_c, int32_t c_count,
                  const int32_t* group_c_index, const int32_t* offsets, int32_t groups, int64_t total_rows,
                  int64_t m, int64_t n, int32_t accumulate) {
  if (!a || !b || !c || !offsets) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (groups < 1 || groups > kMaxGroups) return fail(B200GEMM_ERR_SHAPE, "groups must be in [1, %d]", kMaxGroups);
  if (group_c_index && c_count < 1) return fail(B200GEMM_ERR_SHAPE, "c_count must be positive with a group index");
  const int32_t c_mats = group_c_index ? c_count : groups;
  if (total_rows <= 0 || m <= 0 || n <= 0 || total_rows > (1ll << 30) || m > (1ll << 30) || n > (1ll << 30))
    return fail(B200GEMM_ERR_SHAPE, "bad extent");
  lda = lda ? lda : m;
  ldb = ldb ? ldb : n;
  ldc = ldc ? ldc : n;
  if (lda < m || ldb < n || ldc < n) return fail(B200GEMM_ERR_SHAPE, "leading dimension too small");
  const int64_t bsc = batch_stride_c ? batch_stride_c : ldc * m;
  GemmParams params;
  memset(&params, 0, sizeof(params));
  const auto bf16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // Both operands are [rows = K, width] row-major: MN-major boxes of 64 x 64.
  int rc = encode_map(ctx, &params.map_a, bf16, 2, a, m, total_rows, 1, lda, 0, 64, 64, "A");
  if (rc) return rc;
  rc = encode_map(ctx, &params.map_b, bf16, 2, b, n, total_rows, 1, ldb, 0, 64, 64, "B");
  if (rc) return rc;
  rc = encode_map(ctx, &params.map_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, c, n, m, c_mats, ldc, bsc, 32, 32, "C");
  if (rc) return rc;
  params.status = ctx->status;
  params.m = static_cast<int>(m);
  params.n = static_cast<int>(n);
  params.tiles_m = ceil_div(m, 2 * kTileMCta);
  params.tiles_n = ceil_div(n, kTileN);
  params.batch = c_mats;
  params.a_mn = 1;
  params.b_mn = 1;
  params.reduce = 1;                       // every (group, chunk) item adds its part into C
  params.group_offsets = offsets;
  params.group_b_index = group_c_index;
  params.groups = groups;
  params.split_k = 1;
  // Rows per chunk: short enough that the items outnumber the clusters several times over
  // (hot experts then spread over many clusters instead of serialising on one), long enough
  // that the reduce-add traffic of an item stays small beside its products.
  const int units = std::max(1, ctx->sm_count / 2);
  const int64_t tiles = static_cast<int64_t>(params.tiles_m) * params.tiles_n;
  const int64_t total_kb = ceil_div(total_rows, kBlockK);
  int64_t chunk = total_kb * tiles / (8ll * units);
  chunk = std::max<int64_t>(8, std::min<int64_t>(64, chunk));
  params.kb_per_split = static_cast<int>(chunk);
  params.k_blocks = static_cast<int>(chunk);
  if (!accumulate) {
    for (int e = 0; e < c_mats; ++e)
      CUDA_TRY(cudaMemset2DAsync(c + static_cast<int64_t>(e) * bsc, ldc * sizeof(float), 0, n * sizeof(float), m, stream));
  }
  const int64_t max_items = (ceil_div(total_kb, chunk) + static_cast<int64_t>(groups)) * tiles;
  const int grid = static_cast<int>(std::min<int64_t>(max_items, units)) * 2;
  return launch_kernel<2, kEpiF32Tma, kSchedGroupedWgrad>(ctx, params, grid, stream);
}

// ---------------------------------------------------------------- MoE routing

int moe_check(int64_t tokens, int32_t experts, int32_t top_k) {
  if (tokens <= 0 || tokens > (1ll << 28)) return fail(B200GEMM_ERR_SHAPE, "bad token count");
  if (experts < 1 || experts > kMoeMaxExperts) return fail(B200GEMM_ERR_SHAPE, "experts must be in [1, %d]", kMoeMaxExperts);
  if (top_k < 1 || top_k > kMoeMaxTopK || top_k > experts)
    return fail(B200GEMM_ERR_SHAPE, "top_k must be in [1, min(%d, experts)]", kMoeMaxTopK);
  return B200GEMM_OK;
}


// ---------------------------------------------------------------- allocation-free head forward

// Largest row count b200gemm_lmhead_ce_forward_noalloc accepts, and the bytes
// of scratch that needs (same carving as ce_carve: 256-byte accumulator block,
// one fp32 target logit per row, kCeMaxChunks (max, sum-exp) pairs per row).
constexpr int64_t kCeStaticMaxRows = 32768;
constexpr size_t kCeStaticBytes =
    256 + static_cast<size_t>(kCeStaticMaxRows) * sizeof(float) +
    static_cast<size_t>(kCeMaxChunks) * kCeStaticMaxRows * sizeof(float2);

// The scratch itself: part of the library image, so it exists on every GPU the
// library is loaded on from load until exit, and no call ever allocates it.
static __device__ __align__(256) unsigned char g_ce_static_scratch[kCeStaticBytes];

constexpr int kCeStaticMaxDevices = 64;
std::mutex g_ce_static_mu;
void* g_ce_static_ptr[kCeStaticMaxDevices] = {};

// Device address of the scratch array on `device`.  In host code the array's
// name is only a handle for the runtime, not an address a kernel can use, so
// the address is looked up once per device (that device must be current) and
// remembered.
int ce_static_scratch(int device, void** out) {
  if (device < 0 || device >= kCeStaticMaxDevices)
    return fail(B200GEMM_ERR_UNSUPPORTED, "device ordinal %d is beyond the %d this entry point tracks",
                device, kCeStaticMaxDevices);
  // Every call, not only the first: the launches below go to whichever device is current,
  // with pointers that belong to `device`.
  int current = -1;
  CUDA_TRY(cudaGetDevice(&current));
  if (current != device)
    return fail(B200GEMM_ERR_INVALID, "device %d must be current on the calling thread (device %d is)",
                device, current);
  std::lock_guard<std::mutex> lock(g_ce_static_mu);
  if (!g_ce_static_ptr[device]) {
    void* ptr = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&ptr, g_ce_static_scratch));
    if (!ptr) return fail(B200GEMM_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_ce_static_ptr[device] = ptr;
  }
  *out = g_ce_static_ptr[device];
  return B200GEMM_OK;
}

int check_handle(b200gemm_handle_t h) {
  if (!h) return fail(B200GEMM_ERR_INVALID, "null handle");
  return B200GEMM_OK;
}

}  // namespace

// ==================================================================== C ABI

extern "C" {

int b200gemm_version(void) { return 100; }

int b200gemm_set_sm_limit(b200gemm_handle_t h, int32_t sms) {
  if (!h) return fail(B200GEMM_ERR_INVALID, "null handle");
  if (sms <= 0 || sms > h->sm_total) sms = h->sm_total;
  h->sm_count = sms < 2 ? 2 : sms;
  return B200GEMM_OK;
}

int b200gemm_set_exchange_ctas(b200gemm_handle_t h, int32_t ctas, int32_t bulk) {
  if (!h) return fail(B200GEMM_ERR_INVALID, "null handle");
  if (ctas < 0 || ctas > 4 * h->sm_total) return fail(B200GEMM_ERR_INVALID, "ctas must be 0 (default) .. 4 per SM");
  if (bulk < 0 || bulk > 1) return fail(B200GEMM_ERR_INVALID, "bulk must be 0 or 1");
  h->exchange_ctas = ctas;
  h->exchange_bulk = bulk != 0 && ctas > 0;
  return B200GEMM_OK;
}

int b200gemm_set_scheduler(b200gemm_handle_t h, int32_t mode) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (mode < 0 || mode > 1) return fail(B200GEMM_ERR_INVALID, "scheduler mode must be 0 (static) or 1 (dynamic)");
  h->scheduler = mode;
  return B200GEMM_OK;
}

const char* b200gemm_last_error_string(void) { return g_error; }

int b200gemm_create(int device, b200gemm_handle_t* out) {
  if (!out) return fail(B200GEMM_ERR_INVALID, "null output handle");
  *out = nullptr;
  int count = 0;
  CUDA_TRY(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count) return fail(B200GEMM_ERR_INVALID, "no CUDA device %d", device);
  cudaDeviceProp prop;
  CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(B200GEMM_ERR_UNSUPPORTED,
                "device %d is compute capability %d.%d; this library is sm_100a only and has no "
                "fallback path",
                device, prop.major, prop.minor);
  CUDA_TRY(cudaSetDevice(device));
  b200gemm_context* ctx = new (std::nothrow) b200gemm_context();
  if (!ctx) return fail(B200GEMM_ERR_INVALID, "out of host memory");
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->sm_total = prop.multiProcessorCount;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
    delete ctx;
    return fail(B200GEMM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  }
  ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
  e = cudaMalloc(&ctx->status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ctx->status, 0, sizeof(int));
  if (e != cudaSuccess) {
    delete ctx;
    return fail(B200GEMM_ERR_CUDA, "status word allocation failed: %s", cudaGetErrorString(e));
  }
  *out = ctx;
  return B200GEMM_OK;
}

int b200gemm_destroy(b200gemm_handle_t h) {
  if (!h) return B200GEMM_OK;
  cudaSetDevice(h->device);
  for (void* p : h->stage)
    if (p) cudaFree(p);
  for (auto& kv : h->moe_scratch)
    if (kv.second.ptr) cudaFree(kv.second.ptr);
  for (auto& kv : h->sched_counters)
    if (kv.second) cudaFree(kv.second);
  if (h->status) cudaFree(h->status);
  delete h;
  return B200GEMM_OK;
}

int b200gemm_gemm(b200gemm_handle_t h, void* stream, const b200gemm_desc_t* desc) {
  int rc = check_handle(h);
  if (rc) return rc;
  return launch_gemm(h, static_cast<cudaStream_t>(stream), desc);
}

int b200gemm_gemm_dual(b200gemm_handle_t h, void* stream, const b200gemm_desc_t* desc, void* c_bf16,
                       int64_t ldc_bf16, int64_t batch_stride_c_bf16) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!desc) return fail(B200GEMM_ERR_INVALID, "null descriptor");
  if (!c_bf16) return fail(B200GEMM_ERR_INVALID, "null bf16 output");
  if (desc->out_type != B200GEMM_OUT_F32 || desc->mode != B200GEMM_STORE)
    return fail(B200GEMM_ERR_UNSUPPORTED, "the dual-output form is an fp32 store");
  if (desc->split_k > 1) return fail(B200GEMM_ERR_UNSUPPORTED, "the dual-output form does not split K");
  if (ldc_bf16 == 0) ldc_bf16 = desc->n;
  if (ldc_bf16 < desc->n || (ldc_bf16 % 8) != 0)
    return fail(B200GEMM_ERR_SHAPE, "bf16 row stride must be at least n and a multiple of 8");
  if (batch_stride_c_bf16 == 0) batch_stride_c_bf16 = ldc_bf16 * desc->m;
  if ((batch_stride_c_bf16 % 8) != 0) return fail(B200GEMM_ERR_SHAPE, "bf16 batch stride must be a multiple of 8");
  b200gemm_desc_t d = *desc;
  d.split_k = 1;                       // every element is written once, by one tile
  return launch_gemm(h, static_cast<cudaStream_t>(stream), &d, c_bf16, ldc_bf16, batch_stride_c_bf16);
}

int b200gemm_launch_config(b200gemm_handle_t h, const b200gemm_desc_t* desc, int32_t* grid,
                           int32_t* cluster, int32_t* smem_bytes, int32_t* split_k) {
  int rc = check_handle(h);
  if (rc) return rc;
  Plan plan;
  rc = make_plan(h, desc, &plan);
  if (rc) return rc;
  if (grid) *grid = plan.grid;
  if (cluster) *cluster = plan.cta_group;
  if (smem_bytes) *smem_bytes = plan.smem;
  if (split_k) *split_k = plan.split_k;
  return B200GEMM_OK;
}

int b200gemm_sgemm(b200gemm_handle_t h, void* stream, int32_t op, int32_t accumulate,
                   const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!a || !b || !c) return fail(B200GEMM_ERR_INVALID, "null matrix pointer");
  if (op < 0 || op > 2) return fail(B200GEMM_ERR_INVALID, "bad op");
  if (m <= 0 || n <= 0 || k <= 0 || m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30))
    return fail(B200GEMM_ERR_SHAPE, "bad extent");
  CUDA_TRY(launch_sgemm(static_cast<cudaStream_t>(stream), op, accumulate != 0, a, b, c,
                        static_cast<int>(m), static_cast<int>(n), static_cast<int>(k)));
  return B200GEMM_OK;
}

int b200gemm_convert_f32_to_bf16(b200gemm_handle_t h, void* stream, const float* src,
                                 void* dst_bf16, int64_t count) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!src || !dst_bf16) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (count < 0) return fail(B200GEMM_ERR_SHAPE, "negative count");
  if (count == 0) return B200GEMM_OK;
  CUDA_TRY(launch_f32_to_bf16(static_cast<cudaStream_t>(stream), src,
                              static_cast<uint16_t*>(dst_bf16), count, h->sm_count));
  return B200GEMM_OK;
}

int b200gemm_convert_bf16_to_f32(b200gemm_handle_t h, void* stream, const void* src_bf16,
                                 float* dst, int64_t count) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!src_bf16 || !dst) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (count < 0) return fail(B200GEMM_ERR_SHAPE, "negative count");
  if (count == 0) return B200GEMM_OK;
  CUDA_TRY(launch_bf16_to_f32(static_cast<cudaStream_t>(stream),
                              static_cast<const uint16_t*>(src_bf16), dst, count, h->sm_count));
  return B200GEMM_OK;
}

int b200gemm_transpose_bf16(b200gemm_handle_t h, void* stream, const void* src, void* dst,
                            int64_t rows, int64_t cols) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!src || !dst) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (rows <= 0 || cols <= 0 || rows > (1ll << 30) || cols > (1ll << 30))
    return fail(B200GEMM_ERR_SHAPE, "bad extent");
  CUDA_TRY(launch_transpose_bf16(static_cast<cudaStream_t>(stream),
                                 static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst),
                                 static_cast<int>(rows), static_cast<int>(cols)));
  return B200GEMM_OK;
}

size_t b200gemm_lmhead_ce_workspace_bytes(int64_t m) { return m > 0 ? ce_workspace_bytes(m) : 0; }

int b200gemm_lmhead_ce_forward(b200gemm_handle_t h, void* stream, const void* hidden,
                               const void* weight, int32_t w_layout, const int32_t* targets,
                               int64_t m, int64_t k, int64_t v, int64_t classes, float* lse,
                               float* row_loss, float* loss, void* workspace,
                               size_t workspace_bytes) {
  int rc = check_handle(h);
  if (rc) return rc;
  return ce_forward(h, static_cast<cudaStream_t>(stream), hidden, weight, w_layout, targets, m, k, v,
                    classes, lse, row_loss, loss, workspace, workspace_bytes);
}

int b200gemm_lmhead_ce_backward(b200gemm_handle_t h, void* stream, const void* hidden,
                                const void* weight, int32_t w_layout, const int32_t* targets,
                                const float* lse, float dy, int64_t m, int64_t k, int64_t v,
                                int64_t classes, void* dlogits_bf16, float* d_hidden,
                                float* d_weight, int32_t accumulate_dw) {
  int rc = check_handle(h);
  if (rc) return rc;
  return ce_backward(h, static_cast<cudaStream_t>(stream), hidden, weight, w_layout, targets, lse, dy,
                     m, k, v, classes, dlogits_bf16, d_hidden, d_weight, accumulate_dw);
}

int b200gemm_grouped_gemm(b200gemm_handle_t h, void* stream, const void* a, int64_t lda,
                          const void* b, int32_t b_layout, int64_t ldb, int64_t batch_stride_b,
                          void* c, int64_t ldc, const int32_t* offsets, int32_t groups,
                          int64_t total_rows, int64_t n, int64_t k, int32_t activation) {
  int rc = check_handle(h);
  if (rc) return rc;
  return grouped_gemm(h, static_cast<cudaStream_t>(stream), a, lda, b, b_layout, ldb, batch_stride_b,
                      c, ldc, offsets, groups, total_rows, n, k, activation);
}

int b200gemm_moe_route(b200gemm_handle_t h, void* stream_, const float* scores,
                       int32_t scores_are_logits, int64_t tokens, int32_t experts, int32_t top_k,
                       int64_t capacity, uint32_t* selected, float* gates, uint32_t* slots,
                       uint32_t* assignment_counts, uint32_t* accepted_counts, int32_t* offsets,
                       uint32_t* dest_row) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!scores || !selected || !gates || !slots || !assignment_counts || !accepted_counts ||
      !offsets || !dest_row)
    return fail(B200GEMM_ERR_INVALID, "null pointer");
  rc = moe_check(tokens, experts, top_k);
  if (rc) return rc;
  if (capacity <= 0) return fail(B200GEMM_ERR_SHAPE, "capacity must be positive");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long pairs = tokens * top_k;
  const int topk_blocks = static_cast<int>((tokens * 32 + 255) / 256);
  moe_topk_kernel<<<topk_blocks, 256, 0, stream>>>(scores, scores_are_logits, tokens, experts, top_k,
                                                   selected, gates);
  CUDA_TRY(cudaGetLastError());
  // Slot assignment in three passes over 256-pair segments.  The per-segment
  // count table (segments x experts words) lives in scratch owned by the handle,
  // grown on first use and whenever a larger problem arrives.
  const long long segments = (pairs + kMoeSegment - 1) / kMoeSegment;
  const size_t table_bytes = static_cast<size_t>(segments) * experts * sizeof(uint32_t);
  uint32_t* seg_table = nullptr;
  {
    std::lock_guard<std::mutex> lock(h->mu);
    b200gemm_context::Scratch& sc = h->moe_scratch[stream];
    if (sc.bytes < table_bytes) {
      if (sc.ptr) CUDA_TRY(cudaFree(sc.ptr));   // waits for kernels still using it
      sc.ptr = nullptr;
      sc.bytes = 0;
      CUDA_TRY(cudaMalloc(&sc.ptr, table_bytes));
      sc.bytes = table_bytes;
    }
    seg_table = static_cast<uint32_t*>(sc.ptr);
  }
  const int seg_blocks = static_cast<int>((segments + 7) / 8);
  moe_hist_kernel<<<seg_blocks, 256, 0, stream>>>(selected, pairs, experts, seg_table);
  CUDA_TRY(cudaGetLastError());
  moe_scan_kernel<<<experts, 256, 0, stream>>>(seg_table, segments, experts, capacity, assignment_counts,
                                               accepted_counts);
  CUDA_TRY(cudaGetLastError());
  moe_assign_kernel<<<seg_blocks, 256, 0, stream>>>(selected, seg_table, pairs, experts, capacity, slots);
  CUDA_TRY(cudaGetLastError());
  moe_offsets_kernel<<<1, 32, 0, stream>>>(accepted_counts, experts, offsets);
  CUDA_TRY(cudaGetLastError());
  moe_dest_kernel<<<stream_grid(pairs, h->sm_count), 256, 0, stream>>>(selected, slots, offsets, pairs, dest_row);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_moe_scatter(b200gemm_handle_t h, void* stream, const void* x, const uint32_t* dest_row,
                         int64_t tokens, int32_t top_k, int64_t d, void* x_permuted) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!x || !dest_row || !x_permuted) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (tokens <= 0 || top_k < 1 || d <= 0 || (d % 8) != 0) return fail(B200GEMM_ERR_SHAPE, "need tokens, top_k > 0 and d a multiple of 8");
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(x_permuted)) & 15u) != 0)
    return fail(B200GEMM_ERR_SHAPE, "buffers must be 16-byte aligned");
  if (top_k > 32) return fail(B200GEMM_ERR_SHAPE, "top_k must be at most 32");
  moe_scatter_kernel<<<stream_grid(tokens * 32, h->sm_count), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(x), dest_row, tokens, top_k, d, static_cast<uint16_t*>(x_permuted));
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_moe_combine(b200gemm_handle_t h, void* stream, const void* y_permuted,
                         const uint32_t* dest_row, const float* gates, const void* residual,
                         int64_t tokens, int32_t top_k, int64_t d, void* out, int32_t out_type) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!y_permuted || !dest_row || !out) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (tokens <= 0 || top_k < 1 || top_k > kMoeMaxTopK || d <= 0 || (d % 8) != 0)
    return fail(B200GEMM_ERR_SHAPE, "need tokens > 0, top_k in [1, %d], d a multiple of 8", kMoeMaxTopK);
  if (out_type < 0 || out_type > 1) return fail(B200GEMM_ERR_INVALID, "bad output type");
  const int grid = stream_grid(tokens * 32, h->sm_count);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_type == B200GEMM_OUT_BF16)
    moe_combine_kernel<true><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(y_permuted), dest_row, gates,
                                                  static_cast<const uint16_t*>(residual), tokens, top_k, d, out);
  else
    moe_combine_kernel<false><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(y_permuted), dest_row, gates,
                                                   static_cast<const uint16_t*>(residual), tokens, top_k, d, out);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_lmhead_ce_forward_shard(b200gemm_handle_t h, void* stream, const void* hidden,
                                     const void* weight_shard, int32_t w_layout,
                                     const int32_t* local_targets, int64_t m, int64_t k, int64_t v_local,
                                     int64_t classes_local, float* row_max, float* row_sum,
                                     float* row_target_logit, void* workspace, size_t workspace_bytes) {
  int rc = check_handle(h);
  if (rc) return rc;
  const CeShardOut out = {row_max, row_sum, row_target_logit};
  return ce_forward(h, static_cast<cudaStream_t>(stream), hidden, weight_shard, w_layout, local_targets, m,
                    k, v_local, classes_local, nullptr, nullptr, nullptr, workspace, workspace_bytes, &out);
}

int b200gemm_grouped_gemm_indexed(b200gemm_handle_t h, void* stream, const void* a, int64_t lda,
                                  const void* b, int32_t b_layout, int64_t ldb, int64_t batch_stride_b,
                                  int32_t b_count, const int32_t* group_b_index, void* c, int64_t ldc,
                                  const int32_t* offsets, int32_t groups, int64_t total_rows, int64_t n,
                                  int64_t k, int32_t activation) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!group_b_index) return fail(B200GEMM_ERR_INVALID, "null group index");
  return grouped_gemm(h, static_cast<cudaStream_t>(stream), a, lda, b, b_layout, ldb, batch_stride_b, c,
                      ldc, offsets, groups, total_rows, n, k, activation, group_b_index, b_count);
}

int b200gemm_grouped_gemm_swiglu(b200gemm_handle_t h, void* stream, const void* a, int64_t lda,
                                 const void* b, int32_t b_layout, int64_t ldb, int64_t batch_stride_b,
                                 int32_t b_count, const int32_t* group_b_index, void* y, int64_t ldy,
                                 void* gate_up, int64_t ld_gate_up, const int32_t* offsets,
                                 int32_t groups, int64_t total_rows, int64_t ff, int64_t k) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (group_b_index && b_count < 1) return fail(B200GEMM_ERR_SHAPE, "b_count must be positive with a group index");
  return grouped_gemm(h, static_cast<cudaStream_t>(stream), a, lda, b, b_layout, ldb, batch_stride_b, y,
                      ldy, offsets, groups, total_rows, ff, k, 2, group_b_index, b_count, gate_up,
                      ld_gate_up);
}

int b200gemm_lmhead_ce_forward_noalloc(b200gemm_handle_t h, void* stream, const void* hidden,
                                       const void* weight, int32_t w_layout, const int32_t* targets,
                                       int64_t m, int64_t k, int64_t v, int64_t classes, float* lse,
                                       float* row_loss, float* loss) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (m > kCeStaticMaxRows)
    return fail(B200GEMM_ERR_SHAPE,
                "m = %lld exceeds the %lld rows the built-in scratch holds; use "
                "b200gemm_lmhead_ce_forward with a caller-provided workspace",
                static_cast<long long>(m), static_cast<long long>(kCeStaticMaxRows));
  if (m > 0 && ce_workspace_bytes(m) > kCeStaticBytes)
    return fail(B200GEMM_ERR_SHAPE, "built-in scratch too small for m = %lld", static_cast<long long>(m));
  void* scratch = nullptr;
  rc = ce_static_scratch(h->device, &scratch);
  if (rc) return rc;
  return ce_forward(h, static_cast<cudaStream_t>(stream), hidden, weight, w_layout, targets, m, k, v,
                    classes, lse, row_loss, loss, scratch, kCeStaticBytes, nullptr, /*may_allocate=*/false);
}

int b200gemm_moe_ep_plan(b200gemm_handle_t h, void* stream, const int32_t* all_counts, int32_t world,
                         int32_t rank, int32_t experts, int32_t* dst_base, int32_t* group_offsets,
                         int32_t* group_b_index) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!all_counts || !dst_base || !group_offsets || !group_b_index) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (world < 1 || world > kMoeMaxPeers || rank < 0 || rank >= world)
    return fail(B200GEMM_ERR_SHAPE, "world must be in [1, %d] and rank inside it", kMoeMaxPeers);
  if (experts < world || experts > kMaxGroups || experts % world)
    return fail(B200GEMM_ERR_SHAPE, "experts must be a multiple of world and at most %d", kMaxGroups);
  moe_ep_plan_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(all_counts, world, rank, experts, dst_base,
                                                                      group_offsets, group_b_index);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_moe_ep_return_plan(b200gemm_handle_t h, void* stream, const int32_t* all_counts, int32_t world,
                                int32_t rank, int32_t experts, int32_t* group_dst_rank, int32_t* group_dst_row) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!all_counts || !group_dst_rank || !group_dst_row) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (world < 1 || world > kMoeMaxPeers || rank < 0 || rank >= world)
    return fail(B200GEMM_ERR_SHAPE, "world must be in [1, %d] and rank inside it", kMoeMaxPeers);
  if (experts < world || experts > kMaxGroups || experts % world)
    return fail(B200GEMM_ERR_SHAPE, "experts must be a multiple of world and at most %d", kMaxGroups);
  moe_ep_return_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(all_counts, world, rank, experts,
                                                                               group_dst_rank, group_dst_row);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_grouped_gemm_peer(b200gemm_handle_t h, void* stream, const void* a, int64_t lda, const void* b,
                               int32_t b_layout, int64_t ldb, int64_t batch_stride_b, int32_t b_count,
                               const int32_t* group_b_index, void* const* peer_out, int32_t world,
                               int64_t ld_out, int64_t out_rows, const int32_t* group_dst_rank,
                               const int32_t* group_dst_row, const int32_t* offsets, int32_t groups,
                               int64_t total_rows, int64_t n, int64_t k) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!peer_out) return fail(B200GEMM_ERR_INVALID, "null peer pointer table");
  if (world < 1 || world > kMaxPeerRanks) return fail(B200GEMM_ERR_SHAPE, "world must be in [1, %d]", kMaxPeerRanks);
  if (group_b_index && b_count < 1) return fail(B200GEMM_ERR_SHAPE, "b_count must be positive with a group index");
  PeerBuffers pb = {};
  for (int r = 0; r < world; ++r) {
    if (!peer_out[r] || (reinterpret_cast<uintptr_t>(peer_out[r]) & 15u) != 0)
      return fail(B200GEMM_ERR_INVALID, "peer pointer %d is null or not 16-byte aligned", r);
    pb.ptr[r] = static_cast<uint16_t*>(peer_out[r]);
  }
  return grouped_gemm(h, static_cast<cudaStream_t>(stream), a, lda, b, b_layout, ldb, batch_stride_b, nullptr,
                      ld_out, offsets, groups, total_rows, n, k, 0, group_b_index, b_count, nullptr, 0, nullptr, 0,
                      &pb, group_dst_rank, group_dst_row, out_rows);
}

int b200gemm_peer_barrier(b200gemm_handle_t h, void* stream, void* const* peer_words, int32_t world, int32_t rank,
                          uint64_t epoch, int64_t limit_ms, const int32_t* payload, int32_t payload_count,
                          void* const* peer_tables) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!peer_words) return fail(B200GEMM_ERR_INVALID, "null pointer table");
  if (world < 1 || world > kMoeMaxPeers || rank < 0 || rank >= world)
    return fail(B200GEMM_ERR_SHAPE, "world must be in [1, %d] and rank inside it", kMoeMaxPeers);
  if (epoch == 0) return fail(B200GEMM_ERR_INVALID, "epochs start at 1 (the arrival words start at 0)");
  if (limit_ms < 1 || limit_ms > 10000) return fail(B200GEMM_ERR_INVALID, "limit must be 1..10000 ms");
  if ((payload != nullptr) != (peer_tables != nullptr) || (payload && (payload_count < 1 || payload_count > 4096)))
    return fail(B200GEMM_ERR_INVALID, "payload and peer tables go together, 1..4096 integers per rank");
  PeerWords words = {};
  PeerTables tables = {};
  for (int r = 0; r < world; ++r) {
    if (!peer_words[r] || (reinterpret_cast<uintptr_t>(peer_words[r]) & 7u) != 0)
      return fail(B200GEMM_ERR_INVALID, "peer word array %d is null or not 8-byte aligned", r);
    words.ptr[r] = static_cast<unsigned long long*>(peer_words[r]);
    if (peer_tables) {
      if (!peer_tables[r]) return fail(B200GEMM_ERR_INVALID, "null peer table %d", r);
      tables.ptr[r] = static_cast<int*>(peer_tables[r]);
    }
  }
  peer_barrier_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      words, world, rank, epoch, payload, payload ? payload_count : 0, tables, h->status,
      static_cast<unsigned long long>(limit_ms) * 1000000ull);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_moe_ep_push(b200gemm_handle_t h, void* stream, const void* x, const uint32_t* selected,
                         const uint32_t* slots, const int32_t* dst_base, void* const* peer_inbox,
                         int64_t inbox_rows, int32_t world, int32_t experts, int64_t tokens,
                         int32_t top_k, int64_t d) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!x || !selected || !slots || !dst_base || !peer_inbox) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (inbox_rows <= 0) return fail(B200GEMM_ERR_SHAPE, "inbox_rows must be positive");
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return fail(B200GEMM_ERR_SHAPE, "x is not 16-byte aligned");
  if (world < 1 || world > kMoeMaxPeers || experts % world) return fail(B200GEMM_ERR_SHAPE, "bad world / experts");
  if (tokens <= 0 || top_k < 1 || top_k > kMoeMaxTopK || d <= 0 || (d % 8) != 0)
    return fail(B200GEMM_ERR_SHAPE, "need tokens > 0, top_k in [1, %d], d a multiple of 8", kMoeMaxTopK);
  PeerPointers pp = {};
  for (int r = 0; r < world; ++r) {
    if (!peer_inbox[r]) return fail(B200GEMM_ERR_INVALID, "null peer pointer %d", r);
    if ((reinterpret_cast<uintptr_t>(peer_inbox[r]) & 15u) != 0)
      return fail(B200GEMM_ERR_SHAPE, "peer inbox %d is not 16-byte aligned", r);
    pp.ptr[r] = static_cast<uint16_t*>(peer_inbox[r]);
  }
  if (h->exchange_bulk) {
    // A few blocks were asked for: rows travel by bulk asynchronous copies through a
    // shared-memory ring, which fills the links from few SMs (when the ring is deep enough
    // for the batches of stores in flight).
    int top_k_pad = 1;
    while (top_k_pad < top_k) top_k_pad *= 2;
    const int per_batch = 32 / top_k_pad;
    const size_t row_bytes = static_cast<size_t>(d) * 2;
    const size_t fixed = sizeof(PushBulkSmem) + static_cast<size_t>(experts) * sizeof(int);
    const size_t smem_limit = 200 * 1024;
    const int need = (kPushPendingBatches + 2) * per_batch;
    int stages = std::max(32, need);
    if (smem_limit > fixed) stages = static_cast<int>(std::min<size_t>(stages, (smem_limit - fixed) / row_bytes));
    if (stages >= need && stages <= kPushMaxStages) {
      const size_t smem = stages * row_bytes + fixed;
      if (!h->push_bulk_opt_in) {
        CUDA_TRY(cudaFuncSetAttribute(moe_ep_push_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        h->push_bulk_opt_in = true;
      }
      const int bulk_grid = static_cast<int>(std::min<int64_t>(tokens, h->exchange_ctas));
      moe_ep_push_bulk_kernel<<<bulk_grid, 64, smem, static_cast<cudaStream_t>(stream)>>>(
          static_cast<const uint16_t*>(x), selected, slots, dst_base, pp, experts, experts / world, tokens, top_k,
          top_k_pad, d, inbox_rows, stages, h->status);
      CUDA_TRY(cudaGetLastError());
      return B200GEMM_OK;
    }
  }
  // Two 256-thread CTAs per SM at most: the link, not the SMs, bounds this kernel, and a
  // persistent GEMM CTA (224 threads, nearly all shared memory) must still fit beside them.
  const int push_grid = std::min(stream_grid(tokens * 32, h->sm_total), h->exchange_ctas ? h->exchange_ctas : 2 * h->sm_total);
  moe_ep_push_kernel<<<push_grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(x), selected, slots, dst_base, pp, experts / world, tokens, top_k, d,
      inbox_rows, h->status);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_moe_ep_pull_combine(b200gemm_handle_t h, void* stream, void* const* peer_results,
                                 const uint32_t* selected, const uint32_t* slots,
                                 const int32_t* dst_base, const float* gates, const void* residual,
                                 int64_t result_rows, int32_t world, int32_t experts, int64_t tokens,
                                 int32_t top_k, int64_t d, void* out, int32_t out_type) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!peer_results || !selected || !slots || !dst_base || !gates || !out) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (world < 1 || world > kMoeMaxPeers || experts % world) return fail(B200GEMM_ERR_SHAPE, "bad world / experts");
  if (tokens <= 0 || top_k < 1 || top_k > kMoeMaxTopK || d <= 0 || (d % 8) != 0)
    return fail(B200GEMM_ERR_SHAPE, "need tokens > 0, top_k in [1, %d], d a multiple of 8", kMoeMaxTopK);
  if (out_type < 0 || out_type > 1) return fail(B200GEMM_ERR_INVALID, "bad output type");
  if (((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual)) & 15u) != 0)
    return fail(B200GEMM_ERR_SHAPE, "out / residual not 16-byte aligned");
  PeerPointers pp = {};
  for (int r = 0; r < world; ++r) {
    if (!peer_results[r]) return fail(B200GEMM_ERR_INVALID, "null peer pointer %d", r);
    if ((reinterpret_cast<uintptr_t>(peer_results[r]) & 15u) != 0)
      return fail(B200GEMM_ERR_SHAPE, "peer result buffer %d is not 16-byte aligned", r);
    pp.ptr[r] = static_cast<uint16_t*>(peer_results[r]);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (h->exchange_bulk) {
    // A few blocks were asked for: the form that keeps the links busy from few SMs (bulk
    // asynchronous copies into a shared-memory ring), if a token's rows fit the ring twice.
    int top_k_pad = 1;
    while (top_k_pad < top_k) top_k_pad *= 2;
    const size_t stage_bytes = static_cast<size_t>(top_k) * d * 2;
    const size_t fixed = sizeof(PullBulkSmem) + static_cast<size_t>(experts) * sizeof(int);
    const size_t smem_limit = 200 * 1024;
    int stages = stage_bytes > 0 && smem_limit > fixed ? static_cast<int>(std::min<size_t>(8, (smem_limit - fixed) / stage_bytes)) : 0;
    if (stages >= 2) {
      const size_t smem = stages * stage_bytes + fixed;
      const int bulk_grid = static_cast<int>(std::min<int64_t>(tokens, h->exchange_ctas));
      const int which = out_type == B200GEMM_OUT_BF16 ? 1 : 0;
      if (!h->pull_bulk_opt_in[which]) {
        if (which)
          CUDA_TRY(cudaFuncSetAttribute(moe_ep_pull_bulk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        else
          CUDA_TRY(cudaFuncSetAttribute(moe_ep_pull_bulk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        h->pull_bulk_opt_in[which] = true;
      }
      if (which)
        moe_ep_pull_bulk_kernel<true><<<bulk_grid, 32 * (stages + 1), smem, s>>>(
            pp, selected, slots, dst_base, gates, static_cast<const uint16_t*>(residual), experts, experts / world,
            tokens, top_k, top_k_pad, d, result_rows, stages, h->status, out);
      else
        moe_ep_pull_bulk_kernel<false><<<bulk_grid, 32 * (stages + 1), smem, s>>>(
            pp, selected, slots, dst_base, gates, static_cast<const uint16_t*>(residual), experts, experts / world,
            tokens, top_k, top_k_pad, d, result_rows, stages, h->status, out);
      CUDA_TRY(cudaGetLastError());
      return B200GEMM_OK;
    }
  }
  const int grid = std::min(stream_grid(tokens * 32, h->sm_total),
                            h->exchange_ctas ? h->exchange_ctas : 2 * h->sm_total);   // see b200gemm_moe_ep_push
  if (out_type == B200GEMM_OUT_BF16)
    moe_ep_pull_combine_kernel<true><<<grid, 256, 0, s>>>(pp, selected, slots, dst_base, gates,
                                                          static_cast<const uint16_t*>(residual), experts / world,
                                                          tokens, top_k, d, result_rows, h->status, out);
  else
    moe_ep_pull_combine_kernel<false><<<grid, 256, 0, s>>>(pp, selected, slots, dst_base, gates,
                                                           static_cast<const uint16_t*>(residual), experts / world,
                                                           tokens, top_k, d, result_rows, h->status, out);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_grouped_gemm_act_backward(b200gemm_handle_t h, void* stream, const void* a, int64_t lda,
                                       const void* b, int32_t b_layout, int64_t ldb, int64_t batch_stride_b,
                                       int32_t b_count, const int32_t* group_b_index, int32_t activation,
                                       const void* saved, int64_t ld_saved, void* d_saved, int64_t ld_dsaved,
                                       const int32_t* offsets, int32_t groups, int64_t total_rows, int64_t n,
                                       int64_t k) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (activation != 1 && activation != 2) return fail(B200GEMM_ERR_INVALID, "activation is 1 (SiLU) or 2 (SwiGLU)");
  if (group_b_index && b_count < 1) return fail(B200GEMM_ERR_SHAPE, "b_count must be positive with a group index");
  return grouped_gemm(h, static_cast<cudaStream_t>(stream), a, lda, b, b_layout, ldb, batch_stride_b, d_saved,
                      ld_dsaved, offsets, groups, total_rows, n, k, activation + 2, group_b_index, b_count, nullptr,
                      0, saved, ld_saved);
}

int b200gemm_grouped_wgrad(b200gemm_handle_t h, void* stream, const void* a, int64_t lda, const void* b,
                           int64_t ldb, float* c, int64_t ldc, int64_t batch_stride_c, int32_t c_count,
                           const int32_t* group_c_index, const int32_t* offsets, int32_t groups,
                           int64_t total_rows, int64_t m, int64_t n, int32_t accumulate) {
  int rc = check_handle(h);
  if (rc) return rc;
  return grouped_wgrad(h, static_cast<cudaStream_t>(stream), a, lda, b, ldb, c, ldc, batch_stride_c, c_count,
                       group_c_index, offsets, groups, total_rows, m, n, accumulate);
}

int b200gemm_grouped_gemm_silu(b200gemm_handle_t h, void* stream, const void* a, int64_t lda, const void* b,
                               int32_t b_layout, int64_t ldb, int64_t batch_stride_b, int32_t b_count,
                               const int32_t* group_b_index, void* y, int64_t ldy, void* before,
                               int64_t ld_before, const int32_t* offsets, int32_t groups, int64_t total_rows,
                               int64_t n, int64_t k) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (group_b_index && b_count < 1) return fail(B200GEMM_ERR_SHAPE, "b_count must be positive with a group index");
  return grouped_gemm(h, static_cast<cudaStream_t>(stream), a, lda, b, b_layout, ldb, batch_stride_b, y, ldy,
                      offsets, groups, total_rows, n, k, 1, group_b_index, b_count, before, ld_before);
}

int b200gemm_moe_combine_backward(b200gemm_handle_t h, void* stream, const void* dy, int32_t dy_type,
                                  const void* y_permuted, const uint32_t* dest_row, const float* gates,
                                  int64_t tokens, int32_t top_k, int64_t d, void* dy_permuted,
                                  float* gate_grad) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!dy || !dest_row || !gates || !dy_permuted) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if ((gate_grad != nullptr) != (y_permuted != nullptr))
    return fail(B200GEMM_ERR_INVALID, "y_permuted and gate_grad go together");
  if (dy_type < 0 || dy_type > 1) return fail(B200GEMM_ERR_INVALID, "bad dy type");
  if (tokens <= 0 || top_k < 1 || top_k > kMoeMaxTopK || d <= 0 || (d % 8) != 0)
    return fail(B200GEMM_ERR_SHAPE, "need tokens > 0, top_k in [1, %d], d a multiple of 8", kMoeMaxTopK);
  const int grid = stream_grid(tokens * 32, h->sm_count);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dy_type == B200GEMM_OUT_BF16)
    moe_combine_backward_kernel<true><<<grid, 256, 0, s>>>(dy, static_cast<const uint16_t*>(y_permuted), dest_row,
                                                           gates, tokens, top_k, d,
                                                           static_cast<uint16_t*>(dy_permuted), gate_grad);
  else
    moe_combine_backward_kernel<false><<<grid, 256, 0, s>>>(dy, static_cast<const uint16_t*>(y_permuted), dest_row,
                                                            gates, tokens, top_k, d,
                                                            static_cast<uint16_t*>(dy_permuted), gate_grad);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_activation_backward(b200gemm_handle_t h, void* stream, int32_t activation, const void* saved,
                                 int64_t ld_saved, const void* d_y, int64_t ld_dy, int64_t rows, int64_t ff,
                                 void* d_saved, int64_t ld_dsaved) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!saved || !d_y || !d_saved) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (activation != 1 && activation != 2) return fail(B200GEMM_ERR_INVALID, "activation is 1 (SiLU) or 2 (SwiGLU)");
  if (rows <= 0 || ff <= 0 || (ff % 8) != 0) return fail(B200GEMM_ERR_SHAPE, "need rows > 0 and ff a positive multiple of 8");
  const int64_t width = activation == 2 ? 2 * ff : ff;
  ld_saved = ld_saved ? ld_saved : width;
  ld_dsaved = ld_dsaved ? ld_dsaved : width;
  ld_dy = ld_dy ? ld_dy : ff;
  if (ld_saved < width || ld_dsaved < width || ld_dy < ff || (ld_saved % 8) || (ld_dsaved % 8) || (ld_dy % 8))
    return fail(B200GEMM_ERR_SHAPE, "row strides must cover their rows and be multiples of 8");
  if (((reinterpret_cast<uintptr_t>(saved) | reinterpret_cast<uintptr_t>(d_y) | reinterpret_cast<uintptr_t>(d_saved)) & 15u) != 0)
    return fail(B200GEMM_ERR_SHAPE, "buffers must be 16-byte aligned");
  const int grid = stream_grid(rows * (ff / 8), h->sm_count);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (activation == 2)
    activation_backward_kernel<true><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(saved), ld_saved,
                                                          static_cast<const uint16_t*>(d_y), ld_dy, rows, ff,
                                                          static_cast<uint16_t*>(d_saved), ld_dsaved);
  else
    activation_backward_kernel<false><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(saved), ld_saved,
                                                           static_cast<const uint16_t*>(d_y), ld_dy, rows, ff,
                                                           static_cast<uint16_t*>(d_saved), ld_dsaved);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_moe_route_backward(b200gemm_handle_t h, void* stream, const float* probs, const uint32_t* selected,
                                const float* gates, const float* gate_grad, const uint32_t* assignment_counts,
                                float aux_coefficient, int64_t tokens, int32_t experts, int32_t top_k,
                                float* dlogits) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!probs || !selected || !gates || !gate_grad || !assignment_counts || !dlogits)
    return fail(B200GEMM_ERR_INVALID, "null pointer");
  rc = moe_check(tokens, experts, top_k);
  if (rc) return rc;
  const int blocks = static_cast<int>((tokens * 32 + 255) / 256);
  moe_route_backward_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      probs, selected, gates, gate_grad, assignment_counts, aux_coefficient, tokens, experts, top_k, dlogits);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_router_logits(b200gemm_handle_t h, void* stream, const void* x, const float* w, int64_t tokens,
                           int64_t d, int32_t experts, float* logits) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!x || !w || !logits) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (tokens <= 0 || tokens > (1ll << 28) || d <= 0 || d > (1ll << 24))
    return fail(B200GEMM_ERR_SHAPE, "bad token count or width");
  if (experts < 1 || experts > kMoeMaxExperts) return fail(B200GEMM_ERR_SHAPE, "experts must be in [1, %d]", kMoeMaxExperts);
  dim3 grid(static_cast<unsigned>((tokens + 63) / 64), static_cast<unsigned>((experts + 63) / 64));
  router_logits_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(x), w, tokens, static_cast<int>(d), experts, logits);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_loss_mean_with_aux(b200gemm_handle_t h, void* stream, const float* row_loss, int64_t tokens,
                                const float* aux_terms, int32_t aux_count, float coefficient, float* loss) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!row_loss || !loss || (aux_count > 0 && !aux_terms)) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (tokens <= 0 || aux_count < 0) return fail(B200GEMM_ERR_SHAPE, "need tokens > 0 and aux_count >= 0");
  loss_mean_with_aux_kernel<<<1, kLossTailThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      row_loss, tokens, aux_terms, aux_count, coefficient, loss);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_lmhead_ce_merge_shards(b200gemm_handle_t h, void* stream, const float* stats, int32_t world,
                                    int64_t m, float* lse, float* row_loss, float* loss) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!stats || !lse) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (loss && !row_loss) return fail(B200GEMM_ERR_INVALID, "the mean needs row_loss");
  if (world < 1 || world > 64 || m <= 0 || m > (1ll << 30)) return fail(B200GEMM_ERR_SHAPE, "bad world or row count");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ce_merge_shards_kernel<<<stream_grid(m, h->sm_count), 256, 0, s>>>(stats, world, m, lse, row_loss);
  CUDA_TRY(cudaGetLastError());
  if (loss) {
    loss_mean_with_aux_kernel<<<1, kLossTailThreads, 0, s>>>(row_loss, m, nullptr, 0, 0.f, loss);
    CUDA_TRY(cudaGetLastError());
  }
  return B200GEMM_OK;
}

int b200gemm_sum_parts(b200gemm_handle_t h, void* stream, const void* src, int32_t src_type, int64_t part_stride,
                       int32_t parts, int64_t count, void* dst, int32_t dst_type, int32_t max_blocks) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (!src || !dst) return fail(B200GEMM_ERR_INVALID, "null pointer");
  if (src_type < 0 || src_type > 1 || dst_type < 0 || dst_type > 1) return fail(B200GEMM_ERR_INVALID, "bad element type");
  if (parts < 1 || parts > 64 || count <= 0 || (count % 8) != 0 || part_stride < count || (part_stride % 8) != 0)
    return fail(B200GEMM_ERR_SHAPE, "need 1..64 parts, count a positive multiple of 8, part_stride >= count and a multiple of 8");
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) != 0)
    return fail(B200GEMM_ERR_SHAPE, "buffers must be 16-byte aligned");
  int blocks = stream_grid(count / 8, h->sm_total);
  if (max_blocks > 0 && blocks > max_blocks) blocks = max_blocks;
  CUDA_TRY(launch_sum_parts(static_cast<cudaStream_t>(stream), src, part_stride, parts, count, dst,
                            src_type == B200GEMM_OUT_BF16, dst_type == B200GEMM_OUT_BF16, blocks));
  return B200GEMM_OK;
}

int b200gemm_gemm_host(b200gemm_handle_t h, void* stream_, const b200gemm_desc_t* desc) {
  int rc = check_handle(h);
  if (rc) return rc;
  Plan plan;
  rc = make_plan(h, desc, &plan);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  std::lock_guard<std::mutex> lock(h->mu);
  const bool a_mn = desc->a_layout == B200GEMM_MN_MAJOR, b_mn = desc->b_layout == B200GEMM_MN_MAJOR;
  const size_t c_elem = desc->out_type == B200GEMM_OUT_F32 ? 4 : 2;
  // Each matrix as stored: `rows` rows of `width` elements, `ld` elements apart, `batch`
  // matrices `bs` elements apart.  Only the `width` elements of a row belong to the matrix:
  // with ld > width the rest of the row is the caller's (a column slice of a wider matrix),
  // so it is neither read nor written.  The device copies keep the host's strides.
  struct Mat {
    const void* host;
    int64_t rows, width, ld, bs;
    size_t elem;
  };
  const Mat mats[3] = {
      {desc->a, a_mn ? desc->k : desc->m, a_mn ? desc->m : desc->k, plan.lda, plan.bsa, 2},
      {desc->b, b_mn ? desc->k : desc->n, b_mn ? desc->n : desc->k, plan.ldb, plan.bsb, 2},
      {desc->c, desc->m, desc->n, plan.ldc, plan.bsc, c_elem},
  };
  for (int i = 0; i < 3; ++i) {
    const Mat& t = mats[i];
    const size_t bytes = static_cast<size_t>((desc->batch - 1) * t.bs + (t.rows - 1) * t.ld + t.width) * t.elem;
    if (h->stage_bytes[i] < bytes) {
      if (h->stage[i]) CUDA_TRY(cudaFree(h->stage[i]));
      h->stage[i] = nullptr;
      h->stage_bytes[i] = 0;
      CUDA_TRY(cudaMalloc(&h->stage[i], bytes));
      h->stage_bytes[i] = bytes;
    }
  }
  auto copy = [&](int i, cudaMemcpyKind kind) -> cudaError_t {
    const Mat& t = mats[i];
    for (int e = 0; e < desc->batch; ++e) {
      const size_t off = static_cast<size_t>(e) * t.bs * t.elem;
      uint8_t* dev = static_cast<uint8_t*>(h->stage[i]) + off;
      uint8_t* host = static_cast<uint8_t*>(const_cast<void*>(t.host)) + off;
      const size_t pitch = static_cast<size_t>(t.ld) * t.elem;
      cudaError_t err = kind == cudaMemcpyHostToDevice
                            ? cudaMemcpy2DAsync(dev, pitch, host, pitch, t.width * t.elem, t.rows, kind, stream)
                            : cudaMemcpy2DAsync(host, pitch, dev, pitch, t.width * t.elem, t.rows, kind, stream);
      if (err != cudaSuccess) return err;
    }
    return cudaSuccess;
  };
  CUDA_TRY(copy(0, cudaMemcpyHostToDevice));
  CUDA_TRY(copy(1, cudaMemcpyHostToDevice));
  if (desc->mode == B200GEMM_ACCUMULATE) CUDA_TRY(copy(2, cudaMemcpyHostToDevice));
  b200gemm_desc_t dev = *desc;
  dev.a = h->stage[0];
  dev.b = h->stage[1];
  dev.c = h->stage[2];
  rc = launch_gemm(h, stream, &dev);
  if (rc) return rc;
  CUDA_TRY(copy(2, cudaMemcpyDeviceToHost));
  CUDA_TRY(cudaStreamSynchronize(stream));
  return B200GEMM_OK;
}

int b200gemm_wait_selftest(b200gemm_handle_t h, void* stream, int64_t limit_ms) {
  int rc = check_handle(h);
  if (rc) return rc;
  if (limit_ms < 1 || limit_ms > 5000) return fail(B200GEMM_ERR_INVALID, "limit must be 1..5000 ms");
  wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      h->status, static_cast<unsigned long long>(limit_ms) * 1000000ull);
  CUDA_TRY(cudaGetLastError());
  return B200GEMM_OK;
}

int b200gemm_device_status(b200gemm_handle_t h, void* stream, int32_t* device_code) {
  int rc = check_handle(h);
  if (rc) return rc;
  int code = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUDA_TRY(cudaMemcpyAsync(&code, h->status, sizeof(int), cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  if (device_code) *device_code = code;
  if (code != 0) {
    CUDA_TRY(cudaMemsetAsync(h->status, 0, sizeof(int), s));
    {
      // A launch that gave up may have left its tile counters mid-count.
      std::lock_guard<std::mutex> lock(h->sched_mu);
      for (auto& kv : h->sched_counters) CUDA_TRY(cudaMemsetAsync(kv.second, 0, 2 * sizeof(int), s));
    }
    return fail(B200GEMM_ERR_DEVICE,
                "a kernel reported device status %d (101-104, 106, 108: a bounded wait ran out; 105: a row fell "
                "outside an exchange buffer; 107: a cross-entropy target outside [0, classes))",
                code);
  }
  return B200GEMM_OK;
}

}  // extern "C"
