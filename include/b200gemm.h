/*
 * b200gemm: C ABI of the B200-native (sm_100a) GEMM layer.
 *
 * This is the boundary a host program binds to in place of the reference
 * trainer's `Tcgen05Gemm` (gpu/gemm/src/host.rs:469-1098) and of the fp32
 * `GpuTensor::matmul*` family (gpu/tensor-gpu/src/lib.rs:1754-1851).  Plain
 * pointers and sizes only: every pointer named "device" is a CUDA device
 * pointer owned by the caller, `stream` is a `cudaStream_t` passed as `void*`.
 *
 * All launches are asynchronous on `stream`.  Every function returns a
 * `b200gemm_status_t`; nothing aborts the process.  Contract violations that
 * the reference turns into `assert!` panics (host.rs:81-85, 395-400,
 * 1105-1109, 1168-1171) are reported as B200GEMM_ERR_SHAPE / _INVALID.
 *
 * Differences from the reference boundary, on purpose:
 *  - raw device pointers + runtime shapes replace caller-built TMA descriptors
 *    (host.rs:102-465); tensor maps are encoded inside and passed by value;
 *  - shapes need not be multiples of the tile (256, 256, 64): edges are
 *    zero-filled on load and clipped on store by the copy engine.  Leading
 *    dimensions must keep rows 16-byte aligned (multiples of 8 bf16 / 4 fp32);
 *  - either operand may be MN-major independently, so a `[IN, OUT]` weight can
 *    be read in place without a transposed shadow copy;
 *  - split-K for the deep (K = tokens) weight-gradient shapes;
 *  - fused forms the reference runs as separate passes: the lm-head with its classifier
 *    (b200gemm_lmhead_ce_*), SiLU / SwiGLU in the grouped expert GEMM
 *    (b200gemm_grouped_gemm*), the fp32 result with its bf16 copy (b200gemm_gemm_dual);
 *  - tiles handed out from a device-side counter (b200gemm_set_scheduler), and an SM cap
 *    (b200gemm_set_sm_limit), for running beside a collective's kernels.
 */
#ifndef B200GEMM_H_
#define B200GEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200GEMM_API __attribute__((visibility("default")))
#else
#define B200GEMM_API
#endif

typedef struct b200gemm_context* b200gemm_handle_t;

typedef enum {
  B200GEMM_OK = 0,
  B200GEMM_ERR_INVALID = 1,      /* null pointer, bad enum, bad handle */
  B200GEMM_ERR_SHAPE = 2,        /* extents / leading dimensions / alignment outside the contract */
  B200GEMM_ERR_CUDA = 3,         /* a CUDA runtime or driver call failed (see b200gemm_last_error_string) */
  B200GEMM_ERR_UNSUPPORTED = 4,  /* device is not sm_100, or the combination is not implemented */
  B200GEMM_ERR_DEVICE = 5        /* a kernel reported a bounded-wait timeout (b200gemm_device_status) */
} b200gemm_status_t;

/* Operand orientation (gpu/gemm/src/host.rs:112-125 `TmaLayout`). */
typedef enum {
  B200GEMM_K_MAJOR = 0,  /* stored [rows, K], K contiguous   */
  B200GEMM_MN_MAJOR = 1  /* stored [K, rows], rows contiguous */
} b200gemm_layout_t;

typedef enum { B200GEMM_OUT_F32 = 0, B200GEMM_OUT_BF16 = 1 } b200gemm_out_t;
typedef enum { B200GEMM_STORE = 0, B200GEMM_ACCUMULATE = 1 } b200gemm_mode_t;

/* flags */
#define B200GEMM_FLAG_CTA_GROUP_1 0x1u /* force one-CTA 128x256 tiles               */
#define B200GEMM_FLAG_CTA_GROUP_2 0x2u /* force CTA-pair 256x256 tiles (cta_group::2) */
#define B200GEMM_FLAG_WIDE_TILE   0x4u /* force 256x512 tiles per CTA pair (fp32 output; chosen by itself for deep reductions) */
#define B200GEMM_FLAG_NARROW_TILE 0x8u /* never use 256x512 tiles */

/*
 * One launch: for e in [0, batch):  C[e][m, n] (=|+=) A[e] * B[e]^T
 *   a_layout == K_MAJOR : A[e] is [m, k] with row stride lda;  MN_MAJOR : [k, m] with row stride lda
 *   b_layout == K_MAJOR : B[e] is [n, k] with row stride ldb;  MN_MAJOR : [k, n] with row stride ldb
 *   C[e] is [m, n] row-major with row stride ldc; fp32, or bf16 rounded to nearest even.
 * Inputs are bf16; products are accumulated in fp32.
 * Leading dimensions and batch strides are in elements; 0 means "dense".
 *
 * Covers one-for-one (gpu/gemm/src/host.rs):
 *   store :616  store_batched :658  accumulate :695  accumulate_transposed :875
 *   f32_store :729  f32_store_at :766  f32_store_batched :957  f32_store_transposed :1039
 *   f32_accumulate :802  f32_accumulate_at :837  f32_accumulate_transposed(_at) :1074/:914
 *   f32_accumulate_transposed_batched :997
 * (`_at` = pass `c` already offset; `_batched` = batch > 1.)
 */
typedef struct {
  const void* a;   /* device, bf16 */
  const void* b;   /* device, bf16 */
  void* c;         /* device, fp32 or bf16 */
  int64_t m, n, k;
  int64_t lda, ldb, ldc;
  int32_t a_layout, b_layout; /* b200gemm_layout_t */
  int32_t out_type;           /* b200gemm_out_t    */
  int32_t mode;               /* b200gemm_mode_t   */
  int32_t batch;              /* >= 1 ("experts", host.rs:658-687) */
  int32_t split_k;            /* 0 = choose; 1 = none; >1 = that many K slices (fp32 output only) */
  int64_t batch_stride_a, batch_stride_b, batch_stride_c;
  uint32_t flags;
  uint32_t reserved;
} b200gemm_desc_t;

/* Replaces Tcgen05Gemm::load (host.rs:508-530).  Creates per-device state on
 * CUDA device `device`: opts kernels into large dynamic shared memory and
 * allocates the 4-byte device status word.  Fails with ERR_UNSUPPORTED on a
 * device that is not compute capability 10.x. */
B200GEMM_API int b200gemm_create(int device, b200gemm_handle_t* out);
B200GEMM_API int b200gemm_destroy(b200gemm_handle_t h);

/* Caps the number of SMs the persistent kernels of later launches occupy
 * (0 or a value above the device's SM count restores all of them).  New: lets a
 * caller keep a few SMs free for a collective's kernels that must run at the
 * same time, since a persistent grid would otherwise hold every SM until it ends. */
B200GEMM_API int b200gemm_set_sm_limit(b200gemm_handle_t h, int32_t sms);

/* Thread blocks of the expert exchange's dispatch and combine kernels (b200gemm_moe_ep_push,
 * b200gemm_moe_ep_pull_combine) of later launches; 0 restores the default of two 256-thread
 * blocks per SM.  New: those kernels are bound by the links between the GPUs, not by the SMs,
 * and run beside the expert GEMMs -- fewer blocks take less from the GEMM.
 *   bulk = 0  the store- / load-driven kernels with `ctas` blocks
 *   bulk = 1  rows move by bulk asynchronous copies through a ring in shared memory (two
 *             warps per block dispatch, nine combine); the results are bit-identical
 */
B200GEMM_API int b200gemm_set_exchange_ctas(b200gemm_handle_t h, int32_t ctas, int32_t bulk);

/* How the persistent kernels of later launches hand out their tiles.
 *   0  static: cluster c takes items c, c + clusters, ...  (the reference's walk,
 *      gpu/gemm/src/optimized.rs:776-802)
 *   1  dynamic (the default for 2-CTA launches): every cluster takes its next item from a
 *      counter in device memory.  Same items, same order of hand-out; but a cluster that
 *      runs slower or becomes resident late -- another kernel, e.g. a collective's, held
 *      its SMs -- simply takes fewer items instead of running a fixed share as a second
 *      wave.  Uses 8 bytes of device memory per stream, allocated (cudaMalloc) at the first
 *      launch on that stream: make that launch outside a stream capture, or choose 0.  A
 *      captured graph keeps the counters of the stream it was captured on, so two replays of
 *      one such graph must not run at the same time.
 * Results are the same either way except where a launch reduce-adds split-K slices, whose
 * order of arrival in memory is not fixed in either mode.
 * b200gemm_lmhead_ce_forward_noalloc always uses the static walk. */
B200GEMM_API int b200gemm_set_scheduler(b200gemm_handle_t h, int32_t mode);

/* The tcgen05 GEMM (host.rs:616-1098, kernels gpu/gemm/src/optimized.rs:1138-1268). */
B200GEMM_API int b200gemm_gemm(b200gemm_handle_t h, void* stream, const b200gemm_desc_t* desc);

/* b200gemm_gemm as an fp32 store that ALSO writes the result rounded to bf16 (nearest even)
 * into c_bf16 [m, n] (row stride ldc_bf16 elements, 0 = n; per-batch stride
 * batch_stride_c_bf16, 0 = dense): the packed operand copy the next GEMM reads, produced by
 * the kernel that computes it.  Replaces `f32_store` followed by
 * `convert_f32_to_bf16_pairs` (gpu/model/src/lib.rs:1194-1199; gpu/tensor-gpu/src/lib.rs:322-326).
 * desc->out_type must be F32, desc->mode STORE; K is not split. */
B200GEMM_API int b200gemm_gemm_dual(b200gemm_handle_t h, void* stream, const b200gemm_desc_t* desc,
                                    void* c_bf16, int64_t ldc_bf16, int64_t batch_stride_c_bf16);

/* The launch geometry b200gemm_gemm would use (tcgen05_launch_config,
 * host.rs:47-94): grid, cluster size (1 or 2), dynamic shared memory, chosen
 * split-K.  Any output pointer may be NULL. */
B200GEMM_API int b200gemm_launch_config(b200gemm_handle_t h, const b200gemm_desc_t* desc,
                                        int32_t* grid, int32_t* cluster, int32_t* smem_bytes,
                                        int32_t* split_k);

/*
 * fp32 CUDA-core GEMM family for fp32 operands and arbitrary shapes
 * (gpu/gemm/src/fp32.rs:141-191 register_gemm_{store,accumulate,nt_store,
 * tn_accumulate}; gpu/tensor-gpu/src/lib.rs:1754-1851 GpuTensor::matmul,
 * matmul_nt, matmul_tn).  All matrices dense row-major fp32.
 *   op 0 (NN): C[m,n] = A[m,k] B[k,n]
 *   op 1 (NT): C[m,n] = A[m,k] B[n,k]^T
 *   op 2 (TN): C[m,n] = A[k,m]^T B[k,n]
 * accumulate != 0 adds into C.
 */
typedef enum { B200GEMM_OP_NN = 0, B200GEMM_OP_NT = 1, B200GEMM_OP_TN = 2 } b200gemm_op_t;
B200GEMM_API int b200gemm_sgemm(b200gemm_handle_t h, void* stream, int32_t op, int32_t accumulate,
                                const float* a, const float* b, float* c, int64_t m, int64_t n,
                                int64_t k);

/* Staging converts and the packed transpose the GEMM callers use
 * (gpu/tensor-gpu/src/lib.rs:403-413 convert_f32_to_bf16_pairs, :420-450
 * convert_bf16_pairs_to_f32, :457-507 transpose_bf16_pairs).  `count` in
 * elements; bf16 is round-to-nearest-even. */
B200GEMM_API int b200gemm_convert_f32_to_bf16(b200gemm_handle_t h, void* stream, const float* src,
                                              void* dst_bf16, int64_t count);
B200GEMM_API int b200gemm_convert_bf16_to_f32(b200gemm_handle_t h, void* stream,
                                              const void* src_bf16, float* dst, int64_t count);
/* dst[cols, rows] = src[rows, cols]^T, bf16. */
B200GEMM_API int b200gemm_transpose_bf16(b200gemm_handle_t h, void* stream, const void* src,
                                         void* dst, int64_t rows, int64_t cols);

/*
 * Host-buffer form of b200gemm_gemm for callers that hold their matrices in
 * host memory: copies A and B to the device, runs the GEMM, copies C back, and
 * synchronises `stream`.  With mode == ACCUMULATE the host C is copied in
 * first.  The device staging buffers belong to the handle and grow on demand.
 */
B200GEMM_API int b200gemm_gemm_host(b200gemm_handle_t h, void* stream, const b200gemm_desc_t* desc);

/*
 * lm-head GEMM fused with the softmax cross-entropy classifier.
 *
 * Replaces, in the reference, GpuBf16Head::forward_into + cross_entropy_into
 * (gpu/model/src/lib.rs:3076-3096, 6977-7013: a bf16 `store` of the [m, v]
 * logits followed by fused_classifier_forward_bf16 and loss_mean_with_aux,
 * gpu/ops/src/lib.rs:1721-1829, 2852-2904).  Here the logits
 *     logits[m, v] = hidden[m, k] . W
 * live only in tensor memory: the GEMM's epilogue keeps a running (max,
 * sum-exp) per row, so the [m, v] matrix is never written to HBM.
 *
 *   hidden    device bf16 [m, k], row stride k
 *   weight    device bf16; w_layout == B200GEMM_MN_MAJOR: stored [k, v] (the
 *             reference's [IN, OUT] master), == B200GEMM_K_MAJOR: stored [v, k]
 *   targets   device int32 [m], each in [0, classes) (crates/nn/src/cross_entropy.rs:38 asserts
 *             it); a row whose target is outside gets a NaN loss -- so the mean is NaN -- and
 *             device status 107 is recorded (b200gemm_device_status)
 *   v         padded vocabulary (row stride of a [k, v] weight); columns at or
 *             beyond `classes` are ignored (gpu/ops/src/lib.rs:1721-1829)
 *   lse       device fp32 [m] out: max + ln(sum exp) per row (input of backward)
 *   row_loss  device fp32 [m] out, may be NULL: lse - logit[target]
 *   loss      device fp32 [1] out, may be NULL: mean of row_loss (f64 row sum)
 *   workspace device scratch of at least b200gemm_lmhead_ce_workspace_bytes(m)
 *             bytes, 256-byte aligned; contents need not be preserved between calls
 */
B200GEMM_API size_t b200gemm_lmhead_ce_workspace_bytes(int64_t m);
B200GEMM_API int b200gemm_lmhead_ce_forward(b200gemm_handle_t h, void* stream, const void* hidden,
                                            const void* weight, int32_t w_layout,
                                            const int32_t* targets, int64_t m, int64_t k, int64_t v,
                                            int64_t classes, float* lse, float* row_loss,
                                            float* loss, void* workspace, size_t workspace_bytes);

/*
 * One vocabulary shard of b200gemm_lmhead_ce_forward (new: the reference is
 * single-GPU).  `weight_shard` holds `v_local` columns of the vocabulary, of
 * which the first `classes_local` are real; `local_targets[r]` is the row's
 * target minus the shard's first column, so a target owned by another shard is
 * simply out of [0, classes_local).  Outputs per row, device fp32 [m]:
 *   row_max          max over the shard's real columns
 *   row_sum          sum of exp(logit - row_max) over them
 *   row_target_logit the target's logit if this shard owns it, else 0
 * The caller merges shards: M = max_s row_max; S = sum_s row_sum * exp(row_max - M);
 * lse = M + ln S; loss = lse - sum_s row_target_logit.  Workspace as above.
 */
B200GEMM_API int b200gemm_lmhead_ce_forward_shard(b200gemm_handle_t h, void* stream,
                                                  const void* hidden, const void* weight_shard,
                                                  int32_t w_layout, const int32_t* local_targets,
                                                  int64_t m, int64_t k, int64_t v_local,
                                                  int64_t classes_local, float* row_max,
                                                  float* row_sum, float* row_target_logit,
                                                  void* workspace, size_t workspace_bytes);

/*
 * Merge of the shards' statistics into the global result (the formula above), one launch
 * for all rows instead of a chain of elementwise passes between two all-reduces:
 *   stats   device fp32 [world][3][m]: every shard's row_max, row_sum, row_target_logit
 *           (three consecutive [m] arrays per shard, i.e. what one all-gather of each rank's
 *           [3][m] block produces)
 *   lse, row_loss (may be NULL), loss (may be NULL; needs row_loss): as b200gemm_lmhead_ce_forward
 * New: the reference is single-GPU.
 */
B200GEMM_API int b200gemm_lmhead_ce_merge_shards(b200gemm_handle_t h, void* stream, const float* stats,
                                                 int32_t world, int64_t m, float* lse, float* row_loss,
                                                 float* loss);

/*
 * b200gemm_lmhead_ce_forward for callers that cannot hand the library a
 * workspace.  This entry point has no counterpart in the reference.
 *
 * Who needs it: a trainer that reserves all of HBM for its own arena at
 * start-up and therefore has nothing left to cudaMalloc from, or a step loop
 * that must not call cudaMalloc / cudaFree at all because those calls
 * synchronise the whole device.  For them the per-row softmax statistics go to
 * a fixed array that is part of the library image (about 2.1 MiB of every GPU
 * the library is loaded on, held until the process exits) instead of a
 * caller-provided workspace.  Same arguments and results as
 * b200gemm_lmhead_ce_forward otherwise; this call itself never allocates or
 * frees device or pinned memory.
 *
 * Limits and rules:
 *   - m <= 32768 rows; larger m is refused with B200GEMM_ERR_SHAPE.
 *   - The handle's device must be current on the calling thread at every call
 *     (checked; B200GEMM_ERR_INVALID otherwise).
 *   - The first call on a device looks up the array's device address.  Make
 *     that first call before any stream capture is begun on that device; later
 *     calls only launch kernels.  With lazy module loading the driver may give
 *     the array its memory only at that first call, so a host that is about to
 *     claim all of HBM for its arena makes one warm-up call BEFORE it does so.
 *   - All calls on one device share the one array: two calls whose kernels can
 *     overlap on the GPU (different streams, no ordering between them) race on
 *     it and corrupt each other's loss.  Order them on one stream or with events.
 *   - The array keeps whatever the previous call left in it; the entry point
 *     re-zeroes the part that must start at zero (the loss accumulator) itself.
 */
B200GEMM_API int b200gemm_lmhead_ce_forward_noalloc(b200gemm_handle_t h, void* stream,
                                                    const void* hidden, const void* weight,
                                                    int32_t w_layout, const int32_t* targets,
                                                    int64_t m, int64_t k, int64_t v, int64_t classes,
                                                    float* lse, float* row_loss, float* loss);

/*
 * Backward of the above (reference: fused_classifier_backward_in_place_bf16 +
 * GpuBf16Head::backward_weight / backward_input, gpu/ops/src/lib.rs:1843-2001,
 * gpu/model/src/lib.rs:3103-3145, 5750-5784).  The logits are recomputed tile
 * by tile and turned in the GEMM's epilogue into
 *     dlogits = (dy / m) * (exp(logit - lse) - onehot(target)),  0 in padded columns
 * written once as bf16 [m, v] (`dlogits`, caller-provided); then
 *     d_hidden[m, k] (fp32)  =  dlogits . W^T
 *     d_weight (fp32, same shape as W)  (=|+=)  hidden^T . dlogits
 * `accumulate_dw` != 0 adds into d_weight.  `d_hidden` or `d_weight` may be NULL
 * to skip that product.
 */
B200GEMM_API int b200gemm_lmhead_ce_backward(b200gemm_handle_t h, void* stream, const void* hidden,
                                             const void* weight, int32_t w_layout,
                                             const int32_t* targets, const float* lse, float dy,
                                             int64_t m, int64_t k, int64_t v, int64_t classes,
                                             void* dlogits_bf16, float* d_hidden, float* d_weight,
                                             int32_t accumulate_dw);

/*
 * Grouped ("ragged") expert GEMM over a routed token permutation (new: the
 * reference multiplies fixed-capacity bins, dead rows included,
 * gpu/model/src/lib.rs:1717-1748, 1913-2154).
 *
 *   for g in [0, groups):  rows r in [offsets[g], offsets[g+1])
 *       C[r, 0:n] = act( A[r, 0:k] . B[g]^T )            bf16 out, fp32 accumulate
 *
 *   a        device bf16 [total_rows, k], row stride lda (0 = k)
 *   b        device bf16, `groups` matrices `batch_stride_b` elements apart
 *            (0 = dense): b_layout K_MAJOR [n, k] or MN_MAJOR [k, n], row stride ldb
 *   c        device bf16 [total_rows, n], row stride ldc (0 = n; multiple of 8)
 *   offsets  DEVICE int32 [groups + 1], non-decreasing, offsets[groups] <= total_rows
 *            (the expert offsets the router produces; never read on the host)
 *   activation 0 = none, 1 = SiLU x*sigmoid(x) (crates/nn/src/swiglu.rs:22-28),
 *              2 = SwiGLU: every B matrix holds 2*n columns, [gate(n) | up(n)], and
 *                  C[rows, n] = silu(gate) * up (see b200gemm_grouped_gemm_swiglu)
 * Rows of C outside every group are left untouched.  groups <= 192.
 */
B200GEMM_API int b200gemm_grouped_gemm(b200gemm_handle_t h, void* stream, const void* a, int64_t lda,
                                       const void* b, int32_t b_layout, int64_t ldb,
                                       int64_t batch_stride_b, void* c, int64_t ldc,
                                       const int32_t* offsets, int32_t groups, int64_t total_rows,
                                       int64_t n, int64_t k, int32_t activation);

/* b200gemm_grouped_gemm where group g multiplies B[group_b_index[g]] (device int32
 * [groups], values in [0, b_count)) instead of B[g]: lets rows that arrive from
 * several ranks, each run sorted by local expert, be multiplied in place without
 * re-sorting them (one group per (source rank, local expert)). */
B200GEMM_API int b200gemm_grouped_gemm_indexed(b200gemm_handle_t h, void* stream, const void* a,
                                               int64_t lda, const void* b, int32_t b_layout,
                                               int64_t ldb, int64_t batch_stride_b, int32_t b_count,
                                               const int32_t* group_b_index, void* c, int64_t ldc,
                                               const int32_t* offsets, int32_t groups,
                                               int64_t total_rows, int64_t n, int64_t k,
                                               int32_t activation);

/*
 * The gate/up product of a gated MLP fused with its activation.  Replaces the pair
 * "fused gate/up GEMM into a [rows, 2, ff] panel" + `swiglu_forward_interleaved_packed`
 * (gpu/model/src/lib.rs:1913-2154 expert_linear_forward over `[E,D,2,FF]` weights;
 * gpu/ops/src/lib.rs:1149-1222): every B matrix is [k, 2*ff] (MN-major, the
 * reference's `[D, 2, FF]`) or [2*ff, k] (K-major), gate block first, and
 *   y[rows, ff] = silu(gate) * up            (bf16; the activation is applied to the
 *                                             fp32 accumulators, so the panel's bf16
 *                                             rounding is not in y)
 *   gate_up[rows, 2*ff] = [gate | up]        (bf16, optional: NULL skips it; it is what
 *                                             the backward of the activation reads)
 * in ONE launch: the panel is never read back.  Groups and `group_b_index` (NULL =
 * group g uses B[g], then b_count is ignored) as in b200gemm_grouped_gemm_indexed;
 * one group with offsets {0, rows} is the dense gated MLP.  ff % 8 == 0, and
 * ff % 64 == 0 when the panel is written; ldy, ld_gate_up in elements (0 = packed).
 */
B200GEMM_API int b200gemm_grouped_gemm_swiglu(b200gemm_handle_t h, void* stream, const void* a,
                                              int64_t lda, const void* b, int32_t b_layout,
                                              int64_t ldb, int64_t batch_stride_b, int32_t b_count,
                                              const int32_t* group_b_index, void* y, int64_t ldy,
                                              void* gate_up, int64_t ld_gate_up,
                                              const int32_t* offsets, int32_t groups,
                                              int64_t total_rows, int64_t ff, int64_t k);

/*
 * b200gemm_grouped_gemm with activation 1 (SiLU) that can also keep what the activation
 * was applied to: before[rows, n] (bf16, row stride ld_before, 0 = n; NULL skips it) gets
 * A . B^T rounded to bf16, y[rows, n] gets silu of the fp32 product.  `before` is what
 * b200gemm_activation_backward reads.  group_b_index / b_count as in
 * b200gemm_grouped_gemm_indexed (NULL = group g uses B[g]).  New: the reference's expert
 * is the gated form (b200gemm_grouped_gemm_swiglu).
 */
B200GEMM_API int b200gemm_grouped_gemm_silu(b200gemm_handle_t h, void* stream, const void* a,
                                            int64_t lda, const void* b, int32_t b_layout, int64_t ldb,
                                            int64_t batch_stride_b, int32_t b_count,
                                            const int32_t* group_b_index, void* y, int64_t ldy,
                                            void* before, int64_t ld_before, const int32_t* offsets,
                                            int32_t groups, int64_t total_rows, int64_t n, int64_t k);

/*
 * The input-gradient GEMM of an expert linear with the backward of the activation in front of
 * it fused into its epilogue: replaces `f32_store_batched` + `swiglu_backward_interleaved_packed`
 * (gpu/model/src/lib.rs:2335-2400), i.e. b200gemm_grouped_gemm + b200gemm_activation_backward,
 * without the [rows, n] intermediate and with one rounding instead of two.
 *   d_y[rows, n] = A[rows, k] . B[g]^T                          (fp32, never stored)
 *   activation 1 (SiLU):   d_saved[rows, n]    = d_y * silu'(saved),      saved [rows, n]
 *   activation 2 (SwiGLU): d_saved[rows, 2, n] = {d_y * up * silu'(gate), d_y * silu(gate)},
 *                          saved = the [rows, 2, n] gate/up panel; n % 64 == 0
 * Row strides in elements (0 = packed); n % 8 == 0.  Groups, B and `group_b_index` as in
 * b200gemm_grouped_gemm_indexed (NULL = group g uses B[g]).
 */
B200GEMM_API int b200gemm_grouped_gemm_act_backward(b200gemm_handle_t h, void* stream, const void* a,
                                                    int64_t lda, const void* b, int32_t b_layout,
                                                    int64_t ldb, int64_t batch_stride_b, int32_t b_count,
                                                    const int32_t* group_b_index, int32_t activation,
                                                    const void* saved, int64_t ld_saved, void* d_saved,
                                                    int64_t ld_dsaved, const int32_t* offsets,
                                                    int32_t groups, int64_t total_rows, int64_t n,
                                                    int64_t k);

/*
 * Weight gradients of the expert linears over the routed permutation: the row groups are
 * the REDUCTION axis.
 *
 *   for g in [0, groups):  C[i(g)] [m, n] (=|+=) A[rows_g, 0:m]^T . B[rows_g, 0:n]
 *                          rows_g = [offsets[g], offsets[g+1]),  i(g) = group_c_index ? group_c_index[g] : g
 *
 * Replaces f32_accumulate_transposed_batched over capacity bins
 * (gpu/gemm/src/host.rs:997-1026 as called from expert_linear_backward,
 * gpu/model/src/lib.rs:2011-2055): here a group contributes exactly its own rows, not a
 * bin padded to capacity.
 *   a        device bf16 [total_rows, m], row stride lda (0 = m): the expert linear's input rows
 *   b        device bf16 [total_rows, n], row stride ldb (0 = n): the gradient of its output rows
 *   c        device fp32, c_count (or `groups`) matrices [m, n], row stride ldc (0 = n),
 *            batch_stride_c elements apart (0 = dense)
 *   offsets  DEVICE int32 [groups + 1], as b200gemm_grouped_gemm; groups <= 192
 *   accumulate != 0 adds into C; 0 overwrites it (C is cleared first; an empty group
 *            leaves its matrix zero).  Several groups may share one matrix (rows received
 *            from several ranks for the same expert).
 * Long groups are cut into chunks of a few thousand rows that different CTA pairs multiply
 * at the same time and add into C with the copy engine's fp32 reduction, so a hot expert
 * does not serialise on one pair; the order of those additions is not fixed.
 */
B200GEMM_API int b200gemm_grouped_wgrad(b200gemm_handle_t h, void* stream, const void* a, int64_t lda,
                                        const void* b, int64_t ldb, float* c, int64_t ldc,
                                        int64_t batch_stride_c, int32_t c_count,
                                        const int32_t* group_c_index, const int32_t* offsets,
                                        int32_t groups, int64_t total_rows, int64_t m, int64_t n,
                                        int32_t accumulate);

/*
 * Backward of b200gemm_moe_combine (crates/nn/src/moe.rs:360-381): for every accepted
 * (token, rank) pair
 *   dy_permuted[dest_row, :] = gate * dy[token, :]                         bf16
 *   gate_grad[pair] = sum_d y_permuted[dest_row, d] * dy[token, d]         fp32; 0 for a dropped pair
 * dy is [tokens, d] fp32 or bf16 (dy_type: b200gemm_out_t).  y_permuted (the expert outputs
 * the forward combined) and gate_grad may both be NULL when the router is not trained.
 * Rows of dy_permuted that no pair maps to are left untouched.
 */
B200GEMM_API int b200gemm_moe_combine_backward(b200gemm_handle_t h, void* stream, const void* dy,
                                               int32_t dy_type, const void* y_permuted,
                                               const uint32_t* dest_row, const float* gates,
                                               int64_t tokens, int32_t top_k, int64_t d,
                                               void* dy_permuted, float* gate_grad);

/*
 * Backward of the expert's activation over the routed rows, bf16 in and out.
 *   activation 1 (SiLU, y = silu(a)):       saved = a [rows, ff] (b200gemm_grouped_gemm_silu's
 *       `before`), d_saved[rows, ff] = d_y * s * (1 + a * (1 - s)), s = sigmoid(a)
 *   activation 2 (SwiGLU, y = silu(g) * u): saved = the [rows, 2, ff] gate/up panel
 *       (b200gemm_grouped_gemm_swiglu's `gate_up`), d_saved likewise:
 *       d_g = d_y * u * s * (1 + g * (1 - s)),  d_u = d_y * g * s
 *       (crates/nn/src/swiglu.rs:30-47; gpu/ops/src/lib.rs:1453 swiglu_backward_interleaved_packed)
 * Row strides in elements, 0 = packed; ff % 8 == 0.  d_saved may alias d_y only for SiLU.
 */
B200GEMM_API int b200gemm_activation_backward(b200gemm_handle_t h, void* stream, int32_t activation,
                                              const void* saved, int64_t ld_saved, const void* d_y,
                                              int64_t ld_dy, int64_t rows, int64_t ff, void* d_saved,
                                              int64_t ld_dsaved);

/*
 * Backward of the routing (crates/nn/src/moe.rs:397-445): from the gradients of the combine
 * weights to the gradient of the router's logits, fp32 [tokens, experts].
 *   probs    the router's softmax (the `scores` b200gemm_moe_route selected from)
 *   gate_grad from b200gemm_moe_combine_backward; aux_coefficient weighs the load-balancing
 *   term experts * fraction[e] / tokens, fraction[e] = assignment_counts[e] / (tokens * top_k).
 */
B200GEMM_API int b200gemm_moe_route_backward(b200gemm_handle_t h, void* stream, const float* probs,
                                             const uint32_t* selected, const float* gates,
                                             const float* gate_grad, const uint32_t* assignment_counts,
                                             float aux_coefficient, int64_t tokens, int32_t experts,
                                             int32_t top_k, float* dlogits);

/*
 * Router logits (gpu/ops/src/lib.rs:2319-2429 router_logits_bf16, whose ROUTER_MAX_EXPERTS
 * is 8): logits[tokens, experts] = x[tokens, d] (bf16) . w[d, experts] (fp32), experts <= 256.
 * fp32 arithmetic on CUDA cores, products rounded and added in ascending k: the CPU
 * router's own sums (crates/nn/src/moe.rs:290 `self.router.forward`), bit for bit, so
 * that expert selection cannot differ from the reference's on near-ties.
 */
B200GEMM_API int b200gemm_router_logits(b200gemm_handle_t h, void* stream, const void* x, const float* w,
                                        int64_t tokens, int64_t d, int32_t experts, float* logits);

/*
 * The scalar training loss (gpu/ops/src/lib.rs:2852-2904 loss_mean_with_aux):
 *   loss[0] = mean(row_loss[0:tokens]) + coefficient * sum(aux_terms[0:aux_count])
 * row_loss as written by b200gemm_lmhead_ce_forward; aux_terms one per MoE layer (device
 * fp32, may be NULL with aux_count 0).  The token sum is carried in f64.
 */
B200GEMM_API int b200gemm_loss_mean_with_aux(b200gemm_handle_t h, void* stream, const float* row_loss,
                                             int64_t tokens, const float* aux_terms, int32_t aux_count,
                                             float coefficient, float* loss);

/*
 * MoE routing integers and gates (crates/nn/src/moe.rs:205-254 `MoeFfn::route`;
 * GPU counterparts gpu/ops/src/lib.rs:2435-2511 router_softmax_topk, :2569-2705
 * moe_bin_assign_parallel).  All pointers are device pointers.
 *   scores   fp32 [tokens, experts]: probabilities (scores_are_logits = 0) or raw
 *            router logits (!= 0); selection order is by descending score, ties to
 *            the lower expert index
 *   selected uint32 [tokens*top_k]        gates fp32 [tokens*top_k]
 *   slots    uint32 [tokens*top_k]: arrival order within the expert in flattened
 *            (token, rank) order; 0xFFFFFFFF when the expert was at `capacity`
 *   assignment_counts, accepted_counts uint32 [experts]
 *   offsets  int32 [experts + 1]: exclusive prefix sum of accepted_counts
 *   dest_row uint32 [tokens*top_k]: offsets[selected] + slot (0xFFFFFFFF if dropped)
 * experts <= 256, top_k <= 16 and <= experts.  Integer outputs are bit-exact
 * with the reference's CPU router; so are the gates when scores are probabilities.
 */
B200GEMM_API int b200gemm_moe_route(b200gemm_handle_t h, void* stream, const float* scores,
                                    int32_t scores_are_logits, int64_t tokens, int32_t experts,
                                    int32_t top_k, int64_t capacity, uint32_t* selected, float* gates,
                                    uint32_t* slots, uint32_t* assignment_counts,
                                    uint32_t* accepted_counts, int32_t* offsets, uint32_t* dest_row);

/* Dispatch (gpu/ops/src/lib.rs:2913-2953 moe_scatter_packed_quad):
 * x_permuted[dest_row[t*top_k + r], :] = x[t, :], bf16, d a multiple of 8. */
B200GEMM_API int b200gemm_moe_scatter(b200gemm_handle_t h, void* stream, const void* x,
                                      const uint32_t* dest_row, int64_t tokens, int32_t top_k,
                                      int64_t d, void* x_permuted);

/* Combine (gpu/ops/src/lib.rs:3064-3130 moe_gather_combine_add_quad_packed):
 * out[t, :] = residual[t, :] + sum_r gates[t,r] * y_permuted[dest_row[t,r], :], ranks
 * added in order in fp32.  residual may be NULL.  out_type: b200gemm_out_t.
 * gates == NULL means weights of one: then this is the backward of the dispatch,
 * dx[t, :] = sum_r dx_permuted[dest_row[t,r], :] (crates/nn/src/moe.rs:383-395). */
B200GEMM_API int b200gemm_moe_combine(b200gemm_handle_t h, void* stream, const void* y_permuted,
                                      const uint32_t* dest_row, const float* gates,
                                      const void* residual, int64_t tokens, int32_t top_k, int64_t d,
                                      void* out, int32_t out_type);

/*
 * Expert parallelism over peer-mapped memory (new: the reference is single-GPU).
 * Experts are split in contiguous blocks over `world` GPUs of one box (expert e
 * lives on rank e / (experts / world)); every rank keeps its own tokens.  Each rank
 * owns an inbox and a result buffer that its peers can address (memory mapped into
 * every process, e.g. torch symmetric memory or CUDA IPC; `peer_*[r]` is rank r's
 * buffer as seen from the calling process).  Row layout of rank j's inbox: blocks by
 * source rank, inside a block by local expert, inside an expert by slot.  All three
 * calls take their sizes from device memory: nothing is read back to the host.
 *
 *   plan          from all_counts[world][experts] (every rank's accepted_counts,
 *                 all-gathered; device int32) computes, on the device,
 *                 dst_base[experts]: where MY rows for expert e begin in owner(e)'s inbox;
 *                 group_offsets[experts + 1], group_b_index[experts]: the (source rank,
 *                 local expert) groups of MY inbox, for b200gemm_grouped_gemm_indexed.
 *   push          writes x[token] into owner(e)'s inbox at dst_base[e] + slot for every
 *                 selected expert of every token (peer stores over NVLink).  A row that
 *                 would land at or beyond `inbox_rows` is not written and device status
 *                 105 is recorded (b200gemm_device_status).
 *   pull_combine  out[token] = residual + sum_r gate_r * results_of_owner[dst_base[e_r] + slot_r]
 *                 (peer loads), ranks added in order in fp32; a row at or beyond
 *                 `result_rows` is skipped and device status 105 recorded.
 * The caller orders the phases between ranks (a barrier after every rank's push and
 * after every rank's expert GEMMs, e.g. b200gemm_peer_barrier, which can also gather
 * all_counts); the kernels themselves never wait on a peer.  After
 * b200gemm_set_exchange_ctas(h, n, 1) push and pull_combine move their rows by bulk
 * asynchronous copies through shared memory from n blocks (bit-identical results).
 * world <= 8, experts a multiple of world and <= 192, top_k <= 16, d % 8 == 0; every row buffer
 * (x, the peers' inboxes and result buffers, residual, out) 16-byte aligned.
 */
B200GEMM_API int b200gemm_moe_ep_plan(b200gemm_handle_t h, void* stream, const int32_t* all_counts,
                                      int32_t world, int32_t rank, int32_t experts, int32_t* dst_base,
                                      int32_t* group_offsets, int32_t* group_b_index);
B200GEMM_API int b200gemm_moe_ep_push(b200gemm_handle_t h, void* stream, const void* x,
                                      const uint32_t* selected, const uint32_t* slots,
                                      const int32_t* dst_base, void* const* peer_inbox,
                                      int64_t inbox_rows, int32_t world, int32_t experts,
                                      int64_t tokens, int32_t top_k, int64_t d);
B200GEMM_API int b200gemm_moe_ep_pull_combine(b200gemm_handle_t h, void* stream,
                                              void* const* peer_results, const uint32_t* selected,
                                              const uint32_t* slots, const int32_t* dst_base,
                                              const float* gates, const void* residual,
                                              int64_t result_rows, int32_t world, int32_t experts,
                                              int64_t tokens, int32_t top_k, int64_t d, void* out,
                                              int32_t out_type);

/*
 * A barrier between the GPUs of one box, as a kernel small enough to share an SM with a
 * persistent GEMM CTA (one block, no shared memory) -- which a collective library's kernel is
 * not, so a barrier made of one waits until the GEMM ends or needs SMs kept free for it.
 * New: the reference is single-GPU.
 *   peer_words[r]  rank r's array of `world` 64-bit arrival words (zero at the start) as seen
 *                  from the calling process (peer-mapped memory, e.g. symmetric memory)
 *   epoch          1, 2, 3, ... : the same on every rank for the same barrier, never reused with
 *                  the same arrays
 *   payload / peer_tables  optional all-gather on the way: this rank's `payload_count` int32
 *                  are written into row `rank` of every rank's table (peer_tables[r] = rank r's
 *                  [2][world][payload_count] table; half epoch & 1 is the one written, so a
 *                  rank already at the next barrier does not overwrite what a slower peer
 *                  still reads) before the arrival words, so that after the barrier that
 *                  half of every table holds every rank's integers
 * What this rank stored into peer memory earlier on `stream` is visible to the peers' kernels
 * launched after their barrier.  The wait is bounded: after limit_ms the kernel gives up,
 * records device status 108 (b200gemm_device_status) and returns; the arrays then hold a stale
 * epoch and must not be used again.  Ranks must not share a GPU.  world <= 8.
 */
B200GEMM_API int b200gemm_peer_barrier(b200gemm_handle_t h, void* stream, void* const* peer_words,
                                       int32_t world, int32_t rank, uint64_t epoch, int64_t limit_ms,
                                       const int32_t* payload, int32_t payload_count,
                                       void* const* peer_tables);

/*
 * dst[i] = sum over p in [0, parts), ascending, of src[p * part_stride + i], i in [0, count):
 * the last step of a reduce-scatter whose parts were delivered by copies (one part per rank,
 * e.g. by the copy engines over NVLink while the SMs keep multiplying).  Element types:
 * b200gemm_out_t, sums in fp32; count % 8 == 0.  max_blocks > 0 caps the grid, so that the
 * pass fits beside a persistent GEMM instead of waiting for it.  New: the reference is single-GPU.
 */
B200GEMM_API int b200gemm_sum_parts(b200gemm_handle_t h, void* stream, const void* src, int32_t src_type,
                                    int64_t part_stride, int32_t parts, int64_t count, void* dst,
                                    int32_t dst_type, int32_t max_blocks);

/*
 * The return leg of the expert-parallel exchange fused into the expert GEMM (new, like the
 * calls above): instead of writing its results into a local buffer for the token owners to
 * read later (b200gemm_moe_ep_pull_combine), the grouped GEMM stores every group's rows
 * straight into the buffer of the rank those rows came from, from its epilogue, so the
 * transfer over NVLink runs underneath the tensor-core work of the same kernel.
 *
 *   return_plan  from all_counts[world][experts]: for every group g = (source rank s, local
 *                expert e) of MY inbox, group_dst_rank[g] = s and group_dst_row[g] = the row of
 *                rank s's own permuted order (b200gemm_moe_route's dest_row) where the rows of
 *                that expert begin.  Device int32 [experts] each.
 *   grouped_gemm_peer  b200gemm_grouped_gemm_indexed without activation, whose C is not a
 *                local matrix: rows of group g land in peer_out[group_dst_rank[g]] (bf16,
 *                row stride ld_out elements, 0 = n) at rows group_dst_row[g] + (row - first row
 *                of g).  Plain 16-byte stores, 128 bytes per row and 64-column chunk; a row at
 *                or beyond out_rows is not written and device status 105 is recorded.
 * After every rank's GEMM (one barrier), each rank combines ITS tokens from ITS buffer with
 * b200gemm_moe_combine, exactly as on one GPU.  world <= 8, n % 8 == 0.
 */
B200GEMM_API int b200gemm_moe_ep_return_plan(b200gemm_handle_t h, void* stream, const int32_t* all_counts,
                                             int32_t world, int32_t rank, int32_t experts,
                                             int32_t* group_dst_rank, int32_t* group_dst_row);
B200GEMM_API int b200gemm_grouped_gemm_peer(b200gemm_handle_t h, void* stream, const void* a, int64_t lda,
                                            const void* b, int32_t b_layout, int64_t ldb,
                                            int64_t batch_stride_b, int32_t b_count,
                                            const int32_t* group_b_index, void* const* peer_out,
                                            int32_t world, int64_t ld_out, int64_t out_rows,
                                            const int32_t* group_dst_rank, const int32_t* group_dst_row,
                                            const int32_t* offsets, int32_t groups, int64_t total_rows,
                                            int64_t n, int64_t k);

/* Synchronises `stream`, reads and clears the device status word; returns
 * B200GEMM_ERR_DEVICE if a kernel recorded a timeout, and the raw code in
 * *device_code (may be NULL).  The reference has no counterpart: its kernels
 * never report errors from the device, and its host API returns driver
 * failures only (gpu/gemm/src/host.rs:616-626 `Result<(), DriverError>`). */
B200GEMM_API int b200gemm_device_status(b200gemm_handle_t h, void* stream, int32_t* device_code);

/* Self-test of the bounded waits every kernel here uses: launches a one-block
 * kernel that waits on a barrier nothing completes, gives up after `limit_ms`
 * (1..5000) and records a timeout code, so that the next
 * b200gemm_device_status returns B200GEMM_ERR_DEVICE with code 104.  The
 * kernel returns normally; the context stays usable.  No counterpart in the
 * reference, whose kernels spin without a limit (SPEC.md:725-741 describes the
 * deadlock that cost). */
B200GEMM_API int b200gemm_wait_selftest(b200gemm_handle_t h, void* stream, int64_t limit_ms);

/* Text of the last failure on the calling thread ("" if none). */
B200GEMM_API const char* b200gemm_last_error_string(void);

B200GEMM_API int b200gemm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200GEMM_H_ */
