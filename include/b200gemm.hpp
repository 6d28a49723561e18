// C++ host mirror of the reference's `Tcgen05Gemm` (gpu/gemm/src/host.rs:469-1098)
// over the C ABI in b200gemm.h.  Header-only; method names, argument meaning and
// the store / accumulate / transposed / batched / `_at` split follow the
// reference one for one.  Where the reference panics on a contract violation
// (host.rs:81-85, 1105-1109, 1168-1171) these methods return the library's
// status code instead; `last_error()` has the text.
//
// A "K-major" operand is stored [rows, K]; a "transposed" (MN-major) operand is
// stored [K, rows].  Device pointers are the caller's; `stream` is a
// cudaStream_t passed as void*.
#ifndef B200GEMM_HPP_
#define B200GEMM_HPP_

#include <cstdint>
#include <stdexcept>
#include <string>

#include "b200gemm.h"

namespace b200gemm {

/// TMA panel edge, reduction tile and CTA-pair tile (host.rs:13-19).
constexpr int TC_TILE = 128, TC_BK = 64, TC_M_TILE = 256, TC_N_TILE = 256;

/// A bf16 operand: device pointer + how it is laid out.  Replaces the
/// reference's `Bf16TmaMap` / `Bf16PairsTmaMap(s)` (host.rs:267-465): the
/// tensor map is built inside the library from these fields.
struct Operand {
  const void* ptr = nullptr;
  int64_t rows = 0;          // M or N
  int64_t k = 0;             // reduction extent
  int64_t ld = 0;            // row stride in elements (0 = dense)
  int64_t batch_stride = 0;  // elements between experts (0 = dense)
  b200gemm_layout_t layout = B200GEMM_K_MAJOR;
};

class Tcgen05Gemm {
 public:
  /// Tcgen05Gemm::load (host.rs:508-530).
  explicit Tcgen05Gemm(int device) {
    if (b200gemm_create(device, &h_) != B200GEMM_OK) throw std::runtime_error(last_error());
  }
  ~Tcgen05Gemm() { b200gemm_destroy(h_); }
  Tcgen05Gemm(const Tcgen05Gemm&) = delete;
  Tcgen05Gemm& operator=(const Tcgen05Gemm&) = delete;

  static std::string last_error() { return b200gemm_last_error_string(); }
  b200gemm_handle_t handle() const { return h_; }

  // ---- bf16 output ---------------------------------------------------------
  /// C = A.B^T, packed bf16 (host.rs:616).
  int store(void* stream, const Operand& a, const Operand& b, void* out) const {
    return run(stream, a, b, out, B200GEMM_OUT_BF16, B200GEMM_STORE, 1);
  }
  /// `experts` equal-shaped C = A.B^T in one launch (host.rs:658).
  int store_batched(void* stream, const Operand& a, const Operand& b, void* out, int experts) const {
    return run(stream, a, b, out, B200GEMM_OUT_BF16, B200GEMM_STORE, experts);
  }
  /// C += A.B^T in bf16 (host.rs:695).
  int accumulate(void* stream, const Operand& a, const Operand& b, void* out) const {
    return run(stream, a, b, out, B200GEMM_OUT_BF16, B200GEMM_ACCUMULATE, 1);
  }
  /// C += A^T.B, both operands MN-major (host.rs:875).
  int accumulate_transposed(void* stream, Operand a, Operand b, void* out) const {
    a.layout = b.layout = B200GEMM_MN_MAJOR;
    return run(stream, a, b, out, B200GEMM_OUT_BF16, B200GEMM_ACCUMULATE, 1);
  }

  // ---- fp32 output, overwrite ----------------------------------------------
  int f32_store(void* stream, const Operand& a, const Operand& b, float* out) const {
    return run(stream, a, b, out, B200GEMM_OUT_F32, B200GEMM_STORE, 1);
  }
  /// Writes out[offset .. offset + m*n) (host.rs:766).
  int f32_store_at(void* stream, const Operand& a, const Operand& b, float* out, size_t offset) const {
    return run(stream, a, b, out + offset, B200GEMM_OUT_F32, B200GEMM_STORE, 1);
  }
  int f32_store_batched(void* stream, const Operand& a, const Operand& b, float* out, int experts) const {
    return run(stream, a, b, out, B200GEMM_OUT_F32, B200GEMM_STORE, experts);
  }
  int f32_store_transposed(void* stream, Operand a, Operand b, float* out) const {
    a.layout = b.layout = B200GEMM_MN_MAJOR;
    return run(stream, a, b, out, B200GEMM_OUT_F32, B200GEMM_STORE, 1);
  }

  // ---- fp32 output, accumulate (copy-engine reduce-add) ----------------------
  int f32_accumulate(void* stream, const Operand& a, const Operand& b, float* out) const {
    return run(stream, a, b, out, B200GEMM_OUT_F32, B200GEMM_ACCUMULATE, 1);
  }
  int f32_accumulate_at(void* stream, const Operand& a, const Operand& b, float* out, size_t offset) const {
    return run(stream, a, b, out + offset, B200GEMM_OUT_F32, B200GEMM_ACCUMULATE, 1);
  }
  int f32_accumulate_transposed(void* stream, Operand a, Operand b, float* out) const {
    a.layout = b.layout = B200GEMM_MN_MAJOR;
    return run(stream, a, b, out, B200GEMM_OUT_F32, B200GEMM_ACCUMULATE, 1);
  }
  int f32_accumulate_transposed_at(void* stream, Operand a, Operand b, float* out, size_t offset) const {
    return f32_accumulate_transposed(stream, a, b, out + offset);
  }
  int f32_accumulate_transposed_batched(void* stream, Operand a, Operand b, float* out, int experts) const {
    a.layout = b.layout = B200GEMM_MN_MAJOR;
    return run(stream, a, b, out, B200GEMM_OUT_F32, B200GEMM_ACCUMULATE, experts);
  }

  // ---- lm-head fused with softmax cross-entropy ------------------------------
  // Replaces GpuBf16Head::forward_into + cross_entropy_into and their backward
  // (gpu/model/src/lib.rs:3076-3145, 6977-7040).  `weight` is the [k, v] master
  // when w_layout is MN-major, [v, k] when K-major.
  static size_t lmhead_ce_workspace_bytes(int64_t m) { return b200gemm_lmhead_ce_workspace_bytes(m); }
  int lmhead_ce_forward(void* stream, const void* hidden, const void* weight, b200gemm_layout_t w_layout,
                        const int32_t* targets, int64_t m, int64_t k, int64_t v, int64_t classes,
                        float* lse, float* row_loss, float* loss, void* workspace,
                        size_t workspace_bytes) const {
    return b200gemm_lmhead_ce_forward(h_, stream, hidden, weight, w_layout, targets, m, k, v, classes,
                                      lse, row_loss, loss, workspace, workspace_bytes);
  }
  int lmhead_ce_backward(void* stream, const void* hidden, const void* weight, b200gemm_layout_t w_layout,
                         const int32_t* targets, const float* lse, float dy, int64_t m, int64_t k,
                         int64_t v, int64_t classes, void* dlogits_bf16, float* d_hidden,
                         float* d_weight, bool accumulate_dw) const {
    return b200gemm_lmhead_ce_backward(h_, stream, hidden, weight, w_layout, targets, lse, dy, m, k, v,
                                       classes, dlogits_bf16, d_hidden, d_weight, accumulate_dw ? 1 : 0);
  }

  // ---- MoE: routing integers, dispatch, grouped expert GEMM, combine -----------
  // (crates/nn/src/moe.rs:205-352; gpu/model/src/lib.rs:4971-5130)
  int moe_route(void* stream, const float* scores, bool scores_are_logits, int64_t tokens,
                int32_t experts, int32_t top_k, int64_t capacity, uint32_t* selected, float* gates,
                uint32_t* slots, uint32_t* assignment_counts, uint32_t* accepted_counts,
                int32_t* offsets, uint32_t* dest_row) const {
    return b200gemm_moe_route(h_, stream, scores, scores_are_logits ? 1 : 0, tokens, experts, top_k,
                              capacity, selected, gates, slots, assignment_counts, accepted_counts,
                              offsets, dest_row);
  }
  int moe_scatter(void* stream, const void* x, const uint32_t* dest_row, int64_t tokens, int32_t top_k,
                  int64_t d, void* x_permuted) const {
    return b200gemm_moe_scatter(h_, stream, x, dest_row, tokens, top_k, d, x_permuted);
  }
  int moe_combine(void* stream, const void* y_permuted, const uint32_t* dest_row, const float* gates,
                  const void* residual, int64_t tokens, int32_t top_k, int64_t d, void* out,
                  b200gemm_out_t out_type) const {
    return b200gemm_moe_combine(h_, stream, y_permuted, dest_row, gates, residual, tokens, top_k, d, out,
                                out_type);
  }
  // Expert-parallel exchange over peer memory (no counterpart in the reference, which
  // trains on one GPU): plan -> push (peer stores) -> expert GEMMs -> pull_combine (peer loads).
  int moe_ep_plan(void* stream, const int32_t* all_counts, int32_t world, int32_t rank, int32_t experts,
                  int32_t* dst_base, int32_t* group_offsets, int32_t* group_b_index) const {
    return b200gemm_moe_ep_plan(h_, stream, all_counts, world, rank, experts, dst_base, group_offsets,
                                group_b_index);
  }
  int moe_ep_push(void* stream, const void* x, const uint32_t* selected, const uint32_t* slots,
                  const int32_t* dst_base, void* const* peer_inbox, int64_t inbox_rows, int32_t world,
                  int32_t experts, int64_t tokens, int32_t top_k, int64_t d) const {
    return b200gemm_moe_ep_push(h_, stream, x, selected, slots, dst_base, peer_inbox, inbox_rows, world,
                                experts, tokens, top_k, d);
  }
  int moe_ep_pull_combine(void* stream, void* const* peer_results, const uint32_t* selected,
                          const uint32_t* slots, const int32_t* dst_base, const float* gates,
                          const void* residual, int64_t result_rows, int32_t world, int32_t experts,
                          int64_t tokens, int32_t top_k, int64_t d, void* out, b200gemm_out_t out_type) const {
    return b200gemm_moe_ep_pull_combine(h_, stream, peer_results, selected, slots, dst_base, gates, residual,
                                        result_rows, world, experts, tokens, top_k, d, out, out_type);
  }
  /// Where my inbox's groups return to (rank and first row), for grouped_gemm_peer.
  int moe_ep_return_plan(void* stream, const int32_t* all_counts, int32_t world, int32_t rank, int32_t experts,
                         int32_t* group_dst_rank, int32_t* group_dst_row) const {
    return b200gemm_moe_ep_return_plan(h_, stream, all_counts, world, rank, experts, group_dst_rank, group_dst_row);
  }
  /// The expert GEMM whose epilogue stores each group's rows into the buffer of the rank they came from.
  int grouped_gemm_peer(void* stream, const Operand& a, const Operand& b, int32_t b_count, const int32_t* group_b_index,
                        void* const* peer_out, int32_t world, int64_t ld_out, int64_t out_rows,
                        const int32_t* group_dst_rank, const int32_t* group_dst_row, const int32_t* offsets,
                        int32_t groups) const {
    return b200gemm_grouped_gemm_peer(h_, stream, a.ptr, a.ld, b.ptr, b.layout, b.ld, b.batch_stride, b_count,
                                      group_b_index, peer_out, world, ld_out, out_rows, group_dst_rank, group_dst_row,
                                      offsets, groups, a.rows, b.rows, a.k);
  }
  /// Rows offsets[g]..offsets[g+1] of `a` times expert g's matrix, bf16 out, optional SiLU.
  int grouped_gemm(void* stream, const Operand& a, const Operand& b, void* c, int64_t ldc,
                   const int32_t* offsets, int32_t groups, bool silu) const {
    return b200gemm_grouped_gemm(h_, stream, a.ptr, a.ld, b.ptr, b.layout, b.ld, b.batch_stride, c, ldc,
                                 offsets, groups, a.rows, b.rows, a.k, silu ? 1 : 0);
  }

  /// y = silu(a . W_gate) * (a . W_up) per row group in one launch, `b` holding [gate | up]
  /// (2 * ff columns); `gate_up` (may be null) receives the bf16 [rows, 2, ff] panel.
  /// Replaces the fused gate/up GEMM + swiglu_forward_interleaved_packed pair
  /// (gpu/ops/src/lib.rs:1174-1222).
  int grouped_gemm_swiglu(void* stream, const Operand& a, const Operand& b, int32_t b_count,
                          const int32_t* group_b_index, void* y, int64_t ldy, void* gate_up,
                          int64_t ld_gate_up, const int32_t* offsets, int32_t groups, int64_t ff) const {
    return b200gemm_grouped_gemm_swiglu(h_, stream, a.ptr, a.ld, b.ptr, b.layout, b.ld, b.batch_stride,
                                        b_count, group_b_index, y, ldy, gate_up, ld_gate_up, offsets, groups,
                                        a.rows, ff, a.k);
  }

  /// f32_store that also writes the result rounded to bf16 (the next GEMM's operand copy).
  int f32_store_with_bf16_copy(void* stream, const Operand& a, const Operand& b, float* out, void* out_bf16,
                               int64_t ld_bf16 = 0) const {
    if (a.k != b.k) return B200GEMM_ERR_SHAPE;
    b200gemm_desc_t d = describe(a, b, out, B200GEMM_OUT_F32, B200GEMM_STORE, 1);
    d.split_k = 1;
    return b200gemm_gemm_dual(h_, stream, &d, out_bf16, ld_bf16, 0);
  }

  /// grouped_gemm where group g multiplies matrix group_b_index[g] of `b` (rows received from
  /// several ranks, each run sorted by local expert, multiplied where they landed).
  int grouped_gemm_indexed(void* stream, const Operand& a, const Operand& b, int32_t b_count,
                           const int32_t* group_b_index, void* c, int64_t ldc, const int32_t* offsets,
                           int32_t groups, int activation) const {
    return b200gemm_grouped_gemm_indexed(h_, stream, a.ptr, a.ld, b.ptr, b.layout, b.ld, b.batch_stride, b_count,
                                         group_b_index, c, ldc, offsets, groups, a.rows, b.rows, a.k, activation);
  }

  // ---- backward of the expert path (crates/nn/src/moe.rs:354-445) ----------------
  /// grouped_gemm with SiLU that also keeps the values before the activation (`before`, may be null).
  int grouped_gemm_silu(void* stream, const Operand& a, const Operand& b, int32_t b_count,
                        const int32_t* group_b_index, void* y, int64_t ldy, void* before, int64_t ld_before,
                        const int32_t* offsets, int32_t groups) const {
    return b200gemm_grouped_gemm_silu(h_, stream, a.ptr, a.ld, b.ptr, b.layout, b.ld, b.batch_stride, b_count,
                                      group_b_index, y, ldy, before, ld_before, offsets, groups, a.rows, b.rows, a.k);
  }
  /// Input gradient of an expert linear with the activation's backward in its epilogue
  /// (activation 1 = SiLU, 2 = SwiGLU; `saved` = what the forward kept).
  int grouped_gemm_act_backward(void* stream, const Operand& a, const Operand& b, int32_t b_count,
                                const int32_t* group_b_index, int activation, const void* saved, int64_t ld_saved,
                                void* d_saved, int64_t ld_dsaved, const int32_t* offsets, int32_t groups) const {
    return b200gemm_grouped_gemm_act_backward(h_, stream, a.ptr, a.ld, b.ptr, b.layout, b.ld, b.batch_stride, b_count,
                                              group_b_index, activation, saved, ld_saved, d_saved, ld_dsaved, offsets,
                                              groups, a.rows, b.rows, a.k);
  }
  /// dW[g] (=|+=) A[rows_g]^T . B[rows_g]: the row groups are the reduction axis
  /// (f32_accumulate_transposed_batched over exact groups instead of capacity bins).
  int grouped_wgrad(void* stream, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc,
                    int64_t batch_stride_c, int32_t c_count, const int32_t* group_c_index, const int32_t* offsets,
                    int32_t groups, int64_t total_rows, int64_t m, int64_t n, bool accumulate) const {
    return b200gemm_grouped_wgrad(h_, stream, a, lda, b, ldb, c, ldc, batch_stride_c, c_count, group_c_index,
                                  offsets, groups, total_rows, m, n, accumulate ? 1 : 0);
  }
  int moe_combine_backward(void* stream, const void* dy, b200gemm_out_t dy_type, const void* y_permuted,
                           const uint32_t* dest_row, const float* gates, int64_t tokens, int32_t top_k, int64_t d,
                           void* dy_permuted, float* gate_grad) const {
    return b200gemm_moe_combine_backward(h_, stream, dy, dy_type, y_permuted, dest_row, gates, tokens, top_k, d,
                                         dy_permuted, gate_grad);
  }
  /// activation 1 = SiLU (saved = values before it), 2 = SwiGLU (saved = the [rows, 2, ff] panel).
  int activation_backward(void* stream, int activation, const void* saved, int64_t ld_saved, const void* d_y,
                          int64_t ld_dy, int64_t rows, int64_t ff, void* d_saved, int64_t ld_dsaved) const {
    return b200gemm_activation_backward(h_, stream, activation, saved, ld_saved, d_y, ld_dy, rows, ff, d_saved,
                                        ld_dsaved);
  }
  int moe_route_backward(void* stream, const float* probs, const uint32_t* selected, const float* gates,
                         const float* gate_grad, const uint32_t* assignment_counts, float aux_coefficient,
                         int64_t tokens, int32_t experts, int32_t top_k, float* dlogits) const {
    return b200gemm_moe_route_backward(h_, stream, probs, selected, gates, gate_grad, assignment_counts,
                                       aux_coefficient, tokens, experts, top_k, dlogits);
  }
  /// logits = x (bf16) . w (fp32 [d, experts]); router_logits_bf16 for up to 256 experts.
  int router_logits(void* stream, const void* x, const float* w, int64_t tokens, int64_t d, int32_t experts,
                    float* logits) const {
    return b200gemm_router_logits(h_, stream, x, w, tokens, d, experts, logits);
  }
  /// mean(row_loss) + coefficient * sum(aux_terms)  (loss_mean_with_aux).
  int loss_mean_with_aux(void* stream, const float* row_loss, int64_t tokens, const float* aux_terms,
                         int32_t aux_count, float coefficient, float* loss) const {
    return b200gemm_loss_mean_with_aux(h_, stream, row_loss, tokens, aux_terms, aux_count, coefficient, loss);
  }

  // ---- the lm-head's other forms ----------------------------------------------
  /// One vocabulary shard of the fused forward: per-row max, sum-exp (relative to that max)
  /// and target logit, to be merged across shards by the caller's all-reduces.
  int lmhead_ce_forward_shard(void* stream, const void* hidden, const void* weight_shard,
                              b200gemm_layout_t w_layout, const int32_t* local_targets, int64_t m, int64_t k,
                              int64_t v_local, int64_t classes_local, float* row_max, float* row_sum,
                              float* row_target_logit, void* workspace, size_t workspace_bytes) const {
    return b200gemm_lmhead_ce_forward_shard(h_, stream, hidden, weight_shard, w_layout, local_targets, m, k,
                                            v_local, classes_local, row_max, row_sum, row_target_logit, workspace,
                                            workspace_bytes);
  }
  /// Shards' (max, sum-exp, target logit) blocks, gathered as [world][3][m], into lse / row losses / mean.
  int lmhead_ce_merge_shards(void* stream, const float* stats, int32_t world, int64_t m, float* lse,
                             float* row_loss, float* loss) const {
    return b200gemm_lmhead_ce_merge_shards(h_, stream, stats, world, m, lse, row_loss, loss);
  }
  /// The fused forward on the library's built-in scratch (m <= 32768): allocates nothing.
  int lmhead_ce_forward_noalloc(void* stream, const void* hidden, const void* weight,
                                b200gemm_layout_t w_layout, const int32_t* targets, int64_t m, int64_t k,
                                int64_t v, int64_t classes, float* lse, float* row_loss, float* loss) const {
    return b200gemm_lmhead_ce_forward_noalloc(h_, stream, hidden, weight, w_layout, targets, m, k, v, classes, lse,
                                              row_loss, loss);
  }

  // ---- fp32 family, staging converts (gpu/tensor-gpu/src/lib.rs:403-507, 1754-1851) ----
  /// op 0: C = A.B, 1: C = A^T.B, 2: C = A.B^T (fp32 operands, bit-exact with the CPU loops).
  int sgemm(void* stream, int op, bool accumulate, const float* a, const float* b, float* c, int64_t m,
            int64_t n, int64_t k) const {
    return b200gemm_sgemm(h_, stream, op, accumulate ? 1 : 0, a, b, c, m, n, k);
  }
  int convert_f32_to_bf16(void* stream, const float* src, void* dst_bf16, int64_t count) const {
    return b200gemm_convert_f32_to_bf16(h_, stream, src, dst_bf16, count);
  }
  int convert_bf16_to_f32(void* stream, const void* src_bf16, float* dst, int64_t count) const {
    return b200gemm_convert_bf16_to_f32(h_, stream, src_bf16, dst, count);
  }
  int transpose_bf16(void* stream, const void* src, void* dst, int64_t rows, int64_t cols) const {
    return b200gemm_transpose_bf16(h_, stream, src, dst, rows, cols);
  }

  /// Barrier between the GPUs of one box (optionally gathering a few integers per rank on the way).
  int peer_barrier(void* stream, void* const* peer_words, int32_t world, int32_t rank, uint64_t epoch,
                   int64_t limit_ms = 2000, const int32_t* payload = nullptr, int32_t payload_count = 0,
                   void* const* peer_tables = nullptr) const {
    return b200gemm_peer_barrier(h_, stream, peer_words, world, rank, epoch, limit_ms, payload, payload_count,
                                 peer_tables);
  }
  /// dst = sum of `parts` equally long arrays `part_stride` apart (the tail of a copy-delivered reduce-scatter).
  int sum_parts(void* stream, const void* src, b200gemm_out_t src_type, int64_t part_stride, int32_t parts,
                int64_t count, void* dst, b200gemm_out_t dst_type, int32_t max_blocks = 0) const {
    return b200gemm_sum_parts(h_, stream, src, src_type, part_stride, parts, count, dst, dst_type, max_blocks);
  }

  // ---- launch geometry, host buffers, device status ------------------------------
  /// tcgen05_launch_config (host.rs:47-94) for the GEMM `store`/`f32_store`/... would launch.
  int launch_config(const Operand& a, const Operand& b, void* out, b200gemm_out_t out_type, b200gemm_mode_t mode,
                    int experts, int32_t* grid, int32_t* cluster, int32_t* smem_bytes, int32_t* split_k) const {
    b200gemm_desc_t d = describe(a, b, out, out_type, mode, experts);
    return b200gemm_launch_config(h_, &d, grid, cluster, smem_bytes, split_k);
  }
  /// The GEMM on host-resident matrices (copies in, runs, copies out, synchronises).
  int gemm_host(void* stream, const Operand& a, const Operand& b, void* out, b200gemm_out_t out_type,
                b200gemm_mode_t mode) const {
    b200gemm_desc_t d = describe(a, b, out, out_type, mode, 1);
    return b200gemm_gemm_host(h_, stream, &d);
  }
  /// Synchronises `stream` and returns the device status word (0 = no kernel gave up waiting).
  int device_status(void* stream, int32_t* code = nullptr) const { return b200gemm_device_status(h_, stream, code); }
  /// Exercises the bounded wait: the next device_status reports code 104.
  int wait_selftest(void* stream, int64_t limit_ms) const { return b200gemm_wait_selftest(h_, stream, limit_ms); }
  static int version() { return b200gemm_version(); }

  /// Output row stride (elements) for the next calls; 0 = dense.  Lets a GEMM
  /// write one column block of a wider matrix (the grouped QKV projections,
  /// gpu/model/src/lib.rs:1379-1562).
  void set_ldc(int64_t ldc, int64_t batch_stride_c = 0) { ldc_ = ldc; bsc_ = batch_stride_c; }
  /// 0 = let the library choose, 1 = never split, n = n slices (fp32 output only).
  void set_split_k(int split_k) { split_k_ = split_k; }
  /// Persistent kernels on at most `sms` SMs (0 = all): room for a collective's kernels.
  int set_sm_limit(int sms) const { return b200gemm_set_sm_limit(h_, sms); }
  int set_exchange_ctas(int ctas, bool bulk = false) const { return b200gemm_set_exchange_ctas(h_, ctas, bulk ? 1 : 0); }
  /// Tiles from a device-side counter (true, the default) or the fixed round-robin walk.
  int set_scheduler(bool dynamic) const { return b200gemm_set_scheduler(h_, dynamic ? 1 : 0); }

 private:
  b200gemm_desc_t describe(const Operand& a, const Operand& b, void* out, b200gemm_out_t out_type,
                           b200gemm_mode_t mode, int experts) const {
    b200gemm_desc_t d{};
    d.a = a.ptr; d.b = b.ptr; d.c = out;
    d.m = a.rows; d.n = b.rows; d.k = a.k;
    d.lda = a.ld; d.ldb = b.ld; d.ldc = ldc_;
    d.a_layout = a.layout; d.b_layout = b.layout;
    d.out_type = out_type; d.mode = mode;
    d.batch = experts; d.split_k = split_k_;
    d.batch_stride_a = a.batch_stride; d.batch_stride_b = b.batch_stride; d.batch_stride_c = bsc_;
    return d;
  }
  int run(void* stream, const Operand& a, const Operand& b, void* out, b200gemm_out_t out_type,
          b200gemm_mode_t mode, int experts) const {
    if (a.k != b.k) return B200GEMM_ERR_SHAPE;
    b200gemm_desc_t d = describe(a, b, out, out_type, mode, experts);
    return b200gemm_gemm(h_, stream, &d);
  }

  b200gemm_handle_t h_ = nullptr;
  int64_t ldc_ = 0, bsc_ = 0;
  int split_k_ = 0;
};

}  // namespace b200gemm
#endif  // B200GEMM_HPP_
