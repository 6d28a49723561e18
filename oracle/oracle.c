/*
 * CPU oracle for the GEMM hot path of feitreim/oxide-train.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's CPU crates so that the CUDA kernels can be checked against
 * it.  Nothing in the product library links, loads or calls it; only the test
 * suite, the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Parity status: PINNED.  The reference (Rust) cannot be compiled where this
 * repository is built, so the restatement is pinned by the reference's own
 * known-answer tests instead (see tests/test_oracle.py):
 *   - crates/tensor-cpu/src/ops.rs:194-199   2x2 matmul known answer
 *   - crates/tensor-cpu/src/ops.rs:211-226   _tn/_nt equal explicit transpose
 *   - crates/tensor-core/src/element.rs:72-81 bf16 round-to-nearest-even
 *   - crates/tensor-core/src/rng.rs:71-78     splitmix64 step identity
 *   - crates/nn/tests/moe.rs:182-197          routing tie golden vector
 *
 * Build: gcc -O2 -ffp-contract=off -pthread -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: the reference multiplies in f32 and then adds in
 * f32 (two roundings); a fused multiply-add would change the low bits.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* Row-parallel helper (pthreads).  Each worker owns a contiguous range of    */
/* OUTPUT rows, so no output element is touched by two threads and the order  */
/* of additions per element is the single-threaded one.                       */
/* ------------------------------------------------------------------------ */

typedef void (*orc_row_fn)(void* ctx, size_t row_begin, size_t row_end);
typedef struct {
  orc_row_fn fn;
  void* ctx;
  size_t begin, end;
} orc_task;

static void* orc_task_main(void* p) {
  orc_task* t = (orc_task*)p;
  t->fn(t->ctx, t->begin, t->end);
  return NULL;
}

static void orc_parallel_rows(orc_row_fn fn, void* ctx, size_t rows, int threads) {
  if (threads <= 1 || rows < 2) {
    fn(ctx, 0, rows);
    return;
  }
  if ((size_t)threads > rows) threads = (int)rows;
  pthread_t* ids = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)threads);
  orc_task* tasks = (orc_task*)malloc(sizeof(orc_task) * (size_t)threads);
  size_t chunk = (rows + (size_t)threads - 1) / (size_t)threads;
  int started = 0;
  for (int t = 0; t < threads; ++t) {
    size_t b = (size_t)t * chunk, e = b + chunk < rows ? b + chunk : rows;
    if (b >= e) break;
    tasks[t].fn = fn;
    tasks[t].ctx = ctx;
    tasks[t].begin = b;
    tasks[t].end = e;
    if (pthread_create(&ids[t], NULL, orc_task_main, &tasks[t]) != 0) {
      fn(ctx, b, e); /* could not spawn: do the range here */
      tasks[t].fn = NULL;
    }
    started = t + 1;
  }
  for (int t = 0; t < started; ++t)
    if (tasks[t].fn) pthread_join(ids[t], NULL);
  free(ids);
  free(tasks);
}

typedef struct {
  const float *a, *b;
  float* c;
  size_t M, K, N;
  const int64_t* rows;
} orc_mm_ctx;

/* ------------------------------------------------------------------------ */
/* RNG: crates/tensor-core/src/rng.rs:9-65                                   */
/* ------------------------------------------------------------------------ */

static const uint64_t ORC_GAMMA = 0x9E3779B97F4A7C15ull; /* rng.rs:9 */

/* One mixing round over an already-advanced state (rng.rs:18-23). */
ORC_API uint64_t orc_splitmix64(uint64_t state) {
  uint64_t z = state;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

/* SplitMix64::next_u64 (rng.rs:51-54): advance, then mix. */
ORC_API uint64_t orc_rng_next_u64(uint64_t* state) {
  *state += ORC_GAMMA;
  return orc_splitmix64(*state);
}

/* SplitMix64::next_uniform (rng.rs:57-60): top 24 bits -> [0,1) -> [-1,1). */
ORC_API float orc_rng_next_uniform(uint64_t* state) {
  float unit = (float)(orc_rng_next_u64(state) >> 40) / (float)(1u << 24);
  return unit * 2.0f - 1.0f;
}

/* uniform_vec (rng.rs:63-65). */
ORC_API void orc_uniform_fill(float* out, size_t n, uint64_t seed) {
  uint64_t s = seed;
  for (size_t i = 0; i < n; ++i) out[i] = orc_rng_next_uniform(&s);
}

/*
 * Normal draws for the synthetic workloads (activations ~N(0,1), weights
 * ~N(0,0.02), ...).  The reference has no normal sampler; this is Box-Muller
 * over the same SplitMix64 stream, two uniforms per pair of outputs.  u1 is
 * taken from (0,1] so the logarithm is finite.
 */
ORC_API void orc_normal_fill(float* out, size_t n, uint64_t seed, float mean, float std) {
  uint64_t s = seed;
  const double two_pi = 6.283185307179586476925286766559;
  for (size_t i = 0; i < n; i += 2) {
    double u1 = ((double)(orc_rng_next_u64(&s) >> 40) + 1.0) / 16777216.0;
    double u2 = (double)(orc_rng_next_u64(&s) >> 40) / 16777216.0;
    double r = sqrt(-2.0 * log(u1));
    out[i] = (float)(mean + std * r * cos(two_pi * u2));
    if (i + 1 < n) out[i + 1] = (float)(mean + std * r * sin(two_pi * u2));
  }
}

/* ------------------------------------------------------------------------ */
/* bf16: gpu/tensor-gpu/src/lib.rs:316-326 (the in-repo restatement of        */
/* half::bf16::from_f32 for finite values; crates/tensor-core/element.rs:72) */
/* ------------------------------------------------------------------------ */

ORC_API uint16_t orc_bf16_from_f32(float value) {
  uint32_t bits;
  memcpy(&bits, &value, 4);
  uint32_t round = 0x7fffu + ((bits >> 16) & 1u);
  return (uint16_t)((bits + round) >> 16);
}

ORC_API float orc_bf16_to_f32(uint16_t b) {
  uint32_t bits = (uint32_t)b << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* quantize_bf16 (gpu/gemm/src/main.rs:65-75): words + the widened values. */
ORC_API void orc_quantize_bf16(const float* in, size_t n, uint16_t* bits_out, float* rounded_out) {
  for (size_t i = 0; i < n; ++i) {
    uint16_t b = orc_bf16_from_f32(in[i]);
    if (bits_out) bits_out[i] = b;
    if (rounded_out) rounded_out[i] = orc_bf16_to_f32(b);
  }
}

/* bf16_stochastic (crates/tensor-core/src/element.rs:15-17). */
ORC_API uint16_t orc_bf16_stochastic(float value, uint32_t entropy) {
  uint32_t bits;
  memcpy(&bits, &value, 4);
  return (uint16_t)((bits + (entropy & 0xffffu)) >> 16);
}

/* ------------------------------------------------------------------------ */
/* Matmul family: crates/tensor-cpu/src/ops.rs:85-147                         */
/* `threads` <= 1 runs the loops exactly as written there.  `threads` > 1     */
/* splits the OUTPUT rows over pthreads; every output element still     */
/* sees the same products added in the same order, so results are identical.  */
/* ------------------------------------------------------------------------ */

/* C[M,N] = A[M,K] . B[K,N]   (ops.rs:87-104: i-k-j, c += a*b). */
static void orc_matmul_rows_fn(void* p, size_t r0, size_t r1) {
  orc_mm_ctx* x = (orc_mm_ctx*)p;
  const float *a = x->a, *b = x->b;
  float* c = x->c;
  size_t K = x->K, N = x->N;
  for (size_t i = r0; i < r1; ++i) {
    for (size_t k = 0; k < K; ++k) {
      float aik = a[i * K + k];
      for (size_t j = 0; j < N; ++j) c[i * N + j] += aik * b[k * N + j];
    }
  }
}

ORC_API void orc_matmul(const float* a, const float* b, float* c, size_t M, size_t K, size_t N,
                        int threads) {
  memset(c, 0, M * N * sizeof(float));
  orc_mm_ctx x = {a, b, c, M, K, N, NULL};
  orc_parallel_rows(orc_matmul_rows_fn, &x, M, threads);
}

/* C[K,N] = A[M,K]^T . B[M,N]   (ops.rs:109-125: i-k-j into c[k,j]).
 * Per output element the products arrive in ascending i; the threaded form
 * keeps that order by giving each thread whole output rows k. */
static void orc_matmul_tn_rows_fn(void* p, size_t k0, size_t k1) {
  orc_mm_ctx* x = (orc_mm_ctx*)p;
  const float *a = x->a, *b = x->b;
  float* c = x->c;
  size_t M = x->M, K = x->K, N = x->N;
  for (size_t k = k0; k < k1; ++k) {
    for (size_t i = 0; i < M; ++i) {
      float aik = a[i * K + k];
      for (size_t j = 0; j < N; ++j) c[k * N + j] += aik * b[i * N + j];
    }
  }
}

ORC_API void orc_matmul_tn(const float* a, const float* b, float* c, size_t M, size_t K, size_t N,
                           int threads) {
  memset(c, 0, K * N * sizeof(float));
  if (threads <= 1) {
    for (size_t i = 0; i < M; ++i)
      for (size_t k = 0; k < K; ++k) {
        float aik = a[i * K + k];
        for (size_t j = 0; j < N; ++j) c[k * N + j] += aik * b[i * N + j];
      }
    return;
  }
  orc_mm_ctx x = {a, b, c, M, K, N, NULL};
  orc_parallel_rows(orc_matmul_tn_rows_fn, &x, K, threads);
}

/* C[M,N] = A[M,K] . B[N,K]^T   (ops.rs:130-147: i-j-k with a local acc). */
static void orc_matmul_nt_rows_fn(void* p, size_t r0, size_t r1) {
  orc_mm_ctx* x = (orc_mm_ctx*)p;
  const float *a = x->a, *b = x->b;
  float* c = x->c;
  size_t K = x->K, N = x->N;
  for (size_t i = r0; i < r1; ++i) {
    for (size_t j = 0; j < N; ++j) {
      float acc = 0.0f;
      for (size_t k = 0; k < K; ++k) acc += a[i * K + k] * b[j * K + k];
      c[i * N + j] = acc;
    }
  }
}

ORC_API void orc_matmul_nt(const float* a, const float* b, float* c, size_t M, size_t K, size_t N,
                           int threads) {
  orc_mm_ctx x = {a, b, c, M, K, N, NULL};
  orc_parallel_rows(orc_matmul_nt_rows_fn, &x, M, threads);
}

/* Explicit transpose [M,K] -> [K,M] (ops.rs:151-157). */
ORC_API void orc_transpose(const float* a, float* out, size_t M, size_t K) {
  for (size_t k = 0; k < K; ++k)
    for (size_t i = 0; i < M; ++i) out[k * M + i] = a[i * K + k];
}

/* Selected rows of orc_matmul: C_rows[r,:] = A[rows[r],:] . B.  Used to check
 * full-size GPU results on sampled rows, with the full K per element and the
 * same i-k-j accumulation order. */
static void orc_matmul_sel_rows_fn(void* p, size_t r0, size_t r1) {
  orc_mm_ctx* x = (orc_mm_ctx*)p;
  size_t K = x->K, N = x->N;
  for (size_t r = r0; r < r1; ++r) {
    const float* arow = x->a + (size_t)x->rows[r] * K;
    for (size_t k = 0; k < K; ++k) {
      float aik = arow[k];
      for (size_t j = 0; j < N; ++j) x->c[r * N + j] += aik * x->b[k * N + j];
    }
  }
}

ORC_API void orc_matmul_rows(const float* a, const float* b, float* c_rows, const int64_t* rows,
                             size_t n_rows, size_t K, size_t N, int threads) {
  memset(c_rows, 0, n_rows * N * sizeof(float));
  orc_mm_ctx x = {a, b, c_rows, n_rows, K, N, rows};
  orc_parallel_rows(orc_matmul_sel_rows_fn, &x, n_rows, threads);
}

/* ------------------------------------------------------------------------ */
/* Linear: crates/nn/src/linear.rs:42-49.  W is [IN, OUT].                    */
/* ------------------------------------------------------------------------ */

ORC_API void orc_linear_forward(const float* x, const float* w, float* y, size_t n, size_t in,
                                size_t out, int threads) {
  orc_matmul(x, w, y, n, in, out, threads);
}

/* dW += x^T dy ; dx = dy W^T.  `scratch` holds in*out floats. */
ORC_API void orc_linear_backward(const float* x, const float* w, const float* dy, float* dw,
                                 float* dx, float* scratch, size_t n, size_t in, size_t out,
                                 int threads) {
  orc_matmul_tn(x, dy, scratch, n, in, out, threads);
  for (size_t i = 0; i < in * out; ++i) dw[i] += scratch[i];
  orc_matmul_nt(dy, w, dx, n, out, in, threads);
}

/* ------------------------------------------------------------------------ */
/* Row softmax and cross entropy.                                             */
/* softmax_rows: crates/tensor-cpu/src/ops.rs:166-184                         */
/* SoftmaxCrossEntropy: crates/nn/src/cross_entropy.rs:28-72                  */
/* ------------------------------------------------------------------------ */

ORC_API void orc_softmax_rows(const float* a, float* o, size_t M, size_t N) {
  for (size_t i = 0; i < M; ++i) {
    const float* row = a + i * N;
    float max = -INFINITY;
    for (size_t j = 0; j < N; ++j) max = fmaxf(max, row[j]);
    double denom = 0.0;
    for (size_t j = 0; j < N; ++j) {
      float e = expf(row[j] - max);
      o[i * N + j] = e;
      denom += (double)e;
    }
    for (size_t j = 0; j < N; ++j) o[i * N + j] /= (float)denom;
  }
}

/*
 * Forward (cross_entropy.rs:28-60).  `ld` is the row stride of `logits` and
 * `probs` (>= classes): columns at or beyond `classes` are padding that the
 * classifier ignores, as gpu/ops/src/lib.rs:1721-1829 does for the padded
 * vocabulary.  `row_loss` (optional) receives max + ln(sum) - logit[target]
 * per row in f64.  Returns the mean loss, f64 sum cast to f32.
 */
ORC_API float orc_xent_forward(const float* logits, const int32_t* targets, size_t n,
                               size_t classes, size_t ld, float* probs, double* row_loss) {
  double loss = 0.0;
  for (size_t i = 0; i < n; ++i) {
    const float* row = logits + i * ld;
    float max = -INFINITY;
    for (size_t j = 0; j < classes; ++j) max = fmaxf(max, row[j]);
    double sum_exp = 0.0;
    for (size_t j = 0; j < classes; ++j) {
      float e = expf(row[j] - max);
      if (probs) probs[i * ld + j] = e;
      sum_exp += (double)e;
    }
    if (probs) {
      for (size_t j = 0; j < classes; ++j) probs[i * ld + j] /= (float)sum_exp;
      for (size_t j = classes; j < ld; ++j) probs[i * ld + j] = 0.0f;
    }
    double l = (double)max + log(sum_exp) - (double)row[targets[i]];
    if (row_loss) row_loss[i] = l;
    loss += l;
  }
  return (float)(loss / (double)n);
}

/* Backward (cross_entropy.rs:62-72): dlogits = p*s - s*onehot, s = dy/n.
 * Padded columns stay zero (gpu/ops/src/main.rs:2103). */
ORC_API void orc_xent_backward(const float* probs, const int32_t* targets, size_t n,
                               size_t classes, size_t ld, float dy, float* dlogits) {
  float scale = dy / (float)n;
  for (size_t i = 0; i < n; ++i) {
    for (size_t j = 0; j < classes; ++j) dlogits[i * ld + j] = probs[i * ld + j] * scale;
    for (size_t j = classes; j < ld; ++j) dlogits[i * ld + j] = 0.0f;
    dlogits[i * ld + targets[i]] -= scale;
  }
}

/* ------------------------------------------------------------------------ */
/* MoE routing: crates/nn/src/moe.rs:205-254                                  */
/* ------------------------------------------------------------------------ */

#define ORC_DROPPED 0xFFFFFFFFu /* u32::MAX, gpu/ops/src/lib.rs:2569-2705 */

/*
 * probs [N,E] -> selected[N*K], gates[N*K], slots[N*K] (ORC_DROPPED when the
 * expert was already at capacity), assignment_counts[E], accepted_counts[E].
 * Order per token: descending probability by total order on f32 bits
 * (f32::total_cmp), ties broken towards the lower expert index.  The top-k
 * denominator is summed in f64 and cast to f32 (moe.rs:222-225).  Slots are
 * arrival order in flattened (token, rank) order (moe.rs:228-236).
 */
static int32_t orc_total_key(float f) {
  /* f32::total_cmp: flip the magnitude bits of negatives so that integer
   * comparison orders -NaN < -inf < ... < -0 < +0 < ... < +inf < +NaN. */
  int32_t b;
  memcpy(&b, &f, 4);
  b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
  return b;
}

ORC_API void orc_moe_route(const float* probs, size_t N, size_t E, size_t K, size_t C,
                           uint32_t* selected, float* gates, uint32_t* slots,
                           uint32_t* assignment_counts, uint32_t* accepted_counts) {
  memset(assignment_counts, 0, E * sizeof(uint32_t));
  memset(accepted_counts, 0, E * sizeof(uint32_t));
  uint8_t* taken = (uint8_t*)malloc(E);
  for (size_t token = 0; token < N; ++token) {
    const float* p = probs + token * E;
    memset(taken, 0, E);
    /* Selection sort of the first K places: the unique order defined by the
     * comparator, so any correct sort gives the same prefix. */
    double denom = 0.0;
    for (size_t rank = 0; rank < K; ++rank) {
      size_t best = E;
      for (size_t e = 0; e < E; ++e) {
        if (taken[e]) continue;
        if (best == E || orc_total_key(p[e]) > orc_total_key(p[best])) best = e;
      }
      taken[best] = 1;
      selected[token * K + rank] = (uint32_t)best;
      denom += (double)p[best];
    }
    float denominator = (float)denom;
    for (size_t rank = 0; rank < K; ++rank) {
      size_t pair = token * K + rank;
      uint32_t expert = selected[pair];
      gates[pair] = p[expert] / denominator;
      assignment_counts[expert] += 1;
      if (accepted_counts[expert] < C) {
        slots[pair] = accepted_counts[expert];
        accepted_counts[expert] += 1;
      } else {
        slots[pair] = ORC_DROPPED;
      }
    }
  }
  free(taken);
}

/* Expert offsets = exclusive prefix sum of the accepted counts; permuted row
 * of pair p = offsets[selected[p]] + slots[p] (ORC_DROPPED stays dropped). */
ORC_API void orc_moe_offsets(const uint32_t* accepted_counts, size_t E, uint32_t* offsets) {
  uint32_t run = 0;
  for (size_t e = 0; e < E; ++e) {
    offsets[e] = run;
    run += accepted_counts[e];
  }
  offsets[E] = run;
}

ORC_API void orc_moe_permutation(const uint32_t* selected, const uint32_t* slots,
                                 const uint32_t* offsets, size_t pairs, uint32_t* dest_row) {
  for (size_t p = 0; p < pairs; ++p)
    dest_row[p] = slots[p] == ORC_DROPPED ? ORC_DROPPED : offsets[selected[p]] + slots[p];
}

/* SiLU as crates/nn/src/swiglu.rs:22-28 writes it: g * (1 / (1 + exp(-g))). */
ORC_API void orc_silu(const float* g, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    float sigmoid = 1.0f / (1.0f + expf(-g[i]));
    out[i] = g[i] * sigmoid;
  }
}

/* SwiGLU forward (swiglu.rs:22-28): silu(gate) * up. */
ORC_API void orc_swiglu(const float* gate, const float* up, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    float sigmoid = 1.0f / (1.0f + expf(-gate[i]));
    out[i] = gate[i] * sigmoid * up[i];
  }
}

/* ------------------------------------------------------------------------ */
/* MoE backward: crates/nn/src/moe.rs:354-445, crates/nn/src/swiglu.rs:30-47  */
/* ------------------------------------------------------------------------ */

/* SwiGLU backward (swiglu.rs:30-47): dgate = dy*up*dsilu, dup = dy*silu. */
ORC_API void orc_swiglu_backward(const float* gate, const float* up, const float* dy, float* dgate,
                                 float* dup, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    float sigmoid = 1.0f / (1.0f + expf(-gate[i]));
    float silu = gate[i] * sigmoid;
    float dsilu = sigmoid * (1.0f + gate[i] * (1.0f - sigmoid));
    dgate[i] = dy[i] * up[i] * dsilu;
    dup[i] = dy[i] * silu;
  }
}

/* SiLU backward: the gate half of the above with up = 1. */
ORC_API void orc_silu_backward(const float* g, const float* dy, float* dg, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    float sigmoid = 1.0f / (1.0f + expf(-g[i]));
    float dsilu = sigmoid * (1.0f + g[i] * (1.0f - sigmoid));
    dg[i] = dy[i] * dsilu;
  }
}

/*
 * Backward of the combine (moe.rs:360-381) over the permuted row layout: for every
 * accepted pair, dy_permuted[dest_row] = gate * dy[token] and
 * gate_grad[pair] = sum_d expert_out[dest_row][d] * dy[token][d] summed in f64.
 * Rows of dy_permuted that no pair maps to, and gate_grad of dropped pairs, are zero.
 */
ORC_API void orc_moe_combine_backward(const float* dy, const float* y_permuted, const uint32_t* dest_row,
                                      const float* gates, size_t N, size_t K, size_t D, size_t rows,
                                      float* dy_permuted, float* gate_grad) {
  memset(dy_permuted, 0, rows * D * sizeof(float));
  for (size_t token = 0; token < N; ++token) {
    for (size_t rank = 0; rank < K; ++rank) {
      size_t pair = token * K + rank;
      gate_grad[pair] = 0.0f;
      if (dest_row[pair] == ORC_DROPPED) continue;
      size_t row = dest_row[pair];
      float gate = gates[pair];
      double gg = 0.0;
      for (size_t d = 0; d < D; ++d) {
        dy_permuted[row * D + d] += gate * dy[token * D + d];
        gg += (double)y_permuted[row * D + d] * (double)dy[token * D + d];
      }
      gate_grad[pair] = (float)gg;
    }
  }
}

/* Backward of the dispatch (moe.rs:383-395): dx[token] = sum over accepted ranks, in
 * order, of dx_permuted[dest_row]. */
ORC_API void orc_moe_scatter_backward(const float* dx_permuted, const uint32_t* dest_row, size_t N, size_t K,
                                      size_t D, float* dx) {
  memset(dx, 0, N * D * sizeof(float));
  for (size_t token = 0; token < N; ++token)
    for (size_t rank = 0; rank < K; ++rank) {
      size_t pair = token * K + rank;
      if (dest_row[pair] == ORC_DROPPED) continue;
      for (size_t d = 0; d < D; ++d) dx[token * D + d] += dx_permuted[(size_t)dest_row[pair] * D + d];
    }
}

/* Backward of the routing (moe.rs:397-445): gate gradients -> probability gradients
 * (renormalised top-k + the load-balancing term) -> router logit gradients. */
ORC_API void orc_moe_route_backward(const float* probs, const uint32_t* selected, const float* gates,
                                    const float* gate_grad, const uint32_t* assignment_counts,
                                    float aux_coefficient, size_t N, size_t E, size_t K, float* dlogits) {
  float* dprob = (float*)malloc(E * sizeof(float));
  for (size_t token = 0; token < N; ++token) {
    const float* p = probs + token * E;
    for (size_t e = 0; e < E; ++e) dprob[e] = 0.0f;
    double weighted = 0.0, psum = 0.0;
    for (size_t rank = 0; rank < K; ++rank) {
      size_t pair = token * K + rank;
      weighted += (double)gate_grad[pair] * (double)gates[pair];
      psum += (double)p[selected[pair]];
    }
    float weighted_f = (float)weighted, psum_f = (float)psum;
    for (size_t rank = 0; rank < K; ++rank) {
      size_t pair = token * K + rank;
      dprob[selected[pair]] += (gate_grad[pair] - weighted_f) / psum_f;
    }
    for (size_t e = 0; e < E; ++e) {
      float fraction = (float)assignment_counts[e] / (float)(N * K);
      dprob[e] += aux_coefficient * (float)E * fraction / (float)N;
    }
    double dot = 0.0;
    for (size_t e = 0; e < E; ++e) dot += (double)p[e] * (double)dprob[e];
    float dot_f = (float)dot;
    for (size_t e = 0; e < E; ++e) dlogits[token * E + e] = p[e] * (dprob[e] - dot_f);
  }
  free(dprob);
}
