// cuBLASLt beside the GEMM: the denominator the benchmark prints next to every row.
//
// NOT part of the product: built into its own shared library, loaded only by the
// benchmark's comparator column, never by the package.  The recipe is the reference's
// (gpu/gemm/src/cublaslt.rs:55-61, 434-470): compute type CUBLAS_COMPUTE_32F, bf16 operands,
// a 32 MiB workspace that also caps what the heuristic may return, whatever
// cublasLtMatmulAlgoGetHeuristic ranks first (no search, no tuning pass), fp32 or bf16 C
// at the kernel's own width, beta = 1 on the rows where the kernel adds into C.
//
// cuBLASLt is column-major, the operands here are row-major, so the product asked for is
// the transpose (cublaslt.rs:13-30): with C^T = op(b) . op(a), cuBLASLt's first operand is
// this library's `b` and its second is `a`:
//   b stored [n, k] (K-major):  column-major k x n, ld k, CUBLAS_OP_T
//   b stored [k, n] (MN-major): column-major n x k, ld n, CUBLAS_OP_N
//   a stored [m, k] (K-major):  column-major k x m, ld k, CUBLAS_OP_N
//   a stored [k, m] (MN-major): column-major m x k, ld m, CUBLAS_OP_T
//   c stored [m, n]:            column-major n x m, ld n
#include <cublasLt.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <new>

namespace {

constexpr size_t kWorkspaceBytes = 32ull * 1024 * 1024;   // cublaslt.rs:61

thread_local char g_error[256] = "";

int fail(const char* what, int code) {
  snprintf(g_error, sizeof(g_error), "%s failed with status %d", what, code);
  return 1;
}

struct Session {
  cublasLtHandle_t handle = nullptr;
  void* workspace = nullptr;
};

struct Plan {
  cublasLtMatmulDesc_t desc = nullptr;
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
  cublasLtMatmulAlgo_t algo;
  size_t workspace = 0;
  float beta = 0.f;
};

}  // namespace

#define CMP_API extern "C" __attribute__((visibility("default")))

CMP_API const char* cmp_last_error() { return g_error; }

CMP_API int cmp_create(void** out) {
  Session* s = new (std::nothrow) Session();
  if (!s) return fail("allocation", -1);
  cublasStatus_t st = cublasLtCreate(&s->handle);
  if (st != CUBLAS_STATUS_SUCCESS) { delete s; return fail("cublasLtCreate", st); }
  cudaError_t e = cudaMalloc(&s->workspace, kWorkspaceBytes);
  if (e != cudaSuccess) { cublasLtDestroy(s->handle); delete s; return fail("cudaMalloc(workspace)", e); }
  *out = s;
  return 0;
}

CMP_API void cmp_destroy(void* session) {
  Session* s = static_cast<Session*>(session);
  if (!s) return;
  if (s->workspace) cudaFree(s->workspace);
  if (s->handle) cublasLtDestroy(s->handle);
  delete s;
}

CMP_API void cmp_plan_destroy(void* plan) {
  Plan* p = static_cast<Plan*>(plan);
  if (!p) return;
  if (p->a) cublasLtMatrixLayoutDestroy(p->a);
  if (p->b) cublasLtMatrixLayoutDestroy(p->b);
  if (p->c) cublasLtMatrixLayoutDestroy(p->c);
  if (p->desc) cublasLtMatmulDescDestroy(p->desc);
  delete p;
}

// c[m, n] (=|+=) a . b^T with a, b in either storage order; out_bf16 != 0 for a bf16 C.
CMP_API int cmp_plan(void* session, int64_t m, int64_t n, int64_t k, int a_mn, int b_mn, int out_bf16,
                     int accumulate, void** out) {
  Session* s = static_cast<Session*>(session);
  Plan* p = new (std::nothrow) Plan();
  if (!p) return fail("allocation", -1);
  p->beta = accumulate ? 1.f : 0.f;
  cublasStatus_t st = cublasLtMatmulDescCreate(&p->desc, CUBLAS_COMPUTE_32F, CUDA_R_32F);
  if (st != CUBLAS_STATUS_SUCCESS) { cmp_plan_destroy(p); return fail("cublasLtMatmulDescCreate", st); }
  const cublasOperation_t ta = b_mn ? CUBLAS_OP_N : CUBLAS_OP_T;    // first operand: this library's b
  const cublasOperation_t tb = a_mn ? CUBLAS_OP_T : CUBLAS_OP_N;    // second operand: this library's a
  cublasLtMatmulDescSetAttribute(p->desc, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta));
  cublasLtMatmulDescSetAttribute(p->desc, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb));
  st = b_mn ? cublasLtMatrixLayoutCreate(&p->a, CUDA_R_16BF, n, k, n) : cublasLtMatrixLayoutCreate(&p->a, CUDA_R_16BF, k, n, k);
  if (st == CUBLAS_STATUS_SUCCESS)
    st = a_mn ? cublasLtMatrixLayoutCreate(&p->b, CUDA_R_16BF, m, k, m) : cublasLtMatrixLayoutCreate(&p->b, CUDA_R_16BF, k, m, k);
  if (st == CUBLAS_STATUS_SUCCESS)
    st = cublasLtMatrixLayoutCreate(&p->c, out_bf16 ? CUDA_R_16BF : CUDA_R_32F, n, m, n);
  if (st != CUBLAS_STATUS_SUCCESS) { cmp_plan_destroy(p); return fail("cublasLtMatrixLayoutCreate", st); }
  cublasLtMatmulPreference_t pref = nullptr;
  st = cublasLtMatmulPreferenceCreate(&pref);
  if (st != CUBLAS_STATUS_SUCCESS) { cmp_plan_destroy(p); return fail("cublasLtMatmulPreferenceCreate", st); }
  size_t cap = kWorkspaceBytes;
  cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &cap, sizeof(cap));
  cublasLtMatmulHeuristicResult_t result;
  memset(&result, 0, sizeof(result));
  int found = 0;
  st = cublasLtMatmulAlgoGetHeuristic(s->handle, p->desc, p->a, p->b, p->c, p->c, pref, 1, &result, &found);
  cublasLtMatmulPreferenceDestroy(pref);
  if (st != CUBLAS_STATUS_SUCCESS || found < 1 || result.state != CUBLAS_STATUS_SUCCESS) {
    cmp_plan_destroy(p);
    return fail("cublasLtMatmulAlgoGetHeuristic", st != CUBLAS_STATUS_SUCCESS ? st : -2);
  }
  p->algo = result.algo;
  p->workspace = result.workspaceSize;
  *out = p;
  return 0;
}

CMP_API int cmp_run(void* session, void* plan, void* stream, const void* a, const void* b, void* c) {
  Session* s = static_cast<Session*>(session);
  Plan* p = static_cast<Plan*>(plan);
  const float alpha = 1.f;
  cublasStatus_t st = cublasLtMatmul(s->handle, p->desc, &alpha, b, p->a, a, p->b, &p->beta, c, p->c, c, p->c,
                                     &p->algo, s->workspace, kWorkspaceBytes, static_cast<cudaStream_t>(stream));
  if (st != CUBLAS_STATUS_SUCCESS) return fail("cublasLtMatmul", st);
  return 0;
}
