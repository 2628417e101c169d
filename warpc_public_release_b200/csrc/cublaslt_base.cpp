// The library baseline: cuBLASLt on the same problem, C[M,N] f32 row-major = A[M,K] f16 . Bt[N,K]^T f16,
// alpha 1, beta 0, fp32 compute -- what the reference measures itself against
// (backend/node/cublas_q7.cpp:43-63: every algorithm the heuristic returns is a candidate and the
// fastest exactly-correct one is kept; README.md:516-523).  Row-major C = A . Bt^T is the
// column-major product C^T[N,M] = op_T(Bt viewed K x N) . (A viewed K x M).
// A plain library call: it is a baseline beside the hand-written kernels, never on their path.
#include <cublasLt.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <new>

namespace {
struct Base {
  cublasLtHandle_t lt = nullptr;
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
  cublasLtMatmulHeuristicResult_t algos[32];
  int n_algos = 0;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  const void *a = nullptr, *bt = nullptr;
  void* c = nullptr;
};
}  // namespace

extern "C" int wc_destroy(void* handle) {
  Base* b = static_cast<Base*>(handle);
  if (!b) return 0;
  if (b->la) cublasLtMatrixLayoutDestroy(b->la);
  if (b->lb) cublasLtMatrixLayoutDestroy(b->lb);
  if (b->lc) cublasLtMatrixLayoutDestroy(b->lc);
  if (b->op) cublasLtMatmulDescDestroy(b->op);
  if (b->lt) cublasLtDestroy(b->lt);
  if (b->workspace) cudaFree(b->workspace);
  delete b;
  return 0;
}

// Returns 0 and the number of candidate algorithms, or a cublasStatus_t / 1000 + cudaError_t.
extern "C" int wc_create(int M, int N, int K, const void* dA, const void* dBt, void* dC, size_t workspace_bytes, void** handle,
                         int* n_algos) {
  if (!handle || !n_algos) return -1;
  Base* b = new (std::nothrow) Base();
  if (!b) return -1;
  b->a = dA, b->bt = dBt, b->c = dC, b->workspace_bytes = workspace_bytes;
  int st = 0;
  auto ok = [&](cublasStatus_t s) {
    if (s != CUBLAS_STATUS_SUCCESS && st == 0) st = int(s);
    return s == CUBLAS_STATUS_SUCCESS;
  };
  const cublasOperation_t trans = CUBLAS_OP_T, none = CUBLAS_OP_N;
  if (workspace_bytes && cudaMalloc(&b->workspace, workspace_bytes) != cudaSuccess) st = 1000;
  if (st == 0 && ok(cublasLtCreate(&b->lt)) && ok(cublasLtMatmulDescCreate(&b->op, CUBLAS_COMPUTE_32F, CUDA_R_32F)) &&
      ok(cublasLtMatmulDescSetAttribute(b->op, CUBLASLT_MATMUL_DESC_TRANSA, &trans, sizeof trans)) &&
      ok(cublasLtMatmulDescSetAttribute(b->op, CUBLASLT_MATMUL_DESC_TRANSB, &none, sizeof none)) &&
      ok(cublasLtMatrixLayoutCreate(&b->la, CUDA_R_16F, K, N, K)) && ok(cublasLtMatrixLayoutCreate(&b->lb, CUDA_R_16F, K, M, K)) &&
      ok(cublasLtMatrixLayoutCreate(&b->lc, CUDA_R_32F, N, M, N))) {
    cublasLtMatmulPreference_t pref = nullptr;
    if (ok(cublasLtMatmulPreferenceCreate(&pref))) {
      ok(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_bytes, sizeof workspace_bytes));
      ok(cublasLtMatmulAlgoGetHeuristic(b->lt, b->op, b->la, b->lb, b->lc, b->lc, pref, 32, b->algos, &b->n_algos));
      cublasLtMatmulPreferenceDestroy(pref);
    }
  }
  if (st != 0) {
    wc_destroy(b);
    return st;
  }
  *handle = b;
  *n_algos = b->n_algos;
  return 0;
}

extern "C" int wc_run(void* handle, int algo, void* cuda_stream) {
  Base* b = static_cast<Base*>(handle);
  if (!b || algo < 0 || algo >= b->n_algos) return -1;
  const float alpha = 1.0f, beta = 0.0f;
  return int(cublasLtMatmul(b->lt, b->op, &alpha, b->bt, b->la, b->a, b->lb, &beta, b->c, b->lc, b->c, b->lc, &b->algos[algo].algo,
                            b->workspace, b->workspace_bytes, static_cast<cudaStream_t>(cuda_stream)));
}

extern "C" int wc_version() { return int(cublasLtGetVersion()); }
