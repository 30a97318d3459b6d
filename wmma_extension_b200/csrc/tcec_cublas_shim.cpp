// libtcec_cublas_shim.so: cublasSgemm_v2, cublasSgemmBatched and cublasSgemmStridedBatched with
// cuBLAS's exact signatures, computed by the error-corrected tensor-core GEMM of libtcec_b200.
//
// Host code that calls cuBLAS for its FP32 GEMMs - the reference benchmarks its kernel against
// exactly such a call, cublasSgemmBatched(handle, CUBLAS_OP_T, CUBLAS_OP_N, m, n, k, &alpha, A, k,
// B, k, &beta, C, m, batch) (test/tcec/batch_gemm.cu:619-621) - switches by relinking: put this
// library before libcublas on the link line (or in LD_PRELOAD).  The three entry points below
// then take precedence; every other cuBLAS symbol still resolves to the real library, which this
// one also uses itself (stream and pointer mode of the handle).
//
//   policy   environment variable TCEC_CUBLAS_POLICY = fp16_ec (default) | tf32_ec | fp16_no_ec | tf32_no_ec
//   stream   the handle's (cublasSetStream is honoured)
//   scalars  host pointer mode only; with device pointer mode the call is passed to the real cuBLAS
//   CUBLAS_OP_C is CUBLAS_OP_T for real matrices
#include <cublas_v2.h>
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>

#include "../../include/tcec.h"

namespace {

template <class F>
F real_symbol(const char* name) {
  static_assert(sizeof(F) == sizeof(void*), "function pointer size");
  void* p = dlsym(RTLD_NEXT, name);
  F f;
  memcpy(&f, &p, sizeof(f));
  return f;
}

int shim_policy() {
  const char* e = std::getenv("TCEC_CUBLAS_POLICY");
  if (!e || !*e || !strcmp(e, "fp16_ec")) return TCEC_POLICY_FP16_EC;
  if (!strcmp(e, "tf32_ec")) return TCEC_POLICY_TF32_EC;
  if (!strcmp(e, "fp16_no_ec")) return TCEC_POLICY_FP16_NO_EC;
  if (!strcmp(e, "tf32_no_ec")) return TCEC_POLICY_TF32_NO_EC;
  return -1;
}

cublasStatus_t to_cublas(int st) {
  switch (st) {
    case TCEC_OK: return CUBLAS_STATUS_SUCCESS;
    case TCEC_ERR_INVALID_ARGUMENT: return CUBLAS_STATUS_INVALID_VALUE;
    case TCEC_ERR_UNSUPPORTED: return CUBLAS_STATUS_NOT_SUPPORTED;
    case TCEC_ERR_ALLOC: return CUBLAS_STATUS_ALLOC_FAILED;
    default: return CUBLAS_STATUS_EXECUTION_FAILED;
  }
}

// What the shim needs from the handle; false = hand the call to the real cuBLAS.
bool host_scalars(cublasHandle_t handle, cudaStream_t* stream) {
  typedef cublasStatus_t (*GetStream)(cublasHandle_t, cudaStream_t*);
  typedef cublasStatus_t (*GetMode)(cublasHandle_t, cublasPointerMode_t*);
  static GetStream get_stream = real_symbol<GetStream>("cublasGetStream_v2");
  static GetMode get_mode = real_symbol<GetMode>("cublasGetPointerMode_v2");
  if (!get_stream || !get_mode || !handle) return false;
  cublasPointerMode_t mode;
  if (get_mode(handle, &mode) != CUBLAS_STATUS_SUCCESS || mode != CUBLAS_POINTER_MODE_HOST) return false;
  return get_stream(handle, stream) == CUBLAS_STATUS_SUCCESS;
}

int op_flag(cublasOperation_t op) { return op == CUBLAS_OP_N ? 0 : (op == CUBLAS_OP_T ? 1 : (op == CUBLAS_OP_C ? 2 : -1)); }
int op_layout(cublasOperation_t op) { return op == CUBLAS_OP_N ? TCEC_COL_MAJOR : TCEC_ROW_MAJOR; }

}  // namespace

extern "C" {

cublasStatus_t cublasSgemm_v2(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m, int n,
                              int k, const float* alpha, const float* A, int lda, const float* B, int ldb,
                              const float* beta, float* C, int ldc) {
  cudaStream_t stream = nullptr;
  const int policy = shim_policy();
  if (policy < 0 || !host_scalars(handle, &stream)) {
    typedef cublasStatus_t (*Fn)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const float*,
                                 const float*, int, const float*, int, const float*, float*, int);
    static Fn real = real_symbol<Fn>("cublasSgemm_v2");
    return real ? real(handle, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc)
                : CUBLAS_STATUS_NOT_INITIALIZED;
  }
  return to_cublas(tcec_sgemm_cublas(op_flag(transa), op_flag(transb), m, n, k, alpha, A, lda, B, ldb, beta, C, ldc,
                                     policy, stream));
}

cublasStatus_t cublasSgemmBatched(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb, int m,
                                  int n, int k, const float* alpha, const float* const Aarray[], int lda,
                                  const float* const Barray[], int ldb, const float* beta, float* const Carray[],
                                  int ldc, int batchCount) {
  cudaStream_t stream = nullptr;
  const int policy = shim_policy();
  if (policy < 0 || !host_scalars(handle, &stream)) {
    typedef cublasStatus_t (*Fn)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const float*,
                                 const float* const[], int, const float* const[], int, const float*, float* const[], int,
                                 int);
    static Fn real = real_symbol<Fn>("cublasSgemmBatched");
    return real ? real(handle, transa, transb, m, n, k, alpha, Aarray, lda, Barray, ldb, beta, Carray, ldc, batchCount)
                : CUBLAS_STATUS_NOT_INITIALIZED;
  }
  return to_cublas(tcec_sgemm_batched_cublas(op_flag(transa), op_flag(transb), m, n, k, alpha, Aarray, lda, Barray, ldb,
                                             beta, Carray, ldc, batchCount, policy, stream));
}

cublasStatus_t cublasSgemmStridedBatched(cublasHandle_t handle, cublasOperation_t transa, cublasOperation_t transb,
                                         int m, int n, int k, const float* alpha, const float* A, int lda,
                                         long long int strideA, const float* B, int ldb, long long int strideB,
                                         const float* beta, float* C, int ldc, long long int strideC, int batchCount) {
  cudaStream_t stream = nullptr;
  const int policy = shim_policy();
  if (policy < 0 || !host_scalars(handle, &stream) || op_flag(transa) < 0 || op_flag(transb) < 0) {
    typedef cublasStatus_t (*Fn)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const float*,
                                 const float*, int, long long int, const float*, int, long long int, const float*, float*,
                                 int, long long int, int);
    static Fn real = real_symbol<Fn>("cublasSgemmStridedBatched");
    return real ? real(handle, transa, transb, m, n, k, alpha, A, lda, strideA, B, ldb, strideB, beta, C, ldc, strideC,
                       batchCount)
                : CUBLAS_STATUS_NOT_INITIALIZED;
  }
  if (!alpha || !beta) return CUBLAS_STATUS_INVALID_VALUE;
  return to_cublas(tcec_sgemm_strided_batched(op_layout(transa), op_layout(transb), TCEC_COL_MAJOR, m, n, k, *alpha, A,
                                              lda, strideA, B, ldb, strideB, *beta, C, ldc, strideC, batchCount, policy,
                                              stream));
}

}  // extern "C"
