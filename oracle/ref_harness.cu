// Drives the UNMODIFIED reference (wmma_extension headers and its batched
// example kernel) from where it lies, so the reference itself can be run on the
// GPU box: to produce golden fixtures, and as the GPU comparator of the parity
// tests.  TEST INFRASTRUCTURE ONLY.  Built by oracle/Makefile into
// oracle/_ref/libtcec_ref.so with -I<reference>/include -I<reference>/test/tcec;
// no reference source is copied.
//
// Entry points (all pointers are device pointers):
//   ref_split      cast<T> / correction_scale_0<T> exactly as load_matrix_sync
//                  applies them (include/wmma_extension/tcec/tcec.hpp:219-223)
//   ref_warp_mma   one warp, 32x32x32, the reference's fragment API end to end
//                  (same call sequence as test/tcec/mma.cu:21-96)
//   ref_bgemm      the reference's bgemm_kernel via gen_bgemm_config/launch_bgemm
//                  (test/tcec/batch_gemm.cu:261-443)
#define main ref_batch_gemm_main_unused
#include "batch_gemm.cu"
#undef main

namespace {

template <class T>
__global__ void ref_split_kernel(const float* in, float* hi, float* lo, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = in[i];
    const auto hv = mtk::wmma::detail::common::cast<T>(v);
    const auto dhv = mtk::wmma::detail::common::cast<T>(
        mtk::wmma::tcec::detail::correction_scale_0<T>(v - mtk::wmma::detail::common::cast<float>(hv)));
    hi[i] = mtk::wmma::detail::common::cast<float>(hv);
    lo[i] = mtk::wmma::detail::common::cast<float>(dhv);
  }
}

// A: 32x32 row-major, B: 32x32 col-major, C/D: row-major. One warp.
template <class T, class Policy>
__global__ void ref_warp_mma_kernel(float* d_ptr, const float* a_ptr, const float* b_ptr,
                                    const float* c_ptr, int rz) {
  constexpr unsigned N = 32;
  __shared__ float smem[N * N];
  mtk::wmma::tcec::fragment<nvcuda::wmma::matrix_a, N, N, N, T, nvcuda::wmma::row_major, Policy> frag_a;
  mtk::wmma::tcec::fragment<nvcuda::wmma::matrix_b, N, N, N, T, nvcuda::wmma::col_major, Policy> frag_b;
  mtk::wmma::tcec::fragment<nvcuda::wmma::accumulator, N, N, N, T, void, Policy> frag_c, frag_d;
  for (unsigned i = threadIdx.x; i < N * N; i += 32) smem[i] = a_ptr[i];
  __syncwarp();
  mtk::wmma::tcec::load_matrix_sync<nvcuda::wmma::row_major>(frag_a, smem, N);
  for (unsigned i = threadIdx.x; i < N * N; i += 32) smem[i] = b_ptr[i];
  __syncwarp();
  mtk::wmma::tcec::load_matrix_sync<nvcuda::wmma::col_major>(frag_b, smem, N);
  if (c_ptr) {
    for (unsigned i = threadIdx.x; i < N * N; i += 32) smem[i] = c_ptr[i];
    __syncwarp();
    mtk::wmma::tcec::load_matrix_sync(frag_c, smem, N, nvcuda::wmma::mem_row_major);
  } else {
    mtk::wmma::tcec::fill_zero(frag_c);
  }
  mtk::wmma::tcec::fill_zero(frag_d);
  if (rz)
    mtk::wmma::tcec::mma_rz_sync(frag_d, frag_a, frag_b, frag_c);
  else
    mtk::wmma::tcec::mma_sync(frag_d, frag_a, frag_b, frag_c);
  mtk::wmma::tcec::store_matrix_sync(smem, frag_d, N, nvcuda::wmma::mem_row_major);
  for (unsigned i = threadIdx.x; i < N * N; i += 32) d_ptr[i] = smem[i];
}

template <class T, class EC, class OP>
int launch_warp(float* d, const float* a, const float* b, const float* c, int rz, cudaStream_t s) {
  using Policy = typename mtk::wmma::tcec::detail::default_policy<T, EC, OP>::type;
  ref_warp_mma_kernel<T, Policy><<<1, 32, 0, s>>>(d, a, b, c, rz);
  return (int)cudaGetLastError();
}

template <class T, unsigned PER>
int launch_ref_bgemm(unsigned m, unsigned n, unsigned k, float alpha, const float* const* a, unsigned lda,
                     const float* const* b, unsigned ldb, float beta, float* const* c, unsigned ldc,
                     unsigned batch) {
  using Policy = typename mtk::wmma::tcec::detail::default_policy<T, mtk::wmma::tcec::with_ec,
                                                                  mtk::wmma::tcec::op_mma>::type;
  try {
    const auto conf = gen_bgemm_config<128, 128, 32, 32, 32, 32, 256, PER, PER, 1, 1, 1, T, Policy>();
    launch_bgemm(conf, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, batch);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ref_bgemm: %s\n", e.what());
    return 1;
  }
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

int ref_split(const float* in, float* hi, float* lo, size_t n, int tf32) {
  if (tf32)
    ref_split_kernel<nvcuda::wmma::precision::tf32><<<256, 256>>>(in, hi, lo, n);
  else
    ref_split_kernel<half><<<256, 256>>>(in, hi, lo, n);
  return (int)cudaGetLastError();
}

// op: 0 = op_mma, 1 = op_wmma.  c may be NULL.  rz: use mma_rz_sync.
int ref_warp_mma(int tf32, int op, int ec, float* d, const float* a, const float* b, const float* c, int rz) {
  using namespace mtk::wmma::tcec;
  using tf = nvcuda::wmma::precision::tf32;
  const int key = (tf32 ? 4 : 0) | (op ? 2 : 0) | (ec ? 1 : 0);
  switch (key) {
    case 0: return launch_warp<half, without_ec, op_mma>(d, a, b, c, rz, 0);
    case 1: return launch_warp<half, with_ec, op_mma>(d, a, b, c, rz, 0);
    case 2: return launch_warp<half, without_ec, op_wmma>(d, a, b, c, rz, 0);
    case 3: return launch_warp<half, with_ec, op_wmma>(d, a, b, c, rz, 0);
    case 4: return launch_warp<tf, without_ec, op_mma>(d, a, b, c, rz, 0);
    case 5: return launch_warp<tf, with_ec, op_mma>(d, a, b, c, rz, 0);
    case 6: return launch_warp<tf, without_ec, op_wmma>(d, a, b, c, rz, 0);
    default: return launch_warp<tf, with_ec, op_wmma>(d, a, b, c, rz, 0);
  }
}

// Layout fixed by the reference kernel: A row-major (lda >= k), B col-major
// (ldb >= k), C col-major (ldc >= m).  `per` = CTAs per matrix along m and along n
// (the reference's BLOCK_M_PER_MATRIX = BLOCK_N_PER_MATRIX): 4 (its own test
// value, test/tcec/batch_gemm.cu:660), 16, 32 or 128.  Runs on the default stream.
int ref_bgemm(int tf32, int per, unsigned m, unsigned n, unsigned k, float alpha, const float* const* a,
              unsigned lda, const float* const* b, unsigned ldb, float beta, float* const* c, unsigned ldc,
              unsigned batch) {
  using tf = nvcuda::wmma::precision::tf32;
#define REF_CASE(P)                                                                             \
  case P:                                                                                       \
    return tf32 ? launch_ref_bgemm<tf, P>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, batch)  \
                : launch_ref_bgemm<half, P>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, batch);
  switch (per) {
    REF_CASE(1)
    REF_CASE(4)
    REF_CASE(16)
    REF_CASE(32)
    REF_CASE(128)
    default: return 2;
  }
#undef REF_CASE
}

}  // extern "C"
