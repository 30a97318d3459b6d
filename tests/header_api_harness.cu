// One-warp kernels written against THIS repository's mtk::wmma::tcec headers, exposed through a
// small C ABI so the header surface can be checked from pytest.  Same entry-point shapes as
// oracle/ref_harness.cu, which drives the reference's headers, so the two can be compared.
// TEST INFRASTRUCTURE (built into tests/_build/libtcec_header_test.so by __graft_entry__.build()).
#include <wmma_extension/tcec/tcec.hpp>

#include <cstdio>

namespace {
namespace tc = mtk::wmma::tcec;
using tf32 = nvcuda::wmma::precision::tf32;

// mode bits: 1 = load A from column-major memory, 2 = load B from row-major memory,
//            4 = C/D column-major, 8 = use the *_with_mul forms (A scaled by 2, D by 0.5),
//            16 = mma_rz_sync, 32 = mma_rn_sync (else mma_sync)
template <class T, class Policy, int N>
__global__ void warp_mma_kernel(float* d_ptr, const float* a_ptr, const float* b_ptr, const float* c_ptr,
                                int mode) {
  __shared__ float smem[N * N];
  tc::fragment<nvcuda::wmma::matrix_a, N, N, N, T, nvcuda::wmma::row_major, Policy> frag_a;
  tc::fragment<nvcuda::wmma::matrix_b, N, N, N, T, nvcuda::wmma::col_major, Policy> frag_b;
  tc::fragment<nvcuda::wmma::accumulator, N, N, N, T, void, Policy> frag_c, frag_d;
  for (unsigned i = threadIdx.x; i < N * N; i += 32) smem[i] = a_ptr[i];
  __syncwarp();
  if (mode & 8) {
    if (mode & 1) tc::load_matrix_sync_with_mul<nvcuda::wmma::col_major>(frag_a, smem, N, 2.0f);
    else tc::load_matrix_sync_with_mul(frag_a, smem, N, 2.0f);
  } else {
    if (mode & 1) tc::load_matrix_sync<nvcuda::wmma::col_major>(frag_a, smem, N);
    else tc::load_matrix_sync(frag_a, smem, N);
  }
  for (unsigned i = threadIdx.x; i < N * N; i += 32) smem[i] = b_ptr[i];
  __syncwarp();
  if (mode & 2) tc::load_matrix_sync<nvcuda::wmma::row_major>(frag_b, smem, N);
  else tc::load_matrix_sync(frag_b, smem, N);
  const auto cd_layout = (mode & 4) ? nvcuda::wmma::mem_col_major : nvcuda::wmma::mem_row_major;
  tc::fill_fragment(frag_d, 7.0f);  // must be overwritten
  if (c_ptr) {
    for (unsigned i = threadIdx.x; i < N * N; i += 32) smem[i] = c_ptr[i];
    __syncwarp();
    tc::load_matrix_sync(frag_c, smem, N, cd_layout);
    if (mode & 16) tc::mma_rz_sync(frag_d, frag_a, frag_b, frag_c);
    else if (mode & 32) tc::mma_rn_sync(frag_d, frag_a, frag_b, frag_c);
    else tc::mma_sync(frag_d, frag_a, frag_b, frag_c);
  } else {
    if (mode & 16) tc::mma_rz_sync(frag_d, frag_a, frag_b);
    else if (mode & 32) tc::mma_rn_sync(frag_d, frag_a, frag_b);
    else tc::mma_sync(frag_d, frag_a, frag_b);
  }
  if (mode & 8) tc::store_matrix_sync_with_mul(smem, frag_d, N, 0.5f, cd_layout);
  else tc::store_matrix_sync(smem, frag_d, N, cd_layout);
  for (unsigned i = threadIdx.x; i < N * N; i += 32) d_ptr[i] = smem[i];
  tc::fill_zero(frag_d);
}

// y = A x through load_vector / store_vector (call sequence of the reference's test/tcec/matvec.cu:21-50)
template <class T, class Policy, int N>
__global__ void matvec_kernel(float* y_ptr, const float* a_ptr, const float* x_ptr) {
  __shared__ float smem[N * N];
  tc::fragment<nvcuda::wmma::matrix_a, N, N, N, T, nvcuda::wmma::col_major, Policy> frag_a;
  tc::fragment<nvcuda::wmma::matrix_b, N, N, N, T, nvcuda::wmma::col_major, Policy> frag_x;
  tc::fragment<nvcuda::wmma::accumulator, N, N, N, T, void, Policy> frag_y;
  for (unsigned i = threadIdx.x; i < N * N; i += 32) smem[i] = a_ptr[i];
  __syncwarp();
  tc::load_matrix_sync(frag_a, smem, N);
  __syncwarp();
  for (unsigned i = threadIdx.x; i < N; i += 32) smem[i] = x_ptr[i];
  __syncwarp();
  tc::fill_zero(frag_x);
  tc::load_vector(frag_x, smem);
  tc::mma_sync(frag_y, frag_a, frag_x);
  tc::store_vector(smem, frag_y, nvcuda::wmma::mem_col_major);
  for (unsigned i = threadIdx.x; i < N; i += 32) y_ptr[i] = smem[i];
}

// writes every x(i) / dx(i) (dx scaled back) so the element map can be checked: out[lane][i]
template <class Use, class T, class Policy, int N>
__global__ void dump_kernel(float* hi_out, float* lo_out, const float* src) {
  using L = typename std::conditional<std::is_same<Use, nvcuda::wmma::accumulator>::value, void,
                                      nvcuda::wmma::row_major>::type;
  tc::fragment<Use, N, N, N, T, L, Policy> frag;
  tc::load_matrix_sync<nvcuda::wmma::row_major>(frag, src, N);
  for (unsigned i = 0; i < frag.num_elements; i++) {
    hi_out[threadIdx.x * frag.num_elements + i] = static_cast<float>(frag.x(i));
    if constexpr (decltype(frag)::error_corrected)
      lo_out[threadIdx.x * frag.num_elements + i] = static_cast<float>(frag.dx(i));
  }
}

// Element map of the op_wmma sub-fragments against nvcuda::wmma::load_matrix_sync on the running GPU:
// the same index-coded matrix is loaded both ways; *bad counts registers that differ.
template <class Use, class T, class Layout, int FK>
__global__ void wmma_map_kernel(int* bad) {
  using Policy = tc::Policy<tc::op_wmma, tc::without_ec, 16, 16, FK>;
  constexpr int R = tc::detail::select_value<Use, 16, FK, 16>::value;
  constexpr int C = tc::detail::select_value<Use, FK, 16, 16>::value;
  constexpr bool kAcc = std::is_same<Use, nvcuda::wmma::accumulator>::value;
  constexpr bool kCol = std::is_same<Layout, nvcuda::wmma::col_major>::value;
  using Elem = typename std::conditional<kAcc || !std::is_same<T, half>::value, float, half>::type;
  __shared__ float src[16 * 16];
  __shared__ Elem coded[16 * 16];
  for (int e = threadIdx.x; e < R * C; e += 32) {
    const int i = e / C, j = e % C;
    const float v = static_cast<float>(e + 1);  // exactly representable in half and tf32
    const int at = kCol ? i + j * R : i * C + j;
    src[at] = v;
    coded[at] = static_cast<Elem>(v);
  }
  __syncwarp();
  const unsigned ldm = kCol ? R : C;
  using L = typename std::conditional<kAcc, void, Layout>::type;
  tc::fragment<Use, 16, 16, FK, T, L, Policy> frag;
  using sub_t = typename decltype(frag)::sub_frag_t;
  sub_t ref;
  if constexpr (kAcc) {
    tc::load_matrix_sync(frag, src, ldm, kCol ? nvcuda::wmma::mem_col_major : nvcuda::wmma::mem_row_major);
    nvcuda::wmma::load_matrix_sync(ref, coded, ldm, kCol ? nvcuda::wmma::mem_col_major : nvcuda::wmma::mem_row_major);
  } else {
    tc::load_matrix_sync(frag, src, ldm);
    nvcuda::wmma::load_matrix_sync(ref, coded, ldm);
  }
  static_assert(std::is_same<sub_t, nvcuda::wmma::fragment<Use, 16, 16, FK, typename sub_t::element_type, L>>::value,
                "op_wmma sub-fragments are nvcuda::wmma fragments");
  int n = 0;
  for (unsigned i = 0; i < ref.num_elements; i++)
    if (static_cast<float>(frag.sub_frag[0].x[i]) != static_cast<float>(ref.x[i])) ++n;
  static_assert(decltype(frag)::num_elements == sub_t::num_elements, "one sub-fragment");
  if (n) atomicAdd(bad, n);
}

template <class T, class EC, class OP>
int launch(float* d, const float* a, const float* b, const float* c, int mode) {
  using Policy = typename tc::default_policy<T, EC, OP>::type;
  warp_mma_kernel<T, Policy, 32><<<1, 32>>>(d, a, b, c, mode);
  return (int)cudaGetLastError();
}
template <class T, class EC, class OP>
int launch_matvec(float* y, const float* a, const float* x) {
  using Policy = typename tc::default_policy<T, EC, OP>::type;
  matvec_kernel<T, Policy, 32><<<1, 32>>>(y, a, x);
  return (int)cudaGetLastError();
}
}  // namespace

extern "C" {
// a: 32x32 A as the chosen memory order says, b: 32x32 B likewise, c may be NULL.
int hdr_warp_mma(int tf, int op_wmma, int ec, float* d, const float* a, const float* b, const float* c, int mode) {
  const int key = (tf ? 4 : 0) | (op_wmma ? 2 : 0) | (ec ? 1 : 0);
  switch (key) {
    case 0: return launch<half, tc::without_ec, tc::op_mma>(d, a, b, c, mode);
    case 1: return launch<half, tc::with_ec, tc::op_mma>(d, a, b, c, mode);
    case 2: return launch<half, tc::without_ec, tc::op_wmma>(d, a, b, c, mode);
    case 3: return launch<half, tc::with_ec, tc::op_wmma>(d, a, b, c, mode);
    case 4: return launch<tf32, tc::without_ec, tc::op_mma>(d, a, b, c, mode);
    case 5: return launch<tf32, tc::with_ec, tc::op_mma>(d, a, b, c, mode);
    case 6: return launch<tf32, tc::without_ec, tc::op_wmma>(d, a, b, c, mode);
    default: return launch<tf32, tc::with_ec, tc::op_wmma>(d, a, b, c, mode);
  }
}
int hdr_matvec(int tf, int op_wmma, int ec, float* y, const float* a_colmajor, const float* x) {
  const int key = (tf ? 4 : 0) | (op_wmma ? 2 : 0) | (ec ? 1 : 0);
  switch (key) {
    case 0: return launch_matvec<half, tc::without_ec, tc::op_mma>(y, a_colmajor, x);
    case 1: return launch_matvec<half, tc::with_ec, tc::op_mma>(y, a_colmajor, x);
    case 2: return launch_matvec<half, tc::without_ec, tc::op_wmma>(y, a_colmajor, x);
    case 3: return launch_matvec<half, tc::with_ec, tc::op_wmma>(y, a_colmajor, x);
    case 4: return launch_matvec<tf32, tc::without_ec, tc::op_mma>(y, a_colmajor, x);
    case 5: return launch_matvec<tf32, tc::with_ec, tc::op_mma>(y, a_colmajor, x);
    case 6: return launch_matvec<tf32, tc::without_ec, tc::op_wmma>(y, a_colmajor, x);
    default: return launch_matvec<tf32, tc::with_ec, tc::op_wmma>(y, a_colmajor, x);
  }
}
// element map of the op_mma half fragments: use 0 = matrix_a, 1 = matrix_b, 2 = accumulator
int hdr_dump(int use, float* hi, float* lo, const float* src_rowmajor_32x32) {
  using Policy = typename tc::default_policy<half, tc::with_ec, tc::op_mma>::type;
  if (use == 0) dump_kernel<nvcuda::wmma::matrix_a, half, Policy, 32><<<1, 32>>>(hi, lo, src_rowmajor_32x32);
  else if (use == 1) dump_kernel<nvcuda::wmma::matrix_b, half, Policy, 32><<<1, 32>>>(hi, lo, src_rowmajor_32x32);
  else dump_kernel<nvcuda::wmma::accumulator, half, Policy, 32><<<1, 32>>>(hi, lo, src_rowmajor_32x32);
  return (int)cudaGetLastError();
}
// number of registers of the op_wmma fragments that disagree with nvcuda::wmma::load_matrix_sync (all nine kinds)
int hdr_wmma_map_mismatches(int* bad_dev) {
  using namespace nvcuda::wmma;
  wmma_map_kernel<matrix_a, half, row_major, 16><<<1, 32>>>(bad_dev);
  wmma_map_kernel<matrix_a, half, col_major, 16><<<1, 32>>>(bad_dev);
  wmma_map_kernel<matrix_b, half, row_major, 16><<<1, 32>>>(bad_dev);
  wmma_map_kernel<matrix_b, half, col_major, 16><<<1, 32>>>(bad_dev);
  wmma_map_kernel<accumulator, half, row_major, 16><<<1, 32>>>(bad_dev);
  wmma_map_kernel<accumulator, half, col_major, 16><<<1, 32>>>(bad_dev);
  wmma_map_kernel<matrix_a, tf32, row_major, 8><<<1, 32>>>(bad_dev);
  wmma_map_kernel<matrix_a, tf32, col_major, 8><<<1, 32>>>(bad_dev);
  wmma_map_kernel<matrix_b, tf32, row_major, 8><<<1, 32>>>(bad_dev);
  wmma_map_kernel<matrix_b, tf32, col_major, 8><<<1, 32>>>(bad_dev);
  wmma_map_kernel<accumulator, tf32, row_major, 8><<<1, 32>>>(bad_dev);
  return (int)cudaGetLastError();
}
// the same for the op_mma tf32 fragments (m16n8k8)
int hdr_dump_tf32(int use, float* hi, float* lo, const float* src_rowmajor_32x32) {
  using Policy = typename tc::default_policy<tf32, tc::with_ec, tc::op_mma>::type;
  if (use == 0) dump_kernel<nvcuda::wmma::matrix_a, tf32, Policy, 32><<<1, 32>>>(hi, lo, src_rowmajor_32x32);
  else if (use == 1) dump_kernel<nvcuda::wmma::matrix_b, tf32, Policy, 32><<<1, 32>>>(hi, lo, src_rowmajor_32x32);
  else dump_kernel<nvcuda::wmma::accumulator, tf32, Policy, 32><<<1, 32>>>(hi, lo, src_rowmajor_32x32);
  return (int)cudaGetLastError();
}
}
