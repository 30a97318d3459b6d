// Complex fragments of the TCEC warp-level API: a pair of real fragments, loaded from and stored
// to interleaved cuComplex arrays, multiplied with four real error-corrected products.
//
// Same surface as the reference's include/wmma_extension/tcec/complex.hpp (fragment_complex
// :12-17; fill :19-37; loads :40-394; stores :396-606; mma in its three rounding variants
// :608-727), including the order of the four real products (:617-623, :636-643), so results
// agree with the reference's to the bit wherever its real path does.
#ifndef TCEC_B200_COMPLEX_HPP
#define TCEC_B200_COMPLEX_HPP
#include <cuComplex.h>

#include "tcec.hpp"

namespace mtk {
namespace wmma {
namespace tcec {

template <class Use, int m, int n, int k, class T, class Layout = void,
          class Policy_ = typename mtk::wmma::tcec::detail::default_policy<T>::type>
struct fragment_complex {
  using frag_t = mtk::wmma::tcec::fragment<Use, m, n, k, T, Layout, Policy_>;
  static constexpr unsigned num_sub_frag_m = frag_t::num_sub_frag_m;
  static constexpr unsigned num_sub_frag_n = frag_t::num_sub_frag_n;
  frag_t real, imag;
};

#define TCEC_CFRAG(USE, LAYOUT) fragment_complex<USE, m, n, k, T, LAYOUT, Policy<Op, EC, fm, fn, fk>>
#define TCEC_TPARAMS int m, int n, int k, class T, class Op, class EC, int fm, int fn, int fk

template <class Use, class Layout, TCEC_TPARAMS>
__device__ void fill_fragment(TCEC_CFRAG(Use, Layout) & frag, const float real, const float imag = 0.0f) {
  fill_fragment(frag.real, real);
  fill_fragment(frag.imag, imag);
}
template <class Use, class Layout, TCEC_TPARAMS>
__device__ void fill_zero(TCEC_CFRAG(Use, Layout) & frag) {
  fill_zero(frag.real);
  fill_zero(frag.imag);
}

// ---------------------------------------------------------------- loads
namespace detail {
template <class MemLayout, class Use, class Layout, TCEC_TPARAMS>
__device__ void load_complex(TCEC_CFRAG(Use, Layout) & frag, const cuComplex* const ptr, const unsigned ldm,
                             const float mul, const bool use_mul) {
  load_with<MemLayout>(frag.real, [ptr](unsigned idx) { return ptr[idx].x; }, ldm, mul, use_mul);
  load_with<MemLayout>(frag.imag, [ptr](unsigned idx) { return ptr[idx].y; }, ldm, mul, use_mul);
}
}  // namespace detail

template <class MemLayout, class Use, class Layout, TCEC_TPARAMS,
          typename std::enable_if<detail::is_layout<MemLayout>::value, int>::type = 0>
__device__ void load_matrix_sync(TCEC_CFRAG(Use, Layout) & frag, const cuComplex* const ptr, const unsigned ldm,
                                 const bool sync = true) {
  detail::load_complex<MemLayout>(frag, ptr, ldm, 1.0f, false);
  if (sync) __syncwarp();
}
template <class Use, class Layout, TCEC_TPARAMS,
          typename std::enable_if<detail::is_layout<Layout>::value, int>::type = 0>
__device__ void load_matrix_sync(TCEC_CFRAG(Use, Layout) & frag, const cuComplex* const ptr, const unsigned ldm,
                                 const bool sync = true) {
  load_matrix_sync<Layout>(frag, ptr, ldm, sync);
}
template <TCEC_TPARAMS>
__device__ void load_matrix_sync(TCEC_CFRAG(nvcuda::wmma::accumulator, void) & frag, const cuComplex* const ptr,
                                 const unsigned ldm, const nvcuda::wmma::layout_t layout, const bool sync = true) {
  if (layout == nvcuda::wmma::mem_col_major)
    load_matrix_sync<nvcuda::wmma::col_major>(frag, ptr, ldm, sync);
  else
    load_matrix_sync<nvcuda::wmma::row_major>(frag, ptr, ldm, sync);
}
// real multiplier applied to both parts before the split
template <class MemLayout, class Use, class Layout, TCEC_TPARAMS,
          typename std::enable_if<detail::is_layout<MemLayout>::value, int>::type = 0>
__device__ void load_matrix_sync_with_mul(TCEC_CFRAG(Use, Layout) & frag, const cuComplex* const ptr,
                                          const unsigned ldm, const float mul, const bool sync = true) {
  detail::load_complex<MemLayout>(frag, ptr, ldm, mul, true);
  if (sync) __syncwarp();
}
template <class Use, class Layout, TCEC_TPARAMS,
          typename std::enable_if<detail::is_layout<Layout>::value, int>::type = 0>
__device__ void load_matrix_sync_with_mul(TCEC_CFRAG(Use, Layout) & frag, const cuComplex* const ptr,
                                          const unsigned ldm, const float mul, const bool sync = true) {
  load_matrix_sync_with_mul<Layout>(frag, ptr, ldm, mul, sync);
}

// ---------------------------------------------------------------- stores
namespace detail {
template <class MemLayout, TCEC_TPARAMS>
__device__ void store_complex(cuComplex* const ptr, const TCEC_CFRAG(nvcuda::wmma::accumulator, void) & frag,
                              const unsigned ldm, const float mul, const bool use_mul) {
  store_with<MemLayout>([ptr](unsigned idx, float v) { ptr[idx].x = v; }, frag.real, ldm, mul, use_mul);
  store_with<MemLayout>([ptr](unsigned idx, float v) { ptr[idx].y = v; }, frag.imag, ldm, mul, use_mul);
}
}  // namespace detail

template <class MemLayout, TCEC_TPARAMS, typename std::enable_if<detail::is_layout<MemLayout>::value, int>::type = 0>
__device__ void store_matrix_sync(cuComplex* const ptr, const TCEC_CFRAG(nvcuda::wmma::accumulator, void) & frag,
                                  const unsigned ldm, const bool sync = true) {
  detail::store_complex<MemLayout>(ptr, frag, ldm, 1.0f, false);
  if (sync) __syncwarp();
}
template <TCEC_TPARAMS>
__device__ void store_matrix_sync(cuComplex* const ptr, const TCEC_CFRAG(nvcuda::wmma::accumulator, void) & frag,
                                  const unsigned ldm, const nvcuda::wmma::layout_t layout, const bool sync = true) {
  if (layout == nvcuda::wmma::mem_col_major)
    store_matrix_sync<nvcuda::wmma::col_major>(ptr, frag, ldm, sync);
  else
    store_matrix_sync<nvcuda::wmma::row_major>(ptr, frag, ldm, sync);
}
template <class MemLayout, TCEC_TPARAMS, typename std::enable_if<detail::is_layout<MemLayout>::value, int>::type = 0>
__device__ void store_matrix_sync(cuComplex* const ptr, const TCEC_CFRAG(nvcuda::wmma::accumulator, void) & frag,
                                  const unsigned ldm, const float mul, const bool sync = true) {
  detail::store_complex<MemLayout>(ptr, frag, ldm, mul, true);
  if (sync) __syncwarp();
}
template <TCEC_TPARAMS>
__device__ void store_matrix_sync(cuComplex* const ptr, const TCEC_CFRAG(nvcuda::wmma::accumulator, void) & frag,
                                  const unsigned ldm, const float mul, const nvcuda::wmma::layout_t layout,
                                  const bool sync = true) {
  if (layout == nvcuda::wmma::mem_col_major)
    store_matrix_sync<nvcuda::wmma::col_major>(ptr, frag, ldm, mul, sync);
  else
    store_matrix_sync<nvcuda::wmma::row_major>(ptr, frag, ldm, mul, sync);
}

// ---------------------------------------------------------------- mma: four real products
// (a_r + i a_i)(b_r + i b_i) = (a_r b_r - a_i b_i) + i (a_i b_r + a_r b_i)
#define TCEC_COMPLEX_MMA(NAME)                                                                                  \
  template <class LA, class LB, TCEC_TPARAMS>                                                                   \
  __device__ void NAME(TCEC_CFRAG(nvcuda::wmma::accumulator, void) & d,                                         \
                       const TCEC_CFRAG(nvcuda::wmma::matrix_a, LA) & a,                                        \
                       const TCEC_CFRAG(nvcuda::wmma::matrix_b, LB) & b,                                        \
                       const TCEC_CFRAG(nvcuda::wmma::accumulator, void) & c) {                                 \
    NAME(d.real, a.real, b.real, c.real);                                                                       \
    NAME(d.imag, a.imag, b.real, c.imag);                                                                       \
    NAME(d.imag, a.real, b.imag, d.imag);                                                                       \
    NAME(d.real, a.imag, neg(b.imag), d.real);                                                                  \
  }                                                                                                             \
  template <class LA, class LB, TCEC_TPARAMS>                                                                   \
  __device__ void NAME(TCEC_CFRAG(nvcuda::wmma::accumulator, void) & d,                                         \
                       const TCEC_CFRAG(nvcuda::wmma::matrix_a, LA) & a,                                        \
                       const TCEC_CFRAG(nvcuda::wmma::matrix_b, LB) & b) {                                      \
    NAME(d.imag, a.imag, b.real);                                                                               \
    NAME(d.imag, a.real, b.imag, d.imag);                                                                       \
    NAME(d.real, a.real, b.real);                                                                               \
    NAME(d.real, a.imag, neg(b.imag), d.real);                                                                  \
  }
TCEC_COMPLEX_MMA(mma_sync)
TCEC_COMPLEX_MMA(mma_rn_sync)
TCEC_COMPLEX_MMA(mma_rz_sync)
#undef TCEC_COMPLEX_MMA
#undef TCEC_CFRAG
#undef TCEC_TPARAMS

}  // namespace tcec
}  // namespace wmma
}  // namespace mtk
#endif
