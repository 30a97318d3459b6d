// mtk::wmma::tcec - warp-level error-corrected FP32 matrix fragments on tensor cores.
//
// Source-compatible surface of the reference's include/wmma_extension/tcec/tcec.hpp
// (fragment :13-80; fill :100-137; loads :140-302; stores :305-418; vectors :421-637;
// mma :640-927) and of its without_ec specialisation (tcec/detail/no_cor.hpp), written
// fresh on PTX mma.sync register tiles (detail/tile.hpp).  Arithmetic:
//   load   hi = cast<T>(v), lo = cast<T>((v - hi) * s)            s = 2^11 (half), 1 (tf32)
//   mma    main += A_hi*B_hi (FP32 round-to-nearest add outside the tensor core in the rn
//          variant, inside it in the rz variant); corr += A_lo*B_hi + A_hi*B_lo
//   store  main + corr / s
// All functions are warp-collective: the 32 lanes call them together with the same
// arguments, and they end in __syncwarp() unless `sync` is false.  T is `half` or
// `nvcuda::wmma::precision::tf32`.  A fragment's declared Layout only names the default
// memory order of load_matrix_sync(frag, ptr, ldm); every fragment can be loaded from
// either order through the explicit template argument.
#ifndef TCEC_B200_TCEC_HPP
#define TCEC_B200_TCEC_HPP
#include "detail/policy.hpp"
#include "detail/tile.hpp"

namespace mtk {
namespace wmma {
namespace tcec {

namespace detail {
template <class EC>
struct has_ec : std::is_same<EC, with_ec> {};

template <class Layout>
__device__ inline unsigned mem_index(unsigned i, unsigned j, unsigned ldm) {
  return std::is_same<Layout, nvcuda::wmma::col_major>::value ? i + j * ldm : i * ldm + j;
}
template <class Layout>
struct is_layout : std::integral_constant<bool, std::is_same<Layout, nvcuda::wmma::col_major>::value ||
                                                    std::is_same<Layout, nvcuda::wmma::row_major>::value> {};

// storage of the correction tiles: present with error correction, empty without
template <class Tile, int N, bool kEc>
struct corr_storage {
  Tile sub_d_frag[N];
};
template <class Tile, int N>
struct corr_storage<Tile, N, false> {};
}  // namespace detail

template <class Use, int m, int n, int k, class T, class Layout = void,
          class Policy_ = typename mtk::wmma::tcec::detail::default_policy<T>::type>
struct fragment
    : detail::corr_storage<
          typename detail::sub_tile<typename Policy_::op, Use, Policy_::m, Policy_::n, Policy_::k, T, Layout>::type,
          (detail::select_value<Use, m, k, m>::value /
           detail::select_value<Use, Policy_::m, Policy_::k, Policy_::m>::value) *
              (detail::select_value<Use, k, n, n>::value /
               detail::select_value<Use, Policy_::k, Policy_::n, Policy_::n>::value),
          detail::has_ec<typename Policy_::error_correction>::value> {
  using Policy = Policy_;
  using element_type = float;
  // op_mma: a register tile in PTX mma.sync order; op_wmma: nvcuda::wmma::fragment itself
  using sub_frag_t = typename detail::sub_tile<typename Policy::op, Use, Policy::m, Policy::n, Policy::k, T, Layout>::type;
  using tile_traits = detail::tile_traits<sub_frag_t>;
  using storage_t = typename tile_traits::storage_t;
  static constexpr bool error_corrected = detail::has_ec<typename Policy::error_correction>::value;
  static constexpr int sub_frag_m = Policy::m;
  static constexpr int sub_frag_n = Policy::n;
  static constexpr int sub_frag_k = Policy::k;
  static constexpr int num_sub_frag_m = detail::select_value<Use, m, k, m>::value /
                                        detail::select_value<Use, sub_frag_m, sub_frag_k, sub_frag_m>::value;
  static constexpr int num_sub_frag_n = detail::select_value<Use, k, n, n>::value /
                                        detail::select_value<Use, sub_frag_k, sub_frag_n, sub_frag_n>::value;
  static_assert(detail::select_value<Use, m, k, m>::value % tile_traits::rows == 0 &&
                    detail::select_value<Use, k, n, n>::value % tile_traits::cols == 0,
                "fragment extents must be multiples of the policy's tile");
  static const unsigned num_elements = num_sub_frag_m * num_sub_frag_n * sub_frag_t::num_elements;

  // tiles in column-major order over blocks: block (bm, bn) at bm + num_sub_frag_m * bn
  sub_frag_t sub_frag[num_sub_frag_m * num_sub_frag_n];

  __device__ storage_t& x(const unsigned index) {
    return sub_frag[index / sub_frag_t::num_elements].x[index % sub_frag_t::num_elements];
  }
  __device__ storage_t x(const unsigned index) const {
    return sub_frag[index / sub_frag_t::num_elements].x[index % sub_frag_t::num_elements];
  }
  // correction part; without error correction there is none and dx() is unavailable
  template <bool kE = error_corrected, typename std::enable_if<kE, int>::type = 0>
  __device__ storage_t& dx(const unsigned index) {
    return this->sub_d_frag[index / sub_frag_t::num_elements].x[index % sub_frag_t::num_elements];
  }
  template <bool kE = error_corrected, typename std::enable_if<kE, int>::type = 0>
  __device__ storage_t dx(const unsigned index) const {
    return this->sub_d_frag[index / sub_frag_t::num_elements].x[index % sub_frag_t::num_elements];
  }
  // fold the correction into the main part (accumulators)
  __device__ void integrate() {
    if constexpr (error_corrected) {
      for (int f = 0; f < num_sub_frag_m * num_sub_frag_n; f++)
        for (unsigned i = 0; i < sub_frag_t::num_elements; i++) {
          sub_frag[f].x[i] += static_cast<float>(this->sub_d_frag[f].x[i]) * detail::residual_scale<T>::down;
          this->sub_d_frag[f].x[i] = 0.0f;
        }
    }
  }
};

#define TCEC_FRAG(USE, LAYOUT) fragment<USE, m, n, k, T, LAYOUT, Policy<Op, EC, fm, fn, fk>>
#define TCEC_TPARAMS int m, int n, int k, class T, class Op, class EC, int fm, int fn, int fk

// ---------------------------------------------------------------- fill / neg
template <class Use, class Layout, TCEC_TPARAMS>
__device__ void fill_fragment(TCEC_FRAG(Use, Layout) & frag, const float v) {
  using F = TCEC_FRAG(Use, Layout);
  for (unsigned i = 0; i < F::num_elements; i++) {
    frag.x(i) = static_cast<typename F::storage_t>(v);
    if constexpr (F::error_corrected) frag.dx(i) = static_cast<typename F::storage_t>(0.0f);
  }
}
template <class Use, class Layout, TCEC_TPARAMS>
__device__ void fill_zero(TCEC_FRAG(Use, Layout) & frag) {
  fill_fragment(frag, 0.0f);
}
template <class Use, class Layout, TCEC_TPARAMS>
__device__ TCEC_FRAG(Use, Layout) neg(const TCEC_FRAG(Use, Layout) & frag) {
  using F = TCEC_FRAG(Use, Layout);
  F res;
  for (unsigned i = 0; i < F::num_elements; i++) {
    res.x(i) = -frag.x(i);
    if constexpr (F::error_corrected) res.dx(i) = -frag.dx(i);
  }
  return res;
}

// ---------------------------------------------------------------- loads
namespace detail {
// A / B operands: split on load.  Accumulators: copy (with error correction) or round through T
// (without: the reference's accumulator load does the same, tcec/detail/no_cor.hpp:165-166).
// `get(index)` returns the FP32 value at a linear memory index, so the same code serves plain
// FP32 arrays and the real / imaginary parts of interleaved complex arrays.
template <class MemLayout, class Use, class Layout, TCEC_TPARAMS, class Get>
__device__ void load_with(TCEC_FRAG(Use, Layout) & frag, Get get, const unsigned ldm, const float mul,
                          const bool use_mul) {
  using F = TCEC_FRAG(Use, Layout);
  using tile_t = typename F::tile_traits;
  tile_t::for_each([&](unsigned r, unsigned i, unsigned j) {
    for (int bm = 0; bm < F::num_sub_frag_m; bm++)
      for (int bn = 0; bn < F::num_sub_frag_n; bn++) {
        float v = get(mem_index<MemLayout>(i + bm * tile_t::rows, j + bn * tile_t::cols, ldm));
        if (use_mul) v *= mul;
        const int f = bm + F::num_sub_frag_m * bn;
        if constexpr (std::is_same<Use, nvcuda::wmma::accumulator>::value) {
          if constexpr (F::error_corrected) {
            frag.sub_frag[f].x[r] = v;
            frag.sub_d_frag[f].x[r] = 0.0f;
          } else {
            frag.sub_frag[f].x[r] = round_to<T>(v);
          }
        } else {
          const float hv = round_to<T>(v);
          frag.sub_frag[f].x[r] = static_cast<typename F::storage_t>(hv);
          if constexpr (F::error_corrected)
            frag.sub_d_frag[f].x[r] =
                static_cast<typename F::storage_t>(round_to<T>((v - hv) * residual_scale<T>::up));
        }
      }
  });
}
template <class MemLayout, class Use, class Layout, TCEC_TPARAMS, class MEM_T>
__device__ void load_impl(TCEC_FRAG(Use, Layout) & frag, const MEM_T* const ptr, const unsigned ldm,
                          const float mul, const bool use_mul) {
  load_with<MemLayout>(frag, [ptr](unsigned idx) { return static_cast<float>(ptr[idx]); }, ldm, mul, use_mul);
}
}  // namespace detail

// explicit memory layout
template <class MemLayout, class Use, class Layout, TCEC_TPARAMS, class MEM_T,
          typename std::enable_if<detail::is_layout<MemLayout>::value, int>::type = 0>
__device__ void load_matrix_sync(TCEC_FRAG(Use, Layout) & frag, const MEM_T* const ptr, const unsigned ldm,
                                 const bool sync = true) {
  detail::load_impl<MemLayout>(frag, ptr, ldm, 1.0f, false);
  if (sync) __syncwarp();
}
// A / B: memory layout = the fragment's declared layout
template <class Use, class Layout, TCEC_TPARAMS, class MEM_T,
          typename std::enable_if<detail::is_layout<Layout>::value, int>::type = 0>
__device__ void load_matrix_sync(TCEC_FRAG(Use, Layout) & frag, const MEM_T* const ptr, const unsigned ldm,
                                 const bool sync = true) {
  load_matrix_sync<Layout>(frag, ptr, ldm, sync);
}
// accumulator: run-time layout
template <TCEC_TPARAMS, class MEM_T>
__device__ void load_matrix_sync(TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag, const MEM_T* const ptr,
                                 const unsigned ldm, const nvcuda::wmma::layout_t layout, const bool sync = true) {
  if (layout == nvcuda::wmma::mem_col_major)
    load_matrix_sync<nvcuda::wmma::col_major>(frag, ptr, ldm, sync);
  else
    load_matrix_sync<nvcuda::wmma::row_major>(frag, ptr, ldm, sync);
}
// value * mul is formed in FP32 before the split (reference tcec.hpp:264)
template <class MemLayout, class Use, class Layout, TCEC_TPARAMS, class MEM_T,
          typename std::enable_if<detail::is_layout<MemLayout>::value, int>::type = 0>
__device__ void load_matrix_sync_with_mul(TCEC_FRAG(Use, Layout) & frag, const MEM_T* const ptr,
                                          const unsigned ldm, const MEM_T mul, const bool sync = true) {
  detail::load_impl<MemLayout>(frag, ptr, ldm, static_cast<float>(mul), true);
  if (sync) __syncwarp();
}
template <class Use, class Layout, TCEC_TPARAMS, class MEM_T,
          typename std::enable_if<detail::is_layout<Layout>::value, int>::type = 0>
__device__ void load_matrix_sync_with_mul(TCEC_FRAG(Use, Layout) & frag, const MEM_T* const ptr,
                                          const unsigned ldm, const MEM_T mul, const bool sync = true) {
  load_matrix_sync_with_mul<Layout>(frag, ptr, ldm, mul, sync);
}

// ---------------------------------------------------------------- stores (fold)
namespace detail {
template <class MemLayout, TCEC_TPARAMS, class Put>
__device__ void store_with(Put put, const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag, const unsigned ldm,
                           const float mul, const bool use_mul) {
  using F = TCEC_FRAG(nvcuda::wmma::accumulator, void);
  using tile_t = typename F::tile_traits;
  tile_t::for_each([&](unsigned r, unsigned i, unsigned j) {
    for (int bm = 0; bm < F::num_sub_frag_m; bm++)
      for (int bn = 0; bn < F::num_sub_frag_n; bn++) {
        const int f = bm + F::num_sub_frag_m * bn;
        float v = frag.sub_frag[f].x[r];
        if constexpr (F::error_corrected) v = v + frag.sub_d_frag[f].x[r] * residual_scale<T>::down;
        if (use_mul) v *= mul;
        put(mem_index<MemLayout>(i + bm * tile_t::rows, j + bn * tile_t::cols, ldm), v);
      }
  });
}
template <class MemLayout, TCEC_TPARAMS, class MEM_T>
__device__ void store_impl(MEM_T* const ptr, const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag,
                           const unsigned ldm, const float mul, const bool use_mul) {
  store_with<MemLayout>([ptr](unsigned idx, float v) { ptr[idx] = static_cast<MEM_T>(v); }, frag, ldm, mul, use_mul);
}
}  // namespace detail

template <class MemLayout, TCEC_TPARAMS, class MEM_T,
          typename std::enable_if<detail::is_layout<MemLayout>::value, int>::type = 0>
__device__ void store_matrix_sync(MEM_T* const ptr, const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag,
                                  const unsigned ldm, const bool sync = true) {
  detail::store_impl<MemLayout>(ptr, frag, ldm, 1.0f, false);
  if (sync) __syncwarp();
}
template <TCEC_TPARAMS, class MEM_T>
__device__ void store_matrix_sync(MEM_T* const ptr, const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag,
                                  const unsigned ldm, const nvcuda::wmma::layout_t layout,
                                  const bool sync = true) {
  if (layout == nvcuda::wmma::mem_col_major)
    store_matrix_sync<nvcuda::wmma::col_major>(ptr, frag, ldm, sync);
  else
    store_matrix_sync<nvcuda::wmma::row_major>(ptr, frag, ldm, sync);
}
template <class MemLayout, TCEC_TPARAMS, class MEM_T,
          typename std::enable_if<detail::is_layout<MemLayout>::value, int>::type = 0>
__device__ void store_matrix_sync_with_mul(MEM_T* const ptr,
                                           const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag,
                                           const unsigned ldm, const MEM_T mul, const bool sync = true) {
  detail::store_impl<MemLayout>(ptr, frag, ldm, static_cast<float>(mul), true);
  if (sync) __syncwarp();
}
template <TCEC_TPARAMS, class MEM_T>
__device__ void store_matrix_sync_with_mul(MEM_T* const ptr,
                                           const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag,
                                           const unsigned ldm, const MEM_T mul,
                                           const nvcuda::wmma::layout_t layout, const bool sync = true) {
  if (layout == nvcuda::wmma::mem_col_major)
    store_matrix_sync_with_mul<nvcuda::wmma::col_major>(ptr, frag, ldm, mul, sync);
  else
    store_matrix_sync_with_mul<nvcuda::wmma::row_major>(ptr, frag, ldm, mul, sync);
}

// ---------------------------------------------------------------- vectors
// A vector is the first column (col_major) or the first row (row_major) of the fragment:
// the same elements load_matrix_sync would take from a matrix whose first ld entries hold
// the vector.  Only those elements are written.
namespace detail {
template <bool kFirstColumn, class Use, class Layout, TCEC_TPARAMS, class MEM_T>
__device__ void load_vector_impl(TCEC_FRAG(Use, Layout) & frag, const MEM_T* const ptr, const float mul,
                                 const bool use_mul) {
  using F = TCEC_FRAG(Use, Layout);
  using tile_t = typename F::tile_traits;
  tile_t::for_each([&](unsigned r, unsigned i, unsigned j) {
    if ((kFirstColumn ? j : i) != 0) return;
    const int nblk = kFirstColumn ? F::num_sub_frag_m : F::num_sub_frag_n;
    for (int b = 0; b < nblk; b++) {
      const int f = kFirstColumn ? b : F::num_sub_frag_m * b;
      float v = static_cast<float>(ptr[kFirstColumn ? i + b * tile_t::rows : j + b * tile_t::cols]);
      if (use_mul) v *= mul;
      if constexpr (std::is_same<Use, nvcuda::wmma::accumulator>::value) {
        if constexpr (F::error_corrected) {
          frag.sub_frag[f].x[r] = v;
          frag.sub_d_frag[f].x[r] = 0.0f;
        } else {
          frag.sub_frag[f].x[r] = round_to<T>(v);
        }
      } else {
        const float hv = round_to<T>(v);
        frag.sub_frag[f].x[r] = static_cast<typename F::storage_t>(hv);
        if constexpr (F::error_corrected)
          frag.sub_d_frag[f].x[r] =
              static_cast<typename F::storage_t>(round_to<T>((v - hv) * residual_scale<T>::up));
      }
    }
  });
}
template <bool kFirstColumn, TCEC_TPARAMS, class MEM_T>
__device__ void store_vector_impl(MEM_T* const ptr, const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag,
                                  const float mul, const bool use_mul) {
  using F = TCEC_FRAG(nvcuda::wmma::accumulator, void);
  using tile_t = typename F::tile_traits;
  tile_t::for_each([&](unsigned r, unsigned i, unsigned j) {
    if ((kFirstColumn ? j : i) != 0) return;
    const int nblk = kFirstColumn ? F::num_sub_frag_m : F::num_sub_frag_n;
    for (int b = 0; b < nblk; b++) {
      const int f = kFirstColumn ? b : F::num_sub_frag_m * b;
      float v = frag.sub_frag[f].x[r];
      if constexpr (F::error_corrected) v = v + frag.sub_d_frag[f].x[r] * residual_scale<T>::down;
      if (use_mul) v *= mul;
      ptr[kFirstColumn ? i + b * tile_t::rows : j + b * tile_t::cols] = static_cast<MEM_T>(v);
    }
  });
}
}  // namespace detail

template <class Use, class Layout, TCEC_TPARAMS, class MEM_T,
          typename std::enable_if<detail::is_layout<Layout>::value, int>::type = 0>
__device__ void load_vector(TCEC_FRAG(Use, Layout) & frag, const MEM_T* const ptr) {
  detail::load_vector_impl<std::is_same<Layout, nvcuda::wmma::col_major>::value>(frag, ptr, 1.0f, false);
  __syncwarp();
}
template <class Use, class Layout, TCEC_TPARAMS, class MEM_T,
          typename std::enable_if<detail::is_layout<Layout>::value, int>::type = 0>
__device__ void load_vector(TCEC_FRAG(Use, Layout) & frag, const MEM_T* const ptr, const MEM_T mul) {
  detail::load_vector_impl<std::is_same<Layout, nvcuda::wmma::col_major>::value>(frag, ptr,
                                                                                static_cast<float>(mul), true);
  __syncwarp();
}
template <TCEC_TPARAMS, class MEM_T>
__device__ void load_vector(TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag, const MEM_T* const ptr,
                            const nvcuda::wmma::layout_t layout) {
  if (layout == nvcuda::wmma::mem_col_major)
    detail::load_vector_impl<true>(frag, ptr, 1.0f, false);
  else
    detail::load_vector_impl<false>(frag, ptr, 1.0f, false);
  __syncwarp();
}
template <TCEC_TPARAMS, class MEM_T>
__device__ void store_vector(MEM_T* const ptr, const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag,
                             const nvcuda::wmma::layout_t layout) {
  if (layout == nvcuda::wmma::mem_col_major)
    detail::store_vector_impl<true>(ptr, frag, 1.0f, false);
  else
    detail::store_vector_impl<false>(ptr, frag, 1.0f, false);
  __syncwarp();
}
template <TCEC_TPARAMS, class MEM_T>
__device__ void store_vector(MEM_T* const ptr, const TCEC_FRAG(nvcuda::wmma::accumulator, void) & frag,
                             const MEM_T mul, const nvcuda::wmma::layout_t layout) {
  if (layout == nvcuda::wmma::mem_col_major)
    detail::store_vector_impl<true>(ptr, frag, static_cast<float>(mul), true);
  else
    detail::store_vector_impl<false>(ptr, frag, static_cast<float>(mul), true);
  __syncwarp();
}

// ---------------------------------------------------------------- mma
namespace detail {
// kRn: the main product of every k step is formed on a zero accumulator and added in FP32
// with a round-to-nearest add (reference mma_rn_sync, tcec.hpp:640-770); otherwise it is
// accumulated inside the tensor core (mma_rz_sync, :773-893).  kUseC: d = a*b + c, else d = a*b.
template <bool kRn, bool kUseC, class LA, class LB, TCEC_TPARAMS>
__device__ void mma_impl(TCEC_FRAG(nvcuda::wmma::accumulator, void) & d, const TCEC_FRAG(nvcuda::wmma::matrix_a, LA) & a,
                         const TCEC_FRAG(nvcuda::wmma::matrix_b, LB) & b,
                         const TCEC_FRAG(nvcuda::wmma::accumulator, void) & c) {
  using FD = TCEC_FRAG(nvcuda::wmma::accumulator, void);
  using FA = TCEC_FRAG(nvcuda::wmma::matrix_a, LA);
  using acc_tile = typename FD::sub_frag_t;
  constexpr int MB = FD::num_sub_frag_m, NB = FD::num_sub_frag_n, KB = FA::num_sub_frag_n;
  for (int bm = 0; bm < MB; bm++)
    for (int bn = 0; bn < NB; bn++) {
      const int f = bm + bn * MB;
      acc_tile main_acc, corr_acc;
      for (unsigned i = 0; i < acc_tile::num_elements; i++) {
        main_acc.x[i] = kUseC ? c.sub_frag[f].x[i] : 0.0f;
        if constexpr (FD::error_corrected) corr_acc.x[i] = kUseC ? c.sub_d_frag[f].x[i] : 0.0f;
      }
      for (int bk = 0; bk < KB; bk++) {
        const auto& a_hi = a.sub_frag[bm + bk * MB];
        const auto& b_hi = b.sub_frag[bk + bn * KB];
        if (kRn) {
          acc_tile tmp;
          for (unsigned i = 0; i < acc_tile::num_elements; i++) tmp.x[i] = 0.0f;
          tile_mma(tmp, a_hi, b_hi, tmp);
          for (unsigned i = 0; i < acc_tile::num_elements; i++) main_acc.x[i] = main_acc.x[i] + tmp.x[i];
        } else {
          tile_mma(main_acc, a_hi, b_hi, main_acc);
        }
        if constexpr (FD::error_corrected) {
          tile_mma(corr_acc, a.sub_d_frag[bm + bk * MB], b_hi, corr_acc);
          tile_mma(corr_acc, a_hi, b.sub_d_frag[bk + bn * KB], corr_acc);
        }
      }
      for (unsigned i = 0; i < acc_tile::num_elements; i++) {
        d.sub_frag[f].x[i] = main_acc.x[i];
        if constexpr (FD::error_corrected) d.sub_d_frag[f].x[i] = corr_acc.x[i];
      }
    }
}
}  // namespace detail

template <class LA, class LB, TCEC_TPARAMS>
__device__ void mma_rn_sync(TCEC_FRAG(nvcuda::wmma::accumulator, void) & d, const TCEC_FRAG(nvcuda::wmma::matrix_a, LA) & a,
                            const TCEC_FRAG(nvcuda::wmma::matrix_b, LB) & b,
                            const TCEC_FRAG(nvcuda::wmma::accumulator, void) & c) {
  detail::mma_impl<true, true>(d, a, b, c);
}
template <class LA, class LB, TCEC_TPARAMS>
__device__ void mma_rn_sync(TCEC_FRAG(nvcuda::wmma::accumulator, void) & d, const TCEC_FRAG(nvcuda::wmma::matrix_a, LA) & a,
                            const TCEC_FRAG(nvcuda::wmma::matrix_b, LB) & b) {
  detail::mma_impl<true, false>(d, a, b, d);
}
template <class LA, class LB, TCEC_TPARAMS>
__device__ void mma_rz_sync(TCEC_FRAG(nvcuda::wmma::accumulator, void) & d, const TCEC_FRAG(nvcuda::wmma::matrix_a, LA) & a,
                            const TCEC_FRAG(nvcuda::wmma::matrix_b, LB) & b,
                            const TCEC_FRAG(nvcuda::wmma::accumulator, void) & c) {
  detail::mma_impl<false, true>(d, a, b, c);
}
template <class LA, class LB, TCEC_TPARAMS>
__device__ void mma_rz_sync(TCEC_FRAG(nvcuda::wmma::accumulator, void) & d, const TCEC_FRAG(nvcuda::wmma::matrix_a, LA) & a,
                            const TCEC_FRAG(nvcuda::wmma::matrix_b, LB) & b) {
  detail::mma_impl<false, false>(d, a, b, d);
}
// default rounding: nearest with error correction, inside the tensor core without
// (reference tcec.hpp:896-927, no_cor.hpp:858-897; docs/mma_f32.md:131-135)
template <class LA, class LB, TCEC_TPARAMS>
__device__ void mma_sync(TCEC_FRAG(nvcuda::wmma::accumulator, void) & d, const TCEC_FRAG(nvcuda::wmma::matrix_a, LA) & a,
                         const TCEC_FRAG(nvcuda::wmma::matrix_b, LB) & b,
                         const TCEC_FRAG(nvcuda::wmma::accumulator, void) & c) {
  detail::mma_impl<detail::has_ec<EC>::value, true>(d, a, b, c);
}
template <class LA, class LB, TCEC_TPARAMS>
__device__ void mma_sync(TCEC_FRAG(nvcuda::wmma::accumulator, void) & d, const TCEC_FRAG(nvcuda::wmma::matrix_a, LA) & a,
                         const TCEC_FRAG(nvcuda::wmma::matrix_b, LB) & b) {
  detail::mma_impl<detail::has_ec<EC>::value, false>(d, a, b, d);
}

#undef TCEC_FRAG
#undef TCEC_TPARAMS

}  // namespace tcec
}  // namespace wmma
}  // namespace mtk
#endif
