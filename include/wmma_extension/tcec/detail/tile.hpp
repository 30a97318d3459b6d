// Per-warp register tiles of the TCEC fragments and their element <-> (row, column) maps.
//
// One tile is the operand of one tensor-core step: A is 16 x fk, B is fk x fn, the accumulator
// 16 x fn, with fk = 16 or 8 (half), 8 (tf32) and fn = 8 or 16.
//
// op_mma: `tile` below, in the register order PTX documents for mma.sync.aligned.m16n8k16 /
// m16n8k8 (f16) and m16n8k8 (tf32).  The reference keeps these maps in
// include/wmma_extension/detail/m16n8k16.hpp:100-176, detail/m16n8k8.hpp:136-165 and
// detail/m16n8k8_tf32.hpp:68-112; element order of A/B/C tiles here is the same.
//
// op_wmma: the tile IS nvcuda::wmma::fragment<Use, 16, 16, fk, T, Layout>, as in the reference
// (include/wmma_extension/tcec/detail/policy.hpp:107-112), so sub_frag[] can be handed to
// nvcuda::wmma::* and x(i) follows nvcuda's element order.  That order is not documented; the
// maps below state what sm_80 and later do (the reference states the same facts in
// detail/sm_80.hpp:95-173 and detail/sm_80_tf32.hpp:102-184) and a test compares them with
// nvcuda::wmma::load_matrix_sync on the GPU it runs on.  Half A and B fragments hold every
// element twice (registers x and x + 8).
#ifndef TCEC_B200_DETAIL_TILE_HPP
#define TCEC_B200_DETAIL_TILE_HPP
#include "policy.hpp"

namespace mtk {
namespace wmma {
namespace tcec {
namespace detail {

__device__ inline unsigned lane_id() {
  unsigned l;
  asm("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

// What one register of an operand holds: half for half operands, float otherwise
// (tf32 values live in FP32 registers; accumulators are FP32).
template <class Use, class T>
struct storage {
  using type = float;
};
template <>
struct storage<nvcuda::wmma::matrix_a, half> {
  using type = half;
};
template <>
struct storage<nvcuda::wmma::matrix_b, half> {
  using type = half;
};

template <class T>
__device__ inline float round_to(float v);  // FP32 -> T -> FP32
template <>
__device__ inline float round_to<half>(float v) {
  return __half2float(__float2half_rn(v));
}
template <>
__device__ inline float round_to<nvcuda::wmma::precision::tf32>(float v) {
  unsigned r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}
// scale applied to the residual before it is rounded, and its inverse at the fold
// (reference: include/wmma_extension/tcec/detail/scale.hpp:8-20)
template <class T>
struct residual_scale {
  static constexpr float up = 1.0f, down = 1.0f;
};
template <>
struct residual_scale<half> {
  static constexpr float up = 2048.0f, down = 1.0f / 2048.0f;
};

template <class Use, int FM, int FN, int FK, class T>
struct tile {
  static_assert(FM == 16 && (FN == 8 || FN == 16) && (FK == 16 || FK == 8), "unsupported tile shape");
  static_assert(std::is_same<T, half>::value || (is_tf32<T>::value && FK == 8),
                "half tiles have k = 16 or 8, tf32 tiles k = 8");
  static constexpr bool kPacked = std::is_same<T, half>::value;  // two 16-bit elements per register
  using storage_t = typename storage<Use, T>::type;
  static constexpr int rows = select_value<Use, FM, FK, FM>::value;
  static constexpr int cols = select_value<Use, FK, FN, FN>::value;
  static constexpr unsigned num_elements = rows * cols / 32;
  alignas(8) storage_t x[num_elements];

  // calls f(register index, row, column) for every element this lane holds
  template <class F>
  __device__ static void for_each(F f) {
    const unsigned lane = lane_id(), g = lane >> 2, t = lane & 3;
    if (std::is_same<Use, nvcuda::wmma::matrix_a>::value) {
      if (kPacked && FK == 8) {
#pragma unroll
        for (unsigned r = 0; r < 2; ++r)
#pragma unroll
          for (unsigned e = 0; e < 2; ++e) f(2 * r + e, g + 8 * r, 2 * t + e);
      } else if (FK == 16) {
#pragma unroll
        for (unsigned c = 0; c < 2; ++c)
#pragma unroll
          for (unsigned r = 0; r < 2; ++r)
#pragma unroll
            for (unsigned e = 0; e < 2; ++e) f(4 * c + 2 * r + e, g + 8 * r, 8 * c + 2 * t + e);
      } else {
#pragma unroll
        for (unsigned c = 0; c < 2; ++c)
#pragma unroll
          for (unsigned r = 0; r < 2; ++r) f(2 * c + r, g + 8 * r, t + 4 * c);
      }
    } else if (std::is_same<Use, nvcuda::wmma::matrix_b>::value) {
#pragma unroll
      for (unsigned nb = 0; nb < FN / 8; ++nb) {
        if (kPacked && FK == 8) {
#pragma unroll
          for (unsigned e = 0; e < 2; ++e) f(2 * nb + e, 2 * t + e, 8 * nb + g);
        } else if (FK == 16) {
#pragma unroll
          for (unsigned kh = 0; kh < 2; ++kh)
#pragma unroll
            for (unsigned e = 0; e < 2; ++e) f(4 * nb + 2 * kh + e, 2 * t + 8 * kh + e, 8 * nb + g);
        } else {
#pragma unroll
          for (unsigned kh = 0; kh < 2; ++kh) f(2 * nb + kh, t + 4 * kh, 8 * nb + g);
        }
      }
    } else {
#pragma unroll
      for (unsigned nb = 0; nb < FN / 8; ++nb)
#pragma unroll
        for (unsigned r = 0; r < 2; ++r)
#pragma unroll
          for (unsigned e = 0; e < 2; ++e) f(4 * nb + 2 * r + e, g + 8 * r, 8 * nb + 2 * t + e);
    }
  }
};

// d = a * b + c on tensor cores, FP32 accumulate (d and c may be the same tile)
template <int FN>
__device__ inline void tile_mma(tile<nvcuda::wmma::accumulator, 16, FN, 16, half>& d,
                                const tile<nvcuda::wmma::matrix_a, 16, FN, 16, half>& a,
                                const tile<nvcuda::wmma::matrix_b, 16, FN, 16, half>& b,
                                const tile<nvcuda::wmma::accumulator, 16, FN, 16, half>& c) {
  const unsigned* ar = reinterpret_cast<const unsigned*>(a.x);
  const unsigned* br = reinterpret_cast<const unsigned*>(b.x);
#pragma unroll
  for (int nb = 0; nb < FN / 8; ++nb) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d.x[4 * nb + 0]), "=f"(d.x[4 * nb + 1]), "=f"(d.x[4 * nb + 2]), "=f"(d.x[4 * nb + 3])
        : "r"(ar[0]), "r"(ar[1]), "r"(ar[2]), "r"(ar[3]), "r"(br[2 * nb + 0]), "r"(br[2 * nb + 1]),
          "f"(c.x[4 * nb + 0]), "f"(c.x[4 * nb + 1]), "f"(c.x[4 * nb + 2]), "f"(c.x[4 * nb + 3]));
  }
}
template <int FN>
__device__ inline void tile_mma(tile<nvcuda::wmma::accumulator, 16, FN, 8, half>& d,
                                const tile<nvcuda::wmma::matrix_a, 16, FN, 8, half>& a,
                                const tile<nvcuda::wmma::matrix_b, 16, FN, 8, half>& b,
                                const tile<nvcuda::wmma::accumulator, 16, FN, 8, half>& c) {
  const unsigned* ar = reinterpret_cast<const unsigned*>(a.x);
  const unsigned* br = reinterpret_cast<const unsigned*>(b.x);
#pragma unroll
  for (int nb = 0; nb < FN / 8; ++nb) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
        : "=f"(d.x[4 * nb + 0]), "=f"(d.x[4 * nb + 1]), "=f"(d.x[4 * nb + 2]), "=f"(d.x[4 * nb + 3])
        : "r"(ar[0]), "r"(ar[1]), "r"(br[nb]), "f"(c.x[4 * nb + 0]), "f"(c.x[4 * nb + 1]),
          "f"(c.x[4 * nb + 2]), "f"(c.x[4 * nb + 3]));
  }
}
template <int FN>
__device__ inline void tile_mma(tile<nvcuda::wmma::accumulator, 16, FN, 8, nvcuda::wmma::precision::tf32>& d,
                                const tile<nvcuda::wmma::matrix_a, 16, FN, 8, nvcuda::wmma::precision::tf32>& a,
                                const tile<nvcuda::wmma::matrix_b, 16, FN, 8, nvcuda::wmma::precision::tf32>& b,
                                const tile<nvcuda::wmma::accumulator, 16, FN, 8, nvcuda::wmma::precision::tf32>& c) {
#pragma unroll
  for (int nb = 0; nb < FN / 8; ++nb) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d.x[4 * nb + 0]), "=f"(d.x[4 * nb + 1]), "=f"(d.x[4 * nb + 2]), "=f"(d.x[4 * nb + 3])
        : "r"(__float_as_uint(a.x[0])), "r"(__float_as_uint(a.x[1])), "r"(__float_as_uint(a.x[2])),
          "r"(__float_as_uint(a.x[3])), "r"(__float_as_uint(b.x[2 * nb + 0])),
          "r"(__float_as_uint(b.x[2 * nb + 1])), "f"(c.x[4 * nb + 0]), "f"(c.x[4 * nb + 1]),
          "f"(c.x[4 * nb + 2]), "f"(c.x[4 * nb + 3]));
  }
}

// ---------------------------------------------------------------- op_wmma: nvcuda fragments as tiles
template <class Use, class T>
struct wmma_element {
  using type = T;
};
template <class T>
struct wmma_element<nvcuda::wmma::accumulator, T> {
  using type = float;
};
// nvcuda's A and B fragments need a layout; a TCEC fragment declared without one gets the usual
// one (A row-major, B column-major).  Accumulators have none.
template <class Use, class Layout>
struct wmma_layout {
  using type = Layout;
};
template <>
struct wmma_layout<nvcuda::wmma::matrix_a, void> {
  using type = nvcuda::wmma::row_major;
};
template <>
struct wmma_layout<nvcuda::wmma::matrix_b, void> {
  using type = nvcuda::wmma::col_major;
};
template <class Layout>
struct wmma_layout<nvcuda::wmma::accumulator, Layout> {
  using type = void;
};

// the tile type of a policy
template <class Op, class Use, int FM, int FN, int FK, class T, class Layout>
struct sub_tile {
  using type = tile<Use, FM, FN, FK, T>;
};
template <class Use, int FK, class T, class Layout>
struct sub_tile<op_wmma, Use, 16, 16, FK, T, Layout> {
  using type = nvcuda::wmma::fragment<Use, 16, 16, FK, typename wmma_element<Use, T>::type,
                                      typename wmma_layout<Use, Layout>::type>;
};

// rows, cols, register type and element map of a tile type
template <class Tile>
struct tile_traits;
template <class Use, int FM, int FN, int FK, class T>
struct tile_traits<tile<Use, FM, FN, FK, T>> {
  using tile_t = tile<Use, FM, FN, FK, T>;
  using storage_t = typename tile_t::storage_t;
  static constexpr int rows = tile_t::rows, cols = tile_t::cols;
  template <class F>
  __device__ static void for_each(F f) {
    tile_t::for_each(f);
  }
};
template <class Use, int FK, class E, class L>
struct tile_traits<nvcuda::wmma::fragment<Use, 16, 16, FK, E, L>> {
  using tile_t = nvcuda::wmma::fragment<Use, 16, 16, FK, E, L>;
  using storage_t = typename tile_t::storage_element_type;
  static constexpr int rows = select_value<Use, 16, FK, 16>::value;
  static constexpr int cols = select_value<Use, FK, 16, 16>::value;
  static constexpr bool kTwice = std::is_same<E, half>::value;  // half A and B: every element in registers x and x + 8
  // calls f(register index, row, column) for every register this lane holds
  template <class F>
  __device__ static void for_each(F f) {
    const unsigned lane = lane_id(), g = lane >> 2, t = lane & 3;
    if (std::is_same<Use, nvcuda::wmma::accumulator>::value) {
#pragma unroll
      for (unsigned x = 0; x < 8; ++x) f(x, g + 8 * ((x >> 1) & 1), 2 * t + (x & 1) + 8 * (x >> 2));
    } else if (std::is_same<Use, nvcuda::wmma::matrix_a>::value) {
      if (FK == 16) {
#pragma unroll
        for (unsigned x = 0; x < 8; ++x) {
          f(x, g + 8 * ((x >> 1) & 1), 2 * t + (x & 1) + 8 * (x >> 2));
          f(x + 8, g + 8 * ((x >> 1) & 1), 2 * t + (x & 1) + 8 * (x >> 2));
        }
      } else {
#pragma unroll
        for (unsigned x = 0; x < 4; ++x) f(x, g + 8 * (x & 1), t + 4 * (x >> 1));
      }
    } else {
      if (FK == 16) {
#pragma unroll
        for (unsigned x = 0; x < 8; ++x) {
          f(x, 2 * t + (x & 1) + 8 * ((x >> 1) & 1), g + 8 * (x >> 2));
          f(x + 8, 2 * t + (x & 1) + 8 * ((x >> 1) & 1), g + 8 * (x >> 2));
        }
      } else {
#pragma unroll
        for (unsigned x = 0; x < 4; ++x) f(x, t + 4 * (x & 1), g + 8 * (x >> 1));
      }
    }
  }
};

// d = a * b + c through nvcuda::wmma (d and c may be the same fragment)
template <int FK, class T, class LA, class LB>
__device__ inline void tile_mma(nvcuda::wmma::fragment<nvcuda::wmma::accumulator, 16, 16, FK, float>& d,
                                const nvcuda::wmma::fragment<nvcuda::wmma::matrix_a, 16, 16, FK, T, LA>& a,
                                const nvcuda::wmma::fragment<nvcuda::wmma::matrix_b, 16, 16, FK, T, LB>& b,
                                const nvcuda::wmma::fragment<nvcuda::wmma::accumulator, 16, 16, FK, float>& c) {
  nvcuda::wmma::mma_sync(d, a, b, c);
}

}  // namespace detail
}  // namespace tcec
}  // namespace wmma
}  // namespace mtk
#endif
