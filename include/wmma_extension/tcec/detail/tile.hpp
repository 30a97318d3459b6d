// Per-warp register tiles for mma.sync and their element <-> (row, column) maps.
//
// One tile is the operand of one tensor-core step of the TCEC fragments: A is 16 x fk,
// B is fk x fn, the accumulator 16 x fn, with fk = 16 or 8 (half), 8 (tf32) and fn = 8 or 16.
// Register order is the one PTX documents for mma.sync.aligned.m16n8k16 / m16n8k8 (f16) and
// m16n8k8 (tf32); a 16-wide tile is two n8 blocks back to back.  The reference keeps
// these maps in include/wmma_extension/detail/m16n8k16.hpp:100-176, detail/m16n8k8.hpp:136-165
// and detail/m16n8k8_tf32.hpp:68-112; element order of A/B/C tiles here is the same.
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

}  // namespace detail
}  // namespace tcec
}  // namespace wmma
}  // namespace mtk
#endif
