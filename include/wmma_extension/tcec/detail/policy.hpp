// Tags, policies and default-policy selection of the TCEC warp-level API.
//
// Same names and meaning as the reference's include/wmma_extension/tcec/detail/policy.hpp
// (tags :12-20, sm tags :22-48, Policy :50-57, default_policy :63-99 and :122-125).
// Differences, by design: both instruction tags are implemented on PTX mma.sync with its
// documented register layouts (op_wmma is the 16x16 tile made of two n8 halves), so nothing
// depends on the undocumented nvcuda::wmma fragment layout; and there is no op_simt policy.
#ifndef TCEC_B200_DETAIL_POLICY_HPP
#define TCEC_B200_DETAIL_POLICY_HPP
#include <cuda_fp16.h>
#include <mma.h>

#include <type_traits>

namespace mtk {
namespace wmma {
namespace tcec {

struct op_mma;
struct op_wmma;
struct with_ec;
struct without_ec;
using op_with_error_correction = with_ec;
using op_without_error_correction = without_ec;

struct sm_70;
struct sm_75;
struct sm_80;
struct sm_86;
struct sm_89;
struct sm_90;
struct sm_100;
struct sm_not_specified;
#ifdef __CUDA_ARCH__
#if __CUDA_ARCH__ >= 1000
using sm_auto = sm_100;
#elif __CUDA_ARCH__ >= 900
using sm_auto = sm_90;
#elif __CUDA_ARCH__ >= 800
using sm_auto = sm_80;
#else
#error "this implementation of mtk::wmma::tcec needs sm_80 or newer (mma.sync m16n8k16 / tf32)"
#endif
#else
using sm_auto = sm_not_specified;
#endif

template <class Op, class ErrorCorrection, int m_, int n_, int k_>
struct Policy {
  using op = Op;
  using error_correction = ErrorCorrection;
  static const int m = m_;
  static const int n = n_;
  static const int k = k_;
};

namespace detail {
template <class T>
struct is_tf32 : std::is_same<T, nvcuda::wmma::precision::tf32> {};

// half: 16x16x16 (op_wmma) or 16x8x16 (op_mma); tf32: 16x16x8 or 16x8x8.
template <class T, class ErrorCorrection = mtk::wmma::tcec::with_ec, class Op = mtk::wmma::tcec::op_wmma,
          class Sm = mtk::wmma::tcec::sm_auto>
struct default_policy {
  static_assert(std::is_same<T, half>::value || is_tf32<T>::value, "T must be half or tf32");
  using type = mtk::wmma::tcec::Policy<Op, ErrorCorrection, 16, std::is_same<Op, op_mma>::value ? 8 : 16,
                                       is_tf32<T>::value ? 8 : 16>;
};

template <class Use, int a, int b, int c>
struct select_value;
template <int a, int b, int c>
struct select_value<nvcuda::wmma::matrix_a, a, b, c> {
  static const int value = a;
};
template <int a, int b, int c>
struct select_value<nvcuda::wmma::matrix_b, a, b, c> {
  static const int value = b;
};
template <int a, int b, int c>
struct select_value<nvcuda::wmma::accumulator, a, b, c> {
  static const int value = c;
};
}  // namespace detail

template <class T, class ErrorCorrection = mtk::wmma::tcec::with_ec, class Op = mtk::wmma::tcec::op_wmma,
          class Sm = mtk::wmma::tcec::sm_auto>
using default_policy = detail::default_policy<T, ErrorCorrection, Op, Sm>;

}  // namespace tcec
}  // namespace wmma
}  // namespace mtk
#endif
