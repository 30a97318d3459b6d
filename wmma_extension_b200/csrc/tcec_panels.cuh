// Split pass of the panel path: FP32 matrix -> hi / scaled-lo operand panels.
//
// Follows the reference split (include/wmma_extension/tcec/tcec.hpp:219-223,
// scale include/wmma_extension/tcec/detail/scale.hpp:8-20):
//   hi = cast<T>(v);  lo = cast<T>((v - float(hi)) * s)
// with T = fp16 (round-to-nearest-even, s = 2^11) or tf32 (cvt.rna, s = 1).
// The reference redoes this in every warp that consumes a tile; here every
// element is split once and stored in the exact shared-memory image the
// tensor-core instruction reads, so the GEMM kernel moves panels with linear
// bulk copies and never touches the data with CUDA cores.
//
// Panel = 128 rows x 64 bytes of K (32 fp16 or 16 tf32), 8192 bytes, stored as
// un-swizzled K-major core matrices: element (r, c) with c a 16-byte chunk
// index 0..3 sits at (r/8)*512 + c*128 + (r%8)*16.  For each (row block, k
// block) the hi panel comes first and, with error correction, the lo panel
// directly after it.
#pragma once
#include <cuda_fp16.h>

#include <cstdint>

namespace tcec_sm100 {

constexpr int kPanelRows = 128;
constexpr int kPanelBytes = 8192;

__device__ __forceinline__ float tf32_rna(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

// 8 fp32 -> 8 fp16 hi and 8 fp16 scaled residuals (16 bytes each).
__device__ __forceinline__ void split8_f16(const float (&v)[8], uint4& hi, uint4& lo) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 hv = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    const float2 hf = __half22float2(hv);
    const __half2 lv =
        __floats2half2_rn((v[2 * i] - hf.x) * 2048.0f, (v[2 * i + 1] - hf.y) * 2048.0f);
    h[i] = *reinterpret_cast<const uint32_t*>(&hv);
    l[i] = *reinterpret_cast<const uint32_t*>(&lv);
  }
  hi = make_uint4(h[0], h[1], h[2], h[3]);
  lo = make_uint4(l[0], l[1], l[2], l[3]);
}
// 4 fp32 -> 4 tf32 hi and 4 tf32 residuals (16 bytes each).
__device__ __forceinline__ void split4_tf32(const float (&v)[4], uint4& hi, uint4& lo) {
  float h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    h[i] = tf32_rna(v[i]);
    l[i] = tf32_rna(v[i] - h[i]);
  }
  hi = make_uint4(__float_as_uint(h[0]), __float_as_uint(h[1]), __float_as_uint(h[2]),
                  __float_as_uint(h[3]));
  lo = make_uint4(__float_as_uint(l[0]), __float_as_uint(l[1]), __float_as_uint(l[2]),
                  __float_as_uint(l[3]));
}

struct SplitParams {
  const float* src;              // strided batch base (used when src_array == nullptr)
  const float* const* src_array; // optional pointer array, one matrix per batch entry
  long long ld;                  // leading dimension in elements
  long long batch_stride;        // elements between matrices (strided form)
  int rows;                      // extent along M (for A) or N (for B)
  int k;                         // extent along K
  int k_contiguous;              // 1: element (r,k) at r*ld + k ; 0: at k*ld + r
  int row_blocks;                // padded rows / 128
  int nkb;                       // number of k blocks
  uint8_t* panels;               // output
  long long panels_batch_stride; // bytes
  float mul;                     // value multiplied in before the split (1 for plain loads)
  int elem_stride;               // floats between consecutive elements (0 or 1: dense; 2: one part of
                                 // interleaved complex data, `src` pointing at that part)
  int kb_offset;                 // first k block written (operands concatenated along K)
  int nkb_out;                   // k blocks per row block in the destination (0: nkb)
};

// One CTA's work: the hi(+lo) panel of k block `kb`, row block `rb` of matrix `b`.
template <bool kTf32, bool kEc>
__device__ __forceinline__ void split_one_panel(const SplitParams& p, int kb, int rb, int b) {
  constexpr int KCH = kTf32 ? 4 : 8;    // fp32 elements per 16-byte operand chunk
  constexpr int KOP = 4 * KCH;          // K extent of one panel
  const float* __restrict__ src =
      p.src_array ? p.src_array[b] : p.src + static_cast<long long>(b) * p.batch_stride;
  uint8_t* out = p.panels + static_cast<long long>(b) * p.panels_batch_stride +
                 (static_cast<size_t>(rb) * (p.nkb_out ? p.nkb_out : p.nkb) + p.kb_offset + kb) *
                     (kEc ? 2 : 1) * kPanelBytes;
  const int k0 = kb * KOP;
  const int es = p.elem_stride > 1 ? p.elem_stride : 1;
  const bool vec_ok = (es == 1) && (p.ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int item = threadIdx.x + it * 256;  // 512 (row, chunk) items per panel
    int r, c;
    if (p.k_contiguous) {
      r = item >> 2;
      c = item & 3;
    } else {
      r = item & 127;
      c = item >> 7;
    }
    const int row = rb * kPanelRows + r;
    const int kk = k0 + c * KCH;
    float v[KCH];
    if (p.k_contiguous) {
      const float* s = src + static_cast<long long>(row) * p.ld + static_cast<long long>(kk) * es;
      if (row < p.rows && kk + KCH <= p.k && vec_ok) {
#pragma unroll
        for (int q = 0; q < KCH / 4; ++q) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(s) + q);
          v[4 * q + 0] = t.x;
          v[4 * q + 1] = t.y;
          v[4 * q + 2] = t.z;
          v[4 * q + 3] = t.w;
        }
      } else {
#pragma unroll
        for (int q = 0; q < KCH; ++q) v[q] = (row < p.rows && kk + q < p.k) ? __ldg(s + q * es) : 0.f;
      }
    } else {
#pragma unroll
      for (int q = 0; q < KCH; ++q)
        v[q] = (row < p.rows && kk + q < p.k)
                   ? __ldg(src + static_cast<long long>(kk + q) * p.ld + static_cast<long long>(row) * es)
                   : 0.f;
    }
    if (p.mul != 1.0f) {
#pragma unroll
      for (int q = 0; q < KCH; ++q) v[q] *= p.mul;
    }
    uint4 hi, lo;
    if constexpr (kTf32) {
      split4_tf32(v, hi, lo);
    } else {
      split8_f16(v, hi, lo);
    }
    const int off = (r >> 3) * 512 + c * 128 + (r & 7) * 16;
    *reinterpret_cast<uint4*>(out + off) = hi;
    if constexpr (kEc) *reinterpret_cast<uint4*>(out + kPanelBytes + off) = lo;
  }
}

// grid = (nkb, row_blocks, batch), 256 threads: one CTA writes one hi(+lo) panel.
template <bool kTf32, bool kEc>
__global__ void __launch_bounds__(256) tcec_split_panels_kernel(const SplitParams p) {
  split_one_panel<kTf32, kEc>(p, blockIdx.x, blockIdx.y, blockIdx.z);
}

// Both operands of a product in one launch (grid.x = panels of A + panels of B, all matrices of the
// batch): one launch gap and one grid tail less than two launches, which is what a short call
// notices (4096^3: 3 of 361 us; 1024^3: 3 of 30).
template <bool kTf32, bool kEc>
__global__ void __launch_bounds__(256) tcec_split_both_kernel(const SplitParams pa, const SplitParams pb,
                                                              unsigned int panels_a) {
  const bool second = blockIdx.x >= panels_a;
  const SplitParams& p = second ? pb : pa;
  unsigned int i = second ? blockIdx.x - panels_a : blockIdx.x;
  const int kb = i % p.nkb;
  i /= p.nkb;
  const int rb = i % p.row_blocks;
  split_one_panel<kTf32, kEc>(p, kb, rb, static_cast<int>(i / p.row_blocks));
}

}  // namespace tcec_sm100
