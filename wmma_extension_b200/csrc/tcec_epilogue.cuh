// Store step shared by the GEMM kernels: one epilogue thread holds NC (128, or 64 in half-width
// tiles) consecutive columns of one output row (main + correction already folded) and the warp writes alpha * acc + beta * C.
// Restates the reference's smem2dmem (test/tcec/batch_gemm.cu:119-185): beta == 0 never reads C,
// 128-bit stores where the row allows them, element-wise predicated stores on the ragged edge.
//
// A TMEM load leaves lane = row, so a direct store of a row-major C touches 32 different rows
// per instruction (32 partial sectors).  The warp therefore turns each 32 x 32 block through a
// private shared-memory buffer (pitch 33 floats: conflict-free both ways) and stores it as
// 4 rows x 128 contiguous bytes per instruction.  Column-major C needs no turn: consecutive
// lanes already hold consecutive addresses.
#pragma once
#include <cstdint>

namespace tcec_sm100 {

struct StoreTarget {
  float* cbase;      // first element of this matrix
  long long ldc;
  int M, N;
  int col_major;     // C(row, col) at col * ldc + row, else at row * ldc + col
  bool vec_ok;       // row-major, ldc % 4 == 0 and cbase 16-byte aligned
  float alpha, beta;
};

// alpha * v + beta * old with fixed rounding points (one product rounded, then one fused
// multiply-add), so every store path of every kernel produces the same bits.
__device__ __forceinline__ float axpby(float alpha, float v, float beta, float old) {
  return __fmaf_rn(beta, old, __fmul_rn(alpha, v));
}

template <int NC>
__device__ __forceinline__ void store_row_slice(const float (&acc)[NC], int row, int col0, const StoreTarget& t) {
  if (row >= t.M) return;
#pragma unroll
  for (int cc = 0; cc < NC / 32; ++cc) {
    if (!t.col_major) {
      float* crow = t.cbase + static_cast<long long>(row) * t.ldc;
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const int col = col0 + cc * 32 + i;
        if (t.vec_ok && col + 3 < t.N) {
          float4 o;
          if (t.beta != 0.f) {
            const float4 old = *reinterpret_cast<const float4*>(crow + col);
            o.x = axpby(t.alpha, acc[cc * 32 + i + 0], t.beta, old.x);
            o.y = axpby(t.alpha, acc[cc * 32 + i + 1], t.beta, old.y);
            o.z = axpby(t.alpha, acc[cc * 32 + i + 2], t.beta, old.z);
            o.w = axpby(t.alpha, acc[cc * 32 + i + 3], t.beta, old.w);
          } else {
            o.x = __fmul_rn(t.alpha, acc[cc * 32 + i + 0]);
            o.y = __fmul_rn(t.alpha, acc[cc * 32 + i + 1]);
            o.z = __fmul_rn(t.alpha, acc[cc * 32 + i + 2]);
            o.w = __fmul_rn(t.alpha, acc[cc * 32 + i + 3]);
          }
          *reinterpret_cast<float4*>(crow + col) = o;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (col + e < t.N)
              crow[col + e] = t.beta != 0.f ? axpby(t.alpha, acc[cc * 32 + i + e], t.beta, crow[col + e])
                                            : __fmul_rn(t.alpha, acc[cc * 32 + i + e]);
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int col = col0 + cc * 32 + i;
        if (col < t.N) {
          float* dst = t.cbase + static_cast<long long>(col) * t.ldc + row;
          *dst = t.beta != 0.f ? axpby(t.alpha, acc[cc * 32 + i], t.beta, *dst) : __fmul_rn(t.alpha, acc[cc * 32 + i]);
        }
      }
    }
  }
}

constexpr int kEpiBufFloats = 32 * 33;              // one warp's turn buffer
constexpr int kEpiBufBytes = kEpiBufFloats * 4;      // 4224

// `row0` = first of the warp's 32 rows (lane = row0 + lane holds `acc`), `col0` = first of its
// NC columns, `wbuf` = this warp's buffer of kEpiBufFloats floats.  Warp-collective.
template <int NC>
__device__ __forceinline__ void store_warp_block(const float (&acc)[NC], int row0, int col0, const StoreTarget& t,
                                                 float* wbuf, int lane) {
  if (t.col_major) {
    store_row_slice(acc, row0 + lane, col0, t);
    return;
  }
  const int rsub = lane >> 3, cv = (lane & 7) * 4;
#pragma unroll
  for (int cc = 0; cc < NC / 32; ++cc) {
#pragma unroll
    for (int i = 0; i < 32; ++i) wbuf[lane * 33 + i] = acc[cc * 32 + i];
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = j * 4 + rsub;
      const int row = row0 + r, col = col0 + cc * 32 + cv;
      const float* src = wbuf + r * 33 + cv;
      const float v0 = src[0], v1 = src[1], v2 = src[2], v3 = src[3];
      if (row < t.M) {
        float* dst = t.cbase + static_cast<long long>(row) * t.ldc + col;
        if (t.vec_ok && col + 3 < t.N) {
          float4 o;
          if (t.beta != 0.f) {
            const float4 old = *reinterpret_cast<const float4*>(dst);
            o = make_float4(axpby(t.alpha, v0, t.beta, old.x), axpby(t.alpha, v1, t.beta, old.y),
                            axpby(t.alpha, v2, t.beta, old.z), axpby(t.alpha, v3, t.beta, old.w));
          } else {
            o = make_float4(__fmul_rn(t.alpha, v0), __fmul_rn(t.alpha, v1), __fmul_rn(t.alpha, v2),
                            __fmul_rn(t.alpha, v3));
          }
          *reinterpret_cast<float4*>(dst) = o;
        } else {
          const float v[4] = {v0, v1, v2, v3};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (col + e < t.N)
              dst[e] = t.beta != 0.f ? axpby(t.alpha, v[e], t.beta, dst[e]) : __fmul_rn(t.alpha, v[e]);
          }
        }
      }
    }
    __syncwarp();
  }
}

}  // namespace tcec_sm100
