// Error-corrected GEMM on tcgen05 that reads the FP32 operands directly: TMA loads FP32 tiles
// into shared memory, converter warps split them in registers into fp16 hi and scaled
// residual (reference include/wmma_extension/tcec/tcec.hpp:219-223, scale.hpp:8-20) and write
// the tensor-core operand image, two threads issue the three products into TMEM, and the same
// warps that convert also run the epilogue (RN promotion of the main term, fold of the
// correction term, alpha/beta, stores; tcec.hpp:640-706 and :332-336).
//
// Compared with the panel kernel (tcec_gemm_panels.cuh) nothing is written to or re-read from
// global memory between the split and the products, which halves the DRAM traffic of a GEMM:
// this is the kernel for shapes bound by HBM (batches of small matrices).  It cannot feed the
// tensor pipe at full rate: per K = 32 step a 128x256 tile moves 48 KB of TMA writes, 48 KB of
// converter reads, 48 KB of converter writes and 72 KB of MMA operand reads through shared
// memory, 216 KB against the 96 KB the 768-cycle tensor work of that step leaves room for.
//
// Roles by warp (384 threads, one persistent CTA per SM):
//   warp 0      TMA producer of FP32 tiles (ring of 2 stages x 48 KB, 128-byte swizzle)
//   warp 1 / 2  MMA main / MMA correction (as in the panel kernel)
//   warps 4-11  converter + epilogue
// fp16 policies only; operands must be TMA-addressable (16-byte aligned base, leading
// dimension and batch stride multiples of 4 elements).
#pragma once
#include <cuda.h>

#include "sm100_ptx.cuh"
#include "tcec_gemm_panels.cuh"
#include "tcec_panels.cuh"

namespace tcec_sm100 {

struct GemmFusedParams {
  int M, N, K;
  int batch;
  int nkb;               // K blocks of 32
  int tiles_m, tiles_n;  // 128 x 256 tiles per matrix
  int promo;             // K blocks per RN promotion; 0 = once, at the end
  int a_k_contiguous;    // A is row-major (K contiguous); else column-major
  int b_k_contiguous;    // B is column-major (K contiguous); else row-major
  float alpha, beta;
  float* c;
  long long ldc, c_batch_stride;
  int c_col_major;
  int* status;
};

template <bool kEc>
struct GemmFusedCfg {
  static constexpr int BN = 256;
  static constexpr int NP = kEc ? 2 : 1;
  static constexpr int A_BYTES = kPanelBytes * NP;        // operand image of A: hi (+ lo)
  static constexpr int OP_STAGE = A_BYTES + 2 * kPanelBytes * NP;
  static constexpr int NOP = 2;                           // operand ring
  static constexpr int STG_A = 128 * 128;                 // 128 rows x 32 fp32
  static constexpr int STG_B = 256 * 128;
  static constexpr int STG_STAGE = STG_A + STG_B;
  static constexpr int NSTG = kEc ? 2 : 3;                // FP32 staging ring
  static constexpr int STG_OFFSET = NOP * OP_STAGE;
  static constexpr int SMEM_BYTES = STG_OFFSET + NSTG * STG_STAGE + 1024;
  static constexpr int TMEM_COLS = kEc ? 512 : 256;
  static constexpr int THREADS = 384;
  static constexpr int CONV_WARPS = 8;
  static constexpr int GROUP_M = 16;
};

template <bool kEc>
__global__ void __launch_bounds__(384, 1)
    tcec_gemm_fused_kernel(const GemmFusedParams p, const __grid_constant__ CUtensorMap map_a,
                           const __grid_constant__ CUtensorMap map_b) {
  using Cfg = GemmFusedCfg<kEc>;
  constexpr int NOP = Cfg::NOP, NSTG = Cfg::NSTG, BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[NOP], bar_empty[NOP], bar_stg_full[NSTG], bar_stg_empty[NSTG];
  __shared__ uint64_t bar_main_full, bar_main_free, bar_corr_full, bar_corr_free, bar_drain[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));  // generic pointer to the same place
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = p.tiles_m * p.tiles_n * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NOP; ++s) {
      mbar_init(smem_u32(&bar_full[s]), Cfg::CONV_WARPS);
      mbar_init(smem_u32(&bar_empty[s]), kEc ? 2 : 1);
    }
    for (int s = 0; s < NSTG; ++s) {
      mbar_init(smem_u32(&bar_stg_full[s]), 1);
      mbar_init(smem_u32(&bar_stg_empty[s]), Cfg::CONV_WARPS);
    }
    mbar_init(smem_u32(&bar_main_full), 1);
    mbar_init(smem_u32(&bar_main_free), Cfg::CONV_WARPS);
    mbar_init(smem_u32(&bar_corr_full), 1);
    mbar_init(smem_u32(&bar_corr_free), Cfg::CONV_WARPS);
    mbar_init(smem_u32(&bar_drain[0]), 1);
    mbar_init(smem_u32(&bar_drain[1]), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_main = tmem_base_s;
  const uint32_t tmem_corr = tmem_base_s + BN;
  volatile uint32_t* abortp = &abort_flag;

  if (warp < 4) {
    if (warp == 0) {
      // ---------------------------------------------------------- TMA producer
      if (lane == 0) {
        uint32_t s = 0, ph = 0, armed = 0, armed_parity = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
          const TileCoord tc = decode_tile(tile, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
          for (int kb = 0; kb < p.nkb; ++kb) {
            if (!mbar_wait(smem_u32(&bar_stg_empty[s]), ph ^ 1, abortp, 64)) {
              ok = false;
              break;
            }
            const uint32_t full = smem_u32(&bar_stg_full[s]);
            const uint32_t dst = smem_base + Cfg::STG_OFFSET + s * Cfg::STG_STAGE;
            mbar_arrive_expect_tx(full, Cfg::STG_STAGE);
            armed |= 1u << s;
            armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
            if (p.a_k_contiguous) {
              tma_load_3d(dst, &map_a, full, kb * 32, tc.mt * 128, tc.b);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) tma_load_3d(dst + j * 4096, &map_a, full, tc.mt * 128 + 32 * j, kb * 32, tc.b);
            }
            if (p.b_k_contiguous) {
              tma_load_3d(dst + Cfg::STG_A, &map_b, full, kb * 32, tc.nt * 256, tc.b);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                tma_load_3d(dst + Cfg::STG_A + j * 4096, &map_b, full, tc.nt * 256 + 32 * j, kb * 32, tc.b);
            }
            if (++s == static_cast<uint32_t>(NSTG)) {
              s = 0;
              ph ^= 1;
            }
          }
        }
        if (!ok) {
          abort_flag = 1;
          atomicCAS(p.status, 0, kErrProducerWait);
          for (uint32_t q = 0; q < static_cast<uint32_t>(NSTG); ++q)
            if (armed & (1u << q)) mbar_wait_plain(smem_u32(&bar_stg_full[q]), (armed_parity >> q) & 1);
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------- MMA issuer, main products
      if (lane == 0) {
        const uint32_t idesc = umma_idesc(0u, 128, BN);
        const uint64_t dconst = umma_desc_kmajor_noswizzle(0, 128, 512);
        constexpr uint32_t kBHi = Cfg::A_BYTES >> 4;
        const uint32_t base16 = (smem_base & 0x3ffff) >> 4;
        uint32_t s = 0, ph = 0, chunk = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
          int left_in_chunk = 0;
          for (int kb = 0; kb < p.nkb; ++kb) {
            if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, 32)) {
              ok = false;
              break;
            }
            const bool first_in_chunk = (left_in_chunk == 0);
            if (first_in_chunk) {
              const int rest = p.nkb - kb;
              left_in_chunk = (p.promo && p.promo < rest) ? p.promo : rest;
              if (!mbar_wait(smem_u32(&bar_main_free), (chunk & 1) ^ 1, abortp, 0)) {
                ok = false;
                break;
              }
            }
            tc_fence_after();
            const uint32_t a16 = base16 + s * (Cfg::OP_STAGE >> 4);
#pragma unroll
            for (uint32_t j = 0; j < 2; ++j)
              umma_ss<false>(tmem_main, dconst | (a16 + 16 * j), dconst | (a16 + kBHi + 16 * j), idesc,
                             (first_in_chunk && j == 0) ? 0u : 1u);
            if (--left_in_chunk == 0) {
              umma_commit(smem_u32(&bar_main_full));
              ++chunk;
            }
            umma_commit(smem_u32(&bar_empty[s]));
            if (++s == static_cast<uint32_t>(NOP)) {
              s = 0;
              ph ^= 1;
            }
          }
        }
        if (!ok) {
          abort_flag = 1;
          atomicCAS(p.status, 0, kErrMmaWait);
          umma_commit(smem_u32(&bar_drain[0]));
          mbar_wait_plain(smem_u32(&bar_drain[0]), 0);
        }
      }
    } else if (warp == 2) {
      // ---------------------------------------------------------- MMA issuer, correction products
      if constexpr (kEc) {
        if (lane == 0) {
          const uint32_t idesc = umma_idesc(0u, 128, BN);
          const uint64_t dconst = umma_desc_kmajor_noswizzle(0, 128, 512);
          constexpr uint32_t kALo = kPanelBytes >> 4, kBHi = Cfg::A_BYTES >> 4,
                             kBLo = (Cfg::A_BYTES + 2 * kPanelBytes) >> 4;
          const uint32_t base16 = (smem_base & 0x3ffff) >> 4;
          uint32_t s = 0, ph = 0, tcount = 0;
          bool ok = true;
          for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
            for (int kb = 0; kb < p.nkb; ++kb) {
              if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, 32)) {
                ok = false;
                break;
              }
              if (kb == 0) {
                if (!mbar_wait(smem_u32(&bar_corr_free), (tcount & 1) ^ 1, abortp, 32)) {
                  ok = false;
                  break;
                }
              }
              tc_fence_after();
              const uint32_t c16 = base16 + s * (Cfg::OP_STAGE >> 4);
#pragma unroll
              for (uint32_t j = 0; j < 2; ++j)
                umma_ss<false>(tmem_corr, dconst | (c16 + kALo + 16 * j), dconst | (c16 + kBHi + 16 * j), idesc,
                               (kb == 0 && j == 0) ? 0u : 1u);
#pragma unroll
              for (uint32_t j = 0; j < 2; ++j)
                umma_ss<false>(tmem_corr, dconst | (c16 + 16 * j), dconst | (c16 + kBLo + 16 * j), idesc, 1u);
              umma_commit(smem_u32(&bar_empty[s]));
              if (++s == static_cast<uint32_t>(NOP)) {
                s = 0;
                ph ^= 1;
              }
            }
            if (!ok) break;
            umma_commit(smem_u32(&bar_corr_full));
          }
          if (!ok) {
            abort_flag = 1;
            atomicCAS(p.status, 0, kErrMmaWait);
            umma_commit(smem_u32(&bar_drain[1]));
            mbar_wait_plain(smem_u32(&bar_drain[1]), 0);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ converter + epilogue
    const int ew = warp - 4;
    const int q = warp & 3;
    const int colbase = (ew >> 2) * 128;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const bool vec_store = !p.c_col_major && (p.ldc % 4 == 0);
    uint32_t chunk = 0, tcount = 0;
    uint32_t so = 0, oph = 0, sg = 0, gph = 0;  // operand-ring and staging-ring positions
    bool ok = true;

    // conversion unit = 256 FP32 elements: 8 rows x 32 k (K-contiguous source) or 32 rows x 8 k
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
      const TileCoord tc = decode_tile(tile, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
      float acc[128];
      int left_in_chunk = 0;   // K blocks of the current chunk not yet converted
      int chunks_done = 0;     // chunks of this tile already promoted
      bool owe_drain = false;  // a chunk ended at the previous K block
      auto drain_main = [&]() -> bool {
        if (!mbar_wait_warp(smem_u32(&bar_main_full), chunk & 1, abortp, 64)) return false;
        tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_main + lane_addr + colbase + cc * 32, v);
          tmem_ld_wait();
          if (chunks_done == 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[cc * 32 + i] = __uint_as_float(v[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[cc * 32 + i] += __uint_as_float(v[i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_main_free));
        ++chunk;
        ++chunks_done;
        return true;
      };
      for (int kb = 0; kb < p.nkb && ok; ++kb) {
        if (left_in_chunk == 0) {
          const int rest = p.nkb - kb;
          left_in_chunk = (p.promo && p.promo < rest) ? p.promo : rest;
        }
        // ---- convert K block kb: FP32 staging -> operand image
        if (!mbar_wait_warp(smem_u32(&bar_stg_full[sg]), gph, abortp, 32) ||
            !mbar_wait_warp(smem_u32(&bar_empty[so]), oph ^ 1, abortp, 32)) {
          ok = false;
          break;
        }
        {
          const uint8_t* stg = smem_gen + Cfg::STG_OFFSET + sg * Cfg::STG_STAGE;
          uint8_t* op = smem_gen + so * Cfg::OP_STAGE;
          // 16 units of A and 32 of B, dealt round-robin to the 8 warps
#pragma unroll 1
          for (int u = ew; u < 48; u += Cfg::CONV_WARPS) {
            const bool is_b = u >= 16;
            const int unit = is_b ? u - 16 : u;
            const bool k_contig = is_b ? (p.b_k_contiguous != 0) : (p.a_k_contiguous != 0);
            const uint8_t* src_base = stg + (is_b ? Cfg::STG_A : 0);
            uint8_t* hi_base = op + (is_b ? Cfg::A_BYTES : 0);
            uint8_t* lo_base = hi_base + (is_b ? 2 * kPanelBytes : kPanelBytes);
            float v[8];
            int row, c;
            if (k_contig) {
              const int r = lane & 7;
              c = lane >> 3;
              row = unit * 8 + r;
              const uint8_t* src = src_base + row * 128;
              const float4 x0 = *reinterpret_cast<const float4*>(src + (((2 * c) ^ r) << 4));
              const float4 x1 = *reinterpret_cast<const float4*>(src + (((2 * c + 1) ^ r) << 4));
              v[0] = x0.x; v[1] = x0.y; v[2] = x0.z; v[3] = x0.w;
              v[4] = x1.x; v[5] = x1.y; v[6] = x1.z; v[7] = x1.w;
            } else {
              const int sub = unit >> 2;
              c = unit & 3;
              row = sub * 32 + lane;
              const uint8_t* src = src_base + sub * 4096 + (lane & 3) * 4;
#pragma unroll
              for (int t = 0; t < 8; ++t)
                v[t] = *reinterpret_cast<const float*>(src + (c * 8 + t) * 128 + (((lane >> 2) ^ t) << 4));
            }
            uint4 hi, lo;
            split8_f16(v, hi, lo);
            const int off = (row >> 7) * kPanelBytes + ((row & 127) >> 3) * 512 + c * 128 + (row & 7) * 16;
            *reinterpret_cast<uint4*>(hi_base + off) = hi;
            if constexpr (kEc) *reinterpret_cast<uint4*>(lo_base + off) = lo;
          }
        }
        fence_proxy_async_smem();  // operand image written with ordinary stores, read by the tensor pipe
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bar_full[so]));
          mbar_arrive(smem_u32(&bar_stg_empty[sg]));
        }
        if (++so == static_cast<uint32_t>(NOP)) {
          so = 0;
          oph ^= 1;
        }
        if (++sg == static_cast<uint32_t>(NSTG)) {
          sg = 0;
          gph ^= 1;
        }
        // ---- promote the chunk that ended one K block ago (the block just converted keeps the
        //      tensor pipe busy meanwhile)
        if (owe_drain) {
          if (!drain_main()) {
            ok = false;
            break;
          }
          owe_drain = false;
        }
        if (--left_in_chunk == 0) owe_drain = true;
      }
      if (!ok) break;
      if (owe_drain && !drain_main()) {
        ok = false;
        break;
      }
      // ---- fold the correction term, hand the accumulators back, store
      float* cbase = p.c + tc.b * p.c_batch_stride;
      const int row = tc.mt * 128 + q * 32 + lane;
      const int col0 = tc.nt * BN + colbase;
      const bool vec_ok = vec_store && ((reinterpret_cast<uintptr_t>(cbase) & 15) == 0);
      if constexpr (kEc) {
        if (!mbar_wait_warp(smem_u32(&bar_corr_full), tcount & 1, abortp, 64)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_corr + lane_addr + colbase + cc * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            acc[cc * 32 + i] = acc[cc * 32 + i] + __uint_as_float(v[i]) * (1.0f / 2048.0f);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_corr_free));
      }
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        if (row < p.M) {
          if (!p.c_col_major) {
            float* crow = cbase + static_cast<long long>(row) * p.ldc;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const int col = col0 + cc * 32 + i;
              if (vec_ok && col + 3 < p.N) {
                float4 o;
                o.x = p.alpha * acc[cc * 32 + i + 0];
                o.y = p.alpha * acc[cc * 32 + i + 1];
                o.z = p.alpha * acc[cc * 32 + i + 2];
                o.w = p.alpha * acc[cc * 32 + i + 3];
                if (p.beta != 0.f) {
                  const float4 old = *reinterpret_cast<const float4*>(crow + col);
                  o.x += p.beta * old.x;
                  o.y += p.beta * old.y;
                  o.z += p.beta * old.z;
                  o.w += p.beta * old.w;
                }
                *reinterpret_cast<float4*>(crow + col) = o;
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  if (col + e < p.N) {
                    float o = p.alpha * acc[cc * 32 + i + e];
                    if (p.beta != 0.f) o += p.beta * crow[col + e];
                    crow[col + e] = o;
                  }
                }
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = col0 + cc * 32 + i;
              if (col < p.N) {
                float* dst = cbase + static_cast<long long>(col) * p.ldc + row;
                float o = p.alpha * acc[cc * 32 + i];
                if (p.beta != 0.f) o += p.beta * *dst;
                *dst = o;
              }
            }
          }
        }
      }
    }
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicCAS(p.status, 0, kErrEpilogueWait);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base_s, Cfg::TMEM_COLS);
}

}  // namespace tcec_sm100
