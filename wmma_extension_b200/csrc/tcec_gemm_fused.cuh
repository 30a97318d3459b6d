// Error-corrected GEMM on tcgen05 that reads the FP32 operands directly: TMA loads FP32 tiles
// into shared memory, eight converter warps split them in registers into fp16 hi and scaled
// residual (reference include/wmma_extension/tcec/tcec.hpp:219-223, scale.hpp:8-20) and write
// the tensor-core operand image IN PLACE over the FP32 data, two threads issue the three
// products into TMEM, and eight epilogue warps promote the main term with round-to-nearest
// adds, fold the correction term and store (tcec.hpp:640-706 and :332-336).
//
// Compared with the panel kernel (tcec_gemm_panels.cuh) nothing is written to or re-read from
// global memory between the split and the products, which more than halves the DRAM traffic of
// a GEMM: this is the kernel for shapes bound by HBM (batches of small matrices).  It cannot
// feed the tensor pipe at full rate: per K = 32 step a 128x256 tile moves 48 KB of TMA writes,
// 48 KB of converter reads, 48 KB of converter writes and 72 KB of MMA operand reads through
// shared memory, 216 KB against the 96 KB the 768-cycle tensor work of that step leaves room for.
//
// In-place conversion.  The fp16 hi and lo images of an FP32 block take exactly the block's
// bytes, and the un-swizzled UMMA descriptor leaves the 8-row-group stride free, so every
// 8-row x 32-k group keeps its own 1 KB: FP32 rows (8 x 128 B, TMA 128-byte swizzle) become
// 512 B of hi core matrices followed by 512 B of lo core matrices.  A converter warp reads a
// whole unit into registers, __syncwarp()s, and writes the unit back: a K-contiguous unit is
// one such group (lane = row, 16-byte k chunk); a unit of an operand whose rows are contiguous
// instead (A column-major, B row-major) is a 32-k x 32-row TMA box of 4 KB, four groups, which
// the warp transposes on the way (lane = row).  One ring of four 48 KB stages therefore serves
// as FP32 landing zone and as operand buffer: each stage goes TMA -> convert -> MMA -> free.
//
// Roles by warp (640 threads in five warpgroups, one persistent CTA per SM).  The register file
// is re-balanced at entry with setmaxnreg: the kernel launches with 96 registers per thread, the
// control warpgroup drops to 40, the converters to 56 and the epilogue rises to 160 (the shares
// must sum to no more than the launch allocation, or the raise would never be granted).
//   warp 0       lane 0: TMA producer
//   warp 1       lane 0: MMA issuer, main products
//   warp 2       lane 0: MMA issuer, correction products
//   warps 4-11   epilogue (as in the panel kernel)
//   warps 12-19  converters: one warp cannot issue the split arithmetic faster than one
//                8-element split per 104 clocks (measured), so a K block's 48 splits need
//                several warps per scheduler to stay ahead of the loads
// fp16 policies only; operands must be TMA-addressable (16-byte aligned base, leading
// dimension and batch stride multiples of 4 elements).
#pragma once
#include <cuda.h>

#include "sm100_ptx.cuh"
#include "tcec_epilogue.cuh"
#include "tcec_gemm_panels.cuh"
#include "tcec_gemm_roles.cuh"
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
  unsigned long long* trace;  // develop builds only: hand-off timestamps of CTA 0, rows of 4096 slots
                              // (0 main saw full, 1 main chunk free, 2 landed, 3 converted, 4 corr saw full,
                              //  5 main committed, 6 epilogue: chunk seen / drained, 7 epilogue: corr seen /
                              //  folded / stored, 8 producer: stage issued)
  int debug_flags;  // develop builds only (results invalid): bit 1 = no MMAs, bit 2 = no conversion, bit 3 = no stores
};

template <bool kEc>
struct GemmFusedCfg {
  static constexpr int BN = 256;
  static constexpr int STG_A = 128 * 128;  // 128 rows x 32 fp32, also the size of A's hi + lo image
  static constexpr int STG_B = 256 * 128;
  static constexpr int STAGE = STG_A + STG_B;
  static constexpr int NST = 4;
  static constexpr int EPI_OFFSET = NST * STAGE;           // eight epilogue turn buffers after the ring
  static constexpr int SMEM_BYTES = NST * STAGE + 8 * kEpiBufBytes + 1024;
  static constexpr int TMEM_COLS = kEc ? 512 : 256;
  static constexpr int THREADS = 640;
  static constexpr int CONV_WARPS = 8;
  // setmaxnreg moves registers inside the CTA's launch allocation (640 threads x 96), so the
  // three shares must fit in it: a request beyond it would wait forever.
  static constexpr int REGS_LAUNCH = 96, REGS_CONTROL = 40, REGS_CONVERT = 56, REGS_EPILOGUE = 160;
  static_assert(128 * REGS_CONTROL + 256 * REGS_CONVERT + 256 * REGS_EPILOGUE <= THREADS * REGS_LAUNCH,
                "register shares exceed the launch allocation");
  static constexpr int GROUP_BYTES = 1024;  // one 8-row group: hi at +0, lo at +512
  static constexpr int GROUP_M = 16;
};

// U K-contiguous units, `stride` bytes apart: each is 8 rows x 32 k (1 KB).  Lane = (row r,
// 8-float chunk c).  All units are read before any is written, so the loads overlap.
template <bool kEc, int U>
__device__ __forceinline__ void convert_groups_inplace(uint8_t* g, int stride, int lane) {
  const int r = lane & 7, c = lane >> 3;
  float4 x[U][2];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint8_t* src = g + u * stride + r * 128;
    x[u][0] = *reinterpret_cast<const float4*>(src + (((2 * c) ^ r) << 4));
    x[u][1] = *reinterpret_cast<const float4*>(src + (((2 * c + 1) ^ r) << 4));
  }
  __syncwarp();  // every lane has read its part of every unit
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const float v[8] = {x[u][0].x, x[u][0].y, x[u][0].z, x[u][0].w, x[u][1].x, x[u][1].y, x[u][1].z, x[u][1].w};
    uint4 hi, lo;
    split8_f16(v, hi, lo);
    uint8_t* dst = g + u * stride + c * 128 + r * 16;
    *reinterpret_cast<uint4*>(dst) = hi;
    if constexpr (kEc) *reinterpret_cast<uint4*>(dst + 512) = lo;
  }
}

// U row-contiguous units, `stride` bytes apart: each a 32-k x 32-row box (4 KB, k-row kk at
// kk * 128 B, 16-byte chunk j of it stored at j ^ (kk % 8)).  Lane = row; a box becomes four groups.
template <bool kEc, int U>
__device__ __forceinline__ void convert_boxes_inplace(uint8_t* t, int stride, int lane) {
  float v[U][4][8];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint8_t* src = t + u * stride + (lane & 3) * 4;
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int e = 0; e < 8; ++e)
        v[u][c][e] = *reinterpret_cast<const float*>(src + (c * 8 + e) * 128 + (((lane >> 2) ^ e) << 4));
  }
  __syncwarp();
#pragma unroll
  for (int u = 0; u < U; ++u) {
    uint8_t* g = t + u * stride + (lane >> 3) * 1024 + (lane & 7) * 16;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 hi, lo;
      split8_f16(v[u][c], hi, lo);
      *reinterpret_cast<uint4*>(g + c * 128) = hi;
      if constexpr (kEc) *reinterpret_cast<uint4*>(g + 512 + c * 128) = lo;
    }
  }
}

template <bool kEc>
__global__ void __launch_bounds__(640, 1)
    tcec_gemm_fused_kernel(const GemmFusedParams p, const __grid_constant__ CUtensorMap map_a,
                           const __grid_constant__ CUtensorMap map_b) {
  using Cfg = GemmFusedCfg<kEc>;
  constexpr int NST = Cfg::NST, BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_landed[NST], bar_full[NST], bar_empty[NST];
  __shared__ uint64_t bar_main_full, bar_main_free, bar_corr_full, bar_corr_free, bar_drain[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));  // generic pointer to the same place
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = p.tiles_m * p.tiles_n * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(smem_u32(&bar_landed[s]), 1);
      mbar_init(smem_u32(&bar_full[s]), Cfg::CONV_WARPS);
      mbar_init(smem_u32(&bar_empty[s]), kEc ? 2 : 1);
    }
    mbar_init(smem_u32(&bar_main_full), 1);
    mbar_init(smem_u32(&bar_main_free), 8);
    mbar_init(smem_u32(&bar_corr_full), 1);
    mbar_init(smem_u32(&bar_corr_free), 8);
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
  // Operand descriptors: core matrices 128 B apart along K, 8-row groups 1 KB apart.
  const uint64_t dconst = umma_desc_kmajor_noswizzle(0, 128, Cfg::GROUP_BYTES);
  constexpr uint32_t kALo = 512 >> 4, kBHi = Cfg::STG_A >> 4, kBLo = (Cfg::STG_A + 512) >> 4;

  if (warp >= 12) {
    // ------------------------------------------------------------ converters
    setmaxnreg_dec<Cfg::REGS_CONVERT>();
    const int cw = warp - 12;
    uint32_t s = 0, ph = 0, cit = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < p.nkb; ++kb) {
        if (!mbar_wait_warp(smem_u32(&bar_landed[s]), ph, abortp, 32)) {
          ok = false;
          break;
        }
        mbar_try_wait(smem_u32(&bar_landed[s]), ph);  // each lane observes the completed phase itself
        if (cw == 0 && lane == 0 && blockIdx.x == 0) trace_slot(p.trace, 2, cit);  // landed
        uint8_t* stage = smem_gen + s * Cfg::STAGE;
        // A: 16 groups or 4 boxes; B: 32 groups or 8 boxes.  Groups are dealt warp by warp, a box
        // goes to one warp (A's four boxes to every other warp).
        if (dev_flag(p.debug_flags, 4)) {
        } else {
          if (p.a_k_contiguous) {
            convert_groups_inplace<kEc, 2>(stage + cw * 1024, 8192, lane);
          } else if ((cw & 1) == 0) {
            convert_boxes_inplace<kEc, 1>(stage + (cw >> 1) * 4096, 0, lane);
          }
          if (p.b_k_contiguous) {
            convert_groups_inplace<kEc, 4>(stage + Cfg::STG_A + cw * 1024, 8192, lane);
          } else {
            convert_boxes_inplace<kEc, 1>(stage + Cfg::STG_A + cw * 4096, 0, lane);
          }
        }
        fence_proxy_async_smem();  // image written with ordinary stores, read by the tensor pipe
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_full[s]));
        if (cw == 0 && lane == 0 && blockIdx.x == 0) trace_slot(p.trace, 3, cit);  // converted
        ++cit;
        if (++s == static_cast<uint32_t>(NST)) {
          s = 0;
          ph ^= 1;
        }
      }
    }
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicCAS(p.status, 0, kErrProducerWait);
    }
  } else if (warp < 4) {
    setmaxnreg_dec<Cfg::REGS_CONTROL>();
    if ((warp == 1 || (kEc && warp == 2)) && lane == 0) {
      // ---------------------------------------------------------- MMA issuers (tcec_gemm_roles.cuh)
      OperandImage im;
      im.dconst = dconst;
      im.base16 = (smem_base & 0x3ffff) >> 4;
      im.stage16 = Cfg::STAGE >> 4;
      im.a_lo16 = kALo;
      im.b_hi16 = kBHi;
      im.b_lo16 = kBLo;
      im.idesc = umma_idesc(0u, 128, BN);
      const StridedTiles tiles{static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), ntiles};
      const KWalk walk{p.nkb, p.promo};
      const RingBarriers ring{bar_full, bar_empty};
      if (warp == 1) {
        if (!issue_main_products<false, false, NST>(tiles, walk, im, tmem_main, ring, &bar_main_full, &bar_main_free,
                                                    abortp, p.debug_flags, blockIdx.x == 0 ? p.trace : nullptr))
          mma_thread_gave_up<false>(&abort_flag, p.status, kErrMmaWait, &bar_drain[0]);
      } else {
        if (!issue_corr_products<false, false, NST>(tiles, walk, im, tmem_corr, ring, &bar_corr_full, &bar_corr_free,
                                                    abortp, p.debug_flags, blockIdx.x == 0 ? p.trace : nullptr))
          mma_thread_gave_up<false>(&abort_flag, p.status, kErrMmaWait, &bar_drain[1]);
      }
    } else if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------- TMA producer
      uint32_t s = 0, ph = 0, armed = 0, armed_parity = 0;
      [[maybe_unused]] uint32_t pit = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        const TileCoord tc = decode_tile(tile, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
        for (int kb = 0; kb < p.nkb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, abortp, 64)) {
            ok = false;
            break;
          }
          const uint32_t landed = smem_u32(&bar_landed[s]);
          const uint32_t dst = smem_base + s * Cfg::STAGE;
          mbar_arrive_expect_tx(landed, Cfg::STAGE);
          if (blockIdx.x == 0) trace_slot(p.trace, 8, pit++);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
          if (p.a_k_contiguous) {
            tma_load_3d(dst, &map_a, landed, kb * 32, tc.mt * 128, tc.b);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) tma_load_3d(dst + j * 4096, &map_a, landed, tc.mt * 128 + 32 * j, kb * 32, tc.b);
          }
          if (p.b_k_contiguous) {
            tma_load_3d(dst + Cfg::STG_A, &map_b, landed, kb * 32, tc.nt * 256, tc.b);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              tma_load_3d(dst + Cfg::STG_A + j * 4096, &map_b, landed, tc.nt * 256 + 32 * j, kb * 32, tc.b);
          }
          if (++s == static_cast<uint32_t>(NST)) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0, kErrProducerWait);
        for (uint32_t q = 0; q < static_cast<uint32_t>(NST); ++q)
          if (armed & (1u << q)) mbar_wait_plain(smem_u32(&bar_landed[q]), (armed_parity >> q) & 1);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    setmaxnreg_inc<Cfg::REGS_EPILOGUE>();
    const int ew = warp - 4;
    const int q = warp & 3;
    const int colbase = (ew >> 2) * 128;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    uint32_t chunk = 0, tcount = 0;
    bool ok = true;
    const bool etrace = (warp == 4 && lane == 0 && blockIdx.x == 0);
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
      const TileCoord tc = decode_tile(tile, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
      const int nchunks = p.promo ? (p.nkb + p.promo - 1) / p.promo : 1;
      float acc[128];
      for (int c = 0; c < nchunks; ++c, ++chunk) {
        if (!mbar_wait_warp(smem_u32(&bar_main_full), chunk & 1, abortp)) {
          ok = false;
          break;
        }
        if (etrace) trace_slot(p.trace, 6, 2 * chunk);
        tc_fence_after();
        promote_main_chunk<false>(acc, tmem_main + lane_addr + colbase, c == 0);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_main_free));
        if (etrace) trace_slot(p.trace, 6, 2 * chunk + 1);
      }
      if (!ok) break;
      if constexpr (kEc) {
        if (!mbar_wait_warp(smem_u32(&bar_corr_full), tcount & 1, abortp)) {
          ok = false;
          break;
        }
        if (etrace) trace_slot(p.trace, 7, 3 * tcount);
        tc_fence_after();
        fold_correction(acc, tmem_corr + lane_addr + colbase, 1.0f / 2048.0f);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_corr_free));
        if (etrace) trace_slot(p.trace, 7, 3 * tcount + 1);
      }
      StoreTarget st;
      st.cbase = p.c + tc.b * p.c_batch_stride;
      st.ldc = p.ldc;
      st.M = p.M;
      st.N = p.N;
      st.col_major = p.c_col_major;
      st.vec_ok = !p.c_col_major && (p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(st.cbase) & 15) == 0);
      st.alpha = p.alpha;
      st.beta = p.beta;
      if (!dev_flag(p.debug_flags, 8))
        store_warp_block(acc, tc.mt * 128 + q * 32, tc.nt * BN + colbase, st,
                         reinterpret_cast<float*>(smem_gen + Cfg::EPI_OFFSET) + ew * kEpiBufFloats, lane);
      if (etrace) trace_slot(p.trace, 7, 3 * tcount + 2);
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
