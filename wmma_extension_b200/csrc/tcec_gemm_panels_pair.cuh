// The panel GEMM on CTA pairs (tcgen05 cta_group::2): two SMs share one 256 x 256 output tile.
//
// Same arithmetic, panel format, roles and TMEM layout as tcec_gemm_panels.cuh.  What changes:
// each CTA of a pair loads the A panels of its own 128 rows and only its half of the B panels
// (128 of the tile's 256 N rows), and the leader CTA issues every MMA for both SMs
// (M = 256, N = 256, K = 16): per SM and K block 32 KB instead of 48 KB come through L2 and
// 48 KB instead of 72 KB of operands are read from shared memory, and the ring holds 6 stages
// instead of 4.  Measured: a little faster than one SM per tile while the clocks are high
// (4096^3), but it draws more power per product, so it is slower once the board sits at its
// power cap (16384^3); the host library therefore keeps it behind an option.
//
// Pair protocol (rank 0 = leader, rank 1 = peer):
//   full[s]   leader's barrier: its own copies' bytes + one remote arrive by the peer's relay
//             thread (peer warp 1), which waits on the peer's local full[s] first.  The remote
//             arrive has CTA scope: with cluster-scope release every arrive waited for the
//             SM's copies in flight and the ring degenerated to one stage at a time.
//   empty[s]  committed by the leader's two MMA threads to BOTH CTAs (multicast commit)
//   main_full / corr_full   likewise committed to both CTAs; each CTA drains its own TMEM
//   main_free / corr_free   leader's barriers: 8 local epilogue warps + 8 remote arrives
// Both CTAs meet at a cluster barrier after set-up and before exit.
//
// BN = 128 is the same kernel on 256 x 128 half tiles: a half is one 128-row B panel of which each
// CTA loads its 64 rows (the first or second 4 KB of the panel), multiplied with N = 128, and each
// epilogue warp holds 64 columns.  The host uses it for calls with so few tiles that whole tiles
// would leave at least half of the SM pairs idle (an N = 128 MMA takes ~0.6 of an N = 256 one, so
// halving pays only there); every element of C still sees the same products in the same order.
// A launch covers the pair tiles [tile_first, tile_first + tile_count).
#pragma once
#include "sm100_ptx.cuh"
#include "tcec_gemm_panels.cuh"
#include "tcec_gemm_roles.cuh"

namespace tcec_sm100 {

template <bool kTf32, bool kEc>
struct GemmPairCfg {
  static constexpr int NP = kEc ? 2 : 1;
  static constexpr int A_BYTES = kPanelBytes * NP;   // this CTA's 128 rows of A: hi (+ lo)
  static constexpr int B_BYTES = kPanelBytes * NP;   // this CTA's 128 of the tile's 256 N rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int NST_RAW = (200 * 1024) / STAGE_BYTES;
  static constexpr int NST = NST_RAW > 8 ? 8 : NST_RAW;
  static constexpr int EPI_OFFSET = NST * STAGE_BYTES;
  static constexpr int SMEM_BYTES = NST * STAGE_BYTES + 8 * kEpiBufBytes + 1024;
  static constexpr int TMEM_COLS = kEc ? 512 : 256;
  static constexpr int THREADS = 384;
  // as in the one-SM kernel: the control warpgroup hands registers to the two epilogue warpgroups
  static constexpr int REGS_CONTROL = 40, REGS_EPILOGUE = 232;
  static_assert(128 * REGS_CONTROL + 256 * REGS_EPILOGUE <= THREADS * 168, "register shares");
  static constexpr int GROUP_M = 8;  // pair tiles are 256 rows tall
};

// p.tiles_m counts 256-row pair tiles here.
template <bool kTf32, bool kEc, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(384, 1)
    tcec_gemm_panels_pair_kernel(const GemmPanelParams p) {
  static_assert(BN == 256 || BN == 128, "whole or half-width pair tiles");
  using Cfg = GemmPairCfg<kTf32, kEc>;
  constexpr int NST = Cfg::NST;
  constexpr int HALVES = 256 / BN;            // work items per pair tile
  constexpr int NC = BN / 2;                  // columns per epilogue warp
  constexpr int B_PIECE = kPanelBytes / HALVES;  // bytes of one B image (hi or lo) per CTA and K block
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[NST], bar_empty[NST];
  __shared__ uint64_t bar_main_full, bar_main_free, bar_corr_full, bar_corr_free, bar_drain[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int ntiles = p.tile_count * HALVES;  // work items of this launch

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(smem_u32(&bar_full[s]), leader ? 2 : 1);  // leader: own producer + the peer's relay
      mbar_init(smem_u32(&bar_empty[s]), kEc ? 2 : 1);
    }
    mbar_init(smem_u32(&bar_main_full), 1);
    mbar_init(smem_u32(&bar_main_free), 16);  // used in the leader only: 8 warps of each CTA
    mbar_init(smem_u32(&bar_corr_full), 1);
    mbar_init(smem_u32(&bar_corr_free), 16);
    mbar_init(smem_u32(&bar_drain[0]), 1);
    mbar_init(smem_u32(&bar_drain[1]), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_base_s), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_main = tmem_base_s;
  const uint32_t tmem_corr = tmem_base_s + 256;
  volatile uint32_t* abortp = &abort_flag;
  // What the leader's two MMA threads need (tcec_gemm_roles.cuh): M = 256 across the pair.
  OperandImage im;
  im.dconst = umma_desc_kmajor_noswizzle(0, 128, 512);
  im.base16 = (smem_base & 0x3ffff) >> 4;
  im.stage16 = Cfg::STAGE_BYTES >> 4;
  im.a_lo16 = kPanelBytes >> 4;
  im.b_hi16 = Cfg::A_BYTES >> 4;
  im.b_lo16 = (Cfg::A_BYTES + kPanelBytes) >> 4;
  im.idesc = umma_idesc(kTf32 ? 2u : 0u, 256, BN);
  const StridedTiles tiles{pair, npairs, ntiles};
  const KWalk walk{p.nkb, p.promo};
  const RingBarriers ring{bar_full, bar_empty};

  if (warp < 4) {
    setmaxnreg_dec<Cfg::REGS_CONTROL>();
    if (warp == 0) {
      // ---------------------------------------------------------- producer (each CTA, own panels)
      if (lane == 0) {
        uint32_t s = 0, ph = 0, armed = 0, armed_parity = 0, it = 0;
        bool ok = true;
        for (int tile = pair; tile < ntiles && ok; tile += npairs) {
          const TileCoord tc = decode_tile(p.tile_first + tile / HALVES, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
          const uint8_t* pa = p.panels_a + tc.b * p.panels_a_batch_stride +
                              static_cast<size_t>(tc.mt * 2 + rank) * p.nkb * Cfg::A_BYTES;
          // whole tile: this CTA's 128-row panel of the tile's two; half: its 64 rows of the half's one panel
          const int nblock = tc.nt * 2 + (BN == 256 ? static_cast<int>(rank) : tile % HALVES);
          const uint8_t* pb = p.panels_b + tc.b * p.panels_b_batch_stride +
                              static_cast<size_t>(nblock) * p.nkb * Cfg::B_BYTES + (BN == 256 ? 0u : rank * B_PIECE);
          for (int kb = 0; kb < p.nkb; ++kb, ++it) {
            if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, abortp, 128)) {
              ok = false;
              break;
            }
            if (dev_flag(p.debug_flags, 1) && it >= static_cast<uint32_t>(NST)) {  // develop builds: no loads
              mbar_arrive(smem_u32(&bar_full[s]));
              if (++s == static_cast<uint32_t>(NST)) {
                s = 0;
                ph ^= 1;
              }
              continue;
            }
            const uint32_t full = smem_u32(&bar_full[s]);
            const uint32_t dst = smem_base + s * Cfg::STAGE_BYTES;
            mbar_arrive_expect_tx(full, Cfg::A_BYTES + Cfg::NP * B_PIECE);
            armed |= 1u << s;
            armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
            bulk_load(dst, pa + static_cast<size_t>(kb) * Cfg::A_BYTES, Cfg::A_BYTES, full);
            const uint8_t* srcb = pb + static_cast<size_t>(kb) * Cfg::B_BYTES;
            if constexpr (BN == 256) {
              bulk_load(dst + Cfg::A_BYTES, srcb, Cfg::B_BYTES, full);
            } else {
#pragma unroll
              for (int h = 0; h < Cfg::NP; ++h)  // hi (+ lo): each image keeps its place in the stage
                bulk_load(dst + Cfg::A_BYTES + h * kPanelBytes, srcb + h * kPanelBytes, B_PIECE, full);
            }
            if (++s == static_cast<uint32_t>(NST)) {
              s = 0;
              ph ^= 1;
            }
          }
        }
        if (!ok) {
          raise_abort_pair(&abort_flag);
          atomicCAS(p.status, 0, kErrProducerWait);
          for (uint32_t q = 0; q < static_cast<uint32_t>(NST); ++q)
            if (armed & (1u << q)) mbar_wait_plain(smem_u32(&bar_full[q]), (armed_parity >> q) & 1);
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        if (!leader) {
          // -------------------------------------------------------- peer: relay "my stage landed"
          uint32_t s = 0, ph = 0, it = 0;
          bool ok = true;
          for (int tile = pair; tile < ntiles && ok; tile += npairs) {
            for (int kb = 0; kb < p.nkb; ++kb, ++it) {
              if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, 32)) {
                ok = false;
                break;
              }
              mbar_arrive_cluster(map_to_cta(smem_u32(&bar_full[s]), 0));
              if (++s == static_cast<uint32_t>(NST)) {
                s = 0;
                ph ^= 1;
              }
            }
          }
          if (!ok) {
            raise_abort_pair(&abort_flag);
            atomicCAS(p.status, 0, kErrMmaWait);
          }
        } else {
          // -------------------------------------------------------- leader: main products
          if (!issue_main_products<kTf32, true, NST>(tiles, walk, im, tmem_main, ring, &bar_main_full,
                                                                    &bar_main_free, abortp, p.debug_flags,
                                                                    blockIdx.x == 0 ? p.trace : nullptr))
            mma_thread_gave_up<true>(&abort_flag, p.status, kErrMmaWait, &bar_drain[0]);
        }
      }
    } else if (warp == 2) {
      // ---------------------------------------------------------- leader: correction products
      if constexpr (kEc) {
        if (lane == 0 && leader) {
          if (!issue_corr_products<kTf32, true, NST>(tiles, walk, im, tmem_corr, ring, &bar_corr_full, &bar_corr_free,
                                                     abortp, p.debug_flags, blockIdx.x == 0 ? p.trace : nullptr))
            mma_thread_gave_up<true>(&abort_flag, p.status, kErrMmaWait, &bar_drain[1]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (each CTA, its 128 rows)
    setmaxnreg_inc<Cfg::REGS_EPILOGUE>();
    const int ew = warp - 4;
    const int q = warp & 3;
    const int colbase = (ew >> 2) * NC;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const float corr_scale = kTf32 ? 1.0f : (1.0f / 2048.0f);
    const bool vec_store = !p.c_col_major && (p.ldc % 4 == 0);
    const uint32_t main_free_leader = map_to_cta(smem_u32(&bar_main_free), 0);
    const uint32_t corr_free_leader = map_to_cta(smem_u32(&bar_corr_free), 0);
    uint32_t chunk = 0, tcount = 0;
    bool ok = true;
    for (int tile = pair; tile < ntiles && ok; tile += npairs, ++tcount) {
      const TileCoord tc = decode_tile(p.tile_first + tile / HALVES, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
      const int nchunks = p.promo ? (p.nkb + p.promo - 1) / p.promo : 1;
      float acc[NC];
      for (int c = 0; c < nchunks; ++c, ++chunk) {
        if (!mbar_wait_warp(smem_u32(&bar_main_full), chunk & 1, abortp)) {
          ok = false;
          break;
        }
        if (warp == 4 && lane == 0) trace_mark(p, 2, chunk);
        tc_fence_after();
        if constexpr (BN == 256) promote_main_chunk<true>(acc, tmem_main + lane_addr + colbase, c == 0);
        else promote_main_chunk(acc, tmem_main + lane_addr + colbase, c == 0);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(main_free_leader);
        if (warp == 4 && lane == 0) trace_mark(p, 3, chunk);
      }
      if (!ok) break;
      if constexpr (kEc) {
        if (!mbar_wait_warp(smem_u32(&bar_corr_full), tcount & 1, abortp)) {
          ok = false;
          break;
        }
        tc_fence_after();
      }
      float* cbase = p.c_array ? p.c_array[tc.b] : p.c + tc.b * p.c_batch_stride;
      const int col0 = tc.nt * 256 + (tile % HALVES) * BN + colbase;
      const bool vec_ok = vec_store && ((reinterpret_cast<uintptr_t>(cbase) & 15) == 0);
      if constexpr (kEc) {
        fold_correction(acc, tmem_corr + lane_addr + colbase, corr_scale);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(corr_free_leader);
      }
      StoreTarget st;
      st.cbase = cbase;
      st.ldc = p.ldc;
      st.M = p.M;
      st.N = p.N;
      st.col_major = p.c_col_major;
      st.vec_ok = vec_ok;
      st.alpha = p.alpha;
      st.beta = p.beta;
      store_warp_block(acc, tc.mt * 256 + static_cast<int>(rank) * 128 + q * 32, col0, st, reinterpret_cast<float*>(smem_gen + Cfg::EPI_OFFSET) + ew * kEpiBufFloats, lane);
    }
    if (!ok) {
      raise_abort_pair(&abort_flag);
      if (lane == 0) atomicCAS(p.status, 0, kErrEpilogueWait);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still signal it or read its operands
  if (warp == 1) tmem_dealloc_pair(tmem_base_s, Cfg::TMEM_COLS);
}

}  // namespace tcec_sm100
