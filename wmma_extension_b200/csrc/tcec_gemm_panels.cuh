// Three-product error-corrected GEMM on tcgen05 over pre-split operand panels.
//
// Restates the reference accumulation (include/wmma_extension/tcec/tcec.hpp:640-706,
// fold at :332-336) at tile scale:
//   main  : A_hi*B_hi accumulates in TMEM for `promo` k-blocks, then is added to
//           an FP32 register accumulator with a round-to-nearest FADD (the
//           reference does this every 16 of K because the tensor-core
//           accumulator truncates; the interval here is a launch parameter).
//           The main and the correction products are issued by two different
//           threads, so the correction stream keeps the tensor pipe busy while
//           the main stream waits for the epilogue to drain its accumulator;
//   corr  : A_lo*B_hi + A_hi*B_lo accumulates in a second TMEM region for the
//           whole K loop, as in the reference;
//   store : C = alpha * (main + corr / 2^11) + beta * C   (tf32: corr / 1).
// Without error correction only the main product exists.
//
// One persistent CTA per SM.  Roles by warp:
//   warp 0      producer  - linear bulk copies of operand panels into a ring
//   warp 1      MMA main  - one thread issues the A_hi*B_hi products; owns TMEM
//   warp 2      MMA corr  - one thread issues the A_lo*B_hi and A_hi*B_lo products
//   warps 4..   epilogue  - tcgen05.ld, RN promotion, fold, alpha/beta, stores
// (issuing an MMA, a commit or a barrier wait costs the issuing thread 50 to 200
// cycles each, so a single thread cannot keep a 128-cycle MMA pipe fed with six
// MMAs, a commit and a wait per k block; two threads can.)
// All hand-offs are mbarriers; every wait is bounded and raises `status`.
#pragma once
#include "sm100_ptx.cuh"
#include "tcec_epilogue.cuh"
#include "tcec_gemm_roles.cuh"
#include "tcec_panels.cuh"

namespace tcec_sm100 {

struct GemmPanelParams {
  int M, N, K;
  int batch;
  int nkb;                 // k blocks (panels along K)
  int tiles_m, tiles_n;    // tiles per matrix
  int promo;               // k blocks per RN promotion; 0 = promote once, at the end
  float alpha, beta;
  const uint8_t* panels_a; // [batch][tiles_m][nkb][hi,lo]
  const uint8_t* panels_b; // [batch][n row blocks of 128][nkb][hi,lo]
  long long panels_a_batch_stride, panels_b_batch_stride;  // bytes
  float* c;                // strided base (used when c_array == nullptr)
  float* const* c_array;
  long long ldc, c_batch_stride;
  int c_col_major;
  int* status;             // device word; non-zero after a wait ran out
  unsigned int* sched;     // [0] tiles handed out beyond the first `sched_base`, [1] CTAs finished; both
                           // zero between launches (the last CTA to finish resets them); null = static
                           // striding (tile, tile + gridDim.x, ...)
  int sched_base;          // tiles below this index are the first tiles of a launch's CTAs (CTA i takes tile i)
  int sched_all_dynamic;   // 1: this launch's CTAs draw even their first tile from the counter (a second
                           // launch that shares the counters of one already running)
  int sched_keep;          // 1: the counters are shared by several launches and reset by the host
  const unsigned int* row_ready;  // optional: one word per `ready_rows` rows of A; the producer loads a tile's
  int ready_rows;                 // operands only once the word of the tile's rows equals `ready_epoch` (A is
  unsigned int ready_epoch;       // arriving from another GPU while the kernel runs); the wait is bounded
  int tile_first, tile_count;  // CTA-pair kernel only: the pair tiles this launch covers
  int store_turn;          // 1: stores go through the per-warp shared-memory buffers (launched with
                           // SMEM_BYTES); 0: direct stores, launched with SMEM_BYTES_NO_TURN
  int debug_flags;         // develop builds only (results invalid): bit 0 = no operand copies after the first ring
                           // fill, bit 1 = no MMAs, bit 5 = one stage is never filled (makes the bounded waits run out)
  unsigned long long* trace;  // develop builds only: CTA 0 writes clock64() at hand-off points
};

enum : int { kErrProducerWait = 1, kErrMmaWait = 2, kErrEpilogueWait = 3, kErrOperandWait = 4 };

template <int BN, bool kTf32, bool kEc>
struct GemmPanelCfg {
  static constexpr int BM = 128;
  static constexpr int NB = BN / 128;                  // 128-row B panels per tile
  static constexpr int NP = kEc ? 2 : 1;               // hi (+ lo)
  static constexpr int A_BYTES = kPanelBytes * NP;
  static constexpr int B_BYTES = kPanelBytes * NP * NB;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int NST_RAW = (208 * 1024) / STAGE_BYTES;
  static constexpr int NST = NST_RAW > 8 ? 8 : NST_RAW;
  static constexpr int EPI_WARPS = 4 * NB;
  static constexpr int EPI_OFFSET = NST * STAGE_BYTES;   // epilogue turn buffers follow the ring
  static constexpr int SMEM_BYTES = NST * STAGE_BYTES + EPI_WARPS * kEpiBufBytes + 1024;
  static constexpr int SMEM_BYTES_NO_TURN = NST * STAGE_BYTES + 1024;  // leaves ~30 KB of the SM to others
  static constexpr int TMEM_COLS = kEc ? 2 * BN : BN;  // 128, 256 or 512: powers of two
  static constexpr int THREADS = 128 + 32 * EPI_WARPS;
  // 256-wide tiles run 384 threads (168 registers each at launch).  The control warpgroup needs
  // few, so it hands registers to the two epilogue warpgroups (setmaxnreg; the shares sum to the
  // launch allocation): with 232 the epilogue keeps two 32-column TMEM loads in flight next to
  // its 128 running sums, which shortens every promotion.
  static constexpr bool REBALANCE = (EPI_WARPS == 8);
  static constexpr int REGS_CONTROL = 40, REGS_EPILOGUE = 232;
  static_assert(!REBALANCE || 128 * REGS_CONTROL + 256 * REGS_EPILOGUE <= THREADS * 168, "register shares");
  static constexpr int GROUP_M = 16;                   // m tiles per raster group
};

__device__ __forceinline__ void trace_mark(const GemmPanelParams& p, int role, uint32_t idx) {
  if (blockIdx.x == 0) trace_slot(p.trace, role, idx);
}
struct TileCoord {
  int b, mt, nt;
};
__device__ __forceinline__ TileCoord decode_tile(int tile, int tiles_m, int tiles_n, int group_m) {
  const int per = tiles_m * tiles_n;
  TileCoord t;
  t.b = tile / per;
  const int r = tile - t.b * per;
  const int span = group_m * tiles_n;
  const int g = r / span;
  const int first_m = g * group_m;
  const int gsz = min(group_m, tiles_m - first_m);
  const int in = r - g * span;
  t.mt = first_m + in % gsz;
  t.nt = in / gsz;
  return t;
}

template <int BN, bool kTf32, bool kEc>
__global__ void __launch_bounds__(GemmPanelCfg<BN, kTf32, kEc>::THREADS, 1)
    tcec_gemm_panels_kernel(const GemmPanelParams p) {
  using Cfg = GemmPanelCfg<BN, kTf32, kEc>;
  constexpr int NST = Cfg::NST;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_full[NST], bar_empty[NST];
  __shared__ uint64_t bar_main_full, bar_main_free, bar_corr_full, bar_corr_free, bar_drain[2];
  __shared__ uint64_t bar_tile_full[kTileRing], bar_tile_empty[kTileRing];
  __shared__ int tile_ring[kTileRing];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));  // generic pointer to the same place
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = p.tiles_m * p.tiles_n * p.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), kEc ? 2 : 1);  // one commit per issuing thread
    }
    mbar_init(smem_u32(&bar_main_full), 1);
    mbar_init(smem_u32(&bar_main_free), Cfg::EPI_WARPS);
    mbar_init(smem_u32(&bar_corr_full), 1);
    mbar_init(smem_u32(&bar_corr_free), Cfg::EPI_WARPS);
    mbar_init(smem_u32(&bar_drain[0]), 1);
    mbar_init(smem_u32(&bar_drain[1]), 1);
    for (int i = 0; i < kTileRing; ++i) {
      mbar_init(smem_u32(&bar_tile_full[i]), 1);
      mbar_init(smem_u32(&bar_tile_empty[i]), (kEc ? 2 : 1) + Cfg::EPI_WARPS);  // MMA threads + epilogue warps
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_main = tmem_base_s;
  const uint32_t tmem_corr = tmem_base_s + BN;
  volatile uint32_t* abortp = &abort_flag;

  if (warp < 4) {
    if constexpr (Cfg::REBALANCE) setmaxnreg_dec<Cfg::REGS_CONTROL>();
  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t it = 0, s = 0, ph = 0;
      uint32_t armed = 0, armed_parity = 0;  // per stage: a copy was issued, and in which phase
      bool ok = true;
      // Tile order: the first gridDim.x tiles by CTA index, the rest drawn from a device-wide
      // counter, so a CTA that got its SM late (another kernel was there) takes fewer tiles
      // instead of delaying the launch.  Every tile (and the end mark) is published to the
      // CTA's other roles through the tile ring.
      uint32_t tq = 0, tph = 0;
      int err = kErrProducerWait;
      int ready_upto = -1;  // last row group of A seen to have arrived
      int tile = (p.sched && p.sched_all_dynamic) ? p.sched_base + static_cast<int>(atomicAdd(&p.sched[0], 1u))
                                                  : static_cast<int>(blockIdx.x);
      for (; ok;) {
        TileCoord tc{0, 0, 0};
        if (tile < ntiles) {
          tc = decode_tile(tile, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
          if (p.row_ready) {
            // A is still arriving: wait (bounded, sleeping between polls) for this tile's rows
            const int grp = (tc.mt * 128) / p.ready_rows;
            if (grp > ready_upto) {
              bool seen = false;
              for (uint32_t i = 0; i < TCEC_WAIT_LIMIT && !seen; ++i) {
                if (ld_acquire_gpu(p.row_ready + grp) == p.ready_epoch) seen = true;
                else {
                  __nanosleep(256);
                  if ((i & 0xff) == 0xff && *abortp) break;
                }
              }
              if (!seen) {
                ok = false;
                err = kErrOperandWait;
                break;
              }
              fence_proxy_async_global();  // the bulk copies below read what that flag announced
              ready_upto = grp;
            }
          }
        }
        if (!mbar_wait(smem_u32(&bar_tile_empty[tq]), tph ^ 1, abortp, 64)) {
          ok = false;
          break;
        }
        tile_ring[tq] = tile < ntiles ? tile : kNoMoreTiles;
        mbar_arrive(smem_u32(&bar_tile_full[tq]));
        if (++tq == static_cast<uint32_t>(kTileRing)) {
          tq = 0;
          tph ^= 1;
        }
        if (tile >= ntiles) break;
        // The next tile is claimed late in this one (two ring fills before its end), so the claim
        // follows the CTA's actual progress, and early enough for the atomic's latency to hide.
        int next_tile = tile + static_cast<int>(gridDim.x);
        const int claim_kb = p.nkb > 2 * NST ? p.nkb - 2 * NST : 0;
        const uint8_t* pa = p.panels_a + tc.b * p.panels_a_batch_stride +
                            static_cast<size_t>(tc.mt) * p.nkb * Cfg::A_BYTES;
        const uint8_t* pb = p.panels_b + tc.b * p.panels_b_batch_stride +
                            static_cast<size_t>(tc.nt) * Cfg::NB * p.nkb * (kPanelBytes * Cfg::NP);
        for (int kb = 0; kb < p.nkb; ++kb, ++it, s = (s + 1 == NST ? 0 : s + 1), ph ^= (s == 0)) {
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, abortp, 128)) {
            ok = false;
            break;
          }
          if (p.sched && kb == claim_kb) next_tile = p.sched_base + static_cast<int>(atomicAdd(&p.sched[0], 1u));
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t dst = smem_base + s * Cfg::STAGE_BYTES;
          if (dev_flag(p.debug_flags, 1) && it >= static_cast<uint32_t>(NST)) {
            mbar_arrive(full);
            continue;
          }
          // injected stall (failure-path test): the first stage after the first ring fill is never filled
          if (dev_flag(p.debug_flags, 32) && it == static_cast<uint32_t>(NST)) continue;
          mbar_arrive_expect_tx(full, Cfg::STAGE_BYTES);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
          bulk_load(dst, pa + static_cast<size_t>(kb) * Cfg::A_BYTES, Cfg::A_BYTES, full);
#pragma unroll
          for (int h = 0; h < Cfg::NB; ++h) {
            const uint8_t* src = pb + (static_cast<size_t>(h) * p.nkb + kb) * (kPanelBytes * Cfg::NP);
            bulk_load(dst + Cfg::A_BYTES + h * kPanelBytes, src, kPanelBytes, full);
            if constexpr (kEc)
              bulk_load(dst + Cfg::A_BYTES + (Cfg::NB + h) * kPanelBytes, src + kPanelBytes,
                        kPanelBytes, full);
          }
        }
        tile = next_tile;
      }
      if (!ok) {
        abort_flag = 1;
        atomicCAS(p.status, 0, err);
        // Let this thread's own copies land before the CTA gives up its shared memory.
        for (uint32_t q = 0; q < static_cast<uint32_t>(NST); ++q)
          if (armed & (1u << q)) mbar_wait_plain(smem_u32(&bar_full[q]), (armed_parity >> q) & 1);
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------------------------------------ MMA issuers (tcec_gemm_roles.cuh)
    if (lane == 0 && (warp == 1 || kEc)) {
      OperandImage im;
      im.dconst = umma_desc_kmajor_noswizzle(0, 128, 512);
      im.base16 = (smem_base & 0x3ffff) >> 4;
      im.stage16 = Cfg::STAGE_BYTES >> 4;
      im.a_lo16 = kPanelBytes >> 4;
      im.b_hi16 = Cfg::A_BYTES >> 4;
      im.b_lo16 = (Cfg::A_BYTES + Cfg::NB * kPanelBytes) >> 4;
      im.idesc = umma_idesc(kTf32 ? 2u : 0u, 128, BN);
      RingTiles tiles{tile_ring, bar_tile_full, bar_tile_empty};
      const KWalk walk{p.nkb, p.promo};
      const RingBarriers ring{bar_full, bar_empty};
      unsigned long long* trace = blockIdx.x == 0 ? p.trace : nullptr;
      if (warp == 1) {
        if (!issue_main_products<kTf32, false, NST>(tiles, walk, im, tmem_main, ring, &bar_main_full, &bar_main_free,
                                                    abortp, p.debug_flags, trace))
          mma_thread_gave_up<false>(&abort_flag, p.status, kErrMmaWait, &bar_drain[0]);
      } else {
        if (!issue_corr_products<kTf32, false, NST>(tiles, walk, im, tmem_corr, ring, &bar_corr_full, &bar_corr_free,
                                                    abortp, p.debug_flags, trace))
          mma_thread_gave_up<false>(&abort_flag, p.status, kErrMmaWait, &bar_drain[1]);
      }
    }
  }
  } else {
    // ------------------------------------------------------------ epilogue
    if constexpr (Cfg::REBALANCE) setmaxnreg_inc<Cfg::REGS_EPILOGUE>();
    const int ew = warp - 4;
    const int q = warp & 3;          // TMEM lane quarter this warp may read
    const int colbase = (ew >> 2) * 128;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const float corr_scale = kTf32 ? 1.0f : (1.0f / 2048.0f);
    const bool vec_store = !p.c_col_major && (p.ldc % 4 == 0);
    uint32_t chunk = 0, tcount = 0;
    bool ok = true;
    RingTiles tiles{tile_ring, bar_tile_full, bar_tile_empty};
    for (; ok; ++tcount) {
      const int tile = tiles.next_warp(abortp);
      if (tile == kNoMoreTiles) break;
      if (tile == kTileWaitFailed) {
        ok = false;
        break;
      }
      const TileCoord tc = decode_tile(tile, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
      const int nchunks = p.promo ? (p.nkb + p.promo - 1) / p.promo : 1;
      float acc[128];
      for (int c = 0; c < nchunks; ++c, ++chunk) {
        if (!mbar_wait_warp(smem_u32(&bar_main_full), chunk & 1, abortp)) {
          ok = false;
          break;
        }
        if (warp == 4 && lane == 0) trace_mark(p, 2, chunk);
        tc_fence_after();
        promote_main_chunk<Cfg::REBALANCE>(acc, tmem_main + lane_addr + colbase, c == 0);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_main_free));
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
      const int col0 = tc.nt * BN + colbase;
      const bool vec_ok = vec_store && ((reinterpret_cast<uintptr_t>(cbase) & 15) == 0);
      if constexpr (kEc) {
        // Fold the correction term into the registers first and hand the accumulator back
        // before the stores: the next tile's correction MMAs then overlap this tile's stores.
        fold_correction(acc, tmem_corr + lane_addr + colbase, corr_scale);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_corr_free));
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
      if (p.store_turn)
        store_warp_block(acc, tc.mt * 128 + q * 32, col0, st,
                         reinterpret_cast<float*>(smem_gen + Cfg::EPI_OFFSET) + ew * kEpiBufFloats, lane);
      else
        store_row_slice(acc, tc.mt * 128 + q * 32 + lane, col0, st);
    }
    if (!ok) {
      abort_flag = 1;
      if (lane == 0) atomicCAS(p.status, 0, kErrEpilogueWait);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base_s, Cfg::TMEM_COLS);
  if (threadIdx.x == 0 && p.sched && !p.sched_keep) {
    // Every CTA has drawn its last tile by now; the last one out leaves the counters at zero.
    __threadfence();
    if (atomicAdd(&p.sched[1], 1u) == gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
}

}  // namespace tcec_sm100
