// Error-corrected GEMM on tcgen05 that reads the FP32 operands directly: TMA loads FP32 tiles
// into shared memory, eight converter warps split them in registers into fp16 hi and scaled
// residual (reference include/wmma_extension/tcec/tcec.hpp:219-223, scale.hpp:8-20) and write
// the tensor-core operand image IN PLACE over the FP32 data, two threads issue the three
// products into TMEM, and eight epilogue warps promote the main term with round-to-nearest
// adds, fold the correction term and store (tcec.hpp:640-706 and :332-336).
//
// Compared with the panel kernel (tcec_gemm_panels.cuh) nothing is written to or re-read from
// global memory between the split and the products, which more than halves the DRAM traffic of
// a GEMM: this is the kernel for shapes bound by HBM (batches of small matrices).
//
// What bounds it is shared-memory bandwidth (128 bytes per clock): every FP32 byte is written by
// TMA, read and written back by a converter, and read by the tensor pipe once per product that
// uses it.  The kernel therefore runs on CTA PAIRS (tcgen05 cta_group::2): two SMs share one
// 256 x 256 output tile, each loads and converts its 128 rows of A and only its 128 of the
// tile's 256 B rows (32 KB per K block instead of 48), and the leader CTA issues every MMA for
// both (M = 256).  Per SM and K block that is 144 KB through shared memory instead of 216, and B
// is loaded and converted once per tile row instead of twice.
//
// In-place conversion.  The fp16 hi and lo images of an FP32 block take exactly the block's
// bytes, and the un-swizzled UMMA descriptor leaves the 8-row-group stride free, so every
// 8-row x 32-k group keeps its own 1 KB: FP32 rows (8 x 128 B, TMA 128-byte swizzle) become
// 512 B of hi core matrices followed by 512 B of lo core matrices.  A K-contiguous unit is one
// such group: a warp reads it into registers, __syncwarp()s, and writes it back (lane = row,
// 16-byte k chunk).  A unit of an operand whose rows are contiguous instead (A column-major,
// B row-major) is a 32-k x 32-row TMA box of 4 KB, four groups, transposed on the way by a PAIR
// of warps (lane = row; each warp takes 16 of the 32 k), which meet at a hardware barrier between
// reading and writing.  One ring of five 32 KB stages therefore serves as FP32 landing zone and
// as operand buffer: each stage goes TMA -> convert -> MMA -> free.
//
// C leaves through TMA as well when it can (row-major, beta == 0, 16-byte aligned rows): an
// epilogue warp writes each 32 x 32 block of its results into one of its two 4 KB shared-memory
// boxes (eight 128-bit stores per lane, 128-byte swizzle) and one lane issues a tensor store.
// Measured on 8192 x 256^3: the store phase of a tile takes 5.5 k cycles this way against 10.8 k
// with stores from registers (turned through shared memory into full lines) and 14.6 k with the
// panel kernel's store path, which other C layouts and beta != 0 still take.
//
// Pair protocol (rank 0 = leader, rank 1 = peer), all hand-offs mbarriers with bounded waits:
//   landed[s]   local: the stage's TMA bytes
//   conv[s]     local: one arrive per converter warp
//   full[s]     leader's: one arrive from each CTA's relay thread, which waits on its conv[s]
//   empty[s]    committed by the leader's MMA threads to BOTH CTAs (multicast commit)
//   main_full / corr_full   likewise committed to both CTAs; each CTA drains its own TMEM
//   main_free / corr_free   leader's: 8 local epilogue warps + 8 remote arrives
// Both CTAs meet at a cluster barrier after set-up and before exit.
//
// Roles by warp (640 threads in five warpgroups, one persistent CTA per SM).  The register file
// is re-balanced at entry with setmaxnreg: the kernel launches with 96 registers per thread, the
// control warpgroup drops to 32, the converters to 40 and the epilogue rises to 184 (the shares
// must sum to no more than the launch allocation, or the raise would never be granted).
//   warp 0       lane 0: TMA producer (own rows of A, own half of B)
//   warp 1       lane 0: leader: MMA issuer, main products
//   warp 2       lane 0: leader: MMA issuer, correction products
//   warp 3       lane 0: relay of "my half of the stage is converted" to the leader
//   warps 4-11   epilogue (own 128 rows of the tile)
//   warps 12-19  converters (sixteen warps were measured no faster than eight: the conversion is
//                bound by shared-memory bandwidth, not by issue slots)
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
  int tiles_m, tiles_n;  // 256 x 256 pair tiles per matrix
  int promo;             // K blocks per RN promotion; 0 = once, at the end
  int a_k_contiguous;    // A is row-major (K contiguous); else column-major
  int b_k_contiguous;    // B is column-major (K contiguous); else row-major
  int c_tma;             // C is written with tensor stores through map_c (row-major, beta == 0)
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
  static constexpr int STG_A = 128 * 128;  // this CTA's 128 rows x 32 fp32 of A, also the size of their hi + lo image
  static constexpr int STG_B = 128 * 128;  // this CTA's 128 of the tile's 256 B rows
  static constexpr int STAGE = STG_A + STG_B;
  static constexpr int NST = 5;
  static constexpr int NBOX = 2;  // 4 KB store boxes per epilogue warp
  static constexpr int EPI_WARPS = 8;
  static constexpr int CONV_WARPS = 8;
  static constexpr int EPI_OFFSET = NST * STAGE;  // after the ring: one turn buffer per epilogue warp
  static constexpr int EPI_BYTES = EPI_WARPS * (NBOX * 4096 > kEpiBufBytes ? NBOX * 4096 : kEpiBufBytes);
  static constexpr int SMEM_BYTES = NST * STAGE + EPI_BYTES + 1024;
  static_assert(SMEM_BYTES <= 232448 - 512, "dynamic + static shared memory exceed an SM");
  static constexpr int TMEM_COLS = kEc ? 512 : 256;
  static constexpr int THREADS = 128 + 32 * EPI_WARPS + 32 * CONV_WARPS;
  // setmaxnreg moves registers inside the CTA's launch allocation (896 threads x 72), so the
  // three shares must fit in it: a request beyond it would wait forever.
  static constexpr int REGS_LAUNCH = 96, REGS_CONTROL = 32, REGS_CONVERT = 40, REGS_EPILOGUE = 184;
  static_assert(128 * REGS_CONTROL + 32 * CONV_WARPS * REGS_CONVERT + 32 * EPI_WARPS * REGS_EPILOGUE <=
                    THREADS * REGS_LAUNCH,
                "register shares exceed the launch allocation");
  static_assert(THREADS * REGS_LAUNCH <= 65536, "launch allocation exceeds the register file");
  static constexpr int GROUP_BYTES = 1024;  // one 8-row group: hi at +0, lo at +512
  static constexpr int GROUP_M = 8;         // pair tiles are 256 rows tall
  static constexpr int kBoxBarrier0 = 1;    // hardware barriers 1..4: one per converter warp pair
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

// One row-contiguous unit: a 32-k x 32-row box (4 KB, k-row kk at kk * 128 B, 16-byte chunk j of it
// stored at j ^ (kk % 8)), which becomes four groups.  Two warps share it: lane = row, `half`
// (0 or 1) selects k 0..15 or 16..31.  Both must have read before either writes: they meet at
// hardware barrier `bar_id` (64 threads).
template <bool kEc>
__device__ __forceinline__ void convert_box_inplace_pair(uint8_t* t, int half, uint32_t bar_id, int lane) {
  float v[2][8];
  const uint8_t* src = t + (lane & 3) * 4;
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int e = 0; e < 8; ++e)
      v[c][e] = *reinterpret_cast<const float*>(src + ((2 * half + c) * 8 + e) * 128 + (((lane >> 2) ^ e) << 4));
  named_barrier_sync(bar_id, 64);
  uint8_t* g = t + (lane >> 3) * 1024 + (lane & 7) * 16;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint4 hi, lo;
    split8_f16(v[c], hi, lo);
    *reinterpret_cast<uint4*>(g + (2 * half + c) * 128) = hi;
    if constexpr (kEc) *reinterpret_cast<uint4*>(g + 512 + (2 * half + c) * 128) = lo;
  }
}

// p.tiles_m counts 256-row pair tiles.
template <bool kEc>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GemmFusedCfg<kEc>::THREADS, 1)
    tcec_gemm_fused_kernel(const GemmFusedParams p, const __grid_constant__ CUtensorMap map_a,
                           const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c) {
  using Cfg = GemmFusedCfg<kEc>;
  constexpr int NST = Cfg::NST, BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_landed[NST], bar_conv[NST], bar_full[NST], bar_empty[NST];
  __shared__ uint64_t bar_main_full, bar_main_free, bar_corr_full, bar_corr_free, bar_drain[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_flag;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));  // generic pointer to the same place
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int ntiles = p.tiles_m * p.tiles_n * p.batch;
  const bool tracing = (blockIdx.x == 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(smem_u32(&bar_landed[s]), 1);
      mbar_init(smem_u32(&bar_conv[s]), Cfg::CONV_WARPS);
      mbar_init(smem_u32(&bar_full[s]), 2);  // used in the leader only: one relay arrive per CTA
      mbar_init(smem_u32(&bar_empty[s]), kEc ? 2 : 1);
    }
    mbar_init(smem_u32(&bar_main_full), 1);
    mbar_init(smem_u32(&bar_main_free), 2 * Cfg::EPI_WARPS);  // used in the leader only
    mbar_init(smem_u32(&bar_corr_full), 1);
    mbar_init(smem_u32(&bar_corr_free), 2 * Cfg::EPI_WARPS);
    mbar_init(smem_u32(&bar_drain[0]), 1);
    mbar_init(smem_u32(&bar_drain[1]), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_base_s), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_main = tmem_base_s;
  const uint32_t tmem_corr = tmem_base_s + BN;
  volatile uint32_t* abortp = &abort_flag;

  if (warp >= 4 + Cfg::EPI_WARPS) {
    // ------------------------------------------------------------ converters
    setmaxnreg_dec<Cfg::REGS_CONVERT>();
    const int cw = warp - (4 + Cfg::EPI_WARPS);
    uint32_t s = 0, ph = 0;
    [[maybe_unused]] uint32_t cit = 0;
    bool ok = true;
    for (int tile = pair; tile < ntiles && ok; tile += npairs) {
      for (int kb = 0; kb < p.nkb; ++kb) {
        if (!mbar_wait_warp(smem_u32(&bar_landed[s]), ph, abortp, 32)) {
          ok = false;
          break;
        }
        mbar_try_wait(smem_u32(&bar_landed[s]), ph);  // each lane observes the completed phase itself
        if (cw == 0 && lane == 0 && tracing) trace_slot(p.trace, 2, cit);  // landed
        uint8_t* stage = smem_gen + s * Cfg::STAGE;
        if (!dev_flag(p.debug_flags, 4)) {
          // the stage as 32 groups of 1 KB (A: 0..15, B: 16..31): two per warp; or as 8 boxes of
          // 4 KB (A: 0..3, B: 4..7): one per warp pair
          // The stage is 32 groups of 1 KB (A: 0..15, B: 16..31) where K is contiguous, 4 boxes of
          // 4 KB per operand where rows are; groups are dealt to warps, boxes to warp pairs.
          constexpr int W = Cfg::CONV_WARPS;
          if (p.a_k_contiguous && p.b_k_contiguous) {
#pragma unroll 1
            for (int g = cw; g < 32; g += W) convert_groups_inplace<kEc, 1>(stage + g * 1024, 0, lane);
          } else if (!p.a_k_contiguous && !p.b_k_contiguous) {
#pragma unroll 1
            for (int bx = cw >> 1; bx < 8; bx += W / 2)
              convert_box_inplace_pair<kEc>(stage + bx * 4096, cw & 1, Cfg::kBoxBarrier0 + (cw >> 1), lane);
          } else {
            // one operand in groups (first half of the warps), the other in boxes (pairs of the second half)
            uint8_t* grp = stage + (p.a_k_contiguous ? 0 : Cfg::STG_A);
            uint8_t* bxs = stage + (p.a_k_contiguous ? Cfg::STG_A : 0);
            if (cw < W / 2) {
#pragma unroll 1
              for (int g = cw; g < 16; g += W / 2) convert_groups_inplace<kEc, 1>(grp + g * 1024, 0, lane);
            } else {
#pragma unroll 1
              for (int bx = (cw - W / 2) >> 1; bx < 4; bx += W / 4)
                convert_box_inplace_pair<kEc>(bxs + bx * 4096, cw & 1, Cfg::kBoxBarrier0 + (cw >> 1), lane);
            }
          }
        }
        fence_proxy_async_smem();  // image written with ordinary stores, read by the tensor pipe
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_conv[s]));
        if (cw == 0 && lane == 0 && tracing) trace_slot(p.trace, 3, cit);  // converted
        ++cit;
        if (++s == static_cast<uint32_t>(NST)) {
          s = 0;
          ph ^= 1;
        }
      }
    }
    if (!ok) {
      raise_abort_pair(&abort_flag);
      if (lane == 0) atomicCAS(p.status, 0, kErrProducerWait);
    }
  } else if (warp < 4) {
    setmaxnreg_dec<Cfg::REGS_CONTROL>();
    if (lane == 0 && warp == 0) {
      // ---------------------------------------------------------- TMA producer
      uint32_t s = 0, ph = 0, armed = 0, armed_parity = 0;
      [[maybe_unused]] uint32_t pit = 0;
      bool ok = true;
      for (int tile = pair; tile < ntiles && ok; tile += npairs) {
        const TileCoord tc = decode_tile(tile, p.tiles_m, p.tiles_n, Cfg::GROUP_M);
        const int arow = tc.mt * 256 + static_cast<int>(rank) * 128, brow = tc.nt * 256 + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < p.nkb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, abortp, 64)) {
            ok = false;
            break;
          }
          const uint32_t landed = smem_u32(&bar_landed[s]);
          const uint32_t dst = smem_base + s * Cfg::STAGE;
          mbar_arrive_expect_tx(landed, Cfg::STAGE);
          if (tracing) trace_slot(p.trace, 8, pit++);
          armed |= 1u << s;
          armed_parity = (armed_parity & ~(1u << s)) | (ph << s);
          if (p.a_k_contiguous) {
            tma_load_3d(dst, &map_a, landed, kb * 32, arow, tc.b);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) tma_load_3d(dst + j * 4096, &map_a, landed, arow + 32 * j, kb * 32, tc.b);
          }
          if (p.b_k_contiguous) {
            tma_load_3d(dst + Cfg::STG_A, &map_b, landed, kb * 32, brow, tc.b);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_3d(dst + Cfg::STG_A + j * 4096, &map_b, landed, brow + 32 * j, kb * 32, tc.b);
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
          if (armed & (1u << q)) mbar_wait_plain(smem_u32(&bar_landed[q]), (armed_parity >> q) & 1);
      }
    } else if (lane == 0 && warp == 3) {
      // ---------------------------------------------------------- relay: my half of the stage is converted
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (int tile = pair; tile < ntiles && ok; tile += npairs) {
        for (int kb = 0; kb < p.nkb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_conv[s]), ph, abortp, 32)) {
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
    } else if (lane == 0 && leader && (warp == 1 || (kEc && warp == 2))) {
      // ---------------------------------------------------------- leader: MMA issuers (tcec_gemm_roles.cuh)
      OperandImage im;
      im.dconst = umma_desc_kmajor_noswizzle(0, 128, Cfg::GROUP_BYTES);  // core matrices 128 B apart along K, groups 1 KB apart
      im.base16 = (smem_base & 0x3ffff) >> 4;
      im.stage16 = Cfg::STAGE >> 4;
      im.a_lo16 = 512 >> 4;
      im.b_hi16 = Cfg::STG_A >> 4;
      im.b_lo16 = (Cfg::STG_A + 512) >> 4;
      im.idesc = umma_idesc(0u, 256, BN);
      const StridedTiles tiles{pair, npairs, ntiles};
      const KWalk walk{p.nkb, p.promo};
      const RingBarriers ring{bar_full, bar_empty};
      if (warp == 1) {
        if (!issue_main_products<false, true, NST>(tiles, walk, im, tmem_main, ring, &bar_main_full, &bar_main_free,
                                                   abortp, p.debug_flags, tracing ? p.trace : nullptr))
          mma_thread_gave_up<true>(&abort_flag, p.status, kErrMmaWait, &bar_drain[0]);
      } else {
        if (!issue_corr_products<false, true, NST>(tiles, walk, im, tmem_corr, ring, &bar_corr_full, &bar_corr_free,
                                                   abortp, p.debug_flags, tracing ? p.trace : nullptr))
          mma_thread_gave_up<true>(&abort_flag, p.status, kErrMmaWait, &bar_drain[1]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (each CTA, its 128 rows)
    setmaxnreg_inc<Cfg::REGS_EPILOGUE>();
    const int ew = warp - 4;
    const int q = warp & 3;
    const int colbase = (ew >> 2) * 128;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t main_free_leader = map_to_cta(smem_u32(&bar_main_free), 0);
    const uint32_t corr_free_leader = map_to_cta(smem_u32(&bar_corr_free), 0);
    uint32_t chunk = 0, tcount = 0, nbox = 0;
    bool ok = true;
    const uint32_t box0 = smem_base + Cfg::EPI_OFFSET + ew * (Cfg::NBOX * 4096), box_row = box0 + lane * 128;
    const bool etrace = (warp == 4 && lane == 0 && tracing);
    for (int tile = pair; tile < ntiles && ok; tile += npairs, ++tcount) {
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
        promote_main_chunk_narrow(acc, tmem_main + lane_addr + colbase, c == 0);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(main_free_leader);
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
        fold_correction_narrow(acc, tmem_corr + lane_addr + colbase, 1.0f / 2048.0f);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(corr_free_leader);
        if (etrace) trace_slot(p.trace, 7, 3 * tcount + 1);
      }
      if (dev_flag(p.debug_flags, 8)) continue;
      // alpha is applied in place (one rounding, as in the other kernels' stores), so the store
      // paths below need no temporaries beside the 128 results
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = __fmul_rn(p.alpha, acc[i]);
      const int row0 = tc.mt * 256 + static_cast<int>(rank) * 128 + q * 32, col0 = tc.nt * BN + colbase;
      if (p.c_tma) {
        if (row0 < p.M) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            if (col0 + cc * 32 < p.N) {
              const uint32_t boff = (nbox % Cfg::NBOX) * 4096;
              ++nbox;
              if (lane == 0) bulk_wait_group_read<Cfg::NBOX - 1>();  // the store that used this box has left it
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j)
                st_shared_v4(box_row + boff + ((j ^ (lane & 7)) << 4), acc[cc * 32 + 4 * j + 0],
                             acc[cc * 32 + 4 * j + 1], acc[cc * 32 + 4 * j + 2], acc[cc * 32 + 4 * j + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&map_c, box0 + boff, col0 + cc * 32, row0, tc.b);
                bulk_commit_group();
              }
            }
          }
        }
        if (etrace) trace_slot(p.trace, 7, 3 * tcount + 2);
        continue;
      }
      StoreTarget st;
      st.cbase = p.c + tc.b * p.c_batch_stride;
      st.ldc = p.ldc;
      st.M = p.M;
      st.N = p.N;
      st.col_major = p.c_col_major;
      st.vec_ok = !p.c_col_major && (p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(st.cbase) & 15) == 0);
      st.alpha = 1.0f;  // already applied
      st.beta = p.beta;
      store_warp_block(acc, row0, col0, st,
                       reinterpret_cast<float*>(smem_gen + Cfg::EPI_OFFSET) + ew * (Cfg::EPI_BYTES / Cfg::EPI_WARPS / 4), lane);
      if (etrace) trace_slot(p.trace, 7, 3 * tcount + 2);
    }
    if (p.c_tma && lane == 0) bulk_wait_group<0>();  // this lane's stores are complete before the CTA ends
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
