// Roles shared by the three GEMM kernels (operand panels on one SM, operand panels on a CTA
// pair, FP32 tiles converted in shared memory): the two MMA-issuing threads and the register side
// of the epilogue.  The kernels differ in how a stage of the ring gets filled and in where the
// operand images sit inside it; from `full[s]` onward they do the same thing.
//
// Arithmetic (reference include/wmma_extension/tcec/tcec.hpp:640-706): per K block the main
// accumulator takes A_hi B_hi, the correction accumulator A_lo B_hi + A_hi B_lo; the main
// accumulator is handed to the epilogue every `promo` K blocks (round-to-nearest promotion), the
// correction accumulator once per tile.
#pragma once
#include "sm100_ptx.cuh"

namespace tcec_sm100 {

// Where the operand images of one ring stage live, in the 16-byte units of a UMMA descriptor.
struct OperandImage {
  uint64_t dconst;     // descriptor without its start address (strides, layout type, version)
  uint32_t base16;     // ring base
  uint32_t stage16;    // stage size
  uint32_t a_lo16;     // offsets inside a stage (A hi is at 0)
  uint32_t b_hi16;
  uint32_t b_lo16;
  uint32_t idesc;      // instruction descriptor (type, M, N)
};

// How K is cut.
struct KWalk {
  int nkb;    // K blocks per tile
  int promo;  // K blocks per promotion chunk; 0 = one chunk per tile
};

// Where a consumer role learns its next tile.  next() returns the tile index, kNoMoreTiles, or
// kTileWaitFailed when a bounded wait ran out.
enum : int { kNoMoreTiles = -1, kTileWaitFailed = -2 };

// Static striding: tile, tile + stride, ...
struct StridedTiles {
  int tile, stride, ntiles;
  __device__ __forceinline__ int next(volatile uint32_t*) {
    if (tile >= ntiles) return kNoMoreTiles;
    const int t = tile;
    tile += stride;
    return t;
  }
};

// Tiles published by the CTA's producer thread through a small shared-memory ring (the producer
// draws them from a device-wide counter, so a CTA that starts late simply processes fewer).
// `empty` expects one arrive from every consumer: the MMA threads and each epilogue warp.
constexpr int kTileRing = 4;
struct RingTiles {
  const volatile int* ring;
  uint64_t* full;
  uint64_t* empty;
  uint32_t slot = 0, ph = 0;
  // single-thread consumers
  __device__ __forceinline__ int next(volatile uint32_t* abortp) {
    if (!mbar_wait(smem_u32(&full[slot]), ph, abortp, 64)) return kTileWaitFailed;
    const int t = ring[slot];
    mbar_arrive(smem_u32(&empty[slot]));
    advance();
    return t;
  }
  // warp-collective consumers (all 32 lanes call it)
  __device__ __forceinline__ int next_warp(volatile uint32_t* abortp) {
    if (!mbar_wait_warp(smem_u32(&full[slot]), ph, abortp, 64)) return kTileWaitFailed;
    mbar_try_wait(smem_u32(&full[slot]), ph);  // each lane observes the completed phase itself
    const int t = ring[slot];
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&empty[slot]));
    advance();
    return t;
  }
  __device__ __forceinline__ void advance() {
    if (++slot == static_cast<uint32_t>(kTileRing)) {
      slot = 0;
      ph ^= 1;
    }
  }
};

struct RingBarriers {
  uint64_t* full;   // [NST] stage filled
  uint64_t* empty;  // [NST] stage consumed (one commit per issuing thread)
};

template <bool kTf32, bool kPair>
__device__ __forceinline__ void umma_issue(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if constexpr (kPair) umma_ss_pair<kTf32>(d_tmem, a, b, idesc, acc);
  else umma_ss<kTf32>(d_tmem, a, b, idesc, acc);
}
template <bool kPair>
__device__ __forceinline__ void umma_commit_to(uint32_t bar) {
  if constexpr (kPair) umma_commit_pair(bar);
  else umma_commit(bar);
}

// Development aids exist only in builds with -DTCEC_DEVELOP: switches that leave out parts of a
// kernel for timing experiments (results invalid) and hand-off timestamps (`trace` is null except
// in the CTA that records; kTraceRoles rows of 4096 slots).  The default build compiles both away.
constexpr int kTraceRoles = 12;
#ifdef TCEC_DEVELOP
__device__ __forceinline__ bool dev_flag(int flags, int bit) { return (flags & bit) != 0; }
__device__ __forceinline__ void trace_slot(unsigned long long* trace, int role, uint32_t idx) {
  if (trace && idx < 4096) trace[role * 4096 + idx] = clock64();
}
#else
__device__ __forceinline__ constexpr bool dev_flag(int, int) { return false; }
__device__ __forceinline__ void trace_slot(unsigned long long*, int, uint32_t) {}
#endif

// One thread: the main products of every tile of the walk.  Kept to a handful of integer
// instructions per MMA: descriptors are a constant OR-ed with a 14-bit address field, ring
// positions and the promotion interval are counters.  Returns false when a bounded wait ran out.
// Develop builds only: debug_flags bit 1 issues no MMAs.
template <bool kTf32, bool kPair, int NST, class TileSource>
__device__ __forceinline__ bool issue_main_products(TileSource tiles, const KWalk& w, const OperandImage& im,
                                                    uint32_t tmem_main,
                                                    const RingBarriers& ring, uint64_t* bar_main_full,
                                                    uint64_t* bar_main_free, volatile uint32_t* abortp,
                                                    int debug_flags, unsigned long long* trace) {
  uint32_t it = 0, s = 0, ph = 0, chunk = 0;
  for (;;) {
    const int tile = tiles.next(abortp);
    if (tile == kNoMoreTiles) break;
    if (tile == kTileWaitFailed) return false;
    int left_in_chunk = 0;  // K blocks still to issue in the current chunk
    for (int kb = 0; kb < w.nkb; ++kb, ++it) {
      if (!mbar_wait(smem_u32(&ring.full[s]), ph, abortp, 32u)) return false;
      trace_slot(trace, 0, it);
      const bool first_in_chunk = (left_in_chunk == 0);
      if (first_in_chunk) {
        const int rest = w.nkb - kb;
        left_in_chunk = (w.promo && w.promo < rest) ? w.promo : rest;
        // the epilogue has drained the previous chunk (hot poll: the tensor pipe waits on this)
        if (!mbar_wait(smem_u32(bar_main_free), (chunk & 1) ^ 1, abortp, 0)) return false;
        trace_slot(trace, 1, chunk);
      }
      tc_fence_after();
      const uint32_t a16 = im.base16 + s * im.stage16;
      if (!dev_flag(debug_flags, 2)) {
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j)
          umma_issue<kTf32, kPair>(tmem_main, im.dconst | (a16 + 16 * j), im.dconst | (a16 + im.b_hi16 + 16 * j),
                                   im.idesc, (first_in_chunk && j == 0) ? 0u : 1u);
      }
      if (--left_in_chunk == 0) {
        umma_commit_to<kPair>(smem_u32(bar_main_full));
        ++chunk;
      }
      umma_commit_to<kPair>(smem_u32(&ring.empty[s]));
      trace_slot(trace, 5, it);
      if (++s == static_cast<uint32_t>(NST)) {
        s = 0;
        ph ^= 1;
      }
    }
  }
  return true;
}

// One thread: the correction products of every tile of the walk.
template <bool kTf32, bool kPair, int NST, class TileSource>
__device__ __forceinline__ bool issue_corr_products(TileSource tiles, const KWalk& w, const OperandImage& im,
                                                    uint32_t tmem_corr,
                                                    const RingBarriers& ring, uint64_t* bar_corr_full,
                                                    uint64_t* bar_corr_free, volatile uint32_t* abortp,
                                                    int debug_flags, unsigned long long* trace) {
  uint32_t s = 0, ph = 0, tcount = 0, it = 0;
  for (;; ++tcount) {
    const int tile = tiles.next(abortp);
    if (tile == kNoMoreTiles) break;
    if (tile == kTileWaitFailed) return false;
    for (int kb = 0; kb < w.nkb; ++kb, ++it) {
      if (!mbar_wait(smem_u32(&ring.full[s]), ph, abortp, 32u)) return false;
      if (kb == 0) {
        // the epilogue has folded the previous tile's correction term
        if (!mbar_wait(smem_u32(bar_corr_free), (tcount & 1) ^ 1, abortp, 32)) return false;
      }
      trace_slot(trace, 4, it);
      tc_fence_after();
      const uint32_t c16 = im.base16 + s * im.stage16;
      if (!dev_flag(debug_flags, 2)) {
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j)
          umma_issue<kTf32, kPair>(tmem_corr, im.dconst | (c16 + im.a_lo16 + 16 * j),
                                   im.dconst | (c16 + im.b_hi16 + 16 * j), im.idesc, (kb == 0 && j == 0) ? 0u : 1u);
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j)
          umma_issue<kTf32, kPair>(tmem_corr, im.dconst | (c16 + 16 * j), im.dconst | (c16 + im.b_lo16 + 16 * j),
                                   im.idesc, 1u);
      }
      umma_commit_to<kPair>(smem_u32(&ring.empty[s]));
      if (++s == static_cast<uint32_t>(NST)) {
        s = 0;
        ph ^= 1;
      }
    }
    umma_commit_to<kPair>(smem_u32(bar_corr_full));
  }
  return true;
}

// An MMA thread whose wait ran out: raise the flags, then make sure nothing it issued still
// writes TMEM when the CTA releases it.
template <bool kPair>
__device__ __forceinline__ void mma_thread_gave_up(uint32_t* abort_flag, int* status, int code, uint64_t* bar_drain) {
  if constexpr (kPair) raise_abort_pair(abort_flag);
  else *abort_flag = 1;
  atomicCAS(status, 0, code);
  umma_commit_to<kPair>(smem_u32(bar_drain));
  mbar_wait_plain(smem_u32(bar_drain), 0);
}

// Epilogue thread: add (or, for a tile's first chunk, copy) this thread's 128 columns of the main
// accumulator into its running sums with IEEE round-to-nearest adds (tcec.hpp:676-679).
// kWide keeps two 32-column loads in flight per wait (needs the larger register share).
template <bool kWide>
__device__ __forceinline__ void promote_main_chunk(float (&acc)[128], uint32_t taddr, bool first) {
  if constexpr (kWide) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t v0[32], v1[32];
      tmem_ld_32x32b_x32(taddr + (2 * h) * 32, v0);
      tmem_ld_32x32b_x32(taddr + (2 * h + 1) * 32, v1);
      tmem_ld_wait();
      if (first) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[(2 * h) * 32 + i] = __uint_as_float(v0[i]);
          acc[(2 * h + 1) * 32 + i] = __uint_as_float(v1[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          acc[(2 * h) * 32 + i] += __uint_as_float(v0[i]);
          acc[(2 * h + 1) * 32 + i] += __uint_as_float(v1[i]);
        }
      }
    }
  } else {
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(taddr + cc * 32, v);
      tmem_ld_wait();
      if (first) {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[cc * 32 + i] = __uint_as_float(v[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[cc * 32 + i] += __uint_as_float(v[i]);
      }
    }
  }
}

// The 64-column forms (half-width tiles of the CTA-pair kernel): one wait per step.
__device__ __forceinline__ void promote_main_chunk(float (&acc)[64], uint32_t taddr, bool first) {
  uint32_t v0[32], v1[32];
  tmem_ld_32x32b_x32(taddr, v0);
  tmem_ld_32x32b_x32(taddr + 32, v1);
  tmem_ld_wait();
  if (first) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      acc[i] = __uint_as_float(v0[i]);
      acc[32 + i] = __uint_as_float(v1[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      acc[i] += __uint_as_float(v0[i]);
      acc[32 + i] += __uint_as_float(v1[i]);
    }
  }
}
__device__ __forceinline__ void fold_correction(float (&acc)[64], uint32_t taddr, float scale) {
  uint32_t v0[32], v1[32];
  tmem_ld_32x32b_x32(taddr, v0);
  tmem_ld_32x32b_x32(taddr + 32, v1);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    acc[i] = acc[i] + __uint_as_float(v0[i]) * scale;
    acc[32 + i] = acc[32 + i] + __uint_as_float(v1[i]) * scale;
  }
}

// The same two steps for kernels whose epilogue has a smaller register share (128 sums + 32
// temporaries).  A tile's first chunk is loaded straight into the sums with one wait; later chunks
// and the correction term come in pairs of 16-column loads, both in flight before the one wait
// (a TMEM load costs ~200 cycles whatever its width, so what counts is how many waits there are).
__device__ __forceinline__ void promote_main_chunk_narrow(float (&acc)[128], uint32_t taddr, bool first) {
  if (first) {
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) tmem_ld_32x32b_x32_f(taddr + cc * 32, &acc[cc * 32]);
    tmem_ld_wait();
  } else {
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      uint32_t v0[16], v1[16];
      tmem_ld_32x32b_x16(taddr + cc * 32, v0);
      tmem_ld_32x32b_x16(taddr + cc * 32 + 16, v1);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        acc[cc * 32 + i] += __uint_as_float(v0[i]);
        acc[cc * 32 + 16 + i] += __uint_as_float(v1[i]);
      }
    }
  }
}
__device__ __forceinline__ void fold_correction_narrow(float (&acc)[128], uint32_t taddr, float scale) {
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    uint32_t v0[16], v1[16];
    tmem_ld_32x32b_x16(taddr + cc * 32, v0);
    tmem_ld_32x32b_x16(taddr + cc * 32 + 16, v1);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      acc[cc * 32 + i] = acc[cc * 32 + i] + __uint_as_float(v0[i]) * scale;
      acc[cc * 32 + 16 + i] = acc[cc * 32 + 16 + i] + __uint_as_float(v1[i]) * scale;
    }
  }
}

// Epilogue thread: out = main + corr * scale (tcec.hpp:332-336; scale = 2^-11 for fp16, 1 for tf32).
__device__ __forceinline__ void fold_correction(float (&acc)[128], uint32_t taddr, float scale) {
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + cc * 32, v);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[cc * 32 + i] = acc[cc * 32 + i] + __uint_as_float(v[i]) * scale;
  }
}

}  // namespace tcec_sm100
