// Host side of the C ABI declared in include/tcec.h: argument checks, the
// library-owned workspace, kernel selection and launches.  No CPU compute path
// exists here: every entry point either launches sm_100a kernels or fails.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

#include "tcec_gemm_fused.cuh"
#include "tcec_gemm_panels.cuh"
#include "tcec_gemm_panels_pair.cuh"
#include "tcec_internal.h"
#include "tcec_panels.cuh"

using namespace tcec_sm100;

namespace tcec_host {

namespace {
std::mutex g_mu;
std::map<int, DeviceState> g_dev;
Options g_opt;
}  // namespace

std::mutex& state_mutex() { return g_mu; }
Options snapshot_options() {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_opt;
}

template <int BN, bool T, bool E>
cudaError_t set_smem_attr() {
  return cudaFuncSetAttribute(tcec_gemm_panels_kernel<BN, T, E>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              GemmPanelCfg<BN, T, E>::SMEM_BYTES);
}

template <bool T, bool E>
cudaError_t set_pair_smem_attr() {
  cudaError_t e = cudaFuncSetAttribute(tcec_gemm_panels_pair_kernel<T, E, 256>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, GemmPairCfg<T, E>::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(tcec_gemm_panels_pair_kernel<T, E, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              GemmPairCfg<T, E>::SMEM_BYTES);
}

int get_device_state(DeviceState** out) {
  int dev = 0;
  TCEC_CUDA(cudaGetDevice(&dev));
  DeviceState& st = g_dev[dev];
  if (!st.attrs_done) {
    int major = 0;
    TCEC_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return TCEC_ERR_UNSUPPORTED;  // sm_100a only
    TCEC_CUDA(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
    TCEC_CUDA((set_smem_attr<128, false, false>()));
    TCEC_CUDA((set_smem_attr<128, false, true>()));
    TCEC_CUDA((set_smem_attr<128, true, false>()));
    TCEC_CUDA((set_smem_attr<128, true, true>()));
    TCEC_CUDA((set_smem_attr<256, false, false>()));
    TCEC_CUDA((set_smem_attr<256, false, true>()));
    TCEC_CUDA((set_smem_attr<256, true, false>()));
    TCEC_CUDA((set_smem_attr<256, true, true>()));
    TCEC_CUDA(cudaFuncSetAttribute(tcec_gemm_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   GemmFusedCfg<true>::SMEM_BYTES));
    TCEC_CUDA(cudaFuncSetAttribute(tcec_gemm_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   GemmFusedCfg<false>::SMEM_BYTES));
    TCEC_CUDA((set_pair_smem_attr<false, true>()));
    TCEC_CUDA((set_pair_smem_attr<false, false>()));
    TCEC_CUDA((set_pair_smem_attr<true, true>()));
    TCEC_CUDA((set_pair_smem_attr<true, false>()));
    if (cudaMalloc(&st.status, sizeof(int)) != cudaSuccess) return TCEC_ERR_ALLOC;
    TCEC_CUDA(cudaMemset(st.status, 0, sizeof(int)));
    st.attrs_done = true;
  }
  *out = &st;
  return TCEC_OK;
}

// A workspace that must grow is replaced; the old buffer is handed back in *to_free so that the
// caller can wait for the stream and free it after it has released the state mutex.
int get_workspace(DeviceState* st, cudaStream_t stream, size_t bytes, void** out, void** to_free) {
  Workspace& w = st->ws[stream];
  *to_free = nullptr;
  if (w.bytes < bytes) {
    *to_free = w.ptr;
    w.ptr = nullptr;
    w.bytes = 0;
    if (cudaMalloc(&w.ptr, bytes) != cudaSuccess) {
      w.ptr = nullptr;
      return TCEC_ERR_ALLOC;
    }
    w.bytes = bytes;
  }
  *out = w.ptr;
  return TCEC_OK;
}
// Work queued on the stream may still read a replaced workspace: wait for it, then free.
static int release_old_workspace(void* old, cudaStream_t stream) {
  if (!old) return TCEC_OK;
  const cudaError_t e = cudaStreamSynchronize(stream);
  cudaFree(old);
  return e == cudaSuccess ? TCEC_OK : TCEC_ERR_CUDA;
}

// Launches on one stream are ordered, so they can share one pair of counters (each launch leaves
// them at zero); launches on different streams may overlap and get their own.
int get_sched(DeviceState* st, cudaStream_t stream, unsigned int** out) {
  if (st->sched_fixed) {
    *out = st->sched_fixed;
    return TCEC_OK;
  }
  unsigned int*& p = st->sched[stream];
  if (!p) {
    if (cudaMalloc(&p, 2 * sizeof(unsigned int)) != cudaSuccess) {
      p = nullptr;
      return TCEC_ERR_ALLOC;
    }
    TCEC_CUDA(cudaMemset(p, 0, 2 * sizeof(unsigned int)));
  }
  *out = p;
  return TCEC_OK;
}

bool policy_tf32(int policy) { return policy == TCEC_POLICY_TF32_EC || policy == TCEC_POLICY_TF32_NO_EC; }
bool policy_ec(int policy) { return policy == TCEC_POLICY_FP16_EC || policy == TCEC_POLICY_TF32_EC; }
int padded_row_blocks(int rows) { return ((rows + 255) / 256) * 2; }
size_t packed_bytes(int rows, int k, int policy) {
  const int kop = policy_tf32(policy) ? 16 : 32;
  const size_t nkb = (k + kop - 1) / kop;
  return static_cast<size_t>(padded_row_blocks(rows)) * nkb * (policy_ec(policy) ? 2 : 1) * kPanelBytes;
}
// K extent the tensor-core accumulator may gather before the round-to-nearest add, in k blocks.
// The accumulator truncates, so a longer interval trades accuracy for fewer drains.  Automatic
// choice with error correction: every 64 of K up to K = 2048, 128 up to 4096, 256 below 16384,
// else 512.  Each step is the longest that keeps both acceptance bounds on all-positive inputs,
// where the truncation bias is largest (error vs FP64 at most twice the reference kernel's and
// at most twice an FP32 SGEMM's on identical inputs): at K = 4096 an interval of 256 is 6 %
// faster and still 1.33 x the reference kernel's error, but 2.7 x cuBLAS FP32's.  The policies
// without error correction keep the reference's default for them, accumulation inside the tensor
// core (mma_rz_sync, include/wmma_extension/tcec/detail/no_cor.hpp:858-897).
int promote_blocks(int k, int policy, int kop, const Options& opt) {
  int pk = opt.promote_k;
  if (pk < 0) pk = !policy_ec(policy) ? 0 : (k <= 2048 ? 64 : (k <= 4096 ? 128 : (k < 16384 ? 256 : 512)));
  return pk > 0 ? (pk + kop - 1) / kop : 0;
}
Shape plan(int m, int n, int k, int policy, const Options& opt) {
  Shape s;
  s.kop = policy_tf32(policy) ? 16 : 32;
  s.np = policy_ec(policy) ? 2 : 1;
  s.tile_n = opt.tile_n ? opt.tile_n : (n > 128 ? 256 : 128);
  s.tiles_m = (m + 127) / 128;
  s.tiles_n = (n + s.tile_n - 1) / s.tile_n;
  s.nkb = (k + s.kop - 1) / s.kop;
  s.a_row_blocks = padded_row_blocks(m);
  s.b_row_blocks = padded_row_blocks(n);
  s.a_bytes = packed_bytes(m, k, policy);
  s.b_bytes = packed_bytes(n, k, policy);
  return s;
}

__global__ void scale_c_kernel(float* c, float* const* c_array, long long ldc, long long stride,
                               int rows, int cols, int col_major, float beta) {
  float* base = c_array ? c_array[blockIdx.z] : c + blockIdx.z * stride;
  const int inner = col_major ? rows : cols, outer = col_major ? cols : rows;
  for (int o = blockIdx.y; o < outer; o += gridDim.y)
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inner; i += gridDim.x * blockDim.x) {
      float* p = base + static_cast<long long>(o) * ldc + i;
      *p = (beta == 0.f) ? 0.f : beta * *p;
    }
}

template <bool T>
__global__ void split_flat_kernel(const float* __restrict__ in, float* hi, float* lo, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float v = in[i];
    float h, l;
    if constexpr (T) {
      h = tf32_rna(v);
      l = tf32_rna(v - h);
    } else {
      const __half hh = __float2half_rn(v);
      h = __half2float(hh);
      l = __half2float(__float2half_rn((v - h) * 2048.0f));
    }
    hi[i] = h;
    if (lo) lo[i] = l;
  }
}

template <bool T, bool E>
void launch_split(const SplitParams& sp, int batch, cudaStream_t stream) {
  // the batch index is the grid's z dimension (at most 65535): larger batches go in several launches
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    SplitParams part = sp;
    const int nb = batch - b0 < 65535 ? batch - b0 : 65535;
    if (part.src_array) part.src_array += b0;
    else part.src += static_cast<long long>(b0) * part.batch_stride;
    part.panels += static_cast<long long>(b0) * part.panels_batch_stride;
    dim3 grid(part.nkb, part.row_blocks, nb);
    tcec_split_panels_kernel<T, E><<<grid, 256, 0, stream>>>(part);
  }
}

template <int BN, bool T, bool E>
void launch_gemm(const GemmPanelParams& gp, int grid, cudaStream_t stream) {
  using Cfg = GemmPanelCfg<BN, T, E>;
  tcec_gemm_panels_kernel<BN, T, E>
      <<<grid, Cfg::THREADS, gp.store_turn ? Cfg::SMEM_BYTES : Cfg::SMEM_BYTES_NO_TURN, stream>>>(gp);
}

bool bad_layout(int l) { return l != TCEC_ROW_MAJOR && l != TCEC_COL_MAJOR; }

static SplitParams split_params(bool k_contiguous, int rows, int k, const float* src, const float* const* src_array,
                                long long ld, long long stride, uint8_t* panels, size_t panels_stride, int policy,
                                const PackPart& part) {
  const int kop = policy_tf32(policy) ? 16 : 32;
  SplitParams sp{};
  sp.src = src;
  sp.src_array = src_array;
  sp.ld = ld;
  sp.batch_stride = stride;
  sp.rows = rows;
  sp.k = k;
  sp.k_contiguous = k_contiguous ? 1 : 0;
  sp.row_blocks = padded_row_blocks(rows);
  sp.nkb = (k + kop - 1) / kop;
  sp.panels = panels;
  sp.panels_batch_stride = static_cast<long long>(panels_stride);
  sp.mul = part.mul;
  sp.elem_stride = part.elem_stride;
  sp.kb_offset = part.kb_offset;
  sp.nkb_out = part.nkb_out;
  return sp;
}

void pack_operand(bool k_contiguous, int rows, int k, const float* src, const float* const* src_array,
                  long long ld, long long stride, int batch, uint8_t* panels, size_t panels_stride,
                  int policy, cudaStream_t stream, const PackPart& part) {
  const SplitParams sp = split_params(k_contiguous, rows, k, src, src_array, ld, stride, panels, panels_stride, policy,
                                      part);
  if (policy_tf32(policy)) {
    if (policy_ec(policy)) launch_split<true, true>(sp, batch, stream);
    else launch_split<true, false>(sp, batch, stream);
  } else {
    if (policy_ec(policy)) launch_split<false, true>(sp, batch, stream);
    else launch_split<false, false>(sp, batch, stream);
  }
}

// A (rows = m) and B (rows = n) of one product, in one launch where the grid allows it.
void pack_both(bool a_k_contiguous, int m, const float* a, const float* const* a_array, long long lda, long long stride_a,
               uint8_t* panels_a, size_t a_stride, bool b_k_contiguous, int n, const float* b, const float* const* b_array,
               long long ldb, long long stride_b, uint8_t* panels_b, size_t b_stride, int k, int batch, int policy,
               cudaStream_t stream) {
  const PackPart plain;
  const SplitParams pa = split_params(a_k_contiguous, m, k, a, a_array, lda, stride_a, panels_a, a_stride, policy, plain);
  const SplitParams pb = split_params(b_k_contiguous, n, k, b, b_array, ldb, stride_b, panels_b, b_stride, policy, plain);
  const unsigned long long na = static_cast<unsigned long long>(pa.nkb) * pa.row_blocks * batch;
  const unsigned long long nb = static_cast<unsigned long long>(pb.nkb) * pb.row_blocks * batch;
  if (na + nb > 0x7fffffffull) {  // beyond one grid: one launch (or several) per operand
    pack_operand(a_k_contiguous, m, k, a, a_array, lda, stride_a, batch, panels_a, a_stride, policy, stream);
    pack_operand(b_k_contiguous, n, k, b, b_array, ldb, stride_b, batch, panels_b, b_stride, policy, stream);
    return;
  }
  const unsigned int grid = static_cast<unsigned int>(na + nb), first_b = static_cast<unsigned int>(na);
  if (policy_tf32(policy)) {
    if (policy_ec(policy)) tcec_split_both_kernel<true, true><<<grid, 256, 0, stream>>>(pa, pb, first_b);
    else tcec_split_both_kernel<true, false><<<grid, 256, 0, stream>>>(pa, pb, first_b);
  } else {
    if (policy_ec(policy)) tcec_split_both_kernel<false, true><<<grid, 256, 0, stream>>>(pa, pb, first_b);
    else tcec_split_both_kernel<false, false><<<grid, 256, 0, stream>>>(pa, pb, first_b);
  }
}

int gemm_packed(const Shape& s, int m, int n, int k, float alpha, const uint8_t* panels_a, size_t a_stride,
                const uint8_t* panels_b, size_t b_stride, float beta, float* c, float* const* c_array, long long ldc,
                long long stride_c, int lc, int batch, int policy, DeviceState* st, cudaStream_t stream,
                const Options& opt, const LaunchExtras* extras) {
  const LaunchExtras none;
  const LaunchExtras& ex = extras ? *extras : none;
  GemmPanelParams gp{};
  gp.M = m;
  gp.N = n;
  gp.K = k;
  gp.batch = batch;
  gp.nkb = s.nkb;
  gp.tiles_m = s.tiles_m;
  gp.tiles_n = s.tiles_n;
  gp.promo = promote_blocks(k, policy, s.kop, opt);
  gp.alpha = alpha;
  gp.beta = beta;
  gp.panels_a = panels_a;
  gp.panels_b = panels_b;
  gp.panels_a_batch_stride = static_cast<long long>(a_stride);
  gp.panels_b_batch_stride = static_cast<long long>(b_stride);
  gp.c = c;
  gp.c_array = c_array;
  gp.ldc = ldc;
  gp.c_batch_stride = stride_c;
  gp.c_col_major = (lc == TCEC_COL_MAJOR);
  gp.status = st->status;
  gp.debug_flags = opt.debug_flags;
  gp.store_turn = opt.store_turn;
  gp.trace = opt.trace;
  gp.row_ready = ex.row_ready;
  gp.ready_rows = ex.ready_rows;
  gp.ready_epoch = ex.ready_epoch;
  const int reserve = ex.reserve_sms >= 0 ? ex.reserve_sms : opt.reserve_sms;
  const int sms = st->sm_count - reserve > 1 ? st->sm_count - reserve : 1;
  const bool tf32 = policy_tf32(policy), ec = policy_ec(policy);
  // One product per K block makes the kernel wait on operands from L2, which a CTA pair halves
  // for B: measured 10-15 % faster there.  With three products the pair is faster only while the
  // clocks are high, i.e. for calls too short to reach the board's power cap (2048^3: +8 %,
  // 4096^3: +2 %; 16384^3 back to back: -5 %), so the automatic choice takes it below ~5000^3.
  const double flops = 2.0 * m * static_cast<double>(n) * k * batch;
  const bool want_pair = !ex.force_one_sm && !ex.row_ready && !ex.sched &&
                         (opt.cta_pair == 1 || (opt.cta_pair == -1 && (!ec || flops <= 2.5e11)));
  if (want_pair && s.tile_n == 256 && m > 128) {
    // CTA pairs: 256 x 256 tiles, grid of up to sms/2 clusters of two CTAs
    gp.tiles_m = (m + 255) / 256;
    const long long npair_tiles = static_cast<long long>(gp.tiles_m) * gp.tiles_n * batch;
    if (npair_tiles > 0x3fffffffll) return TCEC_ERR_UNSUPPORTED;  // work items are 32-bit
    const int max_pairs = sms / 2 > 1 ? sms / 2 : 1;
    // A call with so few tiles that they leave at least half of the pairs idle runs in half-width
    // tiles: twice as many work items, each ~0.6 as long (1024^3: 16 tiles become 32 halves,
    // 37 -> 27 us).  Halving only the tiles of an underfilled last wave of a larger call does not
    // pay: an N = 128 MMA takes nearly as long as an N = 256 one (measured at 4096^3 and 5120^3:
    // 1-2 % slower), so such calls stay on whole tiles.
    const int halved = (opt.half_tiles && 2 * npair_tiles <= max_pairs) ? static_cast<int>(npair_tiles) : 0;
    const int whole = static_cast<int>(npair_tiles) - halved;
#define TCEC_PAIR(T, E)                                                                                          \
  do {                                                                                                           \
    if (whole > 0) {                                                                                             \
      gp.tile_first = 0;                                                                                         \
      gp.tile_count = whole;                                                                                     \
      const int grid = 2 * (whole < max_pairs ? whole : max_pairs);                                              \
      tcec_gemm_panels_pair_kernel<T, E, 256><<<grid, 384, GemmPairCfg<T, E>::SMEM_BYTES, stream>>>(gp);         \
    }                                                                                                            \
    if (halved > 0) {                                                                                            \
      gp.tile_first = whole;                                                                                     \
      gp.tile_count = halved;                                                                                    \
      tcec_gemm_panels_pair_kernel<T, E, 128><<<4 * halved, 384, GemmPairCfg<T, E>::SMEM_BYTES, stream>>>(gp);   \
    }                                                                                                            \
  } while (0)
    if (tf32 && ec)
      TCEC_PAIR(true, true);
    else if (tf32)
      TCEC_PAIR(true, false);
    else if (ec)
      TCEC_PAIR(false, true);
    else
      TCEC_PAIR(false, false);
#undef TCEC_PAIR
    return TCEC_OK;
  }
  const long long ntiles = static_cast<long long>(gp.tiles_m) * gp.tiles_n * batch;
  if (ntiles > 0x7fffffffll) return TCEC_ERR_UNSUPPORTED;  // tile indices are 32-bit
  int grid = static_cast<int>(ntiles < sms ? ntiles : sms);
  if (ex.sched) {
    // counters shared with other launches of the same problem; the caller zeroes them
    gp.sched = ex.sched;
    gp.sched_keep = 1;
    gp.sched_base = ex.sched_base;
    gp.sched_all_dynamic = ex.all_from_counter;
    if (ex.grid > 0) grid = ex.grid;
  } else {
    if (!opt.static_tiles) {
      const int rc = get_sched(st, stream, &gp.sched);
      if (rc != TCEC_OK) return rc;
    }
    gp.sched_base = grid;
  }
#define TCEC_DISPATCH(T, E)                         \
  do {                                              \
    if (s.tile_n == 256)                            \
      launch_gemm<256, T, E>(gp, grid, stream);     \
    else                                            \
      launch_gemm<128, T, E>(gp, grid, stream);     \
  } while (0)
  if (tf32 && ec)
    TCEC_DISPATCH(true, true);
  else if (tf32)
    TCEC_DISPATCH(true, false);
  else if (ec)
    TCEC_DISPATCH(false, true);
  else
    TCEC_DISPATCH(false, false);
#undef TCEC_DISPATCH
  return TCEC_OK;
}

// ---------------------------------------------------------------- FP32-tile (fused) path
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// Tensor map of one FP32 operand: `rows` along M (or N), `k` along K.  K-contiguous: element
// (row, kk) at row*ld + kk, box 32 k x box_rows rows.  Otherwise (kk, row) at kk*ld + row, box
// 32 rows x 32 k.  128-byte swizzle; out-of-range elements read as zero.
bool encode_operand_map(CUtensorMap* map, const float* base, bool k_contiguous, int rows, int k, long long ld,
                        long long batch_stride, int batch, int box_rows) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
      return false;
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const cuuint64_t inner = k_contiguous ? k : rows, outer = k_contiguous ? rows : k;
  cuuint64_t dims[3] = {inner, outer, static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 4,
                           static_cast<cuuint64_t>(batch > 1 ? batch_stride : ld * static_cast<long long>(outer)) * 4};
  cuuint32_t box[3] = {32u, static_cast<cuuint32_t>(k_contiguous ? box_rows : 32), 1u};
  cuuint32_t elem[3] = {1, 1, 1};
  return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor map of a row-major C for tensor stores: 32 x 32 boxes, 128-byte swizzle (the layout the
// epilogue writes its store boxes in).  Elements of a box outside the matrix are not written.
bool encode_c_map(CUtensorMap* map, float* base, int m, int n, long long ldc, long long batch_stride, int batch) {
  if (!g_encode) return false;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ldc) * 4,
                           static_cast<cuuint64_t>(batch > 1 ? batch_stride : ldc * static_cast<long long>(m)) * 4};
  cuuint32_t box[3] = {32u, 32u, 1u};
  cuuint32_t elem[3] = {1, 1, 1};
  return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tma_addressable(const float* base, long long ld, long long stride, int batch) {
  return (reinterpret_cast<uintptr_t>(base) & 15) == 0 && ld % 4 == 0 && (batch <= 1 || stride % 4 == 0) &&
         ld < (1ll << 36) && stride < (1ll << 36);
}

// Launches the FP32-tile kernel if the call qualifies; returns false (nothing launched) otherwise.
bool try_fused(int la, int lb, int lc, int m, int n, int k, float alpha, const float* a, long long lda,
               long long stride_a, const float* b, long long ldb, long long stride_b, float beta, float* c,
               long long ldc, long long stride_c, int batch, int policy, const DeviceState* st,
               cudaStream_t stream, const Options& opt) {
  if (policy_tf32(policy) || !a || !b || !c || n <= 128) return false;
  // Worth it only where the GEMM is bound by DRAM traffic, which the split pass doubles: short K.
  const bool wanted = opt.path == 2 || (opt.path == 0 && batch > 1 && k <= 512);
  if (!wanted) return false;
  if (!tma_addressable(a, lda, stride_a, batch) || !tma_addressable(b, ldb, stride_b, batch)) return false;
  const bool a_kc = (la == TCEC_ROW_MAJOR), b_kc = (lb == TCEC_COL_MAJOR);
  CUtensorMap map_a, map_b, map_c;
  if (!encode_operand_map(&map_a, a, a_kc, m, k, lda, stride_a, batch, 128)) return false;
  if (!encode_operand_map(&map_b, b, b_kc, n, k, ldb, stride_b, batch, 128)) return false;
  // C goes out through tensor stores when nothing has to be read back and its rows are addressable.
  const bool c_tma = lc == TCEC_ROW_MAJOR && beta == 0.f && tma_addressable(c, ldc, stride_c, batch) &&
                     encode_c_map(&map_c, c, m, n, ldc, stride_c, batch);
  if (!c_tma) map_c = map_a;  // unused by the kernel
  GemmFusedParams fp{};
  fp.c_tma = c_tma ? 1 : 0;
  fp.M = m;
  fp.N = n;
  fp.K = k;
  fp.batch = batch;
  fp.nkb = (k + 31) / 32;
  fp.tiles_m = (m + 255) / 256;  // 256 x 256 tiles on CTA pairs
  fp.tiles_n = (n + 255) / 256;
  fp.promo = promote_blocks(k, policy, 32, opt);
  fp.a_k_contiguous = a_kc;
  fp.b_k_contiguous = b_kc;
  fp.alpha = alpha;
  fp.beta = beta;
  fp.c = c;
  fp.ldc = ldc;
  fp.c_batch_stride = stride_c;
  fp.c_col_major = (lc == TCEC_COL_MAJOR);
  fp.status = st->status;
  fp.debug_flags = opt.debug_flags;
  fp.trace = opt.trace;
  const long long ntiles = static_cast<long long>(fp.tiles_m) * fp.tiles_n * batch;
  const int sms = st->sm_count - opt.reserve_sms > 2 ? st->sm_count - opt.reserve_sms : 2;
  const int max_pairs = sms / 2;
  const int grid = 2 * static_cast<int>(ntiles < max_pairs ? ntiles : max_pairs);
  if (policy_ec(policy))
    tcec_gemm_fused_kernel<true><<<grid, GemmFusedCfg<true>::THREADS, GemmFusedCfg<true>::SMEM_BYTES, stream>>>(fp, map_a, map_b, map_c);
  else
    tcec_gemm_fused_kernel<false><<<grid, GemmFusedCfg<false>::THREADS, GemmFusedCfg<false>::SMEM_BYTES, stream>>>(fp, map_a, map_b, map_c);
  return true;
}

int scale_only(float beta, float* c, float* const* c_array, long long ldc, long long stride_c, int m,
               int n, int lc, int batch, cudaStream_t stream) {
  if (beta == 1.f) return TCEC_OK;
  const int inner = lc == TCEC_COL_MAJOR ? m : n, outer = lc == TCEC_COL_MAJOR ? n : m;
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = batch - b0 < 65535 ? batch - b0 : 65535;
    dim3 grid((inner + 255) / 256, outer < 65535 ? outer : 65535, nb);
    scale_c_kernel<<<grid, 256, 0, stream>>>(c_array ? nullptr : c + static_cast<long long>(b0) * stride_c,
                                             c_array ? c_array + b0 : nullptr, ldc, stride_c, m, n, lc == TCEC_COL_MAJOR,
                                             beta);
  }
  TCEC_CUDA(cudaGetLastError());
  return TCEC_OK;
}

int gemm_impl(int la, int lb, int lc, int m, int n, int k, float alpha, const float* a,
              const float* const* a_array, long long lda, long long stride_a, const float* b,
              const float* const* b_array, long long ldb, long long stride_b, float beta, float* c,
              float* const* c_array, long long ldc, long long stride_c, int batch, int policy,
              void* stream_v) {
  if (bad_layout(la) || bad_layout(lb) || bad_layout(lc)) return TCEC_ERR_INVALID_ARGUMENT;
  if (m < 0 || n < 0 || k < 0 || batch < 0) return TCEC_ERR_INVALID_ARGUMENT;
  if (policy < 0 || policy > 3) return TCEC_ERR_INVALID_ARGUMENT;
  if (m == 0 || n == 0 || batch == 0) return TCEC_OK;
  if (!c && !c_array) return TCEC_ERR_INVALID_ARGUMENT;
  if (ldc < (lc == TCEC_ROW_MAJOR ? n : m)) return TCEC_ERR_INVALID_ARGUMENT;
  if (k > 0) {
    if ((!a && !a_array) || (!b && !b_array)) return TCEC_ERR_INVALID_ARGUMENT;
    if (lda < (la == TCEC_ROW_MAJOR ? k : m)) return TCEC_ERR_INVALID_ARGUMENT;
    if (ldb < (lb == TCEC_ROW_MAJOR ? n : k)) return TCEC_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  // State is looked up (and a workspace grown) under the mutex; the launches run without it.
  Options opt;
  DeviceState* st = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    opt = g_opt;
    const int rc = get_device_state(&st);
    if (rc != TCEC_OK) return rc;
  }
  if (k == 0 || alpha == 0.f) return scale_only(beta, c, c_array, ldc, stride_c, m, n, lc, batch, stream);

  if (!a_array && !b_array && !c_array &&
      try_fused(la, lb, lc, m, n, k, alpha, a, lda, stride_a, b, ldb, stride_b, beta, c, ldc, stride_c, batch, policy,
                st, stream, opt)) {
    TCEC_CUDA(cudaGetLastError());
    return TCEC_OK;
  }
  const Shape s = plan(m, n, k, policy, opt);
  void* ws = nullptr;
  void* old = nullptr;
  int rc;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    rc = get_workspace(st, stream, (s.a_bytes + s.b_bytes) * batch, &ws, &old);
  }
  const int rel = release_old_workspace(old, stream);
  if (rc != TCEC_OK) return rc;
  if (rel != TCEC_OK) return rel;
  uint8_t* panels_a = static_cast<uint8_t*>(ws);
  uint8_t* panels_b = panels_a + s.a_bytes * batch;
  pack_both(la == TCEC_ROW_MAJOR, m, a, a_array, lda, stride_a, panels_a, s.a_bytes, lb == TCEC_COL_MAJOR, n, b, b_array,
            ldb, stride_b, panels_b, s.b_bytes, k, batch, policy, stream);
  {
    std::lock_guard<std::mutex> lock(g_mu);  // the per-stream tile counters may be created here
    rc = gemm_packed(s, m, n, k, alpha, panels_a, s.a_bytes, panels_b, s.b_bytes, beta, c, c_array, ldc, stride_c,
                     lc, batch, policy, st, stream, opt);
  }
  if (rc != TCEC_OK) return rc;
  TCEC_CUDA(cudaGetLastError());
  return TCEC_OK;
}

// ---------------------------------------------------------------- complex GEMM (four real products)
// C = alpha * (Pr + i Pi) + beta * C on interleaved complex C; Pr, Pi are dense planar products.
__global__ void cgemm_combine_kernel(const float* __restrict__ pr, const float* __restrict__ pi, float2* c,
                                     long long ldc, int inner, int outer, float2 alpha, float2 beta,
                                     int has_product) {
  for (int o = blockIdx.y; o < outer; o += gridDim.y)
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inner; i += gridDim.x * blockDim.x) {
      float2* dst = c + static_cast<long long>(o) * ldc + i;
      float2 out = make_float2(0.f, 0.f);
      if (has_product) {
        const long long q = static_cast<long long>(o) * inner + i;
        const float xr = pr[q], xi = pi[q];
        out.x = alpha.x * xr - alpha.y * xi;
        out.y = alpha.x * xi + alpha.y * xr;
      }
      if (beta.x != 0.f || beta.y != 0.f) {
        const float2 old = *dst;
        out.x += beta.x * old.x - beta.y * old.y;
        out.y += beta.x * old.y + beta.y * old.x;
      }
      *dst = out;
    }
}

// The reference builds a complex product from four real TCEC products
// (include/wmma_extension/tcec/complex.hpp:646-727): real = Ar Br + Ai (-Bi), imag = Ai Br + Ar Bi.
// Here the two products of each part become ONE real GEMM over a K of twice the length:
// [Ar | Ai] x [Br ; -Bi] and [Ar | Ai] x [Bi ; Br].  A is split once into a concatenated panel
// set, B into two; both GEMMs run through the real kernel into planar scratch, and an
// elementwise pass applies the complex alpha and beta into the interleaved C.
int cgemm_impl(int la, int lb, int lc, int m, int n, int k, const float* alpha, const float* a, long long lda,
               const float* b, long long ldb, const float* beta, float* c, long long ldc, int policy,
               void* stream_v) {
  if (bad_layout(la) || bad_layout(lb) || bad_layout(lc) || m < 0 || n < 0 || k < 0 || policy < 0 ||
      policy > 3 || !alpha || !beta)
    return TCEC_ERR_INVALID_ARGUMENT;
  if (m == 0 || n == 0) return TCEC_OK;
  if (!c || ldc < (lc == TCEC_ROW_MAJOR ? n : m)) return TCEC_ERR_INVALID_ARGUMENT;
  const bool has_product = k > 0 && (alpha[0] != 0.f || alpha[1] != 0.f);
  if (has_product) {
    if (!a || !b) return TCEC_ERR_INVALID_ARGUMENT;
    if (lda < (la == TCEC_ROW_MAJOR ? k : m) || ldb < (lb == TCEC_ROW_MAJOR ? n : k))
      return TCEC_ERR_INVALID_ARGUMENT;
  }
  Options opt;
  DeviceState* st = nullptr;
  int rc;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    opt = g_opt;
    rc = get_device_state(&st);
    if (rc != TCEC_OK) return rc;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int inner = lc == TCEC_ROW_MAJOR ? n : m, outer = lc == TCEC_ROW_MAJOR ? m : n;
  const dim3 cgrid((inner + 255) / 256, outer < 32768 ? outer : 32768);
  const float2 al = make_float2(alpha[0], alpha[1]), be = make_float2(beta[0], beta[1]);
  if (!has_product) {
    cgemm_combine_kernel<<<cgrid, 256, 0, stream>>>(nullptr, nullptr, reinterpret_cast<float2*>(c), ldc, inner,
                                                    outer, al, be, 0);
    TCEC_CUDA(cudaGetLastError());
    return TCEC_OK;
  }
  const int kop = policy_tf32(policy) ? 16 : 32;
  const int nkb = (k + kop - 1) / kop;
  const long long k2_ll = 2ll * nkb * kop;
  if (k2_ll > 0x7fffffff) return TCEC_ERR_INVALID_ARGUMENT;
  const int k2 = static_cast<int>(k2_ll);
  const Shape s = plan(m, n, k2, policy, opt);
  const size_t plane = ((static_cast<size_t>(m) * n * sizeof(float)) + 255) & ~static_cast<size_t>(255);
  void* ws = nullptr;
  void* old = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    rc = get_workspace(st, stream, s.a_bytes + 2 * s.b_bytes + 2 * plane, &ws, &old);
  }
  const int rel = release_old_workspace(old, stream);
  if (rc != TCEC_OK) return rc;
  if (rel != TCEC_OK) return rel;
  uint8_t* pa = static_cast<uint8_t*>(ws);
  uint8_t* pbr = pa + s.a_bytes;
  uint8_t* pbi = pbr + s.b_bytes;
  float* prod_r = reinterpret_cast<float*>(pbi + s.b_bytes);
  float* prod_i = reinterpret_cast<float*>(pbi + s.b_bytes + plane);
  const bool a_kc = (la == TCEC_ROW_MAJOR), b_kc = (lb == TCEC_COL_MAJOR);
  PackPart first, second;
  first.elem_stride = second.elem_stride = 2;
  first.nkb_out = second.nkb_out = 2 * nkb;
  second.kb_offset = nkb;
  // A' = [Ar | Ai]
  pack_operand(a_kc, m, k, a, nullptr, 2 * lda, 0, 1, pa, 0, policy, stream, first);
  pack_operand(a_kc, m, k, a + 1, nullptr, 2 * lda, 0, 1, pa, 0, policy, stream, second);
  // B'r = [Br ; -Bi], B'i = [Bi ; Br]
  pack_operand(b_kc, n, k, b, nullptr, 2 * ldb, 0, 1, pbr, 0, policy, stream, first);
  PackPart neg = second;
  neg.mul = -1.0f;
  pack_operand(b_kc, n, k, b + 1, nullptr, 2 * ldb, 0, 1, pbr, 0, policy, stream, neg);
  pack_operand(b_kc, n, k, b + 1, nullptr, 2 * ldb, 0, 1, pbi, 0, policy, stream, first);
  pack_operand(b_kc, n, k, b, nullptr, 2 * ldb, 0, 1, pbi, 0, policy, stream, second);
  {
    std::lock_guard<std::mutex> lock(g_mu);
    rc = gemm_packed(s, m, n, k2, 1.0f, pa, 0, pbr, 0, 0.0f, prod_r, nullptr, inner, 0, lc, 1, policy, st, stream, opt);
    if (rc == TCEC_OK)
      rc = gemm_packed(s, m, n, k2, 1.0f, pa, 0, pbi, 0, 0.0f, prod_i, nullptr, inner, 0, lc, 1, policy, st, stream,
                       opt);
  }
  if (rc != TCEC_OK) return rc;
  cgemm_combine_kernel<<<cgrid, 256, 0, stream>>>(prod_r, prod_i, reinterpret_cast<float2*>(c), ldc, inner,
                                                  outer, al, be, 1);
  TCEC_CUDA(cudaGetLastError());
  return TCEC_OK;
}

}  // namespace tcec_host

using namespace tcec_host;

extern "C" {

int tcec_sgemm(int layout_a, int layout_b, int layout_c, int m, int n, int k, float alpha,
               const float* a, long long lda, const float* b, long long ldb, float beta, float* c,
               long long ldc, int policy, void* stream) {
  return gemm_impl(layout_a, layout_b, layout_c, m, n, k, alpha, a, nullptr, lda, 0, b, nullptr,
                   ldb, 0, beta, c, nullptr, ldc, 0, 1, policy, stream);
}

int tcec_sgemm_batched(int layout_a, int layout_b, int layout_c, int m, int n, int k, float alpha,
                       const float* const* a_array, long long lda, const float* const* b_array,
                       long long ldb, float beta, float* const* c_array, long long ldc, int batch,
                       int policy, void* stream) {
  return gemm_impl(layout_a, layout_b, layout_c, m, n, k, alpha, nullptr, a_array, lda, 0, nullptr,
                   b_array, ldb, 0, beta, nullptr, c_array, ldc, 0, batch, policy, stream);
}

int tcec_sgemm_strided_batched(int layout_a, int layout_b, int layout_c, int m, int n, int k,
                               float alpha, const float* a, long long lda, long long stride_a,
                               const float* b, long long ldb, long long stride_b, float beta,
                               float* c, long long ldc, long long stride_c, int batch, int policy,
                               void* stream) {
  return gemm_impl(layout_a, layout_b, layout_c, m, n, k, alpha, a, nullptr, lda, stride_a, b,
                   nullptr, ldb, stride_b, beta, c, nullptr, ldc, stride_c, batch, policy, stream);
}

size_t tcec_packed_bytes(int rows, int k, int policy) {
  if (rows <= 0 || k <= 0 || policy < 0 || policy > 3) return 0;
  return packed_bytes(rows, k, policy);
}

size_t tcec_packed_row_offset(int row, int k, int policy) {
  // multiples of 256 only: the 256-wide tiles and the CTA-pair kernel read row blocks in pairs
  if (row < 0 || row % 256 != 0 || k <= 0 || policy < 0 || policy > 3) return 0;
  return packed_bytes(256, k, policy) * static_cast<size_t>(row / 256);
}

static int pack_entry(bool is_b, int layout, int rows, int k, const float* src, long long ld, void* packed,
                      int policy, void* stream) {
  if (bad_layout(layout) || rows < 0 || k < 0 || policy < 0 || policy > 3) return TCEC_ERR_INVALID_ARGUMENT;
  if (rows == 0 || k == 0) return TCEC_OK;
  if (!src || !packed) return TCEC_ERR_INVALID_ARGUMENT;
  // A is rows x k, B is k x rows
  const bool k_contig = is_b ? (layout == TCEC_COL_MAJOR) : (layout == TCEC_ROW_MAJOR);
  if (ld < (k_contig ? k : rows)) return TCEC_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(packed) & 15) != 0) return TCEC_ERR_INVALID_ARGUMENT;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* st = nullptr;
    const int rc = get_device_state(&st);
    if (rc != TCEC_OK) return rc;
  }
  pack_operand(k_contig, rows, k, src, nullptr, ld, 0, 1, static_cast<uint8_t*>(packed), 0, policy,
               static_cast<cudaStream_t>(stream));
  TCEC_CUDA(cudaGetLastError());
  return TCEC_OK;
}

int tcec_pack_a(int layout_a, int m, int k, const float* a, long long lda, void* packed, int policy,
                void* stream) {
  return pack_entry(false, layout_a, m, k, a, lda, packed, policy, stream);
}

int tcec_pack_b(int layout_b, int k, int n, const float* b, long long ldb, void* packed, int policy,
                void* stream) {
  return pack_entry(true, layout_b, n, k, b, ldb, packed, policy, stream);
}

int tcec_sgemm_packed(int layout_c, int m, int n, int k, float alpha, const void* a_packed,
                      const void* b_packed, float beta, float* c, long long ldc, int policy, void* stream) {
  if (bad_layout(layout_c) || m < 0 || n < 0 || k < 0 || policy < 0 || policy > 3)
    return TCEC_ERR_INVALID_ARGUMENT;
  if (m == 0 || n == 0) return TCEC_OK;
  if (!c || ldc < (layout_c == TCEC_ROW_MAJOR ? n : m)) return TCEC_ERR_INVALID_ARGUMENT;
  if (k > 0 && (!a_packed || !b_packed)) return TCEC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState* st = nullptr;
  const int rc = get_device_state(&st);
  if (rc != TCEC_OK) return rc;
  const Options opt = g_opt;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (k == 0 || alpha == 0.f) return scale_only(beta, c, nullptr, ldc, 0, m, n, layout_c, 1, s);
  const Shape sh = plan(m, n, k, policy, opt);
  const int grc = gemm_packed(sh, m, n, k, alpha, static_cast<const uint8_t*>(a_packed), 0,
                              static_cast<const uint8_t*>(b_packed), 0, beta, c, nullptr, ldc, 0, layout_c, 1,
                              policy, st, s, opt);
  if (grc != TCEC_OK) return grc;
  TCEC_CUDA(cudaGetLastError());
  return TCEC_OK;
}

// cuBLAS calling convention: column-major storage, transposition flags (0 = N, 1 = T, 2 = C),
// alpha and beta by host pointer.  op(A) is m x k: stored column-major m x k (N) or as its
// transpose k x m (T), which is a row-major m x k matrix with the same leading dimension.
static int cublas_layout(int trans, int* layout) {
  if (trans == 0) *layout = TCEC_COL_MAJOR;
  else if (trans == 1 || trans == 2) *layout = TCEC_ROW_MAJOR;
  else return TCEC_ERR_INVALID_ARGUMENT;
  return TCEC_OK;
}

int tcec_sgemm_cublas(int transa, int transb, int m, int n, int k, const float* alpha, const float* a, int lda,
                      const float* b, int ldb, const float* beta, float* c, int ldc, int policy, void* stream) {
  int la, lb;
  if (!alpha || !beta || cublas_layout(transa, &la) != TCEC_OK || cublas_layout(transb, &lb) != TCEC_OK)
    return TCEC_ERR_INVALID_ARGUMENT;
  return gemm_impl(la, lb, TCEC_COL_MAJOR, m, n, k, *alpha, a, nullptr, lda, 0, b, nullptr, ldb, 0, *beta, c,
                   nullptr, ldc, 0, 1, policy, stream);
}

int tcec_sgemm_batched_cublas(int transa, int transb, int m, int n, int k, const float* alpha,
                              const float* const* a_array, int lda, const float* const* b_array, int ldb,
                              const float* beta, float* const* c_array, int ldc, int batch, int policy,
                              void* stream) {
  int la, lb;
  if (!alpha || !beta || cublas_layout(transa, &la) != TCEC_OK || cublas_layout(transb, &lb) != TCEC_OK)
    return TCEC_ERR_INVALID_ARGUMENT;
  return gemm_impl(la, lb, TCEC_COL_MAJOR, m, n, k, *alpha, nullptr, a_array, lda, 0, nullptr, b_array, ldb, 0,
                   *beta, nullptr, c_array, ldc, 0, batch, policy, stream);
}

int tcec_cgemm(int layout_a, int layout_b, int layout_c, int m, int n, int k, const float* alpha, const float* a,
               long long lda, const float* b, long long ldb, const float* beta, float* c, long long ldc,
               int policy, void* stream) {
  return cgemm_impl(layout_a, layout_b, layout_c, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, policy, stream);
}

int tcec_split(const float* in, float* hi, float* lo, size_t count, int policy, void* stream) {
  if (policy < 0 || policy > 3) return TCEC_ERR_INVALID_ARGUMENT;
  if (count == 0) return TCEC_OK;
  if (!in || !hi) return TCEC_ERR_INVALID_ARGUMENT;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* st = nullptr;
    const int rc = get_device_state(&st);
    if (rc != TCEC_OK) return rc;
  }
  const bool tf32 = policy_tf32(policy);
  const size_t want = (count + 255) / 256;
  const int grid = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
  if (tf32)
    split_flat_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(in, hi, lo, count);
  else
    split_flat_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(in, hi, lo, count);
  TCEC_CUDA(cudaGetLastError());
  return TCEC_OK;
}

#ifdef TCEC_DEVELOP
// Develop builds only (not part of the declared ABI): device buffer of kTraceRoles * 4096 u64 for
// hand-off timestamps.
int tcec_debug_set_trace(unsigned long long* dev_buffer) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_opt.trace = dev_buffer;
  return TCEC_OK;
}
#endif

namespace {
struct OptionEntry {
  const char* name;
  int Options::*field;
  int lo, hi;
  bool (*ok)(int);
};
bool any_value(int) { return true; }
bool tile_value(int v) { return v == 0 || v == 128 || v == 256; }
bool panel_rows_value(int v) { return v % 256 == 0; }
const OptionEntry kOptions[] = {
    {"promote_k", &Options::promote_k, -1, 0x7fffffff, any_value},
    {"tile_n", &Options::tile_n, 0, 256, tile_value},
    {"cta_pair", &Options::cta_pair, -1, 1, any_value},
    {"half_tiles", &Options::half_tiles, 0, 1, any_value},
    {"path", &Options::path, 0, 2, any_value},
    {"store_turn", &Options::store_turn, 0, 1, any_value},
    {"reserve_sms", &Options::reserve_sms, 0, 64, any_value},
    {"static_tiles", &Options::static_tiles, 0, 1, any_value},
    {"comm_sms", &Options::comm_sms, 1, 64, any_value},
    {"comm_panel_rows", &Options::comm_panel_rows, 256, 1 << 20, panel_rows_value},
    {"comm_helper", &Options::comm_helper, 0, 1, any_value},
#ifdef TCEC_DEVELOP
    {"debug_flags", &Options::debug_flags, -0x7fffffff - 1, 0x7fffffff, any_value},
#endif
};
const OptionEntry* find_option(const char* name) {
  for (const OptionEntry& e : kOptions)
    if (!strcmp(name, e.name)) return &e;
  return nullptr;
}
}  // namespace

int tcec_set_option(const char* name, int value) {
  if (!name) return TCEC_ERR_INVALID_ARGUMENT;
  const OptionEntry* e = find_option(name);
  if (!e || value < e->lo || value > e->hi || !e->ok(value)) return TCEC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_mu);
  g_opt.*(e->field) = value;
  return TCEC_OK;
}

int tcec_get_option(const char* name, int* value) {
  if (!name || !value) return TCEC_ERR_INVALID_ARGUMENT;
  const OptionEntry* e = find_option(name);
  if (!e) return TCEC_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_mu);
  *value = g_opt.*(e->field);
  return TCEC_OK;
}

int tcec_device_status(int* detail) {
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState* st = nullptr;
  const int rc = get_device_state(&st);
  if (rc != TCEC_OK) return rc;
  TCEC_CUDA(cudaDeviceSynchronize());
  int word = 0;
  TCEC_CUDA(cudaMemcpy(&word, st->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (detail) *detail = word;
  if (word != 0) {
    TCEC_CUDA(cudaMemset(st->status, 0, sizeof(int)));
    return TCEC_ERR_TIMEOUT;
  }
  return TCEC_OK;
}

size_t tcec_workspace_bytes(int m, int n, int k, int batch, int policy) {
  if (m <= 0 || n <= 0 || k <= 0 || batch <= 0 || policy < 0 || policy > 3) return 0;
  const Shape s = plan(m, n, k, policy, snapshot_options());
  return (s.a_bytes + s.b_bytes) * batch;
}

int tcec_destroy(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  int cur = 0;
  cudaGetDevice(&cur);
  for (auto& kv : g_dev) {
    if (cudaSetDevice(kv.first) != cudaSuccess) continue;
    cudaDeviceSynchronize();
    for (auto& w : kv.second.ws)
      if (w.second.ptr) cudaFree(w.second.ptr);
    kv.second.ws.clear();
    for (auto& sc : kv.second.sched)
      if (sc.second) cudaFree(sc.second);
    kv.second.sched.clear();
    destroy_step_state(&kv.second);
    if (kv.second.status) cudaFree(kv.second.status);
    kv.second.status = nullptr;
    kv.second.attrs_done = false;
  }
  destroy_comm_state();
  g_dev.clear();
  cudaSetDevice(cur);
  return TCEC_OK;
}

// ---------------------------------------------------------------- allocation-free variant
//
// Some callers may not allocate device memory at the moment they need a GEMM: code running
// under a memory pool that owns the whole device, a real-time loop that must not take the
// allocator's locks, a plugin whose host forbids cudaMalloc after start-up.  For them the
// operand panels (the scratch the GEMM kernel streams from) live in a fixed array inside this
// library's device image instead of a workspace obtained with cudaMalloc, and so does the
// status word the kernels raise when a bounded wait runs out.  Every GPU that loads the
// library holds the array until the process exits.
//
// In host code the array's name is only a handle for the runtime, not a device address, so
// the address is looked up once per device with cudaGetSymbolAddress, with that device current.
static __device__ __align__(256) unsigned char g_static_panels[TCEC_STATIC_SCRATCH_BYTES];
static __device__ int g_static_status_word;
static __device__ unsigned int g_static_sched[2];  // the GEMM's tile-scheduler counters (zero between launches)

namespace {
constexpr int kMaxStaticDevices = 64;
struct StaticDevice {
  bool ready = false;
  uint8_t* panels = nullptr;
  int* status = nullptr;
  unsigned int* sched = nullptr;
  int sm_count = 0;
};
StaticDevice g_static_dev[kMaxStaticDevices];  // fixed table: nothing is allocated on the host either

int static_device_state(StaticDevice** out) {
  int dev = 0;
  TCEC_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxStaticDevices) return TCEC_ERR_UNSUPPORTED;
  StaticDevice& sd = g_static_dev[dev];
  if (!sd.ready) {
    int major = 0;
    TCEC_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return TCEC_ERR_UNSUPPORTED;
    TCEC_CUDA(cudaDeviceGetAttribute(&sd.sm_count, cudaDevAttrMultiProcessorCount, dev));
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_panels) != cudaSuccess || p == nullptr) return TCEC_ERR_CUDA;
    sd.panels = static_cast<uint8_t*>(p);
    p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_status_word) != cudaSuccess || p == nullptr) return TCEC_ERR_CUDA;
    sd.status = static_cast<int*>(p);
    p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_sched) != cudaSuccess || p == nullptr) return TCEC_ERR_CUDA;
    sd.sched = static_cast<unsigned int*>(p);
    // opting the kernels into their dynamic shared memory size changes a function attribute; it allocates nothing
    TCEC_CUDA((set_smem_attr<128, false, false>()));
    TCEC_CUDA((set_smem_attr<128, false, true>()));
    TCEC_CUDA((set_smem_attr<128, true, false>()));
    TCEC_CUDA((set_smem_attr<128, true, true>()));
    TCEC_CUDA((set_smem_attr<256, false, false>()));
    TCEC_CUDA((set_smem_attr<256, false, true>()));
    TCEC_CUDA((set_smem_attr<256, true, false>()));
    TCEC_CUDA((set_smem_attr<256, true, true>()));
    TCEC_CUDA((set_pair_smem_attr<false, false>()));
    TCEC_CUDA((set_pair_smem_attr<true, false>()));
    TCEC_CUDA((set_pair_smem_attr<false, true>()));
    TCEC_CUDA((set_pair_smem_attr<true, true>()));
    sd.ready = true;
  }
  *out = &sd;
  return TCEC_OK;
}
}  // namespace

size_t tcec_static_scratch_bytes(void) { return TCEC_STATIC_SCRATCH_BYTES; }

int tcec_sgemm_static(int layout_a, int layout_b, int layout_c, int m, int n, int k, float alpha,
                      const float* a, long long lda, const float* b, long long ldb, float beta, float* c,
                      long long ldc, int policy, void* stream_v) {
  if (bad_layout(layout_a) || bad_layout(layout_b) || bad_layout(layout_c)) return TCEC_ERR_INVALID_ARGUMENT;
  if (m < 0 || n < 0 || k < 0 || policy < 0 || policy > 3) return TCEC_ERR_INVALID_ARGUMENT;
  if (m == 0 || n == 0) return TCEC_OK;
  if (!c || ldc < (layout_c == TCEC_ROW_MAJOR ? n : m)) return TCEC_ERR_INVALID_ARGUMENT;
  if (k > 0) {
    if (!a || !b) return TCEC_ERR_INVALID_ARGUMENT;
    if (lda < (layout_a == TCEC_ROW_MAJOR ? k : m)) return TCEC_ERR_INVALID_ARGUMENT;
    if (ldb < (layout_b == TCEC_ROW_MAJOR ? n : k)) return TCEC_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  std::lock_guard<std::mutex> lock(g_mu);
  if (k == 0 || alpha == 0.f) {
    StaticDevice* sd0 = nullptr;
    const int rc0 = static_device_state(&sd0);
    if (rc0 != TCEC_OK) return rc0;
    return scale_only(beta, c, nullptr, ldc, 0, m, n, layout_c, 1, stream);
  }
  const Options opt = g_opt;
  const Shape s = plan(m, n, k, policy, opt);
  if (s.a_bytes + s.b_bytes > TCEC_STATIC_SCRATCH_BYTES) return TCEC_ERR_TOO_LARGE;
  StaticDevice* sd = nullptr;
  const int rc = static_device_state(&sd);
  if (rc != TCEC_OK) return rc;
  // Nothing in the array has to start at zero: the two split kernels below write every byte of
  // every panel the GEMM reads (rows and K beyond the matrix are written as zeros), and the
  // status word is only ever raised, never relied on to be clear by the kernels.
  uint8_t* panels_a = sd->panels;
  uint8_t* panels_b = sd->panels + s.a_bytes;  // a_bytes is a multiple of 8192
  pack_both(layout_a == TCEC_ROW_MAJOR, m, a, nullptr, lda, 0, panels_a, 0, layout_b == TCEC_COL_MAJOR, n, b, nullptr, ldb,
            0, panels_b, 0, k, 1, policy, stream);
  DeviceState view;  // launch parameters only; owns nothing
  view.status = sd->status;
  view.sm_count = sd->sm_count;
  view.sched_fixed = sd->sched;
  const int grc = gemm_packed(s, m, n, k, alpha, panels_a, 0, panels_b, 0, beta, c, nullptr, ldc, 0, layout_c, 1,
                              policy, &view, stream, opt);
  if (grc != TCEC_OK) return grc;
  TCEC_CUDA(cudaGetLastError());
  return TCEC_OK;
}

int tcec_static_status(int* detail) {
  std::lock_guard<std::mutex> lock(g_mu);
  StaticDevice* sd = nullptr;
  const int rc = static_device_state(&sd);
  if (rc != TCEC_OK) return rc;
  TCEC_CUDA(cudaDeviceSynchronize());
  int word = 0;
  TCEC_CUDA(cudaMemcpy(&word, sd->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (detail) *detail = word;
  if (word != 0) {
    const int zero = 0;
    TCEC_CUDA(cudaMemcpy(sd->status, &zero, sizeof(int), cudaMemcpyHostToDevice));
    return TCEC_ERR_TIMEOUT;
  }
  return TCEC_OK;
}

const char* tcec_status_string(int status) {
  switch (status) {
    case TCEC_OK: return "ok";
    case TCEC_ERR_INVALID_ARGUMENT: return "invalid argument";
    case TCEC_ERR_UNSUPPORTED: return "unsupported (needs an sm_100a device)";
    case TCEC_ERR_CUDA: return "CUDA runtime error";
    case TCEC_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case TCEC_ERR_ALLOC: return "workspace allocation failed";
    case TCEC_ERR_TOO_LARGE: return "operands exceed the fixed scratch of the allocation-free entry point";
    case TCEC_ERR_COMM: return "communication library (NCCL) missing, failed or not initialised";
    default: return "unknown status";
  }
}

const char* tcec_version(void) { return "tcec-b200 0.1 (sm_100a)"; }

}  // extern "C"
