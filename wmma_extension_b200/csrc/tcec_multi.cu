// Host side of the entry points that move operands: the pipelined host-operand GEMM
// (tcec_sgemm_host), the column-sharded GEMM over several GPUs with A broadcast by NCCL
// (tcec_sgemm_multi for one process driving all devices, tcec_sgemm_column_shard[_host] for one
// process per device) and the batch-sharded GEMM (tcec_sgemm_batched_multi, no collective).
//
// The reference is single-GPU and has no host API; the closest counterpart of all of these is
// the launch glue of its batched example (test/tcec/batch_gemm.cu:433-443).  K is never split,
// so no reduction exists anywhere: the only collective is the broadcast of A.
//
// NCCL is loaded at run time (dlopen), so a single-GPU user needs no NCCL at all.  Kernels of this
// library only ever read the GPU's own memory: A reaches it through ncclBroadcast first.
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "tcec_internal.h"

namespace tcec_host {

// ---------------------------------------------------------------- NCCL, loaded at run time
namespace {
struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
};
NcclApi g_nccl;
std::string g_nccl_path;  // empty: the environment variable TCEC_NCCL_LIBRARY, else "libnccl.so.2"

template <class F>
bool bind(void* lib, const char* name, F* out) {
  *out = reinterpret_cast<F>(dlsym(lib, name));
  return *out != nullptr;
}

// Needs the state mutex held.
int load_nccl() {
  if (g_nccl.lib) return TCEC_OK;
  const char* env = std::getenv("TCEC_NCCL_LIBRARY");
  const std::string path = !g_nccl_path.empty() ? g_nccl_path : (env && *env ? env : "libnccl.so.2");
  void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!lib) return TCEC_ERR_COMM;
  NcclApi api;
  api.lib = lib;
  if (!bind(lib, "ncclGetUniqueId", &api.GetUniqueId) || !bind(lib, "ncclCommInitRankConfig", &api.CommInitRankConfig) ||
      !bind(lib, "ncclCommDestroy", &api.CommDestroy) || !bind(lib, "ncclBroadcast", &api.Broadcast) ||
      !bind(lib, "ncclGroupStart", &api.GroupStart) || !bind(lib, "ncclGroupEnd", &api.GroupEnd)) {
    dlclose(lib);
    return TCEC_ERR_COMM;
  }
  g_nccl = api;
  return TCEC_OK;
}

#define TCEC_NCCL(call)                            \
  do {                                             \
    if ((call) != ncclSuccess) return TCEC_ERR_COMM; \
  } while (0)

// Communicators.  One per (process, device): created by tcec_comm_init_rank (one process per
// device) or, for a device list, by the first tcec_sgemm_multi that names it.
struct Comm {
  ncclComm_t comm = nullptr;
  int nranks = 0, rank = 0, device = -1, max_ctas = 0;
};
Comm g_rank_comm;                                // one process per device
std::vector<int> g_multi_devices;                // one process, many devices: the list the comms were made for
std::vector<Comm> g_multi_comms;

ncclConfig_t comm_config(int max_ctas) {
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  // The broadcast runs beside a GEMM that leaves it exactly this many SMs.
  cfg.minCTAs = 1;
  cfg.maxCTAs = max_ctas;
  return cfg;
}

void destroy_comm(Comm* c) {
  if (c->comm && g_nccl.CommDestroy) {
    int cur = 0;
    cudaGetDevice(&cur);
    if (c->device >= 0) cudaSetDevice(c->device);
    g_nccl.CommDestroy(c->comm);
    cudaSetDevice(cur);
  }
  *c = Comm();
}
}  // namespace

void destroy_comm_state() {
  destroy_comm(&g_rank_comm);
  for (Comm& c : g_multi_comms) destroy_comm(&c);
  g_multi_comms.clear();
  g_multi_devices.clear();
}

// ---------------------------------------------------------------- per-device step state
struct StepState {
  cudaStream_t s_in = nullptr, s_out = nullptr, s_comm = nullptr, s_help = nullptr;
  std::vector<cudaEvent_t> events;  // pool, handed out in order within one call
  size_t next_event = 0;
  Workspace packed_a, packed_b, stage;  // stage: FP32 staging of the host-operand pipeline
  unsigned int* words = nullptr;        // [0..1] tile counters, [2..] arrival flags
  unsigned int epoch = 0;
};
namespace {
constexpr int kMaxPanels = 8190;

int step_state(DeviceState* st, StepState** out) {
  if (!st->step) {
    StepState* s = new StepState();
    int lo = 0, hi = 0;
    TCEC_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    TCEC_CUDA(cudaStreamCreateWithFlags(&s->s_in, cudaStreamNonBlocking));
    TCEC_CUDA(cudaStreamCreateWithFlags(&s->s_out, cudaStreamNonBlocking));
    TCEC_CUDA(cudaStreamCreateWithPriority(&s->s_comm, cudaStreamNonBlocking, hi));
    TCEC_CUDA(cudaStreamCreateWithFlags(&s->s_help, cudaStreamNonBlocking));
    if (cudaMalloc(&s->words, (2 + kMaxPanels) * sizeof(unsigned int)) != cudaSuccess) return TCEC_ERR_ALLOC;
    TCEC_CUDA(cudaMemset(s->words, 0, (2 + kMaxPanels) * sizeof(unsigned int)));
    st->step = s;
  }
  st->step->next_event = 0;
  *out = st->step;
  return TCEC_OK;
}
int next_event(StepState* s, cudaEvent_t* out) {
  if (s->next_event == s->events.size()) {
    cudaEvent_t e;
    TCEC_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    s->events.push_back(e);
  }
  *out = s->events[s->next_event++];
  return TCEC_OK;
}
// Grow-only buffer owned by the step state.  Work of earlier calls that may still use the old
// buffer is ordered before this call on every stream involved, so a device synchronisation
// before freeing is enough (growth happens on the first call of a shape only).
int ensure(Workspace* w, size_t bytes) {
  if (w->bytes >= bytes) return TCEC_OK;
  if (w->ptr) {
    TCEC_CUDA(cudaDeviceSynchronize());
    cudaFree(w->ptr);
    w->ptr = nullptr;
    w->bytes = 0;
  }
  if (cudaMalloc(&w->ptr, bytes) != cudaSuccess) return TCEC_ERR_ALLOC;
  w->bytes = bytes;
  return TCEC_OK;
}

// b follows a on stream `b`: record on a, wait on b.
int order(StepState* s, cudaStream_t a, cudaStream_t b) {
  cudaEvent_t e;
  const int rc = next_event(s, &e);
  if (rc != TCEC_OK) return rc;
  TCEC_CUDA(cudaEventRecord(e, a));
  TCEC_CUDA(cudaStreamWaitEvent(b, e, 0));
  return TCEC_OK;
}

// Stream-ordered 32-bit write without a kernel (the GEMM may hold every SM it was given).
typedef CUresult (*WriteValueFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
WriteValueFn g_write_value = nullptr;
bool g_write_value_looked_up = false;
__global__ void set_word_kernel(unsigned int* p, unsigned int v) { *p = v; }
int stream_write(cudaStream_t s, unsigned int* dst, unsigned int value) {
  if (!g_write_value_looked_up) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &fn, cudaEnableDefault, &q) == cudaSuccess && fn)
      g_write_value = reinterpret_cast<WriteValueFn>(fn);
    g_write_value_looked_up = true;
  }
  if (g_write_value) {
    if (g_write_value(s, reinterpret_cast<CUdeviceptr>(dst), value, 0) == CUDA_SUCCESS) return TCEC_OK;
    g_write_value = nullptr;  // not supported here: fall back to a one-thread kernel
  }
  set_word_kernel<<<1, 1, 0, s>>>(dst, value);
  TCEC_CUDA(cudaGetLastError());
  return TCEC_OK;
}

struct Panel {
  int row0, rows;
  size_t offset, bytes;  // in the packed A
};
std::vector<Panel> make_panels(int m, int k, int policy, int panel_rows) {
  std::vector<Panel> v;
  const size_t per_pair = packed_bytes(256, k, policy);  // two 128-row blocks
  for (int r = 0; r < m; r += panel_rows) {
    Panel p;
    p.row0 = r;
    p.rows = m - r < panel_rows ? m - r : panel_rows;
    p.offset = per_pair * static_cast<size_t>(r / 256);
    p.bytes = packed_bytes(p.rows, k, policy);
    v.push_back(p);
  }
  return v;
}

int copy2d(void* dst, size_t dpitch, const void* src, size_t spitch, size_t width, size_t height, cudaMemcpyKind kind,
           cudaStream_t s) {
  if (width == 0 || height == 0) return TCEC_OK;
  if (dpitch == width && spitch == width)
    TCEC_CUDA(cudaMemcpyAsync(dst, src, width * height, kind, s));
  else
    TCEC_CUDA(cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, height, kind, s));
  return TCEC_OK;
}

// One device's part of a column-sharded GEMM.
struct Lane {
  int device = 0;
  int rank = 0;
  ncclComm_t comm = nullptr;
  cudaStream_t stream = nullptr;
  const float* a = nullptr;  // root only
  long long lda = 0;
  const float* b = nullptr;
  long long ldb = 0;
  float* c = nullptr;
  long long ldc = 0;
  int n_local = 0;
  DeviceState* st = nullptr;
  StepState* ss = nullptr;
};

// One packed row panel of A from the root's buffer into every other lane's, in place, on the
// communication streams.  One process driving several devices issues its ncclBroadcast calls
// inside one group (ncclGroupStart / ncclGroupEnd), which is closed on every path out.
int broadcast_panel(std::vector<Lane>& lanes, const Panel& pn, int root) {
  const bool group = lanes.size() > 1;
  if (group) TCEC_NCCL(g_nccl.GroupStart());
  int rc = TCEC_OK;
  for (Lane& ln : lanes) {
    if (cudaSetDevice(ln.device) != cudaSuccess) {
      rc = TCEC_ERR_CUDA;
      break;
    }
    uint8_t* buf = static_cast<uint8_t*>(ln.ss->packed_a.ptr) + pn.offset;
    if (g_nccl.Broadcast(buf, buf, pn.bytes, ncclUint8, root, ln.comm, ln.ss->s_comm) != ncclSuccess) {
      rc = TCEC_ERR_COMM;
      break;
    }
  }
  if (group && g_nccl.GroupEnd() != ncclSuccess && rc == TCEC_OK) rc = TCEC_ERR_COMM;
  return rc;
}

int check_shard_args(int la, int lb, int lc, int m, int k, int policy) {
  if (bad_layout(la) || bad_layout(lb) || bad_layout(lc) || m < 0 || k < 0 || policy < 0 || policy > 3)
    return TCEC_ERR_INVALID_ARGUMENT;
  return TCEC_OK;
}

// Device-resident operands: A on the root lane, every lane its column block of B and C.
// Per lane: B is split once; the root splits A in row panels and broadcasts each as soon as it
// is split; every other lane receives the panels into its packed-A buffer and raises one flag per
// panel; ONE persistent GEMM launch per lane covers all of M, its producers waiting (bounded) on
// the flag of a tile's rows.  The GEMM leaves `comm_sms` SMs to the broadcast, which is limited
// to as many CTAs, and once the broadcast is over a second launch of `comm_sms` CTAs that shares
// the first one's tile counter takes those SMs.
int column_step_device(std::vector<Lane>& lanes, int nranks, int root, int la, int lb, int lc, int m, int k,
                       float alpha, float beta, int policy, const Options& opt) {
  const std::vector<Panel> panels = make_panels(m, k, policy, opt.comm_panel_rows);
  if (panels.size() > static_cast<size_t>(kMaxPanels)) return TCEC_ERR_UNSUPPORTED;
  const size_t a_bytes = packed_bytes(m, k, policy);
  int cur = 0;
  TCEC_CUDA(cudaGetDevice(&cur));
  struct Restore {
    int dev;
    ~Restore() { cudaSetDevice(dev); }
  } restore{cur};

  // ---- buffers, B split, start of the communication stream
  for (Lane& ln : lanes) {
    TCEC_CUDA(cudaSetDevice(ln.device));
    int rc = ensure(&ln.ss->packed_a, a_bytes);
    if (rc != TCEC_OK) return rc;
    rc = ensure(&ln.ss->packed_b, ln.n_local > 0 ? packed_bytes(ln.n_local, k, policy) : 16);
    if (rc != TCEC_OK) return rc;
    ++ln.ss->epoch;
    // the previous call's broadcast and helper launch are over before this call touches the buffers
    rc = order(ln.ss, ln.stream, ln.ss->s_comm);
    if (rc != TCEC_OK) return rc;
    if (ln.n_local > 0)
      pack_operand(lb == TCEC_COL_MAJOR, ln.n_local, k, ln.b, nullptr, ln.ldb, 0, 1,
                   static_cast<uint8_t*>(ln.ss->packed_b.ptr), 0, policy, ln.stream);
  }
  // ---- root: split A panel by panel; every lane: broadcast panel by panel, flags behind it
  Lane* root_lane = nullptr;
  for (Lane& ln : lanes)
    if (ln.rank == root) root_lane = &ln;
  for (size_t p = 0; p < panels.size(); ++p) {
    const Panel& pn = panels[p];
    if (root_lane) {
      TCEC_CUDA(cudaSetDevice(root_lane->device));
      const float* src = la == TCEC_ROW_MAJOR ? root_lane->a + static_cast<long long>(pn.row0) * root_lane->lda
                                              : root_lane->a + pn.row0;
      pack_operand(la == TCEC_ROW_MAJOR, pn.rows, k, src, nullptr, root_lane->lda, 0, 1,
                   static_cast<uint8_t*>(root_lane->ss->packed_a.ptr) + pn.offset, 0, policy, root_lane->stream);
      if (nranks > 1) {
        const int rc = order(root_lane->ss, root_lane->stream, root_lane->ss->s_comm);
        if (rc != TCEC_OK) return rc;
      }
    }
    if (nranks > 1) {
      const int rc = broadcast_panel(lanes, pn, root);
      if (rc != TCEC_OK) return rc;
      for (Lane& ln : lanes) {
        if (ln.rank == root) continue;
        TCEC_CUDA(cudaSetDevice(ln.device));
        const int rc = stream_write(ln.ss->s_comm, ln.ss->words + 2 + p, ln.ss->epoch);
        if (rc != TCEC_OK) return rc;
      }
    }
  }
  // ---- one GEMM launch per lane (+ the helper launch that takes over the broadcast's SMs)
  for (Lane& ln : lanes) {
    TCEC_CUDA(cudaSetDevice(ln.device));
    cudaEvent_t bcast_done = nullptr;
    if (nranks > 1) {
      int rc = next_event(ln.ss, &bcast_done);
      if (rc != TCEC_OK) return rc;
      TCEC_CUDA(cudaEventRecord(bcast_done, ln.ss->s_comm));
    }
    if (ln.n_local > 0 && m > 0) {
      if (k == 0 || alpha == 0.f) {
        const int rc = scale_only(beta, ln.c, nullptr, ln.ldc, 0, m, ln.n_local, lc, 1, ln.stream);
        if (rc != TCEC_OK) return rc;
      } else {
        const Shape s = plan(m, ln.n_local, k, policy, opt);
        LaunchExtras ex;
        ex.force_one_sm = 1;
        if (nranks > 1) {
          TCEC_CUDA(cudaMemsetAsync(ln.ss->words, 0, 2 * sizeof(unsigned int), ln.stream));
          const long long ntiles = static_cast<long long>(s.tiles_m) * s.tiles_n;
          const int sms = ln.st->sm_count - opt.comm_sms > 1 ? ln.st->sm_count - opt.comm_sms : 1;
          ex.reserve_sms = opt.comm_sms;
          ex.sched = ln.ss->words;
          ex.sched_base = static_cast<int>(ntiles < sms ? ntiles : sms);
          if (ln.rank != root) {
            ex.row_ready = ln.ss->words + 2;
            ex.ready_rows = opt.comm_panel_rows;
            ex.ready_epoch = ln.ss->epoch;
          }
        }
        int rc;
        {
          std::lock_guard<std::mutex> lock(state_mutex());  // the per-stream tile counters may be created here
          rc = gemm_packed(s, m, ln.n_local, k, alpha, static_cast<const uint8_t*>(ln.ss->packed_a.ptr), 0,
                           static_cast<const uint8_t*>(ln.ss->packed_b.ptr), 0, beta, ln.c, nullptr, ln.ldc, 0, lc, 1,
                           policy, ln.st, ln.stream, opt, &ex);
        }
        if (rc != TCEC_OK) return rc;
        if (nranks > 1 && opt.comm_helper && ex.sched_base < static_cast<long long>(s.tiles_m) * s.tiles_n) {
          // after the counters were zeroed (the event is recorded behind the main launch, which is
          // queued, not finished) and once the broadcast has left its SMs
          rc = order(ln.ss, ln.stream, ln.ss->s_help);
          if (rc != TCEC_OK) return rc;
          TCEC_CUDA(cudaStreamWaitEvent(ln.ss->s_help, bcast_done, 0));
          LaunchExtras hx = ex;
          hx.row_ready = nullptr;  // everything has arrived by then
          hx.all_from_counter = 1;
          hx.grid = opt.comm_sms;
          hx.reserve_sms = 0;
          rc = gemm_packed(s, m, ln.n_local, k, alpha, static_cast<const uint8_t*>(ln.ss->packed_a.ptr), 0,
                           static_cast<const uint8_t*>(ln.ss->packed_b.ptr), 0, beta, ln.c, nullptr, ln.ldc, 0, lc, 1,
                           policy, ln.st, ln.ss->s_help, opt, &hx);
          if (rc != TCEC_OK) return rc;
          rc = order(ln.ss, ln.ss->s_help, ln.stream);
          if (rc != TCEC_OK) return rc;
        }
      }
    }
    if (nranks > 1) TCEC_CUDA(cudaStreamWaitEvent(ln.stream, bcast_done, 0));
    TCEC_CUDA(cudaGetLastError());
  }
  return TCEC_OK;
}

// Host operands (pinned memory for real overlap): every lane's B block is copied in and split
// once; A travels from the root's host memory in row panels (copy-in, split, broadcast); each
// panel's GEMM runs as its own launch into one of two device buffers and is copied out while the
// next panel is multiplied.  Copy-in, broadcast, GEMM and copy-out run on four streams.
int column_step_host(std::vector<Lane>& lanes, int nranks, int root, int la, int lb, int lc, int m, int k, float alpha,
                     float beta, int policy, int panel_rows, const Options& opt) {
  // Automatic panel height: on one GPU the pipeline is bound by the copy-in of A and B, and what
  // counts is a short tail behind the last copy (16384^3: 43.8 ms with 512 rows, 46.2 with 2048,
  // 49.7 with 4096; the two copies alone take 38.7 ms); with a broadcast per panel, 2048.
  if (panel_rows <= 0) panel_rows = nranks > 1 ? 2048 : 512;
  panel_rows = (panel_rows + 255) / 256 * 256;
  while ((m + panel_rows - 1) / panel_rows > kMaxPanels) panel_rows *= 2;
  const std::vector<Panel> panels = make_panels(m, k, policy, panel_rows);
  if (panels.size() > static_cast<size_t>(kMaxPanels)) return TCEC_ERR_UNSUPPORTED;
  const int prow = m < panel_rows ? (m + 255) / 256 * 256 : panel_rows;
  int cur = 0;
  TCEC_CUDA(cudaGetDevice(&cur));
  struct Restore {
    int dev;
    ~Restore() { cudaSetDevice(dev); }
  } restore{cur};
  struct LaneBufs {
    float *b32 = nullptr, *a32[2] = {nullptr, nullptr}, *c32[2] = {nullptr, nullptr};
    cudaEvent_t a_free[2] = {nullptr, nullptr}, c_free[2] = {nullptr, nullptr};
  };
  std::vector<LaneBufs> bufs(lanes.size());
  const size_t a_panel_bytes = static_cast<size_t>(prow) * k * sizeof(float);
  for (size_t i = 0; i < lanes.size(); ++i) {
    Lane& ln = lanes[i];
    TCEC_CUDA(cudaSetDevice(ln.device));
    const size_t b_bytes = static_cast<size_t>(k) * ln.n_local * sizeof(float);
    const size_t c_panel_bytes = static_cast<size_t>(prow) * ln.n_local * sizeof(float);
    const size_t align = 256;
    auto up = [&](size_t x) { return (x + align - 1) / align * align; };
    const bool is_root = ln.rank == root;
    int rc = ensure(&ln.ss->stage, up(b_bytes) + 2 * up(c_panel_bytes) + (is_root ? 2 * up(a_panel_bytes) : 0) + align);
    if (rc != TCEC_OK) return rc;
    rc = ensure(&ln.ss->packed_a, packed_bytes(m, k, policy));
    if (rc != TCEC_OK) return rc;
    rc = ensure(&ln.ss->packed_b, ln.n_local > 0 ? packed_bytes(ln.n_local, k, policy) : 16);
    if (rc != TCEC_OK) return rc;
    uint8_t* base = static_cast<uint8_t*>(ln.ss->stage.ptr);
    LaneBufs& lb_ = bufs[i];
    lb_.b32 = reinterpret_cast<float*>(base);
    base += up(b_bytes);
    for (int j = 0; j < 2; ++j) {
      lb_.c32[j] = reinterpret_cast<float*>(base);
      base += up(c_panel_bytes);
    }
    if (is_root)
      for (int j = 0; j < 2; ++j) {
        lb_.a32[j] = reinterpret_cast<float*>(base);
        base += up(a_panel_bytes);
      }
    // everything this call queues on the side streams follows what the caller queued before it
    rc = order(ln.ss, ln.stream, ln.ss->s_in);
    if (rc == TCEC_OK) rc = order(ln.ss, ln.stream, ln.ss->s_out);
    if (rc == TCEC_OK) rc = order(ln.ss, ln.stream, ln.ss->s_comm);
    if (rc != TCEC_OK) return rc;
    if (ln.n_local > 0 && k > 0) {
      // B block: k x n_local, dense on the device in the caller's layout
      const bool b_row = lb == TCEC_ROW_MAJOR;
      const size_t width = static_cast<size_t>(b_row ? ln.n_local : k) * 4, height = b_row ? k : ln.n_local;
      rc = copy2d(lb_.b32, width, ln.b, static_cast<size_t>(ln.ldb) * 4, width, height, cudaMemcpyHostToDevice,
                  ln.ss->s_in);
      if (rc == TCEC_OK) rc = order(ln.ss, ln.ss->s_in, ln.stream);
      if (rc != TCEC_OK) return rc;
      pack_operand(!b_row, ln.n_local, k, lb_.b32, nullptr, b_row ? ln.n_local : k, 0, 1,
                   static_cast<uint8_t*>(ln.ss->packed_b.ptr), 0, policy, ln.stream);
    }
  }
  Lane* root_lane = nullptr;
  LaneBufs* root_bufs = nullptr;
  for (size_t i = 0; i < lanes.size(); ++i)
    if (lanes[i].rank == root) {
      root_lane = &lanes[i];
      root_bufs = &bufs[i];
    }
  const bool product = k > 0 && alpha != 0.f;
  for (size_t p = 0; p < panels.size(); ++p) {
    const Panel& pn = panels[p];
    const int slot = static_cast<int>(p & 1);
    if (root_lane && product) {
      // root: panel p of A from host memory, split into its place in the packed A
      Lane& ln = *root_lane;
      TCEC_CUDA(cudaSetDevice(ln.device));
      if (root_bufs->a_free[slot]) TCEC_CUDA(cudaStreamWaitEvent(ln.ss->s_in, root_bufs->a_free[slot], 0));
      const bool a_row = la == TCEC_ROW_MAJOR;
      const size_t width = static_cast<size_t>(a_row ? k : pn.rows) * 4, height = a_row ? pn.rows : k;
      const float* src = a_row ? ln.a + static_cast<long long>(pn.row0) * ln.lda : ln.a + pn.row0;
      int rc = copy2d(root_bufs->a32[slot], width, src, static_cast<size_t>(ln.lda) * 4, width, height,
                      cudaMemcpyHostToDevice, ln.ss->s_in);
      if (rc == TCEC_OK) rc = order(ln.ss, ln.ss->s_in, ln.stream);
      if (rc != TCEC_OK) return rc;
      pack_operand(a_row, pn.rows, k, root_bufs->a32[slot], nullptr, a_row ? k : pn.rows, 0, 1,
                   static_cast<uint8_t*>(ln.ss->packed_a.ptr) + pn.offset, 0, policy, ln.stream);
      rc = next_event(ln.ss, &root_bufs->a_free[slot]);
      if (rc != TCEC_OK) return rc;
      TCEC_CUDA(cudaEventRecord(root_bufs->a_free[slot], ln.stream));
      if (nranks > 1) TCEC_CUDA(cudaStreamWaitEvent(ln.ss->s_comm, root_bufs->a_free[slot], 0));
    }
    if (nranks > 1 && product) {
      const int rc = broadcast_panel(lanes, pn, root);
      if (rc != TCEC_OK) return rc;
    }
    for (size_t i = 0; i < lanes.size(); ++i) {
      Lane& ln = lanes[i];
      LaneBufs& lb_ = bufs[i];
      if (ln.n_local == 0) continue;
      TCEC_CUDA(cudaSetDevice(ln.device));
      int rc;
      if (nranks > 1 && product && ln.rank != root) {
        rc = order(ln.ss, ln.ss->s_comm, ln.stream);  // panel p has arrived
        if (rc != TCEC_OK) return rc;
      }
      if (lb_.c_free[slot]) TCEC_CUDA(cudaStreamWaitEvent(ln.stream, lb_.c_free[slot], 0));
      // C panel on the device: dense, in the caller's layout
      const bool c_row = lc == TCEC_ROW_MAJOR;
      const long long ldc_dev = c_row ? ln.n_local : pn.rows;
      const size_t width = static_cast<size_t>(c_row ? ln.n_local : pn.rows) * 4, height = c_row ? pn.rows : ln.n_local;
      float* c_host = c_row ? ln.c + static_cast<long long>(pn.row0) * ln.ldc : ln.c + pn.row0;
      if (beta != 0.f) {
        rc = order(ln.ss, ln.stream, ln.ss->s_in);  // the buffer is free (c_free was waited for on ln.stream)
        if (rc == TCEC_OK)
          rc = copy2d(lb_.c32[slot], width, c_host, static_cast<size_t>(ln.ldc) * 4, width, height, cudaMemcpyHostToDevice,
                      ln.ss->s_in);
        if (rc == TCEC_OK) rc = order(ln.ss, ln.ss->s_in, ln.stream);
        if (rc != TCEC_OK) return rc;
      }
      if (!product) {
        rc = scale_only(beta, lb_.c32[slot], nullptr, ldc_dev, 0, pn.rows, ln.n_local, lc, 1, ln.stream);
      } else {
        const Shape s = plan(pn.rows, ln.n_local, k, policy, opt);
        LaunchExtras ex;
        if (nranks > 1) ex.reserve_sms = opt.comm_sms;
        std::lock_guard<std::mutex> lock(state_mutex());  // the per-stream tile counters may be created here
        rc = gemm_packed(s, pn.rows, ln.n_local, k, alpha, static_cast<const uint8_t*>(ln.ss->packed_a.ptr) + pn.offset, 0,
                         static_cast<const uint8_t*>(ln.ss->packed_b.ptr), 0, beta, lb_.c32[slot], nullptr, ldc_dev, 0, lc,
                         1, policy, ln.st, ln.stream, opt, &ex);
      }
      if (rc != TCEC_OK) return rc;
      rc = order(ln.ss, ln.stream, ln.ss->s_out);
      if (rc == TCEC_OK)
        rc = copy2d(c_host, static_cast<size_t>(ln.ldc) * 4, lb_.c32[slot], width, width, height, cudaMemcpyDeviceToHost,
                    ln.ss->s_out);
      if (rc == TCEC_OK) rc = next_event(ln.ss, &lb_.c_free[slot]);
      if (rc != TCEC_OK) return rc;
      TCEC_CUDA(cudaEventRecord(lb_.c_free[slot], ln.ss->s_out));
    }
  }
  // the caller's stream ends behind every copy-out and behind the broadcast
  for (Lane& ln : lanes) {
    TCEC_CUDA(cudaSetDevice(ln.device));
    int rc = order(ln.ss, ln.ss->s_out, ln.stream);
    if (rc == TCEC_OK) rc = order(ln.ss, ln.ss->s_comm, ln.stream);
    if (rc == TCEC_OK) rc = order(ln.ss, ln.ss->s_in, ln.stream);
    if (rc != TCEC_OK) return rc;
    TCEC_CUDA(cudaGetLastError());
  }
  return TCEC_OK;
}

// Device and step state of the current device (state mutex held by the caller).
int lane_state(Lane* ln) {
  TCEC_CUDA(cudaSetDevice(ln->device));
  int rc = get_device_state(&ln->st);
  if (rc != TCEC_OK) return rc;
  return step_state(ln->st, &ln->ss);
}

// Communicators for a device list in one process, made on first use and kept until tcec_destroy.
int multi_comms(int ndev, const int* devices, int max_ctas) {
  bool same = static_cast<int>(g_multi_devices.size()) == ndev;
  for (int i = 0; same && i < ndev; ++i) same = g_multi_devices[i] == devices[i] && g_multi_comms[i].max_ctas == max_ctas;
  if (same) return TCEC_OK;
  for (Comm& c : g_multi_comms) destroy_comm(&c);
  g_multi_comms.clear();
  g_multi_devices.clear();
  int rc = load_nccl();
  if (rc != TCEC_OK) return rc;
  ncclUniqueId id;
  TCEC_NCCL(g_nccl.GetUniqueId(&id));
  std::vector<Comm> comms(ndev);
  ncclConfig_t cfg = comm_config(max_ctas);
  TCEC_NCCL(g_nccl.GroupStart());
  for (int i = 0; i < ndev; ++i) {
    if (cudaSetDevice(devices[i]) != cudaSuccess) {
      g_nccl.GroupEnd();
      return TCEC_ERR_CUDA;
    }
    comms[i].nranks = ndev;
    comms[i].rank = i;
    comms[i].device = devices[i];
    comms[i].max_ctas = max_ctas;
    if (g_nccl.CommInitRankConfig(&comms[i].comm, ndev, id, i, &cfg) != ncclSuccess) {
      g_nccl.GroupEnd();
      return TCEC_ERR_COMM;
    }
  }
  TCEC_NCCL(g_nccl.GroupEnd());
  g_multi_comms = comms;
  g_multi_devices.assign(devices, devices + ndev);
  return TCEC_OK;
}
}  // namespace

void destroy_step_state(DeviceState* st) {
  StepState* s = st->step;
  if (!s) return;
  for (cudaEvent_t e : s->events) cudaEventDestroy(e);
  for (cudaStream_t q : {s->s_in, s->s_out, s->s_comm, s->s_help})
    if (q) cudaStreamDestroy(q);
  for (Workspace* w : {&s->packed_a, &s->packed_b, &s->stage})
    if (w->ptr) cudaFree(w->ptr);
  if (s->words) cudaFree(s->words);
  delete s;
  st->step = nullptr;
}

}  // namespace tcec_host

using namespace tcec_host;

extern "C" {

int tcec_sgemm_host(int layout_a, int layout_b, int layout_c, int m, int n, int k, float alpha, const float* a_host,
                    long long lda, const float* b_host, long long ldb, float beta, float* c_host, long long ldc,
                    int policy, int panel_rows, void* stream) {
  int rc = check_shard_args(layout_a, layout_b, layout_c, m, k, policy);
  if (rc != TCEC_OK || n < 0) return TCEC_ERR_INVALID_ARGUMENT;
  if (m == 0 || n == 0) return TCEC_OK;
  if (!c_host || ldc < (layout_c == TCEC_ROW_MAJOR ? n : m)) return TCEC_ERR_INVALID_ARGUMENT;
  if (k > 0 && alpha != 0.f) {
    if (!a_host || !b_host) return TCEC_ERR_INVALID_ARGUMENT;
    if (lda < (layout_a == TCEC_ROW_MAJOR ? k : m) || ldb < (layout_b == TCEC_ROW_MAJOR ? n : k))
      return TCEC_ERR_INVALID_ARGUMENT;
  }
  std::vector<Lane> lanes(1);
  Lane& ln = lanes[0];
  Options opt;
  {
    std::lock_guard<std::mutex> lock(state_mutex());
    TCEC_CUDA(cudaGetDevice(&ln.device));
    rc = lane_state(&ln);
    if (rc != TCEC_OK) return rc;
  }
  opt = snapshot_options();
  ln.stream = static_cast<cudaStream_t>(stream);
  ln.a = a_host;
  ln.lda = lda;
  ln.b = b_host;
  ln.ldb = ldb;
  ln.c = c_host;
  ln.ldc = ldc;
  ln.n_local = n;
  return column_step_host(lanes, 1, 0, layout_a, layout_b, layout_c, m, k, alpha, beta, policy, panel_rows, opt);
}

int tcec_comm_set_library(const char* path) {
  std::lock_guard<std::mutex> lock(state_mutex());
  if (g_nccl.lib) return TCEC_ERR_INVALID_ARGUMENT;  // already loaded
  g_nccl_path = path ? path : "";
  return TCEC_OK;
}

int tcec_comm_unique_id(void* id) {
  if (!id) return TCEC_ERR_INVALID_ARGUMENT;
  static_assert(sizeof(ncclUniqueId) == TCEC_COMM_ID_BYTES, "unique id size");
  std::lock_guard<std::mutex> lock(state_mutex());
  const int rc = load_nccl();
  if (rc != TCEC_OK) return rc;
  ncclUniqueId uid;
  TCEC_NCCL(g_nccl.GetUniqueId(&uid));
  memcpy(id, &uid, sizeof(uid));
  return TCEC_OK;
}

int tcec_comm_init_rank(int nranks, int rank, const void* id) {
  if (nranks < 1 || rank < 0 || rank >= nranks || !id) return TCEC_ERR_INVALID_ARGUMENT;
  const int max_ctas = snapshot_options().comm_sms;  // the broadcast may use as many CTAs as the GEMM leaves SMs
  std::lock_guard<std::mutex> lock(state_mutex());
  int rc = load_nccl();
  if (rc != TCEC_OK) return rc;
  destroy_comm(&g_rank_comm);
  int dev = 0;
  TCEC_CUDA(cudaGetDevice(&dev));
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof(uid));
  ncclConfig_t cfg = comm_config(max_ctas);
  Comm c;
  c.nranks = nranks;
  c.rank = rank;
  c.device = dev;
  c.max_ctas = max_ctas;
  if (g_nccl.CommInitRankConfig(&c.comm, nranks, uid, rank, &cfg) != ncclSuccess) return TCEC_ERR_COMM;
  g_rank_comm = c;
  return TCEC_OK;
}

int tcec_comm_destroy(void) {
  std::lock_guard<std::mutex> lock(state_mutex());
  destroy_comm_state();
  return TCEC_OK;
}

static int column_shard_entry(bool host, int root, int layout_a, int layout_b, int layout_c, int m, int n_local, int k,
                              float alpha, const float* a, long long lda, const float* b, long long ldb, float beta,
                              float* c, long long ldc, int policy, int panel_rows, void* stream) {
  int rc = check_shard_args(layout_a, layout_b, layout_c, m, k, policy);
  if (rc != TCEC_OK || n_local < 0) return TCEC_ERR_INVALID_ARGUMENT;
  std::vector<Lane> lanes(1);
  Lane& ln = lanes[0];
  int nranks = 1;
  {
    std::lock_guard<std::mutex> lock(state_mutex());
    if (g_rank_comm.comm) {
      nranks = g_rank_comm.nranks;
      ln.rank = g_rank_comm.rank;
      ln.comm = g_rank_comm.comm;
    }
    if (root < 0 || root >= nranks) return TCEC_ERR_INVALID_ARGUMENT;
    const bool product = k > 0 && alpha != 0.f;
    if (n_local > 0 && m > 0) {
      if (!c || ldc < (layout_c == TCEC_ROW_MAJOR ? n_local : m)) return TCEC_ERR_INVALID_ARGUMENT;
      if (product && (!b || ldb < (layout_b == TCEC_ROW_MAJOR ? n_local : k))) return TCEC_ERR_INVALID_ARGUMENT;
    }
    if (ln.rank == root && product && m > 0 && (!a || lda < (layout_a == TCEC_ROW_MAJOR ? k : m)))
      return TCEC_ERR_INVALID_ARGUMENT;
    TCEC_CUDA(cudaGetDevice(&ln.device));
    if (g_rank_comm.comm && g_rank_comm.device != ln.device) return TCEC_ERR_INVALID_ARGUMENT;
    rc = lane_state(&ln);
    if (rc != TCEC_OK) return rc;
  }
  if (m == 0) return TCEC_OK;
  const Options opt = snapshot_options();
  ln.stream = static_cast<cudaStream_t>(stream);
  ln.a = a;
  ln.lda = lda;
  ln.b = b;
  ln.ldb = ldb;
  ln.c = c;
  ln.ldc = ldc;
  ln.n_local = n_local;
  if (host)
    return column_step_host(lanes, nranks, root, layout_a, layout_b, layout_c, m, k, alpha, beta, policy, panel_rows, opt);
  return column_step_device(lanes, nranks, root, layout_a, layout_b, layout_c, m, k, alpha, beta, policy, opt);
}

int tcec_sgemm_column_shard(int root, int layout_a, int layout_b, int layout_c, int m, int n_local, int k, float alpha,
                            const float* a, long long lda, const float* b, long long ldb, float beta, float* c,
                            long long ldc, int policy, void* stream) {
  return column_shard_entry(false, root, layout_a, layout_b, layout_c, m, n_local, k, alpha, a, lda, b, ldb, beta, c,
                            ldc, policy, 0, stream);
}

int tcec_sgemm_column_shard_host(int root, int layout_a, int layout_b, int layout_c, int m, int n_local, int k,
                                 float alpha, const float* a_host, long long lda, const float* b_host, long long ldb,
                                 float beta, float* c_host, long long ldc, int policy, int panel_rows, void* stream) {
  return column_shard_entry(true, root, layout_a, layout_b, layout_c, m, n_local, k, alpha, a_host, lda, b_host, ldb,
                            beta, c_host, ldc, policy, panel_rows, stream);
}

int tcec_sgemm_multi(int ndev, const int* devices, int layout_a, int layout_b, int layout_c, int m, const int* n_local,
                     int k, float alpha, const float* a, long long lda, const float* const* b, const long long* ldb,
                     float beta, float* const* c, const long long* ldc, int policy, void* const* streams) {
  if (ndev < 1 || ndev > 64 || !devices || !n_local || !b || !ldb || !c || !ldc) return TCEC_ERR_INVALID_ARGUMENT;
  int rc = check_shard_args(layout_a, layout_b, layout_c, m, k, policy);
  if (rc != TCEC_OK) return rc;
  const bool product = k > 0 && alpha != 0.f;
  for (int i = 0; i < ndev; ++i) {
    if (n_local[i] < 0 || devices[i] < 0) return TCEC_ERR_INVALID_ARGUMENT;
    for (int j = 0; j < i; ++j)
      if (devices[j] == devices[i]) return TCEC_ERR_INVALID_ARGUMENT;
    if (n_local[i] > 0 && m > 0) {
      if (!c[i] || ldc[i] < (layout_c == TCEC_ROW_MAJOR ? n_local[i] : m)) return TCEC_ERR_INVALID_ARGUMENT;
      if (product && (!b[i] || ldb[i] < (layout_b == TCEC_ROW_MAJOR ? n_local[i] : k))) return TCEC_ERR_INVALID_ARGUMENT;
    }
  }
  if (product && m > 0 && (!a || lda < (layout_a == TCEC_ROW_MAJOR ? k : m))) return TCEC_ERR_INVALID_ARGUMENT;
  if (m == 0) return TCEC_OK;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) return TCEC_ERR_CUDA;
  for (int i = 0; i < ndev; ++i)
    if (devices[i] >= count) return TCEC_ERR_INVALID_ARGUMENT;
  const Options opt = snapshot_options();
  std::vector<Lane> lanes(ndev);
  int cur = 0;
  TCEC_CUDA(cudaGetDevice(&cur));
  {
    std::lock_guard<std::mutex> lock(state_mutex());
    if (ndev > 1) {
      rc = multi_comms(ndev, devices, opt.comm_sms);
      if (rc != TCEC_OK) {
        cudaSetDevice(cur);
        return rc;
      }
    }
    for (int i = 0; i < ndev; ++i) {
      Lane& ln = lanes[i];
      ln.device = devices[i];
      ln.rank = i;
      ln.comm = ndev > 1 ? g_multi_comms[i].comm : nullptr;
      rc = lane_state(&ln);
      if (rc != TCEC_OK) {
        cudaSetDevice(cur);
        return rc;
      }
      ln.stream = streams ? static_cast<cudaStream_t>(streams[i]) : nullptr;
      ln.a = i == 0 ? a : nullptr;
      ln.lda = lda;
      ln.b = b[i];
      ln.ldb = ldb[i];
      ln.c = c[i];
      ln.ldc = ldc[i];
      ln.n_local = n_local[i];
    }
    cudaSetDevice(cur);
  }
  return column_step_device(lanes, ndev, 0, layout_a, layout_b, layout_c, m, k, alpha, beta, policy, opt);
}

int tcec_sgemm_batched_multi(int ndev, const int* devices, int layout_a, int layout_b, int layout_c, int m, int n, int k,
                             float alpha, const float* const* a, long long lda, long long stride_a,
                             const float* const* b, long long ldb, long long stride_b, float beta, float* const* c,
                             long long ldc, long long stride_c, const int* batch_local, int policy,
                             void* const* streams) {
  if (ndev < 1 || ndev > 64 || !devices || !a || !b || !c || !batch_local) return TCEC_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < ndev; ++i)
    if (batch_local[i] < 0 || devices[i] < 0) return TCEC_ERR_INVALID_ARGUMENT;
  int cur = 0;
  TCEC_CUDA(cudaGetDevice(&cur));
  int worst = TCEC_OK;
  // independent matrices: every device runs the single-GPU call on its slice, no collective
  for (int i = 0; i < ndev; ++i) {
    if (batch_local[i] == 0) continue;
    if (cudaSetDevice(devices[i]) != cudaSuccess) {
      worst = TCEC_ERR_CUDA;
      continue;
    }
    const int rc = gemm_impl(layout_a, layout_b, layout_c, m, n, k, alpha, a[i], nullptr, lda, stride_a, b[i], nullptr,
                             ldb, stride_b, beta, c[i], nullptr, ldc, stride_c, batch_local[i], policy,
                             streams ? streams[i] : nullptr);
    if (rc != TCEC_OK && worst == TCEC_OK) worst = rc;
  }
  cudaSetDevice(cur);
  return worst;
}

}  // extern "C"
