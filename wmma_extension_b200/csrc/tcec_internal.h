// Host-side internals shared by the translation units of the library: option snapshot, per-device
// state, operand packing and the packed GEMM launch.  Nothing here is part of the C ABI.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <vector>

#include "../../include/tcec.h"

namespace tcec_host {

#define TCEC_CUDA(call)                          \
  do {                                           \
    cudaError_t e_ = (call);                     \
    if (e_ != cudaSuccess) return TCEC_ERR_CUDA; \
  } while (0)

// Process-wide options (tcec_set_option).  Every entry point copies them once, under the state
// mutex, and works from the copy, so a call never sees a half-changed set and holds no lock
// while it launches.
struct Options {
  int promote_k = -1;   // -1: chosen per call from K and the policy
  int tile_n = 0;
  int store_turn = 1;   // 0: the panel kernel stores directly and leaves ~30 KB of shared memory per SM free
  int static_tiles = 0; // 0: tiles beyond the first wave are drawn from a device-wide counter; 1: static striding
  int reserve_sms = 0;  // SMs the GEMM kernels leave idle (for a caller's communication kernels)
  int cta_pair = -1;    // -1: CTA-pair kernel for the policies without error correction; 0: never; 1: whenever it applies
  int half_tiles = 1;   // CTA-pair kernel: calls with very few tiles run on 256 x 128 half tiles
  int path = 0;         // 0: chosen per call, 1: always operand panels, 2: FP32-tile kernel whenever it applies
  int comm_sms = 8;     // SMs the column-sharded step leaves to the broadcast (also the broadcast's CTA limit)
  int comm_panel_rows = 2048;  // rows of A per broadcast
  int comm_helper = 1;  // 1: once the broadcast is over, a second launch takes the SMs it had
  int debug_flags = 0;  // develop builds only
  unsigned long long* trace = nullptr;  // develop builds only
};
Options snapshot_options();

struct Workspace {
  void* ptr = nullptr;
  size_t bytes = 0;
};

// What the multi-GPU step keeps per device (tcec_multi.cu owns the contents).
struct StepState;

struct DeviceState {
  int* status = nullptr;
  int sm_count = 0;
  bool attrs_done = false;
  std::map<cudaStream_t, Workspace> ws;
  std::map<cudaStream_t, unsigned int*> sched;  // per stream: the panel GEMM's two tile-scheduler counters
  unsigned int* sched_fixed = nullptr;          // set instead by the allocation-free entry (a device symbol)
  StepState* step = nullptr;
};

std::mutex& state_mutex();
// Both need the state mutex held.
int get_device_state(DeviceState** out);
int get_workspace(DeviceState* st, cudaStream_t stream, size_t bytes, void** out, void** to_free);
int get_sched(DeviceState* st, cudaStream_t stream, unsigned int** out);
// Called by tcec_destroy for every device, with that device current and the mutex held.
void destroy_step_state(DeviceState* st);
void destroy_comm_state();

struct Shape {
  int tile_n, tiles_m, tiles_n, nkb, kop, np;
  int a_row_blocks, b_row_blocks;  // 128-row panel blocks, padded to an even count
  size_t a_bytes, b_bytes;         // per matrix
};
bool policy_tf32(int policy);
bool policy_ec(int policy);
bool bad_layout(int l);
size_t packed_bytes(int rows, int k, int policy);
Shape plan(int m, int n, int k, int policy, const Options& opt);

// Split one operand (A: rows = m; B: rows = n) into panels on `stream`.
// `part` describes an operand that is one half of a K-concatenated panel set built from
// interleaved complex data: element stride 2, a sign, and where its k blocks go.
struct PackPart {
  int elem_stride = 1;
  float mul = 1.0f;
  int kb_offset = 0;
  int nkb_out = 0;
};
void pack_operand(bool k_contiguous, int rows, int k, const float* src, const float* const* src_array, long long ld,
                  long long stride, int batch, uint8_t* panels, size_t panels_stride, int policy, cudaStream_t stream,
                  const PackPart& part = PackPart());

// What a launch of the packed GEMM may add to the plain call.
struct LaunchExtras {
  int reserve_sms = -1;                    // -1: the option's value
  int grid = 0;                            // > 0: exactly this many CTAs (a helper launch)
  const unsigned int* row_ready = nullptr; // one word per `ready_rows` rows of A: the producer of a tile waits
  int ready_rows = 0;                      //   (bounded) until the word of the tile's rows equals `ready_epoch`
  unsigned int ready_epoch = 0;
  unsigned int* sched = nullptr;           // tile counters shared by several launches (reset by the caller)
  int sched_base = 0;                      // with `sched`: tiles below this index belong to the first launch's CTAs
  int all_from_counter = 0;                // with `sched`: this launch's CTAs draw even their first tile
  int force_one_sm = 0;                    // never the CTA-pair kernel (it knows neither flags nor shared counters)
};
int gemm_packed(const Shape& s, int m, int n, int k, float alpha, const uint8_t* panels_a, size_t a_stride,
                const uint8_t* panels_b, size_t b_stride, float beta, float* c, float* const* c_array, long long ldc,
                long long stride_c, int lc, int batch, int policy, DeviceState* st, cudaStream_t stream,
                const Options& opt, const LaunchExtras* extras = nullptr);
// The whole single-GPU call (argument checks included): tcec_sgemm and its batched forms.
int gemm_impl(int la, int lb, int lc, int m, int n, int k, float alpha, const float* a, const float* const* a_array,
              long long lda, long long stride_a, const float* b, const float* const* b_array, long long ldb,
              long long stride_b, float beta, float* c, float* const* c_array, long long ldc, long long stride_c,
              int batch, int policy, void* stream_v);
int scale_only(float beta, float* c, float* const* c_array, long long ldc, long long stride_c, int m, int n, int lc,
               int batch, cudaStream_t stream);

}  // namespace tcec_host
