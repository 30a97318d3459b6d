/*
 * tcec.h - C ABI of the B200 (sm_100a) error-corrected SGEMM emulation.
 *
 * FP32 GEMM computed on tensor cores: every input is split into a low-precision
 * head and a scaled residual, three tensor-core products are formed, and the
 * correction term is folded back in FP32 (algorithm of wmma_extension's
 * mtk::wmma::tcec, include/wmma_extension/tcec/tcec.hpp).
 *
 * All matrix pointers are DEVICE pointers owned by the caller.  Calls are
 * asynchronous on `stream` (a cudaStream_t passed as void*; NULL = default
 * stream) and return an integer status, never throw and never exit.  The
 * library owns only its cached workspace and two tile-scheduler counters per
 * (device, stream) and a device status word, created on first use and released
 * by tcec_destroy().
 *
 * The reference has no host API: its closest counterpart is the launch glue of
 * its batched example, launch_bgemm() (test/tcec/batch_gemm.cu:433-443) and the
 * cublasSgemmBatched call it is benchmarked against (test/tcec/batch_gemm.cu:619-621).
 * Argument order follows those.
 */
#ifndef TCEC_H_
#define TCEC_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define TCEC_OK 0
#define TCEC_ERR_INVALID_ARGUMENT 1
#define TCEC_ERR_UNSUPPORTED 2
#define TCEC_ERR_CUDA 3
#define TCEC_ERR_TIMEOUT 4 /* a bounded device-side wait ran out */
#define TCEC_ERR_ALLOC 5
#define TCEC_ERR_TOO_LARGE 6 /* tcec_sgemm_static only: operands exceed TCEC_STATIC_SCRATCH_BYTES */
#define TCEC_ERR_COMM 7 /* the communication library (NCCL) is missing, failed, or no communicator exists */

/* storage order of a matrix: element (i,j) at i*ld + j (row) or i + j*ld (col) */
#define TCEC_ROW_MAJOR 0
#define TCEC_COL_MAJOR 1

/*
 * Policies: input type of the tensor-core products x error correction.
 * Mirrors the reference's fragment type T (half / nvcuda::wmma::precision::tf32)
 * and its with_ec / without_ec tags (include/wmma_extension/tcec/detail/policy.hpp:12-20).
 */
#define TCEC_POLICY_FP16_EC 0
#define TCEC_POLICY_TF32_EC 1
#define TCEC_POLICY_FP16_NO_EC 2
#define TCEC_POLICY_TF32_NO_EC 3

/*
 * C = alpha * A(m x k) * B(k x n) + beta * C(m x n).
 * Replaces launch_bgemm() with batch 1 (test/tcec/batch_gemm.cu:433-443); the
 * kernel it stands for is bgemm_kernel (test/tcec/batch_gemm.cu:261-386), whose
 * fixed layout (A row-major, B col-major, C col-major) is one of the eight
 * layout combinations accepted here.  beta == 0 never reads C, as in the
 * reference epilogue (test/tcec/batch_gemm.cu:124-158).
 */
int tcec_sgemm(int layout_a, int layout_b, int layout_c, int m, int n, int k, float alpha,
               const float* a, long long lda, const float* b, long long ldb, float beta, float* c,
               long long ldc, int policy, void* stream);

/*
 * Pointer-array batch: a_array/b_array/c_array are DEVICE arrays of `batch`
 * device pointers, one matrix each, all of the same shape and leading
 * dimensions.  Replaces launch_bgemm() (test/tcec/batch_gemm.cu:433-443), same
 * argument meaning as cublasSgemmBatched (test/tcec/batch_gemm.cu:619-621).
 */
int tcec_sgemm_batched(int layout_a, int layout_b, int layout_c, int m, int n, int k, float alpha,
                       const float* const* a_array, long long lda, const float* const* b_array,
                       long long ldb, float beta, float* const* c_array, long long ldc, int batch,
                       int policy, void* stream);

/*
 * Strided batch: matrix i of A starts at a + i*stride_a (elements), likewise B
 * and C.  Convenience form of the pointer-array batch above for contiguous
 * batches (the reference allocates one buffer per matrix, test/tcec/batch_gemm.cu:469-533).
 */
int tcec_sgemm_strided_batched(int layout_a, int layout_b, int layout_c, int m, int n, int k,
                               float alpha, const float* a, long long lda, long long stride_a,
                               const float* b, long long ldb, long long stride_b, float beta,
                               float* c, long long ldc, long long stride_c, int batch, int policy,
                               void* stream);

/*
 * The same two calls in cuBLAS's convention, for host code that switches by renaming the call:
 * column-major storage, transposition flags with cuBLAS's values (0 = CUBLAS_OP_N, 1 = _T,
 * 2 = _C), alpha and beta by host pointer.  They stand in for the cublasSgemmBatched call the
 * reference times its kernel against (test/tcec/batch_gemm.cu:619-621:
 * cublasSgemmBatched(handle, CUBLAS_OP_T, CUBLAS_OP_N, m, n, k, &alpha, A, k, B, k, &beta, C, m, batch))
 * and for cublasSgemm; the handle is replaced by (policy, stream).
 */
int tcec_sgemm_cublas(int transa, int transb, int m, int n, int k, const float* alpha, const float* a, int lda,
                      const float* b, int ldb, const float* beta, float* c, int ldc, int policy, void* stream);
int tcec_sgemm_batched_cublas(int transa, int transb, int m, int n, int k, const float* alpha,
                              const float* const* a_array, int lda, const float* const* b_array, int ldb,
                              const float* beta, float* const* c_array, int ldc, int batch, int policy,
                              void* stream);

/*
 * tcec_sgemm without any allocation.  This entry point has no counterpart in the reference.
 *
 * For callers that cannot call cudaMalloc when they need the product - a process whose memory
 * pool already owns the device, a latency-critical loop that must stay off the allocator's
 * locks, a plugin host that forbids allocation after start-up.  Same arguments, result and
 * rounding as tcec_sgemm; the split operands go to a fixed TCEC_STATIC_SCRATCH_BYTES array that
 * is part of the library's device image (each GPU that loads the library holds it until the
 * process ends) instead of a cudaMalloc'ed workspace, and the call makes no cudaMalloc, cudaFree
 * or other allocating call, on the device or on the host.
 *
 * Limit: tcec_packed_bytes(m, k, policy) + tcec_packed_bytes(n, k, policy) must not exceed
 * TCEC_STATIC_SCRATCH_BYTES (e.g. up to 2048 x 2048 x 2048 with the fp16 policies, half of that
 * K with tf32); larger problems return TCEC_ERR_TOO_LARGE and launch nothing.
 *
 * The first call on a device looks up the array's device address and sets kernel attributes;
 * make that first call outside any stream capture.  All calls on a device share the one array
 * and it keeps the previous call's panels: two calls whose kernels overlap on the GPU (different
 * streams without an ordering between them) race and give wrong results - order them.  Nothing
 * in the array needs clearing between calls; every byte the GEMM reads is rewritten first.
 * Bounded-wait expiry is reported by tcec_static_status(), the counterpart of
 * tcec_device_status() for this entry point.
 */
#define TCEC_STATIC_SCRATCH_BYTES (32u << 20)
int tcec_sgemm_static(int layout_a, int layout_b, int layout_c, int m, int n, int k, float alpha,
                      const float* a, long long lda, const float* b, long long ldb, float beta, float* c,
                      long long ldc, int policy, void* stream);
size_t tcec_static_scratch_bytes(void);
int tcec_static_status(int* detail);

/*
 * tcec_sgemm on HOST operands (pinned memory makes the copies asynchronous): B is copied in and
 * split once, A travels in panels of `panel_rows` rows (0 = automatic: 512), and the copy-in of panel p+1,
 * the GEMM on panel p and the copy-out of panel p-1 overlap on three streams.  The call returns
 * once everything is queued; the result is complete when `stream` has reached the end of the
 * call's work (synchronise it, or record an event on it, before reading c_host).  The reference
 * example stages its operands with one cudaMemcpy each before and after the launch
 * (test/tcec/batch_gemm.cu:515-533, :548); this is that sequence pipelined.  Device staging
 * buffers are library-owned and cached per device; one such call at a time per device.
 */
int tcec_sgemm_host(int layout_a, int layout_b, int layout_c, int m, int n, int k, float alpha,
                    const float* a_host, long long lda, const float* b_host, long long ldb, float beta,
                    float* c_host, long long ldc, int policy, int panel_rows, void* stream);

/*
 * Several GPUs of one box.  K is never split, so there is no reduction: a batch is divided by
 * matrices (no collective at all), a large GEMM by column blocks of B and C with A broadcast
 * from its owner by NCCL (ncclBroadcast of split row panels, each panel's flag raised behind it;
 * one persistent GEMM launch per GPU consumes the panels as they arrive and leaves "comm_sms"
 * SMs to the broadcast).  The reference has no multi-GPU code and no collective call site; these
 * entries stand where its launch glue does (test/tcec/batch_gemm.cu:433-443).  NCCL is loaded at
 * run time (libnccl.so.2, or the library named by TCEC_NCCL_LIBRARY / tcec_comm_set_library),
 * so single-GPU users need none.  Kernels only read their own GPU's memory.
 *
 * One process drives all devices: tcec_sgemm_multi / tcec_sgemm_batched_multi take a device
 * list; operand i lives on devices[i]; A (m x k) lives on devices[0]; streams may be NULL (the
 * default stream of each device) or one stream per device.  Communicators for the list are made
 * on first use and freed by tcec_destroy().  The calls return when everything is queued; the
 * first status that is not TCEC_OK among the devices is returned.
 *   n_local[i]  columns of B and C held by devices[i] (whole output tiles of 256 columns keep
 *               every GPU's work even); b[i] is k x n_local[i], c[i] is m x n_local[i].
 */
int tcec_sgemm_multi(int ndev, const int* devices, int layout_a, int layout_b, int layout_c, int m,
                     const int* n_local, int k, float alpha, const float* a, long long lda,
                     const float* const* b, const long long* ldb, float beta, float* const* c,
                     const long long* ldc, int policy, void* const* streams);
int tcec_sgemm_batched_multi(int ndev, const int* devices, int layout_a, int layout_b, int layout_c, int m, int n,
                             int k, float alpha, const float* const* a, long long lda, long long stride_a,
                             const float* const* b, long long ldb, long long stride_b, float beta,
                             float* const* c, long long ldc, long long stride_c, const int* batch_local,
                             int policy, void* const* streams);

/*
 * One process per device (what torchrun and MPI launchers give): rank 0 obtains an id with
 * tcec_comm_unique_id, hands its TCEC_COMM_ID_BYTES bytes to the other ranks by whatever means
 * the job has, and every rank calls tcec_comm_init_rank with its device current.  Then
 * tcec_sgemm_column_shard is this rank's part of the column-sharded GEMM: `a` is read on `root`
 * only; b (k x n_local) and c (m x n_local) are this rank's blocks.  Every rank must call it, in
 * the same order.  The _host form takes host operands (A on the root, B and C blocks on every
 * rank) and pipelines copy-in, broadcast, GEMM and copy-out in panels of `panel_rows` rows.
 * Without a communicator (or with one rank) both forms compute locally.
 */
#define TCEC_COMM_ID_BYTES 128
int tcec_comm_set_library(const char* path);
int tcec_comm_unique_id(void* id);
int tcec_comm_init_rank(int nranks, int rank, const void* id);
int tcec_comm_destroy(void);
int tcec_sgemm_column_shard(int root, int layout_a, int layout_b, int layout_c, int m, int n_local, int k,
                            float alpha, const float* a, long long lda, const float* b, long long ldb, float beta,
                            float* c, long long ldc, int policy, void* stream);
int tcec_sgemm_column_shard_host(int root, int layout_a, int layout_b, int layout_c, int m, int n_local, int k,
                                 float alpha, const float* a_host, long long lda, const float* b_host,
                                 long long ldb, float beta, float* c_host, long long ldc, int policy,
                                 int panel_rows, void* stream);

/*
 * Split once, multiply many times.  tcec_pack_a / tcec_pack_b run the split of
 * load_matrix_sync (include/wmma_extension/tcec/tcec.hpp:194-236) over a whole
 * operand and store hi (+ scaled lo) in the layout the GEMM kernel streams;
 * tcec_sgemm_packed is tcec_sgemm on operands packed that way.  `packed` is a
 * caller-owned device buffer of tcec_packed_bytes(rows, k, policy) bytes, 16-byte
 * aligned, where rows = m for A and n for B.  The reference re-splits a tile in
 * every warp that consumes it (test/tcec/batch_gemm.cu:232-255); packing is what
 * lets one operand (B of a column shard, A after its broadcast) be split once.
 * A row sub-range of a packed operand that starts at a multiple of 256 rows is
 * itself a packed operand: it begins tcec_packed_row_offset(row, k, policy) bytes in
 * (0 for any other row: the 256-wide tiles and the CTA-pair kernel read row blocks in pairs).
 */
size_t tcec_packed_bytes(int rows, int k, int policy);
size_t tcec_packed_row_offset(int row, int k, int policy);
int tcec_pack_a(int layout_a, int m, int k, const float* a, long long lda, void* packed, int policy,
                void* stream);
int tcec_pack_b(int layout_b, int k, int n, const float* b, long long ldb, void* packed, int policy,
                void* stream);
int tcec_sgemm_packed(int layout_c, int m, int n, int k, float alpha, const void* a_packed,
                      const void* b_packed, float beta, float* c, long long ldc, int policy, void* stream);

/*
 * Complex GEMM on interleaved (re, im) float pairs: C = alpha * A * B + beta * C.
 * `a`, `b`, `c` point at the real part of the first element; lda, ldb, ldc count
 * complex elements; alpha and beta are two floats each (re, im), read on the host.
 * No conjugation.  Built, like the reference's complex fragments, from four real
 * error-corrected products (include/wmma_extension/tcec/complex.hpp:646-727:
 * real = Ar Br + Ai (-Bi), imag = Ai Br + Ar Bi; its test is test/tcec/mma_complex.cu);
 * here each part is one real GEMM over the concatenated K of its two products, so the
 * promotion rule sees K' = 2K.  Scratch (operand panels and two m x n planes) comes from
 * the per-stream workspace.
 */
int tcec_cgemm(int layout_a, int layout_b, int layout_c, int m, int n, int k, const float* alpha,
               const float* a, long long lda, const float* b, long long ldb, const float* beta, float* c,
               long long ldc, int policy, void* stream);

/*
 * Element-wise split, exposed so the split can be checked bit for bit:
 *   hi[i] = cast<T>(in[i]);  lo[i] = cast<T>((in[i] - hi[i]) * s)
 * returned widened to float (lo still carries the scale s = 2^11 for fp16, 1 for
 * tf32).  Restates load_matrix_sync's per-element arithmetic
 * (include/wmma_extension/tcec/tcec.hpp:219-223; scale.hpp:8-13).  `lo` may be
 * NULL.  Only the input type of `policy` matters.
 */
int tcec_split(const float* in, float* hi, float* lo, size_t count, int policy, void* stream);

/*
 * Options (process-wide):
 *   "promote_k"  K extent accumulated inside the tensor-core accumulator before
 *                it is added to the FP32 running sum with a round-to-nearest add.
 *                -1 (default) = automatic with error correction: 64 up to K = 2048, 128 up to
 *                4096, 256 below 16384, else 512 (error against the reference kernel on
 *                identical inputs: 0.5-0.9 of its error for zero-mean inputs, 0.8-1.4 for
 *                all-positive ones; the acceptance bound is 2); 0 without error correction.
 *                0 = only at the end, the reference's mma_rz_sync behaviour (include/wmma_extension/tcec/tcec.hpp:773-831);
 *                the reference's mma_rn_sync uses 16 or 8 (:640-706).
 *   "tile_n"     0 = automatic, 128 or 256.
 *   "cta_pair"   256-wide tiles on pairs of SMs (tcgen05 cta_group::2: 256 x 256 tiles, each SM
 *                loads its rows of A and half of B; bit-identical results).  -1 (default) = for
 *                the policies without error correction, where one product per K block leaves the
 *                kernel waiting on operands from L2 and the pair is 10-15 % faster (16384^3
 *                fp16: 812 vs 677-735 TFLOP/s), and with error correction for calls below about
 *                5000^3, which are over before the board reaches its power cap (2048^3: +8 %,
 *                4096^3: +2 %; at the cap the pair draws more power per product and is 5 %
 *                slower); 0 = never; 1 = whenever it applies.
 *   "half_tiles" 1 (default) = a call with so few 256 x 256 tiles that they would leave at least half
 *                of the SM pairs idle runs on 256 x 128 half tiles instead (CTA-pair kernel, N = 128
 *                MMAs; 1024^3: 37 -> 27 us); 0 = whole tiles only.  Same results bit for bit.
 *   "reserve_sms" 0..64 (default 0): SMs the GEMM kernels do not occupy.  Their persistent CTAs take
 *                every register of an SM, so a communication kernel launched beside them can only
 *                run where the GEMM has no CTA.
 *   "comm_sms"   1..64 (default 8): SMs the column-sharded step leaves to the broadcast of A; also
 *                the limit on the broadcast's CTAs (read when a communicator is created).
 *   "comm_panel_rows" rows of A per broadcast in the column-sharded step (default 2048, a multiple
 *                of 256).
 *   "comm_helper" 1 (default) = once the broadcast is over, a second GEMM launch that shares the
 *                first one's tile counter takes the SMs it had; 0 = they stay idle.
 *   "static_tiles" 0 (default) = after the first wave the panel GEMM's CTAs draw their tiles from a
 *                device-wide counter, so a CTA that gets its SM late (another kernel was running
 *                there) processes fewer tiles instead of delaying the launch; 1 = static striding
 *                (CTA i takes tiles i, i + grid, ...).  Same results bit for bit.
 *   "store_turn" 1 (default) = the panel kernel turns its C stores through shared memory into full
 *                128-byte lines and uses all 227 KB of the SM; 0 = direct stores and ~30 KB of
 *                shared memory per SM left free.
 *   "path"       0 = automatic; 1 = always split the operands into panels first, then multiply
 *                (two kernels; the faster one whenever the tensor pipe is the limit); 2 = use
 *                the single kernel that TMA-loads FP32 tiles and splits them in registers
 *                whenever the call allows it (fp16 policies, n > 128, 16-byte aligned operands
 *                with leading dimensions that are multiples of 4, no pointer arrays).
 *                Automatic picks it for batches with k <= 512, which are bound by DRAM traffic.
 */
int tcec_set_option(const char* name, int value);
int tcec_get_option(const char* name, int* value);

/*
 * Synchronises the current device and returns TCEC_ERR_TIMEOUT if any kernel
 * of this library gave up a bounded wait since the last call, else TCEC_OK.
 * `detail`, when not NULL, receives the raw device status word.
 */
int tcec_device_status(int* detail);

/* Bytes of library-owned workspace a call of this shape will use (0 on error). */
size_t tcec_workspace_bytes(int m, int n, int k, int batch, int policy);

/* Frees every cached workspace on every device. */
int tcec_destroy(void);

const char* tcec_status_string(int status);
const char* tcec_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TCEC_H_ */
