/*
 * C ABI of the B200 (sm_100a) quantized matvec / matmul library: libint4matmul_b200.so.
 *
 * This is the boundary a foreign-function binding attaches to.  Everything is plain pointers and
 * sizes; all data pointers are DEVICE pointers on the current CUDA device; nothing here allocates
 * device memory unless the entry says so (only i4mm_peer_buffer_create does); every launch goes onto the stream passed in (a
 * cudaStream_t cast to void*, NULL = the legacy default stream the reference launches on).
 * Calls return an i4mm_status; they never abort the process and never trap the device.
 *
 * Tensor contract (identical to the reference's torch extension, int4matmul.cpp:26-48):
 *   x       fp16  (rows, N)          rows = B*M flattened, N = in-features (reduction dim)
 *   matrix  int32 (R, S)             packed weights, S = out-features contiguous;
 *                                    dense: R = N*bits/32; 16:32 sparse int4: R = N/16
 *   mask    int32 (N/32, S) or NULL  16:32 keep-mask, bit l of [b, s] = keep(n = 32b+l, s)
 *   scales  fp16  (n_groups, S)      scale >= 0: W = (q - zero) * scale, both steps rounded to fp16
 *   zeros   fp16  (n_groups, S)      scale <  0: W = fma(+-2^(q & (2^(bits-1)-1)), -scale, zero)
 *   out     fp16  (rows, S)
 *   group_size  positive multiple of 64, or negative for "one group over all of N"
 *   N, S multiples of 64.  sparse is only defined for bits == 4.
 */
#ifndef INT4MATMUL_B200_H
#define INT4MATMUL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum i4mm_status {
    I4MM_OK = 0,
    I4MM_ERR_BITS = 1,         /* bits not in {4, 3, 2}          (int4matmul.cpp:35, 45) */
    I4MM_ERR_UNSUPPORTED = 2,  /* sparse with int3 / int2         (matmul.cuh:188, 331 trap in the reference) */
    I4MM_ERR_SHAPE = 3,        /* a size rule of matmul_kernel.cu:383, 404-416 is violated */
    I4MM_ERR_NULL = 4,         /* a required pointer is NULL */
    I4MM_ERR_ALIGN = 5,        /* a pointer is not 16-byte aligned */
    I4MM_ERR_WORKSPACE = 6,    /* workspace missing or smaller than i4mm_workspace_bytes() */
    I4MM_ERR_LAUNCH = 7,       /* CUDA reported an error at launch; see i4mm_last_cuda_error() */
    I4MM_ERR_MASK = 8,         /* a 32-block of the keep-mask does not hold exactly 16 entries */
    I4MM_ERR_DEVICE = 9,       /* device is not sm_100 or a driver entry point is unavailable */
    I4MM_ERR_TIMEOUT = 10,     /* a bounded device-side wait gave up (status word set by the kernel) */
    I4MM_ERR_TOO_LARGE = 11    /* the problem exceeds the fixed scratch of i4mm_quant_matvec_static */
} i4mm_status;

/* Human-readable name of a status code. */
const char* i4mm_status_string(int status);
/* The cudaError_t (as int) recorded by the last call that returned I4MM_ERR_LAUNCH on this thread. */
int i4mm_last_cuda_error(void);
/* Library version: major*10000 + minor*100 + patch. */
int i4mm_version(void);
/* Kernels this library has launched in this process so far, over all entry points (a multiply is one launch,
 * or two where it cuts K into parts and reduces them).  For accounting in benchmarks; no reference counterpart. */
unsigned long long i4mm_launch_count(void);
/* What the last i4mm_quant_matmul call of this host thread launched on the tcgen05 path: rows per tile (the MMA's N:
 * 16, 32, 64, 128, 160, 192, 224 or 256) + 1000 if it ran as CTA pairs + 10000 * K parts; 0 after a call that took the
 * streaming path.  For tests that must know which kernel instance they exercised; no reference counterpart. */
int i4mm_last_launch_shape(void);

/*
 * Bytes of device scratch the two multiply entries need.  The scratch holds the per-CTA partial tiles
 * of the split-K reduction (tagged words on the tcgen05 path, plus arrival counters on the streaming
 * path) and a status word.  It must be zero-filled once before its first use; the kernels leave it
 * all-zero again when they finish, so one buffer can serve every later call on the same stream.
 * Calls that overlap on the device must not share a buffer.  After a call for which
 * i4mm_device_status reported I4MM_ERR_TIMEOUT, zero the buffer again before reusing it.
 */
size_t i4mm_workspace_bytes(void);

/*
 * out[r, s] (+)= sum_n x[r, n] * W16[n, s], fp32 accumulation, one rounding to fp16.
 *
 * Replaces matvec_packed_int<bits> / MVA_Int4_Half (matvec_kernel.cu:302-383, 198-267) and
 * matmul_packed_int<bits> / MMA_Int4_Half (matmul_kernel.cu:375-459, 219-333).
 *
 *   accumulate != 0  ->  out = half(float(out) + x.W): what the reference's matvec route does to the
 *                        caller's `outs` (matvec_kernel.cu:351, 263, 381-382)
 *   accumulate == 0  ->  out is overwritten, as the reference's matmul route does (matmul_kernel.cu:299-332)
 *
 * rows = B*M may be any value >= 0 (rows == 0 returns I4MM_OK without a launch).  The entry picks the
 * weight-streaming kernel for few rows and the tcgen05 tensor-core kernel for many; `path` forces one:
 *   0 = automatic (the tcgen05 kernel when the driver's tensor-map encoder is found), 1 = streaming (mma.sync,
 *   split-K over the whole GPU), 2 = tcgen05 / TMEM pipeline (128 rows or more run as CTA pairs, two SMs per
 *   MMA), 3 = tcgen05 with single CTAs only.
 *   With path 2 or 3, `path | (T << 8)` also fixes the rows per tile (the MMA's N) to T in {16, 32, 64, 128, 160, 192,
 *   224, 256} instead of choosing it by shape (T >= 128 with path 2 runs as CTA pairs; T <= 64 needs rows <= T):
 *   for tests and tuning, results do not depend on it beyond fp32 summation order.
 *   `path | I4MM_PATH_STATIC_WEIGHTS` is the caller's promise that matrix, mask, scales and zeros are not written by
 *   the kernel that precedes this call in the stream (weights of a loaded model never are).  The tcgen05 kernel is then
 *   launched so that its set-up and its first weight copies overlap the tail of that kernel (programmatic dependent
 *   launch); it still waits for that kernel before it reads x, reads or writes out, or touches the workspace.  Without
 *   the flag every launch is ordered after the whole preceding kernel, as the reference's launches are.
 */
#define I4MM_PATH_STATIC_WEIGHTS 0x100000
int i4mm_quant_matmul(int bits, int accumulate, int path,
                      void* out, const void* matrix, const void* mask /* NULL = dense */,
                      const void* x, const void* scales, const void* zeros,
                      int64_t rows, int64_t N, int64_t S, int64_t n_groups, int64_t group_size,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * The multiply of one rank of a column-sharded matrix, with the all-gather of the outputs done by the kernel's own
 * stores.  No counterpart in the reference (which has no multi-GPU code); it serves the layer-stack configuration,
 * where every matrix is sharded along S over the GPUs of one node and the next matrix needs all of S.
 *
 *   matrix, mask, scales, zeros   this rank's shard: S columns = `parts` pieces of S / parts columns each, piece j being
 *                                 this rank's columns of the j-th matrix of a concatenation (q | k | v, gate | up; 1 = one matrix)
 *   gathered[0 .. n_gathered)     (rows, ld) fp16 buffers, normally one per rank (this rank's own and the peers', opened
 *                                 with i4mm_peer_buffer_open); the result is stored into every one of them, local column
 *                                 c of piece j at column j * (S / parts) * world + rank * (S / parts) + c
 *   ld >= S * world, a multiple of 8.  Always overwrites (no accumulate); tcgen05 kernel only (path 0, 2 or 3).
 * The stores are plain global stores through the peer mappings; i4mm_gather_sync afterwards tells the peers and waits
 * for them.  A buffer may be written again only after another i4mm_gather_sync has passed since its readers ran.
 */
int i4mm_quant_matmul_gather(int bits, int path, void* const* gathered, int n_gathered, int64_t ld, int64_t parts,
                             int64_t rank, int64_t world, const void* matrix, const void* mask /* NULL = dense */,
                             const void* x, const void* scales, const void* zeros,
                             int64_t rows, int64_t N, int64_t S, int64_t n_groups, int64_t group_size,
                             void* workspace, size_t workspace_bytes, void* stream);

/*
 * Device buffers that other processes of the node can map (CUDA IPC), for i4mm_quant_matmul_gather.
 *   create   cudaMalloc + zero-fill + export: *dev_ptr = the buffer, handle_out = i4mm_ipc_handle_bytes() bytes to send to the peers
 *   open     map a peer's buffer from its handle (peer access is enabled on first use); close unmaps it
 *   destroy  frees a buffer made by create (after the peers have closed it)
 * These four and nothing else in the library allocate or free device memory.
 */
size_t i4mm_ipc_handle_bytes(void);
int i4mm_peer_buffer_create(size_t bytes, void** dev_ptr, void* handle_out);
int i4mm_peer_buffer_open(const void* handle, void** dev_ptr);
int i4mm_peer_buffer_close(void* dev_ptr);
int i4mm_peer_buffer_destroy(void* dev_ptr);

/*
 * Hand-shake after a gathering multiply.  Every rank has a flags buffer of i4mm_gather_flags_bytes(slots) bytes made
 * with i4mm_peer_buffer_create (zero-filled) and opened by the peers; flags[r] = rank r's buffer as seen from here
 * (flags[rank] = the local one).  The call enqueues one small kernel that, for slot `slot` (one slot per gathered
 * buffer that is in flight at a time), tells every rank that this rank's stores are done and waits until every rank has
 * said the same.  All ranks must issue the same sequence of calls.  The values exchanged advance by themselves on the
 * device, so the call can be captured in a CUDA graph and replayed.  The wait is bounded (about two seconds): a peer
 * that never arrives sets the status word of `workspace` (see i4mm_device_status) instead of hanging the GPU.
 */
size_t i4mm_gather_flags_bytes(int64_t slots);
int i4mm_gather_sync(void* const* flags, int64_t world, int64_t rank, int64_t slot, int64_t slots, void* workspace, void* stream);

/*
 * The same multiply as i4mm_quant_matmul on its streaming path, for callers that cannot allocate device
 * memory (no cudaMalloc available to them: code running inside someone else's memory pool, inside a
 * latency-critical loop where an allocation would synchronise the device, or in a sandbox that only hands out
 * buffers registered up front).  The caller passes inputs and outputs as usual and NO workspace: the split-K
 * scratch is a fixed 4 882 688-byte array inside the library image, held by every GPU context that loads the
 * library until the process exits.  This entry has no counterpart in the reference.
 *
 *   limits   rows <= 8 and S <= 1 048 576; anything larger returns I4MM_ERR_TOO_LARGE and launches nothing
 *   set-up   the first call on each device looks up the array's device address (cudaGetSymbolAddress) and
 *            configures the kernel; make that first call before any stream capture begins
 *   sharing  every call on a device uses the same array, which keeps the previous call's contents; the entry
 *            clears the counters it needs (one small memset on `stream`) before launching.  Two calls that
 *            overlap on the GPU (different streams, or different host threads) race on it: serialise them.
 *   It calls no cudaMalloc, cudaFree or any allocating library routine.  Results are identical to
 *   i4mm_quant_matmul(path = 1) on the same inputs.
 */
int i4mm_quant_matvec_static(int bits, int accumulate,
                             void* out, const void* matrix, const void* mask /* NULL = dense */,
                             const void* x, const void* scales, const void* zeros,
                             int64_t rows, int64_t N, int64_t S, int64_t n_groups, int64_t group_size, void* stream);

/*
 * Waits for the stream and reports whether a kernel that used `workspace` gave up on one of its bounded
 * device-side waits (every wait on a shared-memory barrier inside the kernels has a poll limit, after which
 * the kernel records a status word in the workspace and returns instead of spinning).  Returns I4MM_OK, or
 * I4MM_ERR_TIMEOUT after clearing the word.  No counterpart in the reference, whose kernels have no waits.
 */
int i4mm_device_status(void* workspace, void* stream);
/* The same check for i4mm_quant_matvec_static, whose status word lives in the library's fixed scratch on the
 * current device: waits for the stream, returns I4MM_OK or (after clearing the word) I4MM_ERR_TIMEOUT. */
int i4mm_static_device_status(void* stream);

/*
 * 16:32 packer.  Replaces sparse_int4_pack / PackMatrix (utils_kernel.cu:67-119, 19-64).
 *   wt_in, msk_in  uint8 (S, N): low nibble of wt_in is the weight, msk_in > 0 means keep
 *   wt_out int32 (N/16, S), msk_out int32 (N/32, S)
 *   violations     optional device int32; incremented once per 32-block that does not keep exactly
 *                  16 entries (the reference device-asserts instead, utils_kernel.cu:41).  May be NULL.
 */
int i4mm_sparse_pack(void* wt_out, void* msk_out, const void* wt_in, const void* msk_in,
                     int64_t S, int64_t N, void* violations, void* stream);

/*
 * Counts the 32-blocks of an already packed keep-mask (N/32, S) whose popcount is not 16 into the
 * device int32 *violations (which the caller zeroes).  No counterpart in the reference, which trusts
 * the mask; offered so callers can validate foreign masks without a device trap.
 */
int i4mm_check_mask(const void* mask, int64_t N, int64_t S, void* violations, void* stream);

/*
 * Row-wise glue of the layer-stack runner: y[r, :] = v / rms(v) per row, computed in fp32, with
 *   mode 0: v = a     mode 1: v = a + b + c     mode 2: v = a + b / rms(b)     mode 3: v = a * b
 *   mode 4: mode 2 into y[0 : rows*width], then mode 0 of that (rounded) result into y[rows*width : 2*rows*width]
 *           (a layer's residual stream and the next layer's normalised input from one launch)
 * a, b, c fp16 (rows, width) with row strides in elements (column slices of a gathered buffer are fine);
 * y fp16 (rows, width) contiguous ((2, rows, width) in mode 4); width even; pointers 4-byte aligned.  No counterpart in the reference
 * (it has no model code): it replaces the handful of eager elementwise kernels between two quantized linears.
 */
int i4mm_row_norm(int mode, void* y, const void* a, const void* b, const void* c, int64_t rows, int64_t width,
                  int64_t stride_a, int64_t stride_b, int64_t stride_c, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INT4MATMUL_B200_H */
