// Peer-visible buffers and the hand-shake of the gathering multiply (i4mm_quant_matmul_gather).
//
// Every rank (one process per GPU) owns a gathered (rows, S) buffer per matrix and a small array of flags, both
// allocated here with cudaMalloc and exported as CUDA IPC handles; the ranks exchange the handles once (over whatever
// channel the host program has: the Python side uses the existing process group) and open each other's buffers.  The
// multiply's epilogue then stores its columns into every rank's buffer with plain global stores through the peer
// mappings: no collective library runs inside a step, so a whole pass can be one CUDA graph per rank.
//
// i4mm_gather_sync is the hand-shake after such a multiply: it tells every peer "my columns of slot s are written"
// and waits until every peer has said the same.  The wait is bounded: after kGatherSpinLimit polls it records a status
// word and returns, so a rank that never arrives ends in an error status on the others, not in a hung GPU.
// No counterpart in the reference, which has no multi-GPU code.
#include "../../include/int4matmul_b200.h"

#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

namespace {

constexpr unsigned int kGatherSpinLimit = 1u << 22;       // x ~0.5 us per poll: about two seconds

struct PeerFlags {
    unsigned int* flags[i4mm::kMaxDst];                   // flags[r] = rank r's flag array (peer-mapped), [slot][source rank]
};

// One block.  Thread t < world: announce to rank t, then wait for rank t's announcement.
// `epochs` (local, one counter per slot) makes the values differ from call to call without a host-side argument, so the
// kernel can be replayed from a CUDA graph: every rank runs the same sequence of calls, hence the same epochs.
__global__ void gather_sync_kernel(PeerFlags pf, unsigned int* epochs, int* status, int world, int rank, int slot, int slots) {
    __shared__ unsigned int s_epoch;
    // launched with programmatic stream serialization: the kernel after this one may be scheduled at once (it waits for
    // this one itself before it reads anything), and nothing happens here before the multiply has completed
    i4mm::ptx::grid_launch_dependents();
    i4mm::ptx::grid_dependency_wait();
    if (threadIdx.x == 0) s_epoch = ++epochs[slot];
    __syncthreads();
    const unsigned int epoch = s_epoch;
    const int t = threadIdx.x;
    if (t < world) {
        // the multiply before this kernel in the stream has completed, its stores to the peers included; the fence orders
        // them before the flag for an observer on another GPU
        __threadfence_system();
        unsigned int* theirs = pf.flags[t] + (size_t)slot * i4mm::kMaxDst + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
        const unsigned int* mine = pf.flags[rank] + (size_t)slot * i4mm::kMaxDst + t;
        unsigned int seen = 0;
        bool ok = false;
        for (unsigned int i = 0; i < kGatherSpinLimit; ++i) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if ((int)(seen - epoch) >= 0) { ok = true; break; }
            __nanosleep(200);
        }
        if (!ok) atomicExch(status, 41);
    }
    (void)slots;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int fail(cudaError_t e) {
    i4mm::record_cuda_error((int)e);
    return I4MM_ERR_LAUNCH;
}

}  // namespace

extern "C" {

size_t i4mm_ipc_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int i4mm_peer_buffer_create(size_t bytes, void** dev_ptr, void* handle_out) {
    if (!dev_ptr || !handle_out || bytes == 0) return I4MM_ERR_NULL;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        return fail(e);
    }
    memcpy(handle_out, &h, sizeof h);
    *dev_ptr = p;
    return I4MM_OK;
}

int i4mm_peer_buffer_open(const void* handle, void** dev_ptr) {
    if (!handle || !dev_ptr) return I4MM_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(e);
    *dev_ptr = p;
    return I4MM_OK;
}

int i4mm_peer_buffer_close(void* dev_ptr) {
    if (!dev_ptr) return I4MM_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    return e == cudaSuccess ? I4MM_OK : fail(e);
}

int i4mm_peer_buffer_destroy(void* dev_ptr) {
    if (!dev_ptr) return I4MM_OK;
    const cudaError_t e = cudaFree(dev_ptr);
    return e == cudaSuccess ? I4MM_OK : fail(e);
}

size_t i4mm_gather_flags_bytes(int64_t slots) {
    // [slot][source rank] flags, then one epoch counter per slot (local use only)
    return slots <= 0 ? 0 : (size_t)slots * i4mm::kMaxDst * sizeof(unsigned int) + (size_t)slots * sizeof(unsigned int);
}

int i4mm_gather_sync(void* const* flags, int64_t world, int64_t rank, int64_t slot, int64_t slots, void* workspace, void* stream) {
    if (!flags || !workspace) return I4MM_ERR_NULL;
    if (world < 1 || world > i4mm::kMaxDst || rank < 0 || rank >= world || slot < 0 || slot >= slots) return I4MM_ERR_SHAPE;
    PeerFlags pf{};
    for (int r = 0; r < world; ++r) {
        if (!flags[r]) return I4MM_ERR_NULL;
        pf.flags[r] = (unsigned int*)flags[r];
    }
    unsigned int* epochs = pf.flags[rank] + (size_t)slots * i4mm::kMaxDst;
    int* status = (int*)((char*)workspace + 256 * 1024 - 64);      // the workspace's status word (see i4mm_device_status)
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3(1, 1, 1);
    cfg.blockDim = dim3(32, 1, 1);
    cfg.stream = (cudaStream_t)stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gather_sync_kernel, pf, epochs, status, (int)world, (int)rank, (int)slot, (int)slots);
    if (e != cudaSuccess) return fail(e);
    i4mm::count_launch();
    return I4MM_OK;
}

}  // extern "C"
