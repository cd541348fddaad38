// i4mm_quant_matvec_static: the matvec / few-row multiply for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: a plugin that runs inside a process whose memory
// pool belongs to someone else, a real-time path where an allocation's implicit synchronisation is
// forbidden, a sandbox that only hands out pre-registered buffers.  They still own their inputs and outputs,
// but the split-K scratch the ordinary entry asks for has nowhere to come from.  This entry keeps that scratch
// in a fixed array that is part of the library image itself.
#include "../../include/int4matmul_b200.h"

#include "common.cuh"

namespace i4mm {
cudaError_t stream_launch(int bits, bool sparse, StreamParams p, int total_rows, int ctas, cudaStream_t stream);
}

namespace {

constexpr int kStaticMaxRows = 8;                       // activation rows per call
constexpr int kStaticMaxTiles = 8192;                   // 128-column tiles: S <= 1 048 576
constexpr int kStaticCtas = 148 * 4;                    // same CTA bound as the ordinary entry, so results are identical
constexpr size_t kCountersBytes = (size_t)kStaticMaxTiles * sizeof(unsigned int);
constexpr size_t kStatusBytes = 256;
constexpr size_t kPartialsBytes = (size_t)kStaticCtas * 2 * kStaticMaxRows * 128 * sizeof(float);
constexpr size_t kStaticBytes = kCountersBytes + kStatusBytes + kPartialsBytes;     // 4 882 688 bytes

// Lives in every GPU context that loads the library, from load to exit.  In host code this name is only a
// handle for cudaGetSymbolAddress: it is not a device address and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// Device address of the array, looked up once per device with that device current.
cudaError_t static_scratch_address(unsigned char** out) {
    static unsigned char* addr[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        addr[dev] = static_cast<unsigned char*>(p);
    }
    *out = addr[dev];
    return cudaSuccess;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int i4mm_quant_matvec_static(int bits, int accumulate, void* out, const void* matrix, const void* mask,
                                        const void* x, const void* scales, const void* zeros, int64_t rows, int64_t N,
                                        int64_t S, int64_t n_groups, int64_t group_size, void* stream) {
    if (bits != 4 && bits != 3 && bits != 2) return I4MM_ERR_BITS;
    const bool sparse = mask != nullptr;
    if (sparse && bits != 4) return I4MM_ERR_UNSUPPORTED;
    if (rows < 0 || N <= 0 || S <= 0 || n_groups <= 0) return I4MM_ERR_SHAPE;
    if (N % 64 != 0 || S % 64 != 0 || N > (1 << 30)) return I4MM_ERR_SHAPE;
    if (group_size == 0 || (group_size > 0 && group_size % 64 != 0)) return I4MM_ERR_SHAPE;
    const int64_t g = group_size < 0 ? (int64_t)i4mm::kSingleGroup : group_size;
    if (g * n_groups < N) return I4MM_ERR_SHAPE;
    // the fixed scratch bounds the problem: say so instead of overrunning it
    if (rows > kStaticMaxRows || (S + 127) / 128 > kStaticMaxTiles) return I4MM_ERR_TOO_LARGE;
    if (rows == 0) return I4MM_OK;
    if (!out || !matrix || !x || !scales || !zeros) return I4MM_ERR_NULL;
    if (!aligned16(out) || !aligned16(matrix) || !aligned16(x) || !aligned16(scales) || !aligned16(zeros) ||
        (mask && !aligned16(mask)))
        return I4MM_ERR_ALIGN;

    unsigned char* scratch = nullptr;
    cudaError_t e = static_scratch_address(&scratch);
    if (e != cudaSuccess) { i4mm::record_cuda_error((int)e); return I4MM_ERR_LAUNCH; }

    i4mm::StreamParams p{};
    p.out = (__half*)out;
    p.matrix = (const uint32_t*)matrix;
    p.mask = (const uint32_t*)mask;
    p.x = (const __half*)x;
    p.scales = (const __half*)scales;
    p.zeros = (const __half*)zeros;
    p.N = (int)N;
    p.S = (int)S;
    p.KB = (int)((N + 127) / 128);
    p.CT = (int)((S + 127) / 128);
    p.accumulate = accumulate ? 1 : 0;
    const uint32_t gq = group_size < 0 ? 0u : (uint32_t)(group_size / 64);
    p.gdiv.div = gq;
    p.gdiv.mul = gq >= 2 ? (uint32_t)((1ull << 32) / gq + 1ull) : 0u;
    p.counters = reinterpret_cast<unsigned int*>(scratch);
    p.status = reinterpret_cast<int*>(scratch + kCountersBytes);
    p.partials = reinterpret_cast<float*>(scratch + kCountersBytes + kStatusBytes);

    // The array keeps whatever the last call left.  The arrival counters must start at zero (a call that was cut
    // short could have left them otherwise); the partial sums are overwritten before they are read.  The status
    // word is left alone: a give-up recorded by an earlier call stays visible until i4mm_static_device_status reads it.
    cudaStream_t st = (cudaStream_t)stream;
    e = cudaMemsetAsync(scratch, 0, (size_t)p.CT * sizeof(unsigned int), st);
    if (e == cudaSuccess) e = i4mm::stream_launch(bits, sparse, p, (int)rows, kStaticCtas, st);
    if (e != cudaSuccess) { i4mm::record_cuda_error((int)e); return I4MM_ERR_LAUNCH; }
    return I4MM_OK;
}

// The status word of the fixed scratch: read (and cleared) the same way i4mm_device_status reads a workspace's.
extern "C" int i4mm_static_device_status(void* stream) {
    unsigned char* scratch = nullptr;
    cudaError_t e = static_scratch_address(&scratch);
    int status = 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&status, scratch + kCountersBytes, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess && status != 0) e = cudaMemsetAsync(scratch + kCountersBytes, 0, kStatusBytes, st);
    if (e != cudaSuccess) { i4mm::record_cuda_error((int)e); return I4MM_ERR_LAUNCH; }
    return status == 0 ? I4MM_OK : I4MM_ERR_TIMEOUT;
}
