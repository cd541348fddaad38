// extern "C" entry points of libint4matmul_b200.so: argument validation, path choice, launches.
// The declarations and the reference interfaces they replace are in include/int4matmul_b200.h.
#include "../../include/int4matmul_b200.h"

#include <atomic>

#include "common.cuh"

namespace i4mm {
static std::atomic<unsigned long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n); }
static thread_local int g_last_cuda_error = 0;        // what i4mm_last_cuda_error returns; every entry point records here
void record_cuda_error(int e) { g_last_cuda_error = e; }
int umma_last_shape();
void umma_clear_last_shape();
cudaError_t stream_launch(int bits, bool sparse, StreamParams p, int total_rows, int ctas, cudaStream_t stream);
cudaError_t sparse_pack_launch(void* wt_out, void* msk_out, const void* wt_in, const void* msk_in,
                               int S, int N, void* violations, cudaStream_t stream);
cudaError_t check_mask_launch(const void* mask, size_t count, void* violations, cudaStream_t stream);
cudaError_t rownorm_launch(int mode, void* y, const void* a, const void* b, const void* c, long long rows, int width,
                           long long sa, long long sb, long long sc, cudaStream_t stream);
int umma_launch(int bits, bool sparse, const StreamParams& p, int total_rows, int n_groups, int group_size, int cta_pairs,
                int force_nt, int overlap, cudaStream_t stream, cudaError_t* cuda_err);
bool umma_supported(int bits, bool sparse, int total_rows, int N, int S);
}  // namespace i4mm

namespace {

constexpr size_t kCounterBytes = 256 * 1024;          // column-tile counters; the last 64 bytes hold the status word
constexpr size_t kStatusOffset = kCounterBytes - 64;
constexpr int kMaxStreamCtas = 148 * 4;               // upper bound on the CTAs of the streaming kernel (sizes the scratch)
constexpr size_t kPartialBytes = (size_t)kMaxStreamCtas * 2 * 32 * 128 * sizeof(float);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int fail_cuda(cudaError_t e) {
    i4mm::record_cuda_error((int)e);
    return I4MM_ERR_LAUNCH;
}

}  // namespace

extern "C" {

const char* i4mm_status_string(int status) {
    switch (status) {
        case I4MM_OK: return "ok";
        case I4MM_ERR_BITS: return "unsupported bit width (must be 4, 3 or 2)";
        case I4MM_ERR_UNSUPPORTED: return "unsupported combination (16:32 sparsity is defined for int4 only)";
        case I4MM_ERR_SHAPE: return "shape rule violated";
        case I4MM_ERR_NULL: return "required pointer is null";
        case I4MM_ERR_ALIGN: return "pointer is not 16-byte aligned";
        case I4MM_ERR_WORKSPACE: return "workspace missing or too small";
        case I4MM_ERR_LAUNCH: return "CUDA launch error";
        case I4MM_ERR_MASK: return "16:32 keep-mask violated";
        case I4MM_ERR_DEVICE: return "device or driver not usable (needs sm_100)";
        case I4MM_ERR_TIMEOUT: return "device-side bounded wait timed out";
        case I4MM_ERR_TOO_LARGE: return "problem exceeds the fixed scratch of the allocation-free entry (rows <= 8, S <= 1048576)";
        default: return "unknown status";
    }
}

int i4mm_last_cuda_error(void) { return i4mm::g_last_cuda_error; }

int i4mm_last_launch_shape(void) { return i4mm::umma_last_shape(); }

int i4mm_version(void) { return 100; }

unsigned long long i4mm_launch_count(void) { return i4mm::g_launches.load(); }

size_t i4mm_workspace_bytes(void) { return kCounterBytes + kPartialBytes; }

}  // extern "C"

namespace {

// The multiply behind both entries.  gather == nullptr: results go to `out` (rows, S).
int multiply(int bits, int accumulate, int path, void* out, const i4mm::OutMap* gather, const void* matrix, const void* mask,
             const void* x, const void* scales, const void* zeros, int64_t rows, int64_t N, int64_t S, int64_t n_groups,
             int64_t group_size, void* workspace, size_t workspace_bytes, void* stream) {
    if (bits != 4 && bits != 3 && bits != 2) return I4MM_ERR_BITS;
    const bool sparse = mask != nullptr;
    if (sparse && bits != 4) return I4MM_ERR_UNSUPPORTED;
    if (rows < 0 || N <= 0 || S <= 0 || n_groups <= 0) return I4MM_ERR_SHAPE;
    if (N % 64 != 0 || S % 64 != 0) return I4MM_ERR_SHAPE;                 // matmul_kernel.cu:416 and the 64-row K tile
    if (N > (1 << 30) || S > (int64_t)128 * 65000 || rows > (1 << 30)) return I4MM_ERR_SHAPE;
    if (group_size == 0 || (group_size > 0 && group_size % 64 != 0)) return I4MM_ERR_SHAPE;   // matmul_kernel.cu:383
    const int64_t g = group_size < 0 ? (int64_t)i4mm::kSingleGroup : group_size;           // matmul_kernel.cu:379-381
    if (g * n_groups < N) return I4MM_ERR_SHAPE;                                               // matmul_kernel.cu:414-415
    if (rows == 0) return I4MM_OK;
    if (!out || !matrix || !x || !scales || !zeros) return I4MM_ERR_NULL;
    if (!aligned16(out) || !aligned16(matrix) || !aligned16(x) || !aligned16(scales) || !aligned16(zeros) ||
        (mask && !aligned16(mask)))
        return I4MM_ERR_ALIGN;
    // bits 8.. of `path`: rows per tile to use on the tcgen05 path instead of the choice by shape (tests, tuning)
    const int overlap = path >= 0 ? (path >> 20) & 1 : 0;         // I4MM_PATH_STATIC_WEIGHTS
    const int force_nt = path >= 0 ? (path >> 8) & 0xFFF : 0;
    if (path >= 0) path &= 0xFF;
    if (path < 0 || path > 3) return I4MM_ERR_SHAPE;
    if (force_nt != 0) {
        const bool known = force_nt == 16 || force_nt == 32 || force_nt == 64 || force_nt == 128 || force_nt == 160 ||
                           force_nt == 192 || force_nt == 224 || force_nt == 256;
        // the few-row tiles reduce split-K partial tiles of one row tile only
        if (!known || path < 2 || (force_nt <= 64 && rows > force_nt)) return I4MM_ERR_SHAPE;
    }

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
    p.gdiv.mul = gq >= 2 ? (uint32_t)((1ull << 32) / gq + 1ull) : 0u;    // gq == 0: one group -> index 0
    if (gather) {
        p.om = *gather;
    } else {
        p.om.dst[0] = (__half*)out;
        p.om.n_dst = 1;
        p.om.part_cols = (int)S;
        p.om.ld = S;
        p.om.part_stride = 0;
        p.om.base = 0;
    }

    if (!workspace || workspace_bytes < i4mm_workspace_bytes()) return I4MM_ERR_WORKSPACE;
    if (!aligned16(workspace)) return I4MM_ERR_ALIGN;
    p.counters = (unsigned int*)workspace;
    p.partials = (float*)((char*)workspace + kCounterBytes);
    p.status = (int*)((char*)workspace + kStatusOffset);

    cudaStream_t st = (cudaStream_t)stream;
    bool use_umma = false;
    if (path >= 2 || gather) {
        if (!i4mm::umma_supported(bits, sparse, (int)rows, (int)N, (int)S)) return I4MM_ERR_UNSUPPORTED;
        use_umma = true;
    } else if (path == 0) {
        use_umma = i4mm::umma_supported(bits, sparse, (int)rows, (int)N, (int)S);
    }
    if (use_umma) {
        cudaError_t ce = cudaSuccess;
        const int rc = i4mm::umma_launch(bits, sparse, p, (int)rows, (int)n_groups, (int)(group_size < 0 ? -1 : group_size), path == 3 ? 1 : 0, force_nt, overlap, st, &ce);
        if (rc == I4MM_ERR_LAUNCH) return fail_cuda(ce);
        return rc;
    }
    i4mm::umma_clear_last_shape();
    const cudaError_t e = i4mm::stream_launch(bits, sparse, p, (int)rows, kMaxStreamCtas, st);
    if (e != cudaSuccess) return fail_cuda(e);
    return I4MM_OK;
}

}  // namespace

extern "C" {

int i4mm_quant_matmul(int bits, int accumulate, int path,
                      void* out, const void* matrix, const void* mask,
                      const void* x, const void* scales, const void* zeros,
                      int64_t rows, int64_t N, int64_t S, int64_t n_groups, int64_t group_size,
                      void* workspace, size_t workspace_bytes, void* stream) {
    return multiply(bits, accumulate, path, out, nullptr, matrix, mask, x, scales, zeros, rows, N, S, n_groups, group_size,
                    workspace, workspace_bytes, stream);
}

int i4mm_quant_matmul_gather(int bits, int path, void* const* gathered, int n_gathered, int64_t ld, int64_t parts,
                             int64_t rank, int64_t world, const void* matrix, const void* mask, const void* x,
                             const void* scales, const void* zeros, int64_t rows, int64_t N, int64_t S, int64_t n_groups,
                             int64_t group_size, void* workspace, size_t workspace_bytes, void* stream) {
    if (!gathered || n_gathered < 1 || n_gathered > i4mm::kMaxDst) return I4MM_ERR_SHAPE;
    if (parts < 1 || world < 1 || rank < 0 || rank >= world || S <= 0 || S % parts != 0) return I4MM_ERR_SHAPE;
    const int64_t part_cols = S / parts;                       // this shard's columns of one part
    if (part_cols % 64 != 0 || ld < S * world || ld % 8 != 0) return I4MM_ERR_SHAPE;
    i4mm::OutMap om{};
    for (int d = 0; d < n_gathered; ++d) {
        if (!gathered[d]) return I4MM_ERR_NULL;
        if (!aligned16(gathered[d])) return I4MM_ERR_ALIGN;
        om.dst[d] = (__half*)gathered[d];
    }
    om.n_dst = n_gathered;
    om.part_cols = (int)part_cols;
    om.ld = ld;
    om.part_stride = part_cols * world;
    om.base = rank * part_cols;
    if ((path & 0xFF) == 1) return I4MM_ERR_UNSUPPORTED;      // the streaming kernel has no gathering epilogue
    return multiply(bits, 0, path, gathered[0], &om, matrix, mask, x, scales, zeros, rows, N, S, n_groups, group_size,
                    workspace, workspace_bytes, stream);
}

int i4mm_device_status(void* workspace, void* stream) {
    if (!workspace) return I4MM_ERR_NULL;
    int status = 0;
    cudaError_t e = cudaMemcpyAsync(&status, (char*)workspace + kStatusOffset, sizeof(int), cudaMemcpyDeviceToHost,
                                    (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return fail_cuda(e);
    if (status == 0) return I4MM_OK;
    e = cudaMemsetAsync((char*)workspace + kStatusOffset, 0, sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return fail_cuda(e);
    return I4MM_ERR_TIMEOUT;
}

int i4mm_row_norm(int mode, void* y, const void* a, const void* b, const void* c, int64_t rows, int64_t width,
                  int64_t stride_a, int64_t stride_b, int64_t stride_c, void* stream) {
    if (mode < 0 || mode > 4 || rows < 0 || width <= 0 || width % 2 != 0 || width > (1 << 30) || rows > (1ll << 31) - 1)
        return I4MM_ERR_SHAPE;
    if (rows == 0) return I4MM_OK;
    if (!y || !a || (mode != 0 && !b) || (mode == 1 && !c)) return I4MM_ERR_NULL;
    if ((stride_a | stride_b | stride_c) & 1) return I4MM_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
         reinterpret_cast<uintptr_t>(c)) & 3u)
        return I4MM_ERR_ALIGN;
    const cudaError_t e = i4mm::rownorm_launch(mode, y, a, b, c, rows, (int)width, stride_a, stride_b, stride_c,
                                               (cudaStream_t)stream);
    if (e != cudaSuccess) return fail_cuda(e);
    return I4MM_OK;
}

int i4mm_sparse_pack(void* wt_out, void* msk_out, const void* wt_in, const void* msk_in,
                     int64_t S, int64_t N, void* violations, void* stream) {
    // utils_kernel.cu:101; S is walked by the grid's y dimension in steps of 32 columns (at most 65535 of them)
    if (S < 0 || N < 0 || N % 32 != 0 || N > (1 << 30) || S > 65535 * 32) return I4MM_ERR_SHAPE;
    if (S == 0 || N == 0) return I4MM_OK;
    if (!wt_out || !msk_out || !wt_in || !msk_in) return I4MM_ERR_NULL;
    if (!aligned16(wt_in) || !aligned16(msk_in) || !aligned16(wt_out) || !aligned16(msk_out)) return I4MM_ERR_ALIGN;
    const cudaError_t e = i4mm::sparse_pack_launch(wt_out, msk_out, wt_in, msk_in, (int)S, (int)N, violations,
                                                   (cudaStream_t)stream);
    if (e != cudaSuccess) return fail_cuda(e);
    return I4MM_OK;
}

int i4mm_check_mask(const void* mask, int64_t N, int64_t S, void* violations, void* stream) {
    if (S < 0 || N < 0 || N % 32 != 0) return I4MM_ERR_SHAPE;
    if (S == 0 || N == 0) return I4MM_OK;
    if (!mask || !violations) return I4MM_ERR_NULL;
    const cudaError_t e = i4mm::check_mask_launch(mask, (size_t)(N / 32) * (size_t)S, violations, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail_cuda(e);
    return I4MM_OK;
}

}  // extern "C"
