// 16:32 sparse packer and keep-mask checker.
//
// Replaces PackMatrix (utils_kernel.cu:19-64).  Same outputs bit for bit; differences in how it gets there:
// one lane owns a whole 32-block of one column (reads its 32 weight bytes and 32 mask bytes as two pairs of
// 16-byte loads) instead of one lane per weight with ballot + 64-bit shuffles, the transposed stores are
// staged through shared memory so both sides of the transpose are coalesced, and a block that does not keep
// exactly 16 weights bumps a counter instead of trapping the device.
#include "common.cuh"

namespace i4mm {

namespace {

constexpr int kPackCols = 32;   // S columns per CTA
constexpr int kPackBlks = 8;    // 32-blocks of N per CTA

__global__ void __launch_bounds__(kPackCols * kPackBlks)
sparse_pack_kernel(uint32_t* __restrict__ wt_out, uint32_t* __restrict__ msk_out,
                   const uint8_t* __restrict__ wt_in, const uint8_t* __restrict__ msk_in,
                   int S, int N, int* __restrict__ violations) {
    __shared__ uint32_t sm_lo[kPackBlks][kPackCols + 1], sm_hi[kPackBlks][kPackCols + 1], sm_m[kPackBlks][kPackCols + 1];
    const int nblk = N / 32;
    // load phase: thread (blk_l, s_l) with blk fastest, so a warp reads 8 blocks x 32 B = 256 contiguous bytes per row
    const int blk_l = threadIdx.x % kPackBlks, s_l = threadIdx.x / kPackBlks;
    const int blk = blockIdx.x * kPackBlks + blk_l, s = blockIdx.y * kPackCols + s_l;
    if (blk < nblk && s < S) {
        const uint4* wp = reinterpret_cast<const uint4*>(wt_in + (size_t)s * N + (size_t)blk * 32);
        const uint4* mp = reinterpret_cast<const uint4*>(msk_in + (size_t)s * N + (size_t)blk * 32);
        const uint4 w0 = wp[0], w1 = wp[1], m0 = mp[0], m1 = mp[1];
        const uint32_t wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const uint32_t mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        uint32_t mask = 0;
        unsigned long long word = 0;
        int rank = 0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const uint32_t keep = ((mv[i >> 2] >> (8 * (i & 3))) & 0xFFu) ? 1u : 0u;   // msk_in > 0 (utils_kernel.cu:34)
            const unsigned long long nib = (wv[i >> 2] >> (8 * (i & 3))) & 0xFu;        // low nibble (utils_kernel.cu:49)
            mask |= keep << i;
            if (keep && rank < 16) word |= nib << (4 * rank);
            rank += keep;
        }
        if (rank != 16 && violations) atomicAdd(violations, 1);
        sm_lo[blk_l][s_l] = (uint32_t)word;
        sm_hi[blk_l][s_l] = (uint32_t)(word >> 32);
        sm_m[blk_l][s_l] = mask;
    }
    __syncthreads();
    // store phase: thread (s fastest) so a warp writes 32 contiguous words of one output row
    const int s_o = threadIdx.x % kPackCols, blk_o = threadIdx.x / kPackCols;
    const int blk2 = blockIdx.x * kPackBlks + blk_o, s2 = blockIdx.y * kPackCols + s_o;
    if (blk2 < nblk && s2 < S) {
        wt_out[(size_t)(2 * blk2) * S + s2] = sm_lo[blk_o][s_o];
        wt_out[(size_t)(2 * blk2 + 1) * S + s2] = sm_hi[blk_o][s_o];
        msk_out[(size_t)blk2 * S + s2] = sm_m[blk_o][s_o];
    }
}

__global__ void check_mask_kernel(const uint32_t* __restrict__ mask, size_t count, int* __restrict__ violations) {
    int bad = 0;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        bad += (__popc(mask[i]) != 16);
    bad = __reduce_add_sync(0xFFFFFFFFu, bad);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(violations, bad);
}

}  // namespace

cudaError_t sparse_pack_launch(void* wt_out, void* msk_out, const void* wt_in, const void* msk_in,
                               int S, int N, void* violations, cudaStream_t stream) {
    const int nblk = N / 32;
    if (nblk == 0 || S == 0) return cudaSuccess;
    dim3 grid((nblk + kPackBlks - 1) / kPackBlks, (S + kPackCols - 1) / kPackCols);
    sparse_pack_kernel<<<grid, kPackCols * kPackBlks, 0, stream>>>(
        (uint32_t*)wt_out, (uint32_t*)msk_out, (const uint8_t*)wt_in, (const uint8_t*)msk_in, S, N, (int*)violations);
    count_launch();
    return cudaGetLastError();
}

cudaError_t check_mask_launch(const void* mask, size_t count, void* violations, cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    const int threads = 256;
    size_t blocks = (count + threads - 1) / threads;
    if (blocks > 148 * 8) blocks = 148 * 8;
    check_mask_kernel<<<(int)blocks, threads, 0, stream>>>((const uint32_t*)mask, count, (int*)violations);
    count_launch();
    return cudaGetLastError();
}

}  // namespace i4mm
