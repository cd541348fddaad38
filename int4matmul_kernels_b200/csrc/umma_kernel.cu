// Tensor-core path: tcgen05.mma with the dequantised weights as the A operand in tensor memory.
//
// Replaces MMA_Int4_Half (matmul_kernel.cu:219-333) and, for one or a few activation rows, MVA_Int4_Half
// (matvec_kernel.cu:198-267).  Per CTA tile: 128 weight columns (S) on the 128 tensor-memory lanes x NT
// activation rows on the MMA's N dimension, accumulated in fp32 in tensor memory over all of N (in-features).
//
//   weight producer   one thread (two, in two warps, for the weight-streaming shapes): tensor-map copies (TMA) of the
//                     packed weight rows, the keep mask and the groups' scales / zeros of one unit (128 k; 256 k for
//                     the weight-streaming shapes) into a shared-memory ring
//   activation prod.  one thread: the activation tile (NT rows x one unit of k as 128-byte-swizzled sub-tiles of 64 k);
//                     for dense int4 weight streaming the whole warp, which reorders k inside the tile (see UFormat)
//   dequant warps     warpgroups of 4 warps take the units in turn; thread i of a group owns weight column i: reads
//                     its packed words from shared memory, rebuilds fp16((q - zero) * scale) in registers and
//                     writes them into its own tensor-memory lane with tcgen05.st (one packed int32 = 8 consecutive
//                     k of one column, which is exactly what a lane of the A operand holds)
//   MMA warp          one elected thread issues 8 (16) x tcgen05.mma (M = 128, N = NT, K = 16) per unit, A from tensor
//                     memory, B from the swizzled shared-memory tile, and commits to mbarriers that recycle the
//                     stages; the accumulator never leaves tensor memory until the tile is done
//   epilogue          4 warps read the accumulator (tcgen05.ld), convert to fp16 and store; a warpgroup of its own
//                     except for 33..64 rows, where dequant warpgroup 0 does it
//
// Configurations (Cfg<NT, PAIR>): NT <= 32 rows stream the weights once from HBM - one CTA per SM, 3 dequant warpgroups,
// 9 weight stages and 3 A / activation stages of 256 k, and the (tile, unit) space cut into equal ranges per CTA
// (split-K over the whole GPU, partial tiles summed through scratch in a fixed order).  NT = 64: two CTAs per SM, whole tiles.
// NT >= 128: one CTA per SM, whole tiles, epilogue stores transposed through shared memory; by default launched as
// clusters of two CTAs that run each MMA together (cta_group::2, M = 256 over two SMs), see PAIR below.
// Every wait is bounded and reports through the status word instead of hanging.
#include "../../include/int4matmul_b200.h"

#include <cuda.h>
#include <dlfcn.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace i4mm {

namespace {


enum : int { MODE_FAST = 0, MODE_GENERAL = 1, MODE_SLOW = 2 };


struct UmmaParams {
    OutMap om;           // where the results go (one array, or this rank's columns of several gathered arrays)
    const uint32_t* matrix;
    const uint32_t* mask;
    const __half* scales;
    const __half* zeros;
    float* partials;
    int* status;
    int rows;            // all activation rows (B * M)
    int N, S;
    int U;               // 128-k units per tile: ceil(N / 128)
    int CT;              // column tiles: ceil(S / 128)
    int MTILES;          // row tiles: ceil(rows / NT)
    int accumulate;
    int overlap;         // host side only: launch with programmatic stream serialization (see launch_nt)
    int kparts;          // > 1: every tile's K range is cut into this many parts, one CTA (pair) each, fp32 partial outputs
                         // go to the scratch as (part, row, S) and kparts_reduce_kernel sums them (more than 32 rows only)
    GroupDiv gdiv;
};

// (mask & a) | (~mask & b)
__device__ __forceinline__ uint32_t bit_select(uint32_t mask, uint32_t a, uint32_t b) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(d) : "r"(mask), "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ---- per-column constants ---------------------------------------------------------------------------------
struct ColK {
    uint32_t s2, z2;
    uint32_t zb;       // sparse fast mode: the integer zero-point replicated into 4 bytes
};

// v = (1024 + q_lo * 2^a, 1024 + q_hi * 2^b) -> the two fp16 weights.  mul / base undo the two shifts exactly.
template <int BITS, int MODE>
__device__ __forceinline__ uint32_t finish(uint32_t v, uint32_t mul, uint32_t base, uint32_t off, const ColK& c) {
    if (MODE == MODE_FAST) return hmul2_u(hfma2_u(v, mul, off), c.s2);         // off = base - zero
    const uint32_t q = hfma2_u(v, mul, base);                                  // exact integers
    if (MODE == MODE_GENERAL) return hmul2_u(hsub2_u(q, c.z2), c.s2);
    const __half2 qh = u32_as_h2(q);
    const __half s = __ushort_as_half((unsigned short)(c.s2 & 0xFFFFu));
    const __half z = __ushort_as_half((unsigned short)(c.z2 & 0xFFFFu));
    const __half lo = dequant_dynamic<BITS>(__half2uint_rz(__low2half(qh)), s, z);
    const __half hi = dequant_dynamic<BITS>(__half2uint_rz(__high2half(qh)), s, z);
    return h2_as_u32(__halves2half2(lo, hi));
}

// half2 constants (hi << 16 | lo)
constexpr uint32_t MUL_1_16 = 0x2C003C00u, BASE_1_16 = 0xD400E400u;      // (x1, x16): int4 nibble pairs
constexpr uint32_t MUL_1_4 = 0x34003C00u, BASE_1_4 = 0xDC00E400u;        // (x1, x4):  int2 crumbs 0, 1
constexpr uint32_t MUL_16_64 = 0x24002C00u, BASE_16_64 = 0xCC00D400u;    // (x16, x64): int2 crumbs 2, 3
constexpr uint32_t MUL_1_8 = 0x30003C00u, BASE_1_8 = 0xD800E400u;        // (x1, x8):  int3 field pairs
constexpr uint32_t MUL_1_1 = 0x3C003C00u, BASE_1_1 = 0xE400E400u;        // (x1, x1): sparse int4 through bytes

// 256-entry table for the sparse expansion, indexed by one byte of the keep-mask (8 positions; see the sparse decode).
// The next 8 kept nibbles are spread over the 8 bytes of a register pair (even nibbles, odd nibbles); for position p
// with rank r among the kept ones the PRMT selector names byte r / 2 of the even or (4 +) of the odd register.
//   x = selector of positions 0..3 | (4 * popcount) << 16 (PRMT reads only the low 16 bits of its selector)
//   y = selector of positions 4..7      z, w = 0xFF in the bytes of the kept positions 0..3, 4..7
constexpr int kSparseLutEntries = 256;
__device__ __forceinline__ uint4 sparse_lut_entry(int mb) {
    uint32_t sel[2] = {0, 0}, keep[2] = {0, 0}, rank = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (mb & (1 << j)) {
            sel[j >> 2] |= ((rank >> 1) + 4u * (rank & 1u)) << (4 * (j & 3));
            keep[j >> 2] |= 0xFFu << (8 * (j & 3));
            ++rank;
        }
    }
    return make_uint4(sel[0] | ((4 * rank) << 16), sel[1], keep[0], keep[1]);
}

// ---- formats: one 64-k part of one column -> 32 registers of fp16 pairs -----------------------------------------
// The pairs are in natural k order, except for dense int4 with PERM: there register 4r + j of packed word r holds
// (k_j, k_{j+4}) of the word's eight k, which needs no byte shuffles; the activation tile is permuted to match
// (kPermutedK: position 2j + i of every group of eight k holds k_{j + 4i}).
template <int BITS, bool SPARSE, bool PERM = false>
struct UFormat;

template <bool PERM>
struct UFormat<4, false, PERM> {
    static constexpr int WROWS = 8, MROWS = 0;       // packed rows / mask rows per 64-k part
    static constexpr bool kPermutedK = PERM;
    template <int MODE>
    __device__ static __forceinline__ void decode(uint32_t wbase, uint32_t, const ColK& c, uint32_t (&A)[32], const uint4*) {
        if (PERM) {
            // nibbles j and j + 4 of a word sit at the same offset of its two 16-bit halves: one LOP3 per pair plants both
            // into the mantissas of (1024, 1024); the odd nibbles come out multiplied by 16
            const uint32_t off1 = hsub2_u(BASE_1_1, c.z2), off16 = hsub2_u(H2_N64, c.z2);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const uint32_t w = ptx::lds32(wbase + r * 512);
                const uint32_t w8 = w >> 8;
                A[4 * r + 0] = finish<4, MODE>(and_or(w, 0x000F000Fu, kMagic1024), MUL_1_1, BASE_1_1, off1, c);      // k0, k4
                A[4 * r + 1] = finish<4, MODE>(and_or(w, 0x00F000F0u, kMagic1024), H2_1_16, H2_N64, off16, c);       // k1, k5
                A[4 * r + 2] = finish<4, MODE>(and_or(w8, 0x000F000Fu, kMagic1024), MUL_1_1, BASE_1_1, off1, c);     // k2, k6
                A[4 * r + 3] = finish<4, MODE>(and_or(w8, 0x00F000F0u, kMagic1024), H2_1_16, H2_N64, off16, c);      // k3, k7
            }
            return;
        }
        const uint32_t off = hsub2_u(BASE_1_16, c.z2);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const uint32_t w = ptx::lds32(wbase + r * 512);
            const uint32_t y0 = prmt(w, w, 0x1010), y1 = prmt(w, w, 0x3232);   // low / high 16 bits in both lanes
            A[4 * r + 0] = finish<4, MODE>(and_or(y0, 0x00F0000Fu, kMagic1024), MUL_1_16, BASE_1_16, off, c);        // k0, k1
            A[4 * r + 1] = finish<4, MODE>(and_or(y0 >> 8, 0x00F0000Fu, kMagic1024), MUL_1_16, BASE_1_16, off, c);   // k2, k3
            A[4 * r + 2] = finish<4, MODE>(and_or(y1, 0x00F0000Fu, kMagic1024), MUL_1_16, BASE_1_16, off, c);        // k4, k5
            A[4 * r + 3] = finish<4, MODE>(and_or(y1 >> 8, 0x00F0000Fu, kMagic1024), MUL_1_16, BASE_1_16, off, c);   // k6, k7
        }
    }
};

template <bool PERM>
struct UFormat<2, false, PERM> {
    static constexpr int WROWS = 4, MROWS = 0;
    static constexpr bool kPermutedK = false;
    template <int MODE>
    __device__ static __forceinline__ void decode(uint32_t wbase, uint32_t, const ColK& c, uint32_t (&A)[32], const uint4*) {
        const uint32_t offa = hsub2_u(BASE_1_4, c.z2), offb = hsub2_u(BASE_16_64, c.z2);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint32_t w = ptx::lds32(wbase + r * 512);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t y = h ? prmt(w, w, 0x3232) : prmt(w, w, 0x1010);   // crumbs 8h .. 8h+7 in both lanes
                const uint32_t y8 = y >> 8;
                A[8 * r + 4 * h + 0] = finish<2, MODE>(and_or(y, 0x000C0003u, kMagic1024), MUL_1_4, BASE_1_4, offa, c);
                A[8 * r + 4 * h + 1] = finish<2, MODE>(and_or(y, 0x00C00030u, kMagic1024), MUL_16_64, BASE_16_64, offb, c);
                A[8 * r + 4 * h + 2] = finish<2, MODE>(and_or(y8, 0x000C0003u, kMagic1024), MUL_1_4, BASE_1_4, offa, c);
                A[8 * r + 4 * h + 3] = finish<2, MODE>(and_or(y8, 0x00C00030u, kMagic1024), MUL_16_64, BASE_16_64, offb, c);
            }
        }
    }
};

template <bool PERM>
struct UFormat<3, false, PERM> {
    static constexpr int WROWS = 6, MROWS = 0;
    static constexpr bool kPermutedK = false;
    template <int MODE>
    __device__ static __forceinline__ void decode(uint32_t wbase, uint32_t, const ColK& c, uint32_t (&A)[32], const uint4*) {
        const uint32_t off = hsub2_u(BASE_1_8, c.z2);
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const uint32_t w0 = ptx::lds32(wbase + (3 * blk) * 512), w1 = ptx::lds32(wbase + (3 * blk + 1) * 512),
                           w2 = ptx::lds32(wbase + (3 * blk + 2) * 512);
            // the 96-bit stream in 12-bit chunks: chunk j holds fields 4j .. 4j+3 = pairs (2j, 2j+1)
            uint32_t ch[8];
            ch[0] = w0;
            ch[1] = w0 >> 12;
            ch[2] = __funnelshift_r(w0, w1, 24);
            ch[3] = w1 >> 4;
            ch[4] = w1 >> 16;
            ch[5] = __funnelshift_r(w1, w2, 28);
            ch[6] = w2 >> 8;
            ch[7] = w2 >> 20;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t y = prmt(ch[j], ch[j], 0x1010);
                A[16 * blk + 2 * j + 0] = finish<3, MODE>(and_or(y, 0x00380007u, kMagic1024), MUL_1_8, BASE_1_8, off, c);
                A[16 * blk + 2 * j + 1] = finish<3, MODE>(and_or(y >> 6, 0x00380007u, kMagic1024), MUL_1_8, BASE_1_8, off, c);
            }
        }
    }
};

template <bool PERM>
struct UFormat<4, true, PERM> {
    static constexpr int WROWS = 4, MROWS = 2;
    static constexpr bool kPermutedK = false;
    template <int MODE>
    __device__ static __forceinline__ void decode(uint32_t wbase, uint32_t mbase, const ColK& c, uint32_t (&A)[32], const uint4* lut) {
        const uint32_t off = hsub2_u(BASE_1_1, c.z2);
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            // a 32-block of this column: the 64-bit word of its 16 kept nibbles (in increasing k) and its keep-mask
            uint32_t lo = ptx::lds32(wbase + (2 * blk) * 512), hi = ptx::lds32(wbase + (2 * blk + 1) * 512);
            const uint32_t m = ptx::lds32(mbase + blk * 512);
#pragma unroll
            for (int byte = 0; byte < 4; ++byte) {               // 8 positions per step
                const uint4 e = lut[(m >> (8 * byte)) & 0xFFu];
                const uint32_t even = lo & 0x0F0F0F0Fu;          // kept nibbles 0, 2, 4, 6 of the next eight, one per byte
                const uint32_t odd = (lo >> 4) & 0x0F0F0F0Fu;    // kept nibbles 1, 3, 5, 7
                uint32_t d[2] = {prmt(even, odd, e.x), prmt(even, odd, e.y)};   // positions 0..3, 4..7 as bytes
                const uint32_t keep[2] = {e.z, e.w};
#pragma unroll
                for (int q4 = 0; q4 < 2; ++q4) {
                    // fast mode: a dropped position gets the (integer) zero-point as its nibble, so it decodes to +0
                    if (MODE == MODE_FAST) d[q4] = bit_select(keep[q4], d[q4], c.zb);
                    uint32_t a = finish<4, MODE>(prmt(d[q4], 0x64646464u, 0x5140), MUL_1_1, BASE_1_1, off, c);
                    uint32_t b = finish<4, MODE>(prmt(d[q4], 0x64646464u, 0x7362), MUL_1_1, BASE_1_1, off, c);
                    if (MODE != MODE_FAST) {                     // exact zeros at dropped positions
                        a &= prmt(keep[q4], keep[q4], 0x1100);
                        b &= prmt(keep[q4], keep[q4], 0x3322);
                    }
                    A[16 * blk + 4 * byte + 2 * q4] = a;
                    A[16 * blk + 4 * byte + 2 * q4 + 1] = b;
                }
                const uint32_t sh = e.x >> 16;                   // 4 bits per kept position, up to 32
                lo = __funnelshift_rc(lo, hi, sh);
                hi = __funnelshift_rc(hi, 0u, sh);
            }
        }
    }
};

template <class F, int H>
struct WStage {     // one stage of the packed-weight ring: one unit = H parts of 64 k
    static constexpr int kW = 0;                                 // H * WROWS packed rows of 512 B
    static constexpr int kMask = H * F::WROWS * 512;             // H * MROWS mask rows of 512 B
    static constexpr int kS = kMask + H * F::MROWS * 512;        // H rows of scales (groups g0 .. g0 + H - 1), 256 B each
    static constexpr int kZ = kS + H * 256;                      // H rows of zeros
    static constexpr int kBytes = kZ + H * 256;
};

constexpr int kMaxWStages = 16;
constexpr int kMaxABStages = 6;

template <int NT, bool PAIR>
struct Cfg {
    // packed-weight ring (128 k per stage).  Few rows: the kernel streams weights from HBM, and the ring has to
    // cover the DRAM latency; many rows: weights are a trickle next to the activation tiles
    static constexpr bool kStream = NT <= 32;                         // weight-streaming shapes: one CTA per SM with everything doubled
    // NT = 128..192: an MMA of N <= 192 takes 512..768 cycles per 128 k, the dequantisation of its weights with two
    // warpgroups ~1400, so these shapes get four warpgroups as well, and a deeper weight ring
    // (single CTAs have the shared memory for the 4 A / activation stages that four warpgroups need only at NT = 128)
    static constexpr bool kDequantBound = NT == 128 || (PAIR && NT >= 128 && NT <= 192);
    // A stage of either ring is waited for by parity, which tells a completed phase only from the one before it.
    // Where the weight stages are not a multiple of the warpgroups, consecutive uses of a stage belong to different
    // warpgroups, and one could poll for a stage's next fill while the previous one, meant for another warpgroup, has
    // not landed yet (tensor-map copies may complete out of order) and take the stale phase for its own: there the
    // dequant warps first wait, like the producer, until the previous use has been released (kWGuard).  And there
    // are at least as many A stages as warpgroups (checked in the kernel).
    // A unit (one stage of every ring) is kHalves parts of 64 k.  The producers and the MMA issuer are single threads
    // whose loops cost ~500 cycles per stage whatever its size (an mbarrier wait ~190 cycles even when it is already
    // complete, expect_tx + the copy's issue another ~190): at 128 k per stage that alone is ~27 us for 16384 x 16384
    // weights on 148 SMs, so the weight-streaming shapes use 256-k units.
    static constexpr int kHalves = kStream ? 4 : 2;
    static constexpr int kWStages = kStream ? (NT <= 16 ? 9 : 6) : NT <= 64 ? 8 : kDequantBound ? 6 : 3;
    // staging slots (units of look-ahead) for activation rows that are reordered on their way into the A / activation
    // stages (umma_kernel's PERM)
    static constexpr int kXStaging = 4;
    static constexpr int kWG = kStream ? 3 : kDequantBound ? 4 : 2;   // dequant warpgroups (4 warps each), taking units in turn
    static constexpr int kABStages = kStream ? 3 : NT == 128 ? 4 : 3;   // ring of (A in tensor memory, activation tile in shared memory) pairs, one unit per stage
    static constexpr bool kWGuard = kWStages % kWG != 0;
    static constexpr bool kEpiWarps = NT >= 128 || kStream;           // a warpgroup of its own for the epilogue (else dequant warpgroup 0 does it)
    static constexpr bool kEpiTransposed = NT >= 128;                 // epilogue stores go through a shared-memory transposition tile
    static constexpr bool kEpiHandoff = kStream;                      // the MMA warp waits for the accumulator and wakes the epilogue warps (named barrier)
    static constexpr bool kDeferArrive = kStream;                     // a dequant warp announces an A stage only before its next wait (hides the tcgen05.wait::st latency)
    // many rows: two epilogue warpgroups, each draining half of the accumulator's columns, so that the next tile's
    // MMAs wait half as long for the accumulator
    static constexpr int kEpiGroups = NT >= 128 ? 2 : 1;
    // The weight-streaming shapes have two weight-producer threads (in two warps) that fill the stages in turn: one
    // thread's loop (wait ~190 cycles, expect_tx + copies ~250) delivers a 16 KB stage per ~500-700 cycles, about
    // 4-5 TB/s over the whole GPU, which is less than the memory system can stream.
    static constexpr int kWProducers = kStream ? 2 : 1;
    static constexpr int kWarps = 4 * kWG + (kEpiWarps ? 4 * kEpiGroups : 0) + 3 + (kWProducers - 1);  // + weight producer(s), activation producer, MMA issuer
    static constexpr int kThreads = kWarps * 32;
    static constexpr int kDCols = NT < 32 ? 32 : NT;                  // accumulator columns
    static constexpr int kACol0 = kDCols;                             // A stages follow: 32 columns per 64 k
    static constexpr int kAStageCols = 32 * kHalves;
    static constexpr int kColsUsed = kDCols + kAStageCols * kABStages;
    static constexpr int kTmemCols = kColsUsed <= 256 ? 256 : 512;
    // split-K over CTAs with a scratch reduction.  The code handles tiles of up to 128 rows, but the reducing CTA reads
    // its partners' partial tiles in dependent L2 round trips (rows x partners / 8 of them): measured at 128 rows that
    // costs 15-30 K cycles per tile and loses more than the better balance gains, so only the few-row shapes split.
    static constexpr bool kSplit = NT <= 32;
    static constexpr int kSlotElems = kDCols * 128;                   // 64-bit words of one CTA's partial tile in the scratch
    static constexpr int kMinBlocks = kStream ? 1 : NT <= 64 ? 2 : 1;
};

// A / activation stages.  A CTA of a pair holds only half of each activation tile, which leaves shared memory for as
// many stages as tensor memory has columns for (accumulator + 64 per stage <= 512).
template <int NT, bool PAIR>
struct ABStages {
    static constexpr int value = !PAIR ? Cfg<NT, false>::kABStages : (Cfg<NT, true>::kDCols + 64 * 5 <= 512 ? 5 : 4);   // pairs: 128-k units
};

struct Barriers {
    unsigned long long w_full[kMaxWStages], w_empty[kMaxWStages];
    unsigned long long ab_full[kMaxABStages];  // 4 dequant warps + the activation producer (with its transaction bytes)
    unsigned long long ab_free[kMaxABStages];  // tcgen05.commit: the MMAs that read the stage are done
    unsigned long long d_full, d_empty;
};

// Non-negative quotient; 64-bit division is a ~500-cycle subroutine on the GPU, so the 32-bit one is used whenever the
// operands allow it (practically always: unit counts are far below 2^32).
__device__ __forceinline__ long long div_nn(long long a, long long b) {
    if (((unsigned long long)a | (unsigned long long)b) >> 32) return a / b;
    return (long long)((uint32_t)a / (uint32_t)b);
}
__device__ __forceinline__ long long range_lo(long long T, long long G, long long b) { return div_nn(T * b, G); }
__device__ __forceinline__ int range_owner(long long T, long long G, long long t) {
    return (int)(div_nn((t + 1) * G + T - 1, T) - 1);
}

struct TensorMaps {
    CUtensorMap x;   // fp16 (rows, N):        box 64 k x NT rows, 128-byte swizzle; weight-streaming shapes: seen as
                     //                        (N / 64, rows, 64) with box kHalves x NT x 64, one copy per unit
    CUtensorMap w;   // int32 (R, S):          box 128 columns x kHalves * WROWS rows
    CUtensorMap m;   // int32 (N / 32, S):     box 128 columns x kHalves * MROWS rows (sparse format only)
    CUtensorMap s;   // fp16 (n_groups, S):    box 128 columns x kHalves rows
    CUtensorMap z;
};

// PAIR: launched as clusters of two CTAs (two SMs) that run every MMA together (cta_group::2, M = 256): the pair's
// tile is 256 weight columns x NT rows, each CTA dequantises its own 128 columns and loads only half of the rows of
// the activation tile, which halves the L2 -> shared-memory traffic that bounds the many-row shapes.
// PERM (up to 8 rows of dense int4 only): the cheaper k order of UFormat, with the activations reordered to match.
template <int BITS, bool SPARSE, int NT, bool PAIR, bool PERM = false>
__global__ void __launch_bounds__(Cfg<NT, PAIR>::kThreads, Cfg<NT, PAIR>::kMinBlocks)
umma_kernel(const __grid_constant__ TensorMaps tm, const UmmaParams p, const __half* x) {
    using C = Cfg<NT, PAIR>;
    using F = UFormat<BITS, SPARSE, PERM>;
    static_assert(!PERM || (C::kStream && F::kPermutedK), "the permuted k order is for dense int4 weight streaming");
    constexpr int H = C::kHalves;                                    // 64-k parts per unit
    using WS = WStage<F, H>;
    static_assert(!PAIR || (NT >= 128 && !C::kEpiHandoff), "CTA pairs are for the many-row shapes");
    static_assert((2 * C::kWStages) % C::kWG == 0, "every second use of a weight stage must be by the same warpgroup");
    static_assert(ABStages<NT, PAIR>::value >= C::kWG, "fewer A stages than warpgroups: a parity wait could see the phase before last");
    constexpr int kBHalfBytes = (PAIR ? NT / 2 : NT) * 128;        // one 64-k activation sub-tile held by this CTA
    constexpr int kBStageBytes = H * kBHalfBytes;
    // single CTAs at NT = 256 have no shared memory left for a second transposition tile: the second epilogue group idles
    constexpr int kEpiGroups = (C::kEpiGroups == 2 && (PAIR || NT < 256)) ? 2 : 1;
    constexpr int kEpiWarp0 = 4 * C::kWG;                           // first epilogue warp (a multiple of 4: lane quarter = warp % 4)
    constexpr int kWProducer = kEpiWarp0 + (C::kEpiWarps ? 4 * C::kEpiGroups : 0), kBProducer = kWProducer + 1, kMma = kWProducer + 2;
    constexpr int kWProducer2 = kWProducer + 3;                     // only when Cfg::kWProducers == 2
    constexpr int kABStages = ABStages<NT, PAIR>::value;
    extern __shared__ __align__(1024) unsigned char smem[];      // [B ring (1024-aligned tiles)][W ring]
    __shared__ __align__(8) Barriers bars;
    __shared__ uint4 lut[SPARSE ? kSparseLutEntries : 1];
    __shared__ uint32_t tmem_base_smem;
    __shared__ volatile int s_abort;     // set by a warp that gives up on the accumulator (the MMA warp before it releases the epilogue
                                         // warps for the last time; an epilogue warp before its group's next named barrier)

    // the shuffle tells the compiler that the warp index is warp-uniform: role dispatch, stage indices and barrier
    // addresses derived from it then live in uniform registers instead of costing vector-ALU instructions
    const int lane = threadIdx.x & 31, warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0);
    const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;       // in the pair; rank 0 leads (issues the MMAs, owns the pair's barriers)
    const uint32_t smem0 = (ptx::smem_u32(smem) + 1023u) & ~1023u;
    const uint32_t b_ring = smem0;
    const uint32_t w_ring = smem0 + kABStages * kBStageBytes;
    const uint32_t epi_tile = w_ring + C::kWStages * WS::kBytes;     // 4 KB transposition tile per epilogue warpgroup (NT >= 128)
    const uint32_t x_staging = epi_tile;                             // weight-streaming shapes (no transposition tile): activation staging ring

    // ---- set-up, spread over warps so that nothing waits for one thread ----
    // The weight producer's warp initialises the weight ring's barriers itself and does not wait for the rest of the
    // CTA (it only arrives on the set-up barrier): its first copies are in flight while tensor memory is allocated.
    if (warp == kWProducer) {
        if (lane == 0) {
            ptx::prefetch_tmap(&tm.w);
            if (SPARSE) ptx::prefetch_tmap(&tm.m);
        }
        if (lane < C::kWStages) {
            ptx::mbar_init(ptx::smem_u32(&bars.w_full[lane]), 1);
            ptx::mbar_init(ptx::smem_u32(&bars.w_empty[lane]), 4);
        }
        ptx::fence_mbar_init();
        __syncwarp();
        if (PAIR) ptx::cluster_sync_all();        // the other CTA arrives on this one's barriers: both must be set up first
        else ptx::named_bar_arrive(3, C::kThreads);
    } else {
        if (warp == 0) {
            if (lane < kABStages) {
                // a pair's stage is full when the dequant warps of both CTAs and both activation halves have arrived
                ptx::mbar_init(ptx::smem_u32(&bars.ab_full[lane]), PAIR ? 4 + 4 + 1 : 4 + 1);
                ptx::mbar_init(ptx::smem_u32(&bars.ab_free[lane]), 1);
            }
            if (lane == 31) {
                ptx::mbar_init(ptx::smem_u32(&bars.d_full), 1);
                ptx::mbar_init(ptx::smem_u32(&bars.d_empty), (PAIR ? 8 : 4) * kEpiGroups);
                s_abort = 0;
            }
            ptx::fence_mbar_init();
        }
        if (SPARSE && warp < 8) lut[warp * 32 + lane] = sparse_lut_entry(warp * 32 + lane);   // (warps 0..7 are dequant warps in every configuration)
        if (warp == kMma) {
            if (PAIR) {
                ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_smem), C::kTmemCols);
                ptx::tmem_relinquish_pair();
            } else {
                ptx::tmem_alloc(ptx::smem_u32(&tmem_base_smem), C::kTmemCols);
                ptx::tmem_relinquish();
            }
        }
        if (warp == kBProducer && lane == 0) {
            ptx::prefetch_tmap(&tm.x);
            ptx::prefetch_tmap(&tm.s);
            ptx::prefetch_tmap(&tm.z);
        }
        ptx::tc_fence_before_sync();
        if (PAIR) ptx::cluster_sync_all();
        else ptx::named_bar_sync(3, C::kThreads);
        ptx::tc_fence_after_sync();
    }
    const uint32_t tmem_base = tmem_base_smem;       // not valid in the weight producer's warp, which never uses it
    // The next kernel of the stream may be scheduled from here on (it takes an SM only when a CTA of this grid has left
    // it); if it is one of these kernels, its set-up and its first weight copies then overlap this grid's tail.
    if (threadIdx.x == 0) ptx::grid_launch_dependents();

    // ---- this CTA's share of the (tile, unit) space; one unit = H x 64 k.  Whole tiles unless the split-K variant ----
    const long long U = p.U;
    const int CTd = PAIR ? (p.CT + 1) / 2 : p.CT;                  // column tiles of a CTA, or column-tile pairs of a CTA pair
    const long long n_tiles = (long long)p.MTILES * CTd;
    const long long G = PAIR ? gridDim.x / 2 : gridDim.x, b = PAIR ? blockIdx.x / 2 : blockIdx.x;
    // tile index -> this CTA's column tile (may lie past the last one in a pair: loads are zero-filled, stores masked) and row tile
    // Column tiles vary fastest.  (Row tiles fastest would read each packed-weight tile from HBM only once, but then every
    // SM asks L2 for the same activation lines at the same moment, and that hot spot cost 3-25 % when measured.)
    auto tile_ct = [&](long long tile) -> int { return (int)(tile % CTd) * (PAIR ? 2 : 1) + (int)rank; };
    auto tile_mt = [&](long long tile) -> int { return (int)(tile / CTd); };
    long long t_lo, t_hi;
    const int kpart = p.kparts > 1 ? (int)(b % p.kparts) : 0;
    if (C::kSplit) {
        t_lo = range_lo(n_tiles * U, G, b);
        t_hi = range_lo(n_tiles * U, G, b + 1);
    } else if (p.kparts > 1) {
        // the grid is exactly tiles x parts: one part of one tile per CTA (pair)
        const long long tile = b / p.kparts;
        t_lo = tile * U + (U * kpart) / p.kparts;
        t_hi = tile * U + (U * (kpart + 1)) / p.kparts;
    } else {
        t_lo = range_lo(n_tiles, G, b) * U;
        t_hi = range_lo(n_tiles, G, b + 1) * U;
    }

    if (warp == kWProducer || (C::kWProducers == 2 && warp == kWProducer2)) {
        // =========================== packed weights (+ scales / zeros): one thread per producer warp ===========================
        if (lane == 0) {
            // every box is copied whole (out-of-range parts are zero-filled)
            constexpr uint32_t kBytes = (uint32_t)WS::kBytes;
            const uint32_t mine = warp == kWProducer ? 0u : 1u;             // with two producers: the stages of this parity
            uint32_t si = 0, ws = 0, wph = 0;
            bool ok = true, ramped = false;
            for (long long t = t_lo; t < t_hi && ok;) {
                const long long tile = div_nn(t, U);                      // one 64-bit division per segment, none per unit
                const int u0 = (int)(t - tile * U);
                const int u1 = (int)min(U, u0 + (t_hi - t));
                const int ct = tile_ct(tile);
                for (int u = u0; u < u1; ++u, ++si) {
                    if (C::kWProducers == 1 || (si & 1u) == mine) {
                        // At the start all CTAs of the GPU ask for their whole rings at once, and the memory system serves
                        // the requests side by side: the first stage would arrive when a third of everything has (measured:
                        // 2.8 us after its copy was issued; 0.9 us for the luckiest CTA).  So the first stages go out alone,
                        // and the rest of the ring only once they have landed: each producer waits once, for the first
                        // stage it issued itself, before its second copy.
                        if (C::kStream && !ramped && si >= (uint32_t)C::kWProducers) {
                            if (!ptx::mbar_wait(ptx::smem_u32(&bars.w_full[mine]), 0u)) { atomicExch(p.status, 15); ok = false; break; }
                            ramped = true;
                        }
                        if (!ptx::mbar_wait(ptx::smem_u32(&bars.w_empty[ws]), wph ^ 1u)) { atomicExch(p.status, 11); ok = false; break; }
                        const uint32_t st = w_ring + ws * WS::kBytes, full = ptx::smem_u32(&bars.w_full[ws]);
                        ptx::mbar_arrive_expect_tx(full, kBytes);
                        ptx::tma_load_2d(st + WS::kW, &tm.w, ct * 128, u * H * F::WROWS, full);
                        if (SPARSE) ptx::tma_load_2d(st + WS::kMask, &tm.m, ct * 128, u * H * F::MROWS, full);
                        const int g0 = (int)p.gdiv((uint32_t)H * (uint32_t)u);
                        ptx::tma_load_2d(st + WS::kS, &tm.s, ct * 128, g0, full);
                        ptx::tma_load_2d(st + WS::kZ, &tm.z, ct * 128, g0, full);
                    }
                    if (++ws == C::kWStages) { ws = 0; wph ^= 1u; }
                }
                t += u1 - u0;
            }
        }
    } else if (PERM && warp == kBProducer) {
        // =========================== activation tiles in the permuted k order: the whole warp ===========================
        // The few valid rows are fetched with plain asynchronous 16-byte copies (eight consecutive k each) into a small
        // staging ring, kXStaging units ahead, every lane its own chunks.  When the unit's A / activation stage is free,
        // each lane reorders its chunks to (k0, k4, k1, k5, k2, k6, k3, k7), the order the dequant warps produce without
        // byte shuffles, and stores them at their place in the stage's 128-byte-swizzled tile; then the stage is
        // announced to the MMA warp.  Rows past the last valid one are zeroed once, up front.  (A tensor-map copy plus
        // a barrier per unit, as for the other formats, costs this warp more per unit than the unit may take.)
        for (uint32_t o = lane * 16; o < (uint32_t)(kABStages * kBStageBytes); o += 32 * 16) ptx::sts128(b_ring + o, make_uint4(0, 0, 0, 0));
        ptx::grid_dependency_wait();      // the activations may be the output of the kernel before this one in the stream
        constexpr int D = C::kXStaging;
        const int total = (int)(t_hi - t_lo);
        const int nrows = min(NT, p.rows);                              // (one row tile: these shapes have at most NT rows)
        const int n_chunks = nrows * 8 * H;                             // chunk index = row * (8 * H) + part * 8 + chunk of the part's 128-byte row segment
        int u_next = (int)(t_lo - div_nn(t_lo, U) * U);                // unit (within its column tile) of the next copy
        auto fetch = [&](int slot) {
            for (int idx = lane; idx < n_chunks; idx += 32) {
                const int r = idx / (8 * H), hc = idx % (8 * H);
                const int k = (u_next * H * 8 + hc) * 8;
                // past the end of the row (N is a multiple of 64, not of 256): zero fill
                ptx::cp_async_16(x_staging + slot * kBStageBytes + idx * 16, x + (size_t)r * p.N + (k < p.N ? k : 0), k < p.N ? 16u : 0u);
            }
            ptx::cp_async_commit();
            if (++u_next == (int)U) u_next = 0;
        };
        for (int j = 0; j < D - 1; ++j) {                                   // (always D - 1 groups, empty ones if need be: wait_group counts groups)
            if (j < total) fetch(j);
            else ptx::cp_async_commit();
        }
        for (int i = 0; i < total; ++i) {
            if (i + D - 1 < total) fetch((i + D - 1) % D);
            else ptx::cp_async_commit();                                  // (keeps the group count per iteration fixed)
            const uint32_t s = (uint32_t)(i % kABStages), ph = (uint32_t)(i / kABStages) & 1u;
            if (!ptx::mbar_wait(ptx::smem_u32(&bars.ab_free[s]), ph ^ 1u)) {
                if (lane == 0) atomicExch(p.status, 12);
                break;
            }
            ptx::cp_async_wait_group<D - 1>();                           // the copies of unit i (this lane's own chunks) have landed
            const uint32_t src = x_staging + (i % D) * kBStageBytes, dst = b_ring + s * kBStageBytes;
            for (int idx = lane; idx < n_chunks; idx += 32) {
                const int r = idx / (8 * H), hc = idx % (8 * H);
                const uint4 a = ptx::lds128(src + idx * 16);
                uint4 o;
                o.x = prmt(a.x, a.z, 0x5410);      // (k0, k4)
                o.y = prmt(a.x, a.z, 0x7632);      // (k1, k5)
                o.z = prmt(a.y, a.w, 0x5410);      // (k2, k6)
                o.w = prmt(a.y, a.w, 0x7632);      // (k3, k7)
                // 128-byte swizzle of the tile a tensor-map copy would have produced: chunk c of row r sits at c ^ (r % 8)
                ptx::sts128(dst + (hc >> 3) * kBHalfBytes + r * 128 + (((hc & 7) ^ (r & 7)) << 4), o);
            }
            ptx::fence_proxy_async_smem();         // the MMAs read the tile through the async proxy
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars.ab_full[s]));
        }
        ptx::cp_async_wait_group<0>();
    } else if (warp == kBProducer) {
        // =========================== activation tiles, one 64-k sub-tile per part of a unit: one thread ===========================
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            // the activations may be the output of the kernel before this one in the stream (the weight-side tensors
            // are not: see the launch attribute in launch_nt)
            ptx::grid_dependency_wait();
            for (long long t = t_lo; t < t_hi && ok;) {
                const long long tile = div_nn(t, U);
                const int u0 = (int)(t - tile * U);
                const int u1 = (int)min(U, u0 + (t_hi - t));
                const int mt = tile_mt(tile);
                for (int u = u0; u < u1; ++u) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&bars.ab_free[s]), ph ^ 1u)) { atomicExch(p.status, 12); ok = false; break; }
                    const uint32_t full = ptx::smem_u32(&bars.ab_full[s]);
                    if (PAIR) {
                        // both CTAs' halves are counted on the leader's barrier, which expects the bytes of both
                        const uint32_t lfull = ptx::map_to_cta(full, 0);
                        if (rank == 0) ptx::mbar_arrive_expect_tx(full, 2u * (uint32_t)kBStageBytes);
                        const int r0 = mt * NT + (int)rank * (NT / 2);
                        ptx::tma_load_2d_pair(b_ring + s * kBStageBytes, &tm.x, u * 128, r0, lfull);
                        ptx::tma_load_2d_pair(b_ring + s * kBStageBytes + kBHalfBytes, &tm.x, u * 128 + 64, r0, lfull);
                    } else if (C::kStream) {
                        // one copy per unit: H sub-tiles of 64 k, laid out one after the other
                        ptx::mbar_arrive_expect_tx(full, (uint32_t)kBStageBytes);
                        ptx::tma_load_3d(b_ring + s * kBStageBytes, &tm.x, 0, mt * NT, u * H, full);
                    } else {
                        ptx::mbar_arrive_expect_tx(full, (uint32_t)kBStageBytes);
                        ptx::tma_load_2d(b_ring + s * kBStageBytes, &tm.x, u * 128, mt * NT, full);
                        ptx::tma_load_2d(b_ring + s * kBStageBytes + kBHalfBytes, &tm.x, u * 128 + 64, mt * NT, full);
                    }
                    if (++s == kABStages) { s = 0; ph ^= 1u; }
                }
                t += u1 - u0;
            }
        }
    } else if (warp == kMma) {
        // =========================== MMA issuer: the warp walks the loop, one elected lane issues ===========================
        {
            const uint32_t idesc = PAIR ? ptx::idesc_f16_m256(NT) : ptx::idesc_f16_m128(NT);
            uint32_t si = 0, seg = 0;
            bool ok = true;
            if (PAIR && rank != 0) t_lo = t_hi;              // the leader issues for both CTAs
            for (long long t = t_lo; t < t_hi && ok;) {
                const long long tile = div_nn(t, U);
                const int u0 = (int)(t - tile * U);
                const int u1 = (int)min(U, u0 + (t_hi - t));
                if (!ptx::mbar_wait(ptx::smem_u32(&bars.d_empty), (seg & 1u) ^ 1u)) {
                    if (lane == 0) atomicExch(p.status, 21);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after_sync();
                uint32_t s = si % kABStages, ph = (si / kABStages) & 1u;
                for (int u = u0; u < u1; ++u, ++si) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&bars.ab_full[s]), ph)) {
                        if (lane == 0) atomicExch(p.status, 22);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint64_t bdesc = ptx::smem_desc_sw128(b_ring + s * kBStageBytes);
                    const uint32_t a0 = tmem_base + C::kACol0 + s * C::kAStageCols;
                    if (ptx::elect_one()) {
#pragma unroll
                        for (int k = 0; k < 4 * H; ++k) {
                            // K = 16 per instruction: +8 columns of A; B: +32 bytes (2 descriptor units) inside a 64-k sub-tile
                            const uint64_t bd = bdesc + (uint64_t)((k >> 2) * (kBHalfBytes >> 4) + (k & 3) * 2);
                            if (PAIR) ptx::umma_f16_ts_pair(tmem_base, a0 + k * 8, bd, idesc, (u > u0 || k > 0) ? 1u : 0u);
                            else ptx::umma_f16_ts(tmem_base, a0 + k * 8, bd, idesc, (u > u0 || k > 0) ? 1u : 0u);
                        }
                        if (PAIR) {                                      // the stage comes free in both CTAs
                            ptx::tc_commit_pair(ptx::map_to_cta(ptx::smem_u32(&bars.ab_free[s]), 0));
                            ptx::tc_commit_pair(ptx::map_to_cta(ptx::smem_u32(&bars.ab_free[s]), 1));
                        } else {
                            ptx::tc_commit(ptx::smem_u32(&bars.ab_free[s]));
                        }
                    }
                    __syncwarp();
                    if (++s == kABStages) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                if (ptx::elect_one()) {
                    if (PAIR) {
                        ptx::tc_commit_pair(ptx::map_to_cta(ptx::smem_u32(&bars.d_full), 0));
                        ptx::tc_commit_pair(ptx::map_to_cta(ptx::smem_u32(&bars.d_full), 1));
                    } else {
                        ptx::tc_commit(ptx::smem_u32(&bars.d_full));
                    }
                }
                __syncwarp();
                if (C::kEpiHandoff) {
                    // the epilogue warps sleep on a hardware barrier instead of polling for the whole segment
                    if (!ptx::mbar_wait(ptx::smem_u32(&bars.d_full), seg & 1u)) {
                        if (lane == 0) atomicExch(p.status, 23);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_before_sync();
                    ptx::named_bar_arrive(2, 128 + 32);
                }
                ++seg;
                t += u1 - u0;
            }
            if (C::kEpiHandoff && !ok) {
                s_abort = 1;
                __threadfence_block();
                ptx::named_bar_arrive(2, 128 + 32);
            }
        }
    } else {
        // =========================== dequant warpgroups; epilogue warps ===========================
        // Accumulator of one finished segment -> fp16 rows of `out`, or a partial tile for the split-K reduction.
        // Run by 4 warps whose index modulo 4 selects the 32 tensor-memory lanes (= weight columns) they may read.
        bool dependency_waited = false;
        auto epilogue = [&](uint32_t seg, long long tile, int u0, int u1) -> bool {
            if (!dependency_waited) {
                // outputs, old outputs and the scratch may still be in use by the kernel before this one in the stream
                ptx::grid_dependency_wait();
                dependency_waited = true;
            }
            const int mt = tile_mt(tile), ct = tile_ct(tile);
            const int col = (warp & 3) * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
            const bool complete = (u0 == 0) && (u1 == (int)U);
            const int scol = ct * 128 + col;
            const bool col_ok = scol < p.S;
            const int row0 = mt * NT;
            const int nrows = min(NT, p.rows - row0);
            // Split-K: the CTAs b_lo .. b_hi share this tile.  b_lo (which owns the tile's first units and reaches them
            // last) adds the others' partial tiles to its own accumulator in CTA order - a fixed order, so results are
            // reproducible.  A partial element is one 64-bit word (fp32 value | tag 1 in the high half), written with a
            // single store, so no fence, counter or second round trip is needed; the reader clears what it has read,
            // which leaves the scratch all-zero for the next launch.  Every other CTA's share of the tile is the first
            // segment of its range, so one slot per CTA is enough.
            int b_lo = 0, b_hi = -1;
            unsigned long long* slot = nullptr;
            unsigned long long* const partials64 = reinterpret_cast<unsigned long long*>(p.partials);
            if (C::kSplit && !complete) {
                const long long T = n_tiles * U, lo_t = tile * U;
                b_lo = range_owner(T, G, lo_t);
                b_hi = range_owner(T, G, lo_t + U - 1);
                if ((int)b != b_lo) slot = partials64 + (size_t)(PAIR ? b * 2 + rank : b) * C::kSlotElems;
            }
            // K parts: fp32 rows j0 .. of this lane's column into the (part, row, S) scratch; the reduce kernel sums the parts
            auto put_kpart = [&](auto& v, int j0) {
                constexpr int CNT = (int)(sizeof(v) / sizeof(uint32_t));
                if (!col_ok) return;
#pragma unroll
                for (int j = 0; j < CNT; ++j)
                    if (j0 + j < nrows)
                        p.partials[((size_t)kpart * p.rows + row0 + j0 + j) * p.S + scol] = __uint_as_float(v[j]);
            };
            // leaves accumulator rows j0 .. j0 + n - 1 of this lane's column in this CTA's slot
            auto put_partial = [&](auto& v, int j0) {
                constexpr int CNT = (int)(sizeof(v) / sizeof(uint32_t));
#pragma unroll
                for (int j = 0; j < CNT; ++j)
                    if (j0 + j < nrows) ptx::st_relaxed_gpu_u64(slot + (j0 + j) * 128 + col, (1ull << 32) | v[j]);
            };
            // adds the other CTAs' partial rows j0 .. j0 + n - 1 to v, in CTA order, and clears them
            auto add_partials = [&](auto& v, int j0) {
                constexpr int CNT = (int)(sizeof(v) / sizeof(uint32_t));
                bool waiting_ok = true;
                for (int bb = b_lo + 1; bb <= b_hi; ++bb) {
                    unsigned long long* src = partials64 + (size_t)(PAIR ? bb * 2 + (int)rank : bb) * C::kSlotElems + col;
#pragma unroll
                    for (int jb = 0; jb < CNT; jb += 8) {
                        if (j0 + jb >= nrows) break;                       // warp-uniform
                        unsigned long long w[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (j0 + jb + i < nrows) w[i] = ptx::ld_relaxed_gpu_u64(src + (j0 + jb + i) * 128);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            if (j0 + jb + i < nrows) {
                                for (uint32_t spins = 0; (uint32_t)(w[i] >> 32) != 1u && waiting_ok; ++spins) {
                                    if (spins >= ptx::kSpinLimit) {        // a contributor never delivered: report, stop waiting
                                        atomicExch(p.status, 34);
                                        waiting_ok = false;
                                        break;
                                    }
                                    __nanosleep(64);
                                    w[i] = ptx::ld_relaxed_gpu_u64(src + (j0 + jb + i) * 128);
                                }
                                v[jb + i] = __float_as_uint(__uint_as_float(v[jb + i]) + __uint_as_float((uint32_t)w[i]));
                                ptx::st_relaxed_gpu_u64(src + (j0 + jb + i) * 128, 0ull);
                            }
                        }
                    }
                }
            };
            // The weight-streaming shapes fetch the other CTAs' partial tiles BEFORE the own accumulator is complete (the
            // partners delivered them early in their run, as their first segment, and these warps have nothing else to
            // do): their sum, in CTA order, then only has to be added, and the dependent round trips to L2 are off the tail.
            constexpr int kPre = (C::kSplit && C::kEpiHandoff) ? C::kDCols : 1;
            uint32_t pre[kPre];
            bool prefetched = false;
            if (C::kSplit && C::kEpiHandoff && !slot && b_hi > b_lo) {
#pragma unroll
                for (int j = 0; j < kPre; ++j) pre[j] = 0u;
                if (kPre >= 16) {
#pragma unroll
                    for (int j0 = 0; j0 < kPre; j0 += 16) add_partials(reinterpret_cast<uint32_t(&)[16]>(pre[j0 < kPre ? j0 : 0]), j0);
                }
                prefetched = true;
            }
            if (C::kEpiHandoff) {
                ptx::named_bar_sync(2, 128 + 32);          // released by the MMA warp once the accumulator is complete
                if (s_abort) return false;
            } else {
                bool got = ptx::mbar_wait(ptx::smem_u32(&bars.d_full), seg & 1u);
                if (!got && lane == 0) atomicExch(p.status, 33);
                if (C::kEpiTransposed) {
                    // the four warps of an epilogue group meet at named barriers further down: a give-up has to be
                    // the whole group's decision, or the warps that went on would wait there for ever
                    if (!got) s_abort = 1;
                    ptx::named_bar_sync(1 + 3 * ((warp - kEpiWarp0) >> 2), 128);
                    got = s_abort == 0;
                }
                if (!got) return false;
            }
            ptx::tc_fence_after_sync();
            // matvec route with more than 64 rows (a batch of one-row products): the caller's old values of rows
            // j0 .. of this lane's column are added to the unrounded sums, so that there is still one rounding
            auto add_old_outs = [&](uint32_t (&v)[16], int j0) {
                if (!col_ok) return;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (j0 + j < nrows)
                        v[j] = __float_as_uint(__uint_as_float(v[j]) + __half2float(p.om.dst[0][(size_t)(row0 + j0 + j) * p.om.ld + p.om.col(scol)]));
            };
            if (C::kEpiTransposed) {
                // 16 accumulator columns (= 16 output rows) at a time: transposed through a 4 KB shared-memory tile so that
                // the global stores are 16-byte rows instead of one 2-byte element per lane
                const int eg = (warp - kEpiWarp0) >> 2;                     // epilogue warpgroup: its share of the accumulator columns
                const uint32_t stage_tile = epi_tile + eg * 4096;          // [16 rows][128 columns] fp16
                const uint32_t bar_id = 1 + 3 * eg;                         // named barriers 1 and 4
                const int t128 = (warp & 3) * 32 + lane;
                constexpr int kShare = NT / kEpiGroups;
                const int j_end = (eg + 1) * kShare;
                if (PAIR) {
                    // A CTA of a pair has the shared memory to stage its whole share as fp16 ([kShare rows][128 columns]):
                    // the accumulator is released after the tensor-memory loads and conversions alone, and the global
                    // stores run while the next tile's MMAs are already under way.
                    const uint32_t stage = epi_tile + eg * (kShare * 256);
#pragma unroll 1
                    for (int j0 = eg * kShare; j0 < j_end; j0 += 16) {
                        uint32_t v[16];
                        ptx::tmem_ld16(lane_addr + j0, v);
                        ptx::tc_wait_ld();
                        if (j0 + 16 >= j_end) {
                            ptx::tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&bars.d_empty), 0));
                        }
                        if (C::kSplit) {
                            if (slot) {
                                put_partial(v, j0);
                                continue;
                            }
                            if (b_hi > b_lo) add_partials(v, j0);
                        }
                        if (p.kparts > 1) {
                            put_kpart(v, j0);
                            continue;
                        }
                        if (p.accumulate) add_old_outs(v, j0);
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            ptx::sts16(stage + (j0 - eg * kShare + j) * 256 + col * 2,
                                       __half_as_ushort(__float2half_rn(__uint_as_float(v[j]))));
                    }
                    ptx::named_bar_sync(bar_id, 128);
#pragma unroll 1
                    for (int idx = t128; idx < ((slot || p.kparts > 1) ? 0 : kShare * 16); idx += 128) {   // 16-byte chunks: row = idx / 16, chunk = idx % 16
                        const int m = eg * kShare + (idx >> 4), c8 = (idx & 15) * 8;
                        if (m < nrows && ct * 128 + c8 < p.S) {
                            const uint4 q = ptx::lds128(stage + (idx >> 4) * 256 + c8 * 2);
                            const size_t at = (size_t)(row0 + m) * p.om.ld + p.om.col(ct * 128 + c8);   // (a chunk of 8 columns never straddles parts)
                            for (int d = 0; d < p.om.n_dst; ++d) *reinterpret_cast<uint4*>(p.om.dst[d] + at) = q;
                        }
                    }
                    ptx::named_bar_sync(bar_id, 128);                       // the staging area may be written again
                } else
#pragma unroll 1
                for (int j0 = eg * kShare; j0 < j_end; j0 += 16) {
                    uint32_t v[16];
                    ptx::tmem_ld16(lane_addr + j0, v);
                    ptx::tc_wait_ld();
                    if (j0 + 16 >= j_end) {                // this group's last columns are in registers: its share of the accumulator is free
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) {
                            if (PAIR) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&bars.d_empty), 0));
                            else ptx::mbar_arrive(ptx::smem_u32(&bars.d_empty));
                        }
                    }
                    if (C::kSplit) {
                        if (slot) {
                            put_partial(v, j0);
                            continue;
                        }
                        if (b_hi > b_lo) add_partials(v, j0);
                    }
                    if (p.kparts > 1) {
                        put_kpart(v, j0);
                        continue;
                    }
                    if (p.accumulate) add_old_outs(v, j0);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        ptx::sts16(stage_tile + j * 256 + col * 2, __half_as_ushort(__float2half_rn(__uint_as_float(v[j]))));
                    ptx::named_bar_sync(bar_id, 128);
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const int idx = t128 + r * 128;                     // 256 chunks of 16 bytes: row = idx / 16, chunk = idx % 16
                        const int m = j0 + (idx >> 4), c8 = (idx & 15) * 8;
                        if (m < nrows && ct * 128 + c8 < p.S) {
                            const uint4 q = ptx::lds128(stage_tile + (idx >> 4) * 256 + c8 * 2);
                            const size_t at = (size_t)(row0 + m) * p.om.ld + p.om.col(ct * 128 + c8);
                            for (int d = 0; d < p.om.n_dst; ++d) *reinterpret_cast<uint4*>(p.om.dst[d] + at) = q;
                        }
                    }
                    ptx::named_bar_sync(bar_id, 128);
                }
            } else {
            constexpr int CH = NT >= 64 ? 32 : 16;          // accumulator columns per tensor-memory load
#pragma unroll 1
            for (int j0 = 0; j0 < NT; j0 += CH) {
                uint32_t v[CH];
                if (CH == 32) ptx::tmem_ld32(lane_addr + j0, reinterpret_cast<uint32_t(&)[32]>(v));
                else ptx::tmem_ld16(lane_addr + j0, reinterpret_cast<uint32_t(&)[16]>(v));
                ptx::tc_wait_ld();
                if (j0 + CH >= NT) {                       // the last columns are in registers: the accumulator is free again
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars.d_empty));
                }
                if (slot) {
                    put_partial(v, j0);
                    continue;
                }
                if (C::kSplit && b_hi > b_lo) {
                    if (prefetched) {
#pragma unroll
                        for (int j = 0; j < CH; ++j)
                            v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(pre[(j0 + j) < kPre ? j0 + j : 0]));
                    } else {
                        add_partials(v, j0);
                    }
                }
                if (p.kparts > 1) {
                    put_kpart(v, j0);
                    continue;
                }
                if (col_ok) {
                    const long long dcol = p.om.col(scol);
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const int m = j0 + j;
                        if (m < nrows) {
                            float f = __uint_as_float(v[j]);
                            const size_t at = (size_t)(row0 + m) * p.om.ld + dcol;
                            if (p.accumulate) f += __half2float(p.om.dst[0][at]);
                            const __half h = __float2half_rn(f);
                            for (int d = 0; d < p.om.n_dst; ++d) p.om.dst[d][at] = h;
                        }
                    }
                }
            }
            }
            // Stores into other GPUs' buffers: every storing thread makes its own stores visible system-wide before the
            // CTA can finish, so that the hand-shake kernel's flag (written by another SM, possibly over another link)
            // cannot reach a peer before this data has.
            if (p.om.n_dst > 1) __threadfence_system();
            return true;
        };

        if (C::kEpiWarps && warp >= kEpiWarp0 + 4 * kEpiGroups) {
            // (an epilogue warpgroup that this configuration does not use)
        } else if (C::kEpiWarps && warp >= kEpiWarp0) {
            // ----- dedicated epilogue warps: one pass per segment -----
            uint32_t seg = 0;
            for (long long t = t_lo; t < t_hi;) {
                const long long tile = div_nn(t, U);
                const int u0 = (int)(t - tile * U);
                const int u1 = (int)min(U, u0 + (t_hi - t));
                if (!epilogue(seg, tile, u0, u1)) break;
                ++seg;
                t += u1 - u0;
            }
        } else {
            // ----- dequant warps -----
            const int wg = warp >> 2;                                           // warpgroup: takes every kWG-th weight stage
            const int col = (warp & 3) * 32 + lane;                             // weight column in the tile = tensor-memory lane
            const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
            uint32_t si0 = 0, seg = 0;                                           // si0: weight stages consumed before this segment
            int pending = -1;                                                    // A stage written but not yet announced (Cfg::kDeferArrive)
            // the stores into tensor memory are complete -> the stage may be read by the MMAs
            auto announce = [&](int stage) {
                ptx::tc_wait_st();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&bars.ab_full[stage]), 0));
                    else ptx::mbar_arrive(ptx::smem_u32(&bars.ab_full[stage]));
                }
            };
            bool ok = true;
            for (long long t = t_lo; t < t_hi && ok;) {
                const long long tile = div_nn(t, U);
                const int u0 = (int)(t - tile * U);
                const int u1 = (int)min(U, u0 + (t_hi - t));
                // this warpgroup's units of the segment: those whose stage index is congruent to wg modulo kWG
                for (int u = u0 + (int)(((uint32_t)wg + (uint32_t)C::kWG - si0 % (uint32_t)C::kWG) % (uint32_t)C::kWG); u < u1; u += C::kWG) {
                    const uint32_t si = si0 + (uint32_t)(u - u0);
                    const uint32_t ws = si % C::kWStages, wph = (si / C::kWStages) & 1u;     // constants: multiply-shift, no division
                    if (C::kWGuard && !ptx::mbar_wait(ptx::smem_u32(&bars.w_empty[ws]), wph ^ 1u)) {   // see Cfg::kWStages
                        if (lane == 0) atomicExch(p.status, 35);
                        ok = false;
                        break;
                    }
                    if (!ptx::mbar_wait(ptx::smem_u32(&bars.w_full[ws]), wph)) {
                        if (lane == 0) atomicExch(p.status, 31);
                        ok = false;
                        break;
                    }
                    const uint32_t st = w_ring + ws * WS::kBytes;
                    const uint32_t g0 = p.gdiv((uint32_t)H * (uint32_t)u);
                    const uint32_t as = si % kABStages, aph = (si / kABStages) & 1u;
                    // polled before the first part is decoded, so that the answer costs no latency when it is needed
                    const bool free_early = ptx::mbar_test_wait(ptx::smem_u32(&bars.ab_free[as]), aph ^ 1u);
                    // scale and zero-point of this thread's column in row `row` of the stage's group box, both halves of a register
                    auto load_group = [&](uint32_t row, ColK& c) {
                        const uint32_t sz = ptx::lds32(st + WS::kS + row * 256 + (col & ~1) * 2) >> (16 * (col & 1));
                        const uint32_t zz = ptx::lds32(st + WS::kZ + row * 256 + (col & ~1) * 2) >> (16 * (col & 1));
                        c.s2 = prmt(sz, sz, 0x1010);
                        c.z2 = prmt(zz, zz, 0x1010);
                        c.zb = 0;
                    };
                    // fast mode needs: scale sign clear, zero-point an integer in [0, 512] ([0, 255] for the sparse format)
                    auto not_fast_bits = [&](const ColK& c) -> uint32_t {
                        const uint32_t zr = hadd2_u(hadd2_u(c.z2, kMagic1024), H2_N1024);
                        constexpr uint32_t kAdd = SPARSE ? 0x2407u : 0x1FFFu;
                        const uint32_t zlo = c.z2 & 0xFFFFu;
                        return ((zlo | ((zlo & 0x7FFFu) + kAdd) | c.s2) & 0x8000u) | (zr ^ c.z2);
                    };
                    // after the last read of the weight stage
                    auto release_weights = [&]() {
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bars.w_empty[ws]));
                    };
                    // before the first store into the A stage
                    auto acquire_a_stage = [&]() -> bool {
                        if (C::kDeferArrive && pending >= 0) announce(pending);       // before any wait: the MMAs must be able to go on
                        // the A stage (and its activation tile) is free once the MMAs of its previous use have completed
                        if (!free_early && !ptx::mbar_wait(ptx::smem_u32(&bars.ab_free[as]), aph ^ 1u)) {
                            if (lane == 0) atomicExch(p.status, 32);
                            return false;
                        }
                        ptx::tc_fence_after_sync();
                        return true;
                    };
                    // The parts are decoded in the fast mode by straight-line code, without a mode decision in between;
                    // whether every group of the unit really is in the fast mode (for every column of the warp) is
                    // voted once, when the last group has been read and before the weight stage is released.  If not,
                    // the unit is decoded again with a decision per part (the stores are simply overwritten).
                    bool redo = false;
                    {
                        ColK c;
                        uint32_t cur_row = 0xFFFFFFFFu, nf = 0;
#pragma unroll
                        for (int h = 0; h < H; ++h) {
                            // scale and zero-point change only where the group does (warp-uniform)
                            const uint32_t row = (h == 0) ? 0u : (p.gdiv((uint32_t)H * (uint32_t)u + (uint32_t)h) - g0);   // 0 .. H - 1
                            if (row != cur_row) {
                                cur_row = row;
                                load_group(row, c);
                                nf |= not_fast_bits(c);
                                if (SPARSE) c.zb = __half2uint_rz(__ushort_as_half((unsigned short)(c.z2 & 0xFFFFu))) * 0x01010101u;
                            }
                            if (h == H - 1 && __any_sync(0xFFFFFFFFu, nf != 0)) {
                                redo = true;
                                break;
                            }
                            uint32_t A[32];
                            F::template decode<MODE_FAST>(st + WS::kW + h * (F::WROWS * 512) + col * 4, st + WS::kMask + h * (F::MROWS * 512) + col * 4, c, A, lut);
                            if (h == H - 1) release_weights();
                            if (h == 0 && !acquire_a_stage()) { ok = false; break; }
                            ptx::tmem_st32(lane_addr + C::kACol0 + as * C::kAStageCols + h * 32, A);
                        }
                    }
                    if (redo && ok) {
                        // some group needs the general or the per-weight mode (rolled loop: three decode bodies in the
                        // instruction cache, not three per part)
                        ptx::tc_wait_st();
                        ColK c;
                        uint32_t cur_row = 0xFFFFFFFFu;
#pragma unroll 1
                        for (int h = 0; h < H; ++h) {
                            const uint32_t row = (h == 0) ? 0u : (p.gdiv((uint32_t)H * (uint32_t)u + (uint32_t)h) - g0);
                            if (row != cur_row) {
                                cur_row = row;
                                load_group(row, c);
                            }
                            const uint32_t wb = st + WS::kW + h * (F::WROWS * 512) + col * 4;
                            const uint32_t mb = st + WS::kMask + h * (F::MROWS * 512) + col * 4;
                            uint32_t A[32];
                            if (!__any_sync(0xFFFFFFFFu, not_fast_bits(c) != 0)) {
                                if (SPARSE) c.zb = __half2uint_rz(__ushort_as_half((unsigned short)(c.z2 & 0xFFFFu))) * 0x01010101u;
                                F::template decode<MODE_FAST>(wb, mb, c, A, lut);
                            } else {
                                c.zb = 0;
                                const bool lin = __hge(__ushort_as_half((unsigned short)(c.s2 & 0xFFFFu)), __ushort_as_half(0));
                                if (__all_sync(0xFFFFFFFFu, lin)) F::template decode<MODE_GENERAL>(wb, mb, c, A, lut);
                                else F::template decode<MODE_SLOW>(wb, mb, c, A, lut);
                            }
                            if (h == H - 1) release_weights();
                            ptx::tmem_st32(lane_addr + C::kACol0 + as * C::kAStageCols + h * 32, A);
                        }
                    }
                    if (!ok) break;
                    // (not deferred for the warpgroup's first stage: the pipeline is still filling and the MMA warp is waiting)
                    if (C::kDeferArrive && si >= (uint32_t)C::kWG) pending = (int)as;
                    else announce((int)as);
                }
                if (!ok) break;
                if (C::kDeferArrive && pending >= 0) { announce(pending); pending = -1; }
                if (!C::kEpiWarps && wg == 0) ok = epilogue(seg, tile, u0, u1);
                ++seg;
                si0 += (uint32_t)(u1 - u0);
                t += u1 - u0;
            }
        }
    }

    // ---- teardown: every role ends up here, also after a timed-out wait ----
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    if (PAIR) ptx::cluster_sync_all();       // neither CTA's barriers or tensor memory may go while the other can still reach them
    if (warp == kMma) {
        if (PAIR) ptx::tmem_dealloc_pair(tmem_base, C::kTmemCols);
        else ptx::tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// Sums the K parts written by umma_kernel (fp32, (part, row, S)) in part order, rounds once to fp16, and puts the
// scratch back to all-zero (the split-K reduction of the few-row shapes relies on that).  8 columns per thread.
// (no __restrict__ here or on umma_kernel's activations: both kernels may start while the kernel that writes what they
// read is still running, and a restrict-qualified pointer would allow the compiler to load above griddepcontrol.wait)
__global__ void kparts_reduce_kernel(float* parts, const OutMap om, int rows, int S, int kparts) {
    // (launched with programmatic stream serialization: the next kernel may be scheduled at once, this one touches
    // nothing before the kernel that wrote the parts has completed)
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int s8 = S / 8;
    const long long n8 = (long long)rows * s8;
    const size_t stride = (size_t)rows * S;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int f = 0; f < kparts; ++f) {
            float4* src = reinterpret_cast<float4*>(parts + f * stride + i * 8);
            const float4 a = src[0], c = src[1];
            acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
            acc[4] += c.x; acc[5] += c.y; acc[6] += c.z; acc[7] += c.w;
            src[0] = make_float4(0.f, 0.f, 0.f, 0.f);
            src[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        const long long row = i / s8;
        const int c8 = (int)(i - row * s8) * 8;
        const size_t at = (size_t)row * om.ld + om.col(c8);
        for (int d = 0; d < om.n_dst; ++d) *reinterpret_cast<uint4*>(om.dst[d] + at) = *reinterpret_cast<uint4*>(h);
    }
    if (om.n_dst > 1) __threadfence_system();        // as in umma_kernel's epilogue
}

// ---- host side -------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, found at run time so that the library does not link against libcuda.
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess && ptr)
            fn = (EncodeTiledFn)ptr;
        if (!fn) {
            (void)cudaGetLastError();
            void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
            if (h) fn = (EncodeTiledFn)dlsym(h, "cuTensorMapEncodeTiled");
        }
    }
    return fn;
}

// 2-D row-major tensor (rows, cols) of `elem_bytes` elements, box (box_rows, box_cols)
bool encode_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows, uint64_t cols,
               uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// what the last tcgen05 launch of this host thread chose: tile rows + 1000 if CTA pairs + 10000 * K parts (tests read it)
thread_local int g_last_shape = 0;

// Encoded tensor maps are a pure function of (base address, shape, box, swizzle): callers multiply with the same
// weight tensors over and over, so the maps are kept in a small direct-mapped table instead of being encoded by the
// driver five times per call (which costs more host time than the launch itself).
struct MapKey {
    const void* base;
    uint64_t rows, cols;
    uint32_t box_rows, box_cols;
    int dt, elem_bytes, swz;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols &&
               dt == o.dt && elem_bytes == o.elem_bytes && swz == o.swz;
    }
};
struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool valid;
};
constexpr int kMapSlots = 512;
std::mutex g_map_mutex;
MapSlot g_map_cache[kMapSlots];

bool encode_2d_cached(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows, uint64_t cols,
                      uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
    const MapKey key{base, rows, cols, box_rows, box_cols, (int)dt, elem_bytes, (int)swz};
    uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
    h ^= (rows * 0xC2B2AE3D27D4EB4Full) ^ (cols << 17) ^ ((uint64_t)box_rows << 40) ^ ((uint64_t)box_cols << 52) ^ (uint64_t)dt;
    MapSlot& slot = g_map_cache[(h >> 32) % kMapSlots];
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        if (slot.valid && slot.key == key) {
            *out = slot.map;
            return true;
        }
    }
    if (!encode_2d(out, base, dt, elem_bytes, rows, cols, box_rows, box_cols, swz)) return false;
    std::lock_guard<std::mutex> lock(g_map_mutex);
    slot.key = key;
    slot.map = *out;
    slot.valid = true;
    return true;
}

// The activations (rows, N) of the weight-streaming shapes seen as (N / 64 blocks, rows, 64 k): one copy fetches the
// `blocks` consecutive 64-k sub-tiles of a unit, each box_rows x 128 bytes in the 128-byte swizzle, one after the other.
bool encode_x_blocks_cached(CUtensorMap* out, const void* base, uint64_t rows, uint64_t n, uint32_t box_rows, uint32_t blocks) {
    const MapKey key{base, rows, n, box_rows, blocks, -3, 2, (int)CU_TENSOR_MAP_SWIZZLE_128B};
    uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
    h ^= (rows * 0xC2B2AE3D27D4EB4Full) ^ (n << 17) ^ ((uint64_t)box_rows << 40) ^ ((uint64_t)blocks << 52) ^ 0x33ull;
    MapSlot& slot = g_map_cache[(h >> 32) % kMapSlots];
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        if (slot.valid && slot.key == key) {
            *out = slot.map;
            return true;
        }
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(n / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)n * 2, 128};
    const cuuint32_t box[3] = {64, box_rows, blocks};
    const cuuint32_t estr[3] = {1, 1, 1};
    if (enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> lock(g_map_mutex);
    slot.key = key;
    slot.map = *out;
    slot.valid = true;
    return true;
}

constexpr long long kPartialWords = 148LL * 4 * 32 * 128;      // 64-bit words of partial tiles in the workspace (capi.cu sizes it)

// More than 32 rows and tiles that fill less than half of the GPU: cut K into parts so that
// tiles x parts CTAs (pairs) run, as long as every part keeps at least 4 stages and the partial outputs fit the scratch.
int choose_kparts(long long capacity, long long tiles, int U, long long rows, long long S) {
    if (tiles <= 0 || tiles * 2 > capacity) return 1;
    long long f = capacity / tiles;
    if (f > 8) f = 8;
    if (f > U / 4) f = U / 4;
    while (f > 1 && f * rows * S * 4 > kPartialWords * 8) --f;
    return f < 2 ? 1 : (int)f;
}

int launch_kparts_reduce(const UmmaParams& p, cudaStream_t stream, cudaError_t* cuda_err) {
    const long long n8 = (long long)p.rows * p.S / 8;
    long long blocks = (n8 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((unsigned)blocks, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kparts_reduce_kernel, p.partials, p.om, p.rows, p.S, p.kparts);
    if (e != cudaSuccess) { *cuda_err = e; return I4MM_ERR_LAUNCH; }
    count_launch();
    return I4MM_OK;
}

template <int BITS, bool SPARSE, int NT, bool PAIR, bool PERM = false>
int launch_nt(const UmmaParams& p_in, const __half* x, int n_groups, cudaStream_t stream, cudaError_t* cuda_err) {
    UmmaParams p = p_in;
    p.kparts = 1;
    using F = UFormat<BITS, SPARSE>;
    using C = Cfg<NT, PAIR>;
    constexpr int H = C::kHalves;
    p.U = (p.N + 64 * H - 1) / (64 * H);
    constexpr int kBStageBytes = H * (PAIR ? NT / 2 : NT) * 128;
    TensorMaps tm;
    const uint64_t R = SPARSE ? (uint64_t)p.N / 16 : (uint64_t)p.N * BITS / 32;
    bool ok = C::kStream ? encode_x_blocks_cached(&tm.x, x, p.rows, p.N, NT, H)
                         : encode_2d_cached(&tm.x, x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.rows, p.N, PAIR ? NT / 2 : NT, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    ok = ok && encode_2d_cached(&tm.w, p.matrix, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, R, p.S, H * F::WROWS, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (SPARSE)
        ok = ok && encode_2d_cached(&tm.m, p.mask, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, (uint64_t)p.N / 32, p.S, H * F::MROWS, 128,
                             CU_TENSOR_MAP_SWIZZLE_NONE);
    else
        tm.m = tm.w;
    ok = ok && encode_2d_cached(&tm.s, p.scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, n_groups, p.S, H, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
    ok = ok && encode_2d_cached(&tm.z, p.zeros, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, n_groups, p.S, H, 128, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!ok) return I4MM_ERR_DEVICE;

    const size_t smem = 1024 + (size_t)ABStages<NT, PAIR>::value * kBStageBytes + (size_t)C::kWStages * WStage<F, H>::kBytes +
                        (!C::kEpiTransposed ? 0 : PAIR ? NT * 256 : 4096 * ((C::kEpiGroups == 2 && NT < 256) ? 2 : 1)) +
                        (PERM ? (size_t)C::kXStaging * kBStageBytes : 0);
    auto kern = umma_kernel<BITS, SPARSE, NT, PAIR, PERM>;
    // per-device caches; atomics because two host threads may make their first call at once (both then compute the same values)
    static std::atomic<int> ctas_per_sm[16];
    static std::atomic<int> sm_count[16];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *cuda_err = e; return I4MM_ERR_LAUNCH; }
    dev &= 15;
    if (ctas_per_sm[dev] == 0) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { *cuda_err = e; return I4MM_ERR_LAUNCH; }
        // CTAs per SM: what the launch bounds and the shared-memory budget were sized for, capped by the tensor
        // memory (512 columns per SM).  The occupancy calculator is not used: it reports 1 for a kernel that
        // allocates tensor memory, whatever amount the kernel asks for at run time.
        int n = C::kMinBlocks, sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) { *cuda_err = e; return I4MM_ERR_LAUNCH; }
        const int tmem_limit = 512 / C::kTmemCols;
        if (n > tmem_limit) n = tmem_limit;
        const int smem_limit = (int)((227 * 1024) / (smem + 2048));
        if (n > smem_limit) n = smem_limit;
        sm_count[dev] = sms;
        ctas_per_sm[dev] = n > 0 ? n : 1;
    }
    if (PAIR) {
        // clusters of two CTAs; as many as can be resident at once, each walking its share of the pair tiles
        static std::atomic<int> max_clusters[16];
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.blockDim = dim3(C::kThreads, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = p.overlap ? 2 : 1;
        if (max_clusters[dev] == 0) {
            cfg.gridDim = dim3(2 * (sm_count[dev] / 2), 1, 1);
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
                (void)cudaGetLastError();
                n = sm_count[dev] / 2;
            }
            if (n > sm_count[dev] / 2) n = sm_count[dev] / 2;
            max_clusters[dev] = n;
        }
        long long clusters = max_clusters[dev];
        const long long tiles2 = (long long)p.MTILES * ((p.CT + 1) / 2);
        if (!C::kSplit && !p.accumulate)
            p.kparts = choose_kparts(clusters, tiles2, p.U, p.rows, p.S);
        const long long work = p.kparts > 1 ? tiles2 * p.kparts : tiles2 * (C::kSplit ? p.U : 1);
        if (C::kSplit && clusters > kPartialWords / C::kSlotElems / 2) clusters = kPartialWords / C::kSlotElems / 2;
        if (clusters > work || p.kparts > 1) clusters = work;
        cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
        e = cudaLaunchKernelEx(&cfg, kern, tm, p, x);
        if (e != cudaSuccess) { *cuda_err = e; return I4MM_ERR_LAUNCH; }
        count_launch();
        g_last_shape = NT + 1000 + 10000 * (p.kparts > 1 ? p.kparts : 0);
        if (p.kparts > 1) return launch_kparts_reduce(p, stream, cuda_err);
        return I4MM_OK;
    }
    const long long n_tiles = (long long)p.MTILES * p.CT;
    long long grid = (long long)sm_count[dev] * ctas_per_sm[dev];
    if (!C::kSplit && !p.accumulate)
        p.kparts = choose_kparts(grid, n_tiles, p.U, p.rows, p.S);
    const long long work = p.kparts > 1 ? n_tiles * p.kparts : C::kSplit ? n_tiles * p.U : n_tiles;
    if (grid > work || p.kparts > 1) grid = work;
    if (C::kSplit && grid > kPartialWords / C::kSlotElems) grid = kPartialWords / C::kSlotElems;   // one partial tile per CTA in the scratch
    {
        // With `overlap` the kernel may start while the kernel before it in the stream is still running: its set-up and
        // its copies of the weight-side tensors (which the caller has declared not to be written by that kernel) overlap
        // that kernel's tail; everything that reads activations, reads or writes outputs or touches the scratch waits
        // for that kernel inside (griddepcontrol.wait).
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.gridDim = dim3((unsigned)grid, 1, 1);
        cfg.blockDim = dim3(C::kThreads, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = p.overlap ? 1 : 0;
        e = cudaLaunchKernelEx(&cfg, kern, tm, p, x);
    }
    if (e != cudaSuccess) { *cuda_err = e; return I4MM_ERR_LAUNCH; }
    count_launch();
    g_last_shape = NT + 10000 * (p.kparts > 1 ? p.kparts : 0);
    if (p.kparts > 1) return launch_kparts_reduce(p, stream, cuda_err);
    return I4MM_OK;
}

// Rows per tile (the MMA's N).  Few rows: the smallest tile that holds them.  Many rows: the tile height that
// minimises (waves of tiles over the SMs) x (time per tile), so that e.g. 320 tiles of 256 rows (2.2 waves on 148
// SMs) become 440 tiles of 192 rows (3.0 waves) when that is faster.
int choose_tile_rows(int rows, int col_tiles, int sms, int max_nt) {
    if (rows <= 16) return 16;
    if (rows <= 32) return 32;
    if (rows <= 64) return 64;
    if (rows <= 128) return 128;
    const int cand[4] = {256, 224, 192, 160};
    int best = max_nt < 256 ? 192 : 256;
    long long best_cost = -1;
    for (int i = 0; i < 4; ++i) {
        const int nt = cand[i];
        if (nt > max_nt) continue;
        const long long tiles = (long long)((rows + nt - 1) / nt) * col_tiles;
        const long long waves = (tiles + sms - 1) / sms;
        const long long cost = waves * (nt + 24);          // + per-tile fill / drain, in row units
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = nt; }
    }
    return best;
}

constexpr int kPairMinRows = 128;

template <int BITS, bool SPARSE>
int launch_fmt(UmmaParams& p, const __half* x, int n_groups, int pair_mode, int force_nt, cudaStream_t stream, cudaError_t* cuda_err) {
    static std::atomic<int> sms_of[16];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    dev &= 15;
    int sms = sms_of[dev].load();
    if (sms == 0) {
        int n = 0;
        sms = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
        sms_of[dev].store(sms);
    }
    // 128 rows or more (the whole-tile configurations) run as CTA pairs, two SMs per MMA, unless the caller asked for single CTAs
    const bool pair = pair_mode == 0 && (force_nt ? force_nt >= 128 : p.rows >= kPairMinRows);
    // Stores into several GPUs' buffers (the gathering multiply) make the epilogue of a tile last longer than the tile's
    // MMAs.  Under exactly that condition the CTA-pair instances with 224 and 256 rows per tile (two dequant warpgroups,
    // three weight stages) were seen, on 8 GPUs, to produce now and then one wrong block of 32 columns x one row tile
    // (one warp's weights of one 128-k unit); the 192-row pair instance (four warpgroups, six stages) and the single-CTA
    // 224 / 256 instances were not, and no run with one destination ever was.  The cause has not been found, so the
    // gathering multiply keeps to tiles of at most 192 rows when it runs as CTA pairs.
    const int max_nt = (pair && p.om.n_dst > 1) ? 192 : 256;
    const int nt = force_nt ? force_nt : pair ? choose_tile_rows(p.rows, (p.CT + 1) / 2, sms / 2, max_nt) : choose_tile_rows(p.rows, p.CT, sms, 256);
    p.MTILES = (p.rows + nt - 1) / nt;
    if (pair) {
        switch (nt) {
            case 128: return launch_nt<BITS, SPARSE, 128, true>(p, x, n_groups, stream, cuda_err);
            case 160: return launch_nt<BITS, SPARSE, 160, true>(p, x, n_groups, stream, cuda_err);
            case 192: return launch_nt<BITS, SPARSE, 192, true>(p, x, n_groups, stream, cuda_err);
            case 224: return launch_nt<BITS, SPARSE, 224, true>(p, x, n_groups, stream, cuda_err);
            case 256: return launch_nt<BITS, SPARSE, 256, true>(p, x, n_groups, stream, cuda_err);
            default: break;
        }
    }
    switch (nt) {
        case 16:
            // up to 8 rows of dense int4: the k order that needs no byte shuffles (more rows would cost the one warp
            // that reorders the activations more per unit than the unit takes)
            if (BITS == 4 && !SPARSE && p.rows <= 8) return launch_nt<BITS, SPARSE, 16, false, BITS == 4 && !SPARSE>(p, x, n_groups, stream, cuda_err);
            return launch_nt<BITS, SPARSE, 16, false>(p, x, n_groups, stream, cuda_err);
        case 32: return launch_nt<BITS, SPARSE, 32, false>(p, x, n_groups, stream, cuda_err);
        case 64: return launch_nt<BITS, SPARSE, 64, false>(p, x, n_groups, stream, cuda_err);
        case 128: return launch_nt<BITS, SPARSE, 128, false>(p, x, n_groups, stream, cuda_err);
        case 160: return launch_nt<BITS, SPARSE, 160, false>(p, x, n_groups, stream, cuda_err);
        case 192: return launch_nt<BITS, SPARSE, 192, false>(p, x, n_groups, stream, cuda_err);
        case 224: return launch_nt<BITS, SPARSE, 224, false>(p, x, n_groups, stream, cuda_err);
        default: return launch_nt<BITS, SPARSE, 256, false>(p, x, n_groups, stream, cuda_err);
    }
}

}  // namespace

int umma_last_shape() { return g_last_shape; }
void umma_clear_last_shape() { g_last_shape = 0; }

bool umma_supported(int bits, bool sparse, int total_rows, int N, int S) {
    (void)bits; (void)sparse; (void)S;
    return total_rows >= 1 && N >= 64 && encode_tiled_fn() != nullptr;
}

int umma_launch(int bits, bool sparse, const StreamParams& sp, int total_rows, int n_groups, int group_size, int cta_pairs /* 0 by shape, 1 never */,
                int force_nt /* 0 = by shape */, int overlap, cudaStream_t stream, cudaError_t* cuda_err) {
    (void)group_size;
    UmmaParams p{};
    p.om = sp.om;
    p.matrix = sp.matrix;
    p.mask = sp.mask;
    p.scales = sp.scales;
    p.zeros = sp.zeros;
    p.partials = sp.partials;
    p.status = sp.status;
    p.rows = total_rows;
    p.N = sp.N;
    p.S = sp.S;
    p.U = 0;                      // set per configuration (units of 128 k or 256 k)
    p.CT = sp.CT;
    p.accumulate = sp.accumulate;
    p.overlap = overlap;
    p.gdiv = sp.gdiv;
    if (sparse) return launch_fmt<4, true>(p, sp.x, n_groups, cta_pairs, force_nt, stream, cuda_err);
    if (bits == 4) return launch_fmt<4, false>(p, sp.x, n_groups, cta_pairs, force_nt, stream, cuda_err);
    if (bits == 3) return launch_fmt<3, false>(p, sp.x, n_groups, cta_pairs, force_nt, stream, cuda_err);
    return launch_fmt<2, false>(p, sp.x, n_groups, cta_pairs, force_nt, stream, cuda_err);
}

}  // namespace i4mm
