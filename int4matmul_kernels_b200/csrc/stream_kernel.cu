// Weight-streaming kernel for few activation rows (matvec and skinny matmul): HBM-bound.
//
// Replaces MVA_Int4_Half (matvec_kernel.cu:198-267) and, for small M, MMA_Int4_Half
// (matmul_kernel.cu:219-333).  Design:
//   * a producer warp streams (128 n x 128 columns) k-blocks of packed words, their scales / zeros and the
//     activation slice into a ring of shared-memory stages with bulk async copies (TMA) that complete on
//     mbarriers, so the bytes in flight per SM are set by the ring depth and not by registers or occupancy;
//   * every consumer lane reads packed words with 128-bit shared loads: one uint4 = 4 adjacent S columns of
//     one packed row; the 4 lanes of a quad take 4 different packed rows, the 8 quads 8 column quartets;
//   * nibbles become fp16 pairs in registers with the 0x6400 mantissa trick (one LOP3 per pair), then
//     (q - zero) * scale exactly as the reference rounds it (sub, then mul);
//   * the multiply-accumulate runs on mma.sync m16n8k16 (fp16 x fp16 -> fp32): the 16 "rows" of A are
//     16 weight columns, the 8 "columns" of B are 8 activation rows, k walks the reduction dim in a
//     permuted order that both operands share, so no data is shuffled between lanes;
//   * the (column tile, k-block) space is cut into equal contiguous ranges, one per CTA, and ranges that
//     split a column tile are summed through fp32 scratch in a fixed order by the last CTA to arrive
//     (no atomics on data, bit-reproducible, no second launch).
#include <atomic>

#include "common.cuh"
#include "ptx.cuh"

namespace i4mm {

namespace {

constexpr int kCTile = 128;    // output columns per CTA tile (4 warps across)

enum : int { MODE_FAST = 0, MODE_GENERAL = 1, MODE_SLOW = 2 };

// (a & b) | c in one LOP3; b and c are kept in registers (an immediate form needs two instructions)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- per-column dequantisation constants ---------------------------------------------------------
struct ColQ {
    uint32_t s2;      // scale in both halves
    uint32_t z2;      // zero in both halves (general / slow modes)
    uint32_t off[4];  // MODE_FAST: -(1024 * mul_j + zero) for shift class j
    uint32_t zb;      // MODE_FAST, sparse: the integer zero as a byte (replicated)
};

// Multiplier and bias that turn (1024 + q * 2^shift) into q exactly, for the field positions a format uses:
//   NJ = 2 (int4): fields at bits 0, 4 of each 16-bit half;  NJ = 4 (int2): bits 0, 2, 4, 6;
//   NJ = 3 (int3): bits 0, 3, 6;  NJ = 1 (sparse int4 through bytes): bit 0 only.
__device__ __forceinline__ constexpr uint32_t shift_mul(int nj, int j) {
    return j == 0 ? H2_ONE
         : nj == 2 ? H2_1_16
         : nj == 4 ? (j == 1 ? H2_1_4 : j == 2 ? H2_1_16 : H2_1_64)
         : (j == 1 ? H2_1_8 : H2_1_64);
}
__device__ __forceinline__ constexpr uint32_t shift_base(int nj, int j) {
    return j == 0 ? H2_N1024
         : nj == 2 ? H2_N64
         : nj == 4 ? (j == 1 ? H2_N256 : j == 2 ? H2_N64 : H2_N16)
         : (j == 1 ? H2_N128 : H2_N16);
}

// sz = (scale bits, zero bits) of one column, each duplicated into both halves already
template <int NJ, int MODE, bool SPARSE>
__device__ __forceinline__ void make_colq(ColQ& c, uint32_t s2, uint32_t z2) {
    c.s2 = s2;
    c.z2 = z2;
    if (MODE == MODE_FAST) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) c.off[j] = hsub2_u(shift_base(NJ, j), z2);
        if (SPARSE) c.zb = __half2uint_rz(__ushort_as_half((unsigned short)(z2 & 0xFFFFu))) * 0x01010101u;
    } else if (SPARSE) {
        c.zb = 0;
    }
}

template <int NJ, int MODE, bool SPARSE>
__device__ __forceinline__ void make_colqs(ColQ (&cq)[4], uint2 s, uint2 z) {
    make_colq<NJ, MODE, SPARSE>(cq[0], dup_lo(s.x), dup_lo(z.x));
    make_colq<NJ, MODE, SPARSE>(cq[1], dup_hi(s.x), dup_hi(z.x));
    make_colq<NJ, MODE, SPARSE>(cq[2], dup_lo(s.y), dup_lo(z.y));
    make_colq<NJ, MODE, SPARSE>(cq[3], dup_hi(s.y), dup_hi(z.y));
}

// v holds (1024 + q * 2^shift_j) in both halves; returns the fp16 weights.
template <int BITS, int NJ, int MODE>
__device__ __forceinline__ uint32_t finish(uint32_t v, int j, const ColQ& c) {
    if (MODE == MODE_FAST) {
        const uint32_t t = (j == 0) ? hadd2_u(v, c.off[0]) : hfma2_u(v, shift_mul(NJ, j), c.off[j]);
        return hmul2_u(t, c.s2);
    }
    const uint32_t q = (j == 0) ? hadd2_u(v, shift_base(NJ, 0))
                                : hfma2_u(v, shift_mul(NJ, j), shift_base(NJ, j));
    if (MODE == MODE_GENERAL) return hmul2_u(hsub2_u(q, c.z2), c.s2);
    // either coding, per column
    const __half2 qh = u32_as_h2(q);
    const __half s = __ushort_as_half((unsigned short)(c.s2 & 0xFFFFu));
    const __half z = __ushort_as_half((unsigned short)(c.z2 & 0xFFFFu));
    const __half lo = dequant_dynamic<BITS>(__half2uint_rz(__low2half(qh)), s, z);
    const __half hi = dequant_dynamic<BITS>(__half2uint_rz(__high2half(qh)), s, z);
    return h2_as_u32(__halves2half2(lo, hi));
}

// Non-zero if this lane's 4 (scale, zero) pairs rule out MODE_FAST: a scale with the sign bit set (exponent
// coding, or -0), or a zero-point that is not an integer of [0, LIM] (LIM = 512, or 255 for the sparse format
// whose fast path carries the zero-point in a byte).  Integer ALU ops on the raw fp16 bits, two halves at a time.
template <bool SPARSE>
__device__ __forceinline__ uint32_t lane_not_fast(uint2 s, uint2 z) {
    // integer test: (z + 1024) - 1024 == z holds exactly for the integers of [0, 1024]
    const uint32_t r0 = hadd2_u(hadd2_u(z.x, kMagic1024), H2_N1024), r1 = hadd2_u(hadd2_u(z.y, kMagic1024), H2_N1024);
    // range test: bit 15 of (m + (0x7FFF - LIMBITS)) is set iff the 15-bit magnitude m exceeds LIMBITS; sign bits pass through
    constexpr uint32_t kAdd = SPARSE ? 0x24072407u /* 0x7FFF - 0x5BF8 (255) */ : 0x1FFF1FFFu /* 0x7FFF - 0x6000 (512) */;
    const uint32_t rz0 = z.x | ((z.x & 0x7FFF7FFFu) + kAdd), rz1 = z.y | ((z.y & 0x7FFF7FFFu) + kAdd);
    return ((rz0 | rz1 | s.x | s.y) & 0x80008000u) | (r0 ^ z.x) | (r1 ^ z.y);
}
// Only evaluated when some lane is not fast: is every scale of this lane linear (>= 0, -0 included)?
__device__ __forceinline__ bool lane_linear(uint2 s) {
    const __half2 zero2 = u32_as_h2(0u);
    return __hbge2(u32_as_h2(s.x), zero2) && __hbge2(u32_as_h2(s.y), zero2);
}

// ---- formats -----------------------------------------------------------------------------------------
// Each format says what one lane loads for one k-block (128 n x its 4 columns) and how it turns one
// "step" of that into NP fp16 pairs per column, in an order the activation side mirrors.

// 16-entry table for the sparse expansion, indexed by 4 mask bits:
//   x: PRMT selector that deposits the next popc(mask) bytes at the kept positions (dropped -> byte 4)
//      | (4 * popc) << 16
//   y, z: pair masks (0xFFFF per kept position) for positions (0,1) and (2,3)
__device__ __forceinline__ uint4 sparse_lut_entry(int mn) {
    uint32_t sel = 0, rank = 0, pm[2] = {0, 0};
    for (int j = 0; j < 4; ++j) {
        if (mn & (1 << j)) {
            sel |= rank << (4 * j);
            pm[j >> 1] |= 0xFFFFu << (16 * (j & 1));
            ++rank;
        } else {
            sel |= 4u << (4 * j);
        }
    }
    return make_uint4(sel | ((4 * rank) << 16), pm[0], pm[1], 0);
}

__device__ __forceinline__ uint32_t pick(const uint4& v, int c) { return c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w; }

// Row pitches inside a stage are padded so that the 8 lanes served by one shared-memory wavefront (2 quads x
// 4 lanes, reading 16 bytes each from 4 different rows) fall into 8 different 16-byte bank groups:
// packed rows 544 B (528 B where a lane reads rows 2t, 2t+1), mask rows 544 B, activation rows 320 B.
constexpr int kMaskPitch = 544;
constexpr int kXPitch = 320;

template <int BITS, bool SPARSE>
struct Format;

// ---------------- dense int4: 8 n per word; lane (g, t) takes packed rows kb*16 + 4*step + t ----------------
template <>
struct Format<4, false> {
    static constexpr int NJ = 2;
    static constexpr int NH = 2;        // (scale, zero) sets per k-block: one per 64-n half
    static constexpr int STEPS = 4;     // lane chunks per k-block
    static constexpr int NP = 4;        // fp16 pairs per column per step
    static constexpr int XREGS = 4;     // activation registers per step (8 halves)
    static constexpr int XSTEP = 32;    // activation elements between steps
    static constexpr int XLANE = 8;     // activation elements between lanes of a quad
    static constexpr bool LANE_TAIL = false;
    static constexpr int WROWS = 16;    // packed rows per k-block
    static constexpr int WPITCH = 544;   // bytes between packed rows in shared memory
    static constexpr int MROWS = 0;     // mask rows per k-block
    struct Frag { uint4 w[4]; uint2 s[2], z[2]; };

    // wbase = shared address of this lane's 16 bytes in packed row 0 of the stage
    __device__ static __forceinline__ void load_smem(Frag& f, uint32_t wbase, uint32_t, int t, bool tail, bool) {
        f.w[0] = ptx::lds128(wbase + (0 + t) * WPITCH);
        f.w[1] = ptx::lds128(wbase + (4 + t) * WPITCH);
        if (!tail) {
            f.w[2] = ptx::lds128(wbase + (8 + t) * WPITCH);
            f.w[3] = ptx::lds128(wbase + (12 + t) * WPITCH);
        }
    }
    template <int MODE>
    __device__ static __forceinline__ void decode(const Frag& f, int step, int c, const ColQ& q, uint32_t (&P)[NP], const uint4*) {
        decode_word<MODE>(pick(f.w[step], c), q, P);
    }
    template <int MODE>
    __device__ static __forceinline__ void decode_word(uint32_t w, const ColQ& q, uint32_t (&P)[NP]) {
        const uint32_t hi = w >> 8;
        P[0] = finish<4, NJ, MODE>(and_or(w, 0x000F000Fu, kMagic1024), 0, q);    // (n0, n4)
        P[1] = finish<4, NJ, MODE>(and_or(w, 0x00F000F0u, kMagic1024), 1, q);    // (n1, n5)
        P[2] = finish<4, NJ, MODE>(and_or(hi, 0x000F000Fu, kMagic1024), 0, q);   // (n2, n6)
        P[3] = finish<4, NJ, MODE>(and_or(hi, 0x00F000F0u, kMagic1024), 1, q);   // (n3, n7)
    }
    __device__ static __forceinline__ void xpairs(const uint32_t (&xr)[XREGS], uint32_t (&X)[NP]) {
        X[0] = prmt(xr[0], xr[2], 0x5410);
        X[1] = prmt(xr[0], xr[2], 0x7632);
        X[2] = prmt(xr[1], xr[3], 0x5410);
        X[3] = prmt(xr[1], xr[3], 0x7632);
    }
};

// ---------------- dense int2: 16 n per word; lane takes packed rows kb*8 + 4*step + t ----------------
template <>
struct Format<2, false> {
    static constexpr int NJ = 4;
    static constexpr int NH = 2;
    static constexpr int STEPS = 2;
    static constexpr int NP = 8;
    static constexpr int XREGS = 8;
    static constexpr int XSTEP = 64;
    static constexpr int XLANE = 16;
    static constexpr bool LANE_TAIL = false;
    static constexpr int WROWS = 8;
    static constexpr int MROWS = 0;
    static constexpr int WPITCH = 544;   // bytes between packed rows in shared memory
    struct Frag { uint4 w[2]; uint2 s[2], z[2]; };

    __device__ static __forceinline__ void load_smem(Frag& f, uint32_t wbase, uint32_t, int t, bool tail, bool) {
        f.w[0] = ptx::lds128(wbase + (0 + t) * WPITCH);
        if (!tail) f.w[1] = ptx::lds128(wbase + (4 + t) * WPITCH);
    }
    template <int MODE>
    __device__ static __forceinline__ void decode(const Frag& f, int step, int c, const ColQ& q, uint32_t (&P)[NP], const uint4*) {
        decode_word<MODE>(pick(f.w[step], c), q, P);
    }
    template <int MODE>
    __device__ static __forceinline__ void decode_word(uint32_t w, const ColQ& q, uint32_t (&P)[NP]) {
        const uint32_t hi = w >> 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t m = 0x00030003u << (2 * j);
            P[j] = finish<2, NJ, MODE>(and_or(w, m, kMagic1024), j, q);        // (n_j,   n_{j+8})
            P[4 + j] = finish<2, NJ, MODE>(and_or(hi, m, kMagic1024), j, q);   // (n_{4+j}, n_{12+j})
        }
    }
    __device__ static __forceinline__ void xpairs(const uint32_t (&xr)[XREGS], uint32_t (&X)[NP]) {
#pragma unroll
        for (int p = 0; p < 8; ++p) X[p] = prmt(xr[p >> 1], xr[4 + (p >> 1)], (p & 1) ? 0x7632 : 0x5410);
    }
};

// ---------------- dense int3: 32 n per 3 words; lane takes the 32-block kb*4 + t ----------------
template <>
struct Format<3, false> {
    static constexpr int NJ = 3;
    static constexpr int NH = 1;        // one set per lane: its block lies in one 64-n half
    static constexpr int STEPS = 1;
    static constexpr int NP = 16;
    static constexpr int XREGS = 16;
    static constexpr int XSTEP = 0;
    static constexpr int XLANE = 32;
    static constexpr bool LANE_TAIL = true;   // in a half k-block lanes t >= 2 have no data
    static constexpr int WROWS = 12;
    static constexpr int WPITCH = 544;   // bytes between packed rows in shared memory
    static constexpr int MROWS = 0;
    struct Frag { uint4 w[3]; uint2 s[1], z[1]; };

    __device__ static __forceinline__ void load_smem(Frag& f, uint32_t wbase, uint32_t, int t, bool, bool lane_ok) {
#pragma unroll
        for (int j = 0; j < 3; ++j) f.w[j] = lane_ok ? ptx::lds128(wbase + (3 * t + j) * WPITCH) : make_uint4(0, 0, 0, 0);
    }
    // pair index p = 3 * wp + f  ->  (n, n') = (6 wp + f, 6 wp + 3 + f); p = 15 -> (30, 31)
    __device__ static __forceinline__ constexpr int pair_lo(int p) { return p == 15 ? 30 : 6 * (p / 3) + (p % 3); }
    __device__ static __forceinline__ constexpr int pair_hi(int p) { return p == 15 ? 31 : 6 * (p / 3) + 3 + (p % 3); }

    template <int MODE>
    __device__ static __forceinline__ void decode(const Frag& f, int, int c, const ColQ& q, uint32_t (&P)[NP], const uint4*) {
        const uint32_t w0 = pick(f.w[0], c), w1 = pick(f.w[1], c), w2 = pick(f.w[2], c);
        // X[wp]: low half = 9-bit window 2wp of the 96-bit stream at bits 0..8, high half = window 2wp+1 at bits 16..24
        uint32_t X[5];
        X[0] = prmt(w0, w0 << 7, 0x7610);                                  // stream bits 0.., 9..
        X[1] = prmt(w0 >> 18, __funnelshift_r(w0, w1, 11), 0x7610);        // 18.., 27..
        X[2] = prmt(w1 >> 4, w1 << 3, 0x7610);                             // 36.., 45..
        X[3] = prmt(w1 >> 22, __funnelshift_r(w1, w2, 15), 0x7610);        // 54.., 63..
        X[4] = prmt(w2 >> 8, w2 >> 1, 0x7610);                             // 72.., 81..
        const uint32_t last = prmt(w2 >> 26, w2 >> 13, 0x7610);            // 90.., 93..
#pragma unroll
        for (int wp = 0; wp < 5; ++wp) {
            P[3 * wp + 0] = finish<3, NJ, MODE>(and_or(X[wp], 0x00070007u, kMagic1024), 0, q);
            P[3 * wp + 1] = finish<3, NJ, MODE>(and_or(X[wp], 0x00380038u, kMagic1024), 1, q);
            P[3 * wp + 2] = finish<3, NJ, MODE>(and_or(X[wp], 0x01C001C0u, kMagic1024), 2, q);
        }
        P[15] = finish<3, NJ, MODE>(and_or(last, 0x00070007u, kMagic1024), 0, q);
    }
    __device__ static __forceinline__ void xpairs(const uint32_t (&xr)[XREGS], uint32_t (&X)[NP]) {
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            const int a = pair_lo(p), b = pair_hi(p);
            const uint32_t sel = ((a & 1) ? 0x32u : 0x10u) | (((b & 1) ? 0x76u : 0x54u) << 8);
            X[p] = prmt(xr[a >> 1], xr[b >> 1], sel);
        }
    }
};

// ---------------- 16:32 sparse int4: 32 n per (64-bit compacted word, 32-bit mask); lane takes block kb*4 + t ----------------
template <>
struct Format<4, true> {
    static constexpr int NJ = 1;
    static constexpr int NH = 1;
    static constexpr int STEPS = 1;
    static constexpr int NP = 16;
    static constexpr int XREGS = 16;
    static constexpr int XSTEP = 0;
    static constexpr int XLANE = 32;
    static constexpr bool LANE_TAIL = true;
    static constexpr int WROWS = 8;
    static constexpr int MROWS = 4;
    static constexpr int WPITCH = 528;   // bytes between packed rows in shared memory
    struct Frag { uint4 w[2]; uint4 m; uint2 s[1], z[1]; };

    __device__ static __forceinline__ void load_smem(Frag& f, uint32_t wbase, uint32_t mbase, int t, bool, bool lane_ok) {
        f.w[0] = lane_ok ? ptx::lds128(wbase + (2 * t) * WPITCH) : make_uint4(0, 0, 0, 0);
        f.w[1] = lane_ok ? ptx::lds128(wbase + (2 * t + 1) * WPITCH) : make_uint4(0, 0, 0, 0);
        f.m = lane_ok ? ptx::lds128(mbase + t * kMaskPitch) : make_uint4(0, 0, 0, 0);
    }
    template <int MODE>
    __device__ static __forceinline__ void decode(const Frag& f, int, int c, const ColQ& q, uint32_t (&P)[NP], const uint4* lut) {
        uint32_t lo = pick(f.w[0], c), hi = pick(f.w[1], c);
        const uint32_t m = pick(f.m, c);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            const uint4 e = lut[(m >> (4 * ch)) & 0xFu];
            uint32_t v = lo & 0xFFFFu;                       // next 4 compacted nibbles
            v = (v | (v << 8)) & 0x00FF00FFu;
            v = (v | (v << 4)) & 0x0F0F0F0Fu;                // one nibble per byte
            const uint32_t dep = prmt(v, q.zb, e.x & 0xFFFFu);   // kept -> its nibble, dropped -> zero-point byte
            uint32_t a = finish<4, NJ, MODE>(prmt(dep, 0x64646464u, 0x5140), 0, q);
            uint32_t b = finish<4, NJ, MODE>(prmt(dep, 0x64646464u, 0x7362), 0, q);
            if (MODE != MODE_FAST) { a &= e.y; b &= e.z; }   // exact zeros at dropped positions
            P[2 * ch] = a;
            P[2 * ch + 1] = b;
            const uint32_t sh = e.x >> 16;
            lo = __funnelshift_r(lo, hi, sh);
            hi >>= sh;
        }
    }
    __device__ static __forceinline__ void xpairs(const uint32_t (&xr)[XREGS], uint32_t (&X)[NP]) {
#pragma unroll
        for (int p = 0; p < 16; ++p) X[p] = xr[p];
    }
};

// ---- stage layout ----------------------------------------------------------------------------------------
// One stage = one k-block (128 n) of one column tile (128 columns):
//   W   : F::WROWS packed rows of 512 B at pitch F::WPITCH   (+ F::MROWS mask rows for the sparse format)
//   SZ  : scales set 0, zeros set 0, scales set 1, zeros set 1, 256 B each (set 1 only if the k-block spans 2 groups)
//   X   : 8 * MT activation rows of 256 B at pitch 320 B (only rows < p.rows are ever written; the others feed output rows
//         that are never stored)
template <class F, int MT>
struct StageLayout {
    static constexpr int kW = 0;
    static constexpr int kMask = kW + F::WROWS * F::WPITCH;
    static constexpr int kSZ = kMask + F::MROWS * kMaskPitch;
    static constexpr int kX = kSZ + 4 * 256;
    static constexpr int kBytes = kX + 8 * MT * kXPitch;
};

struct KBlockInfo {     // what both the producer and the consumers derive from (kb) alone
    bool tail;          // last k-block of an N that is not a multiple of 128: only its first 64 n exist
    bool same;          // both 64-n halves use one (scale, zero) group
    uint32_t g0, g1;
};
__device__ __forceinline__ KBlockInfo kblock_info(const StreamParams& p, int kb) {
    KBlockInfo i;
    i.tail = (kb == p.KB - 1) && (p.N & 127);
    i.g0 = p.gdiv(2u * kb);
    i.g1 = i.tail ? i.g0 : p.gdiv(2u * kb + 1u);
    i.same = i.g0 == i.g1;
    return i;
}

// ---- consumer: one k-block of one warp, read from shared memory ---------------------------------------
struct LanePos {
    int g, t;          // quad index 0..7, lane in quad 0..3
    uint32_t coff;     // byte offset of this lane's 4 columns inside a 512-byte packed row: (wc * 32 + 4 g) * 4
};

template <class F, int BITS, bool SPARSE, int MT, int MODE>
__device__ __forceinline__ void compute_mode(const typename F::Frag& f, const KBlockInfo& info, uint32_t stage,
                                             const LanePos& L, float (&acc)[MT][2][4], const uint4* lut) {
    using SL = StageLayout<F, MT>;
    ColQ cq[4];
    make_colqs<F::NJ, MODE, SPARSE>(cq, f.s[0], f.z[0]);
    constexpr int SPH = F::STEPS / F::NH;
#pragma unroll
    for (int h = 0; h < F::NH; ++h) {
        if (h == 1) {
            if (info.tail) break;
            if (!info.same) make_colqs<F::NJ, MODE, SPARSE>(cq, f.s[F::NH - 1], f.z[F::NH - 1]);
        }
#pragma unroll
        for (int sj = 0; sj < SPH; ++sj) {
            const int step = h * SPH + sj;
            uint32_t X[MT][F::NP];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t xr[F::XREGS];
                const uint32_t xa = stage + SL::kX + (mt * 8 + L.g) * kXPitch + (step * F::XSTEP + L.t * F::XLANE) * 2;
#pragma unroll
                for (int i = 0; i < F::XREGS / 4; ++i) {
                    const uint4 v = ptx::lds128(xa + 16 * i);
                    xr[4 * i + 0] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
                }
                F::xpairs(xr, X[mt]);
            }
#pragma unroll
            for (int cp = 0; cp < 2; ++cp) {
                uint32_t Pa[F::NP], Pb[F::NP];
                F::template decode<MODE>(f, step, 2 * cp, cq[2 * cp], Pa, lut);
                F::template decode<MODE>(f, step, 2 * cp + 1, cq[2 * cp + 1], Pb, lut);
#pragma unroll
                for (int ks = 0; ks < F::NP / 2; ++ks) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        mma16816(acc[mt][cp], Pa[2 * ks], Pb[2 * ks], Pa[2 * ks + 1], Pb[2 * ks + 1],
                                 X[mt][2 * ks], X[mt][2 * ks + 1]);
                }
            }
        }
    }
}

template <class F, int BITS, bool SPARSE, int MT>
__device__ __forceinline__ void consume_stage(const KBlockInfo& info, uint32_t stage, const LanePos& L,
                                              float (&acc)[MT][2][4], const uint4* lut) {
    using SL = StageLayout<F, MT>;
    typename F::Frag f;
    const bool lane_ok = !(F::LANE_TAIL && info.tail && L.t >= 2);
    F::load_smem(f, stage + SL::kW + L.coff, stage + SL::kMask + L.coff, L.t, info.tail, lane_ok);
    {
        // scale / zero of this lane's 4 columns: set 0 for the first 64-n half, set 1 for the second
        const uint32_t so = stage + SL::kSZ + (L.coff >> 1);
        if (F::NH == 2) {
            f.s[0] = ptx::lds64(so);
            f.z[0] = ptx::lds64(so + 256);
            if (!info.same) {
                f.s[F::NH - 1] = ptx::lds64(so + 512);
                f.z[F::NH - 1] = ptx::lds64(so + 768);
            }
        } else {
            const uint32_t set = (!info.same && L.t >= 2) ? 512u : 0u;   // lanes t >= 2 work in the second half
            f.s[0] = lane_ok ? ptx::lds64(so + set) : make_uint2(0, 0);  // scale 0: a lane without data adds nothing
            f.z[0] = lane_ok ? ptx::lds64(so + set + 256) : make_uint2(0, 0);
        }
    }
    // one mode for the whole warp: the cheapest that is exact for every lane
    uint32_t not_fast = lane_not_fast<SPARSE>(f.s[0], f.z[0]);
    if (F::NH == 2 && !info.same) not_fast |= lane_not_fast<SPARSE>(f.s[F::NH - 1], f.z[F::NH - 1]);
    if (!__any_sync(0xFFFFFFFFu, not_fast != 0)) {
        compute_mode<F, BITS, SPARSE, MT, MODE_FAST>(f, info, stage, L, acc, lut);
    } else {
        bool lin = lane_linear(f.s[0]);
        if (F::NH == 2 && !info.same) lin = lin && lane_linear(f.s[F::NH - 1]);
        if (__all_sync(0xFFFFFFFFu, lin)) compute_mode<F, BITS, SPARSE, MT, MODE_GENERAL>(f, info, stage, L, acc, lut);
        else compute_mode<F, BITS, SPARSE, MT, MODE_SLOW>(f, info, stage, L, acc, lut);
    }
}

// ---- producer: fill one stage with bulk copies, spread over the lanes of the producer warp ----------------
template <class F, int MT>
__device__ __forceinline__ void produce_stage(const StreamParams& p, const KBlockInfo& info, int ct, int kb,
                                              uint32_t stage, uint32_t full_bar, int lane) {
    using SL = StageLayout<F, MT>;
    const int cols = min(128, p.S - ct * 128);                       // 128, or 64 in the last tile of an S % 128 == 64
    const int wrows = info.tail ? F::WROWS / 2 : F::WROWS;
    const int mrows = info.tail ? F::MROWS / 2 : F::MROWS;
    const int sets = info.same ? 1 : 2;
    const int xbytes = info.tail ? 128 : 256;
    if (lane == 0) {
        const uint32_t bytes = (uint32_t)((wrows + mrows) * cols * 4 + sets * 2 * cols * 2 + p.rows * xbytes);
        ptx::mbar_arrive_expect_tx(full_bar, bytes);
    }
    __syncwarp();
    const size_t S = (size_t)p.S;
    const size_t c0 = (size_t)ct * 128;
    for (int r = lane; r < wrows; r += 32)
        ptx::bulk_g2s(stage + SL::kW + r * F::WPITCH, p.matrix + ((size_t)kb * F::WROWS + r) * S + c0, cols * 4, full_bar);
    if (F::MROWS > 0) {
        for (int r = lane; r < mrows; r += 32)
            ptx::bulk_g2s(stage + SL::kMask + r * kMaskPitch, p.mask + ((size_t)kb * F::MROWS + r) * S + c0, cols * 4, full_bar);
    }
    if (lane >= 16 && lane < 16 + 2 * sets) {
        const int which = lane - 16;                                  // 0: s0, 1: z0, 2: s1, 3: z1
        const uint32_t grp = which < 2 ? info.g0 : info.g1;
        const __half* src = ((which & 1) ? p.zeros : p.scales) + (size_t)grp * S + c0;
        ptx::bulk_g2s(stage + SL::kSZ + which * 256, src, cols * 2, full_bar);
    }
    for (int m = lane; m < p.rows; m += 32)
        ptx::bulk_g2s(stage + SL::kX + m * kXPitch, p.x + (size_t)m * p.N + (size_t)kb * 128, xbytes, full_bar);
}

// owner of flat tile index t when T tiles are cut into G contiguous ranges [T*b/G, T*(b+1)/G)
__device__ __forceinline__ long long range_lo(long long T, long long G, long long b) { return (T * b) / G; }
__device__ __forceinline__ int range_owner(long long T, long long G, long long t) {
    return (int)(((t + 1) * G + T - 1) / T - 1);
}

constexpr int kStages = 4;              // shared-memory ring stages
constexpr int kMinBlocksOneRow = 3;     // CTAs per SM the one-m-tile kernel is compiled for
constexpr int kConsumerWarps = 4;
constexpr int kStreamThreads = (kConsumerWarps + 1) * 32;

template <int BITS, bool SPARSE, int MT>
__global__ void __launch_bounds__(kStreamThreads, (MT == 1 ? kMinBlocksOneRow : MT == 2 ? 2 : 1))
stream_kernel(const StreamParams p) {
    using F = Format<BITS, SPARSE>;
    using SL = StageLayout<F, MT>;
    extern __shared__ __align__(128) unsigned char smem[];      // kStages stages
    __shared__ __align__(8) unsigned long long full_bar[kStages], empty_bar[kStages];
    __shared__ uint4 lut[16];
    __shared__ int s_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[i]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[i]), kConsumerWarps);
        }
        ptx::fence_mbar_init();
    }
    if (SPARSE && threadIdx.x < 16) lut[threadIdx.x] = sparse_lut_entry(threadIdx.x);
    __syncthreads();

    const uint32_t smem0 = ptx::smem_u32(smem);
    const long long T = (long long)p.CT * p.KB;
    const long long G = gridDim.x, b = blockIdx.x;
    const long long t_lo = range_lo(T, G, b), t_hi = range_lo(T, G, b + 1);
    constexpr int ROWS = 8 * MT;

    if (warp == kConsumerWarps) {
        // ===== producer warp: walks this CTA's tiles in order, at most kStages ahead of the consumers =====
        uint32_t st = 0, ph = 0;
        for (long long tile = t_lo; tile < t_hi; ++tile) {
            const int ct = (int)(tile / p.KB);
            const int kb = (int)(tile - (long long)ct * p.KB);
            if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[st]), ph ^ 1u)) {
                if (lane == 0) atomicExch(p.status, 1);
                break;
            }
            const KBlockInfo info = kblock_info(p, kb);
            produce_stage<F, MT>(p, info, ct, kb, smem0 + st * SL::kBytes, ptx::smem_u32(&full_bar[st]), lane);
            if (++st == kStages) { st = 0; ph ^= 1u; }
        }
        return;
    }

    // ===== consumer warps: warp wc owns columns [32 wc, 32 wc + 32) of the tile =====
    const int wc = warp;
    LanePos L;
    L.g = lane >> 2;
    L.t = lane & 3;
    L.coff = (uint32_t)(wc * 32 + L.g * 4) * 4u;
    uint32_t st = 0, ph = 0;
    bool failed = false;

    long long tile = t_lo;
    bool first_segment = true;
    // A warp whose bounded wait gave up keeps walking its tiles without waiting or computing, so that it still
    // arrives at every named barrier and ring barrier the other warps count on (results are void: the status says so).
    while (tile < t_hi) {
        const int ct = (int)(tile / p.KB);
        const int kb0 = (int)(tile - (long long)ct * p.KB);
        const int kb1 = (int)min((long long)p.KB, kb0 + (t_hi - tile));
        const bool warp_ok = ct * kCTile + wc * 32 < p.S;      // S % 64 == 0: a warp's 32 columns are all in or all out

        float acc[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int cp = 0; cp < 2; ++cp)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][cp][i] = 0.f;

        for (int kb = kb0; kb < kb1; ++kb) {
            if (!failed && !ptx::mbar_wait(ptx::smem_u32(&full_bar[st]), ph)) {
                if (lane == 0) atomicExch(p.status, 2);
                failed = true;
            }
            if (warp_ok && !failed) consume_stage<F, BITS, SPARSE, MT>(kblock_info(p, kb), smem0 + st * SL::kBytes, L, acc, lut);
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&empty_bar[st]));
            if (++st == kStages) { st = 0; ph ^= 1u; }
        }
        // ---- store: lane (g, t) holds, per m-tile, rows m = 2t (c0, c2) and m = 2t + 1 (c1, c3) of columns 4g .. 4g+3 ----
        const bool complete = (kb0 == 0) && (kb1 == p.KB);
        const int col = ct * kCTile + wc * 32 + L.g * 4;
        if (complete) {
            if (warp_ok) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int hrow = 0; hrow < 2; ++hrow) {
                        const int m = mt * 8 + 2 * L.t + hrow;
                        if (m < p.rows) {
                            float v[4] = {acc[mt][0][hrow], acc[mt][0][2 + hrow], acc[mt][1][hrow], acc[mt][1][2 + hrow]};
                            __half* o = p.out + (size_t)m * p.S + col;
                            if (p.accumulate) {
                                const uint2 old = *reinterpret_cast<const uint2*>(o);
                                const float2 o01 = __half22float2(u32_as_h2(old.x)), o23 = __half22float2(u32_as_h2(old.y));
                                v[0] += o01.x; v[1] += o01.y; v[2] += o23.x; v[3] += o23.y;
                            }
                            uint2 r;
                            r.x = h2_as_u32(__floats2half2_rn(v[0], v[1]));
                            r.y = h2_as_u32(__floats2half2_rn(v[2], v[3]));
                            *reinterpret_cast<uint2*>(o) = r;
                        }
                    }
            }
        } else {
            float* slot = p.partials + ((size_t)b * 2 + (first_segment ? 0 : 1)) * (ROWS * kCTile);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int m = mt * 8 + 2 * L.t + hrow;
                    if (m < p.rows)
                        __stcg(reinterpret_cast<float4*>(slot + m * kCTile + wc * 32 + L.g * 4),
                               make_float4(acc[mt][0][hrow], acc[mt][0][2 + hrow], acc[mt][1][hrow], acc[mt][1][2 + hrow]));
                }
            __threadfence();
            ptx::named_bar_sync(1, kConsumerWarps * 32);
            const long long ct_lo = (long long)ct * p.KB, ct_hi = ct_lo + p.KB - 1;
            const int b_lo = range_owner(T, G, ct_lo), b_hi = range_owner(T, G, ct_hi);
            if (threadIdx.x == 0) {
                const unsigned int prev = atomicAdd(p.counters + ct, 1u);
                s_last = (prev == (unsigned int)(b_hi - b_lo)) ? 1 : 0;
            }
            ptx::named_bar_sync(1, kConsumerWarps * 32);
            if (s_last) {
                // the last CTA to arrive sums the partial tiles in CTA order: a fixed order, so results are reproducible
                __threadfence();
                const bool lo_starts_here = range_lo(T, G, b_lo) == ct_lo;
                const int n_elem = p.rows * kCTile;
                for (int idx = threadIdx.x; idx < n_elem; idx += kConsumerWarps * 32) {
                    const int m = idx >> 7, c = idx & 127;
                    const int oc = ct * kCTile + c;
                    float v = 0.f;
                    for (int bb = b_lo; bb <= b_hi; ++bb) {
                        const int which = (bb > b_lo || lo_starts_here) ? 0 : 1;
                        v += __ldcg(p.partials + ((size_t)bb * 2 + which) * (ROWS * kCTile) + idx);
                    }
                    if (oc < p.S) {
                        __half* o = p.out + (size_t)m * p.S + oc;
                        if (p.accumulate) v += __half2float(*o);
                        *o = __float2half_rn(v);
                    }
                }
                if (threadIdx.x == 0) p.counters[ct] = 0;   // leave the scratch ready for the next launch
            }
            ptx::named_bar_sync(1, kConsumerWarps * 32);   // s_last is reused by the next segment
        }
        tile += kb1 - kb0;
        first_segment = false;
    }
}

}  // namespace

// ---- host side --------------------------------------------------------------------------------------

template <int BITS, bool SPARSE, int MT>
static cudaError_t launch_one(const StreamParams& p, int max_ctas, cudaStream_t stream) {
    using SL = StageLayout<Format<BITS, SPARSE>, MT>;
    const size_t smem = (size_t)kStages * SL::kBytes;
    auto kern = stream_kernel<BITS, SPARSE, MT>;
    static std::atomic<int> ctas_per_sm[16];          // per device; concurrent first calls store the same values
    static std::atomic<int> sm_count[16];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    dev &= 15;
    if (ctas_per_sm[dev] == 0) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        int n = 0, sms = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kStreamThreads, smem);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        sm_count[dev] = sms;
        ctas_per_sm[dev] = n > 0 ? n : 1;
    }
    const long long T = (long long)p.CT * p.KB;
    long long grid = (long long)sm_count[dev] * ctas_per_sm[dev];
    if (grid > max_ctas) grid = max_ctas;
    if (grid > T) grid = T;
    kern<<<(int)grid, kStreamThreads, smem, stream>>>(p);
    count_launch();
    return cudaGetLastError();
}

template <int BITS, bool SPARSE>
static cudaError_t launch_mt(const StreamParams& p, int mt, int grid, cudaStream_t stream) {
    switch (mt) {
        case 1: return launch_one<BITS, SPARSE, 1>(p, grid, stream);
        case 2: return launch_one<BITS, SPARSE, 2>(p, grid, stream);
        default: return launch_one<BITS, SPARSE, 4>(p, grid, stream);
    }
}

// Launches the streaming kernel over all rows, 8 * mt rows per pass.  `ctas` = CTAs to fill the device.
cudaError_t stream_launch(int bits, bool sparse, StreamParams p, int total_rows, int ctas, cudaStream_t stream) {
    const int grid = ctas;
    if ((long long)p.CT * p.KB <= 0) return cudaSuccess;
    const __half* x0 = p.x;
    __half* out0 = p.out;
    for (int r0 = 0; r0 < total_rows;) {
        const int left = total_rows - r0;
        const int mt = left <= 8 ? 1 : left <= 16 ? 2 : 4;
        p.rows = left < 8 * mt ? left : 8 * mt;
        p.x = x0 + (size_t)r0 * p.N;
        p.out = out0 + (size_t)r0 * p.S;
        cudaError_t e;
        if (sparse) e = launch_mt<4, true>(p, mt, grid, stream);
        else if (bits == 4) e = launch_mt<4, false>(p, mt, grid, stream);
        else if (bits == 3) e = launch_mt<3, false>(p, mt, grid, stream);
        else e = launch_mt<2, false>(p, mt, grid, stream);
        if (e != cudaSuccess) return e;
        r0 += p.rows;
    }
    return cudaSuccess;
}

}  // namespace i4mm
