// Weight-streaming kernel for few activation rows (matvec and skinny matmul): HBM-bound.
//
// Replaces MVA_Int4_Half (matvec_kernel.cu:198-267) and, for small M, MMA_Int4_Half
// (matmul_kernel.cu:219-333).  Design:
//   * every lane streams packed words with 128-bit loads: one uint4 = 4 adjacent S columns of one packed
//     row; the 4 lanes of a quad take 4 different packed rows, the 8 quads take 8 adjacent column
//     quartets, so a warp load is 4 rows x 128 contiguous bytes;
//   * nibbles become fp16 pairs in registers with the 0x6400 mantissa trick (one LOP3 per pair), then
//     (q - zero) * scale exactly as the reference rounds it (sub, then mul);
//   * the multiply-accumulate runs on mma.sync m16n8k16 (fp16 x fp16 -> fp32): the 16 "rows" of A are
//     16 weight columns, the 8 "columns" of B are 8 activation rows, k walks the reduction dim in a
//     permuted order that both operands share, so no data is shuffled between lanes;
//   * the (column tile, k-block) space is cut into equal contiguous ranges, one per CTA, and ranges that
//     split a column tile are summed through fp32 scratch in a fixed order by the last CTA to arrive
//     (no atomics on data, bit-reproducible, no second launch).
#include "common.cuh"

namespace i4mm {

namespace {

constexpr int kCTile = 128;    // output columns per CTA tile (4 warps across)

enum : int { MODE_FAST = 0, MODE_GENERAL = 1, MODE_SLOW = 2 };

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_keep(const void* p) {
    uint4 v;
    asm("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_keep2(const void* p) {
    uint2 v;
    asm("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
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
    uint32_t z2;      // zero in both halves
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

template <int NJ, int MODE>
__device__ __forceinline__ void make_colq(ColQ& c, uint32_t s_bits16, uint32_t z_bits16) {
    c.s2 = s_bits16 | (s_bits16 << 16);
    c.z2 = z_bits16 | (z_bits16 << 16);
    if (MODE == MODE_FAST) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) c.off[j] = hsub2_u(shift_base(NJ, j), c.z2);
        const uint32_t zi = __half2uint_rz(__ushort_as_half((unsigned short)z_bits16)) & 0xFFu;
        c.zb = zi * 0x01010101u;
    } else {
        c.zb = 0;
    }
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

// ---- formats -----------------------------------------------------------------------------------------
// Each format describes what one lane loads for one k-block (128 n x its 4 columns) and how it turns that
// into NP fp16 pairs per column per "step", in an order the activation side mirrors.

struct LanePos {
    int g, t;       // quad index (0..7), lane in quad (0..3)
    int col;        // first of this lane's 4 columns
    bool col_ok;    // col < S
};

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

template <int BITS, bool SPARSE>
struct Format;

// ---------------- dense int4: 8 n per word ----------------
template <>
struct Format<4, false> {
    static constexpr int NJ = 2;
    static constexpr int NH = 2;        // (scale, zero) sets per lane per k-block
    static constexpr int STEPS = 4;     // lane chunks per k-block
    static constexpr int NP = 4;        // pairs per column per step
    static constexpr int XREGS = 4;     // activation registers per step (8 halves)
    struct Frag { uint4 w[4]; uint2 s[2], z[2]; };

    __device__ static __forceinline__ int n0(int kb, int step, int t) { return kb * 128 + step * 32 + t * 8; }
    __device__ static __forceinline__ int half_of(int step, int) { return step >> 1; }

    __device__ static __forceinline__ void load(Frag& f, const StreamParams& p, const LanePos& L, int kb) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = kb * 16 + j * 4 + L.t;
            f.w[j] = (L.col_ok && r * 8 < p.N) ? ldg_stream(p.matrix + (size_t)r * p.S + L.col) : make_uint4(0, 0, 0, 0);
        }
    }
    template <int MODE>
    __device__ static __forceinline__ void decode(const Frag& f, int step, int c, const ColQ& q, uint32_t (&P)[NP],
                                                  const uint4*) {
        const uint4 v = f.w[step];
        const uint32_t w = c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w;
        const uint32_t hi = w >> 8;
        P[0] = finish<4, NJ, MODE>((w & 0x000F000Fu) | kMagic1024, 0, q);    // (n0, n4)
        P[1] = finish<4, NJ, MODE>((w & 0x00F000F0u) | kMagic1024, 1, q);    // (n1, n5)
        P[2] = finish<4, NJ, MODE>((hi & 0x000F000Fu) | kMagic1024, 0, q);   // (n2, n6)
        P[3] = finish<4, NJ, MODE>((hi & 0x00F000F0u) | kMagic1024, 1, q);   // (n3, n7)
    }
    __device__ static __forceinline__ void xpairs(const uint32_t (&xr)[XREGS], uint32_t (&X)[NP]) {
        X[0] = prmt(xr[0], xr[2], 0x5410);
        X[1] = prmt(xr[0], xr[2], 0x7632);
        X[2] = prmt(xr[1], xr[3], 0x5410);
        X[3] = prmt(xr[1], xr[3], 0x7632);
    }
};

// ---------------- dense int2: 16 n per word ----------------
template <>
struct Format<2, false> {
    static constexpr int NJ = 4;
    static constexpr int NH = 2;
    static constexpr int STEPS = 2;
    static constexpr int NP = 8;
    static constexpr int XREGS = 8;
    struct Frag { uint4 w[2]; uint2 s[2], z[2]; };

    __device__ static __forceinline__ int n0(int kb, int step, int t) { return kb * 128 + step * 64 + t * 16; }
    __device__ static __forceinline__ int half_of(int step, int) { return step; }

    __device__ static __forceinline__ void load(Frag& f, const StreamParams& p, const LanePos& L, int kb) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int r = kb * 8 + j * 4 + L.t;
            f.w[j] = (L.col_ok && r * 16 < p.N) ? ldg_stream(p.matrix + (size_t)r * p.S + L.col) : make_uint4(0, 0, 0, 0);
        }
    }
    template <int MODE>
    __device__ static __forceinline__ void decode(const Frag& f, int step, int c, const ColQ& q, uint32_t (&P)[NP],
                                                  const uint4*) {
        const uint4 v = f.w[step];
        const uint32_t w = c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w;
        const uint32_t hi = w >> 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t m = 0x00030003u << (2 * j);
            P[j] = finish<2, NJ, MODE>((w & m) | kMagic1024, j, q);        // (n_j,   n_{j+8})
            P[4 + j] = finish<2, NJ, MODE>((hi & m) | kMagic1024, j, q);   // (n_{4+j}, n_{12+j})
        }
    }
    __device__ static __forceinline__ void xpairs(const uint32_t (&xr)[XREGS], uint32_t (&X)[NP]) {
#pragma unroll
        for (int p = 0; p < 8; ++p) X[p] = prmt(xr[p >> 1], xr[4 + (p >> 1)], (p & 1) ? 0x7632 : 0x5410);
    }
};

// ---------------- dense int3: 32 n per 3 words ----------------
template <>
struct Format<3, false> {
    static constexpr int NJ = 3;
    static constexpr int NH = 1;
    static constexpr int STEPS = 1;
    static constexpr int NP = 16;
    static constexpr int XREGS = 16;
    struct Frag { uint4 w[3]; uint2 s[1], z[1]; };

    __device__ static __forceinline__ int n0(int kb, int, int t) { return kb * 128 + t * 32; }
    __device__ static __forceinline__ int half_of(int, int t) { return t >> 1; }

    __device__ static __forceinline__ void load(Frag& f, const StreamParams& p, const LanePos& L, int kb) {
        const int blk = kb * 4 + L.t;
        const bool ok = L.col_ok && blk * 32 < p.N;
#pragma unroll
        for (int j = 0; j < 3; ++j)
            f.w[j] = ok ? ldg_stream(p.matrix + (size_t)(blk * 3 + j) * p.S + L.col) : make_uint4(0, 0, 0, 0);
    }
    // pair index p = 3 * wp + f  ->  (n, n') = (6 wp + f, 6 wp + 3 + f); p = 15 -> (30, 31)
    __device__ static __forceinline__ constexpr int pair_lo(int p) { return p == 15 ? 30 : 6 * (p / 3) + (p % 3); }
    __device__ static __forceinline__ constexpr int pair_hi(int p) { return p == 15 ? 31 : 6 * (p / 3) + 3 + (p % 3); }

    template <int MODE>
    __device__ static __forceinline__ void decode(const Frag& f, int, int c, const ColQ& q, uint32_t (&P)[NP],
                                                  const uint4*) {
        const uint32_t w0 = c == 0 ? f.w[0].x : c == 1 ? f.w[0].y : c == 2 ? f.w[0].z : f.w[0].w;
        const uint32_t w1 = c == 0 ? f.w[1].x : c == 1 ? f.w[1].y : c == 2 ? f.w[1].z : f.w[1].w;
        const uint32_t w2 = c == 0 ? f.w[2].x : c == 1 ? f.w[2].y : c == 2 ? f.w[2].z : f.w[2].w;
        // X[wp]: low half = 9-bit window 2wp at bits 0..8, high half = window 2wp+1 at bits 16..24
        uint32_t X[5];
        X[0] = prmt(w0, w0 << 7, 0x7610);                                  // stream bits 0.., 9..
        X[1] = prmt(w0 >> 18, __funnelshift_r(w0, w1, 11), 0x7610);        // 18.., 27..
        X[2] = prmt(w1 >> 4, w1 << 3, 0x7610);                             // 36.., 45..
        X[3] = prmt(w1 >> 22, __funnelshift_r(w1, w2, 15), 0x7610);        // 54.., 63..
        X[4] = prmt(w2 >> 8, w2 >> 1, 0x7610);                             // 72.., 81..
        const uint32_t last = prmt(w2 >> 26, w2 >> 13, 0x7610);            // 90.., 93..
#pragma unroll
        for (int wp = 0; wp < 5; ++wp) {
            P[3 * wp + 0] = finish<3, NJ, MODE>((X[wp] & 0x00070007u) | kMagic1024, 0, q);
            P[3 * wp + 1] = finish<3, NJ, MODE>((X[wp] & 0x00380038u) | kMagic1024, 1, q);
            P[3 * wp + 2] = finish<3, NJ, MODE>((X[wp] & 0x01C001C0u) | kMagic1024, 2, q);
        }
        P[15] = finish<3, NJ, MODE>((last & 0x00070007u) | kMagic1024, 0, q);
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

// ---------------- 16:32 sparse int4: 32 n per (64-bit compacted word, 32-bit mask) ----------------
template <>
struct Format<4, true> {
    static constexpr int NJ = 1;
    static constexpr int NH = 1;
    static constexpr int STEPS = 1;
    static constexpr int NP = 16;
    static constexpr int XREGS = 16;
    struct Frag { uint4 w[2]; uint4 m; uint2 s[1], z[1]; };

    __device__ static __forceinline__ int n0(int kb, int, int t) { return kb * 128 + t * 32; }
    __device__ static __forceinline__ int half_of(int, int t) { return t >> 1; }

    __device__ static __forceinline__ void load(Frag& f, const StreamParams& p, const LanePos& L, int kb) {
        const int blk = kb * 4 + L.t;
        const bool ok = L.col_ok && blk * 32 < p.N;
        f.w[0] = ok ? ldg_stream(p.matrix + (size_t)(blk * 2) * p.S + L.col) : make_uint4(0, 0, 0, 0);
        f.w[1] = ok ? ldg_stream(p.matrix + (size_t)(blk * 2 + 1) * p.S + L.col) : make_uint4(0, 0, 0, 0);
        f.m = ok ? ldg_stream(p.mask + (size_t)blk * p.S + L.col) : make_uint4(0, 0, 0, 0);
    }
    template <int MODE>
    __device__ static __forceinline__ void decode(const Frag& f, int, int c, const ColQ& q, uint32_t (&P)[NP],
                                                  const uint4* lut) {
        uint32_t lo = c == 0 ? f.w[0].x : c == 1 ? f.w[0].y : c == 2 ? f.w[0].z : f.w[0].w;
        uint32_t hi = c == 0 ? f.w[1].x : c == 1 ? f.w[1].y : c == 2 ? f.w[1].z : f.w[1].w;
        const uint32_t m = c == 0 ? f.m.x : c == 1 ? f.m.y : c == 2 ? f.m.z : f.m.w;
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

// ---- one k-block of one warp -------------------------------------------------------------------------
template <class F>
__device__ __forceinline__ void load_frag(typename F::Frag& f, const StreamParams& p, const LanePos& L, int kb) {
    F::load(f, p, L, kb);
#pragma unroll
    for (int h = 0; h < F::NH; ++h) {
        const int hb = kb * 2 + (F::NH == 2 ? h : (L.t >> 1));
        if (L.col_ok && hb * 64 < p.N) {
            const size_t o = (size_t)p.gdiv((uint32_t)hb) * p.S + L.col;
            f.s[h] = ldg_keep2(p.scales + o);
            f.z[h] = ldg_keep2(p.zeros + o);
        } else {
            f.s[h] = make_uint2(0, 0);
            f.z[h] = make_uint2(0, 0);
        }
    }
}

template <bool SPARSE>
__device__ __forceinline__ int classify(uint2 s, uint2 z) {
    const __half2 zero2 = u32_as_h2(0u);
    const __half2 s0 = u32_as_h2(s.x), s1 = u32_as_h2(s.y), z0 = u32_as_h2(z.x), z1 = u32_as_h2(z.y);
    const bool lin = __hbge2(s0, zero2) && __hbge2(s1, zero2);
    const __half2 lim = SPARSE ? u32_as_h2(0x5BF85BF8u) /* 255 */ : u32_as_h2(0x60006000u) /* 512 */;
    bool intz = __hbeq2(h2rint(z0), z0) && __hbeq2(h2rint(z1), z1) &&
                __hble2(__habs2(z0), lim) && __hble2(__habs2(z1), lim);
    if (SPARSE) intz = intz && __hbge2(z0, zero2) && __hbge2(z1, zero2);
    const bool all_lin = __all_sync(0xFFFFFFFFu, lin);
    const bool all_int = __all_sync(0xFFFFFFFFu, lin && intz);
    return all_int ? MODE_FAST : all_lin ? MODE_GENERAL : MODE_SLOW;
}

template <class F, int BITS, int MT, int MODE>
__device__ __forceinline__ void compute_steps(const typename F::Frag& f, int h, const StreamParams& p,
                                              const LanePos& L, int kb, float (&acc)[MT][2][4], const uint4* lut) {
    ColQ cq[4];
    {
        const uint2 s = f.s[h], z = f.z[h];
        make_colq<F::NJ, MODE>(cq[0], s.x & 0xFFFFu, z.x & 0xFFFFu);
        make_colq<F::NJ, MODE>(cq[1], s.x >> 16, z.x >> 16);
        make_colq<F::NJ, MODE>(cq[2], s.y & 0xFFFFu, z.y & 0xFFFFu);
        make_colq<F::NJ, MODE>(cq[3], s.y >> 16, z.y >> 16);
    }
    constexpr int SPH = F::STEPS / F::NH;   // steps that share this (scale, zero) set
#pragma unroll
    for (int sj = 0; sj < SPH; ++sj) {
        const int step = (F::NH == 2 ? h * SPH : 0) + sj;
        const int n0 = F::n0(kb, step, L.t);
        uint32_t X[MT][F::NP];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            uint32_t xr[F::XREGS];
            const int m = mt * 8 + L.g;
            const bool ok = (m < p.rows) && (n0 < p.N);
#pragma unroll
            for (int i = 0; i < F::XREGS / 4; ++i) {
                const uint4 v = ok ? ldg_keep(p.x + (size_t)m * p.N + n0 + 8 * i) : make_uint4(0, 0, 0, 0);
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

template <class F, int BITS, bool SPARSE, int MT>
__device__ __forceinline__ void compute_frag(const typename F::Frag& f, const StreamParams& p, const LanePos& L,
                                             int kb, float (&acc)[MT][2][4], const uint4* lut) {
#pragma unroll
    for (int h = 0; h < F::NH; ++h) {
        const int mode = classify<SPARSE>(f.s[h], f.z[h]);
        if (mode == MODE_FAST) compute_steps<F, BITS, MT, MODE_FAST>(f, h, p, L, kb, acc, lut);
        else if (mode == MODE_GENERAL) compute_steps<F, BITS, MT, MODE_GENERAL>(f, h, p, L, kb, acc, lut);
        else compute_steps<F, BITS, MT, MODE_SLOW>(f, h, p, L, kb, acc, lut);
    }
}

// owner of flat tile index t when T tiles are cut into G contiguous ranges [T*b/G, T*(b+1)/G)
__device__ __forceinline__ long long range_lo(long long T, long long G, long long b) { return (T * b) / G; }
__device__ __forceinline__ int range_owner(long long T, long long G, long long t) {
    return (int)(((t + 1) * G + T - 1) / T - 1);
}

template <int BITS, bool SPARSE, int MT, int WK>
__global__ void __launch_bounds__(128 * WK, (MT <= 2 ? 2 : 1)) stream_kernel(const StreamParams p) {
    using F = Format<BITS, SPARSE>;
    extern __shared__ float red[];                 // [WK][8 * MT][128]
    __shared__ uint4 lut[16];
    __shared__ int s_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wc = warp & 3, wk = warp >> 2;
    LanePos L;
    L.g = lane >> 2;
    L.t = lane & 3;

    if (SPARSE && threadIdx.x < 16) lut[threadIdx.x] = sparse_lut_entry(threadIdx.x);
    __syncthreads();

    const long long T = (long long)p.CT * p.KB;
    const long long G = gridDim.x, b = blockIdx.x;
    const long long t_lo = range_lo(T, G, b), t_hi = range_lo(T, G, b + 1);
    constexpr int ROWS = 8 * MT;

    long long tile = t_lo;
    bool first_segment = true;
    while (tile < t_hi) {
        const int ct = (int)(tile / p.KB);
        const int kb0 = (int)(tile - (long long)ct * p.KB);
        const int kb1 = (int)min((long long)p.KB, kb0 + (t_hi - tile));
        L.col = ct * kCTile + wc * 32 + L.g * 4;
        L.col_ok = L.col < p.S;

        float acc[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int cp = 0; cp < 2; ++cp)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][cp][i] = 0.f;

        {
            typename F::Frag cur, nxt;
            int kb = kb0 + wk;
            if (kb < kb1) load_frag<F>(cur, p, L, kb);
            for (; kb < kb1; kb += WK) {
                const bool more = kb + WK < kb1;
                if (more) load_frag<F>(nxt, p, L, kb + WK);
                compute_frag<F, BITS, SPARSE, MT>(cur, p, L, kb, acc, lut);
                if (more) cur = nxt;
            }
        }

        // ---- reduce the WK warps of this CTA through shared memory ----
        // lane (g, t) holds, per m-tile, rows m = 2t (c0, c2) and m = 2t + 1 (c1, c3) of columns 4g .. 4g+3
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float* r0 = red + ((size_t)wk * ROWS + mt * 8 + 2 * L.t) * kCTile + wc * 32 + L.g * 4;
            *reinterpret_cast<float4*>(r0) = make_float4(acc[mt][0][0], acc[mt][0][2], acc[mt][1][0], acc[mt][1][2]);
            *reinterpret_cast<float4*>(r0 + kCTile) = make_float4(acc[mt][0][1], acc[mt][0][3], acc[mt][1][1], acc[mt][1][3]);
        }
        __syncthreads();

        const bool complete = (kb0 == 0) && (kb1 == p.KB);
        const int n_elem = p.rows * kCTile;
        if (complete) {
            for (int idx = threadIdx.x; idx < n_elem; idx += 128 * WK) {
                const int m = idx >> 7, c = idx & 127;
                const int col = ct * kCTile + c;
                float v = 0.f;
#pragma unroll
                for (int k = 0; k < WK; ++k) v += red[((size_t)k * ROWS + m) * kCTile + c];
                if (col < p.S) {
                    __half* o = p.out + (size_t)m * p.S + col;
                    if (p.accumulate) v += __half2float(*o);
                    *o = __float2half_rn(v);
                }
            }
        } else {
            float* slot = p.partials + ((size_t)b * 2 + (first_segment ? 0 : 1)) * (ROWS * kCTile);
            for (int idx = threadIdx.x; idx < n_elem; idx += 128 * WK) {
                const int m = idx >> 7, c = idx & 127;
                float v = 0.f;
#pragma unroll
                for (int k = 0; k < WK; ++k) v += red[((size_t)k * ROWS + m) * kCTile + c];
                __stcg(slot + idx, v);
            }
            __threadfence();
            __syncthreads();
            const long long ct_lo = (long long)ct * p.KB, ct_hi = ct_lo + p.KB - 1;
            const int b_lo = range_owner(T, G, ct_lo), b_hi = range_owner(T, G, ct_hi);
            if (threadIdx.x == 0) {
                const unsigned int prev = atomicAdd(p.counters + ct, 1u);
                s_last = (prev == (unsigned int)(b_hi - b_lo)) ? 1 : 0;
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                const bool lo_starts_here = range_lo(T, G, b_lo) == ct_lo;
                for (int idx = threadIdx.x; idx < n_elem; idx += 128 * WK) {
                    const int m = idx >> 7, c = idx & 127;
                    const int col = ct * kCTile + c;
                    float v = 0.f;
                    for (int bb = b_lo; bb <= b_hi; ++bb) {
                        const int which = (bb > b_lo || lo_starts_here) ? 0 : 1;
                        v += __ldcg(p.partials + ((size_t)bb * 2 + which) * (ROWS * kCTile) + idx);
                    }
                    if (col < p.S) {
                        __half* o = p.out + (size_t)m * p.S + col;
                        if (p.accumulate) v += __half2float(*o);
                        *o = __float2half_rn(v);
                    }
                }
                if (threadIdx.x == 0) p.counters[ct] = 0;   // leave the scratch ready for the next launch
            }
        }
        __syncthreads();   // `red` and `s_last` are reused by the next segment
        tile += kb1 - kb0;
        first_segment = false;
    }
}

}  // namespace

// ---- host side --------------------------------------------------------------------------------------
size_t stream_partials_bytes(int grid, int mt) { return (size_t)grid * 2 * (8 * mt) * kCTile * sizeof(float); }

template <int BITS, bool SPARSE, int MT>
static cudaError_t launch_one(const StreamParams& p, int grid, cudaStream_t stream) {
    constexpr int WK = 2;
    const size_t smem = (size_t)WK * 8 * MT * kCTile * sizeof(float);
    auto kern = stream_kernel<BITS, SPARSE, MT, WK>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    kern<<<grid, 128 * WK, smem, stream>>>(p);
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
    const long long T = (long long)p.CT * p.KB;
    const int grid = (int)(T < ctas ? T : ctas);
    if (grid <= 0) return cudaSuccess;
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
