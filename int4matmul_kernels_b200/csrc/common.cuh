// Shared device helpers: fp16 bit tricks, the quantization semantics, launch parameter structs.
//
// Quantization semantics restated from the reference (matmul.cuh:93-144, 414-428):
//   scale >= 0 : W16 = hmul(hsub(half(q), zero), scale)            two fp16 roundings
//   otherwise  : W16 = hfma(half(+-2^(q & EXP)), -scale, zero)      one rounding, sign = q's top bit
// Dropped entries of the 16:32 format are exact zeros (matmul.cuh:398).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace i4mm {

constexpr int kSingleGroup = 0x0FFFFFFF;   // group_size < 0 (matmul_kernel.cu:379-381)

// ---- raw half2 arithmetic on 32-bit registers ------------------------------------------------
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

__device__ __forceinline__ uint32_t hadd2_u(uint32_t a, uint32_t b) {
    uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t hsub2_u(uint32_t a, uint32_t b) {
    uint32_t d; asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
    uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d; asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel)); return d;
}
// both halves <- low half / high half of a
__device__ __forceinline__ uint32_t dup_lo(uint32_t a) { return prmt(a, a, 0x1010); }
__device__ __forceinline__ uint32_t dup_hi(uint32_t a) { return prmt(a, a, 0x3232); }

constexpr uint32_t kMagic1024 = 0x64006400u;   // half2(1024, 1024): integer q in the low mantissa bits

// half2 constants as raw bits
constexpr uint32_t H2_ONE      = 0x3C003C00u;  // 1
constexpr uint32_t H2_1_4      = 0x34003400u;  // 1/4
constexpr uint32_t H2_1_8      = 0x30003000u;  // 1/8
constexpr uint32_t H2_1_16     = 0x2C002C00u;  // 1/16
constexpr uint32_t H2_1_64     = 0x24002400u;  // 1/64
constexpr uint32_t H2_N1024    = 0xE400E400u;  // -1024
constexpr uint32_t H2_N256     = 0xDC00DC00u;  // -256
constexpr uint32_t H2_N128     = 0xD800D800u;  // -128
constexpr uint32_t H2_N64      = 0xD400D400u;  // -64
constexpr uint32_t H2_N16      = 0xCC00CC00u;  // -16

// ---- scalar dequantisation in either coding (the slow, always-right path) ------------------------
template <int BITS>
__device__ __forceinline__ __half dequant_dynamic(uint32_t q, __half scale, __half zero) {
    if (__hge(scale, __ushort_as_half(0))) {
        return __hmul(__hsub(__uint2half_rn(q), zero), scale);
    }
    constexpr uint32_t SGN = 1u << (BITS - 1);
    constexpr uint32_t EXPM = SGN - 1u;
    const int iv = ((q & SGN) ? -1 : 1) * (1 << (q & EXPM));
    return __hfma(__int2half_rn(iv), __hneg(scale), zero);
}

// Division of a small index by the number of 64-wide half-blocks per group, by multiply-high.
// mul == 0 encodes "one group"; div == 1 is handled without the multiply.
struct GroupDiv {
    uint32_t div;   // group_size / 64
    uint32_t mul;   // floor(2^32 / div) + 1 for div >= 2
    __device__ __forceinline__ uint32_t operator()(uint32_t half_block) const {
        return div == 1 ? half_block : __umulhi(half_block, mul);
    }
};

// ---- where results go ----------------------------------------------------------------------------------------------
// The ordinary entry writes one (rows, S) array.  The gathering entry writes this rank's S columns into the same place
// of up to 8 arrays (its own and its peers' gathered (rows, ld) buffers, reached through peer-mapped pointers with
// plain stores): local column c belongs to part c / part_cols of a concatenation of matrices that were sharded one by
// one (q | k | v, gate | up), and lands at column part * part_stride + base + c % part_cols.
constexpr int kMaxDst = 8;
struct OutMap {
    __half* dst[kMaxDst];
    int n_dst;
    int part_cols;           // local columns per part (>= S: one part)
    long long ld;            // row stride of every destination, in elements
    long long part_stride;   // destination columns from one part to the next
    long long base;          // destination column of local column 0
    __device__ __forceinline__ long long col(int c) const {
        if (c < part_cols) return base + c;
        const int part = c / part_cols;
        return part * part_stride + base + (c - part * part_cols);
    }
};

// ---- parameters of the weight-streaming kernel ---------------------------------------------------
struct StreamParams {
    __half* out;             // (rows, S)
    const uint32_t* matrix;  // packed weights
    const uint32_t* mask;    // 16:32 keep mask or nullptr
    const __half* x;         // (rows, N)
    const __half* scales;    // (n_groups, S)
    const __half* zeros;     // (n_groups, S)
    float* partials;         // scratch: [2 * grid][8 * MT][128] fp32
    unsigned int* counters;  // scratch: one arrival counter per column tile, zero on entry and on exit
    int* status;             // scratch: set non-zero by a kernel whose bounded wait gave up
    int rows;                // rows handled by this launch (<= 8 * MT)
    int N, S;
    int KB;                  // ceil(N / 128)
    int CT;                  // ceil(S / 128)
    int accumulate;          // out = half(float(out) + acc) instead of overwrite
    GroupDiv gdiv;
    OutMap om;               // tcgen05 kernel only: destinations of the result (dst[0] == out for the ordinary entry)
};

// Counts kernel launches of this library in this process (read through i4mm_launch_count); defined in capi.cu.
void count_launch(int n = 1);
// Stores the cudaError_t that i4mm_last_cuda_error() reports for the calling host thread; defined in capi.cu.
void record_cuda_error(int e);

}  // namespace i4mm
