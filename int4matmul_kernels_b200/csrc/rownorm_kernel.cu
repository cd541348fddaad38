// Row-wise glue between the quantized linears of the layer-stack runner: one launch instead of the five to eight
// elementwise / reduction kernels the same expression costs in eager PyTorch.  y = v / rms(v) per row, in fp32, with
//   mode 0: v = a            mode 1: v = a + b + c            mode 2: v = a + b / rms(b)            mode 3: v = a * b
//   mode 4: mode 2, followed in the same launch by mode 0 of its (rounded) result: two outputs, y and y + rows * width
//           (the residual stream of a layer and the normalised input of the next layer's first linear)
// Rows of up to kCachedWidth elements are read once and kept in registers over the reductions (one block of 512 threads
// per row: the few-row passes are a chain of dependent launches, so a launch's latency is what counts); wider rows take
// the kernel that re-reads its inputs per pass.
// Inputs are fp16 rows of `width` elements with their own row strides (gathered q | k | v and gate | up are column
// slices of one buffer); the output is contiguous.  No counterpart in the reference, which has no model code.
#include "common.cuh"
#include "ptx.cuh"

namespace i4mm {

namespace {

// No pointer of these kernels is __restrict__: they are launched with programmatic stream serialization and may start
// while the kernel that writes their inputs is still running.  A restrict-qualified input promises the compiler that
// nothing else writes that memory during the kernel, which lets it move loads above griddepcontrol.wait (observed: the
// modes with an inner norm read the multiply's output before it was complete).

__device__ __forceinline__ float block_sum(float v, float* red) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = (l < (int)(blockDim.x >> 5)) ? red[l] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
    return t;
}

template <int MODE>
__global__ void __launch_bounds__(256) rownorm_kernel(__half* y, const __half* a,
                                                      const __half* b, const __half* c,
                                                      int width, long long sa, long long sb, long long sc) {
    __shared__ float red[32];
    // Launched with programmatic stream serialization: the kernel after this one may be scheduled at once (a multiply
    // then sets itself up and starts copying weights meanwhile), and nothing is read or written here before the kernel
    // before this one has completed.
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const long long row = blockIdx.x;
    const __half2* a2 = reinterpret_cast<const __half2*>(a + row * sa);
    const __half2* b2 = MODE != 0 ? reinterpret_cast<const __half2*>(b + row * sb) : nullptr;
    const __half2* c2 = MODE == 1 ? reinterpret_cast<const __half2*>(c + row * sc) : nullptr;
    __half2* y2 = reinterpret_cast<__half2*>(y + row * (long long)width);
    const int n2 = width >> 1;
    float rb = 1.f;
    if (MODE == 2) {
        float s = 0.f;
        for (int i = threadIdx.x; i < n2; i += blockDim.x) {
            const float2 v = __half22float2(b2[i]);
            s += v.x * v.x + v.y * v.y;
        }
        rb = rsqrtf(block_sum(s, red) / (float)width + 1e-6f);
    }
    auto value = [&](int i) -> float2 {
        const float2 va = __half22float2(a2[i]);
        if (MODE == 0) return va;
        const float2 vb = __half22float2(b2[i]);
        if (MODE == 1) {
            const float2 vc = __half22float2(c2[i]);
            return make_float2(va.x + vb.x + vc.x, va.y + vb.y + vc.y);
        }
        if (MODE == 2) return make_float2(va.x + vb.x * rb, va.y + vb.y * rb);
        return make_float2(va.x * vb.x, va.y * vb.y);
    };
    float s = 0.f;
    for (int i = threadIdx.x; i < n2; i += blockDim.x) {
        const float2 v = value(i);
        s += v.x * v.x + v.y * v.y;
    }
    const float r = rsqrtf(block_sum(s, red) / (float)width + 1e-6f);
    for (int i = threadIdx.x; i < n2; i += blockDim.x) {
        const float2 v = value(i);
        y2[i] = __floats2half2_rn(v.x * r, v.y * r);
    }
}

constexpr int kCachedThreads = 512;
constexpr int kCachedPer = 14;                                     // fp16 pairs per thread
constexpr int kCachedWidth = 2 * kCachedThreads * kCachedPer;      // 14336

template <int MODE>
__global__ void __launch_bounds__(kCachedThreads) rownorm_cached_kernel(__half* y, const __half* a,
                                                                        const __half* b, const __half* c,
                                                                        int width, long long sa, long long sb, long long sc,
                                                                        long long second_output) {
    __shared__ float red[32];
    ptx::grid_launch_dependents();        // as in rownorm_kernel
    ptx::grid_dependency_wait();
    constexpr bool kHasB = MODE != 0, kHasC = MODE == 1, kInnerNorm = MODE == 2 || MODE == 4;
    const long long row = blockIdx.x;
    const __half2* a2 = reinterpret_cast<const __half2*>(a + row * sa);
    const __half2* b2 = kHasB ? reinterpret_cast<const __half2*>(b + row * sb) : nullptr;
    const __half2* c2 = kHasC ? reinterpret_cast<const __half2*>(c + row * sc) : nullptr;
    __half2* y2 = reinterpret_cast<__half2*>(y + row * (long long)width);
    const int n2 = width >> 1;
    auto pair_at = [&](const __half2* src, int i) -> float2 {     // zero beyond the row: adds nothing to the sums
        return __half22float2(u32_as_h2(i < n2 ? reinterpret_cast<const uint32_t*>(src)[i] : 0u));
    };
    float2 v[kCachedPer], vb[kCachedPer];
#pragma unroll
    for (int k = 0; k < kCachedPer; ++k) {                       // every load of the row is in flight at once
        const int i = threadIdx.x + k * kCachedThreads;
        v[k] = pair_at(a2, i);
        if constexpr (kHasB) vb[k] = pair_at(b2, i);
        if constexpr (kHasC) {
            const float2 vc = pair_at(c2, i);
            v[k] = make_float2(v[k].x + vb[k].x + vc.x, v[k].y + vb[k].y + vc.y);
        }
        if constexpr (MODE == 3) v[k] = make_float2(v[k].x * vb[k].x, v[k].y * vb[k].y);
    }
    if constexpr (kInnerNorm) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < kCachedPer; ++k) s += vb[k].x * vb[k].x + vb[k].y * vb[k].y;
        const float rb = rsqrtf(block_sum(s, red) / (float)width + 1e-6f);
#pragma unroll
        for (int k = 0; k < kCachedPer; ++k) v[k] = make_float2(v[k].x + vb[k].x * rb, v[k].y + vb[k].y * rb);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kCachedPer; ++k) s += v[k].x * v[k].x + v[k].y * v[k].y;
    const float r = rsqrtf(block_sum(s, red) / (float)width + 1e-6f);
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < kCachedPer; ++k) {
        const int i = threadIdx.x + k * kCachedThreads;
        const __half2 h = __floats2half2_rn(v[k].x * r, v[k].y * r);
        if (i < n2) y2[i] = h;
        if constexpr (MODE == 4) {
            v[k] = __half22float2(h);                            // the second norm sees the rounded values, as a second launch would
            s2 += v[k].x * v[k].x + v[k].y * v[k].y;
        }
    }
    if constexpr (MODE == 4) {
        const float r2 = rsqrtf(block_sum(s2, red) / (float)width + 1e-6f);
        __half2* z2 = y2 + (second_output >> 1);
#pragma unroll
        for (int k = 0; k < kCachedPer; ++k) {
            const int i = threadIdx.x + k * kCachedThreads;
            if (i < n2) z2[i] = __floats2half2_rn(v[k].x * r2, v[k].y * r2);
        }
    }
}

}  // namespace

cudaError_t rownorm_launch(int mode, void* y, const void* a, const void* b, const void* c, long long rows, int width,
                           long long sa, long long sb, long long sc, cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    __half* yy = (__half*)y;
    const __half *aa = (const __half*)a, *bb = (const __half*)b, *cc = (const __half*)c;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((unsigned)rows, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e;
    const long long second = rows * (long long)width;             // mode 4: element offset of the second output
    if (width <= kCachedWidth) {
        cfg.blockDim = dim3(kCachedThreads, 1, 1);
        switch (mode) {
            case 0: e = cudaLaunchKernelEx(&cfg, rownorm_cached_kernel<0>, yy, aa, bb, cc, width, sa, sb, sc, second); break;
            case 1: e = cudaLaunchKernelEx(&cfg, rownorm_cached_kernel<1>, yy, aa, bb, cc, width, sa, sb, sc, second); break;
            case 2: e = cudaLaunchKernelEx(&cfg, rownorm_cached_kernel<2>, yy, aa, bb, cc, width, sa, sb, sc, second); break;
            case 3: e = cudaLaunchKernelEx(&cfg, rownorm_cached_kernel<3>, yy, aa, bb, cc, width, sa, sb, sc, second); break;
            default: e = cudaLaunchKernelEx(&cfg, rownorm_cached_kernel<4>, yy, aa, bb, cc, width, sa, sb, sc, second); break;
        }
        if (e == cudaSuccess) count_launch();
        return e;
    }
    if (mode == 4) {                                              // wide rows: the two steps as two launches
        e = cudaLaunchKernelEx(&cfg, rownorm_kernel<2>, yy, aa, bb, cc, width, sa, sb, sc);
        if (e != cudaSuccess) return e;
        count_launch();
        e = cudaLaunchKernelEx(&cfg, rownorm_kernel<0>, yy + second, (const __half*)yy, bb, cc, width, (long long)width, sb, sc);
        if (e == cudaSuccess) count_launch();
        return e;
    }
    switch (mode) {
        case 0: e = cudaLaunchKernelEx(&cfg, rownorm_kernel<0>, yy, aa, bb, cc, width, sa, sb, sc); break;
        case 1: e = cudaLaunchKernelEx(&cfg, rownorm_kernel<1>, yy, aa, bb, cc, width, sa, sb, sc); break;
        case 2: e = cudaLaunchKernelEx(&cfg, rownorm_kernel<2>, yy, aa, bb, cc, width, sa, sb, sc); break;
        default: e = cudaLaunchKernelEx(&cfg, rownorm_kernel<3>, yy, aa, bb, cc, width, sa, sb, sc); break;
    }
    if (e == cudaSuccess) count_launch();
    return e;
}

}  // namespace i4mm
