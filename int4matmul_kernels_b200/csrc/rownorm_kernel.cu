// Row-wise glue between the quantized linears of the layer-stack runner: one launch instead of the five to eight
// elementwise / reduction kernels the same expression costs in eager PyTorch.  y = v / rms(v) per row, in fp32, with
//   mode 0: v = a            mode 1: v = a + b + c            mode 2: v = a + b / rms(b)            mode 3: v = a * b
// Inputs are fp16 rows of `width` elements with their own row strides (gathered q | k | v and gate | up are column
// slices of one buffer); the output is contiguous.  No counterpart in the reference, which has no model code.
#include "common.cuh"
#include "ptx.cuh"

namespace i4mm {

namespace {

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
__global__ void __launch_bounds__(256) rownorm_kernel(__half* __restrict__ y, const __half* __restrict__ a,
                                                      const __half* __restrict__ b, const __half* __restrict__ c,
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
