// The torch extension module `int4matmul`: the operator surface of the reference's int4matmul.cpp
// (same eleven functions, argument order, in-place convention, docstrings) over the C ABI of
// libint4matmul_b200.so.  Host code only: it validates tensors, picks the current CUDA stream, keeps one
// zero-initialised scratch buffer per (device, stream) and turns non-zero statuses into exceptions.
//
// Differences from the reference, all on the side of failing earlier and louder:
//   * every precondition the reference checks with assert() (process abort) or not at all (dtype, device,
//     contiguity; matmul_kernel.cu:404-416, 446-451) raises here;
//   * sparse int3 / int2 and non-fp16 activations raise instead of trapping the device (matmul.cuh:188, 331);
//   * launches go to torch's current stream (the reference uses the legacy default stream, which is the same
//     stream unless the caller switched streams);
//   * weight_matrix_packing raises ValueError when a 32-block does not keep exactly 16 weights (the reference
//     device-asserts, utils_kernel.cu:41); for that it waits for the pack kernel to finish.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <atomic>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/int4matmul_b200.h"

namespace {

using torch::Tensor;

#define I4_TENSOR_MULT_ARGS                                                                            \
    Tensor outs, Tensor matrix, Tensor multiplier, Tensor scales, Tensor zeros, int64_t group_size,    \
        c10::optional<Tensor> sparse_mask
#define I4_TENSOR_MULT_PASS outs, matrix, multiplier, scales, zeros, group_size, sparse_mask

struct Workspace {
    Tensor buffer;
    cudaStream_t stream;
};
std::mutex g_ws_mutex;
std::map<std::pair<int, int64_t>, Workspace> g_workspaces;

Tensor workspace_for(const c10::Device& dev, const c10::cuda::CUDAStream& stream) {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    const auto key = std::make_pair((int)dev.index(), (int64_t)stream.id());
    auto it = g_workspaces.find(key);
    if (it != g_workspaces.end()) return it->second.buffer;
    Tensor ws = torch::zeros({(int64_t)i4mm_workspace_bytes()}, torch::dtype(torch::kUInt8).device(dev));
    g_workspaces.emplace(key, Workspace{ws, stream.stream()});
    return ws;
}

void check_status(int status, const char* what) {
    if (status == I4MM_OK) return;
    std::string msg = std::string(what) + ": " + i4mm_status_string(status);
    if (status == I4MM_ERR_LAUNCH) msg += " (cudaError " + std::to_string(i4mm_last_cuda_error()) + ")";
    if (status == I4MM_ERR_BITS) throw std::invalid_argument(msg);
    TORCH_CHECK(false, msg);
}

enum class Route { AUTO, MATMUL, MATVEC };

// Not in the reference: the caller's promise that the weight-side tensors are never written by the kernel that
// precedes a multiply in the stream (weights of a loaded model), which lets a launch begin while that kernel finishes.
std::atomic<bool> g_static_weights{false};
void set_static_weights(bool flag) { g_static_weights.store(flag); }

void quant_mult(uint32_t bits, Route route, I4_TENSOR_MULT_ARGS) {
    if (bits != 4 && bits != 3 && bits != 2) {
        // int4matmul.cpp:35, 45
        throw std::invalid_argument(multiplier.dim() == 3 && multiplier.size(1) == 1
                                        ? "Unsupported bit width for matvec"
                                        : "Unsupported bit width for matmul");
    }
    const bool is_sparse = sparse_mask.has_value() && sparse_mask.value().defined();
    TORCH_CHECK(multiplier.is_cuda(), "multiplier must be a CUDA tensor");
    const auto dev = multiplier.device();
    auto on_dev = [&](const Tensor& t, const char* name) {
        TORCH_CHECK(t.is_cuda() && t.device() == dev, name, " must be on the same CUDA device as multiplier");
        TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    };
    on_dev(outs, "outs"); on_dev(matrix, "matrix"); on_dev(multiplier, "multiplier");
    on_dev(scales, "scales"); on_dev(zeros, "zeros");
    TORCH_CHECK(multiplier.scalar_type() == torch::kHalf, "multiplier must be float16 (the reference implements fp16 only)");
    TORCH_CHECK(outs.scalar_type() == torch::kHalf, "outs must be float16");
    TORCH_CHECK(scales.scalar_type() == torch::kHalf && zeros.scalar_type() == torch::kHalf, "scales and zeros must be float16");
    TORCH_CHECK(matrix.scalar_type() == torch::kInt, "matrix must be int32");
    TORCH_CHECK(multiplier.dim() == 3, "multiplier must be (batch, seq_len, in_size)");
    TORCH_CHECK(outs.dim() == 3, "outs must be (batch, seq_len, out_size)");
    TORCH_CHECK(matrix.dim() == 2 && scales.dim() == 2 && zeros.dim() == 2, "matrix, scales, zeros must be 2-D");
    TORCH_CHECK(!is_sparse || bits == 4, "16:32 sparsity is only implemented for 4-bit weights");

    const int64_t batch = multiplier.size(0), seq_len = multiplier.size(1), in_size = multiplier.size(2);
    const int64_t mtx_in = matrix.size(0), out_size = matrix.size(1);
    if (route == Route::MATVEC) TORCH_CHECK(seq_len == 1, "the _vec entry needs seq_len == 1 (matvec_kernel.cu:323)");
    if (is_sparse) {
        TORCH_CHECK(mtx_in * 32 * 2 / bits == in_size, "sparse matrix rows * 16 must equal in_size");
    } else {
        TORCH_CHECK(mtx_in * 32 / bits == in_size && (mtx_in * 32) % bits == 0, "matrix rows * 32 / bits must equal in_size");
    }
    TORCH_CHECK(outs.size(0) == batch && outs.size(1) == seq_len && outs.size(2) == out_size, "outs must be (batch, seq_len, out_size)");
    TORCH_CHECK(zeros.size(1) == out_size && scales.size(1) == out_size, "scales/zeros must have out_size columns");
    TORCH_CHECK(zeros.size(0) == scales.size(0), "scales and zeros must have the same number of groups");
    TORCH_CHECK(group_size < 0 || (group_size > 0 && group_size % 64 == 0), "group_size must be a positive multiple of 64, or negative");
    const void* mask_ptr = nullptr;
    if (is_sparse) {
        const Tensor& m = sparse_mask.value();
        on_dev(m, "sparse_mask");
        TORCH_CHECK(m.scalar_type() == torch::kInt && m.dim() == 2, "sparse_mask must be 2-D int32");
        TORCH_CHECK(m.size(0) * 2 == mtx_in && m.size(1) == out_size, "sparse_mask must be (matrix rows / 2, out_size)");
        mask_ptr = m.data_ptr();
    }

    const bool matvec = route == Route::MATVEC || (route == Route::AUTO && seq_len == 1);
    c10::cuda::CUDAGuard guard(dev);
    auto stream = c10::cuda::getCurrentCUDAStream(dev.index());
    Tensor ws = workspace_for(dev, stream);
    const int status = i4mm_quant_matmul(
        (int)bits, matvec ? 1 : 0, /*path=*/g_static_weights.load() ? I4MM_PATH_STATIC_WEIGHTS : 0, outs.data_ptr(), matrix.data_ptr(), mask_ptr, multiplier.data_ptr(),
        scales.data_ptr(), zeros.data_ptr(), batch * seq_len, in_size, out_size, scales.size(0), group_size,
        ws.data_ptr(), (size_t)ws.numel(), (void*)stream.stream());
    check_status(status, "int4matmul");
}

void quant_matmul(uint32_t bits, I4_TENSOR_MULT_ARGS) { quant_mult(bits, Route::AUTO, I4_TENSOR_MULT_PASS); }

#define I4_REGISTER_WIDTH(N)                                                                              \
    void spec_mm_int##N(I4_TENSOR_MULT_ARGS) { quant_mult(N, Route::AUTO, I4_TENSOR_MULT_PASS); }         \
    void matmul_int##N(I4_TENSOR_MULT_ARGS) { quant_mult(N, Route::MATMUL, I4_TENSOR_MULT_PASS); }        \
    void matvec_int##N(I4_TENSOR_MULT_ARGS) { quant_mult(N, Route::MATVEC, I4_TENSOR_MULT_PASS); }
I4_REGISTER_WIDTH(4)
I4_REGISTER_WIDTH(3)
I4_REGISTER_WIDTH(2)

void weight_matrix_packing(Tensor wt_outs, Tensor msk_outs, Tensor wt_in, Tensor msk_in) {
    TORCH_CHECK(wt_in.is_cuda(), "wt_in must be a CUDA tensor");
    const auto dev = wt_in.device();
    for (const Tensor* t : {&wt_outs, &msk_outs, &wt_in, &msk_in}) {
        TORCH_CHECK(t->is_cuda() && t->device() == dev && t->is_contiguous() && t->dim() == 2,
                    "all four tensors must be contiguous 2-D CUDA tensors on one device");
    }
    // utils_kernel.cu:74-82
    TORCH_CHECK(wt_in.size(1) == wt_outs.size(0) * 16, "wt_in columns must be 16 x wt_outs rows");
    TORCH_CHECK(msk_in.size(1) == msk_outs.size(0) * 32, "msk_in columns must be 32 x msk_outs rows");
    TORCH_CHECK(wt_in.size(0) == wt_outs.size(1) && msk_in.size(0) == msk_outs.size(1), "row/column counts must match");
    TORCH_CHECK(wt_in.size(0) == msk_in.size(0) && wt_in.size(1) == msk_in.size(1), "wt_in and msk_in must have one shape");
    TORCH_CHECK(wt_outs.scalar_type() == torch::kInt && msk_outs.scalar_type() == torch::kInt, "outputs must be int32");
    TORCH_CHECK(wt_in.scalar_type() == torch::kByte && msk_in.scalar_type() == torch::kByte, "inputs must be uint8");
    TORCH_CHECK(wt_in.size(1) % 32 == 0, "in_size must be a multiple of 32 (utils_kernel.cu:101)");

    c10::cuda::CUDAGuard guard(dev);
    auto stream = c10::cuda::getCurrentCUDAStream(dev.index());
    Tensor violations = torch::zeros({1}, torch::dtype(torch::kInt).device(dev));
    const int status = i4mm_sparse_pack(wt_outs.data_ptr(), msk_outs.data_ptr(), wt_in.data_ptr(), msk_in.data_ptr(),
                                        wt_in.size(0), wt_in.size(1), violations.data_ptr(), (void*)stream.stream());
    check_status(status, "weight_matrix_packing");
    const int bad = violations.item<int>();
    if (bad != 0) {
        throw std::invalid_argument("weight_matrix_packing: " + std::to_string(bad) +
                                    " block(s) of 32 weights do not keep exactly 16 (16:32 sparsity)");
    }
}

// Not in the reference (its kernels have no waits): waits for every stream this module has launched on, on the
// current device, and raises if a kernel gave up on one of its bounded device-side waits since the last check.
// The multiply entries do not call it themselves, because it synchronises.
void check_device_status() {
    int dev = 0;
    TORCH_CHECK(cudaGetDevice(&dev) == cudaSuccess, "no current CUDA device");
    std::vector<Workspace> mine;
    {
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        for (auto& kv : g_workspaces)
            if (kv.first.first == dev) mine.push_back(kv.second);
    }
    int worst = I4MM_OK;
    for (auto& w : mine) {
        const int st = i4mm_device_status(w.buffer.data_ptr(), (void*)w.stream);
        if (st == I4MM_ERR_TIMEOUT) {                     // the scratch of a cut-short launch is not all-zero any more
            w.buffer.zero_();
            cudaDeviceSynchronize();
        }
        if (st != I4MM_OK) worst = st;
    }
    check_status(worst, "int4matmul device status");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("set_static_weights", &set_static_weights,
          "declare that weight-side tensors are never written by the kernel preceding a multiply in the stream");
    m.def("check_device_status", &check_device_status,
          "raise if a kernel launched by this module gave up on a bounded device-side wait (synchronises)");

    m.def("weight_matrix_packing", &weight_matrix_packing, "int4_sparse_pack");

    m.def("quant_matmul", &quant_matmul, "intn_fp16_mult");

    m.def("quant_int4_linear_mult", &spec_mm_int4, "int4_fp16_mult");
    m.def("quant_int4_linear_mult_mtx", &matmul_int4, "int4_fp16_mult_mtx");
    m.def("quant_int4_linear_mult_vec", &matvec_int4, "int4_fp16_mult_vec");

    m.def("quant_int3_linear_mult", &spec_mm_int3, "int3_fp16_mult");
    m.def("quant_int3_linear_mult_mtx", &matmul_int3, "int3_fp16_mult_mtx");
    m.def("quant_int3_linear_mult_vec", &matvec_int3, "int3_fp16_mult_vec");

    m.def("quant_int2_linear_mult", &spec_mm_int2, "int2_fp16_mult");
    m.def("quant_int2_linear_mult_mtx", &matmul_int2, "int2_fp16_mult_mtx");
    m.def("quant_int2_linear_mult_vec", &matvec_int2, "int2_fp16_mult_vec");
}
