#include "../../include/int4matmul_b200.h"
#include "common.cuh"
namespace i4mm {
bool umma_supported(int, bool, int, int, int) { return false; }
int umma_launch(int, bool, const StreamParams&, int, int, int, cudaStream_t, cudaError_t*) { return I4MM_ERR_UNSUPPORTED; }
}
