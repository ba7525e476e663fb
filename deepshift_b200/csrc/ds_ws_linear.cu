// Warp-specialised kernel for the linear layer: x is [M,K], a producer thread owns one row.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_linear(const GemmParams& p, cudaStream_t st) { return ws_launch_am<AM_LINEAR>(p, st); }
}  // namespace ds
