// Warp-specialised kernel, row mode, windows 3 wide.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_am3(const GemmParams& p, cudaStream_t st) { return ws_launch_am<3>(p, st); }
}  // namespace ds
