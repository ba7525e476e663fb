// Warp-specialised kernel, row mode, windows 1 wide.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_am1(const GemmParams& p, cudaStream_t st) { return ws_launch_am<1>(p, st); }
}  // namespace ds
