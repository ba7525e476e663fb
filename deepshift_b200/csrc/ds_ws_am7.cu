// Warp-specialised kernel, row mode, windows 7 wide.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_am7(const GemmParams& p, cudaStream_t st) { return ws_launch_am<7>(p, st); }
}  // namespace ds
