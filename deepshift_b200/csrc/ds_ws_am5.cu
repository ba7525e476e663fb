// Warp-specialised kernel, row mode, windows 5 wide.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_am5(const GemmParams& p, cudaStream_t st) { return ws_launch_am<5>(p, st); }
}  // namespace ds
