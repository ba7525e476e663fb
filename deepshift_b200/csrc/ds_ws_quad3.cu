// Warp-specialised kernel, row mode for 3-wide windows staged four pixels at a time.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_quad3(const GemmParams& p, cudaStream_t st) { return ws_launch_am<AM_QUAD3>(p, st); }
}  // namespace ds
