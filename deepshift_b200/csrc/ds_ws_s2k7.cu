// Warp-specialised kernel, row mode for 7-wide stride-2 windows staged four output pixels at a time.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_s2k7(const GemmParams& p, cudaStream_t st) { return ws_launch_am<AM_S2K7>(p, st); }
}  // namespace ds
