// Warp-specialised kernel, row mode for 3-wide windows staged two pixels at a time.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_pair3(const GemmParams& p, cudaStream_t st) { return ws_launch_am<AM_PAIR3>(p, st); }
}  // namespace ds
