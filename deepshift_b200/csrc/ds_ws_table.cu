// Warp-specialised kernel, table mode: any window shape, one table entry per k.
#include "ds_gemm_ws.cuh"

namespace ds {
int launch_ws_table(const GemmParams& p, cudaStream_t st) { return ws_launch_am<AM_TABLE>(p, st); }
}  // namespace ds
