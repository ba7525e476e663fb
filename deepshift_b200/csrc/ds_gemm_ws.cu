// Dispatcher of the warp-specialised kernel (ds_gemm_ws.cuh).  The instantiations live in one
// translation unit per window width (ds_ws_am*.cu) so that they compile side by side; this file
// owns what they share: the flag that a kernel sets when one of its bounded waits ran out.
#include "ds_gemm_common.cuh"

namespace ds {

int* kernel_error_flag();
int* bounds_status_ptr();

namespace {

__device__ int g_ws_error = 0;  // never set in a correct run

int* g_ws_error_ptr[kMaxDevices];  // device address of the flag, looked up once per device

__device__ int g_bounds_status = 0;  // checked build: site code of the first access outside its extent
int* g_bounds_status_ptr[kMaxDevices];

}  // namespace

int* kernel_error_flag()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!g_ws_error_ptr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_ws_error) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return nullptr;
        }
        g_ws_error_ptr[dev] = static_cast<int*>(ptr);
    }
    return g_ws_error_ptr[dev];
}

int* bounds_status_ptr()
{
#ifdef DS_BOUNDS_CHECK
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!g_bounds_status_ptr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_bounds_status) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return nullptr;
        }
        g_bounds_status_ptr[dev] = static_cast<int*>(ptr);
    }
    return g_bounds_status_ptr[dev];
#else
    return nullptr;
#endif
}

int launch_ws(const GemmParams& p0, int am, cudaStream_t st)
{
    GemmParams p = p0;
    p.err_flag = kernel_error_flag();
    if (!p.err_flag) return DS_ERR_CUDA;
    switch (am) {
        case AM_LINEAR: return launch_ws_linear(p, st);
        case AM_TABLE: return launch_ws_table(p, st);
        case AM_QUAD3: return launch_ws_quad3(p, st);
        case AM_PAIR3: return launch_ws_pair3(p, st);
        case AM_S2K7: return launch_ws_s2k7(p, st);
        case 1: return launch_ws_am1(p, st);
        case 3: return launch_ws_am3(p, st);
        case 5: return launch_ws_am5(p, st);
        case 7: return launch_ws_am7(p, st);
        default: return DS_ERR_UNSUPPORTED;
    }
}

}  // namespace ds

// Reads and clears the flag that a kernel sets when one of its bounded waits ran out.
// Synchronises the device.  0 = no error.
extern "C" int ds_last_kernel_error(int* flag)
{
    if (!flag) return DS_ERR_BAD_ARG;
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, ds::g_ws_error, sizeof(int)) != cudaSuccess) return DS_ERR_CUDA;
    const int zero = 0;
    if (v && cudaMemcpyToSymbol(ds::g_ws_error, &zero, sizeof(int)) != cudaSuccess) return DS_ERR_CUDA;
    *flag = v;
    return DS_OK;
}

// Checked build (-DDS_BOUNDS_CHECK): reads and clears the status word; *status = 0 means every
// access stayed inside its extent, 1 / 2 / 3 name the first offender (activations, packed weights,
// output or residual).  Synchronises the device.  A normal build reports 0 and *checked = 0.
extern "C" int ds_bounds_status(int* status, int* checked)
{
    if (!status) return DS_ERR_BAD_ARG;
    *status = 0;
#ifdef DS_BOUNDS_CHECK
    if (checked) *checked = 1;
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, ds::g_bounds_status, sizeof(int)) != cudaSuccess) return DS_ERR_CUDA;
    const int zero = 0;
    if (v && cudaMemcpyToSymbol(ds::g_bounds_status, &zero, sizeof(int)) != cudaSuccess) return DS_ERR_CUDA;
    *status = v;
#else
    if (checked) *checked = 0;
#endif
    return DS_OK;
}
