// sx8_api.cu -- error reporting, version and the device error word of libsx8b200.so.
#include <stdarg.h>

#include "sx8_common.cuh"

namespace sx8 {

static thread_local char t_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
    return SX8_E_CUDA;
}

__device__ unsigned g_sx8_error_flag = 0;

}  // namespace sx8

extern "C" int sx8_version(void) { return 100; }

extern "C" const char* sx8_last_error(void) { return sx8::t_err; }

extern "C" int sx8_device_error_flag(unsigned* flag_out) {
    if (!flag_out) {
        sx8::set_error("sx8_device_error_flag: null pointer");
        return SX8_E_INVALID;
    }
    cudaError_t e = cudaMemcpyFromSymbol(flag_out, sx8::g_sx8_error_flag, sizeof(unsigned));
    if (e != cudaSuccess) return sx8::cuda_fail(e, "cudaMemcpyFromSymbol(error flag)");
    return SX8_OK;
}
