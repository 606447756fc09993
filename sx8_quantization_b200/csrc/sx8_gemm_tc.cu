// sx8_gemm_tc.cu -- tcgen05 prefill GEMM (placeholder translation unit until the kernel lands).
#include "sx8_common.cuh"

namespace sx8 {
size_t gemm_tc_workspace_bytes(int, int, int) { return 0; }
bool gemm_tc_supported(int, int, int, int) { return false; }
int gemm_tc_launch(const void*, int, int, long, const void*, const float*, const float*, int, int, void*, int,
                   void*, cudaStream_t) {
    set_error("sx8_gemm: tcgen05 path not built");
    return SX8_E_UNSUPPORTED;
}
}  // namespace sx8
