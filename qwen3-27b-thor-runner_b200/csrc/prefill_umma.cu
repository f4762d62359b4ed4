// placeholder until the kernel lands
#include "nvfp4_internal.h"
namespace nvfp4 {
bool prefill_umma_supported(const LinearArgs&) { return false; }
size_t prefill_umma_scratch_bytes(int, int, int) { return 0; }
cudaError_t launch_prefill_umma(const LinearArgs&, const nvfp4_device_info&, void*, size_t, int*, cudaStream_t) {
    return cudaErrorNotSupported;
}
cudaError_t configure_kernels(const nvfp4_device_info&) { return configure_decode_mma(); }
}  // namespace nvfp4
