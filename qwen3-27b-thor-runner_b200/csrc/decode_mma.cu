// placeholder until the kernel lands
#include "nvfp4_internal.h"
namespace nvfp4 {
bool decode_mma_supported(const LinearArgs&) { return false; }
size_t decode_mma_scratch_bytes(const LinearArgs&, const nvfp4_device_info&) { return 0; }
cudaError_t launch_decode_mma(const LinearArgs&, const nvfp4_device_info&, void*, int*, cudaStream_t) {
    return cudaErrorNotSupported;
}
}  // namespace nvfp4
