// Placeholder translation unit: the tcgen05 backward is not built yet; the dispatcher falls back
// to the CUDA-core backward for every shape.
#include "kernels.cuh"

namespace ember {
bool sm100_bwd_supported(const AttnArgs &) { return false; }
int sm100_attention_bwd(const AttnArgs &, float *, DeviceState *, cudaStream_t)
{
    set_error("tcgen05 backward is not available");
    return EMBER_ERR_UNSUPPORTED;
}
}  // namespace ember
