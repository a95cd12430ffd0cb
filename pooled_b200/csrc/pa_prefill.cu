// placeholder until the tiled prefill kernel lands
#include "pa_params.cuh"
namespace pa {
int prefill_supported(const pa_ctx*) { return 0; }
cudaError_t launch_prefill(const pa_layer*, const PrefillParams&, cudaStream_t) { return cudaErrorNotSupported; }
}
