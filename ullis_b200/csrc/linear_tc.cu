#include "linear_tc.hpp"

namespace ullis {
namespace tc {

bool binary_linear(ullis_cuda_runtime*, const float*, const uint32_t*, const uint16_t*, const uint16_t*, float*,
                   size_t, size_t, size_t) {
    return false;
}
bool fp16_linear(ullis_cuda_runtime*, const float*, const uint16_t*, float*, size_t, size_t, size_t) { return false; }
bool rosa_qkv_bits(ullis_cuda_runtime*, const float*, const LayerWeights&, uint32_t*, uint32_t*, uint32_t*, size_t,
                   size_t, size_t) {
    return false;
}
bool rosa_out_residual(ullis_cuda_runtime*, const uint32_t*, const LayerWeights&, float*, size_t, size_t, size_t) {
    return false;
}
bool cmix_residual(ullis_cuda_runtime*, const LayerWeights&, float*, size_t, size_t, size_t, size_t) { return false; }
bool head_ce(ullis_cuda_runtime*, const float*, const PackedWeights&, const uint32_t*, uint32_t, size_t, size_t,
             size_t, size_t, float*) {
    return false;
}

}  // namespace tc
}  // namespace ullis
