// Tensor-core (tcgen05 / TMEM) delta convolutions. Placeholder translation unit: the
// entry points report "no tensor-core kernel for this shape" until the kernels land.
#include "dc_common.cuh"

namespace dc {

size_t filter_umma_bytes(const dc_conv_desc*, int) { return 0; }

int pack_filter_umma(const dc_conv_desc*, int, const void*, void*, cudaStream_t) { return DC_ERR_UNSUPPORTED; }

int conv2d_umma(const dc_conv_desc*, const void*, const int32_t*, const void*, const void*, void*, int32_t*,
                const dc_epilogue*, cudaStream_t) {
    return DC_ERR_UNSUPPORTED;
}

}  // namespace dc
