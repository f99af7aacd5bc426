// Test infrastructure: a C-ABI shim over the reference project's own host
// launchers (src/cuda/conv_kernel.cuh, deconv_kernel.cuh, other_nn_layers.cuh),
// so that GPU parity tests and the benchmark can run the reference kernels next
// to this library's kernels in one process through ctypes. The reference sources
// are compiled where they lie; nothing of them is stored in this repository.
// The reference launches on the legacy default stream and checks no launch
// error; the shim synchronises the device and reports cudaGetLastError().
#include <stdint.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include "conv_kernel.cuh"
#include "deconv_kernel.cuh"
#include "other_nn_layers.cuh"

namespace {
Dimensions make_dim(int n, int hi, int wi, int ci, int ho, int wo, int co) {
    Dimensions d;
    d.batch_size = (uint16_t)n;
    d.in.h = (uint16_t)hi; d.in.w = (uint32_t)wi; d.in.c = (uint16_t)ci;
    d.out.h = (uint16_t)ho; d.out.w = (uint32_t)wo; d.out.c = (uint16_t)co;
    return d;
}
// geometry: kh kw sh sw pad_top pad_left pad_bottom pad_right dh dw groups
ConvConfig make_cfg(const int* g, bool set_zero) {
    ConvConfig c;
    c.kernel_size[0] = (uint16_t)g[0]; c.kernel_size[1] = (uint16_t)g[1];
    c.stride[0] = (uint16_t)g[2]; c.stride[1] = (uint16_t)g[3];
    c.padding[0] = (uint16_t)g[4]; c.padding[1] = (uint16_t)g[5];
    c.padding[2] = (uint16_t)g[6]; c.padding[3] = (uint16_t)g[7];
    c.dilation[0] = (uint16_t)g[8]; c.dilation[1] = (uint16_t)g[9];
    c.groups = (uint16_t)g[10];
    c.padding_mode = zeros;
    c.sub_tile_sparsity = true;
    c.set_sparse_zero = set_zero;
    return c;
}
int finish(bool sync) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return 100 + (int)e;
    if (sync) {
        e = cudaDeviceSynchronize();
        if (e != cudaSuccess) return 100 + (int)e;
    }
    return 0;
}
}  // namespace

#define REF_GUARD(stmt) try { stmt; } catch (...) { return 1; }

extern "C" {

int ref_conv(int f16, void* in, void* out, void* filter, void* bias, uint32_t* mask, uint32_t* out_mask,
             const int* shape7, const int* geom11, int sync) {
    Dimensions d = make_dim(shape7[0], shape7[1], shape7[2], shape7[3], shape7[4], shape7[5], shape7[6]);
    ConvConfig c = make_cfg(geom11, out_mask == nullptr);
    if (f16) { REF_GUARD(deltacnn_hp((half*)in, (half*)out, (half*)filter, (half*)bias, mask, out_mask, d, c)) }
    else { REF_GUARD(deltacnn<float>((float*)in, (float*)out, (float*)filter, (float*)bias, mask, out_mask, d, c)) }
    return finish(sync);
}

int ref_deconv(int f16, void* in, void* out, void* filter, void* bias, uint32_t* mask, uint32_t* out_mask,
               const int* shape7, const int* geom11, int sync) {
    Dimensions d = make_dim(shape7[0], shape7[1], shape7[2], shape7[3], shape7[4], shape7[5], shape7[6]);
    ConvConfig c = make_cfg(geom11, out_mask == nullptr);
    if (f16) { REF_GUARD(delta_deconv_hp((half*)in, (half*)out, (half*)filter, (half*)bias, mask, out_mask, d, c)) }
    else { REF_GUARD(delta_deconv<float>((float*)in, (float*)out, (float*)filter, (float*)bias, mask, out_mask, d, c)) }
    return finish(sync);
}

int ref_pool(int f16, void* in, void* prev_in, void* out, uint32_t* mask, uint32_t* out_mask,
             const int* shape7, const int* geom11, int pooling_mode, int sync) {
    Dimensions d = make_dim(shape7[0], shape7[1], shape7[2], shape7[3], shape7[4], shape7[5], shape7[6]);
    ConvConfig c = make_cfg(geom11, out_mask == nullptr);
    if (f16) { REF_GUARD(sparse_pool_hp<half>((half*)in, (half*)prev_in, (half*)out, mask, out_mask, d, c, pooling_mode)) }
    else { REF_GUARD(sparse_pool<float>((float*)in, (float*)prev_in, (float*)out, mask, out_mask, d, c, pooling_mode)) }
    return finish(sync);
}

int ref_activate_truncate(int f16, void* delta, void* prev, void* truncated, uint32_t* mask, float threshold,
                          int n, int h, int w, int ch, int activation, int truncation_mode, int sync) {
    Dimensions d = make_dim(n, h, w, ch, h, w, ch);
    if (f16) { REF_GUARD(activate_truncate_hp<half>((half*)delta, (half*)prev, (half*)truncated, mask, threshold, d, activation, truncation_mode)) }
    else { REF_GUARD(activate_truncate<float>((float*)delta, (float*)prev, (float*)truncated, mask, threshold, d, activation, truncation_mode)) }
    return finish(sync);
}

int ref_sparsify(int f16, void* input, void* prev, void* delta, uint32_t* mask, float threshold,
                 int n, int h, int w, int ch, int sync) {
    Dimensions d = make_dim(n, h, w, ch, h, w, ch);
    if (f16) { REF_GUARD(prepare_diff_mask_hp<half>((half*)input, (half*)prev, (half*)delta, mask, threshold, d)) }
    else { REF_GUARD(prepare_diff_mask<float>((float*)input, (float*)prev, (float*)delta, mask, threshold, d)) }
    return finish(sync);
}

int ref_add(int f16, void* a, void* b, void* prev_out, void* out, uint32_t* mask_a, uint32_t* mask_b, uint32_t* mask_out,
            float wa, float wb, int n, int h, int w, int ch, int activation, int dense_out, int sync) {
    Dimensions d = make_dim(n, h, w, ch, h, w, ch);
    if (f16) { REF_GUARD(sparse_add_tensors_hp<half>((half*)a, (half*)b, (half*)prev_out, (half*)out, mask_a, mask_b, mask_out, wa, wb, d, activation, dense_out != 0)) }
    else { REF_GUARD(sparse_add_tensors<float>((float*)a, (float*)b, (float*)prev_out, (float*)out, mask_a, mask_b, mask_out, wa, wb, d, activation, dense_out != 0)) }
    return finish(sync);
}

int ref_add_to_dense(int f16, void* a, void* b, uint32_t* mask_a, int n, int h, int w, int ch, int activation, int sync) {
    Dimensions d = make_dim(n, h, w, ch, h, w, ch);
    if (f16) { REF_GUARD(sparse_add_to_dense_tensor_hp<half>((half*)a, (half*)b, mask_a, d, activation)) }
    else { REF_GUARD(sparse_add_to_dense_tensor_sp<float>((float*)a, (float*)b, mask_a, d, activation)) }
    return finish(sync);
}

int ref_upsample(int f16, void* in, void* out, uint32_t* mask_in, uint32_t* mask_out,
                 int n, int h, int w, int ch, int scale, int sync) {
    Dimensions d = make_dim(n, h, w, ch, h * scale, w * scale, ch);
    if (f16) { REF_GUARD(sparse_upsample_hp<half>((half*)in, (half*)out, mask_in, mask_out, d, scale)) }
    else { REF_GUARD(sparse_upsample<float>((float*)in, (float*)out, mask_in, mask_out, d, scale)) }
    return finish(sync);
}

int ref_concat(int f16, void* a, void* b, void* out, uint32_t* mask_a, uint32_t* mask_b, uint32_t* mask_out,
               int n, int h, int w, int ca, int cb, int sync) {
    // the reference wrapper passes in.c = channels of a, out.c = channels of a + b
    Dimensions d = make_dim(n, h, w, ca, h, w, ca + cb);
    if (f16) { REF_GUARD(sparse_concatenate_hp<half>((half*)a, (half*)b, (half*)out, mask_a, mask_b, mask_out, d)) }
    else { REF_GUARD(sparse_concatenate<float>((float*)a, (float*)b, (float*)out, mask_a, mask_b, mask_out, d)) }
    return finish(sync);
}

int ref_mul_add(int f16, void* in, uint32_t* mask, void* out, uint32_t* mask_out, void* scale, void* bias,
                int n, int h, int w, int ch, int sync) {
    Dimensions d = make_dim(n, h, w, ch, h, w, ch);
    if (f16) { REF_GUARD(sparse_mul_add_hp<half>((half*)in, mask, (half*)out, mask_out, (half*)scale, (half*)bias, d)) }
    else { REF_GUARD(sparse_mul_add<float>((float*)in, mask, (float*)out, mask_out, (float*)scale, (float*)bias, d)) }
    return finish(sync);
}

}  // extern "C"
