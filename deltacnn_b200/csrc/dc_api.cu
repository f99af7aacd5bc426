// C-ABI plumbing: status strings, launch-error bookkeeping, and the convolution entry
// points that choose between the tensor-core and the CUDA-core kernels.
#include <cstdlib>
#include "dc_common.cuh"

namespace dc {

static thread_local int t_last_cuda_error = 0;

int sm_count() {
    static thread_local int cached_dev = -1;
    static thread_local int cached = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cached;
    if (dev != cached_dev) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) cached = v;
        // DC_GRID_SHARE=k sizes every grid for 1/k of the SMs, for callers that run k kernels side by side
        const char* e = getenv("DC_GRID_SHARE");
        const int share = e != nullptr ? atoi(e) : 1;
        if (share > 1 && cached / share >= 1) cached /= share;
        cached_dev = dev;
    }
    return cached;
}

bool pdl_enabled() {
    static const bool on = [] { const char* e = getenv("DC_NO_PDL"); return !(e != nullptr && e[0] == '1'); }();
    return on;
}

int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return DC_OK;
    t_last_cuda_error = (int)e;
    return DC_ERR_LAUNCH;
}

int conv2d_simt(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                int32_t* mo, cudaStream_t st);
int deconv2d_simt(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                  int32_t* mo, cudaStream_t st);
// tensor-core kernels (dc_conv_umma.cu); return DC_ERR_UNSUPPORTED when the shape has none
int conv2d_umma(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st);
size_t filter_umma_bytes(const dc_conv_desc* d, int transposed);
int pack_filter_umma(const dc_conv_desc* d, int transposed, const void* hwio, void* packed, cudaStream_t st);
int umma_error_code();
int stem_umma_error_code();
int irb_error_code();
int halo_error_code();
int conv_stem_umma(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                   int32_t* mo, const dc_epilogue* ep, cudaStream_t st);
int conv_thin(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
              int32_t* mo, cudaStream_t st);
int conv_pw_simt(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                 int32_t* mo, cudaStream_t st);
int conv_stem(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
              int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st);
int dwconv3x3_strip(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                    int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st);
size_t conv_workspace_bytes(const dc_conv_desc* d);
size_t deconv_workspace_bytes(const dc_conv_desc* d);
int deconv2d_umma(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                  int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st);

static int run_epilogue(const dc_conv_desc* d, void* out, int32_t* mo, const dc_epilogue* ep, void* stream) {
    if (ep == nullptr) return DC_OK;
    if (mo == nullptr) return DC_ERR_NULL_POINTER;
    return dc_activate_truncate(out, ep->prev_out, ep->truncated, mo, (int64_t)d->n * d->h_out * d->w_out, d->c_out,
                                d->dtype, ep->threshold, ep->activation, ep->truncation, stream);
}

}  // namespace dc

using namespace dc;

extern "C" {

int dc_version(void) { return 100; }

const char* dc_status_string(int status) {
    switch (status) {
        case DC_OK: return "ok";
        case DC_ERR_NULL_POINTER: return "a required pointer is NULL";
        case DC_ERR_UNSUPPORTED: return "unsupported kernel size, stride, groups or mode";
        case DC_ERR_ALIGNMENT: return "pointer not aligned for the vector width in use";
        case DC_ERR_SHAPE: return "inconsistent or non-positive sizes";
        case DC_ERR_DTYPE: return "dtype must be float32 (0) or float16 (1)";
        case DC_ERR_LAUNCH: return "CUDA launch failed";
        case DC_ERR_WORKSPACE: return "workspace too small";
        default: return "unknown status";
    }
}

int dc_last_cuda_error(void) { return t_last_cuda_error; }

int dc_umma_error(void) {
    const int a = umma_error_code();
    if (a != 0) return a;
    const int b = stem_umma_error_code();
    if (b != 0) return b;
    const int c = irb_error_code();
    return c != 0 ? c : halo_error_code();
}

int dc_conv2d_ws(const dc_conv_desc* desc, const void* in, const int32_t* mask_in, const void* filter, int32_t filter_layout,
                 const void* bias, void* out, int32_t* mask_out, const dc_epilogue* epilogue, void* workspace,
                 size_t workspace_bytes, void* stream) {
    if (desc == nullptr || in == nullptr || filter == nullptr || out == nullptr) return DC_ERR_NULL_POINTER;
    const bool residual_only = epilogue != nullptr && epilogue->residual != nullptr;
    if (epilogue != nullptr && !residual_only && (epilogue->prev_out == nullptr || (epilogue->truncation >= 0 && epilogue->truncated == nullptr)))
        return DC_ERR_NULL_POINTER;
    if (residual_only && filter_layout != DC_FILTER_UMMA) return DC_ERR_UNSUPPORTED;   // the caller adds with dc_add
    if (workspace != nullptr && workspace_bytes < conv_workspace_bytes(desc)) return DC_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    if (filter_layout == DC_FILTER_UMMA)
        return conv2d_umma(desc, in, mask_in, filter, bias, out, mask_out, epilogue, workspace, workspace_bytes, st);
    if (filter_layout != DC_FILTER_HWIO) return DC_ERR_UNSUPPORTED;
    int rc = dwconv3x3_strip(desc, in, mask_in, filter, bias, out, mask_out, epilogue, workspace, workspace_bytes, st);
    if (rc != DC_ERR_UNSUPPORTED) return rc;
    rc = conv_stem_umma(desc, in, mask_in, filter, bias, out, mask_out, epilogue, st);      // RGB stems on the tensor core
    if (rc != DC_ERR_UNSUPPORTED) return rc;
    rc = conv_stem(desc, in, mask_in, filter, bias, out, mask_out, epilogue, workspace, workspace_bytes, st);
    if (rc != DC_ERR_UNSUPPORTED) return rc;
    rc = conv_thin(desc, in, mask_in, filter, bias, out, mask_out, st);
    if (rc == DC_ERR_UNSUPPORTED) rc = conv_pw_simt(desc, in, mask_in, filter, bias, out, mask_out, st);
    if (rc == DC_ERR_UNSUPPORTED) rc = conv2d_simt(desc, in, mask_in, filter, bias, out, mask_out, st);
    if (rc != DC_OK) return rc;
    return run_epilogue(desc, out, mask_out, epilogue, stream);
}

int dc_conv2d(const dc_conv_desc* desc, const void* in, const int32_t* mask_in, const void* filter, int32_t filter_layout,
              const void* bias, void* out, int32_t* mask_out, const dc_epilogue* epilogue, void* stream) {
    return dc_conv2d_ws(desc, in, mask_in, filter, filter_layout, bias, out, mask_out, epilogue, nullptr, 0, stream);
}

size_t dc_conv_workspace_bytes(const dc_conv_desc* desc) { return desc == nullptr ? 0 : conv_workspace_bytes(desc); }

int dc_deconv2d_ws(const dc_conv_desc* desc, const void* in, const int32_t* mask_in, const void* filter, int32_t filter_layout,
                   const void* bias, void* out, int32_t* mask_out, const dc_epilogue* epilogue, void* workspace,
                   size_t workspace_bytes, void* stream) {
    if (desc == nullptr || in == nullptr || filter == nullptr || out == nullptr) return DC_ERR_NULL_POINTER;
    if (epilogue != nullptr && epilogue->residual != nullptr) return DC_ERR_UNSUPPORTED;   // residual connections: 1x1 convolutions only
    if (epilogue != nullptr && (epilogue->prev_out == nullptr || (epilogue->truncation >= 0 && epilogue->truncated == nullptr)))
        return DC_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (filter_layout == DC_FILTER_UMMA) {
        if (workspace != nullptr && workspace_bytes < deconv_workspace_bytes(desc)) return DC_ERR_WORKSPACE;
        return deconv2d_umma(desc, in, mask_in, filter, bias, out, mask_out, epilogue, workspace, workspace_bytes, st);
    }
    if (filter_layout != DC_FILTER_HWIO) return DC_ERR_UNSUPPORTED;
    int rc = deconv2d_simt(desc, in, mask_in, filter, bias, out, mask_out, st);
    if (rc != DC_OK) return rc;
    return run_epilogue(desc, out, mask_out, epilogue, stream);
}

int dc_deconv2d(const dc_conv_desc* desc, const void* in, const int32_t* mask_in, const void* filter, int32_t filter_layout,
                const void* bias, void* out, int32_t* mask_out, const dc_epilogue* epilogue, void* stream) {
    return dc_deconv2d_ws(desc, in, mask_in, filter, filter_layout, bias, out, mask_out, epilogue, nullptr, 0, stream);
}

size_t dc_deconv_workspace_bytes(const dc_conv_desc* desc) { return desc == nullptr ? 0 : deconv_workspace_bytes(desc); }

size_t dc_filter_umma_bytes(const dc_conv_desc* desc, int32_t transposed) {
    if (desc == nullptr) return 0;
    return filter_umma_bytes(desc, transposed);
}

int dc_pack_filter_umma(const dc_conv_desc* desc, int32_t transposed, const void* filter_hwio, void* filter_umma,
                        void* stream) {
    if (desc == nullptr || filter_hwio == nullptr || filter_umma == nullptr) return DC_ERR_NULL_POINTER;
    return pack_filter_umma(desc, transposed, filter_hwio, filter_umma, (cudaStream_t)stream);
}

}  // extern "C"
