/*
 * deltacnn_b200 -- C-ABI of the delta-update inference kernels (sm_100a).
 *
 * Every entry point takes raw DEVICE pointers, plain sizes, and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t; NULL is the legacy default stream), and
 * returns a dc_status. Nothing here allocates, frees or synchronises: all tensors,
 * caches and masks are owned by the caller, as in the reference extension, whose
 * wrappers receive preallocated torch tensors (src/deltacnn/cuda_kernels.py:34-45).
 *
 * Layout: feature/delta tensors are N,H,W,C contiguous ("channels last"), dtype
 * float32 or float16; masks are int32, one word per pixel, values 0/1, N,H,W
 * contiguous. "npix" is N*H*W. Pixels whose mask is 0 are never read; output
 * pixels whose out-mask is 0 are left untouched (undefined, as in the reference).
 *
 * Each declaration cites the reference interface it replaces (path:line within the
 * reference project).
 */
#ifndef DELTACNN_B200_H
#define DELTACNN_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum dc_status {
    DC_OK = 0,
    DC_ERR_NULL_POINTER = 1,   /* a required pointer is NULL */
    DC_ERR_UNSUPPORTED = 2,    /* kernel size / stride / groups / mode not supported */
    DC_ERR_ALIGNMENT = 3,      /* a pointer is not aligned for the vector width in use */
    DC_ERR_SHAPE = 4,          /* inconsistent or non-positive sizes */
    DC_ERR_DTYPE = 5,          /* dtype is neither DC_F32 nor DC_F16 */
    DC_ERR_LAUNCH = 6,         /* the CUDA runtime refused the launch (see dc_last_cuda_error) */
    DC_ERR_WORKSPACE = 7       /* caller-provided workspace too small */
} dc_status;

typedef enum dc_dtype { DC_F32 = 0, DC_F16 = 1 } dc_dtype;

/* Activation codes, as src/deltacnn/sparse_layers.py:20-34 (<=0: identity). */
typedef enum dc_activation {
    DC_ACT_NONE = 0, DC_ACT_RELU = 1, DC_ACT_RELU6 = 2, DC_ACT_LEAKY = 3 /* slope 0.1 */,
    DC_ACT_SIGMOID = 4, DC_ACT_SWISH = 5
} dc_activation;

/* Truncation modes, as DCTruncation in src/deltacnn/sparse_layers.py:102-106. */
typedef enum dc_truncation { DC_TRUNC_NONE = -1, DC_TRUNC_MAX = 0, DC_TRUNC_NORM = 1, DC_TRUNC_RMS = 2 } dc_truncation;

/* Shape and geometry of a convolution, transposed convolution or pooling call.
 * Replaces Dimensions + ConvConfig (src/cuda/common.cuh:14-35), with 32-bit fields. */
typedef struct dc_conv_desc {
    int32_t n, h_in, w_in, c_in;
    int32_t h_out, w_out, c_out;
    int32_t kh, kw;
    int32_t stride_h, stride_w;
    int32_t pad_top, pad_left, pad_bottom, pad_right;
    int32_t dil_h, dil_w;
    int32_t groups;          /* 1, or c_in == c_out == groups (depthwise) */
    int32_t dtype;           /* dc_dtype */
} dc_conv_desc;

/* Optional fused epilogue of dc_conv2d / dc_deconv2d: the accumulate + activation
 * delta + truncation step of dc_activate_truncate applied to the convolution result
 * before it is stored. prev_out / truncated have the shape of the output. */
typedef struct dc_epilogue {
    void* prev_out;
    void* truncated;
    float threshold;
    int32_t activation;      /* dc_activation */
    int32_t truncation;      /* dc_truncation; DC_TRUNC_MAX only when fused */
    /* Optional residual connection (no reference counterpart; replaces a DCAdd behind a linear convolution,
     * sparse_layers.py DCAdd.forward / sparse_add_tensors_wrapper): a delta tensor of the output's shape and its
     * update mask. sum = convolution (where its out-mask is set) + residual (where residual_mask is set), the
     * out-mask is the union. truncation must be DC_TRUNC_NONE. With activation == DC_ACT_NONE out = sum (prev_out
     * and truncated unused, may be NULL); with an activation, prev_out is the add layer's accumulated sum:
     * u = prev_out + sum, out = f(u) - f(prev_out), prev_out = u (the arithmetic of dc_add). fp16, stride 1 and the
     * DC_FILTER_UMMA layout: 1x1 without padding, or KxK called without scratch memory (patch tiles); anything else
     * returns DC_ERR_UNSUPPORTED and the caller adds with dc_add. */
    const void* residual;
    const int32_t* residual_mask;
} dc_epilogue;

/* Filter layouts understood by dc_conv2d / dc_deconv2d. */
typedef enum dc_filter_layout {
    DC_FILTER_HWIO = 0,      /* [kh][kw][c_in/groups][c_out], same dtype as the features */
    DC_FILTER_UMMA = 1       /* private pre-tiled fp16 layout written by dc_pack_filter_umma */
} dc_filter_layout;

int dc_version(void);
const char* dc_status_string(int status);
/* cudaError_t of the most recent failed launch on this thread (0 if none). */
int dc_last_cuda_error(void);

/* Input delta + update mask. Replaces deltacnn_prepare_diff_mask_wrapper
 * (src/cuda/conv_torch_wrapper.cpp:347-384; kernels src/cuda/other_nn_layers.cu:821,1261).
 * d = x - prev_in; mask = any_c(|d| > threshold); active pixels: delta = d, prev_in = x. */
int dc_sparsify(const void* x, void* prev_in, void* delta, int32_t* mask,
                int64_t npix, int32_t channels, int32_t dtype, float threshold, void* stream);

/* Same as dc_sparsify on an 8-bit frame: x_u8 holds N,H,W,C bytes and the pixel
 * value compared and cached is x_u8 * scale[c] + offset[c] (float32 per-channel
 * tables on the device). No reference counterpart; it fuses the preprocessing of
 * example/mobilenetv2_webcam_example.py:79-111 into the first kernel. */
int dc_sparsify_u8(const uint8_t* x_u8, const float* scale, const float* offset, void* prev_in, void* delta,
                   int32_t* mask, int64_t npix, int32_t channels, int32_t dtype, float threshold, void* stream);

/* DCSparsify(dilation = k), the noise-robust input mask (src/deltacnn/sparse_layers.py:1233-1248, where it is four
 * torch operators and a boolean-index copy per frame): delta = x - prev_in at EVERY pixel, mask = 1 where the
 * k x k window centred on the pixel (stride 1, in-bounds elements) holds a pixel with any |delta| > threshold, and
 * prev_in = x where the mask is set. k must be odd, at most 33. hit_scratch: n*h*w bytes of device memory, only
 * meaningful during the call. */
int dc_sparsify_dilated(const void* x, void* prev_in, void* delta, int32_t* mask, uint8_t* hit_scratch, int32_t n, int32_t h,
                        int32_t w, int32_t channels, int32_t dtype, float threshold, int32_t dilation, void* stream);

/* Delta convolution. Replaces sparse_conv_bias_wrapper_masked
 * (src/cuda/conv_torch_wrapper.cpp:62-134 -> deltacnn / deltacnn_hp, src/cuda/conv_kernel.cu:3443,3947).
 * mask_out[q] = OR of mask_in over the in-bounds taps of q; out[q] = sum_taps W^T (in * mask_in) (+ bias).
 * mask_in NULL: every input pixel is active. mask_out NULL: out is written at every
 * pixel (zeros (+bias) where no tap is active), the reference's set_sparse_zero mode.
 * epilogue may be NULL. */
int dc_conv2d(const dc_conv_desc* desc, const void* in, const int32_t* mask_in,
              const void* filter, int32_t filter_layout, const void* bias,
              void* out, int32_t* mask_out, const dc_epilogue* epilogue, void* stream);

/* Scratch bytes dc_conv2d_ws wants for this geometry (16 + 8 bytes per output pixel). */
size_t dc_conv_workspace_bytes(const dc_conv_desc* desc);

/* dc_conv2d with caller-provided scratch memory for the active-pixel work list: a light pass
 * writes the out-mask and compacts the active output pixels into `workspace`, and the convolution
 * kernel then sizes its work by that list (persistent CTAs), which is what makes sparse frames
 * cheap however the active pixels cluster. Same results as dc_conv2d. The scratch is only
 * meaningful during the call; calls on different streams need different scratch. Shapes without a
 * list-driven kernel fall back to dc_conv2d. No reference counterpart (the reference re-derives
 * activity inside every tile, src/cuda/conv_kernel.cu:46-108). */
int dc_conv2d_ws(const dc_conv_desc* desc, const void* in, const int32_t* mask_in,
                 const void* filter, int32_t filter_layout, const void* bias,
                 void* out, int32_t* mask_out, const dc_epilogue* epilogue,
                 void* workspace, size_t workspace_bytes, void* stream);

/* dc_conv2d_ws without any allocation on the caller's side or inside the library. No counterpart in the
 * reference. It exists for hosts that are not allowed to allocate device memory when they call: a
 * plugin that lives inside another application's fixed device-memory allotment, or a control loop that
 * must stay away from the allocator (and the synchronisation it implies) once it runs. The work-list scratch
 * is a fixed array inside this library's device image (4 MiB per GPU that loads the library, held until
 * the process exits), so the call handles at most dc_static_workspace_max_pixels() = 524288 output
 * pixels (n*h_out*w_out) and returns DC_ERR_WORKSPACE beyond that. The first call on a device looks up
 * the array's device address (cudaGetSymbolAddress, with that device current); make that first call
 * before any stream capture. All calls share the one array, which keeps the previous call's list: the
 * counter is cleared at the start of every call, and two calls that overlap on the GPU (different
 * streams, or different threads) race on it -- serialise them or use dc_conv2d_ws with separate scratch.
 * Results are those of dc_conv2d. */
int dc_conv2d_static(const dc_conv_desc* desc, const void* in, const int32_t* mask_in,
                     const void* filter, int32_t filter_layout, const void* bias,
                     void* out, int32_t* mask_out, const dc_epilogue* epilogue, void* stream);
size_t dc_static_workspace_max_pixels(void);

/* Delta transposed convolution (4x4 stride 2, 6x6 stride 4 and any k = m*stride, groups 1).
 * Replaces sparse_deconv_bias_wrapper_masked (src/cuda/conv_torch_wrapper.cpp:136-210 ->
 * delta_deconv / delta_deconv_hp, src/cuda/deconv_kernel.cu:854-932). Filter HWIO:
 * [kh][kw][c_in][c_out] (taps un-flipped, as torch ConvTranspose2d weight[ci][co][ky][kx]). */
int dc_deconv2d(const dc_conv_desc* desc, const void* in, const int32_t* mask_in,
                const void* filter, int32_t filter_layout, const void* bias,
                void* out, int32_t* mask_out, const dc_epilogue* epilogue, void* stream);

/* dc_deconv2d with caller-provided scratch for per-phase active-pixel work lists (16 + 32 bytes per
 * output pixel, dc_deconv_workspace_bytes). With a DC_FILTER_UMMA filter image (stride 2, kernel 2m x 2m,
 * fp16) the four output phases run as m x m implicit GEMMs on the tensor cores. Same results as
 * dc_deconv2d. No reference counterpart. */
int dc_deconv2d_ws(const dc_conv_desc* desc, const void* in, const int32_t* mask_in,
                   const void* filter, int32_t filter_layout, const void* bias,
                   void* out, int32_t* mask_out, const dc_epilogue* epilogue,
                   void* workspace, size_t workspace_bytes, void* stream);
size_t dc_deconv_workspace_bytes(const dc_conv_desc* desc);

/* Bytes of the DC_FILTER_UMMA image of a filter (0 if the shape has no tensor-core kernel). */
size_t dc_filter_umma_bytes(const dc_conv_desc* desc, int32_t transposed);
/* Repack an fp16 HWIO filter on the device into the DC_FILTER_UMMA layout. */
int dc_pack_filter_umma(const dc_conv_desc* desc, int32_t transposed, const void* filter_hwio,
                        void* filter_umma, void* stream);

/* Sticky device-side error code of the tensor-core kernels on the current device: 0 = none,
 * otherwise the bounded wait that gave up (1 stage ring, 2 filter copy, 3 accumulator). The
 * call synchronises with the device. No reference counterpart. */
int dc_umma_error(void);

/* Accumulate + activation delta + truncation, in place on delta, mask and both caches.
 * Replaces deltacnn_activate_truncate (src/cuda/conv_torch_wrapper.cpp:295-344;
 * kernels src/cuda/other_nn_layers.cu:755,1198). truncated may be NULL when
 * truncation == DC_TRUNC_NONE. */
int dc_activate_truncate(void* delta, void* prev_out, void* truncated, int32_t* mask,
                         int64_t npix, int32_t channels, int32_t dtype,
                         float threshold, int32_t activation, int32_t truncation, void* stream);

/* Weighted add of two delta tensors. Replaces sparse_add_tensors_wrapper
 * (src/cuda/conv_torch_wrapper.cpp:387-444; kernels other_nn_layers.cu:1380,1563).
 * prev_out is required when activation > 0 or dense_out != 0. With dense_out the
 * output is f(prev_out) at every pixel and mask_out is not written (may be NULL). */
int dc_add(const void* a, const void* b, void* prev_out, void* out,
           const int32_t* mask_a, const int32_t* mask_b, int32_t* mask_out,
           float weight_a, float weight_b, int64_t npix, int32_t channels, int32_t dtype,
           int32_t activation, int32_t dense_out, void* stream);

/* b += a on the masked pixels of a. Replaces sparse_add_to_dense_tensor_wrapper
 * (src/cuda/conv_torch_wrapper.cpp:446-482; kernels other_nn_layers.cu:1732,1851). */
int dc_add_to_dense(const void* a, void* b, const int32_t* mask_a,
                    int64_t npix, int32_t channels, int32_t dtype, void* stream);

/* out = in * scale[c] (+ bias[c]) on masked pixels; mask copied to mask_out when they
 * differ. Replaces sparse_mul_add_wrapper (src/cuda/conv_torch_wrapper.cpp:569-630;
 * kernels other_nn_layers.cu:3774,3821). scale/bias have the feature dtype. */
int dc_scale_bias(const void* in, const int32_t* mask_in, void* out, int32_t* mask_out,
                  const void* scale, const void* bias,
                  int64_t npix, int32_t channels, int32_t dtype, void* stream);

/* Delta pooling. Replaces sparse_pooling_wrapper_masked (src/cuda/conv_torch_wrapper.cpp:213-293 ->
 * sparse_pool / sparse_pool_hp, other_nn_layers.cu:4509-4661).
 * pooling_mode 0 (max): out = max_win(prev_in + in*mask) - max_win(prev_in); when
 *   update_prev != 0 prev_in += in*mask is applied by the same call (the reference
 *   issues sparse_add_to_dense_tensor afterwards, src/deltacnn/sparse_layers.py:1468).
 * pooling_mode 1 (average): out = sum_win(in*mask) / (kh*kw); with h_out == w_out == 1
 *   and the window covering the image this is the global average pool, reduced in
 *   fp32 in a fixed order and stored in the feature dtype. */
int dc_pool(const dc_conv_desc* desc, const void* in, void* prev_in, const int32_t* mask_in,
            void* out, int32_t* mask_out, int32_t pooling_mode, int32_t update_prev, void* stream);

/* Nearest-neighbour upsampling of values and mask by an integer factor. Replaces
 * sparse_upsample_wrapper (src/cuda/conv_torch_wrapper.cpp:484-521; other_nn_layers.cu:3451,3527). */
int dc_upsample(const void* in, const int32_t* mask_in, void* out, int32_t* mask_out,
                int32_t n, int32_t h, int32_t w, int32_t channels, int32_t scale, int32_t dtype, void* stream);

/* Channel concatenation with mask union; the inactive side is zero-filled. Replaces
 * sparse_concatenate_wrapper (src/cuda/conv_torch_wrapper.cpp:523-567; other_nn_layers.cu:3602,3676). */
int dc_concat(const void* a, const void* b, void* out,
              const int32_t* mask_a, const int32_t* mask_b, int32_t* mask_out,
              int64_t npix, int32_t channels_a, int32_t channels_b, int32_t dtype, void* stream);

/* prev_out += delta on masked pixels and dense_out = f(prev_out) at every pixel, one
 * pass. Replaces the three launches of DCDensify.forward (src/deltacnn/sparse_layers.py:1322-1329:
 * deltacnn_activate_truncate without truncation, clone, torch activation).
 * dense_out may alias nothing; it may be NULL to only accumulate. */
int dc_densify(const void* delta, const int32_t* mask, void* prev_out, void* dense_out,
               int64_t npix, int32_t channels, int32_t dtype, int32_t activation, void* stream);

/* Number of active pixels of a mask and their compacted indices, built
 * with warp ballots and a block prefix scan; count is one int32 on the device,
 * indices holds up to npix int32 (ascending inside a block of 256 pixels, blocks in any order). Used to size work by the active set. No reference
 * counterpart (the reference re-derives activity inside every kernel,
 * src/cuda/conv_kernel.cu:46-108). */
int dc_compact_mask(const int32_t* mask, int64_t npix, int32_t* indices, int32_t* count, void* stream);

/* Fused inverted-residual block (MobileNetV2): expansion 1x1 + activation/truncation, depthwise 3x3 (padding 1,
 * stride 1 or 2) + activation/truncation, projection 1x1, optional residual add of the block input, in ONE launch for
 * steady-state frames (no bias: the reference adds biases on the first frame only, src/deltacnn/sparse_layers.py:616).
 * No reference counterpart: it replaces the three sparse_conv_bias_wrapper_masked calls, two deltacnn_activate_truncate
 * calls and the sparse_add_tensors_wrapper call of a block (example/mobilenet_deltacnn.py:87-128), with the same
 * results and cache updates bit for bit as dc_conv2d with fused epilogues. For small maps: the input rows of a band of
 * output rows, halo included, must fit 128 pixels and at most 8 bands cover the map (14x14 and 7x7 maps); fp16;
 * c_hidden a multiple of 64 (<= 1024), c_in a multiple of 8, c_out a multiple of 16; activations none / ReLU / ReLU6.
 * Other shapes return DC_ERR_UNSUPPORTED (dc_irb_supported tells in advance) and the caller runs the three layers. */
typedef struct dc_irb_desc {
    int32_t n, h, w;                 /* block input: n streams of h x w pixels */
    int32_t c_in, c_hidden, c_out;
    int32_t stride;                  /* of the depthwise convolution */
    int32_t residual;                /* != 0: out = projection + x where x is active (stride 1, c_in == c_out) */
    int32_t act_expand, act_dw;      /* dc_activation of the two truncation layers */
    int32_t dtype;                   /* DC_F16 */
    float thr_expand, thr_dw;        /* their thresholds */
} dc_irb_desc;
int dc_irb_supported(const dc_irb_desc* desc);
/* x, mask_in: block input (delta, mask). w_expand_umma / w_project_umma: DC_FILTER_UMMA images of the two 1x1 filters;
 * w_dw_hwio: depthwise filter [3][3][1][c_hidden]. prev_* / trunc_*: the caches of the two truncation layers (n, h, w,
 * c_hidden and n, h_out, w_out, c_hidden). out, mask_out: block output (n, h_out, w_out, c_out). */
int dc_irb_fused(const dc_irb_desc* desc, const void* x, const int32_t* mask_in, const void* w_expand_umma, const void* w_dw_hwio,
                 const void* w_project_umma, void* prev_expand, void* trunc_expand, void* prev_dw, void* trunc_dw, void* out,
                 int32_t* mask_out, void* stream);

/* Several 3x3 convolutions on the SAME input in one launch (the first layers of detection heads: CenterNet's heat-map,
 * size and offset heads each start with a 3x3 256 -> 64 convolution + ReLU on the same feature map). No reference
 * counterpart: it replaces n_heads sparse_conv_bias_wrapper_masked + deltacnn_activate_truncate pairs
 * (src/cuda/conv_torch_wrapper.cpp:62-134, 295-344) with the same results per head; the input tile is loaded once for
 * all heads. desc describes the concatenated layer (c_out = sum of the heads' output channels, which must be equal per
 * head, a multiple of 16, n_heads 2..4); filter_umma / bias are the DC_FILTER_UMMA image / bias of the filters
 * concatenated along the output channels. outs[h], masks_out[h]: output (n, h_out, w_out, c_out / n_heads) and out-mask of
 * head h. epilogues (array of n_heads, or NULL for plain stores): prev_out / truncated / threshold / activation of each
 * head's truncation layer (truncation DC_TRUNC_MAX). fp16, stride 1, no dilation, padding <= 1. Shapes without this form
 * return DC_ERR_UNSUPPORTED (dc_conv3x3_heads_supported tells in advance) and the caller runs the layers one by one. */
int dc_conv3x3_heads_supported(const dc_conv_desc* desc, int32_t n_heads);
int dc_conv3x3_heads(const dc_conv_desc* desc, const void* in, const int32_t* mask_in, const void* filter_umma, const void* bias,
                     int32_t n_heads, void* const* outs, int32_t* const* masks_out, const dc_epilogue* epilogues, void* stream);

/* ---- task heads behind the delta path -------------------------------------------------------------------
 * No counterpart among the reference's kernels: its networks end with DCDensify and dense torch code
 * (example/mobilenet_deltacnn.py:216-227: adaptive_avg_pooling -> densify -> reshape -> nn.Linear;
 * src/deltacnn/sparse_layers.py:1322-1329). These entry points keep that tail on the device and in delta form;
 * a stream (image of the batch) whose update mask is empty keeps its previous result. */

/* Fully connected layer on the delta of a pooled feature: for every stream n with mask[n] != 0 (all streams when
 * first_frame != 0 or mask is NULL), acc[n][o] += sum_c weight[o][c] * delta[n][c] (+ bias[o] on the first frame,
 * where acc starts from zero), and out[n][o] = acc[n][o] rounded to the feature dtype. delta: n x c_in; weight:
 * c_out x c_in (torch nn.Linear layout) and bias in the feature dtype; acc: n x c_out float32 state owned by the
 * caller. Replaces densify + nn.Linear of example/mobilenet_deltacnn.py:216-227 (a linear layer commutes with the
 * accumulation over frames). */
int dc_linear_delta(const void* delta, const int32_t* mask, const void* weight, const void* bias, float* acc, void* out,
                    int32_t n, int32_t c_in, int32_t c_out, int32_t dtype, int32_t first_frame, void* stream);

/* Arg-max of dense heat maps (n, h, w, joints channels last; the output of dc_densify): out[n][j] = (x, y, value)
 * of the largest element of joint j, the first in row-major order on ties. mask (n*h*w, may be NULL): streams
 * without an active pixel are skipped and out keeps their previous rows. */
int dc_heatmap_argmax(const void* heat, const int32_t* mask, float* out, int32_t n, int32_t h, int32_t w, int32_t joints,
                      int32_t dtype, void* stream);

/* CenterNet decode of dense head outputs (heat n,h,w,classes; wh and offset n,h,w,2; channels last): a peak is an
 * element equal to the maximum of its 3x3 neighbourhood; det[n][k] = (x1, y1, x2, y2, score, class) of the topk
 * best peaks with score > min_score, best first (ties: ascending pixel, class), centre (x + offset_x, y + offset_y),
 * size wh, all multiplied by stride; rows beyond count[n] are zero with class -1. peaks (n*h*w*classes float32) is
 * state owned by the caller: with a mask only pixels next to an updated pixel are re-examined, and streams without
 * an updated pixel keep their rows; mask NULL (first frame) examines everything. topk <= 1024. apply_sigmoid != 0
 * reports sigmoid(score). */
int dc_centernet_decode(const void* heat, const void* wh, const void* offset, const int32_t* mask, float* peaks, float* det,
                        int32_t* count, int32_t n, int32_t h, int32_t w, int32_t classes, int32_t topk, float min_score,
                        float stride, int32_t apply_sigmoid, int32_t dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DELTACNN_B200_H */
