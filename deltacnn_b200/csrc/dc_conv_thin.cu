// Pointwise delta convolution with very few output channels (detection / pose heads: 64 -> 1, 64 -> 2,
// 32 -> 17): too thin for a tensor-core tile, pure bandwidth. An aligned lane group per active pixel reads
// the pixel's channel packs (16 bytes per lane), every lane forms its partial dot products with the filter
// held in shared memory as fp32, and the group reduces them with shuffles.
#include "dc_common.cuh"

namespace dc {

constexpr int kThinMaxCout = 32;

// kCo: compile-time bound on the output channels (1, 2, 4, 8, 16, 32): the accumulators and the inner loops are sized
// by it, so a one-channel head does not pay for thirty-two.
template <typename T, int W, int kCo>
__global__ void __launch_bounds__(256) k_conv_thin(const T* __restrict__ in, const int32_t* __restrict__ mi,
                                                   const T* __restrict__ filt, const T* __restrict__ bias,
                                                   T* __restrict__ out, int32_t* __restrict__ mo, int64_t npix, int cin,
                                                   int cout, int g) {
    extern __shared__ float s_w[];                               // [cin][cout], then bias [cout]
    grid_dep_launch();
    for (int i = threadIdx.x; i < cin * cout; i += 256) s_w[i] = to_f<T>(filt[i]);
    float* s_b = s_w + cin * cout;
    for (int i = threadIdx.x; i < cout; i += 256) s_b[i] = bias ? to_f<T>(bias[i]) : 0.f;
    grid_dep_wait();
    __syncthreads();
    const int nvec = cin / W;
    const int lane = threadIdx.x & 31;
    const int lig = lane & (g - 1);
    const int ppw = 32 / g;
    const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * 8;
    for (int64_t base = warp0 * ppw; base < npix; base += nwarps * ppw) {
        const int64_t px = base + lane / g;
        const bool on = px < npix && mi[px] != 0;
        if (px < npix && lig == 0) mo[px] = on ? 1 : 0;
        if (__ballot_sync(DC_FULL, on) == 0) continue;
        float acc[kCo];
#pragma unroll
        for (int co = 0; co < kCo; ++co) acc[co] = 0.f;
        if (on) {
            for (int i = lig; i < nvec; i += g) {
                Pack<T, W> v;
                v.load(in + px * cin + i * W);
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    const float a = v.get(k);
                    const float* wr = s_w + (i * W + k) * cout;
#pragma unroll
                    for (int co = 0; co < kCo; ++co)
                        if (co < cout) acc[co] = fmaf(a, wr[co], acc[co]);
                }
            }
        }
#pragma unroll
        for (int co = 0; co < kCo; ++co) {
            if (co >= cout) break;
            const float s = group_sum(acc[co], g);
            if (on && (co % g) == lig) out[px * cout + co] = from_f<T>(s + s_b[co]);
        }
    }
}

// 1x1, stride 1, no padding, groups 1, at most 32 output channels, with in- and out-mask.
int conv_thin(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
              int32_t* mo, cudaStream_t st) {
    const bool ok = d->kh == 1 && d->kw == 1 && d->stride_h == 1 && d->stride_w == 1 && d->groups == 1 && d->pad_top == 0 &&
                    d->pad_left == 0 && d->pad_bottom == 0 && d->pad_right == 0 && d->c_out <= kThinMaxCout &&
                    (d->c_out % 8 != 0 || d->c_out < 16) && d->c_in >= 8 && mi != nullptr && mo != nullptr;
    if (!ok) return DC_ERR_UNSUPPORTED;
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    if (npix == 0) return DC_OK;
    const size_t smem = sizeof(float) * ((size_t)d->c_in * d->c_out + d->c_out);
    if (smem > 48 * 1024) return DC_ERR_UNSUPPORTED;
    auto launch = [&](auto kernel, int nvec, auto* tin, auto* tf, auto* tb, auto* tout) {
        const int g = lanes_per_pixel(nvec);
        int64_t blocks = divup64(divup64(npix, 32 / g), 8);
        const int64_t cap = (int64_t)sm_count() * 16;
        if (blocks > cap) blocks = cap;
        return launch_pdl(kernel, dim3((unsigned)blocks), dim3(256), smem, st, tin, mi, tf, tb, tout, mo, npix, d->c_in, d->c_out, g);
    };
#define DC_THIN(T, W, nvec)                                                                                                         \
    do {                                                                                                                            \
        const T* tin = (const T*)in; const T* tf = (const T*)filt; const T* tb = (const T*)bias; T* tout = (T*)out;                  \
        if (d->c_out <= 1) return launch(k_conv_thin<T, W, 1>, nvec, tin, tf, tb, tout);                                             \
        if (d->c_out <= 2) return launch(k_conv_thin<T, W, 2>, nvec, tin, tf, tb, tout);                                             \
        if (d->c_out <= 4) return launch(k_conv_thin<T, W, 4>, nvec, tin, tf, tb, tout);                                             \
        if (d->c_out <= 8) return launch(k_conv_thin<T, W, 8>, nvec, tin, tf, tb, tout);                                             \
        if (d->c_out <= 16) return launch(k_conv_thin<T, W, 16>, nvec, tin, tf, tb, tout);                                           \
        return launch(k_conv_thin<T, W, 32>, nvec, tin, tf, tb, tout);                                                               \
    } while (0)
    if (d->dtype == DC_F16) {
        if (d->c_in % 8 == 0 && aligned16(in)) DC_THIN(__half, 8, d->c_in / 8);
        DC_THIN(__half, 1, d->c_in);
    }
    if (d->dtype == DC_F32) {
        if (d->c_in % 4 == 0 && aligned16(in)) DC_THIN(float, 4, d->c_in / 4);
        DC_THIN(float, 1, d->c_in);
    }
#undef DC_THIN
    return DC_ERR_DTYPE;
}

// Pointwise (1x1, stride 1, no padding) delta convolution on CUDA cores for the cases the tensor-core path does not take
// (fp32; odd channel counts): a CTA owns 16 consecutive pixels x 64 output channels, so a small map still spreads over
// many CTAs through its output channels (the generic tile kernel gives one 8x8 pixel tile all channels: a 7x7 map of a
// single stream ran on one CTA). Thread = one output channel x four pixels; the input chunk (16 pixels x 32 channels)
// and the filter chunk (32 channels x the CTA's output channels) sit in shared memory. fp32 accumulation in a fixed order.
// kCW: output channels per CTA (64: a thread owns four pixels; 16: one pixel, four times the CTAs for layers with few
// output channels and few pixels).
template <typename T, int kCW>
__global__ void __launch_bounds__(256) k_conv_pw_simt(const T* __restrict__ in, const int32_t* __restrict__ mi,
                                                      const T* __restrict__ filt, const T* __restrict__ bias,
                                                      T* __restrict__ out, int32_t* __restrict__ mo, int64_t npix, int cin, int cout) {
    __shared__ float s_x[16][33];
    __shared__ float s_wt[32][kCW + 1];
    __shared__ int s_on[16];
    grid_dep_launch();
    grid_dep_wait();
    constexpr int kPhases = 256 / kCW, kPer = 16 / kPhases;         // pixel phases of the CTA, pixels per thread
    const int tid = threadIdx.x, tx = tid % kCW, ty = tid / kCW;    // output channel within the slab, pixel phase
    const int64_t q0 = (int64_t)blockIdx.x * 16;
    const int co = blockIdx.y * kCW + tx;
    if (tid < 16) {
        const int64_t q = q0 + tid;
        const int on = (q < npix && mi[q] != 0) ? 1 : 0;
        s_on[tid] = on;
        if (q < npix && blockIdx.y == 0) mo[q] = on;
    }
    __syncthreads();
    bool any = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) any |= s_on[i] != 0;
    if (!any) return;
    float acc[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) acc[j] = 0.f;
    for (int c0 = 0; c0 < cin; c0 += 32) {
        // 16 pixels x 32 channels of the input: two elements per thread, channels fastest; inactive pixels read zeros
        for (int e = tid; e < 16 * 32; e += 256) {
            const int pi = e >> 5, c = c0 + (e & 31);
            s_x[pi][e & 31] = (s_on[pi] && c < cin) ? to_f<T>(in[(q0 + pi) * cin + c]) : 0.f;
        }
        // ... and 32 channels x kCW output channels of the filter, coalesced over the output channels: all of a chunk's
        // reads are in flight together
        for (int e = tid; e < 32 * kCW; e += 256) {
            const int c = c0 + e / kCW, o = blockIdx.y * kCW + e % kCW;
            s_wt[e / kCW][e % kCW] = (c < cin && o < cout) ? to_f<T>(filt[(int64_t)c * cout + o]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int c = 0; c < 32; ++c) {
            const float wv = s_wt[c][tx];
#pragma unroll
            for (int j = 0; j < kPer; ++j) acc[j] = fmaf(s_x[ty + kPhases * j][c], wv, acc[j]);
        }
        __syncthreads();
    }
    if (co < cout) {
        const float b = bias != nullptr ? to_f<T>(bias[co]) : 0.f;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
            const int pi = ty + kPhases * j;
            if (s_on[pi]) out[(q0 + pi) * cout + co] = from_f<T>(acc[j] + b);
        }
    }
}

// 1x1, stride 1, no padding, groups 1 on maps of at most 16384 pixels per call (larger maps keep the tile kernel, whose
// tiles skip inactive regions); fp32 and fp16.
int conv_pw_simt(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                 int32_t* mo, cudaStream_t st) {
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    const bool ok = d->kh == 1 && d->kw == 1 && d->stride_h == 1 && d->stride_w == 1 && d->groups == 1 && d->pad_top == 0 &&
                    d->pad_left == 0 && d->pad_bottom == 0 && d->pad_right == 0 && mi != nullptr && mo != nullptr && npix <= 16384 &&
                    d->c_out >= 16;
    if (!ok) return DC_ERR_UNSUPPORTED;
    if (npix == 0) return DC_OK;
    const bool narrow = divup64(npix, 16) * divup(d->c_out, 64) < sm_count();       // few CTAs: narrower channel slabs
    const dim3 grid((unsigned)divup64(npix, 16), (unsigned)divup(d->c_out, narrow ? 16 : 64));
#define DC_PW_SIMT(T)                                                                                                              \
    do {                                                                                                                           \
        if (narrow) return launch_pdl(k_conv_pw_simt<T, 16>, grid, dim3(256), 0, st, (const T*)in, mi, (const T*)filt,             \
                                      (const T*)bias, (T*)out, mo, npix, d->c_in, d->c_out);                                       \
        return launch_pdl(k_conv_pw_simt<T, 64>, grid, dim3(256), 0, st, (const T*)in, mi, (const T*)filt, (const T*)bias,         \
                          (T*)out, mo, npix, d->c_in, d->c_out);                                                                   \
    } while (0)
    if (d->dtype == DC_F32) DC_PW_SIMT(float);
    if (d->dtype == DC_F16) DC_PW_SIMT(__half);
#undef DC_PW_SIMT
    return DC_ERR_DTYPE;
}

}  // namespace dc
