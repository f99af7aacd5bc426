// CUDA-core delta convolutions: the fp32 path of every layer, and the fp16 path of the
// layers that have no tensor-core kernel (depthwise, 3-channel stems, odd shapes).
//
//  k_conv_tile   groups == 1, any kernel size / stride / dilation, and (TRANSPOSED) the
//                transposed convolution. One CTA per 8x8 output tile: the in-mask of the
//                tile's receptive field is staged first; a tile without an active input
//                leaves at once; otherwise the input patch (inactive pixels as zeros) and a
//                slab of the filter are staged per input-channel chunk and every thread
//                accumulates 4 pixels x 4 output channels in fp32 registers.
//  k_dwconv      depthwise: an aligned lane group per output pixel, 16-byte channel packs,
//                per-tap mask skipping, fp32 accumulation.
#include "dc_common.cuh"

namespace dc {

struct ConvGeom {
    int n, hi, wi, ci, ho, wo, co;
    int kh, kw, sh, sw, pt, pl, dh, dw;
    int ph, pw;        // staged input patch (pixels)
    int ck;            // input channels per chunk
    int w_off;         // offset (floats) of the filter slab inside dynamic shared memory, 16-byte aligned
    int tiles_x, tiles_y;
};

constexpr int kTile = 8;      // output tile edge
constexpr int kCT = 64;       // output channels per pass
constexpr int kConvThreads = 256;

__host__ __device__ inline int floordiv(int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }

template <typename T, bool TRANSPOSED>
__global__ void __launch_bounds__(kConvThreads)
k_conv_tile(const T* __restrict__ in, const int32_t* __restrict__ mi, const T* __restrict__ filt,
            const T* __restrict__ bias, T* __restrict__ out, int32_t* __restrict__ mo, ConvGeom g) {
    extern __shared__ float smem[];
    const int npatch = g.ph * g.pw;
    int* s_mask = reinterpret_cast<int*>(smem);                 // [npatch]
    int* s_omask = s_mask + npatch;                             // [64]
    float* s_in = reinterpret_cast<float*>(s_omask + 64);       // [npatch][ck]
    float* s_w = smem + g.w_off;                                // [taps][ck][kCT]

    const int tid = threadIdx.x;
    int bid = blockIdx.x;
    const int tx = bid % g.tiles_x; bid /= g.tiles_x;
    const int ty = bid % g.tiles_y;
    const int b = bid / g.tiles_y;
    const int oy0 = ty * kTile, ox0 = tx * kTile;
    // origin of the staged input patch
    int py0, px0;
    if (TRANSPOSED) {
        py0 = floordiv(oy0 + g.pt - (g.kh - 1), g.sh);
        px0 = floordiv(ox0 + g.pl - (g.kw - 1), g.sw);
    } else {
        py0 = oy0 * g.sh - g.pt;
        px0 = ox0 * g.sw - g.pl;
    }
    const int64_t img_in = (int64_t)b * g.hi * g.wi;

    bool any = false;
    for (int i = tid; i < npatch; i += kConvThreads) {
        const int y = py0 + i / g.pw, x = px0 + i % g.pw;
        int m = 0;
        if (y >= 0 && y < g.hi && x >= 0 && x < g.wi) m = (mi == nullptr) ? 1 : (mi[img_in + (int64_t)y * g.wi + x] != 0);
        s_mask[i] = m;
        any |= m != 0;
    }
    any = __syncthreads_or(any);

    const int taps = g.kh * g.kw;
    // patch index of the input pixel that tap (ky,kx) pairs with output pixel (ly,lx) of the tile, or -1
    auto src_index = [&](int ly, int lx, int ky, int kx) -> int {
        if (TRANSPOSED) {
            const int ty_ = oy0 + ly + g.pt - ky, tx_ = ox0 + lx + g.pl - kx;
            if (ty_ < 0 || tx_ < 0 || ty_ % g.sh != 0 || tx_ % g.sw != 0) return -1;
            const int py = ty_ / g.sh - py0, px = tx_ / g.sw - px0;
            if (py < 0 || py >= g.ph || px < 0 || px >= g.pw) return -1;
            return py * g.pw + px;
        } else {
            return (ly * g.sh + ky * g.dh) * g.pw + lx * g.sw + kx * g.dw;
        }
    };

    if (tid < kTile * kTile) {
        const int ly = tid / kTile, lx = tid % kTile;
        int om = 0;
        const bool inb = (oy0 + ly) < g.ho && (ox0 + lx) < g.wo;
        if (any && inb) {
            for (int t = 0; t < taps && !om; ++t) {
                const int si = src_index(ly, lx, t / g.kw, t % g.kw);
                if (si >= 0) om = s_mask[si];
            }
        }
        if (inb && mo != nullptr) mo[((int64_t)b * g.ho + oy0 + ly) * g.wo + ox0 + lx] = om;
        // without an out-mask every in-bounds pixel is written (zeros + bias where inactive)
        s_omask[tid] = inb ? (mo == nullptr ? 1 : om) : 0;
    }
    __syncthreads();
    if (!any && mo != nullptr) return;

    const int pg = tid >> 4, cg = tid & 15;
    const int ly = pg >> 1, lx0 = (pg & 1) * 4;
    bool mine = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) mine |= s_omask[ly * kTile + lx0 + j] != 0;

    for (int co0 = 0; co0 < g.co; co0 += kCT) {
        float acc[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[j][k] = 0.f;
        const int cw = min(kCT, g.co - co0);
        if (any) {
            for (int ci0 = 0; ci0 < g.ci; ci0 += g.ck) {
                const int cc = min(g.ck, g.ci - ci0);
                __syncthreads();
                for (int i = tid; i < npatch * cc; i += kConvThreads) {
                    const int p = i / cc, c = i % cc;
                    float v = 0.f;
                    if (s_mask[p]) {
                        const int y = py0 + p / g.pw, x = px0 + p % g.pw;
                        v = to_f<T>(in[(img_in + (int64_t)y * g.wi + x) * g.ci + ci0 + c]);
                    }
                    s_in[p * g.ck + c] = v;
                }
                for (int i = tid; i < taps * cc * kCT; i += kConvThreads) {
                    const int o = i % kCT;
                    const int c = (i / kCT) % cc;
                    const int t = i / (kCT * cc);
                    s_w[(t * g.ck + c) * kCT + o] = (o < cw) ? to_f<T>(filt[((int64_t)t * g.ci + ci0 + c) * g.co + co0 + o]) : 0.f;
                }
                __syncthreads();
                if (!mine) continue;
                for (int t = 0; t < taps; ++t) {
                    const int ky = t / g.kw, kx = t % g.kw;
                    int si[4];
                    bool tap_any = false;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        int s = src_index(ly, lx0 + j, ky, kx);
                        if (s >= 0 && s_mask[s] == 0) s = -1;
                        si[j] = s;
                        tap_any |= s >= 0;
                    }
                    if (!tap_any) continue;
                    const float* wrow = s_w + (t * g.ck) * kCT + cg * 4;
                    for (int c = 0; c < cc; ++c) {
                        const float4 w = *reinterpret_cast<const float4*>(wrow + c * kCT);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float a = si[j] >= 0 ? s_in[si[j] * g.ck + c] : 0.f;
                            acc[j][0] = fmaf(a, w.x, acc[j][0]);
                            acc[j][1] = fmaf(a, w.y, acc[j][1]);
                            acc[j][2] = fmaf(a, w.z, acc[j][2]);
                            acc[j][3] = fmaf(a, w.w, acc[j][3]);
                        }
                    }
                }
            }
        }
        if (mine) {
            const int c = co0 + cg * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (s_omask[ly * kTile + lx0 + j] == 0) continue;
                T* o = out + (((int64_t)b * g.ho + oy0 + ly) * g.wo + ox0 + lx0 + j) * g.co + c;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (c + k < g.co) o[k] = from_f<T>(acc[j][k] + (bias ? to_f<T>(bias[c + k]) : 0.f));
                }
            }
        }
    }
}

struct DwGeom {
    int n, hi, wi, c, ho, wo;
    int kh, kw, sh, sw, pt, pl, dh, dw;
};

template <typename T, int W>
__global__ void __launch_bounds__(256)
k_dwconv(const T* __restrict__ in, const int32_t* __restrict__ mi, const T* __restrict__ filt, const T* __restrict__ bias,
         T* __restrict__ out, int32_t* __restrict__ mo, DwGeom p, int g) {
    const int nvec = p.c / W;
    const int64_t npix = (int64_t)p.n * p.ho * p.wo;
    const int lane = threadIdx.x & 31;
    const int lig = lane & (g - 1);
    const int ppw = 32 / g;
    const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t base = warp0 * ppw; base < npix; base += nwarps * ppw) {
        const int64_t px = base + lane / g;
        if (px >= npix) continue;
        const int ox = (int)(px % p.wo);
        const int64_t t = px / p.wo;
        const int oy = (int)(t % p.ho);
        const int64_t b = t / p.ho;
        const int y0 = oy * p.sh - p.pt, x0 = ox * p.sw - p.pl;
        // bit t of `on` = tap t is in bounds and active (kernels up to 8x8... taps <= 64)
        unsigned long long on = 0ull;
        for (int ky = 0; ky < p.kh; ++ky) {
            const int iy = y0 + ky * p.dh;
            if (iy < 0 || iy >= p.hi) continue;
            for (int kx = 0; kx < p.kw; ++kx) {
                const int ix = x0 + kx * p.dw;
                if (ix < 0 || ix >= p.wi) continue;
                if (mi == nullptr || mi[(b * p.hi + iy) * p.wi + ix] != 0) on |= 1ull << (ky * p.kw + kx);
            }
        }
        if (mo != nullptr && lig == 0) mo[px] = on ? 1 : 0;
        if (on == 0ull && mo != nullptr) continue;
        for (int i = lig; i < nvec; i += g) {
            float acc[W];
            if (bias) {
                Pack<T, W> bb; bb.load(bias + i * W);
#pragma unroll
                for (int k = 0; k < W; ++k) acc[k] = bb.get(k);
            } else {
#pragma unroll
                for (int k = 0; k < W; ++k) acc[k] = 0.f;
            }
            unsigned long long rem = on;
            while (rem) {
                const int tp = __ffsll((long long)rem) - 1;
                rem &= rem - 1;
                const int iy = y0 + (tp / p.kw) * p.dh, ix = x0 + (tp % p.kw) * p.dw;
                Pack<T, W> v, w;
                v.load(in + ((b * p.hi + iy) * p.wi + ix) * (int64_t)p.c + i * W);
                w.load(filt + (int64_t)tp * p.c + i * W);
#pragma unroll
                for (int k = 0; k < W; ++k) acc[k] = fmaf(v.get(k), w.get(k), acc[k]);
            }
            Pack<T, W> o;
#pragma unroll
            for (int k = 0; k < W; ++k) o.set(k, acc[k]);
            o.store(out + px * p.c + i * W);
        }
    }
}

static int validate(const dc_conv_desc* d) {
    if (d->n < 0 || d->h_in <= 0 || d->w_in <= 0 || d->c_in <= 0 || d->h_out <= 0 || d->w_out <= 0 || d->c_out <= 0 ||
        d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 || d->stride_w <= 0 || d->dil_h <= 0 || d->dil_w <= 0 ||
        d->pad_top < 0 || d->pad_left < 0 || d->pad_bottom < 0 || d->pad_right < 0 || d->groups <= 0)
        return DC_ERR_SHAPE;
    return DC_OK;
}

template <typename T, bool TRANSPOSED>
static int conv_tile_t(const dc_conv_desc* d, const T* in, const int32_t* mi, const T* filt, const T* bias, T* out,
                       int32_t* mo, cudaStream_t st) {
    ConvGeom g;
    g.n = d->n; g.hi = d->h_in; g.wi = d->w_in; g.ci = d->c_in; g.ho = d->h_out; g.wo = d->w_out; g.co = d->c_out;
    g.kh = d->kh; g.kw = d->kw; g.sh = d->stride_h; g.sw = d->stride_w; g.pt = d->pad_top; g.pl = d->pad_left;
    g.dh = d->dil_h; g.dw = d->dil_w;
    if (TRANSPOSED) {
        g.ph = (kTile - 1 + g.kh - 1) / g.sh + 2;
        g.pw = (kTile - 1 + g.kw - 1) / g.sw + 2;
    } else {
        g.ph = (kTile - 1) * g.sh + (g.kh - 1) * g.dh + 1;
        g.pw = (kTile - 1) * g.sw + (g.kw - 1) * g.dw + 1;
    }
    const int taps = g.kh * g.kw;
    int ck = 8192 / (taps * kCT);
    if (ck > 32) ck = 32;
    if (ck > g.ci) ck = g.ci;
    if (ck < 1) ck = 1;
    g.ck = ck;
    g.tiles_x = divup(g.wo, kTile);
    g.tiles_y = divup(g.ho, kTile);
    g.w_off = ((g.ph * g.pw + 64 + g.ph * g.pw * ck) + 3) & ~3;
    const size_t smem = sizeof(float) * ((size_t)g.w_off + (size_t)taps * ck * kCT);
    if (smem > 200 * 1024) return DC_ERR_UNSUPPORTED;
    auto kern = k_conv_tile<T, TRANSPOSED>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return check_launch();
    }
    const int64_t blocks = (int64_t)g.tiles_x * g.tiles_y * g.n;
    if (blocks > 0x7fffffffLL) return DC_ERR_SHAPE;
    kern<<<(unsigned)blocks, kConvThreads, smem, st>>>(in, mi, filt, bias, out, mo, g);
    return check_launch();
}

template <typename T>
static int dwconv_t(const dc_conv_desc* d, const T* in, const int32_t* mi, const T* filt, const T* bias, T* out,
                    int32_t* mo, cudaStream_t st) {
    constexpr int V = VecTraits<T>::kVec;
    if (d->kh * d->kw > 64) return DC_ERR_UNSUPPORTED;
    DwGeom p{d->n, d->h_in, d->w_in, d->c_in, d->h_out, d->w_out, d->kh, d->kw, d->stride_h, d->stride_w,
             d->pad_top, d->pad_left, d->dil_h, d->dil_w};
    const int C = d->c_in;
    const bool vec_ok = (C % V == 0) && aligned16(in) && aligned16(out) && aligned16(filt) && (bias == nullptr || aligned16(bias));
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    const int g = lanes_per_pixel(vec_ok ? C / V : C);
    int64_t blocks = divup64(divup64(npix, 32 / g), 8);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (vec_ok) k_dwconv<T, V><<<(unsigned)blocks, 256, 0, st>>>(in, mi, filt, bias, out, mo, p, g);
    else k_dwconv<T, 1><<<(unsigned)blocks, 256, 0, st>>>(in, mi, filt, bias, out, mo, p, g);
    return check_launch();
}

// Entry used by the C-ABI layer: CUDA-core convolution for an HWIO filter.
int conv2d_simt(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                int32_t* mo, cudaStream_t st) {
    int rc = validate(d);
    if (rc != DC_OK) return rc;
    const bool depthwise = d->groups > 1 && d->groups == d->c_in && d->c_in == d->c_out;
    if (d->groups != 1 && !depthwise) return DC_ERR_UNSUPPORTED;
    if (d->dtype == DC_F32) {
        return depthwise ? dwconv_t<float>(d, (const float*)in, mi, (const float*)filt, (const float*)bias, (float*)out, mo, st)
                         : conv_tile_t<float, false>(d, (const float*)in, mi, (const float*)filt, (const float*)bias, (float*)out, mo, st);
    }
    if (d->dtype == DC_F16) {
        return depthwise ? dwconv_t<__half>(d, (const __half*)in, mi, (const __half*)filt, (const __half*)bias, (__half*)out, mo, st)
                         : conv_tile_t<__half, false>(d, (const __half*)in, mi, (const __half*)filt, (const __half*)bias, (__half*)out, mo, st);
    }
    return DC_ERR_DTYPE;
}

int deconv2d_simt(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                  int32_t* mo, cudaStream_t st) {
    int rc = validate(d);
    if (rc != DC_OK) return rc;
    if (d->groups != 1 || d->dil_h != 1 || d->dil_w != 1) return DC_ERR_UNSUPPORTED;
    if (d->dtype == DC_F32)
        return conv_tile_t<float, true>(d, (const float*)in, mi, (const float*)filt, (const float*)bias, (float*)out, mo, st);
    if (d->dtype == DC_F16)
        return conv_tile_t<__half, true>(d, (const __half*)in, mi, (const __half*)filt, (const __half*)bias, (__half*)out, mo, st);
    return DC_ERR_DTYPE;
}

}  // namespace dc
