// Delta pooling: window max / average pooling on (delta, mask) with the accumulated
// input cache, and the global average pool. Bandwidth-bound; same pixel-group work
// decomposition as the element-wise kernels, indexed by OUTPUT pixel.
#include "dc_common.cuh"

namespace dc {

struct PoolGeom {
    int n, hi, wi, c, ho, wo;
    int kh, kw, sh, sw, pt, pl, pb, pr, dh, dw;
    uint32_t wo_mul, wo_shift, ho_mul, ho_shift;      // fast_div constants for w_out and h_out (fewer than 2^31 output pixels)
};

// mode 0: out = max_win(prev + in*mask) - max_win(prev) over in-bounds taps (fp32 math);
// mode 1: out = sum_win(in*mask) / (kh*kw).
template <typename T, int W>
__global__ void __launch_bounds__(256) k_pool(const T* __restrict__ in, const T* __restrict__ prev,
                                              const int32_t* __restrict__ mi, T* __restrict__ out,
                                              int32_t* __restrict__ mo, PoolGeom p, int mode, int g) {
    grid_dep_launch();
    grid_dep_wait();
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
        const uint32_t t = fast_div((uint32_t)px, p.wo_mul, p.wo_shift);
        const int ox = (int)((uint32_t)px - t * (uint32_t)p.wo);
        const int64_t b = (int64_t)fast_div(t, p.ho_mul, p.ho_shift);
        const int oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
        const int y0 = oy * p.sh - p.pt, x0 = ox * p.sw - p.pl;
        bool any = false;
        for (int ky = 0; ky < p.kh; ++ky) {
            const int iy = y0 + ky * p.dh;
            if (iy < 0 || iy >= p.hi) continue;
            for (int kx = 0; kx < p.kw; ++kx) {
                const int ix = x0 + kx * p.dw;
                if (ix < 0 || ix >= p.wi) continue;
                any |= mi == nullptr || mi[(b * p.hi + iy) * p.wi + ix] != 0;
            }
        }
        if (mo != nullptr && lig == 0) mo[px] = any ? 1 : 0;
        if (!any && mo != nullptr) continue;
        const float inv = 1.f / (float)(p.kh * p.kw);
        for (int i = lig; i < nvec; i += g) {
            float acc[W], pre[W];
#pragma unroll
            for (int k = 0; k < W; ++k) { acc[k] = mode == 0 ? -1e30f : 0.f; pre[k] = -1e30f; }
            for (int ky = 0; ky < p.kh; ++ky) {
                const int iy = y0 + ky * p.dh;
                if (iy < 0) continue;
                if (iy >= p.hi) {
                    // a zero joins the window below the image when bottom padding differs from top
                    // padding (pad-then-pool behaviour of the reference, other_nn_layers.cu:2402-2409)
                    if (mode == 0 && iy < p.hi + p.pb && p.pt != p.pb) {
#pragma unroll
                        for (int k = 0; k < W; ++k) { acc[k] = fmaxf(acc[k], 0.f); pre[k] = fmaxf(pre[k], 0.f); }
                    }
                    continue;
                }
                for (int kx = 0; kx < p.kw; ++kx) {
                    const int ix = x0 + kx * p.dw;
                    if (ix < 0) continue;
                    if (ix >= p.wi) {
                        if (mode == 0 && ix < p.wi + p.pr && p.pl != p.pr) {
#pragma unroll
                            for (int k = 0; k < W; ++k) { acc[k] = fmaxf(acc[k], 0.f); pre[k] = fmaxf(pre[k], 0.f); }
                        }
                        continue;
                    }
                    const int64_t src = (b * p.hi + iy) * p.wi + ix;
                    const bool on = mi == nullptr || mi[src] != 0;
                    if (mode == 1) {
                        if (!on) continue;
                        Pack<T, W> v; v.load(in + src * p.c + i * W);
#pragma unroll
                        for (int k = 0; k < W; ++k) acc[k] += v.get(k);
                    } else {
                        Pack<T, W> q; q.load(prev + src * p.c + i * W);
                        if (on) {
                            Pack<T, W> v; v.load(in + src * p.c + i * W);
#pragma unroll
                            for (int k = 0; k < W; ++k) {
                                // the accumulated value as the cache will hold it after this call (rounded to the storage
                                // type), so that consecutive frames' deltas telescope exactly
                                acc[k] = fmaxf(acc[k], rnd<T>(q.get(k) + v.get(k)));
                                pre[k] = fmaxf(pre[k], q.get(k));
                            }
                        } else {
#pragma unroll
                            for (int k = 0; k < W; ++k) {
                                acc[k] = fmaxf(acc[k], q.get(k));
                                pre[k] = fmaxf(pre[k], q.get(k));
                            }
                        }
                    }
                }
            }
            Pack<T, W> o;
#pragma unroll
            for (int k = 0; k < W; ++k) o.set(k, mode == 0 ? acc[k] - pre[k] : acc[k] * inv);
            o.store(out + px * p.c + i * W);
        }
    }
}

// Max pooling with a 3x3 window (no dilation, the same padding on opposite sides): the same arithmetic as k_pool with the
// window unrolled, so that the nine mask words are in flight together and every window row's six value reads as well
// (the general kernel walks the window tap by tap, one dependent mask read before each value read).
template <typename T, int W>
__global__ void __launch_bounds__(256) k_maxpool3(const T* __restrict__ in, const T* __restrict__ prev,
                                                  const int32_t* __restrict__ mi, T* __restrict__ out,
                                                  int32_t* __restrict__ mo, PoolGeom p, int g) {
    grid_dep_launch();
    grid_dep_wait();
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
        const uint32_t t = fast_div((uint32_t)px, p.wo_mul, p.wo_shift);
        const int ox = (int)((uint32_t)px - t * (uint32_t)p.wo);
        const int64_t b = (int64_t)fast_div(t, p.ho_mul, p.ho_shift);
        const int oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
        const int y0 = oy * p.sh - p.pt, x0 = ox * p.sw - p.pl;
        bool inb[9], on[9];
        int32_t mv[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) {
            const int iy = y0 + k / 3, ix = x0 + k % 3;
            inb[k] = iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi;
            mv[k] = inb[k] ? mi[(b * p.hi + iy) * p.wi + ix] : 0;
        }
        bool any = false;
#pragma unroll
        for (int k = 0; k < 9; ++k) { on[k] = mv[k] != 0; any |= on[k]; }
        if (mo != nullptr && lig == 0) mo[px] = any ? 1 : 0;
        if (!any && mo != nullptr) continue;
        const int64_t src0 = (b * p.hi + y0) * p.wi + x0;
        for (int i = lig; i < nvec; i += g) {
            float acc[W], pre[W];
#pragma unroll
            for (int k = 0; k < W; ++k) { acc[k] = -1e30f; pre[k] = -1e30f; }
#pragma unroll
            for (int ky = 0; ky < 3; ++ky) {
                Pack<T, W> q[3], v[3];
#pragma unroll
                for (int kx = 0; kx < 3; ++kx) {
                    const int k = ky * 3 + kx;
                    const int64_t src = src0 + (int64_t)ky * p.wi + kx;
                    if (inb[k]) q[kx].load(prev + src * p.c + i * W);
                    if (on[k]) v[kx].load(in + src * p.c + i * W);
                }
#pragma unroll
                for (int kx = 0; kx < 3; ++kx) {
                    const int k = ky * 3 + kx;
                    if (!inb[k]) continue;
#pragma unroll
                    for (int e = 0; e < W; ++e) {
                        const float qe = q[kx].get(e);
                        acc[e] = fmaxf(acc[e], on[k] ? rnd<T>(qe + v[kx].get(e)) : qe);
                        pre[e] = fmaxf(pre[e], qe);
                    }
                }
            }
            Pack<T, W> o;
#pragma unroll
            for (int k = 0; k < W; ++k) o.set(k, acc[k] - pre[k]);
            o.store(out + px * p.c + i * W);
        }
    }
}

// Global average pool: one CTA per (image, slab of 32 channel packs). The 256 threads are 8 pixel lanes x 32
// packs: lane j sums the active pixels j, j+8, ... of its pack in fp32, then the eight partial sums are
// added in a fixed order through shared memory, so the result is reproducible (the reference uses float
// atomics). The image's mask is staged in shared memory in chunks.
template <typename T, int W>
__global__ void __launch_bounds__(256) k_global_avg(const T* __restrict__ in, const int32_t* __restrict__ mi,
                                                    T* __restrict__ out, int32_t* __restrict__ mo, int hw, int C) {
    __shared__ int32_t s_mask[1024];
    __shared__ float s_part[8][32][W];
    __shared__ int s_any;
    grid_dep_launch();
    grid_dep_wait();
    const int b = blockIdx.y;
    const int nvec = C / W;
    const int pk = threadIdx.x & 31, pl = threadIdx.x >> 5;           // pack inside the slab, pixel lane
    const int vec = blockIdx.x * 32 + pk;
    float acc[W];
#pragma unroll
    for (int k = 0; k < W; ++k) acc[k] = 0.f;
    if (threadIdx.x == 0) s_any = 0;
    for (int p0 = 0; p0 < hw; p0 += 1024) {
        __syncthreads();
        const int cnt = min(1024, hw - p0);
        bool any = false;
        for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
            const int32_t m = mi == nullptr ? 1 : mi[(int64_t)b * hw + p0 + i];
            s_mask[i] = m;
            any |= m != 0;
        }
        if (any) s_any = 1;
        __syncthreads();
        if (vec < nvec) {
            for (int i = pl; i < cnt; i += 8) {
                if (s_mask[i] == 0) continue;
                Pack<T, W> v;
                v.load(in + ((int64_t)b * hw + p0 + i) * C + vec * W);
#pragma unroll
                for (int k = 0; k < W; ++k) acc[k] += v.get(k);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < W; ++k) s_part[pl][pk][k] = acc[k];
    __syncthreads();
    if (pl == 0 && vec < nvec) {
        Pack<T, W> o;
        const float inv = 1.f / (float)hw;
#pragma unroll
        for (int k = 0; k < W; ++k) {
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) sum += s_part[j][pk][k];
            o.set(k, sum * inv);
        }
        o.store(out + (int64_t)b * C + vec * W);
    }
    if (mo != nullptr && blockIdx.x == 0 && threadIdx.x == 0) mo[b] = s_any;
}

template <typename T>
static int pool_t(const dc_conv_desc* d, const T* in, T* prev, const int32_t* mi, T* out, int32_t* mo, int mode,
                  cudaStream_t st) {
    constexpr int V = VecTraits<T>::kVec;
    const int C = d->c_in;
    const bool vec_ok = (C % V == 0) && aligned16(in) && aligned16(out) && (prev == nullptr || aligned16(prev));
    const bool global = mode == 1 && d->h_out == 1 && d->w_out == 1 && d->kh == d->h_in && d->kw == d->w_in &&
                        d->pad_top == 0 && d->pad_left == 0 && d->pad_bottom == 0 && d->pad_right == 0 &&
                        d->dil_h == 1 && d->dil_w == 1;
    if (global) {
        const int hw = d->h_in * d->w_in;
        if (vec_ok) {
            dim3 grid(divup(C / V, 32), d->n);
            launch_pdl(k_global_avg<T, V>, grid, dim3(256), 0, st, in, mi, out, mo, hw, C);
        } else {
            dim3 grid(divup(C, 32), d->n);
            launch_pdl(k_global_avg<T, 1>, grid, dim3(256), 0, st, in, mi, out, mo, hw, C);
        }
        return check_launch();
    }
    PoolGeom p{d->n, d->h_in, d->w_in, C, d->h_out, d->w_out, d->kh, d->kw, d->stride_h, d->stride_w,
               d->pad_top, d->pad_left, d->pad_bottom, d->pad_right, d->dil_h, d->dil_w, 0u, 0u, 0u, 0u};
    fast_div_init((uint32_t)d->w_out, &p.wo_mul, &p.wo_shift);
    fast_div_init((uint32_t)d->h_out, &p.ho_mul, &p.ho_shift);
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    if (npix > 0x7fffffffLL) return DC_ERR_SHAPE;
    const int g = lanes_per_pixel(vec_ok ? C / V : C);
    int64_t blocks = divup64(divup64(npix, 32 / g), 8);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    const bool window3 = mode == 0 && vec_ok && mi != nullptr && d->kh == 3 && d->kw == 3 && d->dil_h == 1 && d->dil_w == 1 &&
                         d->pad_top == d->pad_bottom && d->pad_left == d->pad_right;
    if (window3) launch_pdl(k_maxpool3<T, V>, dim3((unsigned)blocks), dim3(256), 0, st, in, prev, mi, out, mo, p, g);
    else if (vec_ok) launch_pdl(k_pool<T, V>, dim3((unsigned)blocks), dim3(256), 0, st, in, prev, mi, out, mo, p, mode, g);
    else launch_pdl(k_pool<T, 1>, dim3((unsigned)blocks), dim3(256), 0, st, in, prev, mi, out, mo, p, mode, g);
    return check_launch();
}

}  // namespace dc

using namespace dc;

extern "C" int dc_pool(const dc_conv_desc* desc, const void* in, void* prev_in, const int32_t* mask_in, void* out,
                       int32_t* mask_out, int32_t pooling_mode, int32_t update_prev, void* stream) {
    if (desc == nullptr || in == nullptr || out == nullptr) return DC_ERR_NULL_POINTER;
    if (pooling_mode != 0 && pooling_mode != 1) return DC_ERR_UNSUPPORTED;
    if (pooling_mode == 0 && prev_in == nullptr) return DC_ERR_NULL_POINTER;
    if (desc->n < 0 || desc->h_in <= 0 || desc->w_in <= 0 || desc->c_in <= 0 || desc->h_out <= 0 || desc->w_out <= 0 ||
        desc->kh <= 0 || desc->kw <= 0 || desc->stride_h <= 0 || desc->stride_w <= 0 || desc->dil_h <= 0 || desc->dil_w <= 0 ||
        desc->c_out != desc->c_in)
        return DC_ERR_SHAPE;
    if (desc->n == 0) return DC_OK;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    if (desc->dtype == DC_F32) rc = pool_t<float>(desc, (const float*)in, (float*)prev_in, mask_in, (float*)out, mask_out, pooling_mode, st);
    else if (desc->dtype == DC_F16) rc = pool_t<__half>(desc, (const __half*)in, (__half*)prev_in, mask_in, (__half*)out, mask_out, pooling_mode, st);
    else return DC_ERR_DTYPE;
    if (rc != DC_OK) return rc;
    if (pooling_mode == 0 && update_prev && mask_in != nullptr)
        rc = dc_add_to_dense(in, prev_in, mask_in, (int64_t)desc->n * desc->h_in * desc->w_in, desc->c_in, desc->dtype, stream);
    return rc;
}
