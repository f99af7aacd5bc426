// First-layer delta convolution: few input channels (RGB), e.g. 3x3/2 3->32 or 7x7/2 3->64, fp16 or
// fp32, optionally fused with the activation/truncation step.
//
// A warp owns a strip of 32 consecutive output pixels. Phase 1: lane i ORs the in-mask over the
// taps of pixel i (coalesced mask reads, no redundancy) and the warp ballots the active set.
// Phase 2: the active pixels are handed out to aligned lane groups (8 output channels per lane);
// a lane reads the pixel's taps straight from global memory (the input has only a few bytes per
// pixel, neighbours share cache lines) against the filter held in shared memory as fp32.
#include "dc_common.cuh"

namespace dc {

struct StemParams {
    const void* in; const int32_t* mi; const void* w; const void* bias; void* out; int32_t* mo;
    void* prev; void* trunc; float thr; int act; int fused;
    int n, hi, wi, ci, ho, wo, co, kh, kw, sh, sw, pt, pl, dh, dw;
};

template <typename T>
__global__ void __launch_bounds__(256) k_conv_stem(StemParams p) {
    extern __shared__ float s_w[];                               // [kh*kw*ci][co] fp32, then bias [co]
    const T* in = reinterpret_cast<const T*>(p.in);
    T* out = reinterpret_cast<T*>(p.out);
    T* prev = reinterpret_cast<T*>(p.prev);
    T* trunc = reinterpret_cast<T*>(p.trunc);
    grid_dep_launch();
    const int taps = p.kh * p.kw;
    const int kdim = taps * p.ci;
    for (int i = threadIdx.x; i < kdim * p.co; i += 256) s_w[i] = to_f<T>(reinterpret_cast<const T*>(p.w)[i]);
    float* s_b = s_w + kdim * p.co;
    for (int i = threadIdx.x; i < p.co; i += 256) s_b[i] = p.bias ? to_f<T>(reinterpret_cast<const T*>(p.bias)[i]) : 0.f;
    grid_dep_wait();
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int npk = p.co >> 3;                                   // 8 output channels per lane
    int g = 1;
    while (g < npk) g <<= 1;                                     // npk <= 32
    const int lig = lane & (g - 1);
    const int ppw = 32 / g;
    const int64_t npix = (int64_t)p.n * p.ho * p.wo;
    const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * 8;
    for (int64_t base = warp0 * 32; base < npix; base += nwarps * 32) {
        // phase 1: lane = pixel
        const int64_t q = base + lane;
        unsigned long long tapbits = 0ull;                       // taps in bounds and active (taps <= 64)
        int ox = 0, oy = 0;
        int64_t b = 0;
        if (q < npix) {
            ox = (int)(q % p.wo);
            const int64_t t = q / p.wo;
            oy = (int)(t % p.ho);
            b = t / p.ho;
            for (int ky = 0; ky < p.kh; ++ky) {
                const int iy = oy * p.sh - p.pt + ky * p.dh;
                if (iy < 0 || iy >= p.hi) continue;
                for (int kx = 0; kx < p.kw; ++kx) {
                    const int ix = ox * p.sw - p.pl + kx * p.dw;
                    if (ix < 0 || ix >= p.wi) continue;
                    if (p.mi[(b * p.hi + iy) * p.wi + ix] != 0) tapbits |= 1ull << (ky * p.kw + kx);
                }
            }
            if (!p.fused || tapbits == 0ull) p.mo[q] = tapbits != 0ull ? 1 : 0;
        }
        unsigned todo = __ballot_sync(DC_FULL, tapbits != 0ull);
        // phase 2: ppw active pixels per round
        while (todo) {
            // the (lane / g)-th set bit of todo, if any
            unsigned rem = todo;
            int src = -1;
            for (int k = 0; k <= lane / g && rem; ++k) {
                src = __ffs(rem) - 1;
                rem &= rem - 1;
                if (k < lane / g) src = -1;
            }
            // drop the ppw lowest set bits
            for (int k = 0; k < ppw && todo; ++k) todo &= todo - 1;
            const int srcl = src < 0 ? 0 : src;
            const unsigned long long tb = __shfl_sync(DC_FULL, tapbits, srcl);
            const int sox = __shfl_sync(DC_FULL, ox, srcl), soy = __shfl_sync(DC_FULL, oy, srcl);
            const long long sb = __shfl_sync(DC_FULL, (long long)b, srcl);
            const bool mine = src >= 0 && lig < npk;
            const int64_t qq = base + srcl;
            float acc[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = mine ? s_b[lig * 8 + k] : 0.f;
            if (mine) {
                unsigned long long r2 = tb;
                while (r2) {
                    const int tp = __ffsll((long long)r2) - 1;
                    r2 &= r2 - 1;
                    const int iy = soy * p.sh - p.pt + (tp / p.kw) * p.dh, ix = sox * p.sw - p.pl + (tp % p.kw) * p.dw;
                    const T* px = in + ((sb * p.hi + iy) * p.wi + ix) * (int64_t)p.ci;
                    for (int c = 0; c < p.ci; ++c) {
                        const float a = to_f<T>(px[c]);
                        const float* wr = s_w + (tp * p.ci + c) * p.co + lig * 8;
                        const float4 w0 = *reinterpret_cast<const float4*>(wr), w1 = *reinterpret_cast<const float4*>(wr + 4);
                        acc[0] = fmaf(a, w0.x, acc[0]); acc[1] = fmaf(a, w0.y, acc[1]);
                        acc[2] = fmaf(a, w0.z, acc[2]); acc[3] = fmaf(a, w0.w, acc[3]);
                        acc[4] = fmaf(a, w1.x, acc[4]); acc[5] = fmaf(a, w1.y, acc[5]);
                        acc[6] = fmaf(a, w1.z, acc[6]); acc[7] = fmaf(a, w1.w, acc[7]);
                    }
                }
            }
            const int64_t off = qq * p.co + lig * 8;
            if (!p.fused) {
                if (mine) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) out[off + k] = from_f<T>(acc[k]);
                }
                continue;
            }
            float yv[8], rv[8], ev[8];
            bool hit = false;
            if (mine) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float yo = to_f<T>(prev[off + k]);
                    const float rr = rnd<T>(to_f<T>(trunc[off + k]) + rnd<T>(acc[k]));
                    const float u = rnd<T>(yo + rr);
                    const float ee = rnd<T>(act_apply(u, p.act) - act_apply(yo, p.act));
                    yv[k] = u; rv[k] = rr; ev[k] = ee;
                    hit |= fabsf(ee) > p.thr;
                }
            }
            const bool active = group_any(hit, g, lane);
            if (mine) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (active) { prev[off + k] = from_f<T>(yv[k]); out[off + k] = from_f<T>(ev[k]); trunc[off + k] = from_f<T>(0.f); }
                    else trunc[off + k] = from_f<T>(rv[k]);
                }
            }
            if (src >= 0 && lig == 0) p.mo[qq] = active ? 1 : 0;
        }
    }
}

// groups == 1, c_in <= 4, c_out a multiple of 8 up to 256, at most 64 taps, with in- and out-mask.
int conv_stem(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
              int32_t* mo, const dc_epilogue* ep, cudaStream_t st) {
    const bool ok = d->groups == 1 && d->c_in <= 4 && d->c_out % 8 == 0 && d->c_out <= 256 && d->kh * d->kw <= 64 &&
                    mi != nullptr && mo != nullptr && (d->dtype == DC_F16 || d->dtype == DC_F32) &&
                    (ep == nullptr || ep->truncation == DC_TRUNC_MAX);
    if (!ok) return DC_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * ((size_t)d->kh * d->kw * d->c_in * d->c_out + d->c_out);
    if (smem > 96 * 1024) return DC_ERR_UNSUPPORTED;
    if (d->n == 0) return DC_OK;
    StemParams p{};
    p.in = in; p.mi = mi; p.w = filt; p.bias = bias; p.out = out; p.mo = mo;
    p.fused = ep != nullptr;
    p.prev = p.fused ? ep->prev_out : nullptr;
    p.trunc = p.fused ? ep->truncated : nullptr;
    p.act = p.fused ? ep->activation : 0;
    p.n = d->n; p.hi = d->h_in; p.wi = d->w_in; p.ci = d->c_in; p.ho = d->h_out; p.wo = d->w_out; p.co = d->c_out;
    p.kh = d->kh; p.kw = d->kw; p.sh = d->stride_h; p.sw = d->stride_w; p.pt = d->pad_top; p.pl = d->pad_left;
    p.dh = d->dil_h; p.dw = d->dil_w;
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    int64_t blocks = divup64(npix, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (d->dtype == DC_F16) {
        p.thr = p.fused ? host_round_threshold<__half>(ep->threshold) : 0.f;
        static thread_local bool set16 = false;
        if (smem > 48 * 1024 && !set16) { cudaFuncSetAttribute(k_conv_stem<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); set16 = true; }
        return launch_pdl(k_conv_stem<__half>, dim3((unsigned)blocks), dim3(256), smem, st, p);
    } else {
        p.thr = p.fused ? ep->threshold : 0.f;
        static thread_local bool set32 = false;
        if (smem > 48 * 1024 && !set32) { cudaFuncSetAttribute(k_conv_stem<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); set32 = true; }
        return launch_pdl(k_conv_stem<float>, dim3((unsigned)blocks), dim3(256), smem, st, p);
    }
    return check_launch();
}

}  // namespace dc
