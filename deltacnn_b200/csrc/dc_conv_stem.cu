// First-layer delta convolution: few input channels (RGB), e.g. 3x3/2 3->32 or 7x7/2 3->64, fp16 or
// fp32, optionally fused with the activation/truncation step.
//
// A warp owns a strip of 32 consecutive output pixels. Phase 1: lane i ORs the in-mask over the
// taps of pixel i (coalesced mask reads, no redundancy) and the warp ballots the active set.
// Phase 2: the active pixels are handed out to aligned lane groups (8 output channels per lane);
// a lane reads the pixel's taps straight from global memory (the input has only a few bytes per
// pixel, neighbours share cache lines) against the filter held in shared memory as fp32.
#include <type_traits>
#include "dc_common.cuh"

namespace dc {

struct StemParams {
    const void* in; const int32_t* mi; const void* w; const void* bias; void* out; int32_t* mo;
    void* prev; void* trunc; float thr; int act; int fused;
    int n, hi, wi, ci, ho, wo, co, kh, kw, sh, sw, pt, pl, dh, dw;
    uint32_t wo_mul, wo_shift, ho_mul, ho_shift;                 // fast_div constants for w_out and h_out
};

// One output pixel per aligned lane group (8 output channels per lane): taps x input channels against the fp32
// filter in shared memory, epilogue in registers. Called by all 32 lanes of a warp.
// kEpi: 0 = plain store, 1 = fused truncation in packed half (fp16, activation of act_exact_in_half), 2 = fused, generic.
template <typename T, int kEpi>
__device__ __forceinline__ void stem_pixel(const StemParams& p, const float* s_w, const float* s_b, const int* s_toff, bool on,
                                           unsigned long long tb, int sin0, int64_t qq, int lig, int g, int npk, int lane,
                                           __half2 thr2) {
    constexpr int W = VecTraits<T>::kVec, NP = 8 / W;            // a lane's 8 output channels as NP 16-byte packs
    const T* in = reinterpret_cast<const T*>(p.in);
    T* out = reinterpret_cast<T*>(p.out);
    T* prev = reinterpret_cast<T*>(p.prev);
    T* trunc = reinterpret_cast<T*>(p.trunc);
    const int taps = p.kh * p.kw;
    const bool mine = on && lig < npk;
    const int cl = mine ? lig * 8 : 0;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = s_b[cl + k];
    // uniform loop over the taps: the reads of a few taps are issued together, inactive taps add zeros
#pragma unroll 3
    for (int tp = 0; tp < taps; ++tp) {
        const bool a = mine && ((tb >> tp) & 1ull) != 0ull;
        const T* px = in + (int64_t)(sin0 + s_toff[tp]) * p.ci;
        float x[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) x[c] = (a && c < p.ci) ? to_f<T>(px[c]) : 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (c < p.ci) {
                const float* wr = s_w + (tp * p.ci + c) * p.co + cl;
                const float4 w0 = *reinterpret_cast<const float4*>(wr), w1 = *reinterpret_cast<const float4*>(wr + 4);
                acc[0] = fmaf(x[c], w0.x, acc[0]); acc[1] = fmaf(x[c], w0.y, acc[1]);
                acc[2] = fmaf(x[c], w0.z, acc[2]); acc[3] = fmaf(x[c], w0.w, acc[3]);
                acc[4] = fmaf(x[c], w1.x, acc[4]); acc[5] = fmaf(x[c], w1.y, acc[5]);
                acc[6] = fmaf(x[c], w1.z, acc[6]); acc[7] = fmaf(x[c], w1.w, acc[7]);
            }
        }
    }
    const int64_t off = qq * p.co + cl;
    Pack<T, W> d[NP], y[NP], r[NP];
#pragma unroll
    for (int h = 0; h < NP; ++h)
#pragma unroll
        for (int k = 0; k < W; ++k) d[h].set(k, acc[h * W + k]);
    if (kEpi == 0) {
        if (mine) {
#pragma unroll
            for (int h = 0; h < NP; ++h) d[h].store(out + off + h * W);
        }
        return;
    }
    bool hit = false;
    if (mine) {
#pragma unroll
        for (int h = 0; h < NP; ++h) {
            y[h].load(prev + off + h * W);
            r[h].load(trunc + off + h * W);
        }
#pragma unroll
        for (int h = 0; h < NP; ++h) {
            if constexpr (sizeof(T) == 2 && kEpi == 1) hit |= truncate_pack_h2(d[h], y[h], r[h], p.act, thr2);
            else hit |= truncate_pack_f32(d[h], y[h], r[h], p.act, p.thr);
        }
    }
    const bool active = group_any(hit, g, lane);
    if (mine) {
#pragma unroll
        for (int h = 0; h < NP; ++h) {
            if (active) {
                Pack<T, W> z; z.zero();
                y[h].store(prev + off + h * W);
                d[h].store(out + off + h * W);
                z.store(trunc + off + h * W);
            } else {
                r[h].store(trunc + off + h * W);
            }
        }
    }
    if (on && lig == 0) p.mo[qq] = active ? 1 : 0;
}

// Filter [kh*kw*ci][co] and bias [co] as fp32 plus the input-pixel offset of every tap, in shared memory.
template <typename T>
__device__ __forceinline__ void stem_stage_filter(const StemParams& p, float* s_w, float** s_b_out, int** s_toff_out) {
    const int taps = p.kh * p.kw;
    const int kdim = taps * p.ci;
    for (int i = threadIdx.x; i < kdim * p.co; i += 256) s_w[i] = to_f<T>(reinterpret_cast<const T*>(p.w)[i]);
    float* s_b = s_w + kdim * p.co;
    for (int i = threadIdx.x; i < p.co; i += 256) s_b[i] = p.bias ? to_f<T>(reinterpret_cast<const T*>(p.bias)[i]) : 0.f;
    int* s_toff = reinterpret_cast<int*>(s_b + p.co);
    for (int i = threadIdx.x; i < taps; i += 256) s_toff[i] = (i / p.kw) * p.dh * p.wi + (i % p.kw) * p.dw;
    *s_b_out = s_b;
    *s_toff_out = s_toff;
}

// Large maps without a work list in global memory: persistent CTAs own the 64-pixel spans blockIdx.x + j * gridDim.x,
// dilate the mask of kStemSpans spans per round (thread = output pixel), compact the active pixels with their tap
// bit sets into shared memory and let the eight warps share them. No scan pass, no counter to reset.
constexpr int kStemSpans = 2;                 // passes per round: a pass looks at four spans of 64 pixels
template <typename T, int kEpi>
__global__ void __launch_bounds__(256) k_conv_stem_cta(StemParams p, int64_t nspans, int rounds) {
    extern __shared__ float s_w[];
    __shared__ uint32_t s_q[kStemSpans * 256];
    __shared__ unsigned long long s_t[kStemSpans * 256];
    __shared__ int s_cnt;
    grid_dep_launch();
    float* s_b;
    int* s_toff;
    stem_stage_filter<T>(p, s_w, &s_b, &s_toff);
    grid_dep_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int npk = p.co >> 3;
    int g = 1;
    while (g < npk) g <<= 1;
    const int lig = lane & (g - 1), gi = lane / g;
    const int ppw = 32 / g;
    const __half2 thr2 = __float2half2_rn(p.thr);
    const uint32_t npix = (uint32_t)p.n * p.ho * p.wo;
    auto in0_of = [&](uint32_t q) {
        const uint32_t t = fast_div(q, p.wo_mul, p.wo_shift);
        const int ox = (int)(q - t * (uint32_t)p.wo);
        const int b = (int)fast_div(t, p.ho_mul, p.ho_shift);
        const int oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
        return (b * p.hi + oy * p.sh - p.pt) * p.wi + ox * p.sw - p.pl;
    };
    for (int round = 0; round < rounds; ++round) {
        if (threadIdx.x == 0) s_cnt = 0;
        __syncthreads();              // also: the filter is staged, the previous round's list has been consumed
#pragma unroll
        for (int j = 0; j < kStemSpans; ++j) {
            const int64_t sid = (int64_t)blockIdx.x + (int64_t)((round * kStemSpans + j) * 4 + (threadIdx.x >> 6)) * gridDim.x;
            const int64_t q64 = sid * 64 + (threadIdx.x & 63);
            const bool valid = sid < nspans && q64 < (int64_t)npix;
            const uint32_t q = valid ? (uint32_t)q64 : 0u;
            unsigned long long tapbits = 0ull;
            if (valid) {
                const uint32_t t = fast_div(q, p.wo_mul, p.wo_shift);
                const int ox = (int)(q - t * (uint32_t)p.wo);
                const int b = (int)fast_div(t, p.ho_mul, p.ho_shift);
                const int oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
                const int y0 = oy * p.sh - p.pt, x0 = ox * p.sw - p.pl;
                const int in0 = (b * p.hi + y0) * p.wi + x0;
                for (int ky = 0; ky < p.kh; ++ky) {
                    const int iy = y0 + ky * p.dh;
                    if (iy < 0 || iy >= p.hi) continue;
                    for (int kx = 0; kx < p.kw; ++kx) {
                        const int ix = x0 + kx * p.dw;
                        if (ix < 0 || ix >= p.wi) continue;
                        if (p.mi[in0 + ky * p.dh * p.wi + kx * p.dw] != 0) tapbits |= 1ull << (ky * p.kw + kx);
                    }
                }
                if (kEpi == 0 || tapbits == 0ull) p.mo[q] = tapbits != 0ull ? 1 : 0;
            }
            const unsigned bal = __ballot_sync(DC_FULL, tapbits != 0ull);
            int base = 0;
            if (lane == 0 && bal != 0u) base = atomicAdd(&s_cnt, __popc(bal));
            base = __shfl_sync(DC_FULL, base, 0);
            if (tapbits != 0ull) {
                const int slot = base + __popc(bal & ((1u << lane) - 1u));
                s_q[slot] = q;
                s_t[slot] = tapbits;
            }
        }
        __syncthreads();
        const int cnt = s_cnt;
        for (int r = warp * ppw; r < cnt; r += 8 * ppw) {
            const int idx = r + gi;
            const bool on = idx < cnt;
            const uint32_t q = on ? s_q[idx] : 0u;
            const unsigned long long tb = on ? s_t[idx] : 0ull;
            stem_pixel<T, kEpi>(p, s_w, s_b, s_toff, on, tb, in0_of(q), (int64_t)q, lig, g, npk, lane, thr2);
        }
    }
}

template <typename T, int kEpi>
__global__ void __launch_bounds__(256) k_conv_stem(StemParams p) {
    extern __shared__ float s_w[];                               // [kh*kw*ci][co] fp32, bias [co], tap offsets [kh*kw]
    grid_dep_launch();
    float* s_b;
    int* s_toff;
    stem_stage_filter<T>(p, s_w, &s_b, &s_toff);
    grid_dep_wait();
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int npk = p.co >> 3;                                   // 8 output channels per lane
    int g = 1;
    while (g < npk) g <<= 1;                                     // npk <= 32
    const int lig = lane & (g - 1), gi = lane / g;
    const int ppw = 32 / g;
    const __half2 thr2 = __float2half2_rn(p.thr);
    const uint32_t npix = (uint32_t)p.n * p.ho * p.wo;
    const uint32_t warp0 = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t nwarps = gridDim.x * 8;
    for (uint32_t base = warp0 * 32u; base < npix; base += nwarps * 32u) {
        // phase 1: lane = pixel
        const uint32_t q = base + lane;
        unsigned long long tapbits = 0ull;                       // taps in bounds and active (taps <= 64)
        int in0 = 0;                                             // input pixel of tap 0 (may lie in the padding)
        if (q < npix) {
            const uint32_t t = fast_div(q, p.wo_mul, p.wo_shift);
            const int ox = (int)(q - t * (uint32_t)p.wo);
            const int b = (int)fast_div(t, p.ho_mul, p.ho_shift);
            const int oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
            const int y0 = oy * p.sh - p.pt, x0 = ox * p.sw - p.pl;
            in0 = (b * p.hi + y0) * p.wi + x0;
            for (int ky = 0; ky < p.kh; ++ky) {
                const int iy = y0 + ky * p.dh;
                if (iy < 0 || iy >= p.hi) continue;
                for (int kx = 0; kx < p.kw; ++kx) {
                    const int ix = x0 + kx * p.dw;
                    if (ix < 0 || ix >= p.wi) continue;
                    if (p.mi[in0 + ky * p.dh * p.wi + kx * p.dw] != 0) tapbits |= 1ull << (ky * p.kw + kx);
                }
            }
            if (kEpi == 0 || tapbits == 0ull) p.mo[q] = tapbits != 0ull ? 1 : 0;
        }
        unsigned todo = __ballot_sync(DC_FULL, tapbits != 0ull);
        // phase 2: ppw active pixels per round
        while (todo) {
            // the gi-th set bit of todo, if any
            unsigned rem = todo;
            int src = -1;
            for (int k = 0; k <= gi && rem; ++k) {
                const int bpos = __ffs(rem) - 1;
                rem &= rem - 1;
                if (k == gi) src = bpos;
            }
            // drop the ppw lowest set bits
            for (int k = 0; k < ppw && todo; ++k) todo &= todo - 1;
            const int srcl = src < 0 ? 0 : src;
            const unsigned long long tb = __shfl_sync(DC_FULL, tapbits, srcl);
            const int sin0 = __shfl_sync(DC_FULL, in0, srcl);
            stem_pixel<T, kEpi>(p, s_w, s_b, s_toff, src >= 0, tb, sin0, (int64_t)base + srcl, lig, g, npk, lane, thr2);
        }
    }
}

// groups == 1, c_in <= 4, c_out a multiple of 8 up to 256, at most 64 taps, with in- and out-mask.
int conv_stem(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
              int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st) {
    const bool ok = d->groups == 1 && d->c_in <= 4 && d->c_out % 8 == 0 && d->c_out <= 256 && d->kh * d->kw <= 64 &&
                    mi != nullptr && mo != nullptr && (d->dtype == DC_F16 || d->dtype == DC_F32) && aligned16(out) &&
                    (ep == nullptr || (ep->truncation == DC_TRUNC_MAX && aligned16(ep->prev_out) && aligned16(ep->truncated)));
    if (!ok) return DC_ERR_UNSUPPORTED;
    const size_t smem = sizeof(float) * ((size_t)d->kh * d->kw * d->c_in * d->c_out + d->c_out + (size_t)d->kh * d->kw);
    if (smem > 96 * 1024) return DC_ERR_UNSUPPORTED;
    if (d->n == 0) return DC_OK;
    if ((int64_t)d->n * d->h_out * d->w_out > 0x7fffffffLL || (int64_t)d->n * d->h_in * d->w_in > 0x7fffffffLL) return DC_ERR_SHAPE;
    StemParams p{};
    p.in = in; p.mi = mi; p.w = filt; p.bias = bias; p.out = out; p.mo = mo;
    p.fused = ep != nullptr;
    p.prev = p.fused ? ep->prev_out : nullptr;
    p.trunc = p.fused ? ep->truncated : nullptr;
    p.act = p.fused ? ep->activation : 0;
    p.n = d->n; p.hi = d->h_in; p.wi = d->w_in; p.ci = d->c_in; p.ho = d->h_out; p.wo = d->w_out; p.co = d->c_out;
    p.kh = d->kh; p.kw = d->kw; p.sh = d->stride_h; p.sw = d->stride_w; p.pt = d->pad_top; p.pl = d->pad_left;
    p.dh = d->dil_h; p.dw = d->dil_w;
    fast_div_init((uint32_t)p.wo, &p.wo_mul, &p.wo_shift);
    fast_div_init((uint32_t)p.ho, &p.ho_mul, &p.ho_shift);
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    int64_t blocks = divup64(npix, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    p.thr = !p.fused ? 0.f : d->dtype == DC_F16 ? host_round_threshold<__half>(ep->threshold) : ep->threshold;
    // epilogue kind of the kernels: plain store, fused truncation in packed half, fused truncation in fp32
    const int epi = !p.fused ? 0 : (d->dtype == DC_F16 && p.act >= DC_ACT_NONE && p.act <= DC_ACT_RELU6) ? 1 : 2;
#define DC_STEM_KERNELS(X) X(__half, 0) X(__half, 1) X(__half, 2) X(float, 0) X(float, 2)
    static PerDeviceOnce attr_once;
    bool* attr_set = attr_once.slot();
    if (attr_set == nullptr) return DC_ERR_LAUNCH;
    if (smem > 48 * 1024 && !*attr_set) {
#define DC_STEM_ATTR(T, E)                                                                                  \
        cudaFuncSetAttribute(k_conv_stem<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);     \
        cudaFuncSetAttribute(k_conv_stem_cta<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        DC_STEM_KERNELS(DC_STEM_ATTR)
#undef DC_STEM_ATTR
        *attr_set = true;
    }
    // large maps: persistent CTAs compact the active pixels of their spans themselves (no scan pass, no scratch)
    (void)ws; (void)ws_bytes;
    if (npix >= 40000) {
        const int64_t nspans = divup64(npix, 64);
        int64_t grid_c = (int64_t)sm_count() * (d->dtype == DC_F16 ? 4 : 3);    // resident CTAs (registers)
        if (grid_c > nspans) grid_c = nspans;
        const int rounds = (int)divup64(divup64(nspans, grid_c), kStemSpans * 4);
#define DC_STEM_CTA(T, E) \
        if (std::is_same<T, __half>::value == (d->dtype == DC_F16) && epi == E) \
            return launch_pdl(k_conv_stem_cta<T, E>, dim3((unsigned)grid_c), dim3(256), smem, st, p, nspans, rounds);
        DC_STEM_KERNELS(DC_STEM_CTA)
#undef DC_STEM_CTA
        return DC_ERR_UNSUPPORTED;
    }
#define DC_STEM_STRIP(T, E) \
    if (std::is_same<T, __half>::value == (d->dtype == DC_F16) && epi == E) \
        return launch_pdl(k_conv_stem<T, E>, dim3((unsigned)blocks), dim3(256), smem, st, p);
    DC_STEM_KERNELS(DC_STEM_STRIP)
#undef DC_STEM_STRIP
#undef DC_STEM_KERNELS
    return DC_ERR_UNSUPPORTED;
}

}  // namespace dc
