// Depthwise 3x3 delta convolution fused with the activation/truncation step (fp16), "warp strip" form.
//
// A warp owns a strip of 32 consecutive output pixels. Phase 1: lane i ORs the in-mask over the nine
// taps of pixel i (each mask word is read once per tap by one lane, coalesced) and the warp ballots the
// active set; strips without an active pixel cost one round of mask loads. Phase 2: the active pixels are
// handed to aligned lane groups (8 channels per lane and step); a lane reads its 16-byte channel packs of
// the active taps straight from global memory (neighbouring output pixels share them through L1/L2),
// multiplies with the filter held in shared memory, accumulates in fp32 and applies the epilogue in
// registers: plain store, or accumulate + activation delta + any-channel truncation against the two
// caches. No staging buffers, so occupancy is bounded by registers only.
#include "dc_common.cuh"

namespace dc {

struct DwStripParams {
    const __half* in; const int32_t* mi; const __half* w; const __half* bias;
    __half* out; int32_t* mo; __half* prev; __half* trunc;
    float thr; int act; int fused;
    int n, hi, wi, c, ho, wo, s, pt, pl;
    int strip;          // output pixels per warp and iteration: a multiple of the pixels a warp processes at once, <= 32
    uint32_t wo_mul, wo_shift, ho_mul, ho_shift;      // fast_div constants for w_out and h_out
};

// One output pixel per aligned lane group: depthwise taps -> fp32 accumulators -> epilogue in registers.
// Must be called by all 32 lanes of a warp (the any-channel decision ballots across the warp).
// `in0` is the element offset of tap (0,0)'s input pixel (it may lie in the padding: only taps whose bit is
// set in `tb` are read). All tap loads of a channel pack are issued before the first is used, so a lane has
// up to eleven 16-byte reads in flight; inactive taps contribute zeros instead of branches.
// kEpi: 0 = plain store, 1 = fused truncation with an activation of act_exact_in_half (packed half only),
// 2 = fused truncation, any activation.
template <int NV, int kEpi>
__device__ __forceinline__ void dw_pixel(const DwStripParams& p, const float* s_w, const float* s_b, bool on, unsigned tb,
                                         int64_t qq, int64_t in0, int lig, int g, int npk, int lane) {
    const int64_t off = qq * p.c;
    Pack<__half, 8> pd[NV], pu[NV], pr[NV];
    const __half2 thr2 = __float2half2_rn(p.thr);
    bool hit = false;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = lig + j * g;
        const bool mine = on && i < npk;
        uint4 v[9];
#pragma unroll
        for (int t9 = 0; t9 < 9; ++t9) {
            v[t9] = make_uint4(0u, 0u, 0u, 0u);
            if (mine && (tb & (1u << t9)))
                v[t9] = __ldg(reinterpret_cast<const uint4*>(p.in + in0 + (int64_t)((t9 / 3) * p.wi + t9 % 3) * p.c) + i);
        }
        if ((kEpi != 0) && mine) {
            pu[j].load(p.prev + off + i * 8);
            pr[j].load(p.trunc + off + i * 8);
        }
        float2 acc[4];                    // fp32 accumulators, two channels per packed FMA (fma.rn.f32x2)
        const int ci = mine ? i * 8 : 0;
        {
            const float4 b0 = *reinterpret_cast<const float4*>(s_b + ci), b1 = *reinterpret_cast<const float4*>(s_b + ci + 4);
            acc[0] = make_float2(b0.x, b0.y); acc[1] = make_float2(b0.z, b0.w); acc[2] = make_float2(b1.x, b1.y); acc[3] = make_float2(b1.z, b1.w);
        }
#pragma unroll
        for (int t9 = 0; t9 < 9; ++t9) {
            const float4 w0 = *reinterpret_cast<const float4*>(s_w + t9 * p.c + ci), w1 = *reinterpret_cast<const float4*>(s_w + t9 * p.c + ci + 4);
            const __half2* h = reinterpret_cast<const __half2*>(&v[t9]);
            acc[0] = __ffma2_rn(__half22float2(h[0]), make_float2(w0.x, w0.y), acc[0]);
            acc[1] = __ffma2_rn(__half22float2(h[1]), make_float2(w0.z, w0.w), acc[1]);
            acc[2] = __ffma2_rn(__half22float2(h[2]), make_float2(w1.x, w1.y), acc[2]);
            acc[3] = __ffma2_rn(__half22float2(h[3]), make_float2(w1.z, w1.w), acc[3]);
        }
        __half2* dh = reinterpret_cast<__half2*>(pd[j].s);
#pragma unroll
        for (int k = 0; k < 4; ++k) dh[k] = __float22half2_rn(acc[k]);
        if ((kEpi == 0)) {
            if (mine) pd[j].store(p.out + off + i * 8);
        } else if (mine) {
            if constexpr (kEpi == 1) hit |= truncate_pack_h2(pd[j], pu[j], pr[j], p.act, thr2);
            else hit |= truncate_pack_f32(pd[j], pu[j], pr[j], p.act, p.thr);
        }
    }
    if ((kEpi == 0)) return;
    const bool active = group_any(hit, g, lane);
    if (!on) return;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = lig + j * g;
        if (i >= npk) continue;
        if (active) {
            Pack<__half, 8> z; z.zero();
            pu[j].store(p.prev + off + i * 8);
            pd[j].store(p.out + off + i * 8);
            z.store(p.trunc + off + i * 8);
        } else {
            pr[j].store(p.trunc + off + i * 8);
        }
    }
    if (lig == 0) p.mo[qq] = active ? 1 : 0;
}

// The filter and the bias as fp32 in shared memory ([9][C] and [C]): converted once per CTA, so that the taps
// cost one conversion (the input) instead of two.
__device__ __forceinline__ void dw_stage_filter(const DwStripParams& p, float* s_w, float* s_b) {
    const int npk = p.c >> 3;
    for (int i = threadIdx.x; i < 10 * npk; i += 256) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (i < 9 * npk) raw = __ldg(reinterpret_cast<const uint4*>(p.w) + i);
        else if (p.bias != nullptr) raw = __ldg(reinterpret_cast<const uint4*>(p.bias) + (i - 9 * npk));
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
        const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
        float* dst = i < 9 * npk ? s_w + i * 8 : s_b + (i - 9 * npk) * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(f0.x, f0.y, f1.x, f1.y);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(f2.x, f2.y, f3.x, f3.y);
    }
}

// List-driven form: persistent warps pull active output pixels from the work list written by
// k_scan_conv_mask, so the active set is spread evenly over the SMs however it clusters in the image.
template <int NV>
__global__ void __launch_bounds__(256) k_dw3x3_list(DwStripParams p, const int32_t* __restrict__ count,
                                                    const uint32_t* __restrict__ list, const uint32_t* __restrict__ taps) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* s_w = reinterpret_cast<float*>(smem);                      // [9][C]
    float* s_b = s_w + 9 * p.c;                                       // [C]
    grid_dep_launch();
    const int npk = p.c >> 3;
    // the filter is constant: stage it while the previous kernel (the mask scan) is still finishing
    dw_stage_filter(p, s_w, s_b);
    grid_dep_wait();
    const int cnt = *count;
    if (cnt == 0) return;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    int g = 1;
    while (g < npk && g < 32) g <<= 1;
    const int lig = lane & (g - 1);
    const int gi = lane / g;
    const int ppw = 32 / g;
    const int warp0 = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * 8;
    const bool exact = act_exact_in_half(p.act);
    for (int r = warp0 * ppw; r < cnt; r += nwarps * ppw) {
        const int idx = r + gi;
        const bool on = idx < cnt;
        const uint32_t q = on ? list[idx] : 0u;
        const unsigned tb = on ? taps[idx] : 0u;
        const uint32_t t = fast_div(q, p.wo_mul, p.wo_shift);
        const int ox = (int)(q - t * (uint32_t)p.wo);
        const uint32_t b = fast_div(t, p.ho_mul, p.ho_shift);
        const int oy = (int)(t - b * (uint32_t)p.ho);
        const int64_t in0 = (((int64_t)b * p.hi + (oy * p.s - p.pt)) * p.wi + (ox * p.s - p.pl)) * p.c;
        if (!p.fused) dw_pixel<NV, 0>(p, s_w, s_b, on, tb, (int64_t)q, in0, lig, g, npk, lane);
        else if (exact) dw_pixel<NV, 1>(p, s_w, s_b, on, tb, (int64_t)q, in0, lig, g, npk, lane);
        else dw_pixel<NV, 2>(p, s_w, s_b, on, tb, (int64_t)q, in0, lig, g, npk, lane);
    }
}

template <int NV, int kEpi>   // channel packs per lane: ceil(C / 8 / lanes-per-pixel)
__global__ void __launch_bounds__(256) k_dw3x3_strip(DwStripParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* s_w = reinterpret_cast<float*>(smem);                      // [9][C]
    float* s_b = s_w + 9 * p.c;                                       // [C]
    grid_dep_launch();
    const int npk = p.c >> 3;
    dw_stage_filter(p, s_w, s_b);
    grid_dep_wait();
    __syncthreads();

    const int lane = threadIdx.x & 31;
    int g = 1;
    while (g < npk && g < 32) g <<= 1;
    const int lig = lane & (g - 1);
    const int gi = lane / g;                                          // lane group inside the warp
    const int ppw = 32 / g;
    const uint32_t npix = (uint32_t)p.n * p.ho * p.wo;
    const uint32_t warp0 = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t nwarps = gridDim.x * 8;
    for (uint32_t base = warp0 * p.strip; base < npix; base += nwarps * p.strip) {
        // ---- phase 1: lane = output pixel ----
        const uint32_t q = base + lane;
        unsigned taps = 0;                                            // bit t: tap t in bounds and active
        int oy = 0, ox = 0, b = 0;
        if (lane < p.strip && q < npix) {
            const uint32_t t = fast_div(q, p.wo_mul, p.wo_shift);
            ox = (int)(q - t * (uint32_t)p.wo);
            b = (int)fast_div(t, p.ho_mul, p.ho_shift);
            oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
            const int y0 = oy * p.s - p.pt, x0 = ox * p.s - p.pl;
            const int32_t* mrow = p.mi + (int64_t)b * p.hi * p.wi;
#pragma unroll
            for (int t9 = 0; t9 < 9; ++t9) {
                const int iy = y0 + t9 / 3, ix = x0 + t9 % 3;
                if (iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi && mrow[iy * p.wi + ix] != 0) taps |= 1u << t9;
            }
            if ((kEpi == 0) || taps == 0) p.mo[q] = taps != 0 ? 1 : 0;
        }
        unsigned todo = __ballot_sync(DC_FULL, taps != 0);
        // ---- phase 2: ppw active pixels per round ----
        while (todo) {
            unsigned rem = todo;
            int src = -1;
            for (int k = 0; k <= gi && rem; ++k) {
                const int bpos = __ffs(rem) - 1;
                rem &= rem - 1;
                if (k == gi) src = bpos;
            }
            for (int k = 0; k < ppw && todo; ++k) todo &= todo - 1;
            const int srcl = src < 0 ? 0 : src;
            const unsigned tb = __shfl_sync(DC_FULL, taps, srcl);
            const int soy = __shfl_sync(DC_FULL, oy, srcl), sox = __shfl_sync(DC_FULL, ox, srcl), sb = __shfl_sync(DC_FULL, b, srcl);
            const int64_t in0 = (((int64_t)sb * p.hi + (soy * p.s - p.pt)) * p.wi + (sox * p.s - p.pl)) * p.c;
            dw_pixel<NV, kEpi>(p, s_w, s_b, src >= 0, tb, (int64_t)base + srcl, in0, lig, g, npk, lane);
        }
    }
}

// Large maps without a work list in global memory: persistent CTAs own the 128-pixel spans blockIdx.x + j * gridDim.x
// (clustered active regions are dealt round-robin to all CTAs). Per round a CTA dilates the mask of kCtaSpans spans
// (thread = output pixel, all mask reads in flight together), compacts the active pixels with their tap bit sets
// into shared memory and lets its eight warps share them, so one active run of pixels is spread over the whole CTA
// instead of being walked by one warp. No scan pass, no counter to reset.
constexpr int kCtaSpans = 4;                  // passes per round: a pass looks at 256 / kCtaSpanPx spans of kCtaSpanPx pixels
constexpr int kCtaSpanPx = 64;
constexpr int kCtaSpanLog2 = 6;
template <int NV, int kEpi>
__global__ void __launch_bounds__(256, 4) k_dw3x3_cta(DwStripParams p, int64_t nspans, int rounds) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* s_w = reinterpret_cast<float*>(smem);                      // [9][C]
    float* s_b = s_w + 9 * p.c;                                       // [C]
    __shared__ uint32_t s_q[kCtaSpans * 256], s_t[kCtaSpans * 256];
    __shared__ int s_cnt;
    grid_dep_launch();
    const int npk = p.c >> 3;
    dw_stage_filter(p, s_w, s_b);
    grid_dep_wait();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int g = 1;
    while (g < npk && g < 32) g <<= 1;
    const int lig = lane & (g - 1);
    const int gi = lane / g;
    const int ppw = 32 / g;
    const uint32_t npix = (uint32_t)p.n * p.ho * p.wo;
    for (int round = 0; round < rounds; ++round) {
        if (threadIdx.x == 0) s_cnt = 0;
        __syncthreads();              // also: the filter is staged, the previous round's list has been consumed
        // ---- phase 1: thread = output pixel of each of the round's spans ----
        unsigned tb4[kCtaSpans];
        uint32_t q4[kCtaSpans];
        bool valid4[kCtaSpans];
#pragma unroll
        for (int j = 0; j < kCtaSpans; ++j) {
            const int64_t sid = (int64_t)blockIdx.x + (int64_t)((round * kCtaSpans + j) * (256 / kCtaSpanPx) + (threadIdx.x >> kCtaSpanLog2)) * gridDim.x;
            const int64_t q64 = sid * kCtaSpanPx + (threadIdx.x & (kCtaSpanPx - 1));
            valid4[j] = sid < nspans && q64 < (int64_t)npix;
            q4[j] = valid4[j] ? (uint32_t)q64 : 0u;
            tb4[j] = 0u;
            if (valid4[j]) {
                const uint32_t t = fast_div(q4[j], p.wo_mul, p.wo_shift);
                const int ox = (int)(q4[j] - t * (uint32_t)p.wo);
                const int b = (int)fast_div(t, p.ho_mul, p.ho_shift);
                const int oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
                const int y0 = oy * p.s - p.pt, x0 = ox * p.s - p.pl;
                const int32_t* mrow = p.mi + (int64_t)b * p.hi * p.wi;
#pragma unroll
                for (int t9 = 0; t9 < 9; ++t9) {
                    const int iy = y0 + t9 / 3, ix = x0 + t9 % 3;
                    if (iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi && mrow[iy * p.wi + ix] != 0) tb4[j] |= 1u << t9;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kCtaSpans; ++j) {
            if (valid4[j] && ((kEpi == 0) || tb4[j] == 0u)) p.mo[q4[j]] = tb4[j] != 0u ? 1 : 0;
            const unsigned bal = __ballot_sync(DC_FULL, tb4[j] != 0u);
            int base = 0;
            if (lane == 0 && bal != 0u) base = atomicAdd(&s_cnt, __popc(bal));
            base = __shfl_sync(DC_FULL, base, 0);
            if (tb4[j] != 0u) {
                const int slot = base + __popc(bal & ((1u << lane) - 1u));
                s_q[slot] = q4[j];
                s_t[slot] = tb4[j];
            }
        }
        __syncthreads();
        const int cnt = s_cnt;
        // ---- phase 2: the CTA's warps share the active pixels ----
        for (int r = warp * ppw; r < cnt; r += 8 * ppw) {
            const int idx = r + gi;
            const bool on = idx < cnt;
            const uint32_t q = on ? s_q[idx] : 0u;
            const unsigned tb = on ? s_t[idx] : 0u;
            const uint32_t t = fast_div(q, p.wo_mul, p.wo_shift);
            const int ox = (int)(q - t * (uint32_t)p.wo);
            const uint32_t b = fast_div(t, p.ho_mul, p.ho_shift);
            const int oy = (int)(t - b * (uint32_t)p.ho);
            const int64_t in0 = (((int64_t)b * p.hi + (oy * p.s - p.pt)) * p.wi + (ox * p.s - p.pl)) * p.c;
            dw_pixel<NV, kEpi>(p, s_w, s_b, on, tb, (int64_t)q, in0, lig, g, npk, lane);
        }
    }
}

// Wide pixels (more than 256 channels): a warp owns one slice of 32 channel packs of one output pixel, the S
// slices of a pixel sit in neighbouring warps of the CTA, and the any-channel decision of the fused epilogue
// goes through shared memory. Compared with one warp walking all slices of a pixel in turn this gives S times
// the warps to hide the read latency with, and a per-warp chain of one round of reads instead of S.
// Persistent CTAs: the filter is staged once per CTA.
template <int kEpi>
__global__ void __launch_bounds__(256) k_dw3x3_sliced(DwStripParams p, int S) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* s_w = reinterpret_cast<float*>(smem);                      // [9][C]
    float* s_b = s_w + 9 * p.c;                                       // [C]
    __shared__ int s_flag[2][8];                                      // [iteration parity][warp]: slice passed the threshold
    grid_dep_launch();
    const int npk = p.c >> 3;
    dw_stage_filter(p, s_w, s_b);
    grid_dep_wait();
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ppi = 8 / S;                                            // pixels per CTA and iteration
    const int my_px = warp / S, my_slice = warp - my_px * S;
    const bool worker = warp < ppi * S;
    const int i = my_slice * 32 + lane;                               // this lane's channel pack
    const __half2 thr2 = __float2half2_rn(p.thr);
    const uint32_t npix = (uint32_t)p.n * p.ho * p.wo;
    int par = 0;
    for (uint32_t base = blockIdx.x * (uint32_t)ppi; base < npix; base += gridDim.x * (uint32_t)ppi, par ^= 1) {
        const uint32_t q = base + (uint32_t)my_px;
        const bool on = worker && q < npix;
        // the pixel's active taps: lane t < 9 looks at tap t
        const uint32_t t = fast_div(on ? q : 0u, p.wo_mul, p.wo_shift);
        const int ox = (int)((on ? q : 0u) - t * (uint32_t)p.wo);
        const int b = (int)fast_div(t, p.ho_mul, p.ho_shift);
        const int oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
        const int y0 = oy * p.s - p.pt, x0 = ox * p.s - p.pl;
        bool tap_on = false;
        if (on && lane < 9) {
            const int iy = y0 + lane / 3, ix = x0 + lane % 3;
            tap_on = iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi && p.mi[((int64_t)b * p.hi + iy) * p.wi + ix] != 0;
        }
        const unsigned tb = __ballot_sync(DC_FULL, tap_on) & 0x1ffu;
        if (on && my_slice == 0 && lane == 0 && ((kEpi == 0) || tb == 0u)) p.mo[q] = tb != 0u ? 1 : 0;
        const bool mine = on && tb != 0u && i < npk;
        const int64_t in0 = (((int64_t)b * p.hi + y0) * p.wi + x0) * p.c;
        const int64_t off = (int64_t)q * p.c + i * 8;
        uint4 v[9];
#pragma unroll
        for (int t9 = 0; t9 < 9; ++t9) {
            v[t9] = make_uint4(0u, 0u, 0u, 0u);
            if (mine && (tb & (1u << t9)))
                v[t9] = __ldg(reinterpret_cast<const uint4*>(p.in + in0 + (int64_t)((t9 / 3) * p.wi + t9 % 3) * p.c) + i);
        }
        Pack<__half, 8> pd, pu, pr;
        if ((kEpi != 0) && mine) {
            pu.load(p.prev + off);
            pr.load(p.trunc + off);
        }
        float2 acc[4];                    // fp32 accumulators, two channels per packed FMA (fma.rn.f32x2)
        const int ci = mine ? i * 8 : 0;
        {
            const float4 b0 = *reinterpret_cast<const float4*>(s_b + ci), b1 = *reinterpret_cast<const float4*>(s_b + ci + 4);
            acc[0] = make_float2(b0.x, b0.y); acc[1] = make_float2(b0.z, b0.w); acc[2] = make_float2(b1.x, b1.y); acc[3] = make_float2(b1.z, b1.w);
        }
#pragma unroll
        for (int t9 = 0; t9 < 9; ++t9) {
            const float4 w0 = *reinterpret_cast<const float4*>(s_w + t9 * p.c + ci), w1 = *reinterpret_cast<const float4*>(s_w + t9 * p.c + ci + 4);
            const __half2* h = reinterpret_cast<const __half2*>(&v[t9]);
            acc[0] = __ffma2_rn(__half22float2(h[0]), make_float2(w0.x, w0.y), acc[0]);
            acc[1] = __ffma2_rn(__half22float2(h[1]), make_float2(w0.z, w0.w), acc[1]);
            acc[2] = __ffma2_rn(__half22float2(h[2]), make_float2(w1.x, w1.y), acc[2]);
            acc[3] = __ffma2_rn(__half22float2(h[3]), make_float2(w1.z, w1.w), acc[3]);
        }
        __half2* dh = reinterpret_cast<__half2*>(pd.s);
#pragma unroll
        for (int k = 0; k < 4; ++k) dh[k] = __float22half2_rn(acc[k]);
        if ((kEpi == 0)) {                                               // uniform over the CTA
            if (mine) pd.store(p.out + off);
            continue;
        }
        bool hit = false;
        if (mine) {
            if constexpr (kEpi == 1) hit = truncate_pack_h2(pd, pu, pr, p.act, thr2);
            else hit = truncate_pack_f32(pd, pu, pr, p.act, p.thr);
        }
        const bool whit = __any_sync(DC_FULL, hit);
        if (lane == 0) s_flag[par][warp] = whit ? 1 : 0;
        __syncthreads();          // the flags of iteration parity `par` are next written two iterations (two barriers) later
        bool active = false;
        if (worker)
            for (int sl = 0; sl < S; ++sl) active |= s_flag[par][my_px * S + sl] != 0;
        if (mine) {
            if (active) {
                Pack<__half, 8> z; z.zero();
                pu.store(p.prev + off);
                pd.store(p.out + off);
                z.store(p.trunc + off);
            } else {
                pr.store(p.trunc + off);
            }
        }
        if (on && tb != 0u && my_slice == 0 && lane == 0) p.mo[q] = active ? 1 : 0;
    }
}

// Depthwise 3x3 (stride 1 or 2, dilation 1) in fp16 with in- and out-mask; DC_ERR_UNSUPPORTED tells the
// caller to use the generic kernels.
int scan_conv_mask(const dc_conv_desc* d, const int32_t* mi, int32_t* mo, void* ws, size_t ws_bytes, int defer_active, cudaStream_t st);

int dwconv3x3_strip(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                    int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st) {
    const bool ok = d->dtype == DC_F16 && d->kh == 3 && d->kw == 3 && d->dil_h == 1 && d->dil_w == 1 &&
                    d->stride_h == d->stride_w && (d->stride_h == 1 || d->stride_h == 2) && d->groups == d->c_in &&
                    d->c_in == d->c_out && d->c_in % 8 == 0 && d->c_in <= 1024 && mi != nullptr && mo != nullptr &&
                    aligned16(in) && aligned16(out) && aligned16(filt) && (bias == nullptr || aligned16(bias)) &&
                    (ep == nullptr || (ep->truncation == DC_TRUNC_MAX && aligned16(ep->prev_out) && aligned16(ep->truncated)));
    if (!ok) return DC_ERR_UNSUPPORTED;
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    if (npix == 0) return DC_OK;
    if (npix > 0x7fffffffLL || (int64_t)d->n * d->h_in * d->w_in > 0x7fffffffLL) return DC_ERR_SHAPE;
    DwStripParams p{};
    p.in = (const __half*)in; p.mi = mi; p.w = (const __half*)filt; p.bias = (const __half*)bias;
    p.out = (__half*)out; p.mo = mo;
    p.fused = ep != nullptr;
    p.prev = p.fused ? (__half*)ep->prev_out : nullptr;
    p.trunc = p.fused ? (__half*)ep->truncated : nullptr;
    p.thr = p.fused ? host_round_threshold<__half>(ep->threshold) : 0.f;
    p.act = p.fused ? ep->activation : 0;
    p.n = d->n; p.hi = d->h_in; p.wi = d->w_in; p.c = d->c_in; p.ho = d->h_out; p.wo = d->w_out; p.s = d->stride_h;
    p.pt = d->pad_top; p.pl = d->pad_left;
    fast_div_init((uint32_t)p.wo, &p.wo_mul, &p.wo_shift);
    fast_div_init((uint32_t)p.ho, &p.ho_mul, &p.ho_shift);
    const int npk = p.c / 8;
    const int nv = divup(npk, 32);
    const int epi = !p.fused ? 0 : (p.act >= DC_ACT_NONE && p.act <= DC_ACT_RELU6) ? 1 : 2;     // epilogue kind of the kernels
    const size_t smem = (size_t)10 * p.c * 4;         // filter and bias as fp32
    // large map, narrow pixels: CTA-level compaction, no scan pass. With scratch memory and so many pixels that a CTA
    // would need several rounds, the work list below spreads the active pixels better.
    const int64_t nspans = divup64(npix, kCtaSpanPx);
    int64_t grid_c = (int64_t)sm_count() * 4;
    if (grid_c > nspans) grid_c = nspans;
    const int rounds = (int)divup64(divup64(nspans, grid_c), kCtaSpans * (256 / kCtaSpanPx));
    if (nv == 1 && npix >= 40000 && (ws == nullptr || rounds <= 1)) {
        return epi == 0 ? launch_pdl(k_dw3x3_cta<1, 0>, dim3((unsigned)grid_c), dim3(256), smem, st, p, nspans, rounds)
             : epi == 1 ? launch_pdl(k_dw3x3_cta<1, 1>, dim3((unsigned)grid_c), dim3(256), smem, st, p, nspans, rounds)
                        : launch_pdl(k_dw3x3_cta<1, 2>, dim3((unsigned)grid_c), dim3(256), smem, st, p, nspans, rounds);
    }
    // the work list costs two extra launches; it pays on large maps where the active pixels cluster
    if (ws != nullptr && npix >= 40000) {             // work-list form: one scan pass, then persistent warps over the active pixels
        int rc = scan_conv_mask(d, mi, mo, ws, ws_bytes, p.fused, st);
        if (rc != DC_OK) return rc;
        const int32_t* count = reinterpret_cast<const int32_t*>(ws);
        const uint32_t* list = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(ws) + 16);
        const uint32_t* taps = list + npix;
        const size_t smem_l = smem;
        const unsigned grid = (unsigned)sm_count() * (nv >= 3 ? 2 : 4);
        switch (nv) {
            case 1: launch_pdl(k_dw3x3_list<1>, dim3(grid), dim3(256), smem_l, st, p, count, list, taps); break;
            case 2: launch_pdl(k_dw3x3_list<2>, dim3(grid), dim3(256), smem_l, st, p, count, list, taps); break;
            case 3: launch_pdl(k_dw3x3_list<3>, dim3(grid), dim3(256), smem_l, st, p, count, list, taps); break;
            default: launch_pdl(k_dw3x3_list<4>, dim3(grid), dim3(256), smem_l, st, p, count, list, taps); break;
        }
        return check_launch();
    }
    if (nv >= 2) {                                    // wide pixels: one warp per slice of 32 channel packs, persistent CTAs
        const int S = nv;                             // c_in <= 1024: at most 4 slices
        const int ppi = 8 / S;
        int64_t blocks_s = divup64(npix, ppi);
        const int64_t cap_s = (int64_t)sm_count() * 4;
        if (blocks_s > cap_s) blocks_s = cap_s;
        return epi == 0 ? launch_pdl(k_dw3x3_sliced<0>, dim3((unsigned)blocks_s), dim3(256), smem, st, p, S)
             : epi == 1 ? launch_pdl(k_dw3x3_sliced<1>, dim3((unsigned)blocks_s), dim3(256), smem, st, p, S)
                        : launch_pdl(k_dw3x3_sliced<2>, dim3((unsigned)blocks_s), dim3(256), smem, st, p, S);
    }
    // wide pixels keep a whole warp busy, so give every warp few of them; narrow pixels share a warp
    int g = 1;
    while (g < npk && g < 32) g <<= 1;
    const int ppw = 32 / g;
    int strip = 32;
    while (strip > ppw && divup64(npix, strip) < (int64_t)sm_count() * 64) strip >>= 1;
    p.strip = strip;
    int64_t blocks = divup64(divup64(npix, strip), 8);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    // wider pixels took the sliced kernel above: one channel pack per lane here
    if (epi == 0) launch_pdl(k_dw3x3_strip<1, 0>, dim3((unsigned)blocks), dim3(256), smem, st, p);
    else if (epi == 1) launch_pdl(k_dw3x3_strip<1, 1>, dim3((unsigned)blocks), dim3(256), smem, st, p);
    else launch_pdl(k_dw3x3_strip<1, 2>, dim3((unsigned)blocks), dim3(256), smem, st, p);
    return check_launch();
}

}  // namespace dc
