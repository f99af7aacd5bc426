// First-layer delta convolution (RGB stems: 3x3/2 3->32, 7x7/2 3->64) on the tensor core, fp16.
//
// With three input channels the contraction length is kh*kw*3 (27 or 147): too ragged for 16-byte gathers, but
// still a GEMM. Persistent CTAs own strided 64-pixel spans of the output, dilate the in-mask with a thread per
// output pixel and compact the active pixels (with the bit set of their active taps) into shared memory. A tile
// of 128 active pixels is then built by an im2col into the 128-byte-swizzled K-major stage (two threads per row,
// 16-bit reads straight from the frame, zeros for inactive / out-of-bounds taps and for the K padding), multiplied
// against the filter (re-tiled into the same layout by the CTA itself, once) with tcgen05.mma into tensor memory,
// and finished by the same epilogue as the other tensor-core kernels: tcgen05.ld -> fp16 staging tile -> coalesced
// rows, plain store or fused accumulate + activation delta + any-channel truncation.
// Every wait on the mbarrier is bounded; a wait that gives up sets the sticky error code read by dc_umma_error.
#include "dc_umma.cuh"

namespace dc {

__device__ int g_stem_umma_error = 0;        // sticky: 5 = the MMA-complete barrier was not reached in time

constexpr int kSuThreads = 256;
constexpr int kSuSpanPx = 64;                 // pixels per span (the unit dealt round-robin to the CTAs)
constexpr int kSuSpans = 8;                   // spans compacted together per round (two passes of 256 threads)
constexpr int kSuMaxK = 192;                  // three K blocks

struct StemUParams {
    const __half* in; const int32_t* mi; const __half* w; const __half* bias;
    __half* out; int32_t* mo; __half* prev; __half* trunc;
    float thr; int act;
    int n, hi, wi, ci, ho, wo, co, kh, kw, sh, sw, pt, pl, dh, dw;
    int kdim, nkb, last_ksteps, kcover;      // kh*kw*ci, K blocks of 64, MMAs in the last block, K values filled (multiple of 16)
    int tmem_cols;
    uint32_t wo_mul, wo_shift, ho_mul, ho_shift;
    int64_t nspans;
    int rounds;
    uint32_t off_b, off_list, off_misc, stage_pitch;
};

// Bit kx of the result: column x0 + kx * dw of the mask row is inside the image and set (kx < min(kw, W)); the W
// reads are issued together.
template <int W>
__device__ __forceinline__ unsigned mask_row_bits(const int32_t* mrow, int x0, int kw, int dw, int wi) {
    int m[W];
#pragma unroll
    for (int kx = 0; kx < W; ++kx) {
        const int ix = x0 + kx * dw;
        m[kx] = (kx < kw && ix >= 0 && ix < wi) ? mrow[kx * dw] : 0;
    }
    unsigned bits = 0u;
#pragma unroll
    for (int kx = 0; kx < W; ++kx)
        if (m[kx] != 0) bits |= 1u << kx;
    return bits;
}

// kEpi: 0 = plain store, 1 = fused truncation in packed half (activation of act_exact_in_half), 2 = fused, fp32 form.
template <int kEpi>
__global__ void __launch_bounds__(kSuThreads, 3) k_stem_umma(const StemUParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;                                            // [nkb] stages of 128 rows x 128 bytes, swizzled
    uint8_t* sStage = smem;                                        // epilogue staging, aliases the stages
    uint8_t* sB = smem + p.off_b;                                  // [nkb][co rows][128 bytes], swizzled
    uint32_t* s_q = reinterpret_cast<uint32_t*>(smem + p.off_list);                       // [512] active output pixels of a round
    unsigned long long* s_t = reinterpret_cast<unsigned long long*>(s_q + kSuSpans * kSuSpanPx);   // their tap bit sets
    uint32_t* s_ktab = reinterpret_cast<uint32_t*>(s_t + kSuSpans * kSuSpanPx);            // [kSuMaxK] (tap << 24) | element offset
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_misc);                       // [0] all MMAs of a tile done
    uint32_t* s_u32 = reinterpret_cast<uint32_t*>(bars + 1);       // [0] tmem base, [1] ok flag, [2] counter
    float* s_bias = reinterpret_cast<float*>(s_u32 + 4);           // [co]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar_done = smem_u32(bars);

    // ---- set-up from constants only: overlaps the previous kernel's tail ----
    for (int k = tid; k < kSuMaxK; k += kSuThreads) {
        uint32_t e = 0xff000000u;                                   // tap 255: never active (K padding)
        if (k < p.kdim) {
            const int tap = k / p.ci, c = k - tap * p.ci;
            const int ky = tap / p.kw, kx = tap - ky * p.kw;
            e = ((uint32_t)tap << 24) | (uint32_t)((ky * p.dh * p.wi + kx * p.dw) * p.ci + c);
        }
        s_ktab[k] = e;
    }
    // the filter [k][co] (kh, kw, ci major to minor in k) re-tiled K-major with the 128-byte swizzle, zeros beyond kdim
    for (int i = tid; i < p.nkb * kKBlock * p.co; i += kSuThreads) {
        const int n = i % p.co, k = i / p.co;
        const int kb = k >> 6, kc = k & 63;
        const __half v = k < p.kdim ? p.w[(size_t)k * p.co + n] : __float2half(0.f);
        uint8_t* dst = sB + (size_t)kb * p.co * 128 + (n >> 3) * 1024 + (n & 7) * 128 + (((kc >> 3) ^ (n & 7)) << 4) + (kc & 7) * 2;
        *reinterpret_cast<__half*>(dst) = v;
    }
    for (int i = tid; i < p.co; i += kSuThreads) s_bias[i] = p.bias != nullptr ? __half2float(p.bias[i]) : 0.f;
    if (tid == 0) {
        mbar_init(bar_done, 1u);
        fence_barrier_init();
        s_u32[1] = 1;
    }
    if (warp == 0) tmem_alloc(smem_u32(&s_u32[0]), (uint32_t)p.tmem_cols);
    fence_proxy_async();               // the filter tile was written with ordinary stores and is read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_dep_launch();                 // only after the tensor memory is held (a dependent CTA allocates before it waits)
    const uint32_t tmem_base = s_u32[0];
    volatile uint32_t* ok_flag = &s_u32[1];
    grid_dep_wait();

    const uint32_t npix = (uint32_t)p.n * p.ho * p.wo;
    const uint32_t idesc = make_idesc(p.co);
    const int nch = p.co >> 3;                                     // 16-byte packs per output row
    int g = 1;
    while (g < nch && g < 32) g <<= 1;
    const int lig = lane & (g - 1), ppw = 32 / g;
    const __half2 thr2 = __float2half2_rn(p.thr);
    auto in0_of = [&](uint32_t q) {                                // input pixel of tap (0, 0) of output pixel q
        const uint32_t t = fast_div(q, p.wo_mul, p.wo_shift);
        const int ox = (int)(q - t * (uint32_t)p.wo);
        const int b = (int)fast_div(t, p.ho_mul, p.ho_shift);
        const int oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
        return (b * p.hi + oy * p.sh - p.pt) * p.wi + ox * p.sw - p.pl;
    };
    int tile = 0;                      // tiles done by this CTA: the barrier's phase
    bool ok = true;
    for (int round = 0; round < p.rounds && ok; ++round) {
        // ---- the round's active pixels: thread = output pixel of a span, two passes over the round's eight spans ----
        if (tid == 0) s_u32[2] = 0u;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kSuSpans * kSuSpanPx / kSuThreads; ++j) {
            const int v = tid + kSuThreads * j;
            const int64_t sid = (int64_t)blockIdx.x + (int64_t)(round * kSuSpans + (v >> 6)) * gridDim.x;
            const int64_t q64 = sid * kSuSpanPx + (v & (kSuSpanPx - 1));
            const bool valid = sid < p.nspans && q64 < (int64_t)npix;
            const uint32_t q = valid ? (uint32_t)q64 : 0u;
            unsigned long long tapbits = 0ull;
            int ox = 0, oy = 0, b = 0;
            if (valid) {
                const uint32_t t = fast_div(q, p.wo_mul, p.wo_shift);
                ox = (int)(q - t * (uint32_t)p.wo);
                b = (int)fast_div(t, p.ho_mul, p.ho_shift);
                oy = (int)(t - (uint32_t)b * (uint32_t)p.ho);
            }
            const int y0 = oy * p.sh - p.pt, x0 = ox * p.sw - p.pl;
            // The 32 output pixels of a warp are consecutive. When they lie in one image row (and the kernel is not dilated,
            // at most 8 wide, stride <= 2) the warp reads the mask words of the input rows together, coalesced and once
            // (31 * stride + kw <= 96 columns per row: three reads per lane and row instead of kw), turns every row into
            // a bit mask with ballots, and each lane cuts its own kw bits out of it.
            const int oy0 = __shfl_sync(DC_FULL, oy, 0), b0 = __shfl_sync(DC_FULL, b, 0), x00 = __shfl_sync(DC_FULL, x0, 0);
            const bool coop = p.dh == 1 && p.dw == 1 && p.kw <= 8 && p.sw <= 2 &&
                              __all_sync(DC_FULL, valid && oy == oy0 && b == b0) != 0;
            if (coop) {
                const int ncol = 31 * p.sw + p.kw;
                const int shift = lane * p.sw;
                for (int ky = 0; ky < p.kh; ++ky) {
                    const int iy = y0 + ky;
                    unsigned w0 = 0u, w1 = 0u, w2 = 0u;
                    if (iy >= 0 && iy < p.hi) {                     // uniform over the warp
                        const int32_t* mrow = p.mi + ((int64_t)b0 * p.hi + iy) * p.wi;
                        int mv[3];
#pragma unroll
                        for (int m = 0; m < 3; ++m) {
                            const int c = lane + 32 * m, ix = x00 + c;
                            mv[m] = (c < ncol && ix >= 0 && ix < p.wi) ? mrow[ix] : 0;
                        }
                        w0 = __ballot_sync(DC_FULL, mv[0] != 0);
                        w1 = __ballot_sync(DC_FULL, mv[1] != 0);
                        w2 = __ballot_sync(DC_FULL, mv[2] != 0);
                    }
                    const unsigned long long lo = (unsigned long long)w0 | ((unsigned long long)w1 << 32);
                    unsigned long long win = lo >> shift;
                    if (shift > 0) win |= (unsigned long long)w2 << (64 - shift);
                    tapbits |= (win & ((1ull << p.kw) - 1ull)) << (ky * p.kw);
                }
                if (kEpi == 0 || tapbits == 0ull) p.mo[q] = tapbits != 0ull ? 1 : 0;
            } else if (valid) {
                const int in0 = (b * p.hi + y0) * p.wi + x0;
                for (int ky = 0; ky < p.kh; ++ky) {
                    const int iy = y0 + ky * p.dh;
                    if (iy < 0 || iy >= p.hi) continue;
                    // the reads of a filter row are issued together: four at a time for kernels up to 4 wide, else eight
                    const int32_t* mrow = p.mi + in0 + ky * p.dh * p.wi;
                    if (p.kw <= 4) tapbits |= (unsigned long long)mask_row_bits<4>(mrow, x0, p.kw, p.dw, p.wi) << (ky * p.kw);
                    else tapbits |= (unsigned long long)mask_row_bits<8>(mrow, x0, p.kw, p.dw, p.wi) << (ky * p.kw);
                }
                for (int kx = 8; kx < p.kw; ++kx) {               // wider rows (not used by any stem): one read at a time
                    const int ix = x0 + kx * p.dw;
                    if (ix < 0 || ix >= p.wi) continue;
                    for (int ky = 0; ky < p.kh; ++ky) {
                        const int iy = y0 + ky * p.dh;
                        if (iy >= 0 && iy < p.hi && p.mi[in0 + ky * p.dh * p.wi + kx * p.dw] != 0) tapbits |= 1ull << (ky * p.kw + kx);
                    }
                }
                if (kEpi == 0 || tapbits == 0ull) p.mo[q] = tapbits != 0ull ? 1 : 0;
            }
            const unsigned bal = __ballot_sync(DC_FULL, tapbits != 0ull);
            int base = 0;
            if (lane == 0 && bal != 0u) base = (int)atomicAdd(&s_u32[2], (uint32_t)__popc(bal));
            base = __shfl_sync(DC_FULL, base, 0);
            if (tapbits != 0ull) {
                const int slot = base + __popc(bal & ((1u << lane) - 1u));
                s_q[slot] = q;
                s_t[slot] = tapbits;
            }
        }
        __syncthreads();
        const int cnt = (int)s_u32[2];
        for (int t0 = 0; t0 < cnt && ok; t0 += kRows, ++tile) {
            const int cnt_t = min(kRows, cnt - t0);
            // ---- im2col of the tile: thread pair per row, each fills half of the K values in pairs of two ----
            {
                const int r = tid >> 1, half = tid & 1;
                if (r < cnt_t) {
                    const unsigned long long tb = s_t[t0 + r];
                    const __half* src = p.in + (int64_t)in0_of(s_q[t0 + r]) * p.ci;
                    const int k0 = half * (p.kcover >> 1), k1 = k0 + (p.kcover >> 1);
                    const uint32_t row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
                    for (int k = k0; k < k1; k += 2) {
                        const uint32_t e0 = s_ktab[k], e1 = s_ktab[k + 1];
                        unsigned short lo = 0, hi = 0;
                        if ((e0 >> 24) < 64u && ((tb >> (e0 >> 24)) & 1ull)) lo = __ldg(reinterpret_cast<const unsigned short*>(src) + (e0 & 0xffffffu));
                        if ((e1 >> 24) < 64u && ((tb >> (e1 >> 24)) & 1ull)) hi = __ldg(reinterpret_cast<const unsigned short*>(src) + (e1 & 0xffffffu));
                        const int kc = k & 63;
                        uint8_t* dst = sA + (size_t)(k >> 6) * kABytes + row_off + (((kc >> 3) ^ (r & 7)) << 4) + (kc & 7) * 2;
                        *reinterpret_cast<uint32_t*>(dst) = (uint32_t)lo | ((uint32_t)hi << 16);
                    }
                }
            }
            fence_proxy_async();
            __syncthreads();
            if (warp == 0 && elect_one()) {            // an elected lane of a converged warp: MMA operands in uniform registers
                tc_fence_after();
                const uint64_t ad0 = make_smem_desc(smem_u32(sA));
                const uint64_t bd0 = make_smem_desc(smem_u32(sB));
                for (int kb = 0; kb < p.nkb; ++kb) {
                    const int ksteps = kb == p.nkb - 1 ? p.last_ksteps : kKBlock / 16;
                    const uint64_t ad = ad0 + (uint64_t)((uint32_t)kb * (kABytes >> 4));
                    const uint64_t bd = bd0 + (uint64_t)((uint32_t)kb * ((uint32_t)p.co * 128u >> 4));
                    for (int ks = 0; ks < ksteps; ++ks)
                        umma_f16(tmem_base, ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(bar_done);
            }
            if (!mbar_wait_warp(bar_done, (uint32_t)(tile & 1), ok_flag)) { *ok_flag = 0; atomicExch(&g_stem_umma_error, 5); }
            __syncthreads();
            if (s_u32[1] == 0) { ok = false; break; }
            tc_fence_after();
            // ---- epilogue 1: tensor memory -> fp16 staging tile (row = TMEM lane) ----
            {
                const int quarter = warp & 3;                          // TMEM lanes a warp may read: 32 * (warp % 4) ...
                const int r = quarter * 32 + lane;
                uint8_t* srow = sStage + (size_t)r * p.stage_pitch;
#pragma unroll 1
                for (int c0 = (warp >> 2) * 16; c0 < p.co; c0 += 32) {
                    uint32_t acc[16];
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, acc);
                    tmem_ld_wait();
                    uint4 o[2];
                    __half2* h = reinterpret_cast<__half2*>(o);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        h[j] = __floats2half2_rn(__uint_as_float(acc[2 * j]) + s_bias[c0 + 2 * j],
                                                 __uint_as_float(acc[2 * j + 1]) + s_bias[c0 + 2 * j + 1]);
                    *reinterpret_cast<uint4*>(srow + c0 * 2) = o[0];
                    *reinterpret_cast<uint4*>(srow + c0 * 2 + 16) = o[1];
                }
            }
            tc_fence_before();
            __syncthreads();
            // ---- epilogue 2: coalesced rows, a lane group per pixel; optional fused truncation ----
#pragma unroll 1
            for (int rb = warp * ppw; rb < cnt_t; rb += (kSuThreads / 32) * ppw) {
                const int r = rb + lane / g;
                const bool mine = r < cnt_t && lig < nch;
                Pack<__half, 8> d, y, tr;
                int64_t off = 0;
                if (mine) {
                    off = (int64_t)s_q[t0 + r] * p.co + lig * 8;
                    d.load(reinterpret_cast<const __half*>(sStage + (size_t)r * p.stage_pitch) + lig * 8);
                    if (kEpi != 0) {
                        y.load(p.prev + off);
                        tr.load(p.trunc + off);
                    }
                }
                if (kEpi == 0) {
                    if (mine) d.store(p.out + off);
                    continue;
                }
                bool hit = false;
                if (mine) {
                    if constexpr (kEpi == 1) hit = truncate_pack_h2(d, y, tr, p.act, thr2);
                    else hit = truncate_pack_f32(d, y, tr, p.act, p.thr);
                }
                const bool active = group_any(hit, g, lane);
                if (mine) {
                    if (active) {
                        Pack<__half, 8> z; z.zero();
                        y.store(p.prev + off);
                        d.store(p.out + off);
                        z.store(p.trunc + off);
                    } else {
                        tr.store(p.trunc + off);
                    }
                }
                if (r < cnt_t && lig == 0) p.mo[s_q[t0 + r]] = active ? 1 : 0;
            }
            __syncthreads();               // the staging tile and the row lists are free again
            tc_fence_after();
        }
    }
    // every MMA that was issued has to finish before shared and tensor memory are released
    if (!ok && tid == 0) {
        for (uint32_t i = 0; i < kWaitLimit && !mbar_try_wait(bar_done, (uint32_t)(tile & 1)); ++i) {}
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
}

// groups == 1, fp16, c_in <= 4, c_out a multiple of 16 up to 256, kh*kw*c_in <= 192, with in- and out-mask, maps of at
// least 4096 output pixels; DC_ERR_UNSUPPORTED sends the caller to the CUDA-core stem kernels.
int conv_stem_umma(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                   int32_t* mo, const dc_epilogue* ep, cudaStream_t st) {
    const int taps = d->kh * d->kw;
    const int kdim = taps * d->c_in;
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    const bool ok = d->dtype == DC_F16 && d->groups == 1 && d->c_in <= 4 && d->c_out % 16 == 0 && d->c_out >= 16 && d->c_out <= 256 &&
                    taps <= 64 && kdim <= kSuMaxK && mi != nullptr && mo != nullptr && aligned16(out) && npix >= 4096 &&
                    (ep == nullptr || (ep->truncation == DC_TRUNC_MAX && aligned16(ep->prev_out) && aligned16(ep->truncated)));
    if (!ok) return DC_ERR_UNSUPPORTED;
    if (npix > 0x7fffffffLL || (int64_t)d->n * d->h_in * d->w_in * d->c_in > 0x7fffffffLL) return DC_ERR_SHAPE;
    StemUParams p{};
    p.in = (const __half*)in; p.mi = mi; p.w = (const __half*)filt; p.bias = (const __half*)bias;
    p.out = (__half*)out; p.mo = mo;
    p.prev = ep ? (__half*)ep->prev_out : nullptr;
    p.trunc = ep ? (__half*)ep->truncated : nullptr;
    p.thr = ep ? host_round_threshold<__half>(ep->threshold) : 0.f;
    p.act = ep ? ep->activation : 0;
    p.n = d->n; p.hi = d->h_in; p.wi = d->w_in; p.ci = d->c_in; p.ho = d->h_out; p.wo = d->w_out; p.co = d->c_out;
    p.kh = d->kh; p.kw = d->kw; p.sh = d->stride_h; p.sw = d->stride_w; p.pt = d->pad_top; p.pl = d->pad_left;
    p.dh = d->dil_h; p.dw = d->dil_w;
    p.kdim = kdim;
    p.nkb = divup(kdim, kKBlock);
    p.last_ksteps = divup(kdim - (p.nkb - 1) * kKBlock, 16);
    p.kcover = (p.nkb - 1) * kKBlock + p.last_ksteps * 16;
    p.tmem_cols = 32;
    while (p.tmem_cols < p.co) p.tmem_cols <<= 1;
    fast_div_init((uint32_t)p.wo, &p.wo_mul, &p.wo_shift);
    fast_div_init((uint32_t)p.ho, &p.ho_mul, &p.ho_shift);
    p.stage_pitch = (uint32_t)p.co * 2 + 16;
    const uint32_t ring = (uint32_t)p.nkb * kABytes, staging = kRows * p.stage_pitch;
    p.off_b = ((ring > staging ? ring : staging) + 1023) & ~1023u;
    p.off_list = (p.off_b + (uint32_t)p.nkb * (uint32_t)p.co * 128u + 15) & ~15u;
    p.off_misc = (p.off_list + kSuSpans * kSuSpanPx * 12u + kSuMaxK * 4u + 15) & ~15u;
    const size_t smem = p.off_misc + 8 + 16 + 4 * (size_t)p.co + 1024 /* alignment slack */;
    if (smem > 227 * 1024) return DC_ERR_UNSUPPORTED;
    static PerDeviceOnce attr_once;
    bool* attr_set = attr_once.slot();
    if (attr_set == nullptr) return DC_ERR_LAUNCH;
    if (!*attr_set) {
        bool okk = cudaFuncSetAttribute(k_stem_umma<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        okk &= cudaFuncSetAttribute(k_stem_umma<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        okk &= cudaFuncSetAttribute(k_stem_umma<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        if (!okk) return check_launch();
        *attr_set = true;
    }
    p.nspans = divup64(npix, kSuSpanPx);
    int64_t per_sm = (int64_t)(227 * 1024) / (int64_t)(smem + 1024);
    if (per_sm > 3) per_sm = 3;
    if (per_sm < 1) per_sm = 1;
    int64_t grid = (int64_t)sm_count() * per_sm;
    if (grid > p.nspans) grid = p.nspans;
    p.rounds = (int)divup64(divup64(p.nspans, grid), kSuSpans);
    const int epi = ep == nullptr ? 0 : (p.act >= DC_ACT_NONE && p.act <= DC_ACT_RELU6) ? 1 : 2;
    if (epi == 0) return launch_pdl(k_stem_umma<0>, dim3((unsigned)grid), dim3(kSuThreads), smem, st, p);
    if (epi == 1) return launch_pdl(k_stem_umma<1>, dim3((unsigned)grid), dim3(kSuThreads), smem, st, p);
    return launch_pdl(k_stem_umma<2>, dim3((unsigned)grid), dim3(kSuThreads), smem, st, p);
}

int stem_umma_error_code() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_stem_umma_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

}  // namespace dc
