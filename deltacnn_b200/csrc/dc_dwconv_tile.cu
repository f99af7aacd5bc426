// Depthwise 3x3 delta convolution fused with the activation/truncation step (fp16).
//
// One CTA per tile of TS x TS output pixels, all channels: the in-mask of the tile's receptive
// field is staged first and a tile without an active input leaves at once (moving objects make
// the active set spatially coherent, so most tiles are either skipped or mostly active). Active
// tiles stage their whole input patch (inactive pixels as zeros, never loaded) and the filter in
// shared memory with 16-byte accesses, every thread computes 8 channels of one output pixel per
// step with fp32 accumulation, and the result goes to a shared staging tile. The epilogue walks
// the active pixels with a lane group per pixel: plain store, or accumulate + activation delta +
// any-channel truncation against the two caches, so the convolution result never visits HBM.
#include "dc_common.cuh"

namespace dc {

struct DwTileParams {
    const __half* in; const int32_t* mi; const __half* w; const __half* bias;
    __half* out; int32_t* mo; __half* prev; __half* trunc;
    float thr; int act; int fused;
    int hi, wi, c, ho, wo, s, pt, pl;
    int ph, pw, tiles_x, tiles_y;
    uint32_t off_w, off_patch, off_stage;
};

template <int TS>
__global__ void __launch_bounds__(256) k_dw3x3_tile(DwTileParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int NPX = TS * TS;
    int* s_mask = reinterpret_cast<int*>(smem);                       // [ph*pw]
    int* s_om = s_mask + p.ph * p.pw;                                 // [NPX]
    __half* s_w = reinterpret_cast<__half*>(smem + p.off_w);          // [9][C]
    __half* s_patch = reinterpret_cast<__half*>(smem + p.off_patch);  // [ph*pw][C]
    __half* s_stage = reinterpret_cast<__half*>(smem + p.off_stage);  // [NPX][C]

    const int tid = threadIdx.x;
    int bid = blockIdx.x;
    const int tx = bid % p.tiles_x; bid /= p.tiles_x;
    const int ty = bid % p.tiles_y;
    const int b = bid / p.tiles_y;
    const int oy0 = ty * TS, ox0 = tx * TS;
    const int py0 = oy0 * p.s - p.pt, px0 = ox0 * p.s - p.pl;
    const int npatch = p.ph * p.pw;
    const int64_t img_in = (int64_t)b * p.hi * p.wi;
    const int64_t img_out = (int64_t)b * p.ho * p.wo;

    bool any = false;
    for (int i = tid; i < npatch; i += 256) {
        const int y = py0 + i / p.pw, x = px0 + i % p.pw;
        int m = 0;
        if (y >= 0 && y < p.hi && x >= 0 && x < p.wi) m = p.mi[img_in + (int64_t)y * p.wi + x] != 0;
        s_mask[i] = m;
        any |= m != 0;
    }
    any = __syncthreads_or(any);
    if (tid < NPX) {
        const int ly = tid / TS, lx = tid % TS;
        const bool inb = (oy0 + ly) < p.ho && (ox0 + lx) < p.wo;
        int om = 0;
        if (any && inb) {
#pragma unroll
            for (int t = 0; t < 9; ++t) om |= s_mask[(ly * p.s + t / 3) * p.pw + lx * p.s + t % 3];
        }
        s_om[tid] = om;
        if (inb && (!p.fused || !om)) p.mo[img_out + (int64_t)(oy0 + ly) * p.wo + ox0 + lx] = om;
    }
    if (!any) return;

    const int npk = p.c >> 3;
    for (int i = tid; i < 9 * npk; i += 256)
        reinterpret_cast<uint4*>(s_w)[i] = __ldg(reinterpret_cast<const uint4*>(p.w) + i);
    for (int i = tid; i < npatch * npk; i += 256) {
        const int pp = i / npk, pk = i - pp * npk;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (s_mask[pp]) {
            const int y = py0 + pp / p.pw, x = px0 + pp % p.pw;
            v = __ldg(reinterpret_cast<const uint4*>(p.in + (img_in + (int64_t)y * p.wi + x) * p.c) + pk);
        }
        reinterpret_cast<uint4*>(s_patch)[i] = v;
    }
    __syncthreads();

    for (int i = tid; i < NPX * npk; i += 256) {
        const int px = i / npk, pk = i - px * npk;
        if (!s_om[px]) continue;
        const int ly = px / TS, lx = px % TS;
        float acc[8];
        if (p.bias != nullptr) {
            Pack<__half, 8> bb; bb.load(p.bias + pk * 8);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = bb.get(k);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        }
#pragma unroll
        for (int t = 0; t < 9; ++t) {
            const int pp = (ly * p.s + t / 3) * p.pw + lx * p.s + t % 3;
            if (!s_mask[pp]) continue;
            Pack<__half, 8> v, w;
            v.load(s_patch + (size_t)pp * p.c + pk * 8);
            w.load(s_w + t * p.c + pk * 8);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = fmaf(v.get(k), w.get(k), acc[k]);
        }
        Pack<__half, 8> o;
#pragma unroll
        for (int k = 0; k < 8; ++k) o.set(k, acc[k]);
        o.store(s_stage + (size_t)px * p.c + pk * 8);
    }
    __syncthreads();

    // epilogue: a lane group per active output pixel
    int g = 1;
    while (g < npk && g < 32) g <<= 1;
    const int lane = tid & 31, warp = tid >> 5;
    const int lig = lane & (g - 1);
    const int ppw = 32 / g;
    constexpr int NV = 4;                                              // packs per lane (C <= 1024)
    for (int pb = warp * ppw; pb < NPX; pb += 8 * ppw) {
        const int px = pb + lane / g;
        const bool on = px < NPX && s_om[px] != 0;
        if (__ballot_sync(DC_FULL, on) == 0) continue;
        const int ly = px / TS, lx = px % TS;
        const int64_t q = img_out + (int64_t)(oy0 + ly) * p.wo + ox0 + lx;
        const int64_t off = q * p.c;
        if (!p.fused) {
            if (on)
                for (int i = lig; i < npk; i += g)
                    reinterpret_cast<uint4*>(p.out + off)[i] = reinterpret_cast<const uint4*>(s_stage + (size_t)px * p.c)[i];
            continue;
        }
        Pack<__half, 8> pe[NV], pu[NV], pr[NV];
        bool hit = false;
        if (on) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int i = lig + j * g;
                if (i >= npk) continue;
                Pack<__half, 8> d;
                d.load(s_stage + (size_t)px * p.c + i * 8);
                pu[j].load(p.prev + off + i * 8);
                pr[j].load(p.trunc + off + i * 8);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float yo = pu[j].get(k);
                    const float rr = rnd<__half>(pr[j].get(k) + d.get(k));
                    const float u = rnd<__half>(yo + rr);
                    const float ee = rnd<__half>(act_apply(u, p.act) - act_apply(yo, p.act));
                    pr[j].set(k, rr); pu[j].set(k, u); pe[j].set(k, ee);
                    hit |= fabsf(ee) > p.thr;
                }
            }
        }
        const bool active = group_any(hit, g, lane);
        if (!on) continue;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = lig + j * g;
            if (i >= npk) continue;
            if (active) {
                Pack<__half, 8> z; z.zero();
                pu[j].store(p.prev + off + i * 8);
                pe[j].store(p.out + off + i * 8);
                z.store(p.trunc + off + i * 8);
            } else {
                pr[j].store(p.trunc + off + i * 8);
            }
        }
        if (lig == 0) p.mo[q] = active ? 1 : 0;
    }
}

// Depthwise 3x3 (stride 1 or 2, dilation 1) in fp16 with an out-mask; DC_ERR_UNSUPPORTED tells the
// caller to use the generic kernels.
int dwconv3x3_tile(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                   int32_t* mo, const dc_epilogue* ep, cudaStream_t st) {
    const bool ok = d->dtype == DC_F16 && d->kh == 3 && d->kw == 3 && d->dil_h == 1 && d->dil_w == 1 &&
                    d->stride_h == d->stride_w && (d->stride_h == 1 || d->stride_h == 2) && d->groups == d->c_in &&
                    d->c_in == d->c_out && d->c_in % 8 == 0 && d->c_in <= 1024 && mi != nullptr && mo != nullptr &&
                    aligned16(in) && aligned16(out) && aligned16(filt) && (bias == nullptr || aligned16(bias)) &&
                    (ep == nullptr || (ep->truncation == DC_TRUNC_MAX && aligned16(ep->prev_out) && aligned16(ep->truncated)));
    if (!ok) return DC_ERR_UNSUPPORTED;
    if (d->n == 0) return DC_OK;
    const int ts = (d->h_out <= 16 || d->w_out <= 16) ? 4 : 8;
    DwTileParams p{};
    p.in = (const __half*)in; p.mi = mi; p.w = (const __half*)filt; p.bias = (const __half*)bias;
    p.out = (__half*)out; p.mo = mo;
    p.fused = ep != nullptr;
    p.prev = p.fused ? (__half*)ep->prev_out : nullptr;
    p.trunc = p.fused ? (__half*)ep->truncated : nullptr;
    p.thr = p.fused ? host_round_threshold<__half>(ep->threshold) : 0.f;
    p.act = p.fused ? ep->activation : 0;
    p.hi = d->h_in; p.wi = d->w_in; p.c = d->c_in; p.ho = d->h_out; p.wo = d->w_out; p.s = d->stride_h;
    p.pt = d->pad_top; p.pl = d->pad_left;
    p.ph = (ts - 1) * p.s + 3; p.pw = p.ph;
    p.tiles_x = divup(p.wo, ts); p.tiles_y = divup(p.ho, ts);
    const uint32_t npatch = (uint32_t)(p.ph * p.pw);
    p.off_w = ((npatch + ts * ts) * 4 + 15) & ~15u;
    p.off_patch = p.off_w + 9u * p.c * 2u;
    p.off_stage = p.off_patch + npatch * p.c * 2u;
    const size_t smem = p.off_stage + (size_t)ts * ts * p.c * 2;
    if (smem > 200 * 1024) return DC_ERR_UNSUPPORTED;
    const int64_t blocks = (int64_t)p.tiles_x * p.tiles_y * d->n;
    if (blocks > 0x7fffffffLL) return DC_ERR_SHAPE;
    static thread_local bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(k_dw3x3_tile<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(k_dw3x3_tile<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return check_launch();
        attr_set = true;
    }
    if (ts == 4) k_dw3x3_tile<4><<<(unsigned)blocks, 256, smem, st>>>(p);
    else k_dw3x3_tile<8><<<(unsigned)blocks, 256, smem, st>>>(p);
    return check_launch();
}

}  // namespace dc
