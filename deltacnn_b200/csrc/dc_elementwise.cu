// Bandwidth-bound per-pixel kernels of the delta-update path: sparsify, activation +
// truncation, add, accumulate, scale/bias, concatenate, densify, upsample, mask compaction.
//
// Work decomposition shared by all of them: a pixel's channel vector is split into
// 16-byte packs; an aligned group of g lanes (g = power of two <= 32) owns one pixel,
// so one warp covers 32/g pixels and a 128-byte sector is always consumed whole.
// Warps whose pixels are all inactive leave after one coalesced mask read. Grids are
// sized in multiples of the SM count with a grid-stride loop.
#include "dc_common.cuh"

namespace dc {

#define DC_PIXEL_LOOP(npix, g)                                                              \
    grid_dep_launch();                                                                      \
    grid_dep_wait();                                                                        \
    const int lane = threadIdx.x & 31;                                                      \
    const int lig = lane & ((g) - 1);                                                       \
    const int ppw = 32 / (g);                                                               \
    const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);     \
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);                          \
    for (int64_t base = warp0 * ppw; base < (npix); base += nwarps * ppw)

static inline dim3 pixel_grid(int64_t npix, int g, int threads = 256) {
    int64_t warps = divup64(npix, 32 / g);
    int64_t blocks = divup64(warps, threads / 32);
    int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return dim3((unsigned)blocks);
}

// ---------------------------------------------------------------------------------------------
// sparsify
// ---------------------------------------------------------------------------------------------
template <typename T, int W>
__global__ void __launch_bounds__(256) k_sparsify(const T* __restrict__ x, T* __restrict__ prev, T* __restrict__ delta,
                                                  int32_t* __restrict__ mask, int64_t npix, int C, int g, float thr) {
    const int nvec = C / W;
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        const bool inb = px < npix;
        const int64_t off = px * C;
        bool hit = false;
        if (inb) {
            for (int i = lig; i < nvec; i += g) {
                Pack<T, W> a, b;
                a.load(x + off + i * W);
                b.load(prev + off + i * W);
#pragma unroll
                for (int k = 0; k < W; ++k) hit |= fabsf(rnd<T>(a.get(k) - b.get(k))) > thr;
            }
        }
        const bool active = group_any(hit, g, lane);
        if (inb) {
            if (lig == 0) mask[px] = active ? 1 : 0;
            if (active) {
                for (int i = lig; i < nvec; i += g) {
                    Pack<T, W> a, b, d;
                    a.load(x + off + i * W);
                    b.load(prev + off + i * W);
#pragma unroll
                    for (int k = 0; k < W; ++k) d.set(k, a.get(k) - b.get(k));
                    d.store(delta + off + i * W);
                    a.store(prev + off + i * W);
                }
            }
        }
    }
}

// RGB frames (3 channels): a thread owns the run of pixels that fills three 16-byte vectors (8 fp16
// pixels or 4 fp32 pixels), so the two full reads of the frame are 16-byte accesses and the mask words go out as
// vectors. A run with at least one active pixel writes its delta and cache vectors whole (the cache keeps its old
// value at the run's inactive pixels; their delta, which the contract leaves undefined, receives the sub-threshold
// difference): element-wise stores of the active pixels alone kept the load/store queue full (ncu: lg_throttle 16
// stalled warps per issue). Runs without an active pixel write nothing but the mask.
template <typename T>
__global__ void __launch_bounds__(256) k_sparsify_c3(const T* __restrict__ x, T* __restrict__ prev, T* __restrict__ delta,
                                                     int32_t* __restrict__ mask, int64_t npix, float thr) {
    constexpr int PPT = sizeof(T) == 2 ? 8 : 4;                         // pixels per thread
    constexpr int NE = PPT * 3;                                         // elements per thread (3 x 16 bytes)
    grid_dep_launch();
    grid_dep_wait();
    const int64_t ngroups = npix / PPT;
    for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < ngroups; gi += (int64_t)gridDim.x * blockDim.x) {
        alignas(16) T xa[NE];
        alignas(16) T pa[NE];
        alignas(16) T da[NE];
        const uint4* xs = reinterpret_cast<const uint4*>(x + gi * NE);
        const uint4* ps = reinterpret_cast<const uint4*>(prev + gi * NE);
#pragma unroll
        for (int i = 0; i < 3; ++i) { reinterpret_cast<uint4*>(xa)[i] = xs[i]; reinterpret_cast<uint4*>(pa)[i] = ps[i]; }
        alignas(16) int32_t m[PPT];
        bool any = false;
#pragma unroll
        for (int px = 0; px < PPT; ++px) {
            bool hit = false;
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                const float d = rnd<T>(to_f<T>(xa[px * 3 + c]) - to_f<T>(pa[px * 3 + c]));
                da[px * 3 + c] = from_f<T>(d);
                hit |= fabsf(d) > thr;
            }
            m[px] = hit ? 1 : 0;
            any |= hit;
            if (hit) {
#pragma unroll
                for (int c = 0; c < 3; ++c) pa[px * 3 + c] = xa[px * 3 + c];
            }
        }
        if (any) {
            uint4* dd = reinterpret_cast<uint4*>(delta + gi * NE);
            uint4* pd = reinterpret_cast<uint4*>(prev + gi * NE);
#pragma unroll
            for (int i = 0; i < 3; ++i) { dd[i] = reinterpret_cast<const uint4*>(da)[i]; pd[i] = reinterpret_cast<const uint4*>(pa)[i]; }
        }
#pragma unroll
        for (int i = 0; i < PPT / 4; ++i) reinterpret_cast<int4*>(mask + gi * PPT)[i] = reinterpret_cast<const int4*>(m)[i];
    }
}

// 8-bit frame: value = u8 * scale[c] + offset[c] (a rounded product, then a rounded sum: the arithmetic of
// frame.float() * scale + offset in torch), rounded to T before the compare.
template <typename T>
__global__ void __launch_bounds__(256) k_sparsify_u8(const uint8_t* __restrict__ x, const float* __restrict__ scale,
                                                     const float* __restrict__ offset, T* __restrict__ prev,
                                                     T* __restrict__ delta, int32_t* __restrict__ mask, int64_t npix, int C,
                                                     int g, float thr) {
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        const bool inb = px < npix;
        const int64_t off = px * C;
        bool hit = false;
        if (inb) {
            for (int c = lig; c < C; c += g) {
                float v = rnd<T>(__fadd_rn(__fmul_rn((float)x[off + c], scale[c]), offset[c]));
                hit |= fabsf(rnd<T>(v - to_f<T>(prev[off + c]))) > thr;
            }
        }
        const bool active = group_any(hit, g, lane);
        if (inb) {
            if (lig == 0) mask[px] = active ? 1 : 0;
            if (active) {
                for (int c = lig; c < C; c += g) {
                    float v = rnd<T>(__fadd_rn(__fmul_rn((float)x[off + c], scale[c]), offset[c]));
                    delta[off + c] = from_f<T>(v - to_f<T>(prev[off + c]));
                    prev[off + c] = from_f<T>(v);
                }
            }
        }
    }
}

// 8-bit RGB frames: the run-of-pixels form of k_sparsify_c3 (a thread owns 8 fp16 or 4 fp32 pixels: 24 or 12 bytes of the
// frame, three 16-byte vectors of the cache and of the delta, the mask words as vectors), with the arithmetic of
// k_sparsify_u8.
template <typename T>
__global__ void __launch_bounds__(256) k_sparsify_u8_c3(const uint8_t* __restrict__ x, const float* __restrict__ scale,
                                                        const float* __restrict__ offset, T* __restrict__ prev,
                                                        T* __restrict__ delta, int32_t* __restrict__ mask, int64_t npix, float thr) {
    constexpr int PPT = sizeof(T) == 2 ? 8 : 4;                         // pixels per thread
    constexpr int NE = PPT * 3;                                         // elements per thread
    grid_dep_launch();
    grid_dep_wait();
    const float sc[3] = {scale[0], scale[1], scale[2]};
    const float of[3] = {offset[0], offset[1], offset[2]};
    const int64_t ngroups = npix / PPT;
    for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < ngroups; gi += (int64_t)gridDim.x * blockDim.x) {
        alignas(8) uint8_t xb[NE];
        alignas(16) T pa[NE];
        alignas(16) T da[NE];
        const uint32_t* xs = reinterpret_cast<const uint32_t*>(x + gi * NE);     // NE is a multiple of 4, the frame 4-byte aligned
        const uint4* ps = reinterpret_cast<const uint4*>(prev + gi * NE);
#pragma unroll
        for (int i = 0; i < NE / 4; ++i) reinterpret_cast<uint32_t*>(xb)[i] = xs[i];
#pragma unroll
        for (int i = 0; i < 3; ++i) reinterpret_cast<uint4*>(pa)[i] = ps[i];
        alignas(16) int32_t m[PPT];
        bool any = false;
#pragma unroll
        for (int px = 0; px < PPT; ++px) {
            bool hit = false;
            T v[3];
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                const float vf = rnd<T>(__fadd_rn(__fmul_rn((float)xb[px * 3 + c], sc[c]), of[c]));
                const float d = rnd<T>(vf - to_f<T>(pa[px * 3 + c]));
                v[c] = from_f<T>(vf);
                da[px * 3 + c] = from_f<T>(d);
                hit |= fabsf(d) > thr;
            }
            m[px] = hit ? 1 : 0;
            any |= hit;
            if (hit) {
#pragma unroll
                for (int c = 0; c < 3; ++c) pa[px * 3 + c] = v[c];
            }
        }
        if (any) {
            uint4* dd = reinterpret_cast<uint4*>(delta + gi * NE);
            uint4* pd = reinterpret_cast<uint4*>(prev + gi * NE);
#pragma unroll
            for (int i = 0; i < 3; ++i) { dd[i] = reinterpret_cast<const uint4*>(da)[i]; pd[i] = reinterpret_cast<const uint4*>(pa)[i]; }
        }
#pragma unroll
        for (int i = 0; i < PPT / 4; ++i) reinterpret_cast<int4*>(mask + gi * PPT)[i] = reinterpret_cast<const int4*>(m)[i];
    }
}

// Noise-robust input mask, DCSparsify(dilation = k) (reference: src/deltacnn/sparse_layers.py:1233-1248, torch ops
// there): delta = x - prev at EVERY pixel, mask = max-pool_{k x k, stride 1}(max_c |delta|) > threshold, and the cache
// takes the new frame where the mask is set. max-pool(v) > t holds exactly when some element of the window has
// v > t, so step 1 writes one hit flag per pixel and step 2 ORs the flags over the window (rows, then columns, in
// shared memory) and updates the cache. Two kernels, because step 2 of a pixel needs step 1 of its neighbours
// against the OLD cache.
template <typename T>
__global__ void __launch_bounds__(256) k_sparsify_hit(const T* __restrict__ x, const T* __restrict__ prev, T* __restrict__ delta,
                                                      uint8_t* __restrict__ hit, int64_t npix, int C, float thr) {
    grid_dep_launch();
    grid_dep_wait();
    for (int64_t px = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; px < npix; px += (int64_t)gridDim.x * blockDim.x) {
        bool h = false;
        for (int c = 0; c < C; ++c) {
            const float d = rnd<T>(to_f<T>(x[px * C + c]) - to_f<T>(prev[px * C + c]));
            delta[px * C + c] = from_f<T>(d);
            h |= fabsf(d) > thr;
        }
        hit[px] = h ? 1 : 0;
    }
}

constexpr int kDilTileW = 32, kDilTileH = 8, kDilMaxR = 16;
template <typename T>
__global__ void __launch_bounds__(256) k_sparsify_dilate(const T* __restrict__ x, T* __restrict__ prev, const uint8_t* __restrict__ hit,
                                                         int32_t* __restrict__ mask, int h, int w, int C, int r) {
    __shared__ uint8_t s_hit[(kDilTileH + 2 * kDilMaxR) * (kDilTileW + 2 * kDilMaxR)];
    __shared__ uint8_t s_row[(kDilTileH + 2 * kDilMaxR) * kDilTileW];
    grid_dep_launch();
    grid_dep_wait();
    const int x0 = blockIdx.x * kDilTileW, y0 = blockIdx.y * kDilTileH;
    const int64_t b = blockIdx.z;
    const int rw = kDilTileW + 2 * r, rh = kDilTileH + 2 * r;
    for (int i = threadIdx.x; i < rw * rh; i += 256) {
        const int yy = y0 - r + i / rw, xx = x0 - r + i % rw;
        s_hit[i] = (yy >= 0 && yy < h && xx >= 0 && xx < w) ? hit[(b * h + yy) * w + xx] : 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rh * kDilTileW; i += 256) {      // OR along the row
        const int ry = i / kDilTileW, cx = i % kDilTileW;
        uint8_t v = 0;
        for (int d = 0; d <= 2 * r; ++d) v |= s_hit[ry * rw + cx + d];
        s_row[i] = v;
    }
    __syncthreads();
    const int tx = threadIdx.x % kDilTileW, ty = threadIdx.x / kDilTileW;
    const int ox = x0 + tx, oy = y0 + ty;
    if (ox >= w || oy >= h) return;
    uint8_t v = 0;
    for (int d = 0; d <= 2 * r; ++d) v |= s_row[(ty + d) * kDilTileW + tx];
    const int64_t px = (b * h + oy) * w + ox;
    mask[px] = v ? 1 : 0;
    if (v)
        for (int c = 0; c < C; ++c) prev[px * C + c] = x[px * C + c];
}

// ---------------------------------------------------------------------------------------------
// activation + truncation
// ---------------------------------------------------------------------------------------------
// NV > 0: every lane keeps its NV packs of (e, u, r) in registers between the
// any-channel decision and the write-back, so each state tensor is read once.
// NV == 0: two passes, the second recomputes (used for very wide pixels).
// kHalfFast: fp16 packs, max-truncation and an activation of act_exact_in_half: only the packed-half step is compiled in.
template <typename T, int W, int NV, bool kHalfFast = false>
__global__ void __launch_bounds__(256) k_act_trunc(T* __restrict__ delta, T* __restrict__ prev, T* __restrict__ trunc,
                                                   int32_t* __restrict__ mask, int64_t npix, int C, int g, float thr,
                                                   int act, int mode) {
    const int nvec = C / W;
    const __half2 thr2 = __float2half2_rn(thr);
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        const bool on = (px < npix) && (mask[px] != 0);
        if (__ballot_sync(DC_FULL, on) == 0) continue;
        const int64_t off = px * C;
        if (mode < 0) {  // no truncation: accumulate, emit activation delta
            if (on) {
                for (int i = lig; i < nvec; i += g) {
                    Pack<T, W> d, y;
                    d.load(delta + off + i * W);
                    y.load(prev + off + i * W);
#pragma unroll
                    for (int k = 0; k < W; ++k) {
                        float yo = y.get(k);
                        float u = rnd<T>(yo + d.get(k));
                        y.set(k, u);
                        if (act > 0) d.set(k, act_apply(u, act) - act_apply(yo, act));
                    }
                    y.store(prev + off + i * W);
                    if (act > 0) d.store(delta + off + i * W);
                }
            }
            continue;
        }
        constexpr int NH = NV > 0 ? NV : 1;
        Pack<T, W> pe[NH], pu[NH], pr[NH];
        bool hit = false;
        float ss = 0.f;
        auto first_pass = [&](int i, Pack<T, W>& e, Pack<T, W>& y, Pack<T, W>& r) {
            Pack<T, W> d;
            d.load(delta + off + i * W);
            y.load(prev + off + i * W);
            r.load(trunc + off + i * W);
            if constexpr (kHalfFast && sizeof(T) == 2 && W == 8) {     // packed half arithmetic, bit-identical (see truncate_pack_h2)
                hit |= truncate_pack_h2(d, y, r, act, thr2);
                e = d;
            } else {
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    float yo = y.get(k);
                    float rr = rnd<T>(r.get(k) + d.get(k));
                    float u = rnd<T>(yo + rr);
                    float ee = rnd<T>(act_apply(u, act) - act_apply(yo, act));
                    r.set(k, rr); y.set(k, u); e.set(k, ee);
                    hit |= fabsf(ee) > thr;
                    ss = fmaf(ee, ee, ss);
                }
            }
        };
        if (on) {
            if constexpr (NV > 0) {
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const int i = lig + j * g;
                    if (i < nvec) first_pass(i, pe[j], pu[j], pr[j]);
                }
            } else {
                for (int i = lig; i < nvec; i += g) first_pass(i, pe[0], pu[0], pr[0]);
            }
        }
        bool active;
        if (mode == DC_TRUNC_MAX) {
            active = group_any(hit, g, lane);
        } else {
            float tot = group_sum(ss, g);
            if (mode == DC_TRUNC_RMS) tot /= (float)C;
            active = sqrtf(tot) > thr;
        }
        if (!on) continue;
        if (NV > 0) {
#pragma unroll
            for (int j = 0; j < NH; ++j) {
                const int i = lig + j * g;
                if (i >= nvec) continue;
                if (active) {
                    Pack<T, W> z; z.zero();
                    pu[j].store(prev + off + i * W);
                    pe[j].store(delta + off + i * W);
                    z.store(trunc + off + i * W);
                } else {
                    pr[j].store(trunc + off + i * W);
                }
            }
        } else {
            for (int i = lig; i < nvec; i += g) {
                Pack<T, W> d, y, r;
                d.load(delta + off + i * W);
                y.load(prev + off + i * W);
                r.load(trunc + off + i * W);
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    float yo = y.get(k);
                    float rr = rnd<T>(r.get(k) + d.get(k));
                    float u = rnd<T>(yo + rr);
                    r.set(k, active ? 0.f : rr);
                    y.set(k, u);
                    d.set(k, act_apply(u, act) - act_apply(yo, act));
                }
                r.store(trunc + off + i * W);
                if (active) {
                    y.store(prev + off + i * W);
                    d.store(delta + off + i * W);
                }
            }
        }
        if (!active && lig == 0) mask[px] = 0;
    }
}

// ---------------------------------------------------------------------------------------------
// add
// ---------------------------------------------------------------------------------------------
template <typename T, int W>
__global__ void __launch_bounds__(256) k_add(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ prev,
                                             T* __restrict__ out, const int32_t* __restrict__ ma,
                                             const int32_t* __restrict__ mb, int32_t* __restrict__ mo, float wa, float wb,
                                             int64_t npix, int C, int act, int dense_out, int g) {
    const int nvec = C / W;
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        if (px >= npix) continue;
        const bool aa = ma[px] != 0, ab = mb[px] != 0;
        const bool any = aa || ab;
        if (!dense_out && lig == 0) mo[px] = any ? 1 : 0;
        if (!any && !dense_out) continue;
        const int64_t off = px * C;
        const bool with_prev = dense_out || act > 0;
        for (int i = lig; i < nvec; i += g) {
            // the three reads of a pack are issued together (none of them waits for another one's data)
            Pack<T, W> o, va, vb, y;
            if (aa) va.load(a + off + i * W); else va.zero();
            if (ab) vb.load(b + off + i * W); else vb.zero();
            if (with_prev) y.load(prev + off + i * W);
            float s[W];
#pragma unroll
            for (int k = 0; k < W; ++k) s[k] = aa ? va.get(k) * wa : 0.f;
            if (ab) {
#pragma unroll
                for (int k = 0; k < W; ++k) s[k] = fmaf(vb.get(k), wb, s[k]);
            }
            if (!with_prev) {
#pragma unroll
                for (int k = 0; k < W; ++k) o.set(k, s[k]);
                o.store(out + off + i * W);
                continue;
            }
#pragma unroll
            for (int k = 0; k < W; ++k) {
                float yo = y.get(k);
                float u = any ? rnd<T>(yo + s[k]) : yo;
                y.set(k, u);
                o.set(k, dense_out ? act_apply(u, act) : act_apply(u, act) - act_apply(yo, act));
            }
            if (any) y.store(prev + off + i * W);
            o.store(out + off + i * W);
        }
    }
}

template <typename T, int W>
__global__ void __launch_bounds__(256) k_add_to_dense(const T* __restrict__ a, T* __restrict__ b,
                                                      const int32_t* __restrict__ ma, int64_t npix, int C, int g) {
    const int nvec = C / W;
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        if (px >= npix || ma[px] == 0) continue;
        const int64_t off = px * C;
        for (int i = lig; i < nvec; i += g) {
            Pack<T, W> u, v;
            u.load(a + off + i * W);
            v.load(b + off + i * W);
#pragma unroll
            for (int k = 0; k < W; ++k) v.set(k, v.get(k) + u.get(k));
            v.store(b + off + i * W);
        }
    }
}

template <typename T, int W>
__global__ void __launch_bounds__(256) k_scale_bias(const T* __restrict__ in, const int32_t* __restrict__ mi,
                                                    T* __restrict__ out, int32_t* __restrict__ mo,
                                                    const T* __restrict__ scale, const T* __restrict__ bias, int64_t npix,
                                                    int C, int g) {
    const int nvec = C / W;
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        if (px >= npix) continue;
        const bool on = mi == nullptr || mi[px] != 0;
        if (mo != nullptr && mo != mi && lig == 0) mo[px] = on ? 1 : 0;
        if (!on) continue;
        const int64_t off = px * C;
        for (int i = lig; i < nvec; i += g) {
            Pack<T, W> v, s, bb;
            v.load(in + off + i * W);
            s.load(scale + i * W);
            if (bias) bb.load(bias + i * W); else bb.zero();
#pragma unroll
            for (int k = 0; k < W; ++k) v.set(k, fmaf(v.get(k), s.get(k), bb.get(k)));
            v.store(out + off + i * W);
        }
    }
}

template <typename T, int W>
__global__ void __launch_bounds__(256) k_concat(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out,
                                                const int32_t* __restrict__ ma, const int32_t* __restrict__ mb,
                                                int32_t* __restrict__ mo, int64_t npix, int Ca, int Cb, int g) {
    const int na = Ca / W, nvec = (Ca + Cb) / W;
    const int C = Ca + Cb;
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        if (px >= npix) continue;
        const bool aa = ma[px] != 0, ab = mb[px] != 0;
        if (lig == 0) mo[px] = (aa || ab) ? 1 : 0;
        if (!aa && !ab) continue;
        for (int i = lig; i < nvec; i += g) {
            Pack<T, W> v;
            v.zero();
            if (i < na) { if (aa) v.load(a + px * Ca + i * W); }
            else        { if (ab) v.load(b + px * Cb + (i - na) * W); }
            v.store(out + px * C + i * W);
        }
    }
}

template <typename T, int W>
__global__ void __launch_bounds__(256) k_densify(const T* __restrict__ delta, const int32_t* __restrict__ mask,
                                                 T* __restrict__ prev, T* __restrict__ dense, int64_t npix, int C, int act,
                                                 int g) {
    const int nvec = C / W;
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        if (px >= npix) continue;
        const bool on = mask[px] != 0;
        if (!on && dense == nullptr) continue;
        const int64_t off = px * C;
        for (int i = lig; i < nvec; i += g) {
            Pack<T, W> y;
            y.load(prev + off + i * W);
            if (on) {
                Pack<T, W> d;
                d.load(delta + off + i * W);
#pragma unroll
                for (int k = 0; k < W; ++k) y.set(k, y.get(k) + d.get(k));
                y.store(prev + off + i * W);
            }
            if (dense != nullptr) {
                if (act > 0) {
#pragma unroll
                    for (int k = 0; k < W; ++k) y.set(k, act_apply(y.get(k), act));
                }
                y.store(dense + off + i * W);
            }
        }
    }
}

template <typename T, int W>
__global__ void __launch_bounds__(256) k_upsample(const T* __restrict__ in, const int32_t* __restrict__ mi,
                                                  T* __restrict__ out, int32_t* __restrict__ mo, int n, int h, int w, int C,
                                                  int scale, int g) {
    const int nvec = C / W;
    const int ho = h * scale, wo = w * scale;
    const int64_t npix = (int64_t)n * ho * wo;
    DC_PIXEL_LOOP(npix, g) {
        const int64_t px = base + lane / g;
        if (px >= npix) continue;
        const int ox = (int)(px % wo);
        const int64_t t = px / wo;
        const int oy = (int)(t % ho);
        const int64_t b = t / ho;
        const int64_t src = (b * h + oy / scale) * w + ox / scale;
        const bool on = mi[src] != 0;
        if (lig == 0) mo[px] = on ? 1 : 0;
        if (!on) continue;
        for (int i = lig; i < nvec; i += g) {
            Pack<T, W> v;
            v.load(in + src * C + i * W);
            v.store(out + px * C + i * W);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// mask compaction: ballot per warp, shared prefix over the block's warps, one atomicAdd per block
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_compact_mask(const int32_t* __restrict__ mask, int64_t npix,
                                                      int32_t* __restrict__ indices, int32_t* __restrict__ count) {
    __shared__ int warp_cnt[8];
    __shared__ int block_base;
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int64_t start = (int64_t)blockIdx.x * 256; start < npix; start += (int64_t)gridDim.x * 256) {
        const int64_t px = start + threadIdx.x;
        const bool on = px < npix && mask[px] != 0;
        const unsigned b = __ballot_sync(DC_FULL, on);
        if (lane == 0) warp_cnt[wid] = __popc(b);
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { int c = warp_cnt[i]; warp_cnt[i] = tot; tot += c; }
            block_base = tot ? atomicAdd(count, tot) : 0;
        }
        __syncthreads();
        if (on) indices[block_base + warp_cnt[wid] + __popc(b & ((1u << lane) - 1u))] = (int32_t)px;
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// host dispatch
// ---------------------------------------------------------------------------------------------
#define DC_REQUIRE(p) do { if ((p) == nullptr) return DC_ERR_NULL_POINTER; } while (0)

template <typename T> static inline int pick_w(int C, std::initializer_list<const void*> ptrs) {
    constexpr int V = VecTraits<T>::kVec;
    if (C % V != 0) return 1;
    for (const void* p : ptrs) if (p != nullptr && !aligned16(p)) return 1;
    return V;
}

template <typename T>
static int sparsify_t(const T* x, T* prev, T* delta, int32_t* mask, int64_t npix, int C, float thr, cudaStream_t st) {
    constexpr int V = VecTraits<T>::kVec;
    const int W = pick_w<T>(C, {x, prev, delta});
    const float t = host_round_threshold<T>(thr);
    if (C == 3 && aligned16(x) && aligned16(prev) && aligned16(delta) && aligned16(mask)) {
        constexpr int PPT = sizeof(T) == 2 ? 8 : 4;
        const int64_t ngroups = npix / PPT;
        if (ngroups > 0) {
            int64_t blocks = divup64(ngroups, 256);
            const int64_t cap = (int64_t)sm_count() * 16;
            if (blocks > cap) blocks = cap;
            launch_pdl(k_sparsify_c3<T>, (unsigned)blocks, dim3(256), 0, st, x, prev, delta, mask, npix, t);
        }
        const int64_t done = ngroups * PPT;
        if (done < npix) {      // ragged tail: the generic kernel on the last few pixels
            const int g = lanes_per_pixel(C);
            launch_pdl(k_sparsify<T, 1>, 1, dim3(256), 0, st, x + done * 3, prev + done * 3, delta + done * 3, mask + done, npix - done, C, g, t);
        }
        return check_launch();
    }
    if (W == V) {
        const int g = lanes_per_pixel(C / V);
        launch_pdl(k_sparsify<T, V>, pixel_grid(npix, g), dim3(256), 0, st, x, prev, delta, mask, npix, C, g, t);
    } else {
        const int g = lanes_per_pixel(C);
        launch_pdl(k_sparsify<T, 1>, pixel_grid(npix, g), dim3(256), 0, st, x, prev, delta, mask, npix, C, g, t);
    }
    return check_launch();
}

template <typename T>
static int act_trunc_t(T* delta, T* prev, T* trunc, int32_t* mask, int64_t npix, int C, float thr, int act, int mode,
                       cudaStream_t st) {
    constexpr int V = VecTraits<T>::kVec;
    const int W = pick_w<T>(C, {delta, prev, trunc});
    const float t = host_round_threshold<T>(thr);
    if (W == V) {
        const int nvec = C / V;
        const int g = lanes_per_pixel(nvec);
        const int per_lane = divup(nvec, g);
        dim3 grid = pixel_grid(npix, g);
        const bool fast = sizeof(T) == 2 && mode == DC_TRUNC_MAX && act >= DC_ACT_NONE && act <= DC_ACT_RELU6;
#define DC_AT(NV)                                                                                                                        \
    do {                                                                                                                                 \
        if (fast) launch_pdl(k_act_trunc<T, V, NV, true>, grid, dim3(256), 0, st, delta, prev, trunc, mask, npix, C, g, t, act, mode);  \
        else launch_pdl(k_act_trunc<T, V, NV, false>, grid, dim3(256), 0, st, delta, prev, trunc, mask, npix, C, g, t, act, mode);      \
    } while (0)
        if (per_lane <= 1) DC_AT(1);
        else if (per_lane <= 2) DC_AT(2);
        else if (per_lane <= 4) DC_AT(4);
        else if (per_lane <= 8) DC_AT(8);
        else DC_AT(0);
#undef DC_AT
    } else {
        const int g = lanes_per_pixel(C);
        dim3 grid = pixel_grid(npix, g);
        if (divup(C, g) <= 4) launch_pdl(k_act_trunc<T, 1, 4>, grid, dim3(256), 0, st, delta, prev, trunc, mask, npix, C, g, t, act, mode);
        else launch_pdl(k_act_trunc<T, 1, 0>, grid, dim3(256), 0, st, delta, prev, trunc, mask, npix, C, g, t, act, mode);
    }
    return check_launch();
}

#define DC_DISPATCH_W(T, C, ptrs, KERNEL, npix_, ...)                                         \
    do {                                                                                      \
        constexpr int V = VecTraits<T>::kVec;                                                 \
        if (pick_w<T>(C, ptrs) == V) {                                                        \
            const int g = lanes_per_pixel((C) / V);                                           \
            launch_pdl(KERNEL<T, V>, pixel_grid(npix_, g), dim3(256), 0, st, __VA_ARGS__, g);               \
        } else {                                                                              \
            const int g = lanes_per_pixel(C);                                                 \
            launch_pdl(KERNEL<T, 1>, pixel_grid(npix_, g), dim3(256), 0, st, __VA_ARGS__, g);               \
        }                                                                                     \
    } while (0)

}  // namespace dc

using namespace dc;

#define DC_PTRS(...) std::initializer_list<const void*>{__VA_ARGS__}

extern "C" {

int dc_sparsify(const void* x, void* prev_in, void* delta, int32_t* mask, int64_t npix, int32_t channels, int32_t dtype,
                float threshold, void* stream) {
    if (npix < 0 || channels <= 0) return DC_ERR_SHAPE;
    if (npix == 0) return DC_OK;
    DC_REQUIRE(x); DC_REQUIRE(prev_in); DC_REQUIRE(delta); DC_REQUIRE(mask);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DC_F32) return sparsify_t<float>((const float*)x, (float*)prev_in, (float*)delta, mask, npix, channels, threshold, st);
    if (dtype == DC_F16) return sparsify_t<__half>((const __half*)x, (__half*)prev_in, (__half*)delta, mask, npix, channels, threshold, st);
    return DC_ERR_DTYPE;
}

int dc_sparsify_u8(const uint8_t* x_u8, const float* scale, const float* offset, void* prev_in, void* delta, int32_t* mask,
                   int64_t npix, int32_t channels, int32_t dtype, float threshold, void* stream) {
    if (npix < 0 || channels <= 0) return DC_ERR_SHAPE;
    if (npix == 0) return DC_OK;
    DC_REQUIRE(x_u8); DC_REQUIRE(scale); DC_REQUIRE(offset); DC_REQUIRE(prev_in); DC_REQUIRE(delta); DC_REQUIRE(mask);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype != DC_F32 && dtype != DC_F16) return DC_ERR_DTYPE;
    const int g = lanes_per_pixel(channels);
    const float thr16 = host_round_threshold<__half>(threshold);
    int64_t done = 0;
    if (channels == 3 && (reinterpret_cast<uintptr_t>(x_u8) & 3u) == 0 && aligned16(prev_in) && aligned16(delta) && aligned16(mask)) {
        // RGB frames: runs of 8 (fp16) or 4 (fp32) pixels per thread with vector accesses; the generic kernel takes the ragged tail
        const int ppt = dtype == DC_F16 ? 8 : 4;
        const int64_t ngroups = npix / ppt;
        if (ngroups > 0) {
            int64_t blocks = divup64(ngroups, 256);
            const int64_t cap = (int64_t)sm_count() * 16;
            if (blocks > cap) blocks = cap;
            if (dtype == DC_F32)
                launch_pdl(k_sparsify_u8_c3<float>, (unsigned)blocks, dim3(256), 0, st, x_u8, scale, offset, (float*)prev_in, (float*)delta, mask, npix, threshold);
            else
                launch_pdl(k_sparsify_u8_c3<__half>, (unsigned)blocks, dim3(256), 0, st, x_u8, scale, offset, (__half*)prev_in, (__half*)delta, mask, npix, thr16);
        }
        done = ngroups * ppt;
        if (done == npix) return check_launch();
    }
    const int64_t rest = npix - done;
    if (dtype == DC_F32)
        launch_pdl(k_sparsify_u8<float>, pixel_grid(rest, g), dim3(256), 0, st, x_u8 + done * channels, scale, offset, (float*)prev_in + done * channels,
                   (float*)delta + done * channels, mask + done, rest, channels, g, threshold);
    else
        launch_pdl(k_sparsify_u8<__half>, pixel_grid(rest, g), dim3(256), 0, st, x_u8 + done * channels, scale, offset, (__half*)prev_in + done * channels,
                   (__half*)delta + done * channels, mask + done, rest, channels, g, thr16);
    return check_launch();
}

int dc_sparsify_dilated(const void* x, void* prev_in, void* delta, int32_t* mask, uint8_t* hit_scratch, int32_t n, int32_t h,
                        int32_t w, int32_t channels, int32_t dtype, float threshold, int32_t dilation, void* stream) {
    if (n < 0 || h <= 0 || w <= 0 || channels <= 0) return DC_ERR_SHAPE;
    if (dilation < 1 || dilation % 2 == 0 || (dilation - 1) / 2 > kDilMaxR) return DC_ERR_UNSUPPORTED;   // odd windows up to 33
    if (n == 0) return DC_OK;
    DC_REQUIRE(x); DC_REQUIRE(prev_in); DC_REQUIRE(delta); DC_REQUIRE(mask); DC_REQUIRE(hit_scratch);
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t npix = (int64_t)n * h * w;
    int64_t blocks = divup64(npix, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    const dim3 tiles((unsigned)divup(w, kDilTileW), (unsigned)divup(h, kDilTileH), (unsigned)n);
    const int r = (dilation - 1) / 2;
    int rc;
    if (dtype == DC_F32) {
        rc = launch_pdl(k_sparsify_hit<float>, dim3((unsigned)blocks), dim3(256), 0, st, (const float*)x, (const float*)prev_in, (float*)delta, hit_scratch, npix, channels, threshold);
        if (rc != DC_OK) return rc;
        return launch_pdl(k_sparsify_dilate<float>, tiles, dim3(256), 0, st, (const float*)x, (float*)prev_in, (const uint8_t*)hit_scratch, mask, h, w, channels, r);
    }
    if (dtype == DC_F16) {
        rc = launch_pdl(k_sparsify_hit<__half>, dim3((unsigned)blocks), dim3(256), 0, st, (const __half*)x, (const __half*)prev_in, (__half*)delta, hit_scratch, npix, channels, host_round_threshold<__half>(threshold));
        if (rc != DC_OK) return rc;
        return launch_pdl(k_sparsify_dilate<__half>, tiles, dim3(256), 0, st, (const __half*)x, (__half*)prev_in, (const uint8_t*)hit_scratch, mask, h, w, channels, r);
    }
    return DC_ERR_DTYPE;
}

int dc_activate_truncate(void* delta, void* prev_out, void* truncated, int32_t* mask, int64_t npix, int32_t channels,
                         int32_t dtype, float threshold, int32_t activation, int32_t truncation, void* stream) {
    if (npix < 0 || channels <= 0) return DC_ERR_SHAPE;
    if (npix == 0) return DC_OK;
    DC_REQUIRE(delta); DC_REQUIRE(prev_out); DC_REQUIRE(mask);
    if (truncation >= 0) DC_REQUIRE(truncated);
    if (truncation > DC_TRUNC_RMS) return DC_ERR_UNSUPPORTED;
    if (activation > DC_ACT_SWISH) return DC_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DC_F32) return act_trunc_t<float>((float*)delta, (float*)prev_out, (float*)truncated, mask, npix, channels, threshold, activation, truncation, st);
    if (dtype == DC_F16) return act_trunc_t<__half>((__half*)delta, (__half*)prev_out, (__half*)truncated, mask, npix, channels, threshold, activation, truncation, st);
    return DC_ERR_DTYPE;
}

int dc_add(const void* a, const void* b, void* prev_out, void* out, const int32_t* mask_a, const int32_t* mask_b,
           int32_t* mask_out, float weight_a, float weight_b, int64_t npix, int32_t channels, int32_t dtype,
           int32_t activation, int32_t dense_out, void* stream) {
    if (npix < 0 || channels <= 0) return DC_ERR_SHAPE;
    if (npix == 0) return DC_OK;
    DC_REQUIRE(a); DC_REQUIRE(b); DC_REQUIRE(out); DC_REQUIRE(mask_a); DC_REQUIRE(mask_b);
    if (!dense_out) DC_REQUIRE(mask_out);
    if (dense_out || activation > 0) DC_REQUIRE(prev_out);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DC_F32)
        DC_DISPATCH_W(float, channels, DC_PTRS(a, b, prev_out, out), k_add, npix, (const float*)a, (const float*)b,
                      (float*)prev_out, (float*)out, mask_a, mask_b, mask_out, weight_a, weight_b, npix, channels,
                      activation, dense_out);
    else if (dtype == DC_F16)
        DC_DISPATCH_W(__half, channels, DC_PTRS(a, b, prev_out, out), k_add, npix, (const __half*)a, (const __half*)b,
                      (__half*)prev_out, (__half*)out, mask_a, mask_b, mask_out, weight_a, weight_b, npix, channels,
                      activation, dense_out);
    else return DC_ERR_DTYPE;
    return check_launch();
}

int dc_add_to_dense(const void* a, void* b, const int32_t* mask_a, int64_t npix, int32_t channels, int32_t dtype,
                    void* stream) {
    if (npix < 0 || channels <= 0) return DC_ERR_SHAPE;
    if (npix == 0) return DC_OK;
    DC_REQUIRE(a); DC_REQUIRE(b); DC_REQUIRE(mask_a);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DC_F32)
        DC_DISPATCH_W(float, channels, DC_PTRS(a, b), k_add_to_dense, npix, (const float*)a, (float*)b, mask_a, npix, channels);
    else if (dtype == DC_F16)
        DC_DISPATCH_W(__half, channels, DC_PTRS(a, b), k_add_to_dense, npix, (const __half*)a, (__half*)b, mask_a, npix, channels);
    else return DC_ERR_DTYPE;
    return check_launch();
}

int dc_scale_bias(const void* in, const int32_t* mask_in, void* out, int32_t* mask_out, const void* scale,
                  const void* bias, int64_t npix, int32_t channels, int32_t dtype, void* stream) {
    if (npix < 0 || channels <= 0) return DC_ERR_SHAPE;
    if (npix == 0) return DC_OK;
    DC_REQUIRE(in); DC_REQUIRE(out); DC_REQUIRE(scale);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DC_F32)
        DC_DISPATCH_W(float, channels, DC_PTRS(in, out, scale, bias), k_scale_bias, npix, (const float*)in, mask_in,
                      (float*)out, mask_out, (const float*)scale, (const float*)bias, npix, channels);
    else if (dtype == DC_F16)
        DC_DISPATCH_W(__half, channels, DC_PTRS(in, out, scale, bias), k_scale_bias, npix, (const __half*)in, mask_in,
                      (__half*)out, mask_out, (const __half*)scale, (const __half*)bias, npix, channels);
    else return DC_ERR_DTYPE;
    return check_launch();
}

int dc_concat(const void* a, const void* b, void* out, const int32_t* mask_a, const int32_t* mask_b, int32_t* mask_out,
              int64_t npix, int32_t channels_a, int32_t channels_b, int32_t dtype, void* stream) {
    if (npix < 0 || channels_a <= 0 || channels_b <= 0) return DC_ERR_SHAPE;
    if (npix == 0) return DC_OK;
    DC_REQUIRE(a); DC_REQUIRE(b); DC_REQUIRE(out); DC_REQUIRE(mask_a); DC_REQUIRE(mask_b); DC_REQUIRE(mask_out);
    cudaStream_t st = (cudaStream_t)stream;
    const int ctot = channels_a + channels_b;
    // the vector path needs both halves to be whole packs
    if (dtype == DC_F32) {
        const int cc = (channels_a % 4 == 0 && channels_b % 4 == 0) ? ctot : 1;
        if (cc == 1) { const int g = lanes_per_pixel(ctot); launch_pdl(k_concat<float, 1>, pixel_grid(npix, g), dim3(256), 0, st, (const float*)a, (const float*)b, (float*)out, mask_a, mask_b, mask_out, npix, channels_a, channels_b, g); }
        else DC_DISPATCH_W(float, ctot, DC_PTRS(a, b, out), k_concat, npix, (const float*)a, (const float*)b, (float*)out, mask_a, mask_b, mask_out, npix, channels_a, channels_b);
    } else if (dtype == DC_F16) {
        const int cc = (channels_a % 8 == 0 && channels_b % 8 == 0) ? ctot : 1;
        if (cc == 1) { const int g = lanes_per_pixel(ctot); launch_pdl(k_concat<__half, 1>, pixel_grid(npix, g), dim3(256), 0, st, (const __half*)a, (const __half*)b, (__half*)out, mask_a, mask_b, mask_out, npix, channels_a, channels_b, g); }
        else DC_DISPATCH_W(__half, ctot, DC_PTRS(a, b, out), k_concat, npix, (const __half*)a, (const __half*)b, (__half*)out, mask_a, mask_b, mask_out, npix, channels_a, channels_b);
    } else return DC_ERR_DTYPE;
    return check_launch();
}

int dc_densify(const void* delta, const int32_t* mask, void* prev_out, void* dense_out, int64_t npix, int32_t channels,
               int32_t dtype, int32_t activation, void* stream) {
    if (npix < 0 || channels <= 0) return DC_ERR_SHAPE;
    if (npix == 0) return DC_OK;
    DC_REQUIRE(delta); DC_REQUIRE(mask); DC_REQUIRE(prev_out);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DC_F32)
        DC_DISPATCH_W(float, channels, DC_PTRS(delta, prev_out, dense_out), k_densify, npix, (const float*)delta, mask,
                      (float*)prev_out, (float*)dense_out, npix, channels, activation);
    else if (dtype == DC_F16)
        DC_DISPATCH_W(__half, channels, DC_PTRS(delta, prev_out, dense_out), k_densify, npix, (const __half*)delta, mask,
                      (__half*)prev_out, (__half*)dense_out, npix, channels, activation);
    else return DC_ERR_DTYPE;
    return check_launch();
}

int dc_upsample(const void* in, const int32_t* mask_in, void* out, int32_t* mask_out, int32_t n, int32_t h, int32_t w,
                int32_t channels, int32_t scale, int32_t dtype, void* stream) {
    if (n < 0 || h <= 0 || w <= 0 || channels <= 0 || scale <= 0) return DC_ERR_SHAPE;
    if (n == 0) return DC_OK;
    DC_REQUIRE(in); DC_REQUIRE(mask_in); DC_REQUIRE(out); DC_REQUIRE(mask_out);
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t npix = (int64_t)n * h * scale * w * scale;
    if (dtype == DC_F32)
        DC_DISPATCH_W(float, channels, DC_PTRS(in, out), k_upsample, npix, (const float*)in, mask_in, (float*)out, mask_out, n, h, w, channels, scale);
    else if (dtype == DC_F16)
        DC_DISPATCH_W(__half, channels, DC_PTRS(in, out), k_upsample, npix, (const __half*)in, mask_in, (__half*)out, mask_out, n, h, w, channels, scale);
    else return DC_ERR_DTYPE;
    return check_launch();
}

int dc_compact_mask(const int32_t* mask, int64_t npix, int32_t* indices, int32_t* count, void* stream) {
    DC_REQUIRE(mask); DC_REQUIRE(indices); DC_REQUIRE(count);
    if (npix < 0 || npix > 0x7fffffffLL) return DC_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(count, 0, sizeof(int32_t), st) != cudaSuccess) return check_launch();
    if (npix == 0) return DC_OK;
    int64_t blocks = divup64(npix, 256);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    launch_pdl(k_compact_mask, dim3((unsigned)blocks), dim3(256), 0, st, mask, npix, indices, count);
    return check_launch();
}

}  // extern "C"
