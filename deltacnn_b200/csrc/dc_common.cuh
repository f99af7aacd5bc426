// Shared device helpers for the delta-update kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "deltacnn_b200.h"

#define DC_WARP 32
#define DC_FULL 0xffffffffu

namespace dc {

__host__ __device__ constexpr inline int64_t divup64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ constexpr inline int divup(int a, int b) { return (a + b - 1) / b; }

// n / d for n < 2^31 with (mul, shift) from fast_div_init(d): exact, no division instruction sequence.
__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint32_t mul, uint32_t shift) {
    return (uint32_t)(((uint64_t)n * mul) >> shift);
}
inline void fast_div_init(uint32_t d, uint32_t* mul, uint32_t* shift) {
    uint32_t s = 0;
    while ((1ull << s) < d) ++s;
    *mul = (uint32_t)((((uint64_t)1 << (31 + s)) + d - 1) / d);   // ceil(2^(31+s) / d) < 2^32
    *shift = 31 + s;
}

// Number of SMs of the current device (cached per thread), for grid sizing.
int sm_count();
// Record a launch failure for dc_last_cuda_error(); returns DC_OK or DC_ERR_LAUNCH.
int check_launch();

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
// Value of x after a round trip through the storage type.
template <typename T> __device__ __forceinline__ float rnd(float x) { return to_f<T>(from_f<T>(x)); }

// Elements of T in one 16-byte vector.
template <typename T> struct VecTraits { static constexpr int kVec = 16 / (int)sizeof(T); };

// W consecutive elements of T held in storage precision: W == VecTraits<T>::kVec is
// one 16-byte access, W == 1 is the scalar fallback for channel counts whose pixel
// stride is not a multiple of 16 bytes.
template <typename T, int W> struct Pack {
    alignas(W * sizeof(T) == 16 ? 16 : alignof(T)) T s[W];
    __device__ __forceinline__ void load(const T* p) {
        if constexpr (W * sizeof(T) == 16) {
            *reinterpret_cast<uint4*>(s) = *reinterpret_cast<const uint4*>(p);
        } else {
#pragma unroll
            for (int i = 0; i < W; ++i) s[i] = p[i];
        }
    }
    __device__ __forceinline__ void store(T* p) const {
        if constexpr (W * sizeof(T) == 16) {
            *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(s);
        } else {
#pragma unroll
            for (int i = 0; i < W; ++i) p[i] = s[i];
        }
    }
    __device__ __forceinline__ float get(int i) const { return to_f<T>(s[i]); }
    __device__ __forceinline__ void set(int i, float x) { s[i] = from_f<T>(x); }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < W; ++i) s[i] = from_f<T>(0.f);
    }
};

__device__ __forceinline__ float act_apply(float x, int code) {
    switch (code) {
        case DC_ACT_RELU: return fmaxf(x, 0.f);
        case DC_ACT_RELU6: return fminf(fmaxf(x, 0.f), 6.f);
        case DC_ACT_LEAKY: return x < 0.f ? 0.1f * x : x;
        case DC_ACT_SIGMOID: return 1.f / (1.f + __expf(-x));
        case DC_ACT_SWISH: return x / (1.f + __expf(-x));
        default: return x;
    }
}

// Activations whose value at a half-precision argument is itself a half: their deltas can be formed in
// packed half arithmetic without changing a bit (identity, ReLU, ReLU6).
__device__ __forceinline__ bool act_exact_in_half(int code) { return code >= DC_ACT_NONE && code <= DC_ACT_RELU6; }

// Accumulate + activation delta + threshold test of one 16-byte pack of fp16 channels.
//   in:  d = incoming delta, y = accumulated pre-activation value, tr = carried residual
//   out: tr = residual + delta, y = y + tr, d = f(y_new) - f(y_old); returns |d| > thr for any channel.
// Packed-half form: adding or subtracting two halves in fp32 and rounding once gives the correctly rounded
// half result, max and min are exact, so this equals truncate_pack_f32 bit for bit for the activations of
// act_exact_in_half at a fifth of the instructions.
__device__ __forceinline__ bool truncate_pack_h2(Pack<__half, 8>& d, Pack<__half, 8>& y, Pack<__half, 8>& tr, int act, __half2 thr2) {
    __half2* dh = reinterpret_cast<__half2*>(d.s);
    __half2* yh = reinterpret_cast<__half2*>(y.s);
    __half2* th = reinterpret_cast<__half2*>(tr.s);
    const __half2 zero = __float2half2_rn(0.f), six = __float2half2_rn(6.f);
    unsigned any = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const __half2 r = __hadd2(th[k], dh[k]);
        const __half2 yo = yh[k];
        const __half2 u = __hadd2(yo, r);
        __half2 fu = u, fy = yo;
        if (act != DC_ACT_NONE) {
            fu = __hmax2(fu, zero);
            fy = __hmax2(fy, zero);
            if (act == DC_ACT_RELU6) {
                fu = __hmin2(fu, six);
                fy = __hmin2(fy, six);
            }
        }
        const __half2 e = __hsub2(fu, fy);
        th[k] = r;
        yh[k] = u;
        dh[k] = e;
        any |= __hgt2_mask(__habs2(e), thr2);
    }
    return any != 0;
}
// The same step in fp32 with one rounding per stored value, for every activation and storage type.
template <typename T, int W>
__device__ __forceinline__ bool truncate_pack_f32(Pack<T, W>& d, Pack<T, W>& y, Pack<T, W>& tr, int act, float thr) {
    bool hit = false;
#pragma unroll
    for (int k = 0; k < W; ++k) {
        const float yo = y.get(k);
        const float rr = rnd<T>(tr.get(k) + d.get(k));
        const float uu = rnd<T>(yo + rr);
        const float ee = rnd<T>(act_apply(uu, act) - act_apply(yo, act));
        tr.set(k, rr);
        y.set(k, uu);
        d.set(k, ee);
        hit |= fabsf(ee) > thr;
    }
    return hit;
}

// Threshold as the storage type sees it (the half kernels compare against the
// threshold rounded to half).
template <typename T> inline float host_round_threshold(float t);
template <> inline float host_round_threshold<float>(float t) { return t; }
template <> inline float host_round_threshold<__half>(float t) { return __half2float(__float2half_rn(t)); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Lanes cooperating on one pixel: smallest power of two >= nvec, capped at 32.
inline int lanes_per_pixel(int nvec) {
    int g = 1;
    while (g < nvec && g < 32) g <<= 1;
    return g;
}

// OR-reduce a predicate over an aligned group of `g` lanes (g power of two <= 32).
__device__ __forceinline__ bool group_any(bool p, int g, int lane) {
    unsigned b = __ballot_sync(DC_FULL, p);
    if (g == 32) return b != 0;
    unsigned base = (unsigned)(lane & ~(g - 1));
    unsigned gm = ((1u << g) - 1u) << base;
    return (b & gm) != 0;
}

// Programmatic dependent launch: a kernel launched through launch_pdl may start while the previous kernel on
// the stream is still draining; everything it does before grid_dep_wait() (shared-memory set-up, loading
// constant filters) overlaps that tail, everything that reads the previous kernel's results comes after it.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// DC_NO_PDL=1 in the environment turns programmatic dependent launch off (plain stream order).
bool pdl_enabled();

// "Done once" flags for set-up that the CUDA runtime keeps per device (function attributes such as the dynamic
// shared-memory limit): slot() is the flag of the current device, or nullptr when the device cannot be queried.
struct PerDeviceOnce {
    bool done[64] = {};
    bool* slot() {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
        return &done[dev];
    }
};

// cluster_y > 1 launches thread-block clusters of (1, cluster_y, 1) CTAs (grid.y must be a multiple of it).
template <typename... KArgs, typename... Args>
inline int launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster_y, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_y > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = (unsigned)cluster_y;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    return check_launch();
}

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    return launch_pdl_cluster(kernel, grid, block, smem, st, 1, args...);
}

// Sum-reduce over an aligned group of g lanes.
__device__ __forceinline__ float group_sum(float x, int g) {
    for (int o = g >> 1; o > 0; o >>= 1) x += __shfl_xor_sync(DC_FULL, x, o);
    return x;
}

}  // namespace dc
