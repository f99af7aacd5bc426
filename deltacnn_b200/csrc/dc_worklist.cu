// Active-pixel work list of a convolution: one light pass dilates the in-mask by the receptive field,
// writes the out-mask and appends every active output pixel (with the bit set of its active taps) to a
// compacted list in caller-provided scratch memory. The convolution kernels then size their work by the
// list (persistent CTAs pulling entries), so inactive regions cost one coalesced mask read and the active
// pixels are spread evenly over the SMs however they cluster in the image.
//
// Scratch layout (dc_conv_workspace_bytes): [0] int32 count, [4..16) padding, then npix_out uint32 pixel
// indices, then npix_out uint32 tap bit sets.
#include "dc_common.cuh"

namespace dc {

struct ScanParams {
    const int32_t* mi; int32_t* mo; int32_t* count; uint32_t* list; uint32_t* taps;
    int n, hi, wi, ho, wo, kh, kw, sh, sw, pt, pl, dh, dw;
    int defer_active;      // fused epilogue: the out-mask of active pixels is written by the epilogue
};

__global__ void __launch_bounds__(256) k_scan_conv_mask(ScanParams p) {
    __shared__ int s_warp[8];
    __shared__ int s_base;
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t npix = (uint32_t)p.n * p.ho * p.wo;
    for (uint32_t start = blockIdx.x * 256u; start < npix; start += gridDim.x * 256u) {
        const uint32_t q = start + threadIdx.x;
        unsigned bits = 0;
        if (q < npix) {
            const int ox = (int)(q % (uint32_t)p.wo);
            const uint32_t t = q / (uint32_t)p.wo;
            const int oy = (int)(t % (uint32_t)p.ho);
            const int b = (int)(t / (uint32_t)p.ho);
            const int32_t* m = p.mi + (int64_t)b * p.hi * p.wi;
            if (p.kh == 1 && p.kw == 1) {
                const int iy = oy * p.sh - p.pt, ix = ox * p.sw - p.pl;
                if (iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi && m[iy * p.wi + ix] != 0) bits = 1u;
            } else {
                for (int ky = 0; ky < p.kh; ++ky) {
                    const int iy = oy * p.sh - p.pt + ky * p.dh;
                    if (iy < 0 || iy >= p.hi) continue;
                    for (int kx = 0; kx < p.kw; ++kx) {
                        const int ix = ox * p.sw - p.pl + kx * p.dw;
                        if (ix < 0 || ix >= p.wi) continue;
                        if (m[iy * p.wi + ix] != 0) bits |= 1u << ((ky * p.kw + kx) & 31);
                    }
                }
            }
            if (!p.defer_active || bits == 0) p.mo[q] = bits != 0 ? 1 : 0;
        }
        const unsigned bal = __ballot_sync(DC_FULL, bits != 0);
        if (lane == 0) s_warp[warp] = __popc(bal);
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { const int c = s_warp[i]; s_warp[i] = tot; tot += c; }
            s_base = tot ? atomicAdd(p.count, tot) : 0;
        }
        __syncthreads();
        if (bits) {
            const int slot = s_base + s_warp[warp] + __popc(bal & ((1u << lane) - 1u));
            p.list[slot] = q;
            p.taps[slot] = bits;
        }
        __syncthreads();
    }
}

size_t conv_workspace_bytes(const dc_conv_desc* d) {
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    return 16 + (size_t)npix * 8;
}

// Fills the work list for `d`; taps beyond 32 per pixel are not representable (kernels up to 5x5).
int scan_conv_mask(const dc_conv_desc* d, const int32_t* mi, int32_t* mo, void* ws, size_t ws_bytes, int defer_active,
                   cudaStream_t st) {
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    if (ws == nullptr || ws_bytes < conv_workspace_bytes(d)) return DC_ERR_WORKSPACE;
    if (npix > 0x7fffffffLL || d->kh * d->kw > 32) return DC_ERR_UNSUPPORTED;
    ScanParams p{};
    p.mi = mi; p.mo = mo;
    p.count = reinterpret_cast<int32_t*>(ws);
    p.list = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(ws) + 16);
    p.taps = p.list + npix;
    p.n = d->n; p.hi = d->h_in; p.wi = d->w_in; p.ho = d->h_out; p.wo = d->w_out; p.kh = d->kh; p.kw = d->kw;
    p.sh = d->stride_h; p.sw = d->stride_w; p.pt = d->pad_top; p.pl = d->pad_left; p.dh = d->dil_h; p.dw = d->dil_w;
    p.defer_active = defer_active;
    if (cudaMemsetAsync(ws, 0, 16, st) != cudaSuccess) return check_launch();
    int64_t blocks = divup64(npix, 256);
    const int64_t cap = (int64_t)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    return launch_pdl(k_scan_conv_mask, dim3((unsigned)blocks), dim3(256), 0, st, p);
}

}  // namespace dc

namespace dc {

// Transposed convolution, stride 2, kernel 2m x 2m: an output pixel (oy, ox) belongs to the phase
// ((oy + pad) % 2, (ox + pad) % 2) and only the m x m taps of that phase reach it, from the input pixels
// ((oy + pad) / 2 - a, (ox + pad) / 2 - b). The active output pixels are listed per phase (four lists of
// npix_out entries each, four counters in the header), so that a tile of rows shares one tap set.
struct ScanDeconvParams {
    const int32_t* mi; int32_t* mo; int32_t* count; uint32_t* list; uint32_t* taps;
    int n, hi, wi, ho, wo, m, pt, pl;
    int defer_active;
};

__global__ void __launch_bounds__(256) k_scan_deconv_mask(ScanDeconvParams p) {
    __shared__ int s_warp[4][8];
    __shared__ int s_base[4];
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t npix = (uint32_t)p.n * p.ho * p.wo;
    for (uint32_t start = blockIdx.x * 256u; start < npix; start += gridDim.x * 256u) {
        const uint32_t q = start + threadIdx.x;
        unsigned bits = 0;
        int phase = 0;
        if (q < npix) {
            const int ox = (int)(q % (uint32_t)p.wo);
            const uint32_t t = q / (uint32_t)p.wo;
            const int oy = (int)(t % (uint32_t)p.ho);
            const int b = (int)(t / (uint32_t)p.ho);
            phase = ((oy + p.pt) & 1) * 2 + ((ox + p.pl) & 1);
            const int by = (oy + p.pt) >> 1, bx = (ox + p.pl) >> 1;
            const int32_t* m = p.mi + (int64_t)b * p.hi * p.wi;
            for (int a = 0; a < p.m; ++a) {
                const int iy = by - a;
                if (iy < 0 || iy >= p.hi) continue;
                for (int c = 0; c < p.m; ++c) {
                    const int ix = bx - c;
                    if (ix < 0 || ix >= p.wi) continue;
                    if (m[iy * p.wi + ix] != 0) bits |= 1u << (a * p.m + c);
                }
            }
            if (!p.defer_active || bits == 0) p.mo[q] = bits != 0 ? 1 : 0;
        }
        unsigned bal[4];
#pragma unroll
        for (int ph = 0; ph < 4; ++ph) {
            bal[ph] = __ballot_sync(DC_FULL, bits != 0 && phase == ph);
            if (lane == 0) s_warp[ph][warp] = __popc(bal[ph]);
        }
        __syncthreads();
        if (threadIdx.x < 4) {
            const int ph = threadIdx.x;
            int tot = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { const int c = s_warp[ph][i]; s_warp[ph][i] = tot; tot += c; }
            s_base[ph] = tot ? atomicAdd(p.count + ph, tot) : 0;
        }
        __syncthreads();
        if (bits) {
            const size_t slot = (size_t)phase * npix + s_base[phase] + s_warp[phase][warp] + __popc(bal[phase] & ((1u << lane) - 1u));
            p.list[slot] = q;
            p.taps[slot] = bits;
        }
        __syncthreads();
    }
}

size_t deconv_workspace_bytes(const dc_conv_desc* d) {
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    return 16 + (size_t)npix * 8 * 4;
}

int scan_deconv_mask(const dc_conv_desc* d, const int32_t* mi, int32_t* mo, void* ws, size_t ws_bytes, int defer_active,
                     cudaStream_t st) {
    const int64_t npix = (int64_t)d->n * d->h_out * d->w_out;
    if (ws == nullptr || ws_bytes < deconv_workspace_bytes(d)) return DC_ERR_WORKSPACE;
    if (npix > 0x3fffffffLL || d->stride_h != 2 || d->stride_w != 2 || d->kh != d->kw || d->kh % 2 != 0 || d->kh > 10) return DC_ERR_UNSUPPORTED;
    ScanDeconvParams p{};
    p.mi = mi; p.mo = mo;
    p.count = reinterpret_cast<int32_t*>(ws);
    p.list = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(ws) + 16);
    p.taps = p.list + 4 * npix;
    p.n = d->n; p.hi = d->h_in; p.wi = d->w_in; p.ho = d->h_out; p.wo = d->w_out; p.m = d->kh / 2; p.pt = d->pad_top; p.pl = d->pad_left;
    p.defer_active = defer_active;
    if (cudaMemsetAsync(ws, 0, 16, st) != cudaSuccess) return check_launch();
    int64_t blocks = divup64(npix, 256);
    const int64_t cap = (int64_t)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    return launch_pdl(k_scan_deconv_mask, dim3((unsigned)blocks), dim3(256), 0, st, p);
}

}  // namespace dc

// ---------------------------------------------------------------------------------------------
// Entry point for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------
// Some hosts of this library may not call cudaMalloc at all: a plugin that runs inside another
// application's fixed device-memory allotment, or a real-time loop that must stay away from the allocator
// (and its implicit synchronisation) once it has started. dc_conv2d_ws wants scratch memory for its work
// list; dc_conv2d_static keeps that scratch in the image of this library instead: a fixed array in device
// global memory that every GPU loading the library holds until the process exits.
namespace dc {

constexpr size_t kStaticWsBytes = 16 + 8u * 524288u;      // work lists of up to 524288 output pixels (4 MiB)
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];

// In host code `g_static_ws` is only a stand-in for the symbol; the device address has to be asked for,
// per device, with that device current.
static void* static_ws_address(int* err) {
    constexpr int kMaxDevices = 64;
    static void* cached[kMaxDevices] = {};
    *err = DC_OK;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { *err = DC_ERR_LAUNCH; return nullptr; }
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_ws) != cudaSuccess || ptr == nullptr) { (void)check_launch(); *err = DC_ERR_LAUNCH; return nullptr; }
        cached[dev] = ptr;
    }
    return cached[dev];
}

}  // namespace dc

extern "C" size_t dc_static_workspace_max_pixels(void) { return (dc::kStaticWsBytes - 16) / 8; }

extern "C" int dc_conv2d_static(const dc_conv_desc* desc, const void* in, const int32_t* mask_in, const void* filter,
                                int32_t filter_layout, const void* bias, void* out, int32_t* mask_out,
                                const dc_epilogue* epilogue, void* stream) {
    if (desc == nullptr) return DC_ERR_NULL_POINTER;
    const int64_t npix = (int64_t)desc->n * desc->h_out * desc->w_out;
    if (npix < 0) return DC_ERR_SHAPE;
    if ((uint64_t)npix > dc_static_workspace_max_pixels()) return DC_ERR_WORKSPACE;   // more output pixels than the built-in scratch holds
    int err = DC_OK;
    void* ws = dc::static_ws_address(&err);
    if (ws == nullptr) return err;
    return dc_conv2d_ws(desc, in, mask_in, filter, filter_layout, bias, out, mask_out, epilogue, ws, dc::kStaticWsBytes, stream);
}
