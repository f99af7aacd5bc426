// Tensor-core delta convolution for sm_100a: pointwise (1x1) layers as a gather-GEMM on
// tcgen05.mma with the accumulator in tensor memory.
//
//   rows (M = 128 per tile)   the ACTIVE output pixels of a span of consecutive pixels, compacted
//                             inside the CTA with warp ballots and a prefix over the warps
//   K                         input channels, streamed in blocks of 64 through a shared-memory ring;
//                             the gathered rows are written in the 128-byte-swizzled K-major layout
//                             the tensor core reads (inactive pixels are never loaded)
//   N                         output channels (<= 256 per CTA); the filter is pre-tiled on the device
//                             into the same swizzled layout, so a K block of it is one contiguous bulk
//                             copy (cp.async.bulk, completion on an mbarrier)
//   epilogue                  tcgen05.ld -> registers (+bias) -> fp16 staging tile in shared memory ->
//                             coalesced rows; optionally the activation/truncation step of
//                             dc_activate_truncate is applied here, so the convolution result never
//                             makes a round trip through HBM
//
// Roles inside a CTA of 8 warps: warps 0-6 gather rows (cp.async into the swizzled stage ring, running up to
// four K blocks ahead; a block is handed over through a "full" mbarrier once the copies have landed and a
// proxy fence has made them visible to the tensor core), one thread of warp 7 waits on those barriers and
// issues the MMAs, tcgen05.commit hands stages back ("empty" barriers); all 8 warps run the epilogue.
// The kernel is bound by instruction issue and dependent latency, not by bandwidth (few warps walk a long
// path once per tile), so the per-tile path is kept short: no integer division (multiply-shift with host
// constants), tap offsets tabulated once, and the truncation step in packed half arithmetic.
//
// Every wait on an mbarrier is bounded; a wait that gives up sets a sticky device-side error code
// (dc_umma_error) and the CTA frees its tensor memory and returns.
#include <cstdlib>
#include <cstring>
#include <cuda.h>          // CUtensorMap and its enums (the encoder is fetched through cudaGetDriverEntryPoint)
#include "dc_umma.cuh"

namespace dc {

__device__ int g_umma_error = 0;

constexpr int kStages = 4;           // shared-memory ring depth
#ifndef DC_KDELAY
#define DC_KDELAY 1
#endif
constexpr int kDelay = DC_KDELAY;    // a producer signals a K block after issuing kDelay more (copies in flight per thread)
constexpr int kPwThreads = 256;
constexpr int kPwWarps = kPwThreads / 32;
constexpr int kProducerWarps = kPwWarps - 1;                  // the last warp feeds the tensor core
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kRowStep = kProducerThreads / 8;                // rows between a producer thread's chunks
constexpr int kChunkPasses = (kRows + kRowStep - 1) / kRowStep;
constexpr uint32_t kRowHasResidual = 0x40000000u;   // bit of a row's tap word: the residual is active at this pixel
constexpr int kMsSpans = 8;                  // spans whose active pixels a persistent CTA compacts together
constexpr int64_t kListMinPixels = 40000;    // below this many output pixels 1x1 layers skip the work list

struct PwParams {
    const __half* in; const int32_t* mi; const uint8_t* wimg; const __half* bias;
    __half* out; int32_t* mo; __half* prev; __half* trunc;
    float thr; int act; int fused;
    const __half* res; const int32_t* res_mask;   // optional residual (delta, mask) added to a linear layer's result
    __half* res_prev; int res_act;                // ... followed by DCAdd's activation: accumulated sum and activation code
    int64_t npix_out;
    int hi, wi, ho, wo, sh, sw;
    int kh, kw, dh, dw, pt, pl;     // kernel geometry; taps = kh * kw (K runs tap-major, then input channels)
    int taps, ncb;                  // ncb = K blocks of 64 input channels per tap; nkb = taps * ncb
    int cin, cout;
    int nkb, bn, span, b_resident, tmem_cols, nslots;
    uint32_t b_kb_stride;           // bytes between consecutive K blocks of the packed filter
    const int32_t* wl_count;        // work-list mode (else nullptr): number of active output pixels
    const uint32_t* wl_list;        //   their indices
    const uint32_t* wl_taps;        //   and the bit sets of their active taps, written by k_scan_conv_mask
    int transposed;                 // transposed convolution with stride sh == sw: blockIdx.z = output phase,
    int m;                          //   m x m taps per phase (kh = m * stride); lists are per phase
    int64_t wl_stride;              //   entries between the per-phase list segments
    uint32_t hw_mul, hw_shift, wo_mul, wo_shift;   // division by h_out*w_out and by w_out (fast_div)
    int ms_rounds;                  // > 0: persistent CTAs over strided 128-pixel spans, kMsSpans of them per round
    int64_t ms_nspans;              //      number of 128-pixel spans of the output
    // patch mode (KxK, stride 1): a tile is a tw x th patch of output pixels (tw * th = 128), persistent CTAs walk the patches
    int patch_mode, patch_tw_log2, patch_px, patch_py;   // patches per image row / column
    int64_t npatches;
    uint32_t ppx_mul, ppx_shift, ppi_mul, ppi_shift;      // division by patch_px and by patch_px * patch_py (fast_div)
    int tma_rows;                   // 2: the tensor map is the 4-D input [n][h][w][c], box {64, tw, th, 1} (patch mode);  1: the kernel got a tensor map of the input as [pixels][channels] and may load whole spans with it
    uint32_t off_b, off_stage, off_list, off_misc, stage_pitch;
};

// ---- kernel -----------------------------------------------------------------------------------
// Shared memory: [ region 0: A stage ring, later reused as the epilogue staging tile ][ filter blocks ]
//                [ row lists ][ mbarriers, scalars, bias ]
// kFront selects how a CTA finds its rows: 0 = one contiguous span of a 1x1 layer, 3 = persistent CTAs over strided
// spans of a 1x1 layer, 1 = work list in global memory (KxK, strided, transposed), 2 = patches of a stride-1 KxK layer, 5 = patches of the
// input lattice of a stride-2 transposed layer.
// One instantiation per form keeps each kernel's code short: their speed depends on it.
// kExactAct: the fused activation is one of act_exact_in_half, so only the packed-half epilogue is compiled in.
// kEpi: 0 = plain store, 1 = fused truncation step, 2 = plain store with a residual added, 3 = residual and the add
// layer's activation.
template <int kFront, bool kExactAct, int kEpi>
__global__ void __launch_bounds__(kPwThreads, 3) k_pw_umma(const PwParams p, const __grid_constant__ CUtensorMap tmap_in) {
    constexpr bool kFused = kEpi == 1;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sStage = smem;                                        // aliases the A ring (dead once a tile's MMAs are done)
    uint8_t* sB = smem + p.off_b;
    int* s_out = reinterpret_cast<int*>(smem + p.off_list);        // [span] output pixel (relative) of every active row
    int* s_base = s_out + p.span;                                  // [span] input pixel of tap 0 of the row (may lie in the padding)
    uint32_t* s_tb = reinterpret_cast<uint32_t*>(s_base + p.span); // [span] bit set of the row's active taps
    int* s_toff = reinterpret_cast<int*>(s_tb + p.span);           // [32] input pixel of every tap relative to the base pixel
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_misc);
    // bars[0..kStages)            empty   (tcgen05.commit of the MMAs that read stage s)
    // bars[kStages..2*kStages)    full    (every producer warp's copies into stage s have landed)
    // bars[2*kStages..3*kStages)  b_full  (bulk copy of the filter block of stage s landed; [0]: the resident filter)
    // bars[3*kStages]             accum   (all MMAs of a tile done)
    uint32_t* s_u32 = reinterpret_cast<uint32_t*>(bars + 3 * kStages + 1);
    // s_u32[0] tmem base, [1] ok flag, [3..3+warps) warp totals
    float* s_bias = reinterpret_cast<float*>(s_u32 + 12);          // [bn]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar0 = smem_u32(bars);
    auto bar_empty = [&](int s) { return bar0 + 8u * s; };
    auto bar_full = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto bar_bfull = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
    const uint32_t bar_accum = bar0 + 8u * (3 * kStages);
    const uint32_t idesc = make_idesc(p.bn);

    const int n0 = blockIdx.y * p.bn;                              // first output channel of this CTA
    const int ncols = min(p.bn, p.cout - n0);                      // real output channels here
    const uint8_t* wimg = p.wimg + (size_t)blockIdx.y * p.bn * 128;   // this CTA's rows inside every K block
    // transposed convolution: this CTA's output phase (py, px) uses the taps ky = py + s*a, kx = px + s*b
    const bool transposed = kFront == 5 || (kFront == 1 && p.transposed != 0);
    const int ph_y = transposed ? (int)blockIdx.z / p.sw : 0, ph_x = transposed ? (int)blockIdx.z % p.sw : 0;
    auto filter_block = [&](int kb_) -> size_t {                  // K block of this CTA -> K block of the packed filter
        if (!transposed) return (size_t)kb_;
        const int j = kb_ / p.ncb, cb = kb_ - j * p.ncb;
        const int t = (ph_y + p.sh * (j / p.m)) * p.kw + ph_x + p.sw * (j % p.m);
        return (size_t)t * p.ncb + cb;
    };

    // ---- set-up that reads nothing the previous kernel wrote: overlaps that kernel's tail ----
    if (tid <= 3 * kStages) {
        // a "full" barrier takes one arrival per producer warp plus one of thread 0, which carries the byte count
        // when the rows of a block come from the copy engine (TMA) instead of the warps' own copies
        mbar_init(bar0 + 8u * tid, (tid >= kStages && tid < 2 * kStages) ? (uint32_t)(kProducerWarps + 1) : 1u);
        fence_barrier_init();
        if (tid == 0) s_u32[1] = 1;
    }
    for (int i = tid; i < p.bn; i += kPwThreads) s_bias[i] = (p.bias != nullptr && i < ncols) ? __half2float(p.bias[n0 + i]) : 0.f;
    if (warp == 0) tmem_alloc(smem_u32(&s_u32[0]), (uint32_t)p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // dependents are released only now: a CTA of the next kernel allocates tensor memory before its own
    // grid_dep_wait(), so it must never compete for columns with a CTA of this grid that is still waiting for its own
    grid_dep_launch();
    const uint32_t tmem_base = s_u32[0];
    auto leave = [&]() {                   // nothing to do for this CTA: give the tensor memory back
        __syncthreads();
        if (warp == 0) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    };
    grid_dep_wait();

    // ---- the rows of this CTA ----
    constexpr bool list_mode = kFront == 1;
    constexpr bool multi = kFront == 3;                               // span mode over several strided spans per CTA
    constexpr bool patch = kFront == 2 || kFront == 5;                             // KxK stride 1: persistent CTAs over patches of output pixels
    const int64_t q0 = (list_mode || multi || patch) ? 0 : (int64_t)blockIdx.x * p.span;
    int cnt = 0;
    bool dense_rows = false;          // span mode: rows = all pixels of the span, loaded by TMA
    if (list_mode) {
        cnt = p.wl_count[blockIdx.z];
        if ((int64_t)blockIdx.x * kRows >= cnt) { leave(); return; }   // persistent CTAs beyond the work
        if (tid < p.taps)                                           // input pixel of tap t relative to a row's base pixel
            s_toff[tid] = transposed ? -((tid / p.m) * p.wi + tid % p.m) : (tid / p.kw) * p.dh * p.wi + (tid % p.kw) * p.dw;
    } else if (multi) {
        if (tid == 0) s_toff[0] = 0;
    } else if (patch) {
        if (tid < p.taps) s_toff[tid] = transposed ? -((tid / p.m) * p.wi + tid % p.m) : (tid / p.kw) * p.dh * p.wi + (tid % p.kw) * p.dw;
    } else {
        // span mode (1x1 kernels, no padding): thread t owns pixel q0 + t; the active ones are compacted in
        // order with a ballot per warp and a prefix over the warp totals
        int pin = 0;
        bool on = false, ron = false;
        const int64_t q = q0 + tid;
        if (tid < p.span && q < p.npix_out) {
            if (p.sh == 1 && p.sw == 1) {
                pin = (int)q;
            } else {
                const uint32_t b = fast_div((uint32_t)q, p.hw_mul, p.hw_shift);
                const uint32_t r = (uint32_t)q - b * (uint32_t)(p.ho * p.wo);
                const uint32_t oy = fast_div(r, p.wo_mul, p.wo_shift);
                pin = (int)((b * p.hi + oy * p.sh) * p.wi + (r - oy * p.wo) * p.sw);
            }
            on = p.mi[pin] != 0;
            if constexpr (kEpi >= 2) ron = p.res_mask[q] != 0;
            if (blockIdx.y == 0 && (!kFused || !(on || ron))) p.mo[q] = (on || ron) ? 1 : 0;
        }
        const uint32_t tbw = (on ? 1u : 0u) | (ron ? kRowHasResidual : 0u);
        const unsigned bal = __ballot_sync(DC_FULL, tbw != 0u);
        if (lane == 0) s_u32[3 + warp] = (uint32_t)__popc(bal);
        if (tid == 0) s_toff[0] = 0;
        __syncthreads();
        int slot = __popc(bal & ((1u << lane) - 1u));
#pragma unroll
        for (int w = 0; w < kPwWarps; ++w) {
            const int c = (int)s_u32[3 + w];
            if (w < warp) slot += c;
            cnt += c;
        }
        if (cnt == 0) { leave(); return; }    // nothing active in this span
        // Mostly active span of a stride-1 layer: its pixels are consecutive rows of the input, so a tile is ONE tiled
        // TMA load per K block instead of a gather; every pixel of the span becomes a row, the inactive ones are
        // computed and dropped in the epilogue.
        const int span_valid = (int)min((int64_t)p.span, p.npix_out - q0);
        dense_rows = p.tma_rows != 0 && 2 * cnt >= span_valid;
        if (dense_rows) {
            cnt = span_valid;
            if (tid < span_valid) {
                s_out[tid] = tid;
                s_base[tid] = pin;
                s_tb[tid] = tbw;
            }
        } else if (tbw != 0u) {
            s_out[slot] = tid;
            s_base[slot] = pin;
            s_tb[slot] = tbw;
        }
    }

    const uint32_t b_block_bytes = (uint32_t)p.bn * 128u;
    const bool is_mma_warp = warp == kPwWarps - 1;
    volatile uint32_t* ok_flag = &s_u32[1];
    bool ok = true;

    // Producer threads (warps 0 .. kProducerWarps-1): thread t owns 16-byte chunk (t & 7) of the rows
    // (t >> 3) + kRowStep * j of every K block and copies it straight into the swizzled stage (cp.async, zero
    // fill for inactive or out-of-bounds taps and beyond the last input channel).
    const int chunk = tid & 7, row0 = tid >> 3;
    auto dst_off = [&](int j) {           // byte offset of this thread's chunk of its j-th row inside a swizzled stage
        const int r = row0 + kRowStep * j;
        return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
    };
    const uint32_t sA_u32 = smem_u32(sA);
    const int last_ksteps = (p.cin - (p.ncb - 1) * kKBlock + 15) >> 4;      // MMAs (K = 16) in the last channel block of a tap
    const int nse = p.nslots;
    // ring positions: producers fill (pslot, pwrap) and signal (sslot); the MMA thread consumes (mslot, mwrap).
    // The wrap counters give the mbarrier phases: use k of a slot completes phase k of its barriers.
    int pslot = 0, pwrap = 0, sslot = 0, mslot = 0, mwrap = 0;
    auto signal_block = [&]() {           // this thread's copies of the oldest unsignalled block have landed
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full(sslot));
        if (tid == 0) mbar_arrive(bar_full(sslot));       // the arrival that carries the byte count in TMA mode
        if (++sslot == nse) sslot = 0;
    };
    // epilogue geometry: an aligned group of g lanes per row, 16 bytes per lane
    const int nch = ncols >> 3;                                   // 16-byte packs per row
    int g = 1;
    while (g < nch && g < 32) g <<= 1;
    const int lig = lane & (g - 1), ppw = 32 / g;
    const __half2 thr2 = __float2half2_rn(p.thr);
    __syncthreads();                  // row lists complete

    const bool plain_1x1 = p.taps == 1 && p.sh == 1 && p.sw == 1 && p.pt == 0 && p.pl == 0 && !transposed;
    int tile = 0;                     // tiles processed by this CTA (the accumulator barrier's phase counts these)
    const int nrounds = multi ? p.ms_rounds : patch ? (int)((p.npatches - blockIdx.x + gridDim.x - 1) / gridDim.x) : 1;
    // patch mode: the origin of the current patch is kept in s_toff[28..30] (x0, y0, image) for the thread that issues the loads
    int carry = 0;                    // multi-span mode: rows of a partly filled tile, kept for the next round
    for (int round = 0; round < nrounds && ok; ++round) {
    if (multi) {
        // Large maps of 1x1 layers without a work list: a persistent CTA owns the spans blockIdx.x + j * gridDim.x
        // (so clustered active regions are dealt round-robin to all CTAs) and compacts the active pixels of kMsSpans
        // of them into one row list. All mask reads of a round are in flight together.
        if (tid == 0) s_u32[2] = (uint32_t)carry;
        __syncthreads();
        int64_t q4[4];
        bool valid4[4];
        uint32_t tb4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int v = tid + kPwThreads * i;                      // 0 .. kMsSpans * 128 - 1
            const int64_t sid = (int64_t)blockIdx.x + (int64_t)(round * kMsSpans + (v >> 7)) * gridDim.x;
            q4[i] = sid * kRows + (v & 127);
            valid4[i] = sid < p.ms_nspans && q4[i] < p.npix_out;
            tb4[i] = (valid4[i] && p.mi[valid4[i] ? q4[i] : 0] != 0) ? 1u : 0u;
            if constexpr (kEpi >= 2) {
                if (valid4[i] && p.res_mask[q4[i]] != 0) tb4[i] |= kRowHasResidual;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (valid4[i] && blockIdx.y == 0 && (!kFused || tb4[i] == 0u)) p.mo[q4[i]] = tb4[i] != 0u ? 1 : 0;
            const unsigned bal = __ballot_sync(DC_FULL, tb4[i] != 0u);
            int base = 0;
            if (lane == 0 && bal != 0u) base = (int)atomicAdd(&s_u32[2], (uint32_t)__popc(bal));
            base = __shfl_sync(DC_FULL, base, 0);
            if (tb4[i] != 0u) {
                const int slot = base + __popc(bal & ((1u << lane) - 1u));
                s_out[slot] = (int)q4[i];
                s_base[slot] = (int)q4[i];
                s_tb[slot] = tb4[i];
            }
        }
        __syncthreads();
        cnt = (int)s_u32[2];
        if (cnt == 0) continue;
    }
    if (patch) {
        // One patch of tw x th output pixels per round. Thread r < 128 looks at pixel r of the patch: ORs the in-mask
        // over the taps (the out-mask), and notes whether every tap inside the image is active. If that holds for the
        // whole patch the tile's rows are loaded by the copy engine, tap by tap (the delta tensor is only defined at
        // active pixels, so a patch with an inactive input pixel in its halo gathers its active rows instead).
        const uint32_t pid = (uint32_t)blockIdx.x + (uint32_t)round * gridDim.x;
        const uint32_t pb = fast_div(pid, p.ppi_mul, p.ppi_shift);
        const uint32_t prem = pid - pb * (uint32_t)(p.patch_px * p.patch_py);
        const uint32_t pyi = fast_div(prem, p.ppx_mul, p.ppx_shift);
        const int patch_b = (int)pb;
        const int patch_y0 = (int)pyi << (7 - p.patch_tw_log2);
        const int patch_x0 = (int)(prem - pyi * (uint32_t)p.patch_px) << p.patch_tw_log2;
        if (tid == 0) { s_toff[28] = patch_x0; s_toff[29] = patch_y0; s_toff[30] = patch_b; }
        // lattice point of this thread inside the patch. Convolution: the output pixel itself. Transposed convolution
        // (stride 2): the patch tiles the lattice (by, bx) = ((oy + pad) / 2, (ox + pad) / 2) of this CTA's output phase,
        // whose taps (a, c) read the input pixels (by - a, bx - c).
        const int ly = patch_y0 + (tid >> p.patch_tw_log2), lx = patch_x0 + (tid & ((1 << p.patch_tw_log2) - 1));
        const int oy = transposed ? 2 * ly + ph_y - p.pt : ly, ox = transposed ? 2 * lx + ph_x - p.pl : lx;
        const bool valid = tid < kRows && oy >= 0 && oy < p.ho && ox >= 0 && ox < p.wo;
        uint32_t tbw = 0u;
        bool all_in = true;
        const int in0 = transposed ? (patch_b * p.hi + ly) * p.wi + lx : (patch_b * p.hi + oy - p.pt) * p.wi + ox - p.pl;
        if (valid) {
            for (int t = 0; t < p.taps; ++t) {
                int iy, ix;
                if (transposed) {
                    const int a = t / p.m;
                    iy = ly - a; ix = lx - (t - a * p.m);
                } else {
                    const int ky = t / p.kw, kx = t - ky * p.kw;
                    iy = oy - p.pt + ky * p.dh; ix = ox - p.pl + kx * p.dw;
                }
                if (iy >= 0 && iy < p.hi && ix >= 0 && ix < p.wi) {
                    if (p.mi[in0 + s_toff[t]] != 0) tbw |= 1u << t;
                    else all_in = false;
                }
            }
        }
        const int q = (patch_b * p.ho + oy) * p.wo + ox;
        if constexpr (kEpi >= 2) {
            if (valid && p.res_mask[q] != 0) tbw |= kRowHasResidual;     // a row of its own even without active taps
        }
        if (valid && blockIdx.y == 0 && (!kFused || tbw == 0u)) p.mo[q] = tbw != 0u ? 1 : 0;
        if (tid == 0) s_u32[2] = 0u;
        const int n_active = __syncthreads_count(tbw != 0u);
        if (n_active == 0) continue;
        dense_rows = p.tma_rows == 2 && __syncthreads_and(!valid || all_in) != 0;
        if (dense_rows) {
            cnt = kRows;
            if (tid < kRows) {
                s_out[tid] = valid ? q : 0;
                s_base[tid] = in0;
                s_tb[tid] = valid ? tbw : 0u;
            }
        } else {
            const unsigned bal = __ballot_sync(DC_FULL, tbw != 0u);
            int base = 0;
            if (lane == 0 && bal != 0u) base = (int)atomicAdd(&s_u32[2], (uint32_t)__popc(bal));
            base = __shfl_sync(DC_FULL, base, 0);
            if (tbw != 0u) {
                const int slot = base + __popc(bal & ((1u << lane) - 1u));
                s_out[slot] = q;
                s_base[slot] = in0;
                s_tb[slot] = tbw;
            }
            cnt = n_active;
        }
        __syncthreads();
    }
    // only the last round runs a partly filled tile; before that the remainder waits for more rows
    const bool full_tiles_only = multi && round + 1 < nrounds;
    // span mode: the tiles of this CTA's own list; list mode: every gridDim.x-th tile of the global list
    const int tile_first = list_mode ? (int)blockIdx.x : 0;
    const int tile_step = list_mode ? (int)gridDim.x : 1;
    const int tiles_total = full_tiles_only ? cnt / kRows : (cnt + kRows - 1) / kRows;
    for (int tg = tile_first; tg < tiles_total && ok; tg += tile_step, ++tile) {
        const int cnt_t = min(kRows, cnt - tg * kRows);
        const int t0 = list_mode ? 0 : tg * kRows;                  // offset of the tile's rows in the shared lists
        if (list_mode) {
            __syncthreads();                                        // previous tile's epilogue has read the lists
            if (tid < cnt_t) {
                const size_t e_ = (size_t)blockIdx.z * p.wl_stride + (size_t)tg * kRows + tid;
                const uint32_t q = p.wl_list[e_];
                s_out[tid] = (int)q;
                s_tb[tid] = p.wl_taps[e_];
                int base = (int)q;
                if (!plain_1x1) {
                    const uint32_t b = fast_div(q, p.hw_mul, p.hw_shift);
                    const uint32_t rr = q - b * (uint32_t)(p.ho * p.wo);
                    const int oy = (int)fast_div(rr, p.wo_mul, p.wo_shift);
                    const int ox = (int)rr - oy * p.wo;
                    if (transposed) base = ((int)b * p.hi + ((oy + p.pt) >> 1)) * p.wi + ((ox + p.pl) >> 1);   // stride 2
                    else base = ((int)b * p.hi + oy * p.sh - p.pt) * p.wi + ox * p.sw - p.pl;
                }
                s_base[tid] = base;
            }
            __syncthreads();
        }

        if (!is_mma_warp && dense_rows) {
            // ---- the copy engine loads the tile's rows, a K block per request of thread 0; every producer warp
            //      still arrives once per block (after the stage is free), so the barriers count the same in both modes ----
            const int y0 = (int)q0 + s_out[t0];                        // first pixel of the tile (stride 1: pixel = input row)
            for (int kb = 0; kb < p.nkb; ++kb) {
                if (pwrap > 0 && !mbar_wait_warp(bar_empty(pslot), (uint32_t)((pwrap - 1) & 1), ok_flag)) {
                    *ok_flag = 0; atomicExch(&g_umma_error, 1);
                    break;
                }
                if (warp == 0 && elect_one()) {        // (elected lane of a converged warp: TMA operands in uniform registers)
                    mbar_expect_tx(bar_full(pslot), (uint32_t)kABytes);
                    if (patch) {
                        const int tap_ = kb / p.ncb, cb_ = kb - tap_ * p.ncb;
                        int cx, cy;
                        if (transposed) {
                            const int a = tap_ / p.m;
                            cx = s_toff[28] - (tap_ - a * p.m); cy = s_toff[29] - a;
                        } else {
                            const int ky = tap_ / p.kw, kx = tap_ - ky * p.kw;
                            cx = s_toff[28] - p.pl + kx * p.dw; cy = s_toff[29] - p.pt + ky * p.dh;
                        }
                        tma_load_patch(sA_u32 + (uint32_t)pslot * kABytes, &tmap_in, cb_ * kKBlock, cx, cy, s_toff[30], bar_full(pslot));
                    } else {
                        tma_load_rows(sA_u32 + (uint32_t)pslot * kABytes, &tmap_in, kb * kKBlock, y0, bar_full(pslot));
                    }
                    if (!p.b_resident) {
                        mbar_expect_tx(bar_bfull(pslot), b_block_bytes);
                        bulk_g2s(smem_u32(sB + (size_t)pslot * b_block_bytes), wimg + filter_block(kb) * p.b_kb_stride, b_block_bytes, bar_bfull(pslot));
                    }
                }
                if (lane == 0) mbar_arrive(bar_full(pslot));
                if (++pslot == nse) { pslot = 0; ++pwrap; }
                if (++sslot == nse) sslot = 0;
            }
        } else if (!is_mma_warp) {
            // ---- producers: run up to nse K blocks ahead of the tensor core; a block is signalled (full
            //      barrier, one arrival per warp) kDelay blocks after it was issued ----
            int rbase[kChunkPasses];
            uint32_t rtb[kChunkPasses];          // tap bit set of the row; bit 31 marks a row that exists
#pragma unroll
            for (int j = 0; j < kChunkPasses; ++j) {
                const int r = row0 + kRowStep * j;
                const bool v = r < cnt_t;
                rbase[j] = v ? s_base[t0 + r] : 0;
                rtb[j] = v ? (s_tb[t0 + r] | 0x80000000u) : 0u;
            }
            int tap = 0, cb = 0, toff = s_toff[0];
            for (int kb = 0; kb < p.nkb; ++kb) {
                if (pwrap > 0 && !mbar_wait_warp(bar_empty(pslot), (uint32_t)((pwrap - 1) & 1), ok_flag)) {
                    *ok_flag = 0; atomicExch(&g_umma_error, 1);
                    break;
                }
                const int kk = cb * kKBlock + chunk * 8;
                const int ksteps_ = cb == p.ncb - 1 ? last_ksteps : kKBlock / 16;
                if (chunk < ksteps_ * 2) {
                    const uint32_t dst0 = sA_u32 + (uint32_t)pslot * kABytes;
                    const bool in_k = kk < p.cin;
#pragma unroll
                    for (int j = 0; j < kChunkPasses; ++j) {
                        if (rtb[j] != 0u) {
                            const bool real = in_k && ((rtb[j] >> tap) & 1u) != 0u;
                            const __half* src = real ? p.in + (int64_t)(rbase[j] + toff) * p.cin + kk : p.in;
                            cp_async16(dst0 + dst_off(j), src, real ? 16u : 0u);
                        }
                    }
                }
                cp_async_commit();
                if (warp == 0 && !p.b_resident && elect_one()) {
                    mbar_expect_tx(bar_bfull(pslot), b_block_bytes);
                    bulk_g2s(smem_u32(sB + (size_t)pslot * b_block_bytes), wimg + filter_block(kb) * p.b_kb_stride, b_block_bytes, bar_bfull(pslot));
                }
                if (++pslot == nse) { pslot = 0; ++pwrap; }
                if (++cb == p.ncb) {
                    cb = 0;
                    if (++tap < p.taps) toff = s_toff[tap];
                }
                if (kb >= kDelay) {
                    cp_async_wait_group<kDelay>();
                    signal_block();
                }
            }
            if (kDelay >= 2 && p.nkb >= 2) { cp_async_wait_group<1>(); signal_block(); }
            cp_async_wait_group<0>();
            signal_block();
        } else {
            // ---- the tensor core's warp: warp-uniform control flow, one elected lane issues the MMAs and the commits
            //      (tcgen05.mma takes its operands from uniform registers; issued from a divergent single-lane loop every
            //      MMA cost ~200 cycles of issue time, under elect.sync ~35) ----
            if (tile == 0 && p.b_resident && elect_one()) {       // the whole filter slab of this CTA: one bulk copy per K block, one barrier
                mbar_expect_tx(bar_bfull(0), (uint32_t)p.nkb * b_block_bytes);
                for (int kb = 0; kb < p.nkb; ++kb)
                    bulk_g2s(smem_u32(sB + (size_t)kb * b_block_bytes), wimg + filter_block(kb) * p.b_kb_stride, b_block_bytes, bar_bfull(0));
            }
            __syncwarp();
            {
                const uint64_t ad0 = make_smem_desc(sA_u32);
                const uint64_t bd0 = make_smem_desc(smem_u32(sB));
                const uint32_t b_step = b_block_bytes >> 4;
                int cb = 0;
                bool got = true;
                for (int kb = 0; kb < p.nkb; ++kb) {
                    got = mbar_wait_warp(bar_full(mslot), (uint32_t)(mwrap & 1), ok_flag);
                    if (got) {
                        if (!p.b_resident) got = mbar_wait_warp(bar_bfull(mslot), (uint32_t)(mwrap & 1), ok_flag);
                        else if (tile == 0 && kb == 0) got = mbar_wait_warp(bar_bfull(0), 0u, ok_flag);
                    }
                    if (!got) { *ok_flag = 0; atomicExch(&g_umma_error, 2); break; }
                    tc_fence_after();
                    const int ksteps = cb == p.ncb - 1 ? last_ksteps : kKBlock / 16;
                    if (elect_one()) {
                        const uint64_t ad = ad0 + (uint64_t)((uint32_t)mslot * (kABytes >> 4));
                        const uint64_t bd = bd0 + (uint64_t)((uint32_t)(p.b_resident ? kb : mslot) * b_step);
                        if (ksteps == kKBlock / 16) {              // a full K block: constant offsets, no loop
#pragma unroll
                            for (int ks = 0; ks < kKBlock / 16; ++ks)
                                umma_f16(tmem_base, ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                        } else {
                            for (int ks = 0; ks < ksteps; ++ks)
                                umma_f16(tmem_base, ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                        }
                        umma_commit(bar_empty(mslot));
                    }
                    __syncwarp();
                    if (++mslot == nse) { mslot = 0; ++mwrap; }
                    if (++cb == p.ncb) cb = 0;
                }
                if (got && *ok_flag != 0 && elect_one()) umma_commit(bar_accum);
                __syncwarp();
            }
        }
        // every MMA of the tile has completed: the accumulator is final and the stage ring is free
        if (!mbar_wait_warp(bar_accum, (uint32_t)(tile & 1), ok_flag)) { *ok_flag = 0; atomicExch(&g_umma_error, 3); }
        __syncthreads();
        if (s_u32[1] == 0) { ok = false; break; }
        tc_fence_after();

        // ---- epilogue 1: tensor memory -> fp16 staging tile (row = TMEM lane) ----
        {
            const int quarter = warp & 3;                          // TMEM lanes a warp may read: 32 * (warp % 4) ...
            const int r = quarter * 32 + lane;
            uint8_t* srow = sStage + (size_t)r * p.stage_pitch;
#pragma unroll 1
            for (int c0 = (warp >> 2) * 16; c0 < p.bn; c0 += 16 * (kPwWarps / 4)) {
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

        // ---- epilogue 2: coalesced rows, kU row groups in flight per warp; optional accumulate +
        //      activation delta + any-channel truncation against the two caches ----
        {
            constexpr int kU = 2;
#pragma unroll 1
            for (int rb = warp * ppw * kU; rb < cnt_t; rb += kPwWarps * ppw * kU) {
                Pack<__half, 8> d[kU], y[kU], tr[kU];
                int64_t off[kU];
                bool mine[kU];
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const int r = rb + u * ppw + lane / g;
                    mine[u] = r < cnt_t && lig < nch && (!dense_rows || s_tb[t0 + r] != 0u);
                    off[u] = 0;
                    if (mine[u]) {
                        off[u] = (q0 + s_out[t0 + r]) * p.cout + n0 + lig * 8;
                        d[u].load(reinterpret_cast<const __half*>(sStage + (size_t)r * p.stage_pitch) + lig * 8);
                        if (kFused) {
                            y[u].load(p.prev + off[u]);
                            tr[u].load(p.trunc + off[u]);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    if (!kFused) {
                        if (mine[u]) {
                            if constexpr (kEpi >= 2) {             // linear layer with a residual connection
                                const uint32_t tbw = s_tb[t0 + rb + u * ppw + lane / g];
                                if ((tbw & 0x3fffffffu) == 0u) d[u].zero();   // the convolution is not active here (stale or zero-filled row)
                                if (tbw & kRowHasResidual) {
                                    Pack<__half, 8> rr;
                                    rr.load(p.res + off[u]);
                                    __half2* dh = reinterpret_cast<__half2*>(d[u].s);
                                    const __half2* rh = reinterpret_cast<const __half2*>(rr.s);
                                    if constexpr (kEpi == 2) {
#pragma unroll
                                        for (int k = 0; k < 4; ++k) dh[k] = __hadd2(dh[k], rh[k]);
                                    } else {
                                        // the add layer's own activation: s = a + b in fp32, u = round(y + s), out = f(u) - f(y)
                                        // (the arithmetic of dc_add, so the result is the same bit for bit)
                                        Pack<__half, 8> yy;
                                        yy.load(p.res_prev + off[u]);
#pragma unroll
                                        for (int k = 0; k < 8; ++k) {
                                            const float yo = yy.get(k);
                                            const float uu = rnd<__half>(yo + (d[u].get(k) + rr.get(k)));
                                            yy.set(k, uu);
                                            d[u].set(k, act_apply(uu, p.res_act) - act_apply(yo, p.res_act));
                                        }
                                        yy.store(p.res_prev + off[u]);
                                    }
                                } else if constexpr (kEpi == 3) {
                                    Pack<__half, 8> yy;
                                    yy.load(p.res_prev + off[u]);
#pragma unroll
                                    for (int k = 0; k < 8; ++k) {
                                        const float yo = yy.get(k);
                                        const float uu = rnd<__half>(yo + d[u].get(k));
                                        yy.set(k, uu);
                                        d[u].set(k, act_apply(uu, p.res_act) - act_apply(yo, p.res_act));
                                    }
                                    yy.store(p.res_prev + off[u]);
                                }
                            }
                            d[u].store(p.out + off[u]);
                        }
                        continue;
                    }
                    bool hit = false;
                    if (mine[u]) {
                        if constexpr (kExactAct) hit = truncate_pack_h2(d[u], y[u], tr[u], p.act, thr2);
                        else hit = truncate_pack_f32(d[u], y[u], tr[u], p.act, p.thr);
                    }
                    const bool active = group_any(hit, g, lane);
                    if (mine[u]) {
                        if (active) {
                            Pack<__half, 8> z; z.zero();
                            y[u].store(p.prev + off[u]);
                            d[u].store(p.out + off[u]);
                            z.store(p.trunc + off[u]);
                        } else {
                            tr[u].store(p.trunc + off[u]);
                        }
                    }
                    const int r = rb + u * ppw + lane / g;
                    if (r < cnt_t && lig == 0 && (!dense_rows || s_tb[t0 + r] != 0u)) p.mo[q0 + s_out[t0 + r]] = active ? 1 : 0;
                }
            }
        }
        __syncthreads();
        tc_fence_after();
    }
    if (full_tiles_only) {            // move the remainder to the front of the lists (source and destination do not overlap)
        carry = cnt - tiles_total * kRows;
        if (tiles_total > 0 && tid < carry) {
            const int src = tiles_total * kRows + tid;
            s_out[tid] = s_out[src];
            s_base[tid] = s_base[src];
            s_tb[tid] = s_tb[src];
        }
        __syncthreads();
    }
    }   // rounds

    // drain: copies in flight and every MMA that was issued have to finish before shared and tensor memory are released
    cp_async_wait_group<0>();
    if (!ok && tid == 0) {
        for (int s = 0; s < kStages; ++s) { (void)mbar_try_wait(bar_empty(s), 0); }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
}

// ---- filter packing ---------------------------------------------------------------------------
// HWIO (1,1,cin,cout) fp16 -> [K block][row = output channel, padded][64 K values], K-major, 128-byte
// swizzled per 8-row group. An N tile of any width (multiple of 16) is a contiguous run of rows inside
// every K block, so the launch can choose its N tiling without repacking.
__global__ void k_pack_pw(const __half* __restrict__ w, __half* __restrict__ img, int cin, int cout, int rows, int taps, int ncb) {
    const int64_t total = (int64_t)taps * ncb * rows * 64;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int e = (int)(i & 7);
        const int cpos = (int)((i >> 3) & 7);       // swizzled chunk position inside the 128-byte row
        const int64_t rowi = i >> 6;
        const int n = (int)(rowi % rows);
        const int kb = (int)(rowi / rows);          // K block = (tap, block of 64 input channels)
        const int tap = kb / ncb, cb = kb - tap * ncb;
        const int c = cpos ^ (n & 7);               // logical chunk stored at this position
        const int k = cb * 64 + c * 8 + e;          // input channel
        img[i] = (k < cin && n < cout) ? w[((int64_t)tap * cin + k) * cout + n] : __float2half(0.f);
    }
}

struct PwPlan {
    bool ok;
    int bn, ntiles, nkb, ncb, taps, rows, tmem_cols, b_resident, span, nslots;
    uint32_t off_b, off_stage, off_list, off_misc, stage_pitch;
    size_t smem, img_bytes;
};

static PwPlan plan_pw(const dc_conv_desc* d, int transposed = 0) {
    PwPlan pl{};
    pl.taps = d->kh * d->kw;
    pl.ok = d->dtype == DC_F16 && d->groups == 1 && pl.taps <= 25 && d->c_in % 8 == 0 && d->c_out % 8 == 0 &&
            d->c_in >= 16 && d->c_out >= 16;
    if (transposed)     // stride 2, kernel 2m x 2m, no dilation: four output phases of m x m taps each
        pl.ok = pl.ok && d->stride_h == 2 && d->stride_w == 2 && d->kh == d->kw && d->kh % 2 == 0 && d->dil_h == 1 && d->dil_w == 1;
    if (!pl.ok) return pl;
    pl.ncb = divup(d->c_in, kKBlock);
    pl.nkb = pl.taps * pl.ncb;
    pl.rows = divup(d->c_out, 256) * 256 + 256;     // room for a ragged last N tile of any width
    pl.img_bytes = (size_t)pl.nkb * pl.rows * 128;
    return pl;
}

// Launch-time choices: N tiling, span of pixels per CTA, shared-memory layout.
static void finish_plan(PwPlan& pl, const dc_conv_desc* d, int64_t npix_out, bool want_fused, bool list_mode, bool multi_span) {
    const int sms = sm_count();
    pl.ntiles = divup(d->c_out, 256);
    pl.bn = divup(divup(d->c_out, pl.ntiles), 16) * 16;
    // few pixels (deep layers): split the output channels over more CTAs, unless the fused epilogue
    // needs a pixel's whole channel vector in one CTA
    if (!(want_fused && pl.ntiles == 1)) {
        const int64_t pix_ctas = divup64(npix_out, 128);
        while (pix_ctas * pl.ntiles < 2 * sms && pl.bn > 32) {
            ++pl.ntiles;
            pl.bn = divup(divup(d->c_out, pl.ntiles), 16) * 16;
        }
        pl.ntiles = divup(d->c_out, pl.bn);
    }
    pl.tmem_cols = 32;
    while (pl.tmem_cols < pl.bn) pl.tmem_cols <<= 1;
    const size_t b_block = (size_t)pl.bn * 128;
    pl.b_resident = pl.nkb * b_block <= 64 * 1024 ? 1 : 0;
    pl.nslots = pl.nkb < kStages ? pl.nkb : kStages;
    const size_t b_bytes = (pl.b_resident ? pl.nkb : pl.nslots) * b_block;
    // spans small enough to give every SM several CTAs, large enough to fill an MMA tile when sparse
    int span = 256;                   // a thread of the CTA looks at one pixel of the span
    const int64_t want = (int64_t)sms * 6;
    while (span > 128 && divup64(npix_out, span) * pl.ntiles < want) span >>= 1;
    if (list_mode) span = kRows;      // the shared row lists hold one tile
    if (multi_span) span = kMsSpans * kRows + kRows;   // ... or the active pixels of a round of spans plus a carried remainder
    pl.span = span;
    pl.stage_pitch = (uint32_t)pl.bn * 2 + 16;
    const uint32_t ring = (uint32_t)pl.nslots * kABytes;
    const uint32_t staging = kRows * pl.stage_pitch;
    pl.off_stage = 0;
    pl.off_b = ((ring > staging ? ring : staging) + 1023) & ~1023u;
    pl.off_list = (pl.off_b + (uint32_t)b_bytes + 15) & ~15u;
    pl.off_misc = (pl.off_list + (3u * (uint32_t)span + 32u) * 4u + 15) & ~15u;
    pl.smem = pl.off_misc + 8 * (3 * kStages + 1) + 48 + 4 * (size_t)pl.bn + 1024 /* alignment slack */;
}

size_t filter_umma_bytes(const dc_conv_desc* d, int transposed) {
    PwPlan pl = plan_pw(d, transposed);
    return pl.ok ? pl.img_bytes : 0;
}

int pack_filter_umma(const dc_conv_desc* d, int transposed, const void* hwio, void* packed, cudaStream_t st) {
    PwPlan pl = plan_pw(d, transposed);
    if (!pl.ok) return DC_ERR_UNSUPPORTED;
    if (!aligned16(packed)) return DC_ERR_ALIGNMENT;
    const int64_t total = (int64_t)pl.img_bytes / 2;
    int64_t blocks = divup64(total, 256);
    if (blocks > 4096) blocks = 4096;
    k_pack_pw<<<(unsigned)blocks, 256, 0, st>>>((const __half*)hwio, (__half*)packed, d->c_in, d->c_out, pl.rows, pl.taps, pl.ncb);
    return check_launch();
}

int scan_conv_mask(const dc_conv_desc* d, const int32_t* mi, int32_t* mo, void* ws, size_t ws_bytes, int defer_active, cudaStream_t st);
int conv3x3_halo(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out, int32_t* mo,
                 const dc_epilogue* ep, uint32_t b_kb_stride, int* fused_out, cudaStream_t st);

int scan_deconv_mask(const dc_conv_desc* d, const int32_t* mi, int32_t* mo, void* ws, size_t ws_bytes, int defer_active, cudaStream_t st);

// Tensor map of the input seen as a matrix [pixels][channels] (fp16), box {64 channels, 128 pixels}, 128-byte
// swizzle: what tma_load_rows reads. The encoder lives in the driver; it is looked up once through the runtime.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static bool encode_rows_map(CUtensorMap* map, const void* in, int64_t npix_in, int cin) {
    static EncodeTiledFn fn = nullptr;
    static bool looked_up = false;
    if (!looked_up) {
        looked_up = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        else
            (void)cudaGetLastError();
    }
    if (fn == nullptr) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)cin, (cuuint64_t)npix_in};
    const cuuint64_t gstride[1] = {(cuuint64_t)cin * 2u};          // bytes between pixels: a multiple of 16 (cin % 8 == 0)
    const cuuint32_t box[2] = {(cuuint32_t)kKBlock, (cuuint32_t)kRows};
    const cuuint32_t estride[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(in), gdim, gstride, box, estride,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor map of the input as [n][h][w][c] (fp16), box {64 channels, tw, th, 1}, 128-byte swizzle: what tma_load_patch reads.
// ``box_c`` = channels per box: 64 (128-byte swizzle) or 32 (64-byte swizzle, rows of 64 bytes).
bool encode_patch_map(CUtensorMap* map, const void* in, const dc_conv_desc* d, int tw, int th, int box_c) {
    CUtensorMap rows_probe;
    if (!encode_rows_map(&rows_probe, in, (int64_t)d->n * d->h_in * d->w_in, d->c_in)) return false;   // looks the encoder up
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(ptr);
    const cuuint64_t c2 = (cuuint64_t)d->c_in * 2u;
    const cuuint64_t gdim[4] = {(cuuint64_t)d->c_in, (cuuint64_t)d->w_in, (cuuint64_t)d->h_in, (cuuint64_t)d->n};
    const cuuint64_t gstride[3] = {c2, c2 * (cuuint64_t)d->w_in, c2 * (cuuint64_t)d->w_in * (cuuint64_t)d->h_in};
    const cuuint32_t box[4] = {(cuuint32_t)box_c, (cuuint32_t)tw, (cuuint32_t)th, 1u};
    const cuuint32_t estride[4] = {1u, 1u, 1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(in), gdim, gstride, box, estride,
              CU_TENSOR_MAP_INTERLEAVE_NONE, box_c == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int conv_umma_impl(const dc_conv_desc* d, int transposed, const void* in, const int32_t* mi, const void* filt, const void* bias,
                          void* out, int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st) {
    PwPlan pl = plan_pw(d, transposed);
    if (!pl.ok || mi == nullptr || mo == nullptr) return DC_ERR_UNSUPPORTED;
    // without scratch for a work list only 1x1 kernels (no receptive field to dilate) have a tensor-core path
    // KxK stride 1 without scratch memory: persistent CTAs over patches of output pixels, no scan pass (with scratch the
    // work list is used: it fills every tile, which wins on sparse maps; patches win on mostly active maps).
    // DC_NO_PATCH=1 turns the patch form off.
    static const bool patch_allowed = [] { const char* e = getenv("DC_NO_PATCH"); return !(e != nullptr && e[0] == '1'); }();
    // (a stride-2 transposed convolution is, per output phase, a 2x2- or 3x3-tap convolution over the input lattice: same form)
    const bool kxk_patch = patch_allowed && (transposed || (pl.taps > 1 && d->stride_h == 1 && d->stride_w == 1));
    if (ws == nullptr && !kxk_patch && (pl.taps != 1 || d->pad_top != 0 || d->pad_left != 0)) return DC_ERR_UNSUPPORTED;
    if (!aligned16(in) || !aligned16(out) || !aligned16(filt)) return DC_ERR_ALIGNMENT;
    const int64_t npix_out = (int64_t)d->n * d->h_out * d->w_out;
    if (npix_out == 0) return DC_OK;
    if ((int64_t)d->n * d->h_in * d->w_in > 0x7fffffffLL) return DC_ERR_SHAPE;
    const bool has_res = ep != nullptr && ep->residual != nullptr;
    if (has_res) {
        // residual connection: linear stride-1 layers whose CTAs find their own rows (pointwise spans, or KxK patch tiles
        // when no scratch is given); with an activation the add layer's accumulated sum (prev_out) is updated too
        const bool unit = d->stride_h == 1 && d->stride_w == 1 && !transposed;
        const bool front_ok = unit && ((pl.taps == 1 && d->pad_top == 0 && d->pad_left == 0) || (pl.taps > 1 && ws == nullptr));
        const bool ok_res = front_ok && ep->truncation == DC_TRUNC_NONE && ep->residual_mask != nullptr && aligned16(ep->residual) &&
                            (ep->activation == DC_ACT_NONE || (ep->prev_out != nullptr && aligned16(ep->prev_out)));
        if (!ok_res) return DC_ERR_UNSUPPORTED;
    }
    bool want_fused = !has_res && ep != nullptr && ep->truncation == DC_TRUNC_MAX && d->c_out <= 256;
    // a handful of tiles with a long K loop (3x3 256 -> 256 on an 8x8 map): one CTA per tile would walk the whole loop while
    // most SMs idle; splitting the output channels over CTAs and truncating in a second pass is faster
    if (want_fused && pl.nkb >= 16 && divup64(npix_out, 128) * 8 <= sm_count()) want_fused = false;
    // 1x1 layers without padding can do without a work list: each CTA compacts its own pixels. On small maps a CTA
    // owns one contiguous span; on large maps persistent CTAs own strided spans (multi-span mode). When the map is so
    // large that a CTA would need several rounds of spans and the caller gave scratch memory, the work list is
    // better: its global compaction fills every tile.
    const bool pointwise = !transposed && pl.taps == 1 && d->pad_top == 0 && d->pad_left == 0;
    const bool unit_stride = d->stride_h == 1 && d->stride_w == 1;
    const int64_t spans_per_cta = divup64(divup64(npix_out, kRows), (int64_t)sm_count() * 3);
    if (pointwise && (npix_out < kListMinPixels || (unit_stride && spans_per_cta <= kMsSpans))) ws = nullptr;
    // the residual forms exist for the fronts whose CTAs find their own rows; the strided-span front takes any number of rounds
    if (pointwise && has_res) ws = nullptr;
    const bool multi_span = ws == nullptr && pointwise && unit_stride && npix_out >= kListMinPixels;
    const bool patch_mode = kxk_patch && ws == nullptr;
    if (patch_mode && !transposed) {
        // 3x3 layers: halo tiles (one load of the patch's halo per channel block instead of one per tap)
        int fused_there = 0;
        const int rc = conv3x3_halo(d, in, mi, filt, bias, out, mo, ep, (uint32_t)pl.rows * 128u, &fused_there, st);
        if (rc != DC_ERR_UNSUPPORTED) {
            if (rc != DC_OK) return rc;
            if (ep != nullptr && !fused_there)
                return dc_activate_truncate(out, ep->prev_out, ep->truncated, mo, npix_out, d->c_out, d->dtype, ep->threshold,
                                            ep->activation, ep->truncation, (void*)st);
            return DC_OK;
        }
    }
    if (transposed) {                 // the kernel sees one phase: m x m taps
        pl.taps = (d->kh / 2) * (d->kw / 2);
        pl.nkb = pl.taps * pl.ncb;
    }
    finish_plan(pl, d, npix_out, want_fused, ws != nullptr || patch_mode, multi_span);
    const bool fused = want_fused && pl.ntiles == 1;
    PwParams p{};
    p.in = (const __half*)in; p.mi = mi; p.wimg = (const uint8_t*)filt; p.bias = (const __half*)bias;
    p.out = (__half*)out; p.mo = mo;
    p.prev = fused ? (__half*)ep->prev_out : nullptr;
    p.trunc = fused ? (__half*)ep->truncated : nullptr;
    p.thr = fused ? host_round_threshold<__half>(ep->threshold) : 0.f;
    p.act = fused ? ep->activation : 0;
    p.fused = fused ? 1 : 0;
    p.res = has_res ? (const __half*)ep->residual : nullptr;
    p.res_mask = has_res ? ep->residual_mask : nullptr;
    p.res_prev = has_res && ep->activation != DC_ACT_NONE ? (__half*)ep->prev_out : nullptr;
    p.res_act = has_res ? ep->activation : 0;
    p.npix_out = npix_out;
    p.hi = d->h_in; p.wi = d->w_in; p.ho = d->h_out; p.wo = d->w_out; p.sh = d->stride_h; p.sw = d->stride_w;
    p.cin = d->c_in; p.cout = d->c_out;
    p.kh = d->kh; p.kw = d->kw; p.dh = d->dil_h; p.dw = d->dil_w; p.pt = d->pad_top; p.pl = d->pad_left;
    p.taps = pl.taps; p.ncb = pl.ncb;
    p.transposed = transposed; p.m = transposed ? d->kh / 2 : 0; p.wl_stride = transposed ? npix_out : 0;
    p.nkb = pl.nkb; p.bn = pl.bn; p.span = pl.span; p.b_resident = pl.b_resident; p.tmem_cols = pl.tmem_cols;
    p.nslots = pl.nslots;
    p.b_kb_stride = (uint32_t)pl.rows * 128u;
    fast_div_init((uint32_t)(d->h_out * d->w_out), &p.hw_mul, &p.hw_shift);
    fast_div_init((uint32_t)d->w_out, &p.wo_mul, &p.wo_shift);
    // span mode on a stride-1 pointwise layer: mostly active spans are loaded as whole tiles by TMA
    alignas(64) CUtensorMap tmap;
    memset(&tmap, 0, sizeof(tmap));
    p.tma_rows = 0;
    if (ws == nullptr && !transposed && pl.taps == 1 && d->stride_h == 1 && d->stride_w == 1 && d->pad_top == 0 && d->pad_left == 0 &&
        d->c_in >= kKBlock && encode_rows_map(&tmap, in, (int64_t)d->n * d->h_in * d->w_in, d->c_in))
        p.tma_rows = 1;
    p.off_b = pl.off_b; p.off_stage = pl.off_stage; p.off_list = pl.off_list; p.off_misc = pl.off_misc; p.stage_pitch = pl.stage_pitch;
    static PerDeviceOnce attr_once;
    bool* attr_set = attr_once.slot();
    if (attr_set == nullptr) return DC_ERR_LAUNCH;
    if (!*attr_set) {
        bool ok_attr = true;
#define DC_SET_ATTR(F, E, U) ok_attr &= cudaFuncSetAttribute(k_pw_umma<F, E, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess
        DC_SET_ATTR(0, true, 0); DC_SET_ATTR(1, true, 0); DC_SET_ATTR(2, true, 0); DC_SET_ATTR(3, true, 0); DC_SET_ATTR(5, true, 0);
        DC_SET_ATTR(0, true, 1); DC_SET_ATTR(1, true, 1); DC_SET_ATTR(2, true, 1); DC_SET_ATTR(3, true, 1); DC_SET_ATTR(5, true, 1);
        DC_SET_ATTR(0, false, 1); DC_SET_ATTR(1, false, 1); DC_SET_ATTR(2, false, 1); DC_SET_ATTR(3, false, 1); DC_SET_ATTR(5, false, 1);
        DC_SET_ATTR(0, true, 2); DC_SET_ATTR(2, true, 2); DC_SET_ATTR(3, true, 2);
        DC_SET_ATTR(0, true, 3); DC_SET_ATTR(2, true, 3); DC_SET_ATTR(3, true, 3);
#undef DC_SET_ATTR
        if (!ok_attr) return check_launch();
        *attr_set = true;
    }
    if (pl.smem > 227 * 1024) return DC_ERR_UNSUPPORTED;
    dim3 grid((unsigned)divup64(npix_out, pl.span), (unsigned)pl.ntiles);
    p.patch_mode = 0;
    if (patch_mode) {
        // patch shape tw x th (tw * th = 128) with the least overhang beyond the image; wide patches on ties
        int best_tw = 128;
        int64_t best_area = -1;
        // extent of the lattice the patches tile: the output, or (transposed) the points ((oy + pad) / 2, (ox + pad) / 2)
        const int lat_w = transposed ? ((d->w_out - 1 + d->pad_left) >> 1) + 1 : d->w_out;
        const int lat_h = transposed ? ((d->h_out - 1 + d->pad_top) >> 1) + 1 : d->h_out;
        for (int tw = 128; tw >= 8; tw >>= 1) {
            const int th = kRows / tw;
            const int64_t area = (int64_t)divup(lat_w, tw) * tw * divup(lat_h, th) * th;
            if (best_area < 0 || area < best_area) { best_area = area; best_tw = tw; }
        }
        const int tw = best_tw, th = kRows / tw;
        p.patch_mode = 1;
        p.patch_tw_log2 = 0;
        while ((1 << p.patch_tw_log2) < tw) ++p.patch_tw_log2;
        p.patch_px = divup(lat_w, tw);
        p.patch_py = divup(lat_h, th);
        p.npatches = (int64_t)d->n * p.patch_px * p.patch_py;
        fast_div_init((uint32_t)p.patch_px, &p.ppx_mul, &p.ppx_shift);
        fast_div_init((uint32_t)(p.patch_px * p.patch_py), &p.ppi_mul, &p.ppi_shift);
        p.tma_rows = encode_patch_map(&tmap, in, d, tw, th, kKBlock) ? 2 : 0;
        int64_t per_sm = (int64_t)(227 * 1024) / (int64_t)(pl.smem + 1024);
        if (per_sm > 3) per_sm = 3;
        if (per_sm < 1) per_sm = 1;
        int64_t persistent = (int64_t)sm_count() * per_sm / pl.ntiles;
        if (persistent < 1) persistent = 1;
        grid.x = (unsigned)(p.npatches < persistent ? p.npatches : persistent);
        if (transposed) grid.z = 4;       // one output phase per z
    }
    p.ms_rounds = 0;
    p.ms_nspans = divup64(npix_out, kRows);
    if (multi_span) {
        int64_t persistent = (int64_t)sm_count() * 3 / pl.ntiles;     // three CTAs of this kernel fit on an SM
        if (persistent < 1) persistent = 1;
        grid.x = (unsigned)(p.ms_nspans < persistent ? p.ms_nspans : persistent);
        p.ms_rounds = (int)divup64(divup64(p.ms_nspans, grid.x), kMsSpans);
        p.tma_rows = 0;
    }
    if (ws != nullptr) {              // work-list mode: scan pass, then persistent CTAs over the active rows
        int rc = transposed ? scan_deconv_mask(d, mi, mo, ws, ws_bytes, fused ? 1 : 0, st)
                            : scan_conv_mask(d, mi, mo, ws, ws_bytes, fused ? 1 : 0, st);
        if (rc != DC_OK) return rc;
        p.wl_count = reinterpret_cast<const int32_t*>(ws);
        p.wl_list = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(ws) + 16);
        p.wl_taps = p.wl_list + (transposed ? 4 * npix_out : npix_out);
        if (transposed) grid.z = 4;
        int64_t persistent = (int64_t)sm_count() * 3 / pl.ntiles;     // three CTAs of this kernel fit on an SM
        if (persistent < 1) persistent = 1;
        if ((int64_t)grid.x > persistent) grid.x = (unsigned)persistent;
    }
    const bool exact_act = !fused || (p.act >= DC_ACT_NONE && p.act <= DC_ACT_RELU6);
    const int front = ws != nullptr ? 1 : patch_mode ? (transposed ? 5 : 2) : multi_span ? 3 : 0;
    int rc;
#define DC_LAUNCH(F, E, U) rc = launch_pdl(k_pw_umma<F, E, U>, grid, dim3(kPwThreads), pl.smem, st, p, tmap)
#define DC_LAUNCH_FRONT(E, U)                                  \
    do {                                                        \
        if (front == 1) DC_LAUNCH(1, E, U);                     \
        else if (front == 2) DC_LAUNCH(2, E, U);                \
        else if (front == 3) DC_LAUNCH(3, E, U);                \
        else if (front == 5) DC_LAUNCH(5, E, U);                \
        else DC_LAUNCH(0, E, U);                                \
    } while (0)
    if (has_res) {                    // residual forms exist for the fronts whose CTAs find their own rows
        const bool with_act = p.res_prev != nullptr;
        if (front == 2) { if (with_act) DC_LAUNCH(2, true, 3); else DC_LAUNCH(2, true, 2); }
        else if (front == 3) { if (with_act) DC_LAUNCH(3, true, 3); else DC_LAUNCH(3, true, 2); }
        else if (front == 0) { if (with_act) DC_LAUNCH(0, true, 3); else DC_LAUNCH(0, true, 2); }
        else return DC_ERR_UNSUPPORTED;
    }
    else if (!fused) DC_LAUNCH_FRONT(true, 0);
    else if (exact_act) DC_LAUNCH_FRONT(true, 1);
    else DC_LAUNCH_FRONT(false, 1);
#undef DC_LAUNCH_FRONT
#undef DC_LAUNCH
    if (rc != DC_OK) return rc;
    if (ep != nullptr && !fused && !has_res)
        return dc_activate_truncate(out, ep->prev_out, ep->truncated, mo, npix_out, d->c_out, d->dtype, ep->threshold,
                                    ep->activation, ep->truncation, (void*)st);
    return DC_OK;
}

int conv2d_umma(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st) {
    return conv_umma_impl(d, 0, in, mi, filt, bias, out, mo, ep, ws, ws_bytes, st);
}

int deconv2d_umma(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out,
                  int32_t* mo, const dc_epilogue* ep, void* ws, size_t ws_bytes, cudaStream_t st) {
    return conv_umma_impl(d, 1, in, mi, filt, bias, out, mo, ep, ws, ws_bytes, st);
}

int umma_error_code() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_umma_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

}  // namespace dc
