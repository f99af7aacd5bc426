// Tensor-core delta convolution for stride-1 3x3 layers on mostly active maps: "halo tiles".
//
// A tile is a patch of 16 rows x 8 pixels of the output (128 MMA rows). Its input, the 18 x 10 pixel halo, is loaded
// ONCE per block of 64 input channels by one 4-D tiled TMA request (box 64 channels x 16 pixels x 18 rows, 128-byte
// swizzle; the padding and everything beyond the image arrive as zeros). The nine taps then read nine shifted views
// of that one copy: an image row of the patch is one 8-row group of the MMA's A operand, so tap (ky, kx) is the same
// shared memory with the start address moved by ky halo rows and kx pixels (stride between 8-row groups = one halo
// row of 16 pixels = 2048 bytes; the swizzle pattern follows the shared-memory address, so the shifted start needs no
// other change). Compared with one request per tap this reads the input from L2 once instead of nine times and
// turns nine dependent load/wait rounds per channel block into one.
//
// Layers with at most 32 input channels keep their halo as rows of 64 bytes (32-channel boxes, 64-byte swizzle on both the
// TMA and the MMA side; the filter keeps its 128-byte rows, every operand has its own descriptor): half the stage, which
// lets two CTAs share an SM (3x3 32->32 @64x64: 32.8 -> 24.6 us).
//
// The delta tensor is only defined at active pixels, so halo pixels inside the image whose in-mask is clear are
// overwritten with zeros in shared memory before the tensor core reads them; every patch with at least one active
// output pixel takes this path, inactive output rows are computed and dropped.
//
// Roles (384 threads, persistent CTAs over the patches, everything double-buffered so that the tiles overlap):
//   warp 0   reads the halo's mask words, derives the out-mask of the patch, publishes the tile record, issues the TMA
//            loads (ring of halo stages)
//   warp 1   one thread issues tcgen05.mma into one of two accumulators in tensor memory
//   warp 2   waits for a halo stage to land, zeroes its inactive pixels, hands it to the MMA thread
//   warp 3   streams filter blocks (one per tap and channel block) through a ring when the filter is too large to stay
//   warps 4-11  epilogue: tensor memory -> fp16 staging tile -> coalesced rows with the optional fused accumulate +
//            activation delta + any-channel truncation; the accumulator is released as soon as it is staged
// Every wait on an mbarrier is bounded; a wait that gives up sets a sticky error code (dc_umma_error) and every role
// leaves its loop.
#include <cstdlib>
#include <cstring>
#include <cuda.h>
#include "dc_umma.cuh"

namespace dc {

__device__ int g_halo_error = 0;

#ifdef DC_HALO_STAMPS
__device__ long long g_halo_stamps[64];
#define HALO_STAMP(i) do { if (blockIdx.x == 0) g_halo_stamps[(i)] = clock64(); } while (0)
#else
#define HALO_STAMP(i) do { } while (0)
#endif

constexpr int kHaloTh = 16, kHaloTw = 8;                  // output patch
constexpr int kHaloRows = kHaloTh + 2, kHaloCols = kHaloTw + 2, kHaloPitch = 16;
constexpr int kHaloPix = kHaloRows * kHaloCols;           // 180 halo pixels that are read
constexpr int kHaloThreads = 384;
constexpr int kHaloEpiWarps = 8, kHaloEpiThreads = kHaloEpiWarps * 32, kHaloFirstEpiWarp = 4;
constexpr int kHaloInfo = 8;                              // ring of tile records
constexpr int kHaloInfoWords = 12;                        // [0..3] rows with active taps, [4] tile runs, [5..8] rows with an active residual
constexpr int kHaloMaxA = 4, kHaloMaxB = 8;
constexpr int kHaloCodesPitch = 192;
constexpr int kHaloRawPitch = kHaloCodesPitch + 128;       // mask words fetched ahead per tile: the halo, then the residual mask of the 128 outputs

struct HaloParams {
    const int32_t* mi; const uint8_t* wimg; const __half* bias;
    __half* out; int32_t* mo; __half* prev; __half* trunc;
    float thr; int act;
    const __half* res; const int32_t* res_mask; __half* res_prev; int res_act;   // residual forms
    // several layers on the same input in one launch (the 3x3 convolutions of detection heads): the output channels are
    // nseg equal segments, each with its own output, out-mask, caches, threshold and activation
    int nseg, seg_cout;
    __half* seg_out[4]; int32_t* seg_mo[4]; __half* seg_prev[4]; __half* seg_trunc[4]; float seg_thr[4]; int seg_act[4];
    int h, w, ho, wo, pt, pl;
    int cin, cout, ncb, bn, tmem_cols, last_ksteps;
    int nA, nB, b_resident;
    uint32_t b_kb_stride;
    int patch_px, patch_py;
    int64_t npatches;
    uint32_t ppx_mul, ppx_shift, ppi_mul, ppi_shift;
    uint32_t off_b, off_stage, off_misc, stage_pitch;
    int dbg;
};

// K-major operand, 128-byte swizzle, 8-row groups sbo bytes apart. The swizzle pattern follows the shared-memory address
// (bits 7-9 select the pattern row), so a start address that is a multiple of 128 bytes inside a 1024-byte pattern needs
// nothing else: the descriptor's base-offset field stays 0 (measured: with the field set to the row position the
// results are wrong).
__device__ __forceinline__ uint64_t make_smem_desc_ex(uint32_t smem_addr, uint32_t sbo, uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout << 61;                              // 2: 128-byte swizzle, 4: 64-byte swizzle
    return d;
}

// every lane polls (no single-lane branch, no shuffle of the result on the fast path); the warp agrees on the outcome
__device__ __forceinline__ bool mbar_wait_all(uint32_t bar, uint32_t parity, volatile uint32_t* ok_flag) {
    return __all_sync(DC_FULL, mbar_wait(bar, parity, ok_flag));
}
// named barrier of the epilogue threads that also ANDs a predicate over them
__device__ __forceinline__ bool epi_bar_and(bool v) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(r) : "r"((uint32_t)(v ? 1u : 0u)), "n"(kHaloEpiThreads) : "memory");
    return r != 0;
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kHaloEpiThreads) : "memory"); }

// kEpi: 0 plain store, 1 fused truncation step, 2 residual added (the DCAdd behind a linear layer), 3 residual and the add
// layer's activation with its accumulated sum. kExactAct: the fused activation is exact in packed half arithmetic.
// kU: groups of rows a warp of the epilogue keeps in flight (4 when the CTA has its SM to itself and the tile needs more
// than one round of cache reads otherwise: then all of a tile's cache rows are asked for in one round trip).
// kA64: halo rows of 64 bytes (layers of at most 32 input channels) instead of 128: compile-time, so that the tap offsets
// of the MMA loop stay constants.
// kSeg: the output channels are p.nseg segments with their own outputs and caches (kEpi 0 or 1).
template <int kEpi, bool kExactAct, int kU, bool kA64, bool kSeg = false>
__global__ void __launch_bounds__(kHaloThreads, kU == 4 ? 1 : 2) k_conv3x3_halo(const HaloParams p, const __grid_constant__ CUtensorMap tmap_in) {
    constexpr bool kFused = kEpi == 1;
    constexpr bool kRes = kEpi >= 2;
    constexpr uint32_t kARow = kA64 ? 64u : 128u;              // bytes of a halo pixel's row in shared memory
    constexpr uint32_t kAStage = (uint32_t)kHaloRows * kHaloPitch * kARow;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + p.off_b;
    uint8_t* sStage = smem + p.off_stage;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_misc);
    // barrier indices
    constexpr int kAFull = 0, kAReady = kHaloMaxA, kAEmpty = 2 * kHaloMaxA, kBFull = 3 * kHaloMaxA, kBEmpty = kBFull + kHaloMaxB,
                  kAccFull = kBEmpty + kHaloMaxB, kAccEmpty = kAccFull + 2, kInfoFull = kAccEmpty + 2, kInfoEmpty = kInfoFull + kHaloInfo,
                  kRowsFull = kInfoEmpty + kHaloInfo, kNumBars = kRowsFull + kHaloInfo;
    uint32_t* s_u32 = reinterpret_cast<uint32_t*>(bars + kNumBars);     // [0] tmem base, [1] ok flag
    uint32_t* s_info = s_u32 + 8;                                       // [kHaloInfo][kHaloInfoWords]
    uint8_t* s_codes = reinterpret_cast<uint8_t*>(s_info + kHaloInfo * kHaloInfoWords);   // [kHaloInfo][192]: 0 outside, 1 active, 2 inactive
    float* s_bias = reinterpret_cast<float*>(s_codes + kHaloInfo * kHaloCodesPitch);
    int32_t* s_raw = reinterpret_cast<int32_t*>(s_bias + 256);          // [4][kHaloRawPitch] mask words of the tiles ahead

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    volatile uint32_t* ok_flag = &s_u32[1];
    const int info_consumers = 3 + (p.b_resident ? 0 : 1);

    if (tid == 0) HALO_STAMP(0);
    if (tid < kNumBars) {
        uint32_t count = 1;
        if (tid >= kInfoEmpty && tid < kRowsFull) count = (uint32_t)info_consumers;
        mbar_init(bar(tid), count);
        fence_barrier_init();
    }
    if (tid == 0) { s_u32[1] = 1; s_u32[2] = 0; s_u32[3] = 0; s_u32[4] = 0; s_u32[5] = 0; }
    for (int i = tid; i < p.bn; i += kHaloThreads) s_bias[i] = (p.bias != nullptr && i < p.cout) ? __half2float(p.bias[i]) : 0.f;
    if (warp == 1) tmem_alloc(smem_u32(&s_u32[0]), (uint32_t)(2 * p.tmem_cols));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) HALO_STAMP(1);
    grid_dep_launch();
    const uint32_t tmem_base = s_u32[0];
    const uint32_t b_block_bytes = (uint32_t)p.bn * 128u;
    const uint32_t sA_u32 = smem_u32(sA), sB_u32 = smem_u32(sB);
    const int tiles_mine = (int)((p.npatches - blockIdx.x + gridDim.x - 1) / gridDim.x);
    auto fail = [&](int code) { *ok_flag = 0; atomicExch(&g_halo_error, code); };
    auto write_mo = [&](int64_t idx, int v) {                 // the out-mask word of a pixel (of every segment)
        if constexpr (kSeg) {
#pragma unroll
            for (int sg = 0; sg < 4; ++sg) if (sg < p.nseg) p.seg_mo[sg][idx] = v;
        } else {
            p.mo[idx] = v;
        }
    };
    auto patch_origin = [&](int t, int& b, int& y0, int& x0) {
        const uint32_t pid = (uint32_t)blockIdx.x + (uint32_t)t * gridDim.x;
        const uint32_t pb = fast_div(pid, p.ppi_mul, p.ppi_shift);
        const uint32_t prem = pid - pb * (uint32_t)(p.patch_px * p.patch_py);
        const uint32_t pyi = fast_div(prem, p.ppx_mul, p.ppx_shift);
        b = (int)pb;
        y0 = (int)pyi * kHaloTh;
        x0 = (int)(prem - pyi * (uint32_t)p.patch_px) * kHaloTw;
    };

    if (warp == 1 && lane == 0 && p.b_resident) {         // the filter does not depend on the previous kernel
        const int nkb = 9 * p.ncb;
        mbar_expect_tx(bar(kBFull), (uint32_t)nkb * b_block_bytes);
        for (int kb = 0; kb < nkb; ++kb)
            bulk_g2s(sB_u32 + (uint32_t)kb * b_block_bytes, p.wimg + (size_t)kb * p.b_kb_stride, b_block_bytes, bar(kBFull));
    }
    grid_dep_wait();
    if (tid == 0) HALO_STAMP(2);

    if (warp == 0) {
        // ---- tile records and halo loads ----
        // The mask words of a halo are fetched two tiles ahead by 4-byte asynchronous copies into a private ring, so the
        // warp never waits a full memory round trip per tile.
        constexpr int kPer = (kHaloPix + 31) / 32, kAhead = 2, kRawRing = 4;
        auto fetch_masks = [&](int t) {
            if (t < tiles_mine) {
                int b, y0, x0;
                patch_origin(t, b, y0, x0);
                int32_t* raw = s_raw + (t % kRawRing) * kHaloRawPitch;
#pragma unroll
                for (int j = 0; j < kPer; ++j) {
                    const int i = lane + 32 * j;
                    const int hy = i / kHaloCols, hx = i - hy * kHaloCols;
                    const int iy = y0 - p.pt + hy, ix = x0 - p.pl + hx;
                    if (i < kHaloPix && iy >= 0 && iy < p.h && ix >= 0 && ix < p.w)
                        cp_async4(smem_u32(raw + i), p.mi + ((int64_t)b * p.h + iy) * p.w + ix);
                }
                if constexpr (kRes) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int r = lane + 32 * j;
                        const int oy = y0 + (r >> 3), ox = x0 + (r & 7);
                        if (oy < p.ho && ox < p.wo) cp_async4(smem_u32(raw + kHaloCodesPitch + r), p.res_mask + ((int64_t)b * p.ho + oy) * p.wo + ox);
                    }
                }
            }
            cp_async_commit();
        };
        for (int t = 0; t < kAhead; ++t) fetch_masks(t);
        int ia = 0;
        for (int t = 0; t < tiles_mine && *ok_flag != 0; ++t) {
            const int slot = t % kHaloInfo, use = t / kHaloInfo;
            fetch_masks(t + kAhead);
            cp_async_wait_group<kAhead>();                         // this thread's words of tile t have landed
            __syncwarp();
            if (use > 0 && !mbar_wait_warp(bar(kInfoEmpty + slot), (uint32_t)((use - 1) & 1), ok_flag)) { fail(11); break; }
            int b, y0, x0;
            patch_origin(t, b, y0, x0);
            uint8_t* codes = s_codes + slot * kHaloCodesPitch;
            bool has_active = false;
            {
                const int32_t* raw = s_raw + (t % kRawRing) * kHaloRawPitch;
#pragma unroll
                for (int j = 0; j < kPer; ++j) {
                    const int i = lane + 32 * j;
                    const int hy = i / kHaloCols, hx = i - hy * kHaloCols;
                    const int iy = y0 - p.pt + hy, ix = x0 - p.pl + hx;
                    const bool inside = iy >= 0 && iy < p.h && ix >= 0 && ix < p.w;
                    if (i < kHaloPix) {
                        const uint8_t code = inside ? (raw[i] != 0 ? 1 : 2) : 0;
                        codes[i] = code;
                        has_active |= code == 1;
                    }
                }
                if constexpr (kRes) {          // rows where the residual is active: a row of their own even without active taps
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int r = lane + 32 * j;
                        const bool ron = y0 + (r >> 3) < p.ho && x0 + (r & 7) < p.wo && raw[kHaloCodesPitch + r] != 0;
                        const unsigned bal = __ballot_sync(DC_FULL, ron);
                        if (lane == 0) s_info[slot * kHaloInfoWords + 5 + j] = bal;
                        has_active |= ron;
                    }
                }
            }
            // an active pixel anywhere in the halo: the tile runs (its row bits come from the warp that prepares the stage)
            const uint32_t any = __any_sync(DC_FULL, has_active) ? 1u : 0u;
            if (lane == 0) s_info[slot * kHaloInfoWords + 4] = any;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kInfoFull + slot));
            if (lane == 0 && t < 4) HALO_STAMP(3 + t);
            if (any == 0u) continue;
            for (int cb = 0; cb < p.ncb; ++cb, ++ia) {
                const int stage = ia % p.nA, ause = ia / p.nA;
                if (ause > 0 && !mbar_wait_warp(bar(kAEmpty + stage), (uint32_t)((ause - 1) & 1), ok_flag)) { fail(12); break; }
                if (elect_one()) {
                    mbar_expect_tx(bar(kAFull + stage), kAStage);
                    tma_load_patch(sA_u32 + (uint32_t)stage * kAStage, &tmap_in, cb * kKBlock, x0 - p.pl, y0 - p.pt, b, bar(kAFull + stage));
                    if (t < 4 && cb == 0) HALO_STAMP(8 + t);
                }
            }
        }
        cp_async_wait_group<0>();
    } else if (warp == 2) {
        // ---- out-mask and row bits of the tile; inactive halo pixels become zeros before the tensor core reads a stage ----
        int ia = 0;
        for (int t = 0; t < tiles_mine && *ok_flag != 0; ++t) {
            const int slot = t % kHaloInfo, use = t / kHaloInfo;
            if (!mbar_wait_all(bar(kInfoFull + slot), (uint32_t)(use & 1), ok_flag)) { fail(21); break; }
            if (s_info[slot * kHaloInfoWords + 4] != 0u) {
                const uint8_t* codes = s_codes + slot * kHaloCodesPitch;
                int b, y0, x0;
                patch_origin(t, b, y0, x0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = lane + 32 * j, y = r >> 3, x = r & 7;
                    const int oy = y0 + y, ox = x0 + x;
                    const bool valid = oy < p.ho && ox < p.wo;
                    bool on = false;
                    if (valid) {
#pragma unroll
                        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                            for (int kx = 0; kx < 3; ++kx) on |= codes[(y + ky) * kHaloCols + x + kx] == 1;
                        bool ron = false;
                        if constexpr (kRes) ron = ((s_info[slot * kHaloInfoWords + 5 + j] >> lane) & 1u) != 0u;
                        if (!kFused || !on) write_mo(((int64_t)b * p.ho + oy) * p.wo + ox, (on || ron) ? 1 : 0);
                    }
                    const unsigned bal = __ballot_sync(DC_FULL, on);
                    if (lane == 0) s_info[slot * kHaloInfoWords + j] = bal;
                }
                bool need = false;
                for (int i = lane; i < kHaloPix; i += 32) need |= codes[i] == 2;
                need = __any_sync(DC_FULL, need);
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kRowsFull + slot));
                bool okw = true;
                for (int cb = 0; cb < p.ncb && okw; ++cb, ++ia) {
                    const int stage = ia % p.nA, ause = ia / p.nA;
                    if (!mbar_wait_all(bar(kAFull + stage), (uint32_t)(ause & 1), ok_flag)) { fail(22); okw = false; break; }
                    if (need) {
                        uint8_t* st = sA + (size_t)stage * kAStage;
                        constexpr int cpr = (int)(kARow >> 4);                  // 16-byte chunks of a pixel's row: 8 or 4
                        for (int i = lane; i < kHaloPix * cpr; i += 32) {
                            const int px = i / cpr;
                            if (codes[px] == 2) {
                                const int hy = px / kHaloCols, hx = px - hy * kHaloCols;
                                *reinterpret_cast<uint4*>(st + (size_t)(hy * kHaloPitch + hx) * kARow + (i - px * cpr) * 16) = make_uint4(0u, 0u, 0u, 0u);
                            }
                        }
                        fence_proxy_async();
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(kAReady + stage));
                    if (lane == 0 && t < 4 && cb == 0) HALO_STAMP(12 + t);
                }
                if (!okw) break;
            } else {
                // nothing active in the halo: the patch's out-mask is all zeros, no other role touches the tile
                int b, y0, x0;
                patch_origin(t, b, y0, x0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = lane + 32 * j;
                    const int oy = y0 + (r >> 3), ox = x0 + (r & 7);
                    if (oy < p.ho && ox < p.wo) write_mo(((int64_t)b * p.ho + oy) * p.wo + ox, 0);
                }
                if (lane == 0) mbar_arrive(bar(kRowsFull + slot));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kInfoEmpty + slot));
        }
    } else if (warp == 3) {
        // ---- filter blocks through the ring (large filters only) ----
        if (!p.b_resident) {
            int ib = 0;
            for (int t = 0; t < tiles_mine && *ok_flag != 0; ++t) {
                const int slot = t % kHaloInfo, use = t / kHaloInfo;
                if (!mbar_wait_warp(bar(kInfoFull + slot), (uint32_t)(use & 1), ok_flag)) { fail(31); break; }
                bool okw = true;
                if (s_info[slot * kHaloInfoWords + 4] != 0u) {
                    for (int cb = 0; cb < p.ncb && okw; ++cb) {
                        for (int tap = 0; tap < 9; ++tap, ++ib) {
                            const int bs = ib % p.nB, buse = ib / p.nB;
                            if (buse > 0 && !mbar_wait_warp(bar(kBEmpty + bs), (uint32_t)((buse - 1) & 1), ok_flag)) { fail(32); okw = false; break; }
                            if (elect_one()) {
                                mbar_expect_tx(bar(kBFull + bs), b_block_bytes);
                                bulk_g2s(sB_u32 + (uint32_t)bs * b_block_bytes, p.wimg + (size_t)(tap * p.ncb + cb) * p.b_kb_stride, b_block_bytes,
                                         bar(kBFull + bs));
                            }
                        }
                    }
                }
                if (!okw) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kInfoEmpty + slot));
            }
        }
    } else if (warp == 1) {
        // ---- the tensor core's warp: warp-uniform control flow, one elected lane issues the MMAs and commits (the
        //      operands of tcgen05.mma live in uniform registers, which a divergent single-lane loop cannot use well) ----
        const uint32_t idesc = make_idesc(p.bn);
        int ia = 0, ib = 0, nt = 0;
        bool okw = true;
        for (int t = 0; t < tiles_mine && okw && *ok_flag != 0; ++t) {
            const int slot = t % kHaloInfo, use = t / kHaloInfo;
            if (!mbar_wait_all(bar(kInfoFull + slot), (uint32_t)(use & 1), ok_flag)) { fail(41); break; }
            if (s_info[slot * kHaloInfoWords + 4] != 0u) {
                const int buf = nt & 1;
                if (nt >= 2 && !mbar_wait_all(bar(kAccEmpty + buf), (uint32_t)(((nt >> 1) - 1) & 1), ok_flag)) { fail(42); break; }
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)(buf * p.tmem_cols);
                for (int cb = 0; cb < p.ncb && okw; ++cb, ++ia) {
                    const int stage = ia % p.nA, ause = ia / p.nA;
                    // (the stage's TMA load was observed complete by the warp that arrives on this barrier)
                    if (!mbar_wait_all(bar(kAReady + stage), (uint32_t)(ause & 1), ok_flag)) { fail(43); okw = false; break; }
                    if (p.b_resident && nt == 0 && cb == 0 && !mbar_wait_all(bar(kBFull), 0u, ok_flag)) { fail(44); okw = false; break; }
                    tc_fence_after();
                    const int ksteps = cb == p.ncb - 1 ? p.last_ksteps : kKBlock / 16;
                    const uint64_t ad0 = make_smem_desc_ex(sA_u32 + (uint32_t)stage * kAStage, kHaloPitch * kARow, kA64 ? 4u : 2u);
                    constexpr uint32_t a_px = kARow >> 4;                       // a halo pixel in descriptor units of 16 bytes
                    if (p.b_resident) {
                        if (elect_one()) {
                            const uint64_t bd0 = make_smem_desc(sB_u32 + (uint32_t)cb * b_block_bytes);
                            const uint64_t b_tap = (uint64_t)(((uint32_t)p.ncb * b_block_bytes) >> 4);
#pragma unroll
                            for (int tap = 0; tap < 9; ++tap) {
                                const int ky = tap / 3, kx = tap - ky * 3;
                                const uint64_t ad = ad0 + (uint64_t)((uint32_t)(ky * kHaloPitch + kx) * a_px);
                                const uint64_t bd = bd0 + (uint64_t)tap * b_tap;
#ifdef DC_HALO_STAMPS
                                if (t == 1 && cb == 0) HALO_STAMP(44 + tap);
                                if (p.dbg & 1) continue;
#endif
                                if (ksteps == kKBlock / 16) {      // a full channel block: constant offsets, no loop
#pragma unroll
                                    for (int ks = 0; ks < kKBlock / 16; ++ks)
                                        umma_f16(tacc, ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc, (cb > 0 || tap > 0 || ks > 0) ? 1u : 0u);
                                } else {
                                    for (int ks = 0; ks < ksteps; ++ks)
                                        umma_f16(tacc, ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc, (cb > 0 || tap > 0 || ks > 0) ? 1u : 0u);
                                }
                            }
                            umma_commit(bar(kAEmpty + stage));
                        }
                        __syncwarp();
                    } else {
                        for (int tap = 0; tap < 9; ++tap, ++ib) {
                            const int ky = tap / 3, kx = tap - ky * 3;
                            const int bs = ib % p.nB;
                            if (!mbar_wait_all(bar(kBFull + bs), (uint32_t)((ib / p.nB) & 1), ok_flag)) { fail(45); okw = false; break; }
                            tc_fence_after();
                            if (elect_one()) {
                                const uint64_t ad = ad0 + (uint64_t)((uint32_t)(ky * kHaloPitch + kx) * a_px);
                                const uint64_t bd = make_smem_desc(sB_u32 + (uint32_t)bs * b_block_bytes);
                                if (ksteps == kKBlock / 16) {
#pragma unroll
                                    for (int ks = 0; ks < kKBlock / 16; ++ks)
                                        umma_f16(tacc, ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc, (cb > 0 || tap > 0 || ks > 0) ? 1u : 0u);
                                } else {
                                    for (int ks = 0; ks < ksteps; ++ks)
                                        umma_f16(tacc, ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc, (cb > 0 || tap > 0 || ks > 0) ? 1u : 0u);
                                }
                                umma_commit(bar(kBEmpty + bs));
                                if (tap == 8) umma_commit(bar(kAEmpty + stage));
                            }
                            __syncwarp();
                        }
                    }
                }
                if (!okw) break;
                if (elect_one()) {
                    umma_commit(bar(kAccFull + buf));
                    if (t < 4) HALO_STAMP(16 + t);
                }
                __syncwarp();
                ++nt;
            }
            if (elect_one()) mbar_arrive(bar(kInfoEmpty + slot));
            __syncwarp();
        }
    } else {
        // ---- epilogue warps ----
        const int ew = warp - kHaloFirstEpiWarp;                   // 0 .. 7
        const int etid = tid - kHaloFirstEpiWarp * 32;
        const int nch = p.cout >> 3;
        int g = 1;
        while (g < nch && g < 32) g <<= 1;
        const int lig = lane & (g - 1), ppw = 32 / g;
        const __half2 thr2 = __float2half2_rn(p.thr);
        const int rb_first = ew * ppw * kU, rb_step = kHaloEpiWarps * ppw * kU;
        int nt = 0;
        for (int t = 0; t < tiles_mine; ++t) {
            const int slot = t % kHaloInfo, use = t / kHaloInfo;
            // every thread waits for the tile's row bits itself; one named barrier per tile makes the outcome uniform (and
            // orders the previous tile's reads of the staging tile before this tile's writes)
            const bool ok1 = *ok_flag != 0 && mbar_wait(bar(kRowsFull + slot), (uint32_t)(use & 1), ok_flag);
            const bool any = ok1 && s_info[slot * kHaloInfoWords + 4] != 0u;
            if (etid == 0 && t < 4) HALO_STAMP(20 + t);
            const int buf = nt & 1;
            uint32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0, r0 = 0, r1 = 0, r2 = 0, r3 = 0;
            if (any) {
                a0 = s_info[slot * kHaloInfoWords + 0]; a1 = s_info[slot * kHaloInfoWords + 1];
                a2 = s_info[slot * kHaloInfoWords + 2]; a3 = s_info[slot * kHaloInfoWords + 3];
                if constexpr (kRes) {
                    r0 = s_info[slot * kHaloInfoWords + 5]; r1 = s_info[slot * kHaloInfoWords + 6];
                    r2 = s_info[slot * kHaloInfoWords + 7]; r3 = s_info[slot * kHaloInfoWords + 8];
                }
            }
            auto row_on = [&](int r) -> bool {                     // the convolution is active at row r
                const uint32_t wv = (r & 64) ? ((r & 32) ? a3 : a2) : ((r & 32) ? a1 : a0);
                return r < kRows && ((wv >> (r & 31)) & 1u) != 0u;
            };
            auto row_res = [&](int r) -> bool {                    // the residual is active at row r
                const uint32_t wv = (r & 64) ? ((r & 32) ? r3 : r2) : ((r & 32) ? r1 : r0);
                return kRes && r < kRows && ((wv >> (r & 31)) & 1u) != 0u;
            };
            int b = 0, y0 = 0, x0 = 0;
            patch_origin(t, b, y0, x0);
            Pack<__half, 8> d[kU], y[kU], tr[kU];
            int64_t off[kU], q[kU];
            bool mine[kU];
            // addresses and cache rows of a group of rows; they do not depend on the convolution's result, so the first
            // group of every warp is asked for before the accumulator is waited for
            auto load_caches = [&](int rb) {
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const int r = rb + u * ppw + lane / g;
                    mine[u] = (row_on(r) || row_res(r)) && lig < nch;
                    q[u] = ((int64_t)b * p.ho + y0 + (r >> 3)) * p.wo + x0 + (r & 7);
                    off[u] = mine[u] ? q[u] * p.cout + lig * 8 : 0;
                    if (kFused && mine[u]) {
                        y[u].load(p.prev + off[u]);
                        tr[u].load(p.trunc + off[u]);
                    }
                    if constexpr (kRes) {                          // tr = the residual's delta, y = the add layer's accumulated sum
                        if (mine[u]) {
                            if (row_res(r)) tr[u].load(p.res + off[u]); else tr[u].zero();
                            if (kEpi == 3) y[u].load(p.res_prev + off[u]);
                        }
                    }
                }
            };
            bool ok2 = true;
            if (any) {
                if (!kSeg && rb_first < kRows) load_caches(rb_first);
                ok2 = mbar_wait(bar(kAccFull + buf), (uint32_t)((nt >> 1) & 1), ok_flag);
            }
            if (!epi_bar_and(ok1 && ok2)) {
                if (etid == 0) fail(51);
                break;
            }
            if (!any) {
                if (etid == 0) mbar_arrive(bar(kInfoEmpty + slot));
                __syncwarp();
                continue;
            }
            if (etid == 0 && t < 4) HALO_STAMP(24 + t);
            tc_fence_after();
            if constexpr (kSeg) {
                // segment by segment: its columns of the accumulator -> staging tile -> rows against the segment's own caches
                const int nch_s = p.seg_cout >> 3;
                int gs = 1;
                while (gs < nch_s && gs < 32) gs <<= 1;
                const int ligs = lane & (gs - 1), ppws = 32 / gs;
                for (int seg = 0; seg < p.nseg; ++seg) {
                    const int c_base = seg * p.seg_cout;
                    if (seg > 0) epi_bar_sync();                   // the previous segment's rows are done with the staging tile
                    {
                        const int quarter = warp & 3;
                        const int r = quarter * 32 + lane;
                        uint8_t* srow = sStage + (size_t)r * p.stage_pitch;
#pragma unroll 1
                        for (int c0 = (ew >> 2) * 16; c0 < p.seg_cout; c0 += 32) {
                            uint32_t acc[16];
                            tmem_ld16(tmem_base + (uint32_t)(buf * p.tmem_cols) + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c_base + c0), acc);
                            tmem_ld_wait();
                            uint4 o[2];
                            __half2* h = reinterpret_cast<__half2*>(o);
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                h[j] = __floats2half2_rn(__uint_as_float(acc[2 * j]) + s_bias[c_base + c0 + 2 * j],
                                                         __uint_as_float(acc[2 * j + 1]) + s_bias[c_base + c0 + 2 * j + 1]);
                            *reinterpret_cast<uint4*>(srow + c0 * 2) = o[0];
                            *reinterpret_cast<uint4*>(srow + c0 * 2 + 16) = o[1];
                        }
                    }
                    tc_fence_before();
                    epi_bar_sync();
                    if (etid == 0 && seg == p.nseg - 1) {          // the accumulator is staged or consumed: the next tile may use it
                        mbar_arrive(bar(kAccEmpty + buf));
                        mbar_arrive(bar(kInfoEmpty + slot));
                    }
                    __syncwarp();
                    __half* out_s = seg == 0 ? p.seg_out[0] : seg == 1 ? p.seg_out[1] : seg == 2 ? p.seg_out[2] : p.seg_out[3];
                    int32_t* mo_s = seg == 0 ? p.seg_mo[0] : seg == 1 ? p.seg_mo[1] : seg == 2 ? p.seg_mo[2] : p.seg_mo[3];
                    __half* prev_s = seg == 0 ? p.seg_prev[0] : seg == 1 ? p.seg_prev[1] : seg == 2 ? p.seg_prev[2] : p.seg_prev[3];
                    __half* trunc_s = seg == 0 ? p.seg_trunc[0] : seg == 1 ? p.seg_trunc[1] : seg == 2 ? p.seg_trunc[2] : p.seg_trunc[3];
                    const float thr_s = seg == 0 ? p.seg_thr[0] : seg == 1 ? p.seg_thr[1] : seg == 2 ? p.seg_thr[2] : p.seg_thr[3];
                    const int act_s = seg == 0 ? p.seg_act[0] : seg == 1 ? p.seg_act[1] : seg == 2 ? p.seg_act[2] : p.seg_act[3];
                    const __half2 thr2_s = __float2half2_rn(thr_s);
#pragma unroll 1
                    for (int rb = ew * ppws * kU; rb < kRows; rb += kHaloEpiWarps * ppws * kU) {
#pragma unroll
                        for (int u = 0; u < kU; ++u) {
                            const int r = rb + u * ppws + lane / gs;
                            mine[u] = row_on(r) && ligs < nch_s;
                            q[u] = ((int64_t)b * p.ho + y0 + (r >> 3)) * p.wo + x0 + (r & 7);
                            off[u] = mine[u] ? q[u] * p.seg_cout + ligs * 8 : 0;
                            if (mine[u]) {
                                if (kFused) {
                                    y[u].load(prev_s + off[u]);
                                    tr[u].load(trunc_s + off[u]);
                                }
                                d[u].load(reinterpret_cast<const __half*>(sStage + (size_t)r * p.stage_pitch) + ligs * 8);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < kU; ++u) {
                            if (!kFused) {
                                if (mine[u]) d[u].store(out_s + off[u]);
                                continue;
                            }
                            bool hit = false;
                            if (mine[u]) {
                                if constexpr (kExactAct) hit = truncate_pack_h2(d[u], y[u], tr[u], act_s, thr2_s);
                                else hit = truncate_pack_f32(d[u], y[u], tr[u], act_s, thr_s);
                            }
                            const bool active = group_any(hit, gs, lane);
                            if (mine[u]) {
                                if (active) {
                                    Pack<__half, 8> z; z.zero();
                                    y[u].store(prev_s + off[u]);
                                    d[u].store(out_s + off[u]);
                                    z.store(trunc_s + off[u]);
                                } else {
                                    tr[u].store(trunc_s + off[u]);
                                }
                            }
                            const int r = rb + u * ppws + lane / gs;
                            if (ligs == 0 && row_on(r)) mo_s[q[u]] = active ? 1 : 0;
                        }
                    }
                }
                ++nt;
                continue;
            }
            // tensor memory -> fp16 staging tile (row = TMEM lane)
            {
                const int quarter = warp & 3;
                const int r = quarter * 32 + lane;
                uint8_t* srow = sStage + (size_t)r * p.stage_pitch;
#pragma unroll 1
                for (int c0 = (ew >> 2) * 16; c0 < p.bn; c0 += 32) {
                    uint32_t acc[16];
                    tmem_ld16(tmem_base + (uint32_t)(buf * p.tmem_cols) + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, acc);
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
            epi_bar_sync();
            if (etid == 0) {                                       // the accumulator is staged: the next tile may use it
                mbar_arrive(bar(kAccEmpty + buf));
                mbar_arrive(bar(kInfoEmpty + slot));
                if (t < 4) HALO_STAMP(28 + t);
            }
            __syncwarp();
#pragma unroll 1
            for (int rb = rb_first; rb < kRows; rb += rb_step) {
                if (rb != rb_first) load_caches(rb);
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const int r = rb + u * ppw + lane / g;
                    if (mine[u]) {
                        if (!kRes || row_on(r)) d[u].load(reinterpret_cast<const __half*>(sStage + (size_t)r * p.stage_pitch) + lig * 8);
                        else d[u].zero();                          // only the residual is active here: the staged row is not a result
                    }
                }
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    if constexpr (kEpi == 2) {                     // the arithmetic of dc_add without activation: one half addition
                        if (mine[u]) {
                            __half2* dh = reinterpret_cast<__half2*>(d[u].s);
                            const __half2* rh = reinterpret_cast<const __half2*>(tr[u].s);
#pragma unroll
                            for (int k = 0; k < 4; ++k) dh[k] = __hadd2(dh[k], rh[k]);
                            d[u].store(p.out + off[u]);
                        }
                        continue;
                    }
                    if constexpr (kEpi == 3) {                     // s = a + b in fp32, u = round(y + s), out = f(u) - f(y): dc_add bit for bit
                        if (mine[u]) {
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                const float yo = y[u].get(k);
                                const float uu = rnd<__half>(yo + (d[u].get(k) + tr[u].get(k)));
                                y[u].set(k, uu);
                                d[u].set(k, act_apply(uu, p.res_act) - act_apply(yo, p.res_act));
                            }
                            y[u].store(p.res_prev + off[u]);
                            d[u].store(p.out + off[u]);
                        }
                        continue;
                    }
                    if (!kFused) {
                        if (mine[u]) d[u].store(p.out + off[u]);
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
                    if (lig == 0 && row_on(r)) p.mo[q[u]] = active ? 1 : 0;
                }
            }
            if (etid == 0 && t < 4) HALO_STAMP(32 + t);
            ++nt;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0) HALO_STAMP(40);
    if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)(2 * p.tmem_cols));
}

// ---- host side ------------------------------------------------------------------------------------

bool encode_patch_map(CUtensorMap* map, const void* in, const dc_conv_desc* d, int tw, int th, int box_c);

struct HaloPlan {
    bool ok;
    int bn, ncb, tmem_cols, nA, nB, b_resident, ctas_per_sm;
    uint32_t off_b, off_stage, off_misc, stage_pitch;
    size_t smem;
};

static HaloPlan plan_halo(const dc_conv_desc* d, bool a64_allowed, int seg_cout = 0) {
    HaloPlan pl{};
    // at most 32 input channels: halo rows of 64 bytes (64-byte swizzle), half the stage
    const size_t a_stage = (size_t)kHaloRows * kHaloPitch * ((d->c_in <= 32 && a64_allowed) ? 64 : 128);
    pl.ok = d->dtype == DC_F16 && d->groups == 1 && d->kh == 3 && d->kw == 3 && d->stride_h == 1 && d->stride_w == 1 &&
            d->dil_h == 1 && d->dil_w == 1 && d->c_in % 8 == 0 && d->c_in >= 16 && d->c_out % 8 == 0 && d->c_out >= 16 && d->c_out <= 256 &&
            d->pad_top <= 1 && d->pad_left <= 1 && d->h_out >= 8 && d->w_out >= 8;
    if (!pl.ok) return pl;
    pl.bn = divup(d->c_out, 16) * 16;
    pl.ncb = divup(d->c_in, kKBlock);
    pl.tmem_cols = 32;
    while (pl.tmem_cols < pl.bn) pl.tmem_cols <<= 1;
    const size_t b_block = (size_t)pl.bn * 128;
    // the staging tile holds one segment of the output channels at a time when the layer has several (else all of them)
    pl.stage_pitch = (uint32_t)(seg_cout > 0 ? seg_cout : pl.bn) * 2 + 16;
    const size_t staging = ((size_t)kRows * pl.stage_pitch + 1023) & ~(size_t)1023;
    const size_t misc = 8 * 72 + 64 + kHaloInfo * kHaloInfoWords * 4 + kHaloInfo * kHaloCodesPitch + 4 * 256 + 4 * kHaloRawPitch * 4 + 64;
    const size_t budget = 227 * 1024 - 1024;
    const size_t resident = 9 * (size_t)pl.ncb * b_block;
    pl.ok = false;
    for (int nA = 3; nA >= 2 && !pl.ok; --nA) {
        if (resident <= 96 * 1024 && nA * a_stage + resident + staging + misc <= budget) {
            pl.ok = true; pl.nA = nA; pl.b_resident = 1; pl.nB = 0;
        }
    }
    // a streamed filter block has to carry enough MMA work to cover its copy: wide N tiles only
    if (!pl.ok && pl.bn >= 128) {
        for (int nA = 3; nA >= 2 && !pl.ok; --nA)
            for (int nB = kHaloMaxB; nB >= 4 && !pl.ok; --nB)
                if (nA * a_stage + nB * b_block + staging + misc <= budget) {
                    pl.ok = true; pl.nA = nA; pl.b_resident = 0; pl.nB = nB;
                }
    }
    if (!pl.ok) return pl;
    const size_t b_bytes = pl.b_resident ? resident : pl.nB * b_block;
    pl.off_b = (uint32_t)((pl.nA * a_stage + 1023) & ~(size_t)1023);
    pl.off_stage = (uint32_t)((pl.off_b + b_bytes + 1023) & ~(size_t)1023);
    pl.off_misc = (uint32_t)(pl.off_stage + staging);
    pl.smem = pl.off_misc + misc + 1024 /* alignment slack */;
    // a smaller footprint (two stages) that lets two CTAs share an SM beats a third stage
    if (pl.b_resident && pl.nA == 3) {
        const size_t two = 2 * a_stage + resident + staging + misc + 2048;
        if (2 * (two + 1024) <= 227 * 1024 && 4 * pl.tmem_cols <= 512) {
            pl.nA = 2;
            pl.off_b = (uint32_t)((2 * a_stage + 1023) & ~(size_t)1023);
            pl.off_stage = (uint32_t)((pl.off_b + b_bytes + 1023) & ~(size_t)1023);
            pl.off_misc = (uint32_t)(pl.off_stage + staging);
            pl.smem = pl.off_misc + misc + 1024;
        }
    }
    pl.ctas_per_sm = (2 * (pl.smem + 1024) <= 227 * 1024 && 4 * pl.tmem_cols <= 512) ? 2 : 1;
    pl.ok = pl.smem <= 227 * 1024;
    return pl;
}

// Returns DC_ERR_UNSUPPORTED when the layer has no halo-tile form (the caller then uses the other kernels); *fused_out
// tells whether the truncation step ran in the epilogue.
int conv3x3_halo(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, void* out, int32_t* mo,
                 const dc_epilogue* ep, uint32_t b_kb_stride, int* fused_out, cudaStream_t st) {
    static const int mode = [] { const char* e = getenv("DC_HALO"); return e != nullptr ? atoi(e) : 1; }();   // DC_HALO=0 turns the halo-tile form off
    if (mode == 0) return DC_ERR_UNSUPPORTED;
    static const bool a64_allowed = [] { const char* e = getenv("DC_HALO_A64"); return !(e != nullptr && e[0] == '0'); }();   // DC_HALO_A64=0: 128-byte rows for every layer
    HaloPlan pl = plan_halo(d, a64_allowed);
    if (!pl.ok || mi == nullptr || mo == nullptr) return DC_ERR_UNSUPPORTED;
    const bool has_res = ep != nullptr && ep->residual != nullptr;
    const bool fused = ep != nullptr && !has_res && ep->truncation == DC_TRUNC_MAX;
    if (fused && (!aligned16(ep->prev_out) || !aligned16(ep->truncated))) return DC_ERR_ALIGNMENT;
    const bool res_act = has_res && ep->activation != DC_ACT_NONE;
    if (has_res && (ep->residual_mask == nullptr || ep->truncation != DC_TRUNC_NONE || !aligned16(ep->residual) ||
                    (res_act && (ep->prev_out == nullptr || !aligned16(ep->prev_out)))))
        return DC_ERR_UNSUPPORTED;
    alignas(64) CUtensorMap tmap;
    memset(&tmap, 0, sizeof(tmap));
    const bool a64 = d->c_in <= 32 && a64_allowed;
    if (!encode_patch_map(&tmap, in, d, kHaloPitch, kHaloRows, a64 ? 32 : kKBlock)) return DC_ERR_UNSUPPORTED;
    HaloParams p{};
    p.mi = mi; p.wimg = (const uint8_t*)filt; p.bias = (const __half*)bias;
    p.out = (__half*)out; p.mo = mo;
    p.prev = fused ? (__half*)ep->prev_out : nullptr;
    p.trunc = fused ? (__half*)ep->truncated : nullptr;
    p.thr = fused ? host_round_threshold<__half>(ep->threshold) : 0.f;
    p.act = fused ? ep->activation : 0;
    p.res = has_res ? (const __half*)ep->residual : nullptr;
    p.res_mask = has_res ? ep->residual_mask : nullptr;
    p.res_prev = res_act ? (__half*)ep->prev_out : nullptr;
    p.res_act = has_res ? ep->activation : 0;
    p.h = d->h_in; p.w = d->w_in; p.ho = d->h_out; p.wo = d->w_out; p.pt = d->pad_top; p.pl = d->pad_left;
    p.cin = d->c_in; p.cout = d->c_out; p.ncb = pl.ncb; p.bn = pl.bn; p.tmem_cols = pl.tmem_cols;
    p.last_ksteps = (d->c_in - (pl.ncb - 1) * kKBlock + 15) >> 4;
    p.nA = pl.nA; p.nB = pl.nB; p.b_resident = pl.b_resident;
    p.b_kb_stride = b_kb_stride;
    p.patch_px = divup(d->w_out, kHaloTw);
    p.patch_py = divup(d->h_out, kHaloTh);
    p.npatches = (int64_t)d->n * p.patch_px * p.patch_py;
    if (p.npatches > 0x7fffffffLL) return DC_ERR_UNSUPPORTED;
    fast_div_init((uint32_t)p.patch_px, &p.ppx_mul, &p.ppx_shift);
    fast_div_init((uint32_t)(p.patch_px * p.patch_py), &p.ppi_mul, &p.ppi_shift);
    p.off_b = pl.off_b; p.off_stage = pl.off_stage; p.off_misc = pl.off_misc; p.stage_pitch = pl.stage_pitch;
    { const char* e = getenv("DC_HALO_DBG"); p.dbg = e != nullptr ? atoi(e) : 0; }
    static PerDeviceOnce attr_once;
    bool* attr_set = attr_once.slot();
    if (attr_set == nullptr) return DC_ERR_LAUNCH;
    if (!*attr_set) {
        bool ok_attr = true;
#define DC_HALO_ATTR(E, X) \
        ok_attr &= cudaFuncSetAttribute(k_conv3x3_halo<E, X, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess; \
        ok_attr &= cudaFuncSetAttribute(k_conv3x3_halo<E, X, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess; \
        ok_attr &= cudaFuncSetAttribute(k_conv3x3_halo<E, X, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess; \
        ok_attr &= cudaFuncSetAttribute(k_conv3x3_halo<E, X, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess
        DC_HALO_ATTR(0, true); DC_HALO_ATTR(1, true); DC_HALO_ATTR(1, false); DC_HALO_ATTR(2, true); DC_HALO_ATTR(3, true);
#undef DC_HALO_ATTR
        if (!ok_attr) return check_launch();
        *attr_set = true;
    }
    int64_t persistent = (int64_t)sm_count() * pl.ctas_per_sm;
    const dim3 grid((unsigned)(p.npatches < persistent ? p.npatches : persistent));
    const bool exact_act = !fused || (p.act >= DC_ACT_NONE && p.act <= DC_ACT_RELU6);
    int rc;
    // rows per round of the epilogue's cache reads: 8 warps x (32 / lanes per row) x kU
    int lanes_row = 1;
    while (lanes_row < d->c_out / 8 && lanes_row < 32) lanes_row <<= 1;
    const bool deep = pl.ctas_per_sm == 1 && 8 * (32 / lanes_row) * 2 < kRows;
#define DC_HALO_LAUNCH(E, X)                                                                                              \
    do {                                                                                                                  \
        if (a64) rc = deep ? launch_pdl(k_conv3x3_halo<E, X, 4, true>, grid, dim3(kHaloThreads), pl.smem, st, p, tmap)    \
                           : launch_pdl(k_conv3x3_halo<E, X, 2, true>, grid, dim3(kHaloThreads), pl.smem, st, p, tmap);   \
        else rc = deep ? launch_pdl(k_conv3x3_halo<E, X, 4, false>, grid, dim3(kHaloThreads), pl.smem, st, p, tmap)       \
                       : launch_pdl(k_conv3x3_halo<E, X, 2, false>, grid, dim3(kHaloThreads), pl.smem, st, p, tmap);      \
    } while (0)
    if (has_res && res_act) DC_HALO_LAUNCH(3, true);
    else if (has_res) DC_HALO_LAUNCH(2, true);
    else if (!fused) DC_HALO_LAUNCH(0, true);
    else if (exact_act) DC_HALO_LAUNCH(1, true);
    else DC_HALO_LAUNCH(1, false);
#undef DC_HALO_LAUNCH
    if (fused_out != nullptr) *fused_out = (fused || has_res) ? 1 : 0;
    return rc;
}

// Several 3x3 layers on the same input in one launch (see HaloParams::nseg): ``d`` describes the concatenated layer
// (c_out = all output channels), the packed filter and the bias are the concatenation along the output channels.
int conv3x3_halo_heads(const dc_conv_desc* d, const void* in, const int32_t* mi, const void* filt, const void* bias, int nseg,
                       void* const* outs, int32_t* const* mos, const dc_epilogue* eps, uint32_t b_kb_stride, bool plan_only, cudaStream_t st) {
    if (nseg < 2 || nseg > 4 || d->c_out % nseg != 0 || (d->c_out / nseg) % 16 != 0) return DC_ERR_UNSUPPORTED;
    const int seg_cout = d->c_out / nseg;
    HaloPlan pl = plan_halo(d, false, seg_cout);
    if (!pl.ok) return DC_ERR_UNSUPPORTED;
    if (plan_only) return DC_OK;
    if (mi == nullptr || in == nullptr || filt == nullptr || outs == nullptr || mos == nullptr) return DC_ERR_NULL_POINTER;
    const bool fused = eps != nullptr;
    bool exact_act = true;
    HaloParams p{};
    for (int sg = 0; sg < nseg; ++sg) {
        if (outs[sg] == nullptr || mos[sg] == nullptr || !aligned16(outs[sg])) return DC_ERR_NULL_POINTER;
        p.seg_out[sg] = (__half*)outs[sg];
        p.seg_mo[sg] = mos[sg];
        if (fused) {
            const dc_epilogue& e = eps[sg];
            if (e.residual != nullptr || e.truncation != DC_TRUNC_MAX || e.prev_out == nullptr || e.truncated == nullptr ||
                !aligned16(e.prev_out) || !aligned16(e.truncated))
                return DC_ERR_UNSUPPORTED;
            p.seg_prev[sg] = (__half*)e.prev_out;
            p.seg_trunc[sg] = (__half*)e.truncated;
            p.seg_thr[sg] = host_round_threshold<__half>(e.threshold);
            p.seg_act[sg] = e.activation;
            exact_act = exact_act && e.activation >= DC_ACT_NONE && e.activation <= DC_ACT_RELU6;
        }
    }
    alignas(64) CUtensorMap tmap;
    memset(&tmap, 0, sizeof(tmap));
    if (!encode_patch_map(&tmap, in, d, kHaloPitch, kHaloRows, kKBlock)) return DC_ERR_UNSUPPORTED;
    p.mi = mi; p.wimg = (const uint8_t*)filt; p.bias = (const __half*)bias;
    p.nseg = nseg; p.seg_cout = seg_cout;
    p.h = d->h_in; p.w = d->w_in; p.ho = d->h_out; p.wo = d->w_out; p.pt = d->pad_top; p.pl = d->pad_left;
    p.cin = d->c_in; p.cout = d->c_out; p.ncb = pl.ncb; p.bn = pl.bn; p.tmem_cols = pl.tmem_cols;
    p.last_ksteps = (d->c_in - (pl.ncb - 1) * kKBlock + 15) >> 4;
    p.nA = pl.nA; p.nB = pl.nB; p.b_resident = pl.b_resident;
    p.b_kb_stride = b_kb_stride;
    p.patch_px = divup(d->w_out, kHaloTw);
    p.patch_py = divup(d->h_out, kHaloTh);
    p.npatches = (int64_t)d->n * p.patch_px * p.patch_py;
    if (p.npatches > 0x7fffffffLL) return DC_ERR_UNSUPPORTED;
    fast_div_init((uint32_t)p.patch_px, &p.ppx_mul, &p.ppx_shift);
    fast_div_init((uint32_t)(p.patch_px * p.patch_py), &p.ppi_mul, &p.ppi_shift);
    p.off_b = pl.off_b; p.off_stage = pl.off_stage; p.off_misc = pl.off_misc; p.stage_pitch = pl.stage_pitch;
    static PerDeviceOnce attr_once;
    bool* attr_set = attr_once.slot();
    if (attr_set == nullptr) return DC_ERR_LAUNCH;
    if (!*attr_set) {
        bool ok_attr = true;
        ok_attr &= cudaFuncSetAttribute(k_conv3x3_halo<0, true, 4, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        ok_attr &= cudaFuncSetAttribute(k_conv3x3_halo<1, true, 4, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        ok_attr &= cudaFuncSetAttribute(k_conv3x3_halo<1, false, 4, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        if (!ok_attr) return check_launch();
        *attr_set = true;
    }
    const int64_t persistent = sm_count();                     // these variants keep an SM to themselves
    const dim3 grid((unsigned)(p.npatches < persistent ? p.npatches : persistent));
    if (!fused) return launch_pdl(k_conv3x3_halo<0, true, 4, false, true>, grid, dim3(kHaloThreads), pl.smem, st, p, tmap);
    if (exact_act) return launch_pdl(k_conv3x3_halo<1, true, 4, false, true>, grid, dim3(kHaloThreads), pl.smem, st, p, tmap);
    return launch_pdl(k_conv3x3_halo<1, false, 4, false, true>, grid, dim3(kHaloThreads), pl.smem, st, p, tmap);
}

#ifdef DC_HALO_STAMPS
extern "C" int dc_halo_debug_stamps(long long* out64) {
    return cudaMemcpyFromSymbol(out64, g_halo_stamps, 64 * sizeof(long long)) == cudaSuccess ? 0 : 1;
}
#endif

int halo_error_code() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_halo_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

}  // namespace dc

using namespace dc;

extern "C" {

// rows of a K block of the packed tensor-core filter image (the layout of dc_pack_filter_umma): the output channels
// rounded up to 256, plus room for a ragged last N tile
static uint32_t umma_kb_stride(const dc_conv_desc* d) { return (uint32_t)(divup(d->c_out, 256) * 256 + 256) * 128u; }

int dc_conv3x3_heads_supported(const dc_conv_desc* desc, int32_t n_heads) {
    if (desc == nullptr) return 0;
    return conv3x3_halo_heads(desc, nullptr, nullptr, nullptr, nullptr, n_heads, nullptr, nullptr, nullptr, 0u, true, nullptr) == DC_OK ? 1 : 0;
}

int dc_conv3x3_heads(const dc_conv_desc* desc, const void* in, const int32_t* mask_in, const void* filter_umma, const void* bias,
                     int32_t n_heads, void* const* outs, int32_t* const* masks_out, const dc_epilogue* epilogues, void* stream) {
    if (desc == nullptr) return DC_ERR_NULL_POINTER;
    if (!aligned16(in) || !aligned16(filter_umma)) return DC_ERR_ALIGNMENT;
    if ((int64_t)desc->n * desc->h_out * desc->w_out == 0) return DC_OK;
    return conv3x3_halo_heads(desc, in, mask_in, filter_umma, bias, n_heads, outs, masks_out, epilogues, umma_kb_stride(desc), false,
                              (cudaStream_t)stream);
}

}  // extern "C"

