// Fused inverted-residual block for small feature maps (sm_100a): expansion 1x1 -> ReLU6 + truncation ->
// depthwise 3x3 -> ReLU6 + truncation -> projection 1x1 (+ residual), one kernel, for steady-state frames.
//
// On small maps (14x14, 7x7) the update masks of a network saturate, so the three convolutions of a block are dense
// work on a few hundred pixels per stream and the separate kernels are bound by launch and dependent-latency floors,
// not by bytes. Here a CTA owns a band of output rows of ONE stream: the expanded tensor of the band (own rows plus
// the halo rows the depthwise filter needs) lives in shared memory from the first GEMM to the second, and only the
// block input, the four truncation caches and the block output touch global memory.
//
//   A  gather the band's input rows (active pixels; zeros otherwise) into the 128-byte-swizzled K-major layout
//   B  expansion GEMM on tcgen05 in chunks of output channels (double-buffered accumulators in tensor memory, filter
//      chunks by bulk copy), each chunk converted to fp16 into the buffer E[K block][pixel slot][64 channels]
//   C  truncation step of the expansion: a warp owns a pixel's whole channel vector (the any-channel decision is a
//      warp vote); halo pixels are computed (they belong to the neighbouring band, which writes their caches) before a
//      cluster barrier, own pixels after it, so a neighbour never reads caches that were already updated
//   D  depthwise 3x3 from E and its truncation step, a warp per output pixel; the result overwrites E in place (the
//      rows of E a finished output row no longer needs), already in the operand layout of the second GEMM
//   E  projection GEMM on tcgen05, filter K blocks streamed through a ring of bulk copies
//   F  tensor memory -> fp16 staging -> coalesced rows, residual added where it is active, out-mask
//
// Arithmetic and rounding are those of the separate kernels (dc_conv_umma.cu, dc_dwconv_strip.cu): fp32 accumulation,
// one rounding to half per stored value, truncation in packed half arithmetic, so the block's outputs and caches
// are the same bit for bit. Every mbarrier wait is bounded; a wait that gives up sets the sticky error code of the
// tensor-core kernels and the CTA still takes part in the cluster barrier and frees its tensor memory.
#include "dc_umma.cuh"

namespace dc {

__device__ int g_irb_error = 0;       // sticky: the bounded wait that gave up (2 filter copy, 3 accumulator)
#ifdef DC_IRB_STAMPS                  // development build: phase time stamps of CTA (0, 0)
__device__ long long g_irb_stamps[16];
#define IRB_STAMP(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) g_irb_stamps[i] = clock64(); } while (0)
#else
#define IRB_STAMP(i) do { } while (0)
#endif

constexpr int kIrbThreads = 512;
constexpr int kIrbWarps = kIrbThreads / 32;
constexpr int kIrbMaxPacks = 4;              // 16-byte channel packs per lane: hidden channels <= 4 * 32 * 8 = 1024

struct IrbParams {
    const __half* x; const int32_t* mask_in;
    const uint8_t* w1; const __half* wd; const uint8_t* w2;
    __half* prev1; __half* trunc1; __half* prev2; __half* trunc2;
    __half* out; int32_t* mask_out;
    float thr1, thr2;
    int act1, act2, residual;
    int h, w, ho, wo, s;
    int cin, chid, cout;
    int nkb1, nkb2, last_ksteps1;
    int nc, nchunks, acc_stride;     // expansion: output channels per chunk, chunks, tensor-memory columns between the two accumulators
    int ntile2, bn2;                 // projection: N tiles (<= 256 wide)
    int rows_per_band, rows_per_round;
    uint32_t w1_kb_stride, w2_kb_stride;      // bytes between K blocks of the packed filter images
    int tmem_cols;
    uint32_t e_kb_bytes;             // bytes of one K block of E / of the gathered input (pixel slots rounded up to 8 rows)
    uint32_t off_x, off_w1, off_wd, off_misc, w1_buf_bytes;
    uint32_t off_w2, w2_stage_bytes; int w2_stages;
    uint32_t stage_pitch;
};

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// byte offset of 16-byte chunk `c` (8 channels) of pixel slot `r` inside one K block of 64 channels
__device__ __forceinline__ uint32_t swz(int r, int c) {
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

template <int NV>
__global__ void __launch_bounds__(kIrbThreads, 1) k_irb_umma(const IrbParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sE = smem;                                   // [nkb2][slot][64 ch], swizzled; later the output staging tile
    uint8_t* sX = smem + p.off_x;                         // [nkb1][slot][64 ch]
    uint8_t* sW1 = smem + p.off_w1;                       // two chunks of the expansion filter
    uint8_t* sW2 = smem + p.off_w2;                       // ring of projection filter K blocks (over sX / sW1, free by then)
    __half* sWd = reinterpret_cast<__half*>(smem + p.off_wd);       // depthwise filter [9][chid]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_misc);
    // bars[0..1] expansion filter chunk landed, [2..3] expansion accumulator done, [4] projection done,
    // [5..5+8) projection filter stage landed, [13..13+8) projection filter stage free
    int* s_pix = reinterpret_cast<int*>(bars + 24);       // [128] global pixel of a slot, -1 outside the image
    uint8_t* s_min = reinterpret_cast<uint8_t*>(s_pix + 128);       // [128] in-mask of the slot
    uint8_t* s_f1 = s_min + 128;                          // [128] slot active after the expansion's truncation
    uint8_t* s_f2 = s_f1 + 128;                           // [128] output pixel active after the depthwise truncation
    uint8_t* s_own = s_f2 + 128;                          // [128] slot belongs to this band (its caches are written here)
    uint8_t* s_lown = s_own + 128;                        // [128] active slots of this band, in slot order
    uint8_t* s_lhalo = s_lown + 128;                      // [128] active halo slots (owned by a neighbouring band)
    uint32_t* s_u32 = reinterpret_cast<uint32_t*>(s_lhalo + 128);   // [0] tmem base, [1] ok flag, [2] halo slots, [3] own slots

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x, band = blockIdx.y;
    const uint32_t bar0 = smem_u32(bars);
    auto bar_w1 = [&](int i) { return bar0 + 8u * i; };
    auto bar_acc = [&](int i) { return bar0 + 8u * (2 + i); };
    const uint32_t bar_fin = bar0 + 8u * 4;
    auto bar_w2_full = [&](int i) { return bar0 + 8u * (5 + i); };
    auto bar_w2_free = [&](int i) { return bar0 + 8u * (13 + i); };

    // ---- geometry of this band ----
    const int o0 = band * p.rows_per_band, o1 = min(p.ho, o0 + p.rows_per_band);     // own output rows
    const int i0 = o0 * p.s - 1;                                                    // first input row of the slots (may be -1)
    const int n_in_rows = (o1 - o0 - 1) * p.s + 3;
    const int r_in = n_in_rows * p.w;                                               // slots in use (<= 128)
    const int rows8 = (r_in + 7) & ~7;
    const int own_lo = o0 * p.s, own_hi = (band == (int)gridDim.y - 1) ? p.h : o1 * p.s;   // own input rows
    const int r_out = (o1 - o0) * p.wo;                                             // own output pixels
    const int npk = p.chid >> 3;                                                    // 16-byte packs of the hidden channel vector

    // ---- set-up from constants: overlaps the previous kernel's tail ----
    if (tid < 21) {
        mbar_init(bar0 + 8u * tid, 1u);
        fence_barrier_init();
    }
    if (tid == 0) s_u32[1] = 1;
    for (int i = tid; i < 9 * npk; i += kIrbThreads)
        reinterpret_cast<uint4*>(sWd)[i] = __ldg(reinterpret_cast<const uint4*>(p.wd) + i);
    if (warp == 0) tmem_alloc(smem_u32(&s_u32[0]), (uint32_t)p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_dep_launch();                 // only after the tensor memory is held (a dependent CTA allocates before it waits)
    const uint32_t tmem_base = s_u32[0];
    volatile uint32_t* ok_flag = &s_u32[1];
    IRB_STAMP(0);
    const uint32_t w1_chunk_bytes = (uint32_t)p.nc * 128u;                          // one K block of a chunk
    auto load_w1 = [&](int j, int buf) {                                            // thread 0 only
        mbar_expect_tx(bar_w1(buf), (uint32_t)p.nkb1 * w1_chunk_bytes);
        for (int kb = 0; kb < p.nkb1; ++kb)
            bulk_g2s(smem_u32(sW1 + (size_t)buf * p.w1_buf_bytes + (size_t)kb * w1_chunk_bytes),
                     p.w1 + (size_t)kb * p.w1_kb_stride + (size_t)j * w1_chunk_bytes, w1_chunk_bytes, bar_w1(buf));
    };
    if (tid == 0) {                    // the filters are constants: start before waiting for the previous kernel
        load_w1(0, 0);
        if (p.nchunks > 1) load_w1(1, 1);
    }
    grid_dep_wait();

    // ---- A: slot table and input gather ----
    IRB_STAMP(1);
    if (tid < 128) {
        const int slot = tid;
        const int ry = slot / p.w, ix = slot - ry * p.w;
        const int iy = i0 + ry;
        const bool inb = slot < r_in && iy >= 0 && iy < p.h;
        const int pix = inb ? (b * p.h + iy) * p.w + ix : -1;
        s_pix[slot] = pix;
        s_min[slot] = (inb && p.mask_in[pix] != 0) ? 1 : 0;
        s_own[slot] = (inb && iy >= own_lo && iy < own_hi) ? 1 : 0;
        s_f1[slot] = 0;
        s_f2[slot] = 0;
    }
    __syncthreads();
    if (warp == kIrbWarps - 1) {          // compact the active slots (own / halo) in slot order: ballots and running counts
        int n_own = 0, n_halo = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int slot = c * 32 + lane;
            const bool a = s_min[slot] != 0, o = s_own[slot] != 0;
            const unsigned bo = __ballot_sync(DC_FULL, a && o), bh = __ballot_sync(DC_FULL, a && !o);
            const unsigned lt = (1u << lane) - 1u;
            if (a && o) s_lown[n_own + __popc(bo & lt)] = (uint8_t)slot;
            if (a && !o) s_lhalo[n_halo + __popc(bh & lt)] = (uint8_t)slot;
            n_own += __popc(bo);
            n_halo += __popc(bh);
        }
        if (lane == 0) { s_u32[2] = (uint32_t)n_halo; s_u32[3] = (uint32_t)n_own; }
    }
    {
        const int chunk = tid & 7, row0 = tid >> 3;                                 // 64 rows per pass
        const uint32_t sX_u32 = smem_u32(sX);
        for (int kb = 0; kb < p.nkb1; ++kb) {
            const int kk = kb * kKBlock + chunk * 8;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int r = row0 + 64 * j;
                if (r < rows8) {
                    const bool real = s_min[r] != 0 && kk < p.cin;
                    const __half* src = real ? p.x + (int64_t)s_pix[r] * p.cin + kk : p.x;
                    cp_async16(sX_u32 + (uint32_t)kb * p.e_kb_bytes + swz(r, chunk), src, real ? 16u : 0u);
                }
            }
        }
        cp_async_commit();
        cp_async_wait_group<0>();
        fence_proxy_async();
    }
    __syncthreads();

    IRB_STAMP(2);

    // ---- B: expansion GEMM, chunk by chunk; chunk j+1 runs on the tensor core while chunk j is converted ----
    const uint32_t idesc1 = make_idesc(p.nc);
    auto issue_expand = [&](int j) {                                                // the elected lane of warp 0 only
        const int buf = j & 1;
        const uint64_t ad0 = make_smem_desc(smem_u32(sX));
        const uint64_t bd0 = make_smem_desc(smem_u32(sW1 + (size_t)buf * p.w1_buf_bytes));
        for (int kb = 0; kb < p.nkb1; ++kb) {
            const int ksteps = kb == p.nkb1 - 1 ? p.last_ksteps1 : kKBlock / 16;
            const uint64_t ad = ad0 + (uint64_t)((uint32_t)kb * (p.e_kb_bytes >> 4));
            const uint64_t bd = bd0 + (uint64_t)((uint32_t)kb * (w1_chunk_bytes >> 4));
            for (int ks = 0; ks < ksteps; ++ks)
                umma_f16(tmem_base + (uint32_t)(buf * p.acc_stride), ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc1, (kb > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(bar_acc(buf));
    };
    // (MMAs are issued by an elected lane of converged warp 0: their operands sit in uniform registers)
    if (warp == 0 && elect_one()) {
        if (mbar_wait(bar_w1(0), 0u, ok_flag)) { tc_fence_after(); issue_expand(0); }
        else { *ok_flag = 0; atomicExch(&g_irb_error, 2); }
    }
    for (int j = 0; j < p.nchunks; ++j) {
        const int buf = j & 1;
        const uint32_t par = (uint32_t)((j >> 1) & 1);
        if (warp == 0 && j + 1 < p.nchunks && *ok_flag != 0 && elect_one()) {
            if (mbar_wait(bar_w1(buf ^ 1), (uint32_t)(((j + 1) >> 1) & 1), ok_flag)) { tc_fence_after(); issue_expand(j + 1); }
            else { *ok_flag = 0; atomicExch(&g_irb_error, 2); }
        }
        // (a wait also gives up when another thread has cleared the ok flag, so this cannot outlast a failure of thread 0)
        if (!mbar_wait_warp(bar_acc(buf), par, ok_flag)) { *ok_flag = 0; atomicExch(&g_irb_error, 3); }
        __syncthreads();
        if (*ok_flag == 0) break;                                                   // uniform: read after the barrier
        tc_fence_after();
        if (tid == 0 && j + 2 < p.nchunks) load_w1(j + 2, buf);                     // this buffer's MMAs are complete
        {   // tensor memory -> fp16 -> E: warp quarter = 32 pixel slots, column groups of 16 channels
            const int quarter = warp & 3;
            const int r = quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = (warp >> 2) * 16; c0 < p.nc; c0 += 16 * (kIrbWarps / 4)) {
                uint32_t acc[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * p.acc_stride + c0), acc);
                tmem_ld_wait();
                if (r < rows8) {
                    uint4 o[2];
                    __half2* hh = reinterpret_cast<__half2*>(o);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        hh[q] = __floats2half2_rn(__uint_as_float(acc[2 * q]) + 0.f, __uint_as_float(acc[2 * q + 1]) + 0.f);
                    const int ch = j * p.nc + c0;                                   // first hidden channel of the group
                    uint8_t* kbp = sE + (size_t)(ch >> 6) * p.e_kb_bytes;
                    const int c = (ch & 63) >> 3;
                    *reinterpret_cast<uint4*>(kbp + swz(r, c)) = o[0];
                    *reinterpret_cast<uint4*>(kbp + swz(r, c + 1)) = o[1];
                }
            }
        }
        tc_fence_before();
        __syncthreads();
    }
    IRB_STAMP(3);
    const bool ok_b = *ok_flag != 0;      // uniform (written before the last barrier of the loop, or read after a barrier)

    // the projection filter's first K blocks can come in while the truncation and depthwise phases run
    auto load_w2 = [&](int item) {                                                  // thread 0 only; item = K block * N tiles + N tile
        const int st = item % p.w2_stages;
        const int kb = item / p.ntile2, nt = item - kb * p.ntile2;
        mbar_expect_tx(bar_w2_full(st), p.w2_stage_bytes);
        bulk_g2s(smem_u32(sW2 + (size_t)st * p.w2_stage_bytes), p.w2 + (size_t)kb * p.w2_kb_stride + (size_t)nt * p.w2_stage_bytes,
                 p.w2_stage_bytes, bar_w2_full(st));
    };
    const int w2_items = p.nkb2 * p.ntile2;
    if (ok_b && tid == 0)
        for (int it = 0; it < p.w2_stages && it < w2_items; ++it) load_w2(it);

    // ---- C: truncation step of the expansion, a warp per pixel slot ----
    const __half2 thr1 = __float2half2_rn(p.thr1), thr2 = __float2half2_rn(p.thr2);
    constexpr int kU = NV >= 4 ? 1 : 2;          // pixel slots a warp has in flight at once (registers: 3 * NV packs each)
    auto truncate_slots = [&](const uint8_t* list, int count, bool own_pass) {
        for (int i = warp * kU; i < count; i += kIrbWarps * kU) {
            int r[kU];
            int64_t off[kU];
            bool val[kU];                                                           // warp-uniform
            Pack<__half, 8> d[kU][NV], y[kU][NV], t[kU][NV];
            bool tz[kU][NV];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                val[u] = i + u < count;
                r[u] = list[val[u] ? i + u : i];
                off[u] = (int64_t)s_pix[r[u]] * p.chid;
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const int pk = lane + 32 * j;
                    if (val[u] && pk < npk) {
                        y[u][j].load(p.prev1 + off[u] + pk * 8);
                        t[u][j].load(p.trunc1 + off[u] + pk * 8);
                        d[u][j].load(reinterpret_cast<const __half*>(sE + (size_t)(pk >> 3) * p.e_kb_bytes + swz(r[u], pk & 7)));
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                if (!val[u]) continue;
                bool hit = false;
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const int pk = lane + 32 * j;
                    if (pk < npk) {
                        const uint4 tv = *reinterpret_cast<const uint4*>(t[u][j].s);
                        tz[u][j] = ((tv.x | tv.y | tv.z | tv.w) & 0x7fff7fffu) == 0u;    // the carried residual is already zero
                        hit |= truncate_pack_h2(d[u][j], y[u][j], t[u][j], p.act1, thr1);
                    }
                }
                const bool active = __any_sync(DC_FULL, hit);
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const int pk = lane + 32 * j;
                    if (pk < npk) {
                        __half* e = reinterpret_cast<__half*>(sE + (size_t)(pk >> 3) * p.e_kb_bytes + swz(r[u], pk & 7));
                        Pack<__half, 8> z; z.zero();
                        if (active) {
                            d[u][j].store(e);
                            if (own_pass) {
                                y[u][j].store(p.prev1 + off[u] + pk * 8);
                                if (!tz[u][j]) z.store(p.trunc1 + off[u] + pk * 8);      // zero is what it holds already otherwise
                            }
                        } else {
                            z.store(e);
                            if (own_pass) t[u][j].store(p.trunc1 + off[u] + pk * 8);
                        }
                    }
                }
                if (lane == 0) s_f1[r[u]] = active ? 1 : 0;
            }
        }
    };
    if (ok_b) truncate_slots(s_lhalo, (int)s_u32[2], false);      // halo pixels: read-only here, the neighbouring band owns their caches
    IRB_STAMP(4);
    if (gridDim.y > 1) cluster_sync_all();        // every band has read its halo before any band updates a cache
    IRB_STAMP(5);
    if (ok_b) truncate_slots(s_lown, (int)s_u32[3], true);
    __syncthreads();

    IRB_STAMP(6);
    // ---- D: depthwise 3x3 + its truncation step, a warp per output pixel; results replace E in place ----
    if (ok_b) {
        const int rounds = (o1 - o0 + p.rows_per_round - 1) / p.rows_per_round;
        Pack<__half, 8> y[NV], t[NV];
        // pixel of round `rd` handled by this warp
        auto pixel_of = [&](int rd, int& orow, int& ox) -> bool {
            const int row_first = rd * p.rows_per_round;
            const int rows_here = min(p.rows_per_round, o1 - o0 - row_first);
            if (warp >= rows_here * p.wo) { orow = 0; ox = 0; return false; }
            orow = row_first + warp / p.wo;
            ox = warp - (warp / p.wo) * p.wo;
            return true;
        };
        // the two cache rows of a pixel are asked for one round ahead, so their latency hides behind the arithmetic
        auto load_caches = [&](int rd) {
            int orow, ox;
            if (!pixel_of(rd, orow, ox)) return;
            const int64_t off = (((int64_t)b * p.ho + o0 + orow) * p.wo + ox) * p.chid;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int pk = lane + 32 * j;
                if (pk < npk) {
                    y[j].load(p.prev2 + off + pk * 8);
                    t[j].load(p.trunc2 + off + pk * 8);
                }
            }
        };
        load_caches(0);
        for (int rd = 0; rd < rounds; ++rd) {
            int orow, ox;
            const bool have = pixel_of(rd, orow, ox);
            const int pout = orow * p.wo + ox;                                      // own output pixel index = slot of the result
            Pack<__half, 8> e2[NV];
            if (have) {
                // active taps: slot of tap (ky, kx) = (orow * s + ky) * w + ox * s - 1 + kx  (slot rows start at input row o0 * s - 1)
                unsigned tb = 0;
                const int sx0 = ox * p.s - 1, srow0 = orow * p.s;
#pragma unroll
                for (int t9 = 0; t9 < 9; ++t9) {
                    const int ix = sx0 + t9 % 3;
                    if (ix >= 0 && ix < p.w && s_f1[(srow0 + t9 / 3) * p.w + ix] != 0) tb |= 1u << t9;
                }
                const int64_t off = (((int64_t)b * p.ho + o0 + orow) * p.wo + ox) * p.chid;
                if (tb == 0u) {
#pragma unroll
                    for (int j = 0; j < NV; ++j) e2[j].zero();
                    if (lane == 0) s_f2[pout] = 0;
                } else {
                    bool tz[NV];
                    bool hit = false;
#pragma unroll
                    for (int j = 0; j < NV; ++j) {
                        const int pk = lane + 32 * j;
                        if (pk < npk) {
                            float2 acc[4];                  // fp32 accumulators, two channels per packed FMA (fma.rn.f32x2)
#pragma unroll
                            for (int q = 0; q < 4; ++q) acc[q] = make_float2(0.f, 0.f);
#pragma unroll
                            for (int t9 = 0; t9 < 9; ++t9) {
                                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                                if (tb & (1u << t9)) {
                                    const int slot = (srow0 + t9 / 3) * p.w + sx0 + t9 % 3;
                                    v = *reinterpret_cast<const uint4*>(sE + (size_t)(pk >> 3) * p.e_kb_bytes + swz(slot, pk & 7));
                                }
                                const uint4 wv = *reinterpret_cast<const uint4*>(sWd + (size_t)t9 * p.chid + pk * 8);
                                const __half2* hv = reinterpret_cast<const __half2*>(&v);
                                const __half2* hw = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
                                for (int q = 0; q < 4; ++q) acc[q] = __ffma2_rn(__half22float2(hv[q]), __half22float2(hw[q]), acc[q]);
                            }
                            __half2* dh = reinterpret_cast<__half2*>(e2[j].s);
#pragma unroll
                            for (int q = 0; q < 4; ++q) dh[q] = __float22half2_rn(acc[q]);
                            const uint4 tv = *reinterpret_cast<const uint4*>(t[j].s);
                            tz[j] = ((tv.x | tv.y | tv.z | tv.w) & 0x7fff7fffu) == 0u;
                            hit |= truncate_pack_h2(e2[j], y[j], t[j], p.act2, thr2);
                        }
                    }
                    const bool active = __any_sync(DC_FULL, hit);
#pragma unroll
                    for (int j = 0; j < NV; ++j) {
                        const int pk = lane + 32 * j;
                        if (pk < npk) {
                            if (active) {
                                y[j].store(p.prev2 + off + pk * 8);
                                if (!tz[j]) { Pack<__half, 8> z; z.zero(); z.store(p.trunc2 + off + pk * 8); }
                            } else {
                                t[j].store(p.trunc2 + off + pk * 8);
                                e2[j].zero();
                            }
                        }
                    }
                    if (lane == 0) s_f2[pout] = active ? 1 : 0;
                }
            }
            if (rd + 1 < rounds) load_caches(rd + 1);
            __syncthreads();              // every read of E for the round's output rows is done
            if (have) {
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const int pk = lane + 32 * j;
                    if (pk < npk)
                        e2[j].store(reinterpret_cast<__half*>(sE + (size_t)(pk >> 3) * p.e_kb_bytes + swz(pout, pk & 7)));
                }
            }
        }
        fence_proxy_async();              // E was written with ordinary stores and is read by the tensor core next
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    IRB_STAMP(7);
    // ---- E: projection GEMM, K = hidden channels in blocks of 64, filter blocks through the ring ----
    if (ok_b && warp == 0 && elect_one()) {
        const uint32_t idesc2 = make_idesc(p.bn2);
        const uint64_t ad0 = make_smem_desc(smem_u32(sE));
        const uint64_t bd0 = make_smem_desc(smem_u32(sW2));
        bool fine = true;
        for (int it = 0; it < w2_items && fine; ++it) {
            const int st = it % p.w2_stages;
            const uint32_t par = (uint32_t)((it / p.w2_stages) & 1);
            const int kb = it / p.ntile2, nt = it - kb * p.ntile2;
            if (!mbar_wait(bar_w2_full(st), par, ok_flag)) { fine = false; break; }
            tc_fence_after();
            const uint64_t ad = ad0 + (uint64_t)((uint32_t)kb * (p.e_kb_bytes >> 4));
            const uint64_t bd = bd0 + (uint64_t)(((uint32_t)st * p.w2_stage_bytes) >> 4);
            for (int ks = 0; ks < kKBlock / 16; ++ks)
                umma_f16(tmem_base + (uint32_t)(nt * p.bn2), ad + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), idesc2, (kb > 0 || ks > 0) ? 1u : 0u);
            umma_commit(bar_w2_free(st));
            if (it + p.w2_stages < w2_items) {
                if (!mbar_wait(bar_w2_free(st), par, ok_flag)) { fine = false; break; }
                load_w2(it + p.w2_stages);
            }
        }
        if (fine) umma_commit(bar_fin);
        else { *ok_flag = 0; atomicExch(&g_irb_error, 2); }
    }
    if (ok_b && !mbar_wait_warp(bar_fin, 0u, ok_flag)) { *ok_flag = 0; atomicExch(&g_irb_error, 3); }
    __syncthreads();
    const bool ok_e = ok_b && *ok_flag != 0;
    tc_fence_after();

    IRB_STAMP(8);
    // ---- F: tensor memory -> fp16 staging tile (over E) -> coalesced rows, residual, out-mask ----
    if (ok_e) {
        {
            const int quarter = warp & 3;
            const int r = quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = (warp >> 2) * 16; c0 < p.cout; c0 += 16 * (kIrbWarps / 4)) {
                uint32_t acc[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, acc);
                tmem_ld_wait();
                if (r < r_out) {
                    uint4 o[2];
                    __half2* hh = reinterpret_cast<__half2*>(o);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        hh[q] = __floats2half2_rn(__uint_as_float(acc[2 * q]) + 0.f, __uint_as_float(acc[2 * q + 1]) + 0.f);
                    uint8_t* srow = sE + (size_t)r * p.stage_pitch + c0 * 2;
                    *reinterpret_cast<uint4*>(srow) = o[0];
                    *reinterpret_cast<uint4*>(srow + 16) = o[1];
                }
            }
        }
        tc_fence_before();
        __syncthreads();
        const int npo = p.cout >> 3;
        for (int pr = warp; pr < r_out; pr += kIrbWarps) {
            const int orow = pr / p.wo, ox = pr - orow * p.wo;
            const int64_t gq = ((int64_t)b * p.ho + o0 + orow) * p.wo + ox;
            const bool on = s_f2[pr] != 0;
            // residual: the block input at the same pixel (stride 1, same shape), where its mask is set; its row is
            // still in the gathered input tile (the projection filter's ring leaves that tile alone in this case)
            const int slot_in = (orow + 1) * p.w + ox;
            const bool ron = p.residual != 0 && s_min[slot_in] != 0;
            if (lane == 0) p.mask_out[gq] = (on || ron) ? 1 : 0;
            if (!(on || ron)) continue;
            for (int pk = lane; pk < npo; pk += 32) {
                Pack<__half, 8> d;
                if (on) d.load(reinterpret_cast<const __half*>(sE + (size_t)pr * p.stage_pitch) + pk * 8);
                else d.zero();
                if (ron) {
                    Pack<__half, 8> rr;
                    rr.load(reinterpret_cast<const __half*>(sX + (size_t)(pk >> 3) * p.e_kb_bytes + swz(slot_in, pk & 7)));
                    __half2* dh = reinterpret_cast<__half2*>(d.s);
                    const __half2* rh = reinterpret_cast<const __half2*>(rr.s);
#pragma unroll
                    for (int q = 0; q < 4; ++q) dh[q] = __hadd2(dh[q], rh[q]);
                }
                d.store(p.out + gq * p.cout + pk * 8);
            }
        }
    }

    // ---- drain: every issued MMA and copy has completed on the success path; release tensor memory ----
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
}

// ---- host side ----------------------------------------------------------------------------------
struct IrbPlan {
    bool ok;
    IrbParams p;
    size_t smem;
    int nbands, nv;
};

static IrbPlan plan_irb(const dc_irb_desc* d) {
    IrbPlan pl{};
    IrbParams& p = pl.p;
    const bool shape_ok = d->dtype == DC_F16 && d->n > 0 && d->h > 0 && d->w > 0 && (d->stride == 1 || d->stride == 2) &&
                          d->c_in % 8 == 0 && d->c_in >= 16 && d->c_hidden % 64 == 0 && d->c_hidden <= 32 * 8 * kIrbMaxPacks &&
                          d->c_out % 16 == 0 && d->c_out >= 16 && d->c_out <= 512 &&
                          d->act_expand >= DC_ACT_NONE && d->act_expand <= DC_ACT_RELU6 && d->act_dw >= DC_ACT_NONE && d->act_dw <= DC_ACT_RELU6 &&
                          (!d->residual || (d->stride == 1 && d->c_in == d->c_out));
    if (!shape_ok) return pl;
    p.h = d->h; p.w = d->w; p.s = d->stride;
    p.ho = (d->h - 1) / d->stride + 1; p.wo = (d->w - 1) / d->stride + 1;        // 3x3, padding 1
    p.cin = d->c_in; p.chid = d->c_hidden; p.cout = d->c_out;
    // bands of output rows whose input rows (with the halo) fit the 128 rows of one MMA tile
    const int max_in_rows = 128 / d->w;
    if (max_in_rows < 3) return pl;
    p.rows_per_band = (max_in_rows - 3) / d->stride + 1;
    if (p.rows_per_band > p.ho) p.rows_per_band = p.ho;
    pl.nbands = divup(p.ho, p.rows_per_band);
    if (pl.nbands > 8) return pl;                        // a portable thread-block cluster holds at most 8 CTAs
    p.rows_per_band = divup(p.ho, pl.nbands);            // even bands
    if (p.wo > kIrbWarps) return pl;
    p.rows_per_round = kIrbWarps / p.wo;
    const int band_in_rows = (p.rows_per_band - 1) * d->stride + 3;
    const int rows8 = (band_in_rows * d->w + 7) & ~7;
    if (rows8 > 128) return pl;
    p.e_kb_bytes = (uint32_t)rows8 * 128u;
    p.nkb1 = divup(d->c_in, kKBlock);
    p.nkb2 = d->c_hidden / kKBlock;
    p.last_ksteps1 = (d->c_in - (p.nkb1 - 1) * kKBlock + 15) >> 4;
    p.ntile2 = divup(d->c_out, 256);
    p.bn2 = divup(divup(d->c_out, p.ntile2), 16) * 16;
    if (p.bn2 * p.ntile2 != d->c_out) return pl;        // equal N tiles only
    pl.nv = divup(d->c_hidden / 8, 32);
    p.stage_pitch = (uint32_t)d->c_out * 2u + 16u;
    // An MMA reads 128 rows of every K block, i.e. up to 16 KB - e_kb_bytes past a block that holds fewer pixel slots: into
    // the next K block or the buffer behind it (its rows beyond the slots are never used). Only the end of the whole
    // layout needs room for that, which the depthwise filter, the tables and the alignment slack provide.
    const uint32_t e_bytes = (uint32_t)p.nkb2 * p.e_kb_bytes;
    if ((uint32_t)(p.rows_per_band * p.wo) * p.stage_pitch > e_bytes) return pl;
    const uint32_t x_bytes = (uint32_t)p.nkb1 * p.e_kb_bytes;
    const uint32_t wd_bytes = ((uint32_t)9 * d->c_hidden * 2u + 1023u) & ~1023u;
    const uint32_t misc_bytes = 24 * 8 + 128 * 4 + 7 * 128 + 64;
    const uint32_t budget = 227u * 1024u - 1024u /* alignment slack */;
    // expansion chunk: the widest that fits shared memory (two buffers) and tensor memory (two accumulators)
    static const int kChunks[] = {256, 192, 160, 128, 96, 64, 48, 32, 16};
    p.nc = 0;
    for (int nc : kChunks) {
        if (d->c_hidden % nc != 0) continue;
        const uint32_t w1b = (uint32_t)p.nkb1 * nc * 128u;
        const uint32_t total = e_bytes + x_bytes + 2u * w1b + wd_bytes + misc_bytes;
        // the projection ring (stages of one N tile of one K block) lives in the expansion-filter area, plus the input tile
        // when no residual needs that tile at the end: at least two stages must fit
        const uint32_t ring = 2u * w1b + (d->residual ? 0u : x_bytes);
        if (total <= budget && ring >= 2u * (uint32_t)p.bn2 * 128u) { p.nc = nc; break; }
    }
    if (p.nc == 0) return pl;
    p.nchunks = d->c_hidden / p.nc;
    p.w1_buf_bytes = (uint32_t)p.nkb1 * p.nc * 128u;
    p.off_x = e_bytes;
    p.off_w1 = p.off_x + x_bytes;
    p.off_wd = p.off_w1 + 2u * p.w1_buf_bytes;
    p.off_misc = p.off_wd + wd_bytes;
    p.off_w2 = d->residual ? p.off_w1 : p.off_x;
    p.w2_stage_bytes = (uint32_t)p.bn2 * 128u;
    p.w2_stages = (int)((2u * p.w1_buf_bytes + (d->residual ? 0u : x_bytes)) / p.w2_stage_bytes);
    if (p.w2_stages > 8) p.w2_stages = 8;
    if (p.w2_stages > p.nkb2 * p.ntile2) p.w2_stages = p.nkb2 * p.ntile2;

    p.acc_stride = (p.nc + 31) & ~31;
    int need = 2 * p.acc_stride > d->c_out ? 2 * p.acc_stride : d->c_out;
    p.tmem_cols = 32;
    while (p.tmem_cols < need) p.tmem_cols <<= 1;
    if (p.tmem_cols > 512) return pl;
    pl.smem = (size_t)p.off_misc + misc_bytes + 1024;
    const size_t reach = (size_t)p.off_x + x_bytes - p.e_kb_bytes + 16u * 1024u + 1024u;      // what the last input K block's MMA reads
    if (pl.smem < reach) pl.smem = reach;
    pl.ok = pl.smem <= 227 * 1024;
    return pl;
}

#ifdef DC_IRB_STAMPS
extern "C" int dc_irb_debug_stamps(long long* out16) {
    return cudaMemcpyFromSymbol(out16, g_irb_stamps, 16 * sizeof(long long)) == cudaSuccess ? 0 : 1;
}
#endif

int irb_error_code() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_irb_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

}  // namespace dc

using namespace dc;

extern "C" {

int dc_irb_supported(const dc_irb_desc* desc) {
    if (desc == nullptr) return 0;
    return plan_irb(desc).ok ? 1 : 0;
}

int dc_irb_fused(const dc_irb_desc* desc, const void* x, const int32_t* mask_in, const void* w_expand_umma, const void* w_dw_hwio,
                 const void* w_project_umma, void* prev_expand, void* trunc_expand, void* prev_dw, void* trunc_dw, void* out,
                 int32_t* mask_out, void* stream) {
    if (desc == nullptr || x == nullptr || mask_in == nullptr || w_expand_umma == nullptr || w_dw_hwio == nullptr ||
        w_project_umma == nullptr || prev_expand == nullptr || trunc_expand == nullptr || prev_dw == nullptr || trunc_dw == nullptr ||
        out == nullptr || mask_out == nullptr)
        return DC_ERR_NULL_POINTER;
    IrbPlan pl = plan_irb(desc);
    if (!pl.ok) return DC_ERR_UNSUPPORTED;
    const void* ptrs[] = {x, w_expand_umma, w_dw_hwio, w_project_umma, prev_expand, trunc_expand, prev_dw, trunc_dw, out};
    for (const void* q : ptrs)
        if (!aligned16(q)) return DC_ERR_ALIGNMENT;
    if ((int64_t)desc->n * desc->h * desc->w > 0x7fffffffLL) return DC_ERR_SHAPE;
    IrbParams& p = pl.p;
    p.x = (const __half*)x; p.mask_in = mask_in;
    p.w1 = (const uint8_t*)w_expand_umma; p.wd = (const __half*)w_dw_hwio; p.w2 = (const uint8_t*)w_project_umma;
    p.prev1 = (__half*)prev_expand; p.trunc1 = (__half*)trunc_expand; p.prev2 = (__half*)prev_dw; p.trunc2 = (__half*)trunc_dw;
    p.out = (__half*)out; p.mask_out = mask_out;
    p.thr1 = host_round_threshold<__half>(desc->thr_expand);
    p.thr2 = host_round_threshold<__half>(desc->thr_dw);
    p.act1 = desc->act_expand; p.act2 = desc->act_dw; p.residual = desc->residual ? 1 : 0;
    // bytes between K blocks of the packed images (dc_pack_filter_umma): rows padded to a multiple of 256 plus 256
    p.w1_kb_stride = (uint32_t)(divup(desc->c_hidden, 256) * 256 + 256) * 128u;
    p.w2_kb_stride = (uint32_t)(divup(desc->c_out, 256) * 256 + 256) * 128u;
    static PerDeviceOnce attr_once;
    bool* attr_set = attr_once.slot();
    if (attr_set == nullptr) return DC_ERR_LAUNCH;
    if (!*attr_set) {
        bool okk = cudaFuncSetAttribute(k_irb_umma<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        okk &= cudaFuncSetAttribute(k_irb_umma<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        okk &= cudaFuncSetAttribute(k_irb_umma<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        okk &= cudaFuncSetAttribute(k_irb_umma<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess;
        if (!okk) return check_launch();
        *attr_set = true;
    }
    const dim3 grid((unsigned)desc->n, (unsigned)pl.nbands);
    cudaStream_t st = (cudaStream_t)stream;
    switch (pl.nv) {
        case 1: return launch_pdl_cluster(k_irb_umma<1>, grid, dim3(kIrbThreads), pl.smem, st, pl.nbands, p);
        case 2: return launch_pdl_cluster(k_irb_umma<2>, grid, dim3(kIrbThreads), pl.smem, st, pl.nbands, p);
        case 3: return launch_pdl_cluster(k_irb_umma<3>, grid, dim3(kIrbThreads), pl.smem, st, pl.nbands, p);
        default: return launch_pdl_cluster(k_irb_umma<4>, grid, dim3(kIrbThreads), pl.smem, st, pl.nbands, p);
    }
}

}  // extern "C"
