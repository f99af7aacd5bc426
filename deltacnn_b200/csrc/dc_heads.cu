// Task heads behind the delta path, kept on the device: the classifier in delta form, the arg-max of pose heat
// maps and the CenterNet peak decode. None of them has a counterpart among the reference's kernels: the reference
// densifies the last feature map and hands it to dense torch code (example/mobilenet_deltacnn.py:216-227,
// src/deltacnn/sparse_layers.py:1322-1329). All three keep their result from the previous frame for streams
// (images of the batch) whose update mask is empty, so an unchanged stream costs one mask read.
#include "dc_umma.cuh"

namespace dc {

// ---------------------------------------------------------------------------------------------
// Linear layer on a pooled delta: acc[n][o] += sum_c W[o][c] * delta[n][c] for streams n whose mask is set;
// out[n][o] = acc[n][o] in the feature dtype. A fully connected layer is linear, so it can consume the delta of
// the pooled feature directly: the dense feature vector is never formed. acc is the fp32 state of the layer
// (bias on the first frame, then the running sum), which keeps the rounding of many frames out of the logits.
// A CTA owns eight outputs (a warp each) and a pass of up to 16 streams (blockIdx.y; further passes in strides of
// gridDim.y): the pass's delta rows and the CTA's weight rows are staged in shared memory by asynchronous copies, all
// in flight together, and the old sums are asked for at the same time; every warp then forms the 16 dot products of
// its weight row without a branch (lanes stride over 16-byte packs; rows of streams without an update hold stale
// data and their sums are dropped) and folds the 32 x 16 partial sums with a butterfly of 31 shuffles, after which
// lane s holds the sum of stream s. Fixed order: reproducible.
// ---------------------------------------------------------------------------------------------
constexpr int kLinStreams = 16;

template <typename T, int W>
__global__ void __launch_bounds__(256) k_linear_delta(const T* __restrict__ delta, const int32_t* __restrict__ mask,
                                                      const T* __restrict__ weight, const T* __restrict__ bias,
                                                      float* __restrict__ acc, T* __restrict__ out, int n, int cin, int cout,
                                                      int first, int spp) {
    extern __shared__ __align__(16) uint8_t lin_smem[];
    constexpr bool kAsync = W > 1;                           // 16-byte packs: rows are staged by asynchronous copies
    T* s_w = reinterpret_cast<T*>(lin_smem);                 // [8][cin] the weight rows of this CTA (kAsync only)
    T* s_d = s_w + (kAsync ? 8 * (size_t)cin : 0);           // [spp][cin], spp <= 16 streams per pass
    __shared__ int s_on[kLinStreams];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int o = blockIdx.x * 8 + warp;
    const int nvec = cin / W;
    const T* wrow = weight + (int64_t)(o < cout ? o : 0) * cin;
    if constexpr (kAsync) {                                  // weights do not depend on the previous kernel
        for (int i = lane; i < nvec; i += 32) cp_async16(smem_u32(s_w + (size_t)warp * cin + i * W), wrow + i * W, 16u);
        cp_async_commit();
    }
    grid_dep_launch();
    grid_dep_wait();
    const float b = (first && bias != nullptr && o < cout) ? to_f<T>(bias[o]) : 0.f;
    for (int n0 = (int)blockIdx.y * spp; n0 < n; n0 += (int)gridDim.y * spp) {
        const int cnt = min(spp, n - n0);
        const bool mine = lane < cnt && (first || mask == nullptr || mask[n0 + lane] != 0);      // stream n0 + lane
        if (warp == 0 && lane < kLinStreams) s_on[lane] = mine ? 1 : 0;
        // the old sum of (stream n0 + lane, output o): in flight while the rows are staged
        const float a_prev = (mine && !first && o < cout) ? acc[(int64_t)(n0 + lane) * cout + o] : 0.f;
        __syncthreads();
        for (int idx = tid; idx < cnt * nvec; idx += 256) {
            const int j = idx / nvec, i = idx - j * nvec;
            if (s_on[j]) {
                if constexpr (kAsync) {
                    cp_async16(smem_u32(s_d + (size_t)j * cin + i * W), delta + (int64_t)(n0 + j) * cin + i * W, 16u);
                } else {
                    s_d[(size_t)j * cin + i] = delta[(int64_t)(n0 + j) * cin + i];
                }
            }
        }
        if constexpr (kAsync) {
            cp_async_commit();
            cp_async_wait_group<0>();
        }
        __syncthreads();
        if (o < cout) {
            float sum[kLinStreams];
#pragma unroll
            for (int j = 0; j < kLinStreams; ++j) sum[j] = 0.f;
            for (int i = lane; i < nvec; i += 32) {
                Pack<T, W> wv;
                wv.load(kAsync ? s_w + (size_t)warp * cin + i * W : wrow + i * W);
                float wf[W];
#pragma unroll
                for (int k = 0; k < W; ++k) wf[k] = wv.get(k);
#pragma unroll
                for (int j = 0; j < kLinStreams; ++j) {
                    const int jj = j < cnt ? j : cnt - 1;     // beyond the pass: a valid row, the sum is not used
                    Pack<T, W> dv;
                    dv.load(s_d + (size_t)jj * cin + i * W);
#pragma unroll
                    for (int k = 0; k < W; ++k) sum[j] = fmaf(wf[k], dv.get(k), sum[j]);
                }
            }
            // fold: lanes L and L ^ 16 first, then after the step with distance w a lane keeps the half of the streams
            // its bit w selects; lane L ends with the sum of stream L & 15
#pragma unroll
            for (int k = 0; k < kLinStreams; ++k) sum[k] += __shfl_xor_sync(DC_FULL, sum[k], 16);
#pragma unroll
            for (int w = kLinStreams / 2; w >= 1; w >>= 1) {
                const bool up = (lane & w) != 0;
#pragma unroll
                for (int k = 0; k < w; ++k) {
                    const float keep = up ? sum[k + w] : sum[k];
                    const float send = up ? sum[k] : sum[k + w];
                    sum[k] = keep + __shfl_xor_sync(DC_FULL, send, w);
                }
            }
            if (mine) {                                      // lane < cnt <= 16
                const int64_t idx = (int64_t)(n0 + lane) * cout + o;
                const float a = a_prev + sum[0] + b;
                acc[idx] = a;
                out[idx] = from_f<T>(a);
            }
        }
        __syncthreads();                                     // s_on and the staged rows are rewritten by the next pass
    }
}

// ---------------------------------------------------------------------------------------------
// Arg-max of dense heat maps (N,H,W,J channels last): per stream and joint the position and value of the largest
// element, the first one in row-major order on ties (torch.argmax). One CTA per stream and slab of 32 joints;
// a thread walks the pixels t, t + 256, ... keeping the best of every joint of the slab, then the 256 candidates
// per joint are reduced through shared memory. Streams whose mask has no active pixel keep their previous result.
// ---------------------------------------------------------------------------------------------
constexpr int kHmJoints = 32;

template <typename T>
__global__ void __launch_bounds__(256) k_heatmap_argmax(const T* __restrict__ heat, const int32_t* __restrict__ mask,
                                                        float* __restrict__ out, int hw, int w, int joints) {
    __shared__ float s_val[8][kHmJoints];
    __shared__ int s_idx[8][kHmJoints];
    __shared__ int s_any;
    grid_dep_launch();
    grid_dep_wait();
    const int b = blockIdx.x, j0 = blockIdx.y * kHmJoints;
    const int nj = min(kHmJoints, joints - j0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (mask != nullptr) {
        if (tid == 0) s_any = 0;
        __syncthreads();
        bool on = false;
        for (int p = tid; p < hw; p += 256) on |= mask[(int64_t)b * hw + p] != 0;
        if (__any_sync(DC_FULL, on) && lane == 0) s_any = 1;
        __syncthreads();
        if (s_any == 0) return;                 // nothing changed in this stream: the previous arg-max stands
    }
    float best[kHmJoints];
    int bidx[kHmJoints];
#pragma unroll
    for (int j = 0; j < kHmJoints; ++j) { best[j] = -INFINITY; bidx[j] = 0x7fffffff; }
    const T* base = heat + (int64_t)b * hw * joints + j0;
    for (int p = tid; p < hw; p += 256) {
#pragma unroll
        for (int j = 0; j < kHmJoints; ++j) {
            if (j < nj) {
                const float v = to_f<T>(base[(int64_t)p * joints + j]);
                if (v > best[j]) { best[j] = v; bidx[j] = p; }      // ascending p: the first maximum stays
            }
        }
    }
    // warp reduce (larger value wins, then the smaller index), then the eight warps through shared memory
#pragma unroll
    for (int j = 0; j < kHmJoints; ++j) {
        float v = best[j];
        int ix = bidx[j];
        for (int o = 16; o > 0; o >>= 1) {
            const float v2 = __shfl_xor_sync(DC_FULL, v, o);
            const int i2 = __shfl_xor_sync(DC_FULL, ix, o);
            if (v2 > v || (v2 == v && i2 < ix)) { v = v2; ix = i2; }
        }
        if (lane == 0) { s_val[warp][j] = v; s_idx[warp][j] = ix; }
    }
    __syncthreads();
    if (tid < nj) {
        float v = s_val[0][tid];
        int ix = s_idx[0][tid];
        for (int k = 1; k < 8; ++k) {
            const float v2 = s_val[k][tid];
            const int i2 = s_idx[k][tid];
            if (v2 > v || (v2 == v && i2 < ix)) { v = v2; ix = i2; }
        }
        float* o = out + ((int64_t)b * joints + j0 + tid) * 3;
        o[0] = (float)(ix % w);
        o[1] = (float)(ix / w);
        o[2] = v;
    }
}

// ---------------------------------------------------------------------------------------------
// CenterNet decode, step 1: peak map. score[p][c] = heat[p][c] when it is the maximum of its 3x3 neighbourhood
// (borders: in-bounds neighbours only; equal neighbours do not suppress, as max_pool == heat in the usual torch
// decode) else -inf. Only pixels whose 3x3 neighbourhood holds an updated pixel are recomputed (a peak can only
// appear or vanish there); mask == NULL recomputes every pixel (first frame).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) k_peak_map(const T* __restrict__ heat, const int32_t* __restrict__ mask,
                                                  float* __restrict__ peaks, int n, int h, int w, int classes) {
    grid_dep_launch();
    grid_dep_wait();
    const int64_t total = (int64_t)n * h * w;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < total; q += (int64_t)gridDim.x * blockDim.x) {
        const int x = (int)(q % w);
        const int y = (int)((q / w) % h);
        const int64_t b = q / ((int64_t)w * h);
        bool touched = mask == nullptr;
        if (!touched) {
            for (int dy = -1; dy <= 1 && !touched; ++dy)
                for (int dx = -1; dx <= 1; ++dx) {
                    const int yy = y + dy, xx = x + dx;
                    if (yy >= 0 && yy < h && xx >= 0 && xx < w && mask[(b * h + yy) * w + xx] != 0) { touched = true; break; }
                }
        }
        if (!touched) continue;
        for (int c = 0; c < classes; ++c) {
            const float v = to_f<T>(heat[q * classes + c]);
            float m = v;
            for (int dy = -1; dy <= 1; ++dy)
                for (int dx = -1; dx <= 1; ++dx) {
                    const int yy = y + dy, xx = x + dx;
                    if (yy >= 0 && yy < h && xx >= 0 && xx < w) m = fmaxf(m, to_f<T>(heat[((b * h + yy) * w + xx) * classes + c]));
                }
            peaks[q * classes + c] = v == m ? v : -INFINITY;
        }
    }
}

// Order-preserving map of a float to an unsigned integer (larger float -> larger key).
__device__ __forceinline__ uint32_t float_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Step 2: the K best peaks of a stream (score above min_score), best first, equal scores by ascending
// (pixel, class) index, and their boxes. One CTA per stream. Candidates are sorted in shared memory as 64-bit keys
// (score key << 32 | ~index) with a bitonic network of kSortN entries; when a stream has more candidates than fit,
// the best K so far are kept and the sort is repeated with the next batch, so the result is exact for any number
// of peaks. det[n][k] = (x1, y1, x2, y2, score, class) in input-image pixels (centre = (x + off_x, y + off_y),
// size = (wh_x, wh_y), all times `stride`); count[n] = number of valid rows. Streams whose mask is empty keep their
// previous rows.
constexpr int kSortN = 2048;

template <typename T>
__global__ void __launch_bounds__(256) k_centernet_topk(const float* __restrict__ peaks, const T* __restrict__ wh,
                                                        const T* __restrict__ off, const int32_t* __restrict__ mask,
                                                        float* __restrict__ det, int32_t* __restrict__ count, int h, int w,
                                                        int classes, int topk, float min_score, float stride, int sigmoid) {
    __shared__ unsigned long long s_key[kSortN];
    __shared__ int s_w[8], s_any;
    grid_dep_launch();
    grid_dep_wait();
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
    const int hw = h * w;
    if (mask != nullptr) {
        if (tid == 0) s_any = 0;
        __syncthreads();
        bool on = false;
        for (int p = tid; p < hw; p += 256) on |= mask[(int64_t)b * hw + p] != 0;
        if (__any_sync(DC_FULL, on) && lane == 0) s_any = 1;
        __syncthreads();
        if (s_any == 0) return;
    }
    const int64_t total = (int64_t)hw * classes;
    const float* pk = peaks + (int64_t)b * total;
    const int warp = tid >> 5;
    int kept = 0;                     // s_key[0..kept) are the best so far, best first
    int64_t next = 0;                 // first candidate index not yet looked at
    do {
        // fill s_key[kept..) with the next candidates in index order, 256 indices per step, while a whole step fits
        int fill = kept;              // uniform over the CTA
        while (next < total && fill + 256 <= kSortN) {
            const int64_t i = next + tid;
            const float v = i < total ? pk[i] : -INFINITY;
            const bool cand = v > min_score && v > -INFINITY;
            const unsigned bal = __ballot_sync(DC_FULL, cand);
            if (lane == 0) s_w[warp] = __popc(bal);
            __syncthreads();
            int before = 0, all = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int c = s_w[k];
                if (k < warp) before += c;
                all += c;
            }
            if (cand)
                s_key[fill + before + __popc(bal & ((1u << lane) - 1u))] =
                    ((unsigned long long)float_key(v) << 32) | (unsigned long long)(~(uint32_t)i);
            fill += all;
            next += 256;
            __syncthreads();          // s_w is rewritten by the next step
        }
        for (int i = fill + tid; i < kSortN; i += 256) s_key[i] = 0ull;       // smallest key: sorts to the end
        __syncthreads();
        // bitonic sort, descending
        for (int k2 = 2; k2 <= kSortN; k2 <<= 1) {
            for (int j = k2 >> 1; j > 0; j >>= 1) {
                for (int i = tid; i < kSortN; i += 256) {
                    const int l = i ^ j;
                    if (l > i) {
                        const unsigned long long a = s_key[i], c = s_key[l];
                        const bool desc = (i & k2) == 0;
                        if (desc ? a < c : a > c) { s_key[i] = c; s_key[l] = a; }
                    }
                }
                __syncthreads();
            }
        }
        kept = min(fill, topk);
    } while (next < total);
    // decode the best `kept`
    for (int k = tid; k < topk; k += 256) {
        float* d = det + ((int64_t)b * topk + k) * 6;
        if (k < kept) {
            const unsigned long long key = s_key[k];
            const uint32_t idx = ~(uint32_t)(key & 0xffffffffull);
            float score = key_float((uint32_t)(key >> 32));
            const int c = (int)(idx % (uint32_t)classes);
            const int p = (int)(idx / (uint32_t)classes);
            const int x = p % w, y = p / w;
            const int64_t q = (int64_t)b * hw + p;
            const float cx = (float)x + to_f<T>(off[q * 2]), cy = (float)y + to_f<T>(off[q * 2 + 1]);
            const float bw = to_f<T>(wh[q * 2]), bh = to_f<T>(wh[q * 2 + 1]);
            if (sigmoid) score = 1.f / (1.f + __expf(-score));
            d[0] = (cx - 0.5f * bw) * stride; d[1] = (cy - 0.5f * bh) * stride;
            d[2] = (cx + 0.5f * bw) * stride; d[3] = (cy + 0.5f * bh) * stride;
            d[4] = score; d[5] = (float)c;
        } else {
            d[0] = d[1] = d[2] = d[3] = d[4] = 0.f; d[5] = -1.f;
        }
    }
    if (tid == 0) count[b] = kept;
}

}  // namespace dc

using namespace dc;

extern "C" {

int dc_linear_delta(const void* delta, const int32_t* mask, const void* weight, const void* bias, float* acc, void* out,
                    int32_t n, int32_t c_in, int32_t c_out, int32_t dtype, int32_t first_frame, void* stream) {
    if (n < 0 || c_in <= 0 || c_out <= 0) return DC_ERR_SHAPE;
    if (n == 0) return DC_OK;
    if (delta == nullptr || weight == nullptr || acc == nullptr || out == nullptr) return DC_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t esz = dtype == DC_F16 ? 2 : 4;
    if (dtype != DC_F16 && dtype != DC_F32) return DC_ERR_DTYPE;
    const bool vec = c_in % (int)(16 / esz) == 0 && aligned16(delta) && aligned16(weight);
    const size_t row = (size_t)c_in * esz, wrows = vec ? 8 * row : 0;    // the vector form also stages its eight weight rows
    if (wrows + row > 200 * 1024) return DC_ERR_UNSUPPORTED;
    int spp = (int)((200 * 1024 - wrows) / row);                         // streams whose rows fit the staging buffer
    if (spp > kLinStreams) spp = kLinStreams;
    if (spp > n) spp = n;
    const size_t smem = wrows + (size_t)spp * row;
    int passes = divup(n, spp);
    if (passes > 8) passes = 8;
    const dim3 grid((unsigned)divup(c_out, 8), (unsigned)passes);
#define DC_LIN(T, W_)                                                                                                                         \
    do {                                                                                                                                      \
        if (smem > 48 * 1024) {                                                                                                               \
            static PerDeviceOnce once;                                                                                                        \
            bool* done = once.slot();                                                                                                         \
            if (done == nullptr) return DC_ERR_LAUNCH;                                                                                        \
            if (!*done) {                                                                                                                     \
                if (cudaFuncSetAttribute(k_linear_delta<T, W_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)      \
                    return check_launch();                                                                                                    \
                *done = true;                                                                                                                 \
            }                                                                                                                                 \
        }                                                                                                                                     \
        launch_pdl(k_linear_delta<T, W_>, grid, dim3(256), smem, st, (const T*)delta, mask, (const T*)weight, (const T*)bias, acc, (T*)out,  \
                   n, c_in, c_out, first_frame, spp);                                                                                         \
    } while (0)
    if (dtype == DC_F16) {
        if (vec) DC_LIN(__half, 8); else DC_LIN(__half, 1);
    } else {
        if (vec) DC_LIN(float, 4); else DC_LIN(float, 1);
    }
#undef DC_LIN
    return check_launch();
}

int dc_heatmap_argmax(const void* heat, const int32_t* mask, float* out, int32_t n, int32_t h, int32_t w, int32_t joints,
                      int32_t dtype, void* stream) {
    if (n < 0 || h <= 0 || w <= 0 || joints <= 0 || (int64_t)h * w > 0x7fffffffLL) return DC_ERR_SHAPE;
    if (n == 0) return DC_OK;
    if (heat == nullptr || out == nullptr) return DC_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid((unsigned)n, (unsigned)divup(joints, kHmJoints));
    if (dtype == DC_F16) launch_pdl(k_heatmap_argmax<__half>, grid, dim3(256), 0, st, (const __half*)heat, mask, out, h * w, w, joints);
    else if (dtype == DC_F32) launch_pdl(k_heatmap_argmax<float>, grid, dim3(256), 0, st, (const float*)heat, mask, out, h * w, w, joints);
    else return DC_ERR_DTYPE;
    return check_launch();
}

int dc_centernet_decode(const void* heat, const void* wh, const void* offset, const int32_t* mask, float* peaks, float* det,
                        int32_t* count, int32_t n, int32_t h, int32_t w, int32_t classes, int32_t topk, float min_score,
                        float stride, int32_t apply_sigmoid, int32_t dtype, void* stream) {
    if (n < 0 || h <= 0 || w <= 0 || classes <= 0 || topk <= 0 || topk > kSortN / 2) return DC_ERR_SHAPE;
    if ((int64_t)h * w * classes > 0x7fffffffLL) return DC_ERR_SHAPE;
    if (n == 0) return DC_OK;
    if (heat == nullptr || wh == nullptr || offset == nullptr || peaks == nullptr || det == nullptr || count == nullptr) return DC_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t total = (int64_t)n * h * w;
    int64_t blocks = divup64(total, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    int rc;
    if (dtype == DC_F16) {
        rc = launch_pdl(k_peak_map<__half>, dim3((unsigned)blocks), dim3(256), 0, st, (const __half*)heat, mask, peaks, n, h, w, classes);
        if (rc != DC_OK) return rc;
        return launch_pdl(k_centernet_topk<__half>, dim3((unsigned)n), dim3(256), 0, st, (const float*)peaks, (const __half*)wh, (const __half*)offset,
                          mask, det, count, h, w, classes, topk, min_score, stride, apply_sigmoid);
    }
    if (dtype == DC_F32) {
        rc = launch_pdl(k_peak_map<float>, dim3((unsigned)blocks), dim3(256), 0, st, (const float*)heat, mask, peaks, n, h, w, classes);
        if (rc != DC_OK) return rc;
        return launch_pdl(k_centernet_topk<float>, dim3((unsigned)n), dim3(256), 0, st, (const float*)peaks, (const float*)wh, (const float*)offset,
                          mask, det, count, h, w, classes, topk, min_score, stride, apply_sigmoid);
    }
    return DC_ERR_DTYPE;
}

}  // extern "C"
