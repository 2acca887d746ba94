// Attention of a ragged step over a per-slot key/value cache: sliding window (or everything before the row), optionally
// with one mean key/value per block of older tokens, and three ways from scores to weights (softmax, softmax with a
// sink, sigmoid).  A key is read where it lives: tokens of the step from the step's own rows, older tokens from the
// slot's cache rows (position p at row p mod kv_len), pooled blocks from the slot's block table -- so a prompt in one
// piece, in portions, and token-by-token decoding all walk the same keys in the same order.
//
// Tile kernel (any step): one block = 64 consecutive query rows of one (sequence, head); 256 threads as 16 x 16, a thread
// owns 4 rows x 4 keys of the score tile and 4 rows x VC value columns of the output; per tile of 64 keys the scores come
// from transposed fp32 tiles in shared memory, the weights go back through shared memory for the value product.  The key
// tile holds 64 dimensions at a time (larger heads add their scores up over several passes), which keeps two blocks on an
// SM for heads of 128.
// Decode kernel (one token per sequence): one block = (sequence, head, split); a warp takes every 8th key of the block's
// share, lanes striding over the head's dimensions; partial (max, sum, output) triples are merged per block and, with more
// than one split, by a second kernel.
// Everything is fp32 arithmetic; T is the storage type of q, the key/value rows and the output.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <algorithm>
#include <stdint.h>

#include "seq_internal.h"

namespace umbs {

constexpr int kCaQ = 64, kCaK = 64, kCaS = 68;        // rows and keys per tile; row stride of the [d][row] tiles
constexpr int kCaD = 64;                              // dimensions of a key tile held at a time

struct CachedAttnArgs {
    const void* q; const void* kv; const void* kv_cache; const void* pool_cache;
    int kv_len, pool_len;
    int heads, kv_heads, dim, vdim, window, pool;
    float scale;
    const float* head_bias; const float* gate; int64_t ldg; int gate_per_head;
    void* out;
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }

// blocks of `pool` tokens that lie wholly before the window of the row at position p
__device__ __forceinline__ int pooled_visible(int p, int window, int pool) {
    const int lim = p - window + 1;                   // tokens [0, lim) have left the window
    return (pool > 0 && lim >= pool) ? lim / pool : 0;
}

template <typename T, int VC, int MODE>
__global__ void __launch_bounds__(256) cached_attention_kernel(CachedAttnArgs a, Batch b) {
    extern __shared__ __align__(16) float sm[];
    constexpr int VW = 16 * VC, VP = VW + 4;
    const int dim = a.dim, vdim = a.vdim;
    float* Qs = sm;                                   // [dim][kCaS]  Qs[d][row]
    float* Ks = Qs + (size_t)dim * kCaS;              // [min(dim, kCaD)][kCaS]  Ks[d][key], kCaD dimensions at a time
    float* Vs = Ks + (size_t)min(dim, kCaD) * kCaS;   // [kCaK][VP]
    float* Ps = Vs + (size_t)kCaK * VP;               // [kCaK][kCaS] Ps[key][row]
    const int s = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * kCaQ;
    const int len = b.seq_len[s], start = b.seq_start[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    if (q0 >= len) return;
    const int g = h / (a.heads / a.kv_heads);
    const int row_kv = a.kv_heads * (dim + vdim), koff = g * dim, voff = a.kv_heads * dim + g * vdim;
    const int window = a.window > 0 ? a.window : (1 << 30);
    const T* q = (const T*)a.q;
    const T* kv = (const T*)a.kv;
    const T* cache = (const T*)a.kv_cache;
    const T* pooled = (const T*)a.pool_cache;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    for (int i = tid; i < kCaQ * dim; i += 256) {
        const int r = i / dim, d = i - r * dim;
        Qs[d * kCaS + r] = (q0 + r < len) ? to_f32(q[(int64_t)(start + q0 + r) * a.heads * dim + (int64_t)h * dim + d]) : 0.f;
    }
    float m[4], l[4], o[4][VC];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m[i] = MODE == UMBS_ATTN_SOFTMAX_SINK ? 0.f : -INFINITY;       // the sink: a key of score 0 ...
        l[i] = MODE == UMBS_ATTN_SOFTMAX_SINK ? 1.f : 0.f;             // ... that counts in the sum and has no value
#pragma unroll
        for (int c = 0; c < VC; ++c) o[i][c] = 0.f;
    }
    const float hb = (MODE == UMBS_ATTN_SIGMOID && a.head_bias) ? a.head_bias[h] : 0.f;
    const int p_lo = pos0 + q0, p_hi = pos0 + min(len, q0 + kCaQ) - 1;      // positions of the block's first and last row
    const int n_pool = pooled_visible(p_hi, window, a.pool);               // blocks the last row sees
    const int tiles_pool = (n_pool + kCaK - 1) / kCaK;
    const int j_lo = max(0, p_lo - window + 1);
    const int tiles_tok = (p_hi - j_lo) / kCaK + 1;
    for (int tile = 0; tile < tiles_pool + tiles_tok; ++tile) {
        const bool in_pool = tile < tiles_pool;
        const int base = in_pool ? tile * kCaK : j_lo + (tile - tiles_pool) * kCaK;
        const int hi = in_pool ? n_pool - 1 : p_hi;                        // last index of this kind any row sees
        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) sc[i][jj] = 0.f;
        for (int d0 = 0; d0 < dim; d0 += kCaD) {
            const int dc = min(kCaD, dim - d0);
            __syncthreads();                          // the previous pass or tile is consumed (the very first time: Qs is written)
            for (int i = tid; i < kCaK * dc; i += 256) {
                const int kk = i / dc, d = i - kk * dc, j = base + kk;
                float val = 0.f;
                if (j <= hi) {
                    const T* src = in_pool ? pooled + ((int64_t)slot * a.pool_len + j) * row_kv
                                 : (j >= pos0 ? kv + (int64_t)(start + j - pos0) * row_kv
                                              : cache + ((int64_t)slot * a.kv_len + j % a.kv_len) * row_kv);
                    val = to_f32(src[koff + d0 + d]);
                }
                Ks[d * kCaS + kk] = val;
            }
            for (int i = tid; d0 == 0 && i < kCaK * VW; i += 256) {
                const int kk = i / VW, c = i - kk * VW, j = base + kk;
                float val = 0.f;
                if (j <= hi && c < vdim) {
                    const T* src = in_pool ? pooled + ((int64_t)slot * a.pool_len + j) * row_kv
                                 : (j >= pos0 ? kv + (int64_t)(start + j - pos0) * row_kv
                                              : cache + ((int64_t)slot * a.kv_len + j % a.kv_len) * row_kv);
                    val = to_f32(src[voff + c]);
                }
                Vs[kk * VP + c] = val;
            }
            __syncthreads();
            for (int d = 0; d < dc; ++d) {
                const float4 qv = *reinterpret_cast<const float4*>(Qs + (d0 + d) * kCaS + ty * 4);
                const float4 kv4 = *reinterpret_cast<const float4*>(Ks + d * kCaS + tx * 4);
                const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) sc[i][jj] = fmaf(qa[i], ka[jj], sc[i][jj]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = q0 + ty * 4 + i, rp = pos0 + r;                  // the row's place in the step and its position
            float p[4];
            bool vis[4];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int j = base + tx * 4 + jj;
                vis[jj] = r < len && (in_pool ? j < pooled_visible(rp, window, a.pool) : (j <= rp && j > rp - window));
            }
            if (MODE == UMBS_ATTN_SIGMOID) {
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) p[jj] = vis[jj] ? sigmoidf_(sc[i][jj] * a.scale + hb) : 0.f;
            } else {
                float val[4], mx = -INFINITY;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    val[jj] = vis[jj] ? sc[i][jj] * a.scale : -INFINITY;
                    mx = fmaxf(mx, val[jj]);
                }
#pragma unroll
                for (int w = 8; w > 0; w >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));   // the row's 16 threads
                const float mn = fmaxf(m[i], mx);
                float sum = 0.f, corr = 1.f;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) p[jj] = 0.f;
                if (mn > -INFINITY) {
                    corr = expf(m[i] - mn);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        p[jj] = vis[jj] ? expf(val[jj] - mn) : 0.f;
                        sum += p[jj];
                    }
                }
#pragma unroll
                for (int w = 8; w > 0; w >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, w);
                l[i] = l[i] * corr + sum;
                m[i] = mn;
#pragma unroll
                for (int c = 0; c < VC; ++c) o[i][c] *= corr;
            }
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) Ps[(tx * 4 + jj) * kCaS + ty * 4 + i] = p[jj];
        }
        __syncthreads();
        for (int kk = 0; kk < kCaK; ++kk) {
            const float4 pv = *reinterpret_cast<const float4*>(Ps + kk * kCaS + ty * 4);
            const float pa[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (int cb = 0; cb < VC / 4; ++cb) {
                const float4 vv = *reinterpret_cast<const float4*>(Vs + kk * VP + cb * 64 + tx * 4);
                const float va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int c = 0; c < 4; ++c) o[i][cb * 4 + c] = fmaf(pa[i], va[c], o[i][cb * 4 + c]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = q0 + ty * 4 + i;
        if (r >= len) continue;
        const int64_t t = start + r;
        const float inv = MODE == UMBS_ATTN_SIGMOID ? 1.f : 1.f / l[i];
        const float* grow = a.gate ? a.gate + t * a.ldg + (a.gate_per_head ? h : h * vdim) : nullptr;
        const float gh = (grow && a.gate_per_head) ? sigmoidf_(grow[0]) : 1.f;
        T* orow = (T*)a.out + t * a.heads * vdim + (int64_t)h * vdim;
#pragma unroll
        for (int cb = 0; cb < VC / 4; ++cb)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = cb * 64 + tx * 4 + c;
                if (col < vdim) {
                    const float gt = (grow && !a.gate_per_head) ? sigmoidf_(grow[col]) : gh;
                    orow[col] = from_f32<T>(o[i][cb * 4 + c] * inv * gt);
                }
            }
    }
}

template <typename T, int VC, int MODE>
static int launch_tiles(const CachedAttnArgs& a, const Batch& b, cudaStream_t st) {
    const size_t smem = ((size_t)(a.dim + std::min(a.dim, kCaD)) * kCaS + (size_t)kCaK * (16 * VC + 4) + (size_t)kCaK * kCaS) * sizeof(float);
    static size_t set = 0;
    if (smem > 48 * 1024 && smem > set) {
        cudaError_t e = cudaFuncSetAttribute(cached_attention_kernel<T, VC, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = smem;
    }
    const dim3 grid((b.max_seq_len + kCaQ - 1) / kCaQ, a.heads, b.n_seqs);
    cached_attention_kernel<T, VC, MODE><<<grid, 256, smem, st>>>(a, b);
    return 0;
}

template <typename T, int MODE>
static int launch_mode(const CachedAttnArgs& a, const Batch& b, cudaStream_t st) {
    if (a.vdim <= 64) return launch_tiles<T, 4, MODE>(a, b, st);
    if (a.vdim <= 128) return launch_tiles<T, 8, MODE>(a, b, st);
    return launch_tiles<T, 16, MODE>(a, b, st);
}

template <typename T>
static int launch_any(int mode, const CachedAttnArgs& a, const Batch& b, cudaStream_t st) {
    switch (mode) {
        case UMBS_ATTN_SOFTMAX: return launch_mode<T, UMBS_ATTN_SOFTMAX>(a, b, st);
        case UMBS_ATTN_SOFTMAX_SINK: return launch_mode<T, UMBS_ATTN_SOFTMAX_SINK>(a, b, st);
        case UMBS_ATTN_SIGMOID: return launch_mode<T, UMBS_ATTN_SIGMOID>(a, b, st);
    }
    return UMB_ERR_ARG;
}


// ------------------------------------------------------------------------------------------------ decode steps
// One block = (split, head, sequence) of a step with one token per sequence.  The row's keys -- pooled blocks first,
// then the tokens of its window -- are numbered 0 .. n - 1 and cut into n_split equal runs; inside a block warp w takes
// keys w, w + 8, ... of the run, lanes striding over the head's dimensions, with its own running (maximum, sum, output).
// The warps' triples are merged in shared memory; one split writes the output itself, several leave their triples in
// `part` [(token, head), split, vdim + 2] for cached_attention_merge_kernel.
constexpr int kCdWarps = 8, kCdMaxPerLane = 8;        // dim, vdim <= 256

template <typename T, int MODE>
__global__ void __launch_bounds__(32 * kCdWarps) cached_attention_decode_kernel(CachedAttnArgs a, Batch b, int n_split,
                                                                                float* __restrict__ part) {
    __shared__ float sm_o[kCdWarps][32 * kCdMaxPerLane];
    __shared__ float sm_ml[kCdWarps][2];
    const int split = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int dim = a.dim, vdim = a.vdim;
    const int t = b.seq_start[s], p = b.seq_pos0[s], slot = b.seq_slot[s];
    const int g = h / (a.heads / a.kv_heads);
    const int row_kv = a.kv_heads * (dim + vdim), koff = g * dim, voff = a.kv_heads * dim + g * vdim;
    const int window = a.window > 0 ? a.window : (1 << 30);
    const int n_pool = pooled_visible(p, window, a.pool), j_lo = max(0, p - window + 1);
    const int n_keys = n_pool + (p - j_lo + 1);
    const int per = (n_keys + n_split - 1) / n_split, lo = split * per, hi = min(n_keys, lo + per);
    const T* qrow = (const T*)a.q + (int64_t)t * a.heads * dim + (int64_t)h * dim;
    float qv[kCdMaxPerLane], o[kCdMaxPerLane];
#pragma unroll
    for (int i = 0; i < kCdMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < dim ? to_f32(qrow[d]) : 0.f;
        o[i] = 0.f;
    }
    const float hb = (MODE == UMBS_ATTN_SIGMOID && a.head_bias) ? a.head_bias[h] : 0.f;
    float m = -INFINITY, l = 0.f;
    for (int k = lo + w; k < hi; k += kCdWarps) {
        const T* src;
        if (k < n_pool) src = (const T*)a.pool_cache + ((int64_t)slot * a.pool_len + k) * row_kv;
        else {
            const int j = j_lo + (k - n_pool);
            src = j >= p ? (const T*)a.kv + (int64_t)t * row_kv : (const T*)a.kv_cache + ((int64_t)slot * a.kv_len + j % a.kv_len) * row_kv;
        }
        float dot = 0.f, vv[kCdMaxPerLane];
#pragma unroll
        for (int i = 0; i < kCdMaxPerLane; ++i) {
            const int d = lane + 32 * i;
            if (d < dim) dot = fmaf(qv[i], to_f32(src[koff + d]), dot);
            vv[i] = d < vdim ? to_f32(src[voff + d]) : 0.f;
        }
#pragma unroll
        for (int x = 16; x > 0; x >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, x);
        float pw;
        if (MODE == UMBS_ATTN_SIGMOID) {
            pw = sigmoidf_(dot * a.scale + hb);
        } else {
            const float sc = dot * a.scale, mn = fmaxf(m, sc), corr = expf(m - mn);      // m = -inf the first time: corr = 0
            pw = expf(sc - mn);
            l = l * corr + pw;
            m = mn;
#pragma unroll
            for (int i = 0; i < kCdMaxPerLane; ++i) o[i] *= corr;
        }
#pragma unroll
        for (int i = 0; i < kCdMaxPerLane; ++i) o[i] = fmaf(pw, vv[i], o[i]);
    }
#pragma unroll
    for (int i = 0; i < kCdMaxPerLane; ++i) sm_o[w][lane + 32 * i] = o[i];
    if (lane == 0) { sm_ml[w][0] = m; sm_ml[w][1] = l; }
    __syncthreads();
    // merge the warps' triples (in warp order); thread c < vdim owns output column c
    const int c = threadIdx.x;
    float M = -INFINITY, L = 0.f, O = 0.f;
    if (MODE == UMBS_ATTN_SIGMOID) {
        if (c < vdim)
            for (int ww = 0; ww < kCdWarps; ++ww) O += sm_o[ww][c];
    } else {
        for (int ww = 0; ww < kCdWarps; ++ww) M = fmaxf(M, sm_ml[ww][0]);
        if (n_split == 1 && MODE == UMBS_ATTN_SOFTMAX_SINK) M = fmaxf(M, 0.f);
        for (int ww = 0; ww < kCdWarps; ++ww) {
            const float mw = sm_ml[ww][0], f = mw > -INFINITY ? expf(mw - M) : 0.f;
            L = fmaf(sm_ml[ww][1], f, L);
            if (c < vdim) O = fmaf(sm_o[ww][c], f, O);
        }
        if (n_split == 1 && MODE == UMBS_ATTN_SOFTMAX_SINK) L += expf(-M);
    }
    if (n_split > 1) {
        float* pr = part + (((int64_t)t * a.heads + h) * n_split + split) * (vdim + 2);
        if (c < vdim) pr[c] = O;
        if (c == 0) { pr[vdim] = M; pr[vdim + 1] = L; }
        return;
    }
    if (c < vdim) {
        const float inv = MODE == UMBS_ATTN_SIGMOID ? 1.f : 1.f / L;
        float gt = 1.f;
        if (a.gate) gt = sigmoidf_(a.gate[(int64_t)t * a.ldg + (a.gate_per_head ? h : h * vdim + c)]);
        ((T*)a.out)[(int64_t)t * a.heads * vdim + (int64_t)h * vdim + c] = from_f32<T>(O * inv * gt);
    }
}

// One block per (token, head): the splits' triples, in split order, then the sink, the division and the output gate.
template <typename T, int MODE>
__global__ void cached_attention_merge_kernel(CachedAttnArgs a, int n_split, const float* __restrict__ part) {
    const int th = blockIdx.x, t = th / a.heads, h = th - t * a.heads, vdim = a.vdim, c = threadIdx.x;
    const float* pr = part + (int64_t)th * n_split * (vdim + 2);
    float M = MODE == UMBS_ATTN_SOFTMAX_SINK ? 0.f : -INFINITY, L = 0.f, O = 0.f;
    if (MODE == UMBS_ATTN_SIGMOID) {
        if (c < vdim)
            for (int i = 0; i < n_split; ++i) O += pr[i * (vdim + 2) + c];
    } else {
        for (int i = 0; i < n_split; ++i) M = fmaxf(M, pr[i * (vdim + 2) + vdim]);
        for (int i = 0; i < n_split; ++i) {
            const float mi = pr[i * (vdim + 2) + vdim], f = mi > -INFINITY ? expf(mi - M) : 0.f;
            L = fmaf(pr[i * (vdim + 2) + vdim + 1], f, L);
            if (c < vdim) O = fmaf(pr[i * (vdim + 2) + c], f, O);
        }
        if (MODE == UMBS_ATTN_SOFTMAX_SINK) L += expf(-M);
    }
    if (c < vdim) {
        const float inv = MODE == UMBS_ATTN_SIGMOID ? 1.f : 1.f / L;
        float gt = 1.f;
        if (a.gate) gt = sigmoidf_(a.gate[(int64_t)t * a.ldg + (a.gate_per_head ? h : h * vdim + c)]);
        ((T*)a.out)[(int64_t)t * a.heads * vdim + (int64_t)h * vdim + c] = from_f32<T>(O * inv * gt);
    }
}

template <typename T, int MODE>
static int launch_decode(const CachedAttnArgs& a, const Batch& b, int n_split, float* part, cudaStream_t st) {
    cached_attention_decode_kernel<T, MODE><<<dim3(n_split, a.heads, b.n_seqs), 32 * kCdWarps, 0, st>>>(a, b, n_split, part);
    if (n_split > 1) cached_attention_merge_kernel<T, MODE><<<b.n_tokens * a.heads, a.vdim <= 128 ? 128 : 256, 0, st>>>(a, n_split, part);
    return 0;
}

template <typename T>
static int launch_decode_any(int mode, const CachedAttnArgs& a, const Batch& b, int n_split, float* part, cudaStream_t st) {
    switch (mode) {
        case UMBS_ATTN_SOFTMAX: return launch_decode<T, UMBS_ATTN_SOFTMAX>(a, b, n_split, part, st);
        case UMBS_ATTN_SOFTMAX_SINK: return launch_decode<T, UMBS_ATTN_SOFTMAX_SINK>(a, b, n_split, part, st);
        case UMBS_ATTN_SIGMOID: return launch_decode<T, UMBS_ATTN_SIGMOID>(a, b, n_split, part, st);
    }
    return UMB_ERR_ARG;
}

}  // namespace umbs

using namespace umbs;

extern "C" int umbs_cached_attention(int dtype, int mode, const void* q, const void* kv, const void* kv_cache, int kv_len,
                                     const void* pool_cache, int pool_len, const umbs_batch_t* batch, int heads,
                                     int kv_heads, int dim, int vdim, int window, int pool, float scale,
                                     const float* head_bias, const float* gate, int64_t ldg, int gate_per_head,
                                     float* split_scratch, size_t split_bytes, void* out, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads != 0 || kv_len < 1) return UMB_ERR_ARG;
    if (pool > 0 && (window <= 0 || pool_cache == nullptr || pool_len < 1)) return UMB_ERR_ARG;
    if (dim < 1 || vdim < 1 || dim > 256 || vdim > 256) return UMB_ERR_UNSUPPORTED;      // tiles and lanes are sized for heads up to 256
    cudaStream_t st = (cudaStream_t)stream;
    CachedAttnArgs a{q, kv, kv_cache, pool_cache, kv_len, pool_len, heads, kv_heads, dim, vdim, window, pool, scale,
                     head_bias, gate, ldg, gate_per_head, out};
    int rc;
    if (batch->max_seq_len == 1) {
        // a decode step: about 256 keys per block, as many splits as the longest context of the step asks for, the GPU
        // has room for (two blocks per SM) and the scratch buffer holds
        const int keys = window > 0 ? (batch->max_pos0 < window ? batch->max_pos0 + 1 : window + (pool > 0 ? batch->max_pos0 / pool : 0))
                                    : batch->max_pos0 + 1;
        int n_split = (keys + 255) / 256;
        const int rows = batch->n_seqs * heads;
        n_split = n_split < 1 ? 1 : (n_split > 32 ? 32 : n_split);
        if (n_split > (296 + rows - 1) / rows) n_split = (296 + rows - 1) / rows;
        const size_t per_split = (size_t)rows * (vdim + 2) * sizeof(float);
        if (split_scratch == nullptr || per_split == 0) n_split = 1;
        else if ((size_t)n_split * per_split > split_bytes) n_split = (int)(split_bytes / per_split);
        if (n_split < 1) n_split = 1;
        if (dtype == UMBS_BF16) rc = launch_decode_any<__nv_bfloat16>(mode, a, *batch, n_split, split_scratch, st);
        else if (dtype == UMBS_F32) rc = launch_decode_any<float>(mode, a, *batch, n_split, split_scratch, st);
        else return UMB_ERR_ARG;
        if (rc) return rc;
        count_launches(n_split > 1 ? 2 : 1);
        return (int)cudaGetLastError();
    }
    if (dtype == UMBS_BF16) rc = launch_any<__nv_bfloat16>(mode, a, *batch, st);
    else if (dtype == UMBS_F32) rc = launch_any<float>(mode, a, *batch, st);
    else return UMB_ERR_ARG;
    if (rc) return rc;
    count_launches(1);
    return (int)cudaGetLastError();
}
