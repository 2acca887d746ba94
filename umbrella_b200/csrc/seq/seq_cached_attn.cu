// Attention of a ragged step over a per-slot key/value cache: sliding window (or everything before the row), optionally
// with one mean key/value per block of older tokens, and three ways from scores to weights (softmax, softmax with a
// sink, sigmoid).  A key is read where it lives: tokens of the step from the step's own rows, older tokens from the
// slot's cache rows (position p at row p mod kv_len), pooled blocks from the slot's block table -- so a prompt in one
// piece, in portions, and token-by-token decoding all walk the same keys in the same order.
//
// Tile kernel (any step): one block = 64 consecutive query rows of one (sequence, head); 256 threads as 16 x 16, a thread
// owns 4 rows x 4 keys of the score tile and 4 rows x VC value columns of the output; per tile of 64 keys the scores come
// from transposed fp32 tiles in shared memory, the weights go back through shared memory for the value product.
// Decode kernel (one token per sequence): one block = (sequence, head, split); a warp takes every 8th key of the block's
// share, lanes striding over the head's dimensions; partial (max, sum, output) triples are merged per block and, with more
// than one split, by a second kernel.
// Everything is fp32 arithmetic; T is the storage type of q, the key/value rows and the output.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "seq_internal.h"

namespace umbs {

constexpr int kCaQ = 64, kCaK = 64, kCaS = 68;        // rows and keys per tile; row stride of the [d][row] tiles

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
    float* Ks = Qs + (size_t)dim * kCaS;              // [dim][kCaS]  Ks[d][key]
    float* Vs = Ks + (size_t)dim * kCaS;              // [kCaK][VP]
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
        __syncthreads();                              // the previous tile is consumed (first time round: Qs is written)
        for (int i = tid; i < kCaK * dim; i += 256) {
            const int kk = i / dim, d = i - kk * dim, j = base + kk;
            float val = 0.f;
            if (j <= hi) {
                const T* src = in_pool ? pooled + ((int64_t)slot * a.pool_len + j) * row_kv
                             : (j >= pos0 ? kv + (int64_t)(start + j - pos0) * row_kv
                                          : cache + ((int64_t)slot * a.kv_len + j % a.kv_len) * row_kv);
                val = to_f32(src[koff + d]);
            }
            Ks[d * kCaS + kk] = val;
        }
        for (int i = tid; i < kCaK * VW; i += 256) {
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
        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) sc[i][jj] = 0.f;
        for (int d = 0; d < dim; ++d) {
            const float4 qv = *reinterpret_cast<const float4*>(Qs + d * kCaS + ty * 4);
            const float4 kv4 = *reinterpret_cast<const float4*>(Ks + d * kCaS + tx * 4);
            const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) sc[i][jj] = fmaf(qa[i], ka[jj], sc[i][jj]);
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
    const size_t smem = ((size_t)2 * a.dim * kCaS + (size_t)kCaK * (16 * VC + 4) + (size_t)kCaK * kCaS) * sizeof(float);
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
    return a.vdim <= 64 ? launch_tiles<T, 4, MODE>(a, b, st) : launch_tiles<T, 8, MODE>(a, b, st);
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
    if (!umbs_window_attention_fits(dim, vdim)) return UMB_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    CachedAttnArgs a{q, kv, kv_cache, pool_cache, kv_len, pool_len, heads, kv_heads, dim, vdim, window, pool, scale,
                     head_bias, gate, ldg, gate_per_head, out};
    (void)split_scratch; (void)split_bytes;
    int rc;
    if (dtype == UMBS_BF16) rc = launch_any<__nv_bfloat16>(mode, a, *batch, st);
    else if (dtype == UMBS_F32) rc = launch_any<float>(mode, a, *batch, st);
    else return UMB_ERR_ARG;
    if (rc) return rc;
    count_launches(1);
    return (int)cudaGetLastError();
}
