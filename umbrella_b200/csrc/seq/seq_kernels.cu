// Kernels of the sequence-state decoders (see include/umbrella_b200_seq.h): group norm + token shift, decayed linear
// attention with rotary positions, sliding-window latent attention over a ring of latents, top-k routing with an
// expert-sorted pair list, the depth-weighted residual mix.  Everything here is fp32 arithmetic on fp32 or bf16
// storage; the matrix products live in seq_gemm.cu.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "seq_internal.h"

namespace umbs {

// Deterministic block sum (fixed tree: shuffles inside a warp, then warp 0 over the per-warp partials).
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ float block_sum(float v, float* red) {   // red: >= 33 floats of shared memory
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float s = lane < nw ? red[lane] : 0.f;
        s = warp_sum(s);
        if (lane == 0) red[32] = s;
    }
    __syncthreads();
    return red[32];
}

// ------------------------------------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table, float* __restrict__ y,
                                 int width) {
    const int t = blockIdx.x;
    const T* row = table + (int64_t)ids[t] * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) y[(int64_t)t * width + e] = to_f32(row[e]);
}

// ------------------------------------------------------------------------------------------------ group norm (+ shift)
// inverse root mean square of group g of row x (all threads get it)
__device__ float group_inv_rms(const float* __restrict__ x, int g, int gsz, float eps, float* red) {
    float s = 0.f;
    for (int e = threadIdx.x; e < gsz; e += blockDim.x) {
        const float v = x[g * gsz + e];
        s += v * v;
    }
    s = block_sum(s, red);
    return 1.f / sqrtf(s / (float)gsz + eps);
}

template <typename T>
__global__ void group_norm_shift_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                        const float* __restrict__ shift_w, float* __restrict__ shift_state, int slots,
                                        Batch b, int width, int groups, float eps, T* __restrict__ h_out,
                                        T* __restrict__ hs_out) {
    extern __shared__ float sm[];     // [groups] own inverse rms, [groups] previous token's, [33] reduction
    float* inv_own = sm;
    float* inv_prev = sm + groups;
    float* red = sm + 2 * groups;
    const int t = blockIdx.x, s = b.tok_seq[t];
    const int start = b.seq_start[s], len = b.seq_len[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s], par = b.seq_parity[s];
    const int gsz = width / groups;
    const bool first = (t == start), last = (t == start + len - 1);
    const float* xr = x + (int64_t)t * width;
    const float* xp = xr - width;
    for (int g = 0; g < groups; ++g) {
        const float a = group_inv_rms(xr, g, gsz, eps, red);
        float p = 0.f;
        if (shift_w != nullptr && !first) p = group_inv_rms(xp, g, gsz, eps, red);
        if (threadIdx.x == 0) { inv_own[g] = a; inv_prev[g] = p; }
    }
    __syncthreads();
    const float* st_in = shift_state + ((int64_t)par * slots + slot) * width;
    float* st_out = shift_state + ((int64_t)(par ^ 1) * slots + slot) * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const int g = e / gsz;
        const float h = xr[e] * inv_own[g] * w[e];
        h_out[(int64_t)t * width + e] = from_f32<T>(h);
        if (shift_w != nullptr) {
            float hp;
            if (!first) hp = xp[e] * inv_prev[g] * w[e];
            else hp = pos0 > 0 ? st_in[e] : 0.f;
            hs_out[(int64_t)t * width + e] = from_f32<T>(h + (hp - h) * shift_w[e]);
            if (last) st_out[e] = h;
        }
    }
}

template <typename T>
__global__ void group_norm_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                       const float* __restrict__ w, int width, int groups, float eps, T* __restrict__ y) {
    extern __shared__ float sm[];
    float* inv = sm;
    float* red = sm + groups;
    const int r = blockIdx.x;
    const float* xr = x + (int64_t)(rows ? rows[r] : r) * width;
    const int gsz = width / groups;
    for (int g = 0; g < groups; ++g) {
        const float a = group_inv_rms(xr, g, gsz, eps, red);
        if (threadIdx.x == 0) inv[g] = a;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < width; e += blockDim.x)
        y[(int64_t)r * width + e] = from_f32<T>(xr[e] * inv[e / gsz] * w[e]);
}

// ------------------------------------------------------------------------------------------------ retention
// One block = (sequence, head, a slice of NC value columns).  The slice's part of the state, S[dim][NC], sits in
// shared memory; thread j owns column j.  Tokens go in order; q and k of TB tokens at a time are rotated into
// shared memory by the whole block.
constexpr int kRetTB = 8;
__global__ void retention_kernel(const float* __restrict__ qkvg, int64_t ld, Batch b, int heads, int dim, int vdim,
                                 int rot_dims, const float* __restrict__ inv_freq, const float* __restrict__ decay,
                                 float* __restrict__ state, float* __restrict__ o_out) {
    extern __shared__ float sm[];
    const int NC = blockDim.x;
    float* S = sm;                         // [dim][NC]
    float* qs = S + (size_t)dim * NC;      // [TB][dim]
    float* ks = qs + kRetTB * dim;         // [TB][dim]
    const int s = blockIdx.x, h = blockIdx.y, j = blockIdx.z * NC + threadIdx.x;
    const int start = b.seq_start[s], len = b.seq_len[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    const bool col = j < vdim;
    const float dec = decay[h];
    const float kscale = 1.f / sqrtf((float)dim);
    const int half = rot_dims / 2;
    float* st = state + (((int64_t)slot * heads + h) * dim) * vdim;
    for (int d = 0; d < dim; ++d) S[d * NC + threadIdx.x] = (col && pos0 > 0) ? st[(int64_t)d * vdim + j] : 0.f;
    const int qoff = h * dim, koff = heads * dim + h * dim, voff = 2 * heads * dim + h * vdim;
    for (int t0 = 0; t0 < len; t0 += kRetTB) {
        const int nb = min(kRetTB, len - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nb * dim; i += NC) {
            const int tt = i / dim, d = i - tt * dim;
            const float* row = qkvg + (int64_t)(start + t0 + tt) * ld;
            float q = row[qoff + d], k = row[koff + d];
            if (d < rot_dims) {
                const int fi = d < half ? d : d - half;
                const float ang = (float)(pos0 + t0 + tt) * inv_freq[fi];
                const float c = cosf(ang), sn = sinf(ang);
                if (d < half) {
                    q = q * c - row[qoff + d + half] * sn;
                    k = k * c - row[koff + d + half] * sn;
                } else {
                    q = q * c + row[qoff + d - half] * sn;
                    k = k * c + row[koff + d - half] * sn;
                }
            }
            qs[tt * dim + d] = q;
            ks[tt * dim + d] = k * kscale;
        }
        __syncthreads();
        if (col) {
            for (int tt = 0; tt < nb; ++tt) {
                const int64_t tok = start + t0 + tt;
                const float v = qkvg[tok * ld + voff + j];
                float acc = 0.f;
                for (int d = 0; d < dim; ++d) {
                    const float sv = dec * S[d * NC + threadIdx.x] + ks[tt * dim + d] * v;
                    S[d * NC + threadIdx.x] = sv;
                    acc += sv * qs[tt * dim + d];
                }
                o_out[tok * ((int64_t)heads * vdim) + h * vdim + j] = acc;
            }
        }
    }
    if (col)
        for (int d = 0; d < dim; ++d) st[(int64_t)d * vdim + j] = S[d * NC + threadIdx.x];
}

// o / rms(o) per head, times silu(g); one warp per (token, head)
template <typename T>
__global__ void retention_gate_kernel(const float* __restrict__ o, const float* __restrict__ qkvg, int64_t ld, int n,
                                      int heads, int dim, int vdim, float eps, T* __restrict__ out) {
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= n * heads) return;
    const int t = w / heads, h = w - t * heads;
    const float* orow = o + (int64_t)t * heads * vdim + h * vdim;
    const float* grow = qkvg + (int64_t)t * ld + 2 * heads * dim + heads * vdim + h * vdim;
    float s = 0.f;
    for (int e = lane; e < vdim; e += 32) s += orow[e] * orow[e];
    s = warp_sum(s);
    const float inv = 1.f / sqrtf(s / (float)vdim + eps);
    for (int e = lane; e < vdim; e += 32) {
        const float g = grow[e];
        out[(int64_t)t * heads * vdim + h * vdim + e] = from_f32<T>(orow[e] * inv * (g / (1.f + expf(-g))));
    }
}

// ------------------------------------------------------------------------------------------------ latent attention
template <typename T>
__global__ void latent_norm_kernel(const float* __restrict__ x, int q_rank, int kv_rank, const float* __restrict__ qw,
                                   const float* __restrict__ kw, float eps, T* __restrict__ cq, T* __restrict__ c) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const float* xr = x + (int64_t)t * (q_rank + kv_rank);
    float s = 0.f;
    for (int e = threadIdx.x; e < q_rank; e += blockDim.x) s += xr[e] * xr[e];
    s = block_sum(s, red);
    const float iq = 1.f / sqrtf(s / (float)q_rank + eps);
    s = 0.f;
    for (int e = threadIdx.x; e < kv_rank; e += blockDim.x) s += xr[q_rank + e] * xr[q_rank + e];
    s = block_sum(s, red);
    const float ik = 1.f / sqrtf(s / (float)kv_rank + eps);
    for (int e = threadIdx.x; e < q_rank; e += blockDim.x) cq[(int64_t)t * q_rank + e] = from_f32<T>(xr[e] * iq * qw[e]);
    for (int e = threadIdx.x; e < kv_rank; e += blockDim.x)
        c[(int64_t)t * kv_rank + e] = from_f32<T>(xr[q_rank + e] * ik * kw[e]);
}

// One warp per (token, head).  Lane l scores key jlo + 32 i + l; the output's kv_rank components are spread over the
// lanes (component r on lane r mod 32), RPL per lane.
template <typename T, int RPL>
__global__ void latent_attention_kernel(const float* __restrict__ q_abs, const T* __restrict__ c, const T* __restrict__ ring,
                                        int ring_len, Batch b, int heads, int R, int window, float scale,
                                        T* __restrict__ out) {
    extern __shared__ float sm[];          // [warps][R] queries
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int w = blockIdx.x * (blockDim.x >> 5) + wib;
    if (w >= b.n_tokens * heads) return;
    const int t = w / heads, h = w - t * heads;
    float* q = sm + (size_t)wib * R;
    for (int r = lane; r < R; r += 32) q[r] = q_abs[((int64_t)t * heads + h) * R + r];
    __syncwarp();
    const int s = b.tok_seq[t], pos = b.tok_pos[t];
    const int start = b.seq_start[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    const T* rbase = ring + (int64_t)slot * ring_len * R;
    const int jlo = max(0, pos - window + 1);
    float m = -INFINITY, l = 0.f, acc[RPL];
#pragma unroll
    for (int i = 0; i < RPL; ++i) acc[i] = 0.f;
    for (int j0 = jlo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const T* row = nullptr;
        if (j <= pos) row = j >= pos0 ? c + (int64_t)(start + j - pos0) * R : rbase + (int64_t)(j % ring_len) * R;
        float sc = -INFINITY;
        if (row != nullptr) {
            float d = 0.f;
            for (int r = 0; r < R; ++r) d += q[r] * to_f32(row[r]);
            sc = d * scale;
        }
        const float mn = fmaxf(m, warp_max(sc));
        const float corr = expf(m - mn);            // m = -inf on the first tile: exp(-inf) = 0
        const float p = row != nullptr ? expf(sc - mn) : 0.f;
        l = l * corr + warp_sum(p);
        m = mn;
#pragma unroll
        for (int i = 0; i < RPL; ++i) acc[i] *= corr;
        const int nk = min(32, pos - j0 + 1);
        for (int jj = 0; jj < nk; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int jk = j0 + jj;
            const T* rj = jk >= pos0 ? c + (int64_t)(start + jk - pos0) * R : rbase + (int64_t)(jk % ring_len) * R;
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int r = lane + 32 * i;
                if (r < R) acc[i] += pj * to_f32(rj[r]);
            }
        }
    }
    const float invl = 1.f / l;
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
        const int r = lane + 32 * i;
        if (r < R) out[((int64_t)t * heads + h) * R + r] = from_f32<T>(acc[i] * invl);
    }
}

template <typename T>
__global__ void ring_append_kernel(const T* __restrict__ c, T* __restrict__ ring, int ring_len, Batch b, int R) {
    const int t = blockIdx.x, s = b.tok_seq[t], pos = b.tok_pos[t];
    if (pos < b.seq_pos0[s] + b.seq_len[s] - ring_len) return;     // a later token of this step takes the row
    T* dst = ring + ((int64_t)b.seq_slot[s] * ring_len + pos % ring_len) * R;
    for (int r = threadIdx.x; r < R; r += blockDim.x) dst[r] = c[(int64_t)t * R + r];
}

// ------------------------------------------------------------------------------------------------ routing
// One warp per token: logits in fp32, `top` rounds of arg-max (lowest index wins a tie), softmax over the chosen.
template <typename T>
__global__ void moe_router_kernel(const T* __restrict__ h, int n, int width, const float* __restrict__ wr, int experts,
                                  int top, float* __restrict__ sel_w, int32_t* __restrict__ sel_e,
                                  int32_t* __restrict__ counts) {
    extern __shared__ float sm[];          // [warps][experts]
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + wib;
    if (t >= n) return;
    float* z = sm + (size_t)wib * experts;
    for (int e = 0; e < experts; ++e) {
        float s = 0.f;
        for (int k = lane; k < width; k += 32) s += to_f32(h[(int64_t)t * width + k]) * wr[(int64_t)e * width + k];
        s = warp_sum(s);
        if (lane == 0) z[e] = s;
    }
    __syncwarp();
    if (lane == 0) {
        float zmax = 0.f, den = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int e = 0; e < experts; ++e)
                if (z[e] > bv) { bv = z[e]; best = e; }
            if (k == 0) zmax = bv;
            const float p = expf(bv - zmax);
            sel_e[(int64_t)t * top + k] = best;
            sel_w[(int64_t)t * top + k] = p;
            den += p;
            z[best] = -INFINITY;
            atomicAdd(counts + best, 1);
        }
        for (int k = 0; k < top; ++k) sel_w[(int64_t)t * top + k] /= den;
    }
}

__global__ void moe_offsets_kernel(const int32_t* __restrict__ counts, int experts, int32_t* __restrict__ grp_off,
                                   int32_t* __restrict__ cursor) {
    if (threadIdx.x == 0) {
        int s = 0;
        for (int e = 0; e < experts; ++e) { grp_off[e] = s; cursor[e] = 0; s += counts[e]; }
        grp_off[experts] = s;
    }
}

__global__ void moe_scatter_kernel(const int32_t* __restrict__ sel_e, int n_pairs, int top,
                                   const int32_t* __restrict__ grp_off, int32_t* __restrict__ cursor,
                                   int32_t* __restrict__ pair_tok, int32_t* __restrict__ pair_pos) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int e = sel_e[i];
    const int p = grp_off[e] + atomicAdd(cursor + e, 1);
    pair_tok[p] = i / top;
    pair_pos[i] = p;
}

// ------------------------------------------------------------------------------------------------ residual + depth mix
__global__ void depth_mix_kernel(const float* x, const float* __restrict__ mix, const float* __restrict__ pair_out,
                                 const float* __restrict__ sel_w, const int32_t* __restrict__ pair_pos, int top,
                                 const float* __restrict__ shared, float* __restrict__ stack, int layer,
                                 const float* __restrict__ depth_w, float* x_out, float* __restrict__ copy_out,
                                 int n, int width) {
    const int t = blockIdx.x;
    const int64_t plane = (int64_t)n * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const int64_t i = (int64_t)t * width + e;
        float ff = 0.f;
        bool any = false;
        if (pair_out != nullptr) {
            for (int k = 0; k < top; ++k)
                ff += sel_w[(int64_t)t * top + k] * pair_out[(int64_t)pair_pos[(int64_t)t * top + k] * width + e];
            any = true;
        }
        if (shared != nullptr) { ff += shared[i]; any = true; }
        const float xn = x[i] + (any ? (mix[i] + ff) : mix[i]);
        stack[(layer + 1) * plane + i] = xn;
        float y = xn;
        if (depth_w != nullptr) {
            y = 0.f;
            for (int j = 0; j <= layer; ++j) y += depth_w[j] * stack[j * plane + i];
            y += depth_w[layer + 1] * xn;
        }
        x_out[i] = y;
        if (copy_out != nullptr) copy_out[i] = y;
    }
}

}  // namespace umbs

// ================================================================================================ host entry points
using namespace umbs;

#define UMBS_DISPATCH_T(dtype, ...)                              \
    do {                                                         \
        if ((dtype) == UMBS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else if ((dtype) == UMBS_F32) { using T = float; __VA_ARGS__; }     \
        else return UMB_ERR_ARG;                                 \
    } while (0)

static inline int threads_for(int width) { return width >= 1024 ? 256 : (width >= 256 ? 128 : 64); }

extern "C" int umbs_embedding(int dtype, const int32_t* ids, const void* table, float* y, int n, int width,
                              umbs_stream_t stream) {
    if (n <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    UMBS_DISPATCH_T(dtype, embedding_kernel<T><<<n, threads_for(width), 0, st>>>(ids, (const T*)table, y, width));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_group_norm_shift(int dtype, const float* x, const float* w, const float* shift_w, float* shift_state,
                                     int slots, const umbs_batch_t* batch, int width, int groups, float eps, void* h,
                                     void* hs, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (groups <= 0 || width % groups != 0) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (2 * groups + 33) * sizeof(float);
    UMBS_DISPATCH_T(dtype, group_norm_shift_kernel<T><<<batch->n_tokens, threads_for(width / groups), smem, st>>>(
                               x, w, shift_w, shift_state, slots, *batch, width, groups, eps, (T*)h, (T*)hs));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_group_norm_rows(int dtype, const float* x, const int32_t* rows, int n_rows, const float* w, int width,
                                    int groups, float eps, void* y, umbs_stream_t stream) {
    if (n_rows <= 0) return 0;
    if (groups <= 0 || width % groups != 0) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (groups + 33) * sizeof(float);
    UMBS_DISPATCH_T(dtype, group_norm_rows_kernel<T><<<n_rows, threads_for(width / groups), smem, st>>>(
                               x, rows, w, width, groups, eps, (T*)y));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_retention(int dtype, const float* qkvg, int64_t ld, const umbs_batch_t* batch, int heads, int dim,
                              int vdim, int rot_dims, const float* inv_freq, const float* decay, float eps, float* state,
                              float* o_scratch, void* out, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (rot_dims < 0 || rot_dims > dim || (rot_dims & 1)) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    // columns per block: as many as keep the state slice in shared memory, at most 128
    int nc = 128;
    while (nc > 32 && (nc / 2 >= vdim || ((size_t)dim * nc + 2 * kRetTB * dim) * sizeof(float) > 200 * 1024)) nc /= 2;
    const size_t smem = ((size_t)dim * nc + 2 * kRetTB * dim) * sizeof(float);
    if (smem > 220 * 1024) return UMB_ERR_UNSUPPORTED;
    static size_t smem_set = 0;
    if (smem > 48 * 1024 && smem > smem_set) {
        cudaError_t e = cudaFuncSetAttribute(retention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        smem_set = smem;
    }
    dim3 grid(batch->n_seqs, heads, (vdim + nc - 1) / nc);
    retention_kernel<<<grid, nc, smem, st>>>(qkvg, ld, *batch, heads, dim, vdim, rot_dims, inv_freq, decay, state, o_scratch);
    const int warps = batch->n_tokens * heads;
    UMBS_DISPATCH_T(dtype, retention_gate_kernel<T><<<(warps + 3) / 4, 128, 0, st>>>(o_scratch, qkvg, ld, batch->n_tokens,
                                                                                   heads, dim, vdim, eps, (T*)out));
    count_launches(2);
    return (int)cudaGetLastError();
}

extern "C" int umbs_latent_norm(int dtype, const float* x, int n, int q_rank, int kv_rank, const float* q_norm,
                                const float* kv_norm, float eps, void* cq, void* c, umbs_stream_t stream) {
    if (n <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    UMBS_DISPATCH_T(dtype, latent_norm_kernel<T><<<n, threads_for(kv_rank), 0, st>>>(x, q_rank, kv_rank, q_norm, kv_norm,
                                                                                   eps, (T*)cq, (T*)c));
    count_launches(1);
    return (int)cudaGetLastError();
}

template <typename T>
static int launch_latent_attention(const float* q_abs, const void* c, const void* ring, int ring_len, const Batch& b,
                                   int heads, int R, int window, float scale, void* out, cudaStream_t st) {
    const int warps = b.n_tokens * heads, wpb = 4;
    const dim3 grid((warps + wpb - 1) / wpb), block(32 * wpb);
    const size_t smem = (size_t)wpb * R * sizeof(float);
#define UMBS_LA(RPL) latent_attention_kernel<T, RPL><<<grid, block, smem, st>>>(q_abs, (const T*)c, (const T*)ring, ring_len, b, heads, R, window, scale, (T*)out)
    if (R <= 32) UMBS_LA(1);
    else if (R <= 64) UMBS_LA(2);
    else if (R <= 128) UMBS_LA(4);
    else if (R <= 256) UMBS_LA(8);
    else if (R <= 512) UMBS_LA(16);
    else return UMB_ERR_UNSUPPORTED;
#undef UMBS_LA
    return 0;
}

extern "C" int umbs_latent_attention(int dtype, const float* q_abs, const void* c, const void* ring, int ring_len,
                                     const umbs_batch_t* batch, int heads, int kv_rank, int window, float scale, void* out,
                                     umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (window < 1 || ring_len < 1) return UMB_ERR_ARG;
    int rc = 0;
    UMBS_DISPATCH_T(dtype, rc = launch_latent_attention<T>(q_abs, c, ring, ring_len, *batch, heads, kv_rank, window, scale,
                                                           out, (cudaStream_t)stream));
    if (rc) return rc;
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_ring_append(int dtype, const void* c, void* ring, int ring_len, const umbs_batch_t* batch, int kv_rank,
                                umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    UMBS_DISPATCH_T(dtype, ring_append_kernel<T><<<batch->n_tokens, 64, 0, st>>>((const T*)c, (T*)ring, ring_len, *batch,
                                                                              kv_rank));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_moe_route(int dtype, const void* h, int n, int width, const float* w_router, int experts, int top,
                              float* sel_w, int32_t* grp_off, int32_t* pair_tok, int32_t* pair_pos, int32_t* scratch,
                              umbs_stream_t stream) {
    if (n <= 0) return 0;
    if (top < 1 || top > experts) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    int32_t* counts = scratch;                 // [experts]
    int32_t* cursor = scratch + experts;       // [experts]
    int32_t* sel_e = scratch + 2 * experts;    // [n top]
    cudaError_t e = cudaMemsetAsync(counts, 0, experts * sizeof(int32_t), st);
    if (e != cudaSuccess) return (int)e;
    const int wpb = 4;
    UMBS_DISPATCH_T(dtype, moe_router_kernel<T><<<(n + wpb - 1) / wpb, 32 * wpb, (size_t)wpb * experts * sizeof(float), st>>>(
                               (const T*)h, n, width, w_router, experts, top, sel_w, sel_e, counts));
    moe_offsets_kernel<<<1, 32, 0, st>>>(counts, experts, grp_off, cursor);
    const int pairs = n * top;
    moe_scatter_kernel<<<(pairs + 255) / 256, 256, 0, st>>>(sel_e, pairs, top, grp_off, cursor, pair_tok, pair_pos);
    count_launches(3);
    return (int)cudaGetLastError();
}

extern "C" int umbs_depth_mix(const float* x, const float* mix, const float* pair_out, const float* sel_w,
                              const int32_t* pair_pos, int top, const float* shared, float* stack, int layer,
                              const float* depth_w, float* x_out, float* copy_out, int n, int width, umbs_stream_t stream) {
    if (n <= 0) return 0;
    depth_mix_kernel<<<n, threads_for(width), 0, (cudaStream_t)stream>>>(x, mix, pair_out, sel_w, pair_pos, top, shared, stack,
                                                                        layer, depth_w, x_out, copy_out, n, width);
    count_launches(1);
    return (int)cudaGetLastError();
}
