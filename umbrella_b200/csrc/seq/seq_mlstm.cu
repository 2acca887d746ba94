// mLSTM: a matrix memory per head with exponential input gates, sigmoid forget gates and a running maximum that keeps
// the exponentials in range (see umbs_mlstm in include/umbrella_b200_seq.h).  Three kernels per step:
//   gates       one warp per (sequence, head): the log gates of 32 tokens at a time, the running maximum by a warp scan
//               of the maps m -> max(m + f, i) (they compose: (f1, i1) then (f2, i2) = (f1 + f2, max(i1 + f2, i2))), and
//               from it each token's decay e^(f + m' - m), input weight e^(i - m) and floor e^(-m);
//   recurrence  one block per (sequence, head, 32 columns) walking the tokens in order with its slice of the state in
//               registers -- the walk of the retention kernel with a decay and an input weight per token; the normaliser
//               n rides along as one more value column whose value is 1, so n . q falls out of the same product;
//   finish      one warp per (token, head): division by max(|n . q|, e^(-m)) + 1e-6, unit RMS, weight, output gate.
// Everything is fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <algorithm>
#include <stdint.h>

#include "seq_internal.h"

namespace umbs {

__device__ __forceinline__ float warp_sum_ml(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// gates[t, h] = (decay, input weight, floor)
__global__ void mlstm_gates_kernel(const float* __restrict__ proj, int64_t ld, int off_i, int off_f,
                                   const float* __restrict__ gate_bias, Batch b, int heads, float cap, float* __restrict__ state,
                                   int64_t state_stride, int m_off, float* __restrict__ gates) {
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (wid >= b.n_seqs * heads) return;
    const int s = wid / heads, h = wid - s * heads;
    const int start = b.seq_start[s], len = b.seq_len[s];
    float* m_state = state + ((int64_t)b.seq_slot[s] * heads + h) * state_stride + m_off;
    float m_in = b.seq_pos0[s] > 0 ? *m_state : 0.f;
    const float bi = gate_bias ? gate_bias[h] : 0.f, bf = gate_bias ? gate_bias[heads + h] : 0.f;
    for (int t0 = 0; t0 < len; t0 += 32) {
        const bool ok = t0 + lane < len;
        const int64_t t = start + t0 + lane;
        float fl = 0.f, il = -INFINITY;                            // the identity map for lanes past the end
        if (ok) {
            il = cap * tanhf((proj[t * ld + off_i + h] + bi) / cap);
            fl = log_sigmoid(cap * tanhf((proj[t * ld + off_f + h] + bf) / cap));
        }
        float A = fl, B = il;                                      // inclusive scan of the composed maps
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float Ae = __shfl_up_sync(0xffffffffu, A, d), Be = __shfl_up_sync(0xffffffffu, B, d);
            if (lane >= d) { B = fmaxf(Be + A, B); A = Ae + A; }
        }
        const float m = fmaxf(m_in + A, B);
        float m_prev = __shfl_up_sync(0xffffffffu, m, 1);
        if (lane == 0) m_prev = m_in;
        if (ok) {
            float* g = gates + (t * heads + h) * 3;
            g[0] = expf(fl + m_prev - m);
            g[1] = expf(il - m);
            g[2] = expf(-m);
        }
        m_in = __shfl_sync(0xffffffffu, m, 31);                     // lanes past the end carry the last token's maximum
    }
    if (lane == 0) *m_state = m_in;
}

// See retention_kernel (seq_kernels.cu) for the walk; here V1 = vdim + 1 columns (the last one is n), per-token factors.
// A sequence may be cut into n_seg segments of seg_len tokens that run as blocks of their own (blockIdx.x = sequence *
// n_seg + segment), in two passes, as retention does: pass 1 runs every segment but a sequence's last from a zero state
// and leaves its end state L_g in seg_state and the product A_g of its tokens' decays in seg_decay; mlstm_chain_kernel
// turns these into start states (S_(g+1) = A_g S_g + L_g); pass 2 starts every segment from its entry and writes the
// outputs, and the last segment stores the slot's state.  pass 0: no segments.  The gates (and with them the running
// maximum every factor refers to) come from the gates kernel, which always walks whole sequences.
template <int DPT, int TB>
__global__ void mlstm_kernel(const float* __restrict__ proj, int64_t ld, Batch b, int heads, int dim, int vdim,
                             const float* __restrict__ gates, float* __restrict__ state, int64_t state_stride,
                             float* __restrict__ o_out, int seg_len, int n_seg, int pass, float* __restrict__ seg_state,
                             float* __restrict__ seg_decay) {
    extern __shared__ __align__(16) float sm[];
    const int DS = blockDim.y, dimP = DS * DPT, nthr = 32 * DS, V1 = vdim + 1;
    float* qs = sm;                          // [TB][dimP]
    float* ks = qs + TB * dimP;              // [TB][dimP]   keys times the token's input weight
    float* part = ks + TB * dimP;            // [DS][TB][32]
    float* vs = part + DS * TB * 32;         // [TB][32]
    float* as = vs + TB * 32;                // [TB]         the tokens' decays
    const int s = blockIdx.x / n_seg, seg = blockIdx.x - s * n_seg;
    const int h = blockIdx.y, lane = threadIdx.x, w = threadIdx.y, tid = w * 32 + lane;
    const int j = blockIdx.z * 32 + lane, d0 = w * DPT;
    const int seq_len = b.seq_len[s], t_first = seg * seg_len;
    if (t_first >= seq_len) return;
    const int len = min(seg_len, seq_len - t_first), start = b.seq_start[s] + t_first;
    const bool last_seg = t_first + len == seq_len;
    if (pass == 1 && last_seg) return;
    const int pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    const bool col = j < V1;
    const float qscale = 1.f / sqrtf((float)dim);
    const int64_t plane = (int64_t)heads * dim * V1;
    float* st = state + ((int64_t)slot * heads + h) * state_stride;
    const float* st_in = st;
    bool have = pos0 > 0;
    if (pass == 1) have = false;
    else if (pass == 2 && !(seg == 0 && last_seg)) {
        // segment 0 of a cut sequence reads the chain kernel's copy of the slot's state (entry n_seg - 1), not the slot,
        // which the sequence's last segment overwrites during this very launch
        st_in = seg_state + ((int64_t)s * n_seg + (seg > 0 ? seg - 1 : n_seg - 1)) * plane + (int64_t)h * dim * V1;
        have = true;
    }
    float S[DPT], decay_product = 1.f;
#pragma unroll
    for (int i = 0; i < DPT; ++i) S[i] = (col && have && d0 + i < dim) ? st_in[(int64_t)(d0 + i) * V1 + j] : 0.f;
    const int qoff = h * dim, koff = heads * dim + h * dim, voff = 2 * heads * dim + h * vdim;
    constexpr int EPT = TB * DPT / 32;
    float pq[EPT], pk[EPT], pv[TB], pa = 1.f;
    auto fetch = [&](int t0) {
        const int nb = min(TB, len - t0);
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
            const int i = tid + e * nthr, tt = i / dimP, d = i - tt * dimP;
            pq[e] = pk[e] = 0.f;
            if (tt < nb && d < dim) {
                const int64_t tok = start + t0 + tt;
                pq[e] = proj[tok * ld + qoff + d] * qscale;
                pk[e] = proj[tok * ld + koff + d] * gates[(tok * heads + h) * 3 + 1];
            }
        }
#pragma unroll
        for (int e = 0; e < TB; ++e) {
            const int i = tid + e * nthr, tt = i >> 5, jj = blockIdx.z * 32 + (i & 31);
            pv[e] = 0.f;
            if (i < nb * 32) {
                if (jj < vdim) pv[e] = proj[(int64_t)(start + t0 + tt) * ld + voff + jj];
                else if (jj == vdim) pv[e] = 1.f;
            }
        }
        if (tid < TB) pa = tid < nb ? gates[((int64_t)(start + t0 + tid) * heads + h) * 3] : 1.f;
    };
    fetch(0);
    for (int t0 = 0; t0 < len; t0 += TB) {
        const int nb = min(TB, len - t0);
        __syncthreads();
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
            const int i = tid + e * nthr;
            qs[i] = pq[e];
            ks[i] = pk[e];
        }
#pragma unroll
        for (int e = 0; e < TB; ++e) {
            const int i = tid + e * nthr;
            if (i < TB * 32) vs[i] = pv[e];
        }
        if (tid < TB) as[tid] = pa;
        __syncthreads();
        if (t0 + TB < len) fetch(t0 + TB);
        for (int tt = 0; tt < nb; ++tt) {
            const float v = vs[tt * 32 + lane], dec = as[tt];
            decay_product *= dec;
            const float4* k4 = reinterpret_cast<const float4*>(ks + tt * dimP + d0);
            const float4* q4 = reinterpret_cast<const float4*>(qs + tt * dimP + d0);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const float4 kv = k4[i], qv = q4[i];
                S[4 * i + 0] = fmaf(dec, S[4 * i + 0], kv.x * v); acc = fmaf(S[4 * i + 0], qv.x, acc);
                S[4 * i + 1] = fmaf(dec, S[4 * i + 1], kv.y * v); acc = fmaf(S[4 * i + 1], qv.y, acc);
                S[4 * i + 2] = fmaf(dec, S[4 * i + 2], kv.z * v); acc = fmaf(S[4 * i + 2], qv.z, acc);
                S[4 * i + 3] = fmaf(dec, S[4 * i + 3], kv.w * v); acc = fmaf(S[4 * i + 3], qv.w, acc);
            }
            part[(w * TB + tt) * 32 + lane] = acc;
        }
        __syncthreads();
        for (int i = tid; i < nb * 32 && pass != 1; i += nthr) {
            const int tt = i >> 5, l = i & 31, jj = blockIdx.z * 32 + l;
            if (jj >= V1) continue;
            float o = 0.f;
            for (int ww = 0; ww < DS; ++ww) o += part[(ww * TB + tt) * 32 + l];
            o_out[((int64_t)(start + t0 + tt) * heads + h) * V1 + jj] = o;
        }
    }
    float* st_out = st;
    if (pass == 1) {
        st_out = seg_state + ((int64_t)s * n_seg + seg) * plane + (int64_t)h * dim * V1;
        if (tid == 0 && blockIdx.z == 0) seg_decay[((int64_t)s * n_seg + seg) * heads + h] = decay_product;
    } else if (pass == 2 && !last_seg) {
        return;
    }
    if (col) {
#pragma unroll
        for (int i = 0; i < DPT; ++i)
            if (d0 + i < dim) st_out[(int64_t)(d0 + i) * V1 + j] = S[i];
    }
}

// Between the two passes: one thread per state element walks the sequence's segments in order, S <- A_g S + L_g, and
// overwrites L_g with the state segment g + 1 starts from; entry n_seg - 1 (never an end state) takes segment 0's start.
__global__ void mlstm_chain_kernel(Batch b, int heads, int dim, int V1, const float* __restrict__ state, int64_t state_stride,
                                   int seg_len, int n_seg, float* __restrict__ seg_state, const float* __restrict__ seg_decay) {
    const int64_t plane = (int64_t)heads * dim * V1;
    const int s = blockIdx.y;
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= plane) return;
    const int full = (b.seq_len[s] - 1) / seg_len;          // segments that are followed by another one
    if (full <= 0) return;
    const int h = (int)(e / ((int64_t)dim * V1));
    const int64_t in_head = e - (int64_t)h * dim * V1;
    float S = b.seq_pos0[s] > 0 ? state[((int64_t)b.seq_slot[s] * heads + h) * state_stride + in_head] : 0.f;
    float* p = seg_state + (int64_t)s * n_seg * plane + e;
    p[(int64_t)(n_seg - 1) * plane] = S;
    for (int g = 0; g < full; ++g) {
        S = fmaf(seg_decay[((int64_t)s * n_seg + g) * heads + h], S, p[(int64_t)g * plane]);
        p[(int64_t)g * plane] = S;
    }
}

template <typename T>
__global__ void mlstm_finish_kernel(const float* __restrict__ o, const float* __restrict__ gates, const float* __restrict__ proj,
                                    int64_t ld, int off_g, int n, int heads, int vdim, float eps,
                                    const float* __restrict__ norm_w, T* __restrict__ out) {
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= n * heads) return;
    const int t = w / heads, h = w - t * heads, V1 = vdim + 1;
    const float* orow = o + (int64_t)w * V1;
    const float* grow = proj + (int64_t)t * ld + off_g + h * vdim;
    const float den = fmaxf(fabsf(orow[vdim]), gates[(int64_t)w * 3 + 2]) + 1e-6f;
    float ss = 0.f;
    for (int e = lane; e < vdim; e += 32) {
        const float v = orow[e] / den;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum_ml(ss);
    const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
    for (int e = lane; e < vdim; e += 32) {
        const float g = 1.f / (1.f + expf(-grow[e]));
        out[(int64_t)t * heads * vdim + h * vdim + e] = from_f32<T>(orow[e] / den * inv * norm_w[h * vdim + e] * g);
    }
}

template <int DPT, int TB>
static int launch_mlstm(const float* proj, int64_t ld, const Batch& b, int heads, int dim, int vdim, const float* gates,
                        float* state, int64_t stride, float* o, int seg_len, int n_seg, int pass, float* seg_state,
                        float* seg_decay, cudaStream_t st) {
    const int ds = (dim + DPT - 1) / DPT;
    const dim3 grid(b.n_seqs * n_seg, heads, (vdim + 1 + 31) / 32), block(32, ds);
    const size_t smem = ((size_t)2 * TB * ds * DPT + (size_t)ds * TB * 32 + TB * 32 + TB) * sizeof(float);
    static size_t set = 0;
    if (smem > 48 * 1024 && smem > set) {
        cudaError_t e = cudaFuncSetAttribute(mlstm_kernel<DPT, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = smem;
    }
    mlstm_kernel<DPT, TB><<<grid, block, smem, st>>>(proj, ld, b, heads, dim, vdim, gates, state, stride, o, seg_len, n_seg, pass,
                                                     seg_state, seg_decay);
    return 0;
}

}  // namespace umbs

using namespace umbs;

extern "C" int umbs_mlstm(int dtype, const float* proj, int64_t ld, const float* gate_bias, const umbs_batch_t* batch,
                          int heads, int dim, int vdim, float gate_cap, float eps, const float* out_norm_w, float* state,
                          float* gates_scratch, float* o_scratch, float* seg_scratch, size_t seg_bytes, void* out,
                          umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (heads < 1 || dim < 1 || vdim < 1 || !(gate_cap > 0.f) || out_norm_w == nullptr) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t stride = (int64_t)dim * (vdim + 1) + 1;
    const int off_g = 2 * heads * dim + heads * vdim, off_i = off_g + heads * vdim, off_f = off_i + heads;
    const int warps = batch->n_seqs * heads;
    mlstm_gates_kernel<<<(warps + 3) / 4, 128, 0, st>>>(proj, ld, off_i, off_f, gate_bias, *batch, heads, gate_cap, state, stride,
                                                        dim * (vdim + 1), gates_scratch);
    // Few blocks and long sequences (one long prompt): cut the sequences into segments that run side by side in two passes.
    // Twice the arithmetic of the recurrence for n_seg times the blocks; differs from the single walk by fp32 rounding only.
    const int V1 = vdim + 1;
    int n_seg = 1, seg_len = batch->max_seq_len;
    const int base_blocks = batch->n_seqs * heads * ((V1 + 31) / 32);
    const size_t per_seg = (size_t)batch->n_seqs * heads * ((size_t)dim * V1 + 1) * sizeof(float);      // states + decay products
    // about four blocks per SM run side by side; two passes pay from three segments on (2 / n_seg of the single walk)
    if (seg_scratch != nullptr && base_blocks * 3 <= 592 && batch->max_seq_len >= 192) {
        int want = std::min(592 / base_blocks, batch->max_seq_len / 64);
        want = (int)std::min<size_t>(want, seg_bytes / per_seg);
        if (want >= 3) {
            seg_len = ((batch->max_seq_len + want - 1) / want + 15) & ~15;
            n_seg = (batch->max_seq_len + seg_len - 1) / seg_len;
        }
    }
    float* seg_decay = n_seg > 1 ? seg_scratch + (size_t)batch->n_seqs * n_seg * heads * dim * V1 : nullptr;
    auto run = [&](int pass) -> int {
        if (dim <= 32) return launch_mlstm<8, 16>(proj, ld, *batch, heads, dim, vdim, gates_scratch, state, stride, o_scratch, seg_len, n_seg, pass, seg_scratch, seg_decay, st);
        if (dim <= 128) return launch_mlstm<16, 16>(proj, ld, *batch, heads, dim, vdim, gates_scratch, state, stride, o_scratch, seg_len, n_seg, pass, seg_scratch, seg_decay, st);
        if (dim <= 512) return launch_mlstm<32, 8>(proj, ld, *batch, heads, dim, vdim, gates_scratch, state, stride, o_scratch, seg_len, n_seg, pass, seg_scratch, seg_decay, st);
        return UMB_ERR_UNSUPPORTED;
    };
    int rc;
    unsigned launches = 3;
    if (n_seg > 1) {
        rc = run(1);
        if (rc) return rc;
        const int64_t plane = (int64_t)heads * dim * V1;
        mlstm_chain_kernel<<<dim3((unsigned)((plane + 255) / 256), batch->n_seqs), 256, 0, st>>>(*batch, heads, dim, V1, state, stride,
                                                                                             seg_len, n_seg, seg_scratch, seg_decay);
        launches += 2;
        rc = run(2);
    } else {
        rc = run(0);
    }
    if (rc) return rc;
    const int fw = batch->n_tokens * heads;
    if (dtype == UMBS_BF16)
        mlstm_finish_kernel<__nv_bfloat16><<<(fw + 3) / 4, 128, 0, st>>>(o_scratch, gates_scratch, proj, ld, off_g, batch->n_tokens,
                                                                        heads, vdim, eps, out_norm_w, (__nv_bfloat16*)out);
    else if (dtype == UMBS_F32)
        mlstm_finish_kernel<float><<<(fw + 3) / 4, 128, 0, st>>>(o_scratch, gates_scratch, proj, ld, off_g, batch->n_tokens, heads,
                                                                vdim, eps, out_norm_w, (float*)out);
    else return UMB_ERR_ARG;
    count_launches(launches);
    return (int)cudaGetLastError();
}
