// Sliding-window softmax attention over per-head keys and values that all sit in the step itself: the form a whole
// prompt takes (no token of the step sees anything older than the step).  Keys and values are then up-projected once
// per token by a matrix product and a (row, key) pair costs dim + vdim multiply-adds, where the latent form -- which a
// decode step needs, because only latents are cached -- costs twice the latent rank.
//
// One block = 64 consecutive query rows of one (sequence, head); 256 threads as 16 x 16, a thread owns 4 rows x 4 keys
// of the score tile and 4 rows x VC value columns of the output.  Per tile of 64 keys:
//   scores   Q K^T from transposed fp32 tiles in shared memory (two 16-byte loads per 16 multiply-adds),
//   softmax  running maximum / sum per row in fp32, reduced over the 16 threads that share the row,
//   values   P V with P handed over through shared memory.
// Everything is fp32 arithmetic; T is the storage type of q, k, v and the output.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "seq_internal.h"

namespace umbs {

constexpr int kWaQ = 64, kWaK = 64, kWaS = 68;        // rows and keys per tile; row stride of the [d][row] tiles

// Options beside the plain form: a key part all heads share (ks: [n_tokens, sdim] with row stride ldks; a head's key is its
// own dim numbers followed by the shared sdim, its query has dim + sdim numbers; here `dim` is that sum and `kdim` the head's
// own part), a sink (a score without key or value that counts once in the sum: sink[h], or 0 without the array) and a
// sigmoid gate per output element.
struct WindowExtra {
    const void* ks; int64_t ldks; int kdim;
    int use_sink; const float* sink;
    const float* gate; int64_t ldg;
};

template <typename T, int VC>
__global__ void __launch_bounds__(256) window_attention_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k,
                                                               int64_t ldk, const T* __restrict__ v, int64_t ldv, Batch b,
                                                               int dim, int vdim, int window, float scale,
                                                               T* __restrict__ out, int64_t ldo, WindowExtra x, int kc) {
    // kc: dimensions of a key tile held at a time (all of them up to 64; larger heads add their scores up over several
    // passes and keep the weights where the key tile was, which leaves room for two blocks on an SM)
    extern __shared__ __align__(16) float sm[];
    const T* ks = (const T*)x.ks;
    const int kdim = x.kdim;
    const bool alias_p = kc < dim;
    constexpr int VW = 16 * VC, VP = VW + 4;          // value columns a block covers; row stride of the value tile
    float* Qs = sm;                                   // [dim][kWaS]  Qs[d][row]
    float* Ks = Qs + (size_t)dim * kWaS;              // [kc][kWaS]   Ks[d][key]
    float* Vs = Ks + (size_t)kc * kWaS;               // [kWaK][VP]
    float* Ps = alias_p ? Ks : Vs + (size_t)kWaK * VP;   // [kWaK][kWaS] Ps[key][row]
    // the last row tiles see the most keys: they are handed out first, so that the short ones fill the tail of the grid
    const int s = blockIdx.z, h = blockIdx.y, q0 = (int)(gridDim.x - 1 - blockIdx.x) * kWaQ;
    const int len = b.seq_len[s], start = b.seq_start[s];
    if (q0 >= len) return;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    for (int i = tid; i < kWaQ * dim; i += 256) {
        const int r = i / dim, d = i - r * dim;
        Qs[d * kWaS + r] = (q0 + r < len) ? to_f32(q[(int64_t)(start + q0 + r) * ldq + (int64_t)h * dim + d]) : 0.f;
    }
    float m[4], l[4], o[4][VC];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m[i] = x.use_sink ? (x.sink ? x.sink[h] : 0.f) : -INFINITY;
        l[i] = x.use_sink ? 1.f : 0.f;
#pragma unroll
        for (int c = 0; c < VC; ++c) o[i][c] = 0.f;
    }
    const int row_hi = min(len, q0 + kWaQ) - 1;       // last row of the block = last key any of its rows sees
    for (int j0 = max(0, q0 - window + 1); j0 <= row_hi; j0 += kWaK) {
        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) sc[i][jj] = 0.f;
        for (int d0 = 0; d0 < dim; d0 += kc) {
            const int dc = min(kc, dim - d0);
            __syncthreads();                          // the previous pass or tile is consumed (first time round: Qs is written)
            for (int i = tid; i < kWaK * dc; i += 256) {
                const int kk = i / dc, d = d0 + i - kk * dc, j = j0 + kk;
                float kvl = 0.f;
                if (j <= row_hi)
                    kvl = d < kdim ? to_f32(k[(int64_t)(start + j) * ldk + (int64_t)h * kdim + d])
                                   : to_f32(ks[(int64_t)(start + j) * x.ldks + (d - kdim)]);
                Ks[(d - d0) * kWaS + kk] = kvl;
            }
            for (int i = tid; d0 == 0 && i < kWaK * VW; i += 256) {
                const int kk = i / VW, c = i - kk * VW, j = j0 + kk;
                Vs[kk * VP + c] = (j <= row_hi && c < vdim) ? to_f32(v[(int64_t)(start + j) * ldv + (int64_t)h * vdim + c]) : 0.f;
            }
            __syncthreads();
            for (int d = 0; d < dc; ++d) {
                const float4 qv = *reinterpret_cast<const float4*>(Qs + (d0 + d) * kWaS + ty * 4);
                const float4 kv = *reinterpret_cast<const float4*>(Ks + d * kWaS + tx * 4);
                const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) sc[i][jj] = fmaf(qa[i], ka[jj], sc[i][jj]);
            }
        }
        if (alias_p) __syncthreads();                 // the weights go where the last key pass sits
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rp = q0 + ty * 4 + i;           // the row's index in its sequence; only differences to keys matter
            float val[4], mx = -INFINITY;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int j = j0 + tx * 4 + jj;
                const bool vis = rp < len && j <= rp && j > rp - window;
                val[jj] = vis ? sc[i][jj] * scale : -INFINITY;
                mx = fmaxf(mx, val[jj]);
            }
#pragma unroll
            for (int w = 8; w > 0; w >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));   // the row's 16 threads
            const float mn = fmaxf(m[i], mx);
            float p[4] = {0.f, 0.f, 0.f, 0.f}, sum = 0.f, corr = 1.f;
            if (mn > -INFINITY) {
                corr = expf(m[i] - mn);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    p[jj] = val[jj] > -INFINITY ? expf(val[jj] - mn) : 0.f;
                    sum += p[jj];
                }
            }
#pragma unroll
            for (int w = 8; w > 0; w >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, w);
            l[i] = l[i] * corr + sum;
            m[i] = mn;
#pragma unroll
            for (int c = 0; c < VC; ++c) o[i][c] *= corr;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) Ps[(tx * 4 + jj) * kWaS + ty * 4 + i] = p[jj];
        }
        __syncthreads();
        for (int kk = 0; kk < kWaK; ++kk) {
            const float4 pv = *reinterpret_cast<const float4*>(Ps + kk * kWaS + ty * 4);
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
        const float inv = 1.f / l[i];
        T* orow = out + (int64_t)(start + r) * ldo + (int64_t)h * vdim;
        const float* grow = x.gate ? x.gate + (int64_t)(start + r) * x.ldg + (int64_t)h * vdim : nullptr;
#pragma unroll
        for (int cb = 0; cb < VC / 4; ++cb)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col = cb * 64 + tx * 4 + c;
                if (col < vdim) {
                    float val = o[i][cb * 4 + c] * inv;
                    if (grow != nullptr) val *= 1.f / (1.f + expf(-grow[col]));
                    orow[col] = from_f32<T>(val);
                }
            }
    }
}

template <typename T, int VC>
static int launch_window_attention(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                                   const Batch& b, int heads, int dim, int vdim, int window, float scale, void* out,
                                   int64_t ldo, const WindowExtra& x, cudaStream_t st) {
    const int kc = dim <= 64 ? dim : 64;
    const size_t smem = ((size_t)(dim + kc) * kWaS + (size_t)kWaK * (16 * VC + 4) + (kc < dim ? 0 : (size_t)kWaK * kWaS)) * sizeof(float);
    static size_t set = 0;
    if (smem > 48 * 1024 && smem > set) {
        cudaError_t e = cudaFuncSetAttribute(window_attention_kernel<T, VC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = smem;
    }
    const dim3 grid((b.max_seq_len + kWaQ - 1) / kWaQ, heads, b.n_seqs);
    window_attention_kernel<T, VC><<<grid, 256, smem, st>>>((const T*)q, ldq, (const T*)k, ldk, (const T*)v, ldv, b, dim, vdim,
                                                            window, scale, (T*)out, ldo, x, kc);
    return 0;
}

}  // namespace umbs

using namespace umbs;

extern "C" int umbs_window_attention_fits(int dim, int vdim) { return dim >= 1 && dim <= 128 && vdim >= 1 && vdim <= 128; }
extern "C" int umbs_window_attention_ex_fits(int dim, int shared_dim, int vdim) {
    return dim >= 1 && shared_dim >= 0 && dim + shared_dim <= 192 && vdim >= 1 && vdim <= 128;
}

extern "C" int umbs_window_attention(int dtype, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                                     int64_t ldv, const umbs_batch_t* batch, int heads, int dim, int vdim, int window,
                                     float scale, void* out, int64_t ldo, umbs_stream_t stream) {
    if (window < 1) return UMB_ERR_ARG;
    if (!umbs_window_attention_fits(dim, vdim)) return UMB_ERR_UNSUPPORTED;
    return umbs_window_attention_ex(dtype, q, ldq, k, ldk, nullptr, 0, 0, v, ldv, batch, heads, dim, vdim, window, scale,
                                    UMBS_ATTN_SOFTMAX, nullptr, nullptr, 0, out, ldo, stream);
}

extern "C" int umbs_window_attention_ex(int dtype, const void* q, int64_t ldq, const void* k, int64_t ldk, const void* k_shared,
                                        int64_t ldks, int shared_dim, const void* v, int64_t ldv, const umbs_batch_t* batch,
                                        int heads, int dim, int vdim, int window, float scale, int mode, const float* sink,
                                        const float* gate, int64_t ldg, void* out, int64_t ldo, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (heads < 1 || (shared_dim > 0 && k_shared == nullptr)) return UMB_ERR_ARG;
    if (mode != UMBS_ATTN_SOFTMAX && mode != UMBS_ATTN_SOFTMAX_SINK) return UMB_ERR_UNSUPPORTED;
    if (!umbs_window_attention_ex_fits(dim, shared_dim, vdim)) return UMB_ERR_UNSUPPORTED;
    if (window <= 0) window = 1 << 30;                       // every earlier token of the step
    cudaStream_t st = (cudaStream_t)stream;
    const WindowExtra x{k_shared, ldks, dim, mode == UMBS_ATTN_SOFTMAX_SINK, sink, gate, ldg};
    const int dq = dim + shared_dim;
    int rc;
    if (dtype == UMBS_BF16) {
        rc = vdim <= 64 ? launch_window_attention<__nv_bfloat16, 4>(q, ldq, k, ldk, v, ldv, *batch, heads, dq, vdim, window, scale, out, ldo, x, st)
                        : launch_window_attention<__nv_bfloat16, 8>(q, ldq, k, ldk, v, ldv, *batch, heads, dq, vdim, window, scale, out, ldo, x, st);
    } else if (dtype == UMBS_F32) {
        rc = vdim <= 64 ? launch_window_attention<float, 4>(q, ldq, k, ldk, v, ldv, *batch, heads, dq, vdim, window, scale, out, ldo, x, st)
                        : launch_window_attention<float, 8>(q, ldq, k, ldk, v, ldv, *batch, heads, dq, vdim, window, scale, out, ldo, x, st);
    } else {
        return UMB_ERR_ARG;
    }
    if (rc) return rc;
    count_launches(1);
    return (int)cudaGetLastError();
}
