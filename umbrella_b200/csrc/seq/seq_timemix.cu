// The time-mix mixer: a matrix memory per head whose decay is a vector per token (one factor per key channel), computed
// from the token itself, with a bonus for the current token in its own read-out; and the token-shifted mixes that feed its
// projections.  fp32 arithmetic throughout; the state is fp32 [slots, heads, dim, dim], key index first.
//
//   umbs_shift_mix : out[t, s, :] = h[t] + (h[t - 1] - h[t]) mu[s, :] for n_mix mixes; the row before a step's first
//                    token comes from the slot's double-buffered shift state, the step's last row goes there.
//   umbs_time_mix  : the recurrence, one warp per (sequence, head, 32 value columns): a lane owns a value column and keeps
//                    that column of the state -- dim numbers -- in registers for the whole step; r, k and the decay of the
//                    next 8 tokens are staged in shared memory (the decay's two exponentials are taken there, once per
//                    token and channel).  Tokens run in order, so a prompt in one piece, in portions or token by token
//                    performs the same additions.  A second kernel takes unit RMS per head, the weight and the silu gate.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "seq_internal.h"

namespace umbs {

template <typename T>
__global__ void shift_mix_kernel(const T* __restrict__ h, const float* __restrict__ mu, int n_mix, float* __restrict__ state,
                                 int slots, Batch b, int width, T* __restrict__ out) {
    const int t = blockIdx.x, s = b.tok_seq[t], pos = b.tok_pos[t];
    const int start = b.seq_start[s], len = b.seq_len[s], slot = b.seq_slot[s], par = b.seq_parity[s];
    const T* hr = h + (int64_t)t * width;
    const bool first = t == start;
    const float* prev_state = state + ((int64_t)par * slots + slot) * width;
    float* next_state = (t == start + len - 1) ? state + ((int64_t)(par ^ 1) * slots + slot) * width : nullptr;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float cur = to_f32(hr[e]);
        const float prev = pos == 0 ? 0.f : (first ? prev_state[e] : to_f32(hr[e - width]));
        for (int m = 0; m < n_mix; ++m)
            out[((int64_t)t * n_mix + m) * width + e] = from_f32<T>(fmaf(prev - cur, mu[(int64_t)m * width + e], cur));
        if (next_state != nullptr) next_state[e] = cur;
    }
}

constexpr int kTmTok = 8;            // tokens staged at a time

// D: the head size rounded up to a multiple of 32 (registers per lane); dim: the real one
template <int D>
__global__ void __launch_bounds__(32) time_mix_kernel(const float* __restrict__ proj, int64_t ld, const float* __restrict__ decay_raw,
                                                      const float* __restrict__ decay_bias, const float* __restrict__ bonus, Batch b,
                                                      int heads, int dim, float* __restrict__ state, float* __restrict__ o) {
    __shared__ __align__(16) float sr[kTmTok][D], sk[kTmTok][D], sw[kTmTok][D], su[D];
    const int lane = threadIdx.x, j = blockIdx.x * 32 + lane, h = blockIdx.y, s = blockIdx.z;
    const int start = b.seq_start[s], len = b.seq_len[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    const int hd = heads * dim;
    const bool col = j < dim;
    float S[D];
    float* st = state + (((int64_t)slot * heads + h) * dim) * dim;          // S[k][j] at st[k dim + j]
#pragma unroll
    for (int k = 0; k < D; ++k) S[k] = (pos0 > 0 && col && k < dim) ? st[(int64_t)k * dim + j] : 0.f;
    for (int k = lane; k < D; k += 32) su[k] = k < dim ? bonus[h * dim + k] : 0.f;
    for (int t0 = 0; t0 < len; t0 += kTmTok) {
        const int nt = min(kTmTok, len - t0);
        __syncwarp();
        for (int i = lane; i < nt * D; i += 32) {
            const int tt = i / D, k = i - tt * D;
            const int64_t t = start + t0 + tt;
            float r = 0.f, kk = 0.f, w = 0.f;
            if (k < dim) {
                r = proj[t * ld + h * dim + k];
                kk = proj[t * ld + hd + h * dim + k];
                w = expf(-expf(decay_raw[t * hd + h * dim + k] + decay_bias[h * dim + k]));
            }
            sr[tt][k] = r; sk[tt][k] = kk; sw[tt][k] = w;
        }
        __syncwarp();
        for (int tt = 0; tt < nt; ++tt) {
            const int64_t t = start + t0 + tt;
            const float v = col ? proj[t * ld + 2 * hd + h * dim + j] : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int k4 = 0; k4 < D; k4 += 4) {
                const float4 r4 = *reinterpret_cast<const float4*>(&sr[tt][k4]);
                const float4 k4v = *reinterpret_cast<const float4*>(&sk[tt][k4]);
                const float4 w4 = *reinterpret_cast<const float4*>(&sw[tt][k4]);
                const float4 u4 = *reinterpret_cast<const float4*>(&su[k4]);
                const float ra[4] = {r4.x, r4.y, r4.z, r4.w}, ka[4] = {k4v.x, k4v.y, k4v.z, k4v.w};
                const float wa[4] = {w4.x, w4.y, w4.z, w4.w}, ua[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float kv = ka[x] * v;
                    acc = fmaf(ra[x], fmaf(ua[x], kv, S[k4 + x]), acc);
                    S[k4 + x] = fmaf(wa[x], S[k4 + x], kv);
                }
            }
            if (col) o[t * hd + h * dim + j] = acc;
        }
    }
    if (col) {
#pragma unroll
        for (int k = 0; k < D; ++k)
            if (k < dim) st[(int64_t)k * dim + j] = S[k];
    }
}

// One warp per (token, head): o / sqrt(mean(o^2) + eps) * weight * silu(gate).
template <typename T>
__global__ void time_mix_finish_kernel(const float* __restrict__ o, const float* __restrict__ proj, int64_t ld, int n_pairs,
                                       int heads, int dim, float eps, const float* __restrict__ w, T* __restrict__ out) {
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const int t = pair / heads, h = pair - t * heads, hd = heads * dim;
    const float* orow = o + (int64_t)t * hd + h * dim;
    const float* grow = proj + (int64_t)t * ld + 3 * hd + h * dim;
    float ss = 0.f;
    for (int c = lane; c < dim; c += 32) ss = fmaf(orow[c], orow[c], ss);
#pragma unroll
    for (int x = 16; x > 0; x >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, x);
    const float inv = 1.f / sqrtf(ss / (float)dim + eps);
    for (int c = lane; c < dim; c += 32) {
        const float g = grow[c];
        out[(int64_t)t * hd + h * dim + c] = from_f32<T>(orow[c] * inv * w[h * dim + c] * (g / (1.f + expf(-g))));
    }
}

}  // namespace umbs

using namespace umbs;

extern "C" int umbs_shift_mix(int dtype, const void* h, const float* mu, int n_mix, float* shift_state, int slots,
                              const umbs_batch_t* batch, int width, void* out, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (h == nullptr || mu == nullptr || shift_state == nullptr || out == nullptr || n_mix < 1 || width < 1) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
    if (dtype == UMBS_BF16)
        shift_mix_kernel<__nv_bfloat16><<<batch->n_tokens, threads, 0, st>>>((const __nv_bfloat16*)h, mu, n_mix, shift_state, slots, *batch,
                                                                          width, (__nv_bfloat16*)out);
    else if (dtype == UMBS_F32)
        shift_mix_kernel<float><<<batch->n_tokens, threads, 0, st>>>((const float*)h, mu, n_mix, shift_state, slots, *batch, width,
                                                                  (float*)out);
    else return UMB_ERR_ARG;
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_time_mix(int dtype, const float* proj, int64_t ld, const float* decay_raw, const float* decay_bias,
                             const float* bonus, const umbs_batch_t* batch, int heads, int dim, float eps,
                             const float* out_norm_w, float* state, float* o_scratch, void* out, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (proj == nullptr || decay_raw == nullptr || decay_bias == nullptr || bonus == nullptr || out_norm_w == nullptr ||
        state == nullptr || o_scratch == nullptr || out == nullptr || heads < 1 || dim < 1)
        return UMB_ERR_ARG;
    if (dim > 128) return UMB_ERR_UNSUPPORTED;              // a lane keeps a column of the state in registers
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid((dim + 31) / 32, heads, batch->n_seqs);
    if (dim <= 32) time_mix_kernel<32><<<grid, 32, 0, st>>>(proj, ld, decay_raw, decay_bias, bonus, *batch, heads, dim, state, o_scratch);
    else if (dim <= 64) time_mix_kernel<64><<<grid, 32, 0, st>>>(proj, ld, decay_raw, decay_bias, bonus, *batch, heads, dim, state, o_scratch);
    else if (dim <= 96) time_mix_kernel<96><<<grid, 32, 0, st>>>(proj, ld, decay_raw, decay_bias, bonus, *batch, heads, dim, state, o_scratch);
    else time_mix_kernel<128><<<grid, 32, 0, st>>>(proj, ld, decay_raw, decay_bias, bonus, *batch, heads, dim, state, o_scratch);
    const int pairs = batch->n_tokens * heads;
    if (dtype == UMBS_BF16)
        time_mix_finish_kernel<__nv_bfloat16><<<(pairs + 3) / 4, 128, 0, st>>>(o_scratch, proj, ld, pairs, heads, dim, eps, out_norm_w,
                                                                              (__nv_bfloat16*)out);
    else if (dtype == UMBS_F32)
        time_mix_finish_kernel<float><<<(pairs + 3) / 4, 128, 0, st>>>(o_scratch, proj, ld, pairs, heads, dim, eps, out_norm_w, (float*)out);
    else return UMB_ERR_ARG;
    count_launches(2);
    return (int)cudaGetLastError();
}
