// The time-mix mixer: a matrix memory per head whose decay is a vector per token (one factor per key channel), computed
// from the token itself, with a bonus for the current token in its own read-out; and the token-shifted mixes that feed its
// projections.  fp32 arithmetic throughout; the state is fp32 [slots, heads, dim, dim], key index first.
//
//   umbs_shift_mix : out[t, s, :] = h[t] + (h[t - 1] - h[t]) mu[s, :] for n_mix mixes; the row before a step's first
//                    token comes from the slot's double-buffered shift state, the step's last row goes there.
//   umbs_time_mix  : the recurrence, one block per (sequence, head, 32 value columns) whose warps each keep 16 key rows of
//                    those columns in registers for the whole step; r, k, v and the decay of 16 tokens at a time are staged in
//                    a ring of shared-memory stages by asynchronous copies (the decay's two exponentials are taken there, once
//                    per token and channel).  Tokens run
//                    in order, so a prompt in one piece, in portions or token by token performs the same additions.  A
//                    second kernel takes unit RMS per head, the weight and the silu gate.
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

constexpr int kTmTok = 16;           // tokens per group staged in shared memory
constexpr int kTmRows = 16;          // key rows of the state a warp keeps (per lane: one value column of them)
constexpr int kTmStages = 4;         // groups in flight: asynchronous copies run three groups ahead of the walk

__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// One block = (32 value columns, head, sequence); warp w keeps key rows [16 w, 16 w + 16) of those columns in registers for
// the whole step.  Tokens are staged 16 at a time in a ring of four shared-memory stages filled by asynchronous copies
// (r, k, the decay's argument and the block's 32 value columns), so that global latency is hidden although a scheduler
// holds a single warp; the decay's two exponentials are taken in place when a stage has landed, once per token and
// channel.  Every warp walks the tokens in order over its rows -- read-out with the bonus first, then decay and the token's
// own outer product -- and leaves its partial read-outs in shared memory, where they are added up warp by warp.  The
// order of every addition is fixed by the layout alone, so a token's result does not depend on how the sequence was cut
// into steps.
__global__ void __launch_bounds__(256) time_mix_kernel(const float* __restrict__ proj, int64_t ld, const float* __restrict__ decay_raw,
                                                       const float* __restrict__ decay_bias, const float* __restrict__ bonus, Batch b,
                                                       int heads, int dim, float* __restrict__ state, float* __restrict__ o) {
    extern __shared__ __align__(16) float tm_sm[];
    const int nw = blockDim.x >> 5, Dp = nw * kTmRows;              // Dp >= dim: the staged rows, zero beyond dim
    const int plane = kTmTok * Dp, stage_floats = 3 * plane + kTmTok * 32;
    float* su = tm_sm + kTmStages * stage_floats;                   // [Dp]
    float* part = su + Dp;                                          // [kTmTok][nw][32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = blockIdx.x * 32 + lane, h = blockIdx.y, s = blockIdx.z, k0 = warp * kTmRows;
    const int start = b.seq_start[s], len = b.seq_len[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    const int hd = heads * dim;
    const bool col = j < dim;
    constexpr int kPerThread = kTmTok * kTmRows / 32;               // (token, row) pairs a thread stages per group
    float S[kTmRows];
    float* st = state + (((int64_t)slot * heads + h) * dim) * dim;          // S[k][j] at st[k dim + j]
#pragma unroll
    for (int i = 0; i < kTmRows; ++i) S[i] = (pos0 > 0 && col && k0 + i < dim) ? st[(int64_t)(k0 + i) * dim + j] : 0.f;
    for (int k = tid; k < Dp; k += blockDim.x) su[k] = k < dim ? bonus[h * dim + k] : 0.f;
    const int groups = (len + kTmTok - 1) / kTmTok;
    // start the copies of group g into its stage (places without a token or beyond dim are zeroed by plain stores)
    auto issue = [&](int g) {
        float* sr = tm_sm + (g % kTmStages) * stage_floats;
        float* sk = sr + plane;
        float* sw = sk + plane;
        float* sv = sw + plane;
        const int t0 = g * kTmTok, nt = min(kTmTok, len - t0);
#pragma unroll
        for (int e = 0; e < kPerThread; ++e) {
            const int i = tid + e * blockDim.x, tt = i / Dp, k = i - tt * Dp;
            if (tt < nt && k < dim) {
                const int64_t t = start + t0 + tt;
                cp_async_f32(sr + i, proj + t * ld + h * dim + k);
                cp_async_f32(sk + i, proj + t * ld + hd + h * dim + k);
                cp_async_f32(sw + i, decay_raw + t * hd + h * dim + k);
            } else {
                sr[i] = 0.f; sk[i] = 0.f; sw[i] = 0.f;
            }
        }
        for (int i = tid; i < kTmTok * 32; i += blockDim.x) {
            const int tt = i >> 5, jj = blockIdx.x * 32 + (i & 31);
            if (tt < nt && jj < dim) cp_async_f32(sv + i, proj + (int64_t)(start + t0 + tt) * ld + 2 * hd + h * dim + jj);
            else sv[i] = 0.f;
        }
    };
    for (int g = 0; g < kTmStages - 1; ++g) {
        if (g < groups) issue(g);
        cp_async_commit();
    }
    for (int g = 0; g < groups; ++g) {
        // (the stage this writes was walked in the previous iteration, which ended with a barrier)
        if (g + kTmStages - 1 < groups) issue(g + kTmStages - 1);
        cp_async_commit();
        cp_async_wait<kTmStages - 1>();                             // this thread's copies of group g have landed
        float* sr = tm_sm + (g % kTmStages) * stage_floats;
        float* sk = sr + plane;
        float* sw = sk + plane;
        float* sv = sw + plane;
        const int t0 = g * kTmTok, nt = min(kTmTok, len - t0);
#pragma unroll
        for (int e = 0; e < kPerThread; ++e) {                      // the decay of the places this thread copied
            const int i = tid + e * blockDim.x, tt = i / Dp, k = i - tt * Dp;
            if (tt < nt && k < dim) sw[i] = expf(-expf(sw[i] + decay_bias[h * dim + k]));
        }
        __syncthreads();
#pragma unroll
        for (int tt = 0; tt < kTmTok; ++tt) {
            if (tt >= nt) break;
            const float* rr = sr + tt * Dp + k0;
            const float* kr = sk + tt * Dp + k0;
            const float* wr = sw + tt * Dp + k0;
            const float v = sv[tt * 32 + lane];
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i4 = 0; i4 < kTmRows; i4 += 4) {
                const float4 r4 = *reinterpret_cast<const float4*>(rr + i4);
                const float4 k4 = *reinterpret_cast<const float4*>(kr + i4);
                const float4 w4 = *reinterpret_cast<const float4*>(wr + i4);
                const float4 u4 = *reinterpret_cast<const float4*>(su + k0 + i4);
                const float ra[4] = {r4.x, r4.y, r4.z, r4.w}, ka[4] = {k4.x, k4.y, k4.z, k4.w};
                const float wa[4] = {w4.x, w4.y, w4.z, w4.w}, ua[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float kv = ka[x] * v;
                    acc[x] = fmaf(ra[x], fmaf(ua[x], kv, S[i4 + x]), acc[x]);
                    S[i4 + x] = fmaf(wa[x], S[i4 + x], kv);
                }
            }
            part[(tt * nw + warp) * 32 + lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
        __syncthreads();
        for (int i = tid; i < nt * 32; i += blockDim.x) {
            const int tt = i >> 5, ln = i & 31, jj = blockIdx.x * 32 + ln;
            if (jj >= dim) continue;
            float sum = 0.f;
            for (int w = 0; w < nw; ++w) sum += part[(tt * nw + w) * 32 + ln];
            o[(int64_t)(start + t0 + tt) * hd + h * dim + jj] = sum;
        }
    }
    if (col) {
#pragma unroll
        for (int i = 0; i < kTmRows; ++i)
            if (k0 + i < dim) st[(int64_t)(k0 + i) * dim + j] = S[i];
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
    const int nw = (dim + kTmRows - 1) / kTmRows, Dp = nw * kTmRows;
    const size_t smem = ((size_t)kTmStages * (3 * kTmTok * Dp + kTmTok * 32) + Dp + (size_t)kTmTok * nw * 32) * sizeof(float);
    static bool big_smem = false;                           // up to 123 KB for heads of 128: above the default limit
    if (!big_smem) {
        cudaError_t e = cudaFuncSetAttribute(time_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
        if (e != cudaSuccess) return (int)e;
        big_smem = true;
    }
    time_mix_kernel<<<grid, 32 * nw, smem, st>>>(proj, ld, decay_raw, decay_bias, bonus, *batch, heads, dim, state, o_scratch);
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
