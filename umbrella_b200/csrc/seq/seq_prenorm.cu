// Kernels of the pre-norm layer form (see include/umbrella_b200_seq.h): residual add fused with the RMS norm that
// follows it, the logit soft cap, and what stands between an attention layer's in-projection and its attention kernel:
// bias, short causal convolution with its carried rows, rotary positions, the step's key/value rows in the cache's
// layout, and the mean key/value of every block of tokens a step completes.  fp32 arithmetic throughout.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <algorithm>
#include <stdint.h>

#include "seq_internal.h"

namespace umbs {

__device__ __forceinline__ float warp_sum_pn(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One block per row.  The row is read once into registers (up to 8 values per thread, more are re-read), its sum of
// squares reduced in a fixed tree (warp shuffles, then warp 0 over the per-warp partials): the result does not depend on
// what else is in the step.
template <typename T>
__global__ void add_rms_norm_kernel(float* __restrict__ x, const float* __restrict__ delta, const int32_t* __restrict__ rows,
                                    const float* __restrict__ w, float w_offset, int width, float eps, T* __restrict__ y,
                                    float* __restrict__ copy) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    float* xr = x + src * width;
    const float* dr = delta ? delta + src * width : nullptr;
    constexpr int KEEP = 8;
    float v[KEEP];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int e = threadIdx.x + i * blockDim.x;
        v[i] = 0.f;
        if (e < width) {
            v[i] = xr[e] + (dr ? dr[e] : 0.f);
            ss = fmaf(v[i], v[i], ss);
        }
    }
    for (int e = threadIdx.x + KEEP * blockDim.x; e < width; e += blockDim.x) {
        const float u = xr[e] + (dr ? dr[e] : 0.f);
        ss = fmaf(u, u, ss);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    ss = warp_sum_pn(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float s = lane < nw ? red[lane] : 0.f;
        s = warp_sum_pn(s);
        if (lane == 0) red[32] = s;
    }
    __syncthreads();
    const float inv = 1.f / sqrtf(red[32] / (float)width + eps);
    const bool write_x = rows == nullptr && dr != nullptr;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int e = threadIdx.x + i * blockDim.x;
        if (e < width) {
            if (write_x) xr[e] = v[i];
            if (copy != nullptr) copy[(int64_t)r * width + e] = v[i];
            if (y != nullptr) y[(int64_t)r * width + e] = from_f32<T>(v[i] * inv * (w_offset + w[e]));
        }
    }
    for (int e = threadIdx.x + KEEP * blockDim.x; e < width; e += blockDim.x) {
        const float u = xr[e] + (dr ? dr[e] : 0.f);
        if (write_x) xr[e] = u;
        if (copy != nullptr) copy[(int64_t)r * width + e] = u;
        if (y != nullptr) y[(int64_t)r * width + e] = from_f32<T>(u * inv * (w_offset + w[e]));
    }
}

// Residual add + norm for any pending block output (dense, routed experts' pairs, gated shared expert; layer scale and
// residual multiplier) and either norm.  One block per row, the row in registers (8 values per thread); sums in a fixed
// tree, so a row's result does not depend on what else is in the step.  The layer norm takes its mean first and the mean
// of the squared deviations second.
__device__ __forceinline__ float block_sum_pn(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum_pn(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float s = lane < nw ? red[lane] : 0.f;
        s = warp_sum_pn(s);
        if (lane == 0) red[32] = s;
    }
    __syncthreads();
    return red[32];
}

template <typename T>
__global__ void add_norm_kernel(float* __restrict__ x, umbs_delta_t d, int has_d, const int32_t* __restrict__ rows, int kind,
                                const float* __restrict__ w, const float* __restrict__ bias, float w_offset, float alpha, int width,
                                float eps, T* __restrict__ y, float* __restrict__ copy) {
    __shared__ float red[33];
    constexpr int KEEP = 8, TOPS = 16;              // up to TOPS routed pairs per token are held in shared memory
    __shared__ float s_w[TOPS];
    __shared__ const float* s_p[TOPS];
    const int r = blockIdx.x;
    const int64_t src = rows ? rows[r] : r;
    float* xr = x + src * width;
    float v[KEEP];
    const float sg = (has_d && d.shared != nullptr && d.shared_gate != nullptr) ? d.shared_gate[src] : 1.f;
    const bool routed = has_d && d.pair_out != nullptr;
    const int top_s = routed ? min(d.top, TOPS) : 0;
    if (threadIdx.x < top_s) {                      // the token's weights and the rows of its experts' outputs, read once
        s_w[threadIdx.x] = d.sel_w[src * d.top + threadIdx.x];
        s_p[threadIdx.x] = d.pair_out + (int64_t)d.pair_pos[src * d.top + threadIdx.x] * width;
    }
    if (routed) __syncthreads();
    // the routed experts' rows first, expert by expert: the thread's eight loads of a row are in flight together
    float ff[KEEP];
#pragma unroll
    for (int i = 0; i < KEEP; ++i) ff[i] = 0.f;
    for (int k = 0; routed && k < d.top; ++k) {
        const float wk = k < top_s ? s_w[k] : d.sel_w[src * d.top + k];
        const float* pk = k < top_s ? s_p[k] : d.pair_out + (int64_t)d.pair_pos[src * d.top + k] * width;
#pragma unroll
        for (int i = 0; i < KEEP; ++i) {
            const int e = threadIdx.x + i * blockDim.x;
            if (e < width) ff[i] = fmaf(wk, pk[e], ff[i]);
        }
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int e = threadIdx.x + i * blockDim.x;
        v[i] = 0.f;
        if (e < width) {
            float dl = 0.f;
            if (has_d) {
                if (d.delta != nullptr) dl = d.delta[src * width + e] * d.delta_mult;
                if (d.delta2 != nullptr) dl = fmaf(d.delta2[src * width + e], d.delta2_mult, dl);
                dl += ff[i];
                if (d.shared != nullptr) dl = fmaf(d.shared[src * width + e], sg, dl);
                if (d.scale != nullptr) dl *= d.scale[e];
                dl *= d.mult;
            }
            v[i] = xr[e] + dl;
            sum += kind == UMBS_NORM_LAYER ? v[i] : v[i] * v[i];
        }
    }
    float mean = 0.f, inv = 0.f;
    if (y != nullptr && kind != UMBS_NORM_DYT) {          // (the tanh norm takes no statistics)
        sum = block_sum_pn(sum, red);
        if (kind == UMBS_NORM_LAYER) {
            mean = sum / (float)width;
            float dev = 0.f;
#pragma unroll
            for (int i = 0; i < KEEP; ++i)
                if (threadIdx.x + i * blockDim.x < width) dev = fmaf(v[i] - mean, v[i] - mean, dev);
            sum = block_sum_pn(dev, red);
        }
        inv = 1.f / sqrtf(sum / (float)width + eps);
    }
    const bool write_x = rows == nullptr && has_d;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int e = threadIdx.x + i * blockDim.x;
        if (e < width) {
            if (write_x) xr[e] = v[i];
            if (copy != nullptr) copy[(int64_t)r * width + e] = v[i];
            if (y != nullptr) {
                float o = kind == UMBS_NORM_DYT ? tanhf(alpha * v[i]) * (w_offset + w[e]) : (v[i] - mean) * inv * (w_offset + w[e]);
                if (kind != UMBS_NORM_RMS && bias != nullptr) o += bias[e];
                y[(int64_t)r * width + e] = from_f32<T>(o);
            }
        }
    }
}

// One block per token of a latent-attention layer with direct queries: RMS norm of the latent, the turn of the shared key
// part and of every head's rope part by the token's position.
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ proj, int64_t ld, Batch b, int heads, int dim, int rope, int R,
                                   const float* __restrict__ kv_norm, float eps, int rot_dims, const float* __restrict__ inv_freq,
                                   float rot_mag, T* __restrict__ q, T* __restrict__ c, float* __restrict__ q_rot, int64_t ld_qrot) {
    extern __shared__ float cs[];                 // cos | sin [rot_dims]
    __shared__ float red[33];
    const int t = blockIdx.x, pos = b.tok_pos[t], half = rot_dims / 2, hd = dim + rope;
    const float* row = proj + (int64_t)t * ld;
    const float* low = row + (int64_t)heads * hd;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        cs[i] = cosf(ang) * rot_mag;
        cs[half + i] = sinf(ang) * rot_mag;
    }
    float ss = 0.f;
    for (int e = threadIdx.x; e < R; e += blockDim.x) ss = fmaf(low[e], low[e], ss);
    ss = block_sum_pn(ss, red);                    // (its barriers also publish cs)
    const float inv = 1.f / sqrtf(ss / (float)R + eps);
    // the turn of component j of a rope part that starts at p
    auto turned = [&](const float* p, int j) -> float {
        if (j < half) return p[j] * cs[j] - p[j + half] * cs[half + j];
        if (j < rot_dims) return p[j] * cs[j - half] + p[j - half] * cs[j];     // cs[j] = sin of pair j - half
        return p[j];
    };
    T* crow = c + (int64_t)t * (R + rope);
    for (int e = threadIdx.x; e < R; e += blockDim.x) crow[e] = from_f32<T>(low[e] * inv * kv_norm[e]);
    for (int j = threadIdx.x; j < rope; j += blockDim.x) crow[R + j] = from_f32<T>(turned(low + R, j));
    T* qrow = q + (int64_t)t * heads * hd;
    for (int i = threadIdx.x; i < heads * hd; i += blockDim.x) {
        const int h = i / hd, e = i - h * hd;
        float o = row[i];
        if (e >= dim) {
            o = turned(row + (int64_t)h * hd + dim, e - dim);
            if (q_rot != nullptr) q_rot[((int64_t)t * heads + h) * ld_qrot + (e - dim)] = o;
        }
        qrow[i] = from_f32<T>(o);
    }
}

__global__ void softcap_kernel(float* __restrict__ z, int64_t n, float cap) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) z[i] = cap * tanhf(z[i] / cap);
}

// One block per token.  Channels of q | k go through bias and convolution into shared memory, are turned there, and leave
// as q and as the key part of the token's kv row; values follow (own projection, or the keys before the turn).
template <typename T>
__global__ void attention_prep_kernel(const float* __restrict__ proj, int64_t ld, const float* __restrict__ bias, Batch b,
                                      int heads, int kv_heads, int dim, int vdim, int values_are_keys, int taps,
                                      const float* __restrict__ conv_w, float* __restrict__ conv_state, int slots, int rot_dims,
                                      const float* __restrict__ inv_freq, float rot_mag, int maps,
                                      const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
                                      T* __restrict__ q_out, T* __restrict__ kv_out) {
    extern __shared__ float sm[];                 // [heads dim + kv_heads dim] convolved q | k, then cos | sin [rot_dims]
    const int Cq = heads * maps * dim, Ck = kv_heads * maps * dim, C = Cq + Ck, Cv = kv_heads * vdim;
    float* y = sm;
    float* cs = sm + C;
    const int t = blockIdx.x, s = b.tok_seq[t], pos = b.tok_pos[t];
    const int start = b.seq_start[s], len = b.seq_len[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s], par = b.seq_parity[s];
    const int keep = taps - 1;
    const float* st_in = conv_state ? conv_state + ((int64_t)par * slots + slot) * keep * C : nullptr;
    const float* row = proj + (int64_t)t * ld;
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        cs[i] = cosf(ang) * rot_mag;
        cs[half + i] = sinf(ang) * rot_mag;
    }
    // u(c, p): the projected value (bias added) of channel c at position p -- this step's row, the carried rows, or zero
    auto u_at = [&](int c, int p) -> float {
        if (p >= pos0) return proj[(int64_t)(start + p - pos0) * ld + c] + (bias ? bias[c] : 0.f);
        if (p < 0 || st_in == nullptr) return 0.f;
        return st_in[(int64_t)(p - (pos0 - keep)) * C + c];       // carried row r holds position pos0 - keep + r
    };
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc;
        if (taps <= 1) {
            acc = row[c] + (bias ? bias[c] : 0.f);
        } else {
            acc = 0.f;
            for (int j = 0; j < taps; ++j) acc = fmaf(conv_w[(int64_t)c * taps + j], u_at(c, pos - keep + j), acc);
        }
        y[c] = acc;
    }
    // the sequence's last token of the step leaves the rows the next step's convolution starts from (other buffer half)
    if (keep > 0 && conv_state != nullptr && t == start + len - 1) {
        float* st_out = conv_state + ((int64_t)(par ^ 1) * slots + slot) * keep * C;
        const int end = pos0 + len;                              // carried row r will hold position end - keep + r
        for (int i = threadIdx.x; i < keep * C; i += blockDim.x) {
            const int r = i / C, c = i - r * C;
            st_out[i] = u_at(c, end - keep + r);
        }
    }
    __syncthreads();
    if (q_norm_w != nullptr || k_norm_w != nullptr) {
        // RMS norm of every (head, map): a warp per group of dim channels, lanes striding over it
        const int lane = threadIdx.x & 31, nw = blockDim.x >> 5;
        for (int grp = threadIdx.x >> 5; grp < C / dim; grp += nw) {
            const float* nwt = grp * dim < Cq ? q_norm_w : k_norm_w;
            if (nwt == nullptr) continue;
            float* yg = y + grp * dim;
            float ss = 0.f;
            for (int d = lane; d < dim; d += 32) ss = fmaf(yg[d], yg[d], ss);
            ss = warp_sum_pn(ss);
            const float inv = 1.f / sqrtf(ss / (float)dim + eps);
            for (int d = lane; d < dim; d += 32) yg[d] = yg[d] * inv * nwt[d];
        }
        __syncthreads();
    }
    const int row_kv = Ck + Cv;
    T* qo = q_out + (int64_t)t * Cq;
    T* ko = kv_out + (int64_t)t * row_kv;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const int d = c % dim;                                   // Cq is a multiple of dim: the same for q and k channels
        float v = y[c];
        if (d < rot_dims) {
            const int f = d < half ? d : d - half;
            const float other = y[d < half ? c + half : c - half];
            v = d < half ? v * cs[f] - other * cs[half + f] : v * cs[f] + other * cs[half + f];
        }
        if (c < Cq) qo[c] = from_f32<T>(v);
        else {
            ko[c - Cq] = from_f32<T>(v);
            if (values_are_keys) ko[Ck + (c - Cq)] = from_f32<T>(y[c]);
        }
    }
    if (!values_are_keys && kv_out != nullptr)
        for (int c = threadIdx.x; c < Cv; c += blockDim.x) ko[Ck + c] = from_f32<T>(row[C + c] + (bias ? bias[C + c] : 0.f));
}

// One block per (block of tokens completed by the step, sequence, 256 columns): the fp32 mean, in position order, of the
// block's kv rows as the cache holds them.  Eight rows are loaded ahead of the additions, which stay in position order.
template <typename T>
__global__ void kv_pool_kernel(const T* __restrict__ kv, const T* __restrict__ kv_cache, int kv_len, T* __restrict__ pool_cache,
                               int pool_len, Batch b, int row, int pool) {
    const int s = blockIdx.y, pos0 = b.seq_pos0[s], len = b.seq_len[s], start = b.seq_start[s], slot = b.seq_slot[s];
    const int blk = pos0 / pool + blockIdx.x;                    // first block whose last token is in the step, onwards
    if ((int64_t)(blk + 1) * pool > (int64_t)pos0 + len || blk >= pool_len) return;
    const int c = blockIdx.z * blockDim.x + threadIdx.x;
    if (c >= row) return;
    auto at = [&](int j) -> float {
        const T* src = j >= pos0 ? kv + (int64_t)(start + j - pos0) * row : kv_cache + ((int64_t)slot * kv_len + j % kv_len) * row;
        return to_f32(src[c]);
    };
    float acc = 0.f;
    const int j0 = blk * pool;
    int j = 0;
    for (; j + 8 <= pool; j += 8) {
        float x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) x[u] = at(j0 + j + u);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc += x[u];
    }
    for (; j < pool; ++j) acc += at(j0 + j);
    pool_cache[((int64_t)slot * pool_len + blk) * row + c] = from_f32<T>(acc / (float)pool);
}

}  // namespace umbs

using namespace umbs;

#define UMBS_DISPATCH_T(dtype, ...)                              \
    do {                                                         \
        if ((dtype) == UMBS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else if ((dtype) == UMBS_F32) { using T = float; __VA_ARGS__; }     \
        else return UMB_ERR_ARG;                                 \
    } while (0)

extern "C" int umbs_add_rms_norm(int dtype, float* x, const float* delta, const int32_t* rows, int n, const float* w,
                                 float w_offset, int width, float eps, void* y, float* copy, umbs_stream_t stream) {
    if (n <= 0) return 0;
    if (x == nullptr || width <= 0 || (y != nullptr && w == nullptr)) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = width >= 2048 ? 256 : (width >= 512 ? 128 : 64);
    UMBS_DISPATCH_T(dtype, add_rms_norm_kernel<T><<<n, threads, 0, st>>>(x, delta, rows, w, w_offset, width, eps, (T*)y, copy));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_add_norm(int dtype, float* x, const umbs_delta_t* d, const int32_t* rows, int n, int kind, const float* w,
                             const float* b, float w_offset, int width, float eps, void* y, float* copy, umbs_stream_t stream) {
    return umbs_add_norm_ex(dtype, x, d, rows, n, kind, w, b, w_offset, 1.f, width, eps, y, copy, stream);
}

extern "C" int umbs_add_norm_ex(int dtype, float* x, const umbs_delta_t* d, const int32_t* rows, int n, int kind, const float* w,
                                const float* b, float w_offset, float alpha, int width, float eps, void* y, float* copy,
                                umbs_stream_t stream) {
    if (n <= 0) return 0;
    if (x == nullptr || width <= 0 || (y != nullptr && w == nullptr)) return UMB_ERR_ARG;
    if (kind != UMBS_NORM_RMS && kind != UMBS_NORM_LAYER && kind != UMBS_NORM_DYT) return UMB_ERR_ARG;
    if (width > 8192) return UMB_ERR_UNSUPPORTED;                 // a row lives in the block's registers
    if (d != nullptr && d->pair_out != nullptr && (d->sel_w == nullptr || d->pair_pos == nullptr || d->top < 1)) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    int threads = ((width + 7) / 8 + 31) / 32 * 32;
    if (threads < 64) threads = 64;
    umbs_delta_t dd{};
    if (d != nullptr) dd = *d;
    if (dd.delta_mult == 0.f && dd.delta2 == nullptr) dd.delta_mult = 1.f;
    UMBS_DISPATCH_T(dtype, add_norm_kernel<T><<<n, threads, 0, st>>>(x, dd, d != nullptr, rows, kind, w, b, w_offset, alpha, width,
                                                                     eps, (T*)y, copy));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_latent_prep(int dtype, const float* proj, int64_t ld, const umbs_batch_t* batch, int heads, int dim,
                                int rope_dim, int kv_rank, const float* kv_norm, float eps, int rot_dims, const float* inv_freq,
                                float rot_mag, void* q, void* c, float* q_rot, int64_t ld_qrot, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (heads < 1 || dim < 0 || rope_dim < 0 || kv_rank < 1 || rot_dims < 0 || rot_dims > rope_dim || (rot_dims & 1)) return UMB_ERR_ARG;
    if (rot_dims > 0 && inv_freq == nullptr) return UMB_ERR_ARG;
    if (proj == nullptr || kv_norm == nullptr || q == nullptr || c == nullptr) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int work = heads * (dim + rope_dim);
    const int threads = work >= 4096 ? 512 : (work >= 1024 ? 256 : 128);
    UMBS_DISPATCH_T(dtype, latent_prep_kernel<T><<<batch->n_tokens, threads, (size_t)(rot_dims + 2) * sizeof(float), st>>>(
                               proj, ld, *batch, heads, dim, rope_dim, kv_rank, kv_norm, eps, rot_dims, inv_freq, rot_mag, (T*)q,
                               (T*)c, q_rot, ld_qrot));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_softcap(float* z, int64_t n, float cap, umbs_stream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return UMB_ERR_ARG;
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(z, n, cap);
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_attention_prep(int dtype, const float* proj, int64_t ld, const float* bias, const umbs_batch_t* batch,
                                   int heads, int kv_heads, int dim, int vdim, int values_are_keys, int taps,
                                   const float* conv_w, float* conv_state, int slots, int rot_dims, const float* inv_freq,
                                   float rot_mag, void* q, void* kv, umbs_stream_t stream) {
    if (kv_heads < 1) return UMB_ERR_ARG;
    return umbs_attention_prep_ex(dtype, proj, ld, bias, batch, heads, kv_heads, dim, vdim, values_are_keys, taps, conv_w, conv_state,
                                  slots, rot_dims, inv_freq, rot_mag, 1, nullptr, nullptr, 0.f, q, kv, stream);
}

extern "C" int umbs_attention_prep_ex(int dtype, const float* proj, int64_t ld, const float* bias, const umbs_batch_t* batch,
                                      int heads, int kv_heads, int dim, int vdim, int values_are_keys, int taps,
                                      const float* conv_w, float* conv_state, int slots, int rot_dims, const float* inv_freq,
                                      float rot_mag, int maps, const float* q_norm_w, const float* k_norm_w, float eps, void* q,
                                      void* kv, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (maps < 1) maps = 1;
    if (rot_dims < 0 || rot_dims > dim || (rot_dims & 1) || taps < 1 || kv_heads < 0 || heads < 1) return UMB_ERR_ARG;
    if (kv_heads > 0 ? (heads % kv_heads != 0 || kv == nullptr) : values_are_keys) return UMB_ERR_ARG;
    if (values_are_keys && vdim != dim) return UMB_ERR_ARG;
    if (taps > 1 && (conv_w == nullptr || conv_state == nullptr)) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int C = (heads + kv_heads) * maps * dim;
    const size_t smem = ((size_t)C + rot_dims + 2) * sizeof(float);
    if (smem > 48 * 1024) return UMB_ERR_UNSUPPORTED;
    // a small step (decoding) has few blocks: spread a token's channels over up to 1024 threads
    const int threads = batch->n_tokens <= 64 ? std::min(1024, (C + 31) / 32 * 32) : (C >= 1024 ? 256 : 128);
    UMBS_DISPATCH_T(dtype, attention_prep_kernel<T><<<batch->n_tokens, threads, smem, st>>>(
                               proj, ld, bias, *batch, heads, kv_heads, dim, vdim, values_are_keys, taps, conv_w, conv_state, slots,
                               rot_dims, inv_freq, rot_mag, maps, q_norm_w, k_norm_w, eps, (T*)q, (T*)kv));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_kv_pool(int dtype, const void* kv, const void* kv_cache, int kv_len, void* pool_cache, int pool_len,
                            const umbs_batch_t* batch, int row, int pool, umbs_stream_t stream) {
    if (batch->n_tokens <= 0 || pool <= 0) return 0;
    if (kv_len < pool) return UMB_ERR_ARG;               // a block's older tokens must still sit in the cache
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(batch->max_seq_len / pool + 1, batch->n_seqs, (row + 255) / 256);
    UMBS_DISPATCH_T(dtype, kv_pool_kernel<T><<<grid, 256, 0, st>>>((const T*)kv, (const T*)kv_cache, kv_len, (T*)pool_cache,
                                                                   pool_len, *batch, row, pool));
    count_launches(1);
    return (int)cudaGetLastError();
}
