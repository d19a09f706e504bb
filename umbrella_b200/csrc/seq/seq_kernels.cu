// Kernels of the sequence-state decoders (see include/umbrella_b200_seq.h): group norm + token shift, decayed linear
// attention with rotary positions, sliding-window latent attention over a ring of latents, top-k routing with an
// expert-sorted pair list, the depth-weighted residual mix.  Everything here is fp32 arithmetic on fp32 or bf16
// storage; the matrix products live in seq_gemm.cu.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <algorithm>
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
// (pos_freq != NULL: sinusoidal positions on top -- sine at the even entries, cosine at the odd ones, one frequency per pair)
template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table, float* __restrict__ y,
                                 int width, float scale, const int32_t* __restrict__ tok_pos, const float* __restrict__ pos_freq) {
    const int t = blockIdx.x;
    const T* row = table + (int64_t)ids[t] * width;
    const float pos = pos_freq != nullptr ? (float)tok_pos[t] : 0.f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        float v = to_f32(row[e]) * scale;
        if (pos_freq != nullptr && (e >> 1) < width / 2) {
            const float ang = pos * pos_freq[e >> 1];
            v += (e & 1) ? cosf(ang) : sinf(ang);
        }
        y[(int64_t)t * width + e] = v;
    }
}

// ------------------------------------------------------------------------------------------------ group norm (+ shift)
// Inverse root mean square of every group of row xr (and of row xp, if given), for all threads of the block.  Each
// group's sum of squares is split over blockDim / 32 / groups warps (at least one), all groups at once, so the row's loads
// are in flight together and the block synchronises twice whatever the number of groups.  The order of the additions
// depends on the block size only.  part: 2 groups max(1, warps / groups)
// floats of shared memory.
__device__ void group_inv_rms_all(const float* __restrict__ xr, const float* __restrict__ xp, int width, int groups, float eps,
                                  float* part, float* inv_own, float* inv_prev) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int gsz = width / groups, wpg = max(1, nw / groups), slots = groups * wpg;
    for (int slot = warp; slot < slots; slot += nw) {
        const int g = slot / wpg, pt = slot - g * wpg;
        float a = 0.f, b = 0.f;
        for (int e = pt * 32 + lane; e < gsz; e += wpg * 32) {
            const float v = xr[g * gsz + e];
            a = fmaf(v, v, a);
            if (xp != nullptr) {
                const float u = xp[g * gsz + e];
                b = fmaf(u, u, b);
            }
        }
        a = warp_sum(a);
        b = warp_sum(b);
        if (lane == 0) { part[slot] = a; part[slots + slot] = b; }
    }
    __syncthreads();
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        float a = 0.f, b = 0.f;
        for (int pt = 0; pt < wpg; ++pt) { a += part[g * wpg + pt]; b += part[slots + g * wpg + pt]; }
        inv_own[g] = 1.f / sqrtf(a / (float)gsz + eps);
        if (inv_prev != nullptr) inv_prev[g] = xp != nullptr ? 1.f / sqrtf(b / (float)gsz + eps) : 0.f;
    }
    __syncthreads();
}

template <typename T>
__global__ void group_norm_shift_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                        const float* __restrict__ shift_w, float* __restrict__ shift_state, int slots,
                                        Batch b, int width, int groups, float eps, T* __restrict__ h_out,
                                        T* __restrict__ hs_out) {
    extern __shared__ float sm[];     // [groups] own inverse rms, [groups] previous token's, partial sums
    float* inv_own = sm;
    float* inv_prev = sm + groups;
    float* part = sm + 2 * groups;
    const int t = blockIdx.x, s = b.tok_seq[t];
    const int start = b.seq_start[s], len = b.seq_len[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s], par = b.seq_parity[s];
    const int gsz = width / groups;
    const bool first = (t == start), last = (t == start + len - 1);
    const float* xr = x + (int64_t)t * width;
    const float* xp = xr - width;
    group_inv_rms_all(xr, (shift_w != nullptr && !first) ? xp : nullptr, width, groups, eps, part, inv_own, inv_prev);
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
    float* part = sm + groups;
    const int r = blockIdx.x;
    const float* xr = x + (int64_t)(rows ? rows[r] : r) * width;
    const int gsz = width / groups;
    group_inv_rms_all(xr, nullptr, width, groups, eps, part, inv, nullptr);
    for (int e = threadIdx.x; e < width; e += blockDim.x)
        y[(int64_t)r * width + e] = from_f32<T>(xr[e] * inv[e / gsz] * w[e]);
}

// ------------------------------------------------------------------------------------------------ retention
// cos / sin of every (token, frequency) pair of the step, once for all heads: tab[t] = cos[half] | sin[half]
__global__ void rotary_table_kernel(const int32_t* __restrict__ tok_pos, const float* __restrict__ inv_freq, int half,
                                    float* __restrict__ tab) {
    const int t = blockIdx.x;
    const float p = (float)tok_pos[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = p * inv_freq[i];
        tab[(int64_t)t * 2 * half + i] = cosf(ang);
        tab[(int64_t)t * 2 * half + half + i] = sinf(ang);
    }
}

// One block = (sequence, head, 32 value columns).  Lane = column; warp w keeps rows [w DPT, (w + 1) DPT) of the
// column's state in registers for the whole step.  Tokens go in order, TB at a time: the block rotates their q and k
// into shared memory, every warp advances its slice of the state through the TB tokens and leaves its part of each
// output in shared memory, and the parts are added in warp order.  TB = 16 (8 for the widest heads, whose staging
// registers would not fit): a round's serial walk then outlasts the latency of the next round's scattered loads.
template <int DPT, int kRetTB>
__global__ void retention_kernel(const float* __restrict__ qkvg, int64_t ld, Batch b, int heads, int dim, int vdim,
                                 int rot_dims, const float* __restrict__ rot_tab, const float* __restrict__ inv_freq,
                                 const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ o_out,
                                 int seg_len, int n_seg, int pass, float* __restrict__ seg_state) {
    extern __shared__ __align__(16) float sm[];
    const int DS = blockDim.y, dimP = DS * DPT, nthr = 32 * DS;
    float* qs = sm;                          // [TB][dimP]
    float* ks = qs + kRetTB * dimP;          // [TB][dimP]
    float* part = ks + kRetTB * dimP;        // [DS][TB][32]
    // A sequence may be cut into n_seg segments of seg_len tokens that run as blocks of their own (blockIdx.x =
    // sequence * n_seg + segment).  pass 0: no segments, the block walks the whole sequence.  pass 1: every segment but a
    // sequence's last starts from zero and leaves its end state in seg_state (no outputs).  Between the passes
    // retention_chain_kernel turns these into the segments' true start states.  pass 2: every segment starts from its
    // entry of seg_state; outputs are written, and the last segment stores the slot's state.
    const int s = blockIdx.x / n_seg, seg = blockIdx.x - s * n_seg;
    const int h = blockIdx.y, lane = threadIdx.x, w = threadIdx.y, tid = w * 32 + lane;
    const int j = blockIdx.z * 32 + lane, d0 = w * DPT;
    const int seq_len = b.seq_len[s], t_first = seg * seg_len;
    if (t_first >= seq_len) return;
    const int len = min(seg_len, seq_len - t_first), start = b.seq_start[s] + t_first;
    const bool last_seg = t_first + len == seq_len;
    if (pass == 1 && last_seg) return;
    const int pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    const bool col = j < vdim;
    const int64_t plane = (int64_t)heads * dim * vdim;
    const float dec = decay[h];
    const float kscale = 1.f / sqrtf((float)dim);
    const int half = rot_dims / 2;
    float* st = state + (((int64_t)slot * heads + h) * dim) * vdim;
    const float* st_in = st;
    bool have = pos0 > 0;
    if (pass == 1) have = false;
    else if (pass == 2 && !(seg == 0 && last_seg)) {
        // segment 0 of a cut sequence reads the chain kernel's copy of the slot's state (entry n_seg - 1), not the slot,
        // which the sequence's last segment overwrites during this very launch
        st_in = seg_state + ((int64_t)s * n_seg + (seg > 0 ? seg - 1 : n_seg - 1)) * plane + (int64_t)h * dim * vdim;
        have = true;
    }
    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) S[i] = (col && have && d0 + i < dim) ? st_in[(int64_t)(d0 + i) * vdim + j] : 0.f;
    const int qoff = h * dim, koff = heads * dim + h * dim, voff = 2 * heads * dim + h * vdim;
    // Each thread stages EPT (token, dim) elements of q and k and up to TB values of v per round; the loads of round
    // r + 1 are issued before round r is consumed, so their latency hides behind the serial walk through the tokens.
    constexpr int EPT = kRetTB * DPT / 32;
    float* vs = part + DS * kRetTB * 32;     // [TB][32]
    float pq[EPT], pq2[EPT], pk[EPT], pk2[EPT], pc[EPT], ps[EPT], pv[kRetTB];
    auto fetch = [&](int t0) {
        const int nb = min(kRetTB, len - t0);
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
            const int i = tid + e * nthr, tt = i / dimP, d = i - tt * dimP;
            pq[e] = pk[e] = pq2[e] = pk2[e] = ps[e] = 0.f;
            pc[e] = 1.f;
            if (tt < nb && d < dim) {
                const int64_t tok = start + t0 + tt;
                const float* row = qkvg + tok * ld;
                pq[e] = row[qoff + d];
                pk[e] = row[koff + d];
                if (d < rot_dims) {
                    const int partner = d < half ? d + half : d - half, f = d < half ? d : d - half;
                    pq2[e] = row[qoff + partner];
                    pk2[e] = row[koff + partner];
                    float cv, sv;
                    if (rot_tab != nullptr) {
                        const float* cs = rot_tab + tok * rot_dims;
                        cv = cs[f];
                        sv = cs[half + f];
                    } else {                     // no table (a decode step): the same angle, cosine and sine, in place
                        const float ang = (float)b.tok_pos[tok] * inv_freq[f];
                        cv = cosf(ang);
                        sv = sinf(ang);
                    }
                    pc[e] = cv;
                    ps[e] = d < half ? -sv : sv;
                }
            }
        }
#pragma unroll
        for (int e = 0; e < kRetTB; ++e) {
            const int i = tid + e * nthr, tt = i >> 5, jj = blockIdx.z * 32 + (i & 31);
            pv[e] = (i < nb * 32 && jj < vdim) ? qkvg[(int64_t)(start + t0 + tt) * ld + voff + jj] : 0.f;
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < len; t0 += kRetTB) {
        const int nb = min(kRetTB, len - t0);
        __syncthreads();
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
            const int i = tid + e * nthr;
            qs[i] = pq[e] * pc[e] + pq2[e] * ps[e];                 // (u cos - v sin) for the first half, (v cos + u sin) for the second
            ks[i] = (pk[e] * pc[e] + pk2[e] * ps[e]) * kscale;
        }
#pragma unroll
        for (int e = 0; e < kRetTB; ++e) {
            const int i = tid + e * nthr;
            if (i < kRetTB * 32) vs[i] = pv[e];
        }
        __syncthreads();
        if (t0 + kRetTB < len) fetch(t0 + kRetTB);
        for (int tt = 0; tt < nb; ++tt) {
            const float v = vs[tt * 32 + lane];
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
            part[(w * kRetTB + tt) * 32 + lane] = acc;
        }
        __syncthreads();
        for (int i = tid; i < nb * 32 && pass != 1; i += nthr) {
            const int tt = i >> 5, l = i & 31, jj = blockIdx.z * 32 + l;
            if (jj >= vdim) continue;
            float o = 0.f;
            for (int ww = 0; ww < DS; ++ww) o += part[(ww * kRetTB + tt) * 32 + l];
            o_out[(int64_t)(start + t0 + tt) * ((int64_t)heads * vdim) + h * vdim + jj] = o;
        }
    }
    float* st_out = st;
    if (pass == 1) st_out = seg_state + ((int64_t)s * n_seg + seg) * plane + (int64_t)h * dim * vdim;
    else if (pass == 2 && !last_seg) return;
    if (col) {
#pragma unroll
        for (int i = 0; i < DPT; ++i)
            if (d0 + i < dim) st_out[(int64_t)(d0 + i) * vdim + j] = S[i];
    }
}

// Between the two passes of a segmented step: seg_state[s][g] holds the end state L_g of segment g run from zero; the
// state segment g + 1 starts from is S_(g+1) = decay^seg_len S_g + L_g with S_0 the slot's state (zero for a fresh
// sequence).  One thread per state element walks the segments in order and overwrites L_g with S_(g+1).
__global__ void retention_chain_kernel(Batch b, int heads, int dim, int vdim, const float* __restrict__ decay,
                                       const float* __restrict__ state, int seg_len, int n_seg, float* __restrict__ seg_state) {
    const int64_t plane = (int64_t)heads * dim * vdim;
    const int s = blockIdx.y;
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= plane) return;
    const int full = (b.seq_len[s] - 1) / seg_len;          // segments that are followed by another one
    if (full <= 0) return;
    const int h = (int)(e / ((int64_t)dim * vdim));
    const float dn = powf(decay[h], (float)seg_len);
    float S = b.seq_pos0[s] > 0 ? state[(int64_t)b.seq_slot[s] * plane + e] : 0.f;
    float* p = seg_state + (int64_t)s * n_seg * plane + e;
    p[(int64_t)(n_seg - 1) * plane] = S;                    // entry n_seg - 1 never holds an end state: segment 0's start state
    for (int g = 0; g < full; ++g) {
        S = fmaf(dn, S, p[(int64_t)g * plane]);
        p[(int64_t)g * plane] = S;
    }
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

// Tiled form.  One block = 32 consecutive (token, head) rows of ONE sequence (token-major), 8 warps x 4 rows.  The keys
// the rows can see are walked in tiles of 32; a tile's latents are converted to fp32 in shared memory once and serve
// every row of the block -- all heads share them, as do neighbouring tokens, whose windows differ by one key.
//   scores:  lane = key; each lane walks its key's latent and the warp's four query rows 4 floats at a time
//   softmax: running maximum / sum per row (fp32), rescaling the accumulators when the maximum moves
//   values:  lane owns components lane, lane + 32, ...; the tile's weights reach it by shuffle
constexpr int kLaRows = 32, kLaKeys = 32, kLaQH = 4;
__device__ __forceinline__ void unpack16(const uint4& v, float* dst, const float*) {
    *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z),
                                                  __uint_as_float(v.w));
}
__device__ __forceinline__ void unpack16(const uint4& v, float* dst, const __nv_bfloat16*) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
    *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <typename T, int RPL>
__global__ void __launch_bounds__(256) latent_attention_kernel(const float* __restrict__ q_abs, const T* __restrict__ c,
                                                               const T* __restrict__ ring, int ring_len, Batch b, int heads,
                                                               int R, int KD, int window, float scale, int rpb, int vec,
                                                               int nsplit, int use_sink, const float* __restrict__ sink,
                                                               float* __restrict__ part, T* __restrict__ out) {
    // A key row holds KD >= R numbers: the latent (R, which is also the value) and a part all heads share; q_abs rows likewise.
    extern __shared__ __align__(16) float sm[];
    const int RS = ((KD + 3) & ~3) + 4;                // row stride: 16-byte rows, lanes 4 banks apart
    float* qs = sm;                                    // [32][RS]
    float* cs = sm + (size_t)kLaRows * RS;             // [32][RS]
    const int s = blockIdx.y;
    const int len = b.seq_len[s], start = b.seq_start[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    const int row0 = blockIdx.x * rpb, nrows = min(len * heads, row0 + rpb);
    if (row0 >= nrows) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* rbase = ring + (int64_t)slot * ring_len * KD;
    // queries of the block's rows, zero beyond KD and beyond the sequence
    for (int i = threadIdx.x; i < kLaRows * RS; i += blockDim.x) {
        const int rr = i / RS, r = i - rr * RS, row = row0 + rr;
        float v = 0.f;
        if (row < nrows && r < KD) v = q_abs[((int64_t)(start + row / heads) * heads + row % heads) * KD + r];
        qs[i] = v;
    }
    int rpos[kLaQH];                                    // position of each of the warp's rows, -1 = no such row
    float m[kLaQH], l[kLaQH], acc[kLaQH][RPL];
#pragma unroll
    for (int a = 0; a < kLaQH; ++a) {
        const int row = row0 + warp * kLaQH + a;
        rpos[a] = row < nrows ? pos0 + row / heads : -1;
        m[a] = -INFINITY;
        l[a] = 0.f;
        if (use_sink && nsplit == 1 && row < nrows) {      // the sink: a score without a key that counts once in the sum
            m[a] = sink ? sink[row % heads] : 0.f;
            l[a] = 1.f;
        }
#pragma unroll
        for (int i = 0; i < RPL; ++i) acc[a][i] = 0.f;
    }
    const int pos_first = pos0 + row0 / heads, pos_last = pos0 + (min(row0 + kLaRows, nrows) - 1) / heads;
    int jlo = max(0, pos_first - window + 1), jhi = pos_last;
    if (nsplit > 1) {
        // this block's share of the key tiles; the partial softmax states are merged by latent_merge_kernel
        const int tiles = (pos_last - jlo) / kLaKeys + 1, per = (tiles + nsplit - 1) / nsplit;
        jhi = min(pos_last, jlo + (int)(blockIdx.z + 1) * per * kLaKeys - 1);
        jlo += blockIdx.z * per * kLaKeys;
    }
    for (int j0 = jlo; j0 <= jhi; j0 += kLaKeys) {
        __syncthreads();                                // the previous tile (and, first time round, qs) is done with
        if (vec) {
            // 16-byte pieces, every thread's loads of the tile in flight together
            constexpr int EP = 16 / sizeof(T);
            const int ppr = KD / EP, pieces = kLaKeys * ppr;
#pragma unroll 4
            for (int i = threadIdx.x; i < pieces; i += 256) {
                const int kk = i / ppr, e0 = (i - kk * ppr) * EP, j = j0 + kk;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (j <= pos_last) {
                    const T* src = j >= pos0 ? c + (int64_t)(start + j - pos0) * KD : rbase + (int64_t)(j % ring_len) * KD;
                    v = *reinterpret_cast<const uint4*>(src + e0);
                }
                unpack16(v, cs + kk * RS + e0, (const T*)nullptr);
            }
            if (threadIdx.x < kLaKeys) {
                for (int r = KD; r < RS; ++r) cs[threadIdx.x * RS + r] = 0.f;
            }
        } else {
            for (int kk = warp; kk < kLaKeys; kk += 8) {
                const int j = j0 + kk;
                const T* src = nullptr;
                if (j <= pos_last) src = j >= pos0 ? c + (int64_t)(start + j - pos0) * KD : rbase + (int64_t)(j % ring_len) * KD;
                for (int r = lane; r < RS; r += 32) cs[kk * RS + r] = (src != nullptr && r < KD) ? to_f32(src[r]) : 0.f;
            }
        }
        __syncthreads();
        // does any of the warp's rows see any key of this tile?
        bool any = false;
#pragma unroll
        for (int a = 0; a < kLaQH; ++a) any |= rpos[a] >= j0 && rpos[a] - window + 1 <= j0 + kLaKeys - 1;
        if (!any) continue;
        float sc[kLaQH] = {};
        const float4* ck = reinterpret_cast<const float4*>(cs + lane * RS);
        const float4* q4 = reinterpret_cast<const float4*>(qs + warp * kLaQH * RS);
        const int n4 = (KD + 3) >> 2, rs4 = RS >> 2;
        for (int r = 0; r < n4; ++r) {
            const float4 cv = ck[r];
#pragma unroll
            for (int a = 0; a < kLaQH; ++a) {
                const float4 qv = q4[a * rs4 + r];
                sc[a] = fmaf(qv.x, cv.x, fmaf(qv.y, cv.y, fmaf(qv.z, cv.z, fmaf(qv.w, cv.w, sc[a]))));
            }
        }
        const int j = j0 + lane;
        float p[kLaQH];
#pragma unroll
        for (int a = 0; a < kLaQH; ++a) {
            const bool vis = rpos[a] >= 0 && j <= rpos[a] && j > rpos[a] - window;
            const float v = vis ? sc[a] * scale : -INFINITY;
            const float mn = fmaxf(m[a], warp_max(v));
            if (mn == -INFINITY) { p[a] = 0.f; continue; }          // the row sees nothing yet
            const float corr = expf(m[a] - mn);
            p[a] = vis ? expf(v - mn) : 0.f;
            l[a] = l[a] * corr + warp_sum(p[a]);
            m[a] = mn;
#pragma unroll
            for (int i = 0; i < RPL; ++i) acc[a][i] *= corr;
        }
        for (int kk = 0; kk < kLaKeys; ++kk) {
            float pk[kLaQH];
#pragma unroll
            for (int a = 0; a < kLaQH; ++a) pk[a] = __shfl_sync(0xffffffffu, p[a], kk);
            const float* cr = cs + kk * RS;
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int r = lane + 32 * i;
                const float cv = r < R ? cr[r] : 0.f;
#pragma unroll
                for (int a = 0; a < kLaQH; ++a) acc[a][i] = fmaf(pk[a], cv, acc[a][i]);
            }
        }
    }
    if (nsplit > 1) {
#pragma unroll
        for (int a = 0; a < kLaQH; ++a) {
            const int row = row0 + warp * kLaQH + a;
            if (row >= nrows) continue;
            float* dst = part + (((int64_t)(start + row / heads) * heads + row % heads) * nsplit + blockIdx.z) * (R + 2);
            if (lane == 0) { dst[0] = m[a]; dst[1] = l[a]; }
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                const int r = lane + 32 * i;
                if (r < R) dst[2 + r] = acc[a][i];
            }
        }
        return;
    }
#pragma unroll
    for (int a = 0; a < kLaQH; ++a) {
        const int row = row0 + warp * kLaQH + a;
        if (row >= nrows) continue;
        const float inv = 1.f / l[a];
        T* o = out + ((int64_t)(start + row / heads) * heads + row % heads) * R;
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            const int r = lane + 32 * i;
            if (r < R) o[r] = from_f32<T>(acc[a][i] * inv);
        }
    }
}

// Merge of the key-split partial states: one block per (token, head) row.  The splits' weights exp(m_i - max) / sum
// are worked out once into shared memory; then every thread owns latent components and adds the splits in order
// (independent loads, so they overlap).
template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ part, int nsplit, int R, int heads, int use_sink,
                                    const float* __restrict__ sink, T* __restrict__ out) {
    extern __shared__ float wgt[];         // [nsplit]
    const int row = blockIdx.x;
    const float* p = part + (int64_t)row * nsplit * (R + 2);
    if (threadIdx.x < 32) {
        const float sk = sink ? sink[row % heads] : 0.f;
        float mx = use_sink ? sk : -INFINITY;
        for (int i = threadIdx.x; i < nsplit; i += 32) mx = fmaxf(mx, p[(int64_t)i * (R + 2)]);
        mx = warp_max(mx);
        float den = (use_sink && threadIdx.x == 0) ? expf(sk - mx) : 0.f;
        for (int i = threadIdx.x; i < nsplit; i += 32) {
            const float mi = p[(int64_t)i * (R + 2)];
            const float e = mi > -INFINITY ? expf(mi - mx) : 0.f;
            wgt[i] = e;
            den += e * p[(int64_t)i * (R + 2) + 1];
        }
        den = warp_sum(den);
        __syncwarp();
        const float inv = 1.f / den;
        for (int i = threadIdx.x; i < nsplit; i += 32) wgt[i] *= inv;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        float v = 0.f;
#pragma unroll 4
        for (int i = 0; i < nsplit; ++i) v = fmaf(wgt[i], p[(int64_t)i * (R + 2) + 2 + r], v);
        out[(int64_t)row * R + r] = from_f32<T>(v);
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
// A router logit: fp32 dot product of one token's activations with one expert's row, lanes striding over the width and
// a shuffle tree at the end.  Both routing kernels below use this one function, so a token's logits -- and with them its
// experts -- do not depend on which of the two ran.
template <typename T>
__device__ __forceinline__ float router_logit(const T* __restrict__ hr, const float* __restrict__ w, int width, int lane) {
    float s = 0.f;
#pragma unroll 8
    for (int k = lane; k < width; k += 32) s = fmaf(to_f32(hr[k]), w[k], s);
    return warp_sum(s);
}

// `top` rounds of arg-max over z (lowest index wins a tie; z is consumed) and the softmax over the chosen logits.
// UMBS_ROUTE_SIGMOID_GROUPS: z becomes sigmoid(z); a group's score is the sum of its two largest scores; `keep` rounds of
// arg-max over the groups mark the eligible ones; `top` rounds of arg-max over the eligible scores; weights = score / sum.
// UMBS_ROUTE_SOFTMAX_ALL: the softmax's sum runs over every expert, the chosen scores are not renormalised.
// Every weight is multiplied by wscale at the end.
__device__ __forceinline__ void route_choose(float* z, int experts, int top, int mode, int groups, int keep, float wscale,
                                             float* __restrict__ w_out, int32_t* __restrict__ e_out, int32_t* counts) {
    if (mode == UMBS_ROUTE_SIGMOID_GROUPS) {
        const int per = experts / groups;
        for (int e = 0; e < experts; ++e) z[e] = 1.f / (1.f + expf(-z[e]));
        unsigned long long kept = 0ull;
        for (int r = 0; r < keep; ++r) {
            int best = -1;
            float bv = -INFINITY;
            for (int g = 0; g < groups; ++g) {
                if ((kept >> g) & 1ull) continue;
                float a = -INFINITY, b2 = -INFINITY;                   // the group's two largest scores
                for (int e = g * per; e < (g + 1) * per; ++e) {
                    const float v = z[e];
                    if (v > a) { b2 = a; a = v; }
                    else if (v > b2) b2 = v;
                }
                const float gs = per > 1 ? a + b2 : a;
                if (gs > bv) { bv = gs; best = g; }
            }
            if (best >= 0) kept |= 1ull << best;
        }
        float den = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < experts; ++e)
                if (((kept >> (e / per)) & 1ull) && z[e] > bv) { bv = z[e]; best = e; }
            e_out[k] = best;
            w_out[k] = bv;
            den += bv;
            z[best] = -INFINITY;
            atomicAdd(counts + best, 1);
        }
        for (int k = 0; k < top; ++k) w_out[k] = w_out[k] / (den + 1e-20f) * wscale;
        return;
    }
    float zmax = 0.f, den = 0.f;
    if (mode == UMBS_ROUTE_SOFTMAX_ALL) {
        zmax = -INFINITY;
        for (int e = 0; e < experts; ++e) zmax = fmaxf(zmax, z[e]);
        for (int e = 0; e < experts; ++e) den += expf(z[e] - zmax);
    }
    for (int k = 0; k < top; ++k) {
        int best = 0;
        float bv = -INFINITY;
        for (int e = 0; e < experts; ++e)
            if (z[e] > bv) { bv = z[e]; best = e; }
        if (k == 0 && mode != UMBS_ROUTE_SOFTMAX_ALL) zmax = bv;
        const float p = expf(bv - zmax);
        e_out[k] = best;
        w_out[k] = p;
        if (mode != UMBS_ROUTE_SOFTMAX_ALL) den += p;
        z[best] = -INFINITY;
        atomicAdd(counts + best, 1);
    }
    for (int k = 0; k < top; ++k) w_out[k] = w_out[k] / den * wscale;
}

// One block per token: the warps share the experts' logits, then one thread chooses.
template <typename T>
__global__ void __launch_bounds__(256) moe_router_kernel(const T* __restrict__ h, int n, int width, const float* __restrict__ wr,
                                                         int experts, int top, int mode, int groups, int keep, float wscale,
                                                         float* __restrict__ sel_w, int32_t* __restrict__ sel_e,
                                                         int32_t* __restrict__ counts, const float* __restrict__ gate_w,
                                                         float* __restrict__ gate_out) {
    extern __shared__ float z[];           // [experts]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int t = blockIdx.x;
    const T* hr = h + (int64_t)t * width;
    for (int e = warp; e < experts + (gate_w != nullptr ? 1 : 0); e += nw) {
        // one more row for the token's gate (the shared expert's factor): sigmoid of its logit
        const float s = router_logit(hr, e < experts ? wr + (int64_t)e * width : gate_w, width, lane);
        if (lane == 0) {
            if (e < experts) z[e] = s;
            else gate_out[t] = 1.f / (1.f + expf(-s));
        }
    }
    __syncthreads();
    if (threadIdx.x == 0)
        route_choose(z, experts, top, mode, groups, keep, wscale, sel_w + (int64_t)t * top, sel_e + (int64_t)t * top, counts);
}

// The whole routing of a small step (a decode step) in one block: logits of every (token, expert) pair, the choice per
// token, the experts' offsets in the sorted pair list and the scatter of the pairs into it.  Pairs of one expert are
// listed in token order (one thread walks each expert's list), so the layout is the same from run to run.
template <typename T>
__global__ void __launch_bounds__(1024) moe_route_small_kernel(const T* __restrict__ h, int n, int width,
                                                              const float* __restrict__ wr, int experts, int top,
                                                              int mode, int groups, int keep, float wscale,
                                                              float* __restrict__ sel_w, int32_t* __restrict__ sel_e,
                                                              int32_t* __restrict__ grp_off, int32_t* __restrict__ pair_tok,
                                                              int32_t* __restrict__ pair_pos, const float* __restrict__ gate_w,
                                                              float* __restrict__ gate_out) {
    extern __shared__ float zs[];                    // [n][experts] logits, then [experts] counts, [n top] chosen experts
    int32_t* counts = reinterpret_cast<int32_t*>(zs + n * experts);
    int32_t* offs = counts + experts;                // [experts + 1]
    int32_t* chosen = offs + experts + 1;            // [n top]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int i = threadIdx.x; i < experts; i += blockDim.x) counts[i] = 0;
    for (int i = warp; i < n * experts; i += nw) {
        const int t = i / experts, e = i - t * experts;
        const float s = router_logit(h + (int64_t)t * width, wr + (int64_t)e * width, width, lane);
        if (lane == 0) zs[i] = s;
    }
    for (int t = warp; gate_w != nullptr && t < n; t += nw) {
        const float s = router_logit(h + (int64_t)t * width, gate_w, width, lane);
        if (lane == 0) gate_out[t] = 1.f / (1.f + expf(-s));
    }
    __syncthreads();
    for (int t = threadIdx.x; t < n; t += blockDim.x)
        route_choose(zs + t * experts, experts, top, mode, groups, keep, wscale, sel_w + (int64_t)t * top, chosen + t * top, counts);
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int e = 0; e < experts; ++e) { offs[e] = s; grp_off[e] = s; s += counts[e]; }
        offs[experts] = s;
        grp_off[experts] = s;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int p = offs[e];
        for (int i = 0; i < n * top && p < offs[e + 1]; ++i)
            if (chosen[i] == e) { pair_tok[p] = i / top; pair_pos[i] = p; ++p; }
    }
    for (int i = threadIdx.x; i < n * top; i += blockDim.x) sel_e[i] = chosen[i];
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

// One warp per token: g[t] = sigmoid(w . h[t]).
template <typename T>
__global__ void token_gate_kernel(const T* __restrict__ h, int n, int width, const float* __restrict__ w, float* __restrict__ g) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n) return;
    const float s = router_logit(h + (int64_t)t * width, w, width, threadIdx.x & 31);
    if ((threadIdx.x & 31) == 0) g[t] = 1.f / (1.f + expf(-s));
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
    return umbs_embedding_scaled(dtype, ids, table, 1.f, y, n, width, stream);
}

extern "C" int umbs_embedding_scaled(int dtype, const int32_t* ids, const void* table, float scale, float* y, int n, int width,
                                     umbs_stream_t stream) {
    return umbs_embedding_pos(dtype, ids, nullptr, table, scale, nullptr, y, n, width, stream);
}

extern "C" int umbs_embedding_pos(int dtype, const int32_t* ids, const int32_t* tok_pos, const void* table, float scale,
                                  const float* pos_freq, float* y, int n, int width, umbs_stream_t stream) {
    if (n <= 0) return 0;
    if (pos_freq != nullptr && tok_pos == nullptr) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    UMBS_DISPATCH_T(dtype, embedding_kernel<T><<<n, threads_for(width), 0, st>>>(ids, (const T*)table, y, width, scale, tok_pos,
                                                                              pos_freq));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_token_gate(int dtype, const void* h, int n, int width, const float* w, float* g, umbs_stream_t stream) {
    if (n <= 0) return 0;
    if (h == nullptr || w == nullptr || g == nullptr) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    UMBS_DISPATCH_T(dtype, token_gate_kernel<T><<<(n + 3) / 4, 128, 0, st>>>((const T*)h, n, width, w, g));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_group_norm_shift(int dtype, const float* x, const float* w, const float* shift_w, float* shift_state,
                                     int slots, const umbs_batch_t* batch, int width, int groups, float eps, void* h,
                                     void* hs, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (groups <= 0 || width % groups != 0) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = threads_for(width);
    const size_t smem = (2 * (size_t)groups + 2 * (size_t)groups * std::max(1, threads / 32 / groups)) * sizeof(float);
    UMBS_DISPATCH_T(dtype, group_norm_shift_kernel<T><<<batch->n_tokens, threads, smem, st>>>(
                               x, w, shift_w, shift_state, slots, *batch, width, groups, eps, (T*)h, (T*)hs));
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_group_norm_rows(int dtype, const float* x, const int32_t* rows, int n_rows, const float* w, int width,
                                    int groups, float eps, void* y, umbs_stream_t stream) {
    if (n_rows <= 0) return 0;
    if (groups <= 0 || width % groups != 0) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = threads_for(width);
    const size_t smem = ((size_t)groups + 2 * (size_t)groups * std::max(1, threads / 32 / groups)) * sizeof(float);
    UMBS_DISPATCH_T(dtype, group_norm_rows_kernel<T><<<n_rows, threads, smem, st>>>(
                               x, rows, w, width, groups, eps, (T*)y));
    count_launches(1);
    return (int)cudaGetLastError();
}

template <int DPT, int kRetTB>
static int launch_retention(const float* qkvg, int64_t ld, const Batch& b, int heads, int dim, int vdim, int rot_dims,
                            const float* rot_tab, const float* inv_freq, const float* decay, float* state, float* o,
                            int seg_len, int n_seg, int pass, float* seg_state, cudaStream_t st) {
    const int ds = (dim + DPT - 1) / DPT;
    const dim3 grid(b.n_seqs * n_seg, heads, (vdim + 31) / 32), block(32, ds);
    const size_t smem = ((size_t)2 * kRetTB * ds * DPT + (size_t)ds * kRetTB * 32 + kRetTB * 32) * sizeof(float);
    static size_t set = 0;
    if (smem > 48 * 1024 && smem > set) {
        cudaError_t e = cudaFuncSetAttribute(retention_kernel<DPT, kRetTB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = smem;
    }
    retention_kernel<DPT, kRetTB><<<grid, block, smem, st>>>(qkvg, ld, b, heads, dim, vdim, rot_dims, rot_tab, inv_freq, decay,
                                                             state, o, seg_len, n_seg, pass, seg_state);
    return 0;
}

extern "C" int umbs_retention(int dtype, const float* qkvg, int64_t ld, const umbs_batch_t* batch, int heads, int dim,
                              int vdim, int rot_dims, const float* inv_freq, const float* decay, float eps, float* state,
                              float* o_scratch, float* rot_scratch, float* seg_scratch, size_t seg_bytes, void* out,
                              umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (rot_dims < 0 || rot_dims > dim || (rot_dims & 1)) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned launches = 2;
    // a step with several tokens per sequence shares one cos | sin table between heads and column blocks; a decode step
    // works the few values out inside the recurrence kernel
    const float* rot_tab = nullptr;
    if (rot_dims > 0 && batch->max_seq_len > 1) {
        rotary_table_kernel<<<batch->n_tokens, 64, 0, st>>>(batch->tok_pos, inv_freq, rot_dims / 2, rot_scratch);
        rot_tab = rot_scratch;
        ++launches;
    }
    // Few blocks and long sequences (one long prompt): cut the sequences into segments that run side by side, in two
    // passes (local end states from zero, chained into start states, then the outputs).  Twice the arithmetic of the
    // recurrence for n_seg times the blocks; the result differs from the single walk by fp32 rounding only.
    int n_seg = 1, seg_len = batch->max_seq_len;
    const int base_blocks = batch->n_seqs * heads * ((vdim + 31) / 32);
    if (seg_scratch != nullptr && base_blocks <= 148 && batch->max_seq_len >= 128) {     // less than a block per SM
        int want = std::min((592 + base_blocks - 1) / base_blocks, batch->max_seq_len / 64);
        const size_t fit = seg_bytes / ((size_t)batch->n_seqs * heads * dim * vdim * sizeof(float));
        want = (int)std::min<size_t>(want, fit);
        if (want >= 2) {
            seg_len = ((batch->max_seq_len + want - 1) / want + 15) & ~15;
            n_seg = (batch->max_seq_len + seg_len - 1) / seg_len;
        }
    }
    auto run = [&](int pass) -> int {
        if (dim <= 32) return launch_retention<8, 16>(qkvg, ld, *batch, heads, dim, vdim, rot_dims, rot_tab, inv_freq, decay, state, o_scratch, seg_len, n_seg, pass, seg_scratch, st);
        if (dim <= 128) return launch_retention<16, 16>(qkvg, ld, *batch, heads, dim, vdim, rot_dims, rot_tab, inv_freq, decay, state, o_scratch, seg_len, n_seg, pass, seg_scratch, st);
        if (dim <= 512) return launch_retention<32, 8>(qkvg, ld, *batch, heads, dim, vdim, rot_dims, rot_tab, inv_freq, decay, state, o_scratch, seg_len, n_seg, pass, seg_scratch, st);
        return UMB_ERR_UNSUPPORTED;
    };
    int rc;
    if (n_seg > 1) {
        rc = run(1);
        if (rc) return rc;
        const int64_t plane = (int64_t)heads * dim * vdim;
        retention_chain_kernel<<<dim3((unsigned)((plane + 255) / 256), batch->n_seqs), 256, 0, st>>>(*batch, heads, dim, vdim, decay, state,
                                                                                                 seg_len, n_seg, seg_scratch);
        launches += 2;
        rc = run(2);
    } else {
        rc = run(0);
    }
    if (rc) return rc;
    const int warps = batch->n_tokens * heads;
    UMBS_DISPATCH_T(dtype, retention_gate_kernel<T><<<(warps + 3) / 4, 128, 0, st>>>(o_scratch, qkvg, ld, batch->n_tokens,
                                                                                   heads, dim, vdim, eps, (T*)out));
    count_launches(launches);
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
                                   int heads, int R, int KD, int window, float scale, int use_sink, const float* sink,
                                   float* part, size_t part_bytes, void* out, cudaStream_t st) {
    const int rpb = kLaRows;
    const size_t smem = (size_t)2 * kLaRows * (((KD + 3) & ~3) + 4) * sizeof(float);
    if (smem > (size_t)200 * 1024) return UMB_ERR_UNSUPPORTED;
    // decode steps: few blocks and a long serial walk over the window -> split the keys over as many blocks per row tile
    // as fill the GPU (as many block slots per SM as the tiles' shared memory allows), as far as the scratch buffer reaches
    int nsplit = 1;
    if (b.max_seq_len == 1 && part != nullptr) {
        const int blocks = ((heads + rpb - 1) / rpb) * b.n_seqs;
        const int tiles = (std::min(window, ring_len + 1) + kLaKeys - 1) / kLaKeys;
        const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(4, (size_t)227 * 1024 / (smem + 1024)));
        nsplit = std::max(1, std::min(tiles, 148 * per_sm / std::max(blocks, 1)));   // down to one key tile per block
        const size_t fit = part_bytes / ((size_t)b.n_tokens * heads * (R + 2) * sizeof(float));   // splits the scratch holds
        nsplit = (int)std::max<size_t>(1, std::min<size_t>(nsplit, fit));
    }
    const int ep = 16 / (int)sizeof(T);
    const int vec = (KD % ep == 0) && ((uintptr_t)c % 16 == 0) && ((uintptr_t)ring % 16 == 0);
    const dim3 grid((b.max_seq_len * heads + rpb - 1) / rpb, b.n_seqs, nsplit), block(256);
#define UMBS_LA(RPL)                                                                                                   \
    do {                                                                                                               \
        static size_t set = 0;                                                                                         \
        if (smem > 48 * 1024 && smem > set) {                                                                          \
            cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<T, RPL>,                                      \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
            if (e != cudaSuccess) return (int)e;                                                                       \
            set = smem;                                                                                                \
        }                                                                                                              \
        latent_attention_kernel<T, RPL><<<grid, block, smem, st>>>(q_abs, (const T*)c, (const T*)ring, ring_len, b,    \
                                                                   heads, R, KD, window, scale, rpb, vec, nsplit,      \
                                                                   use_sink, sink, part, (T*)out);                     \
    } while (0)
    if (R <= 32) UMBS_LA(1);
    else if (R <= 64) UMBS_LA(2);
    else if (R <= 128) UMBS_LA(4);
    else if (R <= 256) UMBS_LA(8);
    else if (R <= 512) UMBS_LA(16);
    else return UMB_ERR_UNSUPPORTED;
#undef UMBS_LA
    if (nsplit > 1) {
        const int rows = b.n_tokens * heads;
        latent_merge_kernel<T><<<rows, R >= 256 ? 256 : (R >= 128 ? 128 : 64), nsplit * sizeof(float), st>>>(part, nsplit, R, heads, use_sink, sink, (T*)out);
        count_launches(1);
    }
    return 0;
}

extern "C" int umbs_latent_attention(int dtype, const float* q_abs, const void* c, const void* ring, int ring_len,
                                     const umbs_batch_t* batch, int heads, int kv_rank, int window, float scale,
                                     float* split_scratch, size_t split_bytes, void* out, umbs_stream_t stream) {
    if (window < 1) return UMB_ERR_ARG;
    return umbs_latent_attention_ex(dtype, q_abs, c, ring, ring_len, batch, heads, kv_rank, 0, window, scale, UMBS_ATTN_SOFTMAX,
                                    nullptr, split_scratch, split_bytes, out, stream);
}

extern "C" int umbs_latent_attention_ex(int dtype, const float* q_abs, const void* c, const void* ring, int ring_len,
                                        const umbs_batch_t* batch, int heads, int kv_rank, int rope_dim, int window,
                                        float scale, int mode, const float* sink, float* split_scratch, size_t split_bytes,
                                        void* out, umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (ring_len < 1 || rope_dim < 0 || kv_rank < 1 || heads < 1) return UMB_ERR_ARG;
    if (mode != UMBS_ATTN_SOFTMAX && mode != UMBS_ATTN_SOFTMAX_SINK) return UMB_ERR_UNSUPPORTED;
    if (window <= 0) window = 1 << 30;                       // every earlier token
    int rc = 0;
    UMBS_DISPATCH_T(dtype, rc = launch_latent_attention<T>(q_abs, c, ring, ring_len, *batch, heads, kv_rank, kv_rank + rope_dim,
                                                           window, scale, mode == UMBS_ATTN_SOFTMAX_SINK, sink, split_scratch,
                                                           split_bytes, out, (cudaStream_t)stream));
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
    return umbs_moe_route_ex(dtype, h, n, width, w_router, experts, top, UMBS_ROUTE_SOFTMAX_TOP, 1, 1, sel_w, grp_off, pair_tok,
                             pair_pos, scratch, nullptr, nullptr, stream);
}

extern "C" int umbs_moe_route_ex(int dtype, const void* h, int n, int width, const float* w_router, int experts, int top,
                                 int mode, int groups, int keep, float* sel_w, int32_t* grp_off, int32_t* pair_tok,
                                 int32_t* pair_pos, int32_t* scratch, const float* gate_w, float* gate_out,
                                 umbs_stream_t stream) {
    return umbs_moe_route_scaled(dtype, h, n, width, w_router, experts, top, mode, groups, keep, 1.f, sel_w, grp_off, pair_tok,
                                 pair_pos, scratch, gate_w, gate_out, stream);
}

extern "C" int umbs_moe_route_scaled(int dtype, const void* h, int n, int width, const float* w_router, int experts, int top,
                                     int mode, int groups, int keep, float weight_scale, float* sel_w, int32_t* grp_off,
                                     int32_t* pair_tok, int32_t* pair_pos, int32_t* scratch, const float* gate_w,
                                     float* gate_out, umbs_stream_t stream) {
    if (n <= 0) return 0;
    if (weight_scale == 0.f) weight_scale = 1.f;
    if (top < 1 || top > experts || (gate_w != nullptr && gate_out == nullptr)) return UMB_ERR_ARG;
    if (mode == UMBS_ROUTE_SIGMOID_GROUPS) {
        if (groups < 1 || experts % groups != 0 || keep < 1 || keep > groups || top > keep * (experts / groups)) return UMB_ERR_ARG;
        if (groups > 64) return UMB_ERR_UNSUPPORTED;
    } else if (mode != UMBS_ROUTE_SOFTMAX_TOP && mode != UMBS_ROUTE_SOFTMAX_ALL) {
        return UMB_ERR_ARG;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if ((size_t)n * experts <= 256 && (size_t)n * top <= 1024) {
        // a small step (decoding): one block does the logits, the choice, the offsets and the sorted pair list
        const size_t smem = ((size_t)n * experts + 2 * (size_t)experts + 1 + (size_t)n * top) * sizeof(float);
        UMBS_DISPATCH_T(dtype, moe_route_small_kernel<T><<<1, 1024, smem, st>>>((const T*)h, n, width, w_router, experts, top,
                                                                              mode, groups, keep, weight_scale, sel_w, scratch + 2 * experts,
                                                                              grp_off, pair_tok, pair_pos, gate_w, gate_out));
        count_launches(1);
        return (int)cudaGetLastError();
    }
    int32_t* counts = scratch;                 // [experts]
    int32_t* cursor = scratch + experts;       // [experts]
    int32_t* sel_e = scratch + 2 * experts;    // [n top]
    cudaError_t e = cudaMemsetAsync(counts, 0, experts * sizeof(int32_t), st);
    if (e != cudaSuccess) return (int)e;
    const int rthreads = experts >= 8 ? 256 : 32 * experts;
    UMBS_DISPATCH_T(dtype, moe_router_kernel<T><<<n, rthreads, (size_t)experts * sizeof(float), st>>>(
                               (const T*)h, n, width, w_router, experts, top, mode, groups, keep, weight_scale, sel_w, sel_e, counts,
                               gate_w, gate_out));
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
