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
// Score options (umbs_attn_opts_t): a tanh cap, a penalty r1 ln(1 + r2 distance) per head, a chunked mask, several maps per
// head and every query head against every value head.  The grid's head axis then counts "virtual heads"
// (h maps + m) value_heads + c, each an independent softmax row; their normalised outputs can be left in fp32
// (raw_out) for umbs_attention_finish, which mixes heads' weights, subtracts maps, norms and gates.
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
    // score options
    float softcap; const float* r1; const float* r2; int chunk, maps, vheads; float* raw;
};

// What a virtual head reads: its query's offset in a q row, its keys' and values' offsets in a key/value row.
struct VHead { int h, qoff, koff, voff, row_kv, qstride, nv; };
__device__ __forceinline__ VHead virtual_head(const CachedAttnArgs& a, int vh) {
    const int C = a.vheads, M = a.maps;
    const int cv = vh % C, hm = vh / C, mp = hm % M, h = hm / M, g = h / (a.heads / a.kv_heads);
    const int kdim = a.kv_heads * M * a.dim;
    VHead v;
    v.h = h; v.qoff = hm * a.dim; v.koff = (g * M + mp) * a.dim; v.voff = kdim + (C > 1 ? cv : g) * a.vdim;
    v.row_kv = kdim + a.kv_heads * a.vdim; v.qstride = a.heads * M * a.dim; v.nv = a.heads * M * C;
    return v;
}

// scale, cap and distance penalty of a raw dot product; dist = row position - key position
__device__ __forceinline__ float shaped_score(const CachedAttnArgs& a, float dot, float r1h, float r2h, int dist) {
    float sv = dot * a.scale;
    if (a.softcap > 0.f) sv = a.softcap * tanhf(sv / a.softcap);
    if (a.r1 != nullptr) sv -= r1h * log1pf(r2h * (float)dist);
    return sv;
}

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
    const int s = blockIdx.z, vh = blockIdx.y, q0 = blockIdx.x * kCaQ;
    const int len = b.seq_len[s], start = b.seq_start[s], pos0 = b.seq_pos0[s], slot = b.seq_slot[s];
    if (q0 >= len) return;
    const VHead vhd = virtual_head(a, vh);
    const int h = vhd.h, row_kv = vhd.row_kv, koff = vhd.koff, voff = vhd.voff;
    const int window = a.window > 0 ? a.window : (1 << 30), chunk = a.chunk;
    const float r1h = a.r1 ? a.r1[h] : 0.f, r2h = a.r1 ? a.r2[h] : 0.f;
    const T* q = (const T*)a.q;
    const T* kv = (const T*)a.kv;
    const T* cache = (const T*)a.kv_cache;
    const T* pooled = (const T*)a.pool_cache;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    for (int i = tid; i < kCaQ * dim; i += 256) {
        const int r = i / dim, d = i - r * dim;
        Qs[d * kCaS + r] = (q0 + r < len) ? to_f32(q[(int64_t)(start + q0 + r) * vhd.qstride + vhd.qoff + d]) : 0.f;
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
    const int j_lo = max(max(0, p_lo - window + 1), chunk > 0 ? p_lo / chunk * chunk : 0);
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
                vis[jj] = r < len && (in_pool ? j < pooled_visible(rp, window, a.pool)
                                              : (j <= rp && j > rp - window && (chunk <= 0 || j / chunk == rp / chunk)));
            }
            if (MODE == UMBS_ATTN_SIGMOID) {
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) p[jj] = vis[jj] ? sigmoidf_(sc[i][jj] * a.scale + hb) : 0.f;
            } else {
                float val[4], mx = -INFINITY;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    val[jj] = vis[jj] ? shaped_score(a, sc[i][jj], r1h, r2h, rp - (base + tx * 4 + jj)) : -INFINITY;
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
        if (a.raw != nullptr) {
            float* rrow = a.raw + (t * vhd.nv + vh) * vdim;
#pragma unroll
            for (int cb = 0; cb < VC / 4; ++cb)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int col = cb * 64 + tx * 4 + c;
                    if (col < vdim) rrow[col] = o[i][cb * 4 + c] * inv;
                }
            continue;
        }
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
    const dim3 grid((b.max_seq_len + kCaQ - 1) / kCaQ, a.heads * a.maps * a.vheads, b.n_seqs);
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
    const int split = blockIdx.x, vh = blockIdx.y, s = blockIdx.z;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int dim = a.dim, vdim = a.vdim;
    const int t = b.seq_start[s], p = b.seq_pos0[s], slot = b.seq_slot[s];
    const VHead vhd = virtual_head(a, vh);
    const int h = vhd.h, row_kv = vhd.row_kv, koff = vhd.koff, voff = vhd.voff;
    const float r1h = a.r1 ? a.r1[h] : 0.f, r2h = a.r1 ? a.r2[h] : 0.f;
    const int window = a.window > 0 ? a.window : (1 << 30);
    const int n_pool = pooled_visible(p, window, a.pool);
    const int j_lo = max(max(0, p - window + 1), a.chunk > 0 ? p / a.chunk * a.chunk : 0);
    const int n_keys = n_pool + (p - j_lo + 1);
    const int per = (n_keys + n_split - 1) / n_split, lo = split * per, hi = min(n_keys, lo + per);
    const T* qrow = (const T*)a.q + (int64_t)t * vhd.qstride + vhd.qoff;
    float qv[kCdMaxPerLane], o[kCdMaxPerLane];
#pragma unroll
    for (int i = 0; i < kCdMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < dim ? to_f32(qrow[d]) : 0.f;
        o[i] = 0.f;
    }
    const float hb = (MODE == UMBS_ATTN_SIGMOID && a.head_bias) ? a.head_bias[h] : 0.f;
    float m = -INFINITY, l = 0.f;
    // Four of the warp's keys at a time: their key and value loads are all in flight before the first is needed; the
    // softmax state then takes them one by one, in key order (the same additions as one key at a time).
    constexpr int KU = 4;
    for (int kb = lo + w; kb < hi; kb += kCdWarps * KU) {
        const T* src[KU];
        int dist[KU];
        float dot[KU], vv[KU][kCdMaxPerLane];
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            const int k = min(kb + u * kCdWarps, hi - 1);           // (a place beyond the run reads the last key; unused)
            dist[u] = 0;
            if (k < n_pool) src[u] = (const T*)a.pool_cache + ((int64_t)slot * a.pool_len + k) * row_kv;
            else {
                const int j = j_lo + (k - n_pool);
                dist[u] = p - j;
                src[u] = j >= p ? (const T*)a.kv + (int64_t)t * row_kv
                                : (const T*)a.kv_cache + ((int64_t)slot * a.kv_len + j % a.kv_len) * row_kv;
            }
        }
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            dot[u] = 0.f;
#pragma unroll
            for (int i = 0; i < kCdMaxPerLane; ++i) {
                const int d = lane + 32 * i;
                if (d < dim) dot[u] = fmaf(qv[i], to_f32(src[u][koff + d]), dot[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < KU; ++u)
#pragma unroll
            for (int i = 0; i < kCdMaxPerLane; ++i) {
                const int d = lane + 32 * i;
                vv[u][i] = d < vdim ? to_f32(src[u][voff + d]) : 0.f;
            }
#pragma unroll
        for (int x = 16; x > 0; x >>= 1)
#pragma unroll
            for (int u = 0; u < KU; ++u) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], x);
#pragma unroll
        for (int u = 0; u < KU; ++u) {
            if (kb + u * kCdWarps >= hi) break;
            float pw;
            if (MODE == UMBS_ATTN_SIGMOID) {
                pw = sigmoidf_(dot[u] * a.scale + hb);
            } else {
                const float sc = shaped_score(a, dot[u], r1h, r2h, dist[u]), mn = fmaxf(m, sc), corr = expf(m - mn);   // m = -inf the first time: corr = 0
                pw = expf(sc - mn);
                l = l * corr + pw;
                m = mn;
#pragma unroll
                for (int i = 0; i < kCdMaxPerLane; ++i) o[i] *= corr;
            }
#pragma unroll
            for (int i = 0; i < kCdMaxPerLane; ++i) o[i] = fmaf(pw, vv[u][i], o[i]);
        }
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
        float* pr = part + (((int64_t)t * vhd.nv + vh) * n_split + split) * (vdim + 2);
        if (c < vdim) pr[c] = O;
        if (c == 0) { pr[vdim] = M; pr[vdim + 1] = L; }
        return;
    }
    if (c < vdim) {
        const float inv = MODE == UMBS_ATTN_SIGMOID ? 1.f : 1.f / L;
        if (a.raw != nullptr) { a.raw[((int64_t)t * vhd.nv + vh) * vdim + c] = O * inv; return; }
        float gt = 1.f;
        if (a.gate) gt = sigmoidf_(a.gate[(int64_t)t * a.ldg + (a.gate_per_head ? h : h * vdim + c)]);
        ((T*)a.out)[(int64_t)t * a.heads * vdim + (int64_t)h * vdim + c] = from_f32<T>(O * inv * gt);
    }
}

// One block per (token, head): the splits' triples, in split order, then the sink, the division and the output gate.
template <typename T, int MODE>
__global__ void cached_attention_merge_kernel(CachedAttnArgs a, int n_split, const float* __restrict__ part) {
    const int nv = a.heads * a.maps * a.vheads;
    const int th = blockIdx.x, t = th / nv, h = th - t * nv, vdim = a.vdim, c = threadIdx.x;      // (without options h is the head)
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
        if (a.raw != nullptr) { a.raw[(int64_t)th * vdim + c] = O * inv; return; }
        float gt = 1.f;
        if (a.gate) gt = sigmoidf_(a.gate[(int64_t)t * a.ldg + (a.gate_per_head ? h : h * vdim + c)]);
        ((T*)a.out)[(int64_t)t * a.heads * vdim + (int64_t)h * vdim + c] = from_f32<T>(O * inv * gt);
    }
}

template <typename T, int MODE>
static int launch_decode(const CachedAttnArgs& a, const Batch& b, int n_split, float* part, cudaStream_t st) {
    const int nv = a.heads * a.maps * a.vheads;
    cached_attention_decode_kernel<T, MODE><<<dim3(n_split, nv, b.n_seqs), 32 * kCdWarps, 0, st>>>(a, b, n_split, part);
    if (n_split > 1) cached_attention_merge_kernel<T, MODE><<<b.n_tokens * nv, a.vdim <= 128 ? 128 : 256, 0, st>>>(a, n_split, part);
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

namespace umbs {
// One warp per (token, head): from the virtual heads' raw outputs to the head's output.
template <typename T>
__global__ void attention_finish_kernel(const float* __restrict__ raw, int n_pairs, int heads, int kv_heads, int vdim, int maps,
                                        int vheads, const float* __restrict__ talk, float lambda, int unit_norm, float eps,
                                        float out_mult, const float* __restrict__ gate, int64_t ldg, T* __restrict__ out) {
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (pair >= n_pairs) return;
    const int t = pair / heads, h = pair - t * heads, nv = heads * maps * vheads;
    const float* rt = raw + (int64_t)t * nv * vdim;
    float v[8], ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        v[i] = 0.f;
        if (c >= vdim) continue;
        if (talk != nullptr) {
            const int own = h / (heads / kv_heads);                       // the value head of query head h
            float acc = 0.f;
            for (int g = 0; g < heads; ++g) acc = fmaf(talk[h * heads + g], rt[(int64_t)(g * vheads + own) * vdim + c], acc);
            v[i] = acc;
        } else if (maps == 2) {
            v[i] = rt[(int64_t)(h * 2) * vdim + c] - lambda * rt[(int64_t)(h * 2 + 1) * vdim + c];
        } else {
            v[i] = rt[(int64_t)h * vdim + c];
        }
        ss = fmaf(v[i], v[i], ss);
    }
#pragma unroll
    for (int x = 16; x > 0; x >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, x);
    const float f = (unit_norm ? 1.f / sqrtf(ss / (float)vdim + eps) : 1.f) * out_mult;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = lane + 32 * i;
        if (c >= vdim) continue;
        float o = v[i] * f;
        if (gate != nullptr) o *= sigmoidf_(gate[(int64_t)t * ldg + h * vdim + c]);
        out[(int64_t)t * heads * vdim + h * vdim + c] = from_f32<T>(o);
    }
}

}  // namespace umbs

extern "C" int umbs_attention_finish(int dtype, const float* raw, int n_tokens, int heads, int kv_heads, int vdim, int maps,
                                     int value_heads, const float* talk, float diff_lambda, int unit_norm, float eps,
                                     float out_mult, const float* gate, int64_t ldg, void* out, umbs_stream_t stream) {
    if (n_tokens <= 0) return 0;
    maps = maps < 1 ? 1 : maps;
    value_heads = value_heads < 1 ? 1 : value_heads;
    if (raw == nullptr || out == nullptr || heads < 1 || kv_heads < 1 || heads % kv_heads != 0) return UMB_ERR_ARG;
    if (vdim < 1 || vdim > 256 || maps > 2) return UMB_ERR_UNSUPPORTED;
    if (talk != nullptr ? (maps != 1 || value_heads != kv_heads) : value_heads != 1) return UMB_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    const int pairs = n_tokens * heads;
    if (dtype == UMBS_BF16)
        attention_finish_kernel<__nv_bfloat16><<<(pairs + 3) / 4, 128, 0, st>>>(raw, pairs, heads, kv_heads, vdim, maps, value_heads, talk,
                                                                               diff_lambda, unit_norm, eps, out_mult != 0.f ? out_mult : 1.f,
                                                                               gate, ldg, (__nv_bfloat16*)out);
    else if (dtype == UMBS_F32)
        attention_finish_kernel<float><<<(pairs + 3) / 4, 128, 0, st>>>(raw, pairs, heads, kv_heads, vdim, maps, value_heads, talk, diff_lambda,
                                                                       unit_norm, eps, out_mult != 0.f ? out_mult : 1.f, gate, ldg, (float*)out);
    else return UMB_ERR_ARG;
    count_launches(1);
    return (int)cudaGetLastError();
}

extern "C" int umbs_cached_attention(int dtype, int mode, const void* q, const void* kv, const void* kv_cache, int kv_len,
                                     const void* pool_cache, int pool_len, const umbs_batch_t* batch, int heads,
                                     int kv_heads, int dim, int vdim, int window, int pool, float scale,
                                     const float* head_bias, const float* gate, int64_t ldg, int gate_per_head,
                                     float* split_scratch, size_t split_bytes, void* out, umbs_stream_t stream) {
    return umbs_cached_attention_ex(dtype, mode, q, kv, kv_cache, kv_len, pool_cache, pool_len, batch, heads, kv_heads, dim, vdim,
                                    window, pool, scale, head_bias, gate, ldg, gate_per_head, nullptr, split_scratch, split_bytes,
                                    out, stream);
}

extern "C" int umbs_cached_attention_ex(int dtype, int mode, const void* q, const void* kv, const void* kv_cache, int kv_len,
                                        const void* pool_cache, int pool_len, const umbs_batch_t* batch, int heads,
                                        int kv_heads, int dim, int vdim, int window, int pool, float scale,
                                        const float* head_bias, const float* gate, int64_t ldg, int gate_per_head,
                                        const umbs_attn_opts_t* opts, float* split_scratch, size_t split_bytes, void* out,
                                        umbs_stream_t stream) {
    if (batch->n_tokens <= 0) return 0;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads != 0 || kv_len < 1) return UMB_ERR_ARG;
    if (pool > 0 && (window <= 0 || pool_cache == nullptr || pool_len < 1)) return UMB_ERR_ARG;
    if (dim < 1 || vdim < 1 || dim > 256 || vdim > 256) return UMB_ERR_UNSUPPORTED;      // tiles and lanes are sized for heads up to 256
    cudaStream_t st = (cudaStream_t)stream;
    CachedAttnArgs a{q, kv, kv_cache, pool_cache, kv_len, pool_len, heads, kv_heads, dim, vdim, window, pool, scale,
                     head_bias, gate, ldg, gate_per_head, out, 0.f, nullptr, nullptr, 0, 1, 1, nullptr};
    if (opts != nullptr) {
        a.softcap = opts->softcap; a.r1 = opts->dist_r1; a.r2 = opts->dist_r2; a.chunk = opts->chunk;
        a.maps = opts->maps > 0 ? opts->maps : 1; a.vheads = opts->value_heads > 0 ? opts->value_heads : 1; a.raw = opts->raw_out;
        const bool any = a.softcap > 0.f || a.r1 != nullptr || a.chunk > 0 || a.maps > 1 || a.vheads > 1;
        if ((a.r1 != nullptr) != (a.r2 != nullptr) || a.chunk < 0) return UMB_ERR_ARG;
        if (any && (pool > 0 || mode == UMBS_ATTN_SIGMOID)) return UMB_ERR_UNSUPPORTED;
        if ((a.maps > 1 || a.vheads > 1) && a.raw == nullptr) return UMB_ERR_ARG;      // several rows per head need the finishing pass
        if (a.vheads != 1 && a.vheads != kv_heads) return UMB_ERR_ARG;
    }
    if (a.raw == nullptr && out == nullptr) return UMB_ERR_ARG;
    heads = a.heads * a.maps * a.vheads;                   // rows per token from here on (splits, scratch)
    int rc;
    if (batch->max_seq_len == 1) {
        // a decode step: about 256 keys per block, as many splits as the longest context of the step asks for, the GPU
        // has room for (two blocks per SM) and the scratch buffer holds
        int keys = window > 0 ? (batch->max_pos0 < window ? batch->max_pos0 + 1 : window + (pool > 0 ? batch->max_pos0 / pool : 0))
                              : batch->max_pos0 + 1;
        if (a.chunk > 0 && keys > a.chunk) keys = a.chunk;
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
