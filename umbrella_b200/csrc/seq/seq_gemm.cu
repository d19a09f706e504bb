// Matrix products of the sequence-state decoders: C = A W^T with W stored [out, in], batched over groups (heads or
// experts), optionally over expert-sorted gathered rows, optionally with the gated feed-forward activation fused
// into the epilogue of a gate|up pair of products.
//
// Three kernels share one argument block:
//   * gemm_simt_kernel  -- fp32 FMA chains over shared-memory tiles; the UMBS_F32 mode (true 32-bit) and every shape
//                          the tensor-core kernel does not take (K not a multiple of 16, unaligned rows);
//   * gemm_mma_kernel   -- bf16 operands through mma.sync.m16n8k16 with fp32 accumulators;
//   * gemm_skinny_kernel -- bf16, at most 16 rows (decoding): a weight stream with the rows' partial sums in registers.
// In each of them an output element is one fp32 sum over k in an order that does not depend on the other rows, so a
// row's result is the same whatever else is in the batch; which kernel runs depends on the row count, and the three
// differ from each other by rounding only.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "seq_internal.h"

namespace umbs {

struct GemmArgs {
    const void* A; int64_t lda; int a_goff;
    const void* W; int64_t ldw; int64_t w_gstride;
    void* C; int64_t ldc; int c_goff;
    int M, N, K;
    const int32_t* grp_off;
    const int32_t* row_src;
    float limit;
    int act;          // UMBS_ACT_*: which gated activation a dual product applies
    const float* bias;       // fp32 [N] (dual: [2 N]) added to the sums, or NULL
    const float* out_gate;   // fp32: the result is multiplied by sigmoid(out_gate[row ld_gate + g gate_goff + n]), or NULL
    int64_t ld_gate;
    int gate_goff;
    int unary;        // UMBS_UNARY_* of a plain product, with its two numbers
    float p0, p1;
};

__device__ __forceinline__ float unary_act(float z, int unary, float p0, float p1) {
    if (unary == UMBS_UNARY_TANH) return tanhf(z);
    if (unary == UMBS_UNARY_XIELU) return z > 0.f ? fmaf(p0 * z, z, 0.5f * z) : fmaf(p1, expm1f(z) - z, 0.5f * z);
    return z;
}

__device__ __forceinline__ float gated_act(float g, float u, float limit, int act) {
    if (act == UMBS_ACT_GELU_TANH) {      // 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * u
        const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.f + tanhf(z)) * u;
    }
    if (act == UMBS_ACT_SILU) return g * (1.f / (1.f + expf(-g))) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * (1.f / (1.f + expf(-1.702f * g))) * (u + 1.f);
}

// What every kernel does with a finished sum (and, for a gate|up pair, its partner): bias, activation, output gate.
template <bool DUAL>
__device__ __forceinline__ float finish(const GemmArgs& a, float s, float s2, int g, int64_t row, int n) {
    if (a.bias != nullptr) {
        s += a.bias[n];
        if (DUAL) s2 += a.bias[a.N + n];
    }
    float v = DUAL ? gated_act(s, s2, a.limit, a.act) : (a.unary ? unary_act(s, a.unary, a.p0, a.p1) : s);
    if (a.out_gate != nullptr) v *= 1.f / (1.f + expf(-a.out_gate[row * a.ld_gate + (int64_t)g * a.gate_goff + n]));
    return v;
}

// ------------------------------------------------------------------------------------------------ SIMT
constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TC, bool DUAL>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmArgs a) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[DUAL ? 2 : 1][BK][BN + 4];
    const int g = blockIdx.z;
    int row_lo = 0, rows = a.M;
    if (a.grp_off != nullptr) { row_lo = a.grp_off[g]; rows = a.grp_off[g + 1] - row_lo; }
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    if (m0 >= rows) return;
    const TA* A = (const TA*)a.A + (int64_t)g * a.a_goff;
    const TA* W = (const TA*)a.W + (int64_t)g * a.w_gstride;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    // loader mapping: 256 threads x 4 elements = a 64 x 16 tile; thread -> (row = tid / 4, k = (tid % 4) * 4 ..)
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    int64_t a_row = -1;
    if (m0 + lr < rows) {
        const int p = row_lo + m0 + lr;
        a_row = a.row_src ? a.row_src[p] : p;
    }
    const int wn = n0 + lr;
    float acc[4][4] = {}, acc2[DUAL ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < a.K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            As[lk + i][lr] = (a_row >= 0 && k < a.K) ? to_f32(A[a_row * a.lda + k]) : 0.f;
            Ws[0][lk + i][lr] = (wn < a.N && k < a.K) ? to_f32(W[(int64_t)wn * a.ldw + k]) : 0.f;
            if (DUAL) Ws[DUAL ? 1 : 0][lk + i][lr] = (wn < a.N && k < a.K) ? to_f32(W[(int64_t)(a.N + wn) * a.ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[4], wv[4], wv2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[k][ty * 4 + i]; wv[i] = Ws[0][k][tx * 4 + i]; }
            if (DUAL) {
#pragma unroll
                for (int i = 0; i < 4; ++i) wv2[i] = Ws[DUAL ? 1 : 0][k][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
                    if (DUAL) acc2[DUAL ? i : 0][j] = fmaf(av[i], wv2[j], acc2[DUAL ? i : 0][j]);
                }
        }
        __syncthreads();
    }
    TC* C = (TC*)a.C + (int64_t)g * a.c_goff;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            const float v = finish<DUAL>(a, acc[i][j], acc2[DUAL ? i : 0][j], g, row_lo + m, n);
            C[(int64_t)(row_lo + m) * a.ldc + n] = from_f32<TC>(v);
        }
    }
}

// ------------------------------------------------------------------------------------------------ bf16 tensor cores
// 128 x 64 output tile per block of 256 threads (8 warps: 4 along m x 2 along n, 32 x 32 each), k in steps of 32
// through a two-stage shared-memory ring filled with 16-byte loads.  Rows are padded to 40 halves so that the
// fragment loads of a warp hit distinct banks.
constexpr int TM = 128, TN = 64, TK = 32, TKP = TK + 8;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename TC, bool DUAL>
__global__ void __launch_bounds__(256) gemm_mma_kernel(GemmArgs a) {
    __shared__ __align__(16) __nv_bfloat16 As[2][TM][TKP];
    __shared__ __align__(16) __nv_bfloat16 Ws[2][DUAL ? 2 : 1][TN][TKP];
    const int g = blockIdx.z;
    int row_lo = 0, rows = a.M;
    if (a.grp_off != nullptr) { row_lo = a.grp_off[g]; rows = a.grp_off[g + 1] - row_lo; }
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    if (m0 >= rows) return;
    const __nv_bfloat16* A = (const __nv_bfloat16*)a.A + (int64_t)g * a.a_goff;
    const __nv_bfloat16* W = (const __nv_bfloat16*)a.W + (int64_t)g * a.w_gstride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = (warp & 3) * 32, wn = (warp >> 2) * 32;
    // loaders: A tile 128 rows x 4 16-byte pieces = 512 pieces, two per thread; W tile 64 x 4 = 256, one per thread
    const int pr = tid >> 2, pc = (tid & 3) * 8;
    int64_t arow[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = pr + 64 * i;
        arow[i] = -1;
        if (m0 + r < rows) {
            const int p = row_lo + m0 + r;
            arow[i] = a.row_src ? a.row_src[p] : p;
        }
    }
    const bool wok = n0 + pr < a.N;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 ra[2], rw[2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
            ra[i] = arow[i] >= 0 ? *reinterpret_cast<const uint4*>(A + arow[i] * a.lda + k0 + pc) : zero;
        rw[0] = wok ? *reinterpret_cast<const uint4*>(W + (int64_t)(n0 + pr) * a.ldw + k0 + pc) : zero;
        if (DUAL) rw[1] = wok ? *reinterpret_cast<const uint4*>(W + (int64_t)(a.N + n0 + pr) * a.ldw + k0 + pc) : zero;
    };
    auto stash = [&](int s) {
#pragma unroll
        for (int i = 0; i < 2; ++i) *reinterpret_cast<uint4*>(&As[s][pr + 64 * i][pc]) = ra[i];
        *reinterpret_cast<uint4*>(&Ws[s][0][pr][pc]) = rw[0];
        if (DUAL) *reinterpret_cast<uint4*>(&Ws[s][DUAL ? 1 : 0][pr][pc]) = rw[1];
    };
    float acc[2][4][4] = {}, acc2[DUAL ? 2 : 1][4][4] = {};
    const int nk = a.K / TK;           // the host routes K % 32 != 0 to the SIMT kernel
    fetch(0);
    stash(0);
    __syncthreads();
    const int gr = lane >> 2, gc = (lane & 3) * 2;
    for (int kt = 0; kt < nk; ++kt) {
        const int s = kt & 1;
        if (kt + 1 < nk) fetch((kt + 1) * TK);
#pragma unroll
        for (int kk = 0; kk < TK; kk += 16) {
            uint32_t af[2][4], bf[4][2], bf2[4][2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = wm + 16 * i + gr;
                af[i][0] = *reinterpret_cast<const uint32_t*>(&As[s][r][kk + gc]);
                af[i][1] = *reinterpret_cast<const uint32_t*>(&As[s][r + 8][kk + gc]);
                af[i][2] = *reinterpret_cast<const uint32_t*>(&As[s][r][kk + gc + 8]);
                af[i][3] = *reinterpret_cast<const uint32_t*>(&As[s][r + 8][kk + gc + 8]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = wn + 8 * j + gr;
                bf[j][0] = *reinterpret_cast<const uint32_t*>(&Ws[s][0][n][kk + gc]);
                bf[j][1] = *reinterpret_cast<const uint32_t*>(&Ws[s][0][n][kk + gc + 8]);
                if (DUAL) {
                    bf2[j][0] = *reinterpret_cast<const uint32_t*>(&Ws[s][DUAL ? 1 : 0][n][kk + gc]);
                    bf2[j][1] = *reinterpret_cast<const uint32_t*>(&Ws[s][DUAL ? 1 : 0][n][kk + gc + 8]);
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    mma_bf16(acc[i][j], af[i], bf[j]);
                    if (DUAL) mma_bf16(acc2[DUAL ? i : 0][j], af[i], bf2[j]);
                }
        }
        if (kt + 1 < nk) {
            stash(s ^ 1);            // the other stage was last read before the barrier that ended step kt - 1
            __syncthreads();
        }
    }
    TC* C = (TC*)a.C + (int64_t)g * a.c_goff;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int m = m0 + wm + 16 * i + gr + (e >> 1) * 8, n = n0 + wn + 8 * j + gc + (e & 1);
                if (m >= rows || n >= a.N) continue;
                const float v = finish<DUAL>(a, acc[i][j][e], acc2[DUAL ? i : 0][j][e], g, row_lo + m, n);
                C[(int64_t)(row_lo + m) * a.ldc + n] = from_f32<TC>(v);
            }
}

// ------------------------------------------------------------------------------------------------ few rows (decode)
// Up to 16 activation rows per group: the product is a stream over the weights.  A warp owns four weight rows (with
// DUAL: the gate and up rows of two outputs) and walks k with one 16-byte load per lane and row, every row's load in
// flight at once; the few activation rows come through L1.  Lanes keep fp32 partial sums per (weight row, activation
// row) and a shuffle tree adds them at the end.  A group without rows returns before touching its weights, so a decode
// step reads only the experts that were chosen.
constexpr int SK_ROWS = 4, SK_WARPS = 4;

__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename TC, bool DUAL, int MT>
__global__ void __launch_bounds__(32 * SK_WARPS) gemm_skinny_kernel(GemmArgs a) {
    const int g = blockIdx.z;
    int row_lo = 0, rows = a.M;
    if (a.grp_off != nullptr) { row_lo = a.grp_off[g]; rows = a.grp_off[g + 1] - row_lo; }
    const int m0 = blockIdx.y * MT;
    if (m0 >= rows) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int OUTS = DUAL ? SK_ROWS / 2 : SK_ROWS;           // outputs per warp
    const int n0 = (blockIdx.x * SK_WARPS + warp) * OUTS;
    if (n0 >= a.N) return;
    const __nv_bfloat16* A = (const __nv_bfloat16*)a.A + (int64_t)g * a.a_goff;
    const __nv_bfloat16* W = (const __nv_bfloat16*)a.W + (int64_t)g * a.w_gstride;
    const __nv_bfloat16* wrow[SK_ROWS];
#pragma unroll
    for (int i = 0; i < SK_ROWS; ++i) {
        int n = DUAL ? (n0 + (i >> 1)) : (n0 + i);
        n = min(n, a.N - 1);                                      // a tail warp recomputes the last row; it is not stored
        wrow[i] = W + (int64_t)(DUAL ? ((i & 1) * a.N + n) : n) * a.ldw;
    }
    const __nv_bfloat16* arow[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const int p = row_lo + min(m0 + m, rows - 1);
        arow[m] = A + (int64_t)(a.row_src ? a.row_src[p] : p) * a.lda;
    }
    float acc[SK_ROWS][MT] = {};
    for (int k = lane * 8; k < a.K; k += 256) {
        uint4 wv[SK_ROWS];
#pragma unroll
        for (int i = 0; i < SK_ROWS; ++i) wv[i] = __ldg(reinterpret_cast<const uint4*>(wrow[i] + k));
        float wf[SK_ROWS][8];
#pragma unroll
        for (int i = 0; i < SK_ROWS; ++i) bf16x8_to_f32(wv[i], wf[i]);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float af[8];
            bf16x8_to_f32(*reinterpret_cast<const uint4*>(arow[m] + k), af);
#pragma unroll
            for (int i = 0; i < SK_ROWS; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i][m] = fmaf(af[e], wf[i][e], acc[i][m]);
        }
    }
#pragma unroll
    for (int i = 0; i < SK_ROWS; ++i)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc[i][m] += __shfl_xor_sync(0xffffffffu, acc[i][m], o);
    TC* C = (TC*)a.C + (int64_t)g * a.c_goff;
    if (lane == 0) {
#pragma unroll
        for (int o = 0; o < OUTS; ++o) {
            if (n0 + o >= a.N) continue;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m0 + m >= rows) continue;
                const float v = finish<DUAL>(a, DUAL ? acc[2 * o][m] : acc[o][m], acc[DUAL ? 2 * o + 1 : o][m], g, row_lo + m0 + m, n0 + o);
                C[(int64_t)(row_lo + m0 + m) * a.ldc + n0 + o] = from_f32<TC>(v);
            }
        }
    }
}

template <typename TC>
static void launch_skinny(const GemmArgs& a, int groups, bool dual, cudaStream_t st) {
    const int outs_per_block = SK_WARPS * (dual ? SK_ROWS / 2 : SK_ROWS);
    const int mt = a.M <= 1 ? 1 : (a.M <= 2 ? 2 : (a.M <= 4 ? 4 : 8));
    const dim3 grid((a.N + outs_per_block - 1) / outs_per_block, (a.M + mt - 1) / mt, groups), block(32 * SK_WARPS);
#define UMBS_SK(MT)                                                                   \
    do {                                                                              \
        if (dual) gemm_skinny_kernel<TC, true, MT><<<grid, block, 0, st>>>(a);        \
        else gemm_skinny_kernel<TC, false, MT><<<grid, block, 0, st>>>(a);            \
    } while (0)
    if (mt == 1) UMBS_SK(1);
    else if (mt == 2) UMBS_SK(2);
    else if (mt == 4) UMBS_SK(4);
    else UMBS_SK(8);
#undef UMBS_SK
}

template <typename TA, typename TC>
static void launch_simt(const GemmArgs& a, int groups, bool dual, cudaStream_t st) {
    const dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM, groups);
    if (dual) gemm_simt_kernel<TA, TC, true><<<grid, 256, 0, st>>>(a);
    else gemm_simt_kernel<TA, TC, false><<<grid, 256, 0, st>>>(a);
}
template <typename TC>
static void launch_mma(const GemmArgs& a, int groups, bool dual, cudaStream_t st) {
    const dim3 grid((a.N + TN - 1) / TN, (a.M + TM - 1) / TM, groups);
    if (dual) gemm_mma_kernel<TC, true><<<grid, 256, 0, st>>>(a);
    else gemm_mma_kernel<TC, false><<<grid, 256, 0, st>>>(a);
}

}  // namespace umbs

using namespace umbs;

static int gemm_run(int dtype, const void* A, int64_t lda, int a_goff, const void* W, int64_t ldw, int64_t w_gstride,
                    void* C, int64_t ldc, int c_goff, int c_f32, int M, int N, int K, int groups,
                    const int32_t* grp_off, const int32_t* row_src, int dual, float limit, const float* bias,
                    const float* out_gate, int64_t ld_gate, int gate_goff, int unary, float p0, float p1, umbs_stream_t stream);

extern "C" int umbs_gemm(int dtype, const void* A, int64_t lda, int a_goff, const void* W, int64_t ldw, int64_t w_gstride,
                         void* C, int64_t ldc, int c_goff, int c_f32, int M, int N, int K, int groups,
                         const int32_t* grp_off, const int32_t* row_src, int dual, float limit, umbs_stream_t stream) {
    return umbs_gemm_ex(dtype, A, lda, a_goff, W, ldw, w_gstride, C, ldc, c_goff, c_f32, M, N, K, groups, grp_off, row_src, dual,
                        limit, nullptr, nullptr, 0, 0, stream);
}

extern "C" int umbs_gemm_ex(int dtype, const void* A, int64_t lda, int a_goff, const void* W, int64_t ldw, int64_t w_gstride,
                            void* C, int64_t ldc, int c_goff, int c_f32, int M, int N, int K, int groups,
                            const int32_t* grp_off, const int32_t* row_src, int dual, float limit, const float* bias,
                            const float* out_gate, int64_t ld_gate, int gate_goff, umbs_stream_t stream) {
    return gemm_run(dtype, A, lda, a_goff, W, ldw, w_gstride, C, ldc, c_goff, c_f32, M, N, K, groups, grp_off, row_src, dual, limit,
                    bias, out_gate, ld_gate, gate_goff, 0, 0.f, 0.f, stream);
}

extern "C" int umbs_gemm_unary(int dtype, const void* A, int64_t lda, int a_goff, const void* W, int64_t ldw, int64_t w_gstride,
                               void* C, int64_t ldc, int c_goff, int c_f32, int M, int N, int K, int groups, const float* bias,
                               int unary, float p0, float p1, umbs_stream_t stream) {
    if (unary != 0 && unary != UMBS_UNARY_TANH && unary != UMBS_UNARY_XIELU) return UMB_ERR_ARG;
    return gemm_run(dtype, A, lda, a_goff, W, ldw, w_gstride, C, ldc, c_goff, c_f32, M, N, K, groups, nullptr, nullptr, 0, 0.f, bias,
                    nullptr, 0, 0, unary, p0, p1, stream);
}

static int gemm_run(int dtype, const void* A, int64_t lda, int a_goff, const void* W, int64_t ldw, int64_t w_gstride,
                    void* C, int64_t ldc, int c_goff, int c_f32, int M, int N, int K, int groups,
                    const int32_t* grp_off, const int32_t* row_src, int dual, float limit, const float* bias,
                    const float* out_gate, int64_t ld_gate, int gate_goff, int unary, float p0, float p1, umbs_stream_t stream) {
    if (M <= 0 || N <= 0 || groups <= 0) return 0;
    if (K <= 0 || A == nullptr || W == nullptr || C == nullptr) return UMB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    GemmArgs a{A, lda, a_goff, W, ldw, w_gstride, C, ldc, c_goff, M, N, K, grp_off, row_src, limit,
               (dual == UMBS_ACT_GELU_TANH || dual == UMBS_ACT_SILU) ? dual : UMBS_ACT_CLAMPED_GLU,
               bias, out_gate, ld_gate, gate_goff, unary, p0, p1};
    if (dtype == UMBS_F32) {
        launch_simt<float, float>(a, groups, dual != 0, st);          // activations are fp32 too: c_f32 changes nothing
    } else if (dtype == UMBS_BF16) {
        // 16-byte loads: every row start and group offset must sit on a 16-byte boundary
        const bool vec = (K % 8 == 0) && (lda % 8 == 0) && (ldw % 8 == 0) && (a_goff % 8 == 0) && (w_gstride % 8 == 0) &&
                         ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
        const bool tc = vec && (K % TK == 0);
        if (vec && M <= 16) {
            if (c_f32) launch_skinny<float>(a, groups, dual != 0, st);
            else launch_skinny<__nv_bfloat16>(a, groups, dual != 0, st);
        } else if (tc) {
            if (c_f32) launch_mma<float>(a, groups, dual != 0, st);
            else launch_mma<__nv_bfloat16>(a, groups, dual != 0, st);
        } else {
            if (c_f32) launch_simt<__nv_bfloat16, float>(a, groups, dual != 0, st);
            else launch_simt<__nv_bfloat16, __nv_bfloat16>(a, groups, dual != 0, st);
        }
    } else {
        return UMB_ERR_ARG;
    }
    count_launches(1);
    return (int)cudaGetLastError();
}
