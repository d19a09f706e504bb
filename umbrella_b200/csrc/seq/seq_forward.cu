// umbs_forward: one batched step of a sequence-state decoder -- the chain of launches for every layer, enqueued on
// the caller's stream from one C call, over a workspace carved up here.
#include <atomic>
#include <cuda_runtime.h>
#include <stdint.h>
#include <vector>

#include "seq_internal.h"

namespace umbs {
static std::atomic<unsigned long long> g_launches{0};
void count_launches(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

struct Arena {
    char* base;
    size_t used, cap;
    void* take(size_t bytes) {
        used = (used + 255) & ~(size_t)255;
        void* p = base ? base + used : nullptr;
        used += bytes;
        return p;
    }
};

struct Scratch {
    float* stack;      // [L + 1, T, width]   X_0 .. X_L
    float* x;          // [T, width]          what the next layer reads (depth-mixed)
    void* h;           // act [T, width]
    void* hs;          // act [T, width]
    float* proj;       // fp32 [T, max in-projection rows]
    float* o32;        // fp32 [T, max(heads vdim)]  retention outputs before the gate
    float* rot;        // fp32 [T, max rot_dims]     the step's cos | sin table
    float* seg;        // fp32 segment states of a retention step cut into segments
    size_t seg_bytes;
    void* mixed;       // act [T, max(heads vdim)]   mixer output before W_o
    void* cq;          // act [T, max q_rank]
    void* c;           // act [T, max kv_rank]
    void* q;           // act [T, max heads dim]
    float* q_abs;      // fp32 [T, max heads kv_rank]
    void* o_lat;       // act [T, max heads kv_rank]
    void* kv;          // act [T, max heads (dim + vdim)]  per-head keys | values of a step of fresh sequences
    float* la_part;    // fp32 [512 (tokens x splits), max heads, max kv_rank + 2]  key-split partial states of decode steps
    size_t la_part_bytes;
    float* mix_out;    // fp32 [T, width]
    float* sel_w;      // fp32 [T, max top]
    int32_t* grp_off;  // [max experts + 1]
    int32_t* pair_tok; // [T max top]
    int32_t* pair_pos; // [T max top]
    int32_t* route_scratch;   // [2 max experts + T max top]
    void* y;           // act [T max top, max ff]
    float* pair_out;   // fp32 [T max top, width]
    void* ys;          // act [T, max shared ff]
    float* shared_out; // fp32 [T, width]
    void* final_h;     // act [n_want, width]
    float* gates;      // fp32 [T, max heads, 3]           mlstm: decay, input weight, floor per (token, head)
    float* ca_part;    // fp32 key-split partial sums of cached attention in decode steps
    size_t ca_part_bytes;
    float* sgate;      // fp32 [T]  the shared expert's factor per token
    float* raw;        // fp32 [T, max heads maps value_heads vdim]  attention outputs in front of umbs_attention_finish
    void* mixes;       // act [T, 5, width]  token-shifted mixes of a time-mix layer
    void* lowrank;     // act [T, max decay_rank]
    float* wraw;       // fp32 [T, max heads dim]  the decay before its exponentials
    float* mix_out2;   // fp32 [T, width]  a second mixer's output
    std::vector<void*> kv_rows;   // per layer: the step's key | value rows (a buffer of its own for a layer others borrow from)
};

// layer j lends its keys and values to a later layer
static bool lends_kv(const umbs_model_t* m, int j) {
    for (int i = j + 1; i < m->n_layers; ++i) {
        if (m->layers[i].kv_from == j + 1) return true;
        if (m->layers[i].second != nullptr && m->layers[i].second->kv_from == j + 1) return true;
    }
    return false;
}

static size_t carve(const umbs_model_t* m, int T, int n_want, char* base, Scratch* s) {
    const size_t es = m->dtype == UMBS_F32 ? 4 : 2;
    size_t segb = 0;
    int hmax = 1, rotd = 1, in_rows = 1, hv = 1, qr = 1, kvr = 1, hd = 1, hkv = 1, hkvw = 1, top = 1, experts = 1, ff = 1, sff = 1;
    int hall = 1, cav = 1, rawd = 1, n_mix = 0, rank = 1, tmhd = 1;
    bool parallel = false, two = false;
    auto up = [](int& a, int b) { if (b > a) a = b; };
    for (int i = 0; i < m->n_layers; ++i)
        if (m->layers[i].form == UMBS_FORM_PARALLEL) parallel = true;
    for (int u = 0; u < 2 * m->n_layers; ++u) {            // every layer's mixer, then its second one
        const int i = u >> 1;
        if ((u & 1) && m->layers[i].second == nullptr) continue;
        const umbs_layer_t& l = (u & 1) ? *m->layers[i].second : m->layers[i];
        if (u & 1) two = true;
        up(hv, l.heads * l.vdim);
        up(hall, l.heads);
        if (l.mixer == UMBS_MIX_CACHED_ATTENTION) {
            const int gate_rows = l.gate_kind == 1 ? l.heads : (l.gate_kind == 2 ? l.heads * l.vdim : 0);
            const int M = l.maps > 1 ? l.maps : 1;
            up(in_rows, l.heads * M * l.dim + l.kv_heads * M * l.dim + (l.values_are_keys ? 0 : l.kv_heads * l.vdim) + gate_rows);
            up(hd, l.heads * M * l.dim); up(hkvw, l.kv_heads * (M * l.dim + l.vdim)); up(cav, l.vdim);
            up(rawd, l.heads * M * (l.talk != nullptr ? l.kv_heads : 1) * l.vdim);
        } else if (l.mixer == UMBS_MIX_TIME_MIX) {
            up(in_rows, 4 * l.heads * l.dim); up(rank, l.decay_rank); up(tmhd, l.heads * l.dim);
            n_mix = 5;
        } else if (l.mixer == UMBS_MIX_MLSTM) {
            up(in_rows, 2 * l.heads * l.dim + 2 * l.heads * l.vdim + 2 * l.heads);
            up(hv, l.heads * (l.vdim + 1));                        // o32 holds n . q as one more column per head
            // segment states (and decay products) of a step of few long sequences: about 592 blocks' worth
            const size_t plane = (size_t)l.heads * ((size_t)l.dim * (l.vdim + 1) + 1) * 4, ent = 592 / ((size_t)l.heads * ((l.vdim + 32) / 32)) + 8;
            if (T >= 128 && ent * plane > segb) segb = ent * plane;
        } else if (l.mixer == UMBS_MIX_RETENTION) {
            up(in_rows, 2 * l.heads * l.dim + 2 * l.heads * l.vdim); up(rotd, l.rot_dims);
            // segment states of a step of few long sequences: about 592 blocks' worth (umbs_retention uses what fits)
            const size_t plane = (size_t)l.heads * l.dim * l.vdim * 4, ent = 592 / ((size_t)l.heads * ((l.vdim + 31) / 32)) + 8;
            if (T >= 128 && ent * plane > segb) segb = ent * plane;
        }
        else {
            // (direct queries: q rows | latent | shared key part | gate rows; keys and queries carry rope_dim more numbers)
            const int gate_rows = l.gate_kind == 2 ? l.heads * l.vdim : 0;
            up(in_rows, l.q_rank > 0 ? l.q_rank + l.kv_rank : l.heads * (l.dim + l.rope_dim) + l.kv_rank + l.rope_dim + gate_rows);
            up(hmax, l.heads); up(qr, l.q_rank); up(kvr, l.kv_rank + l.rope_dim); up(hd, l.heads * (l.dim + l.rope_dim));
            up(hkv, l.heads * (l.kv_rank + l.rope_dim));
            if (l.w_ukv != nullptr) up(hkvw, l.heads * (l.dim + l.rope_dim + l.vdim));
        }
        if (!(u & 1) && l.has_mlp) { up(top, l.mlp.top); up(experts, l.mlp.experts); up(ff, l.mlp.ff); up(sff, l.mlp.shared_ff); }
    }
    Arena a{base, 0, 0};
    const size_t W = m->width, Tz = T;
    Scratch z;
    z.stack = (float*)a.take((size_t)(parallel ? m->n_layers + 1 : 1) * Tz * W * 4);   // pre-norm layers keep one residual stream
    z.x = (float*)a.take(Tz * W * 4);
    z.h = a.take(Tz * W * es);
    z.hs = a.take(Tz * W * es);
    z.proj = (float*)a.take(Tz * in_rows * 4);
    z.o32 = (float*)a.take(Tz * hv * 4);
    z.rot = (float*)a.take(Tz * rotd * 4);
    z.seg_bytes = segb;
    z.seg = (float*)a.take(segb);
    z.mixed = a.take(Tz * hv * es);
    z.cq = a.take(Tz * qr * es);
    z.c = a.take(Tz * kvr * es);
    z.q = a.take(Tz * hd * es);
    z.q_abs = (float*)a.take(Tz * hkv * 4);
    z.o_lat = a.take(Tz * hkv * es);
    z.kv = a.take(Tz * hkvw * es);
    z.la_part_bytes = (size_t)512 * ((size_t)hkv + 2 * (size_t)hmax) * 4;      // tokens x splits <= 512
    z.la_part = (float*)a.take(z.la_part_bytes);
    z.mix_out = (float*)a.take(Tz * W * 4);
    z.sel_w = (float*)a.take(Tz * top * 4);
    z.grp_off = (int32_t*)a.take((size_t)(experts + 1) * 4);
    z.pair_tok = (int32_t*)a.take(Tz * top * 4);
    z.pair_pos = (int32_t*)a.take(Tz * top * 4);
    z.route_scratch = (int32_t*)a.take((2 * (size_t)experts + Tz * top) * 4);
    z.y = a.take(Tz * top * ff * es);
    z.pair_out = (float*)a.take(Tz * top * W * 4);
    z.ys = a.take(Tz * sff * es);
    z.shared_out = (float*)a.take(Tz * W * 4);
    z.final_h = a.take((size_t)(n_want > 0 ? n_want : 1) * W * es);
    z.gates = (float*)a.take(Tz * hall * 3 * 4);
    z.ca_part_bytes = (size_t)2048 * ((size_t)cav + 2) * 4;                 // (token, head, split) triples of a decode step
    z.ca_part = (float*)a.take(z.ca_part_bytes);
    z.sgate = (float*)a.take(Tz * 4);
    z.raw = (float*)a.take(Tz * rawd * 4);
    z.mixes = a.take(Tz * n_mix * W * es);
    z.lowrank = a.take(Tz * rank * es);
    z.wraw = (float*)a.take(Tz * tmhd * 4);
    z.mix_out2 = (float*)a.take(two ? Tz * W * 4 : 0);
    z.kv_rows.assign(m->n_layers, z.kv);
    for (int i = 0; i < m->n_layers; ++i) {
        const umbs_layer_t& l = m->layers[i];
        if (l.mixer == UMBS_MIX_CACHED_ATTENTION && lends_kv(m, i))
            z.kv_rows[i] = a.take(Tz * l.kv_heads * ((l.maps > 1 ? l.maps : 1) * l.dim + l.vdim) * es);
    }
    if (s) *s = z;
    return a.used + 256;
}
}  // namespace umbs

using namespace umbs;

extern "C" const char* umbs_version(void) { return "umbrella_b200_seq 0.1 (sm_100a)"; }
extern "C" unsigned long long umbs_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" size_t umbs_workspace_bytes(const umbs_model_t* model, int max_tokens, int max_want) {
    if (model == nullptr || max_tokens <= 0) return 0;
    return carve(model, max_tokens, max_want, nullptr, nullptr);
}

#define UMBS_TRY(expr) do { int rc__ = (expr); if (rc__ != 0) return rc__; } while (0)

extern "C" int umbs_forward(const umbs_model_t* m, const umbs_batch_t* b, float* logits, float* layer_out, void* workspace,
                            size_t workspace_bytes, umbs_stream_t stream) {
    if (m == nullptr || b == nullptr || workspace == nullptr) return UMB_ERR_ARG;
    const int T = b->n_tokens, W = m->width, dt = m->dtype;
    if (T <= 0) return 0;
    if ((uintptr_t)workspace % 256 != 0) return UMB_ERR_ARG;
    Scratch s;
    if (carve(m, T, b->n_want, (char*)workspace, &s) > workspace_bytes) return UMB_ERR_WORKSPACE;
    const int64_t plane = (int64_t)T * W;
    UMBS_TRY(umbs_embedding_pos(dt, b->tok_ids, b->tok_pos, m->embed, m->embed_scale != 0.f ? m->embed_scale : 1.f, m->pos_freq,
                                s.stack, T, W, stream));
    const float* x = s.stack;                    // layer 0 reads X_0 itself
    bool prenorm = false;
    for (int i = 0; i < m->n_layers; ++i) {
        if (i > 0 && m->layers[i].form != m->layers[0].form) return UMB_ERR_UNSUPPORTED;    // one form per model
        prenorm = m->layers[i].form == UMBS_FORM_PRENORM;
    }
    // Pre-norm layers: one fp32 residual stream, updated in place.  Every block's output waits in `pending` and is added
    // by the kernel that computes the next norm (or, behind the last layer, by the final norm).
    umbs_delta_t pend{};
    bool has_pend = false;
    // the residual add + norm in front of a block: the plain RMS kernel where nothing else is asked for
    auto norm_step = [&](const int32_t* rows, int n, int kind, const float* w, const float* bias, float off, float alpha,
                         void* y, float* copy) -> int {
        const bool plain = kind == UMBS_NORM_RMS && (!has_pend || (pend.pair_out == nullptr && pend.shared == nullptr &&
                                                                   pend.scale == nullptr && pend.mult == 1.f &&
                                                                   pend.delta2 == nullptr && (pend.delta_mult == 0.f || pend.delta_mult == 1.f)));
        if (plain) return umbs_add_rms_norm(dt, s.stack, has_pend ? pend.delta : nullptr, rows, n, w, off, W, m->norm_eps, y, copy, stream);
        return umbs_add_norm_ex(dt, s.stack, has_pend ? &pend : nullptr, rows, n, kind, w, bias, off, alpha, W, m->norm_eps, y, copy,
                                stream);
    };
    // One mixer of a pre-norm layer: from the normed rows s.h to its output, fp32 [T, width] at `out`.  li: the layer's index.
    auto run_mixer = [&](const umbs_layer_t& l, int li, float* out) -> int {
        const int hv = l.heads * l.vdim;
        if (l.mixer == UMBS_MIX_CACHED_ATTENTION) {
            const int M = l.maps > 1 ? l.maps : 1;
            const bool borrowed = l.kv_from > 0;
            const int src = borrowed ? l.kv_from - 1 : li;
            if (borrowed && (src >= li || m->layers[src].mixer != UMBS_MIX_CACHED_ATTENTION || m->layers[src].kv_from > 0 ||
                             l.values_are_keys || l.taps > 1 || l.pool > 0))
                return UMB_ERR_UNSUPPORTED;
            const int cq = l.heads * M * l.dim, ck = borrowed ? 0 : l.kv_heads * M * l.dim;
            const int cv = (borrowed || l.values_are_keys) ? 0 : l.kv_heads * l.vdim;
            const int gate_rows = l.gate_kind == 1 ? l.heads : (l.gate_kind == 2 ? hv : 0);
            const int rows = cq + ck + cv + gate_rows, row_kv = l.kv_heads * (M * l.dim + l.vdim);
            void* kv_rows = s.kv_rows[src];
            const float* gate = gate_rows ? s.proj + cq + ck + cv : nullptr;
            UMBS_TRY(umbs_gemm(dt, s.h, W, 0, l.w_in, W, 0, s.proj, rows, 0, 1, T, rows, W, 1, nullptr, nullptr, 0, 0.f, stream));
            UMBS_TRY(umbs_attention_prep_ex(dt, s.proj, rows, l.bias_in, b, l.heads, borrowed ? 0 : l.kv_heads, l.dim, l.vdim,
                                            l.values_are_keys, l.taps, l.conv_w, l.conv_state, m->slots, l.rot_dims, l.inv_freq,
                                            l.rot_mag, M, l.q_norm_w, l.k_norm_w, m->norm_eps, s.q, borrowed ? nullptr : kv_rows,
                                            stream));
            if (l.pool > 0)
                UMBS_TRY(umbs_kv_pool(dt, kv_rows, l.kv_cache, l.kv_len, l.pool_cache, l.pool_len, b, row_kv, l.pool, stream));
            const bool finish = l.talk != nullptr || M > 1 || l.head_unit_norm || (l.out_mult != 0.f && l.out_mult != 1.f);
            if (finish && l.gate_kind == 1) return UMB_ERR_UNSUPPORTED;
            umbs_attn_opts_t opts{};
            opts.softcap = l.softcap; opts.dist_r1 = l.dist_r1; opts.dist_r2 = l.dist_r2; opts.chunk = l.chunk; opts.maps = M;
            opts.value_heads = l.talk != nullptr ? l.kv_heads : 1;
            opts.raw_out = finish ? s.raw : nullptr;
            UMBS_TRY(umbs_cached_attention_ex(dt, l.attn_mode, s.q, kv_rows, l.kv_cache, l.kv_len, l.pool_cache, l.pool_len, b,
                                              l.heads, l.kv_heads, l.dim, l.vdim, l.window, l.pool, l.scale, l.head_bias,
                                              finish ? nullptr : gate, rows, l.gate_kind == 1, &opts, s.ca_part, s.ca_part_bytes,
                                              s.mixed, stream));
            if (finish)
                UMBS_TRY(umbs_attention_finish(dt, s.raw, T, l.heads, l.kv_heads, l.vdim, M, opts.value_heads, l.talk, l.diff_lambda,
                                               l.head_unit_norm, m->norm_eps, l.out_mult, gate, rows, s.mixed, stream));
            if (!borrowed && !lends_kv(m, li))           // (a lender's rows go to its cache after its last borrower has run)
                UMBS_TRY(umbs_ring_append(dt, kv_rows, l.kv_cache, l.kv_len, b, row_kv, stream));
        } else if (l.mixer == UMBS_MIX_TIME_MIX) {
            const int hd = l.heads * l.dim, rows = 4 * hd;
            const size_t es = dt == UMBS_F32 ? 4 : 2;
            if (l.vdim != l.dim || l.mix_mu == nullptr || l.shift_state == nullptr || l.decay_rank < 1) return UMB_ERR_ARG;
            UMBS_TRY(umbs_shift_mix(dt, s.h, l.mix_mu, 5, l.shift_state, m->slots, b, W, s.mixes, stream));
            // r | k | v | g: one batched product over the first four mixes
            UMBS_TRY(umbs_gemm(dt, s.mixes, (int64_t)5 * W, W, l.w_in, W, (int64_t)hd * W, s.proj, rows, hd, 1, T, hd, W, 4, nullptr,
                               nullptr, 0, 0.f, stream));
            // the decay's low-rank map of the fifth mix, tanh in the first product's epilogue
            UMBS_TRY(umbs_gemm_unary(dt, (const char*)s.mixes + (size_t)4 * W * es, (int64_t)5 * W, 0, l.w_decay1, W, 0, s.lowrank,
                                     l.decay_rank, 0, 0, T, l.decay_rank, W, 1, nullptr, UMBS_UNARY_TANH, 0.f, 0.f, stream));
            UMBS_TRY(umbs_gemm(dt, s.lowrank, l.decay_rank, 0, l.w_decay2, l.decay_rank, 0, s.wraw, hd, 0, 1, T, hd, l.decay_rank, 1,
                               nullptr, nullptr, 0, 0.f, stream));
            UMBS_TRY(umbs_time_mix(dt, s.proj, rows, s.wraw, l.decay_bias, l.bonus, b, l.heads, l.dim, m->norm_eps, l.out_norm_w,
                                   l.tm_state, s.o32, s.mixed, stream));
        } else {
            return UMB_ERR_UNSUPPORTED;
        }
        return umbs_gemm(dt, s.mixed, hv, 0, l.w_o, hv, 0, out, W, 0, 1, T, W, hv, 1, nullptr, nullptr, 0, 0.f, stream);
    };
    for (int i = 0; prenorm && i < m->n_layers; ++i) {
        const umbs_layer_t& l = m->layers[i];
        const int hv = l.heads * l.vdim;
        const float mult = l.residual_mult != 0.f ? l.residual_mult : 1.f;
        UMBS_TRY(norm_step(nullptr, T, l.norm_kind, l.norm_w, l.norm_b, l.norm_offset, l.norm_alpha, s.h,
                           (layer_out && i > 0) ? layer_out + (int64_t)(i - 1) * plane : nullptr));
        const bool generic = l.mixer == UMBS_MIX_CACHED_ATTENTION || l.mixer == UMBS_MIX_TIME_MIX;
        if (generic) {
            UMBS_TRY(run_mixer(l, i, s.mix_out));
            if (l.second != nullptr) UMBS_TRY(run_mixer(*l.second, i, s.mix_out2));
            // rows a layer lent out go to its cache once its last borrower has run
            for (int j = 0; j <= i; ++j) {
                const umbs_layer_t& lj = m->layers[j];
                if (lj.mixer != UMBS_MIX_CACHED_ATTENTION || lj.kv_from > 0 || !lends_kv(m, j)) continue;
                int last = j;
                for (int k = j + 1; k < m->n_layers; ++k)
                    if (m->layers[k].kv_from == j + 1 || (m->layers[k].second && m->layers[k].second->kv_from == j + 1)) last = k;
                if (last == i)
                    UMBS_TRY(umbs_ring_append(dt, s.kv_rows[j], lj.kv_cache, lj.kv_len, b,
                                              lj.kv_heads * ((lj.maps > 1 ? lj.maps : 1) * lj.dim + lj.vdim), stream));
            }
        } else if (l.mixer == UMBS_MIX_MLSTM) {
            const int rows = 2 * l.heads * l.dim + 2 * hv + 2 * l.heads;
            UMBS_TRY(umbs_gemm(dt, s.h, W, 0, l.w_in, W, 0, s.proj, rows, 0, 1, T, rows, W, 1, nullptr, nullptr, 0, 0.f, stream));
            UMBS_TRY(umbs_mlstm(dt, s.proj, rows, l.bias_in, b, l.heads, l.dim, l.vdim, l.gate_cap, m->norm_eps, l.out_norm_w,
                                l.mlstm_state, s.gates, s.o32, s.seg_bytes ? s.seg : nullptr, s.seg_bytes, s.mixed, stream));
        } else if (l.mixer == UMBS_MIX_LATENT_ATTENTION) {
            // direct queries, keys through one normed latent per token plus a rotated part all heads share
            if (l.q_rank != 0 || l.gate_kind == 1 || l.w_ukT == nullptr || l.w_uv == nullptr) return UMB_ERR_UNSUPPORTED;
            const int Rt = l.rope_dim, hd1 = l.dim + Rt, hdq = l.heads * hd1, R = l.kv_rank, KD = R + Rt;
            const int gate_rows = l.gate_kind == 2 ? hv : 0, rows = hdq + KD + gate_rows;
            const float* gate = gate_rows ? s.proj + hdq + KD : nullptr;
            UMBS_TRY(umbs_gemm(dt, s.h, W, 0, l.w_in, W, 0, s.proj, rows, 0, 1, T, rows, W, 1, nullptr, nullptr, 0, 0.f, stream));
            UMBS_TRY(umbs_latent_prep(dt, s.proj, rows, b, l.heads, l.dim, Rt, R, l.kv_norm, m->norm_eps, l.rot_dims, l.inv_freq,
                                      l.rot_mag, s.q, s.c, s.q_abs + R, KD, stream));
            if (b->max_seq_len > 1 && b->max_pos0 == 0 && l.w_ukv != nullptr && umbs_window_attention_ex_fits(l.dim, Rt, l.vdim)) {
                // a step of fresh sequences: every visible key is in the step, so every head's own key part and its values
                // are up-projected once per token and a (row, key) pair costs dim + rope_dim + vdim multiply-adds
                const int hdk = l.heads * l.dim;
                const size_t es = dt == UMBS_F32 ? 4 : 2;
                UMBS_TRY(umbs_gemm(dt, s.c, KD, 0, l.w_ukv, R, 0, s.kv, hdk + hv, 0, 0, T, hdk + hv, R, 1, nullptr, nullptr, 0, 0.f,
                                   stream));
                UMBS_TRY(umbs_window_attention_ex(dt, s.q, hdq, s.kv, hdk + hv, (const char*)s.c + (size_t)R * es, KD, Rt,
                                                  (const char*)s.kv + (size_t)hdk * es, hdk + hv, b, l.heads, l.dim, l.vdim,
                                                  l.window, l.scale, l.attn_mode, l.sink, gate, rows, s.mixed, hv, stream));
                UMBS_TRY(umbs_ring_append(dt, s.c, l.ring, l.ring_len, b, KD, stream));
            } else {
                // q_abs[t, h, :R] = W_uk[h]^T q[t, h, :dim]: scores against the cached latents need no per-key up-projection;
                // q_abs[t, h, R:] is the head's rotated part, written by the kernel above
                UMBS_TRY(umbs_gemm(dt, s.q, hdq, hd1, l.w_ukT, l.dim, (int64_t)R * l.dim, s.q_abs, (int64_t)l.heads * KD, KD, 1, T,
                                   R, l.dim, l.heads, nullptr, nullptr, 0, 0.f, stream));
                UMBS_TRY(umbs_latent_attention_ex(dt, s.q_abs, s.c, l.ring, l.ring_len, b, l.heads, R, Rt, l.window, l.scale,
                                                  l.attn_mode, l.sink, s.la_part, s.la_part_bytes, s.o_lat, stream));
                UMBS_TRY(umbs_ring_append(dt, s.c, l.ring, l.ring_len, b, KD, stream));
                // values per head from the weighted latents, times the sigmoid output gate
                UMBS_TRY(umbs_gemm_ex(dt, s.o_lat, (int64_t)l.heads * R, R, l.w_uv, R, (int64_t)l.vdim * R, s.mixed, hv, l.vdim, 0,
                                      T, l.vdim, R, l.heads, nullptr, nullptr, 0, 0.f, nullptr, gate, rows, l.vdim, stream));
            }
        } else {
            return UMB_ERR_UNSUPPORTED;
        }
        if (!generic) {
            if (l.second != nullptr) return UMB_ERR_UNSUPPORTED;
            UMBS_TRY(umbs_gemm(dt, s.mixed, hv, 0, l.w_o, hv, 0, s.mix_out, W, 0, 1, T, W, hv, 1, nullptr, nullptr, 0, 0.f, stream));
        }
        pend = umbs_delta_t{};
        pend.delta = s.mix_out; pend.scale = l.out_scale; pend.mult = mult;
        pend.delta_mult = 1.f;
        if (l.second != nullptr) {           // two mixers side by side: both factors as given (0 is a factor like any other)
            pend.delta_mult = l.mix_scale;
            pend.delta2 = s.mix_out2; pend.delta2_mult = l.second_scale;
        }
        has_pend = true;
        if (l.has_mlp) {
            const umbs_mlp_t& f = l.mlp;
            if ((f.experts <= 0 && f.shared_ff <= 0) || l.norm2_w == nullptr) return UMB_ERR_UNSUPPORTED;
            const int act = f.act ? f.act : UMBS_ACT_CLAMPED_GLU;
            UMBS_TRY(norm_step(nullptr, T, l.norm_kind, l.norm2_w, l.norm2_b, l.norm_offset, l.norm2_alpha, s.h, nullptr));
            pend = umbs_delta_t{};
            pend.scale = l.out_scale2; pend.mult = mult;
            if (f.experts > 0) {
                // (the shared expert's per-token gate rides along as one more row of the router)
                UMBS_TRY(umbs_moe_route_scaled(dt, s.h, T, W, f.w_router, f.experts, f.top, f.route_mode, f.groups, f.keep,
                                               f.route_scale, s.sel_w, s.grp_off, s.pair_tok, s.pair_pos, s.route_scratch,
                                               f.shared_ff > 0 ? f.w_shared_gate : nullptr, s.sgate, stream));
                UMBS_TRY(umbs_gemm(dt, s.h, W, 0, f.w_gu, W, (int64_t)2 * f.ff * W, s.y, f.ff, 0, 0, T, f.ff, W, f.experts,
                                   s.grp_off, s.pair_tok, act, f.limit, stream));
                UMBS_TRY(umbs_gemm(dt, s.y, f.ff, 0, f.w_down, f.ff, (int64_t)W * f.ff, s.pair_out, W, 0, 1, T, W, f.ff, f.experts,
                                   s.grp_off, nullptr, 0, 0.f, stream));
                pend.pair_out = s.pair_out; pend.sel_w = s.sel_w; pend.pair_pos = s.pair_pos; pend.top = f.top;
            }
            if (f.shared_ff > 0) {
                if (f.plain)           // no gate rows: the activation of the up product alone, in its epilogue
                    UMBS_TRY(umbs_gemm_unary(dt, s.h, W, 0, f.ws_gu, W, 0, s.ys, f.shared_ff, 0, 0, T, f.shared_ff, W, 1, f.bias_gu,
                                             f.unary, f.unary_p0, f.unary_p1, stream));
                else
                UMBS_TRY(umbs_gemm_ex(dt, s.h, W, 0, f.ws_gu, W, 0, s.ys, f.shared_ff, 0, 0, T, f.shared_ff, W, 1, nullptr, nullptr,
                                      act, f.shared_limit, f.bias_gu, nullptr, 0, 0, stream));
                UMBS_TRY(umbs_gemm_ex(dt, s.ys, f.shared_ff, 0, f.ws_down, f.shared_ff, 0, s.shared_out, W, 0, 1, T, W, f.shared_ff, 1,
                                      nullptr, nullptr, 0, 0.f, f.bias_down, nullptr, 0, 0, stream));
                if (f.w_shared_gate != nullptr && f.experts <= 0) UMBS_TRY(umbs_token_gate(dt, s.h, T, W, f.w_shared_gate, s.sgate, stream));
                if (f.experts > 0 || f.w_shared_gate != nullptr) {
                    pend.shared = s.shared_out;
                    pend.shared_gate = f.w_shared_gate != nullptr ? s.sgate : nullptr;
                } else {
                    pend.delta = s.shared_out;           // a dense feed-forward: the plain pending sum
                }
            }
        }
    }
    if (prenorm) {
        if (layer_out != nullptr) {              // the last layer's stream is asked for: finish the sum for every row
            UMBS_TRY(norm_step(nullptr, T, UMBS_NORM_RMS, nullptr, nullptr, 0.f, 1.f, nullptr, layer_out + (int64_t)(m->n_layers - 1) * plane));
            has_pend = false;
        }
        if (logits != nullptr && b->n_want > 0) {
            UMBS_TRY(norm_step(b->want_rows, b->n_want, m->norm_kind, m->final_norm, m->final_norm_b, m->norm_offset,
                               m->final_norm_alpha, s.final_h, nullptr));
            UMBS_TRY(umbs_gemm(dt, s.final_h, W, 0, m->head, W, 0, logits, m->vocab, 0, 1, b->n_want, m->vocab, W, 1, nullptr,
                               nullptr, 0, 0.f, stream));
            if (m->logit_softcap > 0.f) UMBS_TRY(umbs_softcap(logits, (int64_t)b->n_want * m->vocab, m->logit_softcap, stream));
        }
        return 0;
    }
    for (int i = 0; i < m->n_layers; ++i) {
        const umbs_layer_t& l = m->layers[i];
        UMBS_TRY(umbs_group_norm_shift(dt, x, l.norm_w, l.shift_w, l.shift_state, m->slots, b, W, m->norm_groups,
                                       m->norm_eps, s.h, l.shift_w ? s.hs : s.h, stream));
        const void* hs = l.shift_w ? s.hs : s.h;
        const int hv = l.heads * l.vdim;
        if (l.mixer == UMBS_MIX_RETENTION) {
            const int rows = 2 * l.heads * l.dim + 2 * hv;
            UMBS_TRY(umbs_gemm(dt, hs, W, 0, l.w_in, W, 0, s.proj, rows, 0, 1, T, rows, W, 1, nullptr, nullptr, 0, 0.f, stream));
            UMBS_TRY(umbs_retention(dt, s.proj, rows, b, l.heads, l.dim, l.vdim, l.rot_dims, l.inv_freq, l.decay,
                                    m->norm_eps, l.ret_state, s.o32, s.rot, s.seg_bytes ? s.seg : nullptr, s.seg_bytes, s.mixed, stream));
        } else if (l.mixer == UMBS_MIX_LATENT_ATTENTION) {
            const int rows = l.q_rank + l.kv_rank, hd = l.heads * l.dim, R = l.kv_rank;
            UMBS_TRY(umbs_gemm(dt, hs, W, 0, l.w_in, W, 0, s.proj, rows, 0, 1, T, rows, W, 1, nullptr, nullptr, 0, 0.f, stream));
            UMBS_TRY(umbs_latent_norm(dt, s.proj, T, l.q_rank, R, l.q_norm, l.kv_norm, m->norm_eps, s.cq, s.c, stream));
            UMBS_TRY(umbs_gemm(dt, s.cq, l.q_rank, 0, l.w_uq, l.q_rank, 0, s.q, hd, 0, 0, T, hd, l.q_rank, 1, nullptr, nullptr, 0,
                               0.f, stream));
            if (b->max_seq_len > 1 && b->max_pos0 == 0 && l.w_ukv != nullptr && umbs_window_attention_fits(l.dim, l.vdim)) {
                // a step of fresh sequences: every visible key is in the step, so keys and values are up-projected once per
                // token and attention runs over dim + vdim numbers per key instead of twice the latent rank
                UMBS_TRY(umbs_gemm(dt, s.c, R, 0, l.w_ukv, R, 0, s.kv, hd + hv, 0, 0, T, hd + hv, R, 1, nullptr, nullptr, 0, 0.f,
                                   stream));
                const char* kvb = (const char*)s.kv;
                UMBS_TRY(umbs_window_attention(dt, s.q, hd, kvb, hd + hv, kvb + (size_t)hd * (dt == UMBS_F32 ? 4 : 2), hd + hv, b,
                                               l.heads, l.dim, l.vdim, l.window, l.scale, s.mixed, hv, stream));
                UMBS_TRY(umbs_ring_append(dt, s.c, l.ring, l.ring_len, b, R, stream));
            } else {
                // q_abs[t, h, :] = W_uk[h]^T q[t, h, :]: scores against the cached latents need no per-key up-projection
                UMBS_TRY(umbs_gemm(dt, s.q, hd, l.dim, l.w_ukT, l.dim, (int64_t)R * l.dim, s.q_abs, (int64_t)l.heads * R, R, 1, T, R,
                                   l.dim, l.heads, nullptr, nullptr, 0, 0.f, stream));
                UMBS_TRY(umbs_latent_attention(dt, s.q_abs, s.c, l.ring, l.ring_len, b, l.heads, R, l.window, l.scale, s.la_part,
                                               s.la_part_bytes, s.o_lat, stream));
                UMBS_TRY(umbs_ring_append(dt, s.c, l.ring, l.ring_len, b, R, stream));
                UMBS_TRY(umbs_gemm(dt, s.o_lat, (int64_t)l.heads * R, R, l.w_uv, R, (int64_t)l.vdim * R, s.mixed, hv, l.vdim, 0, T,
                                   l.vdim, R, l.heads, nullptr, nullptr, 0, 0.f, stream));
            }
        } else {
            return UMB_ERR_UNSUPPORTED;
        }
        UMBS_TRY(umbs_gemm(dt, s.mixed, hv, 0, l.w_o, hv, 0, s.mix_out, W, 0, 1, T, W, hv, 1, nullptr, nullptr, 0, 0.f, stream));
        const float* pair_out = nullptr;
        const float* shared = nullptr;
        int top = 0;
        if (l.has_mlp) {
            const umbs_mlp_t& f = l.mlp;
            if (f.experts > 0) {
                top = f.top;
                UMBS_TRY(umbs_moe_route(dt, s.h, T, W, f.w_router, f.experts, f.top, s.sel_w, s.grp_off, s.pair_tok, s.pair_pos,
                                        s.route_scratch, stream));
                UMBS_TRY(umbs_gemm(dt, s.h, W, 0, f.w_gu, W, (int64_t)2 * f.ff * W, s.y, f.ff, 0, 0, T, f.ff, W, f.experts,
                                   s.grp_off, s.pair_tok, 1, f.limit, stream));
                UMBS_TRY(umbs_gemm(dt, s.y, f.ff, 0, f.w_down, f.ff, (int64_t)W * f.ff, s.pair_out, W, 0, 1, T, W, f.ff, f.experts,
                                   s.grp_off, nullptr, 0, 0.f, stream));
                pair_out = s.pair_out;
            }
            if (f.shared_ff > 0) {
                UMBS_TRY(umbs_gemm(dt, s.h, W, 0, f.ws_gu, W, 0, s.ys, f.shared_ff, 0, 0, T, f.shared_ff, W, 1, nullptr, nullptr, 1,
                                   f.shared_limit, stream));
                UMBS_TRY(umbs_gemm(dt, s.ys, f.shared_ff, 0, f.ws_down, f.shared_ff, 0, s.shared_out, W, 0, 1, T, W, f.shared_ff, 1,
                                   nullptr, nullptr, 0, 0.f, stream));
                shared = s.shared_out;
            }
        }
        UMBS_TRY(umbs_depth_mix(x, s.mix_out, pair_out, s.sel_w, s.pair_pos, top, shared, s.stack, i, l.depth_w, s.x,
                                layer_out ? layer_out + (int64_t)i * plane : nullptr, T, W, stream));
        x = s.x;
    }
    if (logits != nullptr && b->n_want > 0) {
        UMBS_TRY(umbs_group_norm_rows(dt, x, b->want_rows, b->n_want, m->final_norm, W, m->norm_groups, m->norm_eps, s.final_h,
                                      stream));
        UMBS_TRY(umbs_gemm(dt, s.final_h, W, 0, m->head, W, 0, logits, m->vocab, 0, 1, b->n_want, m->vocab, W, 1, nullptr, nullptr, 0,
                           0.f, stream));
        if (m->logit_softcap > 0.f) UMBS_TRY(umbs_softcap(logits, (int64_t)b->n_want * m->vocab, m->logit_softcap, stream));
    }
    return 0;
}
