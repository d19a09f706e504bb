"""Each mechanism the Subivik family adds to the pre-norm step alone, on the GPU, against the plain statement in
oracle/subivik.py: sinusoidal positions; the tanh norm with two pending outputs; the xielu and tanh epilogues; the
softmax-over-all router; the norm of query and key maps; attention with a score cap, a distance penalty and talking heads;
chunked differential attention; token-shifted mixes; the time-mix memory.  Inputs are shaped so that a fault shows: one
key made dominant far back, just inside or just outside a chunk, slots whose earlier owner left its rows behind."""
import math

import pytest
import torch

from oracle import subivik as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)


def err(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def f32(t):
    return t.to(DEV, torch.float32).contiguous()


def steps_of(lengths_per_step):
    """[[(slot, n), ...], ...] -> per step [(slot, n, pos0, parity)], tracking positions."""
    pos, par, out = {}, {}, []
    for step in lengths_per_step:
        desc = []
        for slot, n in step:
            desc.append((slot, n, pos.get(slot, 0), par.get(slot, 0)))
            pos[slot] = pos.get(slot, 0) + n
            par[slot] = par.get(slot, 0) ^ 1
        out.append(desc)
    return out


def selector(rows, start, total):
    """[rows, total]: picks columns start .. start + rows of a vector (a projection that copies its inputs)."""
    m = torch.zeros(rows, total, dtype=torch.float64)
    m[torch.arange(rows), start + torch.arange(rows)] = 1.0
    return m


# ---------------------------------------------------------------------------------------------- embedding, norm, products
def test_sinusoidal_positions_near_and_far():
    from umbrella_b200 import ops_seq as K
    from umbrella_b200.models.seq_model import rotary_inv_freq
    for width in (6, 50, 256):
        table = rnd(11, width, seed=1)
        ids = torch.tensor([3, 0, 10, 7, 7], dtype=torch.int32, device=DEV)
        pos = [0, 1, 2, 977, 4099]
        y = K.embedding_pos(ids, torch.tensor(pos, dtype=torch.int32, device=DEV), f32(table), rotary_inv_freq(width, 10000.0).to(DEV))
        ref = table.float().double()[ids.cpu().long()] + torch.cat([O.sinusoid_positions(1, width, first=p) for p in pos])
        assert float((y.double().cpu() - ref).abs().max()) < 3e-4          # fp32 angles: position times 6e-8


def test_tanh_norm_with_two_pending_outputs():
    from umbrella_b200 import ops_seq as K
    for width in (40, 200, 1100):
        n = 7
        x, d1, d2 = rnd(n, width, seed=1, scale=2.0), rnd(n, width, seed=2), rnd(n, width, seed=3)
        w, b = rnd(width, seed=4, scale=0.3) + 1, rnd(width, seed=5, scale=0.3)
        xs = f32(x)
        y = K.add_norm_dyt(xs, f32(w), f32(b), 0.37, delta=f32(d1), delta_mult=0.8, delta2=f32(d2), delta2_mult=-1.2)
        tot = x + 0.8 * d1 - 1.2 * d2
        assert err(y, O.dynamic_tanh(tot, 0.37, w, b)) < 3e-6 and err(xs, tot) < 1e-6
        rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
        xs2 = f32(x)
        y2 = K.add_norm_dyt(xs2, f32(w), f32(b), 1.9, rows=rows, delta=f32(d1))
        assert err(y2, O.dynamic_tanh((x + d1)[[5, 0, 5]], 1.9, w, b)) < 3e-6
        assert torch.equal(xs2.cpu(), x.float())                           # chosen rows: nothing is written back


def test_unary_epilogues():
    from umbrella_b200 import _lib_seq as S, ops_seq as K
    for m, n, k in ((5, 24, 40), (70, 100, 64), (300, 48, 96)):
        a, w = rnd(m, k, seed=m), rnd(n, k, seed=n, scale=k ** -0.5 * 2)
        z = a.float().double() @ w.float().double().T
        p, q = 0.3, -0.6
        got = K.gemm_unary(f32(a), f32(w), S.UMBS_UNARY_XIELU, O.softplus(p), 0.5 + O.softplus(q), out_f32=True)
        assert err(got, O.xielu(z, p, q)) < 1e-5
        assert err(K.gemm_unary(f32(a), f32(w), S.UMBS_UNARY_TANH, out_f32=True), torch.tanh(z)) < 1e-5
        ab, wb = a.to(DEV, torch.bfloat16), w.to(DEV, torch.bfloat16)
        zb = ab.double().cpu() @ wb.double().cpu().T
        assert err(K.gemm_unary(ab, wb, S.UMBS_UNARY_XIELU, O.softplus(p), 0.5 + O.softplus(q), out_f32=True), O.xielu(zb, p, q)) < 1e-4


def test_router_softmax_over_all_experts():
    from umbrella_b200 import _lib_seq as S, ops_seq as K
    for n, experts, top in ((5, 7, 3), (400, 12, 4), (9, 4, 4), (33, 1, 1), (300, 40, 1)):
        h, wr = rnd(n, 48, seed=n), rnd(experts, 48, seed=experts, scale=0.5)
        sel_w, grp_off, pair_tok, pair_pos, sel_e = K.moe_route_scaled(f32(h), f32(wr), top, S.UMBS_ROUTE_SOFTMAX_ALL, 2.5)
        s = torch.softmax(h.float().double() @ wr.float().double().T, dim=-1)
        for t in range(n):
            order = sorted(range(experts), key=lambda e: (-float(s[t, e]), e))[:top]
            assert sel_e[t].tolist() == order
            assert err(sel_w[t], 2.5 * s[t, order]) < 1e-5                 # not renormalised over the chosen
        counts = torch.bincount(sel_e.flatten().cpu().long(), minlength=experts)
        assert grp_off.cpu().tolist() == [0] + counts.cumsum(0).tolist()
        assert sorted(pair_pos.cpu().tolist()) == list(range(n * top))


# ---------------------------------------------------------------------------------------------- attention
def feed(run_step, schedule, total):
    """Run `schedule` (token counts of one sequence's steps) and gather the rows; run_step(lo, hi, desc) -> rows."""
    out, lo = [], 0
    for desc in steps_of([[(0, n)] for n in schedule]):
        hi = lo + desc[0][1]
        out.append(run_step(lo, hi, desc))
        lo = hi
    assert lo == total
    return torch.cat(out)


SCHEDULES = ([150], [100] + [1] * 50, [2, 61, 1, 1, 64, 21], [63, 1, 1, 1, 84], [7] * 21 + [3])


def test_talking_attention_with_cap_and_distance_penalty():
    """Every query head against every value head, weights mixed after the softmax; a far key that dominates one head's
    scores, the cap that bounds it, the penalty that grows with the distance."""
    from umbrella_b200 import ops_seq as K
    from umbrella_b200.ops_seq import RaggedBatch
    n = 150
    for H, G, D, V, cap in ((6, 3, 10, 14, 5.0), (4, 1, 72, 40, 0.0), (2, 2, 16, 100, 2.0)):
        cq, ck, cv = H * D, G * D, G * V
        h = rnd(n, cq + ck + cv, seed=H)
        h[3, cq:cq + D] *= 6.0                                   # a key far back that stands out ...
        h[140, :D] = h[3, cq:cq + D] * 0.5                       # ... for a late query of head 0
        h[77, cq:cq + ck] *= 4.0                                 # and one at a place where caches and tiles meet
        h = h.float().double()
        m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=0.31, softcap=cap, q=selector(cq, 0, cq + ck + cv),
                 k=selector(ck, cq, cq + ck + cv), v=selector(cv, cq + ck, cq + ck + cv), r1=rnd(H, seed=1).abs(),
                 r2=rnd(H, seed=2, scale=2.0).abs(), talk=rnd(H, H, seed=3), o=torch.eye(H * V, dtype=torch.float64))
        ref = O.talking_attention(h, m)
        r1, r2, talk = f32(m["r1"]), f32(m["r2"]), f32(m["talk"])
        for schedule in SCHEDULES:
            cache = torch.full((2, 160, ck + cv), 7.0, dtype=torch.float32, device=DEV)       # (a former owner's rows)

            def step(lo, hi, desc):
                b = RaggedBatch(desc, DEV)
                q, kv = K.attention_prep_maps(f32(h[lo:hi]), b, H, G, D, V)
                return K.scored_attention(q, kv, cache, b, H, G, D, V, 0.31, softcap=cap, r1=r1, r2=r2, talk=talk)
            assert err(feed(step, schedule, n), ref) < 2e-5, (H, schedule)


def test_chunked_differential_attention_at_chunk_borders():
    """Two maps over the same values, keys inside the row's own chunk only: a dominant key as the last of the chunk before
    and as the first of the row's chunk, in prompts, portions and token-by-token steps; a ring of one chunk."""
    from umbrella_b200 import ops_seq as K
    from umbrella_b200.ops_seq import RaggedBatch
    n, eps = 150, 1e-5
    for H, G, D, V, chunk in ((4, 2, 12, 20, 16), (2, 1, 48, 64, 64), (3, 3, 8, 8, 1), (2, 2, 20, 28, 0)):
        cq, ck, cv, cg = 2 * H * D, 2 * G * D, G * V, H * V
        tot = cq + ck + cv + cg
        h = rnd(n, tot, seed=H + chunk)
        edge = (chunk or 50) * (2 if chunk and chunk * 3 < n else 1)
        for j in (edge - 1, edge):                               # just outside and just inside the chunk of the rows behind
            if 0 <= j < n:
                h[j, cq:cq + ck] *= 5.0
        h = h.float().double()
        m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=0.4, chunk=chunk, diff=0.35, kv_from=None,
                 q=selector(cq, 0, tot), k=selector(ck, cq, tot), v=selector(cv, cq + ck, tot), g=selector(cg, cq + ck + cv, tot),
                 q_norm=rnd(D, seed=4, scale=0.3) + 1, k_norm=rnd(D, seed=5, scale=0.3) + 2, lq1=rnd(D, seed=6, scale=0.3),
                 lk1=rnd(D, seed=7, scale=0.3), lq2=rnd(D, seed=8, scale=0.3), lk2=rnd(D, seed=9, scale=0.3),
                 o=torch.eye(H * V, dtype=torch.float64))
        k, v = O.differential_keys_values(h, m, eps)
        ref = O.differential_attention(h, m, eps, k, v)
        lam = math.exp(float((m["lq1"] * m["lk1"]).sum())) - math.exp(float((m["lq2"] * m["lk2"]).sum())) + 0.35
        qn, kn = f32(m["q_norm"]), f32(m["k_norm"])
        for schedule in SCHEDULES:
            cache = torch.full((2, chunk or 160, ck + cv), 7.0, dtype=torch.float32, device=DEV)

            def step(lo, hi, desc):
                b = RaggedBatch(desc, DEV)
                proj = f32(h[lo:hi])
                q, kv = K.attention_prep_maps(proj, b, H, G, D, V, maps=2, q_norm=qn, k_norm=kn, eps=eps)
                return K.scored_attention(q, kv, cache, b, H, G, D, V, 0.4, chunk=chunk, maps=2, diff_lambda=lam, unit_norm=True,
                                          eps=eps, out_mult=0.65, gate=proj[:, cq + ck + cv:])
            assert err(feed(step, schedule, n), ref) < 3e-5, (H, chunk, schedule)


def test_borrowed_keys_are_read_before_the_lender_appends():
    """A borrower reads the lender's step rows and the lender's cache as it was before the step: the lender's rows go to
    the ring only afterwards, so a long portion cannot overwrite keys the borrower still needs."""
    from umbrella_b200 import ops_seq as K
    from umbrella_b200.ops_seq import RaggedBatch
    H, G, D, V, chunk, n, eps = 2, 1, 16, 12, 32, 120, 1e-6
    cq, ck, cv = 2 * H * D, 2 * G * D, G * V
    h = rnd(n, cq + ck + cv, seed=3).float().double()
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=0.5, chunk=chunk, diff=0.2, kv_from=None, q=selector(cq, 0, cq + ck + cv),
             k=selector(ck, cq, cq + ck + cv), v=selector(cv, cq + ck, cq + ck + cv), g=torch.zeros(H * V, cq + ck + cv, dtype=torch.float64),
             q_norm=torch.ones(D, dtype=torch.float64), k_norm=torch.ones(D, dtype=torch.float64), lq1=rnd(D, seed=6, scale=0.3),
             lk1=rnd(D, seed=7, scale=0.3), lq2=rnd(D, seed=8, scale=0.3), lk2=rnd(D, seed=9, scale=0.3), o=torch.eye(H * V, dtype=torch.float64))
    k, v = O.differential_keys_values(h, m, eps)
    ref = 2.0 * O.differential_attention(h, m, eps, k, v)                   # (the gate is sigmoid(0) = 1/2 there)
    lam = math.exp(float((m["lq1"] * m["lk1"]).sum())) - math.exp(float((m["lq2"] * m["lk2"]).sum())) + 0.2
    ones = f32(torch.ones(D))
    cache = torch.zeros((1, chunk, ck + cv), dtype=torch.float32, device=DEV)

    def step(lo, hi, desc):
        b = RaggedBatch(desc, DEV)
        q, kv = K.attention_prep_maps(f32(h[lo:hi]), b, H, G, D, V, maps=2, q_norm=ones, k_norm=ones, eps=eps)
        args = dict(chunk=chunk, maps=2, diff_lambda=lam, unit_norm=True, eps=eps, out_mult=0.8)
        own = K.scored_attention(q, kv, cache, b, H, G, D, V, 0.5, append=False, **args)
        again = K.scored_attention(q, kv, cache, b, H, G, D, V, 0.5, append=True, **args)      # the borrower, then the append
        assert torch.equal(own, again)
        return again
    assert err(feed(step, [20, 90, 1, 9], n), ref) < 3e-5


# ---------------------------------------------------------------------------------------------- the recurrent half
def test_token_shifted_mixes_across_steps_and_slots():
    from umbrella_b200 import ops_seq as K
    from umbrella_b200.ops_seq import RaggedBatch
    width, n_mix = 72, 5
    mu = torch.rand(n_mix, width, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    seqs = {0: rnd(40, width, seed=2), 1: rnd(9, width, seed=3)}
    state = torch.full((2, 3, width), 5.0, dtype=torch.float32, device=DEV)           # (a former owner's last rows)
    got = {0: [], 1: []}
    at = {0: 0, 1: 0}
    for desc in steps_of([[(0, 17), (1, 1)], [(1, 3), (0, 1)], [(0, 22), (1, 5)]]):
        rows = torch.cat([seqs[s][at[s]:at[s] + n] for s, n, _, _ in desc])
        out = K.shift_mix(f32(rows), f32(mu), state, RaggedBatch(desc, DEV))
        o = 0
        for s, n, _, _ in desc:
            got[s].append(out[o:o + n])
            at[s] += n
            o += n
    for s, x in seqs.items():
        x = x.float().double()
        ref = x[:, None, :] + (O.shifted(x) - x)[:, None, :] * mu[None]
        assert err(torch.cat(got[s]), ref) < 1e-6


def test_time_mix_memory_in_portions_and_batches():
    from umbrella_b200 import ops_seq as K
    from umbrella_b200.ops_seq import RaggedBatch
    eps = 1e-5
    for heads, dim in ((3, 20), (1, 64), (2, 100), (5, 8)):
        hd = heads * dim
        lens = {0: 130, 2: 37}
        data = {}
        for s, n in lens.items():
            proj, raw = rnd(n, 4 * hd, seed=10 + s), rnd(n, hd, seed=20 + s) - 1.0
            data[s] = (proj.float().double(), raw.float().double())
        bias, u, nw = rnd(hd, seed=1, scale=0.5).float().double(), rnd(hd, seed=2).float().double(), (rnd(hd, seed=3, scale=0.3) + 1).float().double()
        state = torch.full((3, heads, dim, dim), 9.0, dtype=torch.float32, device=DEV)          # (read as zero at position 0)
        got, at = {0: [], 2: []}, {0: 0, 2: 0}
        for desc in steps_of([[(0, 70), (2, 1)], [(2, 1), (0, 1)], [(0, 2), (2, 30)], [(0, 57), (2, 5)]]):
            proj = torch.cat([data[s][0][at[s]:at[s] + n] for s, n, _, _ in desc])
            raw = torch.cat([data[s][1][at[s]:at[s] + n] for s, n, _, _ in desc])
            out = K.time_mix(f32(proj), f32(raw), f32(bias), f32(u), RaggedBatch(desc, DEV), heads, dim, eps, f32(nw), state)
            o = 0
            for s, n, _, _ in desc:
                got[s].append(out[o:o + n])
                at[s] += n
                o += n
        for s, n in lens.items():
            proj, raw = data[s]
            r, k, v = (proj[:, i * hd:(i + 1) * hd].reshape(n, heads, dim) for i in range(3))
            w = torch.exp(-torch.exp(raw + bias)).reshape(n, heads, dim)
            o = O.decayed_memory(r, k, v, w, u.reshape(heads, dim))
            ref = O.unit_rms(o, eps).reshape(n, hd) * nw * O.silu(proj[:, 3 * hd:])
            assert err(torch.cat(got[s]), ref) < 2e-5, (heads, dim, s)
