"""Each mechanism the Kulisun family adds to the pre-norm step alone, on the GPU, against the plain statement in
oracle/kulisun.py: residual + layer norm with layer scale, multiplier and the routed / shared sums; products with bias,
silu gate and sigmoid output gate; the latent's norm and the turn of the rotated parts; the group-limited sigmoid router;
attention over [latent | shared part] keys in the step, in the cache and split over blocks; attention among a step's
own up-projected keys.  Inputs are shaped so that a fault shows: one key made dominant at a chosen distance, scores far
below or above the sink, slots whose earlier owner left its rows behind."""
import math

import pytest
import torch

from oracle import kulisun as O

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


# ---------------------------------------------------------------------------------------------- norm, sums, products
def test_add_norm_layer_norm_scale_and_expert_sums():
    from umbrella_b200 import _lib_seq as S, ops_seq as K
    for width in (40, 200, 1100, 4100):
        n, top = 7, 3
        x, d = rnd(n, width, seed=1, scale=2.0) + 0.7, rnd(n, width, seed=2)
        w, b, ls = rnd(width, seed=3, scale=0.3) + 1, rnd(width, seed=4, scale=0.3), rnd(width, seed=5, scale=0.3) + 1
        xs = f32(x)
        y, copy = K.add_norm(xs, f32(w), f32(b), 1e-5, delta=f32(d), scale=f32(ls), mult=0.6, want_copy=True)
        tot = x + 0.6 * (ls * d)
        assert err(y, O.layer_norm(tot, w, b, 1e-5)) < 3e-6
        assert err(xs, tot) < 1e-6 and err(copy, tot) < 1e-6               # the sum stays in the residual stream
        rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
        xs2 = f32(x)
        y2 = K.add_norm(xs2, f32(w), f32(b), 1e-5, rows=rows, delta=f32(d), scale=f32(ls), mult=0.6)
        assert err(y2, O.layer_norm(tot[[5, 0, 5]], w, b, 1e-5)) < 3e-6
        assert torch.equal(xs2.cpu(), x.float())                           # chosen rows: nothing is written back
        # routed pairs in sorted order + the shared expert times its per-token factor
        pair_out, shared, sg = rnd(n * top, width, seed=6), rnd(n, width, seed=7), torch.rand(n, dtype=torch.float64)
        sel_w = torch.rand(n, top, dtype=torch.float64)
        perm = torch.randperm(n * top, generator=torch.Generator().manual_seed(8))
        ff = torch.stack([sum(sel_w[t, k] * pair_out[perm[t * top + k]] for k in range(top)) for t in range(n)])
        xs3 = f32(x)
        y3 = K.add_norm(xs3, f32(w), f32(b), 1e-5, pair_out=f32(pair_out), sel_w=f32(sel_w),
                        pair_pos=perm.to(DEV, torch.int32), shared=f32(shared), shared_gate=f32(sg), scale=f32(ls), mult=0.5)
        tot3 = x + 0.5 * (ls * (ff + shared * sg[:, None]))
        assert err(xs3, tot3) < 1e-6 and err(y3, O.layer_norm(tot3, w, b, 1e-5)) < 3e-6
        # the RMS kind with an offset on the weight, bf16 output
        yb = K.add_norm(f32(x), f32(w), None, 1e-5, kind=S.UMBS_NORM_RMS, w_offset=1.0, dtype=torch.bfloat16)
        assert err(yb, O.rms_norm(x, 1.0 + w, 1e-5)) < 1e-2
    # a row whose mean dwarfs its spread: the deviations are taken from the mean, not from a difference of large sums
    x = 1000.0 + rnd(3, 96, seed=9, scale=0.05)
    one, zero = torch.ones(96, dtype=torch.float64), torch.zeros(96, dtype=torch.float64)
    assert err(K.add_norm(f32(x), f32(one), f32(zero), 1e-9), O.layer_norm(f32(x).double().cpu(), one, zero, 1e-9)) < 2e-2


def test_products_with_bias_silu_and_output_gate():
    from umbrella_b200 import _lib_seq as S, ops_seq as K
    for M, Kd, N in ((5, 64, 48), (150, 96, 80), (150, 50, 33), (1, 256, 40)):       # few rows, tiles, unaligned, one row
        a, wg, wu = rnd(M, Kd, seed=1), rnd(N, Kd, seed=2, scale=Kd ** -0.5), rnd(N, Kd, seed=3, scale=Kd ** -0.5)
        bg, bu, gate = rnd(N, seed=4, scale=0.5), rnd(N, seed=5, scale=0.5), rnd(M, N + 3, seed=6)
        ref = O.silu(a @ wg.T + bg) * (a @ wu.T + bu)
        got = K.gemm_ex(f32(a), f32(torch.cat([wg, wu])), act=S.UMBS_ACT_SILU, bias=f32(torch.cat([bg, bu])), out_f32=True)
        assert err(got, ref) < 3e-6, (M, Kd, N)
        ref2 = (a @ wg.T + bg) * torch.sigmoid(gate[:, 3:])
        got2 = K.gemm_ex(f32(a), f32(wg), bias=f32(bg), out_gate=f32(gate)[:, 3:], out_f32=True)
        assert err(got2, ref2) < 3e-6, (M, Kd, N)
        bf = lambda t: t.to(DEV, torch.bfloat16).contiguous()
        ab, wb = bf(a).double().cpu(), bf(torch.cat([wg, wu])).double().cpu()
        refb = O.silu(ab @ wb[:N].T + bg) * (ab @ wb[N:].T + bu)
        gotb = K.gemm_ex(bf(a), bf(torch.cat([wg, wu])), act=S.UMBS_ACT_SILU, bias=f32(torch.cat([bg, bu])), out_f32=True)
        assert err(gotb, refb) < 3e-5, (M, Kd, N)
    # batched over heads with a gate column block per head (the value up-projection behind latent attention)
    H, R, V, T = 3, 40, 24, 70
    o_lat, uv, gate = rnd(T, H * R, seed=7), rnd(H * V, R, seed=8, scale=R ** -0.5), rnd(T, 5 + H * V, seed=9)
    ref = torch.cat([o_lat[:, h * R:(h + 1) * R] @ uv[h * V:(h + 1) * V].T for h in range(H)], dim=1) * torch.sigmoid(gate[:, 5:])
    got = K.gemm_ex(f32(o_lat), f32(uv).view(H, V, R), groups=H, a_goff=R, c_goff=V, n=V, k=R, out_gate=f32(gate)[:, 5:], gate_goff=V)
    assert err(got, ref) < 3e-6


def test_token_gate_and_scaled_embedding():
    from umbrella_b200 import ops_seq as K
    h, w = rnd(37, 200, seed=1), rnd(200, seed=2, scale=0.2)
    assert err(K.token_gate(f32(h), f32(w)), torch.sigmoid(h @ w)) < 2e-6
    table = rnd(50, 72, seed=3).to(torch.bfloat16)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    assert err(K.embedding_scaled(ids, table.to(DEV), 13.5), table.double()[[3, 49, 0, 3]] * 13.5) < 1e-6


# ---------------------------------------------------------------------------------------------- router
@pytest.mark.parametrize("n", [6, 300])               # the one-block kernel of small steps and the block-per-token kernel
def test_group_limited_sigmoid_router(n):
    from umbrella_b200 import _lib_seq as S, ops_seq as K
    for E, G, keep, top in ((12, 3, 2, 4), (8, 8, 3, 2), (6, 1, 1, 6), (10, 5, 5, 1), (16, 4, 1, 4)):
        h, wr = rnd(n, 48, seed=E), rnd(E, 48, seed=E + 1, scale=0.4)
        chosen, weights = O.route(h, dict(router=wr, groups=G, keep=keep, top=top))
        gw = rnd(48, seed=E + 2, scale=0.4)          # the per-token gate rides along in the same pass
        sel_w, grp_off, pair_tok, pair_pos, sel_e, gate = K.moe_route_ex(f32(h), f32(wr), top, S.UMBS_ROUTE_SIGMOID_GROUPS, G, keep,
                                                                         gate_w=f32(gw))
        assert err(gate, torch.sigmoid(h @ gw)) < 2e-6
        assert torch.equal(gate, K.token_gate(f32(h), f32(gw)))
        sel_e, sel_w = sel_e.cpu(), sel_w.cpu()
        for t in range(n):
            assert sel_e[t].tolist() == chosen[t], (E, G, keep, top, t)
            assert err(sel_w[t], weights[t]) < 3e-6
        # the sorted pair list: expert e owns [grp_off[e], grp_off[e + 1]), pair_pos inverts pair_tok
        go, pt, pp = grp_off.cpu().tolist(), pair_tok.cpu().tolist(), pair_pos.cpu().view(n, top)
        assert go[0] == 0 and go[-1] == n * top
        for t in range(n):
            for k in range(top):
                p = int(pp[t, k])
                assert pt[p] == t and go[int(sel_e[t, k])] <= p < go[int(sel_e[t, k]) + 1]
    # a group with one towering expert loses to a group with two good ones: the group's score is a sum of two
    E, G = 8, 2
    wr = torch.zeros(E, 4, dtype=torch.float64)
    wr[0, 0], wr[4, 0], wr[5, 0] = 6.0, 2.0, 2.0      # sigmoid: .998 + .5 = 1.498 against .88 + .88 = 1.76
    h = torch.tensor([[1.0, 0, 0, 0]] * n, dtype=torch.float64)
    *_, sel_e = K.moe_route_ex(f32(h), f32(wr), 2, S.UMBS_ROUTE_SIGMOID_GROUPS, G, 1)
    assert sel_e.cpu()[0].tolist() == [4, 5]


# ---------------------------------------------------------------------------------------------- latent preparation
def test_latent_prep_norm_and_turn_across_steps():
    from umbrella_b200 import ops_seq as K
    for H, D, Rt, R, rot in ((3, 16, 8, 40, dict(dims=8, base=100.0, scaling=dict(factor=4.0, original=24, fast=6.0, slow=1.0))),
                             (1, 24, 12, 20, dict(dims=4, base=50.0, scaling=None)),
                             (2, 8, 0, 33, None)):
        n, cols = 45, H * (D + Rt) + R + Rt + 7
        proj, kw = rnd(n, cols, seed=H), rnd(R, seed=9, scale=0.3) + 1
        f, mag = O.rotary_frequencies(rot) if rot else ([], 1.0)
        rd = rot["dims"] if rot else 0
        inv = f32(torch.tensor(f if f else [0.0], dtype=torch.float64))
        q_ref = proj[:, :H * (D + Rt)].reshape(n, H, D + Rt).clone()
        low = proj[:, H * (D + Rt):H * (D + Rt) + R + Rt]
        c_ref = O.rms_norm(low[:, :R], kw, 1e-5)
        kr_ref = low[:, R:]
        if rot:
            q_ref = torch.cat([q_ref[..., :D], O.rotate(q_ref[..., D:], rot)], dim=-1)
            kr_ref = O.rotate(kr_ref, rot)
        got_q, got_c, got_a = [], [], []
        for desc in steps_of([[(0, 30)], [(0, 2)]] + [[(0, 1)]] * 13):          # positions go on from step to step
            s0 = desc[0][2]
            b = K.RaggedBatch(desc, DEV)
            q, c, q_abs = K.latent_prep(f32(proj[s0:s0 + desc[0][1]]), b, H, D, Rt, R, f32(kw), 1e-5, rd, inv, mag)
            got_q.append(q), got_c.append(c), got_a.append(q_abs)
        assert err(torch.cat(got_q), q_ref.reshape(n, -1)) < 3e-6
        assert err(torch.cat(got_c), torch.cat([c_ref, kr_ref], dim=1)) < 3e-6
        if Rt:
            assert err(torch.cat(got_a)[..., R:], q_ref[..., D:]) < 3e-6      # every head's turned part again, in fp32


# ---------------------------------------------------------------------------------------------- attention
def plain_shared_key_attention(q_abs, c, R, scale, sink):
    """q_abs [n, H, KD], c [n, KD]: every head scores against the whole row and reads the first R numbers as the value."""
    n, H, KD = q_abs.shape
    k = c[:, None, :].expand(n, H, KD)
    return O.sink_softmax_attention(q_abs, k, k[..., :R], scale, sink)


def run_latent(q_abs, c, R, Rt, scale, sink, pieces, slot=0, ring=None, cap=None, split=True):
    from umbrella_b200 import ops_seq as K
    n, H, KD = q_abs.shape
    ring = ring if ring is not None else torch.full((slot + 1, cap or n, KD), 7.0, dtype=torch.float32, device=DEV)
    out, pos = [], 0
    for desc in steps_of([[(slot, p)] for p in pieces]):
        b = K.RaggedBatch(desc, DEV)
        m = desc[0][1]
        out.append(K.latent_attention_shared(f32(q_abs[pos:pos + m]), f32(c[pos:pos + m]), ring, b, H, R, Rt, scale,
                                             sink=f32(sink), split=split))
        pos += m
    return torch.cat(out).view(n, H, R), ring


@pytest.mark.parametrize("H,R,Rt", [(4, 40, 8), (1, 33, 0), (6, 120, 24), (3, 20, 12)])
def test_latent_attention_whole_portions_and_decode(H, R, Rt):
    n, scale = 150, 0.2
    q_abs, c, sink = rnd(n, H, R + Rt, seed=1), rnd(n, R + Rt, seed=2), rnd(H, seed=3, scale=1.5)
    ref = plain_shared_key_attention(q_abs, c, R, scale, sink)
    for pieces in ([n], [64, 2, 31, 1, 52], [100] + [1] * 50, [1] * 40 + [110]):
        got, _ = run_latent(q_abs, c, R, Rt, scale, sink, pieces, slot=1)       # the ring starts full of another value
        assert err(got, ref) < 3e-6, pieces
    got, _ = run_latent(q_abs, c, R, Rt, scale, sink, [100] + [1] * 50, split=False)
    assert err(got, ref) < 3e-6


def test_latent_attention_far_key_and_sink():
    """One key made dominant far back, at a tile border and right behind the row; scores far below / above the sink."""
    H, R, Rt, n, scale = 2, 24, 8, 700, 1.0
    for far in (0, 31, 32, 63, 64, 500, 698):
        q_abs, c = rnd(n, H, R + Rt, seed=4, scale=0.3), rnd(n, R + Rt, seed=5, scale=0.3)
        c[far, R:] = 6.0                                    # the shared part carries the match ...
        q_abs[n - 1, :, R:] = 6.0                           # ... for the last row only
        sink = torch.tensor([0.0, -3.0], dtype=torch.float64)
        ref = plain_shared_key_attention(q_abs, c, R, scale, sink)
        assert float((ref[n - 1, 0] - c[far, :R]).abs().max()) < 1e-3          # the row's output is that key's latent
        for pieces in ([n], [n - 1, 1], [far + 1, n - far - 2, 1] if far < n - 2 else [n - 2, 1, 1]):
            got, _ = run_latent(q_abs, c, R, Rt, scale, sink, pieces)
            assert err(got[n - 1], ref[n - 1]) < 3e-6, (far, pieces)
            assert err(got, ref) < 3e-6
    # a sink far above every score leaves (almost) nothing; far below, it changes nothing
    q_abs, c = rnd(40, H, R + Rt, seed=6, scale=0.2), rnd(40, R + Rt, seed=7, scale=0.2)
    plain = plain_shared_key_attention(q_abs, c, R, scale, torch.full((H,), -1e9, dtype=torch.float64))
    for s in (30.0, -60.0):
        sink = torch.full((H,), s, dtype=torch.float64)
        for pieces in ([40], [39, 1]):
            got, _ = run_latent(q_abs, c, R, Rt, scale, sink, pieces)
            assert err(got, plain_shared_key_attention(q_abs, c, R, scale, sink)) < 1e-5
            assert float(got.abs().max()) < 1e-9 if s > 0 else err(got, plain) < 3e-6
    # a learned sink against the fixed one: sink NULL counts exp(0)
    from umbrella_b200 import ops_seq as K
    b = K.RaggedBatch([(0, 40, 0, 0)], DEV)
    ring = torch.zeros((1, 40, R + Rt), dtype=torch.float32, device=DEV)
    got0 = K.latent_attention_shared(f32(q_abs), f32(c), ring, b, H, R, Rt, scale, sink=None).view(40, H, R)
    assert err(got0, plain_shared_key_attention(q_abs, c, R, scale, torch.zeros(H, dtype=torch.float64))) < 3e-6


def test_latent_attention_batch_and_reused_slot():
    from umbrella_b200 import ops_seq as K
    H, R, Rt, scale = 3, 40, 8, 0.25
    lens = [70, 1, 33]
    qs = [rnd(n + 6, H, R + Rt, seed=10 + i) for i, n in enumerate(lens)]
    cs = [rnd(n + 6, R + Rt, seed=20 + i) for i, n in enumerate(lens)]
    sink = rnd(H, seed=30)
    refs = [plain_shared_key_attention(q, c, R, scale, sink) for q, c in zip(qs, cs)]
    ring = torch.full((4, 128, R + Rt), 9.0, dtype=torch.float32, device=DEV)       # slots 3, 0, 2; rows of earlier owners
    slots = [3, 0, 2]
    sched = steps_of([[(s, n) for s, n in zip(slots, lens)]] + [[(s, 1) for s in slots]] * 6)
    got = [[] for _ in lens]
    for step, desc in enumerate(sched):
        b = K.RaggedBatch(desc, DEV)
        take = (lambda i: slice(0, lens[i])) if step == 0 else (lambda i: slice(lens[i] + step - 1, lens[i] + step))
        q = torch.cat([qs[i][take(i)] for i in range(3)])
        c = torch.cat([cs[i][take(i)] for i in range(3)])
        o = K.latent_attention_shared(f32(q), f32(c), ring, b, H, R, Rt, scale, sink=f32(sink)).view(-1, H, R)
        at = 0
        for i in range(3):
            m = desc[i][1]
            got[i].append(o[at:at + m])
            at += m
    for i in range(3):
        assert err(torch.cat(got[i]), refs[i]) < 3e-6, i


@pytest.mark.parametrize("H,D,Rt,V", [(4, 16, 8, 24), (1, 24, 0, 8), (2, 128, 64, 128), (3, 40, 12, 100)])
def test_fresh_attention_over_up_projected_keys(H, D, Rt, V):
    from umbrella_b200 import ops_seq as K
    lens, scale = [130, 1, 64, 65], (D + Rt) ** -0.5
    T = sum(lens)
    q, k, ks, v = rnd(T, H * (D + Rt), seed=1), rnd(T, H * D, seed=2), rnd(T, max(Rt, 1), seed=3), rnd(T, H * V, seed=4)
    gate, sink = rnd(T, H * V + 2, seed=5), rnd(H, seed=6, scale=1.5)
    b = K.RaggedBatch([(i, n, 0, 0) for i, n in enumerate(lens)], DEV)
    kv = f32(torch.cat([k, v], dim=1))                                       # keys and values side by side, as the step holds them
    got = K.window_attention_shared(f32(q), kv[:, :H * D], f32(ks)[:, :Rt] if Rt else None, kv[:, H * D:], b, H, scale,
                                    sink=f32(sink), gate=f32(gate)[:, 2:])
    at = 0
    for n in lens:
        sl = slice(at, at + n)
        kk = torch.cat([k[sl].reshape(n, H, D), ks[sl, :Rt][:, None, :].expand(n, H, Rt)], dim=-1)
        ref = O.sink_softmax_attention(q[sl].reshape(n, H, D + Rt), kk, v[sl].reshape(n, H, V), scale, sink).reshape(n, -1)
        assert err(got[sl], ref * torch.sigmoid(gate[sl, 2:])) < 3e-6, n
        at += n
