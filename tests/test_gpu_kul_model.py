"""The Kulisun family on the GPU against the plain oracle (oracle/kulisun.py): whole prompts and every layer's stream,
the first tokens, decoding token by token through the cache, prompts cut into portions, ragged batches, reused slots,
long decoding with a growing cache, other sizes, both dtypes, greedy generation through the engine and its queue."""
import pytest
import torch

import kul_helpers as H
from oracle import kulisun as O

pytestmark = pytest.mark.gpu
TOL32 = 3e-5          # fp32 product vs float64 oracle: per-row rms of the logit difference over the logits' rms


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.fixture(scope="module")
def mixed():
    t = H.random_tensors(H.MIXED, seed=1)
    return H.MIXED, H.oracle_model(H.MIXED, t), H.product_model(H.MIXED, t, torch.float32)


def run(model, pieces):
    """Feed one sequence as the given portions through a fresh slot; -> logits of every position."""
    slot = model.cache.alloc_slot()
    out = [model.forward([(slot, p, range(len(p)))]) for p in pieces]
    model.cache.free_slot(slot)
    return torch.cat(out)


def cut(seq, sizes):
    out, i = [], 0
    for s in sizes:
        out.append(seq[i:i + s])
        i += s
    if i < len(seq):
        out.append(seq[i:])
    return [p for p in out if p]


def test_whole_prompt_and_layers(mixed):
    cfg, om, pm = mixed
    seq = toks(70, cfg["vocab"], 2)
    ref, streams = O.forward(om, seq, layer_out=True)
    slot = pm.cache.alloc_slot()
    got, ly = pm.forward([(slot, seq, range(len(seq)))], layer_out=True)
    pm.cache.free_slot(slot)
    for i in range(len(cfg["layers"])):
        assert H.row_err(ly[i], streams[i]) < TOL32, f"layer {i}"
    assert H.row_err(got, ref) < TOL32


def test_latent_form_equals_fresh_form(mixed):
    """A whole prompt attends over up-projected keys, every other step over the cached latents: the same numbers."""
    cfg, om, _ = mixed
    t = H.random_tensors(H.MIXED, seed=1)
    pm = H.product_model(H.MIXED, t, torch.float32, fresh_attention=False)
    seq = toks(70, cfg["vocab"], 2)
    assert H.row_err(run(pm, [seq]), O.forward(om, seq)) < TOL32


def test_first_tokens(mixed):
    cfg, om, pm = mixed
    for n in (1, 2, 3):
        seq = toks(n, cfg["vocab"], 10 + n)
        assert H.row_err(run(pm, [seq]), O.forward(om, seq)) < TOL32


def test_prefill_then_token_by_token(mixed):
    cfg, om, pm = mixed
    seq = toks(75, cfg["vocab"], 3)
    ref = O.forward(om, seq)
    for first in (1, 6, 30):
        got = run(pm, [seq[:first]] + [[t] for t in seq[first:]])
        assert H.row_err(got, ref) < TOL32, first


def test_portions_down_to_two_tokens(mixed):
    cfg, om, pm = mixed
    seq = toks(90, cfg["vocab"], 4)
    ref = O.forward(om, seq)
    for sizes in ([2, 2, 2, 3, 1, 2, 17, 4, 31], [64, 2], [3] * 30, [5, 64], [1, 2, 70], [32, 32, 26], [33, 31]):
        assert H.row_err(run(pm, cut(seq, sizes)), ref) < TOL32, sizes


def test_unequal_batch_equals_each_alone(mixed):
    cfg, om, pm = mixed
    seqs = [toks(n, cfg["vocab"], 20 + n) for n in (1, 37, 66, 9)]
    tails = [toks(12, cfg["vocab"], 50 + len(s)) for s in seqs]
    refs = [O.forward(om, s + tl) for s, tl in zip(seqs, tails)]
    slots = [pm.cache.alloc_slot() for _ in seqs]
    got = pm.forward([(slots[i], s, range(len(s))) for i, s in enumerate(seqs)])
    o = 0
    for s, r in zip(seqs, refs):
        assert H.row_err(got[o:o + len(s)], r[:len(s)]) < TOL32
        o += len(s)
    live = list(range(len(seqs)))
    for step in range(12):                             # decode together; one request leaves every fourth step
        if step in (4, 8):
            pm.cache.free_slot(slots[live.pop(1)])
        got = pm.forward([(slots[i], [tails[i][step]], [0]) for i in live])
        for k, i in enumerate(live):
            assert H.row_err(got[k:k + 1], refs[i][len(seqs[i]) + step][None]) < TOL32, (step, i)
    for i in live:
        pm.cache.free_slot(slots[i])


def test_mixed_step_of_portions_and_single_tokens(mixed):
    """One step may hold a fresh prompt, a later portion and a decoded token side by side."""
    cfg, om, pm = mixed
    a, b, c = toks(40, cfg["vocab"], 31), toks(50, cfg["vocab"], 32), toks(21, cfg["vocab"], 33)
    sa, sb, sc = (pm.cache.alloc_slot() for _ in range(3))
    pm.forward([(sa, a[:39], []), (sb, b[:20], [])])
    got = pm.forward([(sa, a[39:], [0]), (sb, b[20:], range(30)), (sc, c, range(21))])
    assert H.row_err(got[:1], O.forward(om, a)[39:]) < TOL32
    assert H.row_err(got[1:31], O.forward(om, b)[20:]) < TOL32
    assert H.row_err(got[31:], O.forward(om, c)) < TOL32
    for s in (sa, sb, sc):
        pm.cache.free_slot(s)


def test_freed_slots_are_used_again(mixed):
    """Nothing is cleared on free: the next owner of a slot must not see its predecessor's latents."""
    cfg, om, pm = mixed
    a, b = toks(80, cfg["vocab"], 5), toks(23, cfg["vocab"], 6)
    s = pm.cache.alloc_slot()
    pm.forward([(s, a, [])])
    pm.cache.free_slot(s)
    s2 = pm.cache.alloc_slot()
    assert s2 == s or pm.cache.live_slots == 1
    got = torch.cat([pm.forward([(s2, b[:7], range(7))])] + [pm.forward([(s2, [t], [0])]) for t in b[7:]])
    pm.cache.free_slot(s2)
    assert H.row_err(got, O.forward(om, b)) < TOL32


def test_long_decoding_with_a_growing_cache():
    cfg = dict(H.MIXED, layers=H.MIXED["layers"][:3])
    t = H.random_tensors(cfg, seed=7)
    om, pm = H.oracle_model(cfg, t), H.product_model(cfg, t, torch.float32, max_tokens=16)
    assert pm.cache.capacity == 16
    seq = toks(300, cfg["vocab"], 8)
    got = run(pm, [seq[:10]] + [[t] for t in seq[10:]])        # decode steps replay a graph; the cache doubles under it
    assert pm.cache.capacity >= 300
    assert H.row_err(got, O.forward(om, seq)) < TOL32


def test_other_sizes_and_bf16():
    t = H.random_tensors(H.ALIGNED, seed=3)
    om = H.oracle_model(H.ALIGNED, t)
    seq = toks(200, H.ALIGNED["vocab"], 9)
    ref = O.forward(om, seq)
    pm = H.product_model(H.ALIGNED, t, torch.float32)
    assert H.row_err(run(pm, [seq]), ref) < TOL32
    assert H.row_err(run(pm, cut(seq, [140, 2, 1, 1, 30])), ref) < TOL32
    pb = H.product_model(H.ALIGNED, t, torch.bfloat16)
    whole, parts = run(pb, [seq]), run(pb, [seq[:170]] + [[x] for x in seq[170:]])
    # bf16 operands: a token whose router scores nearly tie may take another expert, so the bound is on the typical row
    # and on how many rows stray, not on the worst one
    for a, b in ((whole, ref), (parts, ref), (parts, whole)):      # ... and the same numbers however the prompt was cut
        rows = H.row_errs(a, b)
        assert float(rows.median()) < 0.03 and float((rows > 0.1).double().mean()) < 0.05


def test_greedy_generation_through_engine_and_queue(mixed):
    from umbrella_b200.speculation.auto_engine import AutoEngine
    cfg, om, pm = mixed
    eng = AutoEngine.from_config("cuda:0", engine="batch", model=pm.model_name, dtype="float32", max_batch=2, temperature=0.0)
    eng.initialize()                                   # registry -> config reader -> checkpoint loader
    prompts = [toks(n, cfg["vocab"], 70 + n) for n in (5, 21, 2)]
    outs = eng.generate_batch(prompts, max_new_tokens=6)          # three requests, two slots: two batches
    assert eng.model.cache.live_slots == 0
    assert eng.generate(input_ids=prompts[1], max_new_tokens=6)["generated_tokens"] == outs[1]
    for p, out in zip(prompts, outs):
        seq = list(p)
        for tok in out:
            logits = O.forward(om, seq)[-1]
            best = int(logits.argmax())
            if best != tok:                            # only a near tie may differ
                assert float(logits[best] - logits[tok]) < 1e-3
            seq.append(tok)
    eng.update_generation_args(temperature=0.8, topk=8, topp=0.9)
    sampled = eng.generate_batch(prompts[:2], max_new_tokens=5)
    assert all(len(x) == 5 and all(0 <= y < cfg["vocab"] for y in x) for x in sampled)


def _random_config(rng):
    """Sizes, head counts, layer order, ranks, router shapes and constants drawn at random (odd ones included)."""
    layers = []
    for _ in range(rng.randint(2, 5)):
        heads, dim, rd = rng.choice([1, 2, 3, 6, 8]), rng.choice([8, 24, 40, 80, 128]), rng.choice([0, 4, 16, 24, 64])
        rot = None
        if rd:
            dims = rng.choice([rd, rd // 4 * 2]) or rd
            rot = dict(dims=dims, base=rng.choice([100.0, 1e4]), scaling=rng.choice(
                [None, dict(factor=rng.choice([2.0, 16.0]), original=rng.choice([32, 128]), fast=rng.choice([8.0, 32.0]), slow=rng.choice([1.0, 2.0]))]))
        kind = rng.choice(["dense", "moe", "moe", None])
        mlp = None
        if kind == "dense":
            mlp = dict(kind="dense", ff=rng.choice([40, 100, 144]))
        elif kind == "moe":
            groups = rng.choice([1, 2, 3, 5])
            per = rng.choice([1, 2, 4])
            keep = rng.randint(1, groups)
            mlp = dict(kind="moe", experts=groups * per, top=rng.randint(1, keep * per), groups=groups, keep=keep,
                       ff=rng.choice([24, 56, 96]), shared=rng.choice([None, 32, 72]))
        layers.append(dict(heads=heads, dim=dim, rot_dim=rd, vdim=rng.choice([dim, 16, 100]), kv_rank=rng.choice([12, 48, 100, 160]),
                           scale=(dim + rd) ** -0.5, rot=rot, mlp=mlp))
    return dict(width=rng.choice([72, 96, 200]), vocab=rng.choice([130, 301]), eps=rng.choice([1e-5, 1e-6]),
                embed_scale=rng.choice([1.0, 8.5]), residual_mult=rng.choice([1.0, 0.45]), layers=layers)


@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_random_configurations(seed):
    """Nothing rests on one model's sizes: random configurations, a ragged batch prefilled and decoded together."""
    import random
    cfg = _random_config(random.Random(seed))
    t = H.random_tensors(cfg, seed=seed)
    om, pm = H.oracle_model(cfg, t), H.product_model(cfg, t, torch.float32, max_tokens=32)
    seqs = [toks(n, cfg["vocab"], seed + n) for n in (150, 41, 97)]
    refs = [O.forward(om, s) for s in seqs]
    slots = [pm.cache.alloc_slot() for _ in seqs]
    cuts = [len(s) - 25 for s in seqs]
    out = pm.forward([(sl, s[:c], range(c)) for sl, s, c in zip(slots, seqs, cuts)])
    got = [[out[sum(cuts[:i]):sum(cuts[:i + 1])]] for i in range(3)]
    for d in range(25):
        o = pm.forward([(sl, [s[c + d]], [0]) for sl, s, c in zip(slots, seqs, cuts)])
        for i in range(3):
            got[i].append(o[i:i + 1])
    for i in range(3):
        assert H.row_err(torch.cat(got[i]), refs[i]) < TOL32, (seed, i)
