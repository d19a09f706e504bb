"""The Subivik family on the GPU against the plain oracle (oracle/subivik.py): whole prompts and every layer's stream,
the first tokens, decoding token by token through the cache and the recurrent state, prompts cut into portions, ragged
batches, reused slots, long decoding across chunk borders with a growing cache, other sizes, both dtypes, greedy generation
through the engine and its queue."""
import pytest
import torch

import sub_helpers as H
from oracle import subivik as O

pytestmark = pytest.mark.gpu
TOL32 = 3e-5          # fp32 product vs float64 oracle: per-row rms of the logit difference over the logits' rms
TOL_DEEP = 6e-5       # random stacks of several large recurrent heads: fp32 rounding of the decays compounds over the tokens


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
    ref, streams = O.forward(om, seq)
    slot = pm.cache.alloc_slot()
    got, ly = pm.forward([(slot, seq, range(len(seq)))], layer_out=True)
    pm.cache.free_slot(slot)
    for i in range(len(cfg["layers"])):
        assert H.row_err(ly[i], streams[i]) < TOL32, f"layer {i}"
    assert H.row_err(got, ref) < TOL32


def test_first_tokens(mixed):
    cfg, om, pm = mixed
    for n in (1, 2, 3):
        seq = toks(n, cfg["vocab"], 10 + n)
        assert H.row_err(run(pm, [seq]), O.forward(om, seq)[0]) < TOL32


def test_prefill_then_token_by_token(mixed):
    cfg, om, pm = mixed
    seq = toks(75, cfg["vocab"], 3)
    ref = O.forward(om, seq)[0]
    for first in (1, 6, 30):
        got = run(pm, [seq[:first]] + [[t] for t in seq[first:]])
        assert H.row_err(got, ref) < TOL32, first


def test_portions_down_to_two_tokens(mixed):
    cfg, om, pm = mixed
    seq = toks(90, cfg["vocab"], 4)
    ref = O.forward(om, seq)[0]
    # cuts at, just before and just behind the chunk borders (16, 24, 7 and their multiples) among others
    for sizes in ([2, 2, 2, 3, 1, 2, 17, 4, 31], [64, 2], [3] * 30, [5, 64], [1, 2, 70], [16, 16, 16, 24], [15, 2, 7, 24, 1, 23],
                  [48, 2, 2], [33, 31]):
        assert H.row_err(run(pm, cut(seq, sizes)), ref) < TOL32, sizes


def test_unequal_batch_equals_each_alone(mixed):
    cfg, om, pm = mixed
    seqs = [toks(n, cfg["vocab"], 20 + n) for n in (1, 37, 66, 9)]
    tails = [toks(12, cfg["vocab"], 50 + len(s)) for s in seqs]
    refs = [O.forward(om, s + tl)[0] for s, tl in zip(seqs, tails)]
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
    assert H.row_err(got[:1], O.forward(om, a)[0][39:]) < TOL32
    assert H.row_err(got[1:31], O.forward(om, b)[0][20:]) < TOL32
    assert H.row_err(got[31:], O.forward(om, c)[0]) < TOL32
    for s in (sa, sb, sc):
        pm.cache.free_slot(s)


def test_freed_slots_are_used_again(mixed):
    """Nothing is cleared on free: the next owner of a slot must not see its predecessor's keys, memory or last row."""
    cfg, om, pm = mixed
    a, b = toks(80, cfg["vocab"], 5), toks(23, cfg["vocab"], 6)
    s = pm.cache.alloc_slot()
    pm.forward([(s, a, [])])
    pm.cache.free_slot(s)
    s2 = pm.cache.alloc_slot()
    assert s2 == s or pm.cache.live_slots == 1
    got = torch.cat([pm.forward([(s2, b[:7], range(7))])] + [pm.forward([(s2, [t], [0])]) for t in b[7:]])
    pm.cache.free_slot(s2)
    assert H.row_err(got, O.forward(om, b)[0]) < TOL32


def test_long_decoding_with_a_growing_cache():
    """300 tokens, most of them decoded one by one: the chunked rings wrap many times, the lender's ring serves a borrower
    with a wider chunk, the whole-sequence caches double under the replayed graph, the memory decays over hundreds of steps."""
    cfg = H.MIXED
    t = H.random_tensors(cfg, seed=7)
    om, pm = H.oracle_model(cfg, t), H.product_model(cfg, t, torch.float32, max_tokens=16)
    assert pm.cache.capacity == 16
    seq = toks(300, cfg["vocab"], 8)
    got = run(pm, [seq[:10]] + [[t] for t in seq[10:]])
    assert pm.cache.capacity >= 300
    assert H.row_err(got, O.forward(om, seq)[0]) < TOL32


def test_other_sizes_and_bf16():
    t = H.random_tensors(H.ALIGNED, seed=3)
    om = H.oracle_model(H.ALIGNED, t)
    seq = toks(200, H.ALIGNED["vocab"], 9)
    ref = O.forward(om, seq)[0]
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
            logits = O.forward(om, seq)[0][-1]
            best = int(logits.argmax())
            if best != tok:                            # only a near tie may differ
                assert float(logits[best] - logits[tok]) < 1e-3
            seq.append(tok)
    eng.update_generation_args(temperature=0.8, topk=8, topp=0.9)
    sampled = eng.generate_batch(prompts[:2], max_new_tokens=5)
    assert all(len(x) == 5 and all(0 <= y < cfg["vocab"] for y in x) for x in sampled)


def _random_config(rng):
    """Sizes, head counts, layer order, chunks, ranks, router shapes and constants drawn at random (odd ones included)."""
    layers, lenders = [], []
    for i in range(rng.randint(2, 6)):
        kind = rng.choice(["dense", "moe", "moe", None])
        mlp = None
        if kind == "dense":
            mlp = H.dense(rng.choice([40, 100, 144]))
        elif kind == "moe":
            experts = rng.choice([1, 2, 5, 9])
            mlp = H.moe(experts, rng.randint(1, experts), rng.choice([24, 56, 96]), scale=rng.choice([1.0, 0.3, 2.5]))
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            lf = H.left(kv * rng.choice([1, 2, 4]), kv, rng.choice([8, 24, 40, 72]), rng.choice([8, 20, 100]), softcap=rng.choice([0, 4.0, 30.0]))
            layers.append(H.parallel(lf, rng.choice([1, 2, 5]), rng.choice([8, 20, 36, 64, 100]),
                                     scales=(rng.choice([1.0, 0.7]), rng.choice([1.0, 1.4])), mlp=mlp))
        elif lenders and rng.random() < 0.5:
            j = rng.choice(lenders)
            m = layers[j]["mixer"]
            layers.append(H.attention(m["heads"], m["kv_heads"], m["dim"], m["vdim"], chunk=rng.choice([0, 5, 32, 50]),
                                      diff=rng.choice([0.1, 0.5]), kv_from=j, mlp=mlp))
        else:
            kv = rng.choice([1, 2])
            layers.append(H.attention(kv * rng.choice([1, 3]), kv, rng.choice([8, 20, 48]), rng.choice([8, 28, 64]),
                                      chunk=rng.choice([0, 1, 9, 32, 64]), diff=rng.choice([0.05, 0.3]), mlp=mlp))
            lenders.append(i)
    return H.model(rng.choice([72, 96, 200]), rng.choice([130, 301]), layers, eps=rng.choice([1e-5, 1e-6]))


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_random_configurations(seed):
    """Nothing rests on one model's sizes: random configurations, a ragged batch prefilled and decoded together."""
    import random
    cfg = _random_config(random.Random(seed))
    t = H.random_tensors(cfg, seed=seed)
    om, pm = H.oracle_model(cfg, t), H.product_model(cfg, t, torch.float32, max_tokens=32)
    seqs = [toks(n, cfg["vocab"], seed + n) for n in (150, 41, 97)]
    refs = [O.forward(om, s)[0] for s in seqs]
    slots = [pm.cache.alloc_slot() for _ in seqs]
    cuts = [len(s) - 25 for s in seqs]
    out = pm.forward([(sl, s[:c], range(c)) for sl, s, c in zip(slots, seqs, cuts)])
    got = [[out[sum(cuts[:i]):sum(cuts[:i + 1])]] for i in range(3)]
    for d in range(25):
        o = pm.forward([(sl, [s[c + d]], [0]) for sl, s, c in zip(slots, seqs, cuts)])
        for i in range(3):
            got[i].append(o[i:i + 1])
    for i in range(3):
        assert H.row_err(torch.cat(got[i]), refs[i]) < TOL_DEEP, (seed, i)


def test_bf16_at_sizes_no_tensor_core_tile_takes(mixed):
    """bf16 with widths and head sizes that are no multiple of a tile: the products fall back to their plain kernels, the
    cache rows are bf16, and a prompt cut into portions and decoded gives the numbers of the whole prompt within rounding."""
    cfg, om, _ = mixed
    pb = H.product_model(cfg, H.random_tensors(cfg, seed=1), torch.bfloat16)
    seq = toks(120, cfg["vocab"], 41)
    ref = O.forward(om, seq)[0]
    whole, parts = run(pb, [seq]), run(pb, cut(seq, [50, 2, 31]) [:3] + [[x] for x in seq[83:]])
    for a, b in ((whole, ref), (parts, ref), (parts, whole)):
        rows = H.row_errs(a, b)
        assert float(rows.median()) < 0.04 and float((rows > 0.15).double().mean()) < 0.05
