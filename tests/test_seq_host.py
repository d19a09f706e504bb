"""Host-side logic of the sequence-state decoders that needs no GPU: the family's config reader, the slot
bookkeeping of the state cache, the batch engine's queue, and the C ABI table against its header."""
import ctypes
import os
import re

import pytest
import torch

import seq_helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_config_reader_maps_every_key():
    from umbrella_b200.models.radanex import layer_tensor_names, spec_from_config
    spec = spec_from_config(H.config_json(H.MIXED))
    assert (spec.width, spec.vocab, spec.norm_groups, spec.norm_eps) == (64, 96, 2, 1e-5)
    lat, ret = spec.layers[0], spec.layers[1]
    assert (lat.mixer, lat.heads, lat.dim, lat.vdim, lat.q_rank, lat.kv_rank, lat.window, lat.scale) == \
        ("latent_attention", 2, 16, 24, 40, 48, 9, 0.3)
    assert (ret.mixer, ret.rot_dims, ret.rot_base, ret.decay) == ("retention", 8, 100.0, [0.9, 0.97, 0.9990234375])
    assert spec.layers[2].mlp is None and spec.layers[1].mlp.shared_ff == 0
    assert spec.layers[4].mlp.experts == 0 and spec.layers[4].mlp.shared_ff == 24 and spec.layers[3].mlp.top == 1
    names = layer_tensor_names(spec, 3)
    assert names["experts"][2] == ("l3.mlp.e2.gate", "l3.mlp.e2.up", "l3.mlp.e2.down") and names["depth"] == "l3.dwa"
    assert set(n for i in range(5) for v in layer_tensor_names(spec, i).values()
               for n in ([v] if isinstance(v, str) else [x for y in v for x in ([y] if isinstance(y, str) else y)])) \
        | {"embed", "head", "final.norm"} == set(H.random_tensors(H.MIXED))
    with pytest.raises(ValueError):
        spec_from_config(dict(H.config_json(H.MIXED), architecture="Other"))


def test_auto_model_picks_the_family_from_config_json(tmp_path):
    from umbrella_b200.models.auto_model import AutoModelLM
    from umbrella_b200.models.radanex import Radanex
    path = H.write_checkpoint(str(tmp_path / "m"), H.ALIGNED, H.random_tensors(H.ALIGNED))
    m = AutoModelLM.from_pretrained(path, device="cuda:0", dtype=torch.float32)
    assert isinstance(m, Radanex) and m.num_layers == 2 and m.dtype == torch.float32


def test_state_cache_slots():
    from umbrella_b200.attn.state_cache import SequenceStateCache
    from umbrella_b200.models.radanex import spec_from_config
    spec = spec_from_config(H.config_json(H.MIXED))
    c = SequenceStateCache(spec, slots=2, device="cpu", dtype=torch.float32, max_length=20)
    assert c.ring[0].shape == (2, 9, 48) and c.ring[2].shape == (2, 20, 48)        # window 33 capped by max_length
    assert c.ret_state[1].shape == (2, 3, 16, 32) and c.shift[4].shape == (2, 2, 64) and c.ring[1] is None
    a, b = c.alloc_slot(), c.alloc_slot()
    c.ret_state[1][b].fill_(3.0)
    c.advance(b, 5)
    assert (c.position[b], c.parity[b]) == (5, 1)
    d = c.alloc_slot()                                               # full: the cache doubles and keeps its contents
    assert c.slots == 4 and d == 2 and float(c.ret_state[1][b].min()) == 3.0 and c.position[b] == 5
    c.free_slot(b)
    with pytest.raises(ValueError):
        c.free_slot(b)
    assert c.live_slots == 2
    e = c.alloc_slot()
    assert e == 3 and c.alloc_slot() == b and c.position[b] == 0 and c.parity[b] == 0       # freed slots go to the back


class _FakeModel:
    """Counts the steps; the 'logits' make token (last input + 1) the arg-max."""
    eos_tokens = [7]
    device = "cpu"

    def __init__(self):
        from umbrella_b200.attn.state_cache import SequenceStateCache
        from umbrella_b200.models.radanex import spec_from_config
        self.cache = SequenceStateCache(spec_from_config(H.config_json(H.ALIGNED)), slots=2, device="cpu", dtype=torch.float32)
        self.steps = []

    def forward(self, entries):
        self.steps.append([(s, len(t)) for s, t, _ in entries])
        rows = []
        for s, t, w in entries:
            self.cache.advance(s, len(t))
            for i in w:
                row = torch.zeros(16)
                row[(t[i] + 1) % 16] = 1.0
                rows.append(row)
        return torch.stack(rows)


def test_batch_engine_queue_and_slots():
    from umbrella_b200.speculation.auto_engine import AutoEngine
    eng = AutoEngine.from_config("cpu", engine="batch", model="unused", max_batch=2, max_tokens=10)
    fake = _FakeModel()
    eng.initialize(model=fake)
    eng.sample = lambda logits: logits.argmax(-1)
    outs = eng.generate_batch([[1, 2, 3], [4, 5], [9, 9, 9, 9, 9, 9, 9, 9, 9], [0]], max_new_tokens=4)
    assert outs == [[4, 5, 6, 7], [6, 7], [10, 11, 12, 13], [1, 2, 3, 4]]           # 7 is EOS: request 1 leaves early
    assert fake.steps[0] == [(0, 3), (1, 2)]                   # first batch: two requests, prompts in one ragged step
    assert fake.steps[1] == [(0, 1), (1, 1)] and fake.steps[2] == [(0, 1)]          # the shorter one has left
    # second batch: the 9-token prompt alone would fit with the 1-token one only under max_tokens = 10
    assert [len(s) for s in fake.steps[4:6]] == [2, 2] and fake.cache.live_slots == 0
    with pytest.raises(ValueError):
        AutoEngine.from_config("cpu", engine="nope", model="m")


def test_seq_abi_table_matches_header_and_library():
    from umbrella_b200 import _lib_seq, build
    text = open(os.path.join(ROOT, "include", "umbrella_b200_seq.h")).read()
    declared = sorted(set(re.findall(r"\b(umbs_[a-z0-9_]+)\s*\(", text)))
    assert declared == sorted(_lib_seq.SIGNATURES)
    lib = ctypes.CDLL(build.build_seq())                              # nvcc cross-compiles without a GPU
    for n in declared:
        assert hasattr(lib, n), n
    lib.umbs_version.restype = ctypes.c_char_p
    assert lib.umbs_version().startswith(b"umbrella_b200_seq")


# ---------------------------------------------------------------------------------------------- the Zedotar family
def test_zedotar_config_reader_and_tensor_names():
    import zed_helpers as Z
    from umbrella_b200.models.zedotar import layer_tensor_names, spec_from_config
    spec = spec_from_config(Z.config_json(Z.MIXED))
    assert (spec.width, spec.vocab, spec.norm_eps, spec.norm_offset, spec.logit_softcap) == (64, 96, 1e-5, 1.0, 12.0)
    ml, at, a2 = spec.layers[0], spec.layers[1], spec.layers[2]
    assert all(l.form == "prenorm" and not l.shift and not l.depth_average and l.norm_offset == 1.0 for l in spec.layers)
    assert (ml.mixer, ml.heads, ml.dim, ml.vdim, ml.gate_cap, ml.mlp.shared_ff, ml.mlp.act) == ("mlstm", 3, 16, 20, 10.0, 48, "gelu_tanh")
    assert (at.mixer, at.attn_mode, at.gate_kind, at.kv_heads, at.window, at.pool, at.taps, at.values_are_keys, at.bias, at.head_bias) == \
        ("cached_attention", "softmax_sink", 1, 2, 9, 4, 1, False, True, False)
    assert (a2.mixer, a2.attn_mode, a2.gate_kind, a2.window, a2.pool, a2.taps, a2.values_are_keys, a2.head_bias, a2.mlp) == \
        ("cached_attention", "sigmoid", 2, 0, 0, 3, True, True, None)
    assert spec.layers[3].rot_dims == 0 and spec.layers[3].inv_freq is None and spec.layers[5].taps == 1
    assert spec_from_config(Z.config_json(Z.ALIGNED)).logit_softcap == 0.0
    names = {n for i in range(len(spec.layers)) for v in layer_tensor_names(spec, i).values() for n in ([v] if isinstance(v, str) else v)}
    assert names | {"embed", "head", "final.norm"} == set(Z.random_tensors(Z.MIXED))
    bad = Z.config_json(Z.MIXED)
    bad["layers"][2]["mixer"]["vdim"] = 24                            # values are the keys: vdim must equal dim
    with pytest.raises(ValueError):
        spec_from_config(bad)
    with pytest.raises(ValueError):
        spec_from_config(dict(Z.config_json(Z.MIXED), architecture="Radanex"))


def test_zedotar_rotary_frequencies_match_the_plain_statement():
    import zed_helpers as Z
    from oracle import zedotar as O
    from umbrella_b200.models.zedotar import spec_from_config
    cfg = dict(Z.MIXED, layers=[dict(Z.ATT, ff=None), dict(Z.AT2, ff=None),
                                dict(Z.ATT, rot=dict(dims=16, base=500.0, scaling=dict(factor=8.0, low=0.5, high=2.0, original=12)), ff=None),
                                dict(Z.AT2, rot=dict(dims=16, base=40.0, scaling=dict(factor=4.0, original=64, fast=16.0, slow=2.0)), ff=None)])
    spec = spec_from_config(Z.config_json(cfg))
    for L, l in zip(cfg["layers"], spec.layers):
        f, mag = O.rotary_frequencies(Z._rot(L))
        assert torch.allclose(torch.tensor(l.inv_freq, dtype=torch.float64), f, rtol=1e-12, atol=0)
        assert abs(l.rot_mag - mag) < 1e-12
    f = [x for l in spec.layers for x in l.inv_freq]
    assert len(set(f)) > len(f) // 2                                  # the rules leave distinct frequencies (no collapse)


def test_state_cache_of_cached_attention_and_mlstm_layers():
    import zed_helpers as Z
    from umbrella_b200.attn.state_cache import SequenceStateCache
    from umbrella_b200.models.zedotar import spec_from_config
    spec = spec_from_config(Z.config_json(Z.MIXED))
    c = SequenceStateCache(spec, slots=2, device="cpu", dtype=torch.float32, capacity=24)
    assert c.capacity == 24 and c.mlstm_state[0].shape == (2, 3, 16 * 21 + 1) and c.shift[0] is None
    assert c.kv_cache[1].shape == (2, 9, 2 * 40) and c.pool_cache[1].shape == (2, 6, 80)          # ring of the window; 24 / 4 blocks
    assert c.kv_cache[2].shape == (2, 24, 2 * 32) and c.conv_state[2].shape == (2, 2, 2, 96) and c.pool_cache[2] is None
    assert c.kv_cache[6].shape == (2, 7, 40)                                                       # blocks larger than the window
    c.kv_cache[2][1, 23].fill_(4.0), c.pool_cache[1][1, 5].fill_(2.0), c.mlstm_state[0][1].fill_(1.5)
    v = c.version
    c.reserve_length(24)
    assert c.version == v
    c.reserve_length(25)                                              # the growing parts double and keep their rows
    assert c.capacity == 48 and c.version > v
    assert c.kv_cache[2].shape == (2, 48, 64) and float(c.kv_cache[2][1, 23].min()) == 4.0 and float(c.kv_cache[2][1, 24:].abs().max()) == 0
    assert c.pool_cache[1].shape == (2, 12, 80) and float(c.pool_cache[1][1, 5].min()) == 2.0
    assert c.kv_cache[1].shape == (2, 9, 80) and float(c.mlstm_state[0][1].min()) == 1.5
    s = [c.alloc_slot() for _ in range(3)]                            # more slots: every part keeps what it holds
    assert c.slots == 4 and c.kv_cache[2].shape == (4, 48, 64) and float(c.kv_cache[2][1, 23].min()) == 4.0
    capped = SequenceStateCache(spec, slots=1, device="cpu", dtype=torch.float32, max_length=30)
    with pytest.raises(RuntimeError):
        capped.reserve_length(31)


# ---------------------------------------------------------------------------------------------- the Kulisun family
def test_kulisun_config_reader_and_tensor_names():
    import kul_helpers as U
    from umbrella_b200.models.kulisun import layer_tensor_names, spec_from_config
    spec = spec_from_config(U.config_json(U.MIXED))
    assert (spec.width, spec.vocab, spec.norm_eps, spec.norm_kind, spec.embed_scale) == (64, 96, 1e-5, "layer", 3.0)
    assert all(l.form == "prenorm" and l.mixer == "latent_attention" and l.q_rank == 0 and l.window == 0 and l.norm_kind == "layer"
               and l.layer_scale and l.residual_mult == 0.6 and l.attn_mode == "softmax_sink" and l.learned_sink and l.gate_kind == 2
               and not l.shift and not l.depth_average for l in spec.layers)
    a, b, c, d, e = spec.layers[:5]
    assert (a.heads, a.dim, a.rope_dim, a.vdim, a.kv_rank, a.scale, a.rot_dims) == (4, 16, 8, 24, 40, 0.2, 8)
    assert (a.mlp.experts, a.mlp.shared_ff, a.mlp.act, a.mlp.bias, a.mlp.shared_gate) == (0, 48, "silu", True, False)
    assert (b.mlp.experts, b.mlp.top, b.mlp.groups, b.mlp.keep, b.mlp.ff, b.mlp.shared_ff, b.mlp.route, b.mlp.shared_gate, b.mlp.bias) == \
        (8, 3, 4, 2, 24, 32, "sigmoid_groups", True, False)
    assert c.mlp is None and (c.rot_dims, c.rope_dim, c.rot_mag) == (4, 8, 1.0) and len(c.inv_freq) == 2
    assert (d.rope_dim, d.rot_dims, d.inv_freq, d.mlp.shared_ff, d.mlp.groups, d.mlp.top) == (0, 0, None, 0, 1, 1)
    assert e.rot_mag == pytest.approx(0.1 * __import__("math").log(8.0) + 1.0) and spec.layers[5].rot_dims == 0
    names = set()
    for i in range(len(spec.layers)):
        for v in layer_tensor_names(spec, i).values():
            names |= {v} if isinstance(v, str) else set(v) if isinstance(v, tuple) else {n for trio in v for n in trio}
    assert names | {"embed", "head", "final.norm", "final.norm.b"} == set(U.random_tensors(U.MIXED))
    bad = U.config_json(U.MIXED)
    bad["layers"][1]["mlp"]["router"]["top"] = 5                      # two groups of two experts hold no five
    with pytest.raises(ValueError):
        spec_from_config(bad)
    with pytest.raises(ValueError):
        spec_from_config(dict(U.config_json(U.MIXED), architecture="Zedotar"))


def test_kulisun_rotary_frequencies_match_the_plain_statement():
    import kul_helpers as U
    from oracle import kulisun as O
    from umbrella_b200.models.kulisun import spec_from_config
    spec = spec_from_config(U.config_json(U.MIXED))
    for L, l in zip(U.MIXED["layers"], spec.layers):
        if not l.rot_dims:
            continue
        f, mag = O.rotary_frequencies(U._rot(L))
        assert torch.allclose(torch.tensor(l.inv_freq, dtype=torch.float64), torch.tensor(f, dtype=torch.float64), rtol=1e-12, atol=0)
        assert abs(l.rot_mag - mag) < 1e-12


def test_state_cache_of_windowless_latent_attention():
    import kul_helpers as U
    from umbrella_b200.attn.state_cache import SequenceStateCache
    from umbrella_b200.models.kulisun import spec_from_config
    spec = spec_from_config(U.config_json(U.MIXED))
    c = SequenceStateCache(spec, slots=2, device="cpu", dtype=torch.float32, capacity=24)
    assert c.ring[0].shape == (2, 24, 48) and c.ring[3].shape == (2, 24, 40) and c.ring[4].shape == (2, 24, 32)   # latent + shared part
    assert c.shift[0] is None and c.kv_cache[0] is None
    c.ring[0][1, 23].fill_(4.0)
    v = c.version
    c.reserve_length(24)
    assert c.version == v
    c.reserve_length(30)                                              # the rows double and keep their index
    assert c.capacity == 48 and c.version > v and c.ring[0].shape == (2, 48, 48)
    assert float(c.ring[0][1, 23].min()) == 4.0 and float(c.ring[0][1, 24:].abs().max()) == 0
    s = [c.alloc_slot() for _ in range(3)]
    assert c.slots == 4 and c.ring[0].shape == (4, 48, 48) and float(c.ring[0][1, 23].min()) == 4.0


# ---------------------------------------------------------------------------------------------- the Subivik family
def test_subivik_config_reader_and_tensor_names():
    import sub_helpers as SH
    from umbrella_b200.models.subivik import layer_tensor_names, spec_from_config
    spec = spec_from_config(SH.MIXED)
    assert spec.norm_kind == "dyt" and spec.pos_embed == "sinusoid" and spec.width == 80 and spec.norm_eps == 1e-5
    a, p, b = spec.layers[0], spec.layers[1], spec.layers[2]
    assert (a.mixer, a.maps, a.chunk, a.kv_heads, a.diff, a.head_unit_norm, a.qk_norm, a.gate_kind) == \
        ("cached_attention", 2, 16, 2, 0.25, True, True, 2)
    assert (a.mlp.route, a.mlp.experts, a.mlp.top, a.mlp.route_scale, a.mlp.act) == ("softmax_all", 5, 2, 1.7, "silu")
    assert (p.mixer, p.talk, p.dist_bias, p.softcap, p.maps, p.chunk) == ("cached_attention", True, True, 6.0, 1, 0)
    assert (p.second.mixer, p.second.heads, p.second.dim, p.second.vdim) == ("time_mix", 3, 20, 20)
    assert (p.mix_scale, p.second_scale, p.mlp.plain, p.mlp.shared_ff) == (0.6, 1.3, "xielu", 48)
    assert b.kv_from == 0 and b.chunk == 24 and b.mlp is None and spec.layers[3].softcap == 0.0 and spec.layers[4].chunk == 0
    n0, n1, n2 = (layer_tensor_names(spec, i) for i in range(3))
    assert n0["q_norm"] == "l0.mix.q.norm" and n0["k"] == "l0.mix.k" and n0["experts"][4][2] == "l0.mlp.e4.down"
    assert n1["talk"] == "l1.mix.left.talk" and n1["second"]["mu_w"] == "l1.mix.right.mu.w" and n1["dense_act"] == "l1.mlp.act"
    assert "k" not in n2 and "k_norm" not in n2 and "norm2" not in n2 and n2["lq2"] == "l2.mix.lq2"
    every = set()
    for i in range(len(spec.layers)):
        def walk(v):
            if isinstance(v, dict):
                [walk(x) for x in v.values()]
            elif isinstance(v, (list, tuple)):
                [walk(x) for x in v]
            else:
                every.add(v)
        walk(layer_tensor_names(spec, i))
    assert every | {"embed", "final.norm", "final.norm.b", "final.norm.alpha"} == set(SH.random_tensors(SH.MIXED))
    bad = dict(SH.MIXED, layers=[SH.attention(2, 1, 8, 8, kv_from=0)])
    with pytest.raises(ValueError):
        spec_from_config(bad)                                       # a layer cannot borrow from itself or a later one


def test_state_cache_of_subivik_layers():
    import sub_helpers as SH
    from umbrella_b200.attn.state_cache import SequenceStateCache
    from umbrella_b200.models.subivik import spec_from_config
    spec = spec_from_config(SH.MIXED)
    c = SequenceStateCache(spec, slots=2, device="cpu", dtype=torch.float32, capacity=32)
    assert len(c.units) == 8 and spec.layers[1].second.state_index == 6 and spec.layers[3].second.state_index == 7
    assert c.kv_cache[0].shape == (2, 24, 2 * (2 * 12 + 20))        # a ring as long as the borrower's wider chunk
    assert c.kv_cache[1].shape == (2, 32, 3 * (10 + 14))            # the whole sequence
    assert c.kv_cache[2] is None and c.kv_cache[5] is None          # borrowers keep nothing
    assert c.kv_cache[4].shape == (2, 32, 16 + 16 + 16)
    assert c.tm_state[6].shape == (2, 3, 20, 20) and c.shift[6].shape == (2, 2, 80) and c.shift[1] is None
    c.reserve_length(70)
    assert c.capacity == 128 and c.kv_cache[0].shape[1] == 24 and c.kv_cache[1].shape[1] == 128 and c.kv_cache[4].shape[1] == 128
