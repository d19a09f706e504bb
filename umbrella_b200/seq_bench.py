"""Throughput of the sequence-state decoder family beside the framework's Llama at equal size (``bench.py --workload
radanex``): prefill and decode tokens/s of whole models with seeded random weights at layer sizes a real model has,
and the device time of each mechanism's kernels against its roofline, next to the like kernel of the Llama path.

Timing: CUDA events on the launching stream, 3 warm-up runs, a write over a buffer larger than L2 between timed runs
of the kernel table (the whole-model runs read more than L2 by themselves), synchronize on both sides.
"""
from __future__ import annotations

import json
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, "fallback"


def radanex_config(width: int, layers: int = 8, latent_every: int = 4, window: int = 1024) -> dict:
    """A Radanex config with the layer sizes of a model of this width: every fourth layer latent attention (or every
    ``latent_every``-th, over the last ``window`` tokens)."""
    heads = width // 128
    ret = dict(type="retention", mixer=dict(heads=heads, dim=64, vdim=128, rot=dict(dims=64, base=1e6),
                                           decay=[1 - 2.0 ** (-5 - (3 * h) // heads) for h in range(heads)]))
    lat = dict(type="latent_attention", mixer=dict(heads=heads, dim=64, vdim=128, q_rank=3 * width // 8, kv_rank=width // 4,
                                                   scale=0.125, mask=dict(size=window)))
    mlp = dict(kind="moe", router=dict(experts=16, top=2), expert=dict(ff=width // 2, limit=7.0),
               shared=dict(ff=width, limit=7.0))
    return dict(architecture="Radanex", width=width, vocab=32768, norm=dict(eps=1e-6, groups=4),
                layers=[dict(lat if i % latent_every == latent_every - 1 else ret, mlp=mlp) for i in range(layers)])


class Timer:
    def __init__(self, device):
        self.flush = torch.empty(192 << 20, dtype=torch.uint8, device=device)      # > the 126 MB L2

    def __call__(self, fn, reps=5, warm=3, flush=True):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(reps):
            if flush:
                self.flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total / reps


def zedotar_config(width: int, layers: int = 8) -> dict:
    """A Zedotar config with the layer sizes of a model of this width: mLSTM layers with a windowed attention layer as
    every fourth and a convolved sigmoid-attention layer as the last; dense feed-forward of the width Radanex activates."""
    heads = width // 128
    rot = dict(dims=64, base=1e6)
    mls = dict(type="mlstm", mixer=dict(heads=heads, dim=64, vdim=128, gate_cap=15.0))
    att = dict(type="attention", mixer=dict(heads=heads, kv_heads=max(1, heads // 4), dim=128, vdim=128, scale=128 ** -0.5,
                                            mask=dict(size=1024, pool=64),
                                            rot=dict(rot, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192))))
    at2 = dict(type="attention_2", mixer=dict(heads=heads, kv_heads=max(1, heads // 4), dim=128, vdim=128, conv=4, scale=128 ** -0.5,
                                              rot=dict(rot, scaling=dict(factor=4.0, original=4096, fast=32.0, slow=1.0))))
    mlp = dict(kind="dense", ff=2 * width)
    kinds = [at2 if i == layers - 1 else (att if i % 4 == 3 else mls) for i in range(layers)]
    return dict(architecture="Zedotar", width=width, vocab=32768, norm=dict(eps=1e-6), logit_softcap=30.0,
                layers=[dict(k, mlp=mlp) for k in kinds])


def bench_radanex(width, layers, device, prompt, ctx, batches, timer, **config):
    from .models.radanex import Radanex, spec_from_config
    spec = spec_from_config(radanex_config(width, layers, **config))
    m = Radanex(spec, device=device, dtype=torch.bfloat16, slots=max(batches))
    return bench_seq_model(m, spec, prompt, ctx, batches, timer)


def bench_zedotar(width, layers, device, prompt, ctx, batches, timer):
    from .models.zedotar import Zedotar, spec_from_config
    spec = spec_from_config(zedotar_config(width, layers))
    m = Zedotar(spec, device=device, dtype=torch.bfloat16, slots=max(batches), max_tokens=prompt + ctx)
    return bench_seq_model(m, spec, prompt, ctx, batches, timer)


def bench_seq_model(m, spec, prompt, ctx, batches, timer):
    m.alloc()
    m.load_synthetic(7)
    g = torch.Generator().manual_seed(0)
    toks = lambda n: torch.randint(0, spec.vocab, (n,), generator=g).tolist()
    out = {"weight_gb": m.weight_bytes() / 1e9, "state_mb_per_sequence": m.cache.state_bytes_per_slot() / 1e6}

    def prefill(n_seq):
        ps = [toks(prompt) for _ in range(n_seq)]

        def run():
            slots = [m.cache.alloc_slot() for _ in ps]
            m.forward([(s, p, [prompt - 1]) for s, p in zip(slots, ps)])
            for s in slots:
                m.cache.free_slot(s)
        return run
    for n_seq in (1, 4):
        ms = timer(prefill(n_seq), reps=3, flush=False)
        out[f"prefill_{n_seq}x{prompt}_tok_s"] = n_seq * prompt / ms * 1e3
    for B in batches:
        slots = [m.cache.alloc_slot() for _ in range(B)]
        m.forward([(s, toks(ctx), []) for s in slots])
        nxt = toks(B)
        ms = timer(lambda: m.forward([(s, [t], [0]) for s, t in zip(slots, nxt)]), reps=20, flush=False)
        out[f"decode_b{B}_tok_s"] = B / ms * 1e3
        out[f"decode_b{B}_ms_per_step"] = ms
        for s in slots:
            m.cache.free_slot(s)
    return m, out


def bench_llama(width, layers, inter, device, prompt, ctx, timer):
    from .models import llama as L
    heads = width // 128
    shape = L.LlamaShape(hidden_size=width, intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=heads,
                         num_key_value_heads=max(1, heads // 4), vocab_size=32768, rope_scaling=None, rope_theta=1e6)
    m = L.SyntheticLlama(shape, max_length=prompt + ctx + 64, awq=False, seed=7, device=device, gen_device=device)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 32768, (prompt,), generator=g).to(device)
    pos = torch.arange(prompt, device=device)
    out = {"weight_gb": m.weight_bytes() / 1e9}

    def prefill():
        m.clear()
        m.prefill_forward(ids, pos)
    out[f"prefill_1x{prompt}_tok_s"] = prompt / timer(prefill, reps=3, flush=False) * 1e3
    m.clear()
    m.prefill_forward(ids[:ctx], pos[:ctx])
    one, p1 = ids[:1].clone(), torch.tensor([ctx], device=device)

    def decode():
        m.kv_cache.kv_offset = ctx
        m.prefill_forward(one, p1)
    ms = timer(decode, reps=20, flush=False)
    out["decode_b1_tok_s"], out["decode_b1_ms_per_step"] = 1e3 / ms, ms
    return m, out


def kernel_table(rm, lm, device, timer, T=4096):
    """Device time of each mechanism at prefill size (T tokens) and at decode size (8 tokens), with its roofline
    fraction: bytes / measured copy bandwidth, or FLOPs / measured bf16 GEMM throughput for the tensor-core products.
    The fp32 mechanisms (recurrence, scores, norms) have no tensor-core peak to be held against: their bound is the
    bytes they must move, which is what the fraction states."""
    from . import ops, ops_seq as Q
    hbm, tflops, how = _peaks()
    sp = rm.spec
    W = sp.width
    ret = next(l for l in sp.layers if l.mixer == "retention")
    lat = next(l for l in sp.layers if l.mixer == "latent_attention")
    ri, li = sp.layers.index(ret), sp.layers.index(lat)
    rw, lw = rm.weights[ri], rm.weights[li]
    rows = []

    fp32_peak = 148 * 128 * 2 * 1.965e-3            # TFLOP/s: 148 SMs x 128 fp32 FMA lanes at the maximum SM clock (nominal)

    def add(name, ms, nbytes=0, flops=0, like=None, flops32=0):
        r = dict(kernel=name, ms=round(ms, 4))
        if flops32:
            r["fp32_tflops"], r["frac_of_fp32_fma_peak"] = round(flops32 / ms / 1e9, 2), round(flops32 / ms / 1e9 / fp32_peak, 3)
        if flops:
            r["tflops"], r["frac_of_bf16_peak"] = round(flops / ms / 1e9, 1), round(flops / ms / 1e9 / tflops, 3)
        if nbytes:
            r["gb_s"], r["frac_of_hbm_peak"] = round(nbytes / ms / 1e6, 1), round(nbytes / ms / 1e6 / hbm, 3)
        if like:
            r["like"] = like
        rows.append(r)
    bf = dict(dtype=torch.bfloat16, device=device)
    for n, tag in ((T, f"prefill T={T}"), (8, "decode T=8")):
        nseq = 1 if n == T else 8
        per = n // nseq
        batch = Q.RaggedBatch([(s, per, 0 if n == T else 512, 0) for s in range(nseq)], device)
        x = torch.randn(n, W, device=device)
        h = torch.randn(n, W, **bf)
        # dense projection (the retention in-projection) and the routed experts
        w_in = rw["w_in"]
        ms = timer(lambda: Q.gemm(h, w_in, out_f32=True))
        add(f"gemm in-projection [{n} x {W}] x [{w_in.shape[0]} x {W}] ({tag})", ms, nbytes=w_in.numel() * 2 + n * W * 2 + n * w_in.shape[0] * 4,
            flops=2 * n * W * w_in.shape[0])
        f = ret.mlp
        sel_w, grp_off, pair_tok, pair_pos, _ = Q.moe_route(h, rw["router"], f.top)
        ms = timer(lambda: Q.gemm(h, rw["gu"], groups=f.experts, n=f.ff, dual=True, limit=f.limit, grp_off=grp_off, row_src=pair_tok,
                                  rows=n * f.top, max_rows=n))
        touched = min(f.experts, n * f.top)
        add(f"gemm routed gate|up + activation, {f.experts} experts top {f.top} ({tag})", ms,
            nbytes=touched * 2 * f.ff * W * 2 + n * W * 2 + n * f.top * f.ff * 2, flops=2 * n * f.top * W * 2 * f.ff)
        ms = timer(lambda: Q.moe_route(h, rw["router"], f.top))
        add(f"router + expert sort ({tag})", ms, nbytes=n * W * 2)
        # norm + shift
        st = rm.cache.shift[ri]
        ms = timer(lambda: Q.group_norm_shift(x, rw["norm"], rw["shift"], st, batch, sp.norm_groups, sp.norm_eps, torch.bfloat16))
        add(f"group norm + token shift ({tag})", ms, nbytes=n * W * (4 + 2 + 2))
        # retention
        ld = 2 * ret.heads * (ret.dim + ret.vdim)
        qkvg = torch.randn(n, ld, device=device)
        state = rm.cache.ret_state[ri]
        ms = timer(lambda: Q.retention(qkvg, batch, ret.heads, ret.dim, ret.vdim, ret.rot_dims, rw["inv_freq"], rw["decay"],
                                       sp.norm_eps, state, torch.bfloat16))
        sbytes = nseq * ret.heads * ret.dim * ret.vdim * 4 * 2
        add(f"retention: rotary + recurrence + unit norm + gate, fp32 ({tag})", ms,
            nbytes=n * ld * 4 + n * ret.heads * ret.vdim * (4 + 4 + 2) + sbytes, flops32=4 * n * ret.heads * ret.dim * ret.vdim)
        # latent attention
        R = lat.kv_rank
        qa = torch.randn(n, lat.heads * R, device=device)
        c = torch.randn(n, R, **bf)
        ring = rm.cache.ring[li]
        ms = timer(lambda: Q.latent_attention(qa, c, ring, batch, lat.heads, lat.window, lat.scale, append=False))
        keys = sum(min(p + 1, lat.window) for p in range(per)) * nseq if n == T else n * min(513, lat.window)
        add(f"latent attention, window {lat.window}, fp32 scores ({tag})", ms,
            nbytes=n * lat.heads * R * (4 + 2) + (n * R * 2 if n == T else keys * R * 2), flops32=4 * keys * lat.heads * R)
        if n == T:
            # the form a step of fresh sequences takes: per-head keys | values up-projected once, then attention over them
            hd, hvv = lat.heads * lat.dim, lat.heads * lat.vdim
            qh = torch.randn(n, hd, **bf)
            kvh = torch.randn(n, hd + hvv, **bf)
            ms = timer(lambda: Q.window_attention(qh, kvh[:, :hd], kvh[:, hd:], batch, lat.heads, lat.window, lat.scale))
            add(f"window attention over per-head keys, window {lat.window}, fp32 scores ({tag})", ms,
                nbytes=n * (2 * hd + 2 * hvv) * 2, flops32=2 * keys * lat.heads * (lat.dim + lat.vdim))
        # residual + depth mix
        stack = torch.randn(len(sp.layers) + 1, n, W, device=device)
        mix = torch.randn(n, W, device=device)
        dw = rm.weights[-1]["depth"]
        ms = timer(lambda: Q.depth_mix(x, mix, stack, len(sp.layers) - 1, dw, shared=mix))
        add(f"residual + depth average over {len(sp.layers) + 1} streams ({tag})", ms, nbytes=n * W * 4 * (len(sp.layers) + 4))
    # the like kernels of the Llama path: fp16 tcgen05 GEMM at its row limit, attention, rms norm
    sh = lm.config
    Hd, I = sh.hidden_size, sh.intermediate_size
    lwt = lm.layer_weights[0]
    f16 = dict(dtype=torch.float16, device=device)
    for n in (128, 8):
        xx = torch.randn(n, Hd, **f16)
        y = torch.empty(n, I, **f16)
        ms = timer(lambda: ops.gemm_f16(xx, lwt["wgu"], mode=ops.UMB_EPI_SILU_MUL, out=y, workspace=lm._gemm_ws))
        add(f"llama gemm gate|up + silu [{n} x {Hd}] x [{2 * I} x {Hd}] (tcgen05)", ms, nbytes=2 * I * Hd * 2 + n * Hd * 2 + n * I * 2,
            flops=2 * n * Hd * 2 * I, like="gemm")
        ms = timer(lambda: ops.rmsnorm(xx, lwt["input_norm"], 1e-5))
        add(f"llama rms norm, {n} rows", ms, nbytes=n * Hd * 4, like="group norm + token shift")
    S = 2048
    q = torch.randn(128, lm.num_heads, lm.head_dim, **f16)
    k = torch.randn(S, lm.num_key_value_heads, lm.head_dim, **f16)
    v = torch.randn_like(k)
    ws = ops.tree_attn_workspace(128, lm.num_heads, lm.head_dim, device)
    mask = ops.make_mask(ops.UMB_MASK_CAUSAL, prefix_len=S - 128)
    ms = timer(lambda: ops.tree_attn(q, k, v, S, mask, "NHD", workspace=ws))
    add(f"llama causal attention, 128 rows over {S} keys", ms, nbytes=2 * S * lm.num_key_value_heads * lm.head_dim * 2,
        flops=4 * 128 * (S - 64) * lm.num_heads * lm.head_dim, like="latent attention")
    q1 = q[:8].contiguous()
    mask1 = ops.make_mask(ops.UMB_MASK_CAUSAL, prefix_len=S - 8)
    ms = timer(lambda: ops.tree_attn(q1, k, v, S, mask1, "NHD", workspace=ws))
    add(f"llama causal attention, 8 rows over {S} keys", ms, nbytes=2 * S * lm.num_key_value_heads * lm.head_dim * 2,
        like="latent attention / retention (decode)")
    return rows, how


def run(args):
    from . import _lib, _lib_seq
    device = "cuda:0"
    timer = Timer(device)
    hbm, tflops, how = _peaks()
    sizes = []
    launches0 = _lib_seq.load().umbs_launch_count() + _lib.launch_count()
    table = None
    for width in (1024, 2048):
        layers, prompt, ctx = 8, 2048, 512
        rm, r = bench_radanex(width, layers, device, prompt, ctx, (1, 8, 64), timer)
        lm, l = bench_llama(width, layers, 2 * width, device, prompt, ctx, timer)
        sizes.append({"width": width, "layers": layers, "radanex_bf16": {k: round(v, 3) for k, v in r.items()},
                      "llama_fp16": {k: round(v, 3) for k, v in l.items()}})
        if width == 2048:
            table, _ = kernel_table(rm, lm, device, timer)
        del rm, lm
        torch.cuda.empty_cache()
    launches = _lib_seq.load().umbs_launch_count() + _lib.launch_count() - launches0
    head = sizes[-1]["radanex_bf16"]
    line = {"metric": "decode tokens/sec at batch 64 (Radanex bf16, width 2048, 8 layers, synthetic weights)",
            "value": head["decode_b64_tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "vs_baseline": None, "gpu_launches": int(launches),
            "config": {"name": "radanex", "workload": "prefill 1 x 2048 and 4 x 2048 tokens; decode at batch 1 / 8 / 64 behind a "
                       "512-token context; Llama fp16 of the same width, depth and active feed-forward size beside it",
                       "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": how},
                       "l2": "whole-model runs stream more than L2 per step; kernel table flushes L2 between runs"},
            "sizes": sizes, "kernels": table}
    print(json.dumps(line))


def kernel_table_zedotar(zm, rm, device, timer, T=4096):
    """Device time of each Zedotar mechanism at prefill size (one sequence of T tokens) and at decode size (8 sequences behind
    512 tokens), with its roofline fractions, and the like kernel of the Radanex path measured the same way in the same
    run (``like`` names the pairing)."""
    from . import _lib_seq as S, ops_seq as Q
    hbm, tflops, how = _peaks()
    sp, W = zm.spec, zm.spec.width
    fp32_peak = 148 * 128 * 2 * 1.965e-3
    rows = []

    def add(name, ms, nbytes=0, flops=0, like=None, flops32=0):
        r = dict(kernel=name, ms=round(ms, 4))
        if flops32:
            r["fp32_tflops"], r["frac_of_fp32_fma_peak"] = round(flops32 / ms / 1e9, 2), round(flops32 / ms / 1e9 / fp32_peak, 3)
        if flops:
            r["tflops"], r["frac_of_bf16_peak"] = round(flops / ms / 1e9, 1), round(flops / ms / 1e9 / tflops, 3)
        if nbytes:
            r["gb_s"], r["frac_of_hbm_peak"] = round(nbytes / ms / 1e6, 1), round(nbytes / ms / 1e6 / hbm, 3)
        if like:
            r["like"] = like
        rows.append(r)
    mls = next(l for l in sp.layers if l.mixer == "mlstm")
    att = next(l for l in sp.layers if l.mixer == "cached_attention" and l.window > 0)
    at2 = next(l for l in sp.layers if l.mixer == "cached_attention" and l.window == 0)
    mw, aw, sw = (zm.weights[sp.layers.index(l)] for l in (mls, att, at2))
    rsp = rm.spec
    ret = next(l for l in rsp.layers if l.mixer == "retention")
    lat = next(l for l in rsp.layers if l.mixer == "latent_attention")
    rw = rm.weights[rsp.layers.index(ret)]
    bf = dict(dtype=torch.bfloat16, device=device)
    ctx = 512
    zm.cache.reserve_length(T)                       # the windowless cache and the block table hold the whole prompt
    for n, tag in ((T, f"prefill T={T}"), (8, "decode T=8")):
        nseq = 1 if n == T else 8
        per = n // nseq
        pos0 = 0 if n == T else ctx
        batch = Q.RaggedBatch([(s, per, pos0, 0) for s in range(nseq)], device)
        x, d = torch.randn(n, W, device=device), torch.randn(n, W, device=device)
        h = torch.randn(n, W, **bf)
        # feed-forward products
        gu = mw["s_gu"]
        ms = timer(lambda: Q.gemm(h, gu, dual=S.UMBS_ACT_GELU_TANH))
        add(f"gemm dense gate|up + gelu [{n} x {W}] x [{gu.shape[0]} x {W}] ({tag})", ms,
            nbytes=gu.numel() * 2 + n * W * 2 + n * gu.shape[0], flops=2 * n * W * gu.shape[0], like="gemm shared gate|up")
        rgu = rw["s_gu"]
        ms = timer(lambda: Q.gemm(h, rgu, dual=True, limit=7.0))
        add(f"radanex gemm shared gate|up + clamped glu [{n} x {W}] x [{rgu.shape[0]} x {W}] ({tag})", ms,
            nbytes=rgu.numel() * 2 + n * W * 2 + n * rgu.shape[0], flops=2 * n * W * rgu.shape[0])
        # residual + norm
        ms = timer(lambda: Q.add_rms_norm(x, d, mw["norm"], 1.0, sp.norm_eps, torch.bfloat16))
        add(f"residual add + rms norm ({tag})", ms, nbytes=n * W * (4 + 4 + 4 + 2), like="group norm + token shift")
        st = rm.cache.shift[rsp.layers.index(ret)]
        ms = timer(lambda: Q.group_norm_shift(x, rw["norm"], rw["shift"], st, batch, rsp.norm_groups, rsp.norm_eps, torch.bfloat16))
        add(f"radanex group norm + token shift ({tag})", ms, nbytes=n * W * (4 + 2 + 2))
        # mLSTM beside retention (equal heads, dim, vdim)
        ld = 2 * mls.heads * (mls.dim + mls.vdim) + 2 * mls.heads
        proj = torch.randn(n, ld, device=device)
        state = zm.cache.mlstm_state[sp.layers.index(mls)]
        ms = timer(lambda: Q.mlstm(proj, mw["bias_in"], batch, mls.heads, mls.dim, mls.vdim, mls.gate_cap, sp.norm_eps, mw["out_norm"],
                                   state, torch.bfloat16))
        sbytes = nseq * mls.heads * mls.dim * (mls.vdim + 1) * 4 * 2
        add(f"mlstm: gates + recurrence + normaliser + unit norm + gate, fp32 ({tag})", ms,
            nbytes=n * ld * 4 + n * mls.heads * mls.vdim * (4 + 4 + 2) + sbytes, flops32=4 * n * mls.heads * mls.dim * (mls.vdim + 1),
            like="retention")
        rld = 2 * ret.heads * (ret.dim + ret.vdim)
        qkvg = torch.randn(n, rld, device=device)
        rstate = rm.cache.ret_state[rsp.layers.index(ret)]
        ms = timer(lambda: Q.retention(qkvg, batch, ret.heads, ret.dim, ret.vdim, ret.rot_dims, rw["inv_freq"], rw["decay"],
                                       rsp.norm_eps, rstate, torch.bfloat16))
        add(f"radanex retention: rotary + recurrence + unit norm + gate, fp32 ({tag})", ms,
            nbytes=n * rld * 4 + n * ret.heads * ret.vdim * (4 + 4 + 2) + nseq * ret.heads * ret.dim * ret.vdim * 8,
            flops32=4 * n * ret.heads * ret.dim * ret.vdim)
        # the attention kinds
        for l, w, name in ((att, aw, f"window {att.window} + blocks of {att.pool}, sink"), (at2, sw, "causal, sigmoid weights")):
            H, G, D, V = l.heads, l.kv_heads, l.dim, l.vdim
            cq, ck = H * D, G * D
            cv = 0 if l.values_are_keys else G * V
            gate_rows = H if l.gate_kind == 1 else H * V
            pr = torch.randn(n, cq + ck + cv + gate_rows, device=device)
            li = sp.layers.index(l)
            cache, pooled, conv = zm.cache.kv_cache[li], zm.cache.pool_cache[li], zm.cache.conv_state[li]
            ms = timer(lambda: Q.attention_prep(pr, w.get("bias_in"), batch, H, G, D, V, l.rot_dims, w["inv_freq"], l.rot_mag,
                                                l.values_are_keys, l.taps, w.get("conv_w"), conv, torch.bfloat16))
            add(f"attention prep: bias{' + conv' if l.taps > 1 else ''} + rotary -> q, key|value rows ({name}; {tag})", ms,
                nbytes=n * (cq + ck + cv) * 4 + n * (cq + G * (D + V)) * 2)
            q, kv = Q.attention_prep(pr, w.get("bias_in"), batch, H, G, D, V, l.rot_dims, w["inv_freq"], l.rot_mag,
                                     l.values_are_keys, l.taps, w.get("conv_w"), conv, torch.bfloat16)
            mode = S.UMBS_ATTN_SOFTMAX_SINK if l.attn_mode == "softmax_sink" else S.UMBS_ATTN_SIGMOID
            gate = pr[:, cq + ck + cv:]
            ms = timer(lambda: Q.cached_attention(q, kv, cache, batch, H, G, D, V, l.scale, mode=mode, window=l.window, pool=l.pool,
                                                  pool_cache=pooled, head_bias=w.get("head_bias"), gate=gate,
                                                  gate_per_head=l.gate_kind == 1, append=False))
            win = l.window if l.window > 0 else 1 << 30
            seen = lambda p: min(p + 1, win) + (max(0, p - win + 1) // l.pool if l.pool else 0)
            keys = sum(seen(p) for p in range(pos0, pos0 + per)) * nseq
            kv_bytes = n * G * (D + V) * 2 if n == T else nseq * seen(pos0) * G * (D + V) * 2
            add(f"cached attention, {name}, fp32 scores ({tag})", ms, nbytes=n * H * (D + V) * 2 + kv_bytes,
                flops32=2 * keys * H * (D + V), like="window attention over per-head keys" if n == T else "latent attention")
        # Radanex's attention the same way
        R = lat.kv_rank
        lring = rm.cache.ring[rsp.layers.index(lat)]
        keys = sum(min(p + 1, lat.window) for p in range(pos0, pos0 + per)) * nseq
        if n == T:
            hd, hvv = lat.heads * lat.dim, lat.heads * lat.vdim
            qh, kvh = torch.randn(n, hd, **bf), torch.randn(n, hd + hvv, **bf)
            ms = timer(lambda: Q.window_attention(qh, kvh[:, :hd], kvh[:, hd:], batch, lat.heads, lat.window, lat.scale))
            add(f"radanex window attention over per-head keys, window {lat.window}, fp32 scores ({tag})", ms,
                nbytes=n * (2 * hd + 2 * hvv) * 2, flops32=2 * keys * lat.heads * (lat.dim + lat.vdim))
        else:
            qa, c = torch.randn(n, lat.heads * R, device=device), torch.randn(n, R, **bf)
            ms = timer(lambda: Q.latent_attention(qa, c, lring, batch, lat.heads, lat.window, lat.scale, append=False))
            add(f"radanex latent attention, window {lat.window}, fp32 scores ({tag})", ms,
                nbytes=n * lat.heads * R * 6 + keys * R * 2, flops32=4 * keys * lat.heads * R)
    return rows, how


def run_zedotar(args):
    from . import _lib_seq
    device = "cuda:0"
    timer = Timer(device)
    hbm, tflops, how = _peaks()
    sizes, table = [], None
    launches0 = _lib_seq.load().umbs_launch_count()
    for width in (1024, 2048):
        layers, prompt, ctx = 8, 2048, 512
        zm, z = bench_zedotar(width, layers, device, prompt, ctx, (1, 8, 64), timer)
        rm, r = bench_radanex(width, layers, device, prompt, ctx, (1, 8, 64), timer)
        sizes.append({"width": width, "layers": layers, "zedotar_bf16": {k: round(v, 3) for k, v in z.items()},
                      "radanex_bf16": {k: round(v, 3) for k, v in r.items()}})
        if width == 2048:
            table, _ = kernel_table_zedotar(zm, rm, device, timer)
        del zm, rm
        torch.cuda.empty_cache()
    launches = _lib_seq.load().umbs_launch_count() - launches0
    head = sizes[-1]["zedotar_bf16"]
    line = {"metric": "decode tokens/sec at batch 64 (Zedotar bf16, width 2048, 8 layers, synthetic weights)",
            "value": head["decode_b64_tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "vs_baseline": None, "gpu_launches": int(launches),
            "config": {"name": "zedotar", "workload": "prefill 1 x 2048 and 4 x 2048 tokens; decode at batch 1 / 8 / 64 behind a "
                       "512-token context; Radanex bf16 of the same width, depth and active feed-forward size beside it",
                       "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": how},
                       "l2": "whole-model runs stream more than L2 per step; kernel table flushes L2 between runs"},
            "sizes": sizes, "kernels": table}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------- the Kulisun family
def kulisun_config(width: int, layers: int = 8) -> dict:
    """A Kulisun config with the layer sizes of a model of this width: latent attention in every layer (a latent of a
    quarter of the width plus 64 rotated dimensions per cached token, heads of 128 + 64 and values of 128), the first
    layer's feed-forward dense, the others routed with the active width Radanex has (2 of 16 experts in 4 groups of which
    2 stay eligible, plus a shared expert)."""
    heads = width // 128
    mixer = dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=width // 4, scale=192 ** -0.5,
                 rot=dict(dims=64, base=1e4, scaling=dict(factor=40.0, original=4096, fast=32.0, slow=1.0)))
    moe = dict(kind="moe", router=dict(experts=16, top=2, groups=dict(count=4, keep=2)), expert=dict(ff=width // 2),
               shared=dict(ff=width))
    return dict(architecture="Kulisun", width=width, vocab=32768, norm=dict(eps=1e-5), embedding=dict(scale=width ** 0.5),
                residual_mult=0.7,
                layers=[dict(type="latent_attention", mixer=mixer, mlp=dict(kind="dense", ff=2 * width) if i == 0 else moe)
                        for i in range(layers)])


def bench_kulisun(width, layers, device, prompt, ctx, batches, timer):
    from .models.kulisun import Kulisun, spec_from_config
    spec = spec_from_config(kulisun_config(width, layers))
    m = Kulisun(spec, device=device, dtype=torch.bfloat16, slots=max(batches), max_tokens=prompt + ctx)
    return bench_seq_model(m, spec, prompt, ctx, batches, timer)


def kernel_table_kulisun(km, rm, device, timer, T=4096):
    """Device time of each Kulisun mechanism at prefill size (one sequence of T tokens) and at decode size (8 sequences behind
    512 tokens), with its roofline fractions, and the like kernel of the Radanex path measured the same way in the same
    run (``like`` names the pairing)."""
    from . import _lib_seq as S, ops_seq as Q
    hbm, tflops, how = _peaks()
    sp, W = km.spec, km.spec.width
    fp32_peak = 148 * 128 * 2 * 1.965e-3
    rows = []

    def add(name, ms, nbytes=0, flops=0, like=None, flops32=0):
        r = dict(kernel=name, ms=round(ms, 4))
        if flops32:
            r["fp32_tflops"], r["frac_of_fp32_fma_peak"] = round(flops32 / ms / 1e9, 2), round(flops32 / ms / 1e9 / fp32_peak, 3)
        if flops:
            r["tflops"], r["frac_of_bf16_peak"] = round(flops / ms / 1e9, 1), round(flops / ms / 1e9 / tflops, 3)
        if nbytes:
            r["gb_s"], r["frac_of_hbm_peak"] = round(nbytes / ms / 1e6, 1), round(nbytes / ms / 1e6 / hbm, 3)
        if like:
            r["like"] = like
        rows.append(r)
    l = sp.layers[1]
    dw, mw = km.weights[0], km.weights[1]
    rsp = rm.spec
    ret = next(x for x in rsp.layers if x.mixer == "retention")
    lat = next(x for x in rsp.layers if x.mixer == "latent_attention")
    rw, lw = rm.weights[rsp.layers.index(ret)], rm.weights[rsp.layers.index(lat)]
    bf = dict(dtype=torch.bfloat16, device=device)
    ctx = 512
    km.cache.reserve_length(T)
    H, D, Rt, V, R = l.heads, l.dim, l.rope_dim, l.vdim, l.kv_rank
    KD = R + Rt
    for n, tag in ((T, f"prefill T={T}"), (8, "decode T=8")):
        nseq = 1 if n == T else 8
        per = n // nseq
        pos0 = 0 if n == T else ctx
        batch = Q.RaggedBatch([(s, per, pos0, 0) for s in range(nseq)], device)
        x, d = torch.randn(n, W, device=device), torch.randn(n, W, device=device)
        h = torch.randn(n, W, **bf)
        # residual + norm: dense pending output, and the routed + shared sums
        ms = timer(lambda: Q.add_norm(x, dw["norm"], dw["norm_b"], sp.norm_eps, dtype=torch.bfloat16, delta=d, scale=dw["ls1"], mult=0.7))
        add(f"residual add (layer scale, multiplier) + layer norm ({tag})", ms, nbytes=n * W * (4 + 4 + 4 + 2), like="group norm + token shift")
        f = l.mlp
        sel_w, grp_off, pair_tok, pair_pos, _ = Q.moe_route_ex(h, mw["router"], f.top, S.UMBS_ROUTE_SIGMOID_GROUPS, f.groups, f.keep)
        pair_out, sg = torch.randn(n * f.top, W, device=device), torch.rand(n, device=device)
        ms = timer(lambda: Q.add_norm(x, dw["norm"], dw["norm_b"], sp.norm_eps, dtype=torch.bfloat16, pair_out=pair_out, sel_w=sel_w,
                                      pair_pos=pair_pos, shared=d, shared_gate=sg, scale=dw["ls1"], mult=0.7))
        add(f"residual add of {f.top} routed + gated shared outputs + layer norm ({tag})", ms, nbytes=n * W * (4 + 4 + 4 + 2 + 4 * f.top),
            like="residual + depth average")
        st = rm.cache.shift[rsp.layers.index(ret)]
        ms = timer(lambda: Q.group_norm_shift(x, rw["norm"], rw["shift"], st, batch, rsp.norm_groups, rsp.norm_eps, torch.bfloat16))
        add(f"radanex group norm + token shift ({tag})", ms, nbytes=n * W * (4 + 2 + 2))
        stack, dwt = torch.randn(len(rsp.layers) + 1, n, W, device=device), rm.weights[-1]["depth"]
        rpo = torch.randn(n * ret.mlp.top, W, device=device)
        rsel, _, _, rpp, _ = Q.moe_route(h, rw["router"], ret.mlp.top)
        ms = timer(lambda: Q.depth_mix(x, d, stack, len(rsp.layers) - 1, dwt, pair_out=rpo, sel_w=rsel, pair_pos=rpp, shared=d))
        add(f"radanex residual of routed + shared outputs + depth average over {len(rsp.layers) + 1} streams ({tag})", ms,
            nbytes=n * W * 4 * (len(rsp.layers) + 5 + ret.mlp.top))
        # feed-forward products
        gu = dw["s_gu"]
        ms = timer(lambda: Q.gemm_ex(h, gu, act=S.UMBS_ACT_SILU, bias=dw["s_gu_b"]))
        add(f"gemm dense gate|up + bias + silu [{n} x {W}] x [{gu.shape[0]} x {W}] ({tag})", ms,
            nbytes=gu.numel() * 2 + n * W * 2 + n * gu.shape[0], flops=2 * n * W * gu.shape[0], like="gemm shared gate|up")
        rgu = rw["s_gu"]
        ms = timer(lambda: Q.gemm(h, rgu, dual=True, limit=7.0))
        add(f"radanex gemm shared gate|up + clamped glu [{n} x {W}] x [{rgu.shape[0]} x {W}] ({tag})", ms,
            nbytes=rgu.numel() * 2 + n * W * 2 + n * rgu.shape[0], flops=2 * n * W * rgu.shape[0])
        ms = timer(lambda: Q.gemm(h, mw["gu"], groups=f.experts, n=f.ff, dual=S.UMBS_ACT_SILU, grp_off=grp_off, row_src=pair_tok,
                                  rows=n * f.top, max_rows=n))
        touched = min(f.experts, n * f.top)
        add(f"gemm routed gate|up + silu, {f.experts} experts top {f.top} ({tag})", ms,
            nbytes=touched * 2 * f.ff * W * 2 + n * W * 2 + n * f.top * f.ff * 2, flops=2 * n * f.top * W * 2 * f.ff, like="gemm routed gate|up")
        rf = ret.mlp
        _, rgo, rpt, _, _ = Q.moe_route(h, rw["router"], rf.top)
        ms = timer(lambda: Q.gemm(h, rw["gu"], groups=rf.experts, n=rf.ff, dual=True, limit=rf.limit, grp_off=rgo, row_src=rpt,
                                  rows=n * rf.top, max_rows=n))
        add(f"radanex gemm routed gate|up + clamped glu, {rf.experts} experts top {rf.top} ({tag})", ms,
            nbytes=min(rf.experts, n * rf.top) * 2 * rf.ff * W * 2 + n * W * 2 + n * rf.top * rf.ff * 2, flops=2 * n * rf.top * W * 2 * rf.ff)
        # routers
        ms = timer(lambda: Q.moe_route_ex(h, mw["router"], f.top, S.UMBS_ROUTE_SIGMOID_GROUPS, f.groups, f.keep))
        add(f"router (sigmoid, {f.groups} groups keep {f.keep}) + expert sort ({tag})", ms, nbytes=n * W * 2, like="router + expert sort")
        ms = timer(lambda: Q.moe_route(h, rw["router"], rf.top))
        add(f"radanex router (softmax over the top) + expert sort ({tag})", ms, nbytes=n * W * 2)
        ms = timer(lambda: Q.token_gate(h, mw["s_gate"]))
        add(f"shared expert's gate per token ({tag})", ms, nbytes=n * W * 2)
        # between in-projection and attention
        cols = H * (D + Rt) + KD + H * V
        proj = torch.randn(n, cols, device=device)
        ms = timer(lambda: Q.latent_prep(proj, batch, H, D, Rt, R, mw["kv_norm"], sp.norm_eps, l.rot_dims, mw["inv_freq"], l.rot_mag,
                                         torch.bfloat16))
        add(f"latent norm + rotary of the shared key part and of every head's query ({tag})", ms,
            nbytes=n * (H * (D + Rt) + KD) * (4 + 2) + n * H * Rt * 4, like="latent norm")
        rproj = torch.randn(n, lat.q_rank + lat.kv_rank, device=device)
        ms = timer(lambda: Q.latent_norm(rproj, lat.q_rank, lat.kv_rank, lw["q_norm"], lw["kv_norm"], rsp.norm_eps, torch.bfloat16))
        add(f"radanex latent norm of the query and key latents ({tag})", ms, nbytes=n * (lat.q_rank + lat.kv_rank) * (4 + 2))
        # attention
        ring = km.cache.ring[1]
        keys = sum(p + 1 for p in range(pos0, pos0 + per)) * nseq
        gate = proj[:, H * (D + Rt) + KD:]
        RR = lat.kv_rank
        lring = rm.cache.ring[rsp.layers.index(lat)]
        rkeys = sum(min(p + 1, lat.window) for p in range(pos0, pos0 + per)) * nseq
        if n == T:
            q, kvh, ks = torch.randn(n, H * (D + Rt), **bf), torch.randn(n, H * (D + V), **bf), torch.randn(n, KD, **bf)
            ms = timer(lambda: Q.window_attention_shared(q, kvh[:, :H * D], ks[:, R:], kvh[:, H * D:], batch, H, l.scale, sink=mw["sink"],
                                                         gate=gate))
            add(f"attention over per-head keys + shared rotated part, causal, sink, gate, fp32 scores ({tag})", ms,
                nbytes=n * (H * (D + Rt) + H * (D + V) + Rt + H * V) * 2 + n * H * V * 4, flops32=2 * keys * H * (D + Rt + V),
                like="window attention over per-head keys")
            hd, hvv = lat.heads * lat.dim, lat.heads * lat.vdim
            qh, kv2 = torch.randn(n, hd, **bf), torch.randn(n, hd + hvv, **bf)
            ms = timer(lambda: Q.window_attention(qh, kv2[:, :hd], kv2[:, hd:], batch, lat.heads, lat.window, lat.scale))
            add(f"radanex window attention over per-head keys, window {lat.window}, fp32 scores ({tag})", ms,
                nbytes=n * (2 * hd + 2 * hvv) * 2, flops32=2 * rkeys * lat.heads * (lat.dim + lat.vdim))
        qa, c = torch.randn(n, H, KD, device=device), torch.randn(n, KD, **bf)
        ms = timer(lambda: Q.latent_attention_shared(qa, c, ring, batch, H, R, Rt, l.scale, sink=mw["sink"], append=False))
        add(f"latent attention over [latent | shared part] keys, causal, sink, fp32 scores ({tag})", ms,
            nbytes=n * H * (KD * 4 + R * 2) + (n * KD * 2 if n == T else keys * KD * 2), flops32=2 * keys * H * (KD + R),
            like="latent attention")
        qr, cr = torch.randn(n, lat.heads * RR, device=device), torch.randn(n, RR, **bf)
        ms = timer(lambda: Q.latent_attention(qr, cr, lring, batch, lat.heads, lat.window, lat.scale, append=False))
        add(f"radanex latent attention, window {lat.window}, fp32 scores ({tag})", ms,
            nbytes=n * lat.heads * RR * 6 + (n * RR * 2 if n == T else rkeys * RR * 2), flops32=4 * rkeys * lat.heads * RR)
        # value up-projection per head with the output gate in the epilogue
        o_lat = torch.randn(n, H * R, **bf)
        uv = mw["uv"].view(H, V, R)
        ms = timer(lambda: Q.gemm_ex(o_lat, uv, groups=H, a_goff=R, c_goff=V, n=V, k=R, out_gate=gate, gate_goff=V))
        add(f"gemm value up-projection per head + sigmoid output gate ({tag})", ms,
            nbytes=n * H * R * 2 + H * V * R * 2 + n * H * V * (2 + 4), flops=2 * n * H * V * R, like="gemm per head")
        ro = torch.randn(n, lat.heads * RR, **bf)
        ruv = lw["uv"].view(lat.heads, lat.vdim, RR)
        ms = timer(lambda: Q.gemm(ro, ruv, groups=lat.heads, a_goff=RR, c_goff=lat.vdim, n=lat.vdim, k=RR))
        add(f"radanex gemm value up-projection per head ({tag})", ms,
            nbytes=n * lat.heads * RR * 2 + lat.heads * lat.vdim * RR * 2 + n * lat.heads * lat.vdim * 2, flops=2 * n * lat.heads * lat.vdim * RR)
    return rows, how


def run_kulisun(args):
    from . import _lib_seq
    device = "cuda:0"
    timer = Timer(device)
    hbm, tflops, how = _peaks()
    sizes, table = [], None
    launches0 = _lib_seq.load().umbs_launch_count()
    for width in (1024, 2048):
        layers, prompt, ctx = 8, 2048, 512
        km, k = bench_kulisun(width, layers, device, prompt, ctx, (1, 8, 64), timer)
        rm, r = bench_radanex(width, layers, device, prompt, ctx, (1, 8, 64), timer)
        # the closest shape the existing family takes: latent attention in every layer, over the whole context
        ra, a = bench_radanex(width, layers, device, prompt, ctx, (1, 8, 64), timer, latent_every=1, window=4096)
        del ra
        sizes.append({"width": width, "layers": layers, "kulisun_bf16": {a_: round(v, 3) for a_, v in k.items()},
                      "radanex_bf16": {a_: round(v, 3) for a_, v in r.items()},
                      "radanex_all_latent_bf16": {a_: round(v, 3) for a_, v in a.items()}})
        if width == 2048:
            table, _ = kernel_table_kulisun(km, rm, device, timer)
        del km, rm
        torch.cuda.empty_cache()
    launches = _lib_seq.load().umbs_launch_count() - launches0
    head = sizes[-1]["kulisun_bf16"]
    line = {"metric": "decode tokens/sec at batch 64 (Kulisun bf16, width 2048, 8 layers, synthetic weights)",
            "value": head["decode_b64_tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "vs_baseline": None, "gpu_launches": int(launches),
            "config": {"name": "kulisun", "workload": "prefill 1 x 2048 and 4 x 2048 tokens; decode at batch 1 / 8 / 64 behind a "
                       "512-token context; Radanex bf16 of the same width, depth and active feed-forward size beside it, as "
                       "packaged (latent attention in every fourth layer, window 1024) and with latent attention in every layer "
                       "over the whole context",
                       "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": how},
                       "l2": "whole-model runs stream more than L2 per step; kernel table flushes L2 between runs"},
            "sizes": sizes, "kernels": table}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------- the Subivik family
def subivik_config(width: int, layers: int = 8) -> dict:
    """A Subivik config with the layer sizes of a model of this width: heads of 128 with a quarter as many key/value heads
    for the talking attention, recurrent heads of 64 over the whole width beside it; differential attention with two maps
    of 64 per head inside chunks of 1024, one of those layers borrowing an earlier one's keys and values; dense
    feed-forward of 3 x width (the two matrices weigh what Zedotar's three of 2 x width do) or 2 of 16 experts."""
    heads = max(2, width // 128)
    kv = max(1, heads // 4)
    par = dict(type="parallel", mixer=dict(left=dict(heads=heads, kv_heads=kv, dim=128, vdim=128, scale=128 ** -0.5, softcap=50.0),
                                           right=dict(heads=width // 64, dim=64), left_scale=1.0, right_scale=0.5))
    att = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv, dim=64, vdim=128, scale=0.125, diff=0.2, mask=dict(size=1024)))
    dense = dict(kind="dense", ff=3 * width)
    moe = dict(kind="moe", router=dict(experts=16, top=2, scale=2.0), expert=dict(ff=width // 2))
    plan, first_att = [], None
    for i in range(layers):
        if i % 4 == 1:
            first_att = i if first_att is None else first_att
            plan.append(dict(att, mlp=moe))
        elif i % 4 == 3 and first_att is not None:
            plan.append(dict(type="attention", mixer=dict(att["mixer"], kv_from=first_att), mlp=dense))
        else:
            plan.append(dict(par, mlp=moe if i % 4 == 2 else dense))
    return dict(architecture="Subivik", width=width, vocab=32768, norm=dict(eps=1e-6), layers=plan)


def bench_subivik(width, layers, device, prompt, ctx, batches, timer):
    from .models.subivik import Subivik, spec_from_config
    spec = spec_from_config(subivik_config(width, layers))
    m = Subivik(spec, device=device, dtype=torch.bfloat16, slots=max(batches), max_tokens=prompt + ctx)
    return bench_seq_model(m, spec, prompt, ctx, batches, timer)


def kernel_table_subivik(sm, zm, device, timer, T=4096):
    """Device time of each Subivik mechanism at prefill size (one sequence of T tokens) and at decode size (8 sequences
    behind 512 tokens), with its roofline fractions, and the like kernel of the Zedotar path measured the same way in the
    same run (``like`` names the pairing)."""
    from . import _lib_seq as S, ops_seq as Q
    hbm, tflops, how = _peaks()
    sp, W = sm.spec, sm.spec.width
    fp32_peak = 148 * 128 * 2 * 1.965e-3
    rows = []

    def add(name, ms, nbytes=0, flops=0, like=None, flops32=0):
        r = dict(kernel=name, ms=round(ms, 4))
        if flops32:
            r["fp32_tflops"], r["frac_of_fp32_fma_peak"] = round(flops32 / ms / 1e9, 2), round(flops32 / ms / 1e9 / fp32_peak, 3)
        if flops:
            r["tflops"], r["frac_of_bf16_peak"] = round(flops / ms / 1e9, 1), round(flops / ms / 1e9 / tflops, 3)
        if nbytes:
            r["gb_s"], r["frac_of_hbm_peak"] = round(nbytes / ms / 1e6, 1), round(nbytes / ms / 1e6 / hbm, 3)
        if like:
            r["like"] = like
        rows.append(r)
    par = next(l for l in sp.layers if l.second is not None)
    dif = next(l for l in sp.layers if l.maps == 2 and l.kv_from is None)
    pw, dw = sm.weights[sp.layers.index(par)], sm.weights[sp.layers.index(dif)]
    tm, tw = par.second, pw["second"]
    dn = next(sm.weights[i] for i, l in enumerate(sp.layers) if l.mlp is not None and l.mlp.plain)
    zsp = zm.spec
    mls = next(l for l in zsp.layers if l.mixer == "mlstm")
    zat = next(l for l in zsp.layers if l.mixer == "cached_attention" and l.window > 0)
    mw, aw = (zm.weights[zsp.layers.index(l)] for l in (mls, zat))
    bf = dict(dtype=torch.bfloat16, device=device)
    ctx = 512
    sm.cache.reserve_length(T)
    zm.cache.reserve_length(T)
    for n, tag in ((T, f"prefill T={T}"), (8, "decode T=8")):
        nseq = 1 if n == T else 8
        per = n // nseq
        pos0 = 0 if n == T else ctx
        batch = Q.RaggedBatch([(s, per, pos0, 0) for s in range(nseq)], device)
        x, d, d2 = (torch.randn(n, W, device=device) for _ in range(3))
        h = torch.randn(n, W, **bf)
        # feed-forward product with its activation
        up = dn["s_gu"]
        p0, p1 = dn["unary_p"]
        ms = timer(lambda: Q.gemm_unary(h, up, S.UMBS_UNARY_XIELU, p0, p1))
        add(f"gemm dense up + xielu [{n} x {W}] x [{up.shape[0]} x {W}] ({tag})", ms,
            nbytes=up.numel() * 2 + n * W * 2 + n * up.shape[0] * 2, flops=2 * n * W * up.shape[0], like="gemm dense gate|up + gelu")
        gu = mw["s_gu"]
        ms = timer(lambda: Q.gemm(h, gu, dual=S.UMBS_ACT_GELU_TANH))
        add(f"zedotar gemm dense gate|up + gelu [{n} x {W}] x [{gu.shape[0]} x {W}] ({tag})", ms,
            nbytes=gu.numel() * 2 + n * W * 2 + n * gu.shape[0], flops=2 * n * W * gu.shape[0])
        # residual + norm
        ms = timer(lambda: Q.add_norm_dyt(x, pw["norm"], pw["norm_b"], 0.7, torch.bfloat16, delta=d, delta_mult=1.0, delta2=d2, delta2_mult=0.5))
        add(f"residual add of two mixers + tanh norm ({tag})", ms, nbytes=n * W * (4 + 4 + 4 + 4 + 2), like="residual add + rms norm")
        ms = timer(lambda: Q.add_rms_norm(x, d, mw["norm"], 1.0, zsp.norm_eps, torch.bfloat16))
        add(f"zedotar residual add + rms norm ({tag})", ms, nbytes=n * W * (4 + 4 + 4 + 2))
        # token-shifted mixes
        sstate = sm.cache.shift[tm.state_index]
        ms = timer(lambda: Q.shift_mix(h, tw["mu"], sstate, batch))
        add(f"five token-shifted mixes ({tag})", ms, nbytes=n * W * 2 * 6)
        # the time-mix memory beside mLSTM
        hd = tm.heads * tm.dim
        proj, raw = torch.randn(n, 4 * hd, device=device), torch.randn(n, hd, device=device) - 1.0
        tstate = sm.cache.tm_state[tm.state_index]
        ms = timer(lambda: Q.time_mix(proj, raw, tw["w0"], tw["u"], batch, tm.heads, tm.dim, sp.norm_eps, tw["out_norm"], tstate, torch.bfloat16))
        add(f"time mix: decay exponentials + recurrence + unit norm + gate, fp32, {tm.heads} heads of {tm.dim} ({tag})", ms,
            nbytes=n * 5 * hd * 4 + n * hd * (4 + 4 + 2) + nseq * tm.heads * tm.dim * tm.dim * 8,
            flops32=6 * n * tm.heads * tm.dim * tm.dim, like="mlstm")
        ld = 2 * mls.heads * (mls.dim + mls.vdim) + 2 * mls.heads
        mproj = torch.randn(n, ld, device=device)
        mstate = zm.cache.mlstm_state[zsp.layers.index(mls)]
        ms = timer(lambda: Q.mlstm(mproj, mw["bias_in"], batch, mls.heads, mls.dim, mls.vdim, mls.gate_cap, zsp.norm_eps, mw["out_norm"],
                                   mstate, torch.bfloat16))
        add(f"zedotar mlstm: gates + recurrence + normaliser + unit norm + gate, fp32, {mls.heads} heads of {mls.dim} x {mls.vdim} ({tag})", ms,
            nbytes=n * ld * 4 + n * mls.heads * mls.vdim * (4 + 4 + 2) + nseq * mls.heads * mls.dim * (mls.vdim + 1) * 8,
            flops32=4 * n * mls.heads * mls.dim * (mls.vdim + 1))
        # the attention kinds
        for l, w, name in ((par, pw, "causal, cap + distance penalty, talking heads"), (dif, dw, f"differential, chunks of {dif.chunk}")):
            H, G, D, V, M = l.heads, l.kv_heads, l.dim, l.vdim, l.maps
            C_ = G if l.talk else 1
            cq, ck, cv, cg = H * M * D, G * M * D, G * V, (H * V if l.gate_kind else 0)
            pr = torch.randn(n, cq + ck + cv + cg, device=device)
            cache = sm.cache.kv_cache[l.state_index]
            qn, kn = w.get("q_norm"), w.get("k_norm")
            ms = timer(lambda: Q.attention_prep_maps(pr, batch, H, G, D, V, maps=M, q_norm=qn, k_norm=kn, eps=sp.norm_eps, dtype=torch.bfloat16))
            add(f"attention prep{': norm of query and key maps' if qn is not None else ''} -> q, key|value rows ({name}; {tag})", ms,
                nbytes=n * (cq + ck + cv) * 4 + n * (cq + ck + cv) * 2)
            q, kv = Q.attention_prep_maps(pr, batch, H, G, D, V, maps=M, q_norm=qn, k_norm=kn, eps=sp.norm_eps, dtype=torch.bfloat16)
            gate = pr[:, cq + ck + cv:] if cg else None
            ms = timer(lambda: Q.scored_attention(q, kv, cache, batch, H, G, D, V, l.scale, softcap=l.softcap, r1=w.get("r1"), r2=w.get("r2"),
                                                  chunk=l.chunk, maps=M, talk=w.get("talk"), diff_lambda=w.get("diff_lambda", 0.0),
                                                  unit_norm=l.head_unit_norm, eps=sp.norm_eps, out_mult=0.7, gate=gate, append=False))
            reach = l.chunk if l.chunk > 0 else 1 << 30
            seen = lambda p: min(p + 1, p % reach + 1)
            keys = sum(seen(p) for p in range(pos0, pos0 + per)) * nseq
            kv_bytes = n * (ck + cv) * 2 if n == T else nseq * seen(pos0) * (ck + cv) * 2
            add(f"cached attention + finish, {name}, fp32 scores, {H * M * C_} softmax rows per token ({tag})", ms,
                nbytes=n * cq * 2 + kv_bytes + n * H * M * C_ * V * 8 + n * H * V * 2,
                flops32=2 * keys * H * M * C_ * (D + V), like="zedotar cached attention")
        H, G, D, V = zat.heads, zat.kv_heads, zat.dim, zat.vdim
        zpr = torch.randn(n, H * D + G * (D + V) + H, device=device)
        zi = zsp.layers.index(zat)
        zcache, zpool = zm.cache.kv_cache[zi], zm.cache.pool_cache[zi]
        q, kv = Q.attention_prep(zpr, aw.get("bias_in"), batch, H, G, D, V, zat.rot_dims, aw["inv_freq"], zat.rot_mag, False, 1, None, None,
                                 torch.bfloat16)
        zgate = zpr[:, H * D + G * (D + V):]
        ms = timer(lambda: Q.cached_attention(q, kv, zcache, batch, H, G, D, V, zat.scale, mode=S.UMBS_ATTN_SOFTMAX_SINK, window=zat.window,
                                              pool=zat.pool, pool_cache=zpool, gate=zgate, gate_per_head=True, append=False))
        seen = lambda p: min(p + 1, zat.window) + (max(0, p - zat.window + 1) // zat.pool if zat.pool else 0)
        keys = sum(seen(p) for p in range(pos0, pos0 + per)) * nseq
        kv_bytes = n * G * (D + V) * 2 if n == T else nseq * seen(pos0) * G * (D + V) * 2
        add(f"zedotar cached attention, window {zat.window} + blocks of {zat.pool}, sink, fp32 scores, {H} softmax rows per token ({tag})", ms,
            nbytes=n * H * (D + V) * 2 + kv_bytes, flops32=2 * keys * H * (D + V))
    return rows, how


def run_subivik(args):
    from . import _lib_seq
    device = "cuda:0"
    timer = Timer(device)
    hbm, tflops, how = _peaks()
    sizes, table = [], None
    launches0 = _lib_seq.load().umbs_launch_count()
    for width in (1024, 2048):
        layers, prompt, ctx = 8, 2048, 512
        sm, s = bench_subivik(width, layers, device, prompt, ctx, (1, 8, 64), timer)
        zm, z = bench_zedotar(width, layers, device, prompt, ctx, (1, 8, 64), timer)
        sizes.append({"width": width, "layers": layers, "subivik_bf16": {k: round(v, 3) for k, v in s.items()},
                      "zedotar_bf16": {k: round(v, 3) for k, v in z.items()}})
        if width == 2048:
            table, _ = kernel_table_subivik(sm, zm, device, timer)
        del sm, zm
        torch.cuda.empty_cache()
    launches = _lib_seq.load().umbs_launch_count() - launches0
    head = sizes[-1]["subivik_bf16"]
    line = {"metric": "decode tokens/sec at batch 64 (Subivik bf16, width 2048, 8 layers, synthetic weights)",
            "value": head["decode_b64_tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic", "vs_baseline": None, "gpu_launches": int(launches),
            "config": {"name": "subivik", "workload": "prefill 1 x 2048 and 4 x 2048 tokens; decode at batch 1 / 8 / 64 behind a "
                       "512-token context; Zedotar bf16 (the closest family: pre-norm, cached attention, a recurrent matrix memory) "
                       "of the same width and depth beside it",
                       "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": how},
                       "l2": "whole-model runs stream more than L2 per step; kernel table flushes L2 between runs"},
            "sizes": sizes, "kernels": table}
    print(json.dumps(line))
