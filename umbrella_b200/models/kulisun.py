"""Kulisun: a pre-norm decoder family whose every layer mixes tokens by latent attention with direct queries -- keys and
values come from one RMS-normed low-rank latent per token, the keys also carry a rotated part (YaRN-scaled rotary
positions) that all heads share, so a token's cache row is the latent plus that part; causal softmax with a learned
sink score per head; element-wise sigmoid output gate -- followed by a dense silu-gated feed-forward with biases, a
mixture of experts (sigmoid scores, group-limited choice, normalised weights, a shared expert behind a per-token sigmoid
gate), or nothing.  Norms are layer norms with weight and bias; every block's output passes a learned layer scale and a
residual multiplier; the embedding is scaled.

This module is the family's front: config.json -> ``SeqModelSpec``, checkpoint tensor names -> ``load_layer`` dicts,
seeded synthetic weights for benchmarks and tests.  The computation is models/seq_model.py + csrc/seq: the mixer is the
framework's latent-attention mixer with ``q_rank`` 0 and a ``rope_dim``, the router a rule of ``umbs_moe_route_ex``.

config.json keys read here:
    architecture = "Kulisun"; width; vocab; norm.eps; embedding.scale; residual_mult;
    layers[i].type = "latent_attention";
    layers[i].mixer: heads, dim, rot_dim, vdim, kv_rank, scale, rot.{dims, base, scaling: {factor, original, fast, slow}}
    layers[i].mlp = null | {kind: "dense", ff}
                  | {kind: "moe", router: {experts, top, groups: {count, keep}}, expert: {ff}, shared: {ff} | null}
Tensors (safetensors, [out, in]): embed, head, final.norm (+ .b), and per layer ``l<i>.``: norm1, norm2 (+ .b), ls1, ls2,
mix.{q, dkv, dkv.norm, uk, uv, sink, g, o}, mlp.{gate, up, down} (+ .b) or mlp.router, mlp.e<j>.{gate, up, down},
mlp.shared.{gate, up, down, sg}.
"""
from __future__ import annotations

import json
import os

import torch

from .seq_model import (SeqLayerSpec, SeqMlpSpec, SeqModelSpec, SeqStateModel, rotary_inv_freq64, scale_freq_yarn)

ARCHITECTURE = "Kulisun"


def spec_from_config(cfg: dict) -> SeqModelSpec:
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: architecture = {cfg.get('architecture')!r}")
    mult = float(cfg.get("residual_mult", 1.0))
    layers = []
    for entry in cfg["layers"]:
        kind, mx = entry["type"], entry["mixer"]
        if kind != "latent_attention":
            raise ValueError(f"unknown layer type '{kind}'")
        l = SeqLayerSpec(mixer="latent_attention", heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                         form="prenorm", norm_kind="layer", layer_scale=True, residual_mult=mult, shift=False,
                         depth_average=False)
        l.q_rank, l.kv_rank, l.rope_dim, l.scale = 0, int(mx["kv_rank"]), int(mx.get("rot_dim", 0)), float(mx["scale"])
        l.window, l.attn_mode, l.learned_sink, l.gate_kind = 0, "softmax_sink", True, 2
        rot = mx.get("rot")
        if l.rope_dim and rot and int(rot.get("dims", 0)):
            l.rot_dims, l.rot_base = int(rot["dims"]), float(rot["base"])
            if l.rot_dims % 2 or l.rot_dims > l.rope_dim:
                raise ValueError("rot.dims must be even and at most rot_dim")
            f, sc = rotary_inv_freq64(l.rot_dims, l.rot_base), rot.get("scaling")
            if sc:
                f, l.rot_mag = scale_freq_yarn(f, l.rot_dims, l.rot_base, float(sc["factor"]), float(sc["original"]),
                                               float(sc["fast"]), float(sc["slow"]))
            l.inv_freq = [float(x) for x in f]
        mlp = entry.get("mlp")
        if mlp is not None:
            mk = mlp.get("kind", "dense")
            if mk == "dense":
                l.mlp = SeqMlpSpec(shared_ff=int(mlp["ff"]), act="silu", bias=True)
            elif mk == "moe":
                r, groups = mlp["router"], mlp["router"].get("groups") or {}
                m = SeqMlpSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(mlp["expert"]["ff"]), act="silu",
                               route="sigmoid_groups", groups=int(groups.get("count", 1)), keep=int(groups.get("keep", groups.get("count", 1))))
                if m.experts % m.groups or not 1 <= m.keep <= m.groups or m.top > m.keep * (m.experts // m.groups):
                    raise ValueError("router: experts must split into equal groups that hold `top` eligible experts")
                if mlp.get("shared"):
                    m.shared_ff, m.shared_gate = int(mlp["shared"]["ff"]), True
                l.mlp = m
            else:
                raise ValueError(f"unknown feed-forward kind '{mk}'")
        layers.append(l)
    eos = cfg.get("eos_token_id", [])
    return SeqModelSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers, norm_groups=1,
                        norm_eps=float(cfg["norm"]["eps"]), norm_kind="layer",
                        embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                        eos_token_id=list(eos) if isinstance(eos, (list, tuple)) else [int(eos)])


def layer_tensor_names(spec: SeqModelSpec, i: int) -> dict:
    """load_layer key -> checkpoint tensor name(s) of layer i."""
    l, p = spec.layers[i], f"l{i}."
    names = {"norm": p + "norm1", "norm_b": p + "norm1.b", "ls1": p + "ls1", "q": p + "mix.q", "dkv": p + "mix.dkv",
             "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk", "uv": p + "mix.uv", "sink": p + "mix.sink", "g": p + "mix.g",
             "o": p + "mix.o"}
    m = l.mlp
    if m is not None:
        names.update({"norm2": p + "norm2", "norm2_b": p + "norm2.b", "ls2": p + "ls2"})
        if m.experts:
            names["router"] = p + "mlp.router"
            names["experts"] = [tuple(f"{p}mlp.e{e}.{n}" for n in ("gate", "up", "down")) for e in range(m.experts)]
            if m.shared_ff:
                names["shared"] = tuple(f"{p}mlp.shared.{n}" for n in ("gate", "up", "down"))
                names["shared_gate"] = p + "mlp.shared.sg"
        else:
            names["dense"] = tuple(f"{p}mlp.{n}" for n in ("gate", "up", "down"))
            names["dense_b"] = tuple(f"{p}mlp.{n}.b" for n in ("gate", "up", "down"))
    return names


class Kulisun(SeqStateModel):
    """``Kulisun(spec, ...)``; ``alloc()`` then ``load_checkpoint(path)`` or ``load_synthetic(seed)``."""

    def load_checkpoint(self, path: str):
        from .checkpoint import SafetensorsIndex
        idx = SafetensorsIndex(path)
        get = idx.get
        self.load_head(get("embed"), get("head"), get("final.norm"), get("final.norm.b"))
        for i in range(self.num_layers):
            w = {}
            for key, name in layer_tensor_names(self.spec, i).items():
                if isinstance(name, list):
                    w[key] = [tuple(get(n) for n in trio) for trio in name]
                elif isinstance(name, tuple):
                    w[key] = tuple(get(n) for n in name)
                else:
                    w[key] = get(name)
            self.load_layer(i, w)
        idx.close()
        self.weights_source = path
        return self

    def load_synthetic(self, seed: int = 1234, gen_device: str | None = None):
        """Seeded random weights of the architecture (benchmarks, tests)."""
        dev = gen_device or str(self.device)
        head = synth_head(self.spec, seed, dev)
        self.load_head(head["embed"], head["head"], head["final_norm"], head["final_norm_b"])
        for i in range(self.num_layers):
            self.load_layer(i, synth_layer(self.spec, i, seed, dev))
        self.weights_source = f"synthetic(seed={seed})"
        return self


def _rand(gen, shape, scale, dev):
    return (scale * torch.randn(shape, generator=gen, device=dev)).to(torch.bfloat16)


def synth_head(spec: SeqModelSpec, seed: int, dev="cpu") -> dict:
    gen = torch.Generator(device=dev).manual_seed(seed - 1)
    return {"embed": _rand(gen, (spec.vocab, spec.width), 1.0 / max(spec.embed_scale, 1e-6), dev),
            "head": _rand(gen, (spec.vocab, spec.width), spec.width ** -0.5, dev),
            "final_norm": (1 + 0.1 * torch.randn(spec.width, generator=gen, device=dev)).to(torch.bfloat16),
            "final_norm_b": _rand(gen, (spec.width,), 0.1, dev)}


def synth_layer(spec: SeqModelSpec, i: int, seed: int, dev="cpu") -> dict:
    """bf16 tensors (as a checkpoint would hold them), so that every dtype mode sees the same weights."""
    gen = torch.Generator(device=dev).manual_seed(seed + i)
    l, W = spec.layers[i], spec.width
    r = lambda o, k, gain=1.0: _rand(gen, (o, k), gain * k ** -0.5, dev)
    around_one = lambda n: (1 + 0.1 * torch.randn(n, generator=gen, device=dev)).to(torch.bfloat16)
    vec = lambda n, s=0.1: _rand(gen, (n,), s, dev)
    hv = l.heads * l.vdim
    w = {"norm": around_one(W), "norm_b": vec(W), "ls1": around_one(W), "q": r(l.heads * (l.dim + l.rope_dim), W, 2.0),
         "dkv": r(l.kv_rank + l.rope_dim, W, 2.0), "dkv_norm": around_one(l.kv_rank), "uk": r(l.heads * l.dim, l.kv_rank, 2.0),
         "uv": r(hv, l.kv_rank), "sink": vec(l.heads, 1.0), "g": r(hv, W), "o": r(W, hv)}
    m = l.mlp
    if m is not None:
        w.update(norm2=around_one(W), norm2_b=vec(W), ls2=around_one(W))
        if m.experts:
            w["router"] = r(m.experts, W, 2.0)
            w["experts"] = [(r(m.ff, W), r(m.ff, W), r(W, m.ff)) for _ in range(m.experts)]
            if m.shared_ff:
                w["shared"] = (r(m.shared_ff, W), r(m.shared_ff, W), r(W, m.shared_ff))
                w["shared_gate"] = r(1, W, 2.0)
        else:
            w["dense"] = (r(m.shared_ff, W), r(m.shared_ff, W), r(W, m.shared_ff))
            w["dense_b"] = (vec(m.shared_ff), vec(m.shared_ff), vec(W))
    return w


def from_pretrained(path: str, device="cuda:0", dtype=torch.bfloat16, **kw) -> Kulisun:
    """Model of a checkpoint directory (config.json + model.safetensors); ``alloc()`` loads the weights."""
    spec = spec_from_config(json.load(open(os.path.join(path, "config.json"))))
    model = Kulisun(spec, device=device, dtype=dtype, model_name=path, **kw)
    base_alloc = model.alloc

    def alloc(**kwargs):
        base_alloc(**kwargs)
        if kwargs.get("synthetic") or "synthetic_seed" in kwargs:
            model.load_synthetic(kwargs.get("synthetic_seed", 1234))
        else:
            model.load_checkpoint(path)
        torch.cuda.synchronize(model.device)
        return model
    model.alloc = alloc
    return model
