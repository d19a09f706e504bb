"""Subivik: a pre-norm decoder family without statistics in its norms (dynamic tanh: tanh(alpha x) w + b) and with
sinusoidal positions added to the embedding; the logits come from the embedding table itself.  Its layers, in any order
given by config.json (``layers[i].type``), mix tokens by

* ``parallel`` -- two mixers side by side on the same normed input, summed with two constants: grouped-query attention
  over the whole sequence whose scores pass a tanh cap and lose a penalty r1 ln(1 + r2 distance) per head, and whose
  softmax weights are then mixed across heads by a learned matrix ("talking heads" after the softmax; the mixed weights
  meet the values of the head's own key/value head); and a time-mix memory: five token-shifted mixes of the input feed
  r, k, v, a silu gate and a low-rank map whose double exponential is the decay per key channel, the matrix state reads
  out with a bonus for the current token, then unit RMS per head, a weight and the gate;
* ``attention`` -- differential grouped-query attention: every query and key head holds two maps, RMS-normed with one
  weight vector, two softmaxes over the same values inside the row's chunk of ``mask.size`` positions, combined as
  a1 - lambda a2 with one learned lambda per layer, unit RMS per head times (1 - diff), an element-wise sigmoid output
  gate.  A layer with ``kv_from: j`` has no key / value projections and reads layer j's cached keys and values.

Feed-forward: dense W_down xielu(W_up h) (two learned numbers shape the activation), a mixture of silu-gated experts
(softmax over all experts, the ``top`` largest scores times ``router.scale``, not renormalised), or none.

This module is the family's front: config.json -> ``SeqModelSpec``, checkpoint tensor names -> ``load_layer`` dicts,
seeded synthetic weights for benchmarks and tests.  The computation is models/seq_model.py + csrc/seq: both attention
kinds are the framework's cached-attention mixer with score options, the recurrent half its time-mix mixer, the pair a
layer with a ``second`` mixer.

config.json keys read here:
    architecture = "Subivik"; width; vocab; norm.eps;
    layers[i].type = "parallel": mixer.{left: {heads, kv_heads, dim, vdim, scale, softcap}, right: {heads, dim},
                                         left_scale, right_scale}
    layers[i].type = "attention": mixer.{heads, kv_heads, dim, vdim, scale, diff, mask: {size}, kv_from}
    layers[i].mlp = null | {kind: "dense", ff} | {kind: "moe", router: {experts, top, scale}, expert: {ff}}
Tensors (safetensors, [out, in]): embed, final.norm (+ .b, .alpha), and per layer ``l<i>.``: norm1, norm2 (+ .b, .alpha),
mix.left.{q, k, v, r1, r2, talk, o}, mix.right.{mu.{r, k, v, g, w}, r, k, v, g, w1, w2, w0, u, norm, o},
mix.{q, k, v, q.norm, k.norm, lq1, lk1, lq2, lk2, g, o}, mlp.{up, down, act} or mlp.router, mlp.e<j>.{gate, up, down}.
"""
from __future__ import annotations

import json
import os

import torch

from .seq_model import SeqLayerSpec, SeqMlpSpec, SeqModelSpec, SeqStateModel

ARCHITECTURE = "Subivik"


def _attention_spec(mx: dict) -> SeqLayerSpec:
    l = SeqLayerSpec(mixer="cached_attention", heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                     form="prenorm", norm_kind="dyt", shift=False, depth_average=False)
    l.kv_heads, l.scale, l.attn_mode = int(mx.get("kv_heads", mx["heads"])), float(mx["scale"]), "softmax"
    if l.heads % l.kv_heads:
        raise ValueError("heads must be a multiple of kv_heads")
    return l


def spec_from_config(cfg: dict) -> SeqModelSpec:
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: architecture = {cfg.get('architecture')!r}")
    layers = []
    for i, entry in enumerate(cfg["layers"]):
        kind, mx = entry["type"], entry["mixer"]
        if kind == "parallel":
            l = _attention_spec(mx["left"])
            l.softcap, l.dist_bias, l.talk = float(mx["left"].get("softcap") or 0.0), True, True
            r = mx["right"]
            l.second = SeqLayerSpec(mixer="time_mix", heads=int(r["heads"]), dim=int(r["dim"]), vdim=int(r["dim"]),
                                    form="prenorm", shift=False, depth_average=False)
            l.mix_scale, l.second_scale = float(mx.get("left_scale", 1.0)), float(mx.get("right_scale", 1.0))
        elif kind == "attention":
            l = _attention_spec(mx)
            l.maps, l.diff, l.head_unit_norm, l.qk_norm, l.gate_kind = 2, float(mx["diff"]), True, True, 2
            l.chunk = int((mx.get("mask") or {}).get("size", 0))
            if mx.get("kv_from") is not None:
                l.kv_from = int(mx["kv_from"])
                if not 0 <= l.kv_from < i:
                    raise ValueError("kv_from must name an earlier layer")
        else:
            raise ValueError(f"unknown layer type '{kind}'")
        mlp = entry.get("mlp")
        if mlp is not None:
            mk = mlp.get("kind", "dense")
            if mk == "dense":
                l.mlp = SeqMlpSpec(shared_ff=int(mlp["ff"]), plain="xielu")
            elif mk == "moe":
                r = mlp["router"]
                l.mlp = SeqMlpSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(mlp["expert"]["ff"]), act="silu",
                                   route="softmax_all", route_scale=float(r.get("scale", 1.0)))
                if not 1 <= l.mlp.top <= l.mlp.experts:
                    raise ValueError("router: top must lie between 1 and experts")
            else:
                raise ValueError(f"unknown feed-forward kind '{mk}'")
        layers.append(l)
    eos = cfg.get("eos_token_id", [])
    return SeqModelSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers, norm_groups=1,
                        norm_eps=float(cfg["norm"]["eps"]), norm_kind="dyt", pos_embed="sinusoid", pos_base=10000.0,
                        eos_token_id=list(eos) if isinstance(eos, (list, tuple)) else [int(eos)])


def _attention_names(l: SeqLayerSpec, p: str) -> dict:
    names = {"q": p + "q", "o": p + "o"}
    if l.kv_from is None:
        names.update(k=p + "k", v=p + "v")
    if l.talk:
        names.update(r1=p + "r1", r2=p + "r2", talk=p + "talk")
    if l.maps == 2:
        names.update(q_norm=p + "q.norm", lq1=p + "lq1", lk1=p + "lk1", lq2=p + "lq2", lk2=p + "lk2", g=p + "g")
        if l.kv_from is None:
            names["k_norm"] = p + "k.norm"
    return names


def layer_tensor_names(spec: SeqModelSpec, i: int) -> dict:
    """load_layer key -> checkpoint tensor name(s) of layer i (``second``: the same for the layer's second mixer)."""
    l, p = spec.layers[i], f"l{i}."
    names = {"norm": p + "norm1", "norm_b": p + "norm1.b", "norm_alpha": p + "norm1.alpha"}
    if l.second is not None:
        names.update(_attention_names(l, p + "mix.left."))
        r = p + "mix.right."
        names["second"] = {"mu_r": r + "mu.r", "mu_k": r + "mu.k", "mu_v": r + "mu.v", "mu_g": r + "mu.g", "mu_w": r + "mu.w",
                           "r": r + "r", "k": r + "k", "v": r + "v", "g": r + "g", "w1": r + "w1", "w2": r + "w2", "w0": r + "w0",
                           "u": r + "u", "out_norm": r + "norm", "o": r + "o"}
    else:
        names.update(_attention_names(l, p + "mix."))
    m = l.mlp
    if m is not None:
        names.update({"norm2": p + "norm2", "norm2_b": p + "norm2.b", "norm2_alpha": p + "norm2.alpha"})
        if m.experts:
            names["router"] = p + "mlp.router"
            names["experts"] = [tuple(f"{p}mlp.e{e}.{n}" for n in ("gate", "up", "down")) for e in range(m.experts)]
        else:
            names["dense"] = (p + "mlp.up", p + "mlp.down")
            names["dense_act"] = p + "mlp.act"
    return names


def _gather(names, get):
    if isinstance(names, dict):
        return {k: _gather(v, get) for k, v in names.items()}
    if isinstance(names, list):
        return [_gather(v, get) for v in names]
    if isinstance(names, tuple):
        return tuple(get(n) for n in names)
    return get(names)


class Subivik(SeqStateModel):
    """``Subivik(spec, ...)``; ``alloc()`` then ``load_checkpoint(path)`` or ``load_synthetic(seed)``."""

    def load_tensors(self, get):
        """``get(name) -> tensor`` for the family's tensor names."""
        self.load_head(get("embed"), None, get("final.norm"), get("final.norm.b"), float(get("final.norm.alpha")))
        for i in range(self.num_layers):
            self.load_layer(i, _gather(layer_tensor_names(self.spec, i), get))
        return self

    def load_checkpoint(self, path: str):
        from .checkpoint import SafetensorsIndex
        idx = SafetensorsIndex(path)
        self.load_tensors(idx.get)
        idx.close()
        self.weights_source = path
        return self

    def load_synthetic(self, seed: int = 1234, gen_device: str | None = None):
        """Seeded random weights of the architecture (benchmarks, tests)."""
        t = synth_tensors(self.spec, seed, gen_device or str(self.device))
        self.load_tensors(t.__getitem__)
        self.weights_source = f"synthetic(seed={seed})"
        return self


def synth_tensors(spec: SeqModelSpec, seed: int, dev="cpu") -> dict:
    """name -> bf16 tensor (as a checkpoint would hold them), so that every dtype mode sees the same weights."""
    W, t = spec.width, {}
    gen = torch.Generator(device=dev).manual_seed(seed)
    r = lambda o, k, gain=1.0: (gain * k ** -0.5 * torch.randn(o, k, generator=gen, device=dev)).to(torch.bfloat16)
    vec = lambda n, s=0.1: (s * torch.randn(n, generator=gen, device=dev)).to(torch.bfloat16)
    one = lambda n, s=0.1: (1 + s * torch.randn(n, generator=gen, device=dev)).to(torch.bfloat16)

    def norm(name):
        t[name], t[name + ".b"], t[name + ".alpha"] = one(W), vec(W), torch.tensor(0.7, dtype=torch.bfloat16)

    def attention(l, p):
        t[p + "q"], t[p + "o"] = r(l.heads * l.maps * l.dim, W, 2.0), r(W, l.heads * l.vdim)
        if l.kv_from is None:
            t[p + "k"], t[p + "v"] = r(l.kv_heads * l.maps * l.dim, W, 2.0), r(l.kv_heads * l.vdim, W)
        if l.talk:
            t[p + "r1"], t[p + "r2"] = vec(l.heads, 0.3).abs(), vec(l.heads, 0.5).abs()
            t[p + "talk"] = (torch.eye(l.heads, device=dev) + 0.2 * torch.randn(l.heads, l.heads, generator=gen, device=dev)).to(torch.bfloat16)
        if l.maps == 2:
            t[p + "q.norm"], t[p + "g"] = one(l.dim), r(l.heads * l.vdim, W)
            for s in ("lq1", "lk1", "lq2", "lk2"):
                t[p + s] = vec(l.dim, 0.1)
            if l.kv_from is None:
                t[p + "k.norm"] = one(l.dim)

    t["embed"] = (torch.randn(spec.vocab, W, generator=gen, device=dev) * W ** -0.5).to(torch.bfloat16)
    norm("final.norm")
    for i, l in enumerate(spec.layers):
        p = f"l{i}."
        norm(p + "norm1")
        if l.second is not None:
            attention(l, p + "mix.left.")
            s, q = l.second, p + "mix.right."
            hd = s.heads * s.dim
            rank = max(8, min(64, W // 16)) // 8 * 8
            for n in "rkvgw":
                t[q + "mu." + n] = (0.5 + 0.2 * torch.randn(W, generator=gen, device=dev)).clamp(0, 1).to(torch.bfloat16)
            t[q + "r"], t[q + "k"], t[q + "v"], t[q + "g"] = r(hd, W), r(hd, W), r(hd, W), r(hd, W)
            t[q + "w1"], t[q + "w2"], t[q + "w0"] = r(rank, W), r(hd, rank), (vec(hd, 0.5) - 1.0)
            t[q + "u"], t[q + "norm"], t[q + "o"] = vec(hd, 0.3).reshape(s.heads, s.dim), one(hd), r(W, hd)
        else:
            attention(l, p + "mix.")
        m = l.mlp
        if m is None:
            continue
        norm(p + "norm2")
        if m.experts:
            t[p + "mlp.router"] = r(m.experts, W, 2.0)
            for e in range(m.experts):
                t[f"{p}mlp.e{e}.gate"], t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = r(m.ff, W), r(m.ff, W), r(W, m.ff)
        else:
            t[p + "mlp.up"], t[p + "mlp.down"], t[p + "mlp.act"] = r(m.shared_ff, W), r(W, m.shared_ff), vec(2, 0.5)
    return t


def from_pretrained(path: str, device="cuda:0", dtype=torch.bfloat16, **kw) -> Subivik:
    """Model of a checkpoint directory (config.json + model.safetensors); ``alloc()`` loads the weights."""
    spec = spec_from_config(json.load(open(os.path.join(path, "config.json"))))
    model = Subivik(spec, device=device, dtype=dtype, model_name=path, **kw)
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
