"""Test-only helpers for the Subivik family: small random models, built twice from the same tensors -- as the oracle's
plain dict (float64, oracle/subivik.py) and as the product model (a checkpoint directory read by the family's config
reader and loader).  A configuration here is the family's config.json itself."""
import json
import os

import torch


def left(heads, kv_heads, dim, vdim, softcap=6.0):
    d = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=1.3 * dim ** -0.5)
    if softcap:
        d["softcap"] = softcap
    return d


def parallel(lf, heads, dim, scales=(0.6, 1.3), mlp=None):
    return dict(type="parallel", mixer=dict(left=lf, right=dict(heads=heads, dim=dim), left_scale=scales[0], right_scale=scales[1]),
                mlp=mlp)


def attention(heads, kv_heads, dim, vdim, chunk=0, diff=0.25, kv_from=None, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=1.6 * dim ** -0.5, diff=diff)
    if chunk:
        m["mask"] = dict(size=chunk)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m, mlp=mlp)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, scale=1.7):
    return dict(kind="moe", router=dict(experts=experts, top=top, scale=scale), expert=dict(ff=ff))


def model(width, vocab, layers, eps=1e-5):
    return dict(architecture="Subivik", width=width, vocab=vocab, norm=dict(eps=eps), layers=layers)


# every branch: both layer kinds in both orders; dense / routed / no feed-forward; a borrower with a wider chunk than its
# lender and one without a mask; heads = kv_heads and one kv head; no score cap; top = experts and top = 1; one recurrent head
MIXED = model(80, 113, [
    attention(4, 2, 12, 20, chunk=16, mlp=moe(5, 2, 24)),
    parallel(left(6, 3, 10, 14), 3, 20, mlp=dense(48)),
    attention(4, 2, 12, 20, chunk=24, diff=0.4, kv_from=0, mlp=None),
    parallel(left(2, 2, 24, 8, softcap=0), 1, 40, scales=(1.0, 0.5), mlp=moe(3, 3, 16, scale=0.8)),
    attention(2, 1, 16, 16, mlp=dense(40)),
    attention(2, 1, 16, 16, chunk=7, diff=0.1, kv_from=4, mlp=moe(4, 1, 32, scale=2.0)),
])
# dimensions the bf16 tensor-core product takes (every K a multiple of 32)
ALIGNED = model(128, 160, [
    parallel(left(4, 2, 32, 64, softcap=20.0), 2, 64, mlp=dense(256)),
    attention(4, 2, 32, 32, chunk=64, mlp=moe(6, 2, 64)),
    attention(4, 2, 32, 32, chunk=64, kv_from=1, mlp=dense(128)),
], eps=1e-6)


def _bf(t):
    return t.to(torch.bfloat16).to(torch.float32)          # values a bf16 checkpoint can hold


def random_tensors(cfg, seed=0):
    """name -> fp32 tensor (bf16-representable), with the family's checkpoint names."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    r = lambda o, k, gain=1.0: _bf(gain * k ** -0.5 * torch.randn(o, k, generator=g))
    vec = lambda n, s=0.2: _bf(s * torch.randn(n, generator=g))
    one = lambda n, s=0.2: _bf(1 + s * torch.randn(n, generator=g))
    t = {"embed": _bf(torch.randn(cfg["vocab"], W, generator=g))}

    def norm(name):
        t[name], t[name + ".b"], t[name + ".alpha"] = one(W), vec(W), _bf(torch.tensor(0.4 + 0.5 * float(torch.rand(1, generator=g))))
    norm("final.norm")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        norm(p + "norm1")
        if L["type"] == "parallel":
            a, b, q = m["left"], m["right"], p + "mix.left."
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            t[q + "q"], t[q + "k"], t[q + "v"], t[q + "o"] = r(H * D, W, 2.5), r(G * D, W, 2.5), r(G * V, W), r(W, H * V)
            t[q + "r1"], t[q + "r2"] = vec(H, 0.8).abs(), vec(H, 1.5).abs()
            t[q + "talk"] = _bf(0.6 * torch.randn(H, H, generator=g))
            q, hd = p + "mix.right.", b["heads"] * b["dim"]
            for s in "rkvgw":
                t[q + "mu." + s] = _bf(torch.rand(W, generator=g))
            t[q + "r"], t[q + "k"], t[q + "v"], t[q + "g"] = r(hd, W, 1.5), r(hd, W, 1.5), r(hd, W), r(hd, W, 1.5)
            rank = 6 + 2 * i
            t[q + "w1"], t[q + "w2"], t[q + "w0"] = r(rank, W, 2.0), r(hd, rank, 2.0), _bf(vec(hd, 1.0) - 0.5)
            t[q + "u"], t[q + "norm"], t[q + "o"] = vec(hd, 0.6).reshape(b["heads"], b["dim"]), one(hd), r(W, hd)
        else:
            H, G, D, V, q = m["heads"], m["kv_heads"], m["dim"], m["vdim"], p + "mix."
            t[q + "q"], t[q + "g"], t[q + "o"], t[q + "q.norm"] = r(2 * H * D, W, 2.0), r(H * V, W, 2.0), r(W, H * V), one(D, 0.4)
            for s in ("lq1", "lk1", "lq2", "lk2"):
                t[q + s] = vec(D, 0.25)
            if m.get("kv_from") is None:
                t[q + "k"], t[q + "v"], t[q + "k.norm"] = r(2 * G * D, W, 2.0), r(G * V, W), one(D, 0.4) * 2.0
        f = L["mlp"]
        if f is None:
            continue
        norm(p + "norm2")
        if f["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.down"], t[p + "mlp.act"] = r(f["ff"], W, 1.5), r(W, f["ff"]), vec(2, 0.8)
        else:
            t[p + "mlp.router"] = r(f["router"]["experts"], W, 3.0)
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                t[f"{p}mlp.e{e}.gate"], t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = r(ff, W, 1.5), r(ff, W), r(W, ff)
    return t


def oracle_model(cfg, t):
    from oracle import subivik as O
    return O.from_tensors(cfg, t)


def write_checkpoint(path, cfg, t):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    json.dump(cfg, open(os.path.join(path, "config.json"), "w"))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}, os.path.join(path, "model.safetensors"))
    return path


def product_model(cfg, t, dtype=torch.float32, device="cuda:0", slots=4, tmp=None, **kw):
    """The product model over the same tensors, through the registry, the family's config reader and its loader."""
    import tempfile
    from umbrella_b200.models.auto_model import AutoModelLM
    d = write_checkpoint(tmp or tempfile.mkdtemp(prefix="subckpt"), cfg, t)
    m = AutoModelLM.from_pretrained(d, device=device, dtype=dtype, slots=slots, **kw)
    m.alloc()
    return m


def row_errs(a, b):
    """Per-row rms difference relative to the rms of the whole reference."""
    a, b = a.double().cpu(), b.double().cpu()
    return (a - b).pow(2).mean(-1).sqrt() / b.pow(2).mean().sqrt().clamp_min(1e-30)


def row_err(a, b):
    return float(row_errs(a, b).max())
