"""Test-only helpers for the Kulisun family: small random models, built twice from the same tensors -- as the oracle's
plain dict (float64, oracle/kulisun.py) and as the product model (a checkpoint directory read by the family's config
reader and loader)."""
import json
import os

import torch

YARN = dict(factor=4.0, original=24, fast=6.0, slow=1.0)
LAT = dict(heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.2, rot=dict(dims=8, base=100.0, scaling=YARN))
MOE = dict(kind="moe", experts=8, top=3, groups=4, keep=2, ff=24, shared=32)

# every branch: dense / routed / no feed-forward, a shared expert or none, groups of one expert, one group, top 1, one head,
# rotation on part of the rotated dimensions, unscaled rotation, no rotation with and without a shared key part, vdim = dim
MIXED = dict(width=64, vocab=96, eps=1e-5, embed_scale=3.0, residual_mult=0.6, layers=[
    dict(LAT, mlp=dict(kind="dense", ff=48)),
    dict(LAT, mlp=MOE),
    dict(LAT, heads=1, dim=24, vdim=8, rot=dict(dims=4, base=50.0, scaling=None), mlp=None),
    dict(LAT, rot_dim=0, rot=None, vdim=16, mlp=dict(MOE, experts=5, top=1, groups=1, keep=1, shared=None)),
    dict(LAT, heads=3, kv_rank=20, rot_dim=12, rot=dict(dims=12, base=1000.0, scaling=dict(factor=8.0, original=16, fast=4.0, slow=2.0)),
         mlp=dict(MOE, experts=4, top=2, groups=4, keep=3, ff=40, shared=16)),
    dict(LAT, rot=None, mlp=dict(kind="dense", ff=40)),
])
# dimensions the bf16 tensor-core product takes (every K a multiple of 32)
ALIGNED = dict(width=128, vocab=160, eps=1e-6, embed_scale=1.0, residual_mult=1.0, layers=[
    dict(LAT, heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=64, rot=dict(dims=32, base=1e4, scaling=None), mlp=dict(kind="dense", ff=64)),
    dict(LAT, heads=2, dim=64, rot_dim=32, vdim=64, kv_rank=96, rot=dict(dims=32, base=1e4, scaling=dict(factor=16.0, original=64, fast=16.0, slow=1.0)),
         mlp=dict(MOE, experts=6, top=2, groups=3, keep=2, ff=64, shared=64)),
    dict(LAT, heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=64, rot=dict(dims=32, base=1e4, scaling=None), mlp=None),
])


def _bf(t):
    return t.to(torch.bfloat16).to(torch.float32)          # values a bf16 checkpoint can hold


def random_tensors(cfg, seed=0):
    """name -> fp32 tensor (bf16-representable), with the family's checkpoint names."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    r = lambda o, k, gain=1.0: _bf(gain * k ** -0.5 * torch.randn(o, k, generator=g))
    vec = lambda n, s=0.2: _bf(s * torch.randn(n, generator=g))
    one = lambda n, s=0.2: _bf(1 + s * torch.randn(n, generator=g))
    t = {"embed": _bf(torch.randn(cfg["vocab"], W, generator=g) / cfg["embed_scale"]), "head": r(cfg["vocab"], W),
         "final.norm": one(W), "final.norm.b": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        p, H, D, Rt, V, R = f"l{i}.", L["heads"], L["dim"], L["rot_dim"], L["vdim"], L["kv_rank"]
        t[p + "norm1"], t[p + "norm1.b"], t[p + "ls1"] = one(W), vec(W), one(W, 0.3)
        t[p + "mix.q"], t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = r(H * (D + Rt), W, 2.5), r(R + Rt, W, 2.5), one(R)
        t[p + "mix.uk"], t[p + "mix.uv"] = r(H * D, R, 2.0), r(H * V, R)
        t[p + "mix.sink"], t[p + "mix.g"], t[p + "mix.o"] = vec(H, 1.5), r(H * V, W, 2.0), r(W, H * V)
        m = L["mlp"]
        if m is None:
            continue
        t[p + "norm2"], t[p + "norm2.b"], t[p + "ls2"] = one(W), vec(W), one(W, 0.3)
        if m["kind"] == "dense":
            for n, (o, k) in (("gate", (m["ff"], W)), ("up", (m["ff"], W)), ("down", (W, m["ff"]))):
                t[p + "mlp." + n], t[p + "mlp." + n + ".b"] = r(o, k, 1.5), vec(o, 0.3)
        else:
            t[p + "mlp.router"] = r(m["experts"], W, 3.0)
            for e in range(m["experts"]):
                t[f"{p}mlp.e{e}.gate"], t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = r(m["ff"], W, 1.5), r(m["ff"], W), r(W, m["ff"])
            if m["shared"]:
                s = m["shared"]
                t[p + "mlp.shared.gate"], t[p + "mlp.shared.up"], t[p + "mlp.shared.down"] = r(s, W, 1.5), r(s, W), r(W, s)
                t[p + "mlp.shared.sg"] = r(1, W, 3.0)
    return t


def _rot(L):
    rot = L.get("rot")
    if not rot or not L["rot_dim"]:
        return dict(dims=0, base=1.0, scaling=None)
    return dict(dims=rot["dims"], base=rot["base"], scaling=rot.get("scaling"))


def oracle_model(cfg, t):
    d = lambda n: t[n].double()
    layers = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        mix = dict(heads=L["heads"], dim=L["dim"], rot_dim=L["rot_dim"], vdim=L["vdim"], kv_rank=L["kv_rank"], scale=L["scale"],
                   rot=_rot(L), q=d(p + "mix.q"), dkv=d(p + "mix.dkv"), dkv_norm=d(p + "mix.dkv.norm"), uk=d(p + "mix.uk"),
                   uv=d(p + "mix.uv"), sink=d(p + "mix.sink"), g=d(p + "mix.g"), o=d(p + "mix.o"))
        o = dict(norm1=(d(p + "norm1"), d(p + "norm1.b")), ls1=d(p + "ls1"), mix=mix, mlp=None, norm2=None, ls2=None)
        m = L["mlp"]
        if m is not None:
            o["norm2"], o["ls2"] = (d(p + "norm2"), d(p + "norm2.b")), d(p + "ls2")
            if m["kind"] == "dense":
                o["mlp"] = dict(kind="dense", gate=d(p + "mlp.gate"), gate_b=d(p + "mlp.gate.b"), up=d(p + "mlp.up"),
                                up_b=d(p + "mlp.up.b"), down=d(p + "mlp.down"), down_b=d(p + "mlp.down.b"))
            else:
                sh = tuple(d(p + "mlp.shared." + n) for n in ("gate", "up", "down", "sg")) if m["shared"] else None
                o["mlp"] = dict(kind="moe", router=d(p + "mlp.router"), top=m["top"], groups=m["groups"], keep=m["keep"], shared=sh,
                                experts=[tuple(d(f"{p}mlp.e{e}.{n}") for n in ("gate", "up", "down")) for e in range(m["experts"])])
        layers.append(o)
    return dict(width=cfg["width"], vocab=cfg["vocab"], eps=cfg["eps"], embed_scale=cfg["embed_scale"],
                residual_mult=cfg["residual_mult"], embed=d("embed"), head=d("head"),
                final_norm=(d("final.norm"), d("final.norm.b")), layers=layers)


def config_json(cfg):
    """The family's config.json for ``cfg``."""
    layers = []
    for L in cfg["layers"]:
        mixer = dict(heads=L["heads"], dim=L["dim"], rot_dim=L["rot_dim"], vdim=L["vdim"], kv_rank=L["kv_rank"], scale=L["scale"])
        if L.get("rot") and L["rot_dim"]:
            rot = dict(dims=L["rot"]["dims"], base=L["rot"]["base"])
            if L["rot"].get("scaling"):
                rot["scaling"] = L["rot"]["scaling"]
            mixer["rot"] = rot
        m = L["mlp"]
        if m is not None and m["kind"] == "moe":
            m = dict(kind="moe", router=dict(experts=m["experts"], top=m["top"], groups=dict(count=m["groups"], keep=m["keep"])),
                     expert=dict(ff=m["ff"]), shared=dict(ff=m["shared"]) if m["shared"] else None)
        layers.append(dict(type="latent_attention", mixer=mixer, mlp=m))
    return dict(architecture="Kulisun", width=cfg["width"], vocab=cfg["vocab"], norm=dict(eps=cfg["eps"]),
                embedding=dict(scale=cfg["embed_scale"]), residual_mult=cfg["residual_mult"], layers=layers)


def write_checkpoint(path, cfg, t):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    json.dump(config_json(cfg), open(os.path.join(path, "config.json"), "w"))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}, os.path.join(path, "model.safetensors"))
    return path


def product_model(cfg, t, dtype=torch.float32, device="cuda:0", slots=4, tmp=None, **kw):
    """The product model over the same tensors, through the registry, the family's config reader and its loader."""
    import tempfile
    from umbrella_b200.models.auto_model import AutoModelLM
    d = write_checkpoint(tmp or tempfile.mkdtemp(prefix="kulckpt"), cfg, t)
    m = AutoModelLM.from_pretrained(d, device=device, dtype=dtype, slots=slots, **kw)
    m.alloc()
    return m


def row_err(a, b):
    """Largest per-row rms difference relative to the rms of the whole reference."""
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).pow(2).mean(-1).sqrt().max() / b.pow(2).mean().sqrt().clamp_min(1e-30))


def row_errs(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return (a - b).pow(2).mean(-1).sqrt() / b.pow(2).mean().sqrt().clamp_min(1e-30)
