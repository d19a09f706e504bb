"""Plain, slow statement of the Kulisun mechanisms, one function per mechanism, in float64 on the CPU, written from
the equations -- the oracle the CUDA path is tested against.  It shares no code with umbrella_b200.  A model is a dict

    {"width", "vocab", "eps", "embed_scale", "residual_mult", "embed", "head", "final_norm": (w, b), "layers": [...]}
    layer: {"norm1": (w, b), "norm2": (w, b) | None, "ls1", "ls2" | None, "mix": {...}, "mlp": None | {...}}
      mix: heads, dim, rot_dim, vdim, kv_rank, scale, rot (dict), q, dkv, dkv_norm, uk, uv, sink, g, o
      mlp: {"kind": "dense", gate, gate_b, up, up_b, down, down_b}
         | {"kind": "moe", router, top, groups, keep, experts: [(gate, up, down)], shared: None | (gate, up, down, sg)}
    rot: {"dims", "base", "scaling": None | {factor, original, fast, slow}}

Every function takes a whole sequence [n, .]: no cache, no state, no batching.  Position i of a result depends on
tokens 0..i of that one sequence, which is what the product must reproduce however it is fed.
"""
import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------------------------- norms, activations
def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * w + b."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------------------------------------- rotary positions
def rotary_frequencies(rot):
    """-> (f [dims / 2], magnitude): the frequencies after the ramp of the scaling rule and the factor on cos and sin."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    where = lambda turns: dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(where(sc["fast"])), 0), min(math.ceil(where(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, rot):
    """x [n, ..., d]: the first rot.dims components of the last axis are turned, pairs (i, i + dims / 2), by
    position * f_i; the rest passes."""
    dims = rot["dims"]
    f, mag = rotary_frequencies(rot)
    n, half = x.shape[0], dims // 2
    ang = torch.arange(n, dtype=F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]
    shape = [n] + [1] * (x.dim() - 2) + [half]
    cos, sin = (torch.cos(ang) * mag).reshape(shape), (torch.sin(ang) * mag).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------------------------- latent attention
def sink_softmax_attention(q, k, v, scale, sink):
    """q, k [n, heads, d], v [n, heads, e]; causal; every row's denominator also holds exp(sink[head])."""
    n, H = q.shape[0], q.shape[1]
    out = torch.zeros(n, H, v.shape[-1], dtype=F64)
    seen = torch.tril(torch.ones(n, n, dtype=torch.bool))                    # row i sees keys j <= i
    for h in range(H):
        s = (q[:, h] @ k[:, h].T * scale).masked_fill(~seen, -math.inf)
        m = torch.maximum(s.max(-1, keepdim=True).values, sink[h].reshape(1, 1))
        e = torch.exp(s - m)
        out[:, h] = (e @ v[:, h]) / (e.sum(-1, keepdim=True) + torch.exp(sink[h] - m))
    return out


def latent_attention(h, mx, eps):
    """The mixer: queries straight from h, keys and values through one normed latent per token plus one rotated key part
    that all heads share; sigmoid gate on the concatenated heads."""
    n, H, D, Rt, V, R = h.shape[0], mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ mx["q"].T).reshape(n, H, D + Rt)
    low = h @ mx["dkv"].T
    c = rms_norm(low[:, :R], mx["dkv_norm"], eps)
    k_rot = rotate(low[:, R:], mx["rot"])                                   # [n, Rt], one for all heads
    q = torch.cat([q[..., :D], rotate(q[..., D:], mx["rot"])], dim=-1)
    k = torch.cat([(c @ mx["uk"].T).reshape(n, H, D), k_rot[:, None, :].expand(n, H, Rt)], dim=-1)
    v = (c @ mx["uv"].T).reshape(n, H, V)
    o = sink_softmax_attention(q, k, v, mx["scale"], mx["sink"]).reshape(n, H * V)
    return (o * torch.sigmoid(h @ mx["g"].T)) @ mx["o"].T


# ---------------------------------------------------------------------------------------------- feed-forward
def dense_ff(h, m):
    return (silu(h @ m["gate"].T + m["gate_b"]) * (h @ m["up"].T + m["up_b"])) @ m["down"].T + m["down_b"]


def expert_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, m):
    """-> per token the chosen experts and their weights.  Sigmoid scores; groups of neighbouring experts are ranked
    by the sum of their two best scores and only the best ``keep`` groups stay eligible."""
    s = torch.sigmoid(h @ m["router"].T)
    n, E = s.shape
    G, per = m["groups"], E // m["groups"]
    chosen, weights = [], []
    for t in range(n):
        st = s[t]
        gscore = [float(torch.sort(st[g * per:(g + 1) * per], descending=True).values[:2].sum()) for g in range(G)]
        order = sorted(range(G), key=lambda g: (-gscore[g], g))[: m["keep"]]
        ok = [e for e in range(E) if e // per in order]
        pick = sorted(ok, key=lambda e: (-float(st[e]), e))[: m["top"]]
        w = torch.stack([st[e] for e in pick])
        chosen.append(pick)
        weights.append(w / (w.sum() + 1e-20))
    return chosen, weights


def moe_ff(h, m):
    chosen, weights = route(h, m)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * expert_ff(h[t:t + 1], *m["experts"][e])[0]
    if m.get("shared") is not None:
        g, u, d, sg = m["shared"]
        out = out + expert_ff(h, g, u, d) * torch.sigmoid(h @ sg.reshape(1, -1).T)
    return out


# ---------------------------------------------------------------------------------------------- the model
def forward(model, tokens, layer_out=False):
    """Logits [n, vocab] of one whole sequence (and the residual stream after every layer)."""
    eps, mult = model["eps"], model["residual_mult"]
    x = model["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(F64) * model["embed_scale"]
    streams = []
    for l in model["layers"]:
        x = x + mult * (l["ls1"] * latent_attention(layer_norm(x, *l["norm1"], eps), l["mix"], eps))
        if l["mlp"] is not None:
            hn = layer_norm(x, *l["norm2"], eps)
            ff = dense_ff(hn, l["mlp"]) if l["mlp"]["kind"] == "dense" else moe_ff(hn, l["mlp"])
            x = x + mult * (l["ls2"] * ff)
        streams.append(x)
    logits = layer_norm(x, *model["final_norm"], eps) @ model["head"].T
    return (logits, torch.stack(streams)) if layer_out else logits
