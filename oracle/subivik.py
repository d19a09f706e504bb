"""Plain, slow statement of the Subivik mechanisms, one function per mechanism, in float64 on the CPU, written from
the equations -- the oracle the CUDA path is tested against.  It shares no code with umbrella_b200.  A model is

    {"width", "vocab", "eps", "embed", "final_norm": (alpha, w, b), "layers": [...]}
    layer: {"type": "parallel" | "attention", "norm1": (alpha, w, b), "norm2": (alpha, w, b) | None, "mix": {...},
            "mlp": None | {...}}
      parallel mix: {"left": {heads, kv_heads, dim, vdim, scale, softcap, q, k, v, r1, r2, talk, o},
                     "right": {heads, dim, mu: {r, k, v, g, w}, r, k, v, g, w1, w2, w0, u, norm, o},
                     "left_scale", "right_scale"}
      attention mix: {heads, kv_heads, dim, vdim, scale, chunk, diff, kv_from | None, q, k, v, q_norm, k_norm,
                      lq1, lk1, lq2, lk2, g, o}      (k, v, k_norm absent with kv_from)
      mlp: {"kind": "dense", up, down, act: (p, q)}
         | {"kind": "moe", router, top, scale, experts: [(gate, up, down)]}

Every function takes a whole sequence [n, .]: no cache, no state, no batching.  Position i of a result depends on
tokens 0..i of that one sequence, which is what the product must reproduce however it is fed.
"""
import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------------------------- element-wise pieces
def dynamic_tanh(x, alpha, w, b):
    """The norm without statistics: tanh(alpha x) w + b."""
    return torch.tanh(alpha * x) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def softplus(z):
    return math.log1p(math.exp(z))


def xielu(z, p, q):
    """Quadratic on the positive side, exponential on the negative side, slope 1/2 at zero from both."""
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def silu(z):
    return z * torch.sigmoid(z)


def sinusoid_positions(n, width, first=0):
    """[n, width]: column 2i = sin(p f_i), column 2i + 1 = cos(p f_i), f_i = 10000^(-2i / width)."""
    p = torch.arange(first, first + n, dtype=F64)[:, None]
    f = torch.tensor([10000.0 ** (-2.0 * i / width) for i in range(width // 2)], dtype=F64)[None, :]
    out = torch.zeros(n, width, dtype=F64)
    out[:, 0::2], out[:, 1::2] = torch.sin(p * f), torch.cos(p * f)
    return out


# ---------------------------------------------------------------------------------------------- attention pieces
def causal(n):
    return torch.tril(torch.ones(n, n, dtype=torch.bool))


def chunk_mask(n, size):
    """Row i sees j <= i of its own chunk of `size` positions, chunks counted from position 0."""
    i = torch.arange(n)
    return causal(n) & ((i[:, None] // size) == (i[None, :] // size))


def softmax_weights(scores, seen):
    s = scores.masked_fill(~seen, -math.inf)
    e = torch.exp(s - s.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


def distance_penalty(n, r1, r2):
    """r1 ln(1 + r2 (i - j)) for j <= i (0 elsewhere)."""
    i = torch.arange(n, dtype=F64)
    d = (i[:, None] - i[None, :]).clamp(min=0.0)
    return r1 * torch.log1p(r2 * d)


def talking_attention(h, m):
    """Grouped-query attention whose scores pass a tanh cap and lose a penalty growing with the logarithm of the
    distance; after the softmax every head's weights become a learned mix of all heads' weights."""
    n, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ m["q"].T).reshape(n, H, D)
    k = (h @ m["k"].T).reshape(n, G, D)
    v = (h @ m["v"].T).reshape(n, G, V)
    seen, rep = causal(n), H // G
    weights = []
    for a in range(H):
        s = q[:, a] @ k[:, a // rep].T * m["scale"]
        if m.get("softcap"):
            s = m["softcap"] * torch.tanh(s / m["softcap"])
        s = s - distance_penalty(n, m["r1"][a], m["r2"][a])
        weights.append(softmax_weights(s, seen))
    out = torch.zeros(n, H, V, dtype=F64)
    for a in range(H):
        mixed = sum(m["talk"][a, b] * weights[b] for b in range(H))
        out[:, a] = mixed @ v[:, a // rep]
    return out.reshape(n, H * V) @ m["o"].T


def shifted(h):
    """The previous token's row (zeros in front of the first)."""
    return torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)


def decayed_memory(r, k, v, w, u):
    """Per head: o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T.  r, k, v, w [n, heads, d]; u [heads, d]."""
    n, H, D = r.shape
    S = torch.zeros(H, D, D, dtype=F64)
    out = torch.zeros(n, H, D, dtype=F64)
    for t in range(n):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = w[t][:, :, None] * S + kv
    return out


def time_mixing(h, m, eps):
    """The recurrent half: five token-shifted mixes of the input, a decay per key channel from a low-rank map of its
    own mix, the matrix memory with a bonus for the current token, unit RMS per head, a weight, a silu gate."""
    n, H, D = h.shape[0], m["heads"], m["dim"]
    prev = shifted(h)
    mix = {s: h + (prev - h) * m["mu"][s] for s in "rkvgw"}
    r = (mix["r"] @ m["r"].T).reshape(n, H, D)
    k = (mix["k"] @ m["k"].T).reshape(n, H, D)
    v = (mix["v"] @ m["v"].T).reshape(n, H, D)
    gate = silu(mix["g"] @ m["g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mix["w"] @ m["w1"].T) @ m["w2"].T + m["w0"])).reshape(n, H, D)
    o = decayed_memory(r, k, v, w, m["u"])
    o = unit_rms(o, eps).reshape(n, H * D) * m["norm"] * gate
    return o @ m["o"].T


def parallel_mixer(h, m, eps):
    return m["left_scale"] * talking_attention(h, m["left"]) + m["right_scale"] * time_mixing(h, m["right"], eps)


def differential_keys_values(h, m, eps):
    """What the layer caches: keys after their norm [n, kv_heads, 2, dim] and values [n, kv_heads, vdim]."""
    n, G, D, V = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = unit_rms((h @ m["k"].T).reshape(n, G, 2, D), eps) * m["k_norm"]
    return k, (h @ m["v"].T).reshape(n, G, V)


def differential_attention(h, m, eps, k, v):
    """Two softmax maps per head over the same values, the second subtracted with one learned factor per layer; the
    difference gets unit RMS per head, the factor 1 - diff and an element-wise sigmoid gate.  Keys are seen inside the
    row's own chunk only.  k, v: this layer's own, or those of the layer it borrows from."""
    n, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ m["q"].T).reshape(n, H, 2, D), eps) * m["q_norm"]
    lam = math.exp(float((m["lq1"] * m["lk1"]).sum())) - math.exp(float((m["lq2"] * m["lk2"]).sum())) + m["diff"]
    seen, rep = chunk_mask(n, m["chunk"]) if m["chunk"] else causal(n), H // G
    out = torch.zeros(n, H, V, dtype=F64)
    for a in range(H):
        maps = [softmax_weights(q[:, a, j] @ k[:, a // rep, j].T * m["scale"], seen) @ v[:, a // rep] for j in (0, 1)]
        out[:, a] = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    return (out.reshape(n, H * V) * torch.sigmoid(h @ m["g"].T)) @ m["o"].T


# ---------------------------------------------------------------------------------------------- feed-forward
def dense_ff(h, m):
    p, q = float(m["act"][0]), float(m["act"][1])
    return xielu(h @ m["up"].T, p, q) @ m["down"].T


def routed_ff(h, m):
    """Softmax over all experts, the `top` largest scores (ties to the lower index) times `scale`, not renormalised."""
    s = torch.softmax(h @ m["router"].T, dim=-1)
    out = torch.zeros(h.shape[0], m["experts"][0][2].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(s[t, e]), e))[:m["top"]]
        for e in order:
            gate, up, down = m["experts"][e]
            out[t] += m["scale"] * s[t, e] * ((silu(h[t] @ gate.T) * (h[t] @ up.T)) @ down.T)
    return out


# ---------------------------------------------------------------------------------------------- the model
def forward(model, tokens):
    """-> (logits [n, vocab], residual stream after every layer [layers, n, width]) of one sequence, float64."""
    n, eps = len(tokens), model["eps"]
    x = model["embed"][torch.tensor(tokens)] + sinusoid_positions(n, model["width"])
    streams, kept = [], {}
    for i, L in enumerate(model["layers"]):
        h = dynamic_tanh(x, *L["norm1"])
        m = L["mix"]
        if L["type"] == "parallel":
            x = x + parallel_mixer(h, m, eps)
        else:
            if m.get("kv_from") is None:
                kept[i] = differential_keys_values(h, m, eps)
            x = x + differential_attention(h, m, eps, *kept[i if m.get("kv_from") is None else m["kv_from"]])
        if L["mlp"] is not None:
            h = dynamic_tanh(x, *L["norm2"])
            x = x + (dense_ff(h, L["mlp"]) if L["mlp"]["kind"] == "dense" else routed_ff(h, L["mlp"]))
        streams.append(x)
    x = dynamic_tanh(x, *model["final_norm"])
    return x @ model["embed"].T, torch.stack(streams)


def from_tensors(cfg, t):
    """config dict (as config.json holds it) + name -> tensor  ->  the model dict above, float64."""
    f = lambda name: t[name].to(F64)
    norm = lambda name: (float(t[name + ".alpha"]), f(name), f(name + ".b"))
    layers = []
    for i, e in enumerate(cfg["layers"]):
        p, c = f"l{i}.", e["mixer"]
        if e["type"] == "parallel":
            a, b = c["left"], c["right"]
            left = dict(heads=a["heads"], kv_heads=a["kv_heads"], dim=a["dim"], vdim=a["vdim"], scale=a["scale"],
                        softcap=a.get("softcap"), **{s: f(p + "mix.left." + s) for s in ("q", "k", "v", "r1", "r2", "talk", "o")})
            right = dict(heads=b["heads"], dim=b["dim"], mu={s: f(p + "mix.right.mu." + s) for s in "rkvgw"},
                         **{s: f(p + "mix.right." + s) for s in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")})
            mix = dict(left=left, right=right, left_scale=c["left_scale"], right_scale=c["right_scale"])
        else:
            mix = dict(heads=c["heads"], kv_heads=c["kv_heads"], dim=c["dim"], vdim=c["vdim"], scale=c["scale"],
                       chunk=(c.get("mask") or {}).get("size", 0), diff=c["diff"], kv_from=c.get("kv_from"),
                       q_norm=f(p + "mix.q.norm"), **{s: f(p + "mix." + s) for s in ("q", "lq1", "lk1", "lq2", "lk2", "g", "o")})
            if c.get("kv_from") is None:
                mix.update(k=f(p + "mix.k"), v=f(p + "mix.v"), k_norm=f(p + "mix.k.norm"))
        m = e.get("mlp")
        if m is None:
            mlp = None
        elif m["kind"] == "dense":
            mlp = dict(kind="dense", up=f(p + "mlp.up"), down=f(p + "mlp.down"), act=f(p + "mlp.act"))
        else:
            r = m["router"]
            mlp = dict(kind="moe", router=f(p + "mlp.router"), top=r["top"], scale=r["scale"],
                       experts=[tuple(f(f"{p}mlp.e{j}.{s}") for s in ("gate", "up", "down")) for j in range(r["experts"])])
        layers.append(dict(type=e["type"], norm1=norm(p + "norm1"), norm2=norm(p + "norm2") if m is not None else None,
                           mix=mix, mlp=mlp))
    return dict(width=cfg["width"], vocab=cfg["vocab"], eps=cfg["norm"]["eps"], embed=f("embed"),
                final_norm=norm("final.norm"), layers=layers)
