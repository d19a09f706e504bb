"""Tensor-level wrappers over the building blocks of libumbrella_b200_seq.so (torch tensors in, raw pointers out),
the counterpart of ops.py for the sequence-state decoders.  Each call enqueues on ``torch.cuda.current_stream()``.

``dtype`` of the activations / weights is read off the tensors: torch.bfloat16 or torch.float32.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib_seq as S


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _mode(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise RuntimeError("CUDA tensors only (there is no CPU path)")
    if t.dtype == torch.bfloat16:
        return S.UMBS_BF16
    if t.dtype == torch.float32:
        return S.UMBS_F32
    raise TypeError(f"bfloat16 or float32 expected, got {t.dtype}")


def _i32(x, device):
    return torch.as_tensor(x, dtype=torch.int32).to(device)


class RaggedBatch:
    """Device copy of one step's batch description.  ``seqs``: [(slot, n_tokens, pos0, parity)]."""

    def __init__(self, seqs, device, token_ids=None, want=None):
        tok_seq, tok_pos, start = [], [], []
        for b, (slot, n, pos0, par) in enumerate(seqs):
            start.append(len(tok_seq))
            tok_seq += [b] * n
            tok_pos += range(pos0, pos0 + n)
        T = len(tok_seq)
        self.t = dict(tok_ids=_i32(token_ids if token_ids is not None else [0] * T, device), tok_seq=_i32(tok_seq, device),
                      tok_pos=_i32(tok_pos, device), seq_slot=_i32([s[0] for s in seqs], device),
                      seq_start=_i32(start, device), seq_len=_i32([s[1] for s in seqs], device),
                      seq_pos0=_i32([s[2] for s in seqs], device), seq_parity=_i32([s[3] for s in seqs], device),
                      want_rows=_i32(want if want is not None else [], device))
        c = S.Batch()
        c.n_tokens, c.n_seqs, c.n_want = T, len(seqs), len(want) if want is not None else 0
        c.max_seq_len = max(s[1] for s in seqs) if seqs else 0
        c.max_pos0 = max(s[2] for s in seqs) if seqs else 0
        for k, v in self.t.items():
            setattr(c, k, v.data_ptr())
        self.c, self.n_tokens = c, T


def gemm(a: torch.Tensor, w: torch.Tensor, *, out_f32: bool = False, groups: int = 1, a_goff: int = 0, c_goff: int = 0,
         n: int | None = None, k: int | None = None, grp_off=None, row_src=None, rows: int | None = None,
         dual: bool = False, limit: float = 0.0, max_rows: int | None = None) -> torch.Tensor:
    """a [M, lda] x w ([groups,] N(or 2N if dual), K) -> [rows, groups * c_goff or N].  See umbs_gemm."""
    mode = _mode(a)
    assert w.dtype == a.dtype and a.stride(-1) == 1 and w.is_contiguous()
    w3 = w if w.dim() == 3 else w.unsqueeze(0)
    K = w3.shape[2] if k is None else k
    N = (w3.shape[1] // (2 if dual else 1)) if n is None else n
    M = a.shape[0] if rows is None else rows
    cols = N if (groups == 1 or grp_off is not None) else groups * c_goff        # expert groups share the columns
    out = torch.zeros((M, cols), dtype=torch.float32 if out_f32 else a.dtype, device=a.device)
    S.check(S.load().umbs_gemm(mode, _p(a), a.stride(0), a_goff, _p(w3), w3.stride(1), w3.stride(0), _p(out), out.stride(0),
                               c_goff, int(out_f32), M if max_rows is None else max_rows, N, K, groups, _p(grp_off),
                               _p(row_src), int(dual), float(limit), _stream()), "gemm")
    return out


def group_norm_shift(x, w, shift_w, shift_state, batch: RaggedBatch, groups: int, eps: float, dtype=torch.float32):
    T, width = x.shape
    h = torch.empty((T, width), dtype=dtype, device=x.device)
    hs = torch.empty_like(h)
    S.check(S.load().umbs_group_norm_shift(_mode(h), _p(x), _p(w), _p(shift_w), _p(shift_state), shift_state.shape[1],
                                           C.byref(batch.c), width, groups, float(eps), _p(h), _p(hs), _stream()),
            "group_norm_shift")
    return h, hs


def retention(qkvg, batch: RaggedBatch, heads, dim, vdim, rot_dims, inv_freq, decay, eps, state, dtype=torch.float32,
              segments: bool = True):
    """``segments``: give the kernel room to cut few long sequences into segments that run side by side."""
    T = qkvg.shape[0]
    seg = torch.empty(32 * heads * dim * vdim, dtype=torch.float32, device=qkvg.device) if segments and T >= 128 else None
    o32 = torch.empty((T, heads * vdim), dtype=torch.float32, device=qkvg.device)
    out = torch.empty((T, heads * vdim), dtype=dtype, device=qkvg.device)
    rot = torch.empty((T, max(rot_dims, 1)), dtype=torch.float32, device=qkvg.device)
    S.check(S.load().umbs_retention(_mode(out), _p(qkvg), qkvg.stride(0), C.byref(batch.c), heads, dim, vdim, rot_dims,
                                    _p(inv_freq), _p(decay), float(eps), _p(state), _p(o32), _p(rot), _p(seg),
                                    seg.numel() * 4 if seg is not None else 0, _p(out), _stream()),
            "retention")
    return out


def latent_attention(q_abs, c, ring, batch: RaggedBatch, heads, window, scale, append: bool = True):
    T, R = c.shape
    out = torch.empty((T, heads * R), dtype=c.dtype, device=c.device)
    lib = S.load()
    part = torch.empty(512 * heads * (R + 2), dtype=torch.float32, device=c.device) if T <= 64 else None
    S.check(lib.umbs_latent_attention(_mode(c), _p(q_abs), _p(c), _p(ring), ring.shape[1], C.byref(batch.c), heads, R, window,
                                      float(scale), _p(part), part.numel() * 4 if part is not None else 0, _p(out), _stream()),
            "latent_attention")
    if append:
        S.check(lib.umbs_ring_append(_mode(c), _p(c), _p(ring), ring.shape[1], C.byref(batch.c), R, _stream()), "ring_append")
    return out


def latent_norm(x, q_rank, kv_rank, q_norm, kv_norm, eps, dtype=torch.float32):
    n = x.shape[0]
    cq = torch.empty((n, q_rank), dtype=dtype, device=x.device)
    c = torch.empty((n, kv_rank), dtype=dtype, device=x.device)
    S.check(S.load().umbs_latent_norm(_mode(c), _p(x), n, q_rank, kv_rank, _p(q_norm), _p(kv_norm), float(eps), _p(cq), _p(c),
                                      _stream()), "latent_norm")
    return cq, c


def window_attention(q, k, v, batch: RaggedBatch, heads: int, window: int, scale: float):
    """q, k [T, heads dim], v [T, heads vdim] (views with a row stride are fine) -> [T, heads vdim]: sliding-window
    softmax attention among the step's own tokens (fresh sequences)."""
    T = q.shape[0]
    dim, vdim = q.shape[1] // heads, v.shape[1] // heads
    assert q.stride(1) == k.stride(1) == v.stride(1) == 1
    out = torch.empty((T, heads * vdim), dtype=q.dtype, device=q.device)
    S.check(S.load().umbs_window_attention(_mode(q), _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0),
                                           C.byref(batch.c), heads, dim, vdim, window, float(scale), _p(out), heads * vdim,
                                           _stream()), "window_attention")
    return out


def moe_route(h, w_router, top: int):
    """-> (sel_w [n, top] fp32, grp_off [E + 1], pair_tok [n top], pair_pos [n top], sel_e [n top])."""
    n, width = h.shape
    E = w_router.shape[0]
    dev = h.device
    sel_w = torch.empty((n, top), dtype=torch.float32, device=dev)
    grp_off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    pair_tok = torch.empty(n * top, dtype=torch.int32, device=dev)
    pair_pos = torch.empty(n * top, dtype=torch.int32, device=dev)
    scratch = torch.empty(2 * E + n * top, dtype=torch.int32, device=dev)
    S.check(S.load().umbs_moe_route(_mode(h), _p(h), n, width, _p(w_router), E, top, _p(sel_w), _p(grp_off), _p(pair_tok),
                                    _p(pair_pos), _p(scratch), _stream()), "moe_route")
    return sel_w, grp_off, pair_tok, pair_pos, scratch[2 * E:].view(n, top)


def depth_mix(x, mix, stack, layer: int, depth_w, pair_out=None, sel_w=None, pair_pos=None, shared=None):
    n, width = x.shape
    out = torch.empty_like(x)
    top = sel_w.shape[1] if sel_w is not None else 0
    S.check(S.load().umbs_depth_mix(_p(x), _p(mix), _p(pair_out), _p(sel_w), _p(pair_pos), top, _p(shared), _p(stack), layer,
                                    _p(depth_w), _p(out), None, n, width, _stream()), "depth_mix")
    return out


# ---------------------------------------------------------------------------------------------- pre-norm layers
def add_rms_norm(x, delta, w, w_offset: float, eps: float, dtype=torch.float32, rows=None, want_copy: bool = False):
    """x [n, width] fp32 (+= delta in place when ``rows`` is None) -> norm as ``dtype`` (and a copy of the sum)."""
    n = x.shape[0] if rows is None else rows.numel()
    y = torch.empty((n, x.shape[1]), dtype=dtype, device=x.device)
    copy = torch.empty((n, x.shape[1]), dtype=torch.float32, device=x.device) if want_copy else None
    S.check(S.load().umbs_add_rms_norm(_mode(y), _p(x), _p(delta), _p(rows), n, _p(w), float(w_offset), x.shape[1], float(eps),
                                       _p(y), _p(copy), _stream()), "add_rms_norm")
    return (y, copy) if want_copy else y


def softcap(z: torch.Tensor, cap: float) -> torch.Tensor:
    assert z.dtype == torch.float32 and z.is_contiguous()
    S.check(S.load().umbs_softcap(_p(z), z.numel(), float(cap), _stream()), "softcap")
    return z


def attention_prep(proj, bias, batch: RaggedBatch, heads, kv_heads, dim, vdim, rot_dims, inv_freq, rot_mag=1.0,
                   values_are_keys=False, taps=1, conv_w=None, conv_state=None, dtype=torch.float32):
    """proj fp32 [T, q | k | v | ...] -> (q [T, heads dim], kv [T, kv_heads (dim + vdim)]) as ``dtype``."""
    T = proj.shape[0]
    q = torch.empty((T, heads * dim), dtype=dtype, device=proj.device)
    kv = torch.empty((T, kv_heads * (dim + vdim)), dtype=dtype, device=proj.device)
    slots = conv_state.shape[1] if conv_state is not None else 0
    S.check(S.load().umbs_attention_prep(_mode(q), _p(proj), proj.stride(0), _p(bias), C.byref(batch.c), heads, kv_heads, dim,
                                         vdim, int(values_are_keys), taps, _p(conv_w), _p(conv_state), slots, rot_dims,
                                         _p(inv_freq), float(rot_mag), _p(q), _p(kv), _stream()), "attention_prep")
    return q, kv


def cached_attention(q, kv, kv_cache, batch: RaggedBatch, heads, kv_heads, dim, vdim, scale, mode=S.UMBS_ATTN_SOFTMAX,
                     window=0, pool=0, pool_cache=None, head_bias=None, gate=None, gate_per_head=False, append=True,
                     split=True):
    """One attention step over the step's kv rows and the slots' caches (pooling the blocks the step completes first and
    appending the step's rows afterwards, as umbs_forward does)."""
    T = q.shape[0]
    lib, row = S.load(), kv_heads * (dim + vdim)
    out = torch.empty((T, heads * vdim), dtype=q.dtype, device=q.device)
    if pool > 0:
        S.check(lib.umbs_kv_pool(_mode(q), _p(kv), _p(kv_cache), kv_cache.shape[1], _p(pool_cache), pool_cache.shape[1],
                                 C.byref(batch.c), row, pool, _stream()), "kv_pool")
    part = torch.empty(2048 * (vdim + 2), dtype=torch.float32, device=q.device) if split else None
    S.check(lib.umbs_cached_attention(_mode(q), mode, _p(q), _p(kv), _p(kv_cache), kv_cache.shape[1], _p(pool_cache),
                                      pool_cache.shape[1] if pool_cache is not None else 0, C.byref(batch.c), heads, kv_heads,
                                      dim, vdim, window, pool, float(scale), _p(head_bias), _p(gate),
                                      gate.stride(0) if gate is not None else 0, int(gate_per_head), _p(part),
                                      part.numel() * 4 if part is not None else 0, _p(out), _stream()), "cached_attention")
    if append:
        S.check(lib.umbs_ring_append(_mode(q), _p(kv), _p(kv_cache), kv_cache.shape[1], C.byref(batch.c), row, _stream()),
                "ring_append")
    return out


def mlstm(proj, gate_bias, batch: RaggedBatch, heads, dim, vdim, gate_cap, eps, out_norm_w, state, dtype=torch.float32,
          segments: bool = True):
    """proj fp32 [T, q | k | v | gate | i | f] -> [T, heads vdim] as ``dtype``; state fp32 [slots, heads, dim (vdim + 1) + 1].
    ``segments``: give the kernel room to cut few long sequences into segments that run side by side."""
    T = proj.shape[0]
    seg = torch.empty(32 * heads * (dim * (vdim + 1) + 1), dtype=torch.float32, device=proj.device) if segments and T >= 128 else None
    gates = torch.empty((T, heads, 3), dtype=torch.float32, device=proj.device)
    o32 = torch.empty((T, heads, vdim + 1), dtype=torch.float32, device=proj.device)
    out = torch.empty((T, heads * vdim), dtype=dtype, device=proj.device)
    S.check(S.load().umbs_mlstm(_mode(out), _p(proj), proj.stride(0), _p(gate_bias), C.byref(batch.c), heads, dim, vdim,
                                float(gate_cap), float(eps), _p(out_norm_w), _p(state), _p(gates), _p(o32), _p(seg),
                                seg.numel() * 4 if seg is not None else 0, _p(out), _stream()), "mlstm")
    return out


# ---------------------------------------------------------------------------------------------- further options of the pre-norm form
def gemm_ex(a: torch.Tensor, w: torch.Tensor, *, out_f32: bool = False, groups: int = 1, a_goff: int = 0, c_goff: int = 0,
            n: int | None = None, k: int | None = None, act: int = 0, limit: float = 0.0, bias=None, out_gate=None,
            gate_goff: int = 0) -> torch.Tensor:
    """``gemm`` with the epilogue of umbs_gemm_ex: ``act`` = 0 (plain) or UMBS_ACT_* over gate|up rows, ``bias`` fp32 [N] or
    [2 N], ``out_gate`` fp32 [M, .] whose sigmoid multiplies the result (column g gate_goff + n for group g)."""
    mode = _mode(a)
    assert w.dtype == a.dtype and a.stride(-1) == 1 and w.is_contiguous()
    w3 = w if w.dim() == 3 else w.unsqueeze(0)
    K = w3.shape[2] if k is None else k
    N = (w3.shape[1] // (2 if act else 1)) if n is None else n
    M = a.shape[0]
    out = torch.zeros((M, N if groups == 1 else groups * c_goff), dtype=torch.float32 if out_f32 else a.dtype, device=a.device)
    S.check(S.load().umbs_gemm_ex(mode, _p(a), a.stride(0), a_goff, _p(w3), w3.stride(1), w3.stride(0), _p(out), out.stride(0),
                                  c_goff, int(out_f32), M, N, K, groups, None, None, int(act), float(limit), _p(bias),
                                  _p(out_gate), out_gate.stride(0) if out_gate is not None else 0, gate_goff, _stream()),
            "gemm_ex")
    return out


def add_norm(x, w, b, eps: float, kind: int = S.UMBS_NORM_LAYER, w_offset: float = 0.0, dtype=torch.float32, rows=None,
             delta=None, pair_out=None, sel_w=None, pair_pos=None, shared=None, shared_gate=None, scale=None, mult: float = 1.0,
             want_copy: bool = False):
    """x [n, width] fp32 += (delta + routed pairs + gated shared) * scale * mult (in place when ``rows`` is None), then the
    norm of the sum as ``dtype`` (and a copy of the sum)."""
    n = x.shape[0] if rows is None else rows.numel()
    y = torch.empty((n, x.shape[1]), dtype=dtype, device=x.device)
    copy = torch.empty((n, x.shape[1]), dtype=torch.float32, device=x.device) if want_copy else None
    d = None
    if any(t is not None for t in (delta, pair_out, shared)):
        d = S.Delta()
        d.delta, d.pair_out, d.sel_w, d.pair_pos = (t.data_ptr() if t is not None else None for t in (delta, pair_out, sel_w, pair_pos))
        d.top = sel_w.shape[1] if sel_w is not None else 0
        d.shared, d.shared_gate, d.scale = (t.data_ptr() if t is not None else None for t in (shared, shared_gate, scale))
        d.mult = float(mult)
    S.check(S.load().umbs_add_norm(_mode(y), _p(x), C.byref(d) if d is not None else None, _p(rows), n, kind, _p(w), _p(b),
                                   float(w_offset), x.shape[1], float(eps), _p(y), _p(copy), _stream()), "add_norm")
    return (y, copy) if want_copy else y


def latent_prep(proj, batch: RaggedBatch, heads, dim, rope_dim, kv_rank, kv_norm, eps, rot_dims, inv_freq, rot_mag=1.0,
                dtype=torch.float32):
    """proj fp32 [T, q | latent | shared key part | ...] -> (q [T, heads (dim + rope_dim)], c [T, kv_rank + rope_dim]) as
    ``dtype`` and q_abs fp32 [T, heads, kv_rank + rope_dim] whose last rope_dim columns hold every head's turned part (the
    first kv_rank are left for the product with the key up-projection)."""
    T = proj.shape[0]
    KD = kv_rank + rope_dim
    q = torch.empty((T, heads * (dim + rope_dim)), dtype=dtype, device=proj.device)
    c = torch.empty((T, KD), dtype=dtype, device=proj.device)
    q_abs = torch.zeros((T, heads, KD), dtype=torch.float32, device=proj.device)
    S.check(S.load().umbs_latent_prep(_mode(q), _p(proj), proj.stride(0), C.byref(batch.c), heads, dim, rope_dim, kv_rank,
                                      _p(kv_norm), float(eps), rot_dims, _p(inv_freq), float(rot_mag), _p(q), _p(c),
                                      C.c_void_p(q_abs.data_ptr() + 4 * kv_rank), KD, _stream()), "latent_prep")
    return q, c, q_abs


def latent_attention_shared(q_abs, c, ring, batch: RaggedBatch, heads, kv_rank, rope_dim, scale, window: int = 0,
                            sink=None, use_sink: bool = True, append: bool = True, split: bool = True):
    """Attention over [latent | shared part] keys (umbs_latent_attention_ex) -> [T, heads kv_rank]; appends the step's rows."""
    T = c.shape[0]
    out = torch.empty((T, heads * kv_rank), dtype=c.dtype, device=c.device)
    lib = S.load()
    part = torch.empty(512 * heads * (kv_rank + 2), dtype=torch.float32, device=c.device) if split and T <= 64 else None
    S.check(lib.umbs_latent_attention_ex(_mode(c), _p(q_abs), _p(c), _p(ring), ring.shape[1], C.byref(batch.c), heads, kv_rank,
                                         rope_dim, window, float(scale),
                                         S.UMBS_ATTN_SOFTMAX_SINK if use_sink else S.UMBS_ATTN_SOFTMAX, _p(sink), _p(part),
                                         part.numel() * 4 if part is not None else 0, _p(out), _stream()), "latent_attention_ex")
    if append:
        S.check(lib.umbs_ring_append(_mode(c), _p(c), _p(ring), ring.shape[1], C.byref(batch.c), kv_rank + rope_dim, _stream()),
                "ring_append")
    return out


def window_attention_shared(q, k, k_shared, v, batch: RaggedBatch, heads: int, scale: float, window: int = 0, sink=None,
                            use_sink: bool = True, gate=None):
    """q [T, heads (dim + shared)], k [T, heads dim], k_shared [T, shared], v [T, heads vdim] (row-strided views are fine)
    -> [T, heads vdim]: attention among the step's own tokens with a key part all heads share, a sink and an output gate."""
    T = q.shape[0]
    sd = k_shared.shape[1] if k_shared is not None else 0
    dim, vdim = k.shape[1] // heads, v.shape[1] // heads
    assert q.shape[1] == heads * (dim + sd)
    out = torch.empty((T, heads * vdim), dtype=q.dtype, device=q.device)
    S.check(S.load().umbs_window_attention_ex(_mode(q), _p(q), q.stride(0), _p(k), k.stride(0), _p(k_shared),
                                              k_shared.stride(0) if k_shared is not None else 0, sd, _p(v), v.stride(0),
                                              C.byref(batch.c), heads, dim, vdim, window, float(scale),
                                              S.UMBS_ATTN_SOFTMAX_SINK if use_sink else S.UMBS_ATTN_SOFTMAX, _p(sink), _p(gate),
                                              gate.stride(0) if gate is not None else 0, _p(out), heads * vdim, _stream()),
            "window_attention_ex")
    return out


def moe_route_ex(h, w_router, top: int, mode: int, groups: int = 1, keep: int = 1, gate_w=None):
    """``moe_route`` with the rule as an argument (UMBS_ROUTE_*).  With ``gate_w`` the per-token gate sigmoid(gate_w . h) is
    worked out in the same pass and returned as a sixth value."""
    n, width = h.shape
    E = w_router.shape[0]
    dev = h.device
    sel_w = torch.empty((n, top), dtype=torch.float32, device=dev)
    grp_off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    pair_tok = torch.empty(n * top, dtype=torch.int32, device=dev)
    pair_pos = torch.empty(n * top, dtype=torch.int32, device=dev)
    scratch = torch.empty(2 * E + n * top, dtype=torch.int32, device=dev)
    gate = torch.empty(n, dtype=torch.float32, device=dev) if gate_w is not None else None
    S.check(S.load().umbs_moe_route_ex(_mode(h), _p(h), n, width, _p(w_router), E, top, mode, groups, keep, _p(sel_w),
                                       _p(grp_off), _p(pair_tok), _p(pair_pos), _p(scratch), _p(gate_w), _p(gate), _stream()),
            "moe_route_ex")
    out = (sel_w, grp_off, pair_tok, pair_pos, scratch[2 * E:].view(n, top))
    return out + (gate,) if gate_w is not None else out


def token_gate(h, w):
    g = torch.empty(h.shape[0], dtype=torch.float32, device=h.device)
    S.check(S.load().umbs_token_gate(_mode(h), _p(h), h.shape[0], h.shape[1], _p(w), _p(g), _stream()), "token_gate")
    return g


def embedding_scaled(ids, table, scale: float):
    y = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    S.check(S.load().umbs_embedding_scaled(_mode(table), _p(ids), _p(table), float(scale), _p(y), ids.numel(), table.shape[1],
                                           _stream()), "embedding_scaled")
    return y


# ---------------------------------------------------------------------------------------------- score options, time mix
def embedding_pos(ids, tok_pos, table, pos_freq, scale: float = 1.0):
    """table[ids] * scale + sinusoidal positions (entry 2i: sin(p f_i), entry 2i + 1: cos(p f_i)); fp32 [n, width]."""
    y = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    S.check(S.load().umbs_embedding_pos(_mode(table), _p(ids), _p(tok_pos), _p(table), float(scale), _p(pos_freq), _p(y),
                                        ids.numel(), table.shape[1], _stream()), "embedding_pos")
    return y


def add_norm_dyt(x, w, b, alpha: float, dtype=torch.float32, rows=None, delta=None, delta_mult: float = 1.0, delta2=None,
                 delta2_mult: float = 1.0):
    """x [n, width] fp32 += delta_mult delta + delta2_mult delta2 (in place when ``rows`` is None), then
    tanh(alpha x) w + b as ``dtype``."""
    n = x.shape[0] if rows is None else rows.numel()
    y = torch.empty((n, x.shape[1]), dtype=dtype, device=x.device)
    d = None
    if delta is not None or delta2 is not None:
        d = S.Delta()
        d.delta, d.delta2 = (t.data_ptr() if t is not None else None for t in (delta, delta2))
        d.mult, d.delta_mult, d.delta2_mult = 1.0, float(delta_mult), float(delta2_mult)
    S.check(S.load().umbs_add_norm_ex(_mode(y), _p(x), C.byref(d) if d is not None else None, _p(rows), n, S.UMBS_NORM_DYT,
                                      _p(w), _p(b), 0.0, float(alpha), x.shape[1], 0.0, _p(y), None, _stream()), "add_norm_ex")
    return y


def attention_prep_maps(proj, batch: RaggedBatch, heads, kv_heads, dim, vdim, maps=1, q_norm=None, k_norm=None, eps=1e-6,
                        dtype=torch.float32):
    """proj fp32 [T, q (heads maps dim) | k (kv_heads maps dim) | v (kv_heads vdim) | ...] -> (q, kv) as ``dtype``, every
    (head, map) of q and k RMS-normed with the weights given.  kv_heads 0: queries only (kv is None)."""
    T = proj.shape[0]
    q = torch.empty((T, heads * maps * dim), dtype=dtype, device=proj.device)
    kv = torch.empty((T, kv_heads * (maps * dim + vdim)), dtype=dtype, device=proj.device) if kv_heads else None
    S.check(S.load().umbs_attention_prep_ex(_mode(q), _p(proj), proj.stride(0), None, C.byref(batch.c), heads, kv_heads, dim, vdim,
                                            0, 1, None, None, 0, 0, None, 1.0, maps, _p(q_norm), _p(k_norm), float(eps), _p(q),
                                            _p(kv), _stream()), "attention_prep_ex")
    return q, kv


def scored_attention(q, kv, kv_cache, batch: RaggedBatch, heads, kv_heads, dim, vdim, scale, window=0, softcap=0.0, r1=None,
                     r2=None, chunk=0, maps=1, talk=None, diff_lambda=0.0, unit_norm=False, eps=1e-6, out_mult=1.0, gate=None,
                     append=True, split=True):
    """Cached attention with score options, then umbs_attention_finish: a tanh cap, a distance penalty, a chunked mask,
    two maps per head (a1 - diff_lambda a2) or softmax weights mixed across heads by ``talk``; unit RMS per head, a factor,
    an element-wise sigmoid gate.  -> [T, heads vdim] as q's dtype."""
    T = q.shape[0]
    lib, row = S.load(), kv_heads * (maps * dim + vdim)
    vheads = kv_heads if talk is not None else 1
    raw = torch.empty((T, heads * maps * vheads, vdim), dtype=torch.float32, device=q.device)
    out = torch.empty((T, heads * vdim), dtype=q.dtype, device=q.device)
    o = S.AttnOpts()
    o.softcap, o.dist_r1, o.dist_r2, o.chunk, o.maps, o.value_heads = float(softcap), r1.data_ptr() if r1 is not None else None, \
        r2.data_ptr() if r2 is not None else None, chunk, maps, vheads
    o.raw_out = raw.data_ptr()
    part = torch.empty(2048 * (vdim + 2), dtype=torch.float32, device=q.device) if split else None
    S.check(lib.umbs_cached_attention_ex(_mode(q), S.UMBS_ATTN_SOFTMAX, _p(q), _p(kv), _p(kv_cache), kv_cache.shape[1], None, 0,
                                         C.byref(batch.c), heads, kv_heads, dim, vdim, window, 0, float(scale), None, None, 0, 0,
                                         C.byref(o), _p(part), part.numel() * 4 if part is not None else 0, None, _stream()),
            "cached_attention_ex")
    S.check(lib.umbs_attention_finish(_mode(q), _p(raw), T, heads, kv_heads, vdim, maps, vheads, _p(talk), float(diff_lambda),
                                      int(unit_norm), float(eps), float(out_mult), _p(gate), gate.stride(0) if gate is not None else 0,
                                      _p(out), _stream()), "attention_finish")
    if append:
        S.check(lib.umbs_ring_append(_mode(q), _p(kv), _p(kv_cache), kv_cache.shape[1], C.byref(batch.c), row, _stream()),
                "ring_append")
    return out


def shift_mix(h, mu, shift_state, batch: RaggedBatch):
    """h [T, width] -> [T, n_mix, width]: h + (previous row - h) mu[s]; shift_state fp32 [2, slots, width]."""
    out = torch.empty((h.shape[0], mu.shape[0], h.shape[1]), dtype=h.dtype, device=h.device)
    S.check(S.load().umbs_shift_mix(_mode(h), _p(h), _p(mu), mu.shape[0], _p(shift_state), shift_state.shape[1], C.byref(batch.c),
                                    h.shape[1], _p(out), _stream()), "shift_mix")
    return out


def time_mix(proj, decay_raw, decay_bias, bonus, batch: RaggedBatch, heads, dim, eps, out_norm_w, state, dtype=torch.float32):
    """proj fp32 [T, r | k | v | g] and decay_raw fp32 [T, heads dim] -> [T, heads dim] as ``dtype``; state fp32
    [slots, heads, dim, dim]."""
    T = proj.shape[0]
    o32 = torch.empty((T, heads * dim), dtype=torch.float32, device=proj.device)
    out = torch.empty((T, heads * dim), dtype=dtype, device=proj.device)
    S.check(S.load().umbs_time_mix(_mode(out), _p(proj), proj.stride(0), _p(decay_raw), _p(decay_bias), _p(bonus), C.byref(batch.c),
                                   heads, dim, float(eps), _p(out_norm_w), _p(state), _p(o32), _p(out), _stream()), "time_mix")
    return out


def gemm_unary(a: torch.Tensor, w: torch.Tensor, unary: int, p0: float = 0.0, p1: float = 0.0, out_f32: bool = False):
    """unary(a [M, K] x w [N, K]^T): UMBS_UNARY_TANH or UMBS_UNARY_XIELU with its two coefficients."""
    assert w.dtype == a.dtype and a.stride(-1) == 1 and w.is_contiguous()
    out = torch.empty((a.shape[0], w.shape[0]), dtype=torch.float32 if out_f32 else a.dtype, device=a.device)
    S.check(S.load().umbs_gemm_unary(_mode(a), _p(a), a.stride(0), 0, _p(w), w.stride(0), 0, _p(out), out.stride(0), 0,
                                     int(out_f32), a.shape[0], w.shape[0], w.shape[1], 1, None, unary, float(p0), float(p1),
                                     _stream()), "gemm_unary")
    return out


def moe_route_scaled(h, w_router, top: int, mode: int, weight_scale: float = 1.0):
    """``moe_route_ex`` with a factor on the chosen weights (UMBS_ROUTE_SOFTMAX_ALL: softmax over every expert)."""
    n, width = h.shape
    E = w_router.shape[0]
    dev = h.device
    sel_w = torch.empty((n, top), dtype=torch.float32, device=dev)
    grp_off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    pair_tok = torch.empty(n * top, dtype=torch.int32, device=dev)
    pair_pos = torch.empty(n * top, dtype=torch.int32, device=dev)
    scratch = torch.empty(2 * E + n * top, dtype=torch.int32, device=dev)
    S.check(S.load().umbs_moe_route_scaled(_mode(h), _p(h), n, width, _p(w_router), E, top, mode, 1, 1, float(weight_scale),
                                           _p(sel_w), _p(grp_off), _p(pair_tok), _p(pair_pos), _p(scratch), None, None,
                                           _stream()), "moe_route_scaled")
    return sel_w, grp_off, pair_tok, pair_pos, scratch[2 * E:].view(n, top)
