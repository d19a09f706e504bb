"""Sequence-state decoders on the native batched step (umbs_forward of libumbrella_b200_seq.so).

A model is a ``SeqModelSpec``: width, vocabulary, the norm's constants and a list of ``SeqLayerSpec``s, each naming
its form (``"parallel"``: one grouped norm feeds mixer and feed-forward side by side, with token shift and a depth
average as options; ``"prenorm"``: x += mixer(norm1(x)), x += ff(norm2(x)), RMS or layer norms, optionally with a learned
scale vector and a multiplier on every block's output), its mixer (``"retention"``, ``"latent_attention"``,
``"cached_attention"``, ``"mlstm"`` or ``"time_mix"``) with that mixer's sizes and constants -- a pre-norm layer may run a
second mixer beside the first (``second``), both reading the same normed rows --, and its feed-forward (routed experts and /
or a shared expert -- a dense feed-forward is a shared expert alone -- or none).  Model families (models/radanex.py,
models/zedotar.py, models/kulisun.py) translate their config.json into a spec and their tensors into the per-layer
weight dicts ``load_layer`` takes; nothing below knows a family's names.

One ``forward`` call runs a ragged batch: for every sequence its slot of the ``SequenceStateCache`` and its next
tokens (any number: a whole prompt, a portion of one, one decoded token), and the places whose logits are wanted.
The batch description goes host -> device in one pinned copy; one C call enqueues every launch of the step.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import torch

from .. import _lib_seq as S
from ..attn.state_cache import SequenceStateCache


@dataclass
class SeqMlpSpec:
    experts: int = 0
    top: int = 0
    ff: int = 0
    limit: float = 0.0
    shared_ff: int = 0
    shared_limit: float = 0.0
    act: str = "clamped_glu"          # or "gelu_tanh", "silu"
    route: str = "softmax_top"        # "softmax_top": the top logits, softmax over them | "sigmoid_groups": sigmoid
                                      # scores, group-limited choice, chosen scores divided by their sum
    groups: int = 1                   # sigmoid_groups: equal groups of neighbouring experts ...
    keep: int = 1                     # ... of which the best `keep` (by the sum of their two largest scores) stay eligible
    bias: bool = False                # the shared (dense) projections carry biases
    shared_gate: bool = False         # the shared expert's output is multiplied by sigmoid(w . h), a number per token
    route_scale: float = 1.0          # factor on the chosen experts' weights ("softmax_all": softmax over every expert, the
                                      # chosen scores as they are)
    plain: str = ""                   # the dense part has no gate: W_down act(W_up h), act = "xielu" (two learned numbers)


@dataclass
class SeqLayerSpec:
    mixer: str = "retention"
    heads: int = 1
    dim: int = 32
    vdim: int = 32
    # retention
    rot_dims: int = 0
    rot_base: float = 10000.0
    decay: list = field(default_factory=list)
    # latent attention (pre-norm form: q_rank 0 = queries straight from the layer input; also attn_mode, gate_kind 0 / 2,
    # rot_dims <= rope_dim, inv_freq, rot_mag from below; window 0 = every earlier token)
    q_rank: int = 0
    kv_rank: int = 0
    window: int = 0
    scale: float = 1.0
    rope_dim: int = 0                 # rotated query/key dimensions per head beside `dim`; the key's are shared by all heads
    learned_sink: bool = False        # softmax_sink: the sink's score is a learned number per head instead of 0
    # cached attention (also: rot_dims, window (0 = every earlier token), scale)
    kv_heads: int = 0
    attn_mode: str = "softmax"        # "softmax" | "softmax_sink" | "sigmoid"
    gate_kind: int = 0                # 0 none, 1 one sigmoid gate per head, 2 one per output element
    values_are_keys: bool = False     # values = keys before the rotation (no value projection)
    pool: int = 0                     # tokens per pooled block of keys that have left the window
    taps: int = 1                     # short causal convolution on q and k
    bias: bool = False                # q, k, v projections carry biases
    head_bias: bool = False           # a number per head added to the scores
    inv_freq: list | None = None      # rotary frequencies when they are not base^(-2i/rot_dims) (scaled forms)
    rot_mag: float = 1.0              # factor on cos and sin
    # cached attention, score options
    softcap: float = 0.0              # > 0: score <- cap tanh(score / cap)
    dist_bias: bool = False           # score -= r1[h] ln(1 + r2[h] (i - j)), two learned numbers per head
    talk: bool = False                # after the softmax, head h's weights become a learned mix of all heads' weights
    chunk: int = 0                    # > 0: a row sees only keys of its own chunk of this many positions
    maps: int = 1                     # 2: differential attention, a1 - lambda a2 over the same values
    diff: float = 0.0                 # lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff; the output is scaled by 1 - diff
    head_unit_norm: bool = False      # every head's output is divided by its root mean square
    qk_norm: bool = False             # RMS norm (weight [dim]) of every query and key head (and map)
    kv_from: int | None = None        # the layer has no key / value projections and reads that layer's keys and values
    # time mix (dim = vdim)
    decay_rank: int = 0
    # a second mixer beside this one (pre-norm form): x += mix_scale * mixer + second_scale * second
    second: "SeqLayerSpec | None" = None
    mix_scale: float = 1.0
    second_scale: float = 1.0
    # mlstm
    gate_cap: float = 0.0
    # layer
    form: str = "parallel"
    norm_offset: float = 0.0          # added to the layer's norm weights (1: weights stored around zero)
    norm_kind: str = "rms"            # pre-norm form: "rms" | "layer" (mean removed, weight and bias) | "dyt" (tanh(alpha x) w + b)
    layer_scale: bool = False         # pre-norm form: every block's output is multiplied by a learned vector
    residual_mult: float = 1.0        # pre-norm form: x += residual_mult * block output
    shift: bool = True
    depth_average: bool = True
    mlp: SeqMlpSpec | None = None
    state_index: int = -1             # where the state cache keeps this mixer's state (set by the cache)


@dataclass
class SeqModelSpec:
    width: int
    vocab: int
    layers: list
    norm_groups: int = 1
    norm_eps: float = 1e-6
    norm_offset: float = 0.0          # added to the final norm's weight
    logit_softcap: float = 0.0        # > 0: logits <- cap tanh(logits / cap)
    embed_scale: float = 1.0          # factor on the embedding rows
    norm_kind: str = "rms"            # kind of the final norm (pre-norm form)
    pos_embed: str = ""               # "sinusoid": entry 2i of the embedding gets sin(p f_i), entry 2i + 1 cos(p f_i), ...
    pos_base: float = 10000.0         # ... f_i = pos_base^(-2i / width)
    eos_token_id: list = field(default_factory=list)

    # compatibility with the engines' view of a config
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)


def rotary_inv_freq(rot_dims: int, base: float) -> torch.Tensor:
    """f_i = base^(-2 i / rot_dims), i < rot_dims / 2: evaluated in double, rounded once to fp32."""
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / rot_dims).to(torch.float32)


def scale_freq_by_wavelength(f: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Frequency scaling by wavelength l = 2 pi / f against an original context length: kept where l < original / high,
    divided by ``factor`` where l > original / low, blended in between with s = (original / l - low) / (high - low).
    float64 in, float64 out."""
    wave = 2.0 * math.pi / f
    s = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
    mid = (1.0 - s) * f / factor + s * f
    return torch.where(wave < original / high, f, torch.where(wave > original / low, f / factor, mid))


def scale_freq_yarn(f: torch.Tensor, rot_dims: int, base: float, factor: float, original: float, fast: float,
                    slow: float) -> tuple[torch.Tensor, float]:
    """YaRN: frequencies that turn more than ``fast`` times over the original context are kept, those that turn less
    than ``slow`` times are divided by ``factor``, a linear ramp over the dimension index in between; cos and sin are
    scaled by 0.1 ln(factor) + 1.  -> (frequencies, that factor)."""
    turn = lambda t: rot_dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(turn(fast)), 0), min(math.ceil(turn(slow)), rot_dims - 1)
    i = torch.arange(f.numel(), dtype=torch.float64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotary_inv_freq64(rot_dims: int, base: float) -> torch.Tensor:
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / rot_dims)


_MIXERS = {"retention": S.UMBS_MIX_RETENTION, "latent_attention": S.UMBS_MIX_LATENT_ATTENTION,
           "cached_attention": S.UMBS_MIX_CACHED_ATTENTION, "mlstm": S.UMBS_MIX_MLSTM, "time_mix": S.UMBS_MIX_TIME_MIX}
_ATTN_MODES = {"softmax": S.UMBS_ATTN_SOFTMAX, "softmax_sink": S.UMBS_ATTN_SOFTMAX_SINK, "sigmoid": S.UMBS_ATTN_SIGMOID}
_ACTS = {"clamped_glu": S.UMBS_ACT_CLAMPED_GLU, "gelu_tanh": S.UMBS_ACT_GELU_TANH, "silu": S.UMBS_ACT_SILU}
_NORMS = {"rms": S.UMBS_NORM_RMS, "layer": S.UMBS_NORM_LAYER, "dyt": S.UMBS_NORM_DYT}
_ROUTES = {"softmax_top": S.UMBS_ROUTE_SOFTMAX_TOP, "sigmoid_groups": S.UMBS_ROUTE_SIGMOID_GROUPS,
           "softmax_all": S.UMBS_ROUTE_SOFTMAX_ALL}


def _softplus(z: float) -> float:
    return math.log1p(math.exp(-abs(z))) + max(z, 0.0)


class SeqStateModel:
    """Weights + state cache + workspace of one sequence-state decoder on one GPU."""

    def __init__(self, spec: SeqModelSpec, device="cuda:0", dtype=torch.bfloat16, slots: int = 8,
                 max_length: int | None = None, max_tokens: int = 0, model_name: str | None = None,
                 graph_decode: bool = True, fresh_attention: bool = True):
        if dtype not in (torch.bfloat16, torch.float32):
            raise TypeError("sequence-state decoders run in bfloat16 or float32")
        self.spec = self.config = spec
        self.device, self.dtype = torch.device(device), dtype
        self.model_name = model_name
        self.max_length = max_length
        self.num_layers = len(spec.layers)
        self.eos_tokens = list(spec.eos_token_id)
        self._slots0, self._max_tokens0 = slots, max_tokens
        self.weights: list[dict | None] = [None] * self.num_layers
        self.head_weights: dict | None = None
        self.cache: SequenceStateCache | None = None
        self._c_model = None
        self._c_version = -1
        self._ws = None
        self._ws_tokens = self._ws_want = 0
        # decode steps (one token per sequence) replay a CUDA graph of the whole step, captured per batch size once that
        # size has run eagerly twice: slots, positions and parities live in the device-side batch description, so the
        # same graph serves every later step of that size
        self.graph_decode = graph_decode
        # latent attention of a step whose sequences all start at position 0 runs over per-head keys and values
        # up-projected once per token (False: always over the latents, as decode steps and later portions do)
        self.fresh_attention = fresh_attention
        self._graphs: dict = {}
        self._graph_seen: dict = {}

    # ------------------------------------------------------------------ allocation
    def alloc(self, **kwargs):
        S.load()
        if self.device.type != "cuda":
            raise RuntimeError("sequence-state decoders need a CUDA device (there is no CPU path)")
        self.cache = SequenceStateCache(self.spec, slots=kwargs.get("slots", self._slots0), device=self.device,
                                        dtype=self.dtype, max_length=self.max_length, capacity=self._max_tokens0)
        return self

    def _reserve(self, tokens: int, want: int):
        if self._ws is not None and tokens <= self._ws_tokens and want <= self._ws_want:
            return
        tokens, want = max(tokens, self._ws_tokens), max(want, self._ws_want)
        n = S.load().umbs_workspace_bytes(C.byref(self._model_struct()), tokens, want)
        self._ws = None
        self._ws = torch.empty(n, dtype=torch.uint8, device=self.device)
        self._ws_tokens, self._ws_want = tokens, want

    # ------------------------------------------------------------------ weights
    def _act(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.device, self.dtype).contiguous()

    def _f32(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(self.device, torch.float32).contiguous()

    def load_head(self, embed: torch.Tensor, head: torch.Tensor | None, final_norm: torch.Tensor,
                  final_norm_b: torch.Tensor | None = None, final_norm_alpha: float = 1.0):
        """``head`` None: the logits come from the embedding table itself (tied)."""
        e = self._act(embed)
        self.head_weights = dict(embed=e, head=e if head is None else self._act(head), final_norm=self._f32(final_norm))
        if self.spec.norm_kind in ("layer", "dyt"):
            self.head_weights["final_norm_b"] = self._f32(final_norm_b)
        self.final_norm_alpha = float(final_norm_alpha)
        if self.spec.pos_embed == "sinusoid":
            self.head_weights["pos_freq"] = rotary_inv_freq(self.spec.width, self.spec.pos_base).to(self.device)
        elif self.spec.pos_embed:
            raise ValueError(f"unknown position embedding '{self.spec.pos_embed}'")
        self._c_model = None

    def load_layer(self, idx: int, w: dict):
        """``w``: tensors [out, in] as the checkpoint holds them.
        all layers: norm [width]; shift [width] (if the layer shifts); depth [idx + 2] (if it averages); o.
        retention: q, k [heads dim, width]; v, g [heads vdim, width].
        latent attention: dq [q_rank, width], dq_norm, uq [heads dim, q_rank], dkv [kv_rank, width], dkv_norm,
            uk [heads dim, kv_rank], uv [heads vdim, kv_rank].
        cached attention: q [heads dim, width], k [kv_heads dim, width], v [kv_heads vdim, width] (unless the values are
            the keys), g [heads or heads vdim, width] (by gate_kind); q_b, k_b, v_b (biases); q_conv, k_conv [channels, taps];
            pb [heads] (score bias).
        mlstm: q, k [heads dim, width]; v, g [heads vdim, width]; i, f [heads, width] with i_b, f_b [heads]; out_norm [heads vdim].
        latent attention with direct queries (q_rank 0): q [heads (dim + rope_dim), width], dkv [kv_rank + rope_dim, width],
            dkv_norm, uk, uv, g [heads vdim, width] (gate_kind 2), sink [heads] (learned_sink).
        pre-norm layers: norm2 [width] when they have a feed-forward; norm_b, norm2_b (layer norm); ls1, ls2 [width] (layer scale).
        feed-forward: router [experts, width]; experts: list of (gate, up, down); shared (or dense): (gate, up, down);
            dense_b: (gate_b, up_b, down_b) with ``bias``; shared_gate [1, width] or [width]."""
        l = self.spec.layers[idx]
        d = dict(norm=self._f32(w["norm"]))
        if l.form == "prenorm":
            l.shift = l.depth_average = False
            if l.mlp is not None:
                d["norm2"] = self._f32(w["norm2"])
            if l.norm_kind in ("layer", "dyt"):
                d["norm_b"] = self._f32(w["norm_b"])
                if l.mlp is not None:
                    d["norm2_b"] = self._f32(w["norm2_b"])
            if l.norm_kind == "dyt":           # the scalars inside the tanh
                d["norm_alpha"] = float(w["norm_alpha"])
                d["norm2_alpha"] = float(w["norm2_alpha"]) if l.mlp is not None else 1.0
            if l.layer_scale:
                d["ls1"] = self._f32(w["ls1"])
                if l.mlp is not None:
                    d["ls2"] = self._f32(w["ls2"])
        if l.shift:
            d["shift"] = self._f32(w["shift"])
        if l.depth_average:
            d["depth"] = self._f32(w["depth"])
            assert d["depth"].numel() == idx + 2
        self._load_mixer(l, w, d)
        if l.second is not None:
            if l.form != "prenorm" or l.mixer not in ("cached_attention", "time_mix") or \
                    l.second.mixer not in ("cached_attention", "time_mix"):
                raise ValueError("a second mixer goes with pre-norm layers of cached attention and time mix")
            d["second"] = {}
            self._load_mixer(l.second, w["second"], d["second"])
        self._load_mlp(l, w, d)
        self.weights[idx] = d
        self._c_model = None

    def _load_mixer(self, l, w: dict, d: dict):
        """The mixer's tensors of ``w`` (see load_layer) into ``d``, stacked as the kernels read them."""
        d["o"] = self._act(w["o"])
        if l.mixer == "retention":
            d["w_in"] = self._act(torch.cat([w["q"], w["k"], w["v"], w["g"]], dim=0))
            d["inv_freq"] = rotary_inv_freq(l.rot_dims, l.rot_base).to(self.device) if l.rot_dims else \
                torch.zeros(1, dtype=torch.float32, device=self.device)
            d["decay"] = torch.tensor([float(x) for x in l.decay], dtype=torch.float32, device=self.device)
            assert d["decay"].numel() == l.heads and d["w_in"].shape == (2 * l.heads * (l.dim + l.vdim), self.spec.width)
        elif l.mixer == "latent_attention" and l.q_rank == 0:
            if l.form != "prenorm":
                raise ValueError("latent attention with direct queries is a pre-norm mixer")
            hd1 = l.dim + l.rope_dim
            d["w_in"] = self._act(torch.cat([w["q"], w["dkv"]] + ([w["g"]] if l.gate_kind else []), dim=0))
            d["kv_norm"] = self._f32(w["dkv_norm"])
            d["ukT"] = self._act(w["uk"].reshape(l.heads, l.dim, l.kv_rank).transpose(1, 2))
            d["uv"] = self._act(w["uv"])
            # fresh sequences: every head's unrotated keys, then its values, from one product over the latents
            d["ukv"] = self._act(torch.cat([w["uk"], w["uv"]], dim=0))
            if l.learned_sink:
                d["sink"] = self._f32(w["sink"])
            f = torch.tensor(l.inv_freq, dtype=torch.float64) if l.inv_freq is not None else \
                rotary_inv_freq64(l.rot_dims, l.rot_base) if l.rot_dims else None
            d["inv_freq"] = f.to(torch.float32).to(self.device) if l.rot_dims else \
                torch.zeros(1, dtype=torch.float32, device=self.device)
            assert w["q"].shape == (l.heads * hd1, self.spec.width) and w["dkv"].shape == (l.kv_rank + l.rope_dim, self.spec.width)
            assert w["uk"].shape == (l.heads * l.dim, l.kv_rank) and d["uv"].shape == (l.heads * l.vdim, l.kv_rank)
            assert l.gate_kind in (0, 2) and (not l.gate_kind or w["g"].shape[0] == l.heads * l.vdim)
            assert l.rot_dims % 2 == 0 and l.rot_dims <= l.rope_dim and (not l.rot_dims or d["inv_freq"].numel() == l.rot_dims // 2)
        elif l.mixer == "latent_attention":
            d["w_in"] = self._act(torch.cat([w["dq"], w["dkv"]], dim=0))
            d["q_norm"], d["kv_norm"] = self._f32(w["dq_norm"]), self._f32(w["dkv_norm"])
            d["uq"] = self._act(w["uq"])
            # key up-projection transposed per head: [heads, dim, kv_rank] -> [heads, kv_rank, dim]
            d["ukT"] = self._act(w["uk"].reshape(l.heads, l.dim, l.kv_rank).transpose(1, 2))
            d["uv"] = self._act(w["uv"])
            # key rows then value rows in one matrix: a step of fresh sequences up-projects its latents with one product
            d["ukv"] = self._act(torch.cat([w["uk"], w["uv"]], dim=0))
            assert d["uq"].shape == (l.heads * l.dim, l.q_rank) and d["uv"].shape == (l.heads * l.vdim, l.kv_rank)
        elif l.mixer == "cached_attention":
            # in-projection rows: q | k | v (unless the values are the keys) | gate; biases for q | k | v in the same order;
            # with several maps a head's rows are [map 1 | map 2]; a layer that borrows keys and values has q | gate only
            cq, ck = l.heads * l.maps * l.dim, l.kv_heads * l.maps * l.dim
            own = l.kv_from is None
            parts = [w["q"]] + ([w["k"]] if own else []) + ([] if (l.values_are_keys or not own) else [w["v"]]) + \
                ([w["g"]] if l.gate_kind else [])
            d["w_in"] = self._act(torch.cat(parts, dim=0))
            assert w["q"].shape[0] == cq and (not own or w["k"].shape[0] == ck) and l.heads % l.kv_heads == 0
            assert l.maps in (1, 2) and not (l.talk and l.maps > 1)
            if l.dist_bias:
                d["r1"], d["r2"] = self._f32(w["r1"]), self._f32(w["r2"])
                assert d["r1"].numel() == l.heads and d["r2"].numel() == l.heads
            if l.talk:
                d["talk"] = self._f32(w["talk"])
                assert d["talk"].shape == (l.heads, l.heads)
            if l.qk_norm:
                d["q_norm"] = self._f32(w["q_norm"])
                if own:
                    d["k_norm"] = self._f32(w["k_norm"])
                assert d["q_norm"].numel() == l.dim
            if l.maps == 2:        # one number per layer, from four learned vectors: evaluated once, in double
                dot = lambda a, b: float((w[a].double() * w[b].double()).sum())
                d["diff_lambda"] = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + l.diff
            assert not l.gate_kind or w["g"].shape[0] == (l.heads if l.gate_kind == 1 else l.heads * l.vdim)
            assert not l.values_are_keys or l.vdim == l.dim
            if l.bias:
                d["bias_in"] = self._f32(torch.cat([w["q_b"], w["k_b"]] + ([] if l.values_are_keys else [w["v_b"]])))
            if l.taps > 1:
                d["conv_w"] = self._f32(torch.cat([w["q_conv"], w["k_conv"]], dim=0))
                assert d["conv_w"].shape == (cq + ck, l.taps)
            if l.head_bias:
                d["head_bias"] = self._f32(w["pb"])
            f = torch.tensor(l.inv_freq, dtype=torch.float64) if l.inv_freq is not None else \
                rotary_inv_freq64(l.rot_dims, l.rot_base)
            d["inv_freq"] = f.to(torch.float32).to(self.device) if l.rot_dims else \
                torch.zeros(1, dtype=torch.float32, device=self.device)
            assert l.rot_dims == 0 or d["inv_freq"].numel() == l.rot_dims // 2
        elif l.mixer == "time_mix":
            # the four projections that read their own token-shifted mix, stacked for one batched product
            hd = l.heads * l.dim
            d["w_in"] = self._act(torch.stack([w["r"], w["k"], w["v"], w["g"]]))
            d["mu"] = self._f32(torch.stack([w["mu_r"], w["mu_k"], w["mu_v"], w["mu_g"], w["mu_w"]]))
            d["w1"], d["w2"] = self._act(w["w1"]), self._act(w["w2"])
            d["w0"], d["u"], d["out_norm"] = self._f32(w["w0"]), self._f32(w["u"].reshape(-1)), self._f32(w["out_norm"])
            l.decay_rank = int(w["w1"].shape[0])
            assert l.vdim == l.dim and d["w_in"].shape == (4, hd, self.spec.width) and d["mu"].shape == (5, self.spec.width)
            assert d["w2"].shape == (hd, l.decay_rank) and d["w0"].numel() == hd and d["u"].numel() == hd and d["out_norm"].numel() == hd
        elif l.mixer == "mlstm":
            d["w_in"] = self._act(torch.cat([w["q"], w["k"], w["v"], w["g"], w["i"], w["f"]], dim=0))
            d["bias_in"] = self._f32(torch.cat([w["i_b"], w["f_b"]]))
            d["out_norm"] = self._f32(w["out_norm"])
            assert d["w_in"].shape == (2 * l.heads * (l.dim + l.vdim) + 2 * l.heads, self.spec.width)
            assert d["out_norm"].numel() == l.heads * l.vdim and l.gate_cap > 0
        else:
            raise ValueError(f"unknown mixer '{l.mixer}'")
        assert d["o"].shape == (self.spec.width, l.heads * l.vdim)

    def _load_mlp(self, l, w: dict, d: dict):
        if l.mlp is not None:
            m = l.mlp
            if m.plain:
                if m.plain != "xielu" or m.experts or l.form != "prenorm":
                    raise ValueError("a plain feed-forward is W_down xielu(W_up h) of a pre-norm layer")
                up, dn = w["dense"]
                d["s_gu"], d["s_down"] = self._act(up), self._act(dn)
                p, q = (float(x) for x in w["dense_act"].double().reshape(-1))
                d["unary_p"] = (_softplus(p), 0.5 + _softplus(q))        # the two coefficients, evaluated once in double
                assert d["s_gu"].shape == (m.shared_ff, self.spec.width) and d["s_down"].shape == (self.spec.width, m.shared_ff)
                return
            if m.experts:
                d["router"] = self._f32(w["router"])
                d["gu"] = self._act(torch.stack([torch.cat([g, u], dim=0) for g, u, _ in w["experts"]]))
                d["down"] = self._act(torch.stack([dn for _, _, dn in w["experts"]]))
                assert d["gu"].shape == (m.experts, 2 * m.ff, self.spec.width)
            if m.shared_ff:
                g, u, dn = w["shared"] if "shared" in w else w["dense"]
                d["s_gu"], d["s_down"] = self._act(torch.cat([g, u], dim=0)), self._act(dn)
                assert d["s_gu"].shape == (2 * m.shared_ff, self.spec.width)
                if m.bias:
                    gb, ub, db = w["dense_b"]
                    d["s_gu_b"], d["s_down_b"] = self._f32(torch.cat([gb, ub])), self._f32(db)
                    assert d["s_gu_b"].numel() == 2 * m.shared_ff and d["s_down_b"].numel() == self.spec.width
                if m.shared_gate:
                    d["s_gate"] = self._f32(w["shared_gate"].reshape(-1))
                    assert d["s_gate"].numel() == self.spec.width

    def weight_bytes(self) -> int:
        seen, n = set(), 0

        def count(d):
            nonlocal n
            for t in d.values():
                if isinstance(t, dict):
                    count(t)
                elif isinstance(t, torch.Tensor) and t.data_ptr() not in seen:       # (a tied head counts once)
                    seen.add(t.data_ptr())
                    n += t.numel() * t.element_size()
        count(self.head_weights)
        for d in self.weights:
            count(d)
        return n

    # ------------------------------------------------------------------ C structs
    def _model_struct(self) -> S.Model:
        if self._c_model is not None and self._c_version == self.cache.version:
            return self._c_model
        assert self.head_weights is not None and all(w is not None for w in self.weights), "load every layer first"
        sp, cache = self.spec, self.cache
        p = lambda t: t.data_ptr() if t is not None else None
        layers = (S.Layer * self.num_layers)()
        seconds = []

        def fill_mixer(cl, l, w, i):
            """The mixer's part of a layer struct; i: where the cache keeps this mixer's state."""
            cl.mixer = _MIXERS[l.mixer]
            cl.heads, cl.dim, cl.vdim = l.heads, l.dim, l.vdim
            if l.mixer == "retention":
                cl.rot_dims, cl.inv_freq, cl.decay = l.rot_dims, p(w["inv_freq"]), p(w["decay"])
                cl.ret_state = p(cache.ret_state[i])
            elif l.mixer == "cached_attention":
                cl.kv_heads, cl.attn_mode, cl.gate_kind = l.kv_heads, _ATTN_MODES[l.attn_mode], l.gate_kind
                cl.values_are_keys, cl.pool, cl.taps, cl.window, cl.scale = int(l.values_are_keys), l.pool, l.taps, l.window, l.scale
                cl.rot_dims, cl.inv_freq, cl.rot_mag = l.rot_dims, p(w["inv_freq"]), l.rot_mag
                cl.bias_in, cl.conv_w, cl.head_bias = p(w.get("bias_in")), p(w.get("conv_w")), p(w.get("head_bias"))
                src = sp.layers[l.kv_from] if l.kv_from is not None else l           # whose rows the cache holds
                if l.kv_from is not None and (src.mixer != "cached_attention" or src.kv_from is not None or
                                              (src.kv_heads, src.dim, src.vdim, src.maps) != (l.kv_heads, l.dim, l.vdim, l.maps)):
                    raise ValueError("kv_from must name an earlier cached-attention layer of the same key and value shape")
                cl.kv_from = 0 if l.kv_from is None else l.kv_from + 1
                cl.kv_cache, cl.kv_len = p(cache.kv_cache[src.state_index]), cache.kv_len(src)
                cl.pool_cache, cl.pool_len = p(cache.pool_cache[i]), cache.pool_len(l)
                cl.conv_state = p(cache.conv_state[i])
                cl.softcap, cl.dist_r1, cl.dist_r2, cl.talk = l.softcap, p(w.get("r1")), p(w.get("r2")), p(w.get("talk"))
                cl.chunk, cl.maps, cl.diff_lambda = l.chunk, l.maps, w.get("diff_lambda", 0.0)
                cl.head_unit_norm, cl.out_mult = int(l.head_unit_norm), (1.0 - l.diff) if l.maps == 2 else 1.0
                cl.q_norm_w, cl.k_norm_w = p(w.get("q_norm")), p(w.get("k_norm"))
            elif l.mixer == "time_mix":
                cl.mix_mu, cl.decay_rank, cl.w_decay1, cl.w_decay2 = p(w["mu"]), l.decay_rank, p(w["w1"]), p(w["w2"])
                cl.decay_bias, cl.bonus, cl.out_norm_w = p(w["w0"]), p(w["u"]), p(w["out_norm"])
                cl.tm_state, cl.shift_state = p(cache.tm_state[i]), p(cache.shift[i])
            elif l.mixer == "mlstm":
                cl.gate_cap, cl.bias_in, cl.out_norm_w = l.gate_cap, p(w["bias_in"]), p(w["out_norm"])
                cl.mlstm_state = p(cache.mlstm_state[i])
            else:
                cl.q_rank, cl.kv_rank, cl.window, cl.ring_len = l.q_rank, l.kv_rank, l.window, cache.ring_len(l)
                cl.scale = l.scale
                cl.q_norm, cl.kv_norm, cl.w_uq, cl.w_ukT, cl.w_uv = p(w.get("q_norm")), p(w["kv_norm"]), p(w.get("uq")), \
                    p(w["ukT"]), p(w["uv"])
                cl.w_ukv = p(w["ukv"]) if self.fresh_attention else None
                cl.ring = p(cache.ring[i])
                if l.q_rank == 0:
                    cl.rope_dim, cl.rot_dims, cl.inv_freq, cl.rot_mag = l.rope_dim, l.rot_dims, p(w["inv_freq"]), l.rot_mag
                    cl.attn_mode, cl.gate_kind, cl.sink = _ATTN_MODES[l.attn_mode], l.gate_kind, p(w.get("sink"))
            cl.w_in, cl.w_o = p(w["w_in"]), p(w["o"])

        for i, (l, w) in enumerate(zip(sp.layers, self.weights)):
            cl = layers[i]
            fill_mixer(cl, l, w, i)
            cl.form = S.UMBS_FORM_PRENORM if l.form == "prenorm" else S.UMBS_FORM_PARALLEL
            cl.norm_offset, cl.norm2_w = l.norm_offset, p(w.get("norm2"))
            cl.norm_kind, cl.norm_b, cl.norm2_b = _NORMS[l.norm_kind], p(w.get("norm_b")), p(w.get("norm2_b"))
            cl.norm_alpha, cl.norm2_alpha = w.get("norm_alpha", 1.0), w.get("norm2_alpha", 1.0)
            cl.out_scale, cl.out_scale2, cl.residual_mult = p(w.get("ls1")), p(w.get("ls2")), l.residual_mult
            cl.norm_w = p(w["norm"])
            if l.mixer != "time_mix":
                cl.shift_w, cl.shift_state = p(w.get("shift")), p(cache.shift[i])
            cl.depth_w = p(w.get("depth"))
            if l.second is not None:
                sec = S.Layer()
                fill_mixer(sec, l.second, w["second"], l.second.state_index)
                seconds.append(sec)
                cl.second, cl.mix_scale, cl.second_scale = C.pointer(sec), l.mix_scale, l.second_scale
            cl.has_mlp = int(l.mlp is not None)
            if l.mlp is not None:
                m = l.mlp
                cl.mlp.experts, cl.mlp.top, cl.mlp.ff, cl.mlp.limit = m.experts, m.top, m.ff, m.limit
                cl.mlp.w_router, cl.mlp.w_gu, cl.mlp.w_down = p(w.get("router")), p(w.get("gu")), p(w.get("down"))
                cl.mlp.shared_ff, cl.mlp.shared_limit = m.shared_ff, m.shared_limit
                cl.mlp.ws_gu, cl.mlp.ws_down = p(w.get("s_gu")), p(w.get("s_down"))
                cl.mlp.act = _ACTS[m.act]
                cl.mlp.route_mode, cl.mlp.groups, cl.mlp.keep = _ROUTES[m.route], m.groups, m.keep
                cl.mlp.bias_gu, cl.mlp.bias_down = p(w.get("s_gu_b")), p(w.get("s_down_b"))
                cl.mlp.w_shared_gate = p(w.get("s_gate"))
                cl.mlp.route_scale = m.route_scale
                if m.plain:
                    cl.mlp.plain, cl.mlp.unary = 1, S.UMBS_UNARY_XIELU
                    cl.mlp.unary_p0, cl.mlp.unary_p1 = w["unary_p"]
        m = S.Model()
        m.dtype = S.UMBS_BF16 if self.dtype == torch.bfloat16 else S.UMBS_F32
        m.width, m.vocab, m.n_layers, m.norm_groups, m.slots = sp.width, sp.vocab, self.num_layers, sp.norm_groups, cache.slots
        m.norm_eps, m.norm_offset, m.logit_softcap = sp.norm_eps, sp.norm_offset, sp.logit_softcap
        hw = self.head_weights
        m.embed, m.final_norm, m.head = p(hw["embed"]), p(hw["final_norm"]), p(hw["head"])
        m.embed_scale, m.norm_kind, m.final_norm_b = sp.embed_scale, _NORMS[sp.norm_kind], p(hw.get("final_norm_b"))
        m.final_norm_alpha, m.pos_freq = getattr(self, "final_norm_alpha", 1.0), p(hw.get("pos_freq"))
        m.layers = C.cast(layers, C.POINTER(S.Layer))
        self._c_layers = (layers, seconds)
        self._c_model, self._c_version = m, self.cache.version
        return m

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def forward(self, entries, layer_out: bool = False):
        """``entries``: [(slot, tokens, want)], the next tokens of every sequence of the step and the indices among
        them whose logits are wanted.  Returns fp32 logits [sum of wants, vocab] in entry order (and, with
        ``layer_out``, the residual stream after every layer, [layers, tokens, width]).  The slots' positions advance."""
        cache = self.cache
        ids, tok_seq, tok_pos, want = [], [], [], []
        slot, start, length, pos0, parity = [], [], [], [], []
        for b, (s, toks, w) in enumerate(entries):
            n = len(toks)
            if n == 0:
                raise ValueError("an entry without tokens")
            p0 = cache.position[s]
            if self.max_length is not None and p0 + n > self.max_length:
                raise RuntimeError(f"sequence longer than max_length {self.max_length}")
            slot.append(s), start.append(len(ids)), length.append(n), pos0.append(p0), parity.append(cache.parity[s])
            want += [len(ids) + int(i) for i in w]
            ids += [int(t) for t in toks]
            tok_seq += [b] * n
            tok_pos += range(p0, p0 + n)
        T, B, Wn = len(ids), len(entries), len(want)
        if T:
            cache.reserve_length(max(p + n for p, n in zip(pos0, length)))      # growing parts: room for the longest sequence
        if T == 0:
            return torch.empty((0, self.spec.vocab), dtype=torch.float32, device=self.device)
        if len(set(slot)) != B:
            raise ValueError("a slot appears twice in one step")
        flat = ids + tok_seq + tok_pos + slot + start + length + pos0 + parity + want
        host = torch.tensor(flat, dtype=torch.int32).pin_memory()
        self._reserve(max(T, self._max_tokens0), max(Wn, 1))       # sized once for the largest step announced
        model = self._model_struct()

        def describe(base):
            bt, o = S.Batch(), 0
            bt.n_tokens, bt.n_seqs, bt.n_want, bt.max_seq_len = T, B, Wn, max(length)
            bt.max_pos0 = max(pos0)
            for name, n in (("tok_ids", T), ("tok_seq", T), ("tok_pos", T), ("seq_slot", B), ("seq_start", B),
                            ("seq_len", B), ("seq_pos0", B), ("seq_parity", B), ("want_rows", Wn)):
                setattr(bt, name, base + 4 * o)
                o += n
            return bt

        def enqueue(bt, logits, layers=None):
            S.check(S.load().umbs_forward(C.byref(model), C.byref(bt), logits.data_ptr() if Wn else None,
                                          layers.data_ptr() if layers is not None else None, self._ws.data_ptr(),
                                          self._ws.numel(), torch.cuda.current_stream().cuda_stream), "forward")

        logits = None
        if self.graph_decode and T == B and Wn > 0 and not layer_out:
            logits = self._graph_step((B, Wn, cache.version, self._ws.data_ptr()), host, describe, enqueue)
        layers = None
        if logits is None:
            dev = host.to(self.device, non_blocking=True)
            logits = torch.empty((Wn, self.spec.vocab), dtype=torch.float32, device=self.device)
            layers = torch.empty((self.num_layers, T, self.spec.width), dtype=torch.float32, device=self.device) \
                if layer_out else None
            enqueue(describe(dev.data_ptr()), logits, layers)
            self._keep = (host, dev)          # alive until the next step is enqueued behind this one
        for s, n in zip(slot, length):
            cache.advance(s, n)
        return (logits, layers) if layer_out else logits

    def _graph_step(self, key, host, describe, enqueue):
        """Replay (capturing first, on the third step of this shape) the CUDA graph of a decode step; None = run eagerly."""
        g = self._graphs.get(key)
        if g is None:
            seen = self._graph_seen.get(key, 0)
            self._graph_seen[key] = seen + 1
            if seen < 2:
                return None
            for old in [k for k in self._graphs if k[2:] != key[2:]]:      # the cache or the workspace moved
                del self._graphs[old]
            ints = torch.empty(host.numel(), dtype=torch.int32, device=self.device)
            out = torch.empty((key[1], self.spec.vocab), dtype=torch.float32, device=self.device)
            bt = describe(ints.data_ptr())
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.graph(graph, stream=side):
                enqueue(bt, out)
            torch.cuda.current_stream().wait_stream(side)
            g = self._graphs[key] = (graph, ints, out)
        graph, ints, out = g
        ints.copy_(host, non_blocking=True)
        graph.replay()
        self._keep = (host,)
        return out.clone()

    def clear(self):
        self.cache.clear()
