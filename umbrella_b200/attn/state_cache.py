"""Slot-based state of the sequence-state decoders (the counterpart of attn/cache.py's KV_Cache for models whose
per-sequence memory is mostly a fixed-size state).

Every live sequence owns one slot.  A slot holds, per layer,
  * token shift: the previous token's normed activations, fp32 [width], double-buffered (a step reads the half
    ``parity`` names and writes the other, then the parity flips);
  * retention layers: the state matrices, fp32 [heads, dim, vdim];
  * latent-attention layers: a ring of the last ``ring_len`` latents, [ring_len, kv_rank] in the activation dtype,
    position p at row p mod ring_len (ring_len = the layer's window, capped by ``max_length`` when that is given); a
    layer whose keys carry a rotated part shared by all heads keeps it behind the latent, [ring_len, kv_rank + rope_dim];
    a layer without a window keeps a row for every token up to ``capacity`` tokens, as cached attention does;
  * cached-attention layers: key | value rows per token, [kv_len, kv_heads (dim + vdim)] in the activation dtype,
    position p at row p mod kv_len -- with a window a ring of max(window, pool) rows, without one a row for every
    token up to ``capacity`` tokens (the cache reallocates with twice the capacity when a sequence outgrows it);
    with pooled blocks a table of one mean key | value row per block, [capacity / pool, .]; with a short convolution
    the last taps - 1 projected q | k rows, fp32, double-buffered like the shift state;
  * mLSTM layers: per head the matrix S with the normaliser n as one more column and the running maximum m,
    fp32 [heads, dim (vdim + 1) + 1];
  * time-mix layers: per head the matrix memory, fp32 [heads, dim, dim] (key index first), and the previous token's
    normed activations in the token-shift state.
and on the host its position (tokens fed so far) and parity.
A cached-attention layer with several maps per head keeps [kv_heads (maps dim + vdim)] numbers per token; one with a
chunked mask needs a ring of one chunk only; one that borrows another layer's keys and values keeps nothing (the lender's
ring reaches as far back as its furthest-seeing borrower reads).  A layer's second mixer (two mixers side by side) has
state of its own, kept behind the layers' in the same lists (``spec.layers[i].second.state_index``).  Nothing is cleared when a slot is freed or handed out
again: the kernels read a sequence's state as zero while its position is 0, and a ring row is only ever read for a
position that the current owner has written.
"""
from __future__ import annotations

import torch


class SequenceStateCache:
    def __init__(self, spec, slots: int = 8, device="cuda:0", dtype=torch.bfloat16, max_length: int | None = None,
                 capacity: int = 0):
        self.spec, self.device, self.dtype = spec, torch.device(device), dtype
        self.max_length = max_length
        self.slots = 0
        # tokens per sequence that the growing parts (windowless key/value rows, pooled-block tables) hold
        self.capacity = int(max_length or capacity or 512)
        # every mixer that keeps state: the layers' own, then the second mixers of layers that run two side by side
        self.units = []
        for i, l in enumerate(spec.layers):
            l.state_index = i
            self.units.append(l)
        for l in spec.layers:
            if getattr(l, "second", None) is not None:
                l.second.state_index = len(self.units)
                self.units.append(l.second)
        # a layer that lends its keys and values keeps them as far back as its furthest-seeing borrower asks
        self._borrowers = {}
        for l in self.units:
            if l.mixer == "cached_attention" and l.kv_from is not None:
                self._borrowers.setdefault(id(spec.layers[l.kv_from]), []).append(l)
        self._growing = any((l.mixer == "cached_attention" and l.kv_from is None and (self._reach(l) is None or l.pool > 0)) or
                            (l.mixer == "latent_attention" and l.window <= 0) for l in self.units)
        n = len(self.units)
        self.kv_cache: list[torch.Tensor | None] = [None] * n
        self.pool_cache: list[torch.Tensor | None] = [None] * n
        self.conv_state: list[torch.Tensor | None] = [None] * n
        self.mlstm_state: list[torch.Tensor | None] = [None] * n
        self.tm_state: list[torch.Tensor | None] = [None] * n
        self.shift: list[torch.Tensor | None] = [None] * n
        self.ret_state: list[torch.Tensor | None] = [None] * n
        self.ring: list[torch.Tensor | None] = [None] * n
        self.position: list[int] = []
        self.parity: list[int] = []
        self._free: list[int] = []
        self.version = 0                      # bumped whenever the tensors are reallocated (pointers change)
        self.grow(max(1, int(slots)))

    def ring_len(self, layer) -> int:
        """Rows of a latent-attention layer's ring per slot: its window, or -- without one -- a row for every token."""
        n = int(layer.window)
        if n <= 0:
            return self.capacity
        return max(1, min(n, self.max_length) if self.max_length else n)

    def kv_len(self, layer) -> int:
        """Rows of a cached-attention layer's key/value cache per slot: the furthest key a row can see -- its window, or
        its chunk -- bounds the ring; without either, a row per token."""
        reach = self._reach(layer)
        return max(reach, int(layer.pool), 1) if reach is not None else self.capacity

    def _reach(self, layer):
        """How many positions back the rows of ``layer``'s cache are read, by itself and its borrowers; None: any."""
        most = 0
        for l in [layer] + self._borrowers.get(id(layer), []):
            own = [int(n) for n in (l.window, l.chunk) if n > 0]
            if not own:
                return None
            most = max(most, min(own))
        return most

    def pool_len(self, layer) -> int:
        return max(1, -(-self.capacity // int(layer.pool))) if layer.pool > 0 else 0

    def reserve_length(self, tokens: int):
        """Make sure a sequence of ``tokens`` tokens fits the growing parts (doubling the capacity when it does not)."""
        if tokens <= self.capacity or not self._growing:
            return
        if self.max_length is not None and tokens > self.max_length:
            raise RuntimeError(f"sequence longer than max_length {self.max_length}")
        cap = self.capacity
        while cap < tokens:
            cap *= 2
        self._resize(self.slots, min(cap, self.max_length) if self.max_length else cap)

    def grow(self, slots: int):
        """Make room for ``slots`` slots, keeping what the existing ones hold."""
        if slots > self.slots:
            self._resize(slots, self.capacity)

    def _resize(self, slots: int, capacity: int):
        old = self.slots
        f32 = dict(dtype=torch.float32, device=self.device)
        act = dict(dtype=self.dtype, device=self.device)

        def widen(t_old, shape, slot_dim, **kw):
            t = torch.zeros(shape, **kw)
            if t_old is not None:
                part = t.narrow(slot_dim, 0, old)
                if part.shape != t_old.shape:                       # a longer cache: rows keep their index
                    part = part.narrow(slot_dim + 1, 0, t_old.shape[slot_dim + 1])
                part.copy_(t_old)
            return t
        self.capacity = capacity
        for i, l in enumerate(self.units):
            if l.shift or l.mixer == "time_mix":
                self.shift[i] = widen(self.shift[i], (2, slots, self.spec.width), 1, **f32)
            if l.mixer == "retention":
                self.ret_state[i] = widen(self.ret_state[i], (slots, l.heads, l.dim, l.vdim), 0, **f32)
            elif l.mixer == "latent_attention":
                self.ring[i] = widen(self.ring[i], (slots, self.ring_len(l), l.kv_rank + getattr(l, "rope_dim", 0)), 0,
                                     dtype=self.dtype, device=self.device)
            elif l.mixer == "time_mix":
                self.tm_state[i] = widen(self.tm_state[i], (slots, l.heads, l.dim, l.dim), 0, **f32)
            elif l.mixer == "cached_attention" and l.kv_from is None:
                row = l.kv_heads * (l.maps * l.dim + l.vdim)
                self.kv_cache[i] = widen(self.kv_cache[i], (slots, self.kv_len(l), row), 0, **act)
                if l.pool > 0:
                    self.pool_cache[i] = widen(self.pool_cache[i], (slots, self.pool_len(l), row), 0, **act)
                if l.taps > 1:
                    self.conv_state[i] = widen(self.conv_state[i], (2, slots, l.taps - 1, (l.heads + l.kv_heads) * l.maps * l.dim),
                                               1, **f32)
            elif l.mixer == "mlstm":
                self.mlstm_state[i] = widen(self.mlstm_state[i], (slots, l.heads, l.dim * (l.vdim + 1) + 1), 0, **f32)
        self.position += [0] * (slots - old)
        self.parity += [0] * (slots - old)
        self._free += list(range(old, slots))
        self.slots = slots
        self.version += 1

    def alloc_slot(self) -> int:
        """A slot for a new sequence (position 0).  Grows the cache when every slot is taken."""
        if not self._free:
            self.grow(self.slots * 2)
        s = self._free.pop(0)
        self.position[s], self.parity[s] = 0, 0
        return s

    def free_slot(self, slot: int):
        if slot in self._free or not 0 <= slot < self.slots:
            raise ValueError(f"slot {slot} is not in use")
        self.position[slot] = 0
        self._free.append(slot)

    @property
    def live_slots(self) -> int:
        return self.slots - len(self._free)

    def advance(self, slot: int, n_tokens: int):
        self.position[slot] += n_tokens
        self.parity[slot] ^= 1

    def state_bytes_per_slot(self) -> int:
        n = 0
        for t in self.shift + self.ret_state + self.ring + self.kv_cache + self.pool_cache + self.conv_state + self.mlstm_state + \
                self.tm_state:
            if t is not None:
                n += t.numel() * t.element_size() // self.slots
        return n

    def clear(self):
        self._free = list(range(self.slots))
        self.position = [0] * self.slots
        self.parity = [0] * self.slots
