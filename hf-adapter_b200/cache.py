"""Recurrent cache with the reference's layout and methods (rwkv7_hf/model_cache.py:48-465):
``state`` list[L] of ``[B,H,N,N]`` fp32, ``xpa`` / ``xpf`` list[L] of ``[B,D]`` (attention / FFN
token-shift states, the NORMALISED previous inputs), ``v_first [B,H*N]``, plus ``seen_tokens``.
Iterable as the 4-tuple ``(state, xpa, xpf, v_first)``."""
from __future__ import annotations

import torch

_METRIC_NAMES = ("clones", "detaches", "device_moves", "select_batch_calls", "batch_select_calls", "batch_select_indices_calls",
                 "batch_repeat_interleave_calls", "reorder_calls", "crops", "resets", "native_graph_bound_selects")


class NativeRWKV7LegacyCache(tuple):
    """The raw 4-tuple ``(state, xpa, xpf, v_first)`` that still knows how many tokens it has seen
    (rwkv7_hf/model_cache.py:13-45): what ``to_legacy_cache`` returns and ``from_legacy_cache`` takes back."""

    def __new__(cls, state, xpa, xpf, v_first, seen_tokens: int = 0):
        obj = super().__new__(cls, (state, xpa, xpf, v_first))
        obj._seen_tokens = int(seen_tokens)
        return obj

    def get_seq_length(self, layer_idx=0, cache_position=None) -> int:
        if layer_idx is not None:
            state = self[0]
            if int(layer_idx) < 0 or (state is not None and int(layer_idx) >= len(state)) or (state is None and int(layer_idx) != 0):
                return 0
        return self._seen_tokens

    @property
    def seen_tokens(self) -> int:
        return int(self._seen_tokens)

    @seen_tokens.setter
    def seen_tokens(self, value: int) -> None:
        self._seen_tokens = int(value)

    def to_legacy_cache(self):
        return self


class NativeRWKV7Cache:
    is_compileable = True

    def __init__(self, state=None, xpa=None, xpf=None, v_first=None, seen_tokens: int = 0, elapsed=None):
        self._state, self._xpa, self._xpf, self._v_first = state, xpa, xpf, v_first
        self._seen_tokens = int(seen_tokens)
        # FP16-state lane only: per-sequence step counters (int32 [B]) that phase the decay dither
        # (the ``elapsed`` operand of rwkv7_hf/native_wkv_fp16.py:54-71); None for an fp32 state
        self._elapsed = elapsed
        self._graph_owner = None  # decode-graph runner whose static buffers these tensors are, if any
        # how often the cache was copied, moved or re-batched: what a serving layer samples to see whether requests
        # reuse one cache or keep rebuilding it (rwkv7_hf/model_cache.py:71-83,427-436)
        self._rwkv7_cache_metrics = dict.fromkeys(_METRIC_NAMES, 0)

    # -- tuple protocol ---------------------------------------------------
    def __iter__(self):
        return iter((self._state, self._xpa, self._xpf, self._v_first))

    def __len__(self):
        return 4

    def __getitem__(self, i):
        return (self._state, self._xpa, self._xpf, self._v_first)[i]

    @classmethod
    def allocate(cls, num_layers, batch, hidden, heads, head_dim, device, dtype, state_dtype=torch.float32):
        """Zero state (rwkv7_hf/native.py:283-295).  ``state_dtype=torch.float16`` allocates the FP16-state lane's
        cache (half the recurrent-state bytes, plus the ``elapsed`` counters of its decay dither)."""
        z = lambda *s, dt=dtype: torch.zeros(*s, device=device, dtype=dt)
        return cls([z(batch, heads, head_dim, head_dim, dt=state_dtype) for _ in range(num_layers)],
                   [z(batch, hidden) for _ in range(num_layers)], [z(batch, hidden) for _ in range(num_layers)],
                   z(batch, heads * head_dim), 0,
                   elapsed=z(batch, dt=torch.int32) if state_dtype == torch.float16 else None)

    def _tensors(self):
        """Every tensor of the cache as one flat list (the order `_set_tensors` takes)."""
        t = list(self._state) + list(self._xpa) + list(self._xpf) + [self._v_first]
        return t + ([self._elapsed] if self._elapsed is not None else [])

    def _set_tensors(self, tensors):
        L = len(self._state)
        self._state, self._xpa, self._xpf = list(tensors[:L]), list(tensors[L:2 * L]), list(tensors[2 * L:3 * L])
        self._v_first = tensors[3 * L]
        if self._elapsed is not None:
            self._elapsed = tensors[3 * L + 1]

    # -- HF cache contract ---------------------------------------------------
    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen_tokens

    @property
    def seen_tokens(self) -> int:
        return self._seen_tokens

    @seen_tokens.setter
    def seen_tokens(self, value: int) -> None:
        self._seen_tokens = int(value)

    def rwkv7_cache_metrics(self) -> dict:
        metrics = dict(self._rwkv7_cache_metrics)
        metrics.update({"seen_tokens": int(self._seen_tokens), "batch_size": self.get_batch_size(),
                        "layers": len(self._state) if self._state is not None else 0})
        return metrics

    def to_legacy_cache(self):
        return NativeRWKV7LegacyCache(self._state, self._xpa, self._xpf, self._v_first, seen_tokens=self._seen_tokens)

    def get_max_cache_shape(self):
        return None

    def get_batch_size(self):
        if self._state:
            return int(self._state[0].shape[0])
        if self._v_first is not None:
            return int(self._v_first.shape[0])
        return None

    def _is_initialized(self, layer_idx=None) -> bool:
        return bool(self._state) and self._v_first is not None

    def has_previous_state(self, layer_idx=None) -> bool:
        return self._is_initialized(layer_idx) and self._seen_tokens > 0

    def _map(self, fn, *, inplace, count=()):
        ml = lambda vs: None if vs is None else [fn(v) for v in vs]
        state, xpa, xpf = ml(self._state), ml(self._xpa), ml(self._xpf)
        vf = None if self._v_first is None else fn(self._v_first)
        el = None if self._elapsed is None else fn(self._elapsed)
        if inplace:
            if self._graph_owner is not None and "select_batch_calls" in count:
                count = tuple(count) + ("native_graph_bound_selects",)
            self._state, self._xpa, self._xpf, self._v_first, self._elapsed = state, xpa, xpf, vf, el
            self._graph_owner = None
            target = self
        else:
            target = NativeRWKV7Cache(state, xpa, xpf, vf, self._seen_tokens, elapsed=el)
            target._rwkv7_cache_metrics = dict(self._rwkv7_cache_metrics)
        for name in count:
            target._rwkv7_cache_metrics[name] += 1
        return target

    def clone(self):
        return self._map(lambda v: v.clone(), inplace=False, count=("clones",))

    def detach(self, *, inplace: bool = True):
        return self._map(lambda v: v.detach(), inplace=inplace, count=("detaches",))

    def to(self, *args, copy: bool = False, **kwargs):
        def move(v):
            if not v.is_floating_point():  # the elapsed counters only change device
                dev = kwargs.get("device", next((a for a in args if not isinstance(a, torch.dtype)), v.device))
                return v.to(device=dev, copy=copy)
            if v.dtype == torch.float32 and ("dtype" in kwargs or any(isinstance(a, torch.dtype) for a in args)):
                # the fp32 recurrent state keeps its dtype; only the device moves
                dev = kwargs.get("device", next((a for a in args if not isinstance(a, torch.dtype)), v.device))
                return v.to(device=dev, copy=copy)
            return v.to(*args, copy=copy, **kwargs)
        return self._map(move, inplace=False, count=("device_moves",))

    def reset(self) -> None:
        for vs in (self._state, self._xpa, self._xpf):
            for v in vs or ():
                v.zero_()
        if self._v_first is not None:
            self._v_first.zero_()
        if self._elapsed is not None:
            self._elapsed.zero_()
        self._seen_tokens = 0
        self._rwkv7_cache_metrics["resets"] += 1

    def select_batch(self, indices, *, inplace: bool = True, _count=("select_batch_calls",)):
        return self._map(lambda v: v.index_select(0, indices.to(v.device)), inplace=inplace, count=_count)

    compact = select_batch

    def batch_select(self, indices, *, inplace: bool = True):
        return self.select_batch(indices, inplace=inplace, _count=("select_batch_calls", "batch_select_calls"))

    def batch_select_indices(self, indices):
        return self.select_batch(indices, inplace=True, _count=("select_batch_calls", "batch_select_indices_calls"))

    def reorder_cache(self, beam_idx):
        return self.select_batch(beam_idx, inplace=True, _count=("select_batch_calls", "reorder_calls"))

    def batch_repeat_interleave(self, repeats: int):
        return self._map(lambda v: v.repeat_interleave(int(repeats), dim=0), inplace=True,
                         count=("batch_repeat_interleave_calls",))

    def crop(self, max_length: int):
        """A recurrent state cannot be rolled back to a shorter positive prefix
        (rwkv7_hf/model_cache.py:368-380): only no-op crops and a crop to zero are possible."""
        if max_length < 0:
            max_length = self._seen_tokens + max_length
        if max_length >= self._seen_tokens:
            return self
        if max_length == 0:
            self.reset()
            self._rwkv7_cache_metrics["crops"] += 1
            return self
        raise ValueError("a recurrent RWKV-7 cache cannot be cropped to a positive prefix")

    @classmethod
    def from_legacy_cache(cls, legacy, seen_tokens: int = 0):
        if legacy is None:
            return cls(seen_tokens=seen_tokens)
        if isinstance(legacy, cls):
            return legacy
        seen = int(seen_tokens)
        if hasattr(legacy, "get_seq_length"):
            try:
                legacy_seen = int(legacy.get_seq_length())
                if legacy_seen == 0:
                    return cls(seen_tokens=seen_tokens)
                seen = legacy_seen
            except Exception:
                pass
        if hasattr(legacy, "to_legacy_cache"):
            legacy = legacy.to_legacy_cache()
        if legacy is None or (isinstance(legacy, (list, tuple)) and len(legacy) == 0):
            return cls(seen_tokens=seen_tokens)
        if not isinstance(legacy, (list, tuple)) or len(legacy) != 4:
            raise TypeError("NativeRWKV7Cache.from_legacy_cache expects None, an empty cache, or a 4-tuple recurrent cache")
        state, xpa, xpf, v_first = legacy
        return cls(state, xpa, xpf, v_first, seen_tokens=seen)
