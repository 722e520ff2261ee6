"""Serving state pool: persistent per-request recurrent state in slot pools that the decode kernels index directly.

The layout and the allocator interface follow the reference's serving ABI
(docs/integrations/RWKV7_STATE_CACHE_ABI.md): layer-major tensors

    S_pool      [L, capacity + 1, H, N, N]  fp32     xpa_pool / xpf_pool [L, capacity + 1, D]
    vfirst_pool [capacity + 1, A]                    seen_tokens / generation / allocated [capacity]

with one extra row, the scratch slot, that no request owns: padding rows of a fixed-size CUDA-graph batch point at
it, so they can never change live state.  A decode step hands the pools and an int32 ``slot_ids`` vector to the
kernels (rwkv7_*_pool entry points), which read and write row ``slot_ids[b]`` in place: no gather before the step,
no scatter after it, and a captured graph does not depend on which requests are scheduled -- the copies that
``NativeRWKV7Cache.select_batch`` (rwkv7_hf/model_cache.py:301-333) makes on every batch change disappear.
Prefill gathers the scheduled slots into a dense cache, runs the layer-wise prefill and scatters the result back
(once per prompt chunk, where the copies are negligible).
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import torch

from . import norm_mix as _nm
from . import packing as _pk
from .cache import NativeRWKV7Cache


@dataclass
class PrefixEntry:
    """An immutable snapshot of one request's state after a prefix of ``seen_tokens`` tokens."""
    key: str
    state: torch.Tensor   # [L,H,N,N]
    xpa: torch.Tensor     # [L,D]
    xpf: torch.Tensor     # [L,D]
    v_first: torch.Tensor  # [A]
    seen_tokens: int
    checksum: str
    nbytes: int
    last_access: int = 0


@dataclass
class PoolTelemetry:
    allocation_failures: int = 0
    prefix_hits: int = 0
    prefix_misses: int = 0
    prefix_evictions: int = 0
    prefix_bytes_restored: int = 0
    prefix_tokens_saved: int = 0
    gather_scatter_bytes: int = 0
    clones: int = 0
    stale_generation_rejections: int = 0
    high_water: int = 0
    active_rows: int = 0
    graph_bucket_rows: int = 0
    extra: dict = field(default_factory=dict)


class StaleSlotError(RuntimeError):
    """A handle whose generation no longer matches its slot: the slot was freed (and possibly reassigned)."""


def _checksum(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


class RWKV7StatePool:
    """Slot pool for ``capacity`` concurrent requests of ``model`` (an RWKV7ForCausalLM of this package, fp32 state)."""

    LAYOUT_VERSION = 1

    def __init__(self, model, capacity: int, *, prefix_cache_bytes: int = 0, fingerprint: str = ""):
        if model.state_dtype != torch.float32:
            raise ValueError("the state pool holds the fp32 recurrent state")
        if model.tp_world != 1:
            raise ValueError("the state pool serves a single-GPU model")
        cfg = model.config
        self.model = model
        self.capacity = int(capacity)
        if self.capacity < 1:
            raise ValueError("capacity must be positive")
        self.L, self.H, self.N, self.D = cfg.num_hidden_layers, cfg.num_heads, cfg.head_dim, cfg.hidden_size
        self.A = self.H * self.N
        dev, dt = model.device, model.dtype
        rows = self.capacity + 1
        self.scratch_slot = self.capacity
        self.S_pool = torch.zeros(self.L, rows, self.H, self.N, self.N, device=dev, dtype=torch.float32)
        self.xpa_pool = torch.zeros(self.L, rows, self.D, device=dev, dtype=dt)
        self.xpf_pool = torch.zeros(self.L, rows, self.D, device=dev, dtype=dt)
        self.vfirst_pool = torch.zeros(rows, self.A, device=dev, dtype=dt)
        self.seen_tokens = [0] * self.capacity
        self.generation = [0] * self.capacity
        self.allocated = [False] * self.capacity
        self.request_of = [None] * self.capacity
        self._free = list(range(self.capacity - 1, -1, -1))
        self.telemetry = PoolTelemetry()
        self.fingerprint = fingerprint or self._default_fingerprint()
        self._prefix: dict[str, PrefixEntry] = {}
        self._prefix_budget = int(prefix_cache_bytes)
        self._prefix_bytes = 0
        self._clock = 0
        self._graphs: dict[int, "PoolDecodeGraph"] = {}

    # ------------------------------------------------------------------ bookkeeping
    def _default_fingerprint(self) -> str:
        c = self.model.config
        kinds = sorted({type(m).__name__ for m in self.model.modules()})
        return f"layout{self.LAYOUT_VERSION}|L{c.num_hidden_layers}|D{c.hidden_size}|H{c.num_heads}|V{c.vocab_size}|{self.model.dtype}|{','.join(kinds)}"

    @property
    def bytes_per_slot(self) -> int:
        e = self.xpa_pool.element_size()
        return self.L * self.H * self.N * self.N * 4 + 2 * self.L * self.D * e + self.A * e

    def stats(self) -> dict:
        used = sum(self.allocated)
        t = self.telemetry
        return dict(allocated_slots=used, free_slots=self.capacity - used, bytes_per_slot=self.bytes_per_slot,
                    total_state_bytes=self.bytes_per_slot * (self.capacity + 1), allocation_failures=t.allocation_failures,
                    prefix_hits=t.prefix_hits, prefix_misses=t.prefix_misses, prefix_evictions=t.prefix_evictions,
                    prefix_bytes_restored=t.prefix_bytes_restored, prefix_tokens_saved=t.prefix_tokens_saved,
                    prefix_entries=len(self._prefix), prefix_bytes=self._prefix_bytes,
                    gather_scatter_bytes=t.gather_scatter_bytes, clones=t.clones,
                    stale_generation_rejections=t.stale_generation_rejections, high_water=t.high_water,
                    active_rows=t.active_rows, graph_bucket_rows=t.graph_bucket_rows)

    def _check(self, slot_ids, generations=None):
        slots = [int(s) for s in slot_ids]
        if len(set(slots)) != len(slots):
            raise ValueError("a batch must not name a slot twice: two rows would race on one state")
        for i, s in enumerate(slots):
            if not 0 <= s < self.capacity or not self.allocated[s]:
                self.telemetry.stale_generation_rejections += 1
                raise StaleSlotError(f"slot {s} is not allocated")
            if generations is not None and int(generations[i]) != self.generation[s]:
                self.telemetry.stale_generation_rejections += 1
                raise StaleSlotError(f"slot {s}: handle generation {int(generations[i])} != {self.generation[s]}")
        return slots

    def _index(self, slots):
        return torch.tensor(slots, device=self.S_pool.device, dtype=torch.long)

    # ------------------------------------------------------------------ allocator interface
    def allocate(self, request_ids):
        """Zero-initialised, uniquely owned slots: returns ``(slot_ids, generations)`` (lists)."""
        request_ids = list(request_ids)
        if len(request_ids) > len(self._free):
            self.telemetry.allocation_failures += 1
            raise RuntimeError(f"state pool exhausted: {len(request_ids)} requested, {len(self._free)} free")
        slots = [self._free.pop() for _ in request_ids]
        for s, rid in zip(slots, request_ids):
            self.allocated[s], self.request_of[s], self.seen_tokens[s] = True, rid, 0
        self._zero(slots)
        self.telemetry.high_water = max(self.telemetry.high_water, sum(self.allocated))
        return slots, [self.generation[s] for s in slots]

    def free(self, slot_ids, generations=None) -> None:
        """Invalidate the handles (generation bump), then make the slots reusable."""
        for s in self._check(slot_ids, generations):
            self.generation[s] += 1
            self.allocated[s], self.request_of[s], self.seen_tokens[s] = False, None, 0
            self._free.append(s)

    def _zero(self, slots):
        idx = self._index(slots)
        self.S_pool.index_fill_(1, idx, 0)
        self.xpa_pool.index_fill_(1, idx, 0)
        self.xpf_pool.index_fill_(1, idx, 0)
        self.vfirst_pool.index_fill_(0, idx, 0)

    def reset(self, slot_ids, generations=None) -> None:
        """Exact new-request state."""
        slots = self._check(slot_ids, generations)
        self._zero(slots)
        for s in slots:
            self.seen_tokens[s] = 0

    def clone(self, source_slots, destination_slots) -> None:
        """Deep copy for beam / fork / speculative candidates: destinations become independent continuations."""
        src, dst = self._check(source_slots), self._check(destination_slots)
        if len(src) != len(dst) or set(src) & set(dst):
            raise ValueError("clone needs as many distinct destination slots as sources")
        si, di = self._index(src), self._index(dst)
        self.S_pool.index_copy_(1, di, self.S_pool.index_select(1, si))
        self.xpa_pool.index_copy_(1, di, self.xpa_pool.index_select(1, si))
        self.xpf_pool.index_copy_(1, di, self.xpf_pool.index_select(1, si))
        self.vfirst_pool.index_copy_(0, di, self.vfirst_pool.index_select(0, si))
        for s, d in zip(src, dst):
            self.seen_tokens[d] = self.seen_tokens[s]
        self.telemetry.clones += len(src)

    def gather(self, slot_ids, generations=None) -> NativeRWKV7Cache:
        """The scheduled rows as a dense cache in batch order (copies)."""
        slots = self._check(slot_ids, generations)
        idx = self._index(slots)
        cache = NativeRWKV7Cache([self.S_pool[l].index_select(0, idx) for l in range(self.L)],
                                 [self.xpa_pool[l].index_select(0, idx) for l in range(self.L)],
                                 [self.xpf_pool[l].index_select(0, idx) for l in range(self.L)],
                                 self.vfirst_pool.index_select(0, idx), seen_tokens=0)
        self.telemetry.gather_scatter_bytes += self.bytes_per_slot * len(slots)
        return cache

    def scatter(self, slot_ids, cache, generations=None) -> None:
        """Commit a dense cache's rows to exactly those live slots."""
        slots = self._check(slot_ids, generations)
        idx = self._index(slots)
        state, xpa, xpf, v_first = cache
        for l in range(self.L):
            self.S_pool[l].index_copy_(0, idx, state[l])
            self.xpa_pool[l].index_copy_(0, idx, xpa[l])
            self.xpf_pool[l].index_copy_(0, idx, xpf[l])
        self.vfirst_pool.index_copy_(0, idx, v_first)
        self.telemetry.gather_scatter_bytes += self.bytes_per_slot * len(slots)

    # ------------------------------------------------------------------ prefix cache
    def prefix_key(self, token_ids) -> str:
        ids = torch.as_tensor(token_ids, dtype=torch.int64).reshape(-1).cpu().numpy().tobytes()
        return hashlib.sha256(self.fingerprint.encode() + b"|" + ids).hexdigest()

    def snapshot(self, slot_id: int, token_ids=None, *, offload: bool = False) -> PrefixEntry:
        """An immutable copy of one slot (on the CPU with ``offload``).  With ``token_ids`` (the exact prefix that
        produced the state) the entry is also stored in the prefix cache under a key over the model fingerprint
        and those ids."""
        (s,) = self._check([slot_id])
        dev = "cpu" if offload else self.S_pool.device
        parts = [self.S_pool[:, s], self.xpa_pool[:, s], self.xpf_pool[:, s], self.vfirst_pool[s]]
        parts = [p.to(dev, copy=True) for p in parts]
        if token_ids is not None and int(torch.as_tensor(token_ids).numel()) != self.seen_tokens[s]:
            raise ValueError("the prefix ids must be exactly the tokens the slot has consumed (padding is not a prefix)")
        key = self.prefix_key(token_ids) if token_ids is not None else ""
        entry = PrefixEntry(key, *parts, seen_tokens=self.seen_tokens[s], checksum=_checksum(*parts),
                            nbytes=sum(p.numel() * p.element_size() for p in parts))
        if key and self._prefix_budget > 0:
            self._store(entry)
        return entry

    def _store(self, entry):
        old = self._prefix.pop(entry.key, None)
        if old is not None:
            self._prefix_bytes -= old.nbytes
        while self._prefix and self._prefix_bytes + entry.nbytes > self._prefix_budget:
            victim = min(self._prefix.values(), key=lambda e: e.last_access)
            self._prefix_bytes -= victim.nbytes
            del self._prefix[victim.key]
            self.telemetry.prefix_evictions += 1
        if entry.nbytes <= self._prefix_budget:
            self._clock += 1
            entry.last_access = self._clock
            self._prefix[entry.key] = entry
            self._prefix_bytes += entry.nbytes

    def lookup(self, token_ids):
        """Longest cached prefix of ``token_ids``: ``(entry, length)`` or ``(None, 0)``."""
        ids = torch.as_tensor(token_ids, dtype=torch.int64).reshape(-1)
        lengths = sorted({e.seen_tokens for e in self._prefix.values() if e.seen_tokens <= int(ids.numel())}, reverse=True)
        for n in lengths:
            e = self._prefix.get(self.prefix_key(ids[:n]))
            if e is not None:
                self._clock += 1
                e.last_access = self._clock
                self.telemetry.prefix_hits += 1
                return e, n
        self.telemetry.prefix_misses += 1
        return None, 0

    def restore(self, entry: PrefixEntry, destination_slot: int, *, verify: bool = True) -> None:
        """Validate the snapshot and copy it into a live slot (eager clone on hit: entries stay immutable)."""
        (d,) = self._check([destination_slot])
        if tuple(entry.state.shape) != (self.L, self.H, self.N, self.N) or tuple(entry.xpa.shape) != (self.L, self.D):
            raise ValueError("the snapshot does not have this pool's layout")
        if verify and _checksum(entry.state, entry.xpa, entry.xpf, entry.v_first) != entry.checksum:
            raise ValueError("the snapshot fails its checksum")
        self.S_pool[:, d].copy_(entry.state, non_blocking=False)
        self.xpa_pool[:, d].copy_(entry.xpa)
        self.xpf_pool[:, d].copy_(entry.xpf)
        self.vfirst_pool[d].copy_(entry.v_first)
        self.seen_tokens[d] = entry.seen_tokens
        self.telemetry.prefix_bytes_restored += entry.nbytes
        self.telemetry.prefix_tokens_saved += entry.seen_tokens

    # ------------------------------------------------------------------ execution
    def _slot_vector(self, slots, rows):
        """int32 device vector of ``rows`` entries: the scheduled slots, then the scratch slot for padding rows."""
        return torch.tensor(list(slots) + [self.scratch_slot] * (rows - len(slots)), device=self.S_pool.device, dtype=torch.int32)

    @torch.no_grad()
    def decode(self, token_ids, slot_ids, generations=None, *, use_graph: bool = True, greedy: bool = False):
        """One token for every scheduled request, state updated in place inside the pools.  Returns logits
        ``[len(slot_ids), V]`` (or the greedy tokens).  With ``use_graph`` the step replays a CUDA graph captured for the
        next bucket size (1, 2, 4, ...); padding rows read and write the scratch slot only."""
        slots = self._check(slot_ids, generations)
        n = len(slots)
        ids = torch.as_tensor(token_ids, device=self.S_pool.device).reshape(-1)
        if int(ids.numel()) != n:
            raise ValueError("one token per scheduled slot")
        if use_graph:
            bucket = 1 << max(0, (n - 1).bit_length())
            g = self._graphs.get((bucket, greedy))
            if g is None:
                g = self._graphs[(bucket, greedy)] = PoolDecodeGraph(self, bucket, greedy)
            out = g.replay(ids, self._slot_vector(slots, bucket))[:n].clone()
            self.telemetry.graph_bucket_rows = bucket
        else:
            out = self._step(ids, self._slot_vector(slots, n), greedy)
        self.telemetry.active_rows = n
        for s in slots:
            self.seen_tokens[s] += 1
        return out

    def _step(self, ids, slot_vec, greedy):
        m = self.model
        x = torch.nn.functional.embedding(ids, m.model.embeddings.weight)
        ctx = _pk.StepContext(m._side_stream, None, 1, 0, 0, 0, slot_ids=slot_vec)
        packs, _, _, _ = _pk.extract_graph_packs(m)
        for l, p in enumerate(packs):
            x = _pk.block_ip_batched(x, self.S_pool[l], self.xpa_pool[l], self.xpf_pool[l], self.vfirst_pool, p, context=ctx)
        xn = _nm.layer_norm(x, m.model.norm.weight, m.model.norm.bias)
        return m._head(xn, greedy)

    @torch.no_grad()
    def prefill(self, input_ids, slot_ids, generations=None, *, chunk_size: int = 512, scan_chunk: int = 0, use_prefix_cache: bool = False):
        """Consume ``input_ids [n, T]`` (one prompt of T tokens per scheduled slot) continuing from the slots' states.
        Returns the last-token logits ``[n, V]``.  With ``use_prefix_cache`` and a single fresh request the longest cached
        prefix is restored and only the suffix is computed."""
        slots = self._check(slot_ids, generations)
        ids = torch.as_tensor(input_ids, device=self.S_pool.device)
        if ids.dim() != 2 or int(ids.shape[0]) != len(slots):
            raise ValueError("input_ids must be [len(slot_ids), T]")
        T = int(ids.shape[1])
        start = 0
        if use_prefix_cache and len(slots) == 1 and self.seen_tokens[slots[0]] == 0:
            entry, n = self.lookup(ids[0])
            if entry is not None and n < T:  # at least one token must run to produce logits
                self.restore(entry, slots[0])
                start = n
        cache = self.gather(slots)
        logits, cache = self.model.rwkv7_prefill_chunks(ids[:, start:], cache, chunk_size=chunk_size, scan_chunk=scan_chunk)
        self.scatter(slots, cache)
        for s in slots:
            self.seen_tokens[s] += T - start
        return logits[:, -1]


class PoolDecodeGraph:
    """A decode step captured once per bucket size over the pools themselves.  The kernels read the slot vector from a
    static device buffer, so replays serve any set of scheduled requests without rebinding or copying state; the graph
    must be rebuilt only if the pools are reallocated or the model's modules change."""

    def __init__(self, pool: RWKV7StatePool, rows: int, greedy: bool):
        self.pool, self.rows = pool, int(rows)
        dev = pool.S_pool.device
        self.ids = torch.zeros(self.rows, device=dev, dtype=torch.long)
        self.slots = torch.full((self.rows,), pool.scratch_slot, device=dev, dtype=torch.int32)
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up on the scratch slot: lazy initialisations happen outside the capture
                pool._step(self.ids, self.slots, greedy)
        torch.cuda.current_stream(dev).wait_stream(stream)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = pool._step(self.ids, self.slots, greedy)

    def replay(self, ids, slot_vec):
        n = int(ids.numel())
        self.ids[:n].copy_(ids)
        if n < self.rows:
            self.ids[n:].zero_()
        self.slots.copy_(slot_vec)
        self.graph.replay()
        return self.out
