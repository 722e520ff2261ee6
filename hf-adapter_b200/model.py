"""RWKV-7 causal LM running on the CUDA library: the reference's model classes and entry points
(rwkv7_hf/native_model.py:371-853, model_layers.py, model_fast_api.py:58-265) with the same module
tree, parameter names and cache, so a reference ``state_dict`` loads unchanged.

Two execution paths, both made of this package's kernels (dense projections over fewer than 64 rows, or in fp32, are plain
library GEMMs):

* ``_decode_step``: one token for B sequences, every buffer preallocated so the whole step can be
  captured in a CUDA graph (``DecodeGraph``), the role of NativeGraphRunner
  (rwkv7_hf/native_graph_runtime.py:212-711) and ``_block_ip_batched`` (native_jit_decode.py:481-901).
* ``_prefill``: layer-wise over ``[B,T]`` tokens, the role of ``_prefill_current_device_impl``
  (rwkv7_hf/native_jit_prefill.py:223-1057).

Head-sharded tensor parallelism: constructed with ``tp_world > 1`` each rank holds H/P heads of
r/k/v, the LoRA up-projections, the per-head parameters and the recurrent state, F/P of the FFN, and
sums the ``[B,D]`` partial outputs of ``o_proj`` and ``ffn.value`` with an all-reduce.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass
from types import SimpleNamespace

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import gemm as _gemm
from . import norm_mix as _nm
from . import packing as _pk
from . import prep as _prep
from . import recurrent as _rec
from . import sharding as _sh
from .cache import NativeRWKV7Cache


@dataclass
class NativeRWKV7Config:
    """Field names of rwkv7_hf/model_config.py:59-107."""
    vocab_size: int = 65536
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_heads: int = 12
    head_dim: int = 64
    intermediate_size: int = 3072
    decay_low_rank_dim: int = 64
    gate_low_rank_dim: int = 128
    a_low_rank_dim: int = 64
    v_low_rank_dim: int = 32
    use_cache: bool = True

    @property
    def attention_hidden_size(self) -> int:
        return self.num_heads * self.head_dim


class _LoRA(nn.Module):
    def __init__(self, input_size, low_rank, bias, output_size):
        super().__init__()
        self.lora = nn.Sequential(nn.Linear(input_size, low_rank, bias=False), nn.Identity(),
                                  nn.Linear(low_rank, output_size, bias=bias))


class NativeRWKV7Attention(nn.Module):
    def __init__(self, config, layer_idx, tp_world=1):
        super().__init__()
        self.layer_idx = layer_idx
        self.num_heads = config.num_heads // tp_world  # heads held by this rank
        self.head_dim = config.head_dim
        self.hidden_size = config.hidden_size
        hidden, A = config.hidden_size, self.num_heads * self.head_dim
        self.attention_hidden_size = A
        for p in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"):
            setattr(self, p, nn.Parameter(torch.zeros(1, 1, hidden)))
        self.k_k = nn.Parameter(torch.zeros(A))
        self.k_a = nn.Parameter(torch.zeros(A))
        self.r_k = nn.Parameter(torch.zeros(self.num_heads, self.head_dim))
        self.r_proj = nn.Linear(hidden, A, bias=False)
        self.k_proj = nn.Linear(hidden, A, bias=False)
        self.v_proj = nn.Linear(hidden, A, bias=False)
        self.o_proj = nn.Linear(A, hidden, bias=False)
        self.w_lora = _LoRA(hidden, config.decay_low_rank_dim, True, A)
        self.a_lora = _LoRA(hidden, config.a_low_rank_dim, True, A)
        self.g_lora = _LoRA(hidden, config.gate_low_rank_dim, False, A)
        if layer_idx != 0:
            self.v_lora = _LoRA(hidden, config.v_low_rank_dim, True, A)
        self.g_norm = nn.GroupNorm(self.num_heads, A, eps=self.head_dim * 1e-5)


class NativeRWKV7FFN(nn.Module):
    def __init__(self, config, tp_world=1):
        super().__init__()
        self.x_k = nn.Parameter(torch.zeros(config.hidden_size))
        self.key = nn.Linear(config.hidden_size, config.intermediate_size // tp_world, bias=False)
        self.value = nn.Linear(config.intermediate_size // tp_world, config.hidden_size, bias=False)


class NativeRWKV7Layer(nn.Module):
    def __init__(self, config, layer_idx, tp_world=1):
        super().__init__()
        self.attn = NativeRWKV7Attention(config, layer_idx, tp_world)
        self.ffn = NativeRWKV7FFN(config, tp_world)
        self.attn_norm = nn.LayerNorm(config.hidden_size)
        self.ffn_norm = nn.LayerNorm(config.hidden_size)
        if layer_idx == 0:
            self.pre_norm = nn.LayerNorm(config.hidden_size)


class NativeRWKV7Model(nn.Module):
    def __init__(self, config, tp_world=1):
        super().__init__()
        self.embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([NativeRWKV7Layer(config, i, tp_world) for i in range(config.num_hidden_layers)])
        self.norm = nn.LayerNorm(config.hidden_size)


_linear = _pk.apply_linear  # a projection module (quantised or dense) applied with its fused epilogue


def _validate_attention_mask(attention_mask, batch_size: int, seq_len: int, device=None, *, allow_trailing: bool = False):
    """The reference's mask contract (rwkv7_hf/model_backbone.py:28-61): ``[B,T]`` (a longer mask is cut to its last T
    columns when a cache exists), non-zero = token present; an all-ones mask is no mask."""
    if attention_mask is None:
        return None
    if not isinstance(attention_mask, torch.Tensor):
        raise TypeError("NativeRWKV7 attention_mask must be a torch.Tensor when provided")
    if attention_mask.dim() == 1:
        attention_mask = attention_mask.view(1, -1)
    if attention_mask.dim() != 2:
        raise ValueError("NativeRWKV7 attention_mask must be shaped [batch, seq]")
    if int(attention_mask.shape[0]) != int(batch_size):
        raise ValueError("NativeRWKV7 attention_mask batch size must match inputs")
    if int(attention_mask.shape[1]) != int(seq_len):
        if not allow_trailing or int(attention_mask.shape[1]) < int(seq_len):
            raise ValueError("NativeRWKV7 attention_mask must have the same [batch, seq] shape as inputs")
        attention_mask = attention_mask[:, -seq_len:]
    mask = attention_mask.to(device=device) if device is not None else attention_mask
    mask = mask[:, :seq_len] != 0
    if mask.numel() and bool(torch.all(mask)):
        return None
    return mask


def _resolve_logits_to_keep(logits_to_keep, num_logits_to_keep):
    keep = logits_to_keep if logits_to_keep is not None else num_logits_to_keep
    if keep is None:
        return None
    if isinstance(keep, torch.Tensor):
        raise NotImplementedError("logits_to_keep as an index tensor is not supported; pass the number of last tokens")
    keep = int(keep)
    if keep < 0:
        raise ValueError("logits_to_keep must be non-negative")
    return keep


def _causal_lm_output(logits, cache):
    """``transformers.modeling_outputs.CausalLMOutputWithPast`` when that package imports, else an object with the same
    two attributes (this library does not depend on transformers)."""
    try:
        from transformers.modeling_outputs import CausalLMOutputWithPast
    except Exception:  # pragma: no cover - transformers absent
        return SimpleNamespace(logits=logits, past_key_values=cache, loss=None, hidden_states=None, attentions=None)
    return CausalLMOutputWithPast(logits=logits, past_key_values=cache)


def sample_next_token(logits, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, generator=None):
    """One token per row of ``logits [B,V]`` from the temperature-scaled distribution restricted to the ``top_k`` most
    likely tokens and to the smallest set whose probability reaches ``top_p`` (the most likely token always stays)."""
    if temperature <= 0:
        return logits.argmax(-1)
    z = logits.float() / float(temperature)
    if top_k and 0 < int(top_k) < z.shape[-1]:
        kth = torch.topk(z, int(top_k), dim=-1).values[:, -1:]
        z = z.masked_fill(z < kth, float("-inf"))
    if top_p < 1.0:
        sz, idx = torch.sort(z, dim=-1, descending=True)
        pr = torch.softmax(sz, dim=-1)
        before = pr.cumsum(-1) - pr  # probability mass ahead of each token
        sz = sz.masked_fill(before >= float(top_p), float("-inf"))
        z = torch.full_like(z, float("-inf")).scatter(-1, idx, sz)
    return torch.multinomial(torch.softmax(z, dim=-1), 1, generator=generator).squeeze(-1)


class RWKV7ForCausalLM(nn.Module):
    """``RWKV7ForCausalLM`` == the native model, as in the reference (rwkv7_hf/__init__.py:17-20)."""

    def __init__(self, config: NativeRWKV7Config, tp_world: int = 1, tp_rank: int = 0, tp_group=None,
                 state_dtype=torch.float32, tp_shard_head: bool = False, tp_overlap_rows: int = 0, tp_comm: str = "nccl"):
        """``state_dtype=torch.float16`` selects the reference's opt-in FP16-state lane (rwkv7_hf/native_wkv_fp16.py):
        caches hold the recurrent state in fp16 and the decode step dithers the decay; fp16 activations only.
        ``tp_shard_head``: every rank holds ``vocab/P`` rows of the head; full logits are all-gathered, greedy tokens
        come from a local arg-max and one tiny exchange.  ``tp_overlap_rows`` > 0: decode batches of at least twice
        that many rows run as two halves on two streams with their own communicators, so one half's all-reduces hide
        under the other half's kernels (two library communicators are then in flight at once on every GPU: NCCL asks for
        ``NCCL_LAUNCH_ORDER_IMPLICIT=1``, or equal GPU-side order on all ranks, for that to be free of deadlock; with
        "peer_rows" the halves sum with the stand-alone kernel).
        ``tp_comm``: "nccl" sums the partial outputs with the framework's all-reduce,
        "peer" with this library's one-kernel sum over peer-mapped memory (fp16, up to 1024 rows; larger calls use NCCL),
        "peer_rows" moves the sums of a decode step into the LayerNorm / token-shift kernels that consume them (fp16 / bf16,
        up to 1024 rows; otherwise as "peer")."""
        super().__init__()
        if state_dtype not in (torch.float32, torch.float16):
            raise ValueError("state_dtype must be torch.float32 or torch.float16")
        self.state_dtype = state_dtype
        if config.head_dim != 64:
            raise ValueError("the CUDA kernels require head_dim == 64")
        if config.num_heads % tp_world or config.intermediate_size % tp_world:
            raise ValueError("num_heads and intermediate_size must be divisible by the tensor-parallel world size")
        self.config = config
        self.tp_world, self.tp_rank, self.tp_group = int(tp_world), int(tp_rank), tp_group
        self.model = NativeRWKV7Model(config, tp_world)
        self.tp_shard_head = bool(tp_shard_head) and self.tp_world > 1
        if self.tp_shard_head and config.vocab_size % self.tp_world:
            raise ValueError("vocab_size must be divisible by the tensor-parallel world size to shard the head")
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size // (self.tp_world if self.tp_shard_head else 1), bias=False)
        if tp_comm not in ("nccl", "peer", "peer_rows"):
            raise ValueError("tp_comm must be 'nccl', 'peer' or 'peer_rows'")
        self.tp_comm = tp_comm
        self._peer_rows = {}  # lane -> PeerRowSum (the sums taken inside the row kernels; same set-up rule)
        self._peer_ar = {}  # lane -> PeerAllReduce (created on first use: a collective set-up, outside graph capture)
        self.tp_overlap_rows = int(tp_overlap_rows) if self.tp_world > 1 else 0
        # the second half of an overlapped step needs a communicator of its own: two collectives of ONE communicator
        # launched from two graph branches may start in different orders on different ranks
        self._tp_group_b = None
        if self.tp_overlap_rows and tp_group not in (None, False):
            self._tp_group_b = torch.distributed.new_group(ranks=torch.distributed.get_process_group_ranks(tp_group))
        self._graphs = {}
        self._side_streams = {}

    # ------------------------------------------------------------------ helpers
    @property
    def device(self):
        return self.model.embeddings.weight.device

    @property
    def dtype(self):
        return self.model.embeddings.weight.dtype

    def new_cache(self, batch_size: int) -> NativeRWKV7Cache:
        c = self.config
        if self.state_dtype == torch.float16 and self.dtype != torch.float16:
            raise ValueError("the FP16-state lane needs fp16 activations")
        return NativeRWKV7Cache.allocate(c.num_hidden_layers, batch_size, c.hidden_size, c.num_heads // self.tp_world,
                                         c.head_dim, self.device, self.dtype, state_dtype=self.state_dtype)

    def _side_stream(self, device, index: int = 0):
        st = self._side_streams.get((device, index))
        if st is None:
            st = self._side_streams[(device, index)] = torch.cuda.Stream(device=device)
        return st

    PEER_MAX_ROWS = 1024

    def _all_reduce(self, t, lane: int = 0):
        """Sum ``t`` over the tensor-parallel ranks in place.  ``lane`` 1 is the second half of an overlapped step (its own
        communicator / peer buffers)."""
        # tp_group=False: one rank's share of the work without the collective (single-process timing of a shard)
        if self.tp_world == 1 or self.tp_group is False:
            return t
        rows = t.numel() // int(t.shape[-1])
        if self.tp_comm in ("peer", "peer_rows") and t.dtype == torch.float16 and t.is_contiguous() and rows <= self.PEER_MAX_ROWS:
            ar = self._peer_ar.get(lane)
            if ar is None or rows * int(t.shape[-1]) > ar.slot_elems or ar.width != int(t.shape[-1]):
                from .tp_comm import PeerAllReduce, keep_alive
                if torch.cuda.is_current_stream_capturing():
                    raise RuntimeError("the peer all-reduce buffers must exist before graph capture (run one eager step first)")
                # sized for the largest call once and kept by the process, not by the model: a buffer that other ranks
                # have mapped is never released while they run
                ar = self._peer_ar[lane] = keep_alive(PeerAllReduce(self.tp_group, self.PEER_MAX_ROWS, int(t.shape[-1]), t.device))
            return ar.all_reduce(t, out=t)
        torch.distributed.all_reduce(t, group=self._lane_group(lane))
        return t

    def _row_sum(self, partial, lane: int = 0):
        """The communicator whose row kernels sum ``partial [rows, D]`` over the ranks themselves, or None when the sum
        has to run as its own all-reduce (another ``tp_comm``, an unsupported width or dtype, more than 1024 rows; every
        rank decides alike because the answer depends on the shape alone)."""
        if self.tp_comm != "peer_rows" or self.tp_world == 1 or self.tp_group is False:
            return None
        if self.tp_overlap_rows:
            # Two half-batches side by side would run two of these kernels (and two library collectives at the end of
            # the step) at the same time on every GPU; that combination once stalled on two GPUs and stays off: the
            # halves sum with the stand-alone kernel.
            return None
        from .tp_comm import PeerRowSum
        rows, width = int(partial.shape[0]), int(partial.shape[1])
        if not partial.is_contiguous() or rows > self.PEER_MAX_ROWS or PeerRowSum.resident_rows(width, partial.dtype) <= 0:
            return None
        comm = self._peer_rows.get(lane)
        if comm is None or rows > comm.max_rows or comm.width != width or comm.dtype != partial.dtype:
            from .tp_comm import keep_alive
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the peer row-sum buffers must exist before graph capture (run one eager step first)")
            comm = self._peer_rows[lane] = keep_alive(PeerRowSum(self.tp_group, self.PEER_MAX_ROWS, width, partial.device,
                                                                 partial.dtype))
        return comm

    def _lane_group(self, lane: int):
        return self._tp_group_b if (lane and self._tp_group_b is not None) else self.tp_group

    def _head(self, xn, greedy: bool, lane: int = 0):
        """Final projection: logits ``[B,V]`` (all-gathered over the vocabulary shards when the head is sharded) or, with
        ``greedy``, the arg-max token of every row (local arg-max + one [B,2] exchange per rank)."""
        sharded = self.tp_shard_head and self.tp_group is not False
        w = self.lm_head.weight
        if greedy and _gemm.takes(xn, w) and int(xn.shape[0]) >= _gemm.MIN_ROWS:
            # the arg-max rides in the head GEMM's epilogue: the logits are never written
            if not sharded:
                return _gemm.dense_argmax(xn, w)
            idx, val = _gemm.dense_argmax(xn, w, return_values=True)
            return _sh.sharded_argmax(None, self.tp_rank, self.tp_world, self._lane_group(lane), local_best=(val, idx),
                                      shard_width=int(w.shape[0]))
        local = _linear(self.lm_head, xn)
        if not sharded:
            return local.argmax(-1) if greedy else local
        group = self._lane_group(lane)
        if greedy:
            return _sh.sharded_argmax(local, self.tp_rank, self.tp_world, group)
        rows = int(local.shape[0])
        parts = torch.empty((self.tp_world * rows, int(local.shape[1])), device=local.device, dtype=local.dtype)
        torch.distributed.all_gather_into_tensor(parts, local.contiguous(), group=group)  # rank-major concatenation
        return parts.view(self.tp_world, rows, -1).permute(1, 0, 2).reshape(rows, -1)

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def _decode_step(self, ids, cache: NativeRWKV7Cache, greedy: bool = False):
        """One token for every sequence; mutates the cache tensors in place.  Returns logits ``[B,V]`` (or the greedy
        tokens ``[B]``).  With ``tp_overlap_rows`` set and enough rows, the batch runs as two halves on two streams."""
        state, xpa, xpf, v_first = cache
        ids = ids.reshape(-1)
        B = int(ids.shape[0])
        if (self.tp_overlap_rows and B >= 2 * self.tp_overlap_rows and B % 2 == 0
                and (cache._elapsed is None or B % 8 == 0)):  # (a slice of the int32 counters must stay 16-byte aligned)
            dev = ids.device
            main, second = torch.cuda.current_stream(dev), self._side_stream(dev, 7)
            second.wait_stream(main)
            half = B // 2
            outs = []
            for hi, (lo, up) in enumerate(((0, half), (half, B))):
                view = ([t[lo:up] for t in state], [t[lo:up] for t in xpa], [t[lo:up] for t in xpf], v_first[lo:up],
                        None if cache._elapsed is None else cache._elapsed[lo:up])
                with torch.cuda.stream(second if hi else main):
                    outs.append(self._decode_rows(ids[lo:up], view, greedy, hi, 10 * hi))
            main.wait_stream(second)
            for o in outs:
                o.record_stream(main)
            return torch.cat(outs, 0)
        return self._decode_rows(ids, (state, xpa, xpf, v_first, cache._elapsed), greedy, 0, 0)

    def _decode_rows(self, ids, tensors, greedy, lane, stream_base, inputs_embeds=None):
        """The layers of one decode step, each run from its pack tuple (packing.block_ip_batched), then the head."""
        state, xpa, xpf, v_first, elapsed_t = tensors
        x = inputs_embeds if inputs_embeds is not None else F.embedding(ids.reshape(-1), self.model.embeddings.weight)
        elapsed = elapsed_t if state[0].dtype == torch.float16 else None
        ctx = _pk.StepContext(self._side_stream, self._all_reduce, self.tp_world, self.tp_rank, lane, stream_base,
                              row_sum=self._row_sum)
        packs, _, _, _ = _pk.extract_graph_packs(self)
        x, *_ = _pk.step_batched(self, x, state, xpa, xpf, v_first, packs, fp16_elapsed=elapsed, context=ctx)
        xn = _nm.layer_norm(x, self.model.norm.weight, self.model.norm.bias)
        return self._head(xn, greedy, lane)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def _prefill(self, ids, cache: NativeRWKV7Cache, keep: int = 1, scan_chunk: int = 0):
        """Layer-wise prefill of ``ids [B,T]`` continuing from ``cache`` (mutated in place).
        Returns logits for the last ``keep`` tokens ``[B,keep,V]``."""
        state, xpa, xpf, v_first_buf = cache
        H, N = self.model.layers[0].attn.num_heads, self.config.head_dim
        B, T = (int(v) for v in ids.shape)
        x = F.embedding(ids, self.model.embeddings.weight)  # [B,T,D]
        v_first = None
        for i, layer in enumerate(self.model.layers):
            at, ff = layer.attn, layer.ffn
            if i == 0:
                x = _nm.layer_norm(x, layer.pre_norm.weight, layer.pre_norm.bias)
            h = _nm.layer_norm(x, layer.attn_norm.weight, layer.attn_norm.bias)
            xr, xw, xk, xv, xa, xg, nxt = _nm.fused_attn_sequence_shift_mix(
                h, xpa[i], at.x_r, at.x_w, at.x_k, at.x_v, at.x_a, at.x_g)
            xpa[i].copy_(nxt)
            r = _linear(at.r_proj, xr)
            k_raw = _linear(at.k_proj, xk)
            v_raw = _linear(at.v_proj, xv)
            wl, al, gl = at.w_lora.lora, at.a_lora.lora, at.g_lora.lora
            # the rank-R LoRA pairs: dense GEMMs of this library (bias in the epilogue), the activation between them pointwise
            w_raw = _linear(wl[2], torch.tanh(_linear(wl[0], xw)))
            a_pre = _linear(al[2], _linear(al[0], xa))
            g = _linear(gl[2], torch.sigmoid(_linear(gl[0], xg)))
            if i == 0:
                vf, vg = None, None
            else:
                vl = at.v_lora.lora
                vf, vg = v_first, _linear(vl[2], _linear(vl[0], xv))
            a_sig = torch.sigmoid(a_pre)
            chunked = bool(scan_chunk) and T % scan_chunk == 0 and x.dtype == torch.float16
            if chunked:
                # the tensor-core scan forms the decay from the raw logits itself: no decay tensor is written or read.
                # It carries an fp32 state; an fp16 cache is widened for the call and rounded back
                k, v, kk = _prep.fused_prefill_kv_kk_prep(k_raw, v_raw, a_pre, at.k_k, at.k_a, v_first=vf, v_gate=vg, num_heads=H,
                                                          head_dim=N, a_is_raw=True, v_gate_is_raw=True)
                y, new_state = _rec.self_chunk_rwkv7(r, w_raw, k, v, kk, a_sig, state[i].float(), chunk_size=scan_chunk, w_is_raw=True)
                out = _prep.fused_attn_output_prepare(y, r, k, v, g, at.r_k, at.g_norm.weight, at.g_norm.bias,
                                                      num_heads=H, head_dim=N, head_v_dim=N, eps=N * 1e-5)
            else:
                w, k, v, kk = _prep.fused_prefill_state_prep(
                    w_raw, k_raw, v_raw, a_pre, at.k_k, at.k_a, v_first=vf, v_gate=vg, num_heads=H, head_dim=N,
                    a_is_raw=True, v_gate_is_raw=True)
                out, new_state = _rec.fused_recurrent_scan_output_prepare(
                    r, w, k, v, kk, a_sig, state[i], g, at.r_k, at.g_norm.weight, at.g_norm.bias, eps=N * 1e-5)
            if i == 0:
                v_first = v
            state[i].copy_(new_state)
            if self.tp_world == 1:
                x = _linear(at.o_proj, out, residual=x)  # the residual add rides in the projection's epilogue
            else:
                x = x + self._all_reduce(_linear(at.o_proj, out))
            h2 = _nm.layer_norm(x, layer.ffn_norm.weight, layer.ffn_norm.bias)
            mixed, nxt = _nm.fused_ffn_sequence_shift_mix(h2, xpf[i], ff.x_k)
            xpf[i].copy_(nxt)
            hidden = _linear(ff.key, mixed, relu2=True)
            if self.tp_world == 1:
                x = _linear(ff.value, hidden, residual=x)
            else:
                x = x + self._all_reduce(_linear(ff.value, hidden))
        if v_first is not None:
            v_first_buf.copy_(v_first[:, -1])
        cache._seen_tokens += T
        if cache._elapsed is not None:
            cache._elapsed += T
        xn = _nm.layer_norm(x[:, T - keep:].contiguous(), self.model.norm.weight, self.model.norm.bias)
        return self._head(xn.reshape(B * keep, -1), False).reshape(B, keep, -1)

    # ------------------------------------------------------------------ reference-facing API
    @torch.no_grad()
    def rwkv7_forward_token(self, token_ids, cache: NativeRWKV7Cache, *, use_graph: bool = True, return_tokens: bool = False):
        """One decode token per sequence (rwkv7_hf/model_fast_api.py:190-244).  Returns logits ``[B,V]``, or with
        ``return_tokens`` the greedy next tokens ``[B]`` (the head's arg-max inside the step: with a vocabulary-sharded
        head no rank ever holds, or exchanges, the full logits)."""
        ids = token_ids.reshape(-1)
        if use_graph:
            g = self._decode_graph(int(ids.shape[0]), bool(return_tokens))
            logits = g.replay(ids, cache)
        else:
            logits = self._decode_step(ids, cache, greedy=bool(return_tokens))
        cache._seen_tokens += 1
        return logits

    @torch.no_grad()
    def rwkv7_prefill_native(self, input_ids, cache=None, *, logits_to_keep: int = 1, scan_chunk: int = 0):
        """Layer-wise prefill (rwkv7_hf/model_fast_api.py:58-94).  Returns ``(logits [B,keep,V], cache)``."""
        if input_ids.dim() != 2 or int(input_ids.shape[1]) < 1:
            raise ValueError("input_ids must be [batch, tokens] with at least one token")
        if cache is None:
            cache = self.new_cache(int(input_ids.shape[0]))
        keep = int(input_ids.shape[1]) if logits_to_keep in (0, None) else min(int(logits_to_keep), int(input_ids.shape[1]))
        return self._prefill(input_ids, cache, keep=keep, scan_chunk=scan_chunk), cache

    @torch.no_grad()
    def rwkv7_prefill_chunks(self, input_ids, cache=None, *, chunk_size: int = 512, scan_chunk: int = 0):
        """Long prompts: prefill in ``chunk_size`` slices carrying the cache (rwkv7_hf/model_fast_api.py:96-149)."""
        if chunk_size <= 0:
            raise ValueError("chunk_size must be positive")
        logits = None
        for t0 in range(0, int(input_ids.shape[1]), int(chunk_size)):
            logits, cache = self.rwkv7_prefill_native(input_ids[:, t0:t0 + chunk_size], cache, logits_to_keep=1,
                                                      scan_chunk=scan_chunk)
        return logits, cache

    # ------------------------------------------------------------------ Hugging Face surface
    def _masked_run(self, input_ids, inputs_embeds, mask, cache, keep: int):
        """Token-by-token advance for inputs the layer-wise prefill does not take: embeddings instead of ids, or an
        attention mask with holes.  Rows whose mask is 0 at a token keep their recurrent state, shift states and
        ``v_first``, and repeat their previous final hidden state (rwkv7_hf/native_model.py:555-590,
        model_backbone.py:64-75).  Returns logits for the last ``keep`` tokens ``[B,keep,V]``."""
        B = int(input_ids.shape[0] if input_ids is not None else inputs_embeds.shape[0])
        T = int(input_ids.shape[1] if input_ids is not None else inputs_embeds.shape[1])
        logits, last = [], None
        state, xpa, xpf, v_first = cache
        tensors = (state, xpa, xpf, v_first, cache._elapsed)
        for t in range(T):
            m = None if mask is None else mask[:, t]
            if m is not None:
                old = [v.clone() for v in cache._tensors()]
            ids_t = None if input_ids is None else input_ids[:, t]
            emb_t = None if inputs_embeds is None else inputs_embeds[:, t].contiguous()
            lg = self._decode_rows(ids_t, tensors, False, 0, 0, inputs_embeds=emb_t)
            if m is not None:
                for new_t, old_t in zip(cache._tensors(), old):
                    new_t.copy_(torch.where(m.view(-1, *([1] * (new_t.dim() - 1))), new_t, old_t))
                # a masked row repeats its previous logits (zeros before its first token: the head of a zero vector)
                lg = torch.where(m.view(-1, 1), lg, last if last is not None else torch.zeros_like(lg))
            last = lg
            if t >= T - keep:
                logits.append(lg)
        cache._seen_tokens += T
        return torch.stack(logits, dim=1)

    @torch.no_grad()
    def forward(self, input_ids=None, attention_mask=None, inputs_embeds=None, past_key_values=None, use_cache=None,
                output_hidden_states=None, output_attentions=None, return_dict=None, labels=None, logits_to_keep=None,
                num_logits_to_keep=None, position_ids=None, cache_position=None, token_type_ids=None, head_mask=None,
                return_legacy_cache=None, **kwargs):
        """The reference's ``NativeRWKV7ForCausalLM.forward`` for inference (rwkv7_hf/native_model.py:618-853): same
        arguments, same validation messages, ``CausalLMOutputWithPast(logits, past_key_values)`` out (a tuple with
        ``return_dict=False``; a legacy tuple cache with ``return_legacy_cache``).

        Without a cache the logits of every prompt token are returned unless ``logits_to_keep`` asks for the last n;
        with one, a single token takes the decode step (CUDA graph) and a longer continuation the layer-wise
        prefill.  ``attention_mask`` rows that are 0 leave that sequence's recurrent state untouched.  Training
        (``labels``), per-layer hidden states and attention maps are outside this library."""
        if labels is not None:
            raise NotImplementedError("training through labels is not part of this inference library")
        if output_hidden_states:
            raise NotImplementedError("per-layer hidden states are not kept by the fused kernels")
        if output_attentions:
            raise NotImplementedError("NativeRWKV7 does not expose Transformer-style attention maps")
        if input_ids is not None and inputs_embeds is not None:
            raise ValueError("NativeRWKV7ForCausalLM accepts either input_ids or inputs_embeds, not both")
        if input_ids is None and inputs_embeds is None:
            raise ValueError("NativeRWKV7ForCausalLM requires input_ids or inputs_embeds")
        if input_ids is not None and input_ids.dim() == 1:
            input_ids = input_ids.view(1, -1)
        if input_ids is not None and input_ids.dim() != 2:
            raise ValueError("Experimental NativeRWKV7ForCausalLM expects input_ids shaped [batch, seq]")
        if inputs_embeds is not None:
            if inputs_embeds.dim() != 3:
                raise ValueError("NativeRWKV7ForCausalLM expects inputs_embeds shaped [batch, seq, hidden]")
            if int(inputs_embeds.shape[-1]) != int(self.config.hidden_size):
                raise ValueError("NativeRWKV7ForCausalLM inputs_embeds last dimension must match hidden_size")
        B = int(input_ids.shape[0] if input_ids is not None else inputs_embeds.shape[0])
        T = int(input_ids.shape[1] if input_ids is not None else inputs_embeds.shape[1])
        if B <= 0 or T <= 0:
            raise ValueError("NativeRWKV7ForCausalLM requires a non-empty batch and sequence")
        cache = NativeRWKV7Cache.from_legacy_cache(past_key_values) if past_key_values is not None else None
        had_cache = cache is not None and cache._is_initialized()
        if had_cache and cache.get_batch_size() != B:
            raise ValueError(f"NativeRWKV7 cache batch size {cache.get_batch_size()} does not match input batch size {B}")
        if not had_cache:
            cache = self.new_cache(B)
        mask = _validate_attention_mask(attention_mask, B, T, self.device, allow_trailing=had_cache)
        keep = _resolve_logits_to_keep(logits_to_keep, num_logits_to_keep)
        keep_n = T if keep in (None, 0) else min(int(keep), T)
        if not had_cache and keep in (None,):
            keep_n = T  # full forward: all-token logits, Hugging Face CausalLM semantics
        if inputs_embeds is not None or mask is not None:
            logits = self._masked_run(input_ids, inputs_embeds, mask, cache, keep_n)
        elif T == 1:
            logits = self.rwkv7_forward_token(input_ids[:, 0], cache, use_graph=bool(kwargs.get("use_graph", True)))[:, None]
        else:
            logits, cache = self.rwkv7_prefill_native(input_ids, cache, logits_to_keep=keep_n)
        new_cache = cache if (use_cache is None or use_cache) else None
        if new_cache is not None and (return_legacy_cache or (return_legacy_cache is None and isinstance(past_key_values, tuple))):
            new_cache = new_cache.to_legacy_cache()
        if return_dict is not None and not return_dict:
            return tuple(v for v in (logits, new_cache) if v is not None)
        return _causal_lm_output(logits, new_cache)

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, inputs_embeds=None, token_type_ids=None,
                                      head_mask=None, return_legacy_cache=None, **kwargs):
        """What a generation loop feeds ``forward`` next (rwkv7_hf/model_generation.py:53-110): with a cache only the
        last token (and the last column of the mask) is passed on."""
        cache = NativeRWKV7Cache.from_legacy_cache(past_key_values) if past_key_values is not None else None
        has = cache is not None and cache._is_initialized()
        last = lambda t: t[:, -1:] if t is not None else None
        inputs = {}
        if has:
            if input_ids is not None:
                inputs["input_ids"] = last(input_ids)
            elif inputs_embeds is not None:
                inputs["inputs_embeds"] = last(inputs_embeds)
        elif inputs_embeds is not None:
            inputs["inputs_embeds"] = inputs_embeds
        else:
            inputs["input_ids"] = input_ids
        inputs["past_key_values"] = past_key_values
        inputs["use_cache"] = True if kwargs.get("use_cache") is None else kwargs["use_cache"]
        if return_legacy_cache is not None:
            inputs["return_legacy_cache"] = return_legacy_cache
        if kwargs.get("attention_mask") is not None:
            inputs["attention_mask"] = last(kwargs["attention_mask"]) if has else kwargs["attention_mask"]
        for name in ("logits_to_keep", "num_logits_to_keep", "return_dict"):
            if name in kwargs:
                inputs[name] = kwargs[name]
        return inputs

    def _reorder_cache(self, past_key_values, beam_idx):
        """Beam-search reordering of the batch rows of a cache (rwkv7_hf/model_generation.py:25-50)."""
        cache = NativeRWKV7Cache.from_legacy_cache(past_key_values)
        out = cache.select_batch(beam_idx)
        return out.to_legacy_cache() if isinstance(past_key_values, tuple) else out

    @torch.no_grad()
    def generate(self, input_ids=None, attention_mask=None, max_new_tokens: int = 16, do_sample: bool = False,
                 temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, eos_token_id=None, pad_token_id: int = 0,
                 use_graph: bool = True, generator=None, inputs=None, **_):
        """Prefill, then one decode step per new token; returns ``[B, T + new]`` ids.  Greedy by default (the head's
        arg-max runs inside the decode graph); ``do_sample`` draws from the temperature / top-k / top-p filtered
        distribution on the device.  A left-padded batch passes its ``attention_mask``: padded positions leave the
        state untouched.  Sequences that produced ``eos_token_id`` are filled with ``pad_token_id``."""
        if input_ids is None:
            input_ids = inputs
        if input_ids.dim() == 1:
            input_ids = input_ids.view(1, -1)
        B = int(input_ids.shape[0])
        n_new = int(max_new_tokens)
        if n_new <= 0:
            return input_ids
        out = self.forward(input_ids, attention_mask=attention_mask, logits_to_keep=1)
        cache, logits = out.past_key_values, out.logits[:, -1]
        eos = None
        if eos_token_id is not None:
            eos = torch.as_tensor([eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id), device=input_ids.device)
        done = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
        toks = []
        for step in range(n_new):
            if step:
                if do_sample:
                    logits = self.rwkv7_forward_token(tok, cache, use_graph=use_graph)
                else:
                    logits = None
                    tok = self.rwkv7_forward_token(tok, cache, use_graph=use_graph, return_tokens=True)
            if do_sample:
                tok = sample_next_token(logits, temperature=temperature, top_k=top_k, top_p=top_p, generator=generator)
            elif logits is not None:
                tok = logits.argmax(-1)
            if eos is not None:
                tok = torch.where(done, torch.full_like(tok, int(pad_token_id)), tok)
                done = done | torch.isin(tok, eos)
            toks.append(tok[:, None])
            if eos is not None and step + 1 < n_new and bool(done.all()):
                break
        return torch.cat([input_ids] + toks, dim=1)

    def rwkv7_speculative_generate(self, input_ids, draft_model, max_new_tokens: int = 32, draft_tokens: int = 4,
                                   eos_token_id=None, return_stats: bool = False, logits_to_keep: int = 1, **forward_kwargs):
        """Greedy speculative decoding with ``draft_model`` proposing (rwkv7_hf/model_speculative.py:10-231); the result
        equals this model's own greedy continuation.  See ``speculative.rwkv7_speculative_generate``."""
        from .speculative import rwkv7_speculative_generate
        return rwkv7_speculative_generate(self, input_ids, draft_model, max_new_tokens, draft_tokens, eos_token_id,
                                          return_stats, logits_to_keep, **forward_kwargs)

    # ------------------------------------------------------------------ CUDA graph
    def _decode_graph(self, batch: int, greedy: bool = False) -> "DecodeGraph":
        key = (batch, True) if greedy else batch
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = DecodeGraph(self, batch, greedy)
        return g


class DecodeGraph:
    """Fixed-batch CUDA graph of one decode step with its own static cache buffers.

    Binding protocol of the reference runner (rwkv7_hf/native_graph_runtime.py:618-660): a cache that is
    not yet backed by this runner's buffers is copied in once and then re-pointed at them, so later
    replays touch no host-side copies.  Only one cache can alias the buffers at a time: when another
    cache binds, the one bound before gets its own copies of the buffers back and loses its binding
    (``_detach_bound_cache_if_different`` in the reference), so two caches of the same batch size can be
    stepped alternately through one graph.  ``replay`` returns a copy of the static logits buffer unless
    ``copy_logits=False`` (the reference's default is to copy too)."""

    def __init__(self, model: RWKV7ForCausalLM, batch: int, greedy: bool = False):
        self.model, self.batch, self.greedy = model, batch, greedy
        dev = model.device
        self.ids = torch.zeros((batch,), device=dev, dtype=torch.long)
        self.cache = model.new_cache(batch)
        self.launches = 0
        self._bound = None  # weak reference to the cache whose tensors are this runner's static buffers
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up outside capture (allocator, lazy module loading)
                model._decode_step(self.ids, self.cache, greedy)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.cache.reset()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = model._decode_step(self.ids, self.cache, greedy)

    def _static(self):
        return self.cache._tensors()

    def _detach_bound(self):
        """Give the cache bound so far its own copies of the static buffers and drop its binding."""
        old = self._bound() if self._bound is not None else None
        self._bound = None
        if old is None or old._graph_owner is not self:
            return
        old._set_tensors([t.clone() for t in self._static()])
        old._graph_owner = None

    def bind(self, cache: NativeRWKV7Cache):
        if cache._graph_owner is self and self._bound is not None and self._bound() is cache:
            return
        self._detach_bound()
        mine, theirs = self._static(), cache._tensors()
        if len(mine) != len(theirs) or any(a.dtype != b.dtype for a, b in zip(mine, theirs)):
            raise ValueError("the cache does not match this model's state dtype")
        for dst, src in zip(mine, theirs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        cache._set_tensors(list(mine))
        cache._graph_owner = self
        self._bound = weakref.ref(cache)

    def replay(self, ids, cache: NativeRWKV7Cache, *, copy_logits: bool = True):
        self.bind(cache)
        self.ids.copy_(ids)
        self.graph.replay()
        return self.logits.clone() if copy_logits else self.logits


class PrefillGraph:
    """Fixed-shape CUDA graph of the layer-wise prefill of one prompt chunk ``[batch, tokens]`` (the role of the
    reference's prefill graph runner, rwkv7_hf/model_prefill_graph.py): for short chunks and small batches the
    hundred-odd launches per layer cost more host time than device time, and a replay removes it.

    The graph owns static ids and a static cache.  ``replay`` copies the caller's cache in, replays, and copies the
    advanced state back (a few MB against a whole chunk of work), so any cache of the right batch size can be served;
    consecutive chunks of one prompt pass the same cache object, which skips the copy-in."""

    def __init__(self, model: RWKV7ForCausalLM, batch: int, tokens: int, *, logits_to_keep: int = 1, scan_chunk: int = 0):
        self.model, self.batch, self.tokens = model, int(batch), int(tokens)
        self.keep = self.tokens if logits_to_keep in (0, None) else min(int(logits_to_keep), self.tokens)
        dev = model.device
        self.ids = torch.zeros((self.batch, self.tokens), device=dev, dtype=torch.long)
        self.cache = model.new_cache(self.batch)
        self._last = None  # weak reference to the cache whose state the static buffers currently hold
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                model._prefill(self.ids, self.cache, keep=self.keep, scan_chunk=scan_chunk)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.cache.reset()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = model._prefill(self.ids, self.cache, keep=self.keep, scan_chunk=scan_chunk)
        self.cache.reset()

    @torch.no_grad()
    def replay(self, input_ids, cache: NativeRWKV7Cache | None = None):
        """Advance ``cache`` (a fresh one when None) over ``input_ids [batch, tokens]``; returns ``(logits, cache)``."""
        if tuple(input_ids.shape) != (self.batch, self.tokens):
            raise ValueError(f"this graph was captured for input_ids [{self.batch}, {self.tokens}]")
        if cache is None:
            cache = self.model.new_cache(self.batch)
        mine, theirs = self.cache._tensors(), cache._tensors()
        if len(mine) != len(theirs) or any(a.shape != b.shape or a.dtype != b.dtype for a, b in zip(mine, theirs)):
            raise ValueError("the cache does not match the captured batch size or state dtype")
        if self._last is None or self._last() is not cache or cache._seen_tokens != self._seen_after:
            for dst, src in zip(mine, theirs):
                dst.copy_(src)
        self.ids.copy_(input_ids)
        self.graph.replay()
        for dst, src in zip(theirs, mine):
            dst.copy_(src)
        cache._seen_tokens += self.tokens
        self._last, self._seen_after = weakref.ref(cache), cache._seen_tokens
        return self.logits.clone(), cache
