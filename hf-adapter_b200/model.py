"""RWKV-7 causal LM running on the CUDA library: the reference's model classes and entry points
(rwkv7_hf/native_model.py:371-853, model_layers.py, model_fast_api.py:58-265) with the same module
tree, parameter names and cache, so a reference ``state_dict`` loads unchanged.

Two execution paths, both made only of this package's kernels plus plain dense GEMMs:

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

from . import _lib
from . import lora as _lora
from . import norm_mix as _nm
from . import prep as _prep
from . import quant as _q
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


def _rkv_grouped(at, xr, xk, xv):
    """r / k / v through one grouped launch when all three are int4 projections of one shape that the tensor-core
    decode kernel takes; None otherwise."""
    mods = (at.r_proj, at.k_proj, at.v_proj)
    int4 = all(isinstance(m, _q.MM4Linear) for m in mods)
    int8 = all(isinstance(m, _q.MM8Linear) and m.sm7x_rowwise for m in mods)
    if not (int4 or int8) or any(m.bias is not None for m in mods):
        return None
    if len({(m.in_features, m.out_features) for m in mods}) != 1:
        return None
    tiled = [m.tiled_for(x_) for m, x_ in zip(mods, (xr, xk, xv))]
    if any(t is None for t in tiled):
        return None
    if int8:
        return _q.w8_tiled_linear_group((xr, xk, xv), tiled, [m.row_scale for m in mods], mods[0].out_features,
                                        mods[0].in_features)
    return _q.w4_tiled_linear_group((xr, xk, xv), tiled, mods[0].out_features, mods[0].in_features)


def _linear(mod, x, *, relu2=False, residual=None, out=None):
    """Apply a projection operand: a quantised module of this package (epilogues fused through its
    rwkv7_forward_* hooks, as the reference's dispatch probes them: native_jit_graph_dispatch.py:487-523)
    or a dense nn.Linear (one library GEMM)."""
    if isinstance(mod, (_q.MM4Linear, _q.MM8Linear, _q.A8W8Linear)):
        if relu2:
            if hasattr(mod, "rwkv7_forward_relu2"):
                return mod.rwkv7_forward_relu2(x)
            return torch.relu(mod(x)) ** 2
        if residual is not None:
            return mod.rwkv7_forward_add(x, residual)
        if out is not None:
            return mod.rwkv7_forward_into(x, out)
        return mod(x)
    y = F.linear(x, mod.weight, mod.bias)
    if relu2:
        y = torch.relu(y) ** 2
    elif residual is not None:
        y = y + residual
    if out is not None:
        out.copy_(y)
        return out
    return y


class RWKV7ForCausalLM(nn.Module):
    """``RWKV7ForCausalLM`` == the native model, as in the reference (rwkv7_hf/__init__.py:17-20)."""

    def __init__(self, config: NativeRWKV7Config, tp_world: int = 1, tp_rank: int = 0, tp_group=None,
                 state_dtype=torch.float32, tp_shard_head: bool = False, tp_overlap_rows: int = 0, tp_comm: str = "nccl"):
        """``state_dtype=torch.float16`` selects the reference's opt-in FP16-state lane (rwkv7_hf/native_wkv_fp16.py):
        caches hold the recurrent state in fp16 and the decode step dithers the decay; fp16 activations only.
        ``tp_shard_head``: every rank holds ``vocab/P`` rows of the head; full logits are all-gathered, greedy tokens
        come from a local arg-max and one tiny exchange.  ``tp_overlap_rows`` > 0: decode batches of at least twice
        that many rows run as two halves on two streams with their own communicators, so one half's all-reduces hide
        under the other half's kernels.  ``tp_comm``: "nccl" sums the partial outputs with the framework's all-reduce,
        "peer" with this library's one-kernel sum over peer-mapped memory (fp16, up to 1024 rows; larger calls use NCCL)."""
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
        if tp_comm not in ("nccl", "peer"):
            raise ValueError("tp_comm must be 'nccl' or 'peer'")
        self.tp_comm = tp_comm
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
        if self.tp_comm == "peer" and t.dtype == torch.float16 and t.is_contiguous() and rows <= self.PEER_MAX_ROWS:
            ar = self._peer_ar.get(lane)
            if ar is None or rows * int(t.shape[-1]) > ar.slot_elems or ar.width != int(t.shape[-1]):
                from .tp_comm import PeerAllReduce
                if torch.cuda.is_current_stream_capturing():
                    raise RuntimeError("the peer all-reduce buffers must exist before graph capture (run one eager step first)")
                ar = self._peer_ar[lane] = PeerAllReduce(self.tp_group, max(rows, 64), int(t.shape[-1]), t.device)
            return ar.all_reduce(t, out=t)
        torch.distributed.all_reduce(t, group=self._lane_group(lane))
        return t

    def _lane_group(self, lane: int):
        return self._tp_group_b if (lane and self._tp_group_b is not None) else self.tp_group

    def _head(self, xn, greedy: bool, lane: int = 0):
        """Final projection: logits ``[B,V]`` (all-gathered over the vocabulary shards when the head is sharded) or, with
        ``greedy``, the arg-max token of every row (local arg-max + one [B,2] exchange per rank)."""
        local = _linear(self.lm_head, xn)
        if not self.tp_shard_head or self.tp_group is False:
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

    def _decode_rows(self, ids, tensors, greedy, lane, stream_base):
        state, xpa, xpf, v_first, elapsed_t = tensors
        H, N = self.model.layers[0].attn.num_heads, self.config.head_dim
        x = F.embedding(ids.reshape(-1), self.model.embeddings.weight)
        B = int(x.shape[0])
        L = len(self.model.layers)
        elapsed = elapsed_t if state[0].dtype == torch.float16 else None
        for i, layer in enumerate(self.model.layers):
            at, ff = layer.attn, layer.ffn
            if i == 0:
                x = _nm.layer_norm(x, layer.pre_norm.weight, layer.pre_norm.bias)
            xr, xw, xk, xv, xa, xg = _nm.fused_attn_norm_mix6_decode(
                x, xpa[i], layer.attn_norm.weight, layer.attn_norm.bias, at.x_r, at.x_w, at.x_k, at.x_v, at.x_a, at.x_g)
            # The LoRA chain does not depend on r/k/v: it runs on a side stream (a parallel branch of the decode
            # graph once captured) and joins before the recurrence.
            main = torch.cuda.current_stream(x.device)
            side = self._side_stream(x.device, stream_base)
            side.wait_stream(main)
            wl, al, gl = at.w_lora.lora, at.a_lora.lora, at.g_lora.lora
            with torch.cuda.stream(side):
                if i == 0:
                    hs = _lora.small_gemm_group((xw, xa, xg), (wl[0].weight, al[0].weight, gl[0].weight), acts=(1, 0, 2))
                    w_raw, a_pre, g = _lora.small_gemm_group(hs, (wl[2].weight, al[2].weight, gl[2].weight))
                    extra = dict(v_out=v_first)
                else:
                    vl = at.v_lora.lora
                    hs = _lora.small_gemm_group((xw, xa, xg, xv), (wl[0].weight, al[0].weight, gl[0].weight, vl[0].weight),
                                                acts=(1, 0, 2, 0))
                    w_raw, a_pre, g, vg_pre = _lora.small_gemm_group(hs, (wl[2].weight, al[2].weight, gl[2].weight, vl[2].weight))
                    extra = dict(v_first=v_first, v_gate=vg_pre, v_gate_bias=vl[2].bias, v_gate_is_raw=True)
            rkv = _rkv_grouped(at, xr, xk, xv)
            if rkv is not None:
                # int4 r / k / v of equal shape: one launch streams all three weight sets (one pipeline fill, no
                # split-K exchange) instead of three launches competing for the SMs
                r, k, v = rkv
                main.wait_stream(side)
            else:
                # independent projections on separate branches: the tail of one overlaps the ramp-up of the next
                sk, sv = self._side_stream(x.device, stream_base + 1), self._side_stream(x.device, stream_base + 2)
                sk.wait_stream(main)
                sv.wait_stream(main)
                with torch.cuda.stream(sk):
                    k = _linear(at.k_proj, xk)
                with torch.cuda.stream(sv):
                    v = _linear(at.v_proj, xv)
                r = _linear(at.r_proj, xr)
                main.wait_stream(side)
                main.wait_stream(sk)
                main.wait_stream(sv)
                xk.record_stream(sk); k.record_stream(sk); xv.record_stream(sv); v.record_stream(sv)
            for t_ in (xw, xa, xg, xv, w_raw, a_pre, g):
                t_.record_stream(side)
            # the kernel launched just before the recurrence is a projection: it never writes the state
            out, _ = _rec.fused_recurrent_output_prepare_raw(
                r, w_raw, k, v, a_pre, state[i], g, at.k_k, at.k_a, at.r_k, at.g_norm.weight, at.g_norm.bias,
                eps=N * 1e-5, new_state=state[i], w_bias=wl[2].bias, a_bias=al[2].bias, a_is_raw=True,
                state_prefetch=True, elapsed=elapsed, advance_elapsed=elapsed is not None and i == L - 1, **extra)
            attn = self._all_reduce(_linear(at.o_proj, out), lane)
            x, mixed = _nm.fused_ffn_add_norm_mix_decode(x, attn, xpf[i], layer.ffn_norm.weight, layer.ffn_norm.bias, ff.x_k)
            hidden = _linear(ff.key, mixed, relu2=True)
            if self.tp_world > 1:
                # the residual rides in rank 0's partial sum (the projection's add epilogue): no extra add kernel
                x = self._all_reduce(_linear(ff.value, hidden, residual=x if self.tp_rank == 0 else None), lane)
            else:
                x = _linear(ff.value, hidden, residual=x)
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
            w_raw = F.linear(torch.tanh(F.linear(xw, wl[0].weight)), wl[2].weight, wl[2].bias)
            a_pre = F.linear(F.linear(xa, al[0].weight), al[2].weight, al[2].bias)
            g = F.linear(torch.sigmoid(F.linear(xg, gl[0].weight)), gl[2].weight)
            if i == 0:
                vf, vg = None, None
            else:
                vl = at.v_lora.lora
                vf, vg = v_first, F.linear(F.linear(xv, vl[0].weight), vl[2].weight, vl[2].bias)
            w, k, v, kk = _prep.fused_prefill_state_prep(
                w_raw, k_raw, v_raw, a_pre, at.k_k, at.k_a, v_first=vf, v_gate=vg, num_heads=H, head_dim=N,
                a_is_raw=True, v_gate_is_raw=True)
            if i == 0:
                v_first = v
            a_sig = torch.sigmoid(a_pre)
            if scan_chunk and T % scan_chunk == 0 and x.dtype == torch.float16:
                # the tensor-core scan carries an fp32 state; an fp16 cache is widened for the call and rounded back
                y, new_state = _rec.self_chunk_rwkv7(r, w, k, v, kk, a_sig, state[i].float(), chunk_size=scan_chunk)
                out = _prep.fused_attn_output_prepare(y, r, k, v, g, at.r_k, at.g_norm.weight, at.g_norm.bias,
                                                      num_heads=H, head_dim=N, head_v_dim=N, eps=N * 1e-5)
            else:
                out, new_state = _rec.fused_recurrent_scan_output_prepare(
                    r, w, k, v, kk, a_sig, state[i], g, at.r_k, at.g_norm.weight, at.g_norm.bias, eps=N * 1e-5)
            state[i].copy_(new_state)
            x = x + self._all_reduce(_linear(at.o_proj, out))
            h2 = _nm.layer_norm(x, layer.ffn_norm.weight, layer.ffn_norm.bias)
            mixed, nxt = _nm.fused_ffn_sequence_shift_mix(h2, xpf[i], ff.x_k)
            xpf[i].copy_(nxt)
            hidden = _linear(ff.key, mixed, relu2=True)
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

    @torch.no_grad()
    def forward(self, input_ids, past_key_values=None, use_cache=None, logits_to_keep: int = 0, **_):
        """HF-style forward (rwkv7_hf/native_model.py:618-783).  Returns an object with ``.logits``
        ``[B,T or keep,V]`` and ``.past_key_values`` (a NativeRWKV7Cache)."""
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        cache = NativeRWKV7Cache.from_legacy_cache(past_key_values) if past_key_values is not None else None
        if cache is None or not cache._is_initialized():
            cache = self.new_cache(int(input_ids.shape[0]))
        T = int(input_ids.shape[1])
        if T == 1:
            logits = self.rwkv7_forward_token(input_ids[:, 0], cache, use_graph=False)[:, None]
        else:
            logits, cache = self.rwkv7_prefill_native(input_ids, cache, logits_to_keep=logits_to_keep)
        return SimpleNamespace(logits=logits, past_key_values=cache if use_cache is not False else None)

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens: int = 16, do_sample: bool = False, use_graph: bool = True, **_):
        """Greedy generation: prefill, then one decode step per new token.  Returns ``[B, T + new]`` ids."""
        if do_sample:
            raise NotImplementedError("only greedy decoding is implemented")
        logits, cache = self.rwkv7_prefill_native(input_ids, None, logits_to_keep=1)
        tok = logits[:, -1].argmax(-1)
        out = [input_ids, tok[:, None]]
        for _ in range(int(max_new_tokens) - 1):
            tok = self.rwkv7_forward_token(tok, cache, use_graph=use_graph).argmax(-1)
            out.append(tok[:, None])
        return torch.cat(out, dim=1)

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
