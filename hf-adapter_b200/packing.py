"""The per-layer pack tuple of the reference's graph decode path and the in-place layer step that consumes it.

The reference flattens every layer into a 41-slot tuple (rwkv7_hf/native_jit_packing.py:13-146) that its
``_block_ip_batched`` (rwkv7_hf/native_jit_decode.py:481-901) unpacks:

    0 i, 1 H, 2 N, 3 eps (= N * 1e-5), 4 has_pre, 5-6 pre_norm w/b, 7-8 attn_norm w/b, 9-10 ffn_norm w/b,
    11-16 x_r x_w x_k x_v x_a x_g [D], 17 k_k [A], 18 k_a [A], 19 r_k [H,N],
    20-23 Rw Kw Vw Ow, 24-26 w1 w2 w0, 27-29 a1 a2 a0, 30-32 v1 v2 v0 (layer 0: zero dummies), 33-34 g1 g2,
    35-36 g_norm w/b [A], 37 fx_k [D], 38 fK, 39 fV, 40 RKVw ([3,D,A] stacked dense r/k/v, or empty)

A projection slot holds the dense ``[out,in]`` weight tensor of an ``nn.Linear`` or, for a quantised projection,
the module itself as a callable operand whose ``rwkv7_forward_*`` hooks carry the fused epilogues.  This file
builds that tuple from a model of this package (``extract_graph_packs``) and runs one layer from it
(``block_ip_batched``): the model's own decode step is a loop over these calls, so a host that already holds
reference packs drives the same kernels through the same structure.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import gemm as _gemm
from . import lora as _lora
from . import norm_mix as _nm
from . import quant as _q
from . import recurrent as _rec

PACK_SLOTS = 41
_QUANT_TYPES = (_q.MM4Linear, _q.MM8Linear, _q.A8W8Linear)


def graph_linear_operand(mod):
    """What a projection contributes to the pack: a quantised module stays a callable operand, a dense
    ``nn.Linear`` without bias is its weight tensor (rwkv7_hf/native_jit_graph_dispatch.py graph_linear_operand)."""
    if isinstance(mod, _QUANT_TYPES):
        return mod
    if isinstance(mod, nn.Linear) and mod.bias is None:
        return mod.weight
    return mod


def graph_linear_is_dense(op) -> bool:
    return isinstance(op, torch.Tensor)


def extract_graph_packs(model, *, rkv_policy: str = ""):
    """``(packs, H, N, eps)`` for ``model`` (rwkv7_hf/native_jit_packing.py:61-146).  ``rkv_policy="vkwr_auto"`` stacks
    dense r/k/v weights into slot 40; any other value leaves that slot empty."""
    layers = model.model.layers
    H = int(layers[0].attn.num_heads)
    N = int(layers[0].attn.head_dim)
    eps = float(N * 1e-5)
    emb = model.model.embeddings.weight
    hidden = int(emb.shape[1])
    A = H * N
    packs = []
    for i, layer in enumerate(layers):
        a = layer.attn
        vl = getattr(a, "v_lora", None)
        if vl is not None:
            v1, v2, v0 = graph_linear_operand(vl.lora[0]), vl.lora[2].weight, vl.lora[2].bias
        else:
            v1 = torch.zeros(1, hidden, device=emb.device, dtype=emb.dtype)
            v2 = torch.zeros(A, 1, device=emb.device, dtype=emb.dtype)
            v0 = torch.zeros(A, device=emb.device, dtype=emb.dtype)
        if hasattr(layer, "pre_norm"):
            pre_w, pre_b, has_pre = layer.pre_norm.weight, layer.pre_norm.bias, 1
        else:
            pre_w = torch.zeros(hidden, device=emb.device, dtype=emb.dtype)
            pre_b = torch.zeros(hidden, device=emb.device, dtype=emb.dtype)
            has_pre = 0
        r_op, k_op, v_op = (graph_linear_operand(m) for m in (a.r_proj, a.k_proj, a.v_proj))
        if rkv_policy == "vkwr_auto" and all(graph_linear_is_dense(o) for o in (r_op, k_op, v_op)):
            stacked = torch.stack((r_op.t(), k_op.t(), v_op.t())).contiguous()
        else:
            stacked = emb.new_empty((0,))
        packs.append((
            i, H, N, eps, has_pre,
            pre_w, pre_b, layer.attn_norm.weight, layer.attn_norm.bias,
            layer.ffn_norm.weight, layer.ffn_norm.bias,
            a.x_r.reshape(-1), a.x_w.reshape(-1), a.x_k.reshape(-1),
            a.x_v.reshape(-1), a.x_a.reshape(-1), a.x_g.reshape(-1),
            a.k_k, a.k_a, a.r_k,
            r_op, k_op, v_op, graph_linear_operand(a.o_proj),
            graph_linear_operand(a.w_lora.lora[0]), a.w_lora.lora[2].weight, a.w_lora.lora[2].bias,
            graph_linear_operand(a.a_lora.lora[0]), a.a_lora.lora[2].weight, a.a_lora.lora[2].bias,
            v1, v2, v0,
            graph_linear_operand(a.g_lora.lora[0]), a.g_lora.lora[2].weight,
            a.g_norm.weight, a.g_norm.bias,
            layer.ffn.x_k,
            graph_linear_operand(layer.ffn.key), graph_linear_operand(layer.ffn.value),
            stacked,
        ))
    return packs, H, N, eps


def init_batched_from_packs(packs, batch_size: int, device, dtype, *, state_dtype=None):
    """Zero recurrent buffers for ``batch_size`` sequences (rwkv7_hf/native_jit_packing.py:163-182):
    ``(state, xpa, xpf)`` lists with one ``[B,H,N,N]`` / ``[B,D]`` / ``[B,D]`` tensor per layer."""
    n = len(packs)
    H, N = int(packs[0][1]), int(packs[0][2])
    hid = int(packs[0][7].numel())
    if state_dtype is None:
        state_dtype = torch.float32
    state = [torch.zeros(batch_size, H, N, N, device=device, dtype=state_dtype) for _ in range(n)]
    xpa = [torch.zeros(batch_size, hid, device=device, dtype=dtype) for _ in range(n)]
    xpf = [torch.zeros(batch_size, hid, device=device, dtype=dtype) for _ in range(n)]
    return state, xpa, xpf


# ---------------------------------------------------------------------------------------------- operands
def apply_linear(op, x, *, relu2=False, residual=None, out=None):
    """Apply a projection operand of the pack: a quantised module (epilogues fused through its rwkv7_forward_* hooks,
    as the reference's dispatch probes them: rwkv7_hf/native_jit_graph_dispatch.py:487-523), a dense ``[out,in]``
    weight tensor, or an ``nn.Linear`` (this library's GEMM from 64 rows up in fp16 / bf16, else one library GEMM)."""
    if isinstance(op, _QUANT_TYPES):
        if relu2:
            if hasattr(op, "rwkv7_forward_relu2"):
                return op.rwkv7_forward_relu2(x)
            return torch.relu(op(x)) ** 2
        if residual is not None:
            return op.rwkv7_forward_add(x, residual)
        if out is not None:
            return op.rwkv7_forward_into(x, out)
        return op(x)
    weight, bias = (op, None) if isinstance(op, torch.Tensor) else (op.weight, op.bias)
    rows = x.numel() // int(x.shape[-1])
    if rows >= _gemm.MIN_ROWS and _gemm.takes(x, weight) and (bias is None or bias.dtype == x.dtype):
        # many rows over a dense fp16 / bf16 weight: this library's tensor-core GEMM, epilogue fused
        return _gemm.dense_linear(x, weight, bias, relu2=relu2, residual=residual, out=out)
    y = F.linear(x, weight, bias)
    if relu2:
        y = torch.relu(y) ** 2
    elif residual is not None:
        y = y + residual
    if out is not None:
        out.copy_(y)
        return out
    return y


def _weight_of(op):
    return op if isinstance(op, torch.Tensor) else op.weight


def rkv_grouped(ops, xr, xk, xv):
    """r / k / v through one grouped launch when all three are int4 (or row-wise int8) projections of one shape that
    the tensor-core decode kernel takes; None otherwise."""
    int4 = all(isinstance(m, _q.MM4Linear) for m in ops)
    int8 = all(isinstance(m, _q.MM8Linear) and m.sm7x_rowwise for m in ops)
    if not (int4 or int8) or any(m.bias is not None for m in ops):
        return None
    if len({(m.in_features, m.out_features) for m in ops}) != 1:
        return None
    tiled = [m.tiled_for(x_) for m, x_ in zip(ops, (xr, xk, xv))]
    if any(t is None for t in tiled):
        return None
    if int8:
        return _q.w8_tiled_linear_group((xr, xk, xv), tiled, [m.row_scale for m in ops], ops[0].out_features,
                                        ops[0].in_features)
    return _q.w4_tiled_linear_group((xr, xk, xv), tiled, ops[0].out_features, ops[0].in_features)


class StepContext:
    """What a layer step needs beyond the pack when it runs inside a larger program: side streams for the
    independent branches of the layer, and the sum over tensor-parallel ranks.  The default context is a single
    GPU with one side stream per device."""

    def __init__(self, side_stream=None, all_reduce=None, tp_world: int = 1, tp_rank: int = 0, lane: int = 0,
                 stream_base: int = 0, slot_ids=None, row_sum=None):
        # slot_ids (int32 [B] on the device): the recurrent buffers handed to the layer step are slot pools
        # ([capacity, ...]) and batch row b lives in pool row slot_ids[b]
        self.slot_ids = slot_ids
        self._side_stream = side_stream
        self._all_reduce = all_reduce
        # row_sum(partial, lane) -> tp_comm.PeerRowSum or None: the communicator whose row kernels take the sum over
        # ranks in themselves.  defer_sum (set by step_batched between layers): the layer may return its UNSUMMED
        # ffn.value partial and raise `pending`; the next layer's first kernel then sums it.
        self._row_sum = row_sum
        self.defer_sum = False
        self.pending = False
        self.tp_world, self.tp_rank, self.lane, self.stream_base = int(tp_world), int(tp_rank), int(lane), int(stream_base)
        self._own = {}

    def side_stream(self, device, index: int):
        if self._side_stream is not None:
            return self._side_stream(device, self.stream_base + index)
        st = self._own.get((device, index))
        if st is None:
            st = self._own[(device, index)] = torch.cuda.Stream(device=device)
        return st

    def all_reduce(self, t):
        return t if self._all_reduce is None else self._all_reduce(t, self.lane)

    def row_sum(self, partial):
        if self.tp_world == 1 or self._row_sum is None or partial.dim() != 2:
            return None
        return self._row_sum(partial, self.lane)


_DEFAULT_CONTEXT = StepContext()


def block_ip_batched(x, state, xpa, xpf, v_first, p, sparse_ffn_out=None, fp16_elapsed=None,
                     fp16_advance_elapsed=False, route_observer=None, *, context: StepContext | None = None):
    """One layer for ``B`` sequences from its pack tuple, recurrent buffers updated in place
    (rwkv7_hf/native_jit_decode.py:481-901: same arguments, same return value).

    ``x [B,D]`` residual stream in, new residual stream out; ``state [B,H,N,N]`` (fp32, or fp16 with the
    ``fp16_elapsed`` int32 ``[B]`` phase counters of the FP16-state lane), ``xpa``/``xpf [B,D]`` and ``v_first [B,A]``
    are overwritten (with ``context.slot_ids`` they are slot pools ``[capacity, ...]`` and only the rows named there change).  Every launch is capturable in a CUDA graph.  ``sparse_ffn_out`` and ``route_observer`` belong to
    the reference's sparse-FFN experiment and must be None."""
    if sparse_ffn_out is not None or route_observer is not None:
        raise NotImplementedError("the sparse-FFN route of the reference is not part of this library")
    if len(p) != PACK_SLOTS:
        raise ValueError(f"a layer pack has {PACK_SLOTS} slots, got {len(p)}")
    (i, H, N, eps, has_pre,
     pre_w, pre_b, an_w, an_b, fn_w, fn_b,
     x_r, x_w, x_k, x_v, x_a, x_g, k_k, k_a, r_k,
     Rw, Kw, Vw, Ow, w1, w2, w0, a1, a2, a0, v1, v2, v0, g1, g2,
     gn_w, gn_b, fx_k, fK, fV, RKVw) = p
    ctx = context or _DEFAULT_CONTEXT
    if has_pre:
        x = _nm.layer_norm(x, pre_w, pre_b)
    slots = ctx.slot_ids
    rows_comm = ctx.row_sum(x)
    if ctx.pending and rows_comm is None:
        ctx.pending = False
        x = ctx.all_reduce(x)
    if ctx.pending:
        # x is the previous layer's ffn.value partial: the sum over ranks happens inside this kernel
        ctx.pending = False
        x, (xr, xw, xk, xv, xa, xg) = rows_comm.attn_norm_mix6(x, xpa, an_w, an_b, (x_r, x_w, x_k, x_v, x_a, x_g),
                                                              slot_ids=slots)
    else:
        xr, xw, xk, xv, xa, xg = _nm.fused_attn_norm_mix6_decode(x, xpa, an_w, an_b, x_r, x_w, x_k, x_v, x_a, x_g,
                                                                 slot_ids=slots)
    # The LoRA chain does not depend on r/k/v: it runs on a side stream (a parallel branch of the decode graph once
    # captured) and joins before the recurrence.
    main = torch.cuda.current_stream(x.device)
    side = ctx.side_stream(x.device, 0)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        if int(i) == 0:
            hs = _lora.small_gemm_group((xw, xa, xg), (_weight_of(w1), _weight_of(a1), _weight_of(g1)), acts=(1, 0, 2))
            w_raw, a_pre, g = _lora.small_gemm_group(hs, (_weight_of(w2), _weight_of(a2), _weight_of(g2)))
            extra = dict(v_out=v_first)
        else:
            hs = _lora.small_gemm_group((xw, xa, xg, xv), (_weight_of(w1), _weight_of(a1), _weight_of(g1), _weight_of(v1)),
                                        acts=(1, 0, 2, 0))
            w_raw, a_pre, g, vg_pre = _lora.small_gemm_group(
                hs, (_weight_of(w2), _weight_of(a2), _weight_of(g2), _weight_of(v2)))
            extra = dict(v_first=v_first, v_gate=vg_pre, v_gate_bias=v0, v_gate_is_raw=True)
    ops = (Rw, Kw, Vw)
    rkv = rkv_grouped(ops, xr, xk, xv) if all(isinstance(o, _QUANT_TYPES) for o in ops) else None
    if rkv is not None:
        # int4 r / k / v of equal shape: one launch streams all three weight sets (one pipeline fill, no split-K
        # exchange) instead of three launches competing for the SMs
        r, k, v = rkv
        main.wait_stream(side)
    else:
        # independent projections on separate branches: the tail of one overlaps the ramp-up of the next
        sk, sv = ctx.side_stream(x.device, 1), ctx.side_stream(x.device, 2)
        sk.wait_stream(main)
        sv.wait_stream(main)
        with torch.cuda.stream(sk):
            k = apply_linear(Kw, xk)
        with torch.cuda.stream(sv):
            v = apply_linear(Vw, xv)
        r = apply_linear(Rw, xr)
        main.wait_stream(side)
        main.wait_stream(sk)
        main.wait_stream(sv)
        xk.record_stream(sk); k.record_stream(sk); xv.record_stream(sv); v.record_stream(sv)
    for t_ in (xw, xa, xg, xv, w_raw, a_pre, g):
        t_.record_stream(side)
    elapsed = fp16_elapsed if state.dtype == torch.float16 else None
    # the kernel launched just before the recurrence is a projection: it never writes the state
    out, _ = _rec.fused_recurrent_output_prepare_raw(
        r, w_raw, k, v, a_pre, state, g, k_k, k_a, r_k, gn_w, gn_b, eps=float(eps), new_state=state, w_bias=w0, a_bias=a0,
        a_is_raw=True, state_prefetch=True, elapsed=elapsed,
        advance_elapsed=bool(fp16_advance_elapsed) and elapsed is not None, slot_ids=slots, **extra)
    attn = apply_linear(Ow, out)
    if rows_comm is not None:
        x, mixed = rows_comm.ffn_add_norm_mix(x, attn, xpf, fn_w, fn_b, fx_k, slot_ids=slots)
    else:
        x, mixed = _nm.fused_ffn_add_norm_mix_decode(x, ctx.all_reduce(attn), xpf, fn_w, fn_b, fx_k, slot_ids=slots)
    hidden = apply_linear(fK, mixed, relu2=True)
    if ctx.tp_world > 1:
        # the residual rides in rank 0's partial sum (the projection's add epilogue): no extra add kernel
        part = apply_linear(fV, hidden, residual=x if ctx.tp_rank == 0 else None)
        if rows_comm is not None and ctx.defer_sum:
            ctx.pending = True
            return part
        return ctx.all_reduce(part)
    return apply_linear(fV, hidden, residual=x)


def step_batched(model, x, state, xpa, xpf, v_first, packs, *, fp16_elapsed=None, context: StepContext | None = None):
    """All layers of one decode step from their packs (rwkv7_hf/native_jit_decode.py:56-68 ``step_batched``): returns
    ``(x, state, xpa, xpf, v_first)`` with the buffers updated in place.  ``model`` is unused (kept for the
    reference's argument order)."""
    last = len(packs) - 1
    for li, p in enumerate(packs):
        if context is not None:
            context.defer_sum = li != last  # between layers the sum moves into the next layer's first kernel
        x = block_ip_batched(x, state[li], xpa[li], xpf[li], v_first, p, fp16_elapsed=fp16_elapsed,
                             fp16_advance_elapsed=li == last, context=context)
    return x, state, xpa, xpf, v_first
