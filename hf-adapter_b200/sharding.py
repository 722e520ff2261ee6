"""Head-sharded tensor parallelism: how a full ``state_dict`` splits across P ranks.

The WKV-7 recurrence has no cross-head term, so rank p owns heads ``[p*H/P, (p+1)*H/P)``: the matching rows of
``r/k/v_proj`` and of every LoRA up-projection (with their biases), the per-head vectors ``k_k, k_a, r_k`` and the
GroupNorm affine, the matching input columns of ``o_proj``, rows ``[p*F/P, (p+1)*F/P)`` of ``ffn.key`` and the same
columns of ``ffn.value``, and the recurrent state / ``v_first`` of its heads.  LoRA down-projections, LayerNorms,
token-shift vectors, embeddings and the head are replicated.  The ``[B,D]`` partial outputs of ``o_proj`` and
``ffn.value`` are summed with one all-reduce each (the reference keeps the state replicated under its TP plan,
``rwkv7_hf/model_config.py:37-53``; sharding it is what lets the state-bound decode step scale)."""
from __future__ import annotations

import re

_ROWS = re.compile(r"\.attn\.(r_proj|k_proj|v_proj)\.weight$|\.attn\.[wagv]_lora\.lora\.2\.(weight|bias)$|"
                   r"\.attn\.(k_k|k_a|r_k)$|\.attn\.g_norm\.(weight|bias)$|\.ffn\.key\.weight$")
_COLS = re.compile(r"\.attn\.o_proj\.weight$|\.ffn\.value\.weight$")


def shard_spec(name: str):
    """'rows' (dim 0 split), 'cols' (dim 1 split) or None (replicated) for a parameter name."""
    if _ROWS.search(name):
        return "rows"
    if _COLS.search(name):
        return "cols"
    return None


def shard_state_dict(full, world: int, rank: int, shard_head: bool = False):
    """Return rank ``rank``'s share of a full (unsharded) state dict of tensors or arrays.  ``shard_head``: the head's
    vocabulary rows are split as well (``RWKV7ForCausalLM(tp_shard_head=True)``)."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    out = {}
    for name, t in full.items():
        spec = shard_spec(name)
        if shard_head and name == "lm_head.weight":
            spec = "rows"
        if spec is None or world == 1:
            out[name] = t
            continue
        dim = 0 if spec == "rows" else 1
        n = int(t.shape[dim])
        if n % world:
            raise ValueError(f"{name}: dimension {dim} of size {n} is not divisible by {world} ranks")
        step = n // world
        index = [slice(None)] * len(t.shape)
        index[dim] = slice(rank * step, (rank + 1) * step)
        out[name] = t[tuple(index)]
    return out


def pick_sharded_argmax(values, indices):
    """``values`` / ``indices`` ``[P,B]``: every rank's best logit and its GLOBAL vocabulary index.  Returns the arg-max
    per column with torch.argmax's tie rule (the lowest index wins)."""
    import torch
    best = values.max(dim=0).values
    big = torch.iinfo(indices.dtype).max
    return torch.where(values == best[None], indices, torch.full_like(indices, big)).min(dim=0).values


def sharded_argmax(local_logits, rank: int, world: int, group=None, *, local_best=None, shard_width: int = 0):
    """Greedy token over a vocabulary-sharded head: local (max, arg-max) per row, one all-gather of ``[B,2]`` floats per
    rank (indices below 2^24 are exact in fp32), then the pick.  Every rank returns the same ``[B]`` int64 tokens.
    ``local_best = (values [B] fp32, indices [B])`` with ``shard_width`` replaces ``local_logits`` when the head kernel
    already folded its shard (the logits then never exist)."""
    import torch
    import torch.distributed as dist
    if local_best is not None:
        vals, idx = local_best
        width = int(shard_width)
    else:
        vals, idx = local_logits.float().max(dim=-1)
        width = int(local_logits.shape[-1])
    mine = torch.stack([vals.float(), (idx + rank * width).float()], dim=-1).contiguous()  # [B,2]
    parts = torch.empty((world * int(mine.shape[0]), 2), device=mine.device, dtype=mine.dtype)  # rank-major concatenation
    dist.all_gather_into_tensor(parts, mine, group=group)
    parts = parts.view(world, -1, 2)
    return pick_sharded_argmax(parts[..., 0], parts[..., 1].long())
