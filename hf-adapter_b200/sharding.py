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


def shard_state_dict(full, world: int, rank: int):
    """Return rank ``rank``'s share of a full (unsharded) state dict of tensors or arrays."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    out = {}
    for name, t in full.items():
        spec = shard_spec(name)
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
