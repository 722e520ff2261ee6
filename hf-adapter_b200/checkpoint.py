"""Loading upstream RWKV-7 checkpoints: key translation, shape inference, model construction.

Upstream ("official") checkpoints name tensors ``emb.weight``, ``blocks.N.att.receptance.weight``, ``blocks.N.att.w1``
... and store the LoRA factors as ``[in, rank]`` / ``[rank, out]`` matrices; this package (like the reference's native
model) uses ``model.layers.N.attn.r_proj.weight``, ``...w_lora.lora.0.weight`` ``[rank, in]``, ``...lora.2.weight``
``[out, rank]``, ``...lora.2.bias``.  The role of the reference's converter (rwkv7_hf/converter.py:140-365: ``infer_*``,
``validate_layer_shapes``, ``translate_name``, ``prepare_translated_weight``), without its file-layout and Hugging Face
metadata parts: ``convert_state_dict`` maps a dict of upstream tensors to ``(config, state_dict)`` for
``RWKV7ForCausalLM``, ``load_checkpoint`` builds (and optionally quantises) the model, ``to_upstream_state_dict`` is the
inverse mapping.
"""
from __future__ import annotations

import re

import torch

from .model import NativeRWKV7Config, RWKV7ForCausalLM

# upstream sub-module / tensor names -> this package's
_BLOCK_PARTS = {"att": "attn", "ffn": "ffn", "ln0": "pre_norm", "ln1": "attn_norm", "ln2": "ffn_norm"}
_ATT_PROJ = {"receptance": "r_proj", "key": "k_proj", "value": "v_proj", "output": "o_proj", "ln_x": "g_norm"}
_TOP = {"emb.weight": "model.embeddings.weight", "ln_out.weight": "model.norm.weight", "ln_out.bias": "model.norm.bias",
        "head.weight": "lm_head.weight"}
# LoRA factor suffix: upstream digit -> (our tail, stored transposed upstream)
_LORA = {"0": ("lora.2.bias", False), "1": ("lora.0.weight", True), "2": ("lora.2.weight", True)}
_LORA_RE = re.compile(r"^([wavg])([012])$")
# layer 0 has no value-residual gate; upstream checkpoints still carry (unused) v0 / v1 / v2 for it
_UNUSED = {"blocks.0.att.v0", "blocks.0.att.v1", "blocks.0.att.v2"}


def translate_name(name: str, num_layers: int):
    """``(destination key, transposed)`` for an upstream tensor name, or ``("", False)`` for a tensor the model does
    not use (rwkv7_hf/converter.py:333-365)."""
    if name in _UNUSED:
        return "", False
    if name in _TOP:
        return _TOP[name], False
    parts = name.split(".")
    if len(parts) < 4 or parts[0] != "blocks" or not parts[1].isdigit() or parts[2] not in _BLOCK_PARTS:
        raise KeyError(f"Unexpected RWKV weight name: {name}")
    layer = int(parts[1])
    if not 0 <= layer < num_layers:
        raise KeyError(f"Layer index out of range in {name}")
    head = f"model.layers.{layer}.{_BLOCK_PARTS[parts[2]]}"
    tail, transposed = parts[3:], False
    m = _LORA_RE.match(tail[0])
    if m and len(tail) == 1:
        sub, transposed = _LORA[m.group(2)]
        tail = [f"{m.group(1)}_lora", sub]
    elif parts[2] == "att" and tail[0] in _ATT_PROJ:
        tail = [_ATT_PROJ[tail[0]]] + tail[1:]
    return ".".join([head] + tail), transposed


def _shape(weights, name):
    if name not in weights:
        raise KeyError(f"Missing required RWKV-7 weight: {name}")
    return tuple(int(v) for v in weights[name].shape)


def infer_num_layers(weights) -> int:
    """Number of blocks; their indices must be 0..L-1 without gaps (rwkv7_hf/converter.py:147-159)."""
    found = sorted(int(m.group(1)) for k in weights if (m := re.match(r"blocks\.(\d+)\.ffn\.key\.weight$", k)))
    if not found:
        raise KeyError("No blocks.*.ffn.key.weight tensors found in checkpoint")
    if found != list(range(found[-1] + 1)):
        raise ValueError(f"RWKV block indices must be contiguous from 0: got {found[:20]} ...")
    return len(found)


def infer_config(weights) -> NativeRWKV7Config:
    """Model shape from the tensors alone (rwkv7_hf/converter.py:268-319): width and FFN size from ``ffn.key``, heads
    and head size from ``att.r_k``, the LoRA ranks from the second axis of ``w1 / a1 / g1 / v1``."""
    F_, D = _shape(weights, "blocks.0.ffn.key.weight")
    L = infer_num_layers(weights)
    rk = _shape(weights, "blocks.0.att.r_k")
    if len(rk) < 2 or any(d != 1 for d in rk[:-2]):
        raise ValueError(f"Cannot infer attention shape from blocks.0.att.r_k={rk}")
    H, N = rk[-2:]
    A = H * N
    for i in range(L):
        if _shape(weights, f"blocks.{i}.ffn.key.weight") != (F_, D):
            raise ValueError(f"blocks.{i}.ffn.key.weight has inconsistent shape {_shape(weights, f'blocks.{i}.ffn.key.weight')}")
        if _shape(weights, f"blocks.{i}.att.r_k")[-2:] != (H, N):
            raise ValueError(f"blocks.{i}.att.r_k has shape {_shape(weights, f'blocks.{i}.att.r_k')}; expected trailing {(H, N)}")
        for proj in ("receptance", "key", "value"):
            if _shape(weights, f"blocks.{i}.att.{proj}.weight") != (A, D):
                raise ValueError(f"blocks.{i}.att.{proj}.weight has shape {_shape(weights, f'blocks.{i}.att.{proj}.weight')}; expected {(A, D)}")
        if _shape(weights, f"blocks.{i}.att.output.weight") != (D, A):
            raise ValueError(f"blocks.{i}.att.output.weight has shape {_shape(weights, f'blocks.{i}.att.output.weight')}; expected {(D, A)}")
        for affine in ("weight", "bias"):
            if _shape(weights, f"blocks.{i}.att.ln_x.{affine}") != (A,):
                raise ValueError(f"blocks.{i}.att.ln_x.{affine} must have shape {(A,)}")
    if A != D:
        raise ValueError(f"this library's model needs attention width == hidden size (got {A} and {D})")
    v_rank = _shape(weights, "blocks.1.att.v1")[1] if "blocks.1.att.v1" in weights else 32
    return NativeRWKV7Config(vocab_size=_shape(weights, "emb.weight")[0], hidden_size=D, num_hidden_layers=L, num_heads=H,
                             head_dim=N, intermediate_size=F_, decay_low_rank_dim=_shape(weights, "blocks.0.att.w1")[1],
                             a_low_rank_dim=_shape(weights, "blocks.0.att.a1")[1], v_low_rank_dim=v_rank,
                             gate_low_rank_dim=_shape(weights, "blocks.0.att.g1")[1])


def convert_state_dict(weights, dtype=None):
    """``(config, state_dict)`` for ``RWKV7ForCausalLM`` from a dict of upstream tensors.  LoRA factors are transposed,
    vectors stored with other singleton axes (``x_r [1,1,D]`` against ``[D]``, ``r_k [1,H,N]``) are reshaped to the
    module's shape; every destination key must be produced exactly once and no source key may be left over."""
    config = infer_config(weights)
    template = _template_shapes(config)
    out = {}
    for name, tensor in weights.items():
        dst, transposed = translate_name(name, config.num_hidden_layers)
        if not dst:
            continue
        if dst not in template:
            raise KeyError(f"{name} maps to {dst}, which the model does not have")
        if dst in out:
            raise KeyError(f"{dst} is produced twice")
        w = tensor.detach()
        if transposed:
            w = w.t()
        want = template[dst]
        if tuple(w.shape) != want:
            if int(w.numel()) != _numel(want):
                raise ValueError(f"Shape mismatch {name} -> {dst}: {tuple(w.shape)} vs {want}")
            w = w.reshape(want)
        w = w.contiguous()
        if dtype is not None and w.is_floating_point():
            w = w.to(dtype)
        if w.data_ptr() == tensor.data_ptr():
            w = w.clone()  # never alias the caller's (possibly memory-mapped) checkpoint
        out[dst] = w
    missing = sorted(set(template) - set(out))
    if missing:
        raise KeyError(f"checkpoint lacks tensors for: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
    return config, out


def _numel(shape):
    n = 1
    for d in shape:
        n *= int(d)
    return n


def _template_shapes(c: NativeRWKV7Config):
    """Key -> shape of ``RWKV7ForCausalLM(c).state_dict()`` without allocating the model."""
    D, A, F_, V, H, N = c.hidden_size, c.num_heads * c.head_dim, c.intermediate_size, c.vocab_size, c.num_heads, c.head_dim
    s = {"model.embeddings.weight": (V, D), "model.norm.weight": (D,), "model.norm.bias": (D,), "lm_head.weight": (V, D)}
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        for ln in ("attn_norm", "ffn_norm") + (("pre_norm",) if i == 0 else ()):
            s[p + ln + ".weight"] = s[p + ln + ".bias"] = (D,)
        a = p + "attn."
        for mix in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"):
            s[a + mix] = (1, 1, D)
        s[a + "k_k"] = s[a + "k_a"] = (A,)
        s[a + "r_k"] = (H, N)
        for proj in ("r_proj", "k_proj", "v_proj"):
            s[a + proj + ".weight"] = (A, D)
        s[a + "o_proj.weight"] = (D, A)
        s[a + "g_norm.weight"] = s[a + "g_norm.bias"] = (A,)
        ranks = {"w": c.decay_low_rank_dim, "a": c.a_low_rank_dim, "g": c.gate_low_rank_dim}
        if i != 0:
            ranks["v"] = c.v_low_rank_dim
        for t, r in ranks.items():
            s[a + f"{t}_lora.lora.0.weight"] = (r, D)
            s[a + f"{t}_lora.lora.2.weight"] = (A, r)
            if t != "g":
                s[a + f"{t}_lora.lora.2.bias"] = (A,)
        s[p + "ffn.x_k"] = (D,)
        s[p + "ffn.key.weight"] = (F_, D)
        s[p + "ffn.value.weight"] = (D, F_)
    return s


def to_upstream_state_dict(state_dict):
    """The inverse of ``convert_state_dict``: this package's keys and layouts back to the upstream ones."""
    inv_top = {v: k for k, v in _TOP.items()}
    inv_part = {v: k for k, v in _BLOCK_PARTS.items()}
    inv_proj = {v: k for k, v in _ATT_PROJ.items()}
    inv_lora = {tail: (digit, tr) for digit, (tail, tr) in _LORA.items()}
    out = {}
    for key, t in state_dict.items():
        if key in inv_top:
            out[inv_top[key]] = t.clone()
            continue
        m = re.match(r"^model\.layers\.(\d+)\.(attn|ffn|pre_norm|attn_norm|ffn_norm)\.(.+)$", key)
        if not m:
            raise KeyError(f"Unexpected model key: {key}")
        layer, part, tail = m.group(1), inv_part[m.group(2)], m.group(3)
        lm = re.match(r"^([wavg])_lora\.(lora\.\d\.\w+)$", tail)
        if lm:
            digit, transposed = inv_lora[lm.group(2)]
            out[f"blocks.{layer}.{part}.{lm.group(1)}{digit}"] = (t.t() if transposed else t).contiguous().clone()
            continue
        first, _, rest = tail.partition(".")
        if part == "att" and first in inv_proj:
            tail = inv_proj[first] + ("." + rest if rest else "")
        out[f"blocks.{layer}.{part}.{tail}"] = t.clone()
    return out


def load_checkpoint(weights, *, dtype=torch.float16, device="cuda", quant=None, min_params: int = 8_000_000,
                    group_size: int = 128, state_dtype=torch.float32):
    """Build ``RWKV7ForCausalLM`` from upstream weights (a dict of tensors, or the path of a ``torch.save``d one),
    cast to ``dtype``, optionally quantise the projections (``quant`` in {"mm4", "w8", "mm8", "a8w8"}) and move to
    ``device``.  Returns the model in eval mode."""
    if not isinstance(weights, dict):
        weights = torch.load(weights, map_location="cpu", mmap=True, weights_only=True)
    config, sd = convert_state_dict(weights, dtype=dtype)
    model = RWKV7ForCausalLM(config, state_dtype=state_dtype).to(dtype)
    model.load_state_dict(sd)
    if quant:
        from .quant import quantize_model
        quantize_model(model, quant, min_params=min_params, group_size=group_size)
    return model.to(device).eval()
