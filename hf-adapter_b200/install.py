"""Rebinding the reference's operator names to this library.

The reference keeps its optional kernels as module globals of ``rwkv7_hf.native_jit`` and hands them to the modules
that run decode, prefill and the recurrence through ``bind_runtime(runtime_dict)`` (rwkv7_hf/native_jit.py:586-590,
655-694,781-792; native_jit_decode.py:45-48; native_jit_prefill.py:19-32; native_jit_recurrent.py:12-15).  ``install``
replaces every operator this library implements in that facade and re-runs the binding, so the reference's own
decode / prefill code calls the B200 kernels; ``uninstall`` puts the saved originals back.
"""
from __future__ import annotations

import importlib

OPERATOR_NAMES = (
    "fused_recurrent_update", "fused_recurrent_output_prepare", "fused_recurrent_output_prepare_raw",
    "fused_recurrent_scan", "fused_recurrent_scan_clampw", "fused_recurrent_scan_state_prep",
    "fused_recurrent_scan_output_prepare", "self_chunk_rwkv7", "dplr_chunk_scan",
    "native_fp16_recurrent_output_prepare_raw", "native_fp16_sequence",
    "fused_attn_norm_mix6_decode", "fused_ffn_add_norm_mix_decode", "fused_attn_shift_mix",
    "fused_attn_sequence_shift_mix", "fused_ffn_sequence_shift_mix",
    "fused_wag_lora", "fused_wavg_lora",
    "fused_prefill_state_prep", "fused_prefill_kv_kk_prep", "fused_attn_output_prepare", "fused_attn_output_project",
    "fused_sequence_ffn",
)
BOUND_MODULES = ("native_jit_recurrent", "native_jit_graph_dispatch", "native_jit_prefill", "native_jit_decode")


def install(native_jit=None, names=OPERATOR_NAMES):
    """Rebind ``names`` in the reference's ``native_jit`` facade (imported as ``rwkv7_hf.native_jit`` when not given)
    and in the modules it feeds.  Returns ``{name: original}`` for ``uninstall``.  A name the facade does not have is
    skipped: releases of the reference differ in which optional kernels they know."""
    import hf_adapter_b200 as b200
    if native_jit is None:
        native_jit = importlib.import_module("rwkv7_hf.native_jit")
    saved = {}
    for name in names:
        if hasattr(native_jit, name) and hasattr(b200, name):
            saved[name] = getattr(native_jit, name)
            setattr(native_jit, name, getattr(b200, name))
    _rebind(native_jit)
    return saved


def uninstall(saved, native_jit=None):
    if native_jit is None:
        native_jit = importlib.import_module("rwkv7_hf.native_jit")
    for name, original in saved.items():
        setattr(native_jit, name, original)
    _rebind(native_jit)


def _rebind(native_jit):
    package = native_jit.__name__.rsplit(".", 1)[0]
    for sub in BOUND_MODULES:
        try:
            mod = importlib.import_module(f"{package}.{sub}")
        except ImportError:
            continue
        bind = getattr(mod, "bind_runtime", None)
        if callable(bind):
            bind(vars(native_jit))
