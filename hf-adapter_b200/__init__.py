"""rwkv7_b200: B200 (sm_100a) kernels for the RWKV-7 inference hot path behind the operator
contract of rwkv-rs/hf-adapter (package ``rwkv7_hf``).  Importing this package loads the CUDA
library; there is no CPU or PyTorch fallback."""
from . import _lib  # noqa: F401  (fails loudly when the library is missing)
from .cache import NativeRWKV7Cache, NativeRWKV7LegacyCache
from .checkpoint import convert_state_dict, infer_config, load_checkpoint, to_upstream_state_dict, translate_name
from .gemm import dense_argmax, dense_linear
from .install import install, uninstall
from .lora import dense_small, fused_wa_lora, fused_wag_lora, fused_wavg_lora
from .model import DecodeGraph, NativeRWKV7Config, PrefillGraph, RWKV7ForCausalLM, sample_next_token
from .norm_mix import (fused_attn_norm_mix6_decode, fused_attn_sequence_shift_mix, fused_attn_shift_mix,
                       fused_ffn_add_norm_mix_decode, fused_ffn_sequence_shift_mix, layer_norm)
from .packing import (block_ip_batched, extract_graph_packs, graph_linear_is_dense, graph_linear_operand,
                      init_batched_from_packs, step_batched)
from .prep import (fused_attn_output_prepare, fused_attn_output_project, fused_ffn, fused_prefill_kv_kk_prep,
                   fused_prefill_state_prep, fused_sequence_ffn)
from .quant import (A8W8Linear, MM4Linear, MM8Linear, a8w8_ffn, a8w8_linear, dequantize_mm4, dequantize_mm8,
                    dynamic_a8_quant, int8_mm, mm4_matmul, mm4_matmul_triton, mm8_matmul, mm8_matmul_triton,
                    quantize_mm4, quantize_mm8, quantize_model, quantize_w4_groupwise, quantize_w8_row,
                    quantize_weight_per_channel_int8, w4_dequant, w4_groupwise_linear, w4_repack_tiled,
                    w4_tiled_linear, w4_tiled_linear_group, w8_dequant, w8_linear, w8_repack_tiled,
                    w8_tiled_linear_group)
from .recurrent import (dplr_chunk_scan, fused_recurrent_output_prepare, fused_recurrent_output_prepare_raw,
                        fused_recurrent_scan, fused_recurrent_scan_clampw, fused_recurrent_scan_output_prepare,
                        fused_recurrent_scan_state_prep, fused_recurrent_update, native_fp16_recurrent_output_prepare_raw,
                        native_fp16_recurrent_should_use, native_fp16_sequence, self_chunk_rwkv7)

from .sharding import shard_spec, shard_state_dict
from .tokenizer import RWKVWorldTokenizer
from .state_pool import PoolDecodeGraph, PrefixEntry, RWKV7StatePool, StaleSlotError

NativeRWKV7ForCausalLM = RWKV7ForCausalLM
__version__ = "0.1.0"
