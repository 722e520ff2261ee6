/*
 * rwkv7_b200 — C ABI of the B200 (sm_100a) RWKV-7 inference kernels.
 *
 * Every entry point:
 *   - takes plain device pointers owned by the caller, sizes, and the CUDA stream
 *     (a cudaStream_t passed as void*; NULL = the legacy default stream);
 *   - launches asynchronously on that stream, allocates nothing, and can be called from
 *     any host thread with the device current.  What the library keeps between calls:
 *     a thread-local error string; one device-side error word per GPU (set by a
 *     tensor-core kernel whose bounded wait gave up, read by rwkv7_kernel_status) and
 *     its cached address; the set of tiled int4 buffers written by rwkv7_w4g_repack
 *     and not yet read by a projection (mutex-protected); the cached address of the
 *     static scratch of rwkv7_a8w8_linear_static.  No option or mode is process-wide:
 *     everything that changes what a launch does is an argument of the call;
 *   - returns RWKV7_OK or a negative RWKV7_ERR_* code and never aborts;
 *     rwkv7_last_error() returns a thread-local message for the last failure.
 *
 * Tensors are contiguous row-major unless a stride is passed.  `dtype` selects the
 * activation storage type (RWKV7_F16 / RWKV7_BF16 / RWKV7_F32); arithmetic is fp32
 * everywhere, the recurrent state is always fp32 [B,H,64,64] with rows = value
 * index and columns = key index (the reference's "native" orientation).
 *
 * The reference project (rwkv-rs/hf-adapter, package rwkv7_hf) has no C ABI: its
 * boundary is Python functions with a pure-torch fallback plus optional pybind
 * extensions.  Each declaration below cites the reference interface it replaces.
 */
#ifndef RWKV7_B200_H
#define RWKV7_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RWKV7_OK 0
#define RWKV7_ERR_INVALID (-1)     /* null pointer, bad size, bad enum */
#define RWKV7_ERR_UNSUPPORTED (-2) /* shape outside what the kernels handle (e.g. head size != 64) */
#define RWKV7_ERR_ALIGN (-3)       /* pointer or leading dimension not aligned for vector loads */
#define RWKV7_ERR_CUDA (-4)        /* the CUDA runtime reported an error at launch */
#define RWKV7_ERR_WORKSPACE (-5)   /* caller-provided workspace too small */

#define RWKV7_F16 0
#define RWKV7_BF16 1
#define RWKV7_F32 2

/* epilogues of the quantised linears (rwkv7_forward_relu2 / rwkv7_forward_add hooks,
 * rwkv7_hf/native_quant_mm4.py:662-712, native_quant_a8w8.py:555-571) */
#define RWKV7_EPI_NONE 0
#define RWKV7_EPI_RELU2 1 /* out = relu(y)^2, y rounded to the activation dtype first */
#define RWKV7_EPI_ADD 2   /* out = y + residual */

int rwkv7_abi_version(void);
const char* rwkv7_last_error(void);

/* The tensor-core kernels bound every wait on an mbarrier; a wait that gives up records a positive code in a
 * device-side word instead of hanging.  This call synchronises with the device, returns that word (0 = no kernel
 * ever gave up; > 0 = code; < 0 = RWKV7_ERR_*) and clears it when reset != 0.  No counterpart in the reference. */
int rwkv7_kernel_status(int reset);

/* ------------------------------------------------------------------ WKV-7 recurrence, one token
 * Replaces fused_recurrent_update (rwkv7_hf/fused_recurrent_update.py:1214),
 * fused_recurrent_output_prepare (:967) and fused_recurrent_output_prepare_raw (:1089).
 *
 *   sa[i]   = sum_m S[i,m] kk[m]
 *   S'[i,j] = S[i,j] w[j] + v[i] k[j] - sa[i] kk[j] a[j]
 *   y[i]    = sum_j S'[i,j] r[j]
 *
 * state_out may equal state_in (in-place update) or be a different buffer (the reference
 * contract: input state untouched).  Vectors are [B,H,64] in `dtype`; `w` is the decay in
 * fp32 when w_is_f32 != 0, else in `dtype`.
 */
int rwkv7_wkv7_update(const void* r, const void* w, const void* k, const void* v, const void* kk, const void* a,
                      const float* state_in, float* state_out, void* y,
                      int B, int H, int N, int dtype, int w_is_f32, void* stream);

/* update + GroupNorm(eps) + (sum_n r k r_k) v bonus + gate g.  r_k [H,64]; gn_w, gn_b [H*64]. */
int rwkv7_wkv7_output_prepare(const void* r, const void* w, const void* k, const void* v, const void* kk,
                              const void* a, const float* state_in, float* state_out, const void* g,
                              const void* r_k, const void* gn_w, const void* gn_b, void* out,
                              int B, int H, int N, float eps, int dtype, int w_is_f32, void* stream);

/* Same from raw projections: w = exp(-0.606531*sigmoid(w_raw)), kk = l2norm_head(k_raw*k_k),
 * k = k_raw*(1+(a-1)*k_a).  Optional fusions of the LoRA epilogues that precede the step in the
 * decode layer (rwkv7_hf/native_jit_decode.py:747-767); each is enabled by a non-NULL pointer/flag:
 *   w_bias  [H*64] : w_raw += w_bias           (w_lora up bias "w0")
 *   a_bias  [H*64] + a_is_raw : a = sigmoid(a + a_bias)  (a_lora up bias "a0")
 *   v_first [B,H*64], v_gate [B,H*64] (+v_gate_bias, v_gate_is_raw): v = v + (v_first - v)*gate
 *   v_out   [B,H*64] : receives the v actually used (layer 0 stores it as v_first)
 * state_prefetch != 0: the kernel (launched programmatically, under the tail of the kernel that precedes it in the
 * stream) loads its state tile BEFORE waiting for that kernel.  Pass it only when the preceding kernel never writes
 * state_in -- true inside a decode step, where a projection precedes the recurrence; false for back-to-back
 * recurrence calls that feed each other's state.
 */
int rwkv7_wkv7_output_prepare_raw(const void* r, const void* w_raw, const void* k_raw, const void* v, const void* a,
                                  const float* state_in, float* state_out, const void* g,
                                  const void* k_k, const void* k_a, const void* r_k,
                                  const void* gn_w, const void* gn_b, void* out,
                                  const void* w_bias, const void* a_bias, int a_is_raw,
                                  const void* v_first, const void* v_gate, const void* v_gate_bias, int v_gate_is_raw,
                                  void* v_out, int state_prefetch,
                                  int B, int H, int N, float eps, int dtype, void* stream);

/* The same two operators with the recurrent state stored in fp16 [B,H,64,64] (half the state traffic of a decode
 * step); arithmetic stays fp32, the new state is rounded to nearest on the store and the output is formed from the
 * state as stored.  They replace the reference's opt-in FP16-state lanes: the Triton output-prepare kernels given an fp16
 * state (rwkv7_hf/fused_recurrent_update.py:655-699,1030,1149) and, with `elapsed`, the native_wkv_fp16 extension
 * recurrent_output_raw(r,w_raw,k_raw,v,a,state,g,k_k,k_a,r_k,norm_w,norm_b,elapsed,advance,eps)
 * (rwkv7_hf/native_wkv_fp16.py:54-71,200-333).
 *   elapsed [B] int32 (may be NULL): per-sequence step counters.  When given, the decay operand is formed as in that
 *   extension: 1 + fp16(decay - 1 + rot(elapsed[b] + h*64 + j)), rot(x) = 2^-41 * int32(2654435769 * x), a zero-mean
 *   offset below 2^-10 that keeps round-to-nearest from freezing slowly decaying entries (:118-128).
 *   advance_elapsed != 0: elapsed[b] += 1 for every b after the step (a second tiny launch in stream order). */
int rwkv7_wkv7_output_prepare_f16state(const void* r, const void* w, const void* k, const void* v, const void* kk,
                                       const void* a, const void* state_in, void* state_out, const void* g,
                                       const void* r_k, const void* gn_w, const void* gn_b, void* out,
                                       int B, int H, int N, float eps, int dtype, int w_is_f32, void* stream);
int rwkv7_wkv7_output_prepare_raw_f16state(const void* r, const void* w_raw, const void* k_raw, const void* v,
                                           const void* a, const void* state_in, void* state_out, const void* g,
                                           const void* k_k, const void* k_a, const void* r_k,
                                           const void* gn_w, const void* gn_b, void* out,
                                           const void* w_bias, const void* a_bias, int a_is_raw,
                                           const void* v_first, const void* v_gate, const void* v_gate_bias,
                                           int v_gate_is_raw, void* v_out, int* elapsed, int advance_elapsed,
                                           int state_prefetch, int B, int H, int N, float eps, int dtype, void* stream);

/* ------------------------------------------------------------------ WKV-7 scan over T tokens
 * Replaces fused_recurrent_scan (rwkv7_hf/fused_recurrent_update.py:1299), _clampw (:1420),
 * _output_prepare (:1710), self_chunk_rwkv7 (rwkv7_hf/self_chunk_rwkv7.py:33) and dplr_chunk_scan
 * (rwkv7_hf/dplr_prefill.py:505).  Inputs [B,T,H,64]; y [B,T,H,64]; state [B,H,64,64] fp32.
 *   w_mode: 0 = w is the decay in `dtype`, 1 = decay in fp32, 2 = raw w in `dtype` (decay computed in-kernel)
 *   g/r_k/gn_w/gn_b: all NULL = plain scan; all non-NULL = fused per-token GroupNorm/bonus/gate.
 */
int rwkv7_wkv7_scan(const void* r, const void* w, const void* k, const void* v, const void* kk, const void* a,
                    const float* state_in, float* state_out, void* y,
                    const void* g, const void* r_k, const void* gn_w, const void* gn_b, float eps,
                    int B, int T, int H, int N, int dtype, int w_mode, void* stream);

/* The scan with an fp16 state (loaded to fp32 registers, rounded back once at the end of the call) and the operand
 * forms of the reference's FP16-state sequence kernel sequence(r,w,k,v,neg_kk,kka,state,elapsed,w0,add_w0)
 * (rwkv7_hf/native_wkv_fp16.py:335-452,773-821):
 *   ab_mode != 0: `kk` holds -kk and `a` holds kk*a;  w0 [H*64] (may be NULL): added to raw w before the decay (w_mode 2);
 *   elapsed [B] int32 (may be NULL, w_mode 2): token t uses the dither phase elapsed[b] + h*64 + j + t (see above).
 * The reference rounds the state to fp16 after every token; this kernel keeps it in fp32 registers within a call. */
int rwkv7_wkv7_scan_f16state(const void* r, const void* w, const void* k, const void* v, const void* kk, const void* a,
                             const void* state_in, void* state_out, void* y,
                             const void* g, const void* r_k, const void* gn_w, const void* gn_b, float eps,
                             int B, int T, int H, int N, int dtype, int w_mode, int ab_mode, const void* w0,
                             const int* elapsed, void* stream);

/* Chunked (WY / DPLR) form of the same scan with the intra-chunk products on tensor cores.
 * chunk in {16, 32, 64}; T % chunk == 0; fp16 activations only (RWKV7_ERR_UNSUPPORTED otherwise: callers route
 * other dtypes to rwkv7_wkv7_scan, which computes the same recurrence).  Same arguments as above. */
int rwkv7_wkv7_chunk_scan(const void* r, const void* w, const void* k, const void* v, const void* kk, const void* a,
                          const float* state_in, float* state_out, void* y,
                          int B, int T, int H, int N, int chunk, int dtype, int w_mode, void* stream);

/* ------------------------------------------------------------------ LayerNorm + token-shift mixes
 * Replaces fused_attn_norm_mix6_decode (rwkv7_hf/fused_decode_norm_mix.py:161): h = LN(x);
 * out_m = h + (prev - h)*mix_m for m in r,w,k,v,a,g; prev <- h (in place).  outs: 6 device pointers
 * (host array).  x [rows,D]. */
int rwkv7_attn_norm_mix6(const void* x, void* prev, const void* norm_w, const void* norm_b,
                         const void* const mixes[6], void* const outs[6],
                         int rows, int D, float eps, int dtype, void* stream);

/* Replaces fused_ffn_add_norm_mix_decode (rwkv7_hf/fused_decode_norm_mix.py:296) and the sm_120-only
 * ffn_add_norm_mix extension (rwkv7_hf/blackwell_norm_mix.py:56-63): x = residual + attn_out (attn_out
 * may be NULL); h = LN(x); mixed = h + (prev-h)*mix; prev <- h. */
int rwkv7_ffn_add_norm_mix(const void* residual, const void* attn_out, void* prev, const void* norm_w,
                           const void* norm_b, const void* mix, void* residual_out, void* mixed,
                           int rows, int D, float eps, int dtype, void* stream);

/* ------------------------------------------------------------------ serving state pool
 * The three decode operators that touch per-sequence state, reading and writing it in place inside a slot pool
 * (docs/integrations/RWKV7_STATE_CACHE_ABI.md of the reference: layer-major pools indexed by slot id, "production
 * kernels may consume pool pointers and slot_ids directly, removing the gather/scatter copies").  slot_ids: int32 [B]
 * on the device; batch row b uses pool row slot_ids[b].  Rows must be distinct among the live sequences of a call;
 * padding rows of a fixed-size graph batch all point at one scratch row that no sequence owns.  Everything else
 * (activations, outputs) stays batch-ordered.
 *   prev_pool     [capacity, D]        token-shift state of one layer (xpa or xpf)
 *   state_pool    [capacity, H,64,64]  fp32 recurrent state of one layer, updated in place
 *   v_first_pool / v_out_pool [capacity, H*64]  (layer 0 writes v_out_pool, later layers read v_first_pool) */
int rwkv7_attn_norm_mix6_pool(const void* x, void* prev_pool, const int32_t* slot_ids, const void* norm_w,
                              const void* norm_b, const void* const mixes[6], void* const outs[6],
                              int rows, int D, float eps, int dtype, void* stream);
int rwkv7_ffn_add_norm_mix_pool(const void* residual, const void* attn_out, void* prev_pool, const int32_t* slot_ids,
                                const void* norm_w, const void* norm_b, const void* mix, void* residual_out,
                                void* mixed, int rows, int D, float eps, int dtype, void* stream);
int rwkv7_wkv7_output_prepare_raw_pool(const void* r, const void* w_raw, const void* k_raw, const void* v, const void* a,
                                       float* state_pool, const int32_t* slot_ids, const void* g,
                                       const void* k_k, const void* k_a, const void* r_k,
                                       const void* gn_w, const void* gn_b, void* out,
                                       const void* w_bias, const void* a_bias, int a_is_raw,
                                       const void* v_first_pool, const void* v_gate, const void* v_gate_bias,
                                       int v_gate_is_raw, void* v_out_pool, int state_prefetch,
                                       int B, int H, int N, float eps, int dtype, void* stream);

/* Plain LayerNorm (pre_norm of layer 0 and the final norm; rwkv7_hf/native.py:404,450). */
int rwkv7_layer_norm(const void* x, const void* norm_w, const void* norm_b, void* out,
                     int rows, int D, float eps, int dtype, void* stream);

/* Replaces fused_attn_sequence_shift_mix / fused_ffn_sequence_shift_mix (rwkv7_hf/fused_time_mix.py:413,470):
 * x [B,T,D] (already normalised), prev_t = x_{t-1} (initial_prev for t = 0), out_m = x + (prev-x)*mix_m for
 * n_mix in {1,6} mixes; next_state [B,D] = x[:, T-1].  strict_rounding != 0 (fp16 only) reproduces the reference's
 * strict_fp16_rounding=True lowering (:63-134): delta = fp16(prev - x), product = fp16(delta * mix),
 * out = fp16(x + product), three separately rounded fp16 operations like eager PyTorch; 0 = one fp32 expression
 * rounded once at the store. */
int rwkv7_seq_shift_mix(const void* x, const void* initial_prev, const void* const* mixes, void* const* outs,
                        void* next_state, int B, int T, int D, int n_mix, int strict_rounding, int dtype,
                        void* stream);

/* ------------------------------------------------------------------ LoRA group
 * Replaces fused_wa_lora / fused_wag_lora / fused_wavg_lora (rwkv7_hf/fused_lora.py:409,559,706) as a
 * generic small dense linear with fused activation:
 *   out[rows,Nout] = act_out( act_in(x)[rows,K] . W[Nout,K]^T + bias )
 * act codes: 0 none, 1 tanh, 2 sigmoid.  Intended for the rank-R projections (K or Nout <= 256). */
int rwkv7_dense_small(const void* x, const void* W, const void* bias, void* out,
                      int rows, int K, int Nout, int act_in, int act_out, int dtype, void* stream);

/* The same for up to four independent problems in ONE launch (the four rank-R "down" projections, or the four "up"
 * projections, of a layer: the reference's _wavg_lora_down_kernel / _wavg_lora_up_kernel pair,
 * rwkv7_hf/fused_lora.py:244-384), on warp-level tensor-core MMA with split-K inside a thread-block cluster.
 * Arrays have n_problems entries; bias may be NULL or hold NULL entries; any M (64-row blocks); fp16 or bf16.
 *   out_p[M,Nout_p] = act_out_p( x_p[M,K_p] . W_p[Nout_p,K_p]^T + bias_p ) */
int rwkv7_small_gemm_group(int n_problems, const void* const* x, const void* const* W, const void* const* bias,
                           void* const* out, const int* K, const int* Nout, const int* act_out, int M, int dtype,
                           void* stream);

/* ------------------------------------------------------------------ prefill state / output prep
 * Replaces fused_prefill_state_prep (rwkv7_hf/fused_prefill.py:184): per row of [rows,H*64]
 *   w_out = exp(-0.606531*sigmoid(w_raw)) (fp32; the log-decay when log_decay != 0),
 *   kk = l2norm_head(k_raw*k_k), k = k_raw*(1+(a-1)*k_a), v = v_raw + (v_first - v_raw)*v_gate.
 * v_first/v_gate may be NULL (layer 0).  w_raw and w_out may both be NULL: then only k, v, kk are produced, which is
 * fused_prefill_kv_kk_prep (rwkv7_hf/fused_prefill.py:324), the companion of the raw-w scan. */
int rwkv7_prefill_state_prep(const void* w_raw, const void* k_raw, const void* v_raw, const void* a,
                             const void* k_k, const void* k_a, const void* v_first, const void* v_gate,
                             float* w_out, void* k_out, void* v_out, void* kk_out,
                             int rows, int H, int N, int a_is_raw, int v_gate_is_raw, int log_decay,
                             int dtype, void* stream);

/* Replaces fused_attn_output_prepare (rwkv7_hf/fused_output.py:190): (GroupNorm(y) + (sum r k r_k) v) * g. */
int rwkv7_attn_output_prepare(const void* recurrent, const void* r, const void* k, const void* v, const void* g,
                              const void* r_k, const void* gn_w, const void* gn_b, void* out,
                              int rows, int H, int N, float eps, int dtype, void* stream);

/* y = max(x, 0)^2 elementwise over n elements (n % 8 == 0; in place allowed): the activation between the FFN key and
 * value projections when they are dense GEMMs (fused_ffn / fused_sequence_ffn, rwkv7_hf/fused_ffn.py:245-485). */
int rwkv7_relu2(const void* x, void* y, long long n, int dtype, void* stream);

/* ------------------------------------------------------------------ quantised projections
 * int4 group-wise weights, the reference's quantize_w4_groupwise format (rwkv7_hf/sm70_quant.py:502-519):
 * packed [Nout, K/2] u8 (low nibble = even k), scales [Nout, K/group] in `dtype`, optional zeros
 * [Nout, K/group] u8 (NULL = 8).  Replaces w4_groupwise_linear (:579) / MM4Linear(group_size=128).forward:
 *   out[M,Nout] = epilogue( x[M,K] . ((nibble - zero)*scale)^T ).  M <= 64 (decode GEMV regime). */
int rwkv7_w4g_gemv(const void* x, const uint8_t* packed, const void* scales, const uint8_t* zeros,
                   const void* residual, void* out, int M, int K, int Nout, int group, int epilogue,
                   int dtype, void* stream);

/* Tensor-core version of the same projection (any row count; one pass over the weights per 64 rows up to 64 rows, per
 * 128 rows above), reading a TILED
 * copy of the weights built once at load time by rwkv7_w4g_repack: one 8704-byte block per [128 channels x 128 k] tile
 * (packed nibbles, then that tile's fp16 scales and u8 zero-points), blocks of a channel tile consecutive, so each CTA
 * streams one contiguous region.  Same values, same arithmetic as above.  rwkv7_w4g_tiled_bytes returns the size of
 * the tiled buffer (0 for unsupported shapes).  fp16 only, K % 128 == 0.  No counterpart in the reference (its
 * group-wise format has no fused kernel off sm_70). */
int64_t rwkv7_w4g_tiled_bytes(int K, int Nout);
int rwkv7_w4g_repack(const uint8_t* packed, const void* scales, const uint8_t* zeros, uint8_t* tiled, int K, int Nout,
                     int group, int dtype, void* stream);
int rwkv7_w4g_gemv_tiled(const void* x, const uint8_t* tiled, const void* residual, void* out, int M, int K, int Nout,
                         int epilogue, int dtype, void* stream);
/* G (1..4) projections of the same shape in one launch, each with its own activations xs[g] [M,K], tiled weights and
 * output outs[g] [M,Nout] (the r / k / v projections of a layer: rwkv7_hf/native.py:208-211 calls them back to back on
 * different mixes of the same hidden state; the graph path groups them in _native_graph_rkv_project,
 * rwkv7_hf/native_jit_decode.py:175).  The three pointer arrays live in host memory and
 * are read during the call.  Epilogue none or relu^2. */
int rwkv7_w4g_gemv_tiled_group(const void* const* xs, const uint8_t* const* tiled, void* const* outs, int G, int M, int K,
                               int Nout, int epilogue, int dtype, void* stream);

/* Tensor-core version of the int8 per-output-channel projection below (rwkv7_w8_gemv), any row count, from a TILED copy
 * of q built once at load by rwkv7_w8_repack: one 16 KiB block per [128 channels x 128 k] tile, bytes stored as q + 128.
 * G (1..4) projections of one shape per launch (xs, tiled, scales, outs: host arrays of G device pointers; scales[g]
 * [Nout] fp16).  The integer weights enter the MMA exactly and the channel scale multiplies the fp32 accumulator, i.e.
 * out = epilogue(fp16(scale * (x . q^T))): the reference's materialised weight fp16(q * scale) (w8_linear,
 * rwkv7_hf/sm70_quant.py:522-531) differs from q * scale by one fp16 rounding per weight.  The add epilogue takes G = 1
 * and a residual.  fp16 only, K % 128 == 0.  rwkv7_w8_tiled_bytes returns the tiled size (0 = unsupported shape). */
int64_t rwkv7_w8_tiled_bytes(int K, int Nout);
int rwkv7_w8_repack(const int8_t* q, uint8_t* tiled, int K, int Nout, void* stream);
int rwkv7_w8_gemv_tiled_group(const void* const* xs, const uint8_t* const* tiled, const void* const* scales,
                              const void* residual, void* const* outs, int G, int M, int K, int Nout, int epilogue,
                              int dtype, void* stream);

/* int8 per-output-channel weights, quantize_w8_row format (rwkv7_hf/sm70_quant.py:485-489): q [Nout,K] i8,
 * scale [Nout] in `dtype`.  Replaces w8_linear (:522) / the W8A16 GEMV (native_quant_a8w8.py:50-132). */
int rwkv7_w8_gemv(const void* x, const int8_t* q, const void* scale, const void* residual, void* out,
                  int M, int K, int Nout, int epilogue, int dtype, void* stream);

/* Materialise the dense weight W[Nout,K] = (q - zero)*scale in `dtype`, for many-row (prefill) inputs where the
 * reference dequantises and calls a GEMM (w4_dequant, rwkv7_hf/sm70_quant.py:68-71,598-610; :522-531 for int8). */
int rwkv7_w4g_dequant(const uint8_t* packed, const void* scales, const uint8_t* zeros, void* W, int K, int Nout,
                      int group, int dtype, void* stream);
int rwkv7_w8_dequant(const int8_t* q, const void* scale, void* W, int K, int Nout, int dtype, void* stream);

/* Affine 8-bit ("fp16i8") and 4-bit weights in the reference's layouts (quantize_mm8,
 * rwkv7_hf/native_quant_mm8.py:62-97; quantize_mm4, rwkv7_hf/native_quant_mm4.py:77-108):
 *   W[k,n] = (q[k,n] + 0.5)*ry[k]*rx[n] + my[k] + mx[n],  q u8 [K,Nout] (bits 8) or two nibbles per byte
 *   [K,ceil(Nout/2)] (bits 4, low nibble = even n); mx,rx [Nout], my,ry [K] in `dtype`.
 * rwkv7_affine_gemv replaces mm8_gemv_triton / mm8_matmul_triton / mm4_matmul_triton (native_quant_mm8.py:147-215,
 * native_quant_mm4.py:150-330) for 1..8 rows (Nout % 8 == 0): one pass over the weight bytes, fp32 accumulation,
 * fixed summation order; workspace of rwkv7_affine_gemv_workspace_bytes bytes, 16-byte aligned.
 * rwkv7_affine_dequant replaces dequantize_mm8 / dequantize_mm4 (:100-107 / :111-125): W [K,Nout] in `dtype`, every
 * operation rounded to `dtype` in the reference's order, for the many-row route (dequantise, then one GEMM). */
int64_t rwkv7_affine_gemv_workspace_bytes(int M, int K, int Nout);
int rwkv7_affine_gemv(const void* x, const uint8_t* q, const void* mx, const void* rx, const void* my, const void* ry,
                      void* out, float* workspace, int64_t workspace_bytes, int M, int K, int Nout, int bits, int dtype,
                      void* stream);
int rwkv7_affine_dequant(const uint8_t* q, const void* mx, const void* rx, const void* my, const void* ry, void* W,
                         int K, int Nout, int bits, int dtype, void* stream);

/* Dynamic per-row int8 activation quantiser; replaces _dynamic_a8_quant_kernel
 * (rwkv7_hf/native_quant_a8w8.py:134-164) with IEEE fp32 division: s = max(amax/127, 1e-5),
 * q = clamp(round_half_away(x/s), +-127).  q [rows,K] i8, scale [rows] fp32. */
int rwkv7_a8_quant(const void* x, int8_t* q, float* scale, int rows, int K, int dtype, void* stream);

/* int8 x int8 -> int32 GEMM, bit-exact; replaces torch._int_mm (rwkv7_hf/native_quant_a8w8.py:413).
 * qa [M,K] i8 row-major; qw [Nout,K] i8 row-major (the transpose of the reference's q_weight_t);
 * acc [M,Nout] i32. */
int rwkv7_i8_gemm(const int8_t* qa, const int8_t* qw, int32_t* acc, int M, int K, int Nout, void* stream);

/* Dense fp16 / bf16 GEMM with a fused epilogue, for projections over many rows (prefill):
 *   c[M,N] = a[M,K] . b[N,K]^T (+ bias[N])  then  epilogue 0: (+ residual[M,N])   epilogue 1: relu(.)^2 of the rounded value
 * a = activations row-major, b = an nn.Linear weight [out,in]; fp32 accumulation; bias / residual / c in `dtype`.
 * Replaces the tl.dot GEMMs with fused mix / relu^2 / residual of rwkv7_hf/fused_ffn.py:39-232 and the F.linear calls
 * of the layer-wise prefill (rwkv7_hf/native_jit_prefill.py:964-1040).  K % 8 == 0. */
int rwkv7_gemm(const void* a, const void* b, const void* bias, const void* residual, void* c, int M, int K, int N,
               int epilogue, int dtype, void* stream);

/* The output head of a greedy decode step: arg-max over the columns of a[M,K] . b[N,K]^T without ever storing the
 * [M,N] logits (rwkv7_hf/native_jit_decode.py:953-1000 computes the head GEMM and then torch.argmax).  Values are
 * rounded to `dtype` before they are compared and the lowest column wins a tie, so best_index equals torch.argmax of
 * the stored logits.  best_value [M] fp32 may be NULL; best_index [M] int64; workspace of
 * rwkv7_gemm_argmax_workspace_bytes(M, N) bytes, 16-byte aligned. */
int64_t rwkv7_gemm_argmax_workspace_bytes(int M, int N);
int rwkv7_gemm_argmax(const void* a, const void* b, void* workspace, int64_t workspace_bytes, float* best_value,
                      long long* best_index, int M, int K, int N, int dtype, void* stream);

/* Dequant epilogue; replaces _a8w8_dequant_kernel / _a8w8_dequant_add_kernel
 * (rwkv7_hf/native_quant_a8w8.py:166-264): out = fp32(acc)*sa[row]*sw[col] (+bias) (+residual). */
int rwkv7_a8w8_dequant(const int32_t* acc, const float* sa, const float* sw, const void* bias,
                       const void* residual, void* out, int M, int Nout, int dtype, void* stream);

/* The boundary inside a8w8_ffn (rwkv7_hf/native_quant_a8w8.py:189-232, 436-524): per row, h = fp16(acc*sa*sw (+bias)),
 * r = fp16(max(h,0)^2), then the activation quantiser on r; the fp16 hidden activation is never written.  fp16 only. */
int rwkv7_a8w8_relu2_requant(const int32_t* acc, const float* sa, const float* sw, const void* bias, int8_t* q,
                             float* scale, int M, int N, int dtype, void* stream);

/* a8w8_linear (rwkv7_hf/native_quant_a8w8.py:323): quantise rows, integer GEMM, dequantise.  With 64 rows or more
 * the dequantisation runs in the epilogue of the tensor-core GEMM and the accumulators never reach memory.
 * workspace: caller-owned scratch of at least rwkv7_a8w8_workspace_bytes(M,K,Nout) bytes, 256-byte aligned. */
int64_t rwkv7_a8w8_workspace_bytes(int M, int K, int Nout);
int rwkv7_a8w8_linear(const void* x, const int8_t* qw, const float* sw, const void* bias, const void* residual,
                      void* out, void* workspace, int64_t workspace_bytes, int M, int K, int Nout, int dtype,
                      void* stream);

/* The FFN key projection of an A8W8 model: a8w8_linear followed by relu(.)^2 of the value rounded to `dtype`, the
 * activation in the same epilogue (rwkv7_hf/native_jit_prefill.py:964-975 probes rwkv7_forward_relu2 for it). */
int rwkv7_a8w8_linear_relu2(const void* x, const int8_t* qw, const float* sw, const void* bias, void* out,
                            void* workspace, int64_t workspace_bytes, int M, int K, int Nout, int dtype, void* stream);

/* rwkv7_a8w8_linear for callers that cannot allocate device memory when they call (a server that gave the whole
 * GPU to its own memory pool, a thread that must not enter the CUDA allocator, a host that forbids cudaMalloc inside
 * operators).  No counterpart in the reference.  The scratch is a fixed array of rwkv7_a8w8_static_capacity_bytes()
 * bytes (8 MiB) inside the library, held by every GPU that loads it; the call allocates nothing and returns
 * RWKV7_ERR_WORKSPACE when rwkv7_a8w8_workspace_bytes(M,K,Nout) exceeds that capacity.
 *   - The first call on each device looks up the array's device address (one runtime query, no allocation): make
 *     that first call before any stream capture.
 *   - All calls on a device share the one array, which keeps the previous call's contents; nothing in it needs
 *     clearing, but two calls that overlap on the GPU (different streams, no dependency) race on it. */
int64_t rwkv7_a8w8_static_capacity_bytes(void);
int rwkv7_a8w8_linear_static(const void* x, const int8_t* qw, const float* sw, const void* bias, const void* residual,
                             void* out, int M, int K, int Nout, int dtype, void* stream);

/* ------------------------------------------------------------------ tensor-parallel sum over peer memory
 * out[rows,D] = sum over the P ranks of partial[rows,D] (fp16, fp32 accumulation in rank order: bit-identical on every
 * rank): the all-reduce behind the row-sharded o_proj / ffn.value of a head-sharded layer (the reference's TP plan,
 * rwkv7_hf/model_config.py:37-53, uses the framework's all-reduce).  One kernel per GPU: plain peer stores into every
 * peer's inbox, per-CTA flags, bounded waits (wait_ms, default 2000; a wait that runs out sets the device error word,
 * see rwkv7_kernel_status, and the kernel returns without storing).
 *   inbox_ptrs / flag_ptrs: host arrays of P device pointers, entry r = rank r's inbox [2][P][slot_elems] fp16 and flag
 *   array [2][P][rwkv7_tp_allreduce_max_ctas()] u32 as mapped into THIS process (peer-mapped memory; zeroed, with a
 *   barrier, before the first call).  counters: two u32 in local memory, zeroed at set-up.  Every rank must issue the
 *   same sequence of calls with the same rows and D.  Calls that share inbox / flags / counters must not overlap on a GPU. */
int rwkv7_tp_allreduce_max_ctas(void);
int rwkv7_tp_allreduce(const void* partial, void* out, void* const* inbox_ptrs, void* const* flag_ptrs, void* counters,
                       int rank, int world, int rows, int D, long long slot_elems, int wait_ms, int dtype, void* stream);

/* The two row kernels that CONSUME those sums, with the sum inside them: `partial` is this rank's [rows,D] partial
 * output of o_proj (rwkv7_tp_ffn_add_norm_mix: residual_out = residual + sum, then as rwkv7_ffn_add_norm_mix) or of
 * ffn.value (rwkv7_tp_attn_norm_mix6: x_out = sum, then as rwkv7_attn_norm_mix6).  The CTA of a row pushes it to every
 * peer, polls (bounded, as above) for the peers' copies of that row, adds them in rank order and rounds the sum to the
 * storage type - the values rwkv7_tp_allreduce would have stored - before it normalises: one launch replaces the
 * all-reduce kernel, a [rows,D] round trip and a kernel boundary (the reference runs the framework's all-reduce and
 * then its fused norm kernels, rwkv7_hf/native_jit_decode.py:481-901 under rwkv7_hf/model_config.py:37-53).  On the
 * wire every 4 bytes of payload travel with the 4-byte call number in one aligned 8-byte unit, which arrives whole: a
 * unit that shows the call number holds this call's payload, so the exchange needs no fence and no separate flag.
 *   inbox_ptrs: host array of P device pointers, entry r = rank r's inbox as mapped into THIS process,
 *   2 * P * slot_elems * 4 bytes (two buffers, a slot per rank, 4 bytes per 2-byte payload value; zeroed, with a
 *   barrier, before the first call; not shared with rwkv7_tp_allreduce).  slot_elems: a multiple of 8, >= rows * D.
 *   counters: two u32 in local memory, zeroed at set-up.  slot_ids NULL or the state-pool rows of `prev`.
 *   The grid is min(rows, rwkv7_tp_rows_resident(D, dtype)) CTAs, CTA c taking rows c, c + grid, ...: a CTA pushes all
 *   of its rows before it waits for any and waits only for the peers' CTAs of its own index, so with the whole grid
 *   resident at once no CTA waits for one that cannot start.  max_ctas > 0 lowers the grid bound (callers that run two
 *   of these kernels side by side on two streams pass half of rwkv7_tp_rows_resident); 0 = no extra bound.
 *   fp16 or bf16.  The same-sequence and no-overlap rules above apply. */
int rwkv7_tp_rows_resident(int D, int dtype);
int rwkv7_tp_attn_norm_mix6(const void* partial, void* x_out, void* prev, const int32_t* slot_ids, const void* norm_w,
                            const void* norm_b, const void* const mixes[6], void* const outs[6], void* const* inbox_ptrs,
                            void* counters, int rank, int world, int rows, int D, long long slot_elems, int max_ctas,
                            float eps, int wait_ms, int dtype, void* stream);
int rwkv7_tp_ffn_add_norm_mix(const void* residual, const void* partial, void* prev, const int32_t* slot_ids,
                              const void* norm_w, const void* norm_b, const void* mix, void* residual_out, void* mixed,
                              void* const* inbox_ptrs, void* counters, int rank, int world, int rows, int D,
                              long long slot_elems, int max_ctas, float eps, int wait_ms, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RWKV7_B200_H */
