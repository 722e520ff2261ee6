"""Generate the golden fixtures in this folder from the reference itself.

Run where the reference project is importable (it is a pure-Python package
whose operators all have a ``force_fallback=True`` pure-torch branch that
runs on CPU):

    python tests/golden/make_golden.py --reference /path/to/hf-adapter

Outputs ``ops_fp32.npz``, ``ops_fp16.npz``, ``quant.npz``, ``model_tiny.npz``, ``model_masked.npz``,
``config1.npz`` and ``a8w8_ffn.npz`` next to this script (``--only`` selects a subset).  The fixtures hold the seeded inputs
AND the reference's outputs, so the parity tests never need the reference at
run time.  All shapes are small (N=64 heads, a few rows) to keep every file
well under a megabyte.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def npy(t):
    if isinstance(t, torch.Tensor):
        return t.detach().cpu().numpy()
    return np.asarray(t)


def gen_ops(dtype, seed):
    from rwkv7_hf import fused_recurrent_update as fru
    from rwkv7_hf import fused_decode_norm_mix as fdn
    from rwkv7_hf import fused_lora as fl
    from rwkv7_hf import fused_prefill as fp
    from rwkv7_hf import fused_output as fo
    from rwkv7_hf import fused_time_mix as ftm
    from rwkv7_hf import dplr_prefill as dp

    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    B, T, H, N, D = 2, 32, 2, 64, 128
    A = H * N
    out = {}

    # ---- single step ----------------------------------------------------
    r, k, v = (rn(B, H, N).to(dtype) for _ in range(3))
    kk = torch.nn.functional.normalize(rn(B, H, N), dim=-1).to(dtype)
    a = torch.sigmoid(rn(B, H, N)).to(dtype)
    w = torch.exp(-0.606531 * torch.sigmoid(rn(B, H, N)))  # fp32 decay
    state = rn(B, H, N, N) * 0.5
    gate = rn(B, H, N).to(dtype)
    r_k = (rn(H, N) * 0.1).to(dtype)
    gn_w = (1 + 0.1 * rn(A)).to(dtype)
    gn_b = (0.1 * rn(A)).to(dtype)
    eps = N * 1e-5
    y, s1 = fru.torch_recurrent_update(r, w, k, v, kk, a, state)
    out.update(step_r=r, step_w=w, step_k=k, step_v=v, step_kk=kk, step_a=a, step_state=state,
               step_y=y, step_state_out=s1)
    yp, s2 = fru.torch_recurrent_output_prepare(r, w, k, v, kk, a, state, gate, r_k, gn_w, gn_b, eps=eps)
    out.update(step_g=gate, step_r_k=r_k, step_gn_w=gn_w, step_gn_b=gn_b, prep_y=yp, prep_state_out=s2)
    w_raw, k_raw = rn(B, H, N).to(dtype), rn(B, H, N).to(dtype)
    k_k = (0.85 + 0.1 * rn(A)).to(dtype)
    k_a = (1 + 0.1 * rn(A)).to(dtype)
    yr, s3 = fru.fused_recurrent_output_prepare_raw(
        r, w_raw, k_raw, v, a, state, gate, k_k, k_a, r_k, gn_w, gn_b, eps=eps, force_fallback=True)
    out.update(raw_w=w_raw, raw_k=k_raw, raw_k_k=k_k, raw_k_a=k_a, raw_y=yr, raw_state_out=s3)

    # ---- scans ------------------------------------------------------------
    rs, ks, vs = (rn(B, T, H, N).to(dtype) for _ in range(3))
    kks = torch.nn.functional.normalize(ks.float(), dim=-1).to(dtype)
    as_ = torch.sigmoid(rn(B, T, H, N)).to(dtype)
    ws = torch.exp(-0.606531 * torch.sigmoid(rn(B, T, H, N)))
    s0 = rn(B, H, N, N) * 0.1
    ys, sT = fru.torch_recurrent_scan(rs, ws, ks, vs, kks, as_, s0)
    out.update(scan_r=rs, scan_w=ws, scan_k=ks, scan_v=vs, scan_kk=kks, scan_a=as_, scan_state=s0,
               scan_y=ys, scan_state_out=sT)
    yc, sc = dp.dplr_chunk_scan(rs, ws, ks, vs, kks, as_, s0, chunk_size=16, algorithm="wy")
    out.update(chunk_y=yc, chunk_state_out=sc)
    yso, sso = fru.torch_recurrent_scan_output_prepare(
        rs, ws, ks, vs, kks, as_, s0, rn(B, T, H, N).to(dtype), r_k, gn_w, gn_b, eps=eps)
    # regenerate the gate deterministically for the file
    g2 = torch.Generator().manual_seed(seed + 1)
    gate_s = torch.randn(B, T, H, N, generator=g2).to(dtype)
    yso, sso = fru.torch_recurrent_scan_output_prepare(rs, ws, ks, vs, kks, as_, s0, gate_s, r_k, gn_w, gn_b, eps=eps)
    out.update(scan_g=gate_s, scanprep_y=yso, scanprep_state_out=sso)

    # ---- norm / mix -------------------------------------------------------
    x = rn(3, D).to(dtype)
    prev = rn(3, D).to(dtype)
    nw, nb = (1 + 0.1 * rn(D)).to(dtype), (0.1 * rn(D)).to(dtype)
    mixes = [torch.rand(D, generator=g).to(dtype) for _ in range(6)]
    prev_mut = prev.clone()
    outs = fdn.fused_attn_norm_mix6_decode(x, prev_mut, nw, nb, *mixes, force_fallback=True)
    out.update(mix_x=x, mix_prev=prev, mix_nw=nw, mix_nb=nb, mix_mixes=torch.stack(mixes),
               mix_outs=torch.stack(list(outs)), mix_prev_out=prev_mut)
    attn_o = rn(3, D).to(dtype)
    prev_mut2 = prev.clone()
    res_out, mixed = fdn.fused_ffn_add_norm_mix_decode(x, attn_o, prev_mut2, nw, nb, mixes[0], force_fallback=True)
    out.update(ffnmix_attn=attn_o, ffnmix_res_out=res_out, ffnmix_mixed=mixed, ffnmix_prev_out=prev_mut2)
    xs = rn(B, 5, D).to(dtype)
    init_prev = rn(B, D).to(dtype)
    seq = ftm.fused_attn_sequence_shift_mix(xs, init_prev, *mixes)
    out.update(seqmix_x=xs, seqmix_prev=init_prev, seqmix_outs=torch.stack(list(seq[:6])), seqmix_next=seq[6])

    # ---- LoRA -------------------------------------------------------------
    Rw, Ra, Rg, Rv = 16, 16, 32, 8
    xw, xa, xg, xv = (rn(3, D).to(dtype) for _ in range(4))
    sc_ = 0.1
    downs = [(sc_ * rn(R, D)).to(dtype) for R in (Rw, Ra, Rg, Rv)]
    ups = [(sc_ * rn(A, R)).to(dtype) for R in (Rw, Ra, Rg, Rv)]
    wb, ab, vb = (rn(A) * 0.5).to(dtype), (rn(A) * 0.5).to(dtype), (rn(A) * 0.5).to(dtype)
    lw, la, lg, lv = fl.fused_wavg_lora(
        xw, xa, xg, xv, downs[0], downs[1], downs[2], downs[3], ups[0], ups[1], ups[2], ups[3],
        wb, ab, None, vb, force_fallback=True)
    out.update(lora_xw=xw, lora_xa=xa, lora_xg=xg, lora_xv=xv,
               lora_wd=downs[0], lora_ad=downs[1], lora_gd=downs[2], lora_vd=downs[3],
               lora_wu=ups[0], lora_au=ups[1], lora_gu=ups[2], lora_vu=ups[3],
               lora_wb=wb, lora_ab=ab, lora_vb=vb, lora_w=lw, lora_a=la, lora_g=lg, lora_vgate=lv)

    # ---- state prep / output prep ----------------------------------------
    rows = 5
    w_r, k_r, v_r = (rn(rows, A).to(dtype) for _ in range(3))
    a_in = torch.sigmoid(rn(rows, A)).to(dtype)
    vf = rn(rows, A).to(dtype)
    vg = torch.sigmoid(rn(rows, A)).to(dtype)
    pw, pk, pv, pkk = fp.fused_prefill_state_prep(
        w_r, k_r, v_r, a_in, k_k, k_a, v_first=vf, v_gate=vg, num_heads=H, head_dim=N, force_fallback=True)
    out.update(sp_w_raw=w_r, sp_k_raw=k_r, sp_v_raw=v_r, sp_a=a_in, sp_vf=vf, sp_vg=vg,
               sp_w=pw, sp_k=pk, sp_v=pv, sp_kk=pkk)
    rec = rn(rows, A).to(dtype)
    rr, kq, vq, gq = (rn(rows, A).to(dtype) for _ in range(4))
    op = fo.fused_attn_output_prepare(rec, rr.view(rows, H, N), kq.view(rows, H, N), vq.view(rows, H, N),
                                      gq, r_k, gn_w, gn_b, num_heads=H, head_dim=N,
                                      head_v_dim=N, eps=eps, force_fallback=True)
    out.update(op_rec=rec, op_r=rr, op_k=kq, op_v=vq, op_g=gq, op_out=op)

    # ---- later additions (drawn after everything above so the earlier entries keep their values) ----------
    from rwkv7_hf import fused_ffn as ff
    ok_, ov_, okk_ = fp.fused_prefill_kv_kk_prep(k_r, v_r, a_in, k_k, k_a, v_first=vf, v_gate=vg, num_heads=H,
                                                  head_dim=N, force_fallback=True)
    out.update(kvkk_k=ok_, kvkk_v=ov_, kvkk_kk=okk_)
    a_seq = torch.sigmoid(rn(B, T, H, N)).to(dtype)
    w_seq, k_seq, v_seq = (rn(B, T, H, N).to(dtype) for _ in range(3))
    vf_seq, vg_seq = rn(B, T, H, N).to(dtype), torch.sigmoid(rn(B, T, H, N)).to(dtype)
    so, sst, sk, sv = fru.fused_recurrent_scan_state_prep(rs, w_seq, k_seq, v_seq, a_seq, s0, k_k, k_a, v_first=vf_seq,
                                                          v_gate=vg_seq, force_fallback=True)
    out.update(ssp_w_raw=w_seq, ssp_k_raw=k_seq, ssp_v_raw=v_seq, ssp_a=a_seq, ssp_vf=vf_seq, ssp_vg=vg_seq,
               ssp_y=so, ssp_state_out=sst, ssp_k=sk, ssp_v=sv)
    ow = (0.05 * rn(D, A)).to(dtype)
    ob = (0.1 * rn(D)).to(dtype)
    opj = fo.fused_attn_output_project(rec, rr.view(rows, H, N), kq.view(rows, H, N), vq.view(rows, H, N), gq, r_k,
                                       gn_w, gn_b, ow, ob, num_heads=H, head_dim=N, head_v_dim=N, eps=eps,
                                       force_fallback=True)
    out.update(oproj_w=ow, oproj_b=ob, oproj_out=opj)
    Fi = 256
    kw_, vw_ = (0.05 * rn(Fi, D)).to(dtype), (0.05 * rn(D, Fi)).to(dtype)
    fx, fprev = rn(3, D).to(dtype), rn(3, D).to(dtype)
    fo1, fn1 = ff.fused_ffn(fx, fprev, mixes[0], kw_, vw_, force_fallback=True)
    fxs, fps = rn(B, 5, D).to(dtype), rn(B, D).to(dtype)
    fo2, fn2 = ff.fused_sequence_ffn(fxs, fps, mixes[0], kw_, vw_, force_fallback=True)
    out.update(ffn_key=kw_, ffn_value=vw_, ffn_x=fx, ffn_prev=fprev, ffn_out=fo1, ffn_next=fn1,
               sffn_x=fxs, sffn_prev=fps, sffn_out=fo2, sffn_next=fn2)
    return {k_: npy(v_) for k_, v_ in out.items()}


def gen_quant(seed):
    from rwkv7_hf import sm70_quant as sq
    from rwkv7_hf import native_quant_a8w8 as a8
    from rwkv7_hf import native_quant_mm8 as m8

    g = torch.Generator().manual_seed(seed)
    O, K = 96, 256
    W = (0.02 * torch.randn(O, K, generator=g)).half()
    x = torch.randn(5, K, generator=g).half()
    out = dict(W=W, x=x)
    q8, s8 = sq.quantize_w8_row(W)
    out.update(w8_q=q8, w8_s=s8, w8_y=sq.w8_linear(x, q8, s8))
    p4, s4, _ = sq.quantize_w4_groupwise(W, 128)
    out.update(w4g_packed=p4, w4g_scales=s4, w4g_y=sq.w4_groupwise_linear(x, p4, s4, O, K, group_size=128))
    qt, st = a8.quantize_weight_per_channel_int8(W)
    out.update(a8w8_q_t=qt, a8w8_s=st, a8w8_y=a8.a8w8_linear(x, qt, st))
    Wt = W.float().t().contiguous()  # [K, O]
    u8, mx, rx, my, ry = m8.quantize_mm8(Wt)
    out.update(mm8_u8=u8, mm8_mx=mx, mm8_rx=rx, mm8_my=my, mm8_ry=ry,
               mm8_y=m8.mm8_matmul(x.float(), u8, mx, rx, my, ry))
    # the formats as the modules store them (fp16 scales), the dequantised fp16 weight with the reference's operation
    # order, and the 4-bit affine format (even and odd output widths)
    from rwkv7_hf import native_quant_mm4 as m4
    Wh = W.t().contiguous()  # fp16 [K, O]
    u8h, mxh, rxh, myh, ryh = m8.quantize_mm8(Wh)
    out.update(mm8h_u8=u8h, mm8h_mx=mxh, mm8h_rx=rxh, mm8h_my=myh, mm8h_ry=ryh,
               mm8h_W=m8.dequantize_mm8(u8h, mxh, rxh, myh, ryh), mm8h_y=m8.mm8_matmul(x, u8h, mxh, rxh, myh, ryh))
    p4a, mx4, rx4, my4, ry4, mo, mp = m4.quantize_mm4(Wh)
    out.update(mm4a_packed=p4a, mm4a_mx=mx4, mm4a_rx=rx4, mm4a_my=my4, mm4a_ry=ry4,
               mm4a_W=m4.dequantize_mm4(p4a, mx4, rx4, my4, ry4, mo), mm4a_y=m4.mm4_matmul(x, p4a, mx4, rx4, my4, ry4, mo))
    Wodd = Wh[:, :95].contiguous()
    p4o, mxo, rxo, myo, ryo, moo, mpo = m4.quantize_mm4(Wodd)
    out.update(mm4o_packed=p4o, mm4o_mx=mxo, mm4o_rx=rxo, mm4o_my=myo, mm4o_ry=ryo,
               mm4o_W=m4.dequantize_mm4(p4o, mxo, rxo, myo, ryo, moo))
    return {k_: npy(v_) for k_, v_ in out.items()}


def reinit_degenerate(model, seed):
    """The reference constructs the token-shift / key-scale parameters as zeros,
    which makes the delta-rule term vanish; re-initialise them (seeded) so the
    fixture exercises every term."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for i, layer in enumerate(model.model.layers):
            at = layer.attn
            for nme in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"):
                getattr(at, nme).copy_(torch.rand(getattr(at, nme).shape, generator=g))
            at.k_k.copy_(0.85 + 0.1 * torch.randn(at.k_k.shape, generator=g))
            at.k_a.copy_(1.0 + 0.1 * torch.randn(at.k_a.shape, generator=g))
            at.r_k.copy_(0.1 * torch.randn(at.r_k.shape, generator=g))
            at.w_lora.lora[2].bias.copy_(-5 + 4 * torch.rand(at.w_lora.lora[2].bias.shape, generator=g))
            at.a_lora.lora[2].bias.copy_(0.5 * torch.randn(at.a_lora.lora[2].bias.shape, generator=g))
            if i != 0:
                at.v_lora.lora[2].bias.copy_(0.5 * torch.randn(at.v_lora.lora[2].bias.shape, generator=g))
            at.g_norm.weight.copy_(1 + 0.1 * torch.randn(at.g_norm.weight.shape, generator=g))
            at.g_norm.bias.copy_(0.1 * torch.randn(at.g_norm.bias.shape, generator=g))
            layer.ffn.x_k.copy_(torch.rand(layer.ffn.x_k.shape, generator=g))
            for ln in (layer.attn_norm, layer.ffn_norm) + ((layer.pre_norm,) if i == 0 else ()):
                ln.weight.copy_(1 + 0.1 * torch.randn(ln.weight.shape, generator=g))
                ln.bias.copy_(0.1 * torch.randn(ln.bias.shape, generator=g))


def gen_model(seed):
    from rwkv7_hf import NativeRWKV7Config, NativeRWKV7ForCausalLM
    from rwkv7_hf import native

    cfg = NativeRWKV7Config(vocab_size=256, hidden_size=128, num_hidden_layers=2, num_heads=2, head_dim=64,
                            intermediate_size=256, decay_low_rank_dim=16, a_low_rank_dim=16,
                            v_low_rank_dim=8, gate_low_rank_dim=32)
    torch.manual_seed(seed)
    model = NativeRWKV7ForCausalLM(cfg).eval().float()
    reinit_degenerate(model, seed + 1)
    out = {}
    sd = model.state_dict()
    for name, t in sd.items():
        out["param::" + name] = npy(t)
    g = torch.Generator().manual_seed(seed + 2)
    ids = torch.randint(0, 256, (2, 9), generator=g)
    with torch.no_grad():
        logits, state, xpa, xpf, v_first = native.native_prefill_batched(model, ids)
        out.update(ids=ids, prefill_logits=logits)
        toks = []
        tok = logits.argmax(-1)
        for _ in range(4):
            toks.append(tok)
            logits, state, xpa, xpf, v_first = native.native_decode_step_batched(model, tok, state, xpa, xpf, v_first)
            tok = logits.argmax(-1)
        out.update(greedy=torch.stack(toks, 1), final_logits=logits,
                   final_state=torch.stack(state), final_xpa=torch.stack(xpa), final_xpf=torch.stack(xpf),
                   final_v_first=v_first)
        # HF-level API: forward with cache and generate must agree with the loop above
        o = model(ids, use_cache=True)
        out["hf_forward_last_logits"] = o.logits[:, -1]
        gen = model.generate(ids, max_new_tokens=4, do_sample=False)
        out["hf_generate"] = gen
    return {k_: npy(v_) for k_, v_ in out.items()}


def gen_model_masked(seed):
    """The Hugging Face surface of the reference on the tiny model of ``gen_model`` (same seeds, so the weights are
    those of model_tiny.npz): a batch with masked positions (left padding, a hole, a masked first token), the same
    through ``inputs_embeds``, and a cached continuation that passes the full-length mask."""
    from rwkv7_hf import NativeRWKV7Config, NativeRWKV7ForCausalLM

    cfg = NativeRWKV7Config(vocab_size=256, hidden_size=128, num_hidden_layers=2, num_heads=2, head_dim=64,
                            intermediate_size=256, decay_low_rank_dim=16, a_low_rank_dim=16,
                            v_low_rank_dim=8, gate_low_rank_dim=32)
    torch.manual_seed(seed)
    model = NativeRWKV7ForCausalLM(cfg).eval().float()
    reinit_degenerate(model, seed + 1)
    g = torch.Generator().manual_seed(seed + 5)
    ids = torch.randint(0, 256, (3, 7), generator=g)
    mask = torch.tensor([[0, 0, 0, 1, 1, 1, 1], [1, 1, 1, 1, 1, 1, 1], [0, 1, 1, 0, 1, 1, 1]])
    out = dict(ids=ids, mask=mask)
    with torch.no_grad():
        o = model(ids, attention_mask=mask, use_cache=True)
        st, xpa, xpf, vf = o.past_key_values
        out.update(logits=o.logits, state=torch.stack(list(st)), xpa=torch.stack(list(xpa)), xpf=torch.stack(list(xpf)), v_first=vf,
                   seen=np.int64(o.past_key_values.get_seq_length()))
        emb = model.model.embeddings(ids)
        oe = model(inputs_embeds=emb, attention_mask=mask, use_cache=True)
        out["embeds_logits"] = oe.logits
        # continuation: two more tokens with the mask grown to the full length (the second new token of row 0 masked)
        more = torch.randint(0, 256, (3, 2), generator=g)
        mask2 = torch.cat([mask, torch.tensor([[1, 0], [1, 1], [1, 1]])], dim=1)
        o2 = model(more, attention_mask=mask2, past_key_values=o.past_key_values, use_cache=True)
        st2, _, _, _ = o2.past_key_values
        out.update(more=more, mask2=mask2, more_logits=o2.logits, more_state=torch.stack(list(st2)),
                   more_seen=np.int64(o2.past_key_values.get_seq_length()))
    return {k_: (v_ if isinstance(v_, np.generic) else npy(v_)) for k_, v_ in out.items()}


def gen_config1(seed, weight_seed):
    """The 0.1B-shape model (12 layers, d_model 768, 12 heads of 64, FFN 3072, vocabulary 65536, LoRA ranks
    64/64/32/128) in fp32 on the reference's CPU path: a 512-token random prompt through ``forward`` (eager prefill),
    then 128 greedy steps through the cached decode.  The weights come from ``seeded_weights.seeded_state_dict``
    (``weight_seed``: chosen among a few so that no greedy step is a near-tie between its two best logits) and are
    not stored; the fixture keeps their checksum, the prompt, the last-token logits, the greedy tokens with the
    top-1 / top-2 logit gap of every step, and norms of the final cache."""
    from rwkv7_hf import NativeRWKV7Config, NativeRWKV7ForCausalLM
    sys.path.insert(0, HERE)
    from seeded_weights import checksum, seeded_state_dict

    cfg = NativeRWKV7Config(vocab_size=65536, hidden_size=768, num_hidden_layers=12, num_heads=12, head_dim=64,
                            intermediate_size=3072, decay_low_rank_dim=64, a_low_rank_dim=64, v_low_rank_dim=32,
                            gate_low_rank_dim=128)
    torch.manual_seed(seed)
    model = NativeRWKV7ForCausalLM(cfg).eval().float()
    sd = seeded_state_dict({k: v.shape for k, v in model.state_dict().items()}, weight_seed)
    model.load_state_dict(sd)
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 65536, (1, 512), generator=g)
    out = dict(ids=ids, weight_seed=np.int64(weight_seed), weights_checksum=checksum(sd))
    with torch.no_grad():
        o = model(ids, use_cache=True, logits_to_keep=1)
        logits = o.logits[:, -1]
        cache = o.past_key_values
        out["prefill_logits"] = logits
        toks, gaps, tops = [], [], []
        for _ in range(128):
            top2 = logits.topk(2, dim=-1)
            tok = top2.indices[:, 0]
            toks.append(tok)
            tops.append(top2.values[:, 0])
            gaps.append(top2.values[:, 0] - top2.values[:, 1])
            o = model(tok[:, None], past_key_values=cache, use_cache=True)
            logits, cache = o.logits[:, -1], o.past_key_values
        state, xpa, xpf, v_first = tuple(cache)[:4]
        out.update(greedy=torch.stack(toks, 1), top1=torch.stack(tops, 1), top2_gap=torch.stack(gaps, 1),
                   final_logits=logits,
                   final_state_norm=torch.stack([s.double().norm() for s in state]),
                   final_xpa_norm=torch.stack([s.double().norm() for s in xpa]),
                   final_xpf_norm=torch.stack([s.double().norm() for s in xpf]),
                   final_state_l11_h0=state[-1][0, 0], final_v_first=v_first)
    return {k_: npy(v_) for k_, v_ in out.items()}


def gen_a8w8_ffn(seed):
    """The reference's A8W8 FFN pair on its CPU route: ``a8w8_linear`` falls back to the dequantised dense weight off
    CUDA (rwkv7_hf/native_quant_a8w8.py:345-351), so up -> relu^2 (fp16) -> down + residual here is the weight-only
    composition that the fused GPU path approximates; the reference gates the two at cosine >= 0.999
    (tests/test_native_quant_a8w8.py:63,92)."""
    from rwkv7_hf import native_quant_a8w8 as a8

    g = torch.Generator().manual_seed(seed)
    M, D, Fi = 19, 128, 512
    x = torch.randn(M, D, generator=g).half()
    res = torch.randn(M, D, generator=g).half()
    Wu = (0.05 * torch.randn(Fi, D, generator=g)).half()
    Wd = (0.05 * torch.randn(D, Fi, generator=g)).half()
    qu, su = a8.quantize_weight_per_channel_int8(Wu)
    qd, sd_ = a8.quantize_weight_per_channel_int8(Wd)
    h = a8.a8w8_linear(x, qu, su)
    h = torch.relu(h) ** 2
    y = a8.a8w8_linear(h, qd, sd_) + res
    return {k_: npy(v_) for k_, v_ in dict(x=x, res=res, Wu=Wu, Wd=Wd, su=su, sd=sd_, hidden=h, y=y).items()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the hf-adapter checkout")
    ap.add_argument("--only", default="", help="comma-separated subset of: ops,quant,model_tiny,model_masked,config1,a8w8_ffn")
    ap.add_argument("--config1-weight-seed", type=int, default=3)
    ap.add_argument("--out", default=HERE, help="output folder (default: next to this script)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_num_threads(4)
    only = {s for s in args.only.split(",") if s}
    want = lambda name: not only or name in only
    save = lambda name, d: np.savez_compressed(os.path.join(args.out, name), **d)
    if want("ops"):
        save("ops_fp32.npz", gen_ops(torch.float32, 7007))
        save("ops_fp16.npz", gen_ops(torch.float16, 7008))
    if want("quant"):
        save("quant.npz", gen_quant(11))
    if want("model_tiny"):
        save("model_tiny.npz", gen_model(0))
    if want("model_masked"):
        save("model_masked.npz", gen_model_masked(0))
    if want("config1"):
        save("config1.npz", gen_config1(0, args.config1_weight_seed))
    if want("a8w8_ffn"):
        save("a8w8_ffn.npz", gen_a8w8_ffn(21))
    for f in sorted(os.listdir(args.out)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(args.out, f)))


if __name__ == "__main__":
    main()
