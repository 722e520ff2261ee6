"""Greedy speculative decoding for one sequence (the reference's ``rwkv7_speculative_generate``,
rwkv7_hf/model_speculative.py:10-231): a small draft model proposes a block of tokens, the target model checks the
whole block in ONE layer-wise prefill, and the longest agreeing prefix is kept, so the result is exactly the target
model's own greedy continuation whatever the draft proposes.

A recurrent state cannot be rolled back, so both models keep a snapshot of their cache at the block boundary
(``NativeRWKV7Cache.clone``) and, after a rejected proposal, re-advance from it over the accepted tokens plus the
target's correction -- a resync of at most ``draft_tokens`` tokens instead of the whole prefix.  The statistics
dictionary has the reference's keys.
"""
from __future__ import annotations

import torch


def _new_stats():
    return {"generated_tokens": 0, "proposed_tokens": 0, "accepted_tokens": 0, "corrected_tokens": 0, "resyncs": 0,
            "resync_tokens": 0, "full_resync_tokens": 0, "resync_saved_tokens": 0, "target_forward_calls": 0,
            "draft_forward_calls": 0, "acceptance_rate": None}


@torch.no_grad()
def rwkv7_speculative_generate(model, input_ids, draft_model, max_new_tokens: int = 32, draft_tokens: int = 4,
                               eos_token_id=None, return_stats: bool = False, logits_to_keep: int = 1, **forward_kwargs):
    if draft_model is None:
        raise ValueError("rwkv7_speculative_generate requires a draft_model")
    if model.training or getattr(draft_model, "training", False):
        raise RuntimeError("rwkv7_speculative_generate is inference-only; call model.eval() first")
    if input_ids.dim() != 2 or int(input_ids.shape[0]) != 1:
        raise ValueError("rwkv7_speculative_generate currently supports input_ids shaped [1, seq]")
    if int(input_ids.shape[1]) <= 0:
        raise ValueError("rwkv7_speculative_generate requires at least one prompt token")
    max_new_tokens, draft_tokens = int(max_new_tokens), int(draft_tokens)
    if max_new_tokens < 0:
        raise ValueError("max_new_tokens must be non-negative")
    if draft_tokens <= 0:
        raise ValueError("draft_tokens must be positive")
    stats = _new_stats()
    if max_new_tokens == 0:
        return {"sequences": input_ids, "stats": stats} if return_stats else input_ids
    eos = set() if eos_token_id is None else ({int(eos_token_id)} if isinstance(eos_token_id, int) else {int(v) for v in eos_token_id})

    def advance(m, who, tokens, cache, keep=1):
        """Run ``tokens [1,n]`` through ``m`` continuing ``cache`` (None = fresh); returns (logits [1,keep,V], cache)."""
        stats[who + "_forward_calls"] += 1
        out = m(tokens, past_key_values=cache, use_cache=True, logits_to_keep=keep)
        return out.logits, out.past_key_values

    prompt_len = int(input_ids.shape[1])
    logits, target_cache = advance(model, "target", input_ids, None)
    target_next = int(logits[0, -1].argmax())
    logits, draft_cache = advance(draft_model, "draft", input_ids, None)
    draft_next = int(logits[0, -1].argmax())
    out_tokens: list[int] = []
    dev = input_ids.device
    row = lambda toks: torch.tensor([toks], device=dev, dtype=input_ids.dtype)

    while len(out_tokens) < max_new_tokens:
        block = min(draft_tokens, max_new_tokens - len(out_tokens))
        target_mark, draft_mark = target_cache.clone(), draft_cache.clone()  # the block boundary, for a resync
        proposals = []
        for _ in range(block):
            proposals.append(draft_next)
            logits, draft_cache = advance(draft_model, "draft", row([draft_next]), draft_cache)
            draft_next = int(logits[0, -1].argmax())
        stats["proposed_tokens"] += block
        # one prefill of the target over the whole block: its prediction after every proposed token
        verify, target_cache = advance(model, "target", row(proposals), target_cache, keep=block)
        expected = [target_next] + [int(t) for t in verify[0, :-1].argmax(-1)]
        agree = 0
        while agree < block and proposals[agree] == expected[agree]:
            agree += 1
        hit_eos = next((i for i, t in enumerate(proposals[:agree]) if t in eos), None)
        if hit_eos is not None:
            agree = hit_eos + 1
        out_tokens.extend(proposals[:agree])
        stats["accepted_tokens"] += agree
        if hit_eos is not None or len(out_tokens) >= max_new_tokens:
            break
        if agree == block:
            target_next = int(verify[0, -1].argmax())
            continue
        # first disagreement: the target's own token replaces it, and both caches restart from the block boundary
        correction = expected[agree]
        out_tokens.append(correction)
        stats["corrected_tokens"] += 1
        if correction in eos or len(out_tokens) >= max_new_tokens:
            break
        repair = row(proposals[:agree] + [correction])
        logits, target_cache = advance(model, "target", repair, target_mark)
        target_next = int(logits[0, -1].argmax())
        logits, draft_cache = advance(draft_model, "draft", repair, draft_mark)
        draft_next = int(logits[0, -1].argmax())
        stats["resyncs"] += 1
        stats["resync_tokens"] += int(repair.shape[1])
        stats["full_resync_tokens"] += prompt_len + len(out_tokens)
        stats["resync_saved_tokens"] = max(0, stats["full_resync_tokens"] - stats["resync_tokens"])

    stats["generated_tokens"] = len(out_tokens)
    if stats["proposed_tokens"]:
        stats["acceptance_rate"] = stats["accepted_tokens"] / stats["proposed_tokens"]
    sequences = torch.cat([input_ids, row(out_tokens)], dim=1) if out_tokens else input_ids
    return {"sequences": sequences, "stats": stats} if return_stats else sequences
