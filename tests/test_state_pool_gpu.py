"""The serving state pool against independent single-request runs through the ordinary cache: the correctness list
of the reference's serving ABI (docs/integrations/RWKV7_STATE_CACHE_ABI.md, "Correctness tests" 1-8, 10, 12) on
the tiny fp32 model, where the kernels read and write pool rows through slot ids."""
import pytest
import torch

import hf_adapter_b200 as hb
from tests.gpu_util import golden
from tests.test_model_gpu import load_tiny

pytestmark = pytest.mark.gpu
TOL = dict(rtol=2e-4, atol=2e-4)


@pytest.fixture(scope="module")
def model():
    return load_tiny(golden("model_tiny.npz"))


def solo(model, prompt, steps):
    """Reference behaviour: one request alone, ordinary cache.  Returns the logits after the prompt and after every
    following greedy token, and the cache."""
    out = model(prompt[None], logits_to_keep=1)
    cache, logits = out.past_key_values, [out.logits[0, -1]]
    for _ in range(steps):
        logits.append(model.rwkv7_forward_token(logits[-1].argmax()[None], cache, use_graph=False)[0])
    return logits, cache


def pool_rows(pool, slot):
    return (pool.S_pool[:, slot], pool.xpa_pool[:, slot], pool.xpf_pool[:, slot], pool.vfirst_pool[slot])


def cache_rows(cache, row=0):
    st, xpa, xpf, vf = cache
    return (torch.stack([s[row] for s in st]), torch.stack([x[row] for x in xpa]), torch.stack([x[row] for x in xpf]), vf[row])


def test_fresh_slot_is_a_fresh_cache_and_one_token_matches_every_component(model):
    pool = hb.RWKV7StatePool(model, 4)
    (s,), (gen,) = pool.allocate(["a"])
    for t in pool_rows(pool, s):
        assert not t.any()
    tok = torch.tensor([17], device="cuda")
    cache = model.new_cache(1)
    want = model.rwkv7_forward_token(tok, cache, use_graph=False)
    got = pool.decode(tok, [s], [gen], use_graph=False)
    torch.testing.assert_close(got, want, **TOL)
    for a, b in zip(pool_rows(pool, s), cache_rows(cache)):
        torch.testing.assert_close(a, b, **TOL)
    assert pool.seen_tokens[s] == 1


@pytest.mark.parametrize("use_graph", [False, True])
def test_dynamic_batch_equals_independent_requests(model, use_graph):
    """Requests join, leave and change row order between steps; every request's logits stay those of a solo run
    (tests 3, 4, 7, 12 of the ABI list: reorder, insertion / removal, padded graph rows, long mixed decode)."""
    torch.manual_seed(0)
    pool = hb.RWKV7StatePool(model, 6)
    prompts = {r: torch.randint(0, 256, (n,), device="cuda") for r, n in (("A", 5), ("B", 3), ("C", 7), ("D", 4), ("E", 6))}
    steps = 7
    want = {r: solo(model, p, steps)[0] for r, p in prompts.items()}
    slot, pos, last = {}, {}, {}

    def admit(r):
        (s,), _ = pool.allocate([r])
        slot[r], pos[r] = s, 0
        last[r] = pool.prefill(prompts[r][None], [s])[0]
        torch.testing.assert_close(last[r], want[r][0], **TOL)

    for r in "ABCD":
        admit(r)
    schedule = ["ABCD", "DCA", "ACD", "ACDE", "EA", "CAE", "A"]  # B leaves at once; E joins late; rows reorder
    admitted_e = False
    for rows in schedule:
        if "E" in rows and not admitted_e:
            pool.free([slot.pop("B")])
            admit("E")
            admitted_e = True
            assert slot["E"] not in [slot[r] for r in "ACD"]
        toks = torch.stack([last[r].argmax() for r in rows])
        before = {r: [t.clone() for t in pool_rows(pool, slot[r])] for r in slot if r not in rows}
        out = pool.decode(toks, [slot[r] for r in rows], use_graph=use_graph)
        for i, r in enumerate(rows):
            pos[r] += 1
            last[r] = out[i]
            torch.testing.assert_close(out[i], want[r][pos[r]], **TOL)
        for r, saved in before.items():  # unscheduled live slots did not move
            for a, b in zip(pool_rows(pool, slot[r]), saved):
                assert torch.equal(a, b)
    assert pool.seen_tokens[slot["A"]] == len(prompts["A"]) + 7
    st = pool.stats()
    assert st["allocated_slots"] == 4 and st["high_water"] == 4 and st["active_rows"] == 1
    if use_graph:
        assert st["graph_bucket_rows"] == 1 and sorted(k[0] for k in pool._graphs) == [1, 2, 4]


def test_fork_reset_and_stale_handles(model):
    pool = hb.RWKV7StatePool(model, 3)
    prompt = torch.randint(0, 256, (6,), device="cuda")
    (a, b), (ga, gb) = pool.allocate(["a", "b"])
    la = pool.prefill(prompt[None], [a])[0]
    pool.clone([a], [b])
    assert pool.seen_tokens[b] == 6 and pool.stats()["clones"] == 1
    # the fork continues independently: different next tokens give different states, the same token the same logits
    t0, t1 = la.argmax()[None], (la.argmax()[None] + 1) % 256
    oa = pool.decode(t0, [a], use_graph=False)
    ob = pool.decode(t1, [b], use_graph=False)
    assert not torch.allclose(oa, ob)
    pool.clone([a], [b])
    o2 = pool.decode(torch.cat([t0, t0]), [a, b], use_graph=False)
    torch.testing.assert_close(o2[0], o2[1], rtol=0, atol=0)
    # reset removes every trace of the previous request
    pool.reset([b])
    fresh = pool.decode(t0, [b], use_graph=False)
    want = model.rwkv7_forward_token(t0, model.new_cache(1), use_graph=False)
    torch.testing.assert_close(fresh, want, **TOL)
    # stale handles
    pool.free([b], [gb])
    with pytest.raises(hb.StaleSlotError):
        pool.decode(t0, [b], use_graph=False)
    (b2,), (gb2,) = pool.allocate(["c"])
    assert b2 == b and gb2 == gb + 1
    with pytest.raises(hb.StaleSlotError):
        pool.decode(t0, [b2], [gb], use_graph=False)
    assert not pool.S_pool[:, b2].any()  # the reassigned slot starts from zero
    with pytest.raises(ValueError, match="twice"):
        pool.decode(torch.cat([t0, t0]), [a, a], use_graph=False)
    assert pool.stats()["stale_generation_rejections"] == 2
    with pytest.raises(RuntimeError, match="exhausted"):
        pool.allocate(["x", "y"])
    assert pool.stats()["allocation_failures"] == 1


def test_prefix_hit_equals_full_prefill(model):
    pool = hb.RWKV7StatePool(model, 3, prefix_cache_bytes=1 << 20)
    torch.manual_seed(1)
    prefix, suffix = torch.randint(0, 256, (8,), device="cuda"), torch.randint(0, 256, (5,), device="cuda")
    (a, b, c), _ = pool.allocate(["a", "b", "c"])
    pool.prefill(prefix[None], [a])
    entry = pool.snapshot(a, prefix, offload=True)
    assert entry.state.device.type == "cpu" and entry.seen_tokens == 8 and pool.stats()["prefix_entries"] == 1
    full = torch.cat([prefix, suffix])
    want = pool.prefill(full[None], [b])
    got = pool.prefill(full[None], [c], use_prefix_cache=True)
    torch.testing.assert_close(got, want, **TOL)
    for x, y in zip(pool_rows(pool, c), pool_rows(pool, b)):
        torch.testing.assert_close(x, y, **TOL)
    st = pool.stats()
    assert st["prefix_hits"] == 1 and st["prefix_tokens_saved"] == 8 and st["prefix_bytes_restored"] == entry.nbytes
    assert pool.seen_tokens[c] == 13
    assert pool.lookup(torch.randint(0, 256, (4,)))[0] is None and pool.stats()["prefix_misses"] == 1
    with pytest.raises(ValueError, match="exactly the tokens"):
        pool.snapshot(a, prefix[:5])
    entry.xpa[0, 0] += 1  # a corrupted snapshot is refused
    with pytest.raises(ValueError, match="checksum"):
        pool.restore(entry, a)
    # eviction: a budget of one entry keeps the most recent
    small = hb.RWKV7StatePool(model, 2, prefix_cache_bytes=entry.nbytes + 8)
    (s,), _ = small.allocate(["s"])
    small.prefill(prefix[None], [s])
    small.snapshot(s, prefix)
    small.prefill(suffix[None], [s])
    small.snapshot(s, full)
    assert small.stats()["prefix_entries"] == 1 and small.stats()["prefix_evictions"] == 1
    assert small.lookup(full)[1] == 13


def test_pool_operators_leave_other_rows_untouched():
    """The three *_pool operators change exactly the rows named by slot_ids and agree with the dense operators."""
    torch.manual_seed(2)
    B, cap, D, H = 3, 7, 256, 4
    slots = torch.tensor([5, 0, 3], device="cuda", dtype=torch.int32)
    x = torch.randn(B, D, device="cuda").half()
    pool = torch.randn(cap, D, device="cuda").half()
    w, b_ = torch.rand(D, device="cuda").half(), torch.rand(D, device="cuda").half()
    mixes = [torch.rand(D, device="cuda").half() for _ in range(6)]
    dense_prev = pool[slots.long()].clone()
    want = hb.fused_attn_norm_mix6_decode(x, dense_prev, w, b_, *mixes)
    keep = pool.clone()
    got = hb.fused_attn_norm_mix6_decode(x, pool, w, b_, *mixes, slot_ids=slots)
    for a, c in zip(got, want):
        assert torch.equal(a, c)
    assert torch.equal(pool[slots.long()], dense_prev)
    others = [i for i in range(cap) if i not in slots.tolist()]
    assert torch.equal(pool[others], keep[others])
    # ffn add-norm-mix
    attn = torch.randn(B, D, device="cuda").half()
    dense_prev = pool[slots.long()].clone()
    wx, wm = hb.fused_ffn_add_norm_mix_decode(x, attn, dense_prev, w, b_, mixes[0])
    keep = pool.clone()
    gx, gm = hb.fused_ffn_add_norm_mix_decode(x, attn, pool, w, b_, mixes[0], slot_ids=slots)
    assert torch.equal(gx, wx) and torch.equal(gm, wm) and torch.equal(pool[slots.long()], dense_prev)
    assert torch.equal(pool[others], keep[others])
    # recurrence with v_first pools
    A = H * 64
    r, wr, k, v, a, g, vg = (torch.randn(B, A, device="cuda").half() for _ in range(7))
    kk, ka, rk = (torch.rand(A, device="cuda").half() for _ in range(3))
    gw, gb = torch.rand(A, device="cuda").half(), torch.rand(A, device="cuda").half()
    spool = 0.1 * torch.randn(cap, H, 64, 64, device="cuda")
    vpool = torch.randn(cap, A, device="cuda").half()
    dense_state, dense_vf = spool[slots.long()].clone(), vpool[slots.long()].clone()
    wo, ws = hb.fused_recurrent_output_prepare_raw(r, wr, k, v, a, dense_state, g, kk, ka, rk, gw, gb, eps=64e-5,
                                                   a_is_raw=True, v_first=dense_vf, v_gate=vg, v_gate_is_raw=True)
    keep_s = spool.clone()
    go, gs = hb.fused_recurrent_output_prepare_raw(r, wr, k, v, a, spool, g, kk, ka, rk, gw, gb, eps=64e-5, a_is_raw=True,
                                                   v_first=vpool, v_gate=vg, v_gate_is_raw=True, slot_ids=slots)
    assert gs is spool and torch.equal(go, wo) and torch.equal(spool[slots.long()], ws)
    assert torch.equal(spool[others], keep_s[others])
    keep_v = vpool.clone()
    hb.fused_recurrent_output_prepare_raw(r, wr, k, v, a, spool, g, kk, ka, rk, gw, gb, eps=64e-5, v_out=vpool, slot_ids=slots)
    assert torch.equal(vpool[slots.long()], v) and torch.equal(vpool[others], keep_v[others])
    with pytest.raises(ValueError):
        hb.fused_attn_norm_mix6_decode(x, pool, w, b_, *mixes, slot_ids=slots.long())
