"""Head-sharded tensor parallelism on GPUs (needs >= 2 devices; skipped otherwise): two NCCL ranks load their shard
of the reference's tiny model into RWKV7ForCausalLM(tp_world=2) and must reproduce the reference logits / greedy
tokens through prefill, eager decode and CUDA-graph decode (all-reduce captured in the graph)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q, mode):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import hf_adapter_b200 as hb

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = dict(np.load(os.path.join(ROOT, "tests", "golden", "model_tiny.npz")))
        full = {k[len("param::"):]: torch.from_numpy(v) for k, v in g.items() if k.startswith("param::")}
        cfg = hb.NativeRWKV7Config(vocab_size=256, hidden_size=128, num_hidden_layers=2, num_heads=2, head_dim=64,
                                   intermediate_size=256, decay_low_rank_dim=16, a_low_rank_dim=16, v_low_rank_dim=8,
                                   gate_low_rank_dim=32)
        fancy = mode != "plain"  # vocabulary-sharded head, batch decoded as two halves on two communicators
        if mode == "peer_sum":  # the library's own sum over peer memory, alone: against NCCL and identical on all ranks
            from hf_adapter_b200.tp_comm import PeerAllReduce
            ar = PeerAllReduce(dist.group.WORLD, 256, 512, torch.device("cuda", rank))
            gen = torch.Generator(device="cuda").manual_seed(100 + rank)
            for rows in (1, 37, 256, 64):
                part = torch.randn(rows, 512, device="cuda", generator=gen).half()
                want = part.float().clone()
                dist.all_reduce(want)
                got = ar.all_reduce(part.clone())
                np.testing.assert_allclose(got.float().cpu().numpy(), want.cpu().numpy(), rtol=2e-3, atol=4e-3)
                both = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(both, got)
                assert torch.equal(both[0], both[1])
                same = part.clone()
                assert ar.all_reduce(same, out=same) is same and torch.equal(same, got)  # in place
            assert hb._lib.kernel_status(True) == 0
        if mode == "peer_rows":  # the sums inside the row kernels: bit for bit the stand-alone sum + the plain row kernels
            from hf_adapter_b200.tp_comm import PeerAllReduce, PeerRowSum
            dev = torch.device("cuda", rank)
            D = 512
            ar, rs = PeerAllReduce(dist.group.WORLD, 256, D, dev), PeerRowSum(dist.group.WORLD, 256, D, dev)
            few = PeerRowSum(dist.group.WORLD, 256, D, dev, max_ctas=24)  # several rows per CTA
            assert PeerRowSum.resident_rows(D, torch.float16) >= 148
            gen = torch.Generator(device="cuda").manual_seed(200 + rank)
            shared = torch.Generator(device="cuda").manual_seed(7)  # the same on every rank: replicated operands
            rnd = lambda *sh, g=shared: torch.randn(*sh, device="cuda", generator=g).half()
            nw, nb, mixes = 1 + 0.1 * rnd(D), 0.1 * rnd(D), [torch.rand(D, device="cuda", generator=shared).half() for _ in range(6)]
            for rows in (1, 37, 148, 64, 64):
                part, res, prev = rnd(rows, D, g=gen), rnd(rows, D), rnd(rows, D)
                total = ar.all_reduce(part.clone())
                p1, p2 = prev.clone(), prev.clone()
                want_x, want_m = hb.fused_ffn_add_norm_mix_decode(res, total, p1, nw, nb, mixes[0])
                got_x, got_m = rs.ffn_add_norm_mix(res, part, p2, nw, nb, mixes[0])
                assert torch.equal(got_x, want_x) and torch.equal(got_m, want_m) and torch.equal(p1, p2)
                p1, p2 = prev.clone(), prev.clone()
                want6 = hb.fused_attn_norm_mix6_decode(total, p1, nw, nb, *mixes)
                got_t, got6 = rs.attn_norm_mix6(part, p2, nw, nb, mixes)
                assert torch.equal(got_t, total) and torch.equal(p1, p2)
                assert all(torch.equal(a, b) for a, b in zip(got6, want6))
                p2 = prev.clone()
                got_t, got6 = few.attn_norm_mix6(part, p2, nw, nb, mixes)
                assert torch.equal(got_t, total) and torch.equal(p1, p2) and all(torch.equal(a, b) for a, b in zip(got6, want6))
            # pool rows: the shift state of batch row b lives in row slots[b] of a larger pool
            slots = torch.tensor([5, 0, 9, 2], device="cuda", dtype=torch.int32)
            part, res, pool = rnd(4, D, g=gen), rnd(4, D), rnd(12, D)
            total = ar.all_reduce(part.clone())
            q1, q2 = pool.clone(), pool.clone()
            want_x, want_m = hb.fused_ffn_add_norm_mix_decode(res, total, q1, nw, nb, mixes[0], slot_ids=slots)
            got_x, got_m = rs.ffn_add_norm_mix(res, part, q2, nw, nb, mixes[0], slot_ids=slots)
            assert torch.equal(got_x, want_x) and torch.equal(got_m, want_m) and torch.equal(q1, q2)
            assert hb._lib.kernel_status(True) == 0
        comm = {"peer_sum": "peer", "peer_rows": "peer_rows"}.get(mode, "nccl")
        half = comm != "nccl"
        model = hb.RWKV7ForCausalLM(cfg, tp_world=world, tp_rank=rank, tp_group=dist.group.WORLD, tp_shard_head=fancy,
                                    tp_overlap_rows=1 if fancy and mode != "peer_rows" else 0, tp_comm=comm)
        if half:
            model = model.half()
        model.load_state_dict({k: v.contiguous() for k, v in hb.shard_state_dict(full, world, rank, shard_head=fancy).items()})
        model = model.cuda().eval()
        ids = torch.from_numpy(g["ids"]).cuda()
        logits, cache = model.rwkv7_prefill_native(ids, None)
        tol = dict(rtol=3e-2, atol=3e-2) if half else dict(rtol=3e-4, atol=3e-4)  # (the peer modes run in fp16)
        np.testing.assert_allclose(logits[:, -1].float().cpu().numpy(), g["prefill_logits"], **tol)
        assert tuple(cache._state[0].shape) == (2, 1, 64, 64)  # one head per rank
        toks, tok = [], logits[:, -1].argmax(-1)
        for i in range(4):
            toks.append(tok)
            if fancy and i == 3:  # the step that ends in the arg-max token must agree with arg-max of the gathered logits
                tk = model.rwkv7_forward_token(tok, cache.clone(), use_graph=True, return_tokens=True)
            lg = model.rwkv7_forward_token(tok, cache, use_graph=(i >= 2))
            tok = lg.argmax(-1)
            if fancy and i == 3:
                assert torch.equal(tk, tok)
        torch.cuda.synchronize()
        if half:
            assert model._peer_ar and hb._lib.kernel_status(True) == 0  # the decode steps summed over peer memory
            assert bool(model._peer_rows) == (mode == "peer_rows")
        else:
            assert np.array_equal(torch.stack(toks, 1).cpu().numpy(), g["greedy"])
        np.testing.assert_allclose(lg.float().cpu().numpy(), g["final_logits"], **tol)
        result = "ok"
    except Exception as e:  # noqa: BLE001
        result = f"{type(e).__name__}: {e}"
    q.put((rank, result))
    q.close()
    q.join_thread()
    # communicator teardown with captured all-reduces alive was seen to block: leave without it
    os._exit(0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["plain", "sharded_head_overlap", "peer_sum", "peer_rows"])
def test_head_sharded_tp_two_gpus(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + {"plain": 7, "sharded_head_overlap": 13, "peer_sum": 19, "peer_rows": 23}[mode]
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, mode)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_peer_sum_wait_runs_out_without_a_peer():
    """Failure detection without a fault: one GPU plays rank 0 of a two-rank group whose "peer" buffers are local memory
    that nobody ever writes.  The wait for the peer's flag is limited to 30 ms; the kernel must come back by itself, store
    nothing, leave code 7 in the device error word, and the context must stay usable."""
    import ctypes
    import hf_adapter_b200 as hb
    from hf_adapter_b200 import _lib
    rows, D = 64, 1024
    slot = rows * D
    maxc = int(_lib.lib.rwkv7_tp_allreduce_max_ctas())
    inbox = [torch.zeros(2 * 2 * slot, device="cuda", dtype=torch.float16) for _ in range(2)]
    flags = [torch.zeros(2 * 2 * maxc, device="cuda", dtype=torch.int32) for _ in range(2)]
    counters = torch.zeros(2, device="cuda", dtype=torch.int32)
    part = torch.ones(rows, D, device="cuda", dtype=torch.float16)
    out = torch.full((rows, D), -1.0, device="cuda", dtype=torch.float16)
    _lib.kernel_status(True)
    arr = lambda ts: ctypes.cast((ctypes.c_void_p * 2)(*[t.data_ptr() for t in ts]), _lib.PP)
    st = _lib.lib.rwkv7_tp_allreduce(part.data_ptr(), out.data_ptr(), arr(inbox), arr(flags), counters.data_ptr(), 0, 2, rows, D,
                                     slot, 30, _lib.F16, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert _lib.kernel_status(True) == 7          # the bounded wait gave up and said so
    assert float(out.min()) == -1.0 and float(out.max()) == -1.0  # nothing was stored
    assert torch.equal(inbox[1][2 * slot:3 * slot], part.reshape(-1))  # ... but this rank's push (call 1: buffer 1, slot 0) reached the "peer"
    assert int(counters[0]) == 1
    y = hb.layer_norm(part, torch.ones(D, device="cuda", dtype=torch.float16), torch.zeros(D, device="cuda", dtype=torch.float16))
    assert torch.isfinite(y).all() and _lib.kernel_status(True) == 0  # the context still works


@pytest.mark.parametrize("rows,D", [(40, 1024), (128, 4096), (19, 8192)])
def test_row_sum_kernels_with_a_prefilled_inbox(rows, D):
    """The row kernels that take the tensor-parallel sum in themselves, on ONE GPU and without a peer: this GPU plays
    rank 0 of two, the "peer" memory is local, and the test itself puts rank 1's partial rows for call 1 into rank 0's
    inbox before the launch (wire format: every 4-byte payload word followed by the call number).  The results must
    equal the plain row kernels on the rounded sum bit for bit.  A second launch (call 2, nothing prefilled) must give
    up after its 30 ms limit with code 7 and store nothing."""
    import ctypes
    import hf_adapter_b200 as hb
    from hf_adapter_b200 import _lib
    assert int(_lib.lib.rwkv7_tp_rows_resident(D, _lib.F16)) >= 148
    slot = rows * D  # payload values per slot = int32 words per slot on the wire
    g = torch.Generator(device="cuda").manual_seed(3)
    rnd = lambda *sh: torch.randn(*sh, device="cuda", generator=g).half()
    mine, theirs, res, prev = rnd(rows, D), rnd(rows, D), rnd(rows, D), rnd(rows, D)
    nw, nb, mixes = 1 + 0.1 * rnd(D), 0.1 * rnd(D), [torch.rand(D, device="cuda", generator=g).half() for _ in range(6)]
    total = (mine.float() + theirs.float()).half()
    arr = lambda ts: ctypes.cast((ctypes.c_void_p * 2)(*[t.data_ptr() for t in ts]), _lib.PP)
    stream = torch.cuda.current_stream().cuda_stream
    wire = lambda t, call: torch.stack([t.reshape(-1).view(torch.int32), torch.full((slot // 2,), call, device="cuda",
                                                                                    dtype=torch.int32)], 1).reshape(-1)

    def fresh():
        inbox = [torch.zeros(2 * 2 * slot, device="cuda", dtype=torch.int32) for _ in range(2)]
        inbox[0][(1 * 2 + 1) * slot:(1 * 2 + 2) * slot] = wire(theirs, 1)  # call 1 -> buffer 1, slot of rank 1
        return inbox, torch.zeros(2, device="cuda", dtype=torch.int32)

    _lib.kernel_status(True)
    inbox, counters = fresh()
    p1, p2 = prev.clone(), prev.clone()
    want_x, want_m = hb.fused_ffn_add_norm_mix_decode(res, total, p1, nw, nb, mixes[0])
    got_x, got_m = torch.full_like(res, -1.0), torch.full_like(res, -1.0)
    call = lambda: _lib.lib.rwkv7_tp_ffn_add_norm_mix(
        res.data_ptr(), mine.data_ptr(), p2.data_ptr(), None, nw.data_ptr(), nb.data_ptr(), mixes[0].data_ptr(),
        got_x.data_ptr(), got_m.data_ptr(), arr(inbox), counters.data_ptr(), 0, 2, rows, D, slot, 0, 1e-5, 30, _lib.F16, stream)
    assert call() == 0
    torch.cuda.synchronize()
    assert _lib.kernel_status(True) == 0 and int(counters[0]) == 1
    assert torch.equal(got_x, want_x) and torch.equal(got_m, want_m) and torch.equal(p1, p2)
    assert torch.equal(inbox[1][2 * slot:3 * slot], wire(mine, 1))  # this rank's rows reached the "peer" (buffer 1, slot 0)
    # call 2: nobody fills buffer 0 -> every row's wait runs out, nothing is stored
    got_x.fill_(-1.0)
    keep = p2.clone()
    assert call() == 0
    torch.cuda.synchronize()
    assert _lib.kernel_status(True) == 7
    assert float(got_x.min()) == -1.0 and float(got_x.max()) == -1.0 and torch.equal(p2, keep)
    assert int(counters[0]) == 2

    inbox, counters = fresh()
    p1, p2 = prev.clone(), prev.clone()
    want6 = hb.fused_attn_norm_mix6_decode(total, p1, nw, nb, *mixes)
    x_out = torch.empty_like(mine)
    outs = torch.empty(6, rows, D, device="cuda", dtype=torch.float16)
    mp_, _k1 = _lib.ptr_array([m.data_ptr() for m in mixes])
    op_, _k2 = _lib.ptr_array([outs[i].data_ptr() for i in range(6)])
    # 16 CTAs: a CTA pushes all of its rows, then sums them one after the other
    assert _lib.lib.rwkv7_tp_attn_norm_mix6(mine.data_ptr(), x_out.data_ptr(), p2.data_ptr(), None, nw.data_ptr(), nb.data_ptr(),
                                            mp_, op_, arr(inbox), counters.data_ptr(), 0, 2, rows, D, slot, 16, 1e-5, 30,
                                            _lib.F16, stream) == 0
    torch.cuda.synchronize()
    assert _lib.kernel_status(True) == 0
    assert torch.equal(x_out, total) and torch.equal(p1, p2)
    assert all(torch.equal(outs[i], want6[i]) for i in range(6))
