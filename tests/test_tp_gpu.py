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
        model = hb.RWKV7ForCausalLM(cfg, tp_world=world, tp_rank=rank, tp_group=dist.group.WORLD, tp_shard_head=fancy,
                                    tp_overlap_rows=1 if fancy else 0, tp_comm="peer" if mode == "peer_sum" else "nccl")
        if mode == "peer_sum":
            model = model.half()
        model.load_state_dict({k: v.contiguous() for k, v in hb.shard_state_dict(full, world, rank, shard_head=fancy).items()})
        model = model.cuda().eval()
        ids = torch.from_numpy(g["ids"]).cuda()
        logits, cache = model.rwkv7_prefill_native(ids, None)
        tol = dict(rtol=3e-2, atol=3e-2) if mode == "peer_sum" else dict(rtol=3e-4, atol=3e-4)  # (that mode runs in fp16)
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
        if mode == "peer_sum":
            assert model._peer_ar and hb._lib.kernel_status(True) == 0  # the decode steps summed over peer memory
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
@pytest.mark.parametrize("mode", ["plain", "sharded_head_overlap", "peer_sum"])
def test_head_sharded_tp_two_gpus(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + {"plain": 7, "sharded_head_overlap": 13, "peer_sum": 19}[mode]
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
