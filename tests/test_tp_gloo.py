"""Head-sharded tensor parallelism on CPU: two gloo ranks each run the oracle's token step on their shard of the
reference's tiny model (sharded by hf_adapter_b200.shard_state_dict), sum the o_proj / ffn.value partials with
all_reduce, and must reproduce the unsharded logits, greedy tokens and (concatenated over ranks) recurrent state."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from hf_adapter_b200 import shard_spec, shard_state_dict
    from oracle import rwkv7_oracle as O
    from tests.test_oracle_golden import params_from_golden

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = dict(np.load(os.path.join(ROOT, "tests", "golden", "model_tiny.npz")))
        full = {k: v for k, v in g.items() if k.startswith("param::")}
        assert shard_spec("model.layers.1.attn.v_lora.lora.2.bias") == "rows"
        assert shard_spec("model.layers.1.attn.v_lora.lora.0.weight") is None
        assert shard_spec("model.layers.0.ffn.value.weight") == "cols"
        shard = shard_state_dict({k[len("param::"):]: v for k, v in full.items()}, world, rank)
        params = params_from_golden({"param::" + k: v for k, v in shard.items()})

        def reduced(weight):
            def op(x):
                y = torch.from_numpy(np.ascontiguousarray(np.asarray(x, np.float32) @ np.asarray(weight, np.float32).T))
                dist.all_reduce(y)
                return y.numpy()
            return op

        for d in params["layers"]:
            d["Ow"], d["fV"] = reduced(d["Ow"]), reduced(d["fV"])
        H_local, N = 2 // world, 64
        ids = g["ids"]
        B, T = ids.shape
        cache = O.new_cache(2, B, 128, H_local, N, np.float32)
        for t in range(T):
            logits = O.model_step(params, ids[:, t], cache, H_local, N)
        np.testing.assert_allclose(logits, g["prefill_logits"], rtol=3e-4, atol=3e-4)
        toks, tok = [], logits.argmax(-1)
        for _ in range(4):
            toks.append(tok)
            logits = O.model_step(params, tok, cache, H_local, N)
            tok = logits.argmax(-1)
        assert np.array_equal(np.stack(toks, 1), g["greedy"])
        state = torch.from_numpy(np.stack(cache["state"]))  # [L,B,H/P,N,N]
        gathered = [torch.empty_like(state) for _ in range(world)]
        dist.all_gather(gathered, state)
        np.testing.assert_allclose(torch.cat(gathered, dim=2).numpy(), g["final_state"], rtol=3e-4, atol=3e-5)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def test_head_sharded_tp_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_shard_state_dict_errors():
    from hf_adapter_b200 import shard_state_dict
    sd = {"model.layers.0.attn.r_proj.weight": np.zeros((6, 4))}
    assert shard_state_dict(sd, 2, 1)["model.layers.0.attn.r_proj.weight"].shape == (3, 4)
    with pytest.raises(ValueError):
        shard_state_dict(sd, 4, 0)
    with pytest.raises(ValueError):
        shard_state_dict(sd, 2, 2)
