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


def _argmax_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from hf_adapter_b200.sharding import shard_state_dict, sharded_argmax
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        logits = torch.randn(7, 64, generator=g).half()
        logits[0, 5] = logits[0, 40] = 9.0     # a tie across the two shards: the lower index wins, as in torch.argmax
        logits[1, 33] = logits[1, 34] = 9.0    # a tie inside one shard
        logits[2, 63] = 9.0
        Vl = 64 // world
        tok = sharded_argmax(logits[:, rank * Vl:(rank + 1) * Vl], rank, world)
        want = logits.float().argmax(-1)
        assert torch.equal(tok, want), (tok, want)
        assert int(tok[0]) == 5 and int(tok[1]) == 33 and int(tok[2]) == 63
        # the same from a pre-folded shard (what the head kernel's arg-max epilogue hands over): no local logits at all
        local = logits[:, rank * Vl:(rank + 1) * Vl].float()
        val, idx = local.max(dim=-1)
        tok2 = sharded_argmax(None, rank, world, local_best=(val, idx), shard_width=Vl)
        assert torch.equal(tok2, want), (tok2, want)
        head = {"lm_head.weight": np.arange(64 * 4).reshape(64, 4), "model.norm.weight": np.ones(4)}
        sh = shard_state_dict(head, world, rank, shard_head=True)
        assert sh["lm_head.weight"].shape == (Vl, 4) and sh["lm_head.weight"][0, 0] == rank * Vl * 4
        assert shard_state_dict(head, world, rank)["lm_head.weight"].shape == (64, 4)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def test_vocabulary_sharded_head_argmax_two_gloo_ranks():
    """Greedy tokens from a vocabulary-sharded head (local arg-max + one [B,2] all-gather) equal torch.argmax over the
    full logits, ties included."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_argmax_worker, args=(r, 2, port, q)) for r in range(2)]
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
