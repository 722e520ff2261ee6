"""Headline benchmark: decode tok/s at B=64 (+ prefill tok/s) on the 7.2B-shape RWKV-7 with int4
group-128 projections and an fp16 head, random weights, synthetic token ids.

    python bench.py --gpus 1 --steps K --warmup W            # this framework
    python bench.py --impl reference --steps K --warmup W    # CPU baseline arm (host cores)
    torchrun ... bench.py --gpus N ...                       # N>1: head-sharded tensor parallel
    python bench.py --shape 2.9B --quant w8                  # 2.9B shape, int8 per-output-channel projections

One "step" = one decode token for every sequence of the batch (all layers + head), replayed as a
CUDA graph.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = {
    # name: (layers, d_model, heads, ffn, vocab)
    "7.2B": (32, 4096, 64, 16384, 65536),
    "2.9B": (32, 2560, 40, 10240, 65536),
    "0.1B": (12, 768, 12, 3072, 65536),
}
RANKS = dict(decay_low_rank_dim=64, a_low_rank_dim=64, v_low_rank_dim=32, gate_low_rank_dim=128)
METRIC = "decode tok/s @B=64 + prefill tok/s, 7.2B RWKV-7 MM4; WKV scan % HBM/TC peak"


def decode_step_bytes(L, D, H, Fd, V, B, quant="mm4", group=128, ranks=(64, 64, 32, 128), state_bytes=4):
    """Algorithmic HBM bytes of one decode step: quantised weights + scales, fp16 LoRA and head,
    recurrent state read+write, shift states read+write."""
    A = H * 64
    n_w = 4 * D * A + 2 * D * Fd
    if quant == "mm4":
        w_q, w_scales = n_w // 2, n_w // group * 2
    else:  # int8 per output channel (fp16 scales; the a8w8 format keeps them in fp32)
        w_q, w_scales = n_w, (4 * A + 2 * Fd) * (4 if quant == "a8w8" else 2)
    rw, ra, rv, rg = ranks
    lora = (rw + ra + rg + rv) * (D + A) * 2
    weights = L * (w_q + w_scales + lora) + V * D * 2
    state = B * L * H * 64 * 64 * state_bytes * 2
    shift = B * L * 2 * D * 2 * 2
    return weights + state + shift, weights, state


def w4_launch_bytes(M, K, Nout, n=1):
    """Algorithmic bytes of one int4 group-128 projection launch: nibbles, fp16 scale + u8 zero-point per group and
    channel, activations in, outputs out."""
    return n * (K * Nout // 2 + K * Nout // 128 * 3 + M * (K + Nout) * 2)


def w8_launch_bytes(M, K, Nout, n=1):
    """The same for int8 weights with one fp16 scale per output channel."""
    return n * (K * Nout + Nout * 2 + M * (K + Nout) * 2)


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def measured_peaks():
    """(HBM GB/s, bf16 TFLOP/s burst, bf16 TFLOP/s sustained, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        burst = float(p["bf16_tflops"])
        return float(p["hbm_gbs"]), burst, float(p.get("bf16_tflops_sustained", burst)), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def shape_config(shape, quant, batch, layers=0):
    L, D, H, Fd, V = SHAPES[shape]
    fmt = {"mm4": "mm4-g128", "w8": "int8-per-channel", "a8w8": "a8w8 (int8 activations x int8 weights)"}[quant]
    return {"workload": f"rwkv7-{shape}-shape {fmt} decode, batch {batch}, "
                        "fp16 head ending in the greedy token (arg-max fused in the head GEMM), cache resident",
            "layers": layers or L, "d_model": D, "heads": H, "ffn": Fd, "vocab": V, "lora_ranks": RANKS}


# ------------------------------------------------------------------------------------------ model
def build_model(shape, tp_world, tp_rank, tp_group, device, layers_override=0, quant="mm4", seed=0, full_then_shard=False,
                state_dtype=None, overlap_rows=0, tp_comm="nccl"):
    """Random-init model of the named shape, projections quantised on the GPU, fp16 head.
    The token-shift / key-scale parameters the reference constructs as zeros are re-initialised (seeded) so
    that every term of the recurrence is exercised.  ``full_then_shard``: build the unsharded model from the seed
    on every rank and keep this rank's head shard of it (so that sharded and unsharded runs can be compared)."""
    import torch

    import hf_adapter_b200 as hb

    L, D, H, Fd, V = SHAPES[shape]
    if layers_override:
        L = layers_override
    cfg = hb.NativeRWKV7Config(vocab_size=V, hidden_size=D, num_hidden_layers=L, num_heads=H, head_dim=64,
                               intermediate_size=Fd, **RANKS)

    def construct(world, rank, group):
        torch.manual_seed(seed)
        old = torch.get_default_dtype()
        torch.set_default_dtype(torch.float16)
        try:
            with torch.device(device):
                return hb.RWKV7ForCausalLM(cfg, tp_world=world, tp_rank=rank, tp_group=group,
                                           state_dtype=state_dtype or torch.float32, tp_shard_head=world > 1,
                                           tp_overlap_rows=overlap_rows if world > 1 else 0, tp_comm=tp_comm)
        finally:
            torch.set_default_dtype(old)

    def init(model, gseed):
        g = torch.Generator(device=device).manual_seed(gseed)
        with torch.no_grad():
            for name, p in model.named_parameters():
                if p.dim() == 2 and "embeddings" not in name:
                    p.normal_(0.0, 0.02, generator=g)
            for i, layer in enumerate(model.model.layers):
                at = layer.attn
                for nme in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"):
                    getattr(at, nme).uniform_(0, 1, generator=g)
                layer.ffn.x_k.uniform_(0, 1, generator=g)
                at.k_k.normal_(0.85, 0.1, generator=g)
                at.k_a.normal_(1.0, 0.1, generator=g)
                at.r_k.normal_(0.0, 0.1, generator=g)
                at.w_lora.lora[2].bias.uniform_(-5, -1, generator=g)
                at.a_lora.lora[2].bias.normal_(0, 0.5, generator=g)
                if i:
                    at.v_lora.lora[2].bias.normal_(0, 0.5, generator=g)

    if full_then_shard and tp_world > 1:
        full = construct(1, 0, None)
        init(full, 1 + seed)
        sd = hb.shard_state_dict(full.state_dict(), tp_world, tp_rank, shard_head=True)
        model = construct(tp_world, tp_rank, tp_group)
        model.load_state_dict({k: v.contiguous() for k, v in sd.items()})
        del full, sd
    else:
        model = construct(tp_world, tp_rank, tp_group)
        init(model, 1 + seed + (0 if full_then_shard else tp_rank))
    n = hb.quantize_model(model, quant, min_params=1_000_000, group_size=128, skip=("lm_head",))
    torch.cuda.empty_cache()
    return model.eval(), cfg, n


# ------------------------------------------------------------------------------------------ reference arm
def run_cpu_baseline(shape, B, steps, warmup, distinct_layers=4, budget_s=170.0):
    """Times the CPU port of the reference's decode step on the host cores: every step runs ALL L layers and the head
    at batch B (no extrapolation).  To bound the set-up time the L layer calls cycle over `distinct_layers` distinct
    weight sets (400 MB of int4 weights: larger than the host caches, so every call streams its weights from memory
    and dequantises them, as the reference does on CPU); every layer has its own recurrent state."""
    import torch

    from oracle import cpu_port_torch as P

    L, D, H, Fd, V = SHAPES[shape]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ranks = (RANKS["decay_low_rank_dim"], RANKS["a_low_rank_dim"], RANKS["v_low_rank_dim"], RANKS["gate_low_rank_dim"])
    sets = [P.make_layer(D, H, 64, Fd, ranks, layer_id=1 + i, seed=i) for i in range(distinct_layers)]
    g = torch.Generator().manual_seed(0)
    head_w = torch.randn(V, D, generator=g) * 0.02
    nw, nb = torch.ones(D), torch.zeros(D)
    x = torch.randn(B, D, generator=g)
    xpa, xpf = torch.randn(B, D, generator=g), torch.randn(B, D, generator=g)
    vf = torch.randn(B, H * 64, generator=g)
    st = [0.1 * torch.randn(B, H, 64, 64, generator=g) for _ in range(L)]
    times = []
    t_begin = time.perf_counter()
    with torch.no_grad():
        for it in range(warmup + steps):
            if len(times) >= 3 and time.perf_counter() - t_begin > budget_s:
                break  # bounded: the run ends within a few minutes whatever --steps says; `sample` gives the count
            t0 = time.perf_counter()
            y = x
            for i in range(L):
                y, _, _, _, st[i] = P.layer_step(sets[i % distinct_layers], y, xpa, xpf, vf, st[i], H, 64)
            P.head_step(y, nw, nb, head_w)
            if it >= warmup:
                times.append(time.perf_counter() - t0)
    step_s = sum(times) / len(times)
    return {"value": B / step_s, "unit": "tok/s", "cores": cores, "kind": "port", "timed_steps": len(times),
            "sample": f"{len(times)} timed full steps ({L} layers + head) at B={B} after {warmup} warm-up, fp32 activations, int4-g128 "
                      f"weights dequantised per call as the reference does on CPU; the {L} layer calls cycle over "
                      f"{distinct_layers} distinct weight sets, every layer has its own state",
            "ms_per_step": step_s * 1e3}


# ------------------------------------------------------------------------------------------ main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="7.2B", choices=sorted(SHAPES))
    ap.add_argument("--quant", default="mm4", choices=["mm4", "w8", "a8w8"],
                    help="projection format: mm4 = int4 group-128 (headline), w8 = int8 per output channel (the 2.9B configuration), "
                         "a8w8 = per-token int8 activations x int8 weights on the int8 tensor-core GEMM (the prefill kernel)")
    ap.add_argument("--state", default="fp32", choices=["fp32", "fp16"],
                    help="recurrent-state storage: fp32 (the headline contract) or the reference's opt-in FP16-state lane")
    ap.add_argument("--batch", type=int, default=64, help="sequences per GPU group (global batch = batch for N=1)")
    ap.add_argument("--layers", type=int, default=0, help="debug: override the layer count (invalidates the metric)")
    ap.add_argument("--prefill-tokens", type=int, default=1024)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--prefill-scan-chunk", type=int, default=64,
                    help="tile of the tensor-core WKV scan in the prefill sample (0 = sequential scan)")
    ap.add_argument("--parallelism", default="tp", choices=["tp", "dp"],
                    help="N > 1: tp = head-sharded tensor parallelism (headline; independent replicas measured beside "
                         "it), dp = independent sequence batches on full replicas as the headline")
    ap.add_argument("--tp-overlap-rows", type=int, default=0,
                    help="tp: batches of at least twice this many rows per rank decode as two halves on two streams with "
                         "their own communicators, hiding one half's all-reduces under the other half's kernels (0 = off)")
    ap.add_argument("--tp-comm", default="auto", choices=["auto", "peer", "peer_rows", "nccl"],
                    help="tp: sum the [B,D] partial outputs with this library's one-kernel sum over peer-mapped memory (plain "
                         "peer stores, flags, bounded waits) or with NCCL all-reduce; auto = peer at 2 GPUs, NCCL above (one-shot: every "
                         "rank sends its whole partial to every peer, which stops paying from 4 GPUs up)")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-scan", action="store_true")
    ap.add_argument("--no-ops", action="store_true", help="skip the isolated projection-operator table")
    ap.add_argument("--no-b256", action="store_true", help="skip the batch-256 decode measurement")
    ap.add_argument("--no-pool", action="store_true", help="skip the state-pool decode measurement")
    ap.add_argument("--no-side", action="store_true", help="N > 1: skip the side measurements (replicas, strong scaling)")
    ap.add_argument("--stall-limit", type=int, default=480,
                    help="N > 1: seconds after which a run that has not finished ends itself with exit code 5 (a rank "
                         "waiting for a collective that never completes would otherwise sit until the library's own "
                         "10-minute watchdog); 0 = no limit")
    args = ap.parse_args()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    if args.tp_comm == "auto":
        # measured: at 2 GPUs the sums taken inside the row kernels (one trip over the link, no extra launch) give
        # 4.2 ms per step against 5.1 ms with the stand-alone peer kernel; from 4 GPUs up every rank would send its
        # rows to P - 1 peers (6.6 ms at N = 4) and NCCL's in-switch reduction moves fewer bytes (5.9 ms)
        args.tp_comm = "peer_rows" if int(os.environ.get("WORLD_SIZE", "1")) <= 2 else "nccl"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and args.stall_limit > 0 and args.impl == "ours":
        def give_up():
            print(f"[bench rank {rank}] not finished after {args.stall_limit} s: leaving with exit code 5", file=sys.stderr, flush=True)
            os._exit(5)
        stall_timer = threading.Timer(args.stall_limit, give_up)
        stall_timer.daemon = True
        stall_timer.start()
    L, D, H, Fd, V = SHAPES[args.shape]
    base_cfg = shape_config(args.shape, args.quant, args.batch, args.layers)

    if args.impl == "reference":
        if rank != 0:
            return
        cb = run_cpu_baseline(args.shape, args.batch, steps, 1)
        line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
                "steps": cb["timed_steps"], "warmup": 1, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": dict(base_cfg, note="reference's CPU path (torch CPU port) on the host cores; full steps, "
                                              "bounded to about three minutes"),
                "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import torch
    import torch.distributed as dist

    import hf_adapter_b200 as hb
    from hf_adapter_b200 import _lib
    from hf_adapter_b200 import model as hbm
    from hf_adapter_b200 import packing as hpk

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tp_group = None
    if world > 1:
        if args.tp_overlap_rows:
            # two half-batches = two library communicators with collectives in flight at the same time on every GPU;
            # the library orders them by host program order (and so alike on all ranks) only when told to
            os.environ.setdefault("NCCL_LAUNCH_ORDER_IMPLICIT", "1")
        dist.init_process_group("nccl", device_id=dev)
        tp_group = dist.group.WORLD

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def note(msg):
        """Progress on stderr (RWKV7_BENCH_VERBOSE=1): which phase a failed multi-rank run was in."""
        if os.environ.get("RWKV7_BENCH_VERBOSE"):
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def time_decode(model, B, seed, clocks_on_rank0, n_steps=None, e2e=True):
        """Device-resident graph replays (-> ms per step), then the end-to-end loop through the public API; both are
        bracketed by a barrier + synchronize and reduced with MAX over the ranks."""
        n_steps = n_steps or steps
        gen = torch.Generator().manual_seed(seed)
        ids_host = torch.randint(0, V, (n_steps + warmup + 8, B), generator=gen).pin_memory()
        cache = model.new_cache(B)
        # kernels of this library launched per decode step (counted on one eager step through the C ABI; the step
        # before it builds the tiled weight copies, whose one-time repack kernels are not part of a step)
        model.rwkv7_forward_token(ids_host[0].to(dev), cache, use_graph=False)
        _lib.LAUNCHES = 0
        model.rwkv7_forward_token(ids_host[0].to(dev), cache, use_graph=False)
        launches = _lib.LAUNCHES
        greedy = True  # the step ends in the greedy token: arg-max in the head GEMM's epilogue, the logits are never stored
        graph = model._decode_graph(B, greedy)
        graph.bind(cache)
        ids_dev = ids_host.to(dev)
        # the clock sampler starts before the warm-up replays: nvidia-smi needs a moment before its first sample, and
        # the GPU is under the same load from here to the end of the end-to-end loop
        sampler = ClockSampler(local) if (clocks_on_rank0 and rank == 0) else None
        for i in range(warmup):
            graph.ids.copy_(ids_dev[i])
            graph.graph.replay()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(n_steps):
            graph.ids.copy_(ids_dev[warmup + i])
            graph.graph.replay()
        ev1.record()
        barrier()
        ms_step = max_over_ranks(ev0.elapsed_time(ev1)) / n_steps
        e2e_ms = None
        if e2e:
            # end to end: pinned ids -> H2D -> step -> argmax -> D2H, the caller consuming the token before the next step
            tok_host = torch.empty((B,), dtype=torch.long).pin_memory()
            def step_tokens(i):
                out = model.rwkv7_forward_token(ids_host[i].to(dev, non_blocking=True), cache, return_tokens=greedy)
                return out if greedy else out.argmax(-1)

            for i in range(3):
                tok_host.copy_(step_tokens(i), non_blocking=True)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(n_steps):
                tok_host.copy_(step_tokens(warmup + i), non_blocking=True)
                torch.cuda.current_stream().synchronize()
            e1.record()
            barrier()
            e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / n_steps
        return ms_step, e2e_ms, launches, cache, (sampler.stop() if sampler else None), gen

    def drop(model):
        model._graphs.clear()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

    # ---------------- N > 1: parity of the head-sharded form before anything is timed.  Two layers at this shape's
    # width, the unsharded model built from the same seed on every rank: logits and greedy tokens of the sharded run
    # (eager and CUDA-graph steps, NCCL all-reduces inside) must match the single-GPU run of the same weights.
    tp_parity = None
    if world > 1:
        try:
            Bp = 8
            ref_model, _, _ = build_model(args.shape, 1, 0, None, dev, 2, args.quant, seed=7)
            tpm, _, _ = build_model(args.shape, world, rank, tp_group, dev, 2, args.quant, seed=7, full_then_shard=True,
                                    overlap_rows=args.tp_overlap_rows, tp_comm=args.tp_comm)
            gen = torch.Generator().manual_seed(11)
            pids = torch.randint(0, V, (Bp, 6), generator=gen).to(dev)
            c_ref, c_tp = ref_model.new_cache(Bp), tpm.new_cache(Bp)
            worst, same_tokens = 1.0, True
            for t in range(6):
                lr = ref_model.rwkv7_forward_token(pids[:, t], c_ref, use_graph=False)
                lt = tpm.rwkv7_forward_token(pids[:, t], c_tp, use_graph=(t >= 3))
                a, b = lr.double().flatten(), lt.double().flatten()
                worst = min(worst, float(a @ b / a.norm() / b.norm()))
                # the sharded run's best logit may differ from the unsharded choice only within fp16 noise
                top = lr.argmax(-1)
                same_tokens &= bool(((lt.max(-1).values - lt.gather(1, top[:, None])[:, 0]) < 2e-2).all())
                if t == 5:  # the fused arg-max of the sharded head == arg-max of the gathered logits (on a cache copy)
                    tk = tpm.rwkv7_forward_token(pids[:, t], c_chk, use_graph=True, return_tokens=True)
                    same_tokens &= bool(torch.equal(tk, lt.argmax(-1)))
                elif t == 4:
                    c_chk = c_tp.clone()
            s_ref = torch.stack(c_ref._state)[:, :, rank * (H // world):(rank + 1) * (H // world)]
            s_err = float((torch.stack(c_tp._state) - s_ref).norm() / s_ref.norm())
            flag = torch.tensor([1.0 if (worst > 0.9995 and same_tokens and s_err < 1e-2) else 0.0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            tp_parity = {"status": "ok" if float(flag.item()) == 1.0 else "FAILED", "min_logit_cosine": worst,
                         "greedy_tokens_match": same_tokens, "state_rel_err": s_err,
                         "case": f"2 layers at {args.shape} width, batch {Bp}, 6 tokens, eager + graph steps, vs the unsharded model"}
            drop(tpm)
            drop(ref_model)
            del ref_model, tpm, c_ref, c_tp
        except Exception as exc:
            tp_parity = {"status": "FAILED", "error": f"{type(exc).__name__}: {exc}"[:300]}
        torch.cuda.empty_cache()

    # ---------------- N > 1, side measurement: independent sequence batches on full replicas (no collective)
    replicas = None
    use_tp = world > 1 and args.parallelism == "tp"
    if world > 1 and not args.no_side:
        note("side measurement: the other parallelism")
        other_tp = not use_tp
        m2, _, _ = build_model(args.shape, world if other_tp else 1, rank if other_tp else 0, tp_group if other_tp else None,
                               dev, args.layers, args.quant, overlap_rows=args.tp_overlap_rows, tp_comm=args.tp_comm)
        B2 = args.batch * world if other_tp else args.batch
        ms2, _, _, c2, _, _ = time_decode(m2, B2, 0 if other_tp else rank, False, n_steps=min(steps, 20), e2e=False)
        side = {"value": args.batch * world / (ms2 * 1e-3), "unit": "tok/s", "ms_per_step": ms2, "global_batch": args.batch * world,
                "parallelism": (f"tp{world}: heads, state and projections sharded, batch {B2} on every rank" if other_tp else
                                f"dp{world}: independent sequence batches, one full replica per GPU, {args.batch} sequences each, "
                                "no data-path collective")}
        replicas = side
        drop(m2)
        del m2, c2

    # ---------------- headline.  N = 1: the model on one GPU.  N > 1 (default): head-sharded tensor parallelism --
    # heads, their state and the projections sharded, a global batch of batch*N on every rank (per-GPU state work
    # fixed: weak scaling), NCCL all-reduces of the [B,D] partial sums inside the decode graph.
    sdt = torch.float16 if args.state == "fp16" else torch.float32
    if use_tp:
        model, cfg, nq = build_model(args.shape, world, rank, tp_group, dev, args.layers, args.quant, state_dtype=sdt,
                                     overlap_rows=args.tp_overlap_rows, tp_comm=args.tp_comm)
        B, shard = args.batch * world, world
        parallelism = (f"tp{world}: heads, recurrent state, projections and the head's vocabulary sharded, global batch {B} on "
                       "every rank, two sums of the [B,D] partial outputs per layer inside the decode graph ("
                       + ({"peer": "this library's kernel over peer-mapped memory",
                           "peer_rows": "taken over peer-mapped memory inside the LayerNorm / token-shift kernels that consume them"}
                          .get(args.tp_comm, "NCCL all-reduce")) + ")"
                       + (f", batch decoded as two halves of {B // 2} rows on two streams / communicators"
                          if args.tp_overlap_rows and B >= 2 * args.tp_overlap_rows else "")
                       + "; the step ends in the greedy token (local arg-max + one [B,2] all-gather)")
    else:
        model, cfg, nq = build_model(args.shape, 1, 0, None, dev, args.layers, args.quant, state_dtype=sdt)
        B, shard = args.batch, 1
        parallelism = "single GPU" if world == 1 else \
            f"dp{world}: independent sequence batches, one full replica per GPU, {args.batch} sequences each, no data-path collective"
    Lr = cfg.num_hidden_layers
    note(f"headline: batch {B}")
    ms_per_step, e2e_ms, launches_per_step, cache, clocks, gen = time_decode(model, B, 0 if use_tp else rank, True)
    note(f"headline done: {ms_per_step:.3f} ms per step")
    global_batch = B if use_tp else args.batch * world

    # ---------------- N > 1: strong scaling of the head-sharded form (the global batch stays 64 and 256)
    strong = None
    if use_tp and not args.no_side:
        strong = {}
        for Bg in (64, 256):
            note(f"strong scaling: global batch {Bg}")
            ms_s, _, _, c_s, _, _ = time_decode(model, Bg, 0, False, n_steps=min(steps, 20), e2e=False)
            strong[f"global_batch_{Bg}"] = {"value": Bg / (ms_s * 1e-3), "unit": "tok/s", "ms_per_step": ms_s}
            model._graphs.pop((Bg, True), None)
            del c_s
            torch.cuda.empty_cache()

    def leave():
        """Multi-rank exit.  Tearing the NCCL communicator down while CUDA graphs that captured its all-reduces are
        alive was seen to block here, so the graphs go first and the process ends without the destructor chain."""
        if world > 1:
            model._graphs.clear()
            torch.cuda.synchronize()
            dist.barrier()
            sys.stdout.flush()
            os._exit(0)

    if rank != 0:
        leave()  # the remaining sections are rank-0 measurements
        return

    note("rank-0 sections: rooflines, operator table")
    hbm_peak, tc_burst, tc_sustained, peak_src = measured_peaks()
    Hl, Fl, A_l = H // shard, Fd // shard, (H // shard) * 64
    sbytes = 2 if args.state == "fp16" else 4
    step_bytes, w_bytes, s_bytes = decode_step_bytes(Lr, D, Hl, Fl, V, B, args.quant, state_bytes=sbytes)  # per GPU
    N = 64
    f16 = lambda *s: torch.randn(*s, device=dev, dtype=torch.float16)

    def time_graph(fn, launches_inside, reps=None):
        """fn launches `launches_inside` kernels back to back; captured once, replayed, timed with CUDA events on the
        launching stream -> microseconds per launch."""
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        reps = reps or max(3, min(steps, 10))
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            g.replay()
        t1.record()
        torch.cuda.synchronize()
        us = t0.elapsed_time(t1) * 1e3 / (reps * launches_inside)
        del g
        return us

    # ---------------- roofline of the dominant kernel: the int4 projections (four launches per layer), each launch shape
    # timed alone over every layer's own weights (GBs in total: far above the 126 MB L2, so no flush is needed)
    roofline = None
    layers = list(model.model.layers)
    launch_bytes = w4_launch_bytes if args.quant == "mm4" else w8_launch_bytes
    if args.quant != "a8w8" and all(isinstance(l.ffn.key, (hb.MM4Linear, hb.MM8Linear))
                                    and l.ffn.key.tiled_for(f16(B, D)) is not None for l in layers):
        xr, xk, xv, xf = (f16(B, D) for _ in range(4))
        xo, xh, xres = f16(B, A_l), f16(B, Fl).abs_(), f16(B, D)
        per = {}

        def add(name, fn, nbytes):
            us = time_graph(fn, len(layers))
            per[name] = {"us_per_launch": us, "bytes_per_launch": nbytes, "achieved_gbs": nbytes / us / 1e3,
                         "frac": nbytes / us / 1e3 / hbm_peak}

        rkv_of = lambda at: hpk.rkv_grouped((at.r_proj, at.k_proj, at.v_proj), xr, xk, xv)
        assert rkv_of(layers[0].attn) is not None, "r/k/v are not served by the grouped launch"
        add("rkv_grouped", lambda: [rkv_of(l.attn) for l in layers], launch_bytes(B, D, A_l, 3))
        add("o_proj", lambda: [hbm._linear(l.attn.o_proj, xo) for l in layers], launch_bytes(B, A_l, D))
        add("ffn_key_relu2", lambda: [hbm._linear(l.ffn.key, xf, relu2=True) for l in layers], launch_bytes(B, D, Fl))
        add("ffn_value_add", lambda: [hbm._linear(l.ffn.value, xh, residual=xres) for l in layers], launch_bytes(B, Fl, D))
        tot_b = sum(v["bytes_per_launch"] for v in per.values())
        tot_us = sum(v["us_per_launch"] for v in per.values())
        roofline = {"kernel": "w4g_umma_kernel (%s projections on tcgen05: the four launches of a layer)" %
                              ("int4 group-128" if args.quant == "mm4" else "int8 per-channel"),
                    "bound": "hbm", "achieved": tot_b / tot_us / 1e3, "peak": hbm_peak, "unit": "GB/s",
                    "frac": tot_b / tot_us / 1e3 / hbm_peak, "peak_source": peak_src + " (burst copy)",
                    "bytes_per_launch": tot_b / 4, "us_per_launch": tot_us / 4, "launches": per,
                    "share_of_step": tot_us * 1e-3 * len(layers) / ms_per_step,
                    # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the four launches of a 7.2B layer at
                    # B = 64 (profiles/): 36.2 + 38.4 + 28.3 + 9.5 = 112.4 MB against 114.8 MB algorithmic (activations and
                    # outputs stay in L2): scaled by the algorithmic bytes of this run's launches
                    "traffic": (112.4e6 / 114.8e6) * tot_b / 4 if (B == 64 and args.quant == "mm4") else None,
                    "note": "achieved = algorithmic bytes of the four launches / their CUDA-event time, each shape replayed "
                            "alone as a graph over all layers' weights; at 64 rows a [128 x 128] int4 block costs 512 tensor-pipe "
                            "cycles (a 128 x N x 16 MMA takes about 64 cycles for every N <= 128): about 0.65 of the copy peak over 128 CTAs"}
        del xr, xk, xv, xf, xo, xh, xres

    # ---------------- second kernel: the WKV-7 decode recurrence, timed alone over all layers' states
    r, w_raw, k, v, a, g = (f16(B, Hl * N) for _ in range(6))
    at0 = layers[1].attn if Lr > 1 else layers[0].attn
    states = cache._state
    wkv_out = torch.empty((B, Hl * N), device=dev, dtype=torch.float16)

    def wkv_pass():
        for s in states:
            hb.fused_recurrent_output_prepare_raw(r, w_raw, k, v, a, s, g, at0.k_k, at0.k_a, at0.r_k, at0.g_norm.weight,
                                                  at0.g_norm.bias, eps=N * 1e-5, new_state=s, out=wkv_out)

    for _ in range(3):
        wkv_pass()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(3, min(steps, 20))
    k0.record()
    for _ in range(reps):
        wkv_pass()
    k1.record()
    torch.cuda.synchronize()
    wkv_ms = k0.elapsed_time(k1) / (reps * len(states))
    wkv_bytes = B * Hl * (2 * N * N * sbytes + 7 * N * 2)
    achieved = wkv_bytes / (wkv_ms * 1e-3) / 1e9
    roofline_wkv = {"kernel": "wkv7_step_kernel (decode recurrence + fused epilogues)", "bound": "hbm", "achieved": achieved,
                    "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src + " (burst copy)",
                    # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture at B*H = 4096 (profiles/): 87.0 MB per
                    # launch (reads = state in; most of the written state is still dirty in L2 when the kernel ends),
                    # scaled by the sequence-heads of this launch
                    "traffic": 87.0e6 * (B * Hl) / 4096.0 if sbytes == 4 else None, "bytes_per_launch": wkv_bytes, "us_per_launch": wkv_ms * 1e3,
                    "share_of_step": wkv_ms * len(states) / ms_per_step}
    if roofline is None:
        roofline, roofline_wkv = roofline_wkv, None

    extra = {"step_bytes": step_bytes, "step_hbm_frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
             "targets": {"step_hbm_frac": 0.70, "scan_tensor_frac": 0.50,
                         "note": "north-star targets; step_hbm_frac and wkv_scan.*.tensor_frac_of_bf16_burst_peak are the measured values"}}

    # ---------------- decode at batch 256 (the second batch size of the 7.2B configuration), single GPU
    b256 = None
    if not args.no_b256 and world == 1 and args.batch != 256:
        try:
            ms256, _, _, c256, _, _ = time_decode(model, 256, 3, False, n_steps=min(steps, 20), e2e=False)
            sb256 = decode_step_bytes(Lr, D, H, Fd, V, 256, args.quant, state_bytes=sbytes)[0]
            b256 = {"value": 256 / (ms256 * 1e-3), "unit": "tok/s", "ms_per_step": ms256, "step_bytes": sb256,
                    "step_hbm_frac": sb256 / (ms256 * 1e-3) / 1e9 / hbm_peak}
            model._graphs.pop(256, None)
            del c256
        except Exception as exc:
            b256 = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        torch.cuda.empty_cache()

    # ---------------- serving state pool: the same decode step with every sequence's state addressed through slot ids
    pool_stats = None
    if not args.no_pool and world == 1 and args.state == "fp32":
        try:
            cap = B + B // 2
            pool = hb.RWKV7StatePool(model, cap)
            slots_all, _ = pool.allocate(range(cap))
            perm = torch.randperm(cap, generator=gen).tolist()
            sched = [slots_all[i] for i in perm[:B]]  # a scattered, unordered subset of the live slots
            toks = torch.randint(0, V, (B,), generator=gen).to(dev)
            for _ in range(3):
                pool.decode(toks, sched, use_graph=True, greedy=True)
            gph = pool._graphs[(1 << max(0, (B - 1).bit_length()), True)]
            slot_vec = pool._slot_vector(sched, gph.rows)
            torch.cuda.synchronize()
            q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            nrep = max(3, min(steps, 20))
            q0.record()
            for _ in range(nrep):
                gph.replay(toks, slot_vec)
            q1.record()
            torch.cuda.synchronize()
            pms = q0.elapsed_time(q1) / nrep
            pool_stats = {"value": B / (pms * 1e-3), "unit": "tok/s", "ms_per_step": pms, "capacity": cap, "scheduled": B,
                          "bytes_per_slot": pool.bytes_per_slot,
                          "note": "graph replay over the pools with a permuted slot vector; no gather / scatter of state"}
            del pool, gph
        except Exception as exc:
            pool_stats = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        torch.cuda.empty_cache()

    # ---------------- prefill tok/s (bounded sample of the 8192-token prompts: the state carries over chunks)
    prefill = None
    if not args.no_prefill and world == 1:
        Tp, ch = args.prefill_tokens, args.prefill_chunk
        pids = torch.randint(0, V, (B, Tp), generator=gen).to(dev)
        model.rwkv7_prefill_chunks(pids[:, :ch], None, chunk_size=ch, scan_chunk=args.prefill_scan_chunk)
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        model.rwkv7_prefill_chunks(pids, None, chunk_size=ch, scan_chunk=args.prefill_scan_chunk)
        p1.record()
        torch.cuda.synchronize()
        pms = p0.elapsed_time(p1)
        prefill = {"value": B * Tp / (pms * 1e-3), "unit": "tok/s", "batch": B, "tokens": Tp, "chunk": ch, "ms": pms,
                   "wkv_scan": "chunked_tcgen05" if args.prefill_scan_chunk else "sequential",
                   "note": "sample of the 8192-token prompts; throughput is chunk-invariant because only the O(1) state carries over"}
        del pids
        torch.cuda.empty_cache()

    # ---------------- isolated WKV scan (config: B8 T4096 H32 N64)
    scan = None
    if not args.no_scan and world == 1:
        Bs, Ts, Hs = 8, 4096, 32
        rs, ks, vs = (torch.randn(Bs, Ts, Hs, N, device=dev, dtype=torch.float16) for _ in range(3))
        kks = torch.nn.functional.normalize(ks.float(), dim=-1).half()
        as_ = torch.sigmoid(torch.randn(Bs, Ts, Hs, N, device=dev)).half()
        ws = torch.exp(-0.606531 * torch.sigmoid(torch.randn(Bs, Ts, Hs, N, device=dev)))
        s0 = torch.zeros(Bs, Hs, N, N, device=dev)
        scan = {}
        for name, fn in (("sequential", lambda: hb.fused_recurrent_scan(rs, ws, ks, vs, kks, as_, s0)),
                         ("chunked_tcgen05", lambda: hb.self_chunk_rwkv7(rs, ws, ks, vs, kks, as_, s0, chunk_size=64))):
            fn()
            torch.cuda.synchronize()
            s_0, s_1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_0.record()
            for _ in range(3):
                fn()
            s_1.record()
            torch.cuda.synchronize()
            sms = s_0.elapsed_time(s_1) / 3
            sbytes = 5 * Bs * Ts * Hs * N * 2 + Bs * Ts * Hs * N * 4 + Bs * Ts * Hs * N * 2 + 2 * Bs * Hs * N * N * 4
            flops = Bs * Ts * Hs * (16 * 64 * N + 8 * N * N + 2 * 64 * 64)  # chunked-form tensor flops, C = 64
            scan[name] = {"ms": sms, "tok_per_s": Bs * Ts / (sms * 1e-3), "hbm_frac": sbytes / (sms * 1e-3) / 1e9 / hbm_peak,
                          # an isolated kernel: against the burst figure of the measured bf16 GEMM peak
                          "tensor_frac_of_bf16_burst_peak": flops / (sms * 1e-3) / 1e12 / tc_burst}
        del rs, ks, vs, kks, as_, ws
        torch.cuda.empty_cache()

    # ---------------- isolated projection operators: weights [4096,4096], [16384,4096], [4096,16384]; activation rows
    # 1, 8, 64 (decode GEMV) over 32 rotated weight buffers, and the int8 tensor-core GEMM at 4096 rows
    ops = None
    if not args.no_ops and world == 1:
        ops = {"gemv": {}, "a8w8_gemm": {}, "note": "GEMV: 32 distinct weight buffers per shape rotated inside one graph replay "
               "(>= 0.27 GB per shape: above L2); frac = algorithmic bytes / time / measured copy peak.  GEMM: int8 x int8 -> "
               "int32 on tcgen05 kind::i8; frac against 2 x the measured bf16 burst peak (no measured int8 peak is available)"}
        nbuf = 32
        for (Nout, K) in ((4096, 4096), (16384, 4096), (4096, 16384)):
            tiled = []
            for _ in range(nbuf):
                pk = torch.randint(0, 256, (Nout, K // 2), device=dev, dtype=torch.uint8)
                sc = (torch.rand(Nout, K // 128, device=dev) * 0.01 + 0.002).half()
                tiled.append(hb.w4_repack_tiled(pk, sc, K, 128))
                del pk, sc
            q8 = [torch.randint(-127, 128, (Nout, K), device=dev, dtype=torch.int8) for _ in range(nbuf)]
            t8 = [hb.w8_repack_tiled(q) for q in q8]
            s8 = (torch.rand(Nout, device=dev) * 0.01 + 0.002).half()
            for M in (1, 8, 64):
                x = f16(M, K)
                us4 = time_graph(lambda: [hb.w4_tiled_linear(x, t, Nout, K) for t in tiled], nbuf, reps=5)
                us8 = time_graph(lambda: [hb.w8_tiled_linear_group((x,), (t,), (s8,), Nout, K) for t in t8], nbuf, reps=5)
                b4, b8 = w4_launch_bytes(M, K, Nout), w8_launch_bytes(M, K, Nout)
                entry = {"int4_g128_tcgen05": {"us": us4, "gbs": b4 / us4 / 1e3, "frac": b4 / us4 / 1e3 / hbm_peak},
                         "int8_per_channel_tcgen05": {"us": us8, "gbs": b8 / us8 / 1e3, "frac": b8 / us8 / 1e3 / hbm_peak}}
                if M == 1:  # the CUDA-core GEMV on the reference layout, the small-batch route of w8_linear
                    usg = time_graph(lambda: [hb.w8_linear(x, q, s8) for q in q8], nbuf, reps=5)
                    entry["int8_per_channel_gemv"] = {"us": usg, "gbs": b8 / usg / 1e3, "frac": b8 / usg / 1e3 / hbm_peak}
                ops["gemv"][f"w{Nout}x{K}_m{M}"] = entry
            del tiled, q8, t8
            torch.cuda.empty_cache()
        for (Mg, K, Nout) in ((4096, 4096, 4096), (4096, 4096, 16384)):
            qa = torch.randint(-127, 128, (Mg, K), device=dev, dtype=torch.int8)
            qws = [torch.randint(-127, 128, (Nout, K), device=dev, dtype=torch.int8) for _ in range(4)]
            us = time_graph(lambda: [hb.int8_mm(qa, qw) for qw in qws], 4, reps=5)
            tops = 2.0 * Mg * K * Nout / us / 1e6
            ops["a8w8_gemm"][f"m{Mg}_k{K}_n{Nout}"] = {"us": us, "tops": tops, "frac_of_2x_bf16_burst": tops / (2 * tc_burst)}
            del qa, qws
        torch.cuda.empty_cache()
        # prefill-sized projections (64 sequences x 512 tokens) on the persistent CTA-pair GEMM: raw int8 accumulators,
        # the whole A8W8 linear (row quantiser + GEMM with the dequantisation in its epilogue), and the fp16 GEMM with
        # the FFN's relu^2 fused; the library GEMM on the same fp16 operands stands beside as a yardstick
        ops["prefill_gemm"] = {}
        for (Mg, K, Nout) in ((32768, 4096, 4096), (32768, 4096, 16384), (32768, 16384, 4096)):
            xg = torch.randn(Mg, K, device=dev, dtype=torch.float16)
            wg = (torch.randn(Nout, K, device=dev, dtype=torch.float16) / 64)
            qt, sc = hb.quantize_weight_per_channel_int8(wg)
            qrow = qt.t().contiguous()
            qa, _sa = hb.dynamic_a8_quant(xg)
            wsp = hb.quant.a8w8_workspace(Mg, K, Nout, dev)
            fl = 2.0 * Mg * K * Nout
            ent = {}
            for nm, fn, peak in (("int8_raw", lambda: hb.int8_mm(qa, qrow), 2 * tc_burst),
                                 ("a8w8_linear", lambda: hb.a8w8_linear(xg, qt, sc, workspace=wsp), 2 * tc_burst),
                                 ("fp16", lambda: hb.dense_linear(xg, wg), tc_burst),
                                 ("fp16_relu2", lambda: hb.dense_linear(xg, wg, relu2=True), tc_burst),
                                 ("library_fp16", lambda: torch.nn.functional.linear(xg, wg), tc_burst)):
                us = time_graph(fn, 1, reps=5)
                ent[nm] = {"us": us, "tflops": fl / us / 1e6, "frac_of_peak": fl / us / 1e6 / peak}
            ops["prefill_gemm"][f"m{Mg}_k{K}_n{Nout}"] = ent
            del xg, wg, qt, qrow, qa, wsp
            torch.cuda.empty_cache()

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        cb = run_cpu_baseline(args.shape, args.batch, steps=3, warmup=1, budget_s=60.0)
        cpu_baseline = {k_: cb[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}

    line = {
        "metric": METRIC, "value": global_batch / (ms_per_step * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": dict(base_cfg, recurrent_state=args.state, global_batch=global_batch, batch_per_gpu_step=B, layers=Lr, quantised_modules=nq,
                       parallelism=parallelism,
                       l2="working set per step (weights + state, GBs) exceeds the 126 MB L2; no flush needed",
                       cuda_graph=True),
        "e2e": {"value": global_batch / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": global_batch * 8, "d2h_bytes_per_step": global_batch * 8,
                "api": "RWKV7ForCausalLM.rwkv7_forward_token(return_tokens=True)"},
        # kernels of this library launched in the timed region, summed over the GPUs
        "gpu_launches": launches_per_step * steps * world,
        "gpu_launches_per_step": launches_per_step,
        "tp_parity": tp_parity, "replicas" if use_tp else "head_sharded_tp": replicas, "strong_scaling": strong,
        "clocks": clocks, "roofline": roofline, "roofline_secondary": roofline_wkv, "cpu_baseline": cpu_baseline,
        "decode_b256": b256, "state_pool": pool_stats, "prefill": prefill, "wkv_scan": scan, "ops": ops,
        **extra,
    }
    if args.layers:
        line["config"]["INVALID"] = "layer count overridden for debugging"
    if tp_parity is not None and tp_parity.get("status") != "ok":
        line["config"]["INVALID"] = "head-sharded parity check failed: " + json.dumps(tp_parity)[:200]
    note("line ready")
    print(json.dumps(line), flush=True)
    if tp_parity is not None and tp_parity.get("status") != "ok":
        sys.stdout.flush()
        os._exit(3)
    leave()


if __name__ == "__main__":
    main()
