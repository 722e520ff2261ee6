"""Headline benchmark: decode tok/s at B=64 (+ prefill tok/s) on the 7.2B-shape RWKV-7 with int4
group-128 projections and an fp16 head, random weights, synthetic token ids.

    python bench.py --gpus 1 --steps K --warmup W            # this framework
    python bench.py --impl reference --steps K --warmup W    # CPU baseline arm (host cores)
    torchrun ... bench.py --gpus N ...                       # N>1: head-sharded tensor parallel

One "step" = one decode token for every sequence of the batch (all 32 layers + head), replayed as a
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


def decode_step_bytes(L, D, H, Fd, V, B, group=128, ranks=(64, 64, 32, 128)):
    """Algorithmic HBM bytes of one decode step: int4 weights + fp16 group scales, fp16 LoRA and head,
    fp32 state read+write, shift states read+write."""
    A = H * 64
    w_int4 = (4 * D * A + 2 * D * Fd) // 2
    w_scales = (4 * D * A + 2 * D * Fd) // group * 2
    rw, ra, rv, rg = ranks
    lora = (rw + ra + rg + rv) * (D + A) * 2
    weights = L * (w_int4 + w_scales + lora) + V * D * 2
    state = B * L * H * 64 * 64 * 4 * 2
    shift = B * L * 2 * D * 2 * 2
    return weights + state + shift, weights, state


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
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, "fallback"


# ------------------------------------------------------------------------------------------ model
def build_model(shape, tp_world, tp_rank, tp_group, device, layers_override=0):
    """Random-init model of the named shape, projections quantised to int4 group-128 on the GPU, fp16 head.
    The token-shift / key-scale parameters the reference constructs as zeros are re-initialised (seeded) so
    that every term of the recurrence is exercised."""
    import torch

    import hf_adapter_b200 as hb

    L, D, H, Fd, V = SHAPES[shape]
    if layers_override:
        L = layers_override
    cfg = hb.NativeRWKV7Config(vocab_size=V, hidden_size=D, num_hidden_layers=L, num_heads=H, head_dim=64,
                               intermediate_size=Fd, **RANKS)
    torch.manual_seed(0)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.float16)
    try:
        with torch.device(device):
            model = hb.RWKV7ForCausalLM(cfg, tp_world=tp_world, tp_rank=tp_rank, tp_group=tp_group)
    finally:
        torch.set_default_dtype(old)
    g = torch.Generator(device=device).manual_seed(1 + tp_rank)
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
    n = hb.quantize_model(model, "mm4", min_params=1_000_000, group_size=128, skip=("lm_head",))
    torch.cuda.empty_cache()
    return model.eval(), cfg, n


# ------------------------------------------------------------------------------------------ reference arm
def run_cpu_baseline(shape, B, steps, warmup, layers_sample=1):
    """Times the CPU port of the reference's decode layer on the host cores.  A step = `layers_sample`
    layers of the model at batch B (plus the head once per step, scaled); the full-model step time is
    extrapolated as L/layers_sample * t_layers + t_head and says so in `sample`."""
    import torch

    from oracle import cpu_port_torch as P

    L, D, H, Fd, V = SHAPES[shape]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ranks = (RANKS["decay_low_rank_dim"], RANKS["a_low_rank_dim"], RANKS["v_low_rank_dim"], RANKS["gate_low_rank_dim"])
    layers = [P.make_layer(D, H, 64, Fd, ranks, layer_id=1 + i, seed=i) for i in range(layers_sample)]
    g = torch.Generator().manual_seed(0)
    head_w = torch.randn(V, D, generator=g) * 0.02
    nw, nb = torch.ones(D), torch.zeros(D)
    x = torch.randn(B, D, generator=g)
    xpa, xpf = torch.randn(B, D, generator=g), torch.randn(B, D, generator=g)
    vf = torch.randn(B, H * 64, generator=g)
    st = [0.1 * torch.randn(B, H, 64, 64, generator=g) for _ in layers]
    times = []
    t_begin = time.perf_counter()
    with torch.no_grad():
        for it in range(warmup + steps):
            if len(times) >= 3 and time.perf_counter() - t_begin > 180.0:
                break  # bounded: the run ends within a few minutes whatever --steps says; `sample` gives the count
            t0 = time.perf_counter()
            y = x
            for i, p in enumerate(layers):
                y, _, _, _, st[i] = P.layer_step(p, y, xpa, xpf, vf, st[i], H, 64)
            t1 = time.perf_counter()
            P.head_step(y, nw, nb, head_w)
            t2 = time.perf_counter()
            if it >= warmup:
                times.append(((t1 - t0) * L / layers_sample) + (t2 - t1))
    step_s = sum(times) / len(times)
    return {"value": B / step_s, "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{len(times)} timed steps of {layers_sample} of {L} layers + head per step at B={B}, fp32 activations, int4-g128 weights "
                      f"dequantised per call as the reference does on CPU; step time extrapolated x{L // layers_sample} for layers",
            "ms_per_step": step_s * 1e3}


# ------------------------------------------------------------------------------------------ main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="7.2B", choices=sorted(SHAPES))
    ap.add_argument("--batch", type=int, default=64, help="sequences per GPU group (global batch = batch for N=1)")
    ap.add_argument("--layers", type=int, default=0, help="debug: override the layer count (invalidates the metric)")
    ap.add_argument("--prefill-tokens", type=int, default=1024)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--prefill-scan-chunk", type=int, default=64,
                    help="tile of the tensor-core WKV scan in the prefill sample (0 = sequential scan)")
    ap.add_argument("--parallelism", default="dp", choices=["dp", "tp"],
                    help="N > 1: dp = independent sequence batches on full replicas (headline) with the head-sharded "
                         "tensor-parallel form measured beside it; tp = the head-sharded form as the headline")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-scan", action="store_true")
    args = ap.parse_args()
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    L, D, H, Fd, V = SHAPES[args.shape]
    metric = "decode tok/s @B=64 + prefill tok/s, 7.2B RWKV-7 MM4; WKV scan % HBM/TC peak"
    workload = f"rwkv7-{args.shape}-shape mm4-g128 decode, batch {args.batch}, fp16 head, cache resident"

    if args.impl == "reference":
        if rank != 0:
            return
        cb = run_cpu_baseline(args.shape, args.batch, steps, warmup)
        line = {"impl": "reference", "metric": metric, "value": cb["value"], "unit": "tok/s", "n_gpus": args.gpus,
                "steps": steps, "warmup": warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": workload, "note": "reference's CPU path (torch CPU port), host cores"},
                "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": cb["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import torch
    import torch.distributed as dist

    import hf_adapter_b200 as hb
    from hf_adapter_b200 import _lib

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    tp_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        tp_group = dist.group.WORLD

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def time_decode(model, B, seed, clocks_on_rank0):
        """Device-resident graph replays (-> ms per step), then the end-to-end loop through the public API; both are
        bracketed by a barrier + synchronize and reduced with MAX over the ranks."""
        gen = torch.Generator().manual_seed(seed)
        ids_host = torch.randint(0, V, (steps + warmup + 8, B), generator=gen).pin_memory()
        cache = model.new_cache(B)
        # kernels of this library launched per decode step (counted on one eager step through the C ABI; the step
        # before it builds the tiled weight copies, whose one-time repack kernels are not part of a step)
        model.rwkv7_forward_token(ids_host[0].to(dev), cache, use_graph=False)
        _lib.LAUNCHES = 0
        model.rwkv7_forward_token(ids_host[0].to(dev), cache, use_graph=False)
        launches = _lib.LAUNCHES
        graph = model._decode_graph(B)
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
        for i in range(steps):
            graph.ids.copy_(ids_dev[warmup + i])
            graph.graph.replay()
        ev1.record()
        barrier()
        ms_step = max_over_ranks(ev0.elapsed_time(ev1)) / steps
        # end to end: pinned ids -> H2D -> step -> argmax -> D2H, the caller consuming the token before the next step
        tok_host = torch.empty((B,), dtype=torch.long).pin_memory()
        for i in range(3):
            lg = model.rwkv7_forward_token(ids_host[i].to(dev, non_blocking=True), cache)
            tok_host.copy_(lg.argmax(-1), non_blocking=True)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            lg = model.rwkv7_forward_token(ids_host[warmup + i].to(dev, non_blocking=True), cache)
            tok_host.copy_(lg.argmax(-1), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        e1.record()
        barrier()
        e2e = max_over_ranks(e0.elapsed_time(e1)) / steps
        return ms_step, e2e, launches, cache, (sampler.stop() if sampler else None), gen

    # ---------------- more than one GPU, head-sharded form: heads, their state and the projections are sharded, the
    # batch grows with N (B = batch * N on every rank), two NCCL all-reduces per layer.  Measured first and reported
    # beside the headline, which for N > 1 is the partition without any data-path collective (below).
    tp_result = None
    if world > 1 and args.parallelism == "dp":
        try:
            tp_model, tp_cfg, _ = build_model(args.shape, world, rank, tp_group, dev, args.layers)
            tp_ms, tp_e2e, tp_launch, tp_cache, _, _ = time_decode(tp_model, args.batch * world, 0, False)
            tp_result = {"value": args.batch * world / (tp_ms * 1e-3), "unit": "tok/s", "ms_per_step": tp_ms,
                         "e2e_tok_per_s": args.batch * world / (tp_e2e * 1e-3), "global_batch": args.batch * world,
                         "parallelism": f"tp{world}: heads, state and projections sharded, batch {args.batch * world} on "
                                        "every rank, two NCCL all-reduces per layer in the decode graph"}
            tp_model._graphs.clear()
            del tp_cache, tp_model
        except Exception as exc:  # the headline below does not depend on this measurement
            tp_result = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

    # ---------------- headline.  N = 1: the model on one GPU.  N > 1 (default): independent sequence batches -- every
    # GPU holds a full replica and decodes its own `batch` sequences, no collective on the data path (weak scaling);
    # --parallelism tp makes the head-sharded form the headline instead.
    use_tp = world > 1 and args.parallelism == "tp"
    if use_tp:
        model, cfg, nq = build_model(args.shape, world, rank, tp_group, dev, args.layers)
        B, shard = args.batch * world, world
        parallelism = f"tp{world} (heads + projections sharded, batch {B} on every rank, two NCCL all-reduces per layer)"
    else:
        model, cfg, nq = build_model(args.shape, 1, 0, None, dev, args.layers)
        B, shard = args.batch, 1
        parallelism = "single GPU" if world == 1 else \
            f"dp{world}: independent sequence batches, one full replica per GPU, {args.batch} sequences each, no data-path collective"
    Lr = cfg.num_hidden_layers
    ms_per_step, e2e_ms, launches_per_step, cache, clocks, gen = time_decode(model, B, 0 if use_tp else rank, True)
    global_batch = B if use_tp else args.batch * world

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

    hbm_peak, tc_peak, peak_src = measured_peaks()
    step_bytes, w_bytes, s_bytes = decode_step_bytes(Lr, D, H // shard, Fd // shard, V, B)  # per GPU

    # ---------------- roofline of the dominant kernel (WKV-7 decode step), timed alone over all layers' states
    Hl = H // shard
    N = 64
    f16 = lambda *s: torch.randn(*s, device=dev, dtype=torch.float16)
    r, w_raw, k, v, a, g = (f16(B, Hl * N) for _ in range(6))
    at0 = model.model.layers[1].attn if Lr > 1 else model.model.layers[0].attn
    states = cache._state

    def wkv_pass():
        for s in states:
            hb.fused_recurrent_output_prepare_raw(r, w_raw, k, v, a, s, g, at0.k_k, at0.k_a, at0.r_k, at0.g_norm.weight,
                                                  at0.g_norm.bias, eps=N * 1e-5, new_state=s, out=wkv_out)

    wkv_out = torch.empty((B, Hl * N), device=dev, dtype=torch.float16)
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
    wkv_bytes = B * Hl * (2 * N * N * 4 + 7 * N * 2)
    achieved = wkv_bytes / (wkv_ms * 1e-3) / 1e9
    roofline = {"kernel": "wkv7_step_kernel (decode recurrence + fused epilogues)", "bound": "hbm", "achieved": achieved,
                "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src + " (burst copy)",
                # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture at B*H = 4096 (profiles/): 87.0 MB per
                # launch (reads = state in; most of the written state is still dirty in L2 when the kernel ends),
                # scaled by the sequence-heads of this launch
                "traffic": 87.0e6 * (B * Hl) / 4096.0, "bytes_per_launch": wkv_bytes, "us_per_launch": wkv_ms * 1e3}

    extra = {"step_bytes": step_bytes, "step_hbm_frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
             "wkv_share_of_step": wkv_ms * len(states) / ms_per_step}

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
                          "tensor_frac_of_bf16_peak": flops / (sms * 1e-3) / 1e12 / tc_peak}
        del rs, ks, vs, kks, as_, ws
        torch.cuda.empty_cache()

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        cb = run_cpu_baseline(args.shape, args.batch, steps=1, warmup=1)
        cpu_baseline = {k_: cb[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}

    line = {
        "metric": metric, "value": global_batch / (ms_per_step * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload, "global_batch": global_batch, "batch_per_gpu_step": B, "layers": Lr, "d_model": D, "heads": H, "ffn": Fd, "vocab": V,
                   "lora_ranks": RANKS, "quantised_modules": nq, "parallelism": parallelism,
                   "l2": "working set per step (weights + state, GBs) exceeds the 126 MB L2; no flush needed",
                   "cuda_graph": True},
        "e2e": {"value": global_batch / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": global_batch * 8, "d2h_bytes_per_step": global_batch * 8,
                "api": "RWKV7ForCausalLM.rwkv7_forward_token + argmax"},
        # kernels of this library launched in the timed region, summed over the GPUs
        "gpu_launches": launches_per_step * steps * world,
        "gpu_launches_per_step": launches_per_step,
        "head_sharded_tp": tp_result,
        "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu_baseline, "prefill": prefill, "wkv_scan": scan,
        **extra,
    }
    if args.layers:
        line["config"]["INVALID"] = "layer count overridden for debugging"
    print(json.dumps(line), flush=True)
    leave()


if __name__ == "__main__":
    main()
