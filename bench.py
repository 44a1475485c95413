"""Decode benchmark of the mode="flashsvd" hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one greedy decode step (one new token per sequence) of the 32-layer Llama-2-7B-shaped
model whose projections are all factored W = U·V (ranks 1024 / 1488, ~50 % of the dense
parameters), bf16, batch 1, 512 tokens of context: the configuration the reference's decode
benchmark reports (docs/notes/CURRENT_STATUS.md:111-128; utils/evaluator.py:499-540).  Weights and
the cached keys / values are seeded random tensors of those shapes.

N > 1 (torchrun): every rank decodes its own sequence on its own replica, no collective on the
data path; the printed value is the sum over ranks divided by the slowest rank's time.

At N = 1 the line also carries: `parity_check` (the timed engine stepped beside the CPU oracle,
outside the timed region), `cpu_baseline` (the oracle timed on the host cores), and `secondary`
(the other workloads of the benchmark configurations, each timed the same way on a fresh engine).

`--impl reference` times the CPU oracle (the restated PyTorch low-rank path) on the host cores.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode tokens/s (7B-shape SVD 50%, bf16, bs1, ctx512) and % of HBM roofline"
CTX = 512

# DRAM traffic / algorithmic bytes of the decode kernel, from the ncu capture summarised in the file
# named here (a 4-layer launch of the same program; traffic grows with the layer count in
# proportion to the algorithmic bytes).  Reported as an estimate with its source, not as a
# measurement of the run that prints it.
NCU_TRAFFIC_RATIO = 1.005
NCU_TRAFFIC_SOURCE = "profiles/fsvd_decode_kernel_model_4layers_ncu_full.md"


def workload_string(shape_name: str, layers: int, batch: int, ctx: int, share_pairs: bool, factors: str) -> str:
    """One description of the workload, shared by both arms of the benchmark."""
    model = ("llama2-7b shape (d 4096, 32 heads, I 11008), every projection W=U·V, ranks 1024/1488 (0.499 of dense)"
             if shape_name == "7b" else
             "llama2-70b shape (d 8192, GQA 64/8, I 28672), every projection W=U·V, ranks 1312/224/2704 (0.405 of dense)")
    s = f"{model}, {layers} layers, vocab 32000, batch {batch} per GPU, ctx {ctx}, greedy decode"
    if share_pairs:
        s += ", layer pairs share their input-side factors"
    if factors == "int4":
        s += ", int4-g128 factors (fp16 scales)"
    return s


def measured_hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        mx = next((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), None)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_reference_tokens_per_s(budget_s: float = 20.0):
    """The oracle on the host cores: whole tokens of the 32-layer 7B-shape model at ctx 512 (32 layer
    evaluations + final norm + lm_head per token), as many as fit the time budget (at least 2).
    The 32 layer evaluations cycle through 8 distinct sets of full-width factors (1.6 GB, far beyond
    the CPU caches), each layer with its own cache.  Returns (tok/s, threads, sample text)."""
    import torch

    from oracle import lowrank_llama as O

    threads = host_threads()
    torch.set_num_threads(threads)
    shape = O.LLAMA7B_SVD50
    n_sets = 8
    gen = torch.Generator().manual_seed(0)
    # bf16 storage and arithmetic, as the reference's PyTorch low-rank path runs a bf16 checkpoint
    dt = torch.bfloat16
    sets = [O.make_layer_weights(shape, gen, dt) for _ in range(n_sets)]
    lm_head = (torch.randn(shape.vocab, shape.d, generator=gen) / shape.d ** 0.5).to(dt)
    norm = torch.ones(shape.d, dtype=dt)
    S_max = CTX + 8
    ks = [torch.randn(1, S_max, shape.Hk, shape.Dh, generator=gen).to(dt) for _ in range(shape.n_layers)]
    vs = [torch.randn(1, S_max, shape.Hk, shape.Dh, generator=gen).to(dt) for _ in range(shape.n_layers)]
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dt)
    x0 = torch.randn(1, shape.d, generator=gen).to(dt)
    seq = torch.tensor([CTX], dtype=torch.int32)

    def one_token():
        h = x0
        for li in range(shape.n_layers):
            h = O.decode_layer(shape, sets[li % n_sets], h, ks[li], vs[li], seq, cos, sin)
        return torch.argmax(torch.nn.functional.linear(O.rmsnorm(h, norm, shape.eps), lm_head).float(), dim=-1)

    one_token()
    times = []
    t0 = time.perf_counter()
    while len(times) < 2 or (time.perf_counter() - t0 < budget_s and len(times) < 64):
        t1 = time.perf_counter()
        one_token()
        times.append(time.perf_counter() - t1)
    times.sort()
    per_token = times[len(times) // 2]
    sample = (f"{len(times)} whole tokens (median), each 32 layer evaluations at full width over {n_sets} distinct "
              f"factor sets + final norm + lm_head + argmax, ctx {CTX}, bf16 storage and arithmetic, "
              f"torch {torch.__version__} with {threads} threads")
    return 1.0 / per_token, threads, sample


def run_reference(args, rank):
    if rank != 0:
        return
    v, threads, sample = cpu_reference_tokens_per_s(budget_s=max(5.0, min(60.0, 2.0 * args.steps)))
    line = {
        "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"workload": workload_string("7b", 32, 1, CTX, False, "bf16"), "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def time_workload(dev, *, shape_name, layers, batch, ctx, share_pairs, factors, steps, warm, seed, world=1,
                  clocks_index=None, e2e=True, parity_steps=0, profile_range=False):
    """Builds one engine and times it: K kernel-only steps with everything resident, then (e2e)
    K steps in which the host feeds every token from pinned memory and reads every sampled token
    back.  Returns a dict of raw measurements (times are this rank's)."""
    import torch
    import torch.distributed as dist

    from flashsvd_b200 import ops, synthetic

    base = synthetic.LLAMA70B_SVD40 if shape_name == "70b" else synthetic.LLAMA7B_SVD50
    shape = dataclasses.replace(base, n_layers=int(layers))
    eng = synthetic.make_engine(shape, device=dev, dtype=torch.bfloat16, batch=batch, ctx=ctx,
                                max_new=warm + 2 * steps + parity_steps + 16, seed=seed,
                                factors="int4" if factors == "int4" else "dense", share_pairs=bool(share_pairs),
                                keep_raw=(factors == "int4" and parity_steps > 0))
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if profile_range:
        torch.cuda.profiler.start()   # profiler range = warm-up + timed regions (ncu --profile-from-start off)
    launches0 = ops.launch_count()
    eng.step(warm)
    barrier()
    sampler = ClockSampler(clocks_index) if clocks_index is not None else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    eng.step(steps)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    status = eng.status()
    launches = ops.launch_count() - launches0 - warm

    ms_e2e = None
    if e2e:
        pin_in = torch.zeros(batch, dtype=torch.int32).pin_memory()
        pin_out = torch.zeros(batch, dtype=torch.int32).pin_memory()
        tok = eng.tokens
        pin_in.copy_(tok.cpu())
        barrier()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record(stream)
        for _ in range(steps):
            tok.copy_(pin_in, non_blocking=True)      # H2D: the token to feed
            eng.step(1)
            pin_out.copy_(tok, non_blocking=True)     # D2H: the sampled token
            stream.synchronize()
            pin_in.copy_(pin_out)
        e3.record(stream)
        barrier()
        ms_e2e = e2.elapsed_time(e3)

    if profile_range:
        torch.cuda.profiler.stop()
    parity = None
    if parity_steps > 0:
        # the timed engine itself, stepped beside the CPU oracle from its current state (outside
        # every timed region)
        from oracle import check as OC

        res = OC.teacher_forced(eng, shape, parity_steps)
        parity = {"steps": parity_steps, "tokens_equal": res["tokens_equal"],
                  "tokens_explained_by_top2_gap": res["tokens_explained"], "rel_linf": max(res["rel_linf"]),
                  "against": "CPU oracle on the engine's own weights and caches, teacher-forced",
                  "device_status": eng.status()}
    q4 = factors == "int4"
    ctx_mid = ctx + warm + steps // 2
    bytes_step = shape.q4_bytes_per_step(ctx_mid, batch) if q4 else shape.bytes_per_step(ctx_mid, batch)
    layer_bytes = (shape.q4_bytes_per_layer() if q4 else shape.params_per_layer() * 2) + \
        2 * batch * ctx_mid * shape.Hk * shape.Dh * 2
    eng.close()
    del eng
    torch.cuda.empty_cache()
    return {"ms": ms, "ms_e2e": ms_e2e, "clocks": clocks, "status": status, "launches": int(launches),
            "bytes_step": bytes_step, "layer_bytes": layer_bytes, "parity": parity}


def time_prefill(dev, lengths, seed=0):
    """Prompt pass of one sequence through the 32-layer 7B-shape model (128 positions per pass on the
    tiled tensor-core path, the tail in smaller passes): ms per prompt and prompt tokens/s."""
    import torch

    from flashsvd_b200 import synthetic

    shape = synthetic.LLAMA7B_SVD50
    eng = synthetic.make_engine(shape, device=dev, dtype=torch.bfloat16, batch=1, ctx=0, max_new=max(lengths) + 16,
                                seed=seed, fill_cache=False)
    out = {}
    gen = torch.Generator(device=dev).manual_seed(seed)
    for L in lengths:
        prompt = torch.randint(0, shape.vocab, (1, L), device=dev, generator=gen, dtype=torch.int32)
        for it in range(2):      # the first pass builds the 128-row program (CUDA graph capture)
            eng.reset()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.prefill(prompt)
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        out[f"prompt_{L}"] = {"ms": ms, "prompt_tokens_per_s": L / (ms * 1e-3), "device_status": eng.status()}
    eng.close()
    del eng
    torch.cuda.empty_cache()
    return out


def run_tensor_parallel(args, dev, rank, world, local):
    """One model sharded over the ranks (heads and FFN intermediate; NCCL all-reduce of the o_proj and
    down-projection partial sums): tokens/s of the whole job and this path's bytes per GPU."""
    import torch
    import torch.distributed as dist

    from flashsvd_b200 import synthetic
    from flashsvd_b200 import tensor_parallel as TP

    shape = synthetic.LLAMA70B_SVD40 if args.shape == "70b" else synthetic.LLAMA7B_SVD50
    layers = shape.n_layers if args.layers is None else int(args.layers)
    B, ctx0, warm = int(args.batch), int(args.ctx), max(3, args.warmup)
    model = TP.random_tp_model(shape, rank=rank, world=world, device=dev, batch=B, ctx=ctx0,
                               max_new=warm + args.steps + 8, seed=0, n_layers=layers, exchange=args.tp_exchange,
                               shard_of=args.tp_shard_of, trace=args.tp_trace)
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    model.step(warm)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    model.step(args.steps)
    e1.record(stream)
    barrier()
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    status = model.status()
    xtrace = model.exchange.trace_summary() if (args.tp_trace and model.exchange is not None) else None
    how = ("partial sums of the o_proj and down projection pushed to every rank's memory by the GEMM epilogue "
           "(peer stores over NVLink) and summed by the next kernel, no collective call"
           if args.tp_exchange == "peer" else
           "per-op launches with an NCCL all-reduce of the o_proj and down-projection partial sums")
    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        per_gpu = model.bytes_per_step(ctx0 + warm + args.steps // 2)
        achieved = per_gpu / (ms / args.steps * 1e-3) / 1e9
        line = {
            "metric": METRIC + " [secondary workload, see config.workload]",
            "value": B * args.steps / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_string(args.shape, layers, B, ctx0, False, "bf16").replace(" per GPU", " in all") +
                       f", ONE model tensor-parallel over {world} GPUs (heads and FFN intermediate sharded, "
                       f"{how}, step replayed as a CUDA graph)",
                       "exchange": args.tp_exchange, "device_status": status,
                       **({"shard_of": args.tp_shard_of, "note": "one rank's share of a larger partition, timed without "
                           "its peers: not a throughput of the model"} if args.tp_shard_of else {})},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}, per GPU", "bytes_per_launch": per_gpu,
                         "note": "bytes one GPU reads per step: its factor shards + the replicated factors + its K/V rows + lm_head"},
            "clocks": clocks,
        }
        if xtrace:
            line["exchange_trace_rank0"] = xtrace
        print(json.dumps(line), flush=True)
    model.close()


def roofline_of(r, steps, peak, peak_kind):
    achieved = r["bytes_step"] / (r["ms"] / steps * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_kind": f"of {peak_kind}", "bytes_per_launch": r["bytes_step"], "bytes_per_layer": r["layer_bytes"],
            "us_per_layer_equiv": r["ms"] / steps * 1e3 * r["layer_bytes"] / r["bytes_step"]}


SECONDARY = (
    # (name, shape, layers, batch, ctx, share_pairs, factors)
    ("int4_b1_ctx512", "7b", 32, 1, 512, False, "int4"),
    ("int4_b16_ctx512", "7b", 32, 16, 512, False, "int4"),   # two launches of 8 sequences per step
    ("bf16_b8_ctx512", "7b", 32, 8, 512, False, "bf16"),
    ("shared_bases_b1_ctx2048", "7b", 32, 1, 2048, True, "bf16"),
    ("shared_bases_b8_ctx2048", "7b", 32, 8, 2048, True, "bf16"),
    ("70b_shape_replica_b1_ctx512", "70b", 80, 1, 512, False, "bf16"),
    # configuration 4 on ONE GPU (tiled path, tensor-core grouped-query attention); over 8 GPUs: --tp under torchrun
    ("70b_shape_one_gpu_b8_ctx4096", "70b", 80, 8, 4096, False, "bf16"),
    # batches above 8 run as tiled tcgen05 GEMMs + batched attention, one CUDA graph launch per step
    ("tiles_b16_ctx512", "7b", 32, 16, 512, False, "bf16"),
    ("tiles_shared_bases_b32_ctx2048", "7b", 32, 32, 2048, True, "bf16"),
    ("tiles_shared_bases_b128_ctx2048", "7b", 32, 128, 2048, True, "bf16"),   # 137 GB of K / V on the device
)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="flashsvd_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity-check", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads (N = 1 only runs them)")
    ap.add_argument("--shape", choices=("7b", "70b"), default="7b",
                    help="70b: the Llama-2-70B-shaped model (80 layers, GQA 64/8, ranks 1312/224/2704) as one replica "
                         "per GPU; a second workload, not the headline line")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has = a small case of the same kernel for profiler captures; "
                         "its line is marked profile_case and is not a benchmark result")
    ap.add_argument("--factors", choices=("bf16", "int4"), default="bf16",
                    help="int4: the same model with every U and V factor int4-g128 (codes uniform in [-8, 7], fp16 "
                         "scales uniform in [0.005, 0.02]); a second workload, not the headline line")
    ap.add_argument("--batch", type=int, default=1, help="sequences per GPU; other than 1 = a second workload")
    ap.add_argument("--ctx", type=int, default=CTX, help="cached positions before the first timed step")
    ap.add_argument("--share-pairs", action="store_true",
                    help="basis sharing: layers (2i, 2i+1) share their input-side factors")
    ap.add_argument("--tp", action="store_true",
                    help="tensor-parallel decode of ONE model over the ranks (configuration 4: --shape 70b --batch 8 "
                         "--ctx 4096 under torchrun); a secondary workload")
    ap.add_argument("--tp-exchange", default="peer", choices=("peer", "nccl"),
                    help="--tp: partial sums exchanged inside the kernels over peer memory (peer) or with an NCCL "
                         "all-reduce between per-op launches (nccl, the baseline)")
    ap.add_argument("--tp-trace", action="store_true",
                    help="--tp with the peer exchange: time every reduction on the device (%%globaltimer) and add "
                         "the wait for the peers and the reduction time of rank 0 to the line")
    ap.add_argument("--tp-shard-of", type=int, default=None,
                    help="--tp on fewer GPUs than the partition (profiling): the weights are rank 0's share of a "
                         "partition over this many ranks, the exchange has the ranks that run")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: flashsvd_b200 has no CPU path (use --impl reference for the CPU oracle)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if args.tp:
        run_tensor_parallel(args, dev, rank, world, local)
        if world > 1:
            dist.destroy_process_group()
        return

    full_layers = 80 if args.shape == "70b" else 32
    layers = full_layers if args.layers is None else int(args.layers)
    warm = max(3, args.warmup)
    B, ctx0 = int(args.batch), int(args.ctx)
    headline = (args.shape == "7b" and layers == 32 and B == 1 and ctx0 == CTX and not args.share_pairs
                and args.factors == "bf16")
    do_parity = headline and world == 1 and not args.no_parity_check
    r = time_workload(dev, shape_name=args.shape, layers=layers, batch=B, ctx=ctx0, share_pairs=args.share_pairs,
                      factors=args.factors, steps=args.steps, warm=warm, seed=rank, world=world,
                      clocks_index=local if rank == 0 else None, e2e=True, parity_steps=4 if do_parity else 0,
                      profile_range=True)

    times = torch.tensor([r["ms"], r["ms_e2e"]], device=dev, dtype=torch.float64)
    # independent sequences: every rank decodes its own B sequences on a full replica of the factors,
    # the ranks meet only here (max of the step times); no data-path collective
    from flashsvd_b200 import partition
    partition.max_over_ranks(times)
    ms, ms_e2e = float(times[0]), float(times[1])
    r["ms"] = ms

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        roof = roofline_of(r, args.steps, peak, peak_kind)
        roof["traffic"] = NCU_TRAFFIC_RATIO * r["bytes_step"] if headline else None
        roof["traffic_source"] = (f"estimate: algorithmic bytes x {NCU_TRAFFIC_RATIO} (ncu dram bytes of a 4-layer "
                                  f"launch, {NCU_TRAFFIC_SOURCE})") if headline else None
        line = {
            "metric": METRIC if headline else METRIC + " [secondary workload, see config.workload]",
            "value": partition.aggregate_tokens_per_s([B * args.steps] * world, [ms] * world),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warm,
            "ms_per_step": ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": workload_string(args.shape, layers, B, ctx0, args.share_pairs, args.factors),
                "l2": "not flushed: a step streams its factors once, far more than the 126 MB L2",
                "one_step": "one kernel launch",
                "device_status": r["status"],
                **({"profile_case": f"{layers} of {full_layers} layers"} if layers != full_layers else {}),
            },
            "roofline": roof,
            "e2e": {"value": world * B * args.steps / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": r["launches"],
            "clocks": r["clocks"],
            "parity_check": r["parity"] if do_parity else None,
        }
        if not args.no_cpu_baseline and world == 1:
            v, threads, sample = cpu_reference_tokens_per_s(budget_s=15.0)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
        else:
            line["cpu_baseline"] = None
        if headline and world == 1 and not args.no_secondary:
            sec = {}
            for name, sname, lay, b2, c2, share, fac in SECONDARY:
                try:
                    s = time_workload(dev, shape_name=sname, layers=lay, batch=b2, ctx=c2, share_pairs=share,
                                      factors=fac, steps=8, warm=3, seed=0, e2e=False)
                    ro = roofline_of(s, 8, peak, peak_kind)
                    sec[name] = {"workload": workload_string(sname, lay, b2, c2, share, fac),
                                 "value": b2 * 8 / (s["ms"] * 1e-3), "unit": "tokens/s", "ms_per_step": s["ms"] / 8,
                                 "steps": 8, "warmup": 3, "roofline_frac": ro["frac"], "achieved_gbs": ro["achieved"],
                                 "bytes_per_launch": ro["bytes_per_launch"], "device_status": s["status"]}
                except Exception as e:   # a secondary workload must not cost the headline line
                    sec[name] = {"error": f"{type(e).__name__}: {e}"}
            try:
                sec["prefill_7b_shape_b1"] = time_prefill(dev, (512, 2048))
            except Exception as e:
                sec["prefill_7b_shape_b1"] = {"error": f"{type(e).__name__}: {e}"}
            line["secondary"] = sec
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
