"""Decode benchmark of the mode="flashsvd" hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one greedy decode step (one new token per sequence) of the 32-layer Llama-2-7B-shaped
model whose projections are all factored W = U·V (ranks 1024 / 1488, ~50 % of the dense
parameters), bf16, batch 1, 512 tokens of context: the configuration the reference's decode
benchmark reports (docs/notes/CURRENT_STATUS.md:111-128; utils/evaluator.py:499-540).  Weights and
the cached keys / values are seeded random tensors of those shapes.

N > 1 (torchrun): every rank decodes its own sequence on its own replica, no collective on the
data path; the printed value is the sum over ranks divided by the slowest rank's time.

`--impl reference` times the CPU oracle (the restated PyTorch low-rank path) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# DRAM traffic / algorithmic bytes of the decode kernel from one ncu capture of a 4-layer launch
# (profiles/fsvd_decode_kernel_model_4layers_ncu_full.md); traffic grows with the layer count in
# proportion to the algorithmic bytes.
NCU_TRAFFIC_RATIO = 1.003

METRIC = "decode tokens/s (7B-shape SVD 50%, bf16, bs1, ctx512) and % of HBM roofline"
CTX = 512


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


def cpu_reference_tokens_per_s(budget_s: float = 20.0):
    """The oracle on the host cores, bounded sample: a few of the 32 layers at full width, one
    token at ctx 512, scaled to 32 layers plus lm_head.  Returns (tok/s, cores, sample text)."""
    import torch

    from oracle import lowrank_llama as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    shape = O.LLAMA7B_SVD50
    n_l = 2
    # bf16 storage as on the GPU; fp32 arithmetic (bf16 GEMV on this CPU is slower), values bf16-rounded
    gen = torch.Generator().manual_seed(0)
    layers = [{k: v.to(torch.bfloat16).float() for k, v in O.make_layer_weights(shape, gen, torch.float32).items()}
              for _ in range(n_l)]
    lm_head = (torch.randn(shape.vocab, shape.d, generator=gen) / shape.d ** 0.5).to(torch.bfloat16).float()
    S_max = CTX + 8
    ks = [torch.randn(1, S_max, shape.Hk, shape.Dh, generator=gen) for _ in range(n_l)]
    vs = [torch.randn(1, S_max, shape.Hk, shape.Dh, generator=gen) for _ in range(n_l)]
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, torch.float32)
    x = torch.randn(1, shape.d, generator=gen)
    seq = torch.tensor([CTX], dtype=torch.int32)

    def one_token():
        h = x
        for w, k, v in zip(layers, ks, vs):
            h = O.decode_layer(shape, w, h, k, v, seq, cos, sin)
        return torch.nn.functional.linear(O.rmsnorm(h, torch.ones(shape.d), shape.eps), lm_head)

    one_token()
    t0 = time.perf_counter()
    n = 0
    while True:
        t1 = time.perf_counter()
        for w, k, v in zip(layers, ks, vs):
            O.decode_layer(shape, w, x, k, v, seq, cos, sin)
        t_layers = time.perf_counter() - t1
        t2 = time.perf_counter()
        torch.nn.functional.linear(x, lm_head)
        t_head = time.perf_counter() - t2
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 8:
            break
    per_token = t_layers / n_l * shape.n_layers + t_head
    sample = (f"{n_l} of {shape.n_layers} layers at full width + lm_head, 1 token at ctx {CTX}, repeated {n}x, "
              f"scaled to {shape.n_layers} layers; bf16-rounded weights, fp32 arithmetic")
    return 1.0 / per_token, cores, sample


def run_reference(args, rank):
    if rank != 0:
        return
    v, cores, sample = cpu_reference_tokens_per_s(budget_s=max(5.0, min(60.0, 5.0 * args.steps)))
    line = {
        "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"workload": "llama2-7b-shape, every projection W=U·V (ranks 1024/1488), 32 layers, batch 1, ctx 512, greedy decode",
                   "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="flashsvd_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shape", choices=("7b", "70b"), default="7b",
                    help="70b: the Llama-2-70B-shaped model (80 layers, GQA 64/8, ranks 1312/224/2704) as one replica "
                         "per GPU; a second workload, not the headline line")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer than 32 layers = a small case of the same kernel for profiler captures; "
                         "its line is marked profile_case and is not a benchmark result")
    ap.add_argument("--factors", choices=("bf16", "int4"), default="bf16",
                    help="int4: the same model with every U and V factor int4-g128 (codes uniform in [-8, 7], fp16 "
                         "scales uniform in [0.005, 0.02]); a second workload, not the headline line")
    ap.add_argument("--batch", type=int, default=1, help="sequences per GPU (1..8); other than 1 = a second workload")
    ap.add_argument("--ctx", type=int, default=CTX, help="cached positions before the first timed step")
    ap.add_argument("--share-pairs", action="store_true",
                    help="basis sharing: layers (2i, 2i+1) share their input-side factors")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    from flashsvd_b200 import ops, synthetic

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: flashsvd_b200 has no CPU path (use --impl reference for the CPU oracle)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    shape = synthetic.LLAMA70B_SVD40 if args.shape == "70b" else synthetic.LLAMA7B_SVD50
    if args.layers is None:
        args.layers = shape.n_layers
    if args.layers != shape.n_layers:
        import dataclasses

        shape = dataclasses.replace(shape, n_layers=int(args.layers))
    warm = max(3, args.warmup)
    B, ctx0 = int(args.batch), int(args.ctx)
    eng = synthetic.make_engine(shape, device=dev, dtype=torch.bfloat16, batch=B, ctx=ctx0,
                                max_new=warm + 2 * args.steps + 16, seed=rank,
                                factors="int4" if args.factors == "int4" else "dense",
                                share_pairs=bool(args.share_pairs))
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- kernel-only: K steps, inputs resident in HBM, device-side token feedback
    torch.cuda.profiler.start()   # profiler range = warm-up + timed regions (ncu --profile-from-start off)
    launches0 = ops.launch_count()
    eng.step(warm)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    eng.step(args.steps)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    status = eng.status()
    launches = ops.launch_count() - launches0 - warm

    # ---- end to end: the host feeds every token and reads every sampled token back
    pin_in = torch.zeros(B, dtype=torch.int32).pin_memory()
    pin_out = torch.zeros(B, dtype=torch.int32).pin_memory()
    tok = eng.tokens
    pin_in.copy_(tok.cpu())
    barrier()
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record(stream)
    for _ in range(args.steps):
        tok.copy_(pin_in, non_blocking=True)      # H2D: the token to feed
        eng.step(1)
        pin_out.copy_(tok, non_blocking=True)     # D2H: the sampled token
        stream.synchronize()
        pin_in.copy_(pin_out)
    e3.record(stream)
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    torch.cuda.profiler.stop()

    times = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(times[0]), float(times[1])

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        ctx_mid = ctx0 + warm + args.steps // 2
        q4 = args.factors == "int4"
        bytes_step = shape.q4_bytes_per_step(ctx_mid, B) if q4 else shape.bytes_per_step(ctx_mid, B)
        variant = B != 1 or ctx0 != CTX or args.share_pairs or args.shape != "7b"
        achieved = bytes_step / (ms / args.steps * 1e-3) / 1e9
        layer_bytes = (shape.q4_bytes_per_layer() if q4 else shape.params_per_layer() * 2) + \
            2 * B * ctx_mid * shape.Hk * shape.Dh * 2
        line = {
            "metric": METRIC + (" [int4-g128 factors]" if q4 else ""),
            "value": world * B * args.steps / (ms * 1e-3),
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
                "workload": "llama2-7b-shape, every projection W=U·V (ranks 1024/1488, 0.499 of dense), 32 layers, "
                            "vocab 32000, batch 1 per GPU, ctx 512, greedy decode; one step = one kernel launch",
                "l2": "not flushed: a step streams 6.99 GB of factors, far more than the 126 MB L2",
                "device_status": status,
                **({"profile_case": f"{shape.n_layers} layers only"}
                   if shape.n_layers != (80 if args.shape == "70b" else 32) else {}),
                **({"variant": ("llama2-70b shape (80 layers, ranks 1312/224/2704), " if args.shape == "70b" else "") +
                    f"batch {B} per GPU, ctx {ctx0}" + (", layer pairs share input-side factors"
                                                                     if args.share_pairs else "")} if variant else {}),
                **({"factors": "int4-g128 symmetric, fp16 scales, dequantised inside the kernel; "
                               f"{bytes_step / 1e9:.2f} GB per step"} if q4 else {}),
            },
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_kind": f"of {peak_kind}", "traffic": None if (q4 or variant) else NCU_TRAFFIC_RATIO * bytes_step,
                "traffic_note": "ncu dram bytes of a 4-layer launch scaled by algorithmic bytes",
                "bytes_per_launch": bytes_step, "bytes_per_layer": layer_bytes,
                "us_per_layer_equiv": ms / args.steps * 1e3 * layer_bytes / bytes_step,
            },
            "e2e": {"value": world * B * args.steps / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            v, cores, sample = cpu_reference_tokens_per_s(budget_s=15.0)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    eng.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
