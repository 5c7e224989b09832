"""Benchmark of the routed-MoE layer (one "step" = one layer call over one batch of synthetic tokens).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T] [--routing normal|zipf]

Workload at N=1 (BASELINE config 1 of the list after the CPU-runnable case, "c2"): DeepSeek-V4.1-Flash-shaped decode
layer, EXL3 K=3 bank, hidden 5120, inter 2304, 256 routed experts, top-8, one bf16 shared expert, T = 64 tokens per
call.  Weights are synthetic (seeded random trellis codes, +-(0.5+u) sign/scale vectors), activations bf16 N(0,1),
logits N(0,1) or Zipf(1.1)-skewed.  Prints ONE JSON line (rank 0).

`value` = tokens/s with inputs resident in HBM; `e2e` = the same through the host-buffer entry (mlxs_moe_forward_host,
pinned host memory, copies inside the timed region); `roofline` = the gate/up streaming kernel against the measured
HBM peak; `cpu_baseline` = the CPU oracle's fast f32 form on a bounded sample of the same workload.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

H, I, E, K_TOP = 5120, 2304, 256, 8
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_logits(rng, T, routing):
    lg = rng.standard_normal((T, E)).astype(np.float32)
    if routing == "zipf":
        perm = rng.permutation(E)
        p = (np.arange(1, E + 1, dtype=np.float64) ** -1.1)
        p /= p.sum()
        lg = lg + np.log(p)[np.argsort(perm)].astype(np.float32)
    return lg


def reference_arm(args):
    """The reference's CPU path for this layer, timed on the host cores.  The reference's own CPU lane (Zig tests over
    MLX's CPU device) cannot be built here (no zig, no mlx), so this runs the oracle's fast f32 form (kind "port")."""
    import oracle_lib as O
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.cpu_tokens
    rng = np.random.default_rng(1234)
    threads = O.max_threads()
    lg = make_logits(rng, T, args.routing)
    ids, w = O.route(lg, None, K_TOP, O.SCORE_SQRTSOFTPLUS, scale=1.5)
    recs = {int(e): O.exl3_synth_record(0xB200 + int(e), H, I, 1.0, 0.02) for e in np.unique(ids)}
    srng = np.random.default_rng(7)
    shared = [O.f32_to_bf16_bits((srng.standard_normal(s) * 0.02).astype(np.float32))
              for s in ((I, H), (I, H), (H, I))]
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal((T, H)).astype(np.float32)))
    for _ in range(args.warmup):
        O.layer_fast(H, I, E, K_TOP, recs, x, ids, w, shared=shared, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.layer_fast(H, I, E, K_TOP, recs, x, ids, w, shared=shared, threads=threads)
    dt = time.perf_counter() - t0
    v = T * args.steps / dt
    sample = f"{T} tokens x top-{K_TOP} per step ({len(recs)} distinct experts), whole layer incl. shared expert"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 accumulate over f16-valued EXL3 weights", "data": "synthetic",
        "config": workload_config(args, T),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(args, T):
    return {"workload": "c2: DeepSeek-V4.1-Flash-shaped routed MoE decode layer, EXL3 K=3 mul1 bank",
            "hidden": H, "inter": I, "n_experts": E, "top_k": K_TOP, "shared_expert": "bf16", "tokens_per_call": T,
            "routing": args.routing, "l2": "inputs larger than L2 (each call streams >2 GB of distinct expert code)",
            "parallelism": "single GPU" if args.gpus == 1 else f"ep{args.gpus}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--cpu-tokens", type=int, default=8)
    ap.add_argument("--routing", default="normal", choices=["normal", "zipf"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--experts", type=int, default=E, help="routed experts (smaller only for profiler captures)")
    args = ap.parse_args()
    globals()["E"] = args.experts
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    if args.impl == "reference":
        args.steps = min(args.steps, 3)
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T = args.tokens

    cfg = pkg.make_config(H, I, E, K_TOP, n_layers=1, bank_kind=pkg.BANK_EXL3_K3_MUL1, act=pkg.ACT_SWIGLU_CLAMPED,
                          act_limit=10.0, scoring=pkg.SCORE_SQRTSOFTPLUS, norm_topk=True, routed_scale=1.5,
                          shared_expert=True, combine=pkg.COMBINE_F32, max_tokens=max(T, 64), device=local)
    moe = pkg.MoE(cfg)
    logical, stride = moe.record_bytes()
    # synthetic bank generated on the device in the reference's record layout: random trellis codes, +-(0.5+u) scales
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + rank)
    code_bytes = (H // 16) * (I // 16) * 96
    for e in range(E):
        rec = torch.randint(0, 256, (stride,), dtype=torch.uint8, device=dev, generator=g)
        off = 0
        for p in range(3):
            off += code_bytes
            n_out, n_in = (H, I) if p == 2 else (I, H)
            for n, sc in ((n_out, 0.02), (n_in, 1.0)):
                u = torch.rand(n, device=dev, generator=g)
                sgn = torch.where(torch.rand(n, device=dev, generator=g) < 0.5, -1.0, 1.0)
                rec[off:off + 2 * n] = ((0.5 + u) * sgn * sc).to(torch.float16).view(torch.uint8)
                off += 2 * n
        moe.load_expert(0, e, rec.data_ptr(), stride, on_device=True)
    sw = [(torch.randn(s, device=dev, generator=g) * 0.02).to(torch.bfloat16) for s in ((I, H), (I, H), (H, I))]
    moe.set_shared(0, sw[0].data_ptr(), sw[1].data_ptr(), sw[2].data_ptr(), on_device=True)

    rng = np.random.default_rng(99 + rank)
    n_batches = 4  # rotate a few seeded batches so consecutive steps route differently
    xs, lgs, x_host, lg_host = [], [], [], []
    for b in range(n_batches):
        lg = make_logits(rng, T, args.routing)
        x = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
        xs.append(x)
        lgs.append(torch.from_numpy(lg).to(dev))
        x_host.append(x.cpu().pin_memory())
        lg_host.append(torch.from_numpy(lg).pin_memory())
    y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    y_host = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream

    def step(i):
        moe.forward(0, xs[i % n_batches].data_ptr(), lgs[i % n_batches].data_ptr(), T, y.data_ptr(), sp)

    def step_host(i):
        moe.forward_host(0, x_host[i % n_batches].data_ptr(), lg_host[i % n_batches].data_ptr(), T,
                         y_host.data_ptr(), sp)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for i in range(args.warmup):
        step(i)
    # distinct experts per batch (exact, from the routed ids) for the algorithmic byte count
    distinct = []
    for b in range(n_batches):
        step(b)
        distinct.append(int(moe.stats().distinct_experts_last))
    sampler = ClockSampler(local)
    sampler.start()
    moe.profile_enable(True)
    moe.profile_read()
    ms = timed(step, args.steps)
    prof = moe.profile_read()
    moe.profile_enable(False)
    clocks = sampler.stop()
    for i in range(args.warmup):
        step_host(i)
    ms_host = timed(step_host, args.steps)
    st = moe.stats()
    if st.device_status != 0:
        raise SystemExit(f"bench.py: device status {st.device_status}")

    mean_distinct = sum(distinct[i % n_batches] for i in range(args.steps)) / args.steps
    gu_bytes = 2 * code_bytes + 2 * (2 * I + 2 * H)  # one expert's gate + up code and sign/scale vectors
    gu_ms, gu_n = prof["gate_up"]
    peak, which = peaks()
    achieved = mean_distinct * gu_bytes / (gu_ms / max(gu_n, 1) * 1e-3) / 1e9
    layer_bytes = mean_distinct * logical + 3 * H * I * 2 + T * H * 2 * 2 + T * E * 4
    value = world * T * args.steps / (ms * 1e-3)
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 trellis weights x f16 hi/lo activations, f32 accumulate", "data": "synthetic",
        "config": workload_config(args, T),
        "layer_hbm": {"algorithmic_bytes_per_call": layer_bytes, "gb_s": layer_bytes / (ms / args.steps * 1e-3) / 1e9,
                      "frac_of_measured_peak": layer_bytes / (ms / args.steps * 1e-3) / 1e9 / peak,
                      "frac_of_nominal_8000": layer_bytes / (ms / args.steps * 1e-3) / 1e9 / 8000.0,
                      "distinct_experts_mean": mean_distinct},
        "roofline": {"kernel": "exl3_gemv_kernel<2,gate_up>", "bound": "hbm", "achieved": achieved, "peak": peak,
                     "peak_source": which, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "algorithmic_bytes_per_launch": mean_distinct * gu_bytes},
        "stage_ms_per_step": {k: v[0] / max(args.steps, 1) for k, v in prof.items() if v[1]},
        "e2e": {"value": world * T * args.steps / (ms_host * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": T * H * 2 + T * E * 4, "d2h_bytes_per_step": T * H * 2 + 4},
        "gpu_launches": 8 * args.steps,
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle_lib as O
        Tc = args.cpu_tokens
        crng = np.random.default_rng(1234)
        lg = make_logits(crng, Tc, args.routing)
        ids, w = O.route(lg, None, K_TOP, O.SCORE_SQRTSOFTPLUS, scale=1.5)
        recs = {int(e): O.exl3_synth_record(0xB200 + int(e), H, I, 1.0, 0.02) for e in np.unique(ids)}
        shared = [s.view(torch.int16).cpu().numpy().view(np.uint16) for s in sw]
        xc = O.bf16_bits_to_f32(O.f32_to_bf16_bits(crng.standard_normal((Tc, H)).astype(np.float32)))
        threads = O.max_threads()
        t0 = time.perf_counter()
        O.layer_fast(H, I, E, K_TOP, recs, xc, ids, w, shared=shared, threads=threads)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": Tc / dt, "unit": UNIT, "cores": threads, "kind": "port",
                               "sample": f"{Tc} tokens x top-{K_TOP} ({len(recs)} distinct experts), one call, "
                                         "oracle fast f32 form with OpenMP"}
    if rank == 0:
        print(json.dumps(out))
    moe.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
