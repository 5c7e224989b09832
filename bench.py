"""Benchmark of the routed-MoE layer (one "step" = one layer call over one batch of synthetic tokens).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T] [--routing normal|zipf]

Workload at N=1 (the benchmark list's first configuration after the CPU-runnable case, "c2"): DeepSeek-V4.1-Flash-shaped decode
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
# secondary workloads (the MXFP4 and NVFP4 configurations of the benchmark list), selected with --workload
WORKLOADS = {
    "c2": dict(name="c2: DeepSeek-V4.1-Flash-shaped routed MoE decode layer, EXL3 K=3 mul1 bank", H=5120, I=2304, E=256,
               k=8, bank="exl3", shared=True, scoring="sqrtsoftplus", scale=1.5, limit=10.0, chain=False),
    "c3": dict(name="c3: MiMo-shaped routed MoE layer, MXFP4 bank", H=4096, I=2048, E=256, k=8, bank="mxfp4",
               shared=False, scoring="softmax", scale=1.0, limit=0.0, chain=True),
    "c4": dict(name="c4: GLM-shaped routed MoE layer, NVFP4 bank", H=6144, I=2048, E=256, k=8, bank="nvfp4",
               shared=True, scoring="sigmoid", scale=1.0, limit=10.0, chain=True),
    # not in the benchmark list: the reference's other EXL3 shape (GLM-Flash experts, src/arch/glm5_next/exl3_forms_ref.zig:17-37)
    "glm": dict(name="glm: GLM-Flash-shaped routed MoE layer, EXL3 K=3 mul1 bank", H=4096, I=2048, E=256, k=8, bank="exl3",
                shared=True, scoring="sigmoid", scale=2.5, limit=10.0, chain=False),
}
WL = WORKLOADS["c2"]


def fp4_quantise_torch(torch, w, nv):
    """Test tooling: N(0, sigma) weights -> packed FP4 parts on the device (codes u32 [rows, cols/8], scale bytes,
    global scale).  MXFP4: OCP shared exponent floor(log2 amax) - 2; NVFP4: g = tensor amax, block scale =
    e4m3(amax_block / (6 g / 2688)).  Nearest e2m1 by magnitude thresholds."""
    rows, cols = w.shape
    bs = 16 if nv else 32
    blk = w.view(rows, cols // bs, bs)
    amax = blk.abs().amax(dim=2, keepdim=True).clamp_min(1e-30)
    if nv:
        g = w.abs().max()
        inv = g / 2688.0
        t = (amax / (6.0 * inv)).clamp(max=448.0)
        sc8 = t.to(torch.float8_e4m3fn)
        scale = sc8.to(torch.float32) * inv
        sbytes = sc8.view(torch.uint8).reshape(rows, cols // bs)
        scale = scale.clamp_min(1e-30)
    else:
        ex = torch.floor(torch.log2(amax)) - 2
        scale = torch.exp2(ex)
        sbytes = (ex + 127).to(torch.uint8).reshape(rows, cols // bs)
        g = None
    v = blk / scale
    th = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=w.device)
    code = torch.bucketize(v.abs(), th).to(torch.int32) | ((v < 0).to(torch.int32) << 3)
    code = code.view(rows, cols // 8, 8).to(torch.int64)
    shifts = torch.arange(0, 32, 4, device=w.device, dtype=torch.int64)
    words = ((code << shifts).sum(dim=2) & 0xFFFFFFFF).to(torch.int32)  # the low 32 bits, as a bit pattern
    return words.contiguous(), sbytes.contiguous(), g


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
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
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


def zipf_bias(layer):
    """ln p_e of a layer's expert popularity: p_e ~ rank^-1.1 over a permutation seeded by the layer, the same on every
    rank and for every batch (popularity is a property of the layer, which is what a usage-based placement relies on)."""
    perm = np.random.default_rng(4242 + layer).permutation(E)
    p = (np.arange(1, E + 1, dtype=np.float64) ** -1.1)
    p /= p.sum()
    return np.log(p)[np.argsort(perm)].astype(np.float32)


def make_logits(rng, T, routing, layer=0):
    lg = rng.standard_normal((T, E)).astype(np.float32)
    if routing == "zipf":
        lg = lg + zipf_bias(layer)
    return lg


LANE_MIN_ROWS = int(os.environ.get("MLXS_PREFILL_MIN_ROWS", "17"))  # the library's default lane threshold


def own_launches_per_layer(T, world):
    """Kernels of this library one layer call launches (library GEMMs and NCCL kernels are not counted)."""
    A = T * K_TOP
    n = 1                                   # router
    n += 3 if A > 2048 else 1               # dispatch: count / scan / place above 2048 rows, one CTA below
    n += 3                                  # streaming lane: prep, gate/up, down
    # the lane's kernels launch when the local call has enough "tokens" for an expert to reach the threshold (with expert
    # parallelism every received assignment is a token of the local call)
    if (T if world == 1 else A) >= LANE_MIN_ROWS:
        n += 4 if WL["bank"] == "exl3" else 6   # plan, prep, gate/up, down (FP4: two tile shapes of each)
    if WL["shared"]:
        n += 2 if T <= 64 else 1            # skinny kernels, or the activation between the library GEMMs
    n += 1                                  # combine
    if world > 1:
        n += 4                              # destination ranks, rank sort, gather, scatter
    return n


def reference_arm(args):
    """The reference's CPU path for this layer, timed on the host cores.  The reference's own CPU lane (Zig tests over
    MLX's CPU device) cannot be built here (no zig, no mlx), so this runs the oracle's fast f32 form (kind "port")."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # all host threads this process may use (a launcher may have set OMP_NUM_THREADS=1 for its ranks)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(threads)
    import oracle_lib as O
    rng = np.random.default_rng(1234)
    srng = np.random.default_rng(7)
    shared = None
    if WL["shared"]:
        shared = [O.f32_to_bf16_bits((srng.standard_normal(s) * 0.02).astype(np.float32))
                  for s in ((I, H), (I, H), (H, I))]
    if WL["bank"] == "exl3":
        T = args.cpu_tokens
        lg = make_logits(rng, T, args.routing)
        ids, w = O.route(lg, None, K_TOP, O.SCORE_SQRTSOFTPLUS, scale=1.5)
        recs = {int(e): O.exl3_synth_record(0xB200 + int(e), H, I, 1.0, 0.02) for e in np.unique(ids)}
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal((T, H)).astype(np.float32)))
        call = lambda: O.layer_fast(H, I, E, K_TOP, recs, x, ids, w, shared=shared, threads=threads)
        form = "oracle fast f32 form"
    else:
        # FP4 banks: the oracle's f64 layer over exactly decoded weights (there is no faster CPU form of it)
        T = min(args.cpu_tokens, 2)
        nv = WL["bank"] == "nvfp4"
        lg = make_logits(rng, T, args.routing)
        ids, w = O.route(lg, None, K_TOP, O.SCORE_SIGMOID if nv else O.SCORE_SOFTMAX, scale=1.0)
        synth = O.nvfp4_synth_record if nv else O.mxfp4_synth_record
        recs = {int(e): synth(0xB200 + int(e), H, I, 0.02) for e in np.unique(ids)}
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal((T, H)).astype(np.float32)))
        bank = O.BANK_NVFP4 if nv else O.BANK_MXFP4
        call = lambda: O.layer(bank, H, I, E, K_TOP, recs, x, ids, w, shared=shared, limit=10.0 if nv else 0.0,
                               chain_rounding=True, shared_bf16_add=True)
        form = "oracle f64 form"
    for _ in range(args.warmup):
        call()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        call()
    dt = time.perf_counter() - t0
    v = T * args.steps / dt
    sample = f"{T} tokens x top-{K_TOP} per step ({len(recs)} distinct experts), whole layer, {form}"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32" if WL["bank"] == "exl3" else "f64", "data": "synthetic",
        "config": workload_config(args, T),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(args, T):
    return {"workload": WL["name"],
            "hidden": H, "inter": I, "n_experts": E, "top_k": K_TOP, "shared_expert": "bf16" if WL["shared"] else "none",
            "tokens_per_call": T,
            "layers": getattr(args, "layers", 1), "routing": args.routing, "l2": "inputs larger than L2 (each call streams >2 GB of distinct expert code)",
            "parallelism": "single GPU" if args.gpus == 1 else f"ep{args.gpus}, experts placed: {getattr(args, 'placement', 'contiguous')}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--cpu-tokens", type=int, default=8)
    ap.add_argument("--routing", default="normal", choices=["normal", "uniform", "zipf"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--experts", type=int, default=0, help="routed experts (smaller only for profiler captures)")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--graph", action="store_true", help="also time the steps replayed from CUDA graphs (one GPU)")
    ap.add_argument("--placement", default="contiguous", choices=["contiguous", "usage"],
                    help="expert parallel: experts in contiguous blocks, or dealt to the ranks by a routing histogram")
    ap.add_argument("--layers", type=int, default=1,
                    help="stack of identical-shape layers run back to back per step (the stack configuration of the benchmark list uses 24)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    globals().update(WL=wl, H=wl["H"], I=wl["I"], E=args.experts or wl["E"], K_TOP=wl["k"])
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    if args.impl == "reference":
        args.steps = min(args.steps, 3)
        return reference_arm(args)

    # NCCL prints its version banner on stdout at NCCL_DEBUG=VERSION/INFO; the contract is one JSON line
    if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "INFO", "TRACE"):
        os.environ["NCCL_DEBUG"] = "WARN"
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

    bank_kind = {"exl3": pkg.BANK_EXL3_K3_MUL1, "mxfp4": pkg.BANK_MXFP4, "nvfp4": pkg.BANK_NVFP4}[WL["bank"]]
    scoring = {"sqrtsoftplus": pkg.SCORE_SQRTSOFTPLUS, "sigmoid": pkg.SCORE_SIGMOID, "softmax": pkg.SCORE_SOFTMAX}[WL["scoring"]]
    NL = args.layers
    cfg = pkg.make_config(H, I, E, K_TOP, n_layers=NL, bank_kind=bank_kind,
                          act=pkg.ACT_SWIGLU_CLAMPED if WL["limit"] > 0 else pkg.ACT_SWIGLU, act_limit=WL["limit"],
                          scoring=scoring, norm_topk=True, routed_scale=WL["scale"], shared_expert=WL["shared"],
                          combine=pkg.COMBINE_CHAIN if WL["chain"] else pkg.COMBINE_F32, max_tokens=max(T, 64),
                          device=local, ep_world=world, ep_rank=rank)
    moe = pkg.MoE(cfg)
    if world > 1:
        # expert parallel: experts sharded E/N per rank; the NCCL id of the library's own communicator travels through
        # torch.distributed
        idt = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            buf = (C.c_char * 128)()
            if pkg.lib().mlxs_moe_ep_unique_id(buf) != 0:
                raise SystemExit("bench.py: " + pkg.last_error())
            idt.copy_(torch.frombuffer(bytearray(bytes(buf)), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        if pkg.lib().mlxs_moe_ep_init(moe._h, bytes(idt.cpu().numpy().tobytes())) != 0:
            raise SystemExit("bench.py: " + pkg.last_error())
    rng = np.random.default_rng(99 + rank)
    n_batches = 4  # rotate a few seeded batches so consecutive steps route differently
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + rank)
    xs, lgs, x_host, lg_host = [], [], [], []
    biases = [torch.from_numpy(zipf_bias(l)).to(dev) for l in range(NL)] if args.routing == "zipf" else None
    for b in range(n_batches):
        noise = rng.standard_normal((T, E)).astype(np.float32)
        x = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
        xs.append(x)
        nd = torch.from_numpy(noise).to(dev)
        # logits of (batch, layer): the batch's noise + the layer's popularity (one tensor for all layers without skew)
        lgs.append([nd + biases[l] for l in range(NL)] if biases else [nd] * NL)
        x_host.append(x.cpu().pin_memory())
        lg_host.append(lgs[b][0].cpu().pin_memory())
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream

    # where the experts live: contiguous blocks, or dealt out by usage: the library's tally counts the routed ids of the
    # batches on the device, sums them over the ranks, and its planner deals the experts out (most used first, snake order)
    rank_of = [np.arange(E) // (E // world) for _ in range(NL)]
    if world > 1 and args.placement == "usage":
        ids_dev = torch.empty((T, K_TOP), dtype=torch.int32, device=dev)
        w_dev = torch.empty((T, K_TOP), dtype=torch.float32, device=dev)
        moe.usage_enable(True)
        for l in range(NL):
            for b in range(n_batches):
                moe.route(l, lgs[b][l].data_ptr(), T, ids_dev.data_ptr(), w_dev.data_ptr(), sp)
            torch.cuda.synchronize()
            ro = np.asarray(pkg.plan_placement(moe.usage_read(l, all_ranks=True), world), np.uint16)
            rank_of[l] = ro.astype(np.int64)
            moe.set_placement(l, np.ascontiguousarray(ro).ctypes.data)
        moe.usage_enable(False)
    owned = [np.nonzero(rank_of[l] == rank)[0] for l in range(NL)]
    n_local = E // world
    logical, stride = moe.record_bytes()
    code_bytes = (H // 16) * (I // 16) * 96
    if WL["bank"] == "exl3":
        # synthetic bank generated on the device in the reference's record layout: random trellis codes, +-(0.5+u) scales
        for j in range(n_local):
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
            for l in range(NL):  # the stack's layers share one synthetic bank image (same bytes, separate residency)
                moe.load_expert(l, int(owned[l][j]), rec.data_ptr(), stride, on_device=True)
    else:
        nv = WL["bank"] == "nvfp4"
        for j in range(n_local):
            parts = []
            for p in range(3):
                rows, cols = (H, I) if p == 2 else (I, H)
                w = torch.randn((rows, cols), device=dev, generator=g) * 0.02
                words, sbytes, gs = fp4_quantise_torch(torch, w, nv)
                parts += [words.view(torch.uint8).reshape(-1), sbytes.reshape(-1)]
                if nv:
                    parts.append(gs.to(torch.float32).reshape(1).view(torch.uint8))
            rec = torch.cat(parts)
            assert rec.numel() == logical, (rec.numel(), logical)
            for l in range(NL):
                moe.load_expert(l, int(owned[l][j]), rec.data_ptr(), rec.numel(), on_device=True)
    sw = None
    if WL["shared"]:
        sw = [(torch.randn(s, device=dev, generator=g) * 0.02).to(torch.bfloat16) for s in ((I, H), (I, H), (H, I))]
        for l in range(NL):
            moe.set_shared(l, sw[0].data_ptr(), sw[1].data_ptr(), sw[2].data_ptr(), on_device=True)

    y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    y2 = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    y_host = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()

    def step(i):
        # a stack feeds each layer's output to the next one (the trunk between MoE layers is out of scope); every
        # layer routes with its own seeded logits
        src, a, b = xs[i % n_batches], y, y2
        for l in range(NL):
            moe.forward(l, src.data_ptr(), lgs[(i + l) % n_batches][l].data_ptr(), T, a.data_ptr(), sp)
            src, a, b = a, b, a

    x_in = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    lg_in = torch.empty((T, E), dtype=torch.float32, device=dev)

    def step_host(i):
        if NL == 1:
            moe.forward_host(0, x_host[i % n_batches].data_ptr(), lg_host[i % n_batches].data_ptr(), T,
                             y_host.data_ptr(), sp)
            return
        # a stack: the step's inputs come from pinned host memory, the last layer's output goes back
        x_in.copy_(x_host[i % n_batches], non_blocking=True)
        lg_in.copy_(lg_host[i % n_batches], non_blocking=True)
        src, a, b = x_in, y, y2
        for l in range(NL):
            moe.forward(l, src.data_ptr(), (lg_in if l == 0 else lgs[(i + l) % n_batches][l]).data_ptr(), T, a.data_ptr(), sp)
            src, a, b = a, b, a
        y_host.copy_(src, non_blocking=True)
        stream.synchronize()

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
    distinct, lane_counts = [], []
    ids_dev = torch.empty((T, K_TOP), dtype=torch.int32, device=dev)
    w_dev = torch.empty((T, K_TOP), dtype=torch.float32, device=dev)
    for b in range(n_batches):
        step(b)
        distinct.append(int(moe.stats().distinct_experts_last))
        # rows per resident expert of layer 0 (which lane each expert takes is decided on these counts)
        moe.route(0, lgs[b][0].data_ptr(), T, ids_dev.data_ptr(), w_dev.data_ptr(), sp)
        torch.cuda.synchronize()
        all_ids = ids_dev
        if world > 1:
            all_ids = torch.empty((world * T, K_TOP), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(all_ids, ids_dev)
        cnt = torch.bincount(all_ids.reshape(-1).long(), minlength=E).cpu().numpy()
        lane_counts.append(cnt[owned[0]])
    sampler = ClockSampler(local)
    sampler.start()
    moe.profile_enable(True)
    moe.profile_read()
    ms = timed(step, args.steps)
    prof = moe.profile_read()
    moe.profile_enable(False)
    clocks = sampler.stop()
    # the same steps replayed from CUDA graphs (one per batch): what a host gains for launch-bound small batches
    graph_ms = None
    if args.graph and world == 1:
        side = torch.cuda.Stream()
        graphs = []
        for b in range(n_batches):
            gph = torch.cuda.CUDAGraph()
            side.wait_stream(stream)
            with torch.cuda.graph(gph, stream=side):
                cs = torch.cuda.current_stream().cuda_stream
                src, a, bb = xs[b], y, y2
                for l in range(NL):
                    moe.forward(l, src.data_ptr(), lgs[(b + l) % n_batches][l].data_ptr(), T, a.data_ptr(), cs)
                    src, a, bb = a, bb, a
            graphs.append(gph)
        for i in range(args.warmup):
            graphs[i % n_batches].replay()
        graph_ms = timed(lambda i: graphs[i % n_batches].replay(), args.steps)
    for i in range(args.warmup):
        step_host(i)
    ms_host = timed(step_host, args.steps)
    st = moe.stats()
    if st.device_status != 0:
        raise SystemExit(f"bench.py: device status {st.device_status}")

    mean_distinct = sum(distinct[i % n_batches] for i in range(args.steps)) / args.steps * 1.0
    if WL["bank"] == "exl3":
        gu_bytes = 2 * code_bytes + 2 * (2 * I + 2 * H)  # one expert's gate + up code and sign/scale vectors
        kname = "exl3_gemv_kernel<2,gate_up>"
        traffic_ratio = 1.014  # dram read+write / algorithmic bytes of the ncu capture on the small case (profiles/)
    else:
        gu_bytes = 2 * (H * I // 2 + H * I // (16 if WL["bank"] == "nvfp4" else 32))  # gate + up codes and block scales
        kname = "fp4_gemv_kernel<2>"
        traffic_ratio = 1.003
    gu_ms, gu_n = prof["gate_up"]
    peak, which = peaks()
    achieved = mean_distinct * gu_bytes / (gu_ms / max(gu_n, 1) * 1e-3) / 1e9
    tl_ms, tl_n = prof.get("tensor_lane", (0.0, 0))
    # the tensor-core lane is the dominant kernel once most of the rows this rank serves belong to its experts (the lanes
    # run on two streams, so their event spans overlap and do not rank them)
    rows_heavy = float(np.mean([int(c[c >= LANE_MIN_ROWS].sum()) for c in lane_counts])) if lane_counts else 0.0
    rows_served = float(np.mean([int(c.sum()) for c in lane_counts])) if lane_counts else 0.0
    prefill_lane = tl_n > 0 and rows_heavy > 0.5 * rows_served
    layer_bytes = NL * (mean_distinct * logical + (3 * H * I * 2 if WL["shared"] else 0) + T * H * 2 * 2 + T * E * 4)
    value = world * T * args.steps / (ms * 1e-3)
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 decoded weights x f16 activations (hi/lo split for EXL3), f32 accumulate", "data": "synthetic",
        "config": workload_config(args, T),
        "layer_hbm": {"algorithmic_bytes_per_call": layer_bytes, "gb_s": layer_bytes / (ms / args.steps * 1e-3) / 1e9,
                      "frac_of_measured_peak": layer_bytes / (ms / args.steps * 1e-3) / 1e9 / peak,
                      "frac_of_nominal_8000": layer_bytes / (ms / args.steps * 1e-3) / 1e9 / 8000.0,
                      "distinct_experts_mean": mean_distinct},
        "roofline": {"kernel": kname, "bound": "hbm", "achieved": achieved, "peak": peak,
                     "peak_source": which, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic_ratio * mean_distinct * gu_bytes,
                     "traffic_note": "ncu dram bytes of a smaller case (64 experts, 16 tokens) scaled by distinct experts",
                     "algorithmic_bytes_per_launch": mean_distinct * gu_bytes},
        "stage_ms_per_step": {k: v[0] / max(args.steps, 1) for k, v in prof.items() if v[1]},
        "e2e": {"value": world * T * args.steps / (ms_host * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": T * H * 2 + T * E * 4, "d2h_bytes_per_step": T * H * 2 + 4},
        "gpu_launches": NL * own_launches_per_layer(T, world) * args.steps,
        "graph_replay": None if graph_ms is None else {"ms_per_step": graph_ms / args.steps,
                                                        "value": T * args.steps / (graph_ms * 1e-3), "unit": UNIT},
        "exchange": None if world == 1 else {
            "exposed_ms_per_step": prof["exchange"][0] / max(args.steps, 1),
            "bytes_sent_per_step_rank0": st.a2a_bytes_sent / max(st.expert_calls, 1),
            "note": "dispatch + combine all-to-all (NCCL send/recv) incl. the count exchange and its host read"},
        "clocks": clocks,
    }
    if prefill_lane:
        # prefill-sized call: the tcgen05 lane (gate/up and down launches are timed together); tensor roofline
        pk = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        tpeak = float(pk.get("bf16_tflops_sustained", 1400.0))
        heavy_rows = float(np.mean([int(c[c >= LANE_MIN_ROWS].sum()) for c in lane_counts]))
        flops = 6.0 * H * I * heavy_rows
        tf = flops / (tl_ms / max(tl_n, 1) * 1e-3) / 1e12
        out["roofline"] = {"kernel": ("exl3_prefill_kernel" if WL["bank"] == "exl3" else "fp4_prefill_kernel") + "<gate/up> + <down> (tcgen05 kind::f16)", "bound": "tensor", "achieved": tf,
                           "peak": tpeak, "peak_source": "measured sustained bf16" if pk else "fallback", "unit": "TFLOP/s",
                           "frac": tf / tpeak, "traffic": None, "flops_per_launch_pair": flops,
                           "rows_in_lane_mean": heavy_rows, "rows_total": T * K_TOP}
    if rank == 0 and world == 1 and not args.no_cpu and WL["bank"] == "exl3":
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
        # the same form on one thread, over the first two tokens of the sample (their experts only)
        T1 = min(2, Tc)
        recs1 = {int(e): recs[int(e)] for e in np.unique(ids[:T1])}
        t0 = time.perf_counter()
        O.layer_fast(H, I, E, K_TOP, recs1, xc[:T1], ids[:T1], w[:T1], shared=shared, threads=1)
        dt1 = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": Tc / dt, "unit": UNIT, "cores": threads, "kind": "port",
                               "sample": f"{Tc} tokens x top-{K_TOP} ({len(recs)} distinct experts), one call, "
                                         "oracle fast f32 form with OpenMP",
                               "one_thread": {"value": T1 / dt1, "unit": UNIT,
                                              "sample": f"{T1} tokens x top-{K_TOP} ({len(recs1)} distinct experts)"}}
    if rank == 0:
        print(json.dumps(out))
    moe.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
