"""Benchmark of the routed-MoE layer (one "step" = one pass of the hot path over one batch of synthetic tokens).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5|glm]
                  [--tokens T] [--routing normal|zipf] [--layers L] [--placement contiguous|usage]

Default workloads (the benchmark list's configurations; every flag above overrides a piece):
  N = 1   "c2": the DeepSeek-V4.1-Flash-shaped decode layer, EXL3 K=3 bank, hidden 5120, inter 2304, 256 routed experts,
          top-8, one bf16 shared expert, 64 tokens per call, N(0,1) logits, one layer.  The same run also measures the
          24-layer Zipf stack of "c5" on the one GPU and reports it under "c5_stack" (skip with --no-stack).
  N > 1   "c5": the expert-parallel stack of 24 such layers, experts sharded 256/N per GPU and placed by usage,
          Zipf(1.1)-skewed routing, 64 tokens per rank per step (tokens data parallel, so the global batch is 64 N:
          "weak" scaling in tokens while the bank is split N ways; per_gpu_hbm_frac and exchange.exposed_ms_per_step say
          what each GPU streams and how long the exchange shows).
Weights are synthetic (seeded random trellis codes, +-(0.5+u) sign/scale vectors; FP4: N(0, 0.02) quantised on the
device), activations bf16 N(0,1).  Prints ONE JSON line (rank 0).

`value` = tokens/s with inputs resident in HBM; `e2e` = the same through host buffers (pinned memory, copies inside the
timed region); `roofline` = the dominant kernel against the measured peak; `cpu_baseline` = the CPU oracle's fast f32
form on a bounded sample of the same workload; `parity_check` = a handful of each rank's tokens of one timed batch
against the CPU oracle, outside the timed region.  `--impl reference` times the CPU oracle alone on the same workload.
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

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
WORKLOADS = {
    "c2": dict(name="c2: DeepSeek-V4.1-Flash-shaped routed MoE decode layer, EXL3 K=3 mul1 bank", H=5120, I=2304, E=256,
               k=8, bank="exl3", shared=True, scoring="sqrtsoftplus", scale=1.5, limit=10.0, chain=False),
    "c3": dict(name="c3: MiMo-shaped routed MoE layer, MXFP4 bank", H=4096, I=2048, E=256, k=8, bank="mxfp4",
               shared=False, scoring="softmax", scale=1.0, limit=0.0, chain=True),
    "c4": dict(name="c4: GLM-shaped routed MoE layer, NVFP4 bank", H=6144, I=2048, E=256, k=8, bank="nvfp4",
               shared=True, scoring="sigmoid", scale=1.0, limit=10.0, chain=True),
    "c5": dict(name="c5: expert-parallel stack of DeepSeek-V4.1-Flash-shaped layers, EXL3 K=3 mul1 bank", H=5120, I=2304,
               E=256, k=8, bank="exl3", shared=True, scoring="sqrtsoftplus", scale=1.5, limit=10.0, chain=False),
    # not in the benchmark list: the reference's other EXL3 shape (GLM-Flash experts, src/arch/glm5_next/exl3_forms_ref.zig:17-37)
    "glm": dict(name="glm: GLM-Flash-shaped routed MoE layer, EXL3 K=3 mul1 bank", H=4096, I=2048, E=256, k=8, bank="exl3",
                shared=True, scoring="sigmoid", scale=2.5, limit=10.0, chain=False),
}
LANE_MIN_ROWS = int(os.environ.get("MLXS_PREFILL_MIN_ROWS", "0"))  # 0: the library's default for the bank (lane_min_rows)


def lane_min_rows(wl):
    """Rows from which an expert of a call takes the tensor-core lane: the library's default is 13 for EXL3 banks, 17 for FP4."""
    return LANE_MIN_ROWS or (13 if wl["bank"] == "exl3" else 17)
N_BATCHES = 4  # a few seeded batches in rotation, so that consecutive steps route differently


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
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 1400.0)), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons; started before the warm-up so that even a timed region of a few
    milliseconds has samples around it, and read back for the window of the timed region."""

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
            self.lines.append((time.perf_counter(), ln.strip()))

    def window(self, t0, t1):
        """Samples that arrived inside [t0, t1] (perf_counter); if the region was shorter than the sampling period, the
        samples nearest to it."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        rows = [(t, ln) for t, ln in list(self.lines)]
        inside = [r for r in rows if t0 - 0.02 <= r[0] <= t1 + 0.04]
        if not inside and rows:
            inside = sorted(rows, key=lambda r: min(abs(r[0] - t0), abs(r[0] - t1)))[:2]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for _, ln in inside:
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

    def stop(self):
        if self.proc:
            self.proc.terminate()


def zipf_bias(E, layer):
    """ln p_e of a layer's expert popularity: p_e ~ rank^-1.1 over a permutation seeded by the layer, the same on every
    rank and for every batch (popularity is a property of the layer, which is what a usage-based placement relies on)."""
    perm = np.random.default_rng(4242 + layer).permutation(E)
    p = (np.arange(1, E + 1, dtype=np.float64) ** -1.1)
    p /= p.sum()
    return np.log(p)[np.argsort(perm)].astype(np.float32)


def workload_config(wl, E, T, layers, routing, gpus, placement):
    return {"workload": wl["name"],
            "hidden": wl["H"], "inter": wl["I"], "n_experts": E, "top_k": wl["k"],
            "shared_expert": "bf16" if wl["shared"] else "none", "tokens_per_call": T,
            "tokens_meaning": "per rank per step (tokens are data parallel)" if gpus > 1 else "per step",
            "layers": layers, "routing": routing,
            "l2": "inputs larger than L2 (each call streams far more distinct expert code than the 126 MB L2 holds)",
            "parallelism": "single GPU" if gpus == 1 else f"ep{gpus}, experts placed: {placement}"}


FRONT_MAX_TOKENS = int(os.environ.get("MLXS_FRONT_MAX", "16"))   # the library's own default and knob


def own_launches_per_layer(wl, T, world):
    """Kernels of this library one layer call launches (NCCL's kernels are not counted)."""
    A = T * wl["k"]
    if world == 1 and T <= FRONT_MAX_TOKENS:
        n = 1 + 2                           # fused front (route, dispatch, row staging in one launch), gate/up, down
    else:
        n = 1                               # router
        n += 3 if A > 2048 else 1           # dispatch: count / scan / place above 2048 rows, one CTA below
        n += 3                              # streaming lane: prep, gate/up, down
    # the tensor-core lane's kernels launch when the local call has enough "tokens" for an expert to reach the threshold
    # (with expert parallelism every received assignment is a token of the local call)
    if (T if world == 1 else A) >= lane_min_rows(wl):
        n += 6                              # tile plan, row prep, gate/up and down in two tile shapes each
    if wl["shared"]:
        n += 2 if T <= 64 else 3            # skinny gate/up + down, or row staging + the two tcgen05 products
    if world > 1:
        # the exchange: its plan (destination ranks, rank sort, dedup: one launch up to 2048 assignments, three above),
        # push, unpack, partial push, final sum
        n += 5 if A <= 2048 else 7
    else:
        n += 1                              # combine (expert parallel: the partial push and the final sum do its work)
    return n


# ----------------------------------------------------------------------------------------------------------------
# the reference arm: the CPU oracle alone
# ----------------------------------------------------------------------------------------------------------------
def reference_arm(args, wl, E):
    """The reference's CPU path for this workload, timed on the host cores.  The reference's own CPU lane (Zig tests
    over MLX's CPU device) cannot be built here (no zig, no mlx), so this runs the oracle's fast f32 form (kind "port")
    on the same shapes, token count and routing as the GPU arm.  A stack is sampled: as many of its layers per step as
    fit the time budget, scaled to the whole stack."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(threads)   # a launcher may have set 1 for its ranks
    import oracle_lib as O
    H, I, K = wl["H"], wl["I"], wl["k"]
    # the whole job's batch: with N ranks the GPU arm runs `tokens` per rank per step, N x tokens in all
    T, NL = args.tokens * max(args.gpus, 1), args.layers
    rng = np.random.default_rng(1234)
    srng = np.random.default_rng(7)
    shared = None
    if wl["shared"]:
        shared = [O.f32_to_bf16_bits((srng.standard_normal(s) * 0.02).astype(np.float32)) for s in ((I, H), (I, H), (H, I))]
    exl3 = wl["bank"] == "exl3"
    if not exl3:
        T = min(T, 2)   # FP4 banks: only the f64 oracle exists on the CPU; a two-token sample of the call
    score = {"sqrtsoftplus": O.SCORE_SQRTSOFTPLUS, "sigmoid": O.SCORE_SIGMOID, "softmax": O.SCORE_SOFTMAX}[wl["scoring"]]
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal((T, H)).astype(np.float32)))
    noise = rng.standard_normal((T, E)).astype(np.float32)
    recs_cache = {}

    def layer_inputs(l):
        lg = noise + zipf_bias(E, l) if args.routing == "zipf" else noise
        ids, w = O.route(lg, None, K, score, scale=wl["scale"])
        for e in np.unique(ids):
            e = int(e)
            if e not in recs_cache:
                recs_cache[e] = (O.exl3_synth_record(0xB200 + e, H, I, 1.0, 0.02) if exl3 else
                                 (O.nvfp4_synth_record if wl["bank"] == "nvfp4" else O.mxfp4_synth_record)(0xB200 + e, H, I, 0.02))
        return ids, w

    def run_layer(l, ids, w):
        recs = {int(e): recs_cache[int(e)] for e in np.unique(ids)}
        if exl3:
            return O.layer_fast(H, I, E, K, recs, x, ids, w, shared=shared, limit=wl["limit"], threads=threads)
        bank = O.BANK_NVFP4 if wl["bank"] == "nvfp4" else O.BANK_MXFP4
        return O.layer(bank, H, I, E, K, recs, x, ids, w, shared=shared, limit=wl["limit"], chain_rounding=True,
                       shared_bf16_add=True)

    # size the sample: one layer call first, then as many layers per step as the budget allows
    first = layer_inputs(0)
    t0 = time.perf_counter()
    run_layer(0, *first)
    t_layer = time.perf_counter() - t0
    budget_s = float(os.environ.get("MLXS_REF_BUDGET_S", "200"))
    calls = args.steps + args.warmup
    ls = int(max(1, min(NL, budget_s / max(t_layer * calls, 1e-9))))
    plan = [layer_inputs(l) for l in range(ls)]
    distinct = float(np.mean([len(np.unique(p[0])) for p in plan]))
    for _ in range(args.warmup):
        for l in range(ls):
            run_layer(l, *plan[l])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for l in range(ls):
            run_layer(l, *plan[l])
    dt = time.perf_counter() - t0
    ms_step = 1e3 * dt / args.steps * (NL / ls)      # the sampled layers scaled to the stack
    v = T / (ms_step * 1e-3)
    sample = (f"{T} tokens (the global batch of {max(args.gpus, 1)} rank(s)) x top-{K} per layer call ({distinct:.0f} distinct experts per call), {ls} of {NL} layer(s) timed per "
              f"step and scaled to {NL}, whole layer incl. shared expert, oracle {'fast f32' if exl3 else 'f64'} form, OpenMP")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32" if exl3 else "f64", "data": "synthetic",
        "config": workload_config(wl, E, args.tokens, NL, args.routing, args.gpus, args.placement),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------------------------------------------
# the GPU arm
# ----------------------------------------------------------------------------------------------------------------
class Rig:
    """One handle with its synthetic bank, batches and step functions."""

    def __init__(self, env, wl, E, T, NL, routing, placement):
        torch, pkg, dev = env["torch"], env["pkg"], env["dev"]
        self.env, self.wl, self.E, self.T, self.NL, self.routing = env, wl, E, T, NL, routing
        world, rank = env["world"], env["rank"]
        H, I, K = wl["H"], wl["I"], wl["k"]
        bank_kind = {"exl3": pkg.BANK_EXL3_K3_MUL1, "mxfp4": pkg.BANK_MXFP4, "nvfp4": pkg.BANK_NVFP4}[wl["bank"]]
        scoring = {"sqrtsoftplus": pkg.SCORE_SQRTSOFTPLUS, "sigmoid": pkg.SCORE_SIGMOID, "softmax": pkg.SCORE_SOFTMAX}[wl["scoring"]]
        cfg = pkg.make_config(H, I, E, K, n_layers=NL, bank_kind=bank_kind,
                              act=pkg.ACT_SWIGLU_CLAMPED if wl["limit"] > 0 else pkg.ACT_SWIGLU, act_limit=wl["limit"],
                              scoring=scoring, norm_topk=True, routed_scale=wl["scale"], shared_expert=wl["shared"],
                              combine=pkg.COMBINE_CHAIN if wl["chain"] else pkg.COMBINE_F32, max_tokens=max(T, 64),
                              device=env["local"], ep_world=world, ep_rank=rank)
        self.moe = moe = pkg.MoE(cfg)
        dist = env["dist"]
        if world > 1:
            # the NCCL id of the library's own communicator travels through torch.distributed
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
        g = torch.Generator(device=dev)
        g.manual_seed(1000 + rank)
        self.xs, self.lgs, self.x_host, self.lg_host = [], [], [], []
        biases = [torch.from_numpy(zipf_bias(E, l)).to(dev) for l in range(NL)] if routing == "zipf" else None
        for b in range(N_BATCHES):
            noise = rng.standard_normal((T, E)).astype(np.float32)
            x = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
            self.xs.append(x)
            nd = torch.from_numpy(noise).to(dev)
            # logits of (batch, layer): the batch's noise + the layer's popularity (one tensor for all layers without skew)
            self.lgs.append([nd + biases[l] for l in range(NL)] if biases else [nd] * NL)
            self.x_host.append(x.cpu().pin_memory())
            self.lg_host.append(self.lgs[b][0].cpu().pin_memory())
        self.stream = torch.cuda.current_stream()
        self.sp = self.stream.cuda_stream

        # where the experts live: contiguous blocks, or dealt out by usage: the library's tally counts the routed ids of
        # the batches on the device, sums them over the ranks, and its planner deals the experts out
        rank_of = [np.arange(E) // (E // world) for _ in range(NL)]
        if world > 1 and placement == "usage":
            ids_dev = torch.empty((T, K), dtype=torch.int32, device=dev)
            w_dev = torch.empty((T, K), dtype=torch.float32, device=dev)
            moe.usage_enable(True)
            for l in range(NL):
                for b in range(N_BATCHES):
                    moe.route(l, self.lgs[b][l].data_ptr(), T, ids_dev.data_ptr(), w_dev.data_ptr(), self.sp)
                torch.cuda.synchronize()
                ro = np.asarray(pkg.plan_placement(moe.usage_read(l, all_ranks=True), world), np.uint16)
                rank_of[l] = ro.astype(np.int64)
                moe.set_placement(l, np.ascontiguousarray(ro).ctypes.data)
            moe.usage_enable(False)
        self.owned = [np.nonzero(rank_of[l] == rank)[0] for l in range(NL)]
        self.logical, self.stride = moe.record_bytes()
        self._rec_cache = {}
        for l in range(NL):
            for e in self.owned[l]:
                rec = self.expert_record(int(e))
                moe.load_expert(l, int(e), rec.data_ptr(), rec.numel(), on_device=True)
        self._rec_cache.clear()
        self.sw = None
        if wl["shared"]:
            self.sw = [(torch.randn(s, device=dev, generator=g) * 0.02).to(torch.bfloat16) for s in ((I, H), (I, H), (H, I))]
            for l in range(NL):
                moe.set_shared(l, self.sw[0].data_ptr(), self.sw[1].data_ptr(), self.sw[2].data_ptr(), on_device=True)
        self.y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        self.y2 = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        self.y_host = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
        self.x_in = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        self.lg_in = torch.empty((T, E), dtype=torch.float32, device=dev)

    def expert_record(self, e):
        """The synthetic record of expert e in the reference's layout, a function of e alone (every rank and the parity
        check can regenerate it; the layers of a stack hold the same image)."""
        if e in self._rec_cache:
            return self._rec_cache[e]
        torch, dev, wl = self.env["torch"], self.env["dev"], self.wl
        H, I = wl["H"], wl["I"]
        g = torch.Generator(device=dev)
        g.manual_seed(0xB2000 + e)
        if wl["bank"] == "exl3":
            code_bytes = (H // 16) * (I // 16) * 96
            rec = torch.randint(0, 256, (self.stride,), dtype=torch.uint8, device=dev, generator=g)
            off = 0
            for p in range(3):
                off += code_bytes
                n_out, n_in = (H, I) if p == 2 else (I, H)
                for n, sc in ((n_out, 0.02), (n_in, 1.0)):
                    u = torch.rand(n, device=dev, generator=g)
                    sgn = torch.where(torch.rand(n, device=dev, generator=g) < 0.5, -1.0, 1.0)
                    rec[off:off + 2 * n] = ((0.5 + u) * sgn * sc).to(torch.float16).view(torch.uint8)
                    off += 2 * n
        else:
            nv = wl["bank"] == "nvfp4"
            parts = []
            for p in range(3):
                rows, cols = (H, I) if p == 2 else (I, H)
                w = torch.randn((rows, cols), device=dev, generator=g) * 0.02
                words, sbytes, gs = fp4_quantise_torch(torch, w, nv)
                parts += [words.view(torch.uint8).reshape(-1), sbytes.reshape(-1)]
                if nv:
                    parts.append(gs.to(torch.float32).reshape(1).view(torch.uint8))
            rec = torch.cat(parts)
            assert rec.numel() == self.logical, (rec.numel(), self.logical)
        if len(self._rec_cache) < 300:
            self._rec_cache[e] = rec
        return rec

    def step(self, i):
        # a stack feeds each layer's output to the next one (the trunk between MoE layers is out of scope); every
        # layer routes with its own seeded logits
        src, a, b = self.xs[i % N_BATCHES], self.y, self.y2
        for l in range(self.NL):
            self.moe.forward(l, src.data_ptr(), self.lgs[(i + l) % N_BATCHES][l].data_ptr(), self.T, a.data_ptr(), self.sp)
            src, a, b = a, b, a

    def step_host(self, i):
        if self.NL == 1:
            self.moe.forward_host(0, self.x_host[i % N_BATCHES].data_ptr(), self.lg_host[i % N_BATCHES].data_ptr(), self.T,
                                  self.y_host.data_ptr(), self.sp)
            return
        # a stack: the step's inputs come from pinned host memory, the last layer's output goes back
        self.x_in.copy_(self.x_host[i % N_BATCHES], non_blocking=True)
        self.lg_in.copy_(self.lg_host[i % N_BATCHES], non_blocking=True)
        src, a, b = self.x_in, self.y, self.y2
        for l in range(self.NL):
            lg = self.lg_in if l == 0 else self.lgs[(i + l) % N_BATCHES][l]
            self.moe.forward(l, src.data_ptr(), lg.data_ptr(), self.T, a.data_ptr(), self.sp)
            src, a, b = a, b, a
        self.y_host.copy_(src, non_blocking=True)
        self.stream.synchronize()

    def barrier(self):
        if self.env["world"] > 1:
            self.env["dist"].barrier()
        self.env["torch"].cuda.synchronize()

    def timed(self, fn, steps):
        torch = self.env["torch"]
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(self.stream)
        for i in range(steps):
            fn(i)
        e1.record(self.stream)
        self.barrier()
        t1 = time.perf_counter()
        ms = e0.elapsed_time(e1)
        if self.env["world"] > 1:
            t = torch.tensor([ms], device=self.env["dev"])
            self.env["dist"].all_reduce(t, op=self.env["dist"].ReduceOp.MAX)
            ms = float(t.item())
        return ms, (t0, t1)

    def row_counts(self):
        """rows per expert this rank serves, per (batch, layer): from the routed ids of every rank's tokens"""
        torch, dev, dist = self.env["torch"], self.env["dev"], self.env["dist"]
        world, K, E, T = self.env["world"], self.wl["k"], self.E, self.T
        ids_dev = torch.empty((T, K), dtype=torch.int32, device=dev)
        w_dev = torch.empty((T, K), dtype=torch.float32, device=dev)
        out = []
        for b in range(N_BATCHES):
            per_layer = []
            for l in range(self.NL):
                self.moe.route(l, self.lgs[b][l].data_ptr(), T, ids_dev.data_ptr(), w_dev.data_ptr(), self.sp)
                all_ids = ids_dev
                if world > 1:
                    all_ids = torch.empty((world * T, K), dtype=torch.int32, device=dev)
                    dist.all_gather_into_tensor(all_ids, ids_dev)
                cnt = torch.bincount(all_ids.reshape(-1).long(), minlength=E).cpu().numpy()
                per_layer.append(cnt[self.owned[l]])
            out.append(per_layer)
        return out

    def parity_check(self, n_tok=4):
        """A few of this rank's tokens of batch 0 through layer 0 (the whole batch runs, every rank takes part in the
        exchange) against the CPU oracle over the touched experts.  Outside the timed region."""
        import oracle_lib as O
        torch, dev, wl = self.env["torch"], self.env["dev"], self.wl
        H, I, K, E, T = wl["H"], wl["I"], wl["k"], self.E, self.T
        n_tok = min(n_tok, T)
        ids_dev = torch.empty((T, K), dtype=torch.int32, device=dev)
        w_dev = torch.empty((T, K), dtype=torch.float32, device=dev)
        self.moe.route(0, self.lgs[0][0].data_ptr(), T, ids_dev.data_ptr(), w_dev.data_ptr(), self.sp)
        self.moe.forward(0, self.xs[0].data_ptr(), self.lgs[0][0].data_ptr(), T, self.y.data_ptr(), self.sp)
        torch.cuda.synchronize()
        ids = ids_dev[:n_tok].cpu().numpy()
        w = w_dev[:n_tok].cpu().numpy()
        got = self.y[:n_tok].float().cpu().numpy()
        x = self.xs[0][:n_tok].float().cpu().numpy()
        self._rec_cache.clear()
        recs = {}
        for e in np.unique(ids):
            r = self.expert_record(int(e)).cpu().numpy()
            self._rec_cache.clear()
            recs[int(e)] = r
        shared = [s.view(torch.int16).cpu().numpy().view(np.uint16) for s in self.sw] if self.sw else None
        if wl["bank"] == "exl3":
            ref = O.layer_fast(H, I, E, K, recs, x, ids, w, shared=shared, limit=wl["limit"], threads=0)
        else:
            bank = O.BANK_NVFP4 if wl["bank"] == "nvfp4" else O.BANK_MXFP4
            ref = O.layer(bank, H, I, E, K, recs, x, ids, w, shared=shared, limit=wl["limit"], chain_rounding=wl["chain"],
                          shared_bf16_add=wl["chain"])
        ref = np.asarray(ref, np.float64)
        rel = float(np.linalg.norm(got - ref) / (np.linalg.norm(ref) + 1e-30))
        world = self.env["world"]
        if world > 1:
            t = torch.tensor([rel], device=dev, dtype=torch.float64)
            self.env["dist"].all_reduce(t, op=self.env["dist"].ReduceOp.MAX)
            rel = float(t.item())
        return {"rel_l2": rel, "tokens": n_tok * world, "ranks": world, "bar": 1e-2,
                "against": "CPU oracle (fast f32 form) over the touched experts; layer 0, batch 0; max over ranks"}

    def close(self):
        self.moe.close()


def measure(rig, args, sampler, want_e2e=True):
    """Warm-up, the timed steps with per-stage spans, the host-buffer form; returns the pieces of the JSON line."""
    env, wl = rig.env, rig.wl
    torch = env["torch"]
    world = env["world"]
    H, I, K, E, T, NL = wl["H"], wl["I"], wl["k"], rig.E, rig.T, rig.NL
    for i in range(args.warmup):
        rig.step(i)
    counts = rig.row_counts()                      # [batch][layer] -> rows per resident expert
    moe = rig.moe
    moe.profile_enable(True)
    moe.profile_read()
    ms, window = rig.timed(rig.step, args.steps)
    prof = moe.profile_read()
    moe.profile_enable(False)
    clocks = sampler.window(*window) if sampler else None
    graph_ms = None
    if args.graph and world == 1:
        side = torch.cuda.Stream()
        graphs = []
        for b in range(N_BATCHES):
            gph = torch.cuda.CUDAGraph()
            side.wait_stream(rig.stream)
            with torch.cuda.graph(gph, stream=side):
                cs = torch.cuda.current_stream().cuda_stream
                src, a, bb = rig.xs[b], rig.y, rig.y2
                for l in range(NL):
                    moe.forward(l, src.data_ptr(), rig.lgs[(b + l) % N_BATCHES][l].data_ptr(), T, a.data_ptr(), cs)
                    src, a, bb = a, bb, a
            graphs.append(gph)
        for i in range(args.warmup):
            graphs[i % N_BATCHES].replay()
        graph_ms, _ = rig.timed(lambda i: graphs[i % N_BATCHES].replay(), args.steps)
    from_x_ms = None
    if world == 1 and NL == 1 and not args.no_from_x:
        # the layer from x: the router's logits product x . W_g^T inside the call (mlxs_moe_forward_x); W_g ~ N(0, 1/H)
        # so that the logits of N(0,1) rows are N(0,1) like the given ones
        gen = torch.Generator(device=env["dev"]).manual_seed(4321)
        wg = (torch.randn(E, H, generator=gen, device=env["dev"], dtype=torch.float32) * (H ** -0.5)).to(torch.bfloat16).contiguous()
        moe.set_router_weight(0, wg.data_ptr(), on_device=True)
        fx = lambda i: moe.forward_x(0, rig.xs[i % N_BATCHES].data_ptr(), T, rig.y.data_ptr(), rig.sp)
        for i in range(args.warmup):
            fx(i)
        from_x_ms, _ = rig.timed(fx, args.steps)
    ms_host = None
    if want_e2e:
        for i in range(args.warmup):
            rig.step_host(i)
        ms_host, _ = rig.timed(rig.step_host, args.steps)
    st = moe.stats()
    if st.device_status != 0:
        raise SystemExit(f"bench.py: device status {st.device_status}")

    # which (batch, layer) each timed layer call ran: step i, layer l uses batch (i + l) % N_BATCHES
    def mean_over_calls(fn):
        tot = 0.0
        for i in range(args.steps):
            for l in range(NL):
                tot += fn(counts[(i + l) % N_BATCHES][l])
        return tot / args.steps     # per step (summed over the stack's layers)

    distinct_step = mean_over_calls(lambda c: float((c > 0).sum()))
    lmr = lane_min_rows(wl)
    light_step = mean_over_calls(lambda c: float(((c > 0) & (c < lmr)).sum()) if T >= lmr or world > 1 else float((c > 0).sum()))
    rows_heavy = mean_over_calls(lambda c: float(c[c >= lmr].sum()))
    rows_served = mean_over_calls(lambda c: float(c.sum()))
    if wl["bank"] == "exl3":
        code_bytes = (H // 16) * (I // 16) * 96
        gu_bytes = 2 * code_bytes + 2 * (2 * I + 2 * H)  # one expert's gate + up code and sign/scale vectors
        kname = "exl3_gemv_kernel<2,gate_up>"
        traffic_ratio = 1.016  # dram read+write / algorithmic bytes of the ncu capture on the small case (profiles/)
    else:
        gu_bytes = 2 * (H * I // 2 + H * I // (16 if wl["bank"] == "nvfp4" else 32))  # gate + up codes and block scales
        kname = "fp4_gemv_kernel<2>"
        traffic_ratio = 1.015
    hbm_peak, tpeak, which = peaks()
    gu_ms, gu_n = prof["gate_up"]
    per_launch_s = gu_ms / max(gu_n, 1) * 1e-3
    streamed_per_launch = light_step / NL      # experts the streaming lane serves per layer call (the others take the tensor lane)
    achieved = streamed_per_launch * gu_bytes / max(per_launch_s, 1e-12) / 1e9
    tl_ms, tl_n = prof.get("tensor_lane", (0.0, 0))
    prefill_lane = tl_n > 0 and rows_heavy > 0.5 * rows_served
    shared_bytes = 3 * H * I * 2 if wl["shared"] else 0
    step_bytes = distinct_step * rig.logical + NL * (shared_bytes + T * H * 2 * 2 + T * E * 4)
    step_s = ms / args.steps * 1e-3
    if world > 1:
        t = torch.tensor([step_bytes], device=env["dev"], dtype=torch.float64)
        env["dist"].all_reduce(t)
        step_bytes_mean = float(t.item()) / world
    else:
        step_bytes_mean = step_bytes
    out = {
        "value": world * T * args.steps / (ms * 1e-3), "ms_per_step": ms / args.steps,
        "layer_hbm": {"algorithmic_bytes_per_step_per_gpu": step_bytes_mean, "gb_s_per_gpu": step_bytes_mean / step_s / 1e9,
                      "frac_of_measured_peak": step_bytes_mean / step_s / 1e9 / hbm_peak,
                      "frac_of_nominal_8000": step_bytes_mean / step_s / 1e9 / 8000.0,
                      "distinct_experts_per_layer_call_rank0": distinct_step / NL},
        "per_gpu_hbm_frac": step_bytes_mean / step_s / 1e9 / hbm_peak,
        "roofline": {"kernel": kname, "bound": "hbm", "achieved": achieved, "peak": hbm_peak,
                     "peak_source": which, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": traffic_ratio * streamed_per_launch * gu_bytes,
                     "traffic_note": "ncu dram bytes of a smaller case (64 experts, 16 tokens) scaled by the experts streamed",
                     "algorithmic_bytes_per_launch": streamed_per_launch * gu_bytes,
                     "experts_streamed_per_launch": streamed_per_launch, "launch_ms": per_launch_s * 1e3},
        "stage_ms_per_step": {k: v[0] / max(args.steps, 1) for k, v in prof.items()
                              if v[1] and not (k == "tensor_lane" and rows_heavy == 0)},
        "gpu_launches": NL * own_launches_per_layer(wl, T, world) * args.steps,
        "from_x": None if from_x_ms is None else {"ms_per_step": from_x_ms / args.steps, "value": T * args.steps / (from_x_ms * 1e-3),
                                                   "unit": UNIT, "note": "the same layer call with the router's logits product inside it (mlxs_moe_forward_x)"},
        "graph_replay": None if graph_ms is None else {"ms_per_step": graph_ms / args.steps,
                                                        "value": T * args.steps / (graph_ms * 1e-3), "unit": UNIT},
        "exchange": None if world == 1 else {
            "exposed_ms_per_step": prof["exchange"][0] / max(args.steps, 1),
            "frac_of_step": prof["exchange"][0] / max(args.steps, 1) / (ms / args.steps),
            "bytes_sent_per_layer_call_rank0": st.a2a_bytes_sent / max(st.expert_calls, 1),
            "note": "CUDA-event span of the dispatch and combine exchanges on rank 0; with skewed routing it contains the wait for the busiest rank"},
        "clocks": clocks,
    }
    if ms_host is not None:
        out["e2e"] = {"value": world * T * args.steps / (ms_host * 1e-3), "unit": UNIT,
                      "h2d_bytes_per_step": T * H * 2 + T * E * 4, "d2h_bytes_per_step": T * H * 2 + 4}
    if prefill_lane:
        # prefill-sized call: the tcgen05 lane (gate/up and down launches are timed together); tensor roofline
        flops = 6.0 * H * I * rows_heavy / NL
        tf = flops / (tl_ms / max(tl_n, 1) * 1e-3) / 1e12
        native = wl["bank"] == "mxfp4" and os.environ.get("MLXS_MXFP4_NATIVE", "1") != "0"
        kname = "exl3_prefill_kernel" if wl["bank"] == "exl3" else ("mxfp4_native_kernel" if native else "fp4_prefill_kernel")
        out["roofline"] = {"kernel": kname + "<gate/up> + <down> (tcgen05" + (", kind::mxf8f6f4.block_scale" if native else ", kind::f16") + ")",
                           "bound": "tensor", "achieved": tf, "peak": tpeak,
                           "peak_source": "measured sustained bf16" if which == "measured" else "fallback", "unit": "TFLOP/s",
                           "frac": tf / tpeak, "traffic": None, "flops_per_launch_pair": flops,
                           "rows_in_lane_per_layer_call": rows_heavy / NL, "rows_served_per_layer_call": rows_served / NL}
        if native:
            # the block-scaled kind's own ceilings: its issue rate measured on this part (mlxs_moe_fp4_native_probe), of
            # which a pair of MMAs (E4M3 high + low part of a bf16 row) uses half, and the nominal dense FP4 figure
            out["roofline"]["other_peaks"] = {
                "mxf8f6f4_issue_rate_measured_tflops": 4371.0, "frac_of_it_with_two_mmas_per_block": 2.0 * tf / 4371.0,
                "nominal_dense_fp4_tflops": 9000.0, "frac_of_nominal_dense_fp4": tf / 9000.0}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--cpu-tokens", type=int, default=8, help="tokens of the cpu_baseline sample inside the GPU arm")
    ap.add_argument("--routing", default=None, choices=["normal", "uniform", "zipf"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-stack", action="store_true", help="N = 1: skip the 24-layer stack measured beside the layer")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of a few tokens")
    ap.add_argument("--no-from-x", action="store_true", help="N = 1, one layer: skip the measurement of the layer from x (router logits inside)")
    ap.add_argument("--experts", type=int, default=0, help="routed experts (smaller only for profiler captures)")
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--ceiling", action="store_true", help="also measure the EXL3 decode's own ceiling (operands from registers)")
    ap.add_argument("--graph", action="store_true", help="also time the steps replayed from CUDA graphs (one GPU)")
    ap.add_argument("--placement", default=None, choices=["contiguous", "usage"],
                    help="expert parallel: experts in contiguous blocks, or dealt to the ranks by a routing histogram")
    ap.add_argument("--layers", type=int, default=0,
                    help="stack of identical-shape layers run back to back per step (the stack configuration uses 24)")
    args = ap.parse_args()
    default_workload = args.workload is None
    if args.workload is None:
        args.workload = "c2" if args.gpus == 1 else "c5"
    stack = args.workload == "c5"
    if args.routing is None:
        args.routing = "zipf" if stack else "normal"
    if args.layers == 0:
        args.layers = 24 if stack else 1
    if args.placement is None:
        args.placement = "usage" if (stack and args.gpus > 1) else "contiguous"
    wl = WORKLOADS[args.workload]
    E = args.experts or wl["E"]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    if args.impl == "reference":
        return reference_arm(args, wl, E)

    # NCCL writes its INFO lines to stdout by default; the contract is one JSON line there, so they go to stderr
    if os.environ.get("NCCL_DEBUG") and not os.environ.get("NCCL_DEBUG_FILE"):
        os.environ["NCCL_DEBUG_FILE"] = "/dev/stderr"
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
    env = dict(torch=torch, dist=dist, pkg=pkg, dev=dev, rank=rank, world=world, local=local)
    sampler = ClockSampler(local)
    sampler.start()
    T, NL = args.tokens, args.layers
    rig = Rig(env, wl, E, T, NL, args.routing, args.placement)
    m = measure(rig, args, sampler)
    out = {
        "metric": METRIC, "value": m.pop("value"), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": m.pop("ms_per_step"), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 decoded weights x f16 activations (hi/lo split for EXL3), f32 accumulate", "data": "synthetic",
        "config": workload_config(wl, E, T, NL, args.routing, world, args.placement),
    }
    out.update(m)
    if not args.no_parity:
        out["parity_check"] = rig.parity_check()
    if rank == 0 and world == 1 and not args.no_cpu and wl["bank"] == "exl3":
        import oracle_lib as O
        H, I, K = wl["H"], wl["I"], wl["k"]
        Tc = args.cpu_tokens
        crng = np.random.default_rng(1234)
        lg = crng.standard_normal((Tc, E)).astype(np.float32)
        if args.routing == "zipf":
            lg = lg + zipf_bias(E, 0)
        score = {"sqrtsoftplus": O.SCORE_SQRTSOFTPLUS, "sigmoid": O.SCORE_SIGMOID, "softmax": O.SCORE_SOFTMAX}[wl["scoring"]]
        ids, w = O.route(lg, None, K, score, scale=wl["scale"])
        recs = {int(e): O.exl3_synth_record(0xB200 + int(e), H, I, 1.0, 0.02) for e in np.unique(ids)}
        shared = [s.view(torch.int16).cpu().numpy().view(np.uint16) for s in rig.sw] if rig.sw else None
        xc = O.bf16_bits_to_f32(O.f32_to_bf16_bits(crng.standard_normal((Tc, H)).astype(np.float32)))
        threads = O.max_threads()
        t0 = time.perf_counter()
        O.layer_fast(H, I, E, K, recs, xc, ids, w, shared=shared, threads=threads)
        dt = time.perf_counter() - t0
        # the same form on one thread, over the first two tokens of the sample (their experts only)
        T1 = min(2, Tc)
        recs1 = {int(e): recs[int(e)] for e in np.unique(ids[:T1])}
        t0 = time.perf_counter()
        O.layer_fast(H, I, E, K, recs1, xc[:T1], ids[:T1], w[:T1], shared=shared, threads=1)
        dt1 = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": Tc / dt, "unit": UNIT, "cores": threads, "kind": "port",
                               "sample": f"{Tc} tokens x top-{K} ({len(recs)} distinct experts), one layer call, "
                                         "oracle fast f32 form with OpenMP (the whole workload at its own token count: --impl reference)",
                               "one_thread": {"value": T1 / dt1, "unit": UNIT,
                                              "sample": f"{T1} tokens x top-{K} ({len(recs1)} distinct experts)"}}
    if args.ceiling and rank == 0 and wl["bank"] == "exl3":
        hbm_peak = peaks()[0]
        ceil = {}
        for bits in (3, 2):
            for mma in (0, 1):
                tps = pkg.exl3_decode_rate(local, bits, bool(mma), 1 << 15)
                gbs = tps * 32 * bits / 1e9
                ceil[f"k{bits}_{'decode_mma' if mma else 'decode_only'}"] = {"tiles_per_s": tps, "code_gb_s": gbs,
                                                                             "frac_of_measured_hbm": gbs / hbm_peak}
        out["decode_ceiling"] = ceil
    rig.close()
    del rig
    # N = 1, default workload: the 24-layer Zipf stack of the expert-parallel configuration on the one GPU, so that the
    # stack's N = 1 point exists beside the N > 1 lines
    if world == 1 and default_workload and not args.no_stack and not args.experts:
        torch.cuda.empty_cache()
        swl = WORKLOADS["c5"]
        sargs = argparse.Namespace(**vars(args))
        sargs.graph = False
        sargs.steps = max(3, min(args.steps, 10))
        srig = Rig(env, swl, swl["E"], T, 24, "zipf", "contiguous")
        sm = measure(srig, sargs, sampler, want_e2e=False)
        out["c5_stack"] = {"config": workload_config(swl, swl["E"], T, 24, "zipf", 1, "contiguous"), "steps": sargs.steps,
                           "value": sm["value"], "unit": UNIT, "ms_per_step": sm["ms_per_step"],
                           "per_gpu_hbm_frac": sm["per_gpu_hbm_frac"], "stage_ms_per_step": sm["stage_ms_per_step"],
                           "roofline": sm["roofline"]}
        if not args.no_parity:
            out["c5_stack"]["parity_check"] = srig.parity_check()
        srig.close()
    sampler.stop()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
