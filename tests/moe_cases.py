"""Shared fixtures of the GPU parity tests: seeded synthetic banks in the reference's record layouts, the same inputs
given to the CUDA library (through the C ABI) and to the CPU oracle.

Synthetic stand-ins (the reference ships no quantiser and no checkpoints): EXL3 codes are the splitmix64 stream the
reference's golden generator uses (src/arch/glm5_next/exl3_forms_ref.zig:45-66), suh = f16(+-(0.5+u)), svh =
f16(+-(0.5+u) 0.02) so the effective dense weight has element std ~0.02; activations bf16(N(0,1)); logits N(0,1).
"""
import ctypes as C

# rows from which an expert of a call takes the tensor-core lane (the library's defaults; MLXS_PREFILL_MIN_ROWS moves both)
import os as _os
LANE_MIN_EXL3 = int(_os.environ.get("MLXS_PREFILL_MIN_ROWS", "13"))
LANE_MIN_FP4 = int(_os.environ.get("MLXS_PREFILL_MIN_ROWS", "17"))


import numpy as np

import oracle_lib as O
from __graft_entry__ import load_package


def torch_mod():
    import torch
    return torch


class Exl3Case:
    """A routed-MoE layer over one bank kind (EXL3 by default), on the GPU and in the oracle."""

    bank = O.BANK_EXL3

    def __init__(self, hidden, inter, n_experts, top_k, seed=0, shared=True, scoring=None, max_tokens=64,
                 experts_to_load=None, routed_scale=1.5, limit=10.0, device=0, chain=False):
        self.pkg = load_package()
        pkg = self.pkg
        torch = torch_mod()
        self.H, self.I, self.E, self.k = hidden, inter, n_experts, top_k
        self.limit = limit
        self.chain = chain
        self.scoring = pkg.SCORE_SQRTSOFTPLUS if scoring is None else scoring
        self.routed_scale = routed_scale
        self.dev = torch.device("cuda", device)
        cfg = pkg.make_config(hidden, inter, n_experts, top_k, n_layers=1, bank_kind=self.bank,
                              act=pkg.ACT_SWIGLU_CLAMPED if limit > 0 else pkg.ACT_SWIGLU, act_limit=limit,
                              scoring=self.scoring, norm_topk=True, routed_scale=routed_scale, shared_expert=shared,
                              combine=pkg.COMBINE_CHAIN if chain else pkg.COMBINE_F32, max_tokens=max_tokens,
                              device=device)
        self.moe = pkg.MoE(cfg)
        self.records = {}
        self.seed = seed
        todo = range(n_experts) if experts_to_load is None else experts_to_load
        for e in todo:
            self.load(e)
        self.shared = None
        if shared:
            rng = np.random.default_rng(seed + 991)
            ws = [O.f32_to_bf16_bits((rng.standard_normal(s) * 0.02).astype(np.float32))
                  for s in ((inter, hidden), (inter, hidden), (hidden, inter))]
            self.shared = ws
            self.moe.set_shared(0, ws[0].ctypes.data, ws[1].ctypes.data, ws[2].ctypes.data, on_device=False)

    def record_seed(self, e):
        return 0x5EED0000 + 1000 * self.seed + 17 * e

    def synth(self, e):
        return O.exl3_synth_record(self.record_seed(e), self.H, self.I, 1.0, 0.02)

    def load(self, e):
        rec = self.synth(e)
        self.records[e] = rec
        self.moe.load_expert(0, e, rec.ctypes.data, rec.size, on_device=False)

    # ---- inputs ----
    def inputs(self, T, seed=1):
        rng = np.random.default_rng(seed)
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal((T, self.H)).astype(np.float32)))
        logits = rng.standard_normal((T, self.E)).astype(np.float32)
        return x, logits

    def to_dev_bf16(self, x):
        torch = torch_mod()
        return torch.from_numpy(O.f32_to_bf16_bits(x).view(np.int16).reshape(x.shape)).to(self.dev).view(torch.bfloat16)

    # ---- GPU calls through the C ABI ----
    def gpu_route(self, logits):
        torch = torch_mod()
        T = logits.shape[0]
        lg = torch.from_numpy(logits).to(self.dev)
        ids = torch.empty((T, self.k), dtype=torch.int32, device=self.dev)
        w = torch.empty((T, self.k), dtype=torch.float32, device=self.dev)
        self.moe.route(0, lg.data_ptr(), T, ids.data_ptr(), w.data_ptr(), None)
        torch.cuda.synchronize()
        return ids.cpu().numpy(), w.cpu().numpy()

    def gpu_routed(self, x, ids):
        torch = torch_mod()
        T = x.shape[0]
        xd = self.to_dev_bf16(x)
        idd = torch.from_numpy(np.ascontiguousarray(ids, np.int32)).to(self.dev)
        out = torch.full((T, self.k, self.H), float("nan"), dtype=torch.float32, device=self.dev)
        self.moe.routed(0, xd.data_ptr(), idd.data_ptr(), T, out.data_ptr(), None)
        torch.cuda.synchronize()
        return out.cpu().numpy()

    def gpu_experts(self, x, ids, weights):
        torch = torch_mod()
        T = x.shape[0]
        xd = self.to_dev_bf16(x)
        idd = torch.from_numpy(np.ascontiguousarray(ids, np.int32)).to(self.dev)
        wd = torch.from_numpy(np.ascontiguousarray(weights, np.float32)).to(self.dev)
        y = torch.empty((T, self.H), dtype=torch.bfloat16, device=self.dev)
        self.moe.experts(0, xd.data_ptr(), idd.data_ptr(), wd.data_ptr(), T, y.data_ptr(), None)
        torch.cuda.synchronize()
        return y.float().cpu().numpy()

    def gpu_forward(self, x, logits):
        torch = torch_mod()
        T = x.shape[0]
        xd = self.to_dev_bf16(x)
        lg = torch.from_numpy(logits).to(self.dev)
        y = torch.empty((T, self.H), dtype=torch.bfloat16, device=self.dev)
        self.moe.forward(0, xd.data_ptr(), lg.data_ptr(), T, y.data_ptr(), None)
        torch.cuda.synchronize()
        return y.float().cpu().numpy()

    def gpu_forward_host(self, x, logits):
        T = x.shape[0]
        xb = O.f32_to_bf16_bits(x)
        lg = np.ascontiguousarray(logits, np.float32)
        y = np.empty((T, self.H), np.uint16)
        self.moe.forward_host(0, xb.ctypes.data, lg.ctypes.data, T, y.ctypes.data, None)
        return O.bf16_bits_to_f32(y)

    def gpu_gemv(self, expert, proj, xh):
        torch = torch_mod()
        xh = np.ascontiguousarray(xh, np.float32)
        rows = xh.shape[0]
        out_dim = self.H if proj == 2 else self.I
        xd = torch.from_numpy(xh).to(self.dev)
        z = torch.full((rows, out_dim), float("nan"), dtype=torch.float32, device=self.dev)
        self.moe.exl3_gemv(0, expert, proj, xd.data_ptr(), rows, z.data_ptr(), None)
        torch.cuda.synchronize()
        return z.cpu().numpy()

    # ---- oracle ----
    def cpu_route(self, logits, det=True):
        return O.route(logits, None, self.k, self.scoring, norm=True, scale=self.routed_scale, det=det)

    def cpu_layer(self, x, ids, weights, want_ro=False):
        return O.layer(self.bank, self.H, self.I, self.E, self.k, self.records, x, ids, weights, shared=self.shared,
                       limit=self.limit, chain_rounding=self.chain, shared_bf16_add=self.chain, want_ro=want_ro)

    def status(self):
        return self.moe.stats().device_status

    def close(self):
        self.moe.close()


class Exl3K2Case(Exl3Case):
    """The EXL3 bank at 2 bits per weight (the reference's K = 2 layers, src/exl3/kernels.zig:163-177)."""
    bank = O.BANK_EXL3_K2

    def synth(self, e):
        return O.exl3_synth_record(self.record_seed(e), self.H, self.I, 1.0, 0.02, K=2)


class Mxfp4Case(Exl3Case):
    """MiMo-style bank: MXFP4 codes with E8M0 block scales, unclamped SwiGLU, chain combine."""
    bank = O.BANK_MXFP4

    def synth(self, e):
        return O.mxfp4_synth_record(self.record_seed(e), self.H, self.I, 0.02)


class Nvfp4Case(Exl3Case):
    """GLM-Flash-style bank: NVFP4 codes with E4M3 block scales and a global scale, clamped SwiGLU, chain combine."""
    bank = O.BANK_NVFP4

    def synth(self, e):
        return O.nvfp4_synth_record(self.record_seed(e), self.H, self.I, 0.02)


def zipf_bias(n_experts, layer=0, s=1.1):
    """ln p_e with p_e ~ rank^-s over a permutation of the experts seeded by the layer: added to N(0,1) logits it gives
    the skewed routing of the benchmark's Zipf workloads (tau = 1)."""
    perm = np.random.default_rng(4242 + layer).permutation(n_experts)
    p = np.arange(1, n_experts + 1, dtype=np.float64) ** -s
    p /= p.sum()
    return np.log(p)[np.argsort(perm)].astype(np.float32)


def rel_l2(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.linalg.norm(got - ref) / (np.linalg.norm(ref) + 1e-30))


def max_err_over_rms(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.abs(got - ref).max() / (np.sqrt((ref * ref).mean()) + 1e-30))


def run_smoke():
    """One tiny call of the hot path on cuda:0, checked against the oracle (GLM-Flash EXL3 shape, 4 experts, top-2)."""
    case = Exl3Case(512, 256, 4, 2, seed=3, shared=True, max_tokens=8)
    x, logits = case.inputs(3, seed=5)
    y = case.gpu_forward(x, logits)
    ids, w = case.cpu_route(logits)
    ref = case.cpu_layer(x, ids, w)
    err = rel_l2(y, ref)
    st = case.status()
    case.close()
    assert st == 0, f"device status {st}"
    assert err < 1e-2, f"smoke: rel-L2 {err}"
    print(f"smoke ok: rel-L2 {err:.3e}")
