"""GPU parity of the MXFP4 and NVFP4 routed-MoE paths against the CPU oracle, through the C ABI.

The oracle decodes the same packed bytes (src/arch/mimo_v2/moe.zig:379-416, src/arch/glm5_next/decode_kernels_ref.zig:13-65)
and applies the reference decode texts' rounding points (bf16 gate/up, bf16 SiLU product, bf16 down rows, the chain
combine); the bar for the bf16 layer output is 1e-2 relative L2.
"""
import numpy as np
import pytest

import oracle_lib as O
from moe_cases import Mxfp4Case, Nvfp4Case, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.mark.parametrize("cls,limit,shared", [(Mxfp4Case, 0.0, False), (Nvfp4Case, 10.0, True)])
def test_fp4_small_layer(cls, limit, shared):
    case = cls(512, 256, 8, 2, seed=6, shared=shared, scoring=O.SCORE_SIGMOID, max_tokens=64, routed_scale=1.0,
               limit=limit, chain=True)
    try:
        for T in (1, 5, 33, 64):
            x, logits = case.inputs(T, seed=10 + T)
            y = case.gpu_forward(x, logits)
            ids, w = case.cpu_route(logits)
            ref = case.cpu_layer(x, ids, w)
            assert rel_l2(y, ref) < TOL, (T, rel_l2(y, ref))
        # every token to the same experts: more rows than one work item holds
        T = 40
        x, _ = case.inputs(T, seed=3)
        ids = np.tile(np.array([[1, 6]], np.int32), (T, 1))
        w = np.full((T, 2), 0.5, np.float32)
        assert rel_l2(case.gpu_experts(x, ids, w), case.cpu_layer(x, ids, w)) < TOL
        assert case.status() == 0
    finally:
        case.close()


@pytest.mark.parametrize("cls,H,I,limit,shared", [(Mxfp4Case, 4096, 2048, 0.0, False), (Nvfp4Case, 6144, 2048, 10.0, True)])
def test_fp4_config_shapes(cls, H, I, limit, shared):
    # the benchmark list's MXFP4 (MiMo shape) and NVFP4 (GLM shape) configurations at a reduced expert count
    case = cls(H, I, 4, 2, seed=2, shared=shared, scoring=O.SCORE_SIGMOID, max_tokens=16, routed_scale=1.0, limit=limit,
               chain=True)
    try:
        x, logits = case.inputs(6, seed=4)
        ids, w = case.gpu_route(logits)
        rid, rw = case.cpu_route(logits)
        assert (ids == rid).all()
        y = case.gpu_experts(x, ids, w)
        assert rel_l2(y, case.cpu_layer(x, rid, rw)) < TOL
        again = case.gpu_experts(x, ids, w)
        assert (y == again).all()
        one = case.gpu_experts(x[2:3], ids[2:3], w[2:3])
        assert (one[0] == y[2]).all()  # a row does not depend on the batch around it
        assert case.status() == 0
    finally:
        case.close()


def test_fp4_f32_combine_mode():
    # the same bank with the f32 combine (no chain rounding of the rows): against the oracle's unrounded f64 path
    case = Mxfp4Case(512, 256, 8, 2, seed=8, shared=False, scoring=O.SCORE_SOFTMAX, max_tokens=16, routed_scale=1.0,
                     limit=0.0, chain=False)
    try:
        x, logits = case.inputs(9, seed=2)
        y = case.gpu_forward(x, logits)
        ids, w = case.cpu_route(logits)
        assert rel_l2(y, case.cpu_layer(x, ids, w)) < TOL
    finally:
        case.close()


def _skewed_batch(case, T, seed):
    """Expert 0 takes every token, expert 3 a handful: both lanes and several row tiles in one call."""
    x, logits = case.inputs(T, seed=seed)
    logits[:, 0] += 3.0
    logits[:, 3] -= 2.5
    ids, w = case.cpu_route(logits)
    return x, ids, w


@pytest.mark.parametrize("cls,limit,shared", [(Mxfp4Case, 0.0, False), (Nvfp4Case, 10.0, True)])
def test_fp4_tensor_lane(cls, limit, shared):
    """Experts with 17 rows or more go through the tcgen05 lane (the reference's sorted quantised GEMM,
    src/arch/mimo_v2/math.zig:426-447): same decoded weights and rounding chain as the streaming lane, f32 accumulate."""
    case = cls(512, 256, 4, 2, seed=9, shared=shared, scoring=O.SCORE_SIGMOID, max_tokens=512, routed_scale=1.0,
               limit=limit, chain=True)
    try:
        T = 300
        x, ids, w = _skewed_batch(case, T, seed=31)
        counts = np.bincount(ids.reshape(-1), minlength=4)
        assert counts.max() > 256 and 0 < counts.min() < 17
        y = case.gpu_experts(x, ids, w)
        assert case.status() == 0
        assert rel_l2(y, case.cpu_layer(x, ids, w)) < TOL
        # the unweighted rows: the whole call against the same rows taken 8 tokens at a time (16 rows: streaming lane only)
        ro = case.gpu_routed(x, ids)
        assert np.isfinite(ro).all()
        parts = [case.gpu_routed(x[i:i + 8], ids[i:i + 8]) for i in range(0, T, 8)]
        ro_s = np.concatenate(parts, axis=0)
        # both lanes multiply the same exact operands; a bf16 rounding boundary of the gate/up chain may fall either way
        assert rel_l2(ro, ro_s) < 2e-3
        again = case.gpu_routed(x, ids)
        assert (again.view(np.uint32) == ro.view(np.uint32)).all()
        assert case.status() == 0
    finally:
        case.close()


def test_mxfp4_wide_scale_stays_in_streaming_lane():
    """The tensor-core lane builds 2^(b-1) as a bf16, which exists for scale bytes b <= 128; an expert that holds a
    larger byte is marked at load and streams, whatever its row count."""
    case = Mxfp4Case(512, 256, 4, 2, seed=4, shared=False, scoring=O.SCORE_SIGMOID, max_tokens=256, routed_scale=1.0,
                     limit=0.0, chain=True)
    try:
        H, I = case.H, case.I
        rec = case.records[0].copy()
        wbytes, sbytes = H * I // 2, H * I // 32
        s0 = rec[wbytes:wbytes + sbytes]            # the gate projection's E8M0 bytes
        s0[::97] = 131                              # 2^4: beyond the lane's range
        case.records[0] = rec
        case.moe.load_expert(0, 0, rec.ctypes.data, rec.size, on_device=False)
        x, ids, w = _skewed_batch(case, 100, seed=12)
        assert np.bincount(ids.reshape(-1), minlength=4)[0] >= 90
        y = case.gpu_experts(x, ids, w)
        assert case.status() == 0
        assert np.isfinite(y).all()
        assert rel_l2(y, case.cpu_layer(x, ids, w)) < TOL
    finally:
        case.close()


@pytest.mark.parametrize("H,I,T", [(512, 256, 300), (4096, 2048, 280)])
def test_mxfp4_block_scaled_lane_against_decoded_lane(monkeypatch, H, I, T):
    """The MXFP4 tensor-core lane runs on tcgen05.mma.kind::mxf8f6f4.block_scale (codes and E8M0 scales as stored, rows
    split into E4M3 high and low parts); a handle created with MLXS_MXFP4_NATIVE=0 keeps the lane that decodes to bf16
    operands.
    Both multiply the same exact operands with f32 accumulation: the unweighted rows agree to a bf16 rounding boundary of
    the gate/up chain, and both match the f64 oracle."""
    outs = {}
    for native in ("1", "0"):
        monkeypatch.setenv("MLXS_MXFP4_NATIVE", native)
        case = Mxfp4Case(H, I, 4, 2, seed=21, shared=False, scoring=O.SCORE_SIGMOID, max_tokens=512, routed_scale=1.0,
                         limit=0.0, chain=True)
        try:
            x, ids, w = _skewed_batch(case, T, seed=5)
            counts = np.bincount(ids.reshape(-1), minlength=4)
            assert counts.max() > 192 and (counts >= 17).sum() >= 2       # both tile shapes, several tiles
            ro = case.gpu_routed(x, ids)
            assert case.status() == 0
            assert np.isfinite(ro).all()
            y = case.gpu_experts(x, ids, w)
            ref = case.cpu_layer(x[:24], ids[:24], w[:24])
            assert rel_l2(y[:24], ref) < TOL, (native, rel_l2(y[:24], ref))
            again = case.gpu_routed(x, ids)
            assert (again.view(np.uint32) == ro.view(np.uint32)).all()
            outs[native] = ro
        finally:
            case.close()
    assert rel_l2(outs["1"], outs["0"]) < 2e-3, rel_l2(outs["1"], outs["0"])


def test_native_block_scaled_fp4_mma_measured():
    """tcgen05.mma.kind::mxf8f6f4.block_scale on the bank's own bytes: with the bf16 rows split into an E4M3 high and low
    part the product matches the bf16-row product to a few 1e-3 of its rms (the high part alone does not), and the pair
    of 8-bit-rate MMAs it needs per 32 inputs delivers about the 16-bit rate."""
    from __graft_entry__ import load_package
    pkg = load_package()
    r = pkg.fp4_native_probe(0, 4000)
    assert r["rel_l2_hi_lo"] < 4e-3, r
    assert 5e-3 < r["rel_l2_hi_only"] < 0.1, r
    assert r["tflops_f16"] > 100 and r["tflops_mxf8f6f4"] > 1.3 * r["tflops_f16"], r


def test_mma_time_against_the_row_count_of_a_tile():
    """One tcgen05.mma of M 128 x N x K 16 costs the same whether its A operand sits in shared or in tensor memory, takes
    time in proportion to N from 128 rows on and has a floor below that: what the lanes' tile shapes (192-row tiles, A in
    tensor memory) rest on."""
    from __graft_entry__ import load_package
    pkg = load_package()
    t = {(n, a): pkg.mma_rate(0, n, a, 8000) for n in (64, 128, 256) for a in (False, True)}
    for n in (64, 128, 256):
        assert abs(t[(n, True)] - t[(n, False)]) < 0.15 * t[(n, False)], t
    assert 1.6 < t[(256, False)] / t[(128, False)] < 2.4, t          # in proportion from 128 rows on
    assert t[(64, False)] > 0.6 * t[(128, False)], t                  # a floor below
    with pytest.raises(Exception):
        pkg.mma_rate(0, 100, False, 10)
