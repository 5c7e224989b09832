"""GPU parity of the EXL3 routed-MoE path against the CPU oracle, through the C ABI.

Bars: router ids and decoded weights bit-exact; f32 routed rows within the reference's f32-stage tolerance
(max |err| / rms < 1e-4: src/exl3/selfcheck.zig:1167); bf16 layer output within 1e-2 relative L2.
"""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as O
from moe_cases import Exl3Case, Exl3K2Case, max_err_over_rms, rel_l2, LANE_MIN_EXL3

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
TOL_F32 = 1e-4
TOL_LAYER = 1e-2


@pytest.fixture(scope="module")
def c1():
    # the benchmark list's CPU-runnable configuration: hidden 5120, inter 2304, 16 experts, top-4, shared expert, clamped SwiGLU
    case = Exl3Case(5120, 2304, 16, 4, seed=0, shared=True, max_tokens=64)
    yield case
    case.close()


@pytest.mark.parametrize("scoring,E,k", [(0, 256, 8), (1, 256, 8), (2, 256, 8), (0, 16, 4), (1, 288, 8), (2, 16, 4)])
def test_router_bit_exact(scoring, E, k):
    case = Exl3Case(512, 256, E, k, seed=1, shared=False, scoring=scoring, max_tokens=256, experts_to_load=[])
    try:
        for T, seed in ((1, 3), (7, 4), (256, 5)):
            _, logits = case.inputs(T, seed)
            if seed == 5:
                logits[3, :8] = logits[3, 8]  # exact ties -> lower index first
                logits[4, 5] = np.nan
                logits[5] = np.float32(0.25)
            ids, w = case.gpu_route(logits)
            rid, rw = case.cpu_route(logits, det=True)
            assert (ids == rid).all()
            assert (w.view(np.uint32) == rw.view(np.uint32)).all() or np.allclose(w, rw, rtol=1e-6, equal_nan=True)
            lid, lw = case.cpu_route(logits, det=False)
            assert (ids == lid).mean() > 0.999
    finally:
        case.close()


def test_router_bias_changes_selection_not_weights():
    # src/arch/mimo_v2/config.zig:503-514
    case = Exl3Case(512, 256, 4, 2, seed=1, shared=False, scoring=1, max_tokens=8, experts_to_load=[], routed_scale=1.0)
    try:
        bias = np.array([0, 0, 10, 0], np.float32)
        case.moe.set_router_bias(0, bias.ctypes.data)
        ids, w = case.gpu_route(np.array([[0, 2, -2, 1]], np.float32))
        assert ids.tolist() == [[2, 1]]
        low, high = 1 / (1 + np.exp(2.0)), 1 / (1 + np.exp(-2.0))
        assert abs(w[0, 0] - low / (low + high)) < 1e-6 and abs(w[0].sum() - 1) < 1e-6
    finally:
        case.close()


def test_decoded_weights_bit_exact_against_golden_planes():
    """The reference's decode_table check (src/exl3/selfcheck.zig:848-901): one-hot rows through the GEMV return
    W_hat's rows bit for bit; their sha256 is the golden `onehot_rows_sha256` of src/kernels/exl3/manifest.json."""
    dig = json.loads((GOLD / "exl3_digests.json").read_text())["planes"]
    H, I = 5120, 2304
    case = Exl3Case(H, I, 2, 1, seed=0, shared=False, max_tokens=512, experts_to_load=[])
    try:
        g = O.exl3_geometry(H, I)
        rec = np.zeros(g.record_bytes, np.uint8)
        gate = O.fill_code(dig["gate_up"]["seed"], g.len[0] // 2)
        down = O.fill_code(dig["down"]["seed"], g.len[6] // 2)
        rec[g.off[0]:g.off[0] + g.len[0]] = gate.view(np.uint8)
        rec[g.off[3]:g.off[3] + g.len[3]] = gate.view(np.uint8)[::-1].copy()  # up: a different stream
        rec[g.off[6]:g.off[6] + g.len[6]] = down.view(np.uint8)
        case.moe.load_expert(0, 1, rec.ctypes.data, rec.size)
        for proj, name, n_in in ((0, "gate_up", H), (2, "down", I)):
            rows = dig[name]["onehot_rows"]
            xh = np.zeros((rows, n_in), np.float32)
            xh[np.arange(rows), np.arange(rows)] = 1.0
            z = case.gpu_gemv(1, proj, xh)
            z16 = z.astype(np.float16)
            assert (z16.astype(np.float32) == z).all()
            assert hashlib.sha256(z16.tobytes()).hexdigest() == dig[name]["onehot_rows_sha256"]
        # the up projection decodes its own stream
        up_code = rec[g.off[3]:g.off[3] + g.len[3]].view(np.int16)
        w_up = O.reconstruct(up_code, H // 16, I // 16, 3).view(np.float16)
        xh = np.zeros((24, H), np.float32)
        sel = np.arange(24) * 211 % H
        xh[np.arange(24), sel] = 1.0
        assert (case.gpu_gemv(1, 1, xh) == w_up[sel].astype(np.float32)).all()
        assert case.status() == 0
    finally:
        case.close()


def test_gemv_against_f64(c1):
    # src/arch/glm5_next/exl3_parity.zig:132-166: the GEMV against the f64 product
    rng = np.random.default_rng(11)
    g = O.exl3_geometry(c1.H, c1.I)
    for proj, n_in, n_out in ((0, c1.H, c1.I), (1, c1.H, c1.I), (2, c1.I, c1.H)):
        xh = rng.standard_normal((19, n_in)).astype(np.float32)
        z = c1.gpu_gemv(3, proj, xh)
        code = c1.records[3][g.off[3 * proj]:g.off[3 * proj] + g.len[3 * proj]].view(np.int16)
        w = O.reconstruct(code, n_in // 16, n_out // 16, 3).view(np.float16).astype(np.float64)
        ref = xh.astype(np.float64) @ w
        assert max_err_over_rms(z, ref) < 2.0 ** -16 * 8


@pytest.mark.parametrize("T", [1, 8])
def test_layer_config1(c1, T):
    x, logits = c1.inputs(T, seed=20 + T)
    ids, w = c1.gpu_route(logits)
    rid, rw = c1.cpu_route(logits)
    assert (ids == rid).all()
    ref_y, ref_ro = c1.cpu_layer(x, rid, rw, want_ro=True)
    ro = c1.gpu_routed(x, ids)
    assert max_err_over_rms(ro, ref_ro) < TOL_F32
    y = c1.gpu_experts(x, ids, w)
    assert rel_l2(y, ref_y) < TOL_LAYER
    y2 = c1.gpu_forward(x, logits)
    assert (y2 == y).all()
    y3 = c1.gpu_forward_host(x, logits)
    assert (y3 == y).all()
    assert c1.status() == 0


def test_row_invariance_and_determinism(c1):
    # src/exl3/selfcheck.zig:747-846: a row's result does not depend on the batch around it; runs repeat bit for bit
    x, logits = c1.inputs(8, seed=77)
    ids, _ = c1.cpu_route(logits)
    full = c1.gpu_routed(x, ids)
    again = c1.gpu_routed(x, ids)
    assert (full.view(np.uint32) == again.view(np.uint32)).all()
    for t in (0, 5):
        one = c1.gpu_routed(x[t:t + 1], ids[t:t + 1])
        assert (one[0].view(np.uint32) == full[t].view(np.uint32)).all()


def test_ragged_and_heavy_experts(c1):
    # every token to the same experts (rows per expert > one work item), and an empty call
    T = 40
    x, _ = c1.inputs(T, seed=5)
    ids = np.tile(np.array([[2, 9, 11, 0]], np.int32), (T, 1))
    ids[::3, 3] = 15
    w = np.full((T, 4), 0.25, np.float32)
    ref = c1.cpu_layer(x, ids, w)
    y = c1.gpu_experts(x, ids, w)
    assert rel_l2(y, ref) < TOL_LAYER
    assert c1.gpu_experts(x[:0], ids[:0], w[:0]).shape == (0, c1.H)
    assert c1.status() == 0


def test_bad_ids_and_missing_experts_are_reported_not_faulted():
    case = Exl3Case(512, 256, 8, 2, seed=2, shared=False, max_tokens=8, experts_to_load=[0, 1, 2])
    try:
        x, _ = case.inputs(2, seed=1)
        w = np.full((2, 2), 0.5, np.float32)
        case.gpu_experts(x, np.array([[0, 1], [2, 1]], np.int32), w)
        assert case.status() == 0
        case.gpu_experts(x, np.array([[0, 5], [2, 1]], np.int32), w)  # expert 5 never loaded
        assert case.status() == 5
        with pytest.raises(case.pkg.MlxsError) as ei:
            case.gpu_forward_host(x, np.zeros((2, 8), np.float32))
        assert ei.value.rc == -7
    finally:
        case.close()
    case = Exl3Case(512, 256, 8, 2, seed=2, shared=False, max_tokens=8)
    try:
        x, _ = case.inputs(2, seed=1)
        case.gpu_experts(x, np.array([[0, 99], [-4, 1]], np.int32), np.full((2, 2), 0.5, np.float32))
        assert case.status() == 1
        with pytest.raises(case.pkg.MlxsError) as ei:
            case.gpu_experts(np.zeros((9, 512), np.float32), np.zeros((9, 2), np.int32), np.zeros((9, 2), np.float32))
        assert ei.value.rc == -6
    finally:
        case.close()


def test_small_shape_layer_many_seeds():
    case = Exl3Case(512, 256, 8, 2, seed=4, shared=True, max_tokens=64)
    try:
        for T in (1, 3, 17, 64):
            x, logits = case.inputs(T, seed=T)
            y = case.gpu_forward(x, logits)
            ids, w = case.cpu_route(logits)
            assert rel_l2(y, case.cpu_layer(x, ids, w)) < TOL_LAYER
        assert case.status() == 0
    finally:
        case.close()


def test_prefill_lane_tcgen05():
    """Experts with LANE_MIN_EXL3 rows or more take the tensor-core lane, the others of the same call the streaming lane (the
    reference picks the lane on logical M: src/sdk_ext/quant.zig:5-6): f16-rounded rotated activations as the
    reference's prefill chain (src/kernels/exl3/dsv41_prefill_dig_take2v_5120.metal:57-58), f32 accumulate."""
    case = Exl3Case(512, 256, 4, 2, seed=12, shared=True, max_tokens=1024)
    try:
        rng = np.random.default_rng(5)
        # ragged: expert 0 gets 129+ rows (two row tiles), expert 3 a handful, every row count class appears
        T = 300
        x, logits = case.inputs(T, seed=31)
        logits[:, 0] += 3.0
        logits[:, 3] -= 2.5
        ids, w = case.cpu_route(logits)
        counts = np.bincount(ids.reshape(-1), minlength=4)
        assert counts.max() > 128 and 0 < counts.min() < LANE_MIN_EXL3  # both lanes in one call
        ref_y, ref_ro = case.cpu_layer(x, ids, w, want_ro=True)
        ro = case.gpu_routed(x, ids)
        assert case.status() == 0
        assert max_err_over_rms(ro, ref_ro) < 4e-3  # f16 rounding of the two GEMM inputs
        assert rel_l2(ro, ref_ro) < 1e-3
        y = case.gpu_experts(x, ids, w)
        assert rel_l2(y, ref_y) < TOL_LAYER
        again = case.gpu_routed(x, ids)
        assert (again.view(np.uint32) == ro.view(np.uint32)).all()
        # a row does not depend on the batch around it as long as its expert stays in the same lane
        keep = np.arange(0, T, 2)
        sub = case.gpu_routed(x[keep], ids[keep])
        sub_counts = np.bincount(ids[keep].reshape(-1), minlength=4)
        same_lane = (counts >= LANE_MIN_EXL3) == (sub_counts >= LANE_MIN_EXL3)
        assert same_lane.sum() >= 2
        m = same_lane[ids[keep]]
        assert (sub.view(np.uint32)[m] == ro[keep].view(np.uint32)[m]).all()
        # the streaming lane alone (fewer rows than the threshold in the whole call) agrees within the f16 rounding
        few = case.gpu_routed(x[:8], ids[:8])
        assert max_err_over_rms(few, ro[:8]) < 4e-3
    finally:
        case.close()


def test_load_bank_from_reference_format_files(tmp_path):
    """Bank.open + fill (src/expert/bank.zig:208-324): experts.bin + expert-manifest-v2.json written in the
    reference's format, record digests verified, the layer equal to the one loaded record by record."""
    import bank_files
    H, I, E, k = 512, 256, 4, 2
    a = Exl3Case(H, I, E, k, seed=21, shared=False, max_tokens=16)
    b = Exl3Case(H, I, E, k, seed=21, shared=False, max_tokens=16, experts_to_load=[])
    try:
        bank_files.write_exl3_bank(tmp_path, H, I, E, 1, lambda l, e: a.records[e])
        b.moe.load_bank(tmp_path)
        x, logits = a.inputs(9, seed=3)
        assert (a.gpu_forward(x, logits) == b.gpu_forward(x, logits)).all()
        assert b.status() == 0
        # a corrupted record is refused by its digest
        raw = bytearray((tmp_path / "experts.bin").read_bytes())
        raw[5000] ^= 1
        (tmp_path / "experts.bin").write_bytes(bytes(raw))
        with pytest.raises(b.pkg.MlxsError) as ei:
            b.moe.load_bank(tmp_path)
        assert "sha256" in ei.value.msg
    finally:
        a.close()
        b.close()


def test_bank_of_mixed_layer_widths(tmp_path):
    """A bank whose layers differ in K (the reference's 2.9 bpw DeepSeek banks, src/exl3/quant.zig:39-41, 73): the
    load gives every layer its own width from the manifest, and each layer computes what a one-width handle computes
    over the same records, bit for bit."""
    import bank_files
    import torch
    H, I, E, k, T = 512, 256, 4, 2, 9
    bits = [3, 2, 3]
    cases = [(Exl3K2Case if b == 2 else Exl3Case)(H, I, E, k, seed=40 + l, shared=False, max_tokens=16) for l, b in enumerate(bits)]
    pkg = cases[0].pkg
    cfg = pkg.make_config(H, I, E, k, n_layers=3, bank_kind=pkg.BANK_EXL3_K3_MUL1, act=pkg.ACT_SWIGLU_CLAMPED, act_limit=10.0,
                          scoring=pkg.SCORE_SQRTSOFTPLUS, norm_topk=True, routed_scale=1.5, shared_expert=False,
                          combine=pkg.COMBINE_F32, max_tokens=16, device=0)
    moe = pkg.MoE(cfg)
    try:
        bank_files.write_exl3_bank(tmp_path, H, I, E, 3, lambda l, e: cases[l].records[e], bits)
        resident_before = moe.stats().resident_bytes
        moe.load_bank(tmp_path)
        assert [moe.layer_record_bytes(l)[0] for l in range(3)] == bits
        g3, g2 = O.exl3_geometry(H, I, 3), O.exl3_geometry(H, I, 2)
        assert moe.layer_record_bytes(1)[1:] == (g2.logical_bytes, g2.record_bytes)
        assert moe.record_bytes() == (g3.logical_bytes, g3.record_bytes)
        # the narrower layer gave HBM back: one third of its three code planes
        assert resident_before - moe.stats().resident_bytes == E * 3 * (H // 16) * (I // 16) * 32
        for l, c in enumerate(cases):
            x, logits = c.inputs(T, seed=70 + l)
            xd, lg = c.to_dev_bf16(x), torch.from_numpy(logits).to(c.dev)
            y = torch.empty((T, H), dtype=torch.bfloat16, device=c.dev)
            moe.forward(l, xd.data_ptr(), lg.data_ptr(), T, y.data_ptr(), None)
            torch.cuda.synchronize()
            assert (y.float().cpu().numpy() == c.gpu_forward(x, logits)).all(), l
            ids, w = c.cpu_route(logits)
            assert rel_l2(y.float().cpu().numpy(), c.cpu_layer(x, ids, w)) < 1e-2
        assert moe.stats().device_status == 0
        # a layer that holds experts keeps its width; unknown widths are refused by name
        with pytest.raises(pkg.MlxsError) as ei:
            moe.set_layer_bits(0, 2)
        assert "already holds experts" in ei.value.msg
        with pytest.raises(pkg.MlxsError) as ei:
            moe.set_layer_bits(0, 4)
        assert "KNotImplemented" in ei.value.msg
        # a K = 3 record offered to the K = 2 layer's neighbour is fine, a K = 2 record to a K = 3 layer is too short
        rec2 = cases[1].records[0]
        with pytest.raises(pkg.MlxsError) as ei:
            moe.load_expert(0, 0, rec2.ctypes.data, int(g2.logical_bytes), on_device=False)
        assert "RecordGeometry" in ei.value.msg
    finally:
        moe.close()
        for c in cases:
            c.close()


def test_usage_tally_counts_routes_per_layer():
    """The route tally (the reference counts routes per layer and expert, src/sdk_ext/expert/usage.zig:202-224): off
    by default, counts every routed id of route / forward while on, per layer, and adds ids a host routed elsewhere."""
    import torch
    case = Exl3Case(512, 256, 16, 4, seed=8, shared=False, max_tokens=4096)
    try:
        moe, E, k = case.moe, case.E, case.k
        with pytest.raises(case.pkg.MlxsError) as ei:
            moe.usage_read(0)
        assert "tally is off" in ei.value.msg
        moe.usage_enable(True)
        want = np.zeros(E, np.int64)
        for T, seed in ((1, 1), (37, 2), (3000, 3)):
            x, logits = case.inputs(T, seed=seed)
            logits[:, 3] += 2.0                      # a popular expert
            ids, _ = case.gpu_route(logits)
            want += np.bincount(ids.reshape(-1), minlength=E)
        x, logits = case.inputs(9, seed=4)
        case.gpu_forward(x, logits)                  # forward routes too
        want += np.bincount(case.cpu_route(logits)[0].reshape(-1), minlength=E)
        assert moe.usage_read(0) == list(want) and moe.usage_read(0, all_ranks=True) == list(want)
        # ids from elsewhere, out-of-range ones ignored (the dispatch reports those)
        ext = np.array([0, 5, 5, 15, 16, -1, 5], np.int32)
        d = torch.from_numpy(ext).to(case.dev)
        moe.usage_add(0, d.data_ptr(), ext.size, None)
        want += np.bincount(ext[(ext >= 0) & (ext < E)], minlength=E)
        assert moe.usage_read(0) == list(want)
        place = case.pkg.plan_placement(moe.usage_read(0), 4)
        assert sorted(place.count(r) for r in range(4)) == [4, 4, 4, 4] and place[3] == 0   # the hottest expert leads
        moe.usage_enable(False)
        case.gpu_route(logits)
        assert moe.usage_read(0) == list(want)       # off: nothing is counted, the counts stay readable
        moe.usage_reset()
        assert sum(moe.usage_read(0)) == 0
        assert case.status() == 0
    finally:
        case.close()


def test_forward_is_capturable_in_a_cuda_graph():
    """A layer call allocates nothing and never synchronises, so a host can capture it into a CUDA graph and replay it
    (the second stream of the shared expert forks from and joins the capturing stream)."""
    import torch
    case = Exl3Case(512, 256, 8, 2, seed=5, shared=True, max_tokens=8)
    try:
        T = 3
        x, logits = case.inputs(T, seed=9)
        ref = case.gpu_forward(x, logits)          # also warms every kernel up outside the capture
        xd = case.to_dev_bf16(x)
        lg = torch.from_numpy(logits).to(case.dev)
        y = torch.zeros((T, case.H), dtype=torch.bfloat16, device=case.dev)
        side = torch.cuda.Stream(device=case.dev)
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                case.moe.forward(0, xd.data_ptr(), lg.data_ptr(), T, y.data_ptr(), side.cuda_stream)
        torch.cuda.synchronize()
        for _ in range(2):
            y.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert (y.float().cpu().numpy() == ref).all()
        assert case.status() == 0
    finally:
        case.close()


def test_call_with_both_lanes_is_capturable_in_a_cuda_graph():
    """A call whose experts use the streaming lane and both tile lists of the tensor-core lane forks three side streams
    (shared expert, tensor-core lane, the lane's large tiles) and joins them again: the capture stays valid and a replay
    gives the eager call's bits."""
    import torch
    case = Exl3Case(512, 256, 4, 2, seed=12, shared=True, max_tokens=512)
    try:
        T = 300
        x, logits = case.inputs(T, seed=31)
        logits[:, 0] += 3.0          # every token: several large tiles
        logits[:, 3] -= 2.5          # a handful of rows: streaming lane
        ids, _ = case.cpu_route(logits)
        counts = np.bincount(ids.reshape(-1), minlength=4)
        assert counts.max() > 192 and ((counts > 0) & (counts < LANE_MIN_EXL3)).any(), counts   # large tiles and streaming rows
        ref = case.gpu_forward(x, logits)
        xd = case.to_dev_bf16(x)
        lg = torch.from_numpy(logits).to(case.dev)
        y = torch.zeros((T, case.H), dtype=torch.bfloat16, device=case.dev)
        side = torch.cuda.Stream(device=case.dev)
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                case.moe.forward(0, xd.data_ptr(), lg.data_ptr(), T, y.data_ptr(), side.cuda_stream)
        torch.cuda.synchronize()
        for _ in range(2):
            y.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert (y.float().cpu().numpy() == ref).all()
        assert case.status() == 0
    finally:
        case.close()


def test_placement_refusals():
    case = Exl3Case(512, 256, 4, 2, seed=1, shared=False, max_tokens=8, experts_to_load=[])
    try:
        lib = case.pkg.lib()
        ok = np.zeros(4, np.uint16)
        assert lib.mlxs_moe_set_placement(case.moe._h, 0, ok.ctypes.data) == 0      # one rank: everything on rank 0
        bad = np.array([0, 1, 0, 0], np.uint16)
        assert lib.mlxs_moe_set_placement(case.moe._h, 0, bad.ctypes.data) != 0     # rank 1 of a world of 1
        assert "rank" in case.pkg.last_error()
        case.load(2)
        assert lib.mlxs_moe_set_placement(case.moe._h, 0, ok.ctypes.data) != 0      # after loading: refused
        assert "before loading" in case.pkg.last_error()
    finally:
        case.close()


def test_many_assignments_take_the_multi_cta_dispatch():
    """More than 2048 assignment rows: the sort runs over several CTAs (count, scan, place) and both lanes are busy."""
    case = Exl3Case(512, 256, 8, 4, seed=14, shared=True, max_tokens=640)
    try:
        T = 600
        x, logits = case.inputs(T, seed=77)
        logits[:, 5] -= 3.0          # one expert with few rows (streaming lane), the others heavy (tensor-core lane)
        ids, w = case.cpu_route(logits)
        assert ids.size > 2048 and 0 < np.bincount(ids.reshape(-1), minlength=8)[5] < LANE_MIN_EXL3
        y = case.gpu_experts(x, ids, w)
        assert case.status() == 0
        assert rel_l2(y, case.cpu_layer(x, ids, w)) < TOL_LAYER
        gid, gw = case.gpu_route(logits)
        assert (gid == ids).all()
    finally:
        case.close()


def test_limits_empty_call_too_many_tokens_and_the_widest_router():
    case = Exl3Case(512, 256, 1024, 64, seed=2, shared=False, scoring=1, max_tokens=16, experts_to_load=[],
                    routed_scale=1.0)
    try:
        import torch
        # the widest configuration the library accepts: 1024 experts, top-64 (the rank-count selection path)
        _, logits = case.inputs(5, seed=8)
        ids, w = case.gpu_route(logits)
        rid, rw = case.cpu_route(logits)
        assert (ids == rid).all() and np.allclose(w, rw, rtol=1e-6)
        # only the experts a small batch touches are loaded; the layer over them matches the oracle
        x, logits = case.inputs(2, seed=9)
        ids, w = case.cpu_route(logits)
        for e in np.unique(ids):
            case.load(int(e))
        y = case.gpu_experts(x, ids, w)
        assert case.status() == 0
        assert rel_l2(y, case.cpu_layer(x, ids, w)) < TOL_LAYER
        # an empty call is a no-op, one token too many is refused by name
        lib = case.pkg.lib()
        assert lib.mlxs_moe_forward(case.moe._h, 0, None, None, 0, None, None) == 0
        big = torch.zeros((17, 512), dtype=torch.bfloat16, device=case.dev)
        lg = torch.zeros((17, 1024), dtype=torch.float32, device=case.dev)
        rc = lib.mlxs_moe_forward(case.moe._h, 0, big.data_ptr(), lg.data_ptr(), 17, big.data_ptr(), None)
        assert rc == case.pkg.E_TOO_MANY_TOKENS, (rc, case.pkg.last_error())
    finally:
        case.close()


def test_router_logits_product_and_the_layer_from_x():
    """logits = f32(x) . f32(W_g)^T (src/arch/deepseek_v41/graph.zig:2033) in both forms (own kernel up to 64 tokens, the
    library GEMM above), and the layer started from x.  The f32 sum order is the kernel's own, so ids are compared only
    where the k-th and (k+1)-th keys are not a near-tie."""
    import torch
    case = Exl3Case(512, 256, 8, 2, seed=6, shared=True, max_tokens=128)
    try:
        rng = np.random.default_rng(17)
        wg = O.f32_to_bf16_bits((rng.standard_normal((8, 512)) * 0.05).astype(np.float32))
        case.moe.set_router_weight(0, wg.ctypes.data)
        wf = O.bf16_bits_to_f32(wg).astype(np.float64)
        for T in (1, 7, 64, 100):
            x, _ = case.inputs(T, seed=40 + T)
            ref_logits = (x.astype(np.float64) @ wf.T).astype(np.float32)
            xd = case.to_dev_bf16(x)
            lg = torch.full((T, 8), float("nan"), dtype=torch.float32, device=case.dev)
            case.moe.logits(0, xd.data_ptr(), T, lg.data_ptr(), None)
            torch.cuda.synchronize()
            got = lg.cpu().numpy()
            assert np.allclose(got, ref_logits, rtol=2e-5, atol=2e-5), np.abs(got - ref_logits).max()
            again = torch.empty_like(lg)
            case.moe.logits(0, xd.data_ptr(), T, again.data_ptr(), None)
            torch.cuda.synchronize()
            assert (again.cpu().numpy().view(np.uint32) == got.view(np.uint32)).all()
            # the layer from x equals the layer from these logits
            y = torch.empty((T, 512), dtype=torch.bfloat16, device=case.dev)
            case.moe.forward_x(0, xd.data_ptr(), T, y.data_ptr(), None)
            torch.cuda.synchronize()
            assert (y.float().cpu().numpy() == case.gpu_forward(x, got)).all()
            ids, w = case.cpu_route(got)
            assert rel_l2(y.float().cpu().numpy(), case.cpu_layer(x, ids, w)) < TOL_LAYER
        assert case.status() == 0
    finally:
        case.close()


@pytest.mark.parametrize("H,I,proj,which", [(5120, 2304, 0, "gate_up"), (5120, 2304, 2, "down"), (4096, 2048, 0, 0),
                                            (4096, 2048, 2, 1)])
def test_whole_golden_planes_decode_bit_exact(H, I, proj, which):
    """Every row of the reference's seeded planes through the GPU decode: the f16 plane's sha256 is the golden
    `w_hat_sha256` (src/kernels/exl3/manifest.json planes; src/arch/glm5_next/exl3_parity.zig:19-23 for the GLM shape)."""
    gold = json.loads((GOLD / "exl3_digests.json").read_text())
    plane = gold["planes"][which] if isinstance(which, str) else gold["glm_planes"][which]
    n_in, n_out = (I, H) if proj == 2 else (H, I)
    case = Exl3Case(H, I, 1, 1, seed=0, shared=False, max_tokens=1024, experts_to_load=[])
    try:
        g = O.exl3_geometry(H, I)
        rec = np.zeros(g.record_bytes, np.uint8)
        seg = 6 if proj == 2 else 0
        code = O.fill_code(plane["seed"], g.len[seg] // 2)
        assert hashlib.sha256(code.tobytes()).hexdigest() == plane["code_sha256"]
        rec[g.off[seg]:g.off[seg] + g.len[seg]] = code.view(np.uint8)
        case.moe.load_expert(0, 0, rec.ctypes.data, rec.size)
        digest = hashlib.sha256()
        for r0 in range(0, n_in, 1024):
            rows = min(1024, n_in - r0)
            xh = np.zeros((rows, n_in), np.float32)
            xh[np.arange(rows), r0 + np.arange(rows)] = 1.0
            z = case.gpu_gemv(0, proj, xh)
            z16 = z.astype(np.float16)
            assert (z16.astype(np.float32) == z).all()
            digest.update(z16.tobytes())
        assert digest.hexdigest() == plane["w_hat_sha256"]
        assert case.status() == 0
    finally:
        case.close()


# ---- EXL3 at 2 bits per weight (the reference's K = 2 layers) ----
@pytest.mark.parametrize("proj,which", [(0, "gate_up_k2"), (2, "down_k2")])
def test_k2_whole_golden_planes_decode_bit_exact(proj, which):
    """src/kernels/exl3/manifest.json golden planes at K = 2 (scripts/dsv41_exl3_k2_goldens.json): every row of the
    plane through the GPU decode, the f16 plane's sha256 against `w_hat_sha256`."""
    from moe_cases import Exl3K2Case
    plane = json.loads((GOLD / "exl3_digests.json").read_text())["planes"][which]
    H, I = 5120, 2304
    n_in = I if proj == 2 else H
    case = Exl3K2Case(H, I, 1, 1, seed=0, shared=False, max_tokens=1024, experts_to_load=[])
    try:
        g = O.exl3_geometry(H, I, 2)
        rec = np.zeros(g.record_bytes, np.uint8)
        seg = 6 if proj == 2 else 0
        code = O.fill_code(plane["seed"], g.len[seg] // 2)
        assert hashlib.sha256(code.tobytes()).hexdigest() == plane["code_sha256"]
        rec[g.off[seg]:g.off[seg] + g.len[seg]] = code.view(np.uint8)
        case.moe.load_expert(0, 0, rec.ctypes.data, rec.size)
        digest = hashlib.sha256()
        for r0 in range(0, n_in, 1024):
            rows = min(1024, n_in - r0)
            xh = np.zeros((rows, n_in), np.float32)
            xh[np.arange(rows), r0 + np.arange(rows)] = 1.0
            z16 = case.gpu_gemv(0, proj, xh).astype(np.float16)
            digest.update(z16.tobytes())
        assert digest.hexdigest() == plane["w_hat_sha256"]
        assert case.status() == 0
    finally:
        case.close()


def test_k2_layer_both_lanes():
    from moe_cases import Exl3K2Case
    case = Exl3K2Case(512, 256, 4, 2, seed=12, shared=True, max_tokens=512)
    try:
        for T in (1, 9):
            x, logits = case.inputs(T, seed=3 + T)
            y = case.gpu_forward(x, logits)
            ids, w = case.cpu_route(logits)
            assert rel_l2(y, case.cpu_layer(x, ids, w)) < TOL_LAYER
        T = 300
        x, logits = case.inputs(T, seed=31)
        logits[:, 0] += 3.0
        logits[:, 3] -= 2.5
        ids, w = case.cpu_route(logits)
        counts = np.bincount(ids.reshape(-1), minlength=4)
        assert counts.max() > 128 and 0 < counts.min() < LANE_MIN_EXL3
        ref_y, ref_ro = case.cpu_layer(x, ids, w, want_ro=True)
        ro = case.gpu_routed(x, ids)
        assert rel_l2(ro, ref_ro) < 1e-3
        assert rel_l2(case.gpu_experts(x, ids, w), ref_y) < TOL_LAYER
        assert case.status() == 0
    finally:
        case.close()
