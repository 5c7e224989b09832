"""GPU parity at the shapes the benchmark measures, through the C ABI.

  * the DeepSeek-V4.1-Flash-shaped decode layer (hidden 5120, inter 2304, 256 experts, top-8, shared expert) at
    1, 4, 16 and 64 tokens, normal and Zipf-skewed routing;
  * the tensor-core lanes at the real dims of the three banks (EXL3 5120 x 2304, MXFP4 4096 x 2048 with softmax routing
    over 256 experts, NVFP4 6144 x 2048), with experts on both tile shapes and in the streaming lane in one call;
  * the reference's own expert-forward fixture (src/arch/glm5_next/exl3_forms_ref.zig:365-450, seed 0x676C6D35)
    through mlxs_moe_routed, against the reference-held y_mul1.f32: no oracle in between;
  * the dispatch permutation read back from the device against the reference's known answer
    (src/sdk_ext/quant.zig:692-699) and the oracle's counting sort, bit-exact;
  * a bounded wait driven to its limit, the sticky status word and its acknowledgement;
  * an MXFP4 and an NVFP4 bank directory loaded onto the device.
"""
import json
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as O
from moe_cases import Exl3Case, Mxfp4Case, Nvfp4Case, max_err_over_rms, rel_l2, zipf_bias, LANE_MIN_EXL3

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
TOL_F32 = 1e-4
TOL_LAYER = 1e-2


# ---- the decode layer the benchmark times ----
@pytest.fixture(scope="module")
def c2():
    case = Exl3Case(5120, 2304, 256, 8, seed=0, shared=True, max_tokens=64)
    yield case
    case.close()


@pytest.mark.parametrize("routing", ["normal", "zipf"])
@pytest.mark.parametrize("T", [1, 4, 16, 64])
def test_decode_layer_256_experts_top8(c2, T, routing):
    x, logits = c2.inputs(T, seed=300 + T)
    if routing == "zipf":
        logits = logits + zipf_bias(c2.E, layer=0)
    ids, w = c2.gpu_route(logits)
    rid, rw = c2.cpu_route(logits)
    assert (ids == rid).all()
    assert (w.view(np.uint32) == rw.view(np.uint32)).all() or np.allclose(w, rw, rtol=1e-6)
    y = c2.gpu_forward(x, logits)
    assert c2.status() == 0
    # the oracle's f32 form over the touched experts (OpenMP); for the smallest batches also the f64 rows
    ref = O.layer_fast(c2.H, c2.I, c2.E, c2.k, c2.records, x, rid, rw, shared=c2.shared, limit=c2.limit)
    assert rel_l2(y, ref) < TOL_LAYER, rel_l2(y, ref)
    if T <= 4:
        ref_y, ref_ro = c2.cpu_layer(x, rid, rw, want_ro=True)
        ro = c2.gpu_routed(x, ids)
        assert max_err_over_rms(ro, ref_ro) < TOL_F32
        assert rel_l2(y, ref_y) < TOL_LAYER
    assert (c2.gpu_forward_host(x, logits) == y).all()
    assert (c2.gpu_forward(x, logits) == y).all()      # run-to-run determinism


# ---- tensor-core lanes at real dims ----
class _SharedRecords:
    """Mixin: only `distinct` different records are synthesised; expert e holds record e % distinct (the hot experts of
    the tests below are the first ones, so each of them has a record of its own)."""
    distinct = 12

    def synth(self, e):
        key = e % self.distinct
        cache = self.__dict__.setdefault("_synth_cache", {})
        if key not in cache:
            cache[key] = super().synth(key)
        return cache[key]


class _Exl3Shared(_SharedRecords, Exl3Case):
    pass


class _Mxfp4Shared(_SharedRecords, Mxfp4Case):
    pass


class _Nvfp4Shared(_SharedRecords, Nvfp4Case):
    pass


def _lane_mix(case, T, seed, boosts):
    """Logits with some experts boosted, [(experts, boost), ...]: +6 sends every token there (several row tiles), +1 to
    +2 a few dozen to a few hundred (one or two tiles), the rest keep a handful of rows (streaming lane)."""
    x, logits = case.inputs(T, seed=seed)
    for experts, boost in boosts:
        logits[:, experts] += boost
    return x, logits


def _check_sampled_rows(case, x, ids, w, ro, tol_max, tol_l2, sample):
    """The f64 oracle over a sample of the tokens: a routed row depends on its token and expert only."""
    ref_y, ref_ro = case.cpu_layer(x[sample], ids[sample], w[sample], want_ro=True)
    got = ro[sample]
    assert max_err_over_rms(got, ref_ro) < tol_max, max_err_over_rms(got, ref_ro)
    assert rel_l2(got, ref_ro) < tol_l2, rel_l2(got, ref_ro)
    return ref_y


def test_exl3_tensor_lane_at_real_dims():
    """hidden 5120 / inter 2304: K loops of 320 and 144 tiles, 18 and 40 column blocks, experts with two and more row
    tiles of 128 beside streaming-lane experts."""
    case = _Exl3Shared(5120, 2304, 16, 4, seed=3, shared=True, max_tokens=320)
    try:
        T = 300
        x, logits = _lane_mix(case, T, 41, [([0, 1], 6.0), ([2], 2.2), ([3], 0.9), ([4], 0.5), ([10, 13], -1.2)])
        ids, w = case.cpu_route(logits)
        counts = np.bincount(ids.reshape(-1), minlength=case.E)
        assert counts.max() > 256 and ((counts >= LANE_MIN_EXL3) & (counts <= 128)).any() and ((counts > 0) & (counts < LANE_MIN_EXL3)).any(), counts
        gid, gw = case.gpu_route(logits)
        assert (gid == ids).all()
        ro = case.gpu_routed(x, ids)
        assert case.status() == 0 and np.isfinite(ro).all()
        sample = np.r_[0:6, T - 6:T]
        _check_sampled_rows(case, x, ids, w, ro, 4e-3, 1e-3, sample)     # f16-rounded GEMM inputs, as the reference's prefill chain
        y = case.gpu_experts(x, ids, w)
        ref = O.layer_fast(case.H, case.I, case.E, case.k, case.records, x[sample], ids[sample], w[sample],
                           shared=case.shared, limit=case.limit)
        assert rel_l2(y[sample], ref) < TOL_LAYER
        again = case.gpu_routed(x, ids)
        assert (again.view(np.uint32) == ro.view(np.uint32)).all()
    finally:
        case.close()


def test_mxfp4_tensor_lane_at_real_dims_softmax_256_experts():
    """The MiMo-shaped configuration: hidden 4096 / inter 2048, 256 experts, top-8, softmax routing; experts on the
    192-row tile shape, on the 64-row shape and in the streaming lane in one call."""
    case = _Mxfp4Shared(4096, 2048, 256, 8, seed=5, shared=False, scoring=O.SCORE_SOFTMAX, max_tokens=512,
                        routed_scale=1.0, limit=0.0, chain=True)
    try:
        T = 512
        x, logits = _lane_mix(case, T, 43, [([0, 1, 2], 6.0), ([3, 4], 2.2), ([5, 6, 7, 8], 1.0)])
        ids, w = case.gpu_route(logits)
        rid, rw = case.cpu_route(logits)
        assert (ids == rid).all()
        counts = np.bincount(ids.reshape(-1), minlength=case.E)
        assert (counts > 64).any() and ((counts >= 17) & (counts <= 64)).any() and ((counts > 0) & (counts < 17)).any(), counts[:12]
        y = case.gpu_experts(x, ids, w)
        assert case.status() == 0 and np.isfinite(y).all()
        sample = np.r_[0:4, T - 4:T]
        ref = case.cpu_layer(x[sample], rid[sample], rw[sample])
        assert rel_l2(y[sample], ref) < TOL_LAYER, rel_l2(y[sample], ref)
        # the tensor-core lane against the streaming lane on the same rows (8 tokens at a time stay below 17 rows)
        ro = case.gpu_routed(x, ids)
        few = np.concatenate([case.gpu_routed(x[i:i + 2], ids[i:i + 2]) for i in (0, 2, T - 2)], axis=0)
        assert rel_l2(ro[np.r_[0:4, T - 2:T]], few) < 2e-3
        assert (case.gpu_experts(x, ids, w) == y).all()
    finally:
        case.close()


def test_nvfp4_tensor_lane_at_real_dims():
    """The GLM-shaped configuration: hidden 6144 / inter 2048, sigmoid routing, shared expert, both tile shapes."""
    case = _Nvfp4Shared(6144, 2048, 32, 8, seed=7, shared=True, scoring=O.SCORE_SIGMOID, max_tokens=256,
                        routed_scale=1.0, limit=10.0, chain=True)
    try:
        T = 256
        x, logits = _lane_mix(case, T, 47, [([0, 1], 6.0), ([2, 3, 4, 5], 2.2), (list(range(20, 32)), -1.3)])
        ids, w = case.gpu_route(logits)
        rid, rw = case.cpu_route(logits)
        assert (ids == rid).all()
        counts = np.bincount(ids.reshape(-1), minlength=case.E)
        assert (counts > 64).any() and ((counts >= 17) & (counts <= 64)).any() and ((counts > 0) & (counts < 17)).any(), counts
        y = case.gpu_experts(x, ids, w)
        assert case.status() == 0 and np.isfinite(y).all()
        sample = np.r_[0:4, T - 4:T]
        ref = case.cpu_layer(x[sample], rid[sample], rw[sample])
        assert rel_l2(y[sample], ref) < TOL_LAYER, rel_l2(y[sample], ref)
        assert (case.gpu_experts(x, ids, w) == y).all()
    finally:
        case.close()


# ---- the dense bf16 products (shared expert, router logits) on the tensor cores ----
def _shared_ref(x, ws, limit):
    """f64 shared expert (src/arch/deepseek_v41/graph.zig:2162-2172): clamped SwiGLU, h rounded to bf16, down."""
    w1, w3, w2 = [O.bf16_bits_to_f32(w).astype(np.float64) for w in ws]
    g = x.astype(np.float64) @ w1.T
    u = x.astype(np.float64) @ w3.T
    if limit > 0:
        g = np.minimum(g, limit)
        u = np.clip(u, -limit, limit)
    h = g / (1.0 + np.exp(-g)) * u
    h = O.bf16_bits_to_f32(O.f32_to_bf16_bits(h.astype(np.float32))).astype(np.float64)
    return h @ w2.T


@pytest.mark.parametrize("H,I", [(5120, 2304), (6144, 2048)])
def test_shared_expert_alone_at_every_batch_size(H, I):
    """Routed weights of zero leave y = bf16(shared expert): the skinny streaming kernel up to 64 tokens, the tcgen05
    products above (one and several token tiles, a ragged last tile), all against the f64 product."""
    case = Exl3Case(H, I, 2, 1, seed=11, shared=True, max_tokens=600)
    try:
        for T in (1, 8, 64, 65, 256, 300, 600):
            x, _ = case.inputs(T, seed=900 + T)
            ids = np.zeros((T, 1), np.int32)
            w = np.zeros((T, 1), np.float32)
            y = case.gpu_experts(x, ids, w)
            ref = _shared_ref(x, case.shared, case.limit)
            assert case.status() == 0
            assert rel_l2(y, ref) < 4e-3, (T, rel_l2(y, ref))       # one bf16 rounding of the output: 2^-9 relative
            assert (case.gpu_experts(x, ids, w) == y).all()
            if T == 300:
                # the ragged last tile (44 rows) against the same rows through the skinny kernel: two f32 sum orders, so
                # an intermediate h may round to the neighbouring bf16 and move its row by a few 1e-4
                part = case.gpu_experts(x[256:300], ids[256:300], w[256:300])
                assert rel_l2(part, y[256:300]) < 2e-3, rel_l2(part, y[256:300])
    finally:
        case.close()


def test_router_logits_on_the_tensor_cores():
    """logits = f32(x) . W_g^T (src/arch/deepseek_v41/graph.zig:2033) for 256 experts above 64 tokens: the tcgen05
    product against the f64 product, and the layer from x equal to the layer from those logits."""
    import torch
    case = Exl3Case(5120, 2304, 256, 8, seed=2, shared=False, max_tokens=600, experts_to_load=[])
    try:
        rng = np.random.default_rng(5)
        wg = O.f32_to_bf16_bits((rng.standard_normal((256, 5120)) * 0.05).astype(np.float32))
        case.moe.set_router_weight(0, wg.ctypes.data)
        wf = O.bf16_bits_to_f32(wg).astype(np.float64)
        for T in (64, 65, 300, 600):
            x, _ = case.inputs(T, seed=70 + T)
            ref = x.astype(np.float64) @ wf.T
            xd = case.to_dev_bf16(x)
            lg = torch.full((T, 256), float("nan"), dtype=torch.float32, device=case.dev)
            case.moe.logits(0, xd.data_ptr(), T, lg.data_ptr(), None)
            torch.cuda.synchronize()
            got = lg.cpu().numpy()
            assert np.allclose(got, ref, rtol=2e-5, atol=1e-4), (T, np.abs(got - ref).max())
            ids, w = case.gpu_route(got)
            rid, rw = case.cpu_route(got)
            assert (ids == rid).all()
        assert case.status() == 0
    finally:
        case.close()


# ---- the reference's own fixture, no oracle in between ----
def test_reference_expert_forward_fixture_on_the_gpu():
    """src/arch/glm5_next/exl3_forms_ref.zig:365-450: the fixture expert (seed 0x676C6D35, hidden 4096, inter 2048,
    scales f16(+-(0.5+u) x {1, 0.01})) on the fixture's row; the routed row against the reference-held y_mul1.f32 at the
    reference's own tolerance for an f32 chain, max |err| / rms < 1e-4."""
    meta = json.loads((GOLD / "exl3-ref" / "meta.json").read_text())
    seed, H, I = meta["seed"], meta["hidden"], meta["inter"]
    assert seed == 0x676C6D35
    case = Exl3Case(H, I, 2, 1, seed=0, shared=False, max_tokens=64, experts_to_load=[], limit=10.0)
    try:
        rec = O.exl3_synth_record(seed, H, I, 1.0, 0.01)
        case.moe.load_expert(0, 1, rec.ctypes.data, rec.size)
        x = O.fill_x_bf16(seed + 10, H).reshape(1, H)
        want = np.fromfile(GOLD / "exl3-ref" / "y_mul1.f32", "<f4").astype(np.float64)
        got = case.gpu_routed(x, np.array([[1]], np.int32))[0, 0]
        assert case.status() == 0
        assert max_err_over_rms(got, want) < 1e-4, max_err_over_rms(got, want)
        # the same row inside a batch of 40 copies takes the tensor-core lane (f16-rounded GEMM inputs): the reference's
        # bar for that chain is the prefill parity bar
        xs = np.repeat(x, 40, axis=0)
        many = case.gpu_routed(xs, np.full((40, 1), 1, np.int32))
        assert max_err_over_rms(many[7, 0], want) < 4e-3
        assert (many[0, 0].view(np.uint32) == many[39, 0].view(np.uint32)).all()
    finally:
        case.close()


# ---- dispatch tables, bit-exact ----
def test_dispatch_permutation_read_back():
    import torch
    case = Exl3Case(512, 256, 256, 8, seed=1, shared=False, max_tokens=512, experts_to_load=[])
    try:
        def gpu_sort(slot, n_slots):
            d = torch.from_numpy(np.ascontiguousarray(slot, np.int32)).to(case.dev)
            order = torch.full((max(len(slot), 1),), 0x7FFFFFFF, dtype=torch.int32, device=case.dev)
            offs = torch.full((n_slots + 1,), 0x7FFFFFFF, dtype=torch.int32, device=case.dev)
            case.moe.sort_rows(d.data_ptr(), len(slot), n_slots, order.data_ptr(), offs.data_ptr(), None)
            torch.cuda.synchronize()
            return order.cpu().numpy()[:len(slot)].astype(np.uint32), offs.cpu().numpy().astype(np.uint32)

        # src/sdk_ext/quant.zig:692-699: slots {3,1,3,0,1} -> order {3,1,4,0,2}
        order, offs = gpu_sort([3, 1, 3, 0, 1], 4)
        assert order.tolist() == [3, 1, 4, 0, 2] and offs.tolist() == [0, 1, 3, 3, 5]
        rng = np.random.default_rng(8)
        for n, n_slots in ((1, 1), (37, 16), (2048, 256), (3000, 256), (4096, 7)):
            slot = rng.integers(0, n_slots, n).astype(np.int32)
            if n == 3000:
                slot[::3] = 5                      # one heavy slot among ragged ones, some slots empty
                slot[slot == 9] = 10
            order, offs = gpu_sort(slot, n_slots)
            ref_order, sorted_slot, inv, ref_offs = O.dispatch(slot, n_slots)
            assert (order == ref_order).all(), n
            assert (offs == ref_offs).all(), n
            assert (order == np.argsort(slot, kind="stable")).all()
        assert case.status() == 0
    finally:
        case.close()


# ---- bounded waits, the status word ----
def test_a_bounded_wait_runs_out_and_the_handle_recovers():
    """One ring stage of the gate/up stream is withheld with a poll limit of a few hundred: the consumers' wait runs
    out, the CTAs record the status word and return, the call completes, and after the host has acknowledged the
    word the same handle computes the same bits as before."""
    case = Exl3Case(512, 256, 8, 2, seed=4, shared=True, max_tokens=64)
    try:
        x, logits = case.inputs(9, seed=2)
        good = case.gpu_forward(x, logits)
        assert case.status() == 0
        case.moe.debug_wait(poll_limit=300, withhold_stage=1)
        case.gpu_forward(x, logits)                     # completes: nothing hangs, nothing faults
        assert case.status() in (2, 3)                  # ST_WAIT_FULL / ST_WAIT_EMPTY
        case.moe.debug_wait(0, 0)
        with pytest.raises(case.pkg.MlxsError) as ei:   # the word is sticky until acknowledged
            case.gpu_forward_host(x, logits)
        assert ei.value.rc == case.pkg.E_DEVICE_STATUS and "bounded wait" in ei.value.msg
        case.moe.status_clear()
        assert case.status() == 0
        assert (case.gpu_forward_host(x, logits) == good).all()
        assert (case.gpu_forward(x[:1], logits[:1]) == good[:1]).all()   # the K-split path (one token) too
        assert case.status() == 0
        with pytest.raises(case.pkg.MlxsError):
            case.moe.debug_wait(0, 3)                   # a withheld stage needs a short limit
    finally:
        case.close()


def test_misaligned_buffers_are_refused_by_name():
    import torch
    case = Exl3Case(512, 256, 8, 2, seed=4, shared=False, max_tokens=8)
    try:
        x = torch.zeros(4 * 512 + 8, dtype=torch.bfloat16, device=case.dev)
        lg = torch.zeros(4 * 8 + 8, dtype=torch.float32, device=case.dev)
        y = torch.zeros(4 * 512 + 8, dtype=torch.bfloat16, device=case.dev)
        with pytest.raises(case.pkg.MlxsError) as ei:
            case.moe.forward(0, x.data_ptr() + 2, lg.data_ptr(), 4, y.data_ptr(), None)
        assert ei.value.rc == case.pkg.E_ARG and "x_dev" in ei.value.msg
        with pytest.raises(case.pkg.MlxsError) as ei:
            case.moe.forward(0, x.data_ptr(), lg.data_ptr(), 4, y.data_ptr() + 4, None)
        assert "y_dev" in ei.value.msg
        case.moe.forward(0, x.data_ptr() + 16, lg.data_ptr() + 4, 4, y.data_ptr() + 16, None)
        torch.cuda.synchronize()
        assert case.status() == 0
    finally:
        case.close()


# ---- FP4 bank directories onto the device ----
@pytest.mark.parametrize("cls,nv", [(Mxfp4Case, False), (Nvfp4Case, True)])
def test_fp4_load_bank_from_reference_format_files(tmp_path, cls, nv):
    """src/arch/mimo_v2/bank.zig:172-260, src/arch/glm5_next/bank.zig:29-48: experts.bin + expert-manifest.json in the
    reference's format, digests verified, the layer equal bit for bit to the one loaded record by record."""
    import bank_files
    H, I, E, k = 512, 256, 4, 2
    kw = dict(seed=23, shared=False, scoring=O.SCORE_SIGMOID, max_tokens=16, routed_scale=1.0, limit=10.0 if nv else 0.0, chain=True)
    a = cls(H, I, E, k, **kw)
    b = cls(H, I, E, k, experts_to_load=[], **kw)
    try:
        bank_files.write_fp4_bank(tmp_path, H, I, E, 1, nv, lambda l, e: a.records[e])
        b.moe.load_bank(tmp_path)
        x, logits = a.inputs(9, seed=3)
        assert (a.gpu_forward(x, logits) == b.gpu_forward(x, logits)).all()
        assert b.status() == 0
        raw = bytearray((tmp_path / "experts.bin").read_bytes())
        raw[7000] ^= 1
        (tmp_path / "experts.bin").write_bytes(bytes(raw))
        with pytest.raises(b.pkg.MlxsError) as ei:
            b.moe.load_bank(tmp_path)
        assert "sha256" in ei.value.msg.lower() or "digest" in ei.value.msg.lower()
    finally:
        a.close()
        b.close()
