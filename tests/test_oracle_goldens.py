"""The oracle against the reference's own golden vectors (copied by tests/golden/make_golden.py)."""
import ctypes as C
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as O

GOLD = Path(__file__).resolve().parent / "golden"
DIG = json.loads((GOLD / "exl3_digests.json").read_text())


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_mul1_table_digest():
    # src/kernels/exl3/manifest.json golden.mul1_table; src/exl3/kernels.zig:1544-1547
    assert sha(O.mul1_table()) == DIG["mul1_table_sha256"]


@pytest.mark.parametrize("name", ["gate_up", "down", "gate_up_k2", "down_k2"])
def test_seeded_planes(name):
    # src/exl3/kernels.zig:1548-1563: code, W_hat, the one-hot rows and their state coverage
    p = DIG["planes"][name]
    n_in, n_out = p["projection"]
    K = p["K"]
    code = O.fill_code(p["seed"], (n_in // 16) * (n_out // 16) * 16 * K)
    assert sha(code) == p["code_sha256"]
    w, st = O.reconstruct(code, n_in // 16, n_out // 16, K, want_states=True)
    assert sha(w) == p["w_hat_sha256"]
    rows = p["onehot_rows"]
    assert sha(w[:rows]) == p["onehot_rows_sha256"]
    assert np.unique(st[:rows]).size == p["states_covered_by_onehot_rows"] == 65536


@pytest.mark.parametrize("i", [0, 1])
def test_glm_planes(i):
    # src/arch/glm5_next/exl3_parity.zig:19-23
    p = DIG["glm_planes"][i]
    n_in, n_out = p["projection"]
    code = O.fill_code(p["seed"], (n_in // 16) * (n_out // 16) * 48)
    assert sha(code) == p["code_sha256"]
    assert sha(O.reconstruct(code, n_in // 16, n_out // 16, 3)) == p["w_hat_sha256"]


def test_bitstream_definition_and_tile_perm():
    # src/exl3/kernels.zig:1576-1624: every state read bit by bit from the circular MSB-first stream, K = 1..3
    perm = np.empty(256, np.uint8)
    O.lib().orc_tile_perm(perm.ctypes.data_as(C.c_void_p))
    assert sorted(perm.tolist()) == list(range(256))
    rng = np.random.default_rng(0xE3C0DE)
    table = O.mul1_table()
    for K in (1, 2, 3):
        n_i, n_j, tw = 2, 3, 16 * K
        code = rng.integers(0, 65536, n_i * n_j * tw, dtype=np.uint16).view(np.int16)
        w, st = O.reconstruct(code, n_i, n_j, K, table, want_states=True)
        u16 = code.view(np.uint16)
        for ti in range(n_i):
            for tj in range(n_j):
                tile = u16[(ti * n_j + tj) * tw:][:tw]
                bits = 256 * K
                for p in range(256):
                    s = 0
                    for i in range(16):
                        b = ((p + 1) * K + bits - 16 + i) % bits
                        word = int(tile[2 * (b // 32)]) | (int(tile[2 * (b // 32) + 1]) << 16)
                        s = (s << 1) | ((word >> (31 - b % 32)) & 1)
                    pos = int(perm[p])
                    r, c = ti * 16 + pos // 16, tj * 16 + pos % 16
                    assert st[r, c] == s and w[r, c] == table[s]
    # the codebook at its ends
    k_inv = np.array([0x1EEE], np.uint16).view(np.float16)[0]
    k_bias = np.array([0xC931], np.uint16).view(np.float16)[0]
    assert table[0] == np.float16(1024.0 * float(k_inv) + float(k_bias)).view(np.uint16)
    assert np.isfinite(table[0xFFFF:].view(np.float16)[0])


def test_record_geometry():
    # src/arch/glm5_next/exl3_forms_ref.zig:349-357 (GLM-Flash record); src/sdk_ext/expert.zig:339 (DSV41)
    g = O.exl3_geometry(4096, 2048)
    assert g.record_bytes == 9_474_048 and g.record_bytes % 4096 == 0
    want = [(0, 3_145_728), (3_145_728, 4_096), (3_149_824, 8_192), (3_158_016, 3_145_728), (6_303_744, 4_096),
            (6_307_840, 8_192), (6_316_032, 3_145_728), (9_461_760, 8_192), (9_469_952, 4_096)]
    assert [(g.off[i], g.len[i]) for i in range(9)] == want
    d = O.exl3_geometry(5120, 2304)
    assert d.logical_bytes == 13_315_584 and d.record_bytes == 13_316_096 and d.off[6] == 8_877_056
    # src/arch/mimo_v2/bank.zig:341-345
    n, off = O.mxfp4_record_bytes(4096, 2048)
    assert n == 13_369_344 and off[4] == 8_912_896
    n, _ = O.nvfp4_record_bytes(6144, 2048)
    assert n == 21_233_676
    n, _ = O.nvfp4_record_bytes(4096, 2048)
    assert n == 14_155_788


def test_expert_forward_fixture():
    # src/arch/glm5_next/exl3_forms_ref.zig:365-402: W_hat digests, h and y of the fixture expert (seed 0x676C6D35)
    meta = json.loads((GOLD / "exl3-ref" / "meta.json").read_text())
    seed = 0x676C6D35
    assert meta["seed"] == seed
    H, I = meta["hidden"], meta["inter"]
    rec = O.exl3_synth_record(seed, H, I, 1.0, 0.01)
    g = O.exl3_geometry(H, I)
    for p, proj in enumerate(meta["proj"]):
        code = rec[g.off[3 * p]:g.off[3 * p] + g.len[3 * p]].view(np.int16)
        n_in, n_out = proj["in"], proj["out"]
        assert sha(O.reconstruct(code, n_in // 16, n_out // 16, 3)) == proj["w_hat_sha256_mul1"]
    x = O.fill_x_bf16(seed + 10, H)
    h, y = O.exl3_expert_f64(rec, H, I, x, 10.0)
    rh = np.fromfile(GOLD / "exl3-ref" / "h_mul1.f32", "<f4").astype(np.float64)
    ry = np.fromfile(GOLD / "exl3-ref" / "y_mul1.f32", "<f4").astype(np.float64)

    def max_err_over_rms(got, ref):
        return np.abs(got - ref).max() / (np.sqrt((ref * ref).mean()) + 1e-30)

    assert max_err_over_rms(h[0], rh) < 1e-6
    assert max_err_over_rms(y[0], ry) < 1e-6
    # exl3_forms_ref.zig:404-450: the f32 seam chain meets 1e-4 of the f64 truth
    hc, yc = O.exl3_expert_f32chain(rec, H, I, x)
    assert max_err_over_rms(hc[0].astype(np.float64), h[0]) < 1e-4
    assert max_err_over_rms(yc[0].astype(np.float64), y[0]) < 1e-4


def test_swiglu_clamp_literals():
    # src/exl3/quant.zig:1547-1555: the clamp literals are +-10.0 (0x41200000 / 0xC1200000)
    assert np.float32(10.0).view(np.uint32) == 0x41200000 and np.float32(-10.0).view(np.uint32) == 0xC1200000
    L = O.lib()
    assert L.orc_swiglu_clamped(20.0, 30.0, 10.0) == pytest.approx(10.0 / (1 + np.exp(-10.0)) * 10.0)
    assert L.orc_swiglu_clamped(-3.0, -30.0, 10.0) == pytest.approx(-3.0 / (1 + np.exp(3.0)) * -10.0)
    assert np.isnan(L.orc_swiglu_clamped(float("nan"), 1.0, 10.0))


def test_nvfp4_known_answers():
    # src/arch/glm5_next/decode_kernels_ref.zig:170-218
    L = O.lib()
    for b in range(256):
        got, want = L.orc_e4m3_kernel(b), L.orc_e4m3_value(b)
        if np.isnan(want):
            assert np.isnan(got)
        else:
            assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)
    assert L.orc_e4m3_kernel(0x7E) == 448.0 and L.orc_e4m3_kernel(0x01) == 2.0 ** -9
    assert np.float32(L.orc_e4m3_kernel(0x80)).view(np.uint32) == 0x80000000
    for c in range(16):
        hb = np.array([L.orc_e2m1_halfbits(c)], np.uint16).view(np.float16)[0]
        assert np.float32(L.orc_e2m1_value(c)).view(np.uint32) == np.float32(np.float32(hb) * 16384.0).view(np.uint32)
    state = 0x67356E6E
    out = (C.c_uint32 * 4)()
    for pos in range(8):
        for c in range(16):
            state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
            w = (state & ~(0xF << (4 * pos)) & 0xFFFFFFFF) | (c << (4 * pos))
            L.orc_fp4_decode8(C.c_uint32(w), out)
            half = (out[pos] & 0xFFFF) if pos < 4 else (out[pos - 4] >> 16)
            assert half == L.orc_e2m1_halfbits(c)
    fixed = [0x3E200000, 0x3DF00000, 0x3DE00000, 0x3E000000, 0x3E900000, 0x3DC00000, 0x41200000, 0x3F800000]
    gs = [np.array([h], np.uint32).view(np.float32)[0] for h in fixed]
    gs += [np.float32(0.09375) * np.float32(1.36) ** np.float32(i) for i in range(16)]
    n = 0
    for g in gs:
        for b in range(256):
            if b & 0x7F == 0x7F:
                continue
            for c in range(16):
                got = L.orc_nvfp4_kernel_weight(b, c, C.c_float(g))
                want = L.orc_nvfp4_weight(b, c, C.c_float(g))
                assert np.float32(got).view(np.uint32) == np.float32(want).view(np.uint32)
                n += 1
    assert n == 24 * 254 * 16


def test_mxfp4_known_answers():
    # src/arch/mimo_v2/moe.zig:1059-1064 and :408-413
    L = O.lib()
    assert L.orc_silu_mul_ref(0.01171875, 1.0) == 0.005889892578125
    assert L.orc_mxfp4_scale_ref(127) == 2.0 ** -8 and L.orc_mxfp4_scale_ref(128) == 2.0 ** -7
    assert L.orc_mxfp4_scale_ref(0) == 0.0  # 2^-127 x 2^-8 flushes
    assert L.orc_e8m0_value(127) == 1.0 and L.orc_e8m0_value(120) == 2.0 ** -7
    # dequantised weight = e2m1 x 2^(b - 127)
    words = np.array([0x76543210, 0xFEDCBA98, 0, 0], np.uint32)
    scales = np.array([126], np.uint8)
    out = np.empty(32, np.float32)
    L.orc_mxfp4_decode(words.ctypes.data_as(C.c_void_p), scales.ctypes.data_as(C.c_void_p), 1, 32,
                       out.ctypes.data_as(C.c_void_p))
    mags = [0, 0.5, 1, 1.5, 2, 3, 4, 6]
    assert out[:16].tolist() == [m * 0.5 for m in mags] + [-m * 0.5 for m in mags]


def test_router_known_answer():
    # src/arch/mimo_v2/config.zig:503-514
    logits = np.array([[0, 2, -2, 1]], np.float32)
    bias = np.array([0, 0, 10, 0], np.float32)
    for det in (False, True):
        ids, w = O.route(logits, bias, 2, O.SCORE_SIGMOID, det=det)
        assert ids.tolist() == [[2, 1]]
        low, high = 1 / (1 + np.exp(np.float32(2))), 1 / (1 + np.exp(np.float32(-2)))
        assert abs(w[0, 0] - low / (low + high)) < 1e-7 and abs(w[0].sum() - 1) < 1e-7


@pytest.mark.parametrize("scoring", [O.SCORE_SQRTSOFTPLUS, O.SCORE_SIGMOID, O.SCORE_SOFTMAX])
def test_router_fixed_sequence_math_matches_libm(scoring):
    rng = np.random.default_rng(7 + scoring)
    logits = rng.standard_normal((512, 256)).astype(np.float32)
    bias = (rng.standard_normal(256) * 0.1).astype(np.float32)
    scale = 1.5 if scoring == O.SCORE_SQRTSOFTPLUS else 1.0
    a, wa = O.route(logits, bias, 8, scoring, scale=scale, det=False)
    b, wb = O.route(logits, bias, 8, scoring, scale=scale, det=True)
    assert (a == b).mean() > 0.999  # last-place differences can only swap near-ties
    np.testing.assert_allclose(wa[a == b], wb[a == b], rtol=2e-6)
    L = O.lib()
    xs = np.concatenate([np.linspace(-100, 88, 4001), rng.standard_normal(2000) * 3]).astype(np.float32)
    got = np.array([L.orc_det_expf(float(v)) for v in xs], np.float64)
    want = np.exp(xs.astype(np.float64))
    ok = want > 1e-37
    assert np.abs(got[ok] / want[ok] - 1).max() < 3e-7
    xl = np.linspace(1.0, 2.0, 3001).astype(np.float32)
    gl = np.array([L.orc_det_logf(float(v)) for v in xl], np.float64)
    assert np.abs(gl - np.log(xl.astype(np.float64))).max() < 2e-7


def test_router_ties_nan_and_order():
    # ties go to the lower index, NaN ranks last (q3rc_router_tail.metal:17-26)
    logits = np.array([[1, 1, 1, 1], [np.nan, 0, 3, 3], [np.nan, np.nan, np.nan, 5]], np.float32)
    ids, _ = O.route(logits, None, 3, O.SCORE_SIGMOID)
    assert ids.tolist() == [[0, 1, 2], [2, 3, 1], [3, 0, 1]]


def test_dispatch_known_answer():
    # src/sdk_ext/quant.zig:692-699
    order, sorted_slot, inv, offs = O.dispatch([3, 1, 3, 0, 1], 4)
    assert order.tolist() == [3, 1, 4, 0, 2] and sorted_slot.tolist() == [0, 1, 1, 3, 3]
    assert all(inv[o] == i for i, o in enumerate(order))
    assert offs.tolist() == [0, 1, 3, 3, 5]
    rng = np.random.default_rng(1)
    slot = rng.integers(0, 37, 5000)
    order, sorted_slot, inv, offs = O.dispatch(slot, 37)
    assert (order == np.argsort(slot, kind="stable")).all()


def test_k2_expert_forward_uses_the_k2_planes():
    """The oracle's expert forward at K = 2 multiplies by exactly the planes `reconstruct` gives at K = 2 (whose digests
    are pinned above): a dense f64 restatement over those planes gives the same row."""
    H, I = 256, 128
    rec = O.exl3_synth_record(0x1234, H, I, 1.0, 0.02, K=2)
    g = O.exl3_geometry(H, I, 2)
    assert g.len[0] == (H // 16) * (I // 16) * 64          # 16 K int16 per tile
    rng = np.random.default_rng(4)
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal((1, H)).astype(np.float32)))
    ids = np.zeros((1, 1), np.int32)
    w = np.ones((1, 1), np.float32)
    y = O.layer(O.BANK_EXL3_K2, H, I, 1, 1, {0: rec}, x, ids, w, limit=10.0)

    def f16(seg, n):
        return rec[g.off[seg]:g.off[seg] + 2 * n].view(np.float16).astype(np.float64)

    def plane(seg, n_in, n_out):
        code = rec[g.off[seg]:g.off[seg] + g.len[seg]].view(np.int16)
        return O.reconstruct(code, n_in // 16, n_out // 16, 2).view(np.float16).astype(np.float64).reshape(n_in, n_out)

    def had(v):
        v = v.reshape(-1, 128).copy()
        h = 1
        while h < 128:
            v = v.reshape(-1, 128 // (2 * h), 2, h)
            a, b = v[:, :, 0, :].copy(), v[:, :, 1, :].copy()
            v[:, :, 0, :], v[:, :, 1, :] = a + b, a - b
            v = v.reshape(-1, 128)
            h *= 2
        return (v / np.sqrt(128.0)).reshape(-1)

    def proj(v, seg, n_in, n_out):
        return had(had(v * f16(seg + 2, n_in)) @ plane(seg, n_in, n_out)) * f16(seg + 1, n_out)

    xv = x[0].astype(np.float64)
    gate, up = proj(xv, 0, H, I), proj(xv, 3, H, I)
    gate = np.minimum(gate, 10.0)
    up = np.clip(up, -10.0, 10.0)
    hmid = gate / (1.0 + np.exp(-gate)) * up
    ref = proj(hmid, 6, I, H)
    assert np.abs(y[0] - ref).max() / (np.sqrt((ref * ref).mean()) + 1e-30) < 1e-9
