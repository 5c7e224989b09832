"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and refuses by name."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from __graft_entry__ import ROOT, load_package


def header_symbols():
    text = (ROOT / "include" / "mlxs_moe.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mlxs_moe_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    pkg = load_package()
    L = pkg.lib()
    syms = header_symbols()
    assert len(syms) >= 15
    for s in syms:
        assert hasattr(L, s), s
    assert sorted(pkg.EXPORTS) == syms
    assert L.mlxs_moe_abi() == pkg.ABI
    text = (ROOT / "include" / "mlxs_moe.h").read_text()
    assert f"#define MLXS_MOE_ABI {pkg.ABI}" in text


def test_config_struct_matches_header_layout():
    pkg = load_package()
    assert C.sizeof(pkg.Config) == 18 * 4
    assert C.sizeof(pkg.Stats) == 9 * 8 + 8


def test_create_refuses_by_name():
    pkg = load_package()
    bad = [
        (dict(hidden=5000), "hidden"), (dict(inter=100), "inter"), (dict(n_experts=0), "n_experts"),
        (dict(top_k=0), "top_k"), (dict(top_k=99), "top_k"), (dict(bank_kind=7), "bank_kind"), (dict(act=5), "act"),
        (dict(act_limit=0.0), "act_limit"), (dict(scoring=9), "scoring"), (dict(combine=3), "combine"),
        (dict(max_tokens=0), "max_tokens"), (dict(ep_world=3), "ep_world"), (dict(combine=1), "combine"),
    ]
    for kw, name in bad:
        base = dict(hidden=512, inter=256, n_experts=8, top_k=2)
        base.update(kw)
        with pytest.raises(pkg.MlxsError) as ei:
            pkg.MoE(pkg.make_config(**base))
        assert ei.value.rc == -2 and name in ei.value.msg, (kw, ei.value.msg)
    cfg = pkg.make_config(512, 256, 8, 2)
    cfg.struct_size = 12
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.MoE(cfg)
    assert "struct_size" in ei.value.msg


def test_measurement_entries_refuse_bad_arguments_by_name():
    """The probes check their arguments before they touch a device."""
    pkg = load_package()
    for n in (0, 8, 100, 272):
        with pytest.raises(pkg.MlxsError) as ei:
            pkg.mma_rate(0, n, False, 10)
        assert ei.value.rc == -1 and "multiple of 16" in ei.value.msg, ei.value.msg   # MLXS_E_ARG
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.mma_rate(0, 128, False, 0)
    assert ei.value.rc == -1


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    pkg = load_package()
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.MoE(pkg.make_config(512, 256, 8, 2))
    assert ei.value.rc == -3 and "no CPU path" in ei.value.msg


def test_ep_plan_counts():
    pkg = load_package()
    ids = np.array([0, 5, 7, 2, 3, 6, 1, 4, 7, 7], np.int32)
    out = np.zeros(4, np.uint64)
    rc = pkg.lib().mlxs_moe_ep_plan(ids.ctypes.data, ids.size, 8, 4, out.ctypes.data)
    assert rc == 0 and out.tolist() == [2, 2, 2, 4]
    bad = np.array([9], np.int32)
    assert pkg.lib().mlxs_moe_ep_plan(bad.ctypes.data, 1, 8, 4, out.ctypes.data) == -1
    assert "outside" in pkg.last_error()


def test_ep_capacity_refusal_is_the_same_on_every_rank():
    """The NCCL transport's capacity check is a pure function of the gathered count matrix, so every rank reaches the
    same verdict before any send or receive is queued; the peer-store transport's window size is pure arithmetic."""
    pkg = load_package()
    L = pkg.lib()
    W = 4
    counts = np.zeros((W, W), np.int32)
    counts[:, 2] = [300, 200, 100, 500]          # everyone sends most rows to rank 2
    counts[:, 0] = 10
    flat = np.ascontiguousarray(counts)
    assert L.mlxs_moe_ep_overloaded_rank(flat.ctypes.data, W, 1, 1100) == -1
    assert L.mlxs_moe_ep_overloaded_rank(flat.ctypes.data, W, 1, 1099) == 2
    assert L.mlxs_moe_ep_overloaded_rank(flat.ctypes.data, W, 1, 39) == 0     # the lowest overloaded rank
    # the deduplicated form carries two counts per pair: stride 2 reads the assignments
    two = np.zeros((W, W, 2), np.int32)
    two[..., 0] = counts
    two[..., 1] = 1
    assert L.mlxs_moe_ep_overloaded_rank(two.ctypes.data, W, 2, 1099) == 2
    neg = flat.copy(); neg[1, 3] = -5
    assert L.mlxs_moe_ep_overloaded_rank(neg.ctypes.data, W, 1, 10**9) == 3   # a corrupt count overloads its destination
    # every rank evaluates the same matrix: the verdict does not depend on who asks (no rank argument at all)
    b = L.mlxs_moe_ep_window_bytes(8, 64, 8, 256, 5120)
    assert b >= 8 * 64 * 5120 * 6 and b < 8 * 64 * 5120 * 6 + 2 * 1024 * 1024
    assert L.mlxs_moe_ep_window_bytes(3, 64, 8, 256, 5120) == 0              # 256 experts do not shard over 3 ranks


def test_plan_placement_deals_by_use():
    """Most used first (ties to the lower id, as Profile.order, src/sdk_ext/expert/usage.zig:352-366), dealt to the
    ranks in snake order: every rank gets n_experts / world experts and the ranks' loads come out close."""
    import numpy as np
    pkg = load_package()
    assert pkg.plan_placement([5, 9, 9, 1, 0, 7, 3, 3], 2) == [0, 0, 1, 1, 0, 1, 0, 1]
    #   order: 1 2 5 0 6 7 3 4 -> ranks 0 1 1 0 0 1 1 0
    rng = np.random.default_rng(3)
    for E, W in ((384, 8), (256, 4), (16, 16)):
        counts = (1e4 * (1.0 + np.arange(E)) ** -1.1).astype(np.int64)[rng.permutation(E)]
        place = np.asarray(pkg.plan_placement(counts, W))
        assert all((place == r).sum() == E // W for r in range(W))
        loads = np.array([counts[place == r].sum() for r in range(W)])
        blocks = np.array([counts[r * (E // W):(r + 1) * (E // W)].sum() for r in range(W)])
        assert loads.max() - loads.min() <= counts.max()
        assert E == W or loads.max() <= blocks.max()
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.plan_placement([1, 2, 3], 2)
    assert "do not shard" in ei.value.msg


def test_zig_binding_declares_every_header_entry():
    """The Zig host file is shipped as source (no Zig compiler in the build image): at least keep it complete."""
    import re
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    header = (root / "include" / "mlxs_moe.h").read_text()
    zig = (root / "mlx-stream_b200" / "zig" / "mlxs_moe.zig").read_text()
    declared = set(re.findall(r"\b(mlxs_moe_[a-z0-9_]+)\s*\(", header))
    bound = set(re.findall(r"pub extern fn (mlxs_moe_[a-z0-9_]+)\(", zig))
    assert declared - bound == set(), declared - bound
    abi = re.search(r"#define MLXS_MOE_ABI (\d+)", header).group(1)
    assert f"abi_expected: i32 = {abi}" in zig
