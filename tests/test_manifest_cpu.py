"""The manifest reader on the CPU: the reference's v2 sample and its twelve mutations (src/exl3/quant.zig:1395-1421),
the FP4 bank manifests (src/arch/mimo_v2/bank.zig:417-..., src/arch/glm5_next/bank.zig:511-580), refusals by name."""
import json
from pathlib import Path

import pytest

import bank_files
from __graft_entry__ import load_package

GOLD = Path(__file__).resolve().parent / "golden"


def test_v2_sample_of_the_bank_of_record():
    pkg = load_package()
    text = (GOLD / "dsv41_bank_peek.json").read_text()
    info = pkg.bank_peek(text=text)
    assert (info.bank_kind, info.hidden, info.inter, info.n_experts, info.n_layers) == (0, 5120, 2304, 384, 40)
    assert info.logical_bytes == 13_315_584 and info.record_stride == 13_316_096
    assert info.data_bytes == 40 * 384 * 13_316_096


def test_v2_mutations_are_refused_by_name():
    pkg = load_package()
    text = (GOLD / "dsv41_bank_peek.json").read_text()
    cases = [
        ('"mode":"exl3"', '"mode":"exl2"', 'quantization.mode "exl2"'),
        ('"codebook":"mul1"', '"codebook":"3inst"', 'quantization.codebook "3inst"'),
        ('"codebook_multiplier":2212286765', '"codebook_multiplier":2212286766', "codebook_multiplier 2212286766"),
        ('"layout":"exl3-tensor-core"', '"layout":"row-major"', "quantization.tile 16 / row-major"),
        ('"layer":7,"K":3', '"layer":7,"K":4', "layer 7 K 4"),
        ('"hidden":5120', '"hidden":4096', "segment gate_proj.code: its shape"),
        ('"component":"up_proj.rout","dtype":"F16"', '"component":"up_proj.rout","dtype":"F32"', "segment up_proj.rout: its dtype"),
        ('"order":"sylvester-natural"', '"order":"walsh"', "quantization.hadamard 128 / walsh"),
        ('"rin":"exl3.suh"', '"rin":"exl3.sv"', "quantization.scales rin exl3.sv"),
        ('"component":"gate_proj.rout"', '"component":"gate_prj.rout"', "segment gate_prj.rout: an unknown projection"),
        ('"component":"down_proj.rin"', '"component":"down_proj.bias"', "segment down_proj.bias: an unknown tensor"),
        ('"component":"gate_proj.code","dtype":"I16","shape":[320,144,48]',
         '"component":"gate_proj.code","dtype":"I16","shape":[144,320,48]', "segment gate_proj.code: its shape"),
    ]
    for needle, repl, names in cases:
        assert needle in text, needle
        with pytest.raises(pkg.MlxsError) as ei:
            pkg.bank_peek(text=text.replace(needle, repl, 1))
        assert ei.value.rc == -8 and names in ei.value.msg, (names, ei.value.msg)
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text='{"format":"x","quantization":{},"dims":{"hidden":1,"inter":1,"n_experts":1,"n_layers":0},"layers":[]}')
    assert "format" in ei.value.msg
    with pytest.raises(pkg.MlxsError):
        pkg.bank_peek(text="{not json")


def test_v2_full_manifest_records_and_parity():
    pkg = load_package()
    m = bank_files.exl3_manifest(512, 256, 4, 2, ["ab" * 32] * 8)
    info = pkg.bank_peek(text=json.dumps(m))
    assert info.has_sha256 == 1 and info.data_file == b"experts.bin"
    bad = json.loads(json.dumps(m)); bad["parity"]["all_pass"] = False
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "parity.all_pass" in ei.value.msg
    bad = json.loads(json.dumps(m)); bad["records"][3]["sidecar_offset"] += 4096
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "record (0,3)" in ei.value.msg
    bad = json.loads(json.dumps(m)); bad["records"][5] = bad["records"][4]
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "duplicated" in ei.value.msg
    bad = json.loads(json.dumps(m)); bad["sidecar"]["file"] = "../experts.bin"
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "plain file name" in ei.value.msg


def test_v2_bank_of_mixed_layer_widths():
    """The reference's 2.9 bpw banks keep some layers at K = 2 inside a K = 3 bank (src/exl3/quant.zig:73,
    src/expert/bank.zig:288-298): per-layer record sizes, each layer after the ones before it."""
    pkg = load_package()
    H, I, E = 512, 256, 4
    bits = [3, 2, 2, 3]
    m = bank_files.exl3_manifest(H, I, E, 4, ["cd" * 32] * 16, bits)
    info = pkg.bank_peek(text=json.dumps(m))
    g3, g2 = bank_files.O.exl3_geometry(H, I, 3), bank_files.O.exl3_geometry(H, I, 2)
    assert (info.bank_kind, info.bits_min, info.bits_max) == (pkg.BANK_EXL3_K3_MUL1, 2, 3)
    assert info.logical_bytes == g3.logical_bytes and info.data_bytes == 2 * E * (g3.record_bytes + g2.record_bytes)
    assert pkg.bank_layer_bits(json.dumps(m)) == bits
    all2 = bank_files.exl3_manifest(H, I, E, 2, None, [2, 2])
    info = pkg.bank_peek(text=json.dumps(all2))
    assert (info.bank_kind, info.bits_min, info.bits_max, info.logical_bytes) == (pkg.BANK_EXL3_K2_MUL1, 2, 2, g2.logical_bytes)
    # a K = 2 layer that claims the K = 3 record size, and a layer placed as if the one before it were K = 3
    bad = json.loads(json.dumps(m)); bad["layers"][1]["record_bytes"] = int(g3.record_bytes)
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "geometry for K=2" in ei.value.msg
    bad = json.loads(json.dumps(m)); bad["layers"][2]["base_offset"] = 2 * E * int(g3.record_bytes)
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "layer 2 base_offset" in ei.value.msg
    bad = json.loads(json.dumps(m)); bad["layers"][3]["K"] = 1
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "layer 3 K 1 not implemented" in ei.value.msg


@pytest.mark.parametrize("nv", [False, True])
def test_fp4_manifests(nv):
    pkg = load_package()
    # src/arch/mimo_v2/bank.zig:341-345: MiMo geometry; src/arch/glm5_next/bank.zig:557-560: the tiny NVFP4 fixture
    H, I, E, L = (64, 32, 2, 1) if nv else (4096, 2048, 256, 47)
    m = bank_files.fp4_manifest(H, I, E, L, nv, first=3 if nv else 1)
    info = pkg.bank_peek(text=json.dumps(m))
    if nv:
        assert (info.logical_bytes, info.record_stride, info.data_bytes, info.first_layer) == (3468, 4096, 8192, 3)
    else:
        assert info.logical_bytes == 13_369_344 and info.data_bytes == 160_859_947_008
    for key, val, word in (("record_bytes", 1, "record_bytes"), ("gate_up_bytes", 7, "gate_up_bytes"),
                           ("data_file", "x.bin", "data_file")):
        bad = dict(m); bad[key] = val
        with pytest.raises(pkg.MlxsError) as ei:
            pkg.bank_peek(text=json.dumps(bad))
        assert word in ei.value.msg
    bad = json.loads(json.dumps(m)); bad["quantization"]["group_size"] = 64
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "group_size" in ei.value.msg
    bad = json.loads(json.dumps(m)); bad["records"][1]["expert"] = 0
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "record 1" in ei.value.msg


def test_peek_of_a_directory(tmp_path):
    pkg = load_package()
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(directory=tmp_path)
    assert "neither" in ei.value.msg
    (tmp_path / "expert-manifest-v2.json").write_text(json.dumps(bank_files.exl3_manifest(256, 128, 2, 1)))
    assert pkg.bank_peek(directory=tmp_path).hidden == 256
