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
    # a v2 record digest must be 64 lowercase hex digits (src/expert/bank.zig:432-466 decodes nothing else)
    bad = json.loads(json.dumps(m)); bad["records"][2]["sha256"] = "AB" * 32
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(text=json.dumps(bad))
    assert "RecordSha256" in ei.value.msg and "record (0,2)" in ei.value.msg


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
    # the reference's parse refusals by name (src/arch/mimo_v2/bank.zig:210-239, tests :397-403)
    def refused(fn, name):
        bad = json.loads(json.dumps(m))
        fn(bad)
        with pytest.raises(pkg.MlxsError) as ei:
            pkg.bank_peek(text=json.dumps(bad))
        assert name in ei.value.msg, (name, ei.value.msg)
    table = "parts" if nv else "segments"
    refused(lambda d: d["quantization"].update(mode="affine"), "InvalidQuantization")
    refused(lambda d: d[table][0].update(dtype="U16"), "InvalidSegment")
    refused(lambda d: d[table].pop(), "InvalidSegment")
    refused(lambda d: d["records"][0].update(offset=4), "InvalidRecord")
    refused(lambda d: d["records"].pop(), "InvalidRecord")
    refused(lambda d: d["records"][0].update(sha256="12"), "InvalidDigest")
    # 64 characters that are not lowercase hex are no digest either (the reference decodes lowercase hex only)
    refused(lambda d: d["records"][0].update(sha256="A" * 64), "InvalidDigest")
    refused(lambda d: d["output_files"]["experts.bin"].update(sha256="g" * 64), "InvalidDigest")
    refused(lambda d: d["source"].update(revision="z" * 40), "InvalidSource")
    refused(lambda d: d["source"].update(repository=""), "InvalidSource")
    refused(lambda d: d["output_files"]["experts.bin"].update(size=1), "InvalidOutputFile")
    refused(lambda d: d.update(output_files={}), "InvalidOutputFile")
    refused(lambda d: d.update(record_bytes=d["record_bytes"] + 1), "InvalidGeometry")


def test_peek_of_a_directory(tmp_path):
    pkg = load_package()
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_peek(directory=tmp_path)
    assert "neither" in ei.value.msg
    (tmp_path / "expert-manifest-v2.json").write_text(json.dumps(bank_files.exl3_manifest(256, 128, 2, 1)))
    assert pkg.bank_peek(directory=tmp_path).hidden == 256


def _small_bank(tmp_path, bits=(3, 2)):
    import numpy as np
    H, I, E, L = 256, 128, 3, len(bits)
    recs = {(l, e): bank_files.O.exl3_synth_record(900 + 10 * l + e, H, I, 1.0, 0.02, K=bits[l]) for l in range(L) for e in range(E)}
    v2, lshas = bank_files.write_exl3_bank(tmp_path, H, I, E, L, lambda l, e: recs[(l, e)], list(bits))
    return v2, lshas, (H, I, E, L)


def test_bank_open_without_a_device(tmp_path):
    """Bank.open's checks with no device (src/expert/bank.zig:228-251): both manifests, the sidecar, every digest."""
    pkg = load_package()
    v2, lshas, (H, I, E, L) = _small_bank(tmp_path)
    info = pkg.bank_verify(tmp_path)
    assert (info.hidden, info.inter, info.n_experts, info.n_layers, info.bits_min, info.bits_max) == (H, I, E, L, 2, 3)
    assert info.data_bytes == (tmp_path / "experts.bin").stat().st_size
    # a flipped bit inside a record's logical bytes: both digests catch it; in the padding: only the v2 one exists for it
    raw = bytearray((tmp_path / "experts.bin").read_bytes())
    raw[100] ^= 1
    (tmp_path / "experts.bin").write_bytes(bytes(raw))
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_verify(tmp_path)
    assert "RecordSha256" in ei.value.msg and "record (0,0)" in ei.value.msg
    assert pkg.bank_verify(tmp_path, verify_sha256=False).n_experts == E   # the geometry alone still opens


def test_v1_runtime_manifest_refusals_by_name(tmp_path):
    """The v1 half of the reference's refusal table (src/expert/bank.zig:1064-1072): no v1 manifest, another format,
    another mode, a moved record, swapped segments, a gap, a short digest, a dropped record, a truncated file; and the
    sidecar cases (missing, short, a symbolic link)."""
    import os
    pkg = load_package()
    v2, lshas, (H, I, E, L) = _small_bank(tmp_path)
    good = bank_files.exl3_manifest_v1(v2, lshas)
    v1_path = tmp_path / "expert-manifest.json"

    def refused(doc, words, text=None):
        v1_path.write_text(text if text is not None else json.dumps(doc, separators=(",", ":")))
        with pytest.raises(pkg.MlxsError) as ei:
            pkg.bank_verify(tmp_path, verify_sha256=False)
        assert ei.value.rc == -8 and words in ei.value.msg, (words, ei.value.msg)

    def mutated(fn):
        d = json.loads(json.dumps(good))
        fn(d)
        return d

    v1_path.unlink()
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_verify(tmp_path)
    assert "ManifestMissing" in ei.value.msg
    refused(mutated(lambda d: d.update(format="mtplx-expert-manifest-v2")), "ManifestFormat")
    refused(mutated(lambda d: d["quantization"].update(mode="tcq3")), "RuntimeModeNotExl3")
    refused(mutated(lambda d: d["records"][E + 1].update(sidecar_offset=d["records"][E + 1]["sidecar_offset"] + 4096)),
            "record (1,1) offset/length differs")

    def swap(d):
        sg = d["records"][2]["segments"]
        sg[1], sg[2] = sg[2], sg[1]
    refused(mutated(swap), "record (0,2) segments differ")
    refused(mutated(lambda d: d["records"][1]["segments"][6].update(offset=d["records"][1]["segments"][6]["offset"] + 2)),
            "record (0,1) segments differ")
    refused(mutated(lambda d: d["records"][0].update(sha256="abcd")), "record (0,0) has no sha256")
    refused(mutated(lambda d: d["records"].pop(E)), "RecordCount")
    refused(mutated(lambda d: d["records"].__setitem__(1, d["records"][0])), "RecordDuplicate")
    refused(mutated(lambda d: d["records"][0]["segments"][3].update(shard="other.bin")), 'reads shard "other.bin"')
    refused(mutated(lambda d: d["sidecar"].update(size=d["sidecar"]["size"] + 4096)), "SidecarGeometry")
    text = json.dumps(good, separators=(",", ":"))
    refused(None, "ManifestSyntax", text=text[:text.index('},{"expert"') + 1])
    # the good one opens again; then the sidecar cases
    v1_path.write_text(text)
    pkg.bank_verify(tmp_path)
    side = tmp_path / "experts.bin"
    data = side.read_bytes()
    side.write_bytes(data[:-4096])
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_verify(tmp_path, verify_sha256=False)
    assert "SidecarGeometry" in ei.value.msg
    side.unlink()
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_verify(tmp_path, verify_sha256=False)
    assert "cannot open" in ei.value.msg
    (tmp_path / "real.bin").write_bytes(data)
    os.symlink(tmp_path / "real.bin", side)
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_verify(tmp_path, verify_sha256=False)
    assert "cannot open" in ei.value.msg and "SidecarOpen" in ei.value.msg


@pytest.mark.parametrize("nv", [False, True])
def test_fp4_bank_opens_without_a_device(tmp_path, nv):
    import numpy as np
    pkg = load_package()
    H, I, E, L = 128, 64, 2, 2
    O = bank_files.O
    synth = O.nvfp4_synth_record if nv else O.mxfp4_synth_record
    bank_files.write_fp4_bank(tmp_path, H, I, E, L, nv, lambda l, e: synth(50 + 7 * l + e, H, I, 0.02))
    info = pkg.bank_verify(tmp_path)
    assert (info.bank_kind, info.n_experts, info.n_layers) == (pkg.BANK_NVFP4 if nv else pkg.BANK_MXFP4, E, L)
    raw = bytearray((tmp_path / "experts.bin").read_bytes())
    raw[-1 if not nv else 10] ^= 4
    (tmp_path / "experts.bin").write_bytes(bytes(raw))
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_verify(tmp_path)
    assert "RecordSha256" in ei.value.msg


def test_v2_refusal_table_of_the_reference(tmp_path):
    """The v2 half of the reference's refusal table (src/expert/bank.zig:1045-1063), each case on a bank that opens
    before the mutation."""
    import hashlib
    pkg = load_package()
    v2, lshas, (H, I, E, L) = _small_bank(tmp_path, bits=(3, 3))
    v2_path = tmp_path / "expert-manifest-v2.json"
    good = json.loads(v2_path.read_text())
    pkg.bank_verify(tmp_path)

    def refused(fn, words, text=None, verify=False):
        d = json.loads(json.dumps(good))
        if fn:
            fn(d)
        v2_path.write_text(text if text is not None else json.dumps(d, separators=(",", ":")))
        with pytest.raises(pkg.MlxsError) as ei:
            pkg.bank_verify(tmp_path, verify_sha256=verify)
        assert ei.value.rc == -8 and words in ei.value.msg, (words, ei.value.msg)

    text = json.dumps(good, separators=(",", ":"))
    refused(None, "not a JSON object", text=text[:len(text) // 2])                                   # ManifestSyntax
    refused(lambda d: d.update(format="mtplx-expert-manifest-v3"), "format")                        # ManifestFormat
    refused(lambda d: d["quantization"].update(codebook="mcg"), 'codebook "mcg" not implemented')   # CodebookNotImplemented
    refused(lambda d: d["quantization"].update(codebook_multiplier=0x83DCD12E), "codebook_multiplier")
    refused(lambda d: d["dims"].update(hidden=72), "dims hidden=72")                                # DimsInvalid
    refused(lambda d: d["layers"].pop(), "layer entries != dims.n_layers")                          # LayerGeometry
    refused(lambda d: d["layers"][1].update(layer=5), "names layer 5")
    refused(lambda d: d["layers"][0].update(K=4), "K 4 not implemented")                            # KNotImplemented
    refused(lambda d: d["layers"][0]["segments"][0].update(length=d["layers"][0]["segments"][0]["length"] + 2), "its place")
    refused(lambda d: d["layers"][1].update(base_offset=d["layers"][1]["base_offset"] + 4096), "layer 1 base_offset")
    refused(lambda d: d["sidecar"].update(size=d["sidecar"]["size"] + 4096), "sidecar.size")        # SidecarGeometry
    refused(lambda d: d["sidecar"].update(alignment=8192), "sidecar alignment 8192")
    refused(lambda d: d["records"].pop(), "records !=")                                             # RecordCount
    refused(lambda d: d["records"][0].update(expert=E), "out of range")                             # RecordGeometry
    refused(lambda d: d["records"].__setitem__(1, d["records"][0]), "duplicated")                   # RecordDuplicate
    refused(lambda d: d["records"][2].update(sidecar_offset=d["records"][2]["sidecar_offset"] + 4096), "offset/size differs")
    refused(lambda d: d["records"][0].update(sha256=hashlib.sha256(b"x").hexdigest()), "RecordSha256", verify=True)
    refused(lambda d: d["parity"].update(all_pass=False), "parity.all_pass")                        # ParityNotPassed
    v2_path.unlink()
    with pytest.raises(pkg.MlxsError) as ei:
        pkg.bank_verify(tmp_path)
    # without the v2 manifest the v1 one is not a bank description of its own
    assert ei.value.rc == -8 and "ManifestMissing" in ei.value.msg
