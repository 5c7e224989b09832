"""Test tooling: writes synthetic expert banks (experts.bin + manifest) in the reference's own formats, so the
library's manifest reader and bank load are exercised on the formats real packs use.
  EXL3  mtplx-expert-manifest-v2              (src/expert/bank.zig:103-155; sample src/fixtures/dsv41_bank_peek.json)
  MXFP4 mlx-stream-mxfp4-expert-bank-v1       (src/arch/mimo_v2/bank.zig:172-187)
  NVFP4 mlx-stream-nvfp4-expert-bank-v1       (src/arch/glm5_next/bank.zig:262-283, fixture :557-580)
"""
import hashlib
import json
from pathlib import Path

import numpy as np

import oracle_lib as O


def exl3_manifest(H, I, E, L, records_sha=None, bits=None):
    """bits: K per layer (default 3 everywhere); the sidecar places a layer after the layers before it."""
    bits = list(bits) if bits is not None else [3] * L
    geoms = [O.exl3_geometry(H, I, k) for k in bits]
    base = [0]
    for g in geoms:
        base.append(base[-1] + E * int(g.record_bytes))
    names = ["gate_proj", "up_proj", "down_proj"]
    parts = ["code", "rout", "rin"]
    layers = []
    for l in range(L):
        segs = []
        g = geoms[l]
        for p in range(3):
            n_in, n_out = (I, H) if p == 2 else (H, I)
            shapes = [[n_in // 16, n_out // 16, 16 * bits[l]], [n_out], [n_in]]
            for j in range(3):
                segs.append({"component": f"{names[p]}.{parts[j]}", "dtype": "I16" if j == 0 else "F16",
                             "shape": shapes[j], "offset": int(g.off[3 * p + j]), "length": int(g.len[3 * p + j])})
        layers.append({"layer": l, "K": bits[l], "record_bytes": int(g.record_bytes), "logical_bytes": int(g.logical_bytes),
                       "base_offset": base[l], "segments": segs})
    m = {"format": "mtplx-expert-manifest-v2",
         "quantization": {"mode": "exl3", "codebook": "mul1", "codebook_multiplier": 2212286765,
                          "tile": {"size": 16, "layout": "exl3-tensor-core", "bitstream": "msb-first-swap16"},
                          "hadamard": {"size": 128, "order": "sylvester-natural", "scale": "1/sqrt(128)"},
                          "scales": {"rin": "exl3.suh", "rout": "exl3.svh"}},
         "dims": {"hidden": H, "inter": I, "n_experts": E, "n_layers": L}, "layers": layers}
    if records_sha is not None:
        m["sidecar"] = {"file": "experts.bin", "alignment": 4096, "size": base[L]}
        m["records"] = [{"layer": l, "expert": e, "sidecar_offset": base[l] + e * int(geoms[l].record_bytes),
                         "record_bytes": int(geoms[l].record_bytes), "logical_bytes": int(geoms[l].logical_bytes),
                         "sha256": records_sha[l * E + e]} for l in range(L) for e in range(E)]
        m["parity"] = {"all_pass": True}
    return m


def exl3_manifest_v1(v2, logical_shas):
    """The v1 runtime manifest of the same bank (src/expert/bank.zig:924-946): per record the v2 segment table at
    absolute offsets, the digest of the record's logical bytes, the sidecar again."""
    E = v2["dims"]["n_experts"]
    recs = []
    for r in v2["records"]:
        l, e, off = r["layer"], r["expert"], r["sidecar_offset"]
        segs = [{"component": sg["component"], "dtype": sg["dtype"], "length": sg["length"], "offset": off + sg["offset"],
                 "shape": sg["shape"], "shard": v2["sidecar"]["file"], "tensor": f"layers.{l}.ffn.experts.{e}"}
                for sg in v2["layers"][l]["segments"]]
        recs.append({"expert": e, "layer": l, "logical_bytes": r["logical_bytes"], "segments": segs,
                     "sha256": logical_shas[l * E + e], "sidecar_length": r["logical_bytes"], "sidecar_offset": off})
    return {"artifact": {"record_count": len(recs)}, "format": "mtplx-expert-manifest-v1", "model_key": "synthetic",
            "quantization": {"bits": 3, "group_size": 32, "mode": "exl3-mul1"}, "records": recs,
            "shards": [{"name": v2["sidecar"]["file"], "size": v2["sidecar"]["size"]}],
            "sidecar": dict(v2["sidecar"]), "source_repo": "synthetic"}


def write_exl3_bank(directory, H, I, E, L, record_of, bits=None, v1=True):
    """record_of(layer, expert) -> uint8 record (padded to the record stride); bits: K per layer; v1: also write the
    runtime manifest the reference's Bank.open requires beside the v2 one."""
    directory = Path(directory)
    bits = list(bits) if bits is not None else [3] * L
    shas, lshas = [], []
    with open(directory / "experts.bin", "wb") as f:
        for l in range(L):
            g = O.exl3_geometry(H, I, bits[l])
            for e in range(E):
                rec = np.zeros(g.record_bytes, np.uint8)
                r = record_of(l, e)
                rec[:r.size] = r
                shas.append(hashlib.sha256(rec.tobytes()).hexdigest())
                lshas.append(hashlib.sha256(rec[:int(g.logical_bytes)].tobytes()).hexdigest())
                f.write(rec.tobytes())
    v2 = exl3_manifest(H, I, E, L, shas, bits)
    (directory / "expert-manifest-v2.json").write_text(json.dumps(v2, separators=(",", ":")))
    if v1:
        (directory / "expert-manifest.json").write_text(json.dumps(exl3_manifest_v1(v2, lshas), separators=(",", ":")))
    return v2, lshas


def fp4_manifest(H, I, E, L, nv, first=1, shas=None):
    blk = 16 if nv else 32
    part = H * I // 2 + H * I // blk + (4 if nv else 0)
    logical = 3 * part
    stride = (logical + 4095) // 4096 * 4096 if nv else logical
    segs, off = [], 0
    for p, name in enumerate(["gate_proj", "up_proj", "down_proj"]):
        rows, cols = (H, I) if p == 2 else (I, H)
        items = [("weight", "U32", [rows, cols // 8], rows * cols // 2), ("scales", "U8", [rows, cols // blk], rows * cols // blk)]
        if nv:
            items.append(("global_scale", "F32", [], 4))
        for nm, dt, shp, ln in items:
            segs.append({"name": f"{name}.{nm}", "dtype": dt, "shape": shp, "offset": off, "length": ln})
            off += ln
    shas = shas or ["a" * 64] * (L * E)
    m = {"format": "mlx-stream-nvfp4-expert-bank-v1" if nv else "mlx-stream-mxfp4-expert-bank-v1", "data_file": "experts.bin",
         "hidden_size": H, "intermediate_size": I, "num_experts": E, "first_moe_layer": first, "num_moe_layers": L,
         "record_bytes": logical, "gate_up_bytes": 2 * part,
         "quantization": {"mode": "nvfp4" if nv else "mxfp4", "bits": 4, "group_size": blk},
         "source": {"repository": "synthetic", "revision": "0123456789012345678901234567890123456789"},
         ("parts" if nv else "segments"): segs,
         "records": [{"layer": first + i // E, "expert": i % E, "offset": i * stride, "length": logical, "sha256": shas[i]}
                     for i in range(L * E)],
         "output_files": {"experts.bin": {"size": L * E * stride, "sha256": "c" * 64}}}
    if nv:
        m.update(layout="nvfp4-gud-9part", alignment=4096, record_stride=stride, down_bytes=part)
    return m


def write_fp4_bank(directory, H, I, E, L, nv, record_of):
    directory = Path(directory)
    m0 = fp4_manifest(H, I, E, L, nv)
    logical = m0["record_bytes"]
    stride = m0.get("record_stride", logical)
    shas = []
    with open(directory / "experts.bin", "wb") as f:
        for l in range(L):
            for e in range(E):
                r = record_of(l, e)
                assert r.size == logical
                shas.append(hashlib.sha256(r.tobytes()).hexdigest())
                f.write(r.tobytes())
                f.write(b"\0" * (stride - logical))
    (directory / "expert-manifest.json").write_text(json.dumps(fp4_manifest(H, I, E, L, nv, shas=shas), separators=(",", ":")))
