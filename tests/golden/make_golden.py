"""Collects the reference's own golden vectors for the routed-MoE path into this folder.

Run once in a container that has the reference checked out (argument: its root).  It copies only DATA the
reference's tests pin (digests and two small f32 vectors), never source:
  * src/kernels/exl3/manifest.json `golden`        -> the mul1 table digest and the four seeded planes
  * src/arch/glm5_next/exl3_parity.zig:19-23        -> the two GLM-shape plane digests (literals re-typed below)
  * src/arch/glm5_next/testdata/exl3-ref/           -> meta.json, h_mul1.f32, y_mul1.f32 (expert forward fixture)
  * src/fixtures/dsv41_bank_peek.json               -> the v2 manifest sample the reference's claims tests mutate
The parity tests read the copies, so they run where the reference is absent.
"""
import json
import shutil
import sys
from pathlib import Path

here = Path(__file__).resolve().parent


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    manifest = json.loads((ref / "src/kernels/exl3/manifest.json").read_text())
    golden = manifest["golden"]
    planes = {}
    for name, p in golden["planes"].items():
        planes[name] = {k: p[k] for k in ("K", "seed", "projection", "code_sha256", "w_hat_sha256", "onehot_rows",
                                          "onehot_rows_sha256", "states_covered_by_onehot_rows")}
    out = {
        "source": "src/kernels/exl3/manifest.json golden; src/arch/glm5_next/exl3_parity.zig:19-23",
        "mul1_table_sha256": golden["mul1_table"]["sha256"],
        "planes": planes,
        "glm_planes": [
            {"projection": [4096, 2048], "seed": 0x474C4D35E3010001, "K": 3,
             "code_sha256": "334910c3086f12bd760d4d0cd974f2be78ef4d544c9608c8ea94b391c7aa976e",
             "w_hat_sha256": "f22a9f4828c4d119e33ca76201e578d5d0759a6de3f312be7300dd0aec934ba5"},
            {"projection": [2048, 4096], "seed": 0x474C4D35E3010002, "K": 3,
             "code_sha256": "8a2ae8214525ae1b7d8fa2b6b9c288387309fd96a99e3ac1fd1bae7d33549b41",
             "w_hat_sha256": "e2d4731fcb4a17a5a59dab8e99195d51215c1b884d158106b385d43dbc3f4265"},
        ],
    }
    # check the re-typed GLM literals against the reference text, so a typo cannot pass silently
    parity = (ref / "src/arch/glm5_next/exl3_parity.zig").read_text()
    for p in out["glm_planes"]:
        assert p["code_sha256"] in parity and p["w_hat_sha256"] in parity
    (here / "exl3_digests.json").write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    fx = ref / "src/arch/glm5_next/testdata/exl3-ref"
    dst = here / "exl3-ref"
    dst.mkdir(exist_ok=True)
    for f in ("meta.json", "h_mul1.f32", "y_mul1.f32"):
        shutil.copyfile(fx / f, dst / f)
    # the trimmed v2 manifest of the bank of record (format, quantization, dims, 40 layer tables): a data fixture
    shutil.copyfile(ref / "src/fixtures/dsv41_bank_peek.json", here / "dsv41_bank_peek.json")
    print("wrote", here / "exl3_digests.json", "and", dst)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <checkout of the reference project>")
    main(sys.argv[1])
