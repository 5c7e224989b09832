"""The allocation-free EXL3 projection entry against the handle-based one, through the C ABI.

Collected last on purpose (file name): a run that stops at the first failure has then already run everything else.
The entry serves callers that cannot call cudaMalloc (a host with a device-memory budget fixed at load, code inside
a stream capture); its scratch is a fixed array in the library, so the checks are: same bits as
mlxs_moe_exl3_gemv, on two calls in a row that leave different leftovers in the shared scratch, and a clear refusal
beyond the fixed sizes.
"""
import numpy as np
import pytest

import oracle_lib as O
from moe_cases import Exl3Case

pytestmark = pytest.mark.gpu


def test_noalloc_matches_handle_entry_twice_in_a_row():
    import torch
    H, I = 1024, 512
    case = Exl3Case(H, I, 2, 1, seed=9, shared=False, max_tokens=64)
    pkg = case.pkg
    try:
        g = O.exl3_geometry(H, I)
        rng = np.random.default_rng(3)
        # first a 32-row call, then a 5-row call: the second must not see the first one's rows in the scratch
        for proj, rows in ((0, 32), (2, 5), (1, 17), (1, 17)):
            n_in, n_out = (I, H) if proj == 2 else (H, I)
            xh = rng.standard_normal((rows, n_in)).astype(np.float32)
            want = case.gpu_gemv(1, proj, xh)
            code = case.records[1][g.off[3 * proj]:g.off[3 * proj] + g.len[3 * proj]]
            code_d = torch.from_numpy(code.copy()).to(case.dev)
            xd = torch.from_numpy(xh).to(case.dev)
            z = torch.full((rows, n_out), float("nan"), dtype=torch.float32, device=case.dev)
            pkg.exl3_gemv_noalloc(code_d.data_ptr(), n_in, n_out, xd.data_ptr(), rows, z.data_ptr(), None)
            torch.cuda.synchronize()
            got = z.cpu().numpy()
            assert (got.view(np.uint32) == want.view(np.uint32)).all()
        # refusals beyond the fixed scratch, by name
        for kw, word in ((dict(rows=33), "rows"), (dict(n_in=8192 + 128), "in_dim"), (dict(n_in=100), "in_dim"),
                         (dict(n_out=24), "out_dim")):
            a = dict(rows=4, n_in=H, n_out=I)
            a.update(kw)
            with pytest.raises(pkg.MlxsError) as ei:
                pkg.exl3_gemv_noalloc(code_d.data_ptr(), a["n_in"], a["n_out"], xd.data_ptr(), a["rows"], z.data_ptr(), None)
            assert word in ei.value.msg
        # misaligned buffers are refused before any launch (the staging kernel reads 16-byte vectors)
        for bad, word in ((dict(x=4), "xh_dev"), (dict(code=2), "code_dev"), (dict(z=2), "z_dev")):
            with pytest.raises(pkg.MlxsError) as ei:
                pkg.exl3_gemv_noalloc(code_d.data_ptr() + bad.get("code", 0), H, I, xd.data_ptr() + bad.get("x", 0), 4,
                                      z.data_ptr() + bad.get("z", 0), None)
            assert word in ei.value.msg and ei.value.rc == pkg.E_ARG
        assert case.status() == 0
    finally:
        case.close()
