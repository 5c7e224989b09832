"""Expert parallelism on 2 GPUs: each rank's outputs through the library's dispatch / combine exchange against the
CPU oracle over the whole bank.  Ranks are child processes (one per GPU); NVLS is off for the test."""
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


@pytest.mark.parametrize("transport", ["peer-stores", "nccl"])
@pytest.mark.parametrize("placement", ["contiguous", "interleaved", "usage"])
def test_two_rank_exchange_matches_oracle(placement, transport):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if transport == "nccl":
        env["MLXS_EP_NCCL_ONLY"] = "1"
    with tempfile.TemporaryDirectory() as rdv:
        procs = [subprocess.Popen([sys.executable, str(HERE / "ep_worker.py"), str(r), "2", rdv, placement], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=300)
            except subprocess.TimeoutExpired:
                for q in procs:
                    q.kill()
                raise
            outs.append(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and f"rank {r} OK" in out, out[-3000:]
