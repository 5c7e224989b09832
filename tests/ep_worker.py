"""One rank of the 2-GPU expert-parallel parity test (started by tests/test_ep_gpu.py).

argv: rank world rendezvous_dir [placement].  Each rank owns half the experts (contiguous halves; with "interleaved"
the experts dealt alternately through mlxs_moe_set_placement; with "usage" placed by the library's route tally summed
over the ranks and its planner), routes its own tokens, runs the layer through the
library's exchange and checks its output rows against the CPU oracle over the whole bank."""
import os
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    rank, world, rdv = int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3])
    import torch

    import oracle_lib as O
    from __graft_entry__ import load_package
    from moe_cases import rel_l2
    pkg = load_package()
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    H, I, E, k, T = 512, 256, 8, 2, 12 + 5 * rank
    cfg = pkg.make_config(H, I, E, k, bank_kind=pkg.BANK_EXL3_K3_MUL1, act=pkg.ACT_SWIGLU_CLAMPED, act_limit=10.0,
                          scoring=pkg.SCORE_SQRTSOFTPLUS, routed_scale=1.5, shared_expert=True, max_tokens=32, device=rank,
                          ep_world=world, ep_rank=rank)
    moe = pkg.MoE(cfg)

    def batch(r, it):
        """rank r's tokens and logits of iteration it (seeded, so every rank can restate every other rank's)"""
        rs = np.random.default_rng(100 * r + it)
        n = 12 + 5 * r
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rs.standard_normal((n, H)).astype(np.float32)))
        logits = rs.standard_normal((n, E)).astype(np.float32)
        if it == 2:
            logits[:, :E // 2] += 8.0  # every token to the first half of the experts
        return x, logits
    # rendezvous through files: rank 0 publishes the NCCL id
    idf = rdv / "nccl_id.bin"
    if rank == 0:
        buf = (pkg.C.c_char * 128)()
        rc = pkg.lib().mlxs_moe_ep_unique_id(buf)
        assert rc == 0, pkg.last_error()
        (rdv / "nccl_id.tmp").write_bytes(bytes(buf))
        os.rename(rdv / "nccl_id.tmp", idf)
    t0 = time.time()
    while not idf.exists():
        if time.time() - t0 > 60:
            raise SystemExit("rendezvous timed out")
        time.sleep(0.05)
    idb = idf.read_bytes()
    rc = pkg.lib().mlxs_moe_ep_init(moe._h, idb)
    assert rc == 0, pkg.last_error()
    mode = sys.argv[4] if len(sys.argv) > 4 else "contiguous"
    if mode == "interleaved":
        place = (np.arange(E) % world).astype(np.uint16)
        moe.set_placement(0, place.ctypes.data)
    elif mode == "usage":
        # the library's tally over every rank's routes of the run, summed over the ranks, then its planner
        moe.usage_enable(True)
        want = np.zeros(E, np.int64)
        for r in range(world):
            for it in range(3):
                lg_r = batch(r, it)[1]
                want += np.bincount(O.route(lg_r, None, k, O.SCORE_SQRTSOFTPLUS, scale=1.5)[0].reshape(-1), minlength=E)
                if r == rank:
                    n = lg_r.shape[0]
                    lg = torch.from_numpy(lg_r).to(dev)
                    ids_d = torch.empty((n, k), dtype=torch.int32, device=dev)
                    w_d = torch.empty((n, k), dtype=torch.float32, device=dev)
                    moe.route(0, lg.data_ptr(), n, ids_d.data_ptr(), w_d.data_ptr(), None)
        torch.cuda.synchronize()
        counts = moe.usage_read(0, all_ranks=True)
        assert counts == list(want), (counts, list(want))
        mine = moe.usage_read(0)
        assert sum(mine) == 3 * T * k and sum(counts) == 3 * k * sum(12 + 5 * r for r in range(world))
        moe.usage_enable(False)
        place = np.asarray(pkg.plan_placement(counts, world), np.uint16)
        loads = [int(want[place == r].sum()) for r in range(world)]
        assert max(loads) - min(loads) <= int(want.max()), loads
        moe.set_placement(0, place.ctypes.data)
    records = {e: O.exl3_synth_record(0x5EED0000 + 17 * e, H, I, 1.0, 0.02) for e in range(E)}
    for e, rec in records.items():
        moe.load_expert(0, e, rec.ctypes.data, rec.size)  # the library keeps only this rank's shard
    rng = np.random.default_rng(991)
    shared = [O.f32_to_bf16_bits((rng.standard_normal(s) * 0.02).astype(np.float32)) for s in ((I, H), (I, H), (H, I))]
    moe.set_shared(0, shared[0].ctypes.data, shared[1].ctypes.data, shared[2].ctypes.data)
    ok = True
    for it in range(3):
        x, logits = batch(rank, it)  # it == 2: with contiguous halves rank 1 computes nothing, rank 0 everything
        xd = torch.from_numpy(O.f32_to_bf16_bits(x).view(np.int16)).to(dev).view(torch.bfloat16)
        lg = torch.from_numpy(logits).to(dev)
        y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        moe.forward(0, xd.data_ptr(), lg.data_ptr(), T, y.data_ptr(), None)
        torch.cuda.synchronize()
        ids, w = O.route(logits, None, k, O.SCORE_SQRTSOFTPLUS, scale=1.5)
        ref, ref_ro = O.layer(O.BANK_EXL3, H, I, E, k, records, x, ids, w, shared=shared, limit=10.0, want_ro=True)
        err = rel_l2(y.float().cpu().numpy(), ref)
        # the per-assignment form of the exchange (unweighted rows of every assignment, a collective call too)
        idd = torch.from_numpy(np.ascontiguousarray(ids, np.int32)).to(dev)
        ro = torch.full((T, k, H), float("nan"), dtype=torch.float32, device=dev)
        moe.routed(0, xd.data_ptr(), idd.data_ptr(), T, ro.data_ptr(), None)
        torch.cuda.synchronize()
        err_ro = rel_l2(ro.cpu().numpy(), ref_ro)
        print(f"rank {rank} iter {it} rel-L2 layer {err:.3e} rows {err_ro:.3e}", flush=True)
        ok = ok and err < 1e-2 and err_ro < 1e-3
    st = moe.stats()
    print(f"rank {rank} status {st.device_status} transport {st.ep_transport} a2a sent {st.a2a_bytes_sent} recv {st.a2a_bytes_recv}", flush=True)
    # 2 = rows stored straight into the peers' windows, 1 = NCCL send/recv (forced with MLXS_EP_NCCL_ONLY)
    want_transport = 1 if os.environ.get("MLXS_EP_NCCL_ONLY") else 2
    ok = ok and st.device_status == 0 and st.a2a_bytes_sent > 0 and st.ep_transport == want_transport
    moe.close()
    print(f"rank {rank} {'OK' if ok else 'FAIL'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
