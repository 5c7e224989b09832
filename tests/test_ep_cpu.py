"""The expert-parallel protocol on CPU ranks (gloo, world size 2): destination plan, row exchange, local experts,
return and re-ordering, with the oracle as every rank's expert math.  The result must equal the single-rank oracle."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

HERE = Path(__file__).resolve().parent


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, q):
    sys.path.insert(0, str(HERE))
    sys.path.insert(0, str(HERE.parent))
    import torch
    import torch.distributed as dist

    import oracle_lib as O
    from __graft_entry__ import load_package
    pkg = load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, I, E, k, T = 256, 128, 8, 2, 5 + 2 * rank
    e_local = E // world
    records = {e: O.exl3_synth_record(0xABC0 + e, H, I, 1.0, 0.02) for e in range(E)}
    rs = np.random.default_rng(10 + rank)
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rs.standard_normal((T, H)).astype(np.float32)))
    logits = rs.standard_normal((T, E)).astype(np.float32)
    ids, w = O.route(logits, None, k, O.SCORE_SIGMOID)
    flat = ids.reshape(-1)
    # the library's host-side plan: rows per destination rank
    counts = np.zeros(world, np.uint64)
    assert pkg.lib().mlxs_moe_ep_plan(flat.ctypes.data, flat.size, E, world, counts.ctypes.data) == 0
    dest = flat // e_local
    assert (np.bincount(dest, minlength=world) == counts).all()
    order = np.argsort(dest, kind="stable")           # rows in destination order, routed order kept inside a rank
    send_x = x[order // k]
    send_meta = (flat[order] % e_local).astype(np.int32)
    all_counts = [torch.zeros(world, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(all_counts, torch.from_numpy(counts.astype(np.int64)))
    recv_n = [int(all_counts[s][rank]) for s in range(world)]
    send_split = [int(c) for c in counts]
    rx = [torch.zeros((n, H), dtype=torch.float32) for n in recv_n]
    rm = [torch.zeros(n, dtype=torch.int32) for n in recv_n]
    # pairwise exchange with exact counts, as the library's grouped send / recv does
    reqs = []
    sx, sm = torch.from_numpy(send_x).split(send_split), torch.from_numpy(send_meta).split(send_split)
    for peer in range(world):
        if peer == rank:
            rx[peer].copy_(sx[peer]); rm[peer].copy_(sm[peer])
        else:
            reqs += [dist.isend(sx[peer].contiguous(), peer, tag=1), dist.isend(sm[peer].contiguous(), peer, tag=2),
                     dist.irecv(rx[peer], peer, tag=1), dist.irecv(rm[peer], peer, tag=2)]
    for r in reqs:
        r.wait()
    recv_x = torch.cat(rx).numpy()
    recv_meta = torch.cat(rm).numpy()
    # local experts: every received row is its own token with one expert (global id = first + local index)
    R = recv_x.shape[0]
    local_recs = {e: records[rank * e_local + e] for e in range(e_local)}
    if R:
        ro = O.layer(O.BANK_EXL3, H, I, e_local, 1, local_recs, recv_x, recv_meta.reshape(-1, 1),
                     np.ones((R, 1), np.float32), limit=10.0)
    else:
        ro = np.zeros((0, H))
    back = [torch.zeros((n, H), dtype=torch.float64) for n in send_split]
    parts = torch.from_numpy(np.ascontiguousarray(ro)).split(recv_n)
    reqs = []
    for peer in range(world):
        if peer == rank:
            back[peer].copy_(parts[peer])
        else:
            reqs += [dist.isend(parts[peer].contiguous(), peer, tag=3), dist.irecv(back[peer], peer, tag=3)]
    for r in reqs:
        r.wait()
    ret = torch.cat(back).numpy()
    rows = np.empty((T * k, H))
    rows[order] = ret
    y = (rows.reshape(T, k, H) * w[:, :, None].astype(np.float64)).sum(axis=1)
    ref = O.layer(O.BANK_EXL3, H, I, E, k, records, x, ids, w, limit=10.0)
    err = float(np.abs(y - ref).max() / (np.abs(ref).max() + 1e-30))
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, err, int(R)))


def _exchange(dist, torch, rank, world, pieces, recv_shapes, dtype, tag):
    """Pairwise exchange with exact counts: pieces[peer] goes to peer, returns what every peer sent here."""
    got = [torch.zeros(shape, dtype=dtype) for shape in recv_shapes]
    reqs = []
    for peer in range(world):
        if peer == rank:
            got[peer].copy_(pieces[peer])
        else:
            reqs += [dist.isend(pieces[peer].contiguous(), peer, tag=tag), dist.irecv(got[peer], peer, tag=tag)]
    for r in reqs:
        r.wait()
    return got


def _rank_dedup(rank, world, port, q):
    """The layer form of the exchange: a token's row travels once per destination rank, the owning rank folds
    weight x row over the token's experts it holds, one partial row per (token, rank) comes back."""
    sys.path.insert(0, str(HERE))
    sys.path.insert(0, str(HERE.parent))
    import torch
    import torch.distributed as dist

    import oracle_lib as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, I, E, k, T = 256, 128, 8, 4, 6 + 3 * rank
    e_local = E // world
    records = {e: O.exl3_synth_record(0xABC0 + e, H, I, 1.0, 0.02) for e in range(E)}
    rs = np.random.default_rng(20 + rank)
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rs.standard_normal((T, H)).astype(np.float32)))
    logits = rs.standard_normal((T, E)).astype(np.float32)
    ids, w = O.route(logits, None, k, O.SCORE_SIGMOID)
    flat, wflat = ids.reshape(-1), w.reshape(-1)
    dest = flat // e_local
    order = np.argsort(dest, kind="stable")
    tok = order // k
    # first assignment of each (token, rank) pair in sorted order, and the unique row every position reads
    first = np.ones(order.size, bool)
    first[1:] = (tok[1:] != tok[:-1]) | (dest[order][1:] != dest[order][:-1])
    urow = np.cumsum(first) - 1
    n_a = np.bincount(dest, minlength=world)
    n_u = np.array([int(first[dest[order] == r].sum()) for r in range(world)])
    assert n_u.sum() < order.size  # top-4 over 2 ranks: rows are shared
    a0, u0 = np.concatenate([[0], np.cumsum(n_a)]), np.concatenate([[0], np.cumsum(n_u)])
    send_x = x[tok[first]]
    send_meta = (flat[order] % e_local).astype(np.int32)
    send_urow = (urow - u0[dest[order]]).astype(np.int32)
    send_w = wflat[order].astype(np.float32)
    counts = torch.from_numpy(np.stack([n_a, n_u], 1).astype(np.int64))
    allc = [torch.zeros((world, 2), dtype=torch.int64) for _ in range(world)]
    dist.all_gather(allc, counts)
    ra = [int(allc[s][rank][0]) for s in range(world)]
    ru = [int(allc[s][rank][1]) for s in range(world)]
    sp = lambda arr, off: [torch.from_numpy(np.ascontiguousarray(arr[off[r]:off[r + 1]])) for r in range(world)]
    rx = _exchange(dist, torch, rank, world, sp(send_x, u0), [(n, H) for n in ru], torch.float32, 1)
    rm = _exchange(dist, torch, rank, world, sp(send_meta, a0), [(n,) for n in ra], torch.int32, 2)
    rr = _exchange(dist, torch, rank, world, sp(send_urow, a0), [(n,) for n in ra], torch.int32, 3)
    rw = _exchange(dist, torch, rank, world, sp(send_w, a0), [(n,) for n in ra], torch.float32, 4)
    ubase = np.concatenate([[0], np.cumsum(ru)])
    recv_x = torch.cat(rx).numpy()
    recv_meta = torch.cat(rm).numpy()
    recv_w = torch.cat(rw).numpy()
    xrow = np.concatenate([rr[s].numpy() + ubase[s] for s in range(world)]) if sum(ra) else np.zeros(0, np.int64)
    RA = recv_meta.size
    local_recs = {e: records[rank * e_local + e] for e in range(e_local)}
    partial = np.zeros((int(sum(ru)), H))
    if RA:
        ro = O.layer(O.BANK_EXL3, H, I, e_local, 1, local_recs, recv_x[xrow], recv_meta.reshape(-1, 1),
                     np.ones((RA, 1), np.float32), limit=10.0)
        np.add.at(partial, xrow, ro * recv_w[:, None].astype(np.float64))
    back = _exchange(dist, torch, rank, world,
                     [torch.from_numpy(np.ascontiguousarray(partial[ubase[s]:ubase[s + 1]])) for s in range(world)],
                     [(int(n), H) for n in n_u], torch.float64, 5)
    ret = torch.cat(back).numpy()
    y = np.zeros((T, H))
    np.add.at(y, tok[first], ret)
    ref = O.layer(O.BANK_EXL3, H, I, E, k, records, x, ids, w, limit=10.0)
    err = float(np.abs(y - ref).max() / (np.abs(ref).max() + 1e-30))
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, err, int(RA)))


def test_ep_dedup_protocol_world2_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_dedup, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, RA in res:
        assert err < 1e-12, (rank, err)
    assert sum(r[2] for r in res) == (6 + 9) * 4


def test_ep_protocol_world2_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    for rank, err, R in res:
        assert err < 1e-12, (rank, err)
    assert sum(r[2] for r in res) == (5 + 7) * 2


def _rank_placement(rank, world, port, q):
    """Placement by usage on CPU ranks: each rank tallies its own routes (numpy stands in for the device tally), the
    counts are summed over the ranks, and the library's planner must give every rank the same table; the ranks'
    expected rows come out closer than with contiguous blocks."""
    sys.path.insert(0, str(HERE))
    sys.path.insert(0, str(HERE.parent))
    import torch
    import torch.distributed as dist

    import oracle_lib as O
    from __graft_entry__ import load_package
    pkg = load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    E, k, T = 32, 4, 300 + 50 * rank
    rs = np.random.default_rng(77 + rank)
    pop = np.log((1.0 + np.random.default_rng(5).permutation(E)) ** -1.1)   # one popularity order for every rank
    logits = (rs.standard_normal((T, E)) + pop).astype(np.float32)
    ids, _ = O.route(logits, None, k, O.SCORE_SIGMOID)
    mine = np.bincount(ids.reshape(-1), minlength=E).astype(np.int64)
    total = torch.from_numpy(mine.copy())
    dist.all_reduce(total)
    total = total.numpy()
    place = np.asarray(pkg.plan_placement(total, world))
    # every rank must hold the same table
    tables = [torch.zeros(E, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(tables, torch.from_numpy(place.astype(np.int64)))
    same = all((t.numpy() == place).all() for t in tables)
    by_use = [int(total[place == r].sum()) for r in range(world)]
    blocks = [int(total[r * (E // world):(r + 1) * (E // world)].sum()) for r in range(world)]
    # the destination plan of this rank's assignments under the table: counts per rank add up
    dest = place[ids.reshape(-1)]
    sent = np.bincount(dest, minlength=world)
    dist.destroy_process_group()
    q.put((rank, same, by_use, blocks, int(sent.sum()), int(total.sum())))


def test_usage_placement_world2_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_placement, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, same, by_use, blocks, sent, total in res:
        assert same, rank
        assert sent == (300 + 50 * rank) * 4 and total == (300 + 350) * 4
        assert max(by_use) - min(by_use) < max(blocks) - min(blocks), (by_use, blocks)
    assert res[0][2] == res[1][2]


def test_peer_store_protocol_model():
    """The peer-store exchange restated in numpy over W in-process "ranks" with one window each: the same indices the
    kernels use (a token's row once per destination rank at its index inside the pair's block, one 16-byte record per
    assignment, partial rows back at d * Tm + ul, sums in k order of each pair's first assignment).  The result must
    equal the single-rank weighted combine, for skewed and empty ranks, and a window is never larger than its layout."""
    rng = np.random.default_rng(3)
    W, E, k, H, Tm = 4, 16, 4, 8, 12
    e_local = E // W
    Kc = min(k, e_local)
    place_rank = rng.permutation(E) % W                      # a scattered placement
    place_slot = np.zeros(E, np.int64)
    for r in range(W):
        place_slot[place_rank == r] = np.arange(e_local)
    expert_fn = lambda e, rows: rows * (1.0 + e) + 0.25 * e   # any per-expert map of a row
    Ts = [12, 0, 5, 9]                                       # rank 1 has no tokens and still takes part
    xs = [rng.standard_normal((T, H)) for T in Ts]
    ids = [np.stack([rng.permutation(E)[:k] for _ in range(T)]).reshape(T, k) if T else np.zeros((0, k), np.int64) for T in Ts]
    ws = [rng.random((T, k)) for T in Ts]
    # windows
    rx_x = np.full((W, W, Tm, H), np.nan)
    rx_meta = np.full((W, W, Tm * Kc, 3), np.nan)
    disp = np.zeros((W, W, 2), np.int64)
    ret = np.full((W, W, Tm, H), np.nan)
    a_urow, a_first = [], []
    for me in range(W):                                      # push
        A = Ts[me] * k
        flat = ids[me].reshape(-1)
        dest = place_rank[flat]
        order = np.argsort(dest, kind="stable")
        offsets = np.concatenate([[0], np.cumsum(np.bincount(dest, minlength=W))])
        au, af = np.zeros(A, np.int64), np.zeros(A, np.int64)
        u = -1
        ustart = np.zeros(W + 1, np.int64)
        urow = np.zeros(A, np.int64)
        for i in range(A):
            a = order[i]
            first = i == 0 or order[i - 1] // k != a // k or dest[order[i - 1]] != dest[a]
            u += int(first)
            urow[i] = u
        for r in range(W + 1):
            ustart[r] = urow[offsets[r]] if r < W and offsets[r] < A else u + 1
        for i in range(A):
            a, d = order[i], dest[order[i]]
            ul, il = urow[i] - ustart[d], i - offsets[d]
            first = i == 0 or urow[i - 1] != urow[i]
            assert ul < Tm and il < Tm * Kc
            if first:
                rx_x[d, me, ul] = xs[me][a // k]
            rx_meta[d, me, il] = (place_slot[flat[a]], ul, ws[me].reshape(-1)[a])
            au[a], af[a] = d * Tm + ul, int(first)
        for r in range(W):
            disp[r, me] = (offsets[r + 1] - offsets[r], ustart[r + 1] - ustart[r])
        a_urow.append(au); a_first.append(af)
    for me in range(W):                                      # unpack, local experts, partial rows back
        a0 = np.concatenate([[0], np.cumsum(disp[me, :, 0])])
        RA = a0[W]
        slots = np.zeros(RA, np.int64); xrow = np.zeros(RA, np.int64); wt = np.zeros(RA)
        for a in range(RA):
            s = np.searchsorted(a0, a, side="right") - 1
            rec = rx_meta[me, s, a - a0[s]]
            slots[a], xrow[a], wt[a] = int(rec[0]), s * Tm + int(rec[1]), rec[2]
        my_experts = {place_slot[e]: e for e in range(E) if place_rank[e] == me}
        flat_x = rx_x[me].reshape(W * Tm, H)
        ro = np.stack([expert_fn(my_experts[slots[a]], flat_x[xrow[a]]) for a in range(RA)]) if RA else np.zeros((0, H))
        a = 0
        while a < RA:
            b, acc = a, None
            while b < RA and xrow[b] == xrow[a]:
                p = ro[b] * wt[b]
                acc = p if acc is None else p + acc
                b += 1
            s, ul = divmod(xrow[a], Tm)
            ret[s, me, ul] = acc
            a = b
    for me in range(W):                                      # final sums against the single-rank combine
        flat_ret = ret[me].reshape(W * Tm, H)
        for t in range(Ts[me]):
            acc = None
            for j in range(k):
                a = t * k + j
                if a_first[me][a]:
                    v = flat_ret[a_urow[me][a]]
                    acc = v if acc is None else v + acc
            want = sum(expert_fn(ids[me][t, j], xs[me][t]) * ws[me][t, j] for j in range(k))
            assert np.allclose(acc, want, rtol=1e-12), (me, t)
    from __graft_entry__ import load_package
    L = load_package().lib()
    assert L.mlxs_moe_ep_window_bytes(W, Tm, k, E, H) >= W * Tm * H * 6 + W * Tm * Kc * 16 + 2 * W * 128
