"""CPU: batch x head partitioning and the output all-gather, world_size 2 over gloo."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tinytorch_b200 import shard


def test_unit_range_covers_everything():
    for n in (1, 7, 64, 128, 2048):
        for w in (1, 2, 3, 4, 8):
            got = [shard.unit_range(n, r, w) for r in range(w)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(got[i][1] == got[i + 1][0] for i in range(w - 1))
            sizes = [e - b for b, e in got]
            assert max(sizes) - min(sizes) <= 1


def test_balanced_ranges_even_out_ragged_work():
    rng = np.random.default_rng(3)
    lens = np.repeat(rng.integers(1024, 8193, size=64), 32)  # config 4: every kv head of a sequence has its length
    for w in (1, 2, 3, 4, 8):
        rs = shard.balanced_ranges(lens.tolist(), w)
        assert rs[0][0] == 0 and rs[-1][1] == len(lens)
        assert all(rs[i][1] == rs[i + 1][0] for i in range(w - 1))
        sums = [int(lens[b:e].sum()) for b, e in rs]
        assert max(sums) <= 1.01 * (sum(sums) / w)
        eq = [int(lens[slice(*shard.unit_range(len(lens), r, w))].sum()) for r in range(w)]
        assert max(sums) <= max(eq)
    # more ranks than units, and zero weights
    assert shard.balanced_ranges([5.0], 3) in ([(0, 0), (0, 1), (1, 1)], [(0, 1), (1, 1), (1, 1)], [(0, 0), (0, 0), (0, 1)])
    rs = shard.balanced_ranges([0, 0, 0, 0], 2)
    assert rs[0][0] == 0 and rs[-1][1] == 4 and rs[0][1] == rs[1][0]


def test_shard_is_a_view_and_keeps_groups_together():
    q = torch.arange(2 * 8 * 3 * 4, dtype=torch.float32).view(2, 8, 3, 4)  # Hq = 8
    k = torch.arange(2 * 2 * 3 * 4, dtype=torch.float32).view(2, 2, 3, 4)  # Hkv = 2 -> 4 kv units
    qs = shard.shard_bh(q, 4, 1, 2)
    ks = shard.shard_bh(k, 4, 1, 2)
    assert qs.shape == (1, 8, 3, 4) and ks.shape == (1, 2, 3, 4)
    assert qs.data_ptr() == q[1].data_ptr() and ks.data_ptr() == k[1].data_ptr()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_units, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.loader import Oracle
    orc = Oracle(threads=1)
    rng = np.random.default_rng(11)
    B, Hq, Hkv, S, D = 1, 6, 3, 32, 64
    q = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    k, v = (rng.standard_normal((B, Hkv, S, D), dtype=np.float32) for _ in range(2))
    tq, tk, tv = (torch.from_numpy(x) for x in (q, k, v))
    ql, kl, vl = (shard.shard_bh(t, n_units, rank, world) for t in (tq, tk, tv))
    o_local, _ = orc.fwd(ql.numpy(), kl.numpy(), vl.numpy(), causal=True)
    full = shard.all_gather_output(torch.from_numpy(o_local), n_units, world)
    want, _ = orc.fwd(q, k, v, causal=True)
    ok = np.array_equal(full.numpy(), want.reshape(B * Hq, S, D))
    open(os.path.join(out_dir, "rank%d.%s" % (rank, "ok" if ok else "bad")), "w").close()
    dist.destroy_process_group()


def test_two_ranks_gather_equals_single(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), 3, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["rank0.ok", "rank1.ok"]


def _worker_empty(rank, world, port, out_dir):
    # one unit over two ranks: rank 1 owns nothing and still takes part in the gather
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g, L, D = 2, 4, 8
    full = torch.arange(g * L * D, dtype=torch.float32).view(1, g, L, D)
    b0, b1 = shard.unit_range(1, rank, world)
    local = full[:, b0 * g:b1 * g]
    ok = True
    for gs in (g, None):  # group size given / agreed on by the ranks
        got = shard.all_gather_output(local, 1, world, group_size=gs)
        ok = ok and torch.equal(got, full[0])
    # explicit (work-balanced) ranges: three units of g heads, split 2 + 1
    full3 = torch.arange(3 * g * L * D, dtype=torch.float32).view(1, 3 * g, L, D)
    rs = [(0, 2), (2, 3)]
    b0, b1 = rs[rank]
    got = shard.all_gather_output(full3[:, b0 * g:b1 * g], 3, world, group_size=g, ranges=rs)
    ok = ok and torch.equal(got, full3[0])
    open(os.path.join(out_dir, "rank%d.%s" % (rank, "ok" if ok else "bad")), "w").close()
    dist.destroy_process_group()


def test_gather_with_a_rank_that_owns_no_unit(tmp_path):
    world = 2
    mp.spawn(_worker_empty, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["rank0.ok", "rank1.ok"]
