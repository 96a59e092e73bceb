"""The one exchange of the scoring path (sum of per-rank Gram matrices) and the row
sharding, run as two gloo ranks on the CPU.  The per-rank Gram is computed with plain
torch here: what is under test is the host-side sharding and reduction logic."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from trak_b200.score_computers import reduce_gram, shard_rows


def test_shard_rows_partition():
    for n in (1, 7, 100, 1_000_003):
        for world in (1, 2, 3, 8):
            spans = [shard_rows(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        X = torch.randn(101, 16, generator=torch.Generator().manual_seed(5))
        lo, hi = shard_rows(X.shape[0], rank, world)
        local = X[lo:hi].T @ X[lo:hi]
        total = reduce_gram(local.clone(), dist.group.WORLD)
        torch.save(total, os.path.join(tmp, f"gram_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_gram_all_reduce_two_ranks(tmp_path):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    X = torch.randn(101, 16, generator=torch.Generator().manual_seed(5))
    want = X.T @ X
    for r in range(2):
        got = torch.load(os.path.join(tmp_path, f"gram_{r}.pt"))
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)


def _worker_empty_shard(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        X = torch.randn(1, 8, generator=torch.Generator().manual_seed(9))   # one train row, two ranks
        lo, hi = shard_rows(X.shape[0], rank, world)
        # a rank without rows contributes a zero Gram and still joins the reduction (what get_xtx does)
        local = X[lo:hi].T @ X[lo:hi] if hi > lo else torch.zeros(8, 8)
        total = reduce_gram(local.clone(), dist.group.WORLD)
        torch.save((hi - lo, total), os.path.join(tmp, f"gram_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_rank_with_an_empty_shard_still_joins_the_reduction(tmp_path):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker_empty_shard, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    X = torch.randn(1, 8, generator=torch.Generator().manual_seed(9))
    sizes = []
    for r in range(2):
        n, got = torch.load(os.path.join(tmp_path, f"gram_{r}.pt"))
        sizes.append(n)
        torch.testing.assert_close(got, X.T @ X)
    assert sorted(sizes) == [0, 1]


def test_reduce_gram_single_process_is_identity():
    g = torch.eye(3)
    assert reduce_gram(g, None) is g
