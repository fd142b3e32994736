"""Host logic of the sharded APSP solves (cuasr_b200/apsp.py) on CPU: two gloo ranks, with the CPU oracle standing
in for the device SRGEMM; a gloo all-gather (repeated squaring) or broadcast (blocked Floyd-Warshall) for the
exchange."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from cuasr_b200 import DType, Layout, Op
from cuasr_b200.apsp import ShardedSquaring, random_graph

COL = Layout.COLUMN_MAJOR
INF = np.float32(np.inf)


class OracleBackend:
    """Backend of ShardedSquaring that computes each block with the CPU oracle and exchanges with torch.distributed."""

    def __init__(self, n, flat, world):
        self.n, self.world = n, world
        self.bufs = [flat.copy(), np.zeros_like(flat)]

    def srgemm_block(self, cur, nxt, c0, cols):
        n = self.n
        src, dst = self.bufs[cur], self.bufs[nxt]
        blk = slice(c0 * n, (c0 + cols) * n)
        out = np.empty(cols * n, np.float32)
        oracle.srgemm(Op.MINIMUM, Op.PLUS, DType.F32, (COL, COL, COL), (n, cols, n), 0.0, src, n,
                      np.ascontiguousarray(src[blk]), n, 0.0, np.ascontiguousarray(src[blk]), n, out, n, INF, 1)
        dst[blk] = out

    def exchange(self, nxt, c0, cols):
        if self.world == 1:
            return
        n = self.n
        mine = torch.from_numpy(self.bufs[nxt][c0 * n:(c0 + cols) * n].copy())
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine)
        self.bufs[nxt][:] = torch.cat(parts).numpy()

    def matrix(self, which):
        return self.bufs[which]


def floyd_warshall(adj):
    d = adj.astype(np.float64).copy()
    for k in range(d.shape[0]):
        d = np.minimum(d, d[:, k:k + 1] + d[k:k + 1, :])
    return d


def _worker(rank, world, port, n, seed, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    flat = random_graph(n, 0.05, seed, "cpu").numpy()
    solver = ShardedSquaring(n, rank, world, OracleBackend(n, flat, world))
    steps = solver.solve()
    assert steps == ShardedSquaring.squarings_needed(n)
    out[rank] = solver.result().copy()
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_ranks_equal_one_rank_and_floyd_warshall():
    n, seed, world = 96, 5, 2
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), n, seed, out), nprocs=world, join=True)
    flat = random_graph(n, 0.05, seed, "cpu").numpy()
    single = ShardedSquaring(n, 0, 1, OracleBackend(n, flat, 1))
    single.solve()
    for rank in range(world):
        assert np.array_equal(out[rank], single.result()), f"rank {rank} differs from the single-rank solve"
    # weights are small integers, so fp32 path lengths are exact and must equal Floyd-Warshall's
    want = floyd_warshall(flat.reshape(n, n).T)
    got = single.result().reshape(n, n).T.astype(np.float64)
    assert np.array_equal(got, want)


def test_sharding_arithmetic():
    assert ShardedSquaring.squarings_needed(16384) == 14
    assert ShardedSquaring.squarings_needed(2) == 1
    s = ShardedSquaring(64, 3, 4, backend=None)
    assert (s.c0, s.cols) == (48, 16)
    with pytest.raises(ValueError):
        ShardedSquaring(10, 0, 4, backend=None)


def test_graph_generator_blocks_match_the_whole():
    n = 40
    whole = random_graph(n, 0.2, 9, "cpu")
    part = random_graph(n, 0.2, 9, "cpu", rows=(8, 16))
    assert torch.equal(whole[8 * n:24 * n], part)
    m = whole.view(n, n)
    assert torch.all(m.diagonal() == 0)
    present = m[~torch.eye(n, dtype=torch.bool)]
    present = present[torch.isfinite(present)]
    assert present.min() >= 1 and present.max() <= 100 and torch.all(present == present.round())


# ---- blocked Floyd-Warshall over ranks: ownership, look-ahead and panel rotation on CPU -----------------------
def _host_floyd_warshall_class():
    from cuasr_b200.apsp import BlockedFloydWarshall

    _, fn = oracle._load(oracle.ORACLE_PATH, "cuasr_oracle_srgemm")
    zero, inf = np.zeros(1, np.float32), np.full(1, np.inf, np.float32)

    class HostFloydWarshall(BlockedFloydWarshall):
        """The multi-rank driver unchanged, with the CPU oracle as the block product: its "device addresses" are
        addresses of CPU tensors here.  Broadcast mode only (the push mode needs peer-mapped GPU memory)."""

        def _srgemm(self, m, n, k, A, lda, B, ldb, C, ldc, D, ldd, extras=()):
            assert not extras
            st = fn(int(Op.MINIMUM), int(Op.PLUS), int(DType.F32), int(COL), int(COL), int(COL), m, n, k,
                    zero.ctypes.data, A, lda, B, ldb, zero.ctypes.data, C, ldc, D, ldd, inf.ctypes.data, 1)
            assert st == 0
            self.launches += 1

    return HostFloydWarshall


def _fw_worker(rank, world, port, n, block, seed, distribution, look_ahead, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    solver = _host_floyd_warshall_class()(n, block, rank, world, "cpu", mode="allgather", distribution=distribution,
                                          look_ahead=look_ahead)
    solver.load_columns(torch.cat([random_graph(n, 0.05, seed, "cpu", rows=(kb * block, block))
                                   for kb in solver.owned_blocks()]))
    solver.solve()
    solver.solve()        # the closure is a fixed point; the second solve re-uses every panel buffer
    out[rank] = (solver.owned_blocks(), solver.result_columns().numpy().copy())
    dist.destroy_process_group()


@pytest.mark.parametrize("distribution,look_ahead", [("cyclic", True), ("cyclic", False), ("contiguous", True)])
def test_blocked_floyd_warshall_two_ranks(distribution, look_ahead):
    n, block, seed, world = 96, 16, 11, 2
    out = mp.Manager().dict()
    mp.spawn(_fw_worker, args=(world, _free_port(), n, block, seed, distribution, look_ahead, out), nprocs=world,
             join=True)
    flat = random_graph(n, 0.05, seed, "cpu").numpy()
    want = floyd_warshall(flat.reshape(n, n).T).T.astype(np.float32).reshape(-1)       # column-major, like `flat`
    blocks_seen = []
    for rank in range(world):
        blocks, cols = out[rank]
        blocks_seen += blocks
        mine = np.concatenate([want[kb * block * n:(kb + 1) * block * n] for kb in blocks])
        assert np.array_equal(cols, mine), f"{distribution}: rank {rank}"
    assert sorted(blocks_seen) == list(range(n // block))
    expect0 = [0, 2, 4] if distribution == "cyclic" else [0, 1, 2]
    assert out[0][0] == expect0


def test_floyd_warshall_ownership_arithmetic():
    cls = _host_floyd_warshall_class()
    s = cls(64, 8, 1, 4, "cpu", mode="allgather")
    assert s.owned_blocks() == [1, 5] and s.owner(6) == 2 and s.local_column(5) == 8 and s.look_ahead
    c = cls(64, 8, 1, 4, "cpu", mode="allgather", distribution="contiguous")
    assert c.owned_blocks() == [2, 3] and c.owner(6) == 3 and c.local_column(3) == 8
    with pytest.raises(ValueError):
        cls(64, 12, 0, 4, "cpu", mode="allgather")
    with pytest.raises(ValueError):
        cls(64, 8, 0, 4, "cpu", mode="allgather", distribution="random")
