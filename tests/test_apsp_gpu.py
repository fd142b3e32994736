"""Repeated-squaring APSP on the GPU against the CPU oracle and Floyd-Warshall; multi-GPU modes where two or more
GPUs are visible."""
import os
import socket

import numpy as np
import pytest

import oracle
from cuasr_b200 import DType, Layout, Op
from cuasr_b200.apsp import BlockedFloydWarshall, CudaBackend, ShardedSquaring, random_graph

pytestmark = pytest.mark.gpu
COL = Layout.COLUMN_MAJOR


def cpu_apsp(flat, n, squarings):
    cur = flat.copy()
    inf = np.float32(np.inf)
    for _ in range(squarings):
        nxt = np.empty_like(cur)
        oracle.srgemm(Op.MINIMUM, Op.PLUS, DType.F32, (COL, COL, COL), (n, n, n), 0.0, cur, n, cur, n, 0.0, cur, n,
                      nxt, n, inf, 0)
        cur = nxt
    return cur


def test_single_gpu_apsp_matches_cpu(cuda_device):
    """Full solve at n = 1024 (the whole algorithm on the CPU as well), every squaring compared bit for bit."""
    import torch
    n, seed = 1024, 11
    flat = random_graph(n, 0.01, seed, cuda_device)
    backend = CudaBackend(n, 0, 1, cuda_device)
    backend.load(0, flat)
    solver = ShardedSquaring(n, 0, 1, backend)
    host = flat.cpu().numpy()
    for step in range(ShardedSquaring.squarings_needed(n)):
        solver.step()
        host = cpu_apsp(host, n, 1)
        torch.cuda.synchronize()
        assert np.array_equal(solver.result().cpu().numpy(), host), f"squaring {step} differs"
    # the fixed point: one more squaring changes nothing, and distances satisfy the triangle inequality
    again = cpu_apsp(host, n, 1)
    assert np.array_equal(again, host)


def test_apsp_blocks_at_full_size_property(cuda_device):
    """n = 4096: sampled column blocks of one squaring against the oracle fed the same input."""
    import torch
    n = 4096
    flat = random_graph(n, 0.01, 3, cuda_device)
    backend = CudaBackend(n, 0, 1, cuda_device)
    backend.load(0, flat)
    solver = ShardedSquaring(n, 0, 1, backend)
    solver.step()
    solver.step()
    before = backend.matrix(solver.cur).clone()
    solver.step()
    torch.cuda.synchronize()
    src = before.cpu().numpy()
    got = solver.result().cpu().numpy()
    inf = np.float32(np.inf)
    for c0 in (0, 1504, 4064):
        blk = slice(c0 * n, (c0 + 32) * n)
        want = np.empty(32 * n, np.float32)
        oracle.srgemm(Op.MINIMUM, Op.PLUS, DType.F32, (COL, COL, COL), (n, 32, n), 0.0, src, n,
                      np.ascontiguousarray(src[blk]), n, 0.0, np.ascontiguousarray(src[blk]), n, want, n, inf, 0)
        assert np.array_equal(got[blk], want), f"columns {c0}..{c0 + 31}"
    # squaring never lengthens a path
    assert bool((solver.result() <= before).all())


def test_blocked_floyd_warshall_equals_repeated_squaring(cuda_device):
    """Integer weights: both algorithms are exact, so the distances must be identical bit for bit."""
    import torch
    n, seed = 1024, 13
    flat = random_graph(n, 0.01, seed, cuda_device)
    want = cpu_apsp(flat.cpu().numpy(), n, ShardedSquaring.squarings_needed(n))
    for block, look_ahead in ((256, False), (512, False), (1024, False), (128, True), (256, True), (1024, True)):
        # look_ahead reorders the launches the way the multi-rank solve does (next block's columns first)
        solver = BlockedFloydWarshall(n, block, 0, 1, cuda_device, look_ahead=look_ahead)
        solver.load_columns(flat)
        solver.solve()
        torch.cuda.synchronize()
        assert np.array_equal(solver.result_columns().cpu().numpy(), want), f"block {block} look_ahead {look_ahead}"


def _fw_rank(rank, world, port, n, seed, mode, distribution, out):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    cols = n // world
    solver = BlockedFloydWarshall(n, 128, rank, world, dev, mode=mode, distribution=distribution)
    solver.load_columns(torch.cat([random_graph(n, 0.01, seed, dev, rows=(kb * 128, 128)) for kb in solver.owned_blocks()]))
    out[("blocks", mode, rank)] = solver.owned_blocks()
    solver.solve()
    solver.solve()          # a second solve of the closed matrix changes nothing and reuses the panel buffers
    torch.cuda.synchronize()
    from cuasr_b200 import device_status
    out[("status", mode, rank)] = device_status()     # 3 would mean a wait for a peer's flag ran out
    out[(mode, rank)] = solver.result_columns().cpu().numpy()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("distribution", ["cyclic", "contiguous"])
@pytest.mark.parametrize("mode", ["allgather", "push"])
def test_multi_gpu_blocked_floyd_warshall(mode, distribution):
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    n, seed = 1024, 27
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_fw_rank, args=(world, port, n, seed, mode, distribution, out), nprocs=world, join=True)
    want = cpu_apsp(random_graph(n, 0.01, seed, "cpu").numpy(), n, ShardedSquaring.squarings_needed(n))
    for rank in range(world):
        assert out[("status", mode, rank)] == 0
        mine = np.concatenate([want[kb * 128 * n:(kb + 1) * 128 * n] for kb in out[("blocks", mode, rank)]])
        assert np.array_equal(out[(mode, rank)], mine), f"{mode} {distribution}: rank {rank}"


def _rank(rank, world, port, n, seed, mode, out):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    backend = CudaBackend(n, rank, world, dev, mode=mode)
    backend.load(0, random_graph(n, 0.01, seed, dev))
    solver = ShardedSquaring(n, rank, world, backend)
    solver.solve()
    torch.cuda.synchronize()
    out[(mode, rank)] = solver.result().cpu().numpy()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["allgather", "push"])
def test_multi_gpu_apsp(mode):
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    n, seed = 1024, 21
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_rank, args=(world, port, n, seed, mode, out), nprocs=world, join=True)
    want = cpu_apsp(random_graph(n, 0.01, seed, "cpu").numpy(), n, ShardedSquaring.squarings_needed(n))
    for rank in range(world):
        assert np.array_equal(out[(mode, rank)], want), f"{mode}: rank {rank} differs from the CPU solve"


def _host_pipeline_rank(rank, world, port, m, n, k, exchange, out):
    """One rank of a sharded host-buffer SRGEMM: its columns of D, its columns of B, its share of every K piece of A."""
    import torch
    import torch.distributed as dist
    from cuasr_b200 import DType, HostSrgemm, Layout, RINGS, Srgemm, device_status
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    g = torch.Generator().manual_seed(1234)
    A = torch.randint(-8, 9, (m * k,), generator=g).float()
    B = torch.randint(-8, 9, (k * n,), generator=g).float()
    C = torch.randint(-8, 9, (m * n,), generator=g).float()
    cols = n // world
    col = Layout.COLUMN_MAJOR
    op = Srgemm(*RINGS["minimum_plus"], DType.F32, col, col, col)
    pipe = HostSrgemm(op, m, cols, k, 0.0, 0.0, dev, chunks=2, group=dist.group.WORLD, rank=rank, world=world,
                      exchange=exchange)
    share = torch.cat([A[a:b] for a, b in pipe.shared_share_layout()]).pin_memory()
    hB = B[rank * cols * k:(rank + 1) * cols * k].clone().pin_memory()
    hC = C[rank * cols * m:(rank + 1) * cols * m].clone().pin_memory()
    hD = torch.empty(cols * m, dtype=torch.float32).pin_memory()
    for _ in range(2):
        hD.zero_()
        pipe(share, hB, hC, hD)
        torch.cuda.synchronize()
    out[("k_pieces", rank)] = pipe.k_pieces
    out[("status", rank)] = device_status()
    out[("D", rank)] = hD.numpy().copy()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["p2p", "nccl"])
def test_multi_gpu_host_buffer_pipeline(exchange):
    """Ranks that shard the columns of D bring 1/world of every K piece of A each and complete the pieces over
    NVLink (peer copies + arrival words, or NCCL all-gathers); the result is the one-shot host SRGEMM's, bit for
    bit."""
    import torch
    import torch.multiprocessing as mp
    import oracle
    from cuasr_b200 import DType, Layout, Op
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    m, n, k = 1024, 1024 * world, 1024
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_host_pipeline_rank, args=(world, port, m, n, k, exchange, out), nprocs=world, join=True)
    g = torch.Generator().manual_seed(1234)
    A = torch.randint(-8, 9, (m * k,), generator=g).float().numpy()
    B = torch.randint(-8, 9, (k * n,), generator=g).float().numpy()
    C = torch.randint(-8, 9, (m * n,), generator=g).float().numpy()
    col = Layout.COLUMN_MAJOR
    want = np.empty_like(C)
    oracle.srgemm(Op.MINIMUM, Op.PLUS, DType.F32, (col, col, col), (m, n, k), 0.0, A, m, B, k, 0.0, C, m, want, m,
                  np.finfo(np.float32).max)
    cols = n // world
    for rank in range(world):
        assert out[("status", rank)] == 0
        assert out[("k_pieces", rank)] == 4
        assert np.array_equal(out[("D", rank)], want[rank * cols * m:(rank + 1) * cols * m]), f"rank {rank}"
