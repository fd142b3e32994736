"""The C entry points of include/cuasr_b200_apsp.h: argument checks and sizes without a GPU, whole solves on one."""
import numpy as np
import pytest

from cuasr_b200 import DType, Status, apsp


def test_workspace_sizes_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("with a device the sizes also hold the optional SRGEMM scratch")
    assert apsp.device_solve_workspace_size(DType.F32, apsp.REPEATED_SQUARING, 1024) == 4 * 1024 * 1024
    assert apsp.device_solve_workspace_size(DType.F64, apsp.REPEATED_SQUARING, 1000) == 8 * 1000 * 1000
    # Floyd-Warshall: column panel + row panel + two diagonal blocks
    assert apsp.device_solve_workspace_size(DType.F32, apsp.BLOCKED_FLOYD_WARSHALL, 4096, 512) == 4 * (2 * 4096 * 512 + 2 * 512 * 512)
    assert apsp.device_solve_workspace_size(DType.F32, apsp.BLOCKED_FLOYD_WARSHALL, 4096) == 4 * (2 * 4096 * 1024 + 2 * 1024 * 1024)
    assert apsp.device_solve_workspace_size(DType.S32, apsp.REPEATED_SQUARING, 1024) == 0      # not a distance type
    assert apsp.device_solve_workspace_size(DType.F32, 7, 1024) == 0
    assert apsp.device_solve_workspace_size(DType.F32, apsp.BLOCKED_FLOYD_WARSHALL, 1024, 30) == 0   # block % 4


def test_argument_checks_need_no_device():
    import ctypes
    from cuasr_b200 import _lib
    lib = _lib.load()
    call = lambda **kw: Status(lib.cuasr_b200_apsp(ctypes.byref(apsp._apsp_args(**kw))))
    ok = dict(dtype=DType.F32, algorithm=apsp.REPEATED_SQUARING, n=64, D=4096, workspace=8192, workspace_bytes=1 << 20)
    assert call(**dict(ok, D=0)) == Status.kErrorInvalidProblem
    assert call(**dict(ok, n=0)) == Status.kErrorInvalidProblem
    assert call(**dict(ok, ldd=63)) == Status.kErrorInvalidProblem
    assert call(**dict(ok, D=4098)) == Status.kErrorMisalignedOperand
    assert call(**dict(ok, workspace=0)) == Status.kErrorWorkspaceNull
    assert call(**dict(ok, workspace_bytes=64 * 64 * 4 - 1)) == Status.kErrorWorkspaceNull
    assert call(**dict(ok, workspace=8200)) == Status.kErrorMisalignedOperand
    assert lib.cuasr_b200_apsp(None) == int(Status.kErrorInvalidProblem)
    assert apsp.shard_squaring(DType.F32, 64, 32, 64, 4096, 64, 8192, 64) == Status.kErrorInvalidProblem   # columns past n
    assert apsp.shard_squaring(DType.F32, 64, 0, 32, 0, 64, 8192, 64) == Status.kErrorInvalidProblem
    assert apsp.shard_squaring(DType.F32, 64, 0, 32, 4096, 64, 8192, 64, peer_next=[1] * 8) == Status.kErrorInvalidProblem
    assert lib.cuasr_b200_apsp_shard_squaring(None) == int(Status.kErrorInvalidProblem)


def test_multi_gpu_entry_point_partition_and_argument_checks():
    """cuasr_b200_apsp_multi: how the columns are dealt out, and what is refused before any GPU is touched."""
    assert apsp.multi_partition(16384, 8, 0) == (0, 2048)
    assert apsp.multi_partition(16384, 8, 7) == (14336, 2048)
    assert apsp.multi_partition(1000, 4, 2) == (500, 250)
    assert apsp.multi_partition(1000, 3, 0) is None          # n must divide
    assert apsp.multi_partition(1024, 9, 0) is None          # at most 8 GPUs (one launch has 8 destinations)
    assert apsp.multi_partition(1024, 2, 2) is None
    st, _, _ = apsp.multi_device_solve(DType.F32, 1000, [0, 1, 2], [4096] * 3, [8192] * 3)
    assert st == Status.kErrorInvalidProblem                 # 1000 columns over 3 GPUs
    st, _, _ = apsp.multi_device_solve(DType.F32, 1024, [0, 0], [4096] * 2, [8192] * 2)
    assert st == Status.kErrorInvalidProblem                 # the same device twice
    st, _, _ = apsp.multi_device_solve(DType.F32, 1024, [0, 1], [4096, 0], [8192] * 2)
    assert st == Status.kErrorInvalidProblem                 # a missing buffer
    st, _, _ = apsp.multi_device_solve(DType.S32, 1024, [0], [4096], [8192])
    assert st == Status.kErrorInvalidProblem                 # not a distance type
    st, _, _ = apsp.multi_device_solve(DType.F32, 1024, [0], [4096], [8192], ldd=1000)
    assert st == Status.kErrorInvalidProblem
    # the Floyd-Warshall form: whole blocks per GPU, and a workspace on every GPU
    fw = dict(algorithm=apsp.BLOCKED_FLOYD_WARSHALL, block=256)
    need = apsp.multi_device_workspace_size(DType.F32, 4096, 2, block=512)
    assert need == 4 * (3 * 4096 * 512 + 512 * 2048 + 2 * 512 * 512)      # three column panels, a row piece, two blocks
    assert apsp.multi_device_workspace_size(DType.F32, 4096, 3) == 0
    assert apsp.multi_device_workspace_size(DType.F32, 4096, 2, apsp.REPEATED_SQUARING) == 0
    st, _, _ = apsp.multi_device_solve(DType.F32, 1024, [0, 1], [4096] * 2, **fw)
    assert st == Status.kErrorWorkspaceNull
    st, _, _ = apsp.multi_device_solve(DType.F32, 1024, [0, 1], [4096] * 2, workspaces=[4096] * 2, workspace_bytes=100, **fw)
    assert st == Status.kErrorWorkspaceNull
    st, _, _ = apsp.multi_device_solve(DType.F32, 1024, [0, 1], [4096] * 2, workspaces=[4096, 4100], workspace_bytes=1 << 30, **fw)
    assert st == Status.kErrorMisalignedOperand
    st, _, _ = apsp.multi_device_solve(DType.F32, 1024, [0, 1], [4096] * 2, workspaces=[4096] * 2, workspace_bytes=1 << 30,
                                       algorithm=apsp.BLOCKED_FLOYD_WARSHALL, block=384)     # 1024 % (2 x 384)
    assert st == Status.kErrorInvalidProblem


@pytest.mark.gpu
@pytest.mark.parametrize("n,block,pad,dt", [(1024, 128, 0, DType.F32), (1536, 256, 8, DType.F32), (768, 64, 0, DType.F64)])
def test_multi_gpu_floyd_warshall_from_one_process(cuda_device, n, block, pad, dt):
    """cuasr_b200_apsp_multi, blocked Floyd-Warshall: column blocks dealt out cyclically over the GPUs of the box
    (one GPU included), the column panel of every step stored into every GPU's panel buffer by the owner's
    epilogue; the distributed closure, put together again, must equal the host's."""
    import torch
    np_t, t_t = (np.float32, torch.float32) if dt == DType.F32 else (np.float64, torch.float64)
    w = _graph(n, n + block, np_t)
    want = _closure(w)
    G = min(torch.cuda.device_count(), 4)
    while n % (G * block):
        G -= 1
    ld, cols, blocks = n + pad, n // G, n // block
    owned = [[kb for kb in range(blocks) if kb % G == g] for g in range(G)]
    bufs = []
    for g in range(G):
        buf = np.full((cols, ld), 7.0, dtype=np_t)               # column c of the piece is row c of this array
        for i, kb in enumerate(owned[g]):
            buf[i * block:(i + 1) * block, :n] = w[:, kb * block:(kb + 1) * block].T
        bufs.append(torch.from_numpy(buf).to(f"cuda:{g}"))
    need = apsp.multi_device_workspace_size(dt, n, G, block=block)
    assert need > 0
    ws = [torch.empty(need, dtype=torch.uint8, device=f"cuda:{g}") for g in range(G)]
    for g in range(G):
        torch.cuda.synchronize(g)
    st, which, status = apsp.multi_device_solve(dt, n, list(range(G)), [t.data_ptr() for t in bufs], ldd=ld,
                                                workspaces=[t.data_ptr() for t in ws], workspace_bytes=need,
                                                algorithm=apsp.BLOCKED_FLOYD_WARSHALL, block=block)
    assert st == Status.kSuccess and which == 0 and status == [0] * G
    got = np.empty((n, n), dtype=np.float64)
    for g in range(G):
        piece = bufs[g].cpu().numpy()
        assert np.all(piece[:, n:] == 7.0)                       # the padding of the leading dimension stays
        for i, kb in enumerate(owned[g]):
            got[:, kb * block:(kb + 1) * block] = piece[i * block:(i + 1) * block, :n].T
    assert np.array_equal(got, want)
    torch.cuda.set_device(0)


@pytest.mark.gpu
@pytest.mark.parametrize("n,ld", [(1024, 1024), (768, 776)])
def test_multi_gpu_solve_from_one_process(cuda_device, n, ld):
    """cuasr_b200_apsp_multi on every GPU of the box that divides n (one GPU included: the same code path with no
    peers): plain cudaMalloc'ed buffers, host threads and peer stores only; the closure must equal the host's."""
    import torch
    w = _graph(n, n, np.float32)
    want = _closure(w)
    G = torch.cuda.device_count()
    while n % G:
        G -= 1
    G = min(G, 4)
    buf = np.full((n, ld), 7.0, dtype=np.float32)
    buf[:, :n] = w.T
    b0 = [torch.from_numpy(buf).to(f"cuda:{g}") for g in range(G)]
    b1 = [torch.full((n * ld,), -3.0, dtype=torch.float32, device=f"cuda:{g}") for g in range(G)]
    for g in range(G):
        torch.cuda.synchronize(g)
    st, which, status = apsp.multi_device_solve(DType.F32, n, list(range(G)), [t.data_ptr() for t in b0],
                                                [t.data_ptr() for t in b1], ldd=ld)
    assert st == Status.kSuccess and status == [0] * G
    for g in range(G):
        got = (b0 if which == 0 else b1)[g].cpu().numpy().reshape(n, ld)
        assert np.array_equal(got[:, :n].T.astype(np.float64), want), f"GPU {g}"
    torch.cuda.set_device(0)


def _graph(n, seed, dtype):
    rng = np.random.default_rng(seed)
    w = rng.integers(1, 101, size=(n, n)).astype(dtype)
    w[rng.random((n, n)) >= 0.02] = np.inf
    np.fill_diagonal(w, 0)
    return w


def _closure(w):
    from scipy.sparse.csgraph import floyd_warshall
    return floyd_warshall(np.where(np.isinf(w), 0, w).astype(np.float64), directed=True)


@pytest.mark.gpu
@pytest.mark.parametrize("algorithm", [apsp.REPEATED_SQUARING, apsp.BLOCKED_FLOYD_WARSHALL])
@pytest.mark.parametrize("n,ld,block,dt", [(1024, 1024, 256, DType.F32), (1000, 1008, 256, DType.F32), (333, 333, 0, DType.F64),
                                           (1537, 1540, 512, DType.F32)])
def test_device_solve_equals_floyd_warshall_on_the_host(cuda_device, algorithm, n, ld, block, dt):
    import torch
    np_t = np.float32 if dt == DType.F32 else np.float64
    w = _graph(n, n + block, np_t)
    want = _closure(w)              # integer weights: exact in either element type, so equality is bit for bit
    buf = np.full((n, ld), 7.0, dtype=np_t)          # column j of the matrix is row j of this array
    buf[:, :n] = w.T
    D = torch.from_numpy(buf).cuda()
    assert apsp.device_solve(D, n, dt, algorithm, ldd=ld, block=block) == Status.kSuccess
    torch.cuda.synchronize()
    got = D.cpu().numpy()
    assert np.array_equal(got[:, :n].T.astype(np.float64), want)
    assert np.all(got[:, n:] == 7.0)                 # the padding of every column is untouched


@pytest.mark.gpu
def test_shard_squaring_pushes_to_every_destination(cuda_device):
    """Two ranks emulated one after the other on one GPU: each computes its half of the columns and stores it into
    both next-iterate matrices; together they must equal one unsharded squaring."""
    import torch
    n = 512
    w = _graph(n, 5, np.float32)
    cur = torch.from_numpy(np.ascontiguousarray(w.T)).cuda()
    nxt = [torch.zeros_like(cur) for _ in range(2)]
    s = torch.cuda.current_stream().cuda_stream
    for rank in range(2):
        st = apsp.shard_squaring(DType.F32, n, rank * 256, 256, cur.data_ptr(), n, nxt[rank].data_ptr(), n,
                                 peer_next=[nxt[1 - rank].data_ptr()], stream=s)
        assert st == Status.kSuccess
    whole = cur.clone()
    assert apsp.device_solve(whole, n, DType.F32, apsp.REPEATED_SQUARING, iterations=1) == Status.kSuccess
    torch.cuda.synchronize()
    assert torch.equal(nxt[0], whole) and torch.equal(nxt[1], whole)


@pytest.mark.gpu
def test_flags_raise_wait_and_a_wait_that_runs_out(cuda_device):
    """The one-sided flags of the sharded Floyd-Warshall solve, on one stream of one GPU: a raised word lets the wait
    through, values only grow, and a wait nothing answers ends by itself with status 3 instead of hanging."""
    import ctypes
    import torch
    from cuasr_b200 import _lib, device_status
    lib = _lib.load()
    words = torch.zeros(8, dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    ptrs = (ctypes.c_void_p * 3)(*[words.data_ptr() + 4 * i for i in range(3)])
    assert lib.cuasr_b200_flag_raise(ptrs, 3, 5, s) == 0
    assert lib.cuasr_b200_flag_wait(words.data_ptr(), 3, 5, 100, s) == 0
    assert lib.cuasr_b200_flag_raise(ptrs, 3, 3, s) == 0                     # lower than what is there: no effect
    assert device_status() == 0
    assert words.tolist() == [5, 5, 5, 0, 0, 0, 0, 0]
    assert lib.cuasr_b200_flag_wait(words.data_ptr() + 12, 1, 1, 50, s) == 0   # word 3 stays 0: runs out after 50 ms
    assert device_status() == 3
    assert device_status() == 0                                              # reading the status clears it
    assert lib.cuasr_b200_flag_wait(words.data_ptr(), 1, 1, 0, s) == int(Status.kErrorInvalidProblem)
    assert lib.cuasr_b200_flag_raise(ptrs, 9, 1, s) == int(Status.kErrorInvalidProblem)


def test_walk_follows_a_predecessor_matrix():
    P = [[-1] * 5 for _ in range(5)]
    P[0][4], P[0][2], P[2][4] = 2, 1, 3                 # 0 -> 4 splits at 2; 0 -> 2 at 1; 2 -> 4 at 3
    assert apsp.walk(P, 0, 4) == [0, 1, 2, 3, 4]
    assert apsp.walk(P, 3, 4) == [3, 4]
    with pytest.raises(ValueError):                     # a matrix that describes no path must not loop for ever
        apsp.walk([[0, 1], [0, 1]], 0, 1)


def test_predecessor_arguments_are_checked_without_a_device():
    import ctypes
    from cuasr_b200 import _lib
    lib = _lib.load()
    call = lambda **kw: Status(lib.cuasr_b200_apsp(ctypes.byref(apsp._apsp_args(**kw))))
    ok = dict(dtype=DType.F32, algorithm=apsp.BLOCKED_FLOYD_WARSHALL, n=64, D=4096, workspace=8192, workspace_bytes=1 << 20,
              parent=1 << 16)
    assert call(**dict(ok, ld_parent=63)) == Status.kErrorInvalidProblem
    assert call(**dict(ok, parent=(1 << 16) + 2)) == Status.kErrorMisalignedOperand


@pytest.mark.gpu
@pytest.mark.parametrize("algorithm", [apsp.REPEATED_SQUARING, apsp.BLOCKED_FLOYD_WARSHALL])
@pytest.mark.parametrize("n,ld,ldp,block,dt", [(512, 512, 512, 128, DType.F32), (1000, 1008, 1004, 256, DType.F32),
                                               (300, 300, 300, 64, DType.F64)])
def test_device_solve_with_predecessors(cuda_device, algorithm, n, ld, ldp, block, dt):
    """The solve with `parent`: the same distances, bit for bit, and a predecessor matrix every entry of which
    splits its pair into two shorter shortest paths; walking it gives paths made of edges of the input whose weights
    add up to the distance."""
    import torch
    np_t = np.float32 if dt == DType.F32 else np.float64
    w = _graph(n, 3 * n + block, np_t)
    want = _closure(w)
    buf = np.full((n, ld), 7.0, dtype=np_t)
    buf[:, :n] = w.T
    D = torch.from_numpy(buf).cuda()
    P = torch.full((n, ldp), -1, dtype=torch.int32, device="cuda")
    assert apsp.device_solve(D, n, dt, algorithm, ldd=ld, block=block, parent=P, ld_parent=ldp) == Status.kSuccess
    torch.cuda.synchronize()
    dist = D.cpu().numpy()[:, :n].T.astype(np.float64)          # dist[i, j]
    par = P.cpu().numpy()[:, :n].T                              # par[i, j]
    assert np.array_equal(dist, want)
    assert np.all(P.cpu().numpy()[:, n:] == -1)                 # the padding of the predecessor matrix is untouched
    i, j = np.nonzero(par >= 0)
    k = par[i, j]
    assert np.all((k != i) & (k != j) & (k < n))
    assert np.array_equal(dist[i, j], dist[i, k] + dist[k, j])  # every predecessor splits its pair exactly
    direct = par < 0
    assert np.array_equal(dist[direct], w.astype(np.float64)[direct])   # no predecessor: an edge (or nothing) of the input
    rng = np.random.default_rng(n)
    checked = 0
    for a, b in rng.integers(0, n, size=(400, 2)):
        if a == b or not np.isfinite(dist[a, b]):
            continue
        path = apsp.walk(par, int(a), int(b))
        assert path[0] == a and path[-1] == b and len(set(path)) == len(path)
        assert sum(float(w[u, v]) for u, v in zip(path, path[1:])) == dist[a, b]
        checked += 1
    assert checked > 50


def test_multi_gpu_solve_stops_together_when_no_device_can_be_used():
    """A GPU that cannot be selected fails its host thread before the first step; the threads agree on that at their
    first barrier and all of them leave without launching anything (no thread is left waiting for the others).
    Without any GPU every thread fails that way."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("the buffers below are not real")
    st, _, _ = apsp.multi_device_solve(DType.F32, 256, [0, 1], [4096, 4096], [8192, 8192])
    assert st == Status.kErrorInternal
    st, _, _ = apsp.multi_device_solve(DType.F32, 256, [0, 1], [4096, 4096], workspaces=[4096, 8192], workspace_bytes=1 << 30,
                                       algorithm=apsp.BLOCKED_FLOYD_WARSHALL, block=64)
    assert st == Status.kErrorInternal


@pytest.mark.gpu
def test_multi_gpu_solve_stops_together_when_one_device_cannot_be_used(cuda_device):
    """The same with one good GPU and an ordinal that does not exist: the good GPU's thread learns of the failure at
    the first barrier and launches nothing."""
    import torch
    n = 256
    D = [torch.zeros(n * n, dtype=torch.float32, device="cuda:0") for _ in range(2)]
    st, _, _ = apsp.multi_device_solve(DType.F32, n, [0, 99], [D[0].data_ptr(), 4096], [D[1].data_ptr(), 8192])
    assert st in (Status.kErrorInternal, Status.kErrorNotSupported)
    torch.cuda.synchronize()
    assert float(D[0].abs().sum()) == 0.0 and float(D[1].abs().sum()) == 0.0
