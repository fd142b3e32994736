"""All-pairs shortest paths by repeated min-plus squaring, sharded over the GPUs of one node.

The reference stops at one GPU; its README only motivates the epilogue (+) with C by distributed APSP
(README.md:338-342).  This layer is the multi-GPU side the north star adds:

    D  <-  min(D, D (x) D)        ceil(log2 n) times, D the n x n matrix of path lengths (column-major)

Rank g of G owns n/G consecutive columns (one contiguous block of a column-major matrix).  A squaring step is one
SRGEMM per rank, `D_next[:, block] = min(D_cur[:, block], D_cur (x) D_cur[:, block])`, followed by the only
exchange of the algorithm: every rank needs the whole of D_next.  Two exchange modes:

  "allgather"  NCCL all-gather of D_next (torch.distributed) after the kernel.
  "push"       the SRGEMM epilogue itself stores each finished tile into every rank's D_next through peer
               pointers (cuasr_b200_srgemm_push), so the transfer overlaps the computation tile by tile; the
               step ends with a stream-ordered barrier.  Peer pointers come from torch symmetric memory.

The host logic (sharding, buffer rotation, exchange) is independent of the device: `ShardedSquaring` drives a
small backend interface, `CudaBackend` is the product, and the CPU tests plug in a gloo/numpy backend.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

from .semiring import DType, Layout, Op, Status, identity


class ShardedSquaring:
    """Sharding and buffer rotation of the repeated-squaring solve; all data movement goes through `backend`."""

    def __init__(self, n: int, rank: int, world: int, backend):
        if n % world != 0:
            raise ValueError(f"n = {n} is not divisible by the {world} ranks")
        self.n, self.rank, self.world, self.backend = n, rank, world, backend
        self.cols = n // world
        self.c0 = rank * self.cols
        self.cur, self.nxt = 0, 1         # indices of the two full-size matrices the backend holds
        self.steps_done = 0

    @staticmethod
    def squarings_needed(n: int) -> int:
        """Paths have at most n - 1 edges and every squaring doubles the covered length: ceil(log2 n) steps."""
        return max(1, math.ceil(math.log2(n)))

    def step(self) -> None:
        b = self.backend
        b.srgemm_block(self.cur, self.nxt, self.c0, self.cols)   # D_next[:, block] (and, in push mode, every peer's)
        b.exchange(self.nxt, self.c0, self.cols)                 # afterwards every rank holds all of D_next
        self.cur, self.nxt = self.nxt, self.cur
        self.steps_done += 1

    def solve(self, squarings: Optional[int] = None) -> int:
        squarings = self.squarings_needed(self.n) if squarings is None else squarings
        for _ in range(squarings):
            self.step()
        return squarings

    def result(self):
        return self.backend.matrix(self.cur)


class CudaBackend:
    """Two n x n fp32 matrices per GPU, the min-plus SRGEMM of this library, and the exchange over NVLink."""

    def __init__(self, n: int, rank: int, world: int, device, mode: str = "push", group=None,
                 true_infinity: bool = True):
        import torch
        import torch.distributed as dist

        from .srgemm import Arguments, Srgemm, Status

        if mode not in ("push", "allgather"):
            raise ValueError(mode)
        self.n, self.rank, self.world, self.device, self.mode = n, rank, world, device, mode
        self.torch, self.dist, self.group = torch, dist, group
        self.Status, self.Arguments = Status, Arguments
        self.inf = math.inf if true_infinity else float(identity(Op.MINIMUM, DType.F32))
        self.peer_ptrs: List[List[int]] = [[], []]
        if world > 1 and mode == "push":
            import torch.distributed._symmetric_memory as symm_mem

            self.bufs = [symm_mem.empty(n * n, dtype=torch.float32, device=device) for _ in range(2)]
            self._handles = [symm_mem.rendezvous(t, dist.group.WORLD if group is None else group) for t in self.bufs]
            self.peer_ptrs = [[int(p) for p in h.buffer_ptrs] for h in self._handles]
        else:
            self.bufs = [torch.empty(n * n, dtype=torch.float32, device=device) for _ in range(2)]
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        col = Layout.COLUMN_MAJOR
        self.op = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, col, col, col, add_identity=self.inf)
        self.workspace = None     # optional load-balancing scratch of the SRGEMM, sized on first use
        self.launches = 0

    # -- data ---------------------------------------------------------------------------------------------
    def load(self, which: int, flat) -> None:
        self.bufs[which].copy_(flat)

    def matrix(self, which: int):
        return self.bufs[which]

    # -- the two operations ShardedSquaring needs -----------------------------------------------------------
    def srgemm_block(self, cur: int, nxt: int, c0: int, cols: int) -> None:
        n, es = self.n, 4
        src, dst = self.bufs[cur], self.bufs[nxt]
        off = c0 * n * es
        # A = D_cur (n x n), B = C = D_cur[:, block], D = D_next[:, block]; alpha = beta = 0 = the (x) identity
        args = self.Arguments((n, cols, n), (src, n), (src.data_ptr() + off, n), (src.data_ptr() + off, n),
                              (dst.data_ptr() + off, n), (0.0, 0.0))
        stream = self.torch.cuda.current_stream(self.device)
        if self.workspace is None:
            need = self.op.get_optional_workspace_size(args)
            self.workspace = self.torch.empty(max(need, 1), dtype=self.torch.uint8, device=self.device)
        st = self.op.initialize(args, self.workspace, stream)
        if st != self.Status.kSuccess:
            raise RuntimeError(f"SRGEMM rejected the squaring step: {st!r}")
        if self.world > 1 and self.mode == "push":
            extras = [p + off for r, p in enumerate(self.peer_ptrs[nxt]) if r != self.rank]
            st = self.op.run_push(extras, stream)
        else:
            st = self.op.run(stream)
        if st != self.Status.kSuccess:
            raise RuntimeError(f"SRGEMM launch failed: {st!r}")
        self.launches += 1

    def exchange(self, nxt: int, c0: int, cols: int) -> None:
        if self.world == 1:
            return
        if self.mode == "allgather":
            buf = self.bufs[nxt]
            self.dist.all_gather_into_tensor(buf, buf[c0 * self.n:(c0 + cols) * self.n], group=self.group)
        else:
            # every rank's kernel has written into every rank's D_next; a stream-ordered collective on one word
            # orders "all kernels of this step are done" before anything that follows on any rank
            self.dist.all_reduce(self._flag, group=self.group)


def random_graph(n: int, p: float, seed: int, device, absent: float = math.inf, rows: Optional[Sequence[int]] = None):
    """Flat column-major (= row-major, the generator is symmetric) weighted adjacency matrix of a random directed
    graph: each edge present with probability p, integer weights uniform in [1, 100] stored as fp32, diagonal 0,
    absent edges = `absent`."""
    import torch

    from . import datagen

    if rows is None:
        return datagen.sparse_graph(seed, n, p, absent, dtype=torch.float32, device=device, weight_lo=1,
                                    weight_hi=100, integer_weights=True)
    start, count = rows
    return datagen.sparse_graph(seed, n, p, absent, dtype=torch.float32, device=device, weight_lo=1, weight_hi=100,
                                integer_weights=True, row_start=start, rows=count)


class BlockedFloydWarshall:
    """All-pairs shortest paths by the three-phase blocked Floyd-Warshall scheme on top of the same min-plus
    SRGEMM (its epilogue (+) with C is what the reference's README.md:338-342 positions for exactly this): 2 n^3
    semiring operations in total instead of 2 n^3 log2(n) for repeated squaring.

    D is column-major, n x n; rank g of G owns n / G columns (every G-th block of `block` columns by default, see
    `distribution`) and stores only those.  For every block
    K = [kb * b, (kb + 1) * b) of vertices:
      1. the rank that owns columns K closes the diagonal block (paths inside K) by ceil(log2 b) squarings of it;
      2. it updates the column panel  P_col = min(D[:, K], D[:, K] (x) D[K, K]*)  and every rank receives P_col
         (pushed by that SRGEMM's epilogue into symmetric memory, or broadcast with NCCL); every rank updates its
         piece of the row panel  P_row = min(D[K, mine], D[K, K]* (x) D[K, mine]);
      3. every rank updates its columns in place:  D[:, mine] = min(D[:, mine], P_col (x) P_row).
    Panels are computed out of place, so no SRGEMM reads memory another CTA of the same launch writes.  With
    integer edge weights every sum is exact and the result equals repeated squaring bit for bit; with general
    floating-point weights the two orders of summation may round differently.
    """

    def __init__(self, n: int, block: int, rank: int, world: int, device, mode: str = "push", group=None,
                 look_ahead: Optional[bool] = None, distribution: str = "cyclic"):
        import torch
        import torch.distributed as dist

        from .srgemm import Arguments, Srgemm, Status

        self.look_ahead = world > 1 if look_ahead is None else bool(look_ahead)
        if distribution not in ("cyclic", "contiguous"):
            raise ValueError(distribution)
        # "cyclic": rank g owns the column blocks g, g + G, g + 2G, ... so the extra work of the owner (closure and
        # column panel) moves to another rank every step; "contiguous": one run of n / G columns per rank
        self.distribution = distribution
        if n % world or (n // world) % block:
            raise ValueError(f"block size {block} must divide the {n // max(world, 1)} columns each rank owns")
        if mode not in ("push", "allgather"):
            raise ValueError(mode)
        self.n, self.b, self.rank, self.world, self.device, self.mode = n, block, rank, world, device, mode
        self.torch, self.dist, self.group = torch, dist, group
        self.Status, self.Arguments = Status, Arguments
        self.cols = n // world
        self.c0 = rank * self.cols
        f32 = torch.float32
        self.D = torch.empty(n * self.cols, dtype=f32, device=device)          # my columns, ld = n
        self.p_row = torch.empty(block * self.cols, dtype=f32, device=device)  # ld = block
        self.diag = [torch.empty(block * block, dtype=f32, device=device) for _ in range(2)]
        self.peer_pcol: List[List[int]] = [[], [], []]
        if world > 1 and mode == "push":
            import torch.distributed._symmetric_memory as symm_mem

            self.p_col = [symm_mem.empty(n * block, dtype=f32, device=device) for _ in range(3)]
            handles = [symm_mem.rendezvous(t, dist.group.WORLD if group is None else group) for t in self.p_col]
            self._handles = handles
            self.peer_pcol = [[int(p) for p in h.buffer_ptrs] for h in handles]
            # word 0: number of column panels delivered to me so far; words 1 + r: steps rank r has finished
            self.sig = symm_mem.empty(64, dtype=torch.int32, device=device)
            self._sig_handle = symm_mem.rendezvous(self.sig, dist.group.WORLD if group is None else group)
            self.peer_sig = [int(p) for p in self._sig_handle.buffer_ptrs]
            self.sig.zero_()
            torch.cuda.synchronize(device)
            dist.barrier(group=group)            # nobody raises a word that is about to be cleared
        else:
            self.p_col = [torch.empty(n * block, dtype=f32, device=device) for _ in range(3)]
        self.epoch = 0
        self.wait_ms = 5000
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        col = Layout.COLUMN_MAJOR
        self.op = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, col, col, col, add_identity=math.inf)
        self._workspaces = {}
        self.launches = 0

    def owner(self, kb: int) -> int:
        return kb % self.world if self.distribution == "cyclic" else (kb * self.b) // self.cols

    def local_column(self, kb: int) -> int:
        """First local column of block kb on the rank that owns it."""
        return (kb // self.world) * self.b if self.distribution == "cyclic" else kb * self.b - self.c0

    def owned_blocks(self) -> List[int]:
        """Global indices of the column blocks this rank holds, in the order it stores them."""
        return [kb for kb in range(self.n // self.b) if self.owner(kb) == self.rank]

    def load_columns(self, flat) -> None:
        """`flat`: this rank's columns of the weighted adjacency matrix (column-major, n x cols, diagonal 0): the
        column blocks `owned_blocks()` one after the other."""
        self.D.copy_(flat)

    def _srgemm(self, m, n, k, A, lda, B, ldb, C, ldc, D, ldd, extras=()):
        """D = min(C, A (x) B); all arguments are device addresses."""
        args = self.Arguments((m, n, k), (A, lda), (B, ldb), (C, ldc), (D, ldd), (0.0, 0.0))
        key = (m, n, k)
        if key not in self._workspaces:
            need = self.op.get_optional_workspace_size(args)
            self._workspaces[key] = self.torch.empty(max(need, 1), dtype=self.torch.uint8, device=self.device)
        stream = self.torch.cuda.current_stream(self.device)
        st = self.op.initialize(args, self._workspaces[key], stream)
        if st == self.Status.kSuccess:
            st = self.op.run_push(list(extras), stream) if extras else self.op.run(stream)
        if st != self.Status.kSuccess:
            raise RuntimeError(f"SRGEMM failed: {st!r}")
        self.launches += 1

    def _closure_and_column_panel(self, kb: int) -> None:
        """Run by the rank that owns block K = kb: phase 1 and the column panel of phase 2, delivered to every rank."""
        n, b, es = self.n, self.b, 4
        k0 = kb * b
        lc = self.local_column(kb)                              # first local column of block K
        # phase 1: closure of the diagonal block by repeated squaring of a private copy
        self.diag[0].view(b, b).copy_(self.D.view(self.cols, n)[lc:lc + b, k0:k0 + b])
        cur = 0
        for _ in range(max(1, math.ceil(math.log2(b)))):
            s, d = self.diag[cur].data_ptr(), self.diag[1 - cur].data_ptr()
            self._srgemm(b, b, b, s, b, s, b, s, b, d, b)
            cur = 1 - cur
        star = self.diag[cur].data_ptr()
        # phase 2, column panel: P_col = min(D[:, K], D[:, K] (x) D[K, K]*)
        panel = self.D.data_ptr() + lc * n * es
        extras = [p for r, p in enumerate(self.peer_pcol[kb % 3]) if r != self.rank]
        self._srgemm(n, b, b, panel, n, star, b, panel, n, self.p_col[kb % 3].data_ptr(), n, extras)

    def _phase3(self, pcp: int, lo: int, hi: int) -> None:
        """D[:, lo:hi] = min(D[:, lo:hi], P_col (x) P_row[:, lo:hi]) over my local columns lo..hi, in place (C aliases
        D; the operands are copies)."""
        if hi <= lo:
            return
        n, b, es = self.n, self.b, 4
        d = self.D.data_ptr() + lo * n * es
        self._srgemm(n, hi - lo, b, pcp, n, self.p_row.data_ptr() + lo * b * es, b, d, n, d, n)

    # -- ordering between ranks ------------------------------------------------------------------------------
    # "allgather" mode: one NCCL broadcast per panel.  "push" mode: the owner's SRGEMM epilogue has already stored the
    # panel into every rank's buffer; what remains is ordering, and that is one-sided (cuasr_b200_flag_raise / _wait):
    # the owner raises "panels delivered" on every rank and goes on, a consumer waits for its own copy of that word.
    # A collective here would make the owner wait until the slowest consumer arrives, i.e. run in lockstep with it.
    def _raise(self, word: int, value: int) -> None:
        import ctypes

        from . import _lib

        ptrs = (ctypes.c_void_p * self.world)(*[p + 4 * word for p in self.peer_sig])
        stream = self.torch.cuda.current_stream(self.device).cuda_stream
        st = _lib.load().cuasr_b200_flag_raise(ptrs, self.world, value, stream)
        if st != 0:
            raise RuntimeError(f"flag raise failed: {Status(st)!r}")
        self.launches += 1

    def _wait(self, word: int, count: int, value: int) -> None:
        from . import _lib

        stream = self.torch.cuda.current_stream(self.device).cuda_stream
        st = _lib.load().cuasr_b200_flag_wait(self.sig.data_ptr() + 4 * word, count, value, self.wait_ms, stream)
        if st != 0:
            raise RuntimeError(f"flag wait failed: {Status(st)!r}")
        self.launches += 1

    def _send_panel(self, kb: int, base: int) -> None:
        """Run by the owner of block kb.  The panel goes into buffer kb % 3, which every rank last read in step
        kb - 3: wait until all of them have reported that step finished, then compute, push and announce."""
        flags = self.world > 1 and self.mode == "push"
        if flags and kb >= 3:
            self._wait(1, self.world, base + kb - 2)
        self._closure_and_column_panel(kb)
        if flags:
            self._raise(0, base + kb + 1)

    def _receive_panel(self, kb: int, base: int) -> None:
        """Every rank, once per block and in block order: afterwards P_col of block kb is complete in buffer kb % 3."""
        if self.world == 1:
            return
        owner = self.owner(kb)
        if self.mode == "push":
            if owner != self.rank:
                self._wait(0, 1, base + kb + 1)
        else:
            self.dist.broadcast(self.p_col[kb % 3], src=owner, group=self.group)

    def solve(self) -> None:
        """With look-ahead (the default with more than one rank) the owner of the NEXT block works ahead: it updates
        that block's columns first, closes the block and sends its column panel before it finishes phase 3 of the
        current block.  The chain panel -> next panel is then (row-panel piece, one block of phase 3, closure, column
        panel) instead of a whole step, and the ranks that only consume never wait.  Three panel buffers plus the
        "step finished" words keep a fast owner from overwriting a panel a slow rank still reads."""
        n, b, es = self.n, self.b, 4
        Dp = self.D.data_ptr()
        blocks = n // b
        ahead = self.look_ahead
        base = self.epoch * (blocks + 4)          # flag values of this solve start above those of the last one
        self.epoch += 1
        if self.world > 1:
            # a rank may still be reading the panels of a previous solve: nobody sends before everybody is here
            self.dist.all_reduce(self._flag, group=self.group)
        if self.rank == 0:
            self._send_panel(0, base)
        for kb in range(blocks):
            k0 = kb * b
            pcp = self.p_col[kb % 3].data_ptr()
            if not (ahead and self.mode != "push" and kb > 0 and self.owner(kb) == self.rank):
                self._receive_panel(kb, base)     # (a broadcasting owner that worked ahead has already joined it)
            # phase 2, my piece of the row panel: P_row = min(D[K, mine], D[K, K]* (x) D[K, mine]); D[K, K]* = P_col[K, :]
            rows = Dp + k0 * es
            self._srgemm(b, self.cols, b, pcp + k0 * es, n, rows, n, rows, n, self.p_row.data_ptr(), b)
            nxt = kb + 1
            mine_next = nxt < blocks and self.owner(nxt) == self.rank
            if ahead and mine_next:
                lc = self.local_column(nxt)
                self._phase3(pcp, lc, lc + b)
                self._send_panel(nxt, base)
                if self.mode != "push":
                    self._receive_panel(nxt, base)          # the root's side of the broadcast, early
                self._phase3(pcp, 0, lc)
                self._phase3(pcp, lc + b, self.cols)
            else:
                self._phase3(pcp, 0, self.cols)
                if mine_next:
                    self._send_panel(nxt, base)
            if self.world > 1 and self.mode == "push":
                self._raise(1 + self.rank, base + kb + 1)   # step kb finished here: its panel buffer may be reused

    def result_columns(self):
        return self.D


# ---- the C entry points of include/cuasr_b200_apsp.h --------------------------------------------------------
REPEATED_SQUARING, BLOCKED_FLOYD_WARSHALL = 0, 1


def _apsp_args(dtype: DType, algorithm: int, n: int, D=0, ldd: Optional[int] = None, block: int = 0,
               iterations: int = 0, workspace=0, workspace_bytes: int = 0, stream: int = 0, parent=0,
               ld_parent: Optional[int] = None):
    from . import _lib

    a = _lib.ApspArgs()
    a.dtype, a.algorithm, a.n, a.block, a.iterations = int(dtype), int(algorithm), int(n), int(block), int(iterations)
    a.D, a.ldd = int(D) or None, int(n if ldd is None else ldd)
    a.workspace, a.workspace_bytes = int(workspace) or None, int(workspace_bytes)
    a.stream = int(stream) or None
    a.parent, a.ld_parent = int(parent) or None, int(n if ld_parent is None else ld_parent)
    return a


def device_solve_workspace_size(dtype: DType, algorithm: int, n: int, block: int = 0) -> int:
    """cuasr_b200_apsp_workspace_size: bytes of device scratch `device_solve` needs."""
    import ctypes

    from . import _lib

    return int(_lib.load().cuasr_b200_apsp_workspace_size(ctypes.byref(_apsp_args(dtype, algorithm, n, block=block))))


def device_solve(D, n: int, dtype: DType = DType.F32, algorithm: int = BLOCKED_FLOYD_WARSHALL, ldd: Optional[int] = None,
                 block: int = 0, iterations: int = 0, workspace=None, stream=None, parent=None,
                 ld_parent: Optional[int] = None) -> Status:
    """cuasr_b200_apsp: closes the n x n distance matrix `D` (a torch CUDA tensor or a device address) in place on
    one GPU; enqueues on `stream` (default: the current torch stream) and returns.  `workspace`: a uint8 CUDA
    tensor of at least `device_solve_workspace_size` bytes; allocated here when omitted.  `parent`: optional int32
    n x n matrix (column-major like D, filled with -1 by the caller) that receives, for every pair whose distance
    improved, a vertex k with D[i, j] == D[i, k] + D[k, j] (`walk` turns it into vertex sequences)."""
    import ctypes

    import torch

    from . import _lib

    if workspace is None:
        workspace = torch.empty(max(1, device_solve_workspace_size(dtype, algorithm, n, block)), dtype=torch.uint8,
                                device="cuda")
    s = torch.cuda.current_stream().cuda_stream if stream is None else getattr(stream, "cuda_stream", stream)
    ptr = D.data_ptr() if hasattr(D, "data_ptr") else int(D)
    par = 0 if parent is None else (parent.data_ptr() if hasattr(parent, "data_ptr") else int(parent))
    a = _apsp_args(dtype, algorithm, n, ptr, ldd, block, iterations, workspace.data_ptr(), workspace.numel(), s, par,
                   ld_parent)
    return Status(_lib.load().cuasr_b200_apsp(ctypes.byref(a)))


def walk(parent, i: int, j: int):
    """The vertices of the shortest path i -> j, end points included, from the predecessor matrix a solve with
    `parent` left behind: parent[i][j] = k >= 0 splits the path at k, a negative entry means the pair is joined by
    an edge of the input (the caller checks beforehand that j can be reached at all).  `parent` is indexed
    [i][j] (pass the transpose of the column-major device matrix)."""
    path, todo = [i], [(i, j)]
    steps = 0
    while todo:
        # a simple path over n vertices has at most n - 1 edges and n - 2 splits
        steps += 1
        if steps > 2 * len(parent):
            raise ValueError("the predecessor matrix does not describe a simple path (zero-weight cycle?)")
        u, v = todo.pop()
        k = int(parent[u][v])
        if k < 0:
            path.append(v)
        else:
            todo.append((k, v))
            todo.append((u, k))
    return path


def shard_squaring(dtype: DType, n: int, col0: int, cols: int, d_cur: int, ld_cur: int, d_next: int, ld_next: int,
                   peer_next: Sequence[int] = (), workspace: int = 0, workspace_bytes: int = 0, stream: int = 0) -> Status:
    """cuasr_b200_apsp_shard_squaring on device addresses: one rank's share of one squaring, pushed to the peers."""
    import ctypes

    from . import _lib

    a = _lib.ApspShardArgs()
    a.dtype, a.n, a.col0, a.cols = int(dtype), int(n), int(col0), int(cols)
    a.D_cur, a.ld_cur, a.D_next, a.ld_next = int(d_cur) or None, int(ld_cur), int(d_next) or None, int(ld_next)
    peers = (ctypes.c_void_p * max(1, len(peer_next)))(*[int(p) for p in peer_next])
    a.n_peers, a.peer_next = len(peer_next), ctypes.cast(peers, ctypes.POINTER(ctypes.c_void_p))
    a.workspace, a.workspace_bytes, a.stream = int(workspace) or None, int(workspace_bytes), int(stream) or None
    return Status(_lib.load().cuasr_b200_apsp_shard_squaring(ctypes.byref(a)))


def multi_partition(n: int, n_devices: int, g: int):
    """cuasr_b200_apsp_multi_partition: (first column, number of columns) of GPU g, or None for invalid arguments."""
    import ctypes

    from . import _lib

    col0, cols = ctypes.c_int32(), ctypes.c_int32()
    st = _lib.load().cuasr_b200_apsp_multi_partition(n, n_devices, g, ctypes.byref(col0), ctypes.byref(cols))
    return (col0.value, cols.value) if st == 0 else None


def multi_device_workspace_size(dtype: DType, n: int, n_devices: int, algorithm: int = BLOCKED_FLOYD_WARSHALL,
                                block: int = 0) -> int:
    """cuasr_b200_apsp_multi_workspace_size: bytes of scratch every GPU needs (0 for repeated squaring, whose
    workspace is optional, and for arguments the solve would refuse)."""
    import ctypes

    from . import _lib

    a = _lib.ApspMultiArgs()
    a.dtype, a.algorithm, a.n, a.block, a.n_devices, a.ldd = int(dtype), int(algorithm), int(n), int(block), int(n_devices), int(n)
    return int(_lib.load().cuasr_b200_apsp_multi_workspace_size(ctypes.byref(a)))


def multi_device_solve(dtype: DType, n: int, devices: Sequence[int], buf0: Sequence[int], buf1: Sequence[int] = (),
                       ldd: Optional[int] = None, iterations: int = 0, workspaces: Sequence[int] = (),
                       workspace_bytes: int = 0, streams: Sequence[int] = (), algorithm: int = REPEATED_SQUARING,
                       block: int = 0):
    """cuasr_b200_apsp_multi on device addresses: the sharded solve on the GPUs `devices` of this machine from one
    process (one host thread per GPU inside the library, peer stores between the GPUs).
    Repeated squaring: buf0[g] holds the whole distance matrix on every GPU, buf1[g] is a second matrix.
    Blocked Floyd-Warshall: buf0[g] holds the column blocks g, g + G, ... of `block` vertices (n x n/G, leading
    dimension ldd), buf1 is not used and `workspaces` (multi_device_workspace_size bytes each) are required.
    Returns (Status, index of the buffer that holds the result, list of per-GPU device status words).  Blocks until
    the solve is done."""
    import ctypes

    from . import _lib

    G = len(devices)
    a = _lib.ApspMultiArgs()
    a.dtype, a.algorithm, a.n, a.block, a.iterations, a.n_devices = int(dtype), int(algorithm), int(n), int(block), int(iterations), G
    dev_arr = (ctypes.c_int32 * max(G, 1))(*[int(d) for d in devices])
    b0 = (ctypes.c_void_p * max(G, 1))(*[int(p) or None for p in buf0])
    a.devices = ctypes.cast(dev_arr, ctypes.POINTER(ctypes.c_int32))
    a.buf0 = ctypes.cast(b0, ctypes.POINTER(ctypes.c_void_p))
    a.ldd = int(n if ldd is None else ldd)
    keep = [dev_arr, b0]
    if buf1:
        b1 = (ctypes.c_void_p * max(G, 1))(*[int(p) or None for p in buf1])
        a.buf1 = ctypes.cast(b1, ctypes.POINTER(ctypes.c_void_p))
        keep.append(b1)
    if workspaces:
        ws = (ctypes.c_void_p * G)(*[int(p) or None for p in workspaces])
        a.workspace, a.workspace_bytes = ctypes.cast(ws, ctypes.POINTER(ctypes.c_void_p)), int(workspace_bytes)
        keep.append(ws)
    if streams:
        st_arr = (ctypes.c_void_p * G)(*[int(p) or None for p in streams])
        a.streams = ctypes.cast(st_arr, ctypes.POINTER(ctypes.c_void_p))
        keep.append(st_arr)
    result = ctypes.c_int32(-1)
    status = (ctypes.c_int32 * max(G, 1))()
    a.result_buffer = ctypes.pointer(result)
    a.device_status = ctypes.cast(status, ctypes.POINTER(ctypes.c_int32))
    st = Status(_lib.load().cuasr_b200_apsp_multi(ctypes.byref(a)))
    return st, result.value, list(status)[:G]
