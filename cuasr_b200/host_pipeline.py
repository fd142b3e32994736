"""SRGEMM for callers whose matrices live in host memory.

The reference's operators take device pointers only; a caller with host data pays for the copies around the call.
`HostSrgemm` is that whole path as one object: pinned host operands in, result out, with the copies overlapped with
the kernel.  The output is cut into chunks of storage lines (columns of a column-major D, rows of a row-major D).
The operand that is needed by every chunk (A for column-major D) is copied first; then, per chunk, the matching
lines of the other operand and of C go in on one stream, the SRGEMM of that chunk runs on a second stream as soon as
its inputs have arrived, and the finished chunk of D goes out on a third, so host-to-device copies, math and
device-to-host copies of different chunks run at the same time.  The arithmetic is the same SRGEMM, chunk by chunk,
so the result is bit-identical to the one-shot call.

The first chunk would otherwise wait for the whole shared operand.  Where that operand's K range is a run of whole
storage lines (column-major A, or row-major B for a row-major D) it is sent in a few K pieces instead, and the first
chunk is computed piece by piece, `D <- (alpha (x) A_p (x)(+) B_p) (+) D`, each piece as soon as it has arrived;
(x) distributes over (+), and every ring except floating-point plus-times is exact, so the bits do not change
(plus-times on floats keeps the one-piece schedule).

Several ranks that shard the output (each computes its own lines of D) all need the shared operand.  With `group`
set, every rank brings only its 1/world share of each K piece over its own host link and the ranks complete the
piece on every GPU over NVLink, so each byte of the shared operand crosses a host link once per node and the
first chunk still starts after the first piece.  Two ways to complete a piece (`exchange`):
  "p2p"   the shared operand lives in symmetric memory; a rank copies its share into every peer's buffer with plain
          device-to-device copies (copy engines) and raises a word on each peer (cuasr_b200_flag_raise); a rank's
          compute stream waits until the words of all ranks have arrived (cuasr_b200_flag_wait, bounded).  No SM is
          needed, which matters because the SRGEMM kernel is persistent and fills every SM: a collective kernel
          would have to wait for it, and piece p + 1 could not arrive while piece p computes.
  "nccl"  an NCCL all-gather per piece on a communication stream.
"""
from __future__ import annotations

from typing import Optional

from .semiring import DType, Layout, Op, Status
from .srgemm import Arguments, Srgemm, pack_k_contiguous


def share_ranges(shared_elems: int, k_pieces: int, rank: int, world: int):
    """Element ranges [(start, stop), ...] of the shared operand's flat storage that rank `rank` of `world` brings
    over its own host link: the rank-th of `world` equal parts of each of the `k_pieces` K pieces, in piece order.
    The ranges of all ranks tile the operand exactly once."""
    if shared_elems % (k_pieces * world):
        raise ValueError("the shared operand does not divide into equal shares for the ranks")
    piece = shared_elems // k_pieces
    sub = piece // world
    return [(p * piece + rank * sub, p * piece + (rank + 1) * sub) for p in range(k_pieces)]


def device_numa_node(device_index: int):
    """(NUMA node the GPU's host link hangs off, CPUs of that node this process may run on), or (None, set()) where
    the system does not say (no sysfs entry, a single node, a virtual machine that hides the topology)."""
    import os

    import torch
    try:
        props = torch.cuda.get_device_properties(device_index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None, set()
        cpus = set()
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        return node, cpus & os.sched_getaffinity(0)
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None, set()


class numa_local:
    """`with numa_local(device_index):` runs the calling thread on the CPUs next to the GPU's host link for the
    length of the block.  Pinned host buffers allocated inside get their pages from that node's memory (Linux
    places pages on the node of the thread that first touches them), so the GPU's copies do not cross the link
    between the CPU sockets; with eight GPUs of one box copying at once that link is otherwise the narrow spot.
    Only this process's own CPU affinity is touched, and it is put back on exit.  `.node` is the node, or None
    where the system does not tell (then the block runs unchanged)."""

    def __init__(self, device_index: int):
        self.node, self._cpus = device_numa_node(device_index)
        self._before = None

    def __enter__(self):
        import os
        if self._cpus:
            self._before = os.sched_getaffinity(0)
            os.sched_setaffinity(0, self._cpus)
        return self

    def __exit__(self, *exc):
        import os
        if self._before is not None:
            os.sched_setaffinity(0, self._before)
        return False


def _address(ref) -> int:
    return ref.data_ptr() if hasattr(ref, "data_ptr") else int(ref)


class HostSrgemm:
    def __init__(self, operator: Srgemm, m: int, n: int, k: int, alpha, beta, device, chunks: int = 8,
                 extra_outputs_per_chunk=None, buffers=None, shared_on_device: bool = False, group=None,
                 rank: int = 0, world: int = 1, exchange: str = "p2p"):
        """shared_on_device: the operand every chunk needs (A for a column-major D) is already in its device buffer
        when the call starts; it is not copied here.
        group, rank, world: torch.distributed group whose ranks all need the same shared operand (m, n, k describe
        THIS rank's product).  The host tensor passed for the shared operand then holds this rank's share only:
        for each of the `k_pieces` K pieces in turn, the rank-th of `world` equal parts of that piece's storage
        (`shared_share_layout` gives the element ranges).  exchange: "p2p" or "nccl", see the module docstring;
        with "p2p" the shared operand is kept in symmetric memory allocated here (the matching entry of `buffers`
        is not used)."""
        import torch

        self.torch = torch
        self.op, self.m, self.n, self.k, self.alpha, self.beta, self.device = operator, m, n, k, alpha, beta, device
        la, lb, lc = operator.layout_a, operator.layout_b, operator.layout_c
        col_c = lc == Layout.COLUMN_MAJOR
        # the chunked dimension must be the line dimension of C and of the operand that shares it
        self.chunkable = (col_c and lb == Layout.COLUMN_MAJOR) or (not col_c and la == Layout.ROW_MAJOR)
        lines = n if col_c else m
        self.col_c = col_c
        self.es = 8 if operator.dtype == DType.F64 else 4
        count = max(1, min(int(chunks), lines // 128)) if self.chunkable else 1
        while lines % count:
            count -= 1
        self.chunk_lines = [lines // count] * count
        self.chunks = len(self.chunk_lines)
        self.chunk_start = [sum(self.chunk_lines[:j]) for j in range(self.chunks)]
        tdt = {DType.F32: torch.float32, DType.F64: torch.float64, DType.S32: torch.int32, DType.U32: torch.int32}[operator.dtype]
        if buffers is not None:      # device storage supplied by the caller: flat A (m*k), B (k*n), C and D (m*n)
            self.dA, self.dB, self.dC, self.dD = buffers
        else:
            self.dA = torch.empty(m * k, dtype=tdt, device=device)
            self.dB = torch.empty(k * n, dtype=tdt, device=device)
            self.dC = torch.empty(m * n, dtype=tdt, device=device)
            self.dD = torch.empty(m * n, dtype=tdt, device=device)
        self.lda = m if la == Layout.COLUMN_MAJOR else k
        self.ldb = k if lb == Layout.COLUMN_MAJOR else n
        self.ldc = m if col_c else n
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        self.extra = extra_outputs_per_chunk       # optional: callable(chunk_index, byte_offset) -> list of peer pointers
        self.workspace = None
        self.launches = 0
        # K pieces of the shared operand for the first chunk (see the module docstring)
        shared_lines_are_k = (col_c and la == Layout.COLUMN_MAJOR) or (not col_c and lb == Layout.ROW_MAJOR)
        exact = not (operator.add_op == Op.PLUS and operator.dtype in (DType.F32, DType.F64))
        # every piece applies alpha to its own partial result, which is only right where alpha (x) distributes over
        # (+): with (x) = multiplies under min or max that needs alpha >= 0 (a negative factor swaps min and max)
        if operator.mul_op == Op.MULTIPLIES and operator.add_op in (Op.MINIMUM, Op.MAXIMUM) and not (alpha >= 0):
            exact = False
        self.k_pieces = 4 if (self.chunkable and shared_lines_are_k and exact and k % 4 == 0 and k >= 512) else 1
        self.shared_on_device = bool(shared_on_device)
        if self.shared_on_device:
            self.k_pieces = 1
        # Every chunk multiplies by the same shared operand.  Where its storage lines run along M (or N) the kernel
        # would make a K-contiguous copy of it for every launch; the pipeline makes that copy once, K piece by K
        # piece as the operand arrives, and hands the launches the copy (a row-major A, a column-major B).
        self.packed = None
        if self.chunkable and shared_lines_are_k and not self.shared_on_device:
            rows = m if col_c else n
            self.packed = torch.empty(rows * k, dtype=tdt, device=device)
            self.op_packed = Srgemm(operator.add_op, operator.mul_op, operator.dtype,
                                    Layout.ROW_MAJOR if col_c else la, lb if col_c else Layout.COLUMN_MAJOR, lc,
                                    add_identity=operator.add_identity, mul_identity=operator.mul_identity)
        self.group, self.rank, self.world = group, int(rank), int(world)
        if self.world > 1:
            shared_elems = (m * k) if col_c else (k * n)
            if self.k_pieces > 1 and (shared_elems // self.k_pieces) % self.world:
                self.k_pieces = 1
            if shared_elems % (self.k_pieces * self.world):
                raise ValueError("the shared operand does not divide into equal shares for the ranks")
            if exchange not in ("p2p", "nccl"):
                raise ValueError(exchange)
            self.s_comm = torch.cuda.Stream(device=device)
            self.exchange = exchange
            self._flag = torch.zeros(1, dtype=torch.int32, device=device)
            if exchange == "p2p":
                import torch.distributed as dist
                import torch.distributed._symmetric_memory as symm_mem
                grp = dist.group.WORLD if group is None else group
                shared = symm_mem.empty(shared_elems, dtype=tdt, device=device)
                handle = symm_mem.rendezvous(shared, grp)
                # views of every rank's copy of the shared operand (element r is this rank's own buffer for r == rank)
                self._peer_shared = [handle.get_buffer(r, (shared_elems,), tdt) for r in range(self.world)]
                if col_c:
                    self.dA = shared
                else:
                    self.dB = shared
                # arrival words: word p * world + r = "rank r's share of piece p has been delivered", per call epoch
                self._sig = symm_mem.empty(64, dtype=torch.int32, device=device)
                self._sig_handle = symm_mem.rendezvous(self._sig, grp)
                self._peer_sig = [int(ptr) for ptr in self._sig_handle.buffer_ptrs]
                self._handles = (handle, self._sig_handle)
                self._sig.zero_()
                torch.cuda.synchronize(device)
                dist.barrier(group=group)
                self._epoch = 0
                self.wait_ms = 5000

    def shared_share_layout(self):
        """Element ranges [(start, stop), ...] of the shared operand's flat storage that make up this rank's share,
        in the order the share's host tensor holds them (one range per K piece)."""
        shared_elems = (self.m * self.k) if self.col_c else (self.k * self.n)
        return share_ranges(shared_elems, self.k_pieces, self.rank, self.world)

    def _open_exchange(self, start) -> None:
        """Start of a call with several ranks.  With the p2p exchange the peers are about to write into this rank's
        copy of the shared operand: nobody may send before everybody has finished computing on the previous
        contents, i.e. has reached this point on its device (a one-word collective on the communication stream)."""
        self.s_comm.wait_event(start)
        if self.exchange == "p2p":
            import torch.distributed as dist
            self._epoch += 1
            with self.torch.cuda.stream(self.s_comm):
                dist.all_reduce(self._flag, group=self.group)

    def _bring_shared_piece(self, shared_dev, shared_host, p: int):
        """Starts the transfer of K piece p of the shared operand and returns the event that marks its arrival on
        this GPU: a plain copy, or (several ranks) the copy of this rank's share followed by an all-gather."""
        torch = self.torch
        shared_elems = shared_dev.numel()
        piece = shared_elems // self.k_pieces
        arrived = torch.cuda.Event()
        if self.world == 1:
            rng = slice(p * piece, (p + 1) * piece)
            with torch.cuda.stream(self.s_in):
                shared_dev[rng].copy_(shared_host[rng], non_blocking=True)
                arrived.record(self.s_in)
            return arrived
        import torch.distributed as dist
        sub = piece // self.world
        mine = slice(p * piece + self.rank * sub, p * piece + (self.rank + 1) * sub)
        copied = torch.cuda.Event()
        with torch.cuda.stream(self.s_in):
            shared_dev[mine].copy_(shared_host[p * sub:(p + 1) * sub], non_blocking=True)
            copied.record(self.s_in)
        with torch.cuda.stream(self.s_comm):
            self.s_comm.wait_event(copied)
            if self.exchange == "nccl":
                dist.all_gather_into_tensor(shared_dev[p * piece:(p + 1) * piece], shared_dev[mine], group=self.group)
            else:
                import ctypes

                from . import _lib
                lib = _lib.load()
                for r in range(self.world):
                    if r != self.rank:
                        self._peer_shared[r][mine].copy_(shared_dev[mine], non_blocking=True)
                word = 4 * (p * self.world + self.rank)
                ptrs = (ctypes.c_void_p * self.world)(*[ptr + word for ptr in self._peer_sig])
                st = lib.cuasr_b200_flag_raise(ptrs, self.world, self._epoch, self.s_comm.cuda_stream)
                if st == 0:
                    st = lib.cuasr_b200_flag_wait(self._sig.data_ptr() + 4 * p * self.world, self.world, self._epoch,
                                                  self.wait_ms, self.s_comm.cuda_stream)
                if st != 0:
                    raise RuntimeError(f"exchange of the shared operand failed: {Status(st)!r}")
            arrived.record(self.s_comm)
        return arrived

    def _pack_shared(self, shared_dev, p: int) -> None:
        """K piece p of the shared operand (all of it when there is one piece), which the compute stream has just
        been told to wait for, into the K-contiguous copy the launches read."""
        if self.packed is None:
            return
        kp = self.k // self.k_pieces
        rows, ld = (self.m, self.lda) if self.col_c else (self.n, self.ldb)
        st = pack_k_contiguous(self.op.dtype, shared_dev.data_ptr() + p * kp * ld * self.es, ld, False, rows, kp,
                               self.packed.data_ptr() + p * kp * self.es, self.k, self.s_run)
        if st != Status.kSuccess:
            raise RuntimeError(f"packing the shared operand failed: {st!r}")

    def _chunk_args(self, j: int):
        """Arguments of chunk j and the element ranges of B (or A), C and D it touches."""
        m, n, k = self.m, self.n, self.k
        w, l0 = self.chunk_lines[j], self.chunk_start[j]
        if self.col_c:
            moving, fixed = slice(l0 * k, (l0 + w) * k), None             # columns of B
            out = slice(l0 * m, (l0 + w) * m)
            shared = (self.packed, k) if self.packed is not None else (self.dA, self.lda)
            args = Arguments((m, w, k), shared, (self.dB.data_ptr() + moving.start * self.es, self.ldb),
                             (self.dC.data_ptr() + out.start * self.es, self.ldc),
                             (self.dD.data_ptr() + out.start * self.es, self.ldc), (self.alpha, self.beta))
        else:
            moving = slice(l0 * k, (l0 + w) * k)                           # rows of A
            out = slice(l0 * n, (l0 + w) * n)
            shared = (self.packed, k) if self.packed is not None else (self.dB, self.ldb)
            args = Arguments((w, n, k), (self.dA.data_ptr() + moving.start * self.es, self.lda), shared,
                             (self.dC.data_ptr() + out.start * self.es, self.ldc),
                             (self.dD.data_ptr() + out.start * self.es, self.ldc), (self.alpha, self.beta))
        return args, moving, out

    def _launch(self, args, extras, what: str) -> None:
        torch = self.torch
        op = self.op_packed if self.packed is not None else self.op
        with torch.cuda.stream(self.s_run):
            st = op.initialize(args, self.workspace, self.s_run)
            if st == Status.kSuccess:
                st = op.run_push(extras, self.s_run) if extras else op.run(self.s_run)
            if st != Status.kSuccess:
                raise RuntimeError(f"SRGEMM failed on {what}: {st!r}")
            self.launches += 1

    def _first_chunk_by_k_pieces(self, args, shared_dev, shared_host, extras, first_piece, inputs) -> None:
        """Chunk 0 as k_pieces accumulating launches, piece p as soon as K piece p of the shared operand is there.
        first_piece: arrival of K piece 0 (already on its way); inputs: arrival of the chunk's other operand and C."""
        torch = self.torch
        kp = self.k // self.k_pieces
        (m, n, _), es = args.problem_size, self.es
        self.s_run.wait_event(inputs)
        for p in range(self.k_pieces):
            self.s_run.wait_event(first_piece if p == 0 else self._bring_shared_piece(shared_dev, shared_host, p))
            self._pack_shared(shared_dev, p)
            # a K piece of the packed shared operand is a run of kp elements in every line: offset p * kp
            if self.col_c:      # A column-major: K piece = columns of A; B chunk column-major: K piece = rows of B
                a = ((_address(args.ref_A[0]) + p * kp * es, self.k) if self.packed is not None
                     else (_address(args.ref_A[0]) + p * kp * self.lda * es, self.lda))
                b = (_address(args.ref_B[0]) + p * kp * es, self.ldb)
            else:               # A chunk row-major: K piece = columns of A; B row-major: K piece = rows of B
                a = (_address(args.ref_A[0]) + p * kp * es, self.lda)
                b = ((_address(args.ref_B[0]) + p * kp * es, self.k) if self.packed is not None
                     else (_address(args.ref_B[0]) + p * kp * self.ldb * es, self.ldb))
            first, last = p == 0, p == self.k_pieces - 1
            c = args.ref_C if first else args.ref_D
            beta = self.beta if first else self.op.mul_identity
            piece_args = Arguments((m, n, kp), a, b, c, args.ref_D, (self.alpha, beta))
            self._launch(piece_args, extras if last else [], f"K piece {p} of chunk 0")

    def __call__(self, hA, hB, hC, hD, stream=None) -> None:
        """hA, hB, hC: pinned host tensors (flat storage, leading dimension = contiguous extent); hD receives the
        result.  Work is ordered after `stream` (default: the current stream) and `stream` waits for its end."""
        torch = self.torch
        cur = torch.cuda.current_stream(self.device) if stream is None else stream
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)
        shared_dev, shared_host = (self.dA, hA) if self.col_c else (self.dB, hB)
        moving_dev, moving_host = (self.dB, hB) if self.col_c else (self.dA, hA)
        if self.workspace is None:
            # one optional workspace for every launch shape of the pipeline (whole chunks and K pieces of chunk 0)
            whole = self._chunk_args(0)[0]
            (cm, cn, ck) = whole.problem_size
            shapes = [whole, Arguments((cm, cn, ck // self.k_pieces), whole.ref_A, whole.ref_B, whole.ref_C,
                                       whole.ref_D, whole.epilogue)]
            need = max((self.op_packed if self.packed is not None else self.op).get_optional_workspace_size(a)
                       for a in shapes)
            self.workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=self.device)
        whole_shared = None
        if self.k_pieces == 1 and not self.shared_on_device:
            if self.world == 1:
                with torch.cuda.stream(self.s_in):
                    shared_dev.copy_(shared_host, non_blocking=True)
            else:
                self._open_exchange(start)
                whole_shared = self._bring_shared_piece(shared_dev, shared_host, 0)
        elif self.world > 1:
            self._open_exchange(start)
        for j in range(self.chunks):
            args, moving, out = self._chunk_args(j)
            by_pieces = j == 0 and self.k_pieces > 1
            # K piece 0 of the shared operand goes first: with several ranks its exchange then runs under the copies
            # of the chunk's own inputs
            first_piece = self._bring_shared_piece(shared_dev, shared_host, 0) if by_pieces else None
            with torch.cuda.stream(self.s_in):
                moving_dev[moving].copy_(moving_host[moving], non_blocking=True)
                self.dC[out].copy_(hC[out], non_blocking=True)
            extras = self.extra(j, out.start * self.es) if self.extra else []
            done = torch.cuda.Event()
            if by_pieces:
                inputs = torch.cuda.Event()
                inputs.record(self.s_in)
                self._first_chunk_by_k_pieces(args, shared_dev, shared_host, extras, first_piece, inputs)
            else:
                arrived = torch.cuda.Event()
                arrived.record(self.s_in)
                self.s_run.wait_event(arrived)
                if whole_shared is not None:
                    self.s_run.wait_event(whole_shared)
                if j == 0 and self.k_pieces == 1:
                    self._pack_shared(shared_dev, 0)
                self._launch(args, extras, f"chunk {j}")
            done.record(self.s_run)
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                hD[out].copy_(self.dD[out], non_blocking=True)
        for s in (self.s_run, self.s_out) + ((self.s_comm,) if self.world > 1 else ()):
            end = torch.cuda.Event()
            end.record(s)
            cur.wait_event(end)
