"""SRGEMM for callers whose matrices live in host memory.

The reference's operators take device pointers only; a caller with host data pays for the copies around the call.
`HostSrgemm` is that whole path as one object: pinned host operands in, result out, with the copies overlapped with
the kernel.  The output is cut into chunks of storage lines (columns of a column-major D, rows of a row-major D).
The operand that is needed by every chunk (A for column-major D) is copied first; then, per chunk, the matching
lines of the other operand and of C go in on one stream, the SRGEMM of that chunk runs on a second stream as soon as
its inputs have arrived, and the finished chunk of D goes out on a third, so host-to-device copies, math and
device-to-host copies of different chunks run at the same time.  The arithmetic is the same SRGEMM, chunk by chunk,
so the result is bit-identical to the one-shot call.
"""
from __future__ import annotations

from typing import Optional

from .semiring import DType, Layout, Status
from .srgemm import Arguments, Srgemm


class HostSrgemm:
    def __init__(self, operator: Srgemm, m: int, n: int, k: int, alpha, beta, device, chunks: int = 8,
                 extra_outputs_per_chunk=None, buffers=None):
        import torch

        self.torch = torch
        self.op, self.m, self.n, self.k, self.alpha, self.beta, self.device = operator, m, n, k, alpha, beta, device
        la, lb, lc = operator.layout_a, operator.layout_b, operator.layout_c
        col_c = lc == Layout.COLUMN_MAJOR
        # the chunked dimension must be the line dimension of C and of the operand that shares it
        self.chunkable = (col_c and lb == Layout.COLUMN_MAJOR) or (not col_c and la == Layout.ROW_MAJOR)
        lines = n if col_c else m
        self.chunks = max(1, min(chunks, lines // 128)) if self.chunkable else 1
        while lines % self.chunks:
            self.chunks -= 1
        self.col_c = col_c
        self.es = 8 if operator.dtype == DType.F64 else 4
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

    def _chunk_args(self, j: int):
        """Arguments of chunk j and the element ranges of B (or A), C and D it touches."""
        m, n, k = self.m, self.n, self.k
        if self.col_c:
            w = n // self.chunks
            moving, fixed = slice(j * w * k, (j + 1) * w * k), None       # columns of B
            out = slice(j * w * m, (j + 1) * w * m)
            args = Arguments((m, w, k), (self.dA, self.lda), (self.dB.data_ptr() + moving.start * self.es, self.ldb),
                             (self.dC.data_ptr() + out.start * self.es, self.ldc),
                             (self.dD.data_ptr() + out.start * self.es, self.ldc), (self.alpha, self.beta))
        else:
            w = m // self.chunks
            moving = slice(j * w * k, (j + 1) * w * k)                     # rows of A
            out = slice(j * w * n, (j + 1) * w * n)
            args = Arguments((w, n, k), (self.dA.data_ptr() + moving.start * self.es, self.lda), (self.dB, self.ldb),
                             (self.dC.data_ptr() + out.start * self.es, self.ldc),
                             (self.dD.data_ptr() + out.start * self.es, self.ldc), (self.alpha, self.beta))
        return args, moving, out

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
        with torch.cuda.stream(self.s_in):
            shared_dev.copy_(shared_host, non_blocking=True)
        for j in range(self.chunks):
            args, moving, out = self._chunk_args(j)
            arrived, done = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(self.s_in):
                moving_dev[moving].copy_(moving_host[moving], non_blocking=True)
                self.dC[out].copy_(hC[out], non_blocking=True)
                arrived.record(self.s_in)
            self.s_run.wait_event(arrived)
            with torch.cuda.stream(self.s_run):
                if self.workspace is None:
                    need = self.op.get_optional_workspace_size(args)
                    self.workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=self.device)
                st = self.op.initialize(args, self.workspace, self.s_run)
                if st == Status.kSuccess:
                    extras = self.extra(j, out.start * self.es) if self.extra else []
                    st = self.op.run_push(extras, self.s_run) if extras else self.op.run(self.s_run)
                if st != Status.kSuccess:
                    raise RuntimeError(f"SRGEMM failed on chunk {j}: {st!r}")
                self.launches += 1
                done.record(self.s_run)
            self.s_out.wait_event(done)
            with torch.cuda.stream(self.s_out):
                hD[out].copy_(self.dD[out], non_blocking=True)
        for s in (self.s_run, self.s_out):
            end = torch.cuda.Event()
            end.record(s)
            cur.wait_event(end)
