"""Benchmark of the SRGEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `minplus_f32_8192`: min-plus fp32 SRGEMM D = min(C, A (x) B), M = N = K = 8192, all matrices
column-major, A and B uniform in [0, 100) from a seed, C filled with the additive identity.  One step is one
SRGEMM.  At N > 1 GPUs the columns of D (contiguous blocks of a column-major matrix) are sharded over the ranks
and the step ends with an all-gather of D: exactly one squaring step of the sharded all-pairs-shortest-paths
solve.  Rank 0 prints ONE JSON line.  The other workloads of cuasr_b200/workloads.py run the same way on one GPU.

`--impl reference` times the reference's own host SRGEMM (oracle/_ref when it was built, else the C restatement
in oracle/) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "minplus_f32_srgemm_throughput"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "sm_max_mhz": 1965.0}, "fallback"


def dram_traffic(workload: str):
    """Bytes one launch of `workload` moved to and from DRAM in the committed ncu capture (None when there is none).
    The figures live in one tracked table beside the profile summaries so that this file and they cannot drift."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            entry = json.load(f).get(workload)
        return int(entry["bytes_per_launch"]) if entry else None
    except (OSError, ValueError, KeyError):
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs: through NVML every 10 ms where it is
    available, else by polling nvidia-smi."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._thread = index, [], threading.Event(), None

    def _nvml(self):
        """(module, handle) for this process's GPU `index` through NVML, or None where NVML cannot be used (then
        nvidia-smi is polled instead).  Reading only: no setting of the GPU is touched."""
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            try:        # CUDA's device order need not be NVML's: go by UUID where torch knows it
                import torch
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
                for candidate in (uuid, uuid.encode()):
                    try:
                        handle = pynvml.nvmlDeviceGetHandleByUUID(candidate)
                        break
                    except Exception:
                        continue
            except Exception:
                handle = None
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)      # fails here if the handle is unusable
            return pynvml, handle
        except Exception:
            return None

    def _sample_nvml(self, nvml, handle):
        sm = nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)
        top = nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM)
        reasons = getattr(nvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nvml.nvmlDeviceGetCurrentClocksThrottleReasons
        mask = int(reasons(handle))
        # bits of the NVML reasons mask: software power cap 0x4, hardware slowdown 0x8, software thermal 0x20,
        # hardware thermal 0x40
        flag = lambda bit: "Active" if mask & bit else "Not Active"
        return [str(sm), str(top), flag(0x8), flag(0x40), flag(0x20), flag(0x4)]

    def _run(self):
        nvml = self._nvml()
        while not self._stop.is_set():
            try:
                if nvml is not None:
                    self.samples.append(self._sample_nvml(*nvml))
                    self._stop.wait(0.01)
                    continue
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) == 6:
                    self.samples.append(parts)
            except Exception:
                nvml = None             # an NVML call failed mid-run: fall back to polling nvidia-smi
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [int(s[0]) for s in self.samples if s[0].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": int(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples)}


def host_threads() -> int:
    """Host threads the CPU arm uses: the cores this process may run on.  OpenMP's own default is not used because
    launchers such as torchrun export OMP_NUM_THREADS=1 to every rank."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def identity_of(wl):
    from cuasr_b200 import RINGS, identity
    return identity(RINGS[wl.ring][0], wl.dtype) if wl.add_identity is None else wl.add_identity


def cpu_sample(wl, lines: int):
    """Host operands for the first `lines` storage lines of D (columns of a column-major D, rows of a row-major
    one): returns (mnk, A, lda, B, ldb, C, ldc) as numpy arrays.  The sampled operand is the one whose lines
    follow D's lines (B for column-major D, A for row-major D); the other operand is needed in full."""
    import numpy as np
    from cuasr_b200 import Layout
    from cuasr_b200.semiring import NUMPY_DTYPE

    np_t = NUMPY_DTYPE[wl.dtype]

    def host(which, count=None):
        t = wl.operand(which, "cpu", 0, count).numpy()
        return t.view(np.uint32) if np_t == np.uint32 else t

    ident = identity_of(wl)
    if wl.layouts[2] == Layout.COLUMN_MAJOR:
        assert wl.layouts[1] == Layout.COLUMN_MAJOR
        A, B = host("A"), host("B", wl.k * lines)
        mnk = (wl.m, lines, wl.k)
        C = np.full(wl.m * lines, ident, np_t)
        lda = wl.m if wl.layouts[0] == Layout.COLUMN_MAJOR else wl.k
        return mnk, A, lda, B, wl.k, C, wl.m
    assert wl.layouts[0] == Layout.ROW_MAJOR
    A, B = host("A", wl.k * lines), host("B")
    mnk = (lines, wl.n, wl.k)
    C = np.full(lines * wl.n, ident, np_t)
    ldb = wl.k if wl.layouts[1] == Layout.COLUMN_MAJOR else wl.n
    return mnk, A, wl.k, B, ldb, C, wl.n


def cpu_run(wl, lines: int, repeats: int = 1, warmup: int = 0):
    """Times the CPU SRGEMM on a `lines`-wide sample.  Returns (GOP/s, kind, cores, seconds, D)."""
    import numpy as np
    import oracle
    from cuasr_b200 import RINGS

    use_ref = oracle.have_ref()
    fn = oracle.ref_srgemm if use_ref else oracle.srgemm
    cores = host_threads()
    mnk, A, lda, B, ldb, C, ldc = cpu_sample(wl, lines)
    D = np.empty_like(C)
    add_op, mul_op = RINGS[wl.ring]
    alpha = np.asarray(wl.alpha).astype(C.dtype)
    beta = np.asarray(wl.beta).astype(C.dtype)
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        fn(add_op, mul_op, wl.dtype, wl.layouts, mnk, alpha, A, lda, B, ldb, beta, C, ldc, D, ldc, identity_of(wl), cores)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return 2.0 * mnk[0] * mnk[1] * mnk[2] / sec / 1e9, ("reference" if use_ref else "port"), cores, sec, D


def reference_device_kernel(wl, A, lda, B, ldb, C, ldc, D, reps: int = 3):
    """The reference's own SIMT kernel (default configuration, recompiled for sm_100a into oracle/_ref) on the
    buffers the timed region used: its time, and whether its output has the bits of `D`.  None where that library
    was not built or does not cover the workload (it is column-major only, without split-K)."""
    import torch

    import oracle
    from cuasr_b200 import Layout, RINGS

    if not oracle.have_ref_device() or wl.split_k_slices > 1 or any(l != Layout.COLUMN_MAJOR for l in wl.layouts):
        return None
    add_op, mul_op = RINGS[wl.ring]
    out = torch.empty_like(D)
    stream = torch.cuda.current_stream()

    def run():
        return oracle.ref_device_srgemm(add_op, mul_op, wl.dtype, (wl.m, wl.n, wl.k), A.data_ptr(), lda, B.data_ptr(),
                                        ldb, C.data_ptr(), ldc, out.data_ptr(), ldc, wl.alpha, wl.beta,
                                        stream.cuda_stream)

    st = run()
    if st != 0:
        return None if st == -1 else {"error": f"status {st}"}
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(reps):
        run()
    t1.record(stream)
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / reps
    return {"value": round(wl.ops / (ms * 1e-3) / 1e9, 2), "unit": "GOP/s", "ms": round(ms, 4), "launches": reps,
            "bit_identical_to_ours": bool(torch.equal(out, D)),
            "what": "the reference's cuasr::gemm::device::Srgemm, default configuration, recompiled for sm_100a, "
                    "same device buffers"}


def sample_lines(wl, target_gop: float = 9.0) -> int:
    """Lines of D whose product costs about `target_gop` GOP (a multiple of 32: the host SRGEMM works in
    32 x 32 blocks, tools/include/cuasr/reference/srgemm/host_srgemm.h:56-57)."""
    from cuasr_b200 import Layout
    total = wl.n if wl.layouts[2] == Layout.COLUMN_MAJOR else wl.m
    per_line = wl.ops / total
    lines = int(target_gop * 1e9 / per_line) // 32 * 32
    return max(32, min(total, lines))


def run_reference(args, wl):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    lines = sample_lines(wl, 40.0)
    gops, kind, cores, sec, _ = cpu_run(wl, lines, repeats=args.steps, warmup=args.warmup)
    total_lines = wl.n if int(wl.layouts[2]) == 0 else wl.m
    sample = (f"first {lines} storage lines of D of the {wl.m}x{wl.n}x{wl.k} problem per step "
              f"({wl.ops / total_lines * lines / 1e9:.1f} GOP), all {cores} host threads")
    line = {
        "impl": "reference", "metric": metric_name(wl), "value": round(gops, 3), "unit": "GOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": wl.dtype.name.lower(), "data": "synthetic",
        "config": workload_config(wl),
        "cpu_baseline": {"value": round(gops, 3), "unit": "GOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": round(gops, 3), "unit": "GOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(wl):
    from cuasr_b200 import DType
    if wl.ring == "minimum_plus" and wl.dtype == DType.F32:
        return METRIC
    return f"{wl.ring}_{wl.dtype.name.lower()}_srgemm_throughput"


def workload_config(wl):
    return {"workload": wl.name, "m": wl.m, "n": wl.n, "k": wl.k, "semiring": wl.ring,
            "layout": "/".join("col" if int(l) == 0 else "row" for l in wl.layouts) + " (A/B/C,D)",
            "split_k_slices": wl.split_k_slices}


def run_ours(args, wl):
    import numpy as np
    import torch
    import torch.distributed as dist

    from cuasr_b200 import (Arguments, DType, Layout, RINGS, Srgemm, SrgemmSplitKParallel, Status, device_status,
                            launch_count)
    from cuasr_b200.workloads import TORCH_DTYPE

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    col_major_c = wl.layouts[2] == Layout.COLUMN_MAJOR
    if world > 1:
        assert col_major_c and wl.layouts[1] == Layout.COLUMN_MAJOR and wl.n % world == 0, \
            "only column-major workloads shard over ranks"
    m, n, k = wl.m, wl.n, wl.k
    es = 8 if wl.dtype == DType.F64 else 4
    tdt = TORCH_DTYPE[wl.dtype]
    ident = identity_of(wl)
    add_op, mul_op = RINGS[wl.ring]

    # this rank's share: `cols` columns of D and of B (everything when world == 1)
    cols = n // world
    c0 = rank * cols
    lda = m if wl.layouts[0] == Layout.COLUMN_MAJOR else k
    ldb = k if wl.layouts[1] == Layout.COLUMN_MAJOR else n
    ldc = m if col_major_c else n
    A = wl.operand("A", dev)
    B = wl.operand("B", dev, c0 * k, cols * k) if world > 1 else wl.operand("B", dev)
    if wl.ld_pad:
        # same matrices, stored with padded leading dimensions
        def padded(flat, ld):
            lines = flat.numel() // ld
            out = torch.zeros(lines * (ld + wl.ld_pad), dtype=flat.dtype, device=dev)
            out.view(lines, ld + wl.ld_pad)[:, :ld].copy_(flat.view(lines, ld))
            return out
        A, B = padded(A, lda), padded(B, ldb)
        lda, ldb = lda + wl.ld_pad, ldb + wl.ld_pad
    fill = float(ident) if tdt.is_floating_point else int(ident)
    C = torch.full((m * n,), fill, dtype=tdt, device=dev)
    push = world > 1 and args.exchange == "push"
    peer_d = []
    if push:
        import torch.distributed._symmetric_memory as symm_mem
        D = symm_mem.empty(m * n, dtype=tdt, device=dev)
        handle = symm_mem.rendezvous(D, dist.group.WORLD)
        peer_d = [int(p) for p in handle.buffer_ptrs]
        D.zero_()
    else:
        D = torch.zeros(m * n, dtype=tdt, device=dev)
    off = c0 * m * es if world > 1 else 0
    extras = [p + off for r, p in enumerate(peer_d) if r != rank]
    flag = torch.zeros(1, dtype=torch.int32, device=dev)

    cls = SrgemmSplitKParallel if wl.split_k_slices > 1 else Srgemm
    op = cls(add_op, mul_op, wl.dtype, *wl.layouts, add_identity=ident)
    margs = Arguments((m, cols if world > 1 else n, k), (A, lda), (B, ldb), (C.data_ptr() + off, ldc),
                      (D.data_ptr() + off, ldc), (wl.alpha, wl.beta), wl.split_k_slices)
    ws = None
    need = op.get_workspace_size(margs)
    if not need and not args.no_workspace:
        need = op.get_optional_workspace_size(margs)            # never required: balanced last wave, re-packed operands
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream()
    st = op.initialize(margs, ws, stream)
    assert st == Status.kSuccess, st

    def launch():
        return op.run_push(extras, stream) if push else op.run(stream)

    def gather():
        if push:
            dist.all_reduce(flag)          # stream-ordered: every rank's stores into every D are complete
        elif world > 1:
            dist.all_gather_into_tensor(D, D[c0 * m:(c0 + cols) * m])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        assert launch() == Status.kSuccess
        gather()
    barrier()
    kernel_name = op.last_kernel()

    # ---- device-resident timing: CUDA events on the launching stream; kernel-only events inside ----
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record(stream)
        for i in range(args.steps):
            kev[i][0].record(stream)
            st = launch()
            kev[i][1].record(stream)
            gather()
        ev1.record(stream)
        barrier()
    launches = launch_count() - launches0
    assert st == Status.kSuccess and device_status() == 0
    t = torch.tensor([ev0.elapsed_time(ev1), statistics.mean(a.elapsed_time(b) for a, b in kev)],
                     dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step, kernel_ms = float(t[0]) / args.steps, float(t[1])
    value = wl.ops / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the host-buffer call: pinned host operands in, D out, every step ----
    # HostSrgemm = the library's host-buffer call: chunked copies overlapped with the kernel (split-K workloads and
    # layouts it cannot chunk fall back to copy, run, copy).  With several ranks every byte of A crosses a host link
    # once per node: each rank holds 1/world of every K piece of A in pinned memory, and the pipeline completes the
    # pieces on every GPU with all-gathers over NVLink while earlier pieces compute.
    from cuasr_b200 import HostSrgemm
    share = m * cols
    Cs, Ds = C[c0 * m: c0 * m + share], D[c0 * m: c0 * m + share]
    pipe = None
    if wl.split_k_slices == 1 and not wl.ld_pad:
        extra_fn = (lambda j, byte_off: [p + off + byte_off for r, p in enumerate(peer_d) if r != rank]) if push else None
        pipe = HostSrgemm(op, m, cols if world > 1 else n, k, wl.alpha, wl.beta, dev,
                          chunks=args.e2e_chunks or (8 if world == 1 else max(1, min(8, cols // 512))),
                          extra_outputs_per_chunk=extra_fn, buffers=(A, B, Cs, Ds),
                          group=dist.group.WORLD if world > 1 else None, rank=rank, world=world)
    if pipe is not None and world > 1:
        ranges = pipe.shared_share_layout()
    else:
        a_part = A.numel() // world
        ranges = [(rank * a_part, (rank + 1) * a_part)]
    # the pinned buffers of a rank come from the memory next to its GPU's host link
    from cuasr_b200.host_pipeline import numa_local
    with numa_local(dev.index if dev.index is not None else 0) as numa:
        hA = torch.empty(sum(b - a for a, b in ranges), dtype=tdt).pin_memory()
        hB = torch.empty(B.numel(), dtype=tdt).pin_memory()
        hC = torch.empty(share, dtype=tdt).pin_memory(); hC.fill_(fill)
        hD = torch.empty(share, dtype=tdt).pin_memory(); hD.zero_()
    pos = 0
    for a, b in ranges:
        hA[pos:pos + b - a].copy_(A[a:b])
        pos += b - a
    hB.copy_(B)
    e2e_steps = max(1, min(args.steps, 5))

    def e2e_step():
        if pipe is not None:
            pipe(hA, hB, hC, hD, stream)
            if world > 1:
                if push:
                    dist.all_reduce(flag)
                else:
                    dist.all_gather_into_tensor(D, Ds)
            return
        a0, a1 = ranges[0]
        A[a0:a1].copy_(hA, non_blocking=True)
        if world > 1:
            dist.all_gather_into_tensor(A, A[a0:a1])
        B.copy_(hB, non_blocking=True); Cs.copy_(hC, non_blocking=True)
        if launch() != Status.kSuccess:
            raise RuntimeError("SRGEMM launch failed")
        gather()
        hD.copy_(Ds, non_blocking=True)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t[0]) / e2e_steps
    # bytes of the whole job per step: every rank's part of A, its columns of B and C in, its columns of D out
    h2d = (hA.numel() + hB.numel() + hC.numel()) * es * world
    d2h = hD.numel() * es * world

    # ---- the north star's second metric, at every N: the whole n = 16384 APSP solve, sharded over the ranks ----
    apsp_rec = None
    if wl.name == "minplus_f32_8192" and not args.no_apsp:
        from cuasr_b200.workloads import WORKLOADS
        apsp_rec = apsp_solve_record(WORKLOADS["apsp_16384"], rank, world, dev, args.exchange)

    # ---- rank 0: spot check against the CPU oracle, CPU baseline, JSON line ----
    if rank == 0:
        _, _, _, _, want = cpu_run(wl, 32)
        got = D[: want.size].cpu().numpy()
        got = got.view(np.uint32) if want.dtype == np.uint32 else got
        if wl.ring == "plus_multiplies":
            parity = bool(np.allclose(got, want, rtol=0, atol=8 * k * np.finfo(want.dtype).eps * (wl.hi ** 2)))
        else:
            parity = bool(np.array_equal(got, want))
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            lines = sample_lines(wl, 400.0)     # about ten seconds of host work
            gops, kind, cores, sec, _ = cpu_run(wl, lines)
            cpu = {"value": round(gops, 3), "unit": "GOP/s", "cores": cores, "kind": kind,
                   "sample": f"first {lines} storage lines of D, one pass ({sec:.1f} s), all {cores} host threads"}
        refdev = None
        if world == 1 and not args.no_cpu_baseline:
            assert op.initialize(margs, ws, stream) == Status.kSuccess and launch() == Status.kSuccess
            torch.cuda.synchronize()
            refdev = reference_device_kernel(wl, A, lda, B, ldb, C, ldc, D)
        peaks, peak_kind = measured_peaks()
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        peak_tops = sms * 128 * 2 * peaks["sm_max_mhz"] * 1e6 / 1e12
        achieved = (wl.ops / world) / (kernel_ms * 1e-3) / 1e12
        algorithmic_bytes = es * (m * k + k * cols + 2 * m * cols)   # A + B block + C block read + D block written
        line = {
            "metric": metric_name(wl),
            "value": round(value, 2), "unit": "GOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": wl.dtype.name.lower(), "data": "synthetic",
            "config": dict(workload_config(wl), kernel=kernel_name,
                           sharding=f"{cols} columns of D per rank" + (
                               "" if world == 1 else ", epilogue stores D to every peer + barrier" if push
                               else ", NCCL all-gather of D"),
                           l2="operands exceed the 126 MB L2" if es * (m * k + k * n) > 126e6 else
                              "L2 flushed between steps by the other operands' traffic: NO (operands fit L2)"),
            "e2e": {"value": round(wl.ops / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps,
                    "pinned_memory_numa_node": numa.node},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "CUDA cores (issue / register-file ports); HBM is orders of magnitude below",
                         "achieved": round(achieved, 3), "peak": round(peak_tops, 2), "unit": "TOP/s",
                         "frac": round(achieved / peak_tops, 4),
                         # against one semiring operation per lane per clock (half the FP32-FMA line): the ceiling
                         # of any formulation that spends one issued lane-instruction per operation
                         "achieved_vs_1op_per_lane_clk": round(achieved / (peak_tops / 2), 4),
                         "peak_source": f"{sms} SMs x 128 lanes x 2 x sm_max_mhz ({peak_kind} clock {peaks['sm_max_mhz']:.0f} MHz)",
                         "kernel_ms": round(kernel_ms, 4),
                         "hbm_achieved_gbs": round(algorithmic_bytes / (kernel_ms * 1e-3) / 1e9, 2),
                         "hbm_peak_gbs": peaks["hbm_gbs"],
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from an ncu capture
                         "traffic": dram_traffic(wl.name) if world == 1 else None},
            "cpu_baseline": cpu,
            "reference_device_kernel": refdev,
            "parity_spot_check": parity,
            "apsp_16384": apsp_rec,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def apsp_solve_record(wl, rank, world, dev, exchange):
    """One whole sharded APSP solve by repeated squaring (ceil(log2 n) squarings of the graph of `wl`): the adjacency
    matrix comes from pinned host memory, every rank's block of distances goes back.  Returns, on rank 0, seconds of
    the squarings alone and end to end (device events, max over ranks) and a check of the last squaring against the
    host SRGEMM; None on the other ranks."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import oracle
    from cuasr_b200 import DType, Layout, Op, device_status
    from cuasr_b200.apsp import CudaBackend, ShardedSquaring

    n = wl.n
    squarings = ShardedSquaring.squarings_needed(n)
    backend = CudaBackend(n, rank, world, dev, mode=exchange)
    solver = ShardedSquaring(n, rank, world, backend)
    stream = torch.cuda.current_stream()
    host_in = torch.empty(n * n, dtype=torch.float32).pin_memory()
    host_in.copy_(wl.operand("A", dev))
    host_out = torch.empty(n * n // world, dtype=torch.float32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    backend.bufs[0].copy_(host_in, non_blocking=True)
    solver.step()                                   # warm-up: workspace allocation, first-launch costs
    barrier()
    e0, k0, k1, e1 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
    solver.cur, solver.nxt = 0, 1
    e0.record(stream)
    backend.bufs[0].copy_(host_in, non_blocking=True)
    k0.record(stream)
    for _ in range(squarings - 1):
        solver.step()
    k1.record(stream)
    before_last = backend.matrix(solver.cur).clone()
    k2, k3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k2.record(stream)
    solver.step()
    k3.record(stream)
    mine = backend.matrix(solver.cur)[solver.c0 * n:(solver.c0 + solver.cols) * n]
    host_out.copy_(mine, non_blocking=True)
    e1.record(stream)
    barrier()
    clone_ms = k1.elapsed_time(k2)                 # the copy kept for the check is not part of the solve
    t = torch.tensor([k0.elapsed_time(k1) + k2.elapsed_time(k3), e0.elapsed_time(e1) - clone_ms],
                     dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = device_status() == 0
    if rank != 0:
        return None
    src = before_last.cpu().numpy()
    blk = np.ascontiguousarray(src[: 32 * n])
    want = np.empty(32 * n, np.float32)
    fn = oracle.ref_srgemm if oracle.have_ref() else oracle.srgemm
    col = Layout.COLUMN_MAJOR
    fn(Op.MINIMUM, Op.PLUS, DType.F32, (col, col, col), (n, 32, n), 0.0, src, n, blk, n, 0.0, blk, n, want, n,
       np.float32(np.inf), host_threads())
    return {"n": n, "squarings": squarings, "seconds": round(float(t[0]) * 1e-3, 4),
            "seconds_end_to_end": round(float(t[1]) * 1e-3, 4), "exchange": exchange if world > 1 else "none",
            "sharding": f"{n // world} columns of D per rank",
            "parity_spot_check": bool(ok and np.array_equal(host_out.numpy()[: 32 * n], want))}


def run_path(args, wl):
    """Path-tracking product: one step = dist <- min(dist, A (x) B) from dist = +inf with the index of the first best
    k recorded for every element (cuasr_b200_srgemm_path), single GPU."""
    import numpy as np
    import torch

    import oracle
    from cuasr_b200 import DType, RINGS, Srgemm, Status, device_status, launch_count, srgemm_path

    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    m, n, k = wl.m, wl.n, wl.k
    A, B = wl.operand("A", dev), wl.operand("B", dev)
    D = torch.empty(m * n, dtype=torch.float32, device=dev)
    P = torch.empty(m * n, dtype=torch.int32, device=dev)
    op = Srgemm(*RINGS[wl.ring], wl.dtype, *wl.layouts, add_identity=identity_of(wl))
    stream = torch.cuda.current_stream()

    def step():
        D.fill_(float("inf")); P.fill_(-1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        st = srgemm_path(op, (m, n, k), (A, m), (B, k), (D, m), (P, m), stream=stream)
        e1.record(stream)
        assert st == Status.kSuccess
        return e0, e1

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    launches0 = launch_count()
    with ClockSampler(0) as clocks:
        events = [step() for _ in range(args.steps)]
        torch.cuda.synchronize()
    launches = launch_count() - launches0
    assert device_status() == 0
    ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    # the same product once more on the finished distances: nothing improves any more (the state of a late
    # Floyd-Warshall or squaring step), so the index bookkeeping is never entered
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record(stream)
    assert srgemm_path(op, (m, n, k), (A, m), (B, k), (D, m), (P, m), stream=stream) == Status.kSuccess
    w1.record(stream)
    torch.cuda.synchronize()
    settled_ms = w0.elapsed_time(w1)
    # end to end: operands from pinned host memory, distances and parents back
    hA = torch.empty(A.numel(), dtype=torch.float32).pin_memory(); hA.copy_(A)
    hB = torch.empty(B.numel(), dtype=torch.float32).pin_memory(); hB.copy_(B)
    hD = torch.empty(D.numel(), dtype=torch.float32).pin_memory()
    hP = torch.empty(P.numel(), dtype=torch.int32).pin_memory()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    A.copy_(hA, non_blocking=True); B.copy_(hB, non_blocking=True)
    step()
    hD.copy_(D, non_blocking=True); hP.copy_(P, non_blocking=True)
    e1.record(stream)
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    # 8 columns against the host routine
    d0, p0 = np.full(8 * m, np.inf, np.float32), np.full(8 * m, -1, np.int32)
    t0 = time.perf_counter()
    want_d, want_p = oracle.srgemm_path(DType.F32, wl.layouts, (m, 8, k), hA.numpy(), m, hB.numpy()[: 8 * k], k, d0, m, p0, m)
    cpu_sec = time.perf_counter() - t0
    parity = bool(np.array_equal(hD.numpy()[: 8 * m], want_d) and np.array_equal(hP.numpy()[: 8 * m], want_p))
    peaks, peak_kind = measured_peaks()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    peak_tops = sms * 128 * 2 * peaks["sm_max_mhz"] * 1e6 / 1e12
    achieved = wl.ops / (ms * 1e-3) / 1e12
    line = {
        "metric": "minplus_path_f32_srgemm_throughput", "value": round(wl.ops / (ms * 1e-3) / 1e9, 2), "unit": "GOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(workload_config(wl), kernel=op.last_kernel(), l2="operands (128 MiB) exceed the 126 MB L2"),
        "e2e": {"value": round(wl.ops / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GOP/s", "h2d_bytes_per_step": 4 * (m * k + k * n),
                "d2h_bytes_per_step": 8 * m * n, "ms_per_step": round(e2e_ms, 3), "steps": 1},
        "gpu_launches": int(launches), "clocks": clocks.summary(),
        "roofline": {"bound": "CUDA cores (issue / register-file ports)", "achieved": round(achieved, 3),
                     "peak": round(peak_tops, 2), "unit": "TOP/s", "frac": round(achieved / peak_tops, 4),
                     "peak_source": f"{sms} SMs x 128 lanes x 2 x sm_max_mhz ({peak_kind})", "kernel_ms": round(ms, 4),
                     "kernel_ms_when_nothing_improves": round(settled_ms, 4), "traffic": None},
        "cpu_baseline": {"value": round(2.0 * m * 8 * k / cpu_sec / 1e9, 3), "unit": "GOP/s", "cores": 1, "kind": "port",
                         "sample": f"8 columns of D ({2.0 * m * 8 * k / 1e9:.2f} GOP), the scalar path-tracking loop"},
        "parity_spot_check": parity,
    }
    print(json.dumps(line), flush=True)


def run_apsp_fw(args, wl):
    """Blocked Floyd-Warshall workload: one step = one whole APSP solve (2 n^3 semiring operations)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from cuasr_b200 import device_status
    from cuasr_b200.apsp import BlockedFloydWarshall

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n = wl.n
    cols = n // world
    block = min(args.fw_block or (1024 if world <= 2 else 512), cols)
    solver = BlockedFloydWarshall(n, block, rank, world, dev, mode=args.exchange)
    # this rank's column blocks of the adjacency matrix, in the order the solver stores them (block-cyclic)
    mine = torch.cat([wl.operand("A", dev, kb * block * n, block * n) for kb in solver.owned_blocks()])
    host_in = torch.empty(cols * n, dtype=torch.float32).pin_memory()
    host_in.copy_(mine)
    host_out = torch.empty(cols * n, dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def solve_from_host():
        solver.D.copy_(host_in, non_blocking=True)
        solver.solve()
        host_out.copy_(solver.D, non_blocking=True)

    for _ in range(max(1, min(args.warmup, 2))):
        solver.load_columns(mine)
        solver.solve()
    barrier()
    times = []
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.steps):
            solver.load_columns(mine)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            solver.solve()
            e1.record(stream)
            barrier()
            times.append(e0.elapsed_time(e1))
    launches_per_solve = solver.launches // (args.steps + max(1, min(args.warmup, 2)))
    assert device_status() == 0
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    solve_from_host()
    e1.record(stream)
    barrier()
    t = torch.tensor([sum(times) / len(times), e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    # fixed point, at every world size: one more min-plus step over sampled columns must change nothing (checked by
    # the host SRGEMM on rank 0).  With several ranks the distributed result is first gathered over NCCL.
    blocks_of = lambda r: [kb for kb in range(n // block) if solver.owner(kb) == r]
    if world > 1:
        gathered = torch.empty(world * cols * n, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(gathered, solver.D)
    else:
        gathered = solver.D
    parity = None
    if rank == 0:
        import oracle
        from cuasr_b200 import DType, Layout, Op
        full_dev = torch.empty(n * n, dtype=torch.float32, device=dev)
        for r in range(world):
            for i, kb in enumerate(blocks_of(r)):
                src = gathered[(r * cols + i * block) * n:(r * cols + (i + 1) * block) * n]
                full_dev[kb * block * n:(kb + 1) * block * n].copy_(src)
        full = full_dev.cpu().numpy()
        del full_dev
        fn = oracle.ref_srgemm if oracle.have_ref() else oracle.srgemm
        col = Layout.COLUMN_MAJOR
        parity = True
        # the first columns (rank 0's), 32 in the middle, and the last (another rank's where there is one)
        for c0 in sorted({0, (n // 2) // 32 * 32, n - 32}):
            blk = np.ascontiguousarray(full[c0 * n:(c0 + 32) * n])
            again = np.empty_like(blk)
            fn(Op.MINIMUM, Op.PLUS, DType.F32, (col, col, col), (n, 32, n), 0.0, full, n, blk, n, 0.0, blk, n, again, n,
               np.float32(np.inf), host_threads())
            parity = parity and bool(np.array_equal(again, blk))
        line = {
            "metric": "apsp_blocked_floyd_warshall_seconds", "value": round(ms * 1e-3, 5), "unit": "s", "n_gpus": world,
            "steps": args.steps, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": round(ms, 3),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload_config(wl), block=block, exchange=args.exchange if world > 1 else "none",
                           distribution=f"block-{solver.distribution} columns" if world > 1 else "one rank",
                           algorithm="three-phase blocked Floyd-Warshall on the min-plus SRGEMM"),
            "semiring_gops": round(2.0 * n ** 3 / (ms * 1e-3) / 1e9, 1),
            "e2e": {"value": round(e2e_ms * 1e-3, 5), "unit": "s", "h2d_bytes_per_step": cols * n * 4,
                    "d2h_bytes_per_step": cols * n * 4},
            "gpu_launches": int(launches_per_solve),
            "clocks": clocks.summary(),
            "parity_spot_check": parity,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_apsp(args, wl):
    """APSP workloads: one step = one squaring D <- min(D, D (x) D) of the sharded solve (cuasr_b200/apsp.py);
    the line also carries the whole solve (ceil(log2 n) squarings) in seconds."""
    import numpy as np
    import torch
    import torch.distributed as dist

    import oracle
    from cuasr_b200 import DType, Layout, Op, device_status, launch_count
    from cuasr_b200.apsp import CudaBackend, ShardedSquaring

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n = wl.n
    squarings = ShardedSquaring.squarings_needed(n)
    backend = CudaBackend(n, rank, world, dev, mode=args.exchange)
    graph = wl.operand("A", dev)
    backend.load(0, graph)
    solver = ShardedSquaring(n, rank, world, backend)
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        solver.step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = launch_count()
    before_last = None
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record(stream)
        for _ in range(args.steps):
            solver.step()
        ev1.record(stream)
        barrier()
    launches = launch_count() - launches0
    assert device_status() == 0
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t[0]) / args.steps
    value = wl.ops / (ms_per_step * 1e-3) / 1e9

    # ---- the whole solve end to end: adjacency matrix from pinned host memory, distances back ----
    host_in = torch.empty(n * n, dtype=torch.float32).pin_memory()
    host_in.copy_(graph)
    host_out = torch.empty(n * n // world, dtype=torch.float32).pin_memory()
    del graph
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    solver.cur, solver.nxt = 0, 1
    backend.bufs[0].copy_(host_in, non_blocking=True)
    for s in range(squarings):
        if s == squarings - 1:
            before_last = backend.matrix(solver.cur).clone()
        solver.step()
    mine = backend.matrix(solver.cur)[solver.c0 * n:(solver.c0 + solver.cols) * n]
    host_out.copy_(mine, non_blocking=True)
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    solve_ms = float(t[0])

    if rank == 0:
        # 32 columns of the last squaring against the oracle fed that squaring's input
        src = before_last.cpu().numpy()
        blk = np.ascontiguousarray(src[: 32 * n])
        want = np.empty(32 * n, np.float32)
        fn = oracle.ref_srgemm if oracle.have_ref() else oracle.srgemm
        col = Layout.COLUMN_MAJOR
        t0 = time.perf_counter()
        fn(Op.MINIMUM, Op.PLUS, DType.F32, (col, col, col), (n, 32, n), 0.0, src, n, blk, n, 0.0, blk, n, want, n,
           np.float32(np.inf), host_threads())
        cpu_sec = time.perf_counter() - t0
        parity = bool(np.array_equal(host_out.numpy()[: 32 * n], want))
        cores = host_threads()
        peaks, peak_kind = measured_peaks()
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        peak_tops = sms * 128 * 2 * peaks["sm_max_mhz"] * 1e6 / 1e12
        achieved = (wl.ops / world) / (ms_per_step * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload_config(wl), kernel="tma", exchange=args.exchange if world > 1 else "none",
                           sharding=f"{n // world} columns of D per rank", l2="matrix (%d MiB) exceeds the 126 MB L2" % (n * n * 4 >> 20)),
            "apsp": {"n": n, "squarings": squarings, "seconds": round(squarings * ms_per_step * 1e-3, 4),
                     "seconds_end_to_end": round(solve_ms * 1e-3, 4)},
            "e2e": {"value": round(squarings * wl.ops / (solve_ms * 1e-3) / 1e9, 2), "unit": "GOP/s",
                    "h2d_bytes_per_step": n * n * 4 // squarings, "d2h_bytes_per_step": n * n * 4 // world // squarings,
                    "ms_per_step": round(solve_ms / squarings, 3), "steps": squarings,
                    "note": "one whole solve: adjacency matrix in from pinned host memory, all squarings, this rank's block of distances out"},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "CUDA cores (issue / register-file ports)", "achieved": round(achieved, 3),
                         "peak": round(peak_tops, 2), "unit": "TOP/s", "frac": round(achieved / peak_tops, 4),
                         "peak_source": f"{sms} SMs x 128 lanes x 2 x sm_max_mhz ({peak_kind})",
                         "kernel_ms": round(ms_per_step, 4), "note": "step time includes the exchange", "traffic": None},
            "cpu_baseline": {"value": round(2.0 * n * n * 32 / cpu_sec / 1e9, 3), "unit": "GOP/s", "cores": cores,
                             "kind": "reference" if oracle.have_ref() else "port",
                             "sample": f"32 columns of the last squaring ({2.0 * n * n * 32 / 1e9:.1f} GOP), all {cores} host threads"},
            "parity_spot_check": parity,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    from cuasr_b200.workloads import WORKLOADS

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="minplus_f32_8192")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU-baseline leg (profiling runs)")
    ap.add_argument("--e2e-chunks", type=int, default=0,
                    help="column chunks of the end-to-end (host buffer) step; 0 = 8 on one GPU, 512-column chunks beyond")
    ap.add_argument("--no-workspace", action="store_true",
                    help="do not hand the library the optional workspace (no balanced last wave, no re-packed operands)")
    ap.add_argument("--no-apsp", action="store_true",
                    help="skip the n = 16384 APSP solve appended to the default workload's line (profiling runs)")
    ap.add_argument("--fw-block", type=int, default=0,
                    help="block size of the blocked Floyd-Warshall workload (0: 1024 up to 2 GPUs, 512 beyond)")
    ap.add_argument("--exchange", choices=("push", "allgather"), default="push",
                    help="N > 1: how D reaches every rank -- stored to peers by the SRGEMM epilogue, or NCCL all-gather")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        args.warmup = max(args.warmup, 3)
        if wl.path:
            run_path(args, wl)
        elif wl.name.startswith("apsp_fw"):
            run_apsp_fw(args, wl)
        elif wl.fill == "apsp":
            run_apsp(args, wl)
        else:
            run_ours(args, wl)


if __name__ == "__main__":
    main()
