"""Benchmark of the SRGEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (`minplus_f32_8192`): min-plus fp32 SRGEMM D = min(C, A (x) B) with M = N = K = 8192, all
matrices column-major, A and B uniform in [0, 100) from a seed, C filled with the additive identity.  One step
is one SRGEMM; at N > 1 GPUs the columns of D (contiguous blocks of a column-major matrix) are sharded over
the ranks and the step ends with an all-gather of D, which is exactly one squaring step of the sharded
all-pairs-shortest-paths solve.  Prints ONE JSON line on rank 0.

`--impl reference` times the reference's own host SRGEMM (oracle/_ref, else the C restatement in oracle/)
on the host cores, on a bounded sample of the same workload.
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

WORKLOADS = {
    # name: (n, description)
    "minplus_f32_8192": 8192,
    "minplus_f32_4096": 4096,
    "minplus_f32_16384": 16384,
}
SEED_A, SEED_B = 3090, 3091  # the seeds of examples/00_minplus_srgemm/minplus_srgemm.cu:108-110


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "sm_max_mhz": 1965.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._thread = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) == 6:
                    self.samples.append(parts)
            except Exception:
                pass
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


def host_operands(n: int, rows_of_d: int | None = None):
    """Column-major A (n x n), B (n x n) as flat numpy float32 arrays (the CPU arm's inputs)."""
    from cuasr_b200 import datagen
    A = datagen.uniform_f32(SEED_A, n * n, 0.0, 100.0).numpy()
    B = datagen.uniform_f32(SEED_B, n * n, 0.0, 100.0).numpy()
    return A, B


def cpu_arm(n: int, cols: int, repeats: int = 1, warmup: int = 0):
    """Times the CPU SRGEMM on the first `cols` columns of D (D[:, :cols] = A (x) B[:, :cols]; 2 n^2 cols ops).
    Returns (GOP/s, kind, cores, seconds per repeat)."""
    import numpy as np
    import oracle
    from cuasr_b200 import DType, Layout, Op, identity

    use_ref = oracle.have_ref()
    fn = oracle.ref_srgemm if use_ref else oracle.srgemm
    cores = oracle.max_threads(use_ref)
    A, B = host_operands(n)
    ident = identity(Op.MINIMUM, DType.F32)
    C = np.full(n * cols, ident, np.float32)
    D = np.empty(n * cols, np.float32)
    col = Layout.COLUMN_MAJOR
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        fn(Op.MINIMUM, Op.PLUS, DType.F32, (col, col, col), (n, cols, n), 0.0, A, n, B, n, 0.0, C, n, D, n, ident, cores)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return 2.0 * n * n * cols / sec / 1e9, ("reference" if use_ref else "port"), cores, sec


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = WORKLOADS[args.workload]
    cols = 64 if n >= 8192 else 256
    gops, kind, cores, sec = cpu_arm(n, cols, repeats=args.steps, warmup=args.warmup)
    sample = f"D[:, :{cols}] of the {n}^3 problem per step ({2.0 * n * n * cols / 1e9:.1f} GOP), all {cores} host threads"
    line = {
        "impl": "reference", "metric": "minplus_f32_srgemm_throughput", "value": round(gops, 3), "unit": "GOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "m": n, "n": n, "k": n, "layout": "column-major A, B, C, D",
                   "semiring": "min-plus"},
        "cpu_baseline": {"value": round(gops, 3), "unit": "GOP/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": round(gops, 3), "unit": "GOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    from cuasr_b200 import Arguments, DType, Layout, Op, Srgemm, Status, datagen, device_status, identity, launch_count

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    n = WORKLOADS[args.workload]
    assert n % world == 0
    cols = n // world                      # columns of D (and of B) this rank owns
    c0 = rank * cols
    ident = identity(Op.MINIMUM, DType.F32)
    col = Layout.COLUMN_MAJOR

    # operands resident in HBM: full A, this rank's column block of B, full C and D (column-major, ld = n)
    A = datagen.uniform_f32(SEED_A, n * n, 0.0, 100.0, device=dev)
    B = datagen.uniform_f32(SEED_B, n * cols, 0.0, 100.0, device=dev, start=c0 * n)
    C = torch.full((n * n,), float(ident), dtype=torch.float32, device=dev)
    D = torch.zeros(n * n, dtype=torch.float32, device=dev)
    es = 4
    op = Srgemm(Op.MINIMUM, Op.PLUS, DType.F32, col, col, col)
    margs = Arguments((n, cols, n), (A, n), (B, n), (C.data_ptr() + c0 * n * es, n), (D.data_ptr() + c0 * n * es, n),
                      (0.0, 0.0))
    stream = torch.cuda.current_stream()
    assert op.initialize(margs, None, stream) == Status.kSuccess

    def step():
        st = op.run(stream)
        if st != Status.kSuccess:
            raise RuntimeError(f"SRGEMM launch failed: {st!r}")
        if world > 1:
            dist.all_gather_into_tensor(D, D[c0 * n:(c0 + cols) * n])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()

    # ---- device-resident timing: CUDA events on the launching stream, kernel events inside ----
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record(stream)
        for i in range(args.steps):
            kev[i][0].record(stream)
            st = op.run(stream)
            kev[i][1].record(stream)
            if world > 1:
                dist.all_gather_into_tensor(D, D[c0 * n:(c0 + cols) * n])
        ev1.record(stream)
        barrier()
    launches = launch_count() - launches0
    assert st == Status.kSuccess and device_status() == 0
    ms_total = ev0.elapsed_time(ev1)
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in kev)
    t = torch.tensor([ms_total, kernel_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, kernel_ms = float(t[0]), float(t[1])
    ms_per_step = ms_total / args.steps
    ops_per_step = 2.0 * n * n * n
    value = ops_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the host-buffer call: pinned host operands in, D out, every step ----
    hA = torch.empty(n * n, dtype=torch.float32).pin_memory()
    hB = torch.empty(n * cols, dtype=torch.float32).pin_memory()
    hC = torch.empty(n * cols, dtype=torch.float32).pin_memory()
    hD = torch.empty(n * cols, dtype=torch.float32).pin_memory()
    hA.copy_(A); hB.copy_(B); hC.fill_(float(ident))
    Cs, Ds = C[c0 * n:(c0 + cols) * n], D[c0 * n:(c0 + cols) * n]
    e2e_steps = max(1, min(args.steps, 5))

    def e2e_step():
        A.copy_(hA, non_blocking=True); B.copy_(hB, non_blocking=True); Cs.copy_(hC, non_blocking=True)
        if op.run(stream) != Status.kSuccess:
            raise RuntimeError("SRGEMM launch failed")
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
    e2e_value = ops_per_step / (e2e_ms * 1e-3) / 1e9
    h2d = (hA.numel() + hB.numel() + hC.numel()) * es
    d2h = hD.numel() * es

    # ---- spot check of the timed result against the CPU oracle (a few columns of D) ----
    parity = None
    cpu = None
    if rank == 0:
        import numpy as np
        import oracle
        check_cols = 4
        hostA, hostB = host_operands(n)
        want = np.empty(n * check_cols, np.float32)
        Cc = np.full(n * check_cols, ident, np.float32)
        fn = oracle.ref_srgemm if oracle.have_ref() else oracle.srgemm
        fn(Op.MINIMUM, Op.PLUS, DType.F32, (col, col, col), (n, check_cols, n), 0.0, hostA, n, hostB, n, 0.0, Cc, n,
           want, n, ident, 0)
        got = D[: n * check_cols].cpu().numpy()
        parity = bool(np.array_equal(got, want))
        if world == 1 and not args.no_cpu_baseline:
            sample_cols = 64 if n >= 8192 else 256
            gops, kind, cores, sec = cpu_arm(n, sample_cols, repeats=1, warmup=0)
            cpu = {"value": round(gops, 3), "unit": "GOP/s", "cores": cores, "kind": kind,
                   "sample": f"D[:, :{sample_cols}] of the {n}^3 problem, one pass ({sec:.1f} s), all {cores} host threads"}

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        props = torch.cuda.get_device_properties(dev)
        sms = props.multi_processor_count
        peak_tops = sms * 128 * 2 * peaks["sm_max_mhz"] * 1e6 / 1e12
        k_ops = 2.0 * n * cols * n                     # one launch on one rank
        achieved = k_ops / (kernel_ms * 1e-3) / 1e12
        algorithmic_bytes = es * (n * n + n * cols + 2 * n * cols)   # A + B block + C block read + D block written
        line = {
            "metric": "minplus_f32_srgemm_throughput", "value": round(value, 2), "unit": "GOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "m": n, "n": n, "k": n, "layout": "column-major A, B, C, D",
                       "semiring": "min-plus", "sharding": f"{cols} columns of D per rank" + (", all-gather of D" if world > 1 else ""),
                       "l2": "operands (3 x %d MiB) exceed the 126 MB L2" % (n * n * es >> 20)},
            "e2e": {"value": round(e2e_value, 2), "unit": "GOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "fp32 CUDA cores (issue/ALU pipes); HBM is three orders below", "achieved": round(achieved, 3),
                         "peak": round(peak_tops, 2), "unit": "TOP/s", "frac": round(achieved / peak_tops, 4),
                         "peak_source": f"{sms} SMs x 128 lanes x 2 x sm_max_mhz ({peak_kind} clock {peaks['sm_max_mhz']:.0f} MHz)",
                         "kernel_ms": round(kernel_ms, 4),
                         "hbm_achieved_gbs": round(algorithmic_bytes / (kernel_ms * 1e-3) / 1e9, 2),
                         "hbm_peak_gbs": peaks["hbm_gbs"], "traffic": None},
            "cpu_baseline": cpu,
            "parity_spot_check": parity,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="minplus_f32_8192")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU-baseline leg (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
