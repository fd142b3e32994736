"""The benchmark configurations, as seeded synthetic operands.

Each workload describes one SRGEMM: ring, element type, shape, layouts, how A, B and C are filled (on any torch
device, or any sub-range on the host for spot checks) and the epilogue scalars.  No dataset is involved; the
generators below are the workloads.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Callable, Optional, Tuple

import torch

from . import datagen
from .semiring import DType, Layout, Op, RINGS

COL, ROW = Layout.COLUMN_MAJOR, Layout.ROW_MAJOR
TORCH_DTYPE = {DType.F32: torch.float32, DType.F64: torch.float64, DType.S32: torch.int32, DType.U32: torch.int32}
SEED_A, SEED_B, SEED_C = 3090, 3091, 3092  # examples/00_minplus_srgemm/minplus_srgemm.cu:108-110


@dataclasses.dataclass(frozen=True)
class Workload:
    name: str
    ring: str
    dtype: DType
    m: int
    n: int
    k: int
    layouts: Tuple[Layout, Layout, Layout]
    fill: str                      # "uniform", "graph", "apsp", "ints", "words"
    lo: float = 0.0
    hi: float = 1.0
    density: float = 1.0           # "graph": probability that an entry is present
    add_identity: Optional[float] = None   # None: the reference's constant for the ring
    alpha: float = 0.0
    beta: float = 0.0
    split_k_slices: int = 1
    description: str = ""
    path: bool = False             # path-tracking product (distances and the index of the best k)
    ld_pad: int = 0                # elements added to the leading dimensions of A and B (an odd value makes them
                                   # operands TMA cannot describe)

    @property
    def ops(self) -> float:
        return 2.0 * self.m * self.n * self.k

    def operand(self, which: str, device="cpu", start: int = 0, count: Optional[int] = None) -> torch.Tensor:
        """Elements [start, start + count) of the flat storage of operand "A" or "B" (leading dimension = the
        contiguous extent)."""
        total = self.m * self.k if which == "A" else self.k * self.n
        count = total - start if count is None else count
        seed = SEED_A if which == "A" else SEED_B
        if self.fill == "uniform":
            fn = datagen.uniform_f32 if self.dtype == DType.F32 else datagen.uniform_f64
            return fn(seed, count, self.lo, self.hi, device=device, start=start)
        if self.fill == "ints":
            # whole numbers in [lo, hi): sums stay far from the 32-bit range, so nothing wraps on either side
            return datagen.uniform_f32(seed, count, self.lo, self.hi, device=device, start=start).to(TORCH_DTYPE[self.dtype])
        if self.fill == "words":
            return datagen.words_u32(seed, count, device=device, start=start)
        if self.fill == "apsp":
            # A and B are the same matrix: the weighted adjacency matrix of the graph being solved
            assert self.m == self.n == self.k and start % self.n == 0 and count % self.n == 0
            return datagen.sparse_graph(SEED_A, self.n, self.density, self.absent(), dtype=torch.float32,
                                        device=device, weight_lo=int(self.lo), weight_hi=int(self.hi),
                                        integer_weights=True, row_start=start // self.n, rows=count // self.n)
        if self.fill == "graph":
            # square matrices only; storage line index = start // n works for either layout because the
            # generator is symmetric in how it treats rows and columns of the flat index
            assert self.m == self.n == self.k and start % self.n == 0 and count % self.n == 0
            return datagen.sparse_graph(seed, self.n, self.density, self.absent(), dtype=TORCH_DTYPE[self.dtype],
                                        device=device, weight_lo=int(self.lo), weight_hi=int(self.hi),
                                        integer_weights=False, row_start=start // self.n, rows=count // self.n)
        raise ValueError(self.fill)

    def absent(self) -> float:
        add_op = RINGS[self.ring][0]
        return math.inf if add_op == Op.MINIMUM else -math.inf


WORKLOADS = {w.name: w for w in [
    Workload("minplus_f32_8192", "minimum_plus", DType.F32, 8192, 8192, 8192, (COL, COL, COL), "uniform", 0.0, 100.0,
             description="north star: min-plus fp32, M = N = K = 8192, column-major, A, B uniform [0, 100), C = additive identity"),
    Workload("minplus_f32_4096", "minimum_plus", DType.F32, 4096, 4096, 4096, (COL, COL, COL), "uniform", 0.0, 100.0),
    Workload("minplus_f32_4096_ld4097", "minimum_plus", DType.F32, 4096, 4096, 4096, (COL, COL, COL), "uniform", 0.0, 100.0,
             ld_pad=1, description="min-plus fp32 4096^3 with leading dimension 4097 for A and B: operands TMA cannot "
                                   "describe (the reference accepts any leading dimension)"),
    Workload("minplus_path_f32_4096", "minimum_plus", DType.F32, 4096, 4096, 4096, (COL, COL, COL), "uniform", 0.0, 100.0,
             add_identity=math.inf, path=True,
             description="path-tracking min-plus fp32 4096^3: distances (from +inf) and the first best k of every element"),
    Workload("minplus_f32_512", "minimum_plus", DType.F32, 512, 512, 512, (COL, COL, COL), "uniform", 0.0, 100.0,
             description="config 1: the reference's own CPU-runnable case"),
    Workload("minplus_f64_8192", "minimum_plus", DType.F64, 8192, 8192, 8192, (COL, COL, COL), "graph", 1.0, 1000.0,
             density=0.1, add_identity=math.inf,
             description="config 2: weighted adjacency matrices, 10 % present in [1, 1000), absent = +inf, diagonal 0"),
    Workload("minplus_f64_4096", "minimum_plus", DType.F64, 4096, 4096, 4096, (COL, COL, COL), "graph", 1.0, 1000.0,
             density=0.1, add_identity=math.inf, description="config 2 at half the size (profiling captures)"),
    Workload("maxplus_f64_8192", "maximum_plus", DType.F64, 8192, 8192, 8192, (COL, COL, COL), "graph", 1.0, 1000.0,
             density=0.1, add_identity=-math.inf,
             description="config 2: as above with absent = -inf"),
    Workload("splitk_minplus_f32_s16", "minimum_plus", DType.F32, 256, 256, 1048576, (ROW, COL, ROW), "uniform", 0.0, 1.0,
             split_k_slices=16, description="config 3: tall-skinny contraction, 16 slices"),
    Workload("splitk_minplus_f32_s32", "minimum_plus", DType.F32, 256, 256, 1048576, (ROW, COL, ROW), "uniform", 0.0, 1.0,
             split_k_slices=32, description="config 3: 32 slices"),
    Workload("splitk_minplus_f32_s64", "minimum_plus", DType.F32, 256, 256, 1048576, (ROW, COL, ROW), "uniform", 0.0, 1.0,
             split_k_slices=64, description="config 3: 64 slices"),
    Workload("apsp_16384", "minimum_plus", DType.F32, 16384, 16384, 16384, (COL, COL, COL), "apsp", 1.0, 100.0,
             density=0.01, add_identity=math.inf,
             description="config 4: APSP by repeated squaring, G(n = 16384, p = 0.01), integer weights 1..100 as fp32, "
                         "14 squarings; one step = one squaring D <- min(D, D (x) D)"),
    Workload("apsp_fw_16384", "minimum_plus", DType.F32, 16384, 16384, 16384, (COL, COL, COL), "apsp", 1.0, 100.0,
             density=0.01, add_identity=math.inf,
             description="the graph of config 4 solved by blocked Floyd-Warshall on the same SRGEMM (one step = one solve)"),
    Workload("apsp_4096", "minimum_plus", DType.F32, 4096, 4096, 4096, (COL, COL, COL), "apsp", 1.0, 100.0,
             density=0.01, add_identity=math.inf, description="config 4 at a quarter of the size (12 squarings)"),
    Workload("maxmin_f32_4096", "maximum_minimum", DType.F32, 4096, 4096, 4096, (COL, COL, COL), "uniform", 0.0, 1.0,
             add_identity=-math.inf, alpha=math.inf, beta=math.inf,
             description="config 5: max-min fp32, values uniform [0, 1)"),
    Workload("plustimes_f64_4096", "plus_multiplies", DType.F64, 4096, 4096, 4096, (COL, COL, COL), "uniform", -1.0, 1.0,
             alpha=1.0, beta=1.0, description="config 5: plus-times fp64, values uniform [-1, 1)"),
    Workload("minplus_s32_4096", "minimum_plus", DType.S32, 4096, 4096, 4096, (COL, COL, COL), "ints", 0.0, 1000.0,
             description="min-plus over 32-bit integers (one fused add-min instruction per product), values 0..999"),
    Workload("xorand_u32_4096", "bit_xor_bit_and", DType.U32, 4096, 4096, 4096, (COL, COL, COL), "words",
             alpha=-1, beta=-1, description="config 5: xor-and over uniform 32-bit words"),
]}
