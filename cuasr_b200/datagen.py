"""Seeded synthetic operands for the benchmark and the large parity checks.

Values come from a counter-based generator (splitmix64 of seed and element index), so an operand can be made
on the device at full size and any sub-block of it re-made on the host, bit for bit, without storing it.
Everything is written with 64-bit integer tensor operations that behave identically on CPU and CUDA.
"""
from __future__ import annotations

import torch

_MASK = {s: (1 << (64 - s)) - 1 for s in (11, 27, 30, 31, 40)}


def _c(v: int) -> int:
    """A 64-bit constant as the signed integer with the same bits."""
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical shift right of int64 tensors (torch's >> is arithmetic)."""
    return (x >> s) & _MASK[s]


def splitmix64(seed: int, index: torch.Tensor) -> torch.Tensor:
    """splitmix64 output for state = seed + (index + 1) * golden-gamma; int64 tensor holding the 64 bits."""
    z = index * _c(0x9E3779B97F4A7C15) + _c((seed * 0x9E3779B97F4A7C15 + 0x9E3779B97F4A7C15) & ((1 << 64) - 1))
    z = (z ^ _lsr(z, 30)) * _c(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _c(0x94D049BB133111EB)
    return z ^ _lsr(z, 31)


def _indices(start: int, count: int, device) -> torch.Tensor:
    return torch.arange(start, start + count, dtype=torch.int64, device=device)


def uniform_f32(seed: int, count: int, lo: float, hi: float, device="cpu", start: int = 0) -> torch.Tensor:
    """`count` floats uniform in [lo, hi): lo + (hi - lo) * u / 2^24 with u the top 24 bits of the hash."""
    u = _lsr(splitmix64(seed, _indices(start, count, device)), 40).to(torch.float32)
    return (u * ((hi - lo) / 16777216.0) + lo).to(torch.float32)


def uniform_f64(seed: int, count: int, lo: float, hi: float, device="cpu", start: int = 0) -> torch.Tensor:
    u = _lsr(splitmix64(seed, _indices(start, count, device)), 11).to(torch.float64)
    return u * ((hi - lo) / 9007199254740992.0) + lo


def words_u32(seed: int, count: int, device="cpu", start: int = 0) -> torch.Tensor:
    """Uniform 32-bit words, returned as int32 bit patterns."""
    w = splitmix64(seed, _indices(start, count, device)) & 0xFFFFFFFF
    return torch.where(w >= (1 << 31), w - (1 << 32), w).to(torch.int32)


def sparse_graph(seed: int, n: int, p: float, absent: float, dtype=torch.float32, device="cpu",
                 weight_lo: int = 1, weight_hi: int = 100, integer_weights: bool = True,
                 row_start: int = 0, rows: int | None = None) -> torch.Tensor:
    """Rows [row_start, row_start + rows) of the n x n weighted adjacency matrix of a random directed graph:
    each edge present with probability p (decided by one hash), weight uniform in [weight_lo, weight_hi]
    (integers) or [weight_lo, weight_hi) (reals) from a second hash, absent edges = `absent`, diagonal 0.
    Returned flat, row-major over the selected rows."""
    rows = n if rows is None else rows
    idx = _indices(row_start * n, rows * n, device)
    present = _lsr(splitmix64(seed ^ 0x5DEECE66D, idx), 11).to(torch.float64) < p * 9007199254740992.0
    h = _lsr(splitmix64(seed, idx), 11)
    if integer_weights:
        w = (h % (weight_hi - weight_lo + 1) + weight_lo).to(dtype)
    else:
        w = (h.to(torch.float64) * ((weight_hi - weight_lo) / 9007199254740992.0) + weight_lo).to(dtype)
    out = torch.where(present, w, torch.full_like(w, absent))
    r = idx // n
    c = idx - r * n
    return torch.where(r == c, torch.zeros_like(out), out)
