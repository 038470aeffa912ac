"""Seeded synthetic workloads for the PAM hot path.

Every tensor is drawn on the CPU in float32 from ``torch.Generator().manual_seed(seed)``
in a fixed order and only then cast / copied, so the CPU oracle, the reference and the
CUDA kernels all see identical values (CUDA and CPU RNG streams differ, so nothing is
drawn on the device).  Shapes and distributions follow the five benchmark configurations
of this project: complex-normal Q/K/V with per-component std 1/sqrt(2d), decay
gamma = sigmoid(N(3,1)), unit-variance complex upstream gradient.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


@dataclass
class ScanInputs:
    q: torch.Tensor       # [B,H,T,d,2]
    k: torch.Tensor
    v: torch.Tensor
    g: torch.Tensor       # [B,H,T] pre-sigmoid decay logits, gamma = sigmoid(g)
    dy: torch.Tensor      # [B,H,T,d,2]

    @property
    def gamma(self) -> torch.Tensor:
        return torch.sigmoid(self.g)


def scan_inputs(B: int, H: int, T: int, d: int, seed: int = 0, dtype=torch.float32) -> ScanInputs:
    """Config-1 style inputs: draw order q, k, v, g, dy."""
    gen = _gen(seed)
    std = 1.0 / math.sqrt(2.0 * d)
    q = torch.randn(B, H, T, d, 2, generator=gen) * std
    k = torch.randn(B, H, T, d, 2, generator=gen) * std
    v = torch.randn(B, H, T, d, 2, generator=gen) * std
    g = torch.randn(B, H, T, generator=gen) + 3.0
    dy = torch.randn(B, H, T, d, 2, generator=gen) / math.sqrt(2.0)
    return ScanInputs(q.to(dtype), k.to(dtype), v.to(dtype), g, dy.to(dtype))


def config1() -> ScanInputs:
    """B=2, H=4, d=32, T=512 (chunk 64), complex64, seed 0."""
    return scan_inputs(2, 4, 512, 32, seed=0)


@dataclass
class CEInputs:
    h: torch.Tensor        # [N, 2D]  = [h_r | h_i]
    w: torch.Tensor        # [V, 2D]  = [E_r | E_i]
    targets: torch.Tensor  # [N] int64


def ce_inputs(N: int, D: int, V: int, seed: int = 0, dtype=torch.bfloat16) -> CEInputs:
    """Config-2 style inputs: hidden ~ N(0,1), tied embedding ~ N(0,0.02), uniform targets."""
    gen = _gen(seed)
    h = torch.randn(N, D, 2, generator=gen).to(dtype)
    e = (torch.randn(V, D, 2, generator=gen) * 0.02).to(dtype)
    targets = torch.randint(0, V, (N,), generator=gen, dtype=torch.int64)
    hcat = torch.cat([h[..., 0], h[..., 1]], dim=-1).contiguous()
    wcat = torch.cat([e[..., 0], e[..., 1]], dim=-1).contiguous()
    return CEInputs(hcat, wcat, targets)


def config2() -> CEInputs:
    """N=8192 rows, complex dim 384, vocab 50261, bf16, seed 0."""
    return ce_inputs(8192, 384, 50261, seed=0)


@dataclass
class PackedInputs:
    q: torch.Tensor            # [H, Ttot, d, 2]
    k: torch.Tensor
    v: torch.Tensor
    gamma: torch.Tensor        # [H, Ttot] fp32
    cu_seqlens: torch.Tensor   # [S+1] int32
    lengths: torch.Tensor


def packed_inputs(n_seq: int, lo: int, hi: int, H: int, d: int, seed: int = 0,
                  dtype=torch.bfloat16) -> PackedInputs:
    """Config-4 style packed ragged batch: lengths uniform in [lo, hi]."""
    gen = _gen(seed)
    lengths = torch.randint(lo, hi + 1, (n_seq,), generator=gen, dtype=torch.int64)
    total = int(lengths.sum())
    std = 1.0 / math.sqrt(2.0 * d)
    q = (torch.randn(H, total, d, 2, generator=gen) * std).to(dtype)
    k = (torch.randn(H, total, d, 2, generator=gen) * std).to(dtype)
    v = (torch.randn(H, total, d, 2, generator=gen) * std).to(dtype)
    gamma = torch.sigmoid(torch.randn(H, total, generator=gen) + 3.0)
    cu = torch.zeros(n_seq + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lengths, 0).to(torch.int32)
    return PackedInputs(q, k, v, gamma, cu, lengths)


def config4() -> PackedInputs:
    """32 sequences, lengths uniform in [512,16384], H=16, d=64, bf16, seed 0."""
    return packed_inputs(32, 512, 16384, 16, 64, seed=0)


def decode_prompts(n_seq: int, lo: int, hi: int, vocab: int, seed: int = 0):
    """Config-5 style prompts: lengths uniform in [lo,hi], ids uniform over the vocab."""
    gen = _gen(seed)
    lengths = torch.randint(lo, hi + 1, (n_seq,), generator=gen, dtype=torch.int64)
    return [torch.randint(0, vocab, (int(n),), generator=gen, dtype=torch.int64) for n in lengths]
