"""Seeded synthetic inputs and rotary tables for the fused attention path.

The generator is structured like the reference's ``make_inputs``
(src/e1_rope_publication_v1.py:172-183: draw q, k, v, gamma_q, gamma_k in that
order from one seeded generator; ``angle = pos * theta^(-2i/D)`` in fp32;
cos/sin tables cast to the activation dtype with the half-width table
duplicated into both halves), with the value distributions of the benchmark
configurations (q, k, v ~ N(0,1); gammas ~ 1 + 0.1 N(0,1)).  Everything is
generated on the CPU so that every rank count sees identical data.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    S: int
    Hq: int
    Hkv: int
    D: int
    dtype: torch.dtype
    theta: float
    causal: bool = True
    eps: float = 1e-6


# The five named configurations (C1 is the CPU known-answer case).
WORKLOADS = {
    "C1": Workload("C1", 1, 128, 32, 8, 128, torch.float32, 1e6),
    "C2": Workload("C2", 1, 2048, 32, 8, 128, torch.bfloat16, 1e6),
    "C3": Workload("C3", 4, 1000, 32, 8, 128, torch.float16, 1e6),
    "C4": Workload("C4", 16, 4096, 32, 8, 128, torch.bfloat16, 1e6),
    "C5": Workload("C5", 8, 8192, 16, 8, 256, torch.bfloat16, 1e4),
}


def rope_tables(positions: torch.Tensor, d: int, theta: float, dtype: torch.dtype):
    """cos/sin tables [len(positions), D]: the half-width table duplicated in
    the split-half layout, computed in fp32 and cast to ``dtype``
    (src/e1_rope_publication_v1.py:180-183)."""
    pos = positions.to(torch.float32)
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=pos.device) / d))
    ang = pos[:, None] * inv[None, :]
    cos = torch.cat([torch.cos(ang), torch.cos(ang)], dim=1).to(dtype)
    sin = torch.cat([torch.sin(ang), torch.sin(ang)], dim=1).to(dtype)
    return cos.contiguous(), sin.contiguous()


def make_inputs(b, s, hq, hkv, d, *, dtype=torch.bfloat16, theta=1e6, seed=0,
                sigma=1.0, gamma_sigma=0.1, rope=True):
    """Returns (q, k, v, gq, gk, cos, sin) on the CPU; cos/sin are None when
    ``rope`` is False.  Values are drawn in fp32 and cast to ``dtype``."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    rn = lambda *shape: torch.randn(*shape, generator=gen, dtype=torch.float32)
    q = (rn(b, hq, s, d) * sigma).to(dtype)
    k = (rn(b, hkv, s, d) * sigma).to(dtype)
    v = (rn(b, hkv, s, d) * sigma).to(dtype)
    gq = (1 + rn(d) * gamma_sigma).to(dtype)
    gk = (1 + rn(d) * gamma_sigma).to(dtype)
    if rope:
        cos, sin = rope_tables(torch.arange(s), d, theta, dtype)
    else:
        cos = sin = None
    return q, k, v, gq, gk, cos, sin


def make_workload_inputs(w: Workload, seed=0, B=None, dtype=None):
    """Inputs of a named workload; ``B`` overrides the batch (bounded CPU
    samples) and ``dtype`` the activation dtype."""
    return make_inputs(w.B if B is None else B, w.S, w.Hq, w.Hkv, w.D,
                       dtype=w.dtype if dtype is None else dtype, theta=w.theta, seed=seed)
