"""Seeded synthetic inputs for the benchmark configurations.

All tensors are drawn on the CPU from a seeded ``torch.Generator`` and cast to the
working dtype, so the CPU oracle and the GPU kernels see identical bits.  There is no
public dataset behind these workloads: the shapes and value distributions below *are* the
workload definition.

Seeds: partial of rank ``r`` in config ``c`` uses ``1000*c + r``; the outlier mask uses
``1000*c + 500 + r``; the residual ``1000*c + 900``; the RMSNorm weight ``1000*c + 901``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass(frozen=True)
class Config:
    cfg: int
    name: str
    tokens: int
    hidden: int
    quant_type: int
    static_scale: Optional[float] = None
    partial_std_div_sqrt_n: bool = False
    outlier_prob: float = 0.0
    outlier_mult: float = 1.0
    eps: float = 1e-6


CONFIGS = {
    "c1": Config(1, "c1_cpu_gloo_128x4096_dynamic", 128, 4096, 3),
    "c2": Config(2, "c2_decode_8x8192_static0.05", 8, 8192, 4, static_scale=0.05,
                 partial_std_div_sqrt_n=True),
    "c3": Config(3, "c3_mid_1024x8192_dynamic", 1024, 8192, 3),
    "c4": Config(4, "c4_prefill_16384x7168_dynamic_outliers", 16384, 7168, 3,
                 outlier_prob=0.001, outlier_mult=20.0),
    "c5": Config(5, "c5_model_ar_32x8192_dynamic", 32, 8192, 3),
}


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def make_partial(cfg: Config, rank: int, world: int, tokens: Optional[int] = None,
                 dtype=torch.bfloat16) -> torch.Tensor:
    m = cfg.tokens if tokens is None else tokens
    x = torch.randn(m, cfg.hidden, generator=_gen(1000 * cfg.cfg + rank), dtype=torch.float32)
    if cfg.partial_std_div_sqrt_n:
        x = x / math.sqrt(8.0)
    if cfg.outlier_prob > 0:
        mask = torch.rand(m, cfg.hidden, generator=_gen(1000 * cfg.cfg + 500 + rank)) < cfg.outlier_prob
        x = torch.where(mask, x * cfg.outlier_mult, x)
    return x.to(dtype)


def make_residual(cfg: Config, tokens: Optional[int] = None, dtype=torch.bfloat16) -> torch.Tensor:
    m = cfg.tokens if tokens is None else tokens
    return torch.randn(m, cfg.hidden, generator=_gen(1000 * cfg.cfg + 900), dtype=torch.float32).to(dtype)


def make_weight(cfg: Config, dtype=torch.bfloat16) -> torch.Tensor:
    w = 1.0 + 0.1 * torch.randn(cfg.hidden, generator=_gen(1000 * cfg.cfg + 901), dtype=torch.float32)
    return w.to(dtype)


def make_case(cfg: Config, world: int, tokens: Optional[int] = None, dtype=torch.bfloat16):
    parts: List[torch.Tensor] = [make_partial(cfg, r, world, tokens, dtype) for r in range(world)]
    return parts, make_residual(cfg, tokens, dtype), make_weight(cfg, dtype)
