"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations (there are no
checkpoints or datasets here: every tensor is drawn from a torch CPU generator with a stated seed and draw order)."""
from __future__ import annotations

import numpy as np
import torch


def gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def int4_matrix(rows: int, cols: int, g: torch.Generator, group: int = 128):
    """codes uint8 [rows][cols] uniform in 0..15 (signed value + 8), scales f32 [rows][cols/group] =
    |N(0, 0.02)| / 7 + 1e-4 rounded to bf16 (exactly representable in f16)."""
    codes = torch.randint(0, 16, (rows, cols), generator=g, dtype=torch.uint8).numpy()
    sc = (torch.randn(rows, cols // group, generator=g).abs() * 0.02 / 7 + 1e-4).to(torch.bfloat16).float().numpy()
    return codes, sc


def activations(rows: int, cols: int, g: torch.Generator) -> np.ndarray:
    """f16 [rows][cols], N(0, 1)."""
    return torch.randn(rows, cols, generator=g).to(torch.float16).numpy()
