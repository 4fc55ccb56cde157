"""PyTorch value model of NVFP4 quantisation (runs on any device).

Counterpart of the reference project's ``src/nvfp4_decode_kernel/reference.py``
(``round_e2m1`` :8-27, ``nvfp4_round_trip`` :30-46): same names, same results.
It models VALUES, not bytes: an exact E2M1 midpoint goes to the smaller
magnitude here, while the device converters round such ties to even.
"""

from __future__ import annotations

import torch

_E2M1_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_E2M1_STEPS = (0.5, 0.5, 0.5, 0.5, 1.0, 1.0, 2.0)


def round_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 value {0, .5, 1, 1.5, 2, 3, 4, 6}; ties toward zero; non-finite -> 0."""
    magnitude = x.abs()
    rounded = torch.zeros_like(magnitude, dtype=torch.float32)
    for midpoint, step in zip(_E2M1_MIDPOINTS, _E2M1_STEPS):
        rounded = rounded + (magnitude > midpoint).to(torch.float32) * step
    rounded = torch.where(torch.isfinite(magnitude), rounded, torch.zeros_like(rounded))
    return torch.sign(x) * rounded


def nvfp4_round_trip(x: torch.Tensor, group: int = 16) -> torch.Tensor:
    """Quantise to NVFP4 and back along the last axis, one E4M3 scale per ``group``."""
    if group <= 0:
        raise ValueError(f"group must be positive, got {group}")
    if x.shape[-1] % group != 0:
        raise ValueError(
            f"last dimension {x.shape[-1]} must be divisible by group {group}"
        )
    blocks = x.float().unflatten(-1, (-1, group))
    scale = (blocks.abs().amax(dim=-1, keepdim=True) / 6.0).to(torch.float8_e4m3fn).float()
    dead = scale == 0
    divisor = torch.where(dead, torch.ones_like(scale), scale)
    restored = torch.where(dead, blocks, round_e2m1(blocks / divisor) * scale)
    return restored.reshape(x.shape)
