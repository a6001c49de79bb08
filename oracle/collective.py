"""All-reduce rule: f32 sum of the bf16 partials in rank order, then the residual, one bf16 rounding
(test/kernels/deepseek_v41/check_ffn.py:251-258 `reduced`; sgl_amd_mono/common/ops.py:377-385)."""

from __future__ import annotations

import numpy as np
import torch


def allreduce(partials, residual=None) -> torch.Tensor:
    acc = np.zeros(partials[0].shape, np.float32)
    for p in partials:
        acc = (acc + p.detach().cpu().float().numpy()).astype(np.float32)
    if residual is not None:
        acc = (acc + residual.detach().cpu().float().numpy()).astype(np.float32)
    return torch.from_numpy(acc).to(torch.bfloat16)


def slot_sum(contrib) -> torch.Tensor:
    """[slots, rows, hidden] bf16 -> bf16 sum in slot order with a bf16 rounding at every add
    (sgl_amd_mono/deepseek_v41/gfx950/stages/moe.py:1166-1173)."""
    acc = torch.zeros(contrib.shape[1:], dtype=torch.float32)
    for s in range(contrib.shape[0]):
        acc = (acc + contrib[s].detach().cpu().float()).to(torch.bfloat16).float()
    return acc.to(torch.bfloat16)
