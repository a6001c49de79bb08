"""MXFP4 expert weights: the tile packing the kernels read (made once at load time, the counterpart of the
reference's shuffle_weight / e8m0_shuffle calls, sgl_amd_mono/muse_spark/weights.py and
test/kernels/deepseek_v41/check_ffn.py:169-172) and its inverse.

Checkpoint form: codes u8 [N, K/2] (byte b of a row = dims 2b in the low nibble, 2b+1 in the high nibble), scales
u8 [N, K/32] (E8M0).  Packed form: codes u8 [N/16, K/64, 32, 16]: lane (g, c) of a warp holds, for the two 32-wide
scale groups G of a 64-wide k unit, the four code bytes (dims 8c..8c+7 of the group) of row g and of row g+8, in the
order (G0, g), (G0, g+8), (G1, g), (G1, g+8); scales u8 [N/16, K/64, 8, 4] in the same (G, half) order.
N is whatever the caller stacks (all experts' rows); N % 16 == 0 and K % 64 == 0.
"""

from __future__ import annotations

import torch


def pack_mxfp4(codes: torch.Tensor, scales: torch.Tensor):
    n, kb = codes.shape[-2], codes.shape[-1]
    k = kb * 2
    if n % 16 or k % 64 or scales.shape[-2:] != (n, k // 32):
        raise ValueError(f"pack_mxfp4: codes {tuple(codes.shape)} scales {tuple(scales.shape)}: rows must be a multiple of 16, "
                         "k a multiple of 64, one scale per 32")
    lead = codes.shape[:-2]
    c = codes.reshape(*lead, n // 16, 2, 8, k // 64, 2, 4, 4)         # tile, half, g, unit, G, c, byte
    c = c.permute(*range(len(lead)), -7, -4, -5, -2, -3, -6, -1)      # tile, unit, g, c, G, half, byte
    s = scales.reshape(*lead, n // 16, 2, 8, k // 64, 2)              # tile, half, g, unit, G
    s = s.permute(*range(len(lead)), -5, -2, -3, -1, -4)              # tile, unit, g, G, half
    return (c.reshape(*lead, n // 16, k // 64, 32, 16).contiguous(), s.reshape(*lead, n // 16, k // 64, 8, 4).contiguous())


def unpack_mxfp4(packed: torch.Tensor, pscales: torch.Tensor):
    lead = packed.shape[:-4]
    t, u = packed.shape[-4], packed.shape[-3]
    c = packed.reshape(*lead, t, u, 8, 4, 2, 2, 4)                    # tile, unit, g, c, G, half, byte
    c = c.permute(*range(len(lead)), -7, -2, -5, -6, -3, -4, -1)      # tile, half, g, unit, G, c, byte
    s = pscales.reshape(*lead, t, u, 8, 2, 2)                         # tile, unit, g, G, half
    s = s.permute(*range(len(lead)), -5, -1, -3, -4, -2)              # tile, half, g, unit, G
    return c.reshape(*lead, t * 16, u * 32).contiguous(), s.reshape(*lead, t * 16, u * 2).contiguous()
