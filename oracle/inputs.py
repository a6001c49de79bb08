"""Seeded synthetic tensors of the benchmark configurations.

They stand in for the checkpoints and serving traffic the reference measures on
(none are available offline): weights ~N(0, 0.02) quantised by the oracle's own
rules, activations bf16 ~N(0, 1), norm weights 1 + 0.1 N(0, 1), router bias
N(0, 0.02), as the reference's kernel checks draw them
(test/kernels/glm53/check_layer.py:154; test/kernels/deepseek_v41/check_ffn.py:127-160).
"""

from __future__ import annotations

import torch

from . import quant as Q

C1 = dict(name="c1_moe_ffn", rows=4, hidden=2048, experts=64, topk=6, inter=768, has_shared=True,
          score_fn=0, route_scale=1.0, eps=1e-6, swiglu_limit=0.0)
# per-rank slice of the sparse-MLA MoE layer's FFN at tensor-parallel size tp
def c2_ffn(tp: int, rows: int):
    return dict(name=f"c2_moe_ffn_tp{tp}", rows=rows, hidden=7168, experts=256, topk=8, inter=2048 // tp,
                has_shared=True, score_fn=1, route_scale=2.5, eps=1e-6, swiglu_limit=0.0)


def moe_weights(cfg, seed: int = 0, experts_chunk: int = 16, device="cpu"):
    """Weights of one MoE block.  On a CUDA device the same rules run there (the stream of
    random numbers differs from the CPU generator's; a test uses one device throughout)."""
    g = torch.Generator(device=device).manual_seed(1000 * seed + 7)
    _randn = torch.randn

    def randn(*shape, generator):
        return _randn(*shape, generator=generator, device=device)

    H, E, I = cfg["hidden"], cfg["experts"], cfg["inter"]
    n = E + (1 if cfg["has_shared"] else 0)
    w = dict(
        norm=(1 + 0.1 * randn(H, generator=g)).to(torch.bfloat16),
        gate_w=(0.02 * randn(E, H, generator=g)).to(torch.bfloat16),
        bias=(0.02 * randn(E, generator=g)).float() if cfg["score_fn"] == 1 else None,
    )
    w13 = torch.empty(n, 2 * I, H, dtype=torch.float8_e4m3fn, device=device)
    w13_s = torch.empty(n, -(-2 * I // 128), H // 128, device=device)
    w2 = torch.empty(n, H, I, dtype=torch.float8_e4m3fn, device=device)
    w2_s = torch.empty(n, H // 128, I // 128, device=device)
    for e0 in range(0, n, experts_chunk):
        e1 = min(n, e0 + experts_chunk)
        q, s = Q.quant_weight_block128(0.02 * randn(e1 - e0, 2 * I, H, generator=g))
        w13[e0:e1], w13_s[e0:e1] = q, s
        q, s = Q.quant_weight_block128(0.02 * randn(e1 - e0, H, I, generator=g))
        w2[e0:e1], w2_s[e0:e1] = q, s
    w.update(w13=w13, w13_s=w13_s, w2=w2, w2_s=w2_s)
    return w


def rows_bf16(rows: int, hidden: int, seed: int = 0, scale: float = 1.0):
    g = torch.Generator().manual_seed(77 + seed)
    return (scale * torch.randn(rows, hidden, generator=g)).to(torch.bfloat16)
