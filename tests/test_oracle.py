"""The oracle against the reference's own helpers (golden vectors made by
tests/golden/make_golden.py) and against the known-answer values in the reference's
unit tests."""

import os

import numpy as np
import torch

from oracle import detmath as dm
from oracle import moe as M
from oracle import quant as Q

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_helpers.npz"))


def t(name):
    return torch.from_numpy(G[name])


def test_quant128_matches_reference_helpers():
    x = t("q128_x").bfloat16()
    q, s = Q.quant128(x, zero_rule=True)
    assert torch.equal(Q.dequant128(q, s), t("q128_glm"))
    assert torch.equal(Q.dequant128(q, s), t("q128_rows"))
    # the floor rule differs from the zero rule only on all-zero groups
    q2, s2 = Q.quant128(x, zero_rule=False)
    nz = (x.float().reshape(6, 4, 128).abs().amax(-1) > 0)
    assert torch.equal(s[nz], s2[nz]) and torch.equal(q.view(torch.uint8), q2.view(torch.uint8))


def test_block_fp8_gemv_matches_reference():
    x = t("q128_x").bfloat16()
    wq = t("gemv_w_bytes").view(torch.float8_e4m3fn)
    ws = t("gemv_ws")
    assert torch.equal(Q.deq_weight_block128(wq, ws), t("slices_f32"))
    q, s = Q.quant128(x, zero_rule=True)
    y = Q.gemv_fp8(q, s, wq, ws).bfloat16().float()
    ref = t("gemv_y")
    assert ((y - ref).norm() / ref.norm()).item() < 2e-3  # f64 vs f32 accumulation, then bf16
    # weight quantiser is the inverse of the reference's dequantiser
    w = Q.deq_weight_block128(wq, ws)
    q2, s2 = Q.quant_weight_block128(w)
    assert torch.equal(Q.deq_weight_block128(q2, s2), w)


def test_rmsnorm_matches_reference_value():
    x = t("q128_x").bfloat16()
    w = t("rms_w").bfloat16()
    _, y, _, _ = M.rmsnorm_quant(x, w, 1e-5)
    ref = t("rms_y")
    # same formula, different (but defined) order of the sum of squares: within 1 bf16 ulp
    assert torch.allclose(y.float(), ref, rtol=2**-7, atol=1e-30)
    assert (y.float() == ref.bfloat16().float()).float().mean() > 0.98


def test_radix_key_matches_reference():
    assert np.array_equal(dm.radix_key(G["radix_in"]).astype(np.int64), G["radix_keys"])


def test_mxfp4_matches_reference_and_kat():
    p, s = Q.quantize_mxfp4(t("mx4_in"))
    assert torch.equal(p, t("mx4_packed")) and torch.equal(s, t("mx4_scales"))
    assert torch.equal(Q.dequantize_mxfp4(p, s), t("mx4_deq"))
    assert torch.equal(Q.dequantize_mxfp4(p, s), t("mx4_deq_glm"))
    # test/unit/test_muse_spark_mxfp4_quant.py:68-76: (1.0, -0.5) -> scale code 125, byte 0xC6
    p, s = Q.quantize_mxfp4(torch.tensor([[1.0, -0.5] + [0.0] * 30]))
    assert int(s[0, 0]) == 125 and int(p[0, 0]) == 0xC6


def test_mxfp8_scale_rules():
    # test/kernels/deepseek_v41/check_ffn.py:92-104: power-of-two scale >= amax/448
    x = torch.tensor([[448.0] + [0.0] * 31, [449.0] + [0.0] * 31, [0.0] * 32])
    _, c = Q.mxfp8_quant(x, "aiter")
    assert c[:, 0].tolist() == [127, 128, 85]  # 1e-10/448 = 2.23e-13 -> 2^-42 -> code 85
    _, c = Q.mxfp8_quant(x, "vllm")
    assert c[:2, 0].tolist() == [127, 128] and int(c[2, 0]) == 1  # FLT_MIN/448 is subnormal: exponent field 0, +1
    q, c = Q.mxfp8_quant(torch.randn(4, 64), "aiter")
    assert (Q.mxfp8_dequant(q, c) - torch.randn(4, 64)).isfinite().all()


def test_det_math_accuracy_and_bits():
    x = np.linspace(-30, 30, 200001).astype(np.float32)
    e = dm.det_exp(x).astype(np.float64)
    ref = np.exp(x.astype(np.float64))
    assert (np.abs(e - ref) / ref).max() < 6e-7
    assert dm.det_exp(np.float32(0.0)) == np.float32(1.0)
    s = dm.det_sigmoid(x)
    assert s.dtype == np.float32 and np.all(np.diff(s) >= 0) and s[0] < 1e-12 and s[-1] == 1.0
    v = np.arange(32, dtype=np.float32)[None]
    assert dm.warp_sum_tree(v)[0] == 496.0


def test_route_ties_go_to_the_smaller_id():
    logits = np.zeros((2, 16), np.float32)
    logits[1, [3, 9]] = 1.0
    ids, w = M.route(logits, None, 4, M.SCORE_SOFTMAX, 1.0)
    assert ids[0].tolist() == [0, 1, 2, 3] and ids[1].tolist() == [3, 9, 0, 1]
    assert np.allclose(w.sum(1), 1.0, atol=1e-6)
    ids, w = M.route(logits, np.linspace(0, -0.1, 16).astype(np.float32), 4, M.SCORE_SIGMOID_BIAS, 2.5)
    assert ids[1].tolist() == [3, 9, 0, 1] and np.allclose(w.sum(1), 2.5, atol=1e-5)
    # selection uses sigmoid + bias, weights the unbiased sigmoid (sgl_amd_mono/glm53/check.py:184-195)
    bias = np.zeros(16, np.float32)
    bias[15] = 10.0
    ids, w = M.route(logits, bias, 2, M.SCORE_SIGMOID_BIAS, 1.0)
    assert ids[1].tolist() == [15, 3] and w[1, 0] < w[1, 1]


def test_router_logits_order_is_close_to_plain_matmul():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(3, 2048, generator=g).bfloat16()
    w = (0.02 * torch.randn(64, 2048, generator=g)).bfloat16()
    l = M.router_logits(x, w)
    ref = (x.double() @ w.double().T).numpy()
    assert np.abs(l - ref).max() < 2e-5


def test_moe_ffn_small_block_properties():
    from oracle import inputs

    cfg = dict(inputs.C1, hidden=256, inter=128, experts=8, topk=2, rows=3)
    w = inputs.moe_weights(cfg, seed=3)
    x = inputs.rows_bf16(3, 256, seed=3)
    r = M.moe_ffn(x, w, cfg)
    assert r["ids"].shape == (3, 2) and r["union"][-1] == 8
    assert sorted(set(r["ids"].reshape(-1).tolist())) == r["union"][:-1].tolist()
    for tt in range(3):
        for sl in range(2):
            u = r["union"].tolist().index(int(r["ids"][tt, sl]))
            assert r["pick"][u, tt] == sl + 1
    # a row's output does not depend on the other rows of the step
    r1 = M.moe_ffn(x[1:2], w, cfg)
    assert torch.equal(r1["out"][0], r["out"][1])
    # residual: out = bf16(moe + s)
    res = inputs.rows_bf16(3, 256, seed=9)
    rr = M.moe_ffn(x, w, cfg, residual=res, add_residual=True)
    assert torch.equal(rr["s"], (x.float() + res.float()).bfloat16())


def test_mxfp4_tile_packing_round_trip_and_positions():
    import sgl_amd_mono_b200  # noqa: F401
    from sgl_amd_mono_b200 import mx4
    g = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 256, (3, 32, 64), generator=g, dtype=torch.uint8)
    sc = torch.randint(100, 140, (3, 32, 4), generator=g, dtype=torch.uint8)
    p, ps = mx4.pack_mxfp4(codes, sc)
    assert p.shape == (3, 2, 2, 32, 16) and ps.shape == (3, 2, 2, 8, 4)
    c2, s2 = mx4.unpack_mxfp4(p, ps)
    assert torch.equal(c2, codes) and torch.equal(s2, sc)
    # lane (g, c) of tile t, k unit u: group G, row g + 8 * half -> bytes [(2G + half) * 4, +4) = dims 8c .. 8c+7 of the group
    for t, u, gg, cc, G, half in [(0, 0, 0, 0, 0, 0), (1, 1, 3, 2, 1, 1), (1, 0, 7, 3, 0, 1)]:
        row, b0 = t * 16 + half * 8 + gg, (64 * u + 32 * G + 8 * cc) // 2
        assert torch.equal(p[0, t, u, gg * 4 + cc, (2 * G + half) * 4:(2 * G + half) * 4 + 4], codes[0, row, b0:b0 + 4])
        assert int(ps[0, t, u, gg, 2 * G + half]) == int(sc[0, row, 2 * u + G])
    import pytest
    with pytest.raises(ValueError):
        mx4.pack_mxfp4(codes[:, :24], sc[:, :24])
