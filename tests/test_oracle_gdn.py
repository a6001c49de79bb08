"""The GDN oracle against outputs of the reference's own Triton kernels (run on f32 tensors under the Triton
interpreter by tests/golden/make_golden_gdn.py), and its bf16 rules against hand-checked cases."""

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

from oracle import gdn as O  # noqa: E402

GOLD = np.load(os.path.join(ROOT, "tests", "golden", "gdn_reference.npz"))
CASE = dict(seed=11, requests=3, tokens=4, hk=1, hv=2, k_in=256, dead=(1,), no_snapshot=(2,))
DECODE = dict(seed=12, requests=3, tokens=1, hk=1, hv=2, k_in=256, dead=(0,))
SCALE, EPS = 128 ** -0.5, 1e-6


def trunc_bf16(x):
    """f32 -> bf16 by truncation: the Triton interpreter's cast (compiled Triton rounds to nearest even)."""
    return (x.contiguous().view(torch.int32) & -65536).view(torch.float32)


def close(a, b, tol):
    a, b = torch.as_tensor(a).double(), torch.as_tensor(b).double()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item() < tol


def test_case_constants_match_the_generator():
    import make_golden_gdn as M
    assert M.CASE == CASE and M.DECODE == DECODE and M.SCALE == SCALE and M.EPS == EPS


def test_verify_chain_matches_reference_kernels():
    qkvz, hidden, w, st, step = O.make_case(act=torch.float32, **CASE)
    ssm0 = st["ssm_state"].clone()
    r = O.gdn_core(qkvz, hidden, w, st, step, CASE["tokens"], CASE["hk"], CASE["hv"], SCALE, EPS, verify=True, act=torch.float32,
                   bf=trunc_bf16)
    # conv: same operation order, elementwise -> exact except exp's last ulp
    assert np.allclose(r["mixed"].numpy(), GOLD["v_mixed"], rtol=0, atol=2e-6)
    assert np.array_equal(st["conv_state"].numpy(), GOLD["v_conv_state"])
    assert np.array_equal(st["inter_conv"].numpy(), GOLD["v_inter_conv"])
    assert close(r["out"], GOLD["v_out"], 2e-5)
    assert close(r["out_scale"], GOLD["v_scale"], 2e-5)
    assert close(r["out_q"], GOLD["v_out_q"], 2e-5)
    assert close(st["inter_ssm"][..., ::8, ::8], GOLD["v_inter_ssm_sub"], 2e-6)
    assert np.allclose(st["inter_ssm"].double().sum((-1, -2)).numpy(), GOLD["v_inter_ssm_sum"], rtol=1e-5, atol=1e-4)
    assert torch.equal(st["ssm_state"], ssm0)  # verify never writes the committed state
    dead = slice(4, 8)  # request 1
    assert not r["out"][dead].any() and not GOLD["v_out"][dead].any()
    assert not st["inter_ssm"][int(step["inter_slot"][1])].any()  # dead request: no snapshot either
    assert int(step["inter_slot"][2]) == -1


def test_decode_matches_reference_kernel():
    qkvz, hidden, w, st, step = O.make_case(act=torch.float32, **DECODE)
    r = O.gdn_core(qkvz, hidden, w, st, step, 1, DECODE["hk"], DECODE["hv"], SCALE, EPS, verify=False, act=torch.float32,
                   bf=trunc_bf16)
    assert close(r["out"], GOLD["d_out"], 2e-5)
    assert close(r["out_scale"], GOLD["d_scale"], 2e-5)
    assert close(st["ssm_state"][..., ::8, ::8], GOLD["d_state_sub"], 2e-6)
    assert np.allclose(st["ssm_state"].double().sum((-1, -2)).numpy(), GOLD["d_state_sum"], rtol=1e-5, atol=1e-4)


def test_bf16_tap_rounding_and_window_shift():
    # one channel, taps chosen so that the bf16 rounding of a product is visible
    w = torch.tensor([[1.0, 1.0, 1.0, 1.0078125]]).bfloat16()  # 1 + 2^-7 is a bf16 value
    state = torch.tensor([[[0.0], [0.0], [0.0]]]).bfloat16()
    x = torch.tensor([[1.0078125], [2.0]]).bfloat16()
    inter = torch.zeros(1, 2, 3, 1, dtype=torch.bfloat16)
    m = O.conv_chain(x, w, None, state, torch.tensor([0]), torch.tensor([0]), inter, 2, 1, verify=True)
    # (1+2^-7)^2 = 1 + 2^-6 + 2^-14 -> bf16 1 + 2^-6; silu
    acc0 = 1.015625
    assert m[0, 0].item() == torch.tensor(acc0 / (1 + np.exp(-acc0))).bfloat16().item()
    assert inter[0, 0, :, 0].tolist() == [0.0, 0.0, 1.0078125] and inter[0, 1, :, 0].tolist() == [0.0, 1.0078125, 2.0]
    assert state[0, :, 0].tolist() == [0.0, 1.0078125, 2.0]
    # decode keeps the product in f32
    state = torch.zeros(1, 3, 1, dtype=torch.bfloat16)
    m2 = O.conv_chain(x[:1], w, None, state, torch.tensor([0]), torch.tensor([-1]), None, 1, 1, verify=False)
    acc = 1.0078125 ** 2
    assert m2[0, 0].item() == torch.tensor(acc / (1 + np.exp(-acc))).bfloat16().item()
