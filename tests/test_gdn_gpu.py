"""GDN core (conv chain + delta chain) on the GPU against the oracle, through the C ABI."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import sgl_amd_mono_b200  # noqa: E402,F401
from oracle import gdn as O  # noqa: E402
from sgl_amd_mono_b200 import cabi  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCALE, EPS = 128 ** -0.5, 1e-6


def stream():
    return torch.cuda.current_stream().cuda_stream


def rel(a, b):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def run(lib, qkvz, hidden, w, st, step, tokens, hk, hv, commit):
    d = lambda t: t.to(DEV)
    rows = qkvz.shape[0]
    conv_dim = (2 * hk + hv) * 128
    g = dict(conv_state=d(st["conv_state"]), ssm_state=d(st["ssm_state"]), inter_conv=d(st["inter_conv"]),
             inter_ssm=d(st["inter_ssm"]),
             mixed=torch.full((rows, conv_dim), float("nan"), dtype=torch.bfloat16, device=DEV),
             out=torch.full((rows, hv * 128), float("nan"), dtype=torch.bfloat16, device=DEV),
             out_q=torch.full((rows, hv * 128), 0x7f, dtype=torch.uint8, device=DEV),
             out_scale=torch.full((rows, hv), float("nan"), device=DEV))
    keep = [d(qkvz), d(hidden), d(w["ba_w"]), d(w["conv_w"]), d(step["slot"]), d(step["inter_slot"]), d(w["a_log"]),
            d(w["dt_bias"]), d(w["norm_w"])]
    lib.call("gdn", cabi.fill("B200GdnArgs", qkvz=keep[0], hidden=keep[1], ba_w=keep[2], conv_w=keep[3],
                              conv_state=g["conv_state"], ssm_state=g["ssm_state"], slot=keep[4], inter_slot=keep[5],
                              inter_conv=g["inter_conv"], inter_ssm=g["inter_ssm"], a_log=keep[6], dt_bias=keep[7],
                              norm_w=keep[8], mixed=g["mixed"], out=g["out"], out_q=g["out_q"], out_scale=g["out_scale"],
                              requests=rows // tokens, tokens=tokens, hk=hk, hv=hv, k_in=hidden.shape[1],
                              qkvz_stride=qkvz.shape[1], commit=commit, scale=SCALE, eps=EPS), stream())
    torch.cuda.synchronize()
    return g


@pytest.mark.parametrize("requests,tokens,hk,hv,k_in,dead,nosnap", [
    (3, 4, 1, 2, 256, (1,), (2,)),
    (8, 4, 16, 32, 2048, (), ()),      # the hybrid layer's verify step: 8 requests x 4 draft tokens
    (2, 3, 2, 8, 1024, (), (0,)),
])
def test_verify_chain_against_oracle(lib, requests, tokens, hk, hv, k_in, dead, nosnap):
    qkvz, hidden, w, st, step = O.make_case(5 + requests, requests, tokens, hk, hv, k_in, dead=dead, no_snapshot=nosnap)
    ref_st = {k: v.clone() for k, v in st.items()}
    ref = O.gdn_core(qkvz, hidden, w, ref_st, step, tokens, hk, hv, SCALE, EPS, verify=True)
    g = run(lib, qkvz, hidden, w, st, step, tokens, hk, hv, commit=0)
    # the convolution is elementwise with a fixed operation order: windows bit-exact, outputs to one bf16 ulp of exp
    assert torch.equal(g["conv_state"].cpu(), ref_st["conv_state"])
    assert torch.equal(g["inter_conv"].cpu(), ref_st["inter_conv"])
    dm = (g["mixed"].cpu().float() - ref["mixed"].float()).abs()
    assert (dm <= ref["mixed"].float().abs() * 2 ** -7 + 1e-30).all()
    assert (dm > 0).float().mean() < 1e-3
    # committed recurrent state untouched; snapshots after every token
    assert torch.equal(g["ssm_state"].cpu(), st["ssm_state"])
    assert rel(g["inter_ssm"], ref_st["inter_ssm"]) < 1e-4          # the reference's own bound for this buffer
    live = [r for r in range(requests) if r not in dead]
    rows_live = torch.tensor([r * tokens + t for r in live for t in range(tokens)])
    assert rel(g["out"][rows_live], ref["out"][rows_live]) < 5e-3
    assert rel(g["out_scale"], ref["out_scale"]) < 5e-3
    deq = g["out_q"].view(torch.float8_e4m3fn).float().view(-1, hv, 128) * g["out_scale"][:, :, None]
    assert rel(deq.view(-1, hv * 128)[rows_live], ref["out"][rows_live].float()) < 4e-2  # e4m3 grid
    for r in dead:
        sl = slice(r * tokens, (r + 1) * tokens)
        assert not g["out"][sl].any() and not g["out_q"][sl].any() and not g["mixed"][sl].any()
    for r in nosnap:
        pass  # inter_slot -1: nothing to check beyond the buffers matching the oracle's above


def test_decode_commits_state(lib):
    requests, hk, hv, k_in = 5, 4, 8, 512
    qkvz, hidden, w, st, step = O.make_case(77, requests, 1, hk, hv, k_in, dead=(3,))
    ref_st = {k: v.clone() for k, v in st.items()}
    ref = O.gdn_core(qkvz, hidden, w, ref_st, step, 1, hk, hv, SCALE, EPS, verify=False)
    g = run(lib, qkvz, hidden, w, st, step, 1, hk, hv, commit=1)
    assert torch.equal(g["conv_state"].cpu(), ref_st["conv_state"])
    assert rel(g["ssm_state"], ref_st["ssm_state"]) < 1e-5
    untouched = [s for s in range(st["ssm_state"].shape[0]) if s not in step["slot"].tolist()]
    assert torch.equal(g["ssm_state"].cpu()[untouched], st["ssm_state"][untouched])
    assert not g["inter_ssm"].any() and not g["inter_conv"].any()   # decode writes no snapshots
    live = torch.tensor([r for r in range(requests) if r != 3])
    assert rel(g["out"][live], ref["out"][live]) < 5e-3
    assert not g["out"][3].any()


def test_chain_equals_single_steps(lib):
    """A 4-token verify chain leaves the same snapshots as four decode steps that commit (up to the decode rules'
    roundings): the size-independent property of the recurrence."""
    requests, tokens, hk, hv, k_in = 2, 4, 2, 4, 256
    qkvz, hidden, w, st, step = O.make_case(9, requests, tokens, hk, hv, k_in)
    g = run(lib, qkvz, hidden, w, {k: v.clone() for k, v in st.items()}, step, tokens, hk, hv, commit=0)
    cur = {k: v.clone() for k, v in st.items()}
    for t in range(tokens):
        rows = torch.tensor([r * tokens + t for r in range(requests)])
        g1 = run(lib, qkvz[rows], hidden[rows], w, cur, step, 1, hk, hv, commit=1)
        cur["ssm_state"], cur["conv_state"] = g1["ssm_state"].cpu(), g1["conv_state"].cpu()
        for r in range(requests):
            snap = g["inter_ssm"][int(step["inter_slot"][r]), t].cpu()
            assert rel(cur["ssm_state"][int(step["slot"][r])], snap) < 2e-2  # beta / tap roundings differ by rule
            assert torch.equal(cur["conv_state"][int(step["slot"][r])], g["inter_conv"][int(step["inter_slot"][r]), t].cpu())


def test_gdn_refuses_chain_commit(lib):
    z = torch.zeros(64, device=DEV)
    a = cabi.fill("B200GdnArgs", qkvz=z, hidden=z, ba_w=z, conv_w=z, conv_state=z, ssm_state=z, slot=z, a_log=z, dt_bias=z,
                  norm_w=z, mixed=z, out=z, out_q=z, out_scale=z, requests=1, tokens=4, hk=1, hv=1, k_in=256,
                  qkvz_stride=512, commit=1, scale=1.0, eps=1e-6)
    with pytest.raises(cabi.B200MonoError, match="decode form"):
        lib.call("gdn", a, stream())
