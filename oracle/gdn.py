"""Test oracle (CPU, torch f32) for the gated-delta-network core of the hybrid layers: causal depthwise
convolution over [window(3) | new tokens] + SiLU, the gated delta-rule recurrence with a snapshot of the window and
of the state after every token, the gated RMSNorm of the head outputs and their per-head FP8 quantisation.

This file is test infrastructure: only tests, the smoke check and the benchmark's CPU baseline import it.

Follows sgl_amd_mono/qwen35_a17b/fp8/gfx950/verify.py:56-233 (verify chains) and gdn.py:95-140,225-281 (decode):
  conv:   acc = sum_i tap_i(c_i * w_i) + tap(x * w_3) [+ bias];  y = acc / (1 + exp(-acc)) -> bf16;
          tap() rounds each product to bf16 in verify, keeps f32 in decode;  window <- (c1, c2, x).
  gates:  b, a = bf16(hidden . w_b), bf16(hidden . w_a);  beta = sigmoid(b) (decode: rounded to bf16);
          g = -exp(a_log) * softplus(a + dt_bias) (softplus(x) = x above 20);  decay = exp(g).
  chain:  q <- q / sqrt(sum q^2 + 1e-6) * scale;  k <- k / sqrt(sum k^2 + 1e-6);
          S <- S * decay;  v' = (v - S k) * beta;  S <- S + v' (x) k;  o = S q      (S is [v, k], f32)
  norm:   o <- bf16(o);  y = bf16(o * rsqrt(mean o^2 + eps) * w * z * sigmoid(z));  dead requests give y = 0
  quant:  scale = max(amax|y|, 1e-10) / 448 per head (128 values);  yq = e4m3(clamp(y * (1 / scale), +-448)).
Formats (this library's): conv state bf16 [slots, 3, conv_dim]; recurrent state f32 [slots, HV, D, D] ([v][k]);
snapshots bf16 [islots, T, 3, conv_dim] and f32 [islots, T, HV, D, D]; qkvz columns q (HK*D) | k (HK*D) | v (HV*D) |
z (HV*D).  In verify the committed recurrent state is not written (the engine commits a snapshot after acceptance);
the conv window is advanced in place, as the reference's chain kernel does.
"""

from __future__ import annotations

import torch

D = 128
FP8_MAX = 448.0


def _bf(x):
    return x.bfloat16().float()


def conv_chain(qkvz, conv_w, conv_bias, conv_state, slot, inter_slot, inter_conv, tokens, conv_dim, verify,
               act=torch.bfloat16):
    """Returns mixed `act` [rows, conv_dim]; updates conv_state and inter_conv in place.  `act` is the activation
    dtype (bf16 in the product; f32 only to compare with the reference kernels run on f32 tensors)."""
    rows = qkvz.shape[0]
    R = rows // tokens
    w = conv_w.float()
    mixed = torch.zeros(rows, conv_dim, dtype=act)
    tap = (lambda v: v.to(act).float()) if verify else (lambda v: v)
    for r in range(R):
        s = int(slot[r])
        if s < 0:
            continue
        c = [conv_state[s, i].float() for i in range(3)]
        for t in range(tokens):
            x = qkvz[r * tokens + t, :conv_dim].float()
            acc = tap(c[0] * w[:, 0]) + tap(c[1] * w[:, 1])
            acc = acc + tap(c[2] * w[:, 2]) + tap(x * w[:, 3])
            if conv_bias is not None:
                acc = acc + conv_bias.float()
            mixed[r * tokens + t] = (acc / (1.0 + torch.exp(-acc))).to(act)
            c = [c[1], c[2], x]
            if inter_conv is not None and int(inter_slot[r]) >= 0:
                for i in range(3):
                    inter_conv[int(inter_slot[r]), t, i] = c[i].to(act)
        for i in range(3):
            conv_state[s, i] = c[i].to(act)
    return mixed


def delta_chain(mixed, qkvz, hidden, ba_w, ssm_state, slot, inter_slot, inter_ssm, a_log, dt_bias, norm_w, tokens, hk, hv,
                scale, eps, verify, act=torch.bfloat16, bf=_bf):
    """Returns (out bf16 [rows, hv*D], out_q e4m3 [rows, hv*D], out_scale f32 [rows, hv]); updates inter_ssm (verify)
    or ssm_state (decode) in place.  `bf` is the f32 -> bf16 -> f32 rounding of the gate scalars (round to nearest
    even; the pin against the reference kernels passes truncation, which is what the Triton interpreter's cast does)."""
    rows = mixed.shape[0]
    R = rows // tokens
    q8 = torch.float8_e4m3fn if act == torch.bfloat16 else torch.float32
    out = torch.zeros(rows, hv * D, dtype=act)
    out_q = torch.zeros(rows, hv * D, dtype=q8)
    out_s = torch.full((rows, hv), 1e-10) * (1.0 / FP8_MAX)
    ba = hidden.float() @ ba_w.float().T  # [rows, 2 hv]
    b, a = bf(ba[:, :hv]), bf(ba[:, hv:])
    nw = norm_w.float()
    for r in range(R):
        s = int(slot[r])
        if s < 0:
            continue
        S = ssm_state[s].float().clone()  # [hv, v, k]
        for t in range(tokens):
            row = r * tokens + t
            q = mixed[row, : hk * D].float().view(hk, D)
            k = mixed[row, hk * D : 2 * hk * D].float().view(hk, D)
            v = mixed[row, 2 * hk * D :].float().view(hv, D)
            z = qkvz[row, 2 * hk * D + hv * D : 2 * hk * D + 2 * hv * D].float().view(hv, D)
            q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * scale
            k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            q = q.repeat_interleave(hv // hk, 0)
            k = k.repeat_interleave(hv // hk, 0)
            x = a[row] + dt_bias.float()
            softplus = torch.where(x <= 20.0, torch.log1p(torch.exp(torch.clamp(x, max=20.0))), x)
            g = -torch.exp(a_log.float()) * softplus
            beta = torch.sigmoid(b[row])
            if not verify:
                beta = bf(beta)
            S = S * torch.exp(g)[:, None, None]
            vn = (v - torch.einsum("hvk,hk->hv", S, k)) * beta[:, None]
            S = S + vn[:, :, None] * k[:, None, :]
            o = torch.einsum("hvk,hk->hv", S, q).to(act).float()
            if verify and inter_ssm is not None and int(inter_slot[r]) >= 0:
                inter_ssm[int(inter_slot[r]), t] = S
            rstd = torch.rsqrt((o * o).sum(-1, keepdim=True) / D + eps)
            y = (o * rstd * nw[None, :] * (z * torch.sigmoid(z))).to(act)
            out[row] = y.view(-1)
            yf = y.float()
            sc = torch.clamp(yf.abs().amax(-1), min=1e-10) * (1.0 / FP8_MAX)
            out_s[row] = sc
            out_q[row] = torch.clamp(yf * (1.0 / sc)[:, None], -FP8_MAX, FP8_MAX).to(q8).view(-1)
        if not verify:
            ssm_state[s] = S
    return out, out_q, out_s


def gdn_core(qkvz, hidden, w, state, step, tokens, hk, hv, scale, eps, verify, act=torch.bfloat16, bf=_bf):
    """Both stages.  `w`: conv_w bf16 [conv_dim, 4], conv_bias or None, ba_w bf16 [2 hv, k_in], a_log, dt_bias f32 [hv],
    norm_w bf16 [D].  `state`: conv_state, ssm_state, inter_conv, inter_ssm (updated in place).  `step`: slot,
    inter_slot int32 [requests]."""
    conv_dim = 2 * hk * D + hv * D
    mixed = conv_chain(qkvz, w["conv_w"], w.get("conv_bias"), state["conv_state"], step["slot"], step["inter_slot"],
                       state.get("inter_conv"), tokens, conv_dim, verify, act)
    out, out_q, out_s = delta_chain(mixed, qkvz, hidden, w["ba_w"], state["ssm_state"], step["slot"], step["inter_slot"],
                                    state.get("inter_ssm"), w["a_log"], w["dt_bias"], w["norm_w"], tokens, hk, hv, scale, eps,
                                    verify, act, bf)
    return dict(mixed=mixed, out=out, out_q=out_q, out_scale=out_s)


def make_case(seed, requests, tokens, hk, hv, k_in, act=torch.bfloat16, slots=None, dead=(), no_snapshot=()):
    """Seeded inputs of one step: (qkvz, hidden, w, state, step).  Requests in `dead` have slot -1, requests in
    `no_snapshot` have inter_slot -1.  Value ranges follow the reference's verify test
    (test/kernels/test_qwen35_a17b_fp8_verify.py:118-150): unit-normal activations, state 0.1 N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    rows = requests * tokens
    conv_dim = 2 * hk * D + hv * D
    n_slots = slots or requests + 1
    qkvz = torch.randn(rows, conv_dim + hv * D, generator=g).to(act)
    hidden = torch.randn(rows, k_in, generator=g).to(act)
    w = dict(conv_w=(torch.randn(conv_dim, 4, generator=g) * 0.5).to(act), ba_w=(torch.randn(2 * hv, k_in, generator=g) * 0.05).to(act),
             a_log=torch.randn(hv, generator=g) * 0.5, dt_bias=torch.randn(hv, generator=g),
             norm_w=(1 + 0.1 * torch.randn(D, generator=g)).to(act))
    state = dict(conv_state=torch.randn(n_slots, 3, conv_dim, generator=g).to(act),
                 ssm_state=torch.randn(n_slots, hv, D, D, generator=g) * 0.1,
                 inter_conv=torch.zeros(requests, tokens, 3, conv_dim, dtype=act),
                 inter_ssm=torch.zeros(requests, tokens, hv, D, D))
    perm = torch.randperm(n_slots, generator=g)[:requests].to(torch.int32)
    iperm = torch.randperm(requests, generator=g).to(torch.int32)
    for r in dead:
        perm[r] = -1
    for r in no_snapshot:
        iperm[r] = -1
    return qkvz, hidden, w, state, dict(slot=perm, inter_slot=iperm)
