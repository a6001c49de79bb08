"""The sparse-MLA FP8 MoE decoder layer as the composition of the stage restatements, plus its
seeded synthetic weights, caches and step metadata.

The reference pins the whole layer only against SGLang's own layer with loose bounds
(sgl_amd_mono/glm53/spec.py:168-226); its kernel tests pin stages.  The layer oracle here is
therefore the composition of the stage rules in oracle/{moe,quant,attn,collective}.py, in the
launch order of sgl_amd_mono/deepseek_v41/spec.py:716-779 (K1, K2i, K2).
"""

from __future__ import annotations

import numpy as np
import torch

from . import attn as A
from . import collective as C
from . import moe as M
from . import quant as Q

Q_LORA, KV_LORA, ROPE, NOPE, V_HEAD = 1536, 512, 64, 128, 128
IDX_HEADS, IDX_DIM, TOPK_KEYS = 64, 128, 2048
COL_KV, COL_ROPE, COL_IDX, COL_W, YA_COLS = 1536, 2048, 2112, 2240, 2304


def layer_cfg(tp=8, hidden=7168, heads=128, experts=256, topk=8, inter=2048, max_ctx=65536):
    return dict(tp=tp, hidden=hidden, heads=heads, experts=experts, topk=topk, inter=inter, max_ctx=max_ctx, eps=1e-6,
                route_scale=2.5, index_weight_scale=0.125 / 8.0, has_shared=True, score_fn=1, swiglu_limit=0.0)


def _q(gen, n, k, device, std=0.02):
    return Q.quant_weight_block128(std * torch.randn(n, k, generator=gen, device=device))


def make_weights(cfg, rank: int, seed: int = 0, device="cpu"):
    """Weights of one rank.  Replicated tensors (norms, q_a/kv_a, index projections, router) are drawn from a
    rank-independent generator; sharded ones (q_b, W_UK, W_UV, W_o columns, expert slices) from a per-rank one
    (sharding by head and by expert-intermediate slice: sgl_amd_mono/deepseek_v41/gfx950/attention/plan.py:48-50,
    stages/dims.py:29-37)."""
    g = torch.Generator(device=device).manual_seed(1000 * seed + 7)
    gr = torch.Generator(device=device).manual_seed(1000 * seed + 7 + 100 * (rank + 1))
    H, hl = cfg["hidden"], cfg["heads"] // cfg["tp"]

    def norm(n):
        return (1 + 0.1 * torch.randn(n, generator=g, device=device)).to(torch.bfloat16)

    w = dict(attn_norm=norm(H), q_norm=norm(Q_LORA), kv_norm=norm(KV_LORA))
    w["wa"], w["wa_s"] = _q(g, YA_COLS, H, device)
    w["wiq_b"], w["wiq_b_s"] = _q(g, IDX_HEADS * IDX_DIM, Q_LORA, device, std=0.05)
    w["wq_b"], w["wq_b_s"] = _q(gr, hl * 192, Q_LORA, device, std=0.05)
    w["w_uk"], w["w_uk_s"] = _q(gr, hl * KV_LORA, NOPE, device, std=0.08)
    w["w_uv"], w["w_uv_s"] = _q(gr, hl * V_HEAD, KV_LORA, device, std=0.05)
    w["w_o"], w["w_o_s"] = _q(gr, H, hl * V_HEAD, device)
    # MoE block: router replicated, expert slices per rank
    E, I = cfg["experts"], cfg["inter"] // cfg["tp"]
    w["ffn_norm"] = norm(H)
    w["gate_w"] = (0.02 * torch.randn(E, H, generator=g, device=device)).to(torch.bfloat16)
    w["bias"] = (0.02 * torch.randn(E, generator=g, device=device)).float()
    w13 = torch.empty(E + 1, 2 * I, H, dtype=torch.float8_e4m3fn, device=device)
    w13_s = torch.empty(E + 1, -(-2 * I // 128), H // 128, device=device)
    w2 = torch.empty(E + 1, H, I, dtype=torch.float8_e4m3fn, device=device)
    w2_s = torch.empty(E + 1, H // 128, I // 128, device=device)
    for e0 in range(0, E + 1, 32):
        e1 = min(E + 1, e0 + 32)
        w13[e0:e1], w13_s[e0:e1] = Q.quant_weight_block128(0.02 * torch.randn(e1 - e0, 2 * I, H, generator=gr, device=device))
        w2[e0:e1], w2_s[e0:e1] = Q.quant_weight_block128(0.02 * torch.randn(e1 - e0, H, I, generator=gr, device=device))
    w.update(w13=w13, w13_s=w13_s, w2=w2, w2_s=w2_s)
    return w


def make_step(cfg, rows: int, ctx_lo: int, ctx_hi: int, seed: int = 0, tokens_per_request: int = 1, device="cpu"):
    """Caches filled with random records for every earlier position, a permuted page table (page 0 = pad page,
    test/kernels/glm53/check_layer.py:248-261), positions uniform in [ctx_lo, ctx_hi); with tokens_per_request > 1
    the rows of a request sit at consecutive positions (verify step)."""
    g = torch.Generator().manual_seed(9000 + seed)
    n_req = rows // tokens_per_request
    first = torch.randint(ctx_lo, ctx_hi - tokens_per_request + 1, (n_req,), generator=g)
    pos = (first[:, None] + torch.arange(tokens_per_request)[None, :]).reshape(-1).to(torch.int32)
    req = torch.arange(n_req).repeat_interleave(tokens_per_request).to(torch.int32)
    max_pages = (int(pos.max()) + 64) // 64
    n_pages = n_req * max_pages + 1
    table = (torch.randperm(n_pages - 1, generator=g)[: n_req * max_pages] + 1).view(n_req, max_pages).to(torch.int32)
    kv = torch.randint(0, 256, (n_pages * 64, A.KV_REC), generator=g, dtype=torch.uint8)
    lat = kv[:, :KV_LORA]
    lat[(lat & 0x7F) == 0x7F] = 0x38
    kv[:, KV_LORA:KV_LORA + 16] = (torch.rand(n_pages * 64, 4, generator=g) * 0.02 + 0.002).view(torch.uint8).reshape(-1, 16)
    kv[:, KV_LORA + 16:] = torch.randn(n_pages * 64, ROPE, generator=g).to(torch.bfloat16).view(torch.uint8).reshape(-1, 2 * ROPE)
    idx = torch.randint(0, 256, (n_pages, 4352), generator=g, dtype=torch.uint8)
    idx[:, 4096:] = torch.randint(120, 128, (n_pages, 256), generator=g, dtype=torch.uint8)
    slots = (table[req.long(), (pos // 64).long()].long() * 64 + (pos % 64).long()).to(torch.int32)
    step = dict(positions=pos, slots=slots, req_of_row=req, ctx_len=(pos + 1).to(torch.int32), page_table=table)
    caches = dict(kv=kv, idx=idx, rope_table=A.rope_table(cfg["max_ctx"] + 64))
    return {k: v.to(device) for k, v in caches.items()}, {k: v.to(device) for k, v in step.items()}


def _cpu(t):
    return t.detach().cpu()


def k1(x, w, caches, step, cfg):
    """Front of the layer on one rank; writes the new records into `caches` (CPU copies) and returns intermediates."""
    hl = cfg["heads"] // cfg["tp"]
    rows = x.shape[0]
    pos = _cpu(step["positions"])
    tab = _cpu(caches["rope_table"])
    _, _, xq, xs = M.rmsnorm_quant(_cpu(x), w["attn_norm"], cfg["eps"])
    ya = Q.gemv_fp8(xq, xs, w["wa"], w["wa_s"]).to(torch.bfloat16)
    return k1_from_ya(ya, w, caches, step, cfg) | dict(xq=xq, xs=xs, ya=ya)


def k1_from_ya(ya, w, caches, step, cfg, q=None, qi=None):
    """Everything after the fused q_a/kv_a projection, from given bf16 `ya` (a launch's own, or the oracle's)."""
    hl = cfg["heads"] // cfg["tp"]
    ya = _cpu(ya)
    rows = ya.shape[0]
    pos = _cpu(step["positions"])
    tab = _cpu(caches["rope_table"])
    _, _, qa_q, qa_s = M.rmsnorm_quant(ya[:, :Q_LORA].contiguous(), w["q_norm"], cfg["eps"])
    _, _, kv_q, kv_s = M.rmsnorm_quant(ya[:, COL_KV:COL_ROPE].contiguous(), w["kv_norm"], cfg["eps"])
    kv_rec = A.kv_record(kv_q, kv_s, A.rope_gptj(ya[:, COL_ROPE:COL_IDX].contiguous(), pos, tab))
    ik = ya[:, COL_IDX:COL_W].clone()
    ik[:, 64:] = A.rope_gptj(ik[:, 64:].contiguous(), pos, tab)
    idx_rec = A.index_record(ik)
    if q is None:
        q = Q.gemv_fp8(qa_q, qa_s, w["wq_b"], w["wq_b_s"]).to(torch.bfloat16)
    qh = _cpu(q).view(rows, hl, 192)
    qn_q, qn_s = Q.quant128(qh[:, :, :NOPE].contiguous())
    q_rope = A.rope_gptj(qh[:, :, NOPE:].contiguous(), pos, tab)
    q_lat = Q.gemv_fp8(qn_q.view(rows, hl * NOPE), qn_s.view(rows, hl), w["w_uk"], w["w_uk_s"], groups=hl).to(torch.bfloat16)
    if qi is None:
        qi = Q.gemv_fp8(qa_q, qa_s, w["wiq_b"], w["wiq_b_s"]).to(torch.bfloat16)
    qih = _cpu(qi).view(rows, IDX_HEADS, IDX_DIM).clone()
    qih[:, :, 64:] = A.rope_gptj(qih[:, :, 64:].contiguous(), pos, tab)
    q_rec = A.index_record(qih.reshape(rows * IDX_HEADS, IDX_DIM)).view(rows, IDX_HEADS, 68)
    iw = (ya[:, COL_W:YA_COLS].float().numpy().astype(np.float32) * np.float32(cfg["index_weight_scale"])).astype(np.float32)
    return dict(qa_q=qa_q, qa_s=qa_s, kv_rec=kv_rec, idx_rec=idx_rec, q=q, q_rope=q_rope.reshape(rows, hl * ROPE),
                q_lat=q_lat, qi=qi, q_rec=q_rec, iw=torch.from_numpy(iw))


def write_records(caches, step, kv_rec, idx_rec):
    kv, idx = caches["kv"], caches["idx"]
    for t, s in enumerate(_cpu(step["slots"]).tolist()):
        if s <= 0:
            continue
        kv[s] = kv_rec[t]
        idx[s // 64, (s % 64) * 64:(s % 64) * 64 + 64] = idx_rec[t, :64]
        idx[s // 64, 4096 + (s % 64) * 4:4096 + (s % 64) * 4 + 4] = idx_rec[t, 64:]


def keys_of(caches, step, t):
    n = int(step["ctx_len"][t])
    req = int(step["req_of_row"][t])
    pages = caches["idx"][_cpu(step["page_table"])[req, : (n + 63) // 64].long()]
    return torch.cat([pages[:, :4096].reshape(-1, 64)[:n], pages[:, 4096:].reshape(-1, 4)[:n]], 1)


def k2i(q_rec, iw, caches, step):
    """Per row: (scores f32 [ctx], selected positions ascending)."""
    out = []
    for t in range(q_rec.shape[0]):
        s = A.index_scores(q_rec[t], iw[t], keys_of(caches, step, t))
        out.append((s, A.exact_topk(s, TOPK_KEYS)))
    return out


def attention(q_lat, q_rope, sel, caches, step, cfg):
    """o_lat bf16 [rows, heads_local*512] from the selected positions of every row."""
    hl = cfg["heads"] // cfg["tp"]
    rows = q_lat.shape[0]
    out = torch.empty(rows, hl, KV_LORA, dtype=torch.bfloat16)
    table = _cpu(step["page_table"])
    for t in range(rows):
        pos = torch.from_numpy(np.asarray(sel[t])).long()
        req = int(step["req_of_row"][t])
        slots = table[req, pos // 64].long() * 64 + pos % 64
        out[t] = A.sparse_mla(_cpu(q_lat)[t].view(hl, KV_LORA), _cpu(q_rope)[t].view(hl, ROPE), caches["kv"][slots], 192 ** -0.5)
    return out.view(rows, hl * KV_LORA)


def attn_out_partial(o_lat, w, cfg):
    """W_UV per head, o_proj: this rank's bf16 partial of the attention output."""
    hl = cfg["heads"] // cfg["tp"]
    ol_q, ol_s = Q.quant128(_cpu(o_lat))
    o_h = Q.gemv_fp8(ol_q, ol_s, w["w_uv"], w["w_uv_s"], groups=hl).to(torch.bfloat16)
    oh_q, oh_s = Q.quant128(o_h)
    return Q.gemv_fp8(oh_q, oh_s, w["w_o"], w["w_o_s"]).to(torch.bfloat16), o_h


def ffn_contrib(a, w, cfg):
    """This rank's per-slot MoE contributions [topk+1, rows, hidden] bf16 (the all-reduce sums the slots)."""
    ffn_w = dict(norm=w["ffn_norm"], gate_w=w["gate_w"], bias=w["bias"], w13=w["w13"], w13_s=w["w13_s"], w2=w["w2"], w2_s=w["w2_s"])
    fcfg = dict(cfg, inter=cfg["inter"] // cfg["tp"])
    r = M.moe_ffn(a, ffn_w, fcfg)
    return r


def forward(x, weights_by_rank, caches, step, cfg):
    """Whole layer on all ranks (CPU).  `caches` are CPU tensors and receive the step's new records."""
    caches = {k: _cpu(v) for k, v in caches.items()}
    step_c = {k: _cpu(v) for k, v in step.items()}
    x = _cpu(x)
    parts, inter = [], []
    for r, w in enumerate(weights_by_rank):
        f = k1(x, w, caches, step_c, cfg)
        if r == 0:
            write_records(caches, step_c, f["kv_rec"], f["idx_rec"])
            sel = k2i(f["q_rec"], f["iw"], caches, step_c)
        o_lat = attention(f["q_lat"], f["q_rope"], [s for _, s in sel], caches, step_c, cfg)
        part, _ = attn_out_partial(o_lat, w, cfg)
        parts.append(part)
        inter.append(dict(f, o_lat=o_lat, attn_part=part))
    a = C.allreduce(parts, x)
    contribs = [ffn_contrib(a, w, cfg) for w in weights_by_rank]
    out = C.allreduce([c["out"] for c in contribs], a)
    return dict(out=out, a=a, sel=sel, ranks=inter, ffn=contribs, caches=caches)
