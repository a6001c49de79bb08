"""Generate the golden vectors under tests/golden/ by running the reference's own
importable Python helpers on seeded inputs.  Run once in a container where the
reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

The vectors (inputs and the reference's outputs) are committed; the tests only read
the .npz files, so they run where the reference is absent.
"""

from __future__ import annotations

import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref: str) -> None:
    sys.path.insert(0, ref)
    warnings.filterwarnings("ignore")
    from sgl_amd_mono.glm53 import check as G
    from sgl_amd_mono.muse_spark import mxfp4_quant as MX
    from sgl_amd_mono.qwen35_a17b.fp8.gfx950 import gemv as GV

    g = torch.Generator().manual_seed(20240607)
    out = {}

    # per-128 FP8 activation quant (glm53/check.py:416-424, qwen35 gemv.py:256-266)
    x = (torch.randn(6, 512, generator=g) * torch.tensor([1e-3, 0.1, 1.0, 3.0, 30.0, 0.0])[:, None]).bfloat16()
    out["q128_x"] = x.float().numpy()
    out["q128_glm"] = G._q128(x).numpy()
    out["q128_rows"] = GV._quantize_rows(x).numpy()

    # block-FP8 GEMV (qwen35 gemv.py:268-273)
    w = torch.randn(256, 512, generator=g) * 0.02
    blk = w.reshape(2, 128, 4, 128)
    ws = blk.abs().amax(dim=(1, 3)) / 448.0
    wq = (blk / ws[:, None, :, None]).reshape(256, 512).to(torch.float8_e4m3fn)
    out["gemv_w_bytes"] = wq.view(torch.uint8).numpy()
    out["gemv_ws"] = ws.numpy()
    out["gemv_y"] = GV._plain_gemv(x, wq, ws).float().numpy()
    out["slices_f32"] = G.slices_f32(wq[None], ws[None], False)[0].numpy()

    # RMSNorm (glm53/check.py:391-393)
    gw = (1 + 0.1 * torch.randn(512, generator=g)).bfloat16()
    out["rms_w"] = gw.float().numpy()
    out["rms_y"] = G._rms(x, gw, 1e-5).numpy()

    # radix key (glm53/check.py:111-114)
    f = torch.tensor([0.0, -0.0, 1.0, -1.0, 3.5e-39, -3.5e-39, 65504.0, -1e30, 1e30, 2.5, 2.5000002])
    out["radix_in"] = f.numpy()
    out["radix_keys"] = G._radix_keys(f.view(torch.int32)).numpy()

    # MXFP4 (muse_spark/mxfp4_quant.py:15-80; glm53/check.py:438-444)
    m = torch.randn(3, 8, 128, generator=g) * torch.tensor([0.02, 1.0, 50.0])[:, None, None]
    m[0, 0, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.5]) * 2.0**-6
    p, s = MX.quantize_mxfp4(m)
    out["mx4_in"] = m.numpy()
    out["mx4_packed"] = p.numpy()
    out["mx4_scales"] = s.numpy()
    out["mx4_deq"] = MX.dequantize_mxfp4(p, s).numpy()
    out["mx4_deq_glm"] = G.mx_f32(p, s).numpy()

    np.savez_compressed(os.path.join(HERE, "reference_helpers.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_helpers.npz"), {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
