"""The CUDA path against the committed golden fixtures (outputs of the compiled reference CPU
route, written by tests/golden/make_golden.py): int8-route outputs byte for byte, Q4_1 within
the fixture's tolerance.  These need no oracle and no reference tree at run time."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from nnops_b200 import ops

pytestmark = pytest.mark.gpu
GOLDEN = sorted((Path(__file__).resolve().parent / "golden").glob("*.npz"))


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_cuda_matches_golden(cuda_device, nnb200_lib, path):
    z = np.load(path)
    meta = json.loads(str(z["meta"]))
    dev = cuda_device
    if meta["op"] == "gemm_i8":
        kw = {k: (z[k] if k in z.files else meta["scalars"][k]) for k in meta["kw"]}
        a = torch.from_numpy(z["a"]).to(dev)
        w = torch.from_numpy(z["w"]).to(dev)
        a = a.t() if meta.get("a_transposed") else a        # logical [M,K] view of [K,M] storage
        w = w.t() if meta.get("w_kn") else w                # logical [N,K] view of [K,N] storage
        got = ops.gemm_i8(a, w, out_kind=meta["out_kind"], relu=meta["relu"],
                          activation="relu" if meta["relu"] and meta["out_kind"] in ("f32", "f16") else "none", **kw)
        assert np.array_equal(got.cpu().numpy().view(np.uint8), z["out"].view(np.uint8))
    elif meta["op"] == "conv2d_i8":
        g = meta["geom"]
        fp = meta["out_kind"] in ("f32", "f16")
        got = ops.conv2d_i8(torch.from_numpy(z["x"]).to(dev), torch.from_numpy(z["w"]).to(dev),
                            out_kind=meta["out_kind"], bias=torch.from_numpy(z["bias"]), relu=meta["relu"],
                            activation="relu" if meta["relu"] and fp else "none",
                            scale_w=torch.from_numpy(z["scale_w"]), zp_w=torch.from_numpy(z["zp_w"]),
                            stride=tuple(g["stride"]), dilation=tuple(g["dilation"]), padding=tuple(g["padding"]),
                            groups=g["groups"], **meta["scalars"])
        assert np.array_equal(got.cpu().numpy().view(np.uint8), z["out"].view(np.uint8))
    elif meta["op"] == "fp_act":
        pt = meta["per_token"]
        got = ops.linear_fp_act(torch.from_numpy(z["a"]).to(dev), torch.from_numpy(z["w"]).to(dev),
                                scale_a=torch.from_numpy(z["scale_a"]) if pt else float(z["scale_a"][0]),
                                zp_a=torch.from_numpy(z["zp_a"]) if pt else int(z["zp_a"][0]),
                                bias=torch.from_numpy(z["bias"]), relu=meta["relu"],
                                activation="relu" if meta["relu"] else "none", scale_w=torch.from_numpy(z["scale_w"]))
        assert np.array_equal(got.cpu().numpy().view(np.uint8), z["out"].view(np.uint8))
    elif meta["op"] == "quant_linear":
        scale, zp = torch.from_numpy(z["scale"]), torch.from_numpy(z["zero_point"])
        q = ops.quantize_linear(torch.from_numpy(z["x"]).to(dev), scale, zp, axis=meta["axis"],
                                out_dtype=torch.from_numpy(z["quantized"]).dtype)
        assert np.array_equal(q.cpu().numpy(), z["quantized"])
        dq = ops.dequantize_linear(torch.from_numpy(z["xq"]).to(dev), scale, zp, axis=meta["axis"],
                                   out_dtype=torch.from_numpy(z["dequantized"]).dtype)
        assert np.array_equal(dq.cpu().numpy().view(np.uint8), z["dequantized"].view(np.uint8))
    else:
        a = torch.from_numpy(z["a"]).to(dev)
        w = torch.from_numpy(z["w_blocks"]).to(dev)
        tdt = torch.float16 if meta["out_dtype"] == "f16" else torch.float32
        for engine in ("auto", "gemv_simt") if a.shape[0] <= 8 else ("auto",):
            got = ops.linear_q4_1(a, w, meta["k"], out_dtype=tdt, engine=engine).cpu().numpy().astype(np.float32)
            ref = z["out"].astype(np.float32)
            tol = meta["rtol"] * np.abs(ref) + meta["rtol"] * float(np.sqrt(np.mean(ref * ref)))
            assert np.all(np.abs(got - ref) <= tol), f"{engine}: max err {np.abs(got - ref).max()}"
