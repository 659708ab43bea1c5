"""Golden vectors for the checkpoint-materialisation rules, from the reference's own Python code (CPU only).

    python tests/golden/make_golden_io.py <reference checkout>

Calls forge/utils/io.py::_apply_block_scale (packed int4 + group scales), ::_dequant_mxfp4_blocks_to_fp (MXFP4) and
::_apply_block_scale_inv_2d followed by the cast of materialize_block_weights_to_fp (fp8 e4m3 + 128x128 block scales) of
the reference on small seeded inputs and stores inputs and outputs in tests/golden/io_materialise.npz.  The module
imports accelerate and huggingface_hub at its top for unrelated functions; where those packages are absent they
are replaced by empty stand-ins, which the two functions used here never touch.
"""
import os
import sys
import types

import numpy as np
import torch

ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FORGE_REFERENCE_ROOT", "")
sys.path.insert(0, ref_root)
for name, attrs in (("accelerate", ()), ("accelerate.utils", ("set_module_tensor_to_device",)),
                    ("huggingface_hub", ("hf_hub_download",))):
    try:
        __import__(name)
    except Exception:
        m = types.ModuleType(name)
        for a in attrs:
            setattr(m, a, None)
        sys.modules[name] = m
import importlib.util  # noqa: E402

spec = importlib.util.spec_from_file_location("ref_io", os.path.join(ref_root, "forge", "utils", "io.py"))
rio = importlib.util.module_from_spec(spec)
spec.loader.exec_module(rio)

g = torch.Generator().manual_seed(77)
out = {}
O, I, gs = 24, 256, 32
packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (O, I // 8), generator=g, dtype=torch.int64).to(torch.int32)
scales = (torch.rand(O, I // gs, generator=g) * 0.02 + 1e-3).to(torch.float32)
out["int4_packed"], out["int4_scales"] = packed, scales
for sym in (True, False):
    for inv in (False, True):
        w = rio._apply_block_scale(packed, scales, [O, I], bits=4, symmetric=sym, scale_is_inv=inv)
        out[f"int4_out_sym{int(sym)}_inv{int(inv)}"] = w
rows, NB = 40, 3
blocks = torch.randint(0, 256, (2, rows, NB, 16), generator=g, dtype=torch.int64).to(torch.uint8)
sc = torch.randint(110, 135, (2, rows, NB), generator=g, dtype=torch.int64).to(torch.uint8)
sc[0, 0, 0] = 0          # the e == 0 rule
sc[1, 5, 2] = 254
out["mx_blocks"], out["mx_scales"] = blocks, sc
out["mx_out"] = rio._dequant_mxfp4_blocks_to_fp(blocks, sc).contiguous()
# fp8 e4m3 weights with fp32 block scales: whole tiles, a partial last row tile, and a scale grid whose row tile is
# not the column tile (the `so` fall-back of the reference's inference rule)
for tag, (O8, I8, nO, nI) in {"sq": (256, 256, 2, 2), "ragged": (200, 384, 2, 3), "tall": (96, 128, 3, 1)}.items():
    w8 = (torch.randn(O8, I8, generator=g) * 60.0).to(torch.float8_e4m3fn)
    sinv = (torch.rand(nO, nI, generator=g) * 2e-3 + 1e-5).to(torch.float32)
    w = rio._apply_block_scale_inv_2d(w8.to(torch.float32), sinv).to(torch.bfloat16)   # io.py:864-874
    out[f"fp8_{tag}_w"] = w8.view(torch.uint8)
    out[f"fp8_{tag}_sinv"] = sinv
    out[f"fp8_{tag}_out_bits"] = w.view(torch.int16)
path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "io_materialise.npz")
np.savez_compressed(path, **{k: v.numpy() for k, v in out.items()})
print(path, os.path.getsize(path), "bytes")
