"""Generate the golden vectors under ``tests/golden/`` from the reference's own code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/MatGPTQ

It imports ``src/quant_utils_matgpqt.py`` and ``src/quant_utils_gptq.py`` from that
checkout (pure torch, CPU) and records their outputs on seeded inputs.  The tests
only read the resulting ``.npz`` files; they never import the reference.
bf16 tensors are stored as their raw uint16 bit patterns, fp16 as float16.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
BITS = (2, 3, 4, 6, 8)


def _bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from src.quant_utils_matgpqt import (FakeMatryoshkaLinear, MatryoshkaQuantizer,
                                         dequantize, matryoshka_slice)
    from src.quant_utils_gptq import quantize as rtn_quantize

    out: dict[str, np.ndarray] = {}

    # 1. slicing table: every byte value, every supported slice, master 8; plus the
    #    pass-through case master == slice for a non-8 master.
    allbytes = torch.arange(256, dtype=torch.uint8)
    for b in BITS:
        out[f"slice_m8_b{b}"] = matryoshka_slice(allbytes, 8, b).numpy()
    out["slice_m4_b4"] = matryoshka_slice(allbytes, 4, 4).numpy()
    out["slice_m6_b4"] = matryoshka_slice(allbytes, 6, 4).numpy()

    # 2. dequantize on seeded inputs, both dtypes, asymmetric and symmetric zero,
    #    including tiny and huge scales (subnormal / overflow edges of fp16).
    g = torch.Generator().manual_seed(1234)
    n, groups, gs = 16, 3, 128
    q = torch.randint(0, 256, (n, groups, gs), dtype=torch.uint8, generator=g)
    out["dq_q"] = q.numpy()
    for dname, dtype in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        scale = (torch.rand(n, groups, 1, generator=g) * 0.02 + 1e-4).to(dtype)
        scale[0, 0, 0] = 6e-8 if dtype == torch.float16 else 1e-38      # subnormal products
        scale[1, 0, 0] = 400.0 if dtype == torch.float16 else 3e36     # overflow to inf
        scale[2, 0, 0] = 0.0
        zero_asym = torch.randint(60, 190, (n, groups, 1), generator=g).to(dtype)
        zero_sym = torch.full((n, groups, 1), 128.0).to(dtype)
        out[f"dq_scale_{dname}"] = _bits16(scale)
        out[f"dq_zero_asym_{dname}"] = _bits16(zero_asym)
        for b in BITS:
            out[f"dq_asym_{dname}_b{b}"] = _bits16(dequantize(q, scale, zero_asym, 8, b))
            out[f"dq_sym_{dname}_b{b}"] = _bits16(dequantize(q, scale, zero_sym, 8, b))

    # 3. FakeMatryoshkaLinear forward (dequantise-then-matmul) on a small layer.
    g = torch.Generator().manual_seed(99)
    n, k, gs, m = 32, 256, 128, 3
    qw = torch.randint(0, 256, (n, k), dtype=torch.uint8, generator=g)
    sc = (torch.rand(n, k // gs, generator=g) * 0.02 + 1e-3).half()
    zp = torch.randint(100, 150, (n, k // gs), generator=g).half()
    xx = torch.randn(m, k, generator=g).half()
    out["fl_q"] = qw.numpy()
    out["fl_scale"] = sc.numpy()
    out["fl_zero"] = zp.numpy()
    out["fl_x"] = xx.numpy()
    for b in BITS:
        layer = FakeMatryoshkaLinear(qw, sc, zp, master_bitwidth=8, slice_bitwidth=b)
        with torch.no_grad():
            out[f"fl_w_b{b}"] = layer.get_weight().numpy()
            out[f"fl_y_b{b}"] = layer(xx).numpy()

    # 4. min-max parameters + RTN codes (how synthetic master codes are drawn).
    g = torch.Generator().manual_seed(7)
    w = torch.randn(8, 512, generator=g) * 0.02
    wg = w.reshape(-1, 128)
    out["mm_w"] = w.numpy()
    for sym in (False, True):
        quantizer = MatryoshkaQuantizer()
        quantizer.configure(bits=8, perchannel=True, sym=sym)
        quantizer.find_params(wg, weight=True)
        tag = "sym" if sym else "asym"
        out[f"mm_scale_{tag}"] = quantizer.scale.numpy()
        out[f"mm_zero_{tag}"] = quantizer.zero.numpy()
        codes = rtn_quantize(wg, quantizer.scale, quantizer.zero, quantizer.maxq)
        out[f"mm_codes_{tag}"] = codes.to(torch.uint8).numpy()

    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print(f"wrote {len(out)} arrays to {os.path.join(HERE, 'reference_vectors.npz')}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the MatGPTQ checkout>")
    main(sys.argv[1])
