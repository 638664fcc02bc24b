"""CPU oracle for the bit-sliced mixed-precision linear layer.

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU, the arithmetic of
the reference implementation of the path.  It is imported by ``tests/``, by the
smoke check and by the CPU-baseline / reference arm of ``bench.py`` and by
nothing else: the product path never routes through it and raises when the
CUDA library is missing.

Parity status: PINNED.  Every function below is checked against outputs of the
reference's own Python code (``src/quant_utils_matgpqt.py``) that were generated
by importing it and are committed as ``tests/golden/*.npz`` together with the
script that made them (``tests/golden/make_golden.py``), and against the
closed-form expected weight of the reference's kernel test
(``inference_lib/test_matgptq_matmul.py:40``).

Each function cites the reference lines it follows.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

SUPPORTED_BITWIDTHS = (2, 3, 4, 6, 8)


# --------------------------------------------------------------------------- #
# integer part: slicing
# --------------------------------------------------------------------------- #
def matryoshka_slice_np(x: np.ndarray, master_bitwidth: int, slice_bitwidth: int) -> np.ndarray:
    """Round-to-nearest MSB slice with saturation, numpy restatement.

    Follows ``src/quant_utils_matgpqt.py:9-17``: the number of dropped bits is
    ``8 - slice_bitwidth`` whatever the master bitwidth (codes are stored in a
    byte); the rounding bit is added unless the slice equals the master; the
    result saturates at ``2**slice_bitwidth - 1``.
    """
    assert x.dtype == np.uint8
    drop = 8 - slice_bitwidth
    floor = x.astype(np.int32) >> drop
    if master_bitwidth == slice_bitwidth:
        return np.clip(floor, 0, 2 ** slice_bitwidth - 1).astype(np.uint8)
    round_bit = (x.astype(np.int32) >> (drop - 1)) & 1
    return np.clip(floor + round_bit, 0, 2 ** slice_bitwidth - 1).astype(np.uint8)


def matryoshka_slice(x: torch.Tensor, master_bitwidth: int, slice_bitwidth: int) -> torch.Tensor:
    """Torch restatement of ``src/quant_utils_matgpqt.py:9-17`` (uint8 in, uint8 out)."""
    assert x.dtype == torch.uint8
    drop = 8 - slice_bitwidth
    floor = x >> drop
    if master_bitwidth == slice_bitwidth:
        return torch.clamp(floor, 0, 2 ** slice_bitwidth - 1)
    round_bit = (x >> (drop - 1)) & 1
    return torch.clamp(floor + round_bit, 0, 2 ** slice_bitwidth - 1)


# --------------------------------------------------------------------------- #
# floating-point part: dequantise, dequantise-then-matmul
# --------------------------------------------------------------------------- #
def dequantize(q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
               master_bitwidth: int, slice_bitwidth: int) -> torch.Tensor:
    """``scale * ((slice(q) << (master - slice)) - zero)``; result has the scale's dtype.

    Follows ``src/quant_utils_matgpqt.py:19-22``.  ``q_shifted - zero`` is an
    exact integer in the scale dtype; the multiplication rounds once.
    """
    q_slices = matryoshka_slice(q, master_bitwidth, slice_bitwidth)
    q_shifted = q_slices << (master_bitwidth - slice_bitwidth)
    return scale * (q_shifted - zero)


def dequantize_weight(qweight: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
                      master_bitwidth: int, slice_bitwidth: int) -> torch.Tensor:
    """Grouped dequantisation of a whole ``[N, K]`` code matrix.

    Follows ``FakeMatryoshkaLinear.get_weight`` (``src/quant_utils_matgpqt.py:202-216``):
    ``scale``/``zero`` are ``[N, G]``; codes are viewed ``[N, G, K/G]``.
    """
    n = qweight.shape[0]
    scale3 = scale.reshape(n, -1, 1)
    zero3 = zero.reshape(n, -1, 1)
    groups = scale3.shape[1]
    w = dequantize(qweight.reshape(n, groups, -1), scale3, zero3, master_bitwidth, slice_bitwidth)
    return w.reshape(qweight.shape)


def fake_matryoshka_linear(x: torch.Tensor, qweight: torch.Tensor, scale: torch.Tensor,
                           zero: torch.Tensor, master_bitwidth: int, slice_bitwidth: int,
                           bias: torch.Tensor | None = None,
                           perm: torch.Tensor | None = None) -> torch.Tensor:
    """Dequantise-then-matmul in the scale dtype, as the reference's fake layer does.

    Follows ``FakeMatryoshkaLinear.forward`` (``src/quant_utils_matgpqt.py:218-224``).
    This is the CPU path that the benchmark times as the reference arm.
    """
    if perm is not None:
        x = x[..., perm]
    w = dequantize_weight(qweight, scale, zero, master_bitwidth, slice_bitwidth)
    return F.linear(x, w, bias)


def linear_fp32_accumulate(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with both operands widened to fp32: the accumulation target
    that fp16/bf16 outputs are compared with (tolerance 1e-2, see ``rel_err``)."""
    return F.linear(x.float(), w.float())


def op_dequantized_weight(codes: torch.Tensor, scales: torch.Tensor, bitwidth: int,
                          group_size: int) -> torch.Tensor:
    """Expected weight of the three-op path for pre-sliced codes.

    Follows ``inference_lib/test_matgptq_matmul.py:40``:
    ``((q - 2**(b-1)) * s) * 2**(8-b)`` with ``s`` broadcast over each group
    (``group_size == -1`` means one group per row), computed in the scale dtype.
    """
    n, k = codes.shape
    gs = group_size if group_size != -1 else k
    dtype = scales.dtype
    w = (codes.to(torch.int32).unflatten(-1, (-1, gs)) - 2 ** (bitwidth - 1)) * scales.to(dtype)[..., None]
    return w.flatten(-2) * (2 ** (8 - bitwidth))


def rel_err(y: torch.Tensor, y_ref32: torch.Tensor) -> float:
    """``max|y - y_ref| / max|y_ref|`` — the error measure used for outputs (<= 1e-2)."""
    denom = y_ref32.abs().max().item()
    if denom == 0.0:
        return (y.float() - y_ref32).abs().max().item()
    return (y.float() - y_ref32).abs().max().item() / denom


def elementwise_err(y: torch.Tensor, y_ref32: torch.Tensor, rtol: float = 1e-2, atol_rms: float = 1e-2) -> float:
    """Element-wise companion of ``rel_err``: the largest ``|y - y_ref| / (rtol*|y_ref| + atol)`` with the
    absolute floor ``atol = atol_rms * rms(y_ref)``; a value <= 1 means every element is within
    ``rtol`` relative error or within the floor.  The floor is needed because sums of thousands of
    products land arbitrarily close to zero, where no relative bound on a single element is meaningful."""
    ref = y_ref32.float()
    atol = atol_rms * ref.pow(2).mean().sqrt().item()
    bound = rtol * ref.abs() + max(atol, 1e-30)
    return ((y.float() - ref).abs() / bound).max().item()


# --------------------------------------------------------------------------- #
# quantiser parameters (used only to build synthetic master codes)
# --------------------------------------------------------------------------- #
def minmax_params(w: torch.Tensor, bits: int, sym: bool) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-row min-max scale and zero-point for a ``[rows, cols]`` fp32 matrix.

    Follows ``MatryoshkaQuantizer.find_params`` with ``perchannel=True, weight=True``
    (``src/quant_utils_matgpqt.py:92-151``): asymmetric ``scale = (max-min)/maxq``,
    ``zero = round(-min/scale)``; symmetric ``zero = (maxq+1)/2``.
    """
    maxq = 2 ** bits - 1
    x = w.flatten(1)
    xmin = x.min(1).values.clone()
    xmax = x.max(1).values.clone()
    if sym:
        xmax = torch.maximum(torch.abs(xmin), xmax)
        neg = xmin < 0
        if torch.any(neg):
            xmin[neg] = -xmax[neg]
    same = xmin == xmax
    xmin[same] = -1
    xmax[same] = +1
    scale = (xmax - xmin) / maxq
    if sym:
        zero = torch.full_like(scale, (maxq + 1) / 2)
    else:
        zero = torch.round(-xmin / scale)
    return scale.reshape(-1, 1), zero.reshape(-1, 1)


def rtn_quantize(w: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, maxq: int) -> torch.Tensor:
    """Round-to-nearest codes ``clamp(round(w/scale + zero), 0, maxq)`` as uint8.

    Follows the plain quantiser of the GPTQ baseline (``src/quant_utils_gptq.py:23-25``).
    """
    q = torch.clamp(torch.round(w / scale.clamp_min(1e-9) + zero), 0, maxq)
    return q.to(torch.uint8)
