"""Grouped product: several weight matrices with their own bitwidths over the same activations in one launch
(the fused qkv / gate_up layers of a model with per-layer bitwidths).  Every segment's column block is compared
with the oracle's dequantise-then-matmul for that segment, and with the single-segment operator."""
import pytest
import torch

from matgptq_b200 import synth
from oracle import matgptq_oracle as oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _segments(rows_bits, n_in, gs, dtype, cuda, seed=0):
    from matgptq_b200 import ops  # noqa: F401  registers torch.ops.matgptq_cuda.*
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    packed, scales, refs = [], [], []
    for i, (rows, b) in enumerate(rows_bits):
        layer = synth.make_layer(rows, n_in, gs, seed=seed + 7 * i, sym=True, dtype=dtype, device=cuda)
        packed.append(torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, rows, n_in, 8, b, gs, flag))
        scales.append(torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, rows, n_in, gs))
        refs.append(oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b))
    return packed, scales, refs, flag


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("gs", [-1, 32, 128])
@pytest.mark.parametrize("m", [1, 5, 16, 23, 40, 130, 300])
def test_mixed_bitwidth_segments(cuda, dtype, gs, m):
    from matgptq_b200 import _native
    rows_bits = [(64, 2), (208, 3), (16, 4), (96, 6), (48, 8)]  # every bitwidth, ragged row counts
    n_in = 1152
    packed, scales, refs, flag = _segments(rows_bits, n_in, gs, dtype, cuda)
    x = synth.make_activations(m, n_in, seed=m, dtype=dtype, device=cuda)
    y = torch.ops.matgptq_cuda.matmul_matgptq_grouped(x, packed, scales, [r for r, _ in rows_bits], n_in,
                                                      [b for _, b in rows_bits], gs, flag)
    assert _native.device_status() == 0
    assert y.shape == (m, sum(r for r, _ in rows_bits)) and y.dtype == dtype
    col = 0
    for (rows, b), w_ref, w, s in zip(rows_bits, refs, packed, scales):
        y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
        assert oracle.rel_err(y[:, col:col + rows].cpu(), y_ref) <= TOL, f"segment b={b}"
        single = torch.ops.matgptq_cuda.matmul_matgptq(x, w, s, rows, n_in, b, gs, flag)
        assert oracle.rel_err(y[:, col:col + rows].cpu(), single.float().cpu()) <= 2e-3
        col += rows


@pytest.mark.parametrize("m", [1, 8, 16, 32, 100])  # from 32 rows: one grouped launch of the tensor-core path
@pytest.mark.parametrize("layer", ["qkv", "gate_up"])
def test_llama_fused_layers(cuda, layer, m):
    """The two fused layers of the Llama-3.1-8B architecture with the bitwidths a mean-3-bit assignment gives them."""
    from matgptq_b200 import ops
    n_in = 4096
    rows_bits = [(4096, 4), (1024, 2), (1024, 8)] if layer == "qkv" else [(14336, 3), (14336, 6)]
    packed, scales, refs, flag = _segments(rows_bits, n_in, 128, torch.float16, cuda, seed=3)
    x = synth.make_activations(m, n_in, seed=m, dtype=torch.float16, device=cuda)
    y = ops.matmul_matgptq_grouped_raw(x, packed, scales, [r for r, _ in rows_bits], n_in, [b for _, b in rows_bits], 128, flag | 4)
    y2 = ops.matmul_matgptq_grouped_raw(x, packed, scales, [r for r, _ in rows_bits], n_in, [b for _, b in rows_bits], 128, flag | 4)
    assert torch.equal(y, y2)  # fixed summation order
    col = 0
    for (rows, b), w_ref in zip(rows_bits, refs):
        assert oracle.rel_err(y[:, col:col + rows].cpu(), oracle.linear_fp32_accumulate(x.cpu(), w_ref)) <= TOL, f"b={b}"
        col += rows


def test_grouped_contract(lib, cuda):
    packed, scales, _, flag = _segments([(32, 4), (32, 2)], 256, 128, torch.float16, cuda)
    x = synth.make_activations(2, 256, seed=1, dtype=torch.float16, device=cuda)
    with pytest.raises(RuntimeError, match="per segment"):
        torch.ops.matgptq_cuda.matmul_matgptq_grouped(x, packed, scales, [32], 256, [4, 2], 128, flag)
    with pytest.raises(RuntimeError, match="wrong size"):
        torch.ops.matgptq_cuda.matmul_matgptq_grouped(x, packed, scales, [32, 48], 256, [4, 2], 128, flag)
    with pytest.raises(RuntimeError, match="at most 8"):
        torch.ops.matgptq_cuda.matmul_matgptq_grouped(x, packed * 5, scales * 5, [32] * 10, 256, [4, 2] * 5, 128, flag)
    empty = torch.ops.matgptq_cuda.matmul_matgptq_grouped(x[:0], packed, scales, [32, 32], 256, [4, 2], 128, flag)
    assert empty.shape == (0, 64)
    # fake tensors: shape and dtype without a launch
    meta = torch.ops.matgptq_cuda.matmul_matgptq_grouped(x.to("meta"), [p.to("meta") for p in packed],
                                                         [s.to("meta") for s in scales], [32, 32], 256, [4, 2], 128, flag)
    assert meta.shape == (2, 64) and meta.dtype == torch.float16
