"""Parity of the packed matmul with the reference's dequantise-then-matmul.

* the reference's own kernel test grid (inference_lib/test_matgptq_matmul.py:11-49): integer-valued
  scales and activations make every partial sum exact, so the comparison is exact;
* real-valued layers in the benchmark's shapes: outputs within 1e-2 of an fp32 accumulation over the
  oracle's dequantised weights (max |y - y_ref| / max |y_ref|).
"""
import pytest
import torch
import torch.nn.functional as F

from matgptq_b200 import synth
from oracle import matgptq_oracle as oracle

pytestmark = pytest.mark.gpu
BITS = (2, 3, 4, 6, 8)
TOL = 1e-2

torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


@pytest.mark.parametrize("bitwidth", BITS)
@pytest.mark.parametrize("n_out_features", [16])
@pytest.mark.parametrize("n_in_features", [1024, 4096, 8192])
@pytest.mark.parametrize("batch_size", [1, 8, 16])
@pytest.mark.parametrize("group_size", [-1, 32, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_reference_kernel_grid_exact(cuda, bitwidth, n_out_features, n_in_features, batch_size, group_size, dtype):
    from matgptq_b200.matgptq_linear import MatGPTQLinear
    torch.random.manual_seed(1)
    gs = group_size if group_size != -1 else n_in_features
    qweights = torch.randint(0, 2 ** bitwidth, (n_out_features, n_in_features), dtype=torch.uint8)
    scales = torch.rand(n_out_features, n_in_features // gs, dtype=dtype).round()
    x = torch.randn(batch_size, n_in_features, dtype=dtype).round()
    weight_dq = oracle.op_dequantized_weight(qweights, scales, bitwidth, group_size)
    y_true = F.linear(x.to(cuda).to(weight_dq.dtype), weight_dq.to(cuda))
    layer = MatGPTQLinear(qweights, scales, bitwidth, group_size)
    y = layer(x.to(cuda))
    torch.cuda.synchronize()
    assert y.shape == (batch_size, n_out_features) and y.dtype == dtype
    assert torch.allclose(y, y_true), f"b={bitwidth} K={n_in_features} M={batch_size} g={group_size} {dtype}"
    # exact, not just close: every partial sum is an integer below 2^24
    y_exact = F.linear(x.double(), weight_dq.double()).to(dtype)
    assert torch.equal(y.cpu(), y_exact)


def _layer_and_ref(n_out, n_in, gs, b, dtype, seed, cuda):
    layer = synth.make_layer(n_out, n_in, gs, seed=seed, sym=True, dtype=dtype, device=cuda)
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n_out, n_in, 8, b, gs, flag)
    scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n_out, n_in, gs)
    # oracle weights on the CPU (the GPU only holds inputs and the product's outputs)
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    return packed, scales_r, w_ref, flag


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("shape", [(4096, 4096), (4096, 1024)])
@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
def test_llama_shapes_fp16(cuda, b, shape, m):
    from matgptq_b200 import ops  # noqa: F401
    n_in, n_out = shape
    packed, scales_r, w_ref, flag = _layer_and_ref(n_out, n_in, 128, b, torch.float16, 11 + b, cuda)
    x = synth.make_activations(m, n_in, seed=m, dtype=torch.float16, device=cuda)
    y = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, 128, flag)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert oracle.rel_err(y.cpu(), y_ref) <= TOL


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("shape", [(4096, 14336), (14336, 4096)])
def test_llama_mlp_shapes_fp16(cuda, b, shape):
    """gate/up and down at every bitwidth and every batch size of the sweep (their launch shapes differ from
    the small layers': clusters, K slices inside the CTA, two batch tiles).  Besides the global measure the
    element-wise one is checked: |y - y_ref| <= 1e-2 * |y_ref| + 1e-2 * rms(y_ref)."""
    from matgptq_b200 import ops  # noqa: F401
    n_in, n_out = shape
    packed, scales_r, w_ref, flag = _layer_and_ref(n_out, n_in, 128, b, torch.float16, 5, cuda)
    for m in (1, 2, 4, 8, 16):
        x = synth.make_activations(m, n_in, seed=m, dtype=torch.float16, device=cuda)
        y = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, 128, flag)
        y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
        assert oracle.rel_err(y.cpu(), y_ref) <= TOL, f"M={m}"
        assert oracle.elementwise_err(y.cpu(), y_ref, rtol=1e-2, atol_rms=1e-2) <= 1.0, f"M={m}"


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("b", [2, 3, 8])
@pytest.mark.parametrize("m", [1, 16])
def test_tensor_parallel_arithmetic_on_one_gpu(cuda, world, b, m):
    """The arithmetic of tensor parallelism through the CUDA kernels, every rank's shard run on one GPU:
    column-parallel shards (out-features split) concatenated in rank order and row-parallel shards
    (in-features split) summed in rank order must give the unsharded operator's result and the oracle's."""
    from matgptq_b200 import ops  # noqa: F401
    n_in, n_out = 4096, 1024
    layer = synth.make_layer(n_out, n_in, 128, seed=31, sym=True, dtype=torch.float16, device=cuda)
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    x = synth.make_activations(m, n_in, seed=m, dtype=torch.float16, device=cuda)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)

    def run(q, s, xs):
        n, k = q.shape
        packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(q.contiguous(), n, k, 8, b, 128, 1)
        scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(s.contiguous(), n, k, 128)
        return torch.ops.matgptq_cuda.matmul_matgptq(xs.contiguous(), packed, scales_r, n, k, b, 128, 1)

    y_full = run(layer.qweight, layer.scales, x)
    rows, cols = n_out // world, n_in // world
    y_col = torch.cat([run(layer.qweight[r * rows:(r + 1) * rows], layer.scales[r * rows:(r + 1) * rows], x)
                       for r in range(world)], dim=1)
    partial = [run(layer.qweight[:, r * cols:(r + 1) * cols], layer.scales[:, r * cols // 128:(r + 1) * cols // 128],
                   x[:, r * cols:(r + 1) * cols]) for r in range(world)]
    y_row = partial[0].float()
    for part in partial[1:]:
        y_row = y_row + part.float()
    for name, y in (("unsharded", y_full), ("column-parallel", y_col), ("row-parallel", y_row)):
        assert oracle.rel_err(y.cpu(), y_ref) <= TOL, name
    # out-feature shards do not change any output's arithmetic beyond the order of the K split
    assert oracle.rel_err(y_col.cpu(), y_full.float().cpu()) <= 2e-3


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("gs", [-1, 32, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 3, 7, 9, 13, 17, 31, 33, 64])
def test_ragged_batches_and_groups(cuda, b, gs, dtype, m):
    """Every batch size is valid here, including the ones the reference kernel cannot run."""
    from matgptq_b200 import ops  # noqa: F401
    n_out, n_in = 208, 1152      # 13 row tiles, 9 blocks: nothing divides evenly
    packed, scales_r, w_ref, flag = _layer_and_ref(n_out, n_in, gs, b, dtype, 3, cuda)
    x = synth.make_activations(m, n_in, seed=m, dtype=dtype, device=cuda)
    y = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, gs, flag)
    assert y.shape == (m, n_out)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert oracle.rel_err(y.cpu(), y_ref) <= TOL


@pytest.mark.parametrize("b", [3, 4])
@pytest.mark.parametrize("m", [5, 13])
@pytest.mark.parametrize("warps,split", [(1, 1), (2, 8), (4, 2), (8, 1), (8, 4), (8, 8), (3, 4), (16, 2), (13, 1),
                                         # warps | K slices inside the CTA << 8
                                         (8 | 2 << 8, 1), (8 | 2 << 8, 4), (16 | 8 << 8, 1), (16 | 16 << 8, 1),
                                         (12 | 4 << 8, 2), (6 | 3 << 8, 2)])
def test_every_launch_shape_gives_the_same_answer(cuda, b, warps, split, m):
    from matgptq_b200 import ops
    n_out, n_in = 272, 2048
    packed, scales_r, w_ref, flag = _layer_and_ref(n_out, n_in, 128, b, torch.float16, 9, cuda)
    x = synth.make_activations(m, n_in, seed=1, dtype=torch.float16, device=cuda)
    try:
        y = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag, warps_per_cta=warps, split_k=split)
    except RuntimeError as e:
        # K slices inside a CTA need its whole K slice of the activations in shared memory; a forced shape
        # that does not fit is refused (the automatic choice falls back to the plain cluster split)
        assert (warps >> 8) > 1 and "status 3" in str(e)
        return
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert oracle.rel_err(y.cpu(), y_ref) <= TOL
    # the cluster reduction adds partial sums in a fixed order: repeated launches are bit-identical
    y2 = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag, warps_per_cta=warps, split_k=split)
    assert torch.equal(y, y2)


def test_pdl_flag_and_linearity(cuda):
    from matgptq_b200 import ops
    n_out, n_in, m, b = 1024, 4096, 4, 4
    packed, scales_r, w_ref, flag = _layer_and_ref(n_out, n_in, 128, b, torch.float16, 21, cuda)
    x = synth.make_activations(m, n_in, seed=2, dtype=torch.float16, device=cuda)
    y = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag)
    y_pdl = x
    for _ in range(3):  # back-to-back launches with programmatic dependent launch
        y_pdl = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag | 4)
    assert torch.equal(y, y_pdl)
    # f(2x) == 2 f(x) exactly (scaling by two is exact in fp16 away from overflow)
    y2 = ops.matmul_matgptq_raw(x * 2, packed, scales_r, n_out, n_in, b, 128, flag)
    assert torch.equal(y2, y * 2)


def test_input_views_and_errors(cuda):
    from matgptq_b200 import ops  # noqa: F401
    n_out, n_in, b = 64, 256, 4
    packed, scales_r, w_ref, flag = _layer_and_ref(n_out, n_in, 128, b, torch.float16, 2, cuda)
    x = synth.make_activations(6, n_in + 8, seed=2, dtype=torch.float16, device=cuda)[:, 4:4 + n_in]  # strided, misaligned
    y = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, 128, flag)
    assert oracle.rel_err(y.cpu(), oracle.linear_fp32_accumulate(x.cpu(), w_ref)) <= TOL
    with pytest.raises(RuntimeError, match="wrong size"):
        torch.ops.matgptq_cuda.matmul_matgptq(x, packed[:-1], scales_r, n_out, n_in, b, 128, flag)
    with pytest.raises(RuntimeError, match="bitwidth"):
        wrong = torch.zeros(5 * n_out * n_in // 32, dtype=torch.uint32, device=cuda)
        torch.ops.matgptq_cuda.matmul_matgptq(x, wrong, scales_r, n_out, n_in, 5, 128, flag)
    with pytest.raises(RuntimeError, match="CUDA"):
        torch.ops.matgptq_cuda.matmul_matgptq(x.cpu(), packed, scales_r, n_out, n_in, b, 128, flag)
    empty = torch.ops.matgptq_cuda.matmul_matgptq(x[:0], packed, scales_r, n_out, n_in, b, 128, flag)
    assert empty.shape == (0, n_out)


@pytest.mark.parametrize("m", [1, 16, 48])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_out_form_writes_the_callers_tensor(cuda, m, dtype):
    """matmul_matgptq_out: the same bits as the allocating operator, written into a slice of a larger buffer (GEMV
    and tensor-core path), nothing around the slice touched; a wrong `out` is an error."""
    from matgptq_b200 import ops  # noqa: F401
    n_out, n_in, b = 384, 1024, 3
    packed, scales_r, w_ref, flag = _layer_and_ref(n_out, n_in, 128, b, dtype, 5, cuda)
    x = synth.make_activations(m, n_in, seed=m, dtype=dtype, device=cuda)
    y = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, 128, flag)
    buf = torch.full((3 * m * n_out,), 7.0, dtype=dtype, device=cuda)
    out = buf[m * n_out:2 * m * n_out].view(m, n_out)
    assert torch.ops.matgptq_cuda.matmul_matgptq_out(x, packed, scales_r, n_out, n_in, b, 128, flag, out) is None
    assert torch.equal(out, y)
    assert (buf[:m * n_out] == 7.0).all() and (buf[2 * m * n_out:] == 7.0).all()
    assert oracle.rel_err(out.cpu(), oracle.linear_fp32_accumulate(x.cpu(), w_ref)) <= TOL
    with pytest.raises(RuntimeError, match="out must be"):
        torch.ops.matgptq_cuda.matmul_matgptq_out(x, packed, scales_r, n_out, n_in, b, 128, flag, out[:, :-1])
    with pytest.raises(RuntimeError, match="out must be"):
        torch.ops.matgptq_cuda.matmul_matgptq_out(x, packed, scales_r, n_out, n_in, b, 128, flag, out.float())


# ---- extension: per-group zero points (asymmetric quantisation) ---------------------------------------------

def _asym_layer_and_ref(n_out, n_in, gs, b, dtype, seed, cuda):
    layer = synth.make_layer(n_out, n_in, gs, seed=seed, sym=False, dtype=dtype, device=cuda)
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n_out, n_in, 8, b, gs, flag)
    scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n_out, n_in, gs)
    zeros_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.zeros, n_out, n_in, gs)
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    return layer, packed, scales_r, zeros_r, w_ref, flag


def test_config0_asymmetric_minmax_4096_b4(cuda):
    """The CPU-runnable case of the benchmark definition: K = N = 4096, one fp16 activation row, weights
    N(0, 0.02) quantised per group of 128 with asymmetric min-max at 8 bits (fp16 scales and zero points),
    sliced to 4 bits; output against the dequantise-then-matmul of the oracle on the CPU."""
    layer, packed, scales_r, zeros_r, w_ref, flag = _asym_layer_and_ref(4096, 4096, 128, 4, torch.float16, 0, cuda)
    z = layer.zeros.float()
    assert z.min() < 120 and z.max() > 136  # really asymmetric
    x = synth.make_activations(1, 4096, seed=0, dtype=torch.float16, device=cuda)
    y = torch.ops.matgptq_cuda.matmul_matgptq_zeros(x, packed, scales_r, zeros_r, 4096, 4096, 4, 128, flag)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert y.shape == (1, 4096) and y.dtype == torch.float16
    assert oracle.rel_err(y.cpu(), y_ref) <= TOL
    # the three-op path on the same codes (implicit zero point 128) must NOT agree: the zero points matter
    y_sym = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, 4096, 4096, 4, 128, flag)
    assert oracle.rel_err(y_sym.cpu(), y_ref) > 10 * TOL


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("gs", [-1, 32, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m", [1, 5, 16, 37])
def test_zero_points_ragged(cuda, b, gs, dtype, m):
    n_out, n_in = 208, 1152
    layer, packed, scales_r, zeros_r, w_ref, flag = _asym_layer_and_ref(n_out, n_in, gs, b, dtype, 7, cuda)
    x = synth.make_activations(m, n_in, seed=m, dtype=dtype, device=cuda)
    y = torch.ops.matgptq_cuda.matmul_matgptq_zeros(x, packed, scales_r, zeros_r, n_out, n_in, b, gs, flag)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert oracle.rel_err(y.cpu(), y_ref) <= TOL


def test_zero_points_equal_to_128_match_the_three_op_path(cuda):
    n_out, n_in, b, m = 1024, 4096, 3, 4
    packed, scales_r, w_ref, flag = _layer_and_ref(n_out, n_in, 128, b, torch.float16, 5, cuda)
    zeros_r = torch.full_like(scales_r, 128.0)
    x = synth.make_activations(m, n_in, seed=3, dtype=torch.float16, device=cuda)
    y = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, 128, flag)
    yz = torch.ops.matgptq_cuda.matmul_matgptq_zeros(x, packed, scales_r, zeros_r, n_out, n_in, b, 128, flag)
    assert torch.equal(y, yz)
