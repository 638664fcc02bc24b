"""Tensor-core path (tcgen05, batches >= 32): parity with the reference's dequantise-then-matmul.

Dense weights inside the kernel are the oracle's dequantised weights bit for bit, so the only
difference from `F.linear(x, W)` in fp32 is the order of accumulation: integer-valued inputs give
exact results, real-valued ones stay within 1e-2 (max |y - y_ref| / max |y_ref|).
"""
import pytest
import torch
import torch.nn.functional as F

from matgptq_b200 import synth
from oracle import matgptq_oracle as oracle

pytestmark = pytest.mark.gpu
BITS = (2, 3, 4, 6, 8)
TOL = 1e-2


def _pack(layer, n_out, n_in, gs, b, dtype):
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n_out, n_in, 8, b, gs, flag)
    scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n_out, n_in, gs)
    return packed, scales_r, flag


def _status_ok():
    from matgptq_b200 import _native
    return _native.device_status() == 0


@pytest.mark.parametrize("bitwidth", BITS)
@pytest.mark.parametrize("group_size", [-1, 32, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch_size,n_in_features", [(32, 1024), (64, 4096)])
def test_integer_inputs_are_exact(cuda, bitwidth, group_size, dtype, batch_size, n_in_features):
    """The reference's kernel test (inference_lib/test_matgptq_matmul.py:11-49) at tensor-core batch sizes."""
    from matgptq_b200.matgptq_linear import MatGPTQLinear
    torch.random.manual_seed(1)
    n_out = 128
    gs = group_size if group_size != -1 else n_in_features
    q = torch.randint(0, 2 ** bitwidth, (n_out, n_in_features), dtype=torch.uint8)
    scales = torch.rand(n_out, n_in_features // gs, dtype=dtype).round()
    x = torch.randn(batch_size, n_in_features, dtype=dtype).round()
    w = oracle.op_dequantized_weight(q, scales, bitwidth, group_size)
    y = MatGPTQLinear(q, scales, bitwidth, group_size)(x.to(cuda))
    assert _status_ok()
    assert torch.equal(y.cpu(), F.linear(x.double(), w.double()).to(dtype))


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape,m", [((256, 208), 33), ((1152, 384), 100), ((512, 128), 300), ((4096, 1024), 128)])
def test_real_valued_parity(cuda, b, dtype, shape, m):
    from matgptq_b200 import ops
    n_in, n_out = shape
    layer = synth.make_layer(n_out, n_in, 128, seed=b, sym=True, dtype=dtype, device=cuda)
    packed, scales_r, flag = _pack(layer, n_out, n_in, 128, b, dtype)
    x = synth.make_activations(m, n_in, seed=m, dtype=dtype, device=cuda)
    y = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag, path=2)
    assert _status_ok()
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert y.shape == (m, n_out)
    assert oracle.rel_err(y.cpu(), y_ref) <= TOL


@pytest.mark.parametrize("split", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("m", [5, 16, 64, 256])
def test_split_k_and_small_batches_agree_with_gemv(cuda, split, m):
    """Any batch size may be forced onto the tensor-core path; every K split gives the GEMV's answer."""
    from matgptq_b200 import ops
    n_in, n_out, b = 2048, 384, 4
    layer = synth.make_layer(n_out, n_in, 128, seed=4, sym=True, dtype=torch.float16, device=cuda)
    packed, scales_r, flag = _pack(layer, n_out, n_in, 128, b, torch.float16)
    x = synth.make_activations(m, n_in, seed=m, dtype=torch.float16, device=cuda)
    y_tc = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag, path=2, split_k=split)
    y_gemv = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag, path=1)
    assert _status_ok()
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert oracle.rel_err(y_tc.cpu(), y_ref) <= TOL
    assert oracle.rel_err(y_gemv.cpu(), y_ref) <= TOL
    # repeated launches are bit-identical (fixed summation order in the split-K reduction)
    y_again = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag, path=2, split_k=split)
    assert torch.equal(y_tc, y_again)


def test_workspace_contract(lib, cuda):
    """The sums of a split K meet inside a thread-block cluster; with FLAG_SCRATCH_REDUCE they go through scratch
    and a second kernel.  Both add in the order of the K ranges: identical bits."""
    from matgptq_b200 import _native
    assert lib.matgptq_b200_matmul_workspace_bytes(4096, 4096, 16) == 0      # GEMV family: no scratch
    need = lib.matgptq_b200_matmul_workspace_bytes(1024, 4096, 64)           # 8 tiles only: K is split
    assert need > 0 and need % (64 * 1024 * 4) == 0
    n_in, n_out, b, m = 4096, 1024, 3, 64
    layer = synth.make_layer(n_out, n_in, 128, seed=1, sym=True, dtype=torch.bfloat16, device=cuda)
    packed, scales_r, flag = _pack(layer, n_out, n_in, 128, b, torch.bfloat16)
    x = synth.make_activations(m, n_in, seed=1, dtype=torch.bfloat16, device=cuda)
    y_op = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, 128, flag)
    stream = torch.cuda.current_stream().cuda_stream
    # no scratch: the plain entry point splits K in the same way
    y_plain = torch.empty_like(y_op)
    st = lib.matgptq_b200_matmul(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(), x.data_ptr(),
                                 y_plain.data_ptr(), stream, flag)
    assert st == 0
    # through scratch
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    y_scratch = torch.empty_like(y_op)
    st = lib.matgptq_b200_matmul_ws(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(), x.data_ptr(),
                                    y_scratch.data_ptr(), stream, flag | _native.FLAG_SCRATCH_REDUCE, ws.data_ptr(), need, 2, 0)
    assert st == 0
    torch.cuda.synchronize()
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert oracle.rel_err(y_op.cpu(), y_ref) <= TOL
    assert torch.equal(y_op, y_plain) and torch.equal(y_op, y_scratch)
    # the scratch form without enough scratch, and more CTAs along K than a cluster holds, are argument
    # errors, not silent fallbacks
    small = torch.empty(16, dtype=torch.uint8, device=cuda)
    st = lib.matgptq_b200_matmul_ws(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(), x.data_ptr(),
                                    y_plain.data_ptr(), stream, flag | _native.FLAG_SCRATCH_REDUCE, small.data_ptr(), 16, 2, 4)
    assert st == 1
    st = lib.matgptq_b200_matmul_ws(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(), x.data_ptr(),
                                    y_plain.data_ptr(), stream, flag, None, 0, 2, 9)
    assert st == 1
    assert _status_ok()


_LLAMA = {"q_o": (4096, 4096), "k_v": (4096, 1024), "gate_up": (4096, 14336), "down": (14336, 4096)}


@pytest.mark.parametrize("b", [3, 4, 8])
@pytest.mark.parametrize("shape", list(_LLAMA))
def test_tensor_core_regime_grid_bf16(cuda, shape, b):
    """Every cell of the tensor-core regime the benchmark times: the four Llama-3-8B shapes x M in
    {32, 64, 128, 256} x b in {3, 4, 8}, bf16, through the operator (automatic path and K split), against the
    oracle's dequantise-then-matmul.  For the two large layers the comparison runs on every seventh
    out-feature (all 128-row tiles are hit) to bound the CPU time of the oracle."""
    from matgptq_b200 import ops  # noqa: F401
    n_in, n_out = _LLAMA[shape]
    layer = synth.make_layer(n_out, n_in, 128, seed=300 + b, sym=True, dtype=torch.bfloat16, device=cuda)
    packed, scales_r, flag = _pack(layer, n_out, n_in, 128, b, torch.bfloat16)
    rows = torch.arange(0, n_out, 7 if n_out * n_in > 4096 * 4096 else 1)
    w_ref = oracle.dequantize_weight(layer.qweight.cpu()[rows], layer.scales.cpu()[rows], layer.zeros.cpu()[rows], 8, b)
    for m in (32, 64, 128, 256):
        x = synth.make_activations(m, n_in, seed=m, dtype=torch.bfloat16, device=cuda)
        y = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, 128, flag)
        assert _status_ok()
        y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
        assert oracle.rel_err(y.cpu()[:, rows], y_ref) <= TOL, f"M={m}"
        assert oracle.elementwise_err(y.cpu()[:, rows], y_ref, rtol=1e-2, atol_rms=2e-2) <= 1.0, f"M={m}"


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("gs", [-1, 32, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dense_tile_is_bit_exact(cuda, b, gs, dtype):
    """The weights the tensor-core path builds in shared memory, read back through the product itself: with
    one-hot activation rows (row i = unit vector k0 + i) every output is a single weight times one, so
    y[i, n] must equal dequantize()[n, k0 + i] bit for bit (fp32 accumulation of one term, exact rounding).
    With one scale per row (gs == -1) the kernel scales the fp32 sum instead: still one rounding."""
    from matgptq_b200 import ops
    n_out, n_in, m = 256, 512, 256
    layer = synth.make_layer(n_out, n_in, gs, seed=40 + b, sym=True, dtype=dtype, device=cuda)
    packed, scales_r, flag = _pack(layer, n_out, n_in, gs, b, dtype)
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    for k0 in (0, 256):
        x = torch.zeros(m, n_in, dtype=dtype, device=cuda)
        x[torch.arange(m), k0 + torch.arange(m)] = 1.0
        y = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, gs, flag, path=2)
        assert _status_ok()
        assert torch.equal(y.cpu(), w_ref[:, k0:k0 + m].t().contiguous()), f"k0={k0}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dense_tile_scale_edges_b2(cuda, dtype):
    """b = 2 folds a factor two into the scale.  A finite scale whose double leaves the finite range must
    still give dequantize()'s weight for the code on the zero point: exactly zero (the doubled scale is
    clamped to the largest finite value; an infinite one would turn 0 * scale into NaN).  Groups with such
    scales hold only that code here, because any other code times such a scale is infinite in dequantize()
    too and an infinite weight cannot be read back through a product.  Tiny, negative and zero scales ride
    along with random codes."""
    from matgptq_b200 import ops
    n_out, n_in, m, b = 128, 256, 256, 2
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    big = torch.finfo(dtype).max
    tiny = torch.finfo(dtype).tiny
    edge = torch.tensor([big, -big, big / 1.5, 0.0, -0.0, tiny, tiny / 4, -3.0, 1.0, 6e-5], dtype=torch.float32).to(dtype)
    scales = edge[torch.arange(n_out * 2) % len(edge)].reshape(n_out, 2).contiguous()
    g = torch.Generator().manual_seed(3)
    q = torch.randint(0, 256, (n_out, n_in), dtype=torch.uint8, generator=g)
    huge = (scales.float().abs() * 2 > big).repeat_interleave(128, dim=1)
    assert huge.any() and not huge.all()
    q[huge] = 128  # slices to code 2 = the implicit zero point of 2-bit codes
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(q.to(cuda), n_out, n_in, 8, b, 128, flag)
    scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(scales.to(cuda), n_out, n_in, 128)
    w_ref = oracle.dequantize_weight(q, scales, torch.full_like(scales, 128.0), 8, b)
    assert torch.isfinite(w_ref.float()).all() and (w_ref[huge] == 0).all()
    x = torch.zeros(m, n_in, dtype=dtype, device=cuda)
    x[torch.arange(m), torch.arange(m)] = 1.0
    y = ops.matmul_matgptq_raw(x, packed, scales_r, n_out, n_in, b, 128, flag, path=2)
    assert _status_ok()
    assert torch.equal(y.cpu().t().contiguous(), w_ref)
