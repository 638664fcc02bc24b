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
    from matgptq_b200 import ops
    assert lib.matgptq_b200_matmul_workspace_bytes(4096, 4096, 16) == 0      # GEMV family: no scratch
    need = lib.matgptq_b200_matmul_workspace_bytes(1024, 4096, 64)           # 8 tiles only: K is split
    assert need > 0 and need % (64 * 1024 * 4) == 0
    n_in, n_out, b, m = 4096, 1024, 3, 64
    layer = synth.make_layer(n_out, n_in, 128, seed=1, sym=True, dtype=torch.bfloat16, device=cuda)
    packed, scales_r, flag = _pack(layer, n_out, n_in, 128, b, torch.bfloat16)
    x = synth.make_activations(m, n_in, seed=1, dtype=torch.bfloat16, device=cuda)
    y_split = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales_r, n_out, n_in, b, 128, flag)
    # no scratch: the plain entry point runs without a K split and must agree
    y_plain = torch.empty_like(y_split)
    st = lib.matgptq_b200_matmul(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(), x.data_ptr(),
                                 y_plain.data_ptr(), torch.cuda.current_stream().cuda_stream, flag)
    assert st == 0
    torch.cuda.synchronize()
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
    assert oracle.rel_err(y_split.cpu(), y_ref) <= TOL and oracle.rel_err(y_plain.cpu(), y_ref) <= TOL
    # a forced split without enough scratch is an argument error, not a silent fallback
    small = torch.empty(16, dtype=torch.uint8, device=cuda)
    st = lib.matgptq_b200_matmul_ws(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(), x.data_ptr(),
                                    y_plain.data_ptr(), torch.cuda.current_stream().cuda_stream, flag,
                                    small.data_ptr(), 16, 2, 4)
    assert st == 1
