"""Dequantised weights from the packed layout: bit-exact against the oracle for every bitwidth."""
import numpy as np
import pytest
import torch

from oracle import matgptq_oracle as oracle

pytestmark = pytest.mark.gpu
BITS = (2, 3, 4, 6, 8)


def _bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _reorder(t, n, k, gs):
    return torch.ops.matgptq_cuda.reorder_matgptq_scales(t.contiguous(), n, k, gs)


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("gs", [-1, 32, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dequant_symmetric_bit_exact(cuda, b, gs, dtype):
    from matgptq_b200 import ops  # noqa: F401
    n, k = 64, 512
    g = torch.Generator().manual_seed(b * 100 + (gs % 11))
    master = torch.randint(0, 256, (n, k), dtype=torch.uint8, generator=g)
    master[0, :256] = torch.arange(256, dtype=torch.uint8)
    groups = 1 if gs == -1 else k // gs
    scales = (torch.rand(n, groups, generator=g) * 0.02 + 1e-4).to(dtype)
    # edges: product subnormal, zero scale, negative scale, large scale
    scales[0, 0] = 6e-8 if dtype == torch.float16 else 1e-38
    scales[1, 0] = 0.0
    scales[2, 0] = -0.013
    scales[3, 0] = 400.0 if dtype == torch.float16 else 3e36
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(master, n, k, 8, b, gs, flag)
    w = torch.ops.matgptq_cuda.dequantize_matgptq(packed, _reorder(scales, n, k, gs), n, k, b, gs, flag)
    want = oracle.dequantize_weight(master, scales, torch.full_like(scales, 128.0), 8, b)
    assert w.dtype == dtype
    assert np.array_equal(_bits(w), _bits(want))


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("dname,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
@pytest.mark.parametrize("mode", ["asym", "sym"])
def test_dequant_golden_vectors(lib, cuda, golden, b, dname, dtype, mode):
    """The vectors recorded from the reference's dequantize(), through the GPU path (with zero points)."""
    from matgptq_b200 import ops  # noqa: F401
    q = torch.from_numpy(golden["dq_q"])                       # [16, 3, 128]
    n, groups, gs = q.shape
    k = groups * gs
    scale = torch.from_numpy(golden[f"dq_scale_{dname}"].view(np.int16).copy()).view(dtype).reshape(n, groups)
    if mode == "asym":
        zero = torch.from_numpy(golden[f"dq_zero_asym_{dname}"].view(np.int16).copy()).view(dtype).reshape(n, groups)
    else:
        zero = torch.full_like(scale, 128.0)
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(q.reshape(n, k).contiguous(), n, k, 8, b, gs, flag)
    s_r = _reorder(scale, n, k, gs)
    z_r = _reorder(zero, n, k, gs)
    out = torch.empty(n, k, dtype=dtype, device=cuda)
    st = lib.matgptq_b200_dequantize(packed.data_ptr(), s_r.data_ptr(), z_r.data_ptr(), out.data_ptr(), n, k, b, gs,
                                     flag, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    want = golden[f"dq_{mode}_{dname}_b{b}"].reshape(n, k)
    assert np.array_equal(_bits(out), want)


@pytest.mark.parametrize("b", BITS)
def test_dequant_fake_linear_golden(lib, cuda, golden, b):
    from matgptq_b200 import ops  # noqa: F401
    q = torch.from_numpy(golden["fl_q"])
    n, k = q.shape
    sc = torch.from_numpy(golden["fl_scale"])
    zp = torch.from_numpy(golden["fl_zero"])
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(q, n, k, 8, b, 128, 1)
    out = torch.empty(n, k, dtype=torch.float16, device=cuda)
    s_r, z_r = _reorder(sc, n, k, 128), _reorder(zp, n, k, 128)  # keep alive across the raw-pointer call
    st = lib.matgptq_b200_dequantize(packed.data_ptr(), s_r.data_ptr(), z_r.data_ptr(), out.data_ptr(), n, k, b, 128, 1,
                                     torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), golden[f"fl_w_b{b}"])
