"""Load-time kernels on the GPU against the oracle and the host twins (bit-exact)."""
import numpy as np
import pytest
import torch

from oracle import matgptq_oracle as oracle

pytestmark = pytest.mark.gpu
BITS = (2, 3, 4, 6, 8)


def _stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("master", [8])
@pytest.mark.parametrize("numel", [0, 1, 255, 256, 4096 + 3, 1 << 20])
def test_slice_kernel(lib, cuda, b, master, numel):
    g = torch.Generator().manual_seed(numel + b)
    x = torch.randint(0, 256, (numel,), dtype=torch.uint8, generator=g)
    if numel >= 256:
        x[:256] = torch.arange(256, dtype=torch.uint8)
    xd = x.to(cuda)
    out = torch.full_like(xd, 77)
    assert lib.matgptq_b200_slice(xd.data_ptr(), out.data_ptr(), numel, master, b, _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), oracle.matryoshka_slice(x, master, b))


def test_slice_kernel_unaligned_and_in_place(lib, cuda):
    x = torch.randint(0, 256, (10001,), dtype=torch.uint8)
    xd = x.to(cuda)
    view = xd[1:]  # not 16-byte aligned
    assert lib.matgptq_b200_slice(view.data_ptr(), view.data_ptr(), view.numel(), 8, 3, _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(view.cpu(), oracle.matryoshka_slice(x[1:], 8, 3))
    assert xd[0].item() == x[0].item()


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("shape", [(16, 128), (80, 640), (1024, 4096)])
@pytest.mark.parametrize("fused", [0, 8])
def test_gpu_pack_equals_host_pack(lib, cuda, b, shape, fused):
    n, k = shape
    g = torch.Generator().manual_seed(n + k + b)
    hi = 256 if fused else 2 ** b
    codes = torch.randint(0, hi, (n, k), dtype=torch.uint8, generator=g)
    host = np.zeros(b * n * k // 32, dtype=np.uint32)
    cn = codes.numpy()
    assert lib.matgptq_b200_pack_qweights_host(cn.ctypes.data, host.ctypes.data, n, k, b, fused) == 0
    cd = codes.to(cuda)
    dev = torch.zeros(b * n * k // 32, dtype=torch.uint32, device=cuda)
    assert lib.matgptq_b200_pack_qweights(cd.data_ptr(), dev.data_ptr(), n, k, b, fused, _stream()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(dev.cpu().numpy(), host)
    # and the packed words decode back to the (sliced) codes
    back = np.zeros((n, k), dtype=np.uint8)
    assert lib.matgptq_b200_unpack_qweights_host(host.ctypes.data, back.ctypes.data, n, k, b) == 0
    want = oracle.matryoshka_slice_np(cn, 8, b) if fused else cn
    assert np.array_equal(back, want)


@pytest.mark.parametrize("gs", [-1, 32, 128])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_reorder_scales_op(cuda, gs, dtype):
    from matgptq_b200 import ops  # noqa: F401
    n, k = 64, 1024
    groups = 1 if gs == -1 else k // gs
    s = torch.randn(n, groups).to(dtype)
    out = torch.ops.matgptq_cuda.reorder_matgptq_scales(s, n, k, gs)
    assert out.is_cuda and out.shape == s.shape and out.dtype == dtype
    want = s.reshape(n // 16, 16, groups).transpose(1, 2).reshape(n, groups)
    assert torch.equal(out.cpu(), want)
    # same result from a CUDA input
    out2 = torch.ops.matgptq_cuda.reorder_matgptq_scales(s.to(cuda), n, k, gs)
    assert torch.equal(out2, out)


def test_pack_op_contract(cuda):
    from matgptq_b200 import ops  # noqa: F401
    q = torch.randint(0, 16, (32, 256), dtype=torch.uint8)
    p_cpu_in = torch.ops.matgptq_cuda.pack_matgptq_qweights(q, 32, 256, 4, 128, 1)
    p_gpu_in = torch.ops.matgptq_cuda.pack_matgptq_qweights(q.to(cuda), 32, 256, 4, 128, 1)
    assert p_cpu_in.is_cuda and p_cpu_in.dtype == torch.uint32 and p_cpu_in.dim() == 1
    assert p_cpu_in.numel() == 4 * 32 * 256 // 32
    assert torch.equal(p_cpu_in, p_gpu_in)
    master = torch.randint(0, 256, (32, 256), dtype=torch.uint8)
    fused = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(master, 32, 256, 8, 3, 128, 1)
    two = torch.ops.matgptq_cuda.pack_matgptq_qweights(oracle.matryoshka_slice(master, 8, 3), 32, 256, 3, 128, 1)
    assert torch.equal(fused, two)


@pytest.mark.parametrize("code", [101, 102, 103])
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(lib, cuda, code):
    """Bounded waits: one warp waits on a barrier that nothing completes; the wait gives up, the status word
    carries the code, reading it clears it, and kernels launched afterwards work."""
    from matgptq_b200 import _native
    assert _native.device_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device=cuda)
    st = lib.matgptq_b200_selftest_wait_timeout(code, flag.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    assert _native.device_status(reset=False) == code   # synchronises; the kernel has ended by itself
    assert int(flag.item()) == 1
    assert _native.device_status(reset=True) == code
    assert _native.device_status() == 0
    assert lib.matgptq_b200_selftest_wait_timeout(7, None, None) == 1  # not one of the wait codes
    # the context is intact: a real launch right after
    x = torch.arange(256, dtype=torch.uint8, device=cuda)
    out = torch.empty_like(x)
    assert lib.matgptq_b200_slice(x.data_ptr(), out.data_ptr(), 256, 8, 4, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert int(out.max()) == 15


def test_runtime_bitwidth_switch_from_resident_master(cuda):
    """One resident copy of the 8-bit master codes serves every bitwidth: set_bitwidth re-slices and re-packs on
    the GPU, and after every switch the layer computes what the oracle computes at that bitwidth."""
    from matgptq_b200 import synth
    from matgptq_b200.matgptq_linear import MatGPTQLinear
    n_out, n_in = 512, 1024
    layer = synth.make_layer(n_out, n_in, 128, seed=2, sym=True, dtype=torch.float16, device=cuda)
    lin = MatGPTQLinear.from_master(layer.qweight, layer.scales, 8, 8, 128, keep_master=True)
    x = synth.make_activations(5, n_in, seed=3, dtype=torch.float16, device=cuda)
    for b in (8, 2, 4, 3, 6, 8):
        lin.set_bitwidth(b)
        assert lin.bitwidth == b and lin.matgptq_qweight.numel() == b * n_out * n_in // 32
        w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
        assert oracle.rel_err(lin(x).cpu(), oracle.linear_fp32_accumulate(x.cpu(), w_ref)) <= 1e-2
    plain = MatGPTQLinear.from_master(layer.qweight, layer.scales, 8, 4, 128)
    with pytest.raises(RuntimeError, match="keep_master"):
        plain.set_bitwidth(2)
