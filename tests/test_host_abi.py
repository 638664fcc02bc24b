"""C-ABI library on the CPU: it loads, exports what the header declares, and its host packer
inverts itself.  No kernel is launched here."""
import os
import re

import numpy as np
import pytest

from oracle import matgptq_oracle as oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BITS = (2, 3, 4, 6, 8)


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "matgptq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(matgptq_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from matgptq_b200 import _native
    names = _declared_functions()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/matgptq_b200.h but not exported"
        assert name in _native.SIGNATURES, f"{name} has no ctypes signature"
    assert lib.matgptq_b200_version() >= 100
    assert lib.matgptq_b200_strerror(0) == b"ok"


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("shape", [(16, 128), (48, 384), (128, 1024)])
def test_host_pack_roundtrip(lib, b, shape):
    n, k = shape
    rng = np.random.default_rng(b * 1000 + n)
    codes = rng.integers(0, 2 ** b, (n, k), dtype=np.uint8)
    packed = np.zeros(b * n * k // 32, dtype=np.uint32)
    assert lib.matgptq_b200_pack_qweights_host(codes.ctypes.data, packed.ctypes.data, n, k, b, 0) == 0
    back = np.full_like(codes, 255)
    assert lib.matgptq_b200_unpack_qweights_host(packed.ctypes.data, back.ctypes.data, n, k, b) == 0
    assert np.array_equal(back, codes)
    # every packed bit is a code bit: nothing is stored twice and nothing is lost
    assert int(np.unpackbits(packed.view(np.uint8)).sum()) == int(np.unpackbits(codes).sum())


@pytest.mark.parametrize("b", BITS)
def test_host_pack_extreme_codes(lib, b):
    n, k = 16, 128
    for fill in (0, 2 ** b - 1):
        codes = np.full((n, k), fill, dtype=np.uint8)
        packed = np.zeros(b * n * k // 32, dtype=np.uint32)
        assert lib.matgptq_b200_pack_qweights_host(codes.ctypes.data, packed.ctypes.data, n, k, b, 0) == 0
        assert (packed == (0 if fill == 0 else 0xFFFFFFFF)).all()


@pytest.mark.parametrize("b", BITS)
def test_host_fused_slice_equals_oracle_slice(lib, b):
    n, k = 32, 256
    rng = np.random.default_rng(b)
    master = rng.integers(0, 256, (n, k), dtype=np.uint8)
    master[0, :256] = np.arange(256, dtype=np.uint8)  # every byte value
    fused = np.zeros(b * n * k // 32, dtype=np.uint32)
    assert lib.matgptq_b200_pack_qweights_host(master.ctypes.data, fused.ctypes.data, n, k, b, 8) == 0
    sliced = oracle.matryoshka_slice_np(master, 8, b)
    two_step = np.zeros_like(fused)
    assert lib.matgptq_b200_pack_qweights_host(sliced.ctypes.data, two_step.ctypes.data, n, k, b, 0) == 0
    assert np.array_equal(fused, two_step)


@pytest.mark.parametrize("gs", [-1, 32, 128])
def test_host_reorder_scales(lib, gs):
    n, k = 48, 512
    groups = 1 if gs == -1 else k // gs
    s = np.arange(n * groups, dtype=np.uint16).reshape(n, groups)
    out = np.zeros_like(s)
    assert lib.matgptq_b200_reorder_scales_host(s.ctypes.data, out.ctypes.data, n, k, gs) == 0
    want = s.reshape(n // 16, 16, groups).transpose(0, 2, 1).reshape(n, groups)
    assert np.array_equal(out, want)


def test_bad_arguments_return_status_codes(lib):
    buf = np.zeros(16 * 128, dtype=np.uint8)
    out = np.zeros(16 * 128, dtype=np.uint32)
    p, q = buf.ctypes.data, out.ctypes.data
    assert lib.matgptq_b200_pack_qweights_host(p, q, 16, 128, 5, 0) == 1      # bitwidth
    assert lib.matgptq_b200_pack_qweights_host(p, q, 15, 128, 4, 0) == 1      # N % 16
    assert lib.matgptq_b200_pack_qweights_host(p, q, 16, 100, 4, 0) == 1      # K % 64
    assert lib.matgptq_b200_pack_qweights_host(p, q, 16, 192, 4, 0) == 3      # K % 128 == 64: unsupported
    assert lib.matgptq_b200_pack_qweights_host(None, q, 16, 128, 4, 0) == 1   # null pointer
    assert lib.matgptq_b200_reorder_scales_host(p, q, 16, 128, 64) == 1       # group size
    assert lib.matgptq_b200_matmul(4, 128, 16, 128, 1, None, None, None, None, None, 1) == 1
    assert lib.matgptq_b200_matmul(4, 128, 16, 128, 0, None, None, None, None, None, 1) == 0  # empty batch: nothing to do
    for code in range(5):
        assert len(lib.matgptq_b200_strerror(code)) > 0


def test_operator_checks_raise_without_gpu():
    import torch
    from matgptq_b200 import ops  # noqa: F401
    q = torch.zeros(16, 128, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="bitwidth"):
        torch.ops.matgptq_cuda.pack_matgptq_qweights(q, 16, 128, 5, 128, 1)
    with pytest.raises(RuntimeError, match="uint8"):
        torch.ops.matgptq_cuda.pack_matgptq_qweights(q.float(), 16, 128, 4, 128, 1)
    with pytest.raises(RuntimeError, match="n_out_features"):
        torch.ops.matgptq_cuda.pack_matgptq_qweights(q, 32, 128, 4, 128, 1)
    with pytest.raises(RuntimeError, match="group_size"):
        torch.ops.matgptq_cuda.reorder_matgptq_scales(torch.zeros(16, 2, dtype=torch.float16), 16, 128, 64)
    if not torch.cuda.is_available():
        # no silent CPU path: the operator refuses to run without a CUDA device
        with pytest.raises(RuntimeError, match="CUDA"):
            torch.ops.matgptq_cuda.pack_matgptq_qweights(q, 16, 128, 4, 128, 1)


def test_fake_tensor_shapes():
    import torch
    from matgptq_b200 import ops  # noqa: F401
    x = torch.empty(3, 5, 128, dtype=torch.float16, device="meta")
    w = torch.empty(4 * 16 * 128 // 32, dtype=torch.uint32, device="meta")
    s = torch.empty(16, 1, dtype=torch.float16, device="meta")
    y = torch.ops.matgptq_cuda.matmul_matgptq(x, w, s, 16, 128, 4, 128, 1)
    assert y.shape == (5, 16) and y.dtype == torch.float16
    y = torch.ops.matgptq_cuda.matmul_matgptq(x.bfloat16(), w, s.bfloat16(), 16, 128, 4, 128, 3)
    assert y.dtype == torch.bfloat16
