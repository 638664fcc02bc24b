"""The CPU oracle against vectors recorded from the reference's own code (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import matgptq_oracle as oracle

BITS = (2, 3, 4, 6, 8)


def _from_bits(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(dtype)


@pytest.mark.parametrize("b", BITS)
def test_slice_table(golden, b):
    allbytes = np.arange(256, dtype=np.uint8)
    want = golden[f"slice_m8_b{b}"]
    assert np.array_equal(oracle.matryoshka_slice_np(allbytes, 8, b), want)
    assert np.array_equal(oracle.matryoshka_slice(torch.from_numpy(allbytes), 8, b).numpy(), want)


def test_slice_non8_master(golden):
    allbytes = np.arange(256, dtype=np.uint8)
    assert np.array_equal(oracle.matryoshka_slice_np(allbytes, 4, 4), golden["slice_m4_b4"])
    assert np.array_equal(oracle.matryoshka_slice_np(allbytes, 6, 4), golden["slice_m6_b4"])


def test_slice_known_answers():
    # b=2 maps 0..31 -> 0, 32..95 -> 1, 96..159 -> 2, 160..255 -> 3 (224..255 would round to 4 and saturate)
    x = np.arange(256, dtype=np.uint8)
    s = oracle.matryoshka_slice_np(x, 8, 2)
    assert (s[:32] == 0).all() and (s[32:96] == 1).all() and (s[96:160] == 2).all() and (s[160:] == 3).all()
    assert np.array_equal(oracle.matryoshka_slice_np(x, 8, 8), x)


@pytest.mark.parametrize("dname,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("mode", ["asym", "sym"])
def test_dequantize_bit_exact(golden, dname, dtype, b, mode):
    q = torch.from_numpy(golden["dq_q"])
    scale = _from_bits(golden[f"dq_scale_{dname}"], dtype)
    if mode == "asym":
        zero = _from_bits(golden[f"dq_zero_asym_{dname}"], dtype)
    else:
        zero = torch.full_like(scale, 128.0)
    got = oracle.dequantize(q, scale, zero, 8, b)
    assert got.dtype == dtype
    want = golden[f"dq_{mode}_{dname}_b{b}"]
    assert np.array_equal(got.contiguous().view(torch.int16).numpy().view(np.uint16), want)


@pytest.mark.parametrize("b", BITS)
def test_fake_linear(golden, b):
    q = torch.from_numpy(golden["fl_q"])
    sc = torch.from_numpy(golden["fl_scale"])
    zp = torch.from_numpy(golden["fl_zero"])
    x = torch.from_numpy(golden["fl_x"])
    w = oracle.dequantize_weight(q, sc, zp, 8, b)
    assert np.array_equal(w.numpy(), golden[f"fl_w_b{b}"])
    y = oracle.fake_matryoshka_linear(x, q, sc, zp, 8, b)
    assert np.array_equal(y.numpy(), golden[f"fl_y_b{b}"])


@pytest.mark.parametrize("b", BITS)
@pytest.mark.parametrize("gs", [-1, 32, 128])
def test_op_weight_equals_dequantize_with_zero_128(b, gs):
    # the three-op path implies zero = 128 in master units: its weight formula
    # (test_matgptq_matmul.py:40) must agree with dequantize() on sliced codes
    g = torch.Generator().manual_seed(b * 10 + (gs % 7))
    n, k = 16, 256
    master = torch.randint(0, 256, (n, k), dtype=torch.uint8, generator=g)
    groups = 1 if gs == -1 else k // gs
    scales = (torch.rand(n, groups, generator=g) * 0.01 + 1e-3).half()
    sliced = oracle.matryoshka_slice(master, 8, b)
    w_op = oracle.op_dequantized_weight(sliced, scales, b, gs)
    w_ref = oracle.dequantize_weight(master, scales, torch.full_like(scales, 128.0), 8, b)
    assert torch.equal(w_op.half(), w_ref)


@pytest.mark.parametrize("sym", [False, True])
def test_minmax_and_rtn(golden, sym):
    tag = "sym" if sym else "asym"
    w = torch.from_numpy(golden["mm_w"]).reshape(-1, 128)
    scale, zero = oracle.minmax_params(w, 8, sym)
    assert np.array_equal(scale.numpy(), golden[f"mm_scale_{tag}"])
    assert np.array_equal(zero.numpy(), golden[f"mm_zero_{tag}"])
    codes = oracle.rtn_quantize(w, scale, zero, 255)
    assert np.array_equal(codes.numpy(), golden[f"mm_codes_{tag}"])
