"""The three operators of the reference's ``matgptq_cuda`` package, on the B200 library.

Same names, schemas and argument meaning as ``inference_lib/matgptq_cuda/__init__.py:5-63``
(Python custom ops) and ``csrc/bindings.cpp:43-191,197-207`` (checks, allocation,
stream): ``torch.ops.matgptq_cuda.{pack_matgptq_qweights, reorder_matgptq_scales,
matmul_matgptq}``.  PyTorch supplies device memory and the current stream; the
work is done by ``libmatgptq_b200.so`` through its C ABI.  Two additions sit beside
them: ``slice_pack_matgptq_qweights`` (slicing fused into packing) and
``dequantize_matgptq`` (dense weights for checks).
"""
from __future__ import annotations

import torch

from . import _native

_lib = _native.load()

_BITWIDTHS = (2, 3, 4, 6, 8)
_GROUPS = (-1, 32, 128)


def _check_common(bitwidth: int, group_size: int, n_in_features: int) -> None:
    # csrc/bindings.cpp:55-59
    if bitwidth not in _BITWIDTHS:
        raise RuntimeError("bitwidth must be one of {2, 3, 4, 6, 8}")
    if group_size not in _GROUPS:
        raise RuntimeError("group_size must be one of {-1, 32, 128}")
    if group_size != -1 and n_in_features % group_size != 0:
        raise RuntimeError(
            f"group_size must divide n_in_features. Got group_size={group_size}, n_in_features={n_in_features}")


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _cuda_device_of(t: torch.Tensor) -> torch.device:
    if t.is_cuda:
        return t.device
    if not torch.cuda.is_available():
        raise RuntimeError("matgptq_b200 needs a CUDA device: there is no CPU implementation of this operator")
    return torch.device("cuda", torch.cuda.current_device())


def _pack_impl(qweights: torch.Tensor, n_out_features: int, n_in_features: int, bitwidth: int,
               group_size: int, slice_from_master: int) -> torch.Tensor:
    # csrc/bindings.cpp:50-59
    if qweights.dtype != torch.uint8:
        raise RuntimeError("qweights must be uint8")
    if not qweights.is_contiguous():
        raise RuntimeError("qweights must be contiguous")
    if qweights.dim() != 2:
        raise RuntimeError("qweights must be 2D (n_out_features, n_in_features)")
    if qweights.size(0) != n_out_features:
        raise RuntimeError("n_out_features does not match qweights.size(0)")
    if qweights.size(1) != n_in_features:
        raise RuntimeError("n_in_features does not match qweights.size(1)")
    _check_common(bitwidth, group_size, n_in_features)
    dev = _cuda_device_of(qweights)
    with torch.cuda.device(dev):
        codes = qweights.to(dev, non_blocking=True)
        packed = torch.empty(bitwidth * n_out_features * n_in_features // 32, dtype=torch.uint32, device=dev)
        st = _lib.matgptq_b200_pack_qweights(codes.data_ptr(), packed.data_ptr(), n_out_features, n_in_features,
                                             bitwidth, slice_from_master, _stream_ptr(dev))
        _native.check(st, "pack_matgptq_qweights")
        if codes is not qweights:
            codes.record_stream(torch.cuda.current_stream(dev))
    return packed


@torch.library.custom_op("matgptq_cuda::pack_matgptq_qweights", mutates_args=())
def pack_matgptq_qweights(
    qweights: torch.Tensor,
    n_out_features: int,
    n_in_features: int,
    bitwidth: int,
    group_size: int,
    feature_flag: int,
) -> torch.Tensor:
    """Pack already-sliced b-bit codes ``[N, K]`` (uint8, CPU or CUDA) into the 1-D
    uint32 CUDA tensor of ``b*N*K/32`` words that ``matmul_matgptq`` reads."""
    return _pack_impl(qweights, n_out_features, n_in_features, bitwidth, group_size, 0)


@pack_matgptq_qweights.register_fake
def _pack_fake(qweights, n_out_features, n_in_features, bitwidth, group_size, feature_flag):
    return qweights.new_empty((bitwidth * n_out_features * n_in_features // 32,), dtype=torch.uint32)


@torch.library.custom_op("matgptq_cuda::slice_pack_matgptq_qweights", mutates_args=())
def slice_pack_matgptq_qweights(
    qweights: torch.Tensor,
    n_out_features: int,
    n_in_features: int,
    master_bitwidth: int,
    bitwidth: int,
    group_size: int,
    feature_flag: int,
) -> torch.Tensor:
    """``pack_matgptq_qweights(matryoshka_slice(qweights, master_bitwidth, bitwidth), ...)`` in one
    pass over the master codes (the two steps of ``vllm_matgptq.py:152-166``)."""
    if not (bitwidth <= master_bitwidth <= 8):
        raise RuntimeError("need bitwidth <= master_bitwidth <= 8")
    return _pack_impl(qweights, n_out_features, n_in_features, bitwidth, group_size, master_bitwidth)


@slice_pack_matgptq_qweights.register_fake
def _slice_pack_fake(qweights, n_out_features, n_in_features, master_bitwidth, bitwidth, group_size, feature_flag):
    return qweights.new_empty((bitwidth * n_out_features * n_in_features // 32,), dtype=torch.uint32)


def _reorder_impl(scales: torch.Tensor, m: int, n: int, group_size: int) -> torch.Tensor:
    # csrc/bindings.cpp:92-97
    if not scales.is_contiguous():
        raise RuntimeError("scales must be contiguous")
    if scales.dim() != 2:
        raise RuntimeError("scales must be 2D (n_out_features, n_groups)")
    if scales.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("scales must be float16 or bfloat16")
    _check_common(8, group_size, n)
    groups = 1 if group_size == -1 else n // group_size
    if scales.size(0) != m or scales.size(1) != groups:
        raise RuntimeError(f"scales must have shape ({m}, {groups})")
    dev = _cuda_device_of(scales)
    with torch.cuda.device(dev):
        src = scales.to(dev, non_blocking=True)
        out = torch.empty_like(src)
        st = _lib.matgptq_b200_reorder_scales(src.data_ptr(), out.data_ptr(), m, n, group_size, _stream_ptr(dev))
        _native.check(st, "reorder_matgptq_scales")
        if src is not scales:
            src.record_stream(torch.cuda.current_stream(dev))
    return out


@torch.library.custom_op("matgptq_cuda::reorder_matgptq_scales", mutates_args=())
def reorder_matgptq_scales(scales: torch.Tensor, m: int, n: int, group_size: int) -> torch.Tensor:
    """Reorder scales ``[N, G]`` for the kernels; same shape and dtype, on CUDA
    (``m`` = out features, ``n`` = in features, as in the reference)."""
    return _reorder_impl(scales, m, n, group_size)


@reorder_matgptq_scales.register_fake
def _reorder_fake(scales, m, n, group_size):
    return torch.empty_like(scales)


def _check_matmul_args(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidth, group_size):
    # csrc/bindings.cpp:155-168
    for name, t in (("input", input), ("matgptq_weights", matgptq_weights), ("matgptq_scales", matgptq_scales)):
        if not t.is_cuda:
            raise RuntimeError(f"matmul_matgptq: expected {name} to be a CUDA tensor")
    if not (input.device == matgptq_weights.device == matgptq_scales.device):
        raise RuntimeError("matmul_matgptq: input, matgptq_weights and matgptq_scales must be on the same GPU")
    if matgptq_weights.dtype != torch.uint32:
        raise RuntimeError("matgptq_weights must be uint32")
    if not matgptq_weights.is_contiguous():
        raise RuntimeError("matgptq_weights must be contiguous")
    if matgptq_weights.dim() != 1:
        raise RuntimeError("qweights must be 1D")
    if matgptq_weights.size(0) != bitwidth * n_out_features * n_in_features // 32:
        raise RuntimeError("matgptq_weights has the wrong size")
    _check_common(bitwidth, group_size, n_in_features)
    if input.dim() < 2 or input.size(-1) != n_in_features:
        raise RuntimeError("input must have shape [..., M, n_in_features]")


def _launch_matmul(what: str, dev, bitwidth: int, group_size: int, n_out_features: int, n_in_features: int, batch: int,
                   weights: torch.Tensor, scales: torch.Tensor, x: torch.Tensor, out: torch.Tensor, feature_flag: int) -> None:
    """One call of the C-ABI product.  Scratch is only allocated when it is used: with FLAG_SCRATCH_REDUCE, or for
    the second attempt on a device that could not place the thread-block cluster of a split K."""
    def call(ws):
        return _lib.matgptq_b200_matmul_ws(bitwidth, group_size, n_out_features, n_in_features, batch,
                                           weights.data_ptr(), scales.data_ptr(), x.data_ptr(), out.data_ptr(),
                                           _stream_ptr(dev), feature_flag,
                                           ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, 0, 0)

    def scratch():
        need = _lib.matgptq_b200_matmul_workspace_bytes(n_out_features, n_in_features, batch)
        return torch.empty(need, dtype=torch.uint8, device=dev) if need > 0 else None

    st = call(scratch() if feature_flag & _native.FLAG_SCRATCH_REDUCE else None)
    if st == _native.ERR_CUDA and not feature_flag & _native.FLAG_SCRATCH_REDUCE:
        ws = scratch()
        if ws is not None:
            st = call(ws)
    _native.check(st, what)


def _prepare_input(input: torch.Tensor, batch: int, n_in_features: int) -> torch.Tensor:
    x = input
    if input.dim() > 2:
        # the reference reads the last two dimensions only (csrc/bindings.cpp:171)
        x = input.reshape(-1, batch, n_in_features)[0]
    if not x.is_contiguous():
        x = x.contiguous()
    if x.data_ptr() % 16 != 0:
        x = x.clone()
    return x


def _matmul_impl(input: torch.Tensor, matgptq_weights: torch.Tensor, matgptq_scales: torch.Tensor, n_out_features: int,
                 n_in_features: int, bitwidth: int, group_size: int, feature_flag: int) -> torch.Tensor:
    _check_matmul_args(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidth, group_size)
    bf16 = bool(feature_flag & _native.FLAG_BF16)
    dtype = torch.bfloat16 if bf16 else torch.float16
    if input.dtype != dtype or matgptq_scales.dtype != dtype:
        raise RuntimeError(f"input and matgptq_scales must be {dtype} for feature_flag={feature_flag}")
    dev = matgptq_weights.device
    batch = input.size(-2)
    x = _prepare_input(input, batch, n_in_features)
    with torch.cuda.device(dev):
        out = torch.empty((batch, n_out_features), dtype=dtype, device=dev)
        _launch_matmul("matmul_matgptq", dev, bitwidth, group_size, n_out_features, n_in_features, batch,
                       matgptq_weights, matgptq_scales, x, out, feature_flag)
    return out


@torch.library.custom_op("matgptq_cuda::matmul_matgptq", mutates_args=())
def matmul_matgptq(
    input: torch.Tensor,
    matgptq_weights: torch.Tensor,
    matgptq_scales: torch.Tensor,
    n_out_features: int,
    n_in_features: int,
    bitwidth: int,
    group_size: int,
    feature_flag: int,
) -> torch.Tensor:
    """``y[M, N] = x[M, K] @ Wdq.T`` for packed b-bit weights; ``M = input.size(-2)``.
    Output is float16, or bfloat16 when ``feature_flag & 2``."""
    return _matmul_impl(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidth, group_size,
                        feature_flag)


@matmul_matgptq.register_fake
def _matmul_fake(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidth, group_size,
                 feature_flag):
    # inference_lib/matgptq_cuda/__init__.py:49-63
    return input.new_empty((input.shape[-2], n_out_features),
                           dtype=torch.bfloat16 if feature_flag & 2 else torch.float16)


@torch.library.custom_op("matgptq_cuda::matmul_matgptq_out", mutates_args=("out",))
def matmul_matgptq_out(
    input: torch.Tensor,
    matgptq_weights: torch.Tensor,
    matgptq_scales: torch.Tensor,
    n_out_features: int,
    n_in_features: int,
    bitwidth: int,
    group_size: int,
    feature_flag: int,
    out: torch.Tensor,
) -> None:
    """``matmul_matgptq`` into a tensor the caller owns (``out [M, N]``, contiguous, float16 or bfloat16 like the
    input): nothing is allocated, which is what callers that gather several layers' outputs in one buffer, or that
    capture the call in a CUDA graph with their own memory plan, want.  The reference's operator only has the
    allocating form (csrc/bindings.cpp:158-201)."""
    _check_matmul_args(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidth, group_size)
    dtype = torch.bfloat16 if feature_flag & _native.FLAG_BF16 else torch.float16
    if input.dtype != dtype or matgptq_scales.dtype != dtype:
        raise RuntimeError(f"input and matgptq_scales must be {dtype} for feature_flag={feature_flag}")
    batch = input.size(-2)
    dev = matgptq_weights.device
    if (out.dtype != dtype or out.device != dev or tuple(out.shape) != (batch, n_out_features) or not out.is_contiguous()
            or out.data_ptr() % 2 != 0):
        raise RuntimeError(f"out must be a contiguous {dtype} tensor of shape ({batch}, {n_out_features}) on {dev}")
    x = _prepare_input(input, batch, n_in_features)
    with torch.cuda.device(dev):
        _launch_matmul("matmul_matgptq_out", dev, bitwidth, group_size, n_out_features, n_in_features, batch,
                       matgptq_weights, matgptq_scales, x, out, feature_flag)


def matmul_matgptq_grouped_raw(x: torch.Tensor, packed, scales, n_out, n_in: int, bitwidths, group_size: int,
                               flags: int, out: torch.Tensor | None = None,
                               workspace: torch.Tensor | None = None) -> torch.Tensor:
    """The C-ABI grouped product without checks: segment ``i`` (``packed[i]``, ``scales[i]``, ``n_out[i]`` rows at
    ``bitwidths[i]`` bits) fills its column block of ``out [M, sum(n_out)]``.  One kernel launch up to 16 rows."""
    batch = x.size(-2)
    total = int(sum(n_out))
    if out is None:
        out = torch.empty((batch, total), dtype=x.dtype, device=x.device)
    segs = (_native.Segment * len(packed))()
    need = 0
    for i, (w, s, n, b) in enumerate(zip(packed, scales, n_out, bitwidths)):
        segs[i] = _native.Segment(w.data_ptr(), s.data_ptr(), int(n), int(b))
        if batch >= 32 and workspace is None and flags & _native.FLAG_SCRATCH_REDUCE:
            need = max(need, _lib.matgptq_b200_matmul_workspace_bytes(int(n), n_in, batch))
    if need > 0:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    st = _lib.matgptq_b200_matmul_grouped(segs, len(packed), group_size, n_in, batch, x.data_ptr(), out.data_ptr(),
                                          torch.cuda.current_stream(x.device).cuda_stream, flags,
                                          workspace.data_ptr() if workspace is not None else None,
                                          workspace.numel() if workspace is not None else 0)
    _native.check(st, "matgptq_b200_matmul_grouped")
    return out


@torch.library.custom_op("matgptq_cuda::matmul_matgptq_grouped", mutates_args=())
def matmul_matgptq_grouped(
    input: torch.Tensor,
    matgptq_weights: list[torch.Tensor],
    matgptq_scales: list[torch.Tensor],
    n_out_features: list[int],
    n_in_features: int,
    bitwidths: list[int],
    group_size: int,
    feature_flag: int,
) -> torch.Tensor:
    """Addition: ``matmul_matgptq`` for a fused layer whose output partitions have their own bitwidths
    (``vllm_matgptq.py:113-121`` fuses q/k/v and gate/up; ``evo_quant_search.py:659-671`` gives each checkpoint
    layer its own bitwidth).  ``y[M, sum N_i] = x[M, K] @ cat(Wdq_i).T`` in one launch up to 16 rows;
    the reference's operator takes a single bitwidth per call."""
    if not (len(matgptq_weights) == len(matgptq_scales) == len(n_out_features) == len(bitwidths)) or not matgptq_weights:
        raise RuntimeError("matmul_matgptq_grouped: one weight, scale, n_out_features and bitwidth per segment")
    if len(matgptq_weights) > 8:
        raise RuntimeError("matmul_matgptq_grouped: at most 8 segments")
    bf16 = bool(feature_flag & _native.FLAG_BF16)
    dtype = torch.bfloat16 if bf16 else torch.float16
    for w, s, n, b in zip(matgptq_weights, matgptq_scales, n_out_features, bitwidths):
        _check_matmul_args(input, w, s, n, n_in_features, b, group_size)
        if s.dtype != dtype:
            raise RuntimeError(f"matgptq_scales must be {dtype} for feature_flag={feature_flag}")
    if input.dtype != dtype:
        raise RuntimeError(f"input must be {dtype} for feature_flag={feature_flag}")
    batch = input.size(-2)
    x = input
    if input.dim() > 2:
        x = input.reshape(-1, batch, n_in_features)[0]
    if not x.is_contiguous():
        x = x.contiguous()
    if x.data_ptr() % 16 != 0:
        x = x.clone()
    with torch.cuda.device(x.device):
        return matmul_matgptq_grouped_raw(x, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidths,
                                          group_size, feature_flag)


@matmul_matgptq_grouped.register_fake
def _matmul_grouped_fake(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidths, group_size,
                         feature_flag):
    return input.new_empty((input.shape[-2], sum(n_out_features)),
                           dtype=torch.bfloat16 if feature_flag & 2 else torch.float16)


@torch.library.custom_op("matgptq_cuda::matmul_matgptq_zeros", mutates_args=())
def matmul_matgptq_zeros(
    input: torch.Tensor,
    matgptq_weights: torch.Tensor,
    matgptq_scales: torch.Tensor,
    matgptq_zeros: torch.Tensor,
    n_out_features: int,
    n_in_features: int,
    bitwidth: int,
    group_size: int,
    feature_flag: int,
) -> torch.Tensor:
    """Extension: ``matmul_matgptq`` with per-group zero points, ``Wdq = s * (code * 2^(8-b) - zero)`` as in the
    reference's ``dequantize`` (``src/quant_utils_matgpqt.py:19-22``).  ``matgptq_zeros`` are the zero points in
    master (8-bit) units, in the dtype of the scales, passed through ``reorder_matgptq_scales`` like the scales.
    The reference's operator has no such argument (its zero point is the implicit ``2^(b-1)``)."""
    _check_matmul_args(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidth, group_size)
    bf16 = bool(feature_flag & _native.FLAG_BF16)
    dtype = torch.bfloat16 if bf16 else torch.float16
    if input.dtype != dtype or matgptq_scales.dtype != dtype or matgptq_zeros.dtype != dtype:
        raise RuntimeError(f"input, matgptq_scales and matgptq_zeros must be {dtype} for feature_flag={feature_flag}")
    if matgptq_zeros.shape != matgptq_scales.shape or matgptq_zeros.device != matgptq_scales.device:
        raise RuntimeError("matgptq_zeros must have the shape and device of matgptq_scales")
    dev = matgptq_weights.device
    batch = input.size(-2)
    x = input
    if input.dim() > 2:
        x = input.reshape(-1, batch, n_in_features)[0]
    if not x.is_contiguous():
        x = x.contiguous()
    if x.data_ptr() % 16 != 0:
        x = x.clone()
    z = matgptq_zeros.contiguous()
    with torch.cuda.device(dev):
        out = torch.empty((batch, n_out_features), dtype=dtype, device=dev)
        st = _lib.matgptq_b200_matmul_zp(bitwidth, group_size, n_out_features, n_in_features, batch,
                                         matgptq_weights.data_ptr(), matgptq_scales.data_ptr(), z.data_ptr(),
                                         x.data_ptr(), out.data_ptr(), _stream_ptr(dev), feature_flag)
        _native.check(st, "matmul_matgptq_zeros")
    return out


@matmul_matgptq_zeros.register_fake
def _matmul_zeros_fake(input, matgptq_weights, matgptq_scales, matgptq_zeros, n_out_features, n_in_features, bitwidth,
                       group_size, feature_flag):
    return input.new_empty((input.shape[-2], n_out_features),
                           dtype=torch.bfloat16 if feature_flag & 2 else torch.float16)


@torch.library.custom_op("matgptq_cuda::dequantize_matgptq", mutates_args=())
def dequantize_matgptq(
    matgptq_weights: torch.Tensor,
    matgptq_scales: torch.Tensor,
    n_out_features: int,
    n_in_features: int,
    bitwidth: int,
    group_size: int,
    feature_flag: int,
) -> torch.Tensor:
    """Dense ``W[N, K]`` (fp16/bf16) from packed weights and reordered scales, bit-exact with the
    reference's ``dequantize`` for zero point 128."""
    _check_common(bitwidth, group_size, n_in_features)
    dev = matgptq_weights.device
    dtype = torch.bfloat16 if feature_flag & _native.FLAG_BF16 else torch.float16
    if matgptq_scales.dtype != dtype:
        raise RuntimeError(f"matgptq_scales must be {dtype} for feature_flag={feature_flag}")
    with torch.cuda.device(dev):
        out = torch.empty((n_out_features, n_in_features), dtype=dtype, device=dev)
        st = _lib.matgptq_b200_dequantize(matgptq_weights.data_ptr(), matgptq_scales.data_ptr(), None, out.data_ptr(),
                                          n_out_features, n_in_features, bitwidth, group_size, feature_flag,
                                          _stream_ptr(dev))
        _native.check(st, "dequantize_matgptq")
    return out


@dequantize_matgptq.register_fake
def _dequant_fake(matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidth, group_size, feature_flag):
    return matgptq_scales.new_empty((n_out_features, n_in_features))


def matmul_matgptq_raw(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, n_out: int, n_in: int,
                       bitwidth: int, group_size: int, flags: int, out: torch.Tensor | None = None,
                       warps_per_cta: int = 0, split_k: int = 0, path: int = 0,
                       workspace: torch.Tensor | None = None) -> torch.Tensor:
    """The C-ABI matmul without the dispatcher around it: no argument checks beyond the library's own,
    optional preallocated output and scratch, forced path (1 GEMV, 2 tensor cores) and launch shape.
    Used by the decode loop, the benchmarks and the tests."""
    batch = x.size(-2)
    if out is None:
        out = torch.empty((batch, n_out), dtype=x.dtype, device=x.device)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    if warps_per_cta:
        st = _lib.matgptq_b200_matmul_tuned(bitwidth, group_size, n_out, n_in, batch, packed.data_ptr(),
                                            scales.data_ptr(), x.data_ptr(), out.data_ptr(), stream, flags,
                                            warps_per_cta, split_k)
    else:
        if workspace is None and path != 1 and flags & _native.FLAG_SCRATCH_REDUCE:  # scratch only where it is used
            if path == 2 and split_k > 1:
                need = split_k * batch * n_out * 4
            elif path == 2:
                need = _lib.matgptq_b200_matmul_workspace_bytes(n_out, n_in, max(batch, 64))
            else:
                need = _lib.matgptq_b200_matmul_workspace_bytes(n_out, n_in, batch)
            if need > 0:
                workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
        st = _lib.matgptq_b200_matmul_ws(bitwidth, group_size, n_out, n_in, batch, packed.data_ptr(),
                                         scales.data_ptr(), x.data_ptr(), out.data_ptr(), stream, flags,
                                         workspace.data_ptr() if workspace is not None else None,
                                         workspace.numel() if workspace is not None else 0, path, split_k)
    _native.check(st, "matgptq_b200_matmul")
    return out
