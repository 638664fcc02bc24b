"""The matmul entry point that allocates nothing (scratch built into the library image).

It exists for callers that have no device memory to hand over and no way to get any: a host
whose pool already owns the GPU, a plugin without access to that pool, a loop in which
cudaMalloc is off limits.  Its result must be the one `matgptq_b200_matmul_ws` gives with
caller-provided scratch: same kernels, same K split, so bit-identical.  Two calls in a row share
the built-in array; the second must not see anything of the first.

The file name sorts last on purpose: a run that stops at the first failure has by then run every
other test.
"""
import pytest
import torch

from matgptq_b200 import synth

pytestmark = pytest.mark.gpu


def _layer(n_out, n_in, b, dtype, seed, cuda):
    from matgptq_b200 import ops  # noqa: F401
    layer = synth.make_layer(n_out, n_in, 128, seed=seed, sym=True, dtype=dtype, device=cuda)
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n_out, n_in, 8, b, 128, flag)
    scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n_out, n_in, 128)
    return packed, scales_r, flag


SCRATCH_REDUCE = 8  # MATGPTQ_B200_FLAG_SCRATCH_REDUCE: the sums of a split K go through the scratch


def _both(lib, packed, scales_r, flag, x, n_out, n_in, b):
    m = x.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    need = lib.matgptq_b200_matmul_workspace_bytes(n_out, n_in, m)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    y_ws = torch.empty(m, n_out, dtype=x.dtype, device=x.device)
    st = lib.matgptq_b200_matmul_ws(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(), x.data_ptr(),
                                    y_ws.data_ptr(), stream, flag, ws.data_ptr() if need else None, need, 0, 0)
    assert st == 0
    y_static = torch.full_like(y_ws, float("nan"))
    st = lib.matgptq_b200_matmul_static_scratch(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(),
                                                x.data_ptr(), y_static.data_ptr(), stream, flag)
    assert st == 0
    torch.cuda.synchronize()
    return y_ws, y_static, need


def test_static_scratch_matches_caller_scratch_twice_in_a_row(lib, cuda):
    from matgptq_b200 import _native
    # k/v shape: 8 row tiles of 128, so the tensor-core path splits K and needs scratch
    n_in, n_out = 4096, 1024
    packed_a, scales_a, flag_a = _layer(n_out, n_in, 4, torch.float16, 1, cuda)
    packed_b, scales_b, flag_b = _layer(n_out, n_in, 3, torch.bfloat16, 2, cuda)
    x_a = synth.make_activations(64, n_in, seed=1, dtype=torch.float16, device=cuda)
    x_b = synth.make_activations(48, n_in, seed=2, dtype=torch.bfloat16, device=cuda)

    y_ws, y_static, need = _both(lib, packed_a, scales_a, flag_a | SCRATCH_REDUCE, x_a, n_out, n_in, 4)
    assert need > 0, "this shape is meant to exercise the scratch"
    assert torch.isfinite(y_static.float()).all()
    assert torch.equal(y_static, y_ws)

    # second call, other weights, dtype and batch: the array still holds the first call's sums
    y_ws2, y_static2, need2 = _both(lib, packed_b, scales_b, flag_b | SCRATCH_REDUCE, x_b, n_out, n_in, 3)
    assert need2 > 0
    assert torch.equal(y_static2, y_ws2)
    # and the first problem again gives the first answer again
    _, y_static3, _ = _both(lib, packed_a, scales_a, flag_a | SCRATCH_REDUCE, x_a, n_out, n_in, 4)
    assert torch.equal(y_static3, y_ws)
    # without the flag the sums meet inside the cluster and the array is only a fallback: the same bits
    y_ws4, y_static4, _ = _both(lib, packed_a, scales_a, flag_a, x_a, n_out, n_in, 4)
    assert torch.equal(y_static4, y_ws) and torch.equal(y_ws4, y_ws)
    assert _native.device_status() == 0


def test_static_scratch_later_calls_leave_free_memory_unchanged(lib, cuda):
    """Only the first call that needs scratch on a device may change the free device memory (it brings the
    built-in array in); the calls after it must not, which is what a host whose pool owns the rest of the
    device relies on.  Inputs and outputs are allocated before the measurement starts."""
    n_in, n_out, b, m = 4096, 1024, 4, 64
    packed, scales_r, flag = _layer(n_out, n_in, b, torch.float16, 5, cuda)
    x = synth.make_activations(m, n_in, seed=5, dtype=torch.float16, device=cuda)
    y = torch.empty(m, n_out, dtype=torch.float16, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.matgptq_b200_matmul_workspace_bytes(n_out, n_in, m) > 0

    def call(extra=0):
        st = lib.matgptq_b200_matmul_static_scratch(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(),
                                                    x.data_ptr(), y.data_ptr(), stream, flag | extra)
        assert st == 0
        torch.cuda.synchronize()

    call()  # set-up (if no earlier test did it) happens here
    call(SCRATCH_REDUCE)  # both forms of the K split have run once: their kernels are loaded
    free_before, _ = torch.cuda.mem_get_info(cuda)
    first = y.clone()
    free_before, _ = torch.cuda.mem_get_info(cuda)  # taken after the clone: nothing below allocates through torch
    call()
    call(SCRATCH_REDUCE)
    call()
    free_after, _ = torch.cuda.mem_get_info(cuda)
    assert free_after == free_before
    assert torch.equal(y, first)


def test_static_scratch_small_batches_and_limit(lib, cuda):
    n_in, n_out, b = 4096, 4096, 4
    packed, scales_r, flag = _layer(n_out, n_in, b, torch.float16, 3, cuda)
    # a batch of the cluster GEMV: no scratch involved at all, same answer
    x = synth.make_activations(8, n_in, seed=3, dtype=torch.float16, device=cuda)
    y_ws, y_static, need = _both(lib, packed, scales_r, flag, x, n_out, n_in, b)
    assert need == 0 and torch.equal(y_static, y_ws)
    # a shape whose sums want more than the built-in 8 MiB: with the flag it is refused and nothing is launched
    m = 256
    need = lib.matgptq_b200_matmul_workspace_bytes(n_out, n_in, m)
    assert need > 8 * 1024 * 1024
    xb = synth.make_activations(m, n_in, seed=4, dtype=torch.float16, device=cuda)
    y = torch.full((m, n_out), 7.0, dtype=torch.float16, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    st = lib.matgptq_b200_matmul_static_scratch(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(),
                                                xb.data_ptr(), y.data_ptr(), stream, flag | SCRATCH_REDUCE)
    assert st == 5
    assert b"scratch" in lib.matgptq_b200_strerror(st)
    torch.cuda.synchronize()
    assert (y == 7.0).all()
    # without the flag the sums meet inside the cluster, no scratch is involved, and the call goes through
    st = lib.matgptq_b200_matmul_static_scratch(b, 128, n_out, n_in, m, packed.data_ptr(), scales_r.data_ptr(),
                                                xb.data_ptr(), y.data_ptr(), stream, flag)
    assert st == 0
    y_ws = torch.ops.matgptq_cuda.matmul_matgptq(xb, packed, scales_r, n_out, n_in, b, 128, flag)
    torch.cuda.synchronize()
    assert torch.equal(y, y_ws)
