"""Row-parallel product fused with its all-reduce over peer memory.

On one GPU the ranks of a tensor-parallel group are emulated: every rank's buffers are local, the ranks'
products run one after the other in store-and-publish mode and a finishing kernel adds up what each rank
received (kernels that wait for one another must not be separate launches on one GPU).  That covers the
addressing of slots and flags, the alternation of the two slot sets, the epochs and the rank-order sum; the
in-kernel wait runs where there are really several GPUs (test_two_gpus_fused_equals_nccl)."""
import os
import subprocess
import sys

import pytest
import torch

from matgptq_b200 import synth
from oracle import matgptq_oracle as oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _shards(n_out, n_in, world, b, dtype, cuda, seed):
    from matgptq_b200 import ops  # noqa: F401
    layer = synth.make_layer(n_out, n_in, 128, seed=seed, sym=True, dtype=dtype, device=cuda)
    flag = 1 | (2 if dtype == torch.bfloat16 else 0)
    cols = n_in // world
    shards = []
    for r in range(world):
        q = layer.qweight[:, r * cols:(r + 1) * cols].contiguous()
        s = layer.scales[:, r * cols // 128:(r + 1) * cols // 128].contiguous()
        shards.append((torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(q, n_out, cols, 8, b, 128, flag),
                       torch.ops.matgptq_cuda.reorder_matgptq_scales(s, n_out, cols, 128)))
    w_ref = oracle.dequantize_weight(layer.qweight.cpu(), layer.scales.cpu(), layer.zeros.cpu(), 8, b)
    return shards, w_ref, flag, cols


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("b,dtype", [(2, torch.float16), (3, torch.bfloat16), (4, torch.float16), (8, torch.float16)])
@pytest.mark.parametrize("m", [1, 5, 16, 19])
def test_emulated_ranks_sum_in_rank_order(cuda, world, b, dtype, m):
    from matgptq_b200 import _native
    from matgptq_b200.tp_comm import LoopbackRanks
    n_out, n_in = 1024, 4096
    shards, w_ref, flag, cols = _shards(n_out, n_in, world, b, dtype, cuda, seed=11)
    ranks = LoopbackRanks(world, cuda, max_rows=32, max_cols=n_out)
    for call in range(3):  # three reductions in a row: both slot sets and a reuse of the first
        x = synth.make_activations(m, n_in, seed=m + call, dtype=dtype, device=cuda)
        for r in range(world):
            ranks.push(r, x[:, r * cols:(r + 1) * cols].contiguous(), shards[r][0], shards[r][1], n_out, cols, b, 128, flag)
        outs = [ranks.finish(r, m, n_out, dtype, flag) for r in range(world)]
        assert _native.device_status() == 0
        for o in outs[1:]:
            assert torch.equal(o, outs[0])  # every rank adds the same slots in the same order
        y_ref = oracle.linear_fp32_accumulate(x.cpu(), w_ref)
        assert oracle.rel_err(outs[0].cpu(), y_ref) <= 1e-2
        # against the unfused arithmetic: per-rank products (fp16/bf16 outputs) added in fp32
        parts = [torch.ops.matgptq_cuda.matmul_matgptq(x[:, r * cols:(r + 1) * cols].contiguous(), shards[r][0], shards[r][1],
                                                       n_out, cols, b, 128, flag).float() for r in range(world)]
        # (the per-rank outputs carry one rounding to the output type, the fused sum does not)
        assert oracle.rel_err(outs[0].cpu(), sum(parts).cpu()) <= (3e-3 if dtype == torch.float16 else 2e-2)
        assert int(ranks.ctrl[0][0]) == call + 1  # the epoch of rank 0 advanced by one


def test_a_missing_rank_is_reported_not_waited_for(cuda):
    """Rank 1 never publishes: the finishing kernel of rank 0 finds its flags missing and records status 105."""
    from matgptq_b200 import _native
    from matgptq_b200.tp_comm import LoopbackRanks
    n_out, n_in, world, b, m = 256, 1024, 2, 4, 3
    shards, _, flag, cols = _shards(n_out, n_in, world, b, torch.float16, cuda, seed=5)
    ranks = LoopbackRanks(world, cuda, max_rows=32, max_cols=n_out)
    x = synth.make_activations(m, n_in, seed=1, dtype=torch.float16, device=cuda)
    ranks.push(0, x[:, :cols].contiguous(), shards[0][0], shards[0][1], n_out, cols, b, 128, flag)
    ranks.finish(0, m, n_out, torch.float16, flag)
    assert _native.device_status() == 105
    assert _native.device_status() == 0


def test_unsupported_shapes_are_refused(lib, cuda):
    import ctypes
    from matgptq_b200.tp_comm import LoopbackRanks
    shards, _, flag, cols = _shards(256, 1024, 2, 4, torch.float16, cuda, seed=5)
    ranks = LoopbackRanks(2, cuda, max_rows=4, max_cols=256)
    x = synth.make_activations(40, cols, seed=1, dtype=torch.float16, device=cuda)
    y = torch.empty(40, 256, dtype=torch.float16, device=cuda)
    st = lib.matgptq_b200_matmul_allreduce(4, 128, 256, cols, 40, shards[0][0].data_ptr(), shards[0][1].data_ptr(), x.data_ptr(),
                                           y.data_ptr(), None, flag, ctypes.byref(ranks.comms[0]))
    assert st == 3  # 32 rows and more: tensor-core path, not fused
    st = lib.matgptq_b200_matmul_allreduce(4, 128, 256, cols, 8, shards[0][0].data_ptr(), shards[0][1].data_ptr(), x.data_ptr(),
                                           y.data_ptr(), None, flag, ctypes.byref(ranks.comms[0]))
    assert st == 3  # 8 * 256 outputs do not fit in slots of 4 * 256
    assert int(ranks.ctrl[0][1]) == 0  # nothing was launched


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_fused_equals_nccl():
    """Two processes on two GPUs: the fused kernel (in-kernel wait on the peer's flags) against per-rank products
    followed by an NCCL all-reduce; both ranks must hold identical bits."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "two_rank_allreduce_check.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert proc.returncode == 0 and "ALLREDUCE OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-3000:]
