"""Child of tests/test_gpu_allreduce.py::test_two_gpus_fused_equals_nccl, one process per GPU (torchrun)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from matgptq_b200 import _native, ops, synth  # noqa: F401
    from matgptq_b200.tp_comm import PeerAllReduce
    ar = PeerAllReduce(device=dev, max_rows=32, max_cols=4096)
    n_out, n_in = 4096, 4096
    cols = n_in // world
    worst = 0.0
    for b, m in ((4, 1), (2, 8), (8, 16), (3, 5)):
        layer = synth.make_layer(n_out, n_in, 128, seed=b, sym=True, dtype=torch.float16, device=dev)
        q = layer.qweight[:, rank * cols:(rank + 1) * cols].contiguous()
        s = layer.scales[:, rank * cols // 128:(rank + 1) * cols // 128].contiguous()
        packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(q, n_out, cols, 8, b, 128, 1)
        scales = torch.ops.matgptq_cuda.reorder_matgptq_scales(s, n_out, cols, 128)
        for rep in range(4):
            x = synth.make_activations(m, n_in, seed=10 * b + rep, dtype=torch.float16, device=dev)[:, rank * cols:(rank + 1) * cols].contiguous()
            fused = ar.matmul(x, packed, scales, n_out, cols, b, 128, 1 | 4)
            part = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales, n_out, cols, b, 128, 1).float()
            dist.all_reduce(part)
            torch.cuda.synchronize()
            assert _native.device_status() == 0
            err = (fused.float() - part).abs().max().item() / part.abs().max().item()
            worst = max(worst, err)
            gathered = [torch.empty_like(fused) for _ in range(world)]
            dist.all_gather(gathered, fused)
            assert all(torch.equal(g, gathered[0]) for g in gathered), "ranks hold different bits"
    assert worst <= 3e-3, worst
    dist.barrier()
    if rank == 0:
        print("ALLREDUCE OK", worst, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
