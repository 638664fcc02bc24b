"""Decode harness: a small Llama-architecture model over packed linears against the same model over
the oracle's dequantised dense weights, and the tensor-parallel sharding arithmetic on CPU ranks."""
import os

import pytest
import torch
import torch.nn.functional as F

from oracle import matgptq_oracle as oracle

SMALL = dict(hidden=256, intermediate=512, n_heads=4, n_kv_heads=2, n_layers=2, vocab=512)


def _dense_linear_factory(model):
    """Dense stand-in for PackedLlama.linear built from the master codes with the CPU oracle."""
    dense = {}
    for li, L in enumerate(model.layers):
        for which in ("qkv", "o", "gate_up", "down"):
            ws = [oracle.dequantize_weight(q, s, torch.full_like(s, 128.0), 8, bits) for _, bits, q, s in L[which].master]
            dense[(li, which)] = torch.cat(ws).float().to(model.dev)

    def linear(layer, which, x):
        return F.linear(x.float(), dense[(layer, which)]).to(x.dtype)
    return linear


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch", [1, 3])
def test_small_model_matches_dense_reference(cuda, dtype, batch):
    from matgptq_b200 import decode
    shape = decode.LlamaShape(**SMALL)
    bits = decode.mixed_bitwidths(shape, 4.0, seed=1)
    assert len(set(bits.values())) >= 3
    model = decode.PackedLlama(shape, bits, dtype=dtype, batch=batch, max_seq=48, device=cuda, keep_master=True, seed=3)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, shape.vocab, (batch, 24), generator=g).to(cuda)
    pos = torch.arange(24, device=cuda)
    logits = model.forward(prompt, pos)
    packed_linear = model.linear
    model.linear = _dense_linear_factory(model)
    for k in model.k_cache + model.v_cache:
        k.zero_()
    logits_ref = model.forward(prompt, pos)
    model.linear = packed_linear
    assert logits.shape == (batch, shape.vocab)
    assert oracle.rel_err(logits, logits_ref) <= (2e-2 if dtype == torch.bfloat16 else 1e-2)
    # greedy generation: graph replay and eager stepping produce the same tokens
    for k in model.k_cache + model.v_cache:
        k.zero_()
    a = model.generate(prompt, 12, use_graph=True)
    for k in model.k_cache + model.v_cache:
        k.zero_()
    b = model.generate(prompt, 12, use_graph=False)
    assert torch.equal(a["tokens"], b["tokens"]) and a["decode_steps"] == 11
    assert a["decode_s"] > 0 and a["prefill_s"] > 0


def _shard_worker(rank, world, port, out):
    import torch.distributed as dist
    from matgptq_b200 import decode
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, I, gs = 256, 512, 128
    seed_of = lambda n: 7  # noqa: E731
    bits_of = lambda n: 4  # noqa: E731
    # column-parallel: rows split; row-parallel: columns (and their scale groups) split
    col = decode._make_segments([("up", I)], H, H, 0, bits_of, gs, torch.float16, seed_of, "cpu",
                                [(rank * I // world, (rank + 1) * I // world)])[0]
    row = decode._make_segments([("down", H)], I // world, I, rank * I // world, bits_of, gs, torch.float16, seed_of, "cpu",
                                [(0, H)])[0]
    gathered_q = [torch.empty_like(col[2].contiguous()) for _ in range(world)]
    dist.all_gather(gathered_q, col[2].contiguous())
    gathered_rq = [torch.empty_like(row[2].contiguous()) for _ in range(world)]
    dist.all_gather(gathered_rq, row[2].contiguous())
    gathered_rs = [torch.empty_like(row[3].contiguous()) for _ in range(world)]
    dist.all_gather(gathered_rs, row[3].contiguous())
    # the row-parallel partial products add up to the full product (what the all-reduce computes)
    x = torch.randn(3, I, generator=torch.Generator().manual_seed(1))
    w_loc = oracle.dequantize_weight(row[2].contiguous(), row[3].contiguous(), torch.full_like(row[3], 128.0), 8, 4).float()
    part = x[:, rank * I // world:(rank + 1) * I // world] @ w_loc.T
    dist.all_reduce(part)
    if rank == 0:
        from matgptq_b200 import synth
        full_up = synth.make_layer(I, H, gs, seed=7, dtype=torch.float16)
        full_down = synth.make_layer(H, I, gs, seed=7, dtype=torch.float16)
        ok = torch.equal(torch.cat(gathered_q), full_up.qweight)
        ok &= torch.equal(torch.cat(gathered_rq, dim=1), full_down.qweight)
        ok &= torch.equal(torch.cat(gathered_rs, dim=1), full_down.scales)
        w_full = oracle.dequantize_weight(full_down.qweight, full_down.scales, full_down.zeros, 8, 4).float()
        ok &= torch.allclose(part, x @ w_full.T, rtol=1e-4, atol=1e-4)
        out.put(bool(ok))
    dist.destroy_process_group()


def test_tensor_parallel_sharding_two_cpu_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_shard_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(timeout=5) is True
