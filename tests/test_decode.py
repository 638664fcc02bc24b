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


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [1, 8])
def test_full_width_layers_match_dense_reference(cuda, batch):
    """Two decoder layers at the full width of the Llama-3.1-8B architecture (hidden 4096, MLP 14336, 32 heads
    / 8 KV heads; small vocabulary), seeded per-layer bitwidths with mean 3 bits: the logits of the prefill
    AND of the first decode step (one row per sequence: the GEMV launch shapes of the timed decode) against
    the same model over the oracle's dequantised dense weights."""
    from matgptq_b200 import decode
    shape = decode.LlamaShape(4096, 14336, 32, 8, 2, 4096)
    bits = decode.mixed_bitwidths(shape, 3.0, seed=0)
    model = decode.PackedLlama(shape, bits, dtype=torch.float16, batch=batch, max_seq=64, device=cuda, keep_master=True, seed=0)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, shape.vocab, (batch, 32), generator=g).to(cuda)
    nxt = torch.randint(0, shape.vocab, (batch, 1), generator=g).to(cuda)
    pos, pos1 = torch.arange(32, device=cuda), torch.tensor([32], device=cuda)

    def run():
        for k in model.k_cache + model.v_cache:
            k.zero_()
        return model.forward(prompt, pos), model.forward(nxt, pos1)

    got_prefill, got_step = run()
    packed_linear = model.linear
    model.linear = _dense_linear_factory(model)
    ref_prefill, ref_step = run()
    model.linear = packed_linear
    assert oracle.rel_err(got_prefill, ref_prefill) <= 1e-2
    assert oracle.rel_err(got_step, ref_step) <= 1e-2


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


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_helper_kernels_match_torch(cuda, dtype):
    """add_rmsnorm, rope_kv and silu_mul against the same arithmetic in torch (fp32 inside, results rounded
    to the model dtype at the same places)."""
    from matgptq_b200 import _native
    lib = _native.load()
    flag = _native.FLAG_BF16 if dtype == torch.bfloat16 else 0
    stream = torch.cuda.current_stream(cuda).cuda_stream
    g = torch.Generator(device=cuda).manual_seed(5)
    rows, hidden, eps = 7, 384, 1e-5
    x = torch.randn(rows, hidden, generator=g, device=cuda).to(dtype)
    delta = torch.randn(rows, hidden, generator=g, device=cuda).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, generator=g, device=cuda)).to(dtype)
    for use_delta in (False, True):
        xs, h = x.clone(), torch.empty_like(x)
        _native.check(lib.matgptq_b200_add_rmsnorm(xs.data_ptr(), delta.data_ptr() if use_delta else None, w.data_ptr(),
                                                   h.data_ptr(), rows, hidden, eps, flag, stream), "add_rmsnorm")
        x_ref = (x + delta) if use_delta else x
        xf = x_ref.float()
        h_ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype) * w
        assert torch.equal(xs, x_ref)
        assert (h.float() - h_ref.float()).abs().max() <= 2 * torch.finfo(dtype).eps * h_ref.float().abs().max()

    B, S, H, KV, d, max_seq = 2, 5, 4, 2, 64, 16
    qkv = torch.randn(B, S, (H + 2 * KV) * d, generator=g, device=cuda).to(dtype)
    positions = torch.tensor([3, 4, 5, 6, 7], device=cuda)
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, device=cuda, dtype=torch.float32) / d))
    ang = torch.arange(max_seq, device=cuda, dtype=torch.float32)[:, None] * inv[None, :]
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    q = torch.empty(B, H, S, d, dtype=dtype, device=cuda)
    kc = torch.zeros(B, KV, max_seq, d, dtype=dtype, device=cuda)
    vc = torch.zeros_like(kc)
    _native.check(lib.matgptq_b200_rope_kv(qkv.data_ptr(), positions.data_ptr(), cos.data_ptr(), sin.data_ptr(), q.data_ptr(),
                                           kc.data_ptr(), vc.data_ptr(), B, S, H, KV, d, max_seq, flag, stream), "rope_kv")

    def rope(t):  # [B, S, h, d]
        tf = t.float()
        a, c = tf[..., 0::2], tf[..., 1::2]
        cs, sn = cos[positions][None, :, None, :], sin[positions][None, :, None, :]
        return torch.stack([a * cs - c * sn, a * sn + c * cs], dim=-1).flatten(-2).to(dtype)

    parts = qkv.view(B, S, H + 2 * KV, d)
    q_ref = rope(parts[:, :, :H]).transpose(1, 2)
    k_ref = rope(parts[:, :, H:H + KV]).transpose(1, 2)
    v_ref = parts[:, :, H + KV:].transpose(1, 2)
    tol = 2 * torch.finfo(dtype).eps * 4
    assert (q.float() - q_ref.float()).abs().max() <= tol * q_ref.float().abs().max()
    assert (kc[:, :, 3:8].float() - k_ref.float()).abs().max() <= tol * k_ref.float().abs().max()
    assert torch.equal(vc[:, :, 3:8], v_ref)
    assert kc[:, :, :3].abs().max() == 0 and kc[:, :, 8:].abs().max() == 0 and vc[:, :, 8:].abs().max() == 0

    inter = 320
    gu = torch.randn(rows, 2 * inter, generator=g, device=cuda).to(dtype)
    out = torch.empty(rows, inter, dtype=dtype, device=cuda)
    _native.check(lib.matgptq_b200_silu_mul(gu.data_ptr(), out.data_ptr(), rows, inter, flag, stream), "silu_mul")
    ref = F.silu(gu[:, :inter].float()).to(dtype) * gu[:, inter:]
    assert (out.float() - ref.float()).abs().max() <= 4 * torch.finfo(dtype).eps * ref.float().abs().max()
    assert lib.matgptq_b200_add_rmsnorm(None, None, w.data_ptr(), h.data_ptr(), 1, hidden, eps, flag, stream) != 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 128256), (3, 4096), (8, 512), (2, 8)])
def test_argmax_kernel_matches_torch(cuda, dtype, rows, cols):
    """Greedy sampling helper: the first index of each row's maximum, ties and -inf included."""
    from matgptq_b200 import _native
    lib = _native.load()
    g = torch.Generator(device=cuda).manual_seed(rows * cols)
    logits = torch.randn(rows, cols, generator=g, device=cuda).to(dtype)
    logits[0, cols // 2] = logits[0].max()       # a tie: the first of the two equal maxima wins
    if rows > 1:
        logits[1] = float("-inf")                # nothing is larger than anything: index 0
        logits[1, cols - 1] = -3.0
    out = torch.full((rows,), -1, dtype=torch.int64, device=cuda)
    flag = _native.FLAG_BF16 if dtype == torch.bfloat16 else 0
    _native.check(lib.matgptq_b200_argmax(logits.data_ptr(), out.data_ptr(), rows, cols, flag,
                                          torch.cuda.current_stream(cuda).cuda_stream), "argmax")
    want = torch.stack([(row == row.max()).nonzero()[0, 0] for row in logits.float()])
    assert torch.equal(out, want)
    assert lib.matgptq_b200_argmax(logits.data_ptr(), out.data_ptr(), rows, 12, flag, None) == 1  # cols % 8 != 0
