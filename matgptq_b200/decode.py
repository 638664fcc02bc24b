"""Whole-model decode over the packed linear layers: a thin Llama-architecture harness.

Stands in for the two serving loops of the reference — vLLM with ``tensor_parallel_size``
(``inference_lib/inference_demo_vllm.py:16-30``; the all-reduce after row-parallel layers is vLLM's
``RowParallelLinear``) and the HF-transformers static-cache loop
(``inference_lib/inference_demo_transformers.py:141-173``) — so that tensor parallelism, per-layer
bitwidths and CUDA-graph replay are under this package's control.  Every block linear goes through
``libmatgptq_b200`` (GEMV family for decode, tensor-core path for prefill); attention, RMSNorm, RoPE,
embedding and the unquantised ``lm_head`` are plain torch ops (plumbing, as in the reference, which
leaves them to vLLM / transformers).  Weights are random-init (no checkpoints exist here): master codes
and scales are drawn per layer on the GPU from a seed (``matgptq_b200.synth``).

Tensor parallelism: q/k/v and gate/up are column-parallel (out-features split), o and down are
row-parallel (in-features split, one all-reduce each), ``lm_head`` is vocabulary-parallel with an
all-gather of the logits.  One process per GPU over ``torch.distributed`` (NCCL).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _native, ops, synth


@dataclass
class LlamaShape:
    hidden: int
    intermediate: int
    n_heads: int
    n_kv_heads: int
    n_layers: int
    vocab: int
    rope_theta: float = 500000.0
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.hidden // self.n_heads


LLAMA31_8B = LlamaShape(4096, 14336, 32, 8, 32, 128256)
LLAMA31_70B = LlamaShape(8192, 28672, 64, 8, 80, 128256)


def layer_names(shape: LlamaShape) -> dict[str, int]:
    """``checkpoint layer name -> parameter count`` of every quantised linear."""
    d = shape.head_dim
    out = {}
    for i in range(shape.n_layers):
        p = f"model.layers.{i}"
        out[f"{p}.self_attn.q_proj"] = shape.hidden * shape.hidden
        out[f"{p}.self_attn.k_proj"] = shape.n_kv_heads * d * shape.hidden
        out[f"{p}.self_attn.v_proj"] = shape.n_kv_heads * d * shape.hidden
        out[f"{p}.self_attn.o_proj"] = shape.hidden * shape.hidden
        out[f"{p}.mlp.gate_proj"] = shape.intermediate * shape.hidden
        out[f"{p}.mlp.up_proj"] = shape.intermediate * shape.hidden
        out[f"{p}.mlp.down_proj"] = shape.hidden * shape.intermediate
    return out


class PackedLinear:
    """One (possibly fused) linear layer: consecutive output segments, each with its own bitwidth."""

    def __init__(self, segments, n_in: int, group_size: int, dtype: torch.dtype, keep_master: bool = False):
        # segments: list of (rows, bits, qweight_master_u8 [rows, n_in], scales [rows, G])
        self.n_in = n_in
        self.group_size = group_size
        self.flag = _native.FLAG_ASYNC | (_native.FLAG_BF16 if dtype == torch.bfloat16 else 0)
        self.parts = []
        self.master = [] if keep_master else None
        merged = []
        for rows, bits, q, s in segments:
            if merged and merged[-1][1] == bits:
                merged[-1] = (merged[-1][0] + rows, bits, torch.cat([merged[-1][2], q]), torch.cat([merged[-1][3], s]))
            else:
                merged.append((rows, bits, q, s))
        for rows, bits, q, s in merged:
            packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(q.contiguous(), rows, n_in, 8, bits, group_size, self.flag)
            scales = torch.ops.matgptq_cuda.reorder_matgptq_scales(s.contiguous(), rows, n_in, group_size)
            self.parts.append((rows, bits, packed, scales))
            if keep_master:
                self.master.append((rows, bits, q.cpu(), s.cpu()))
        self.n_out = sum(p[0] for p in self.parts)

    def __call__(self, x: torch.Tensor, pdl: bool = False) -> torch.Tensor:
        flag = self.flag | (_native.FLAG_PDL if pdl else 0)
        if len(self.parts) == 1:
            rows, bits, packed, scales = self.parts[0]
            return ops.matmul_matgptq_raw(x, packed, scales, rows, self.n_in, bits, self.group_size, flag)
        # segments of different bitwidths: ONE grouped launch writes them side by side
        # (running the segments on parallel streams was measured: 419 tok/s against 446 at batch 1; the fork
        # and join events cost more than the overlap gives, and the launches lose their programmatic chaining)
        return ops.matmul_matgptq_grouped_raw(x, [p[2] for p in self.parts], [p[3] for p in self.parts],
                                              [p[0] for p in self.parts], self.n_in, [p[1] for p in self.parts],
                                              self.group_size, flag)

    def weight_bytes(self) -> int:
        return sum(p.numel() * 4 + s.numel() * 2 for _, _, p, s in self.parts)


def _make_segments(names_rows, n_in, n_in_total, col0, bits_of, group_size, dtype, seed_of, dev, row_slices):
    """Draw master codes/scales of each named layer (full shape from its seed) and cut this rank's shard."""
    segs = []
    for (name, rows_total), (r0, r1) in zip(names_rows, row_slices):
        layer = synth.make_layer(rows_total, n_in_total, group_size, seed=seed_of(name), sym=True, dtype=dtype, device=dev)
        g0, g1 = col0 // group_size, (col0 + n_in) // group_size
        q = layer.qweight[r0:r1, col0:col0 + n_in]
        s = layer.scales[r0:r1, g0:g1]
        segs.append((r1 - r0, bits_of(name), q, s))
    return segs


class PackedLlama:
    """Llama-architecture decoder over packed linears, one tensor-parallel rank of it."""

    def __init__(self, shape: LlamaShape, bits, *, group_size: int = 128, dtype: torch.dtype = torch.float16,
                 tp_rank: int = 0, tp_size: int = 1, seed: int = 0, batch: int = 1, max_seq: int = 256,
                 device: torch.device | str = "cuda", keep_master: bool = False, pdl: bool = True, peer_allreduce=None):
        """``peer_allreduce``: a ``tp_comm.PeerAllReduce`` of the tensor-parallel group.  With it the row-parallel
        layers (o, down) run the product fused with its all-reduce over peer memory for fewer than 32 rows; without
        it (and for larger batches) the product is followed by an NCCL all-reduce."""
        self.shape, self.dtype, self.dev = shape, dtype, torch.device(device)
        self.peer_ar = peer_allreduce
        self.tp_rank, self.tp_size, self.batch, self.max_seq, self.pdl = tp_rank, tp_size, batch, max_seq, pdl
        T, r, d = tp_size, tp_rank, shape.head_dim
        assert shape.n_heads % T == 0 and shape.n_kv_heads % T == 0 and shape.intermediate % (T * 128) == 0
        assert (shape.hidden // T) % 128 == 0 and shape.vocab % T == 0
        self.h_loc, self.kv_loc = shape.n_heads // T, shape.n_kv_heads // T
        names = list(layer_names(shape))
        bits_of = (lambda n: bits) if isinstance(bits, int) else (lambda n: bits[n])
        seed_of = lambda n: seed * 100003 + names.index(n)  # noqa: E731
        H, I = shape.hidden, shape.intermediate
        qr, kvr, ir = H // T, shape.n_kv_heads * d // T, I // T
        mk = lambda nr, n_in, n_tot, c0, rs: PackedLinear(  # noqa: E731
            _make_segments(nr, n_in, n_tot, c0, bits_of, group_size, dtype, seed_of, self.dev, rs), n_in, group_size, dtype, keep_master)
        self.layers = []
        gen = torch.Generator(device=self.dev).manual_seed(seed + 17)
        for i in range(shape.n_layers):
            p = f"model.layers.{i}"
            qkv = mk([(f"{p}.self_attn.q_proj", H), (f"{p}.self_attn.k_proj", shape.n_kv_heads * d), (f"{p}.self_attn.v_proj", shape.n_kv_heads * d)],
                     H, H, 0, [(r * qr, (r + 1) * qr), (r * kvr, (r + 1) * kvr), (r * kvr, (r + 1) * kvr)])
            o = mk([(f"{p}.self_attn.o_proj", H)], H // T, H, r * (H // T), [(0, H)])
            gate_up = mk([(f"{p}.mlp.gate_proj", I), (f"{p}.mlp.up_proj", I)], H, H, 0, [(r * ir, (r + 1) * ir)] * 2)
            down = mk([(f"{p}.mlp.down_proj", H)], I // T, I, r * ir, [(0, H)])
            norms = [(1.0 + 0.1 * torch.randn(H, generator=gen, device=self.dev)).to(dtype) for _ in range(2)]
            self.layers.append({"qkv": qkv, "o": o, "gate_up": gate_up, "down": down, "ln1": norms[0], "ln2": norms[1]})
        self.final_norm = (1.0 + 0.1 * torch.randn(H, generator=gen, device=self.dev)).to(dtype)
        self.embed = (torch.randn(shape.vocab, H, generator=gen, device=self.dev) * 0.02).to(dtype)
        v_loc = shape.vocab // T
        head = (torch.randn(shape.vocab, H, generator=gen, device=self.dev) * 0.02).to(dtype)
        self.lm_head = head[r * v_loc:(r + 1) * v_loc].contiguous()
        del head
        inv = 1.0 / (shape.rope_theta ** (torch.arange(0, d, 2, device=self.dev, dtype=torch.float32) / d))
        ang = torch.arange(max_seq, device=self.dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()
        self.k_cache = [torch.zeros(batch, self.kv_loc, max_seq, d, dtype=dtype, device=self.dev) for _ in range(shape.n_layers)]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        self.key_index = torch.arange(max_seq, device=self.dev)

    # -- pieces ------------------------------------------------------------------------------
    def linear(self, layer: int, which: str, x: torch.Tensor) -> torch.Tensor:
        """x [M, n_in] -> [M, n_out] through the packed layer (tests swap this for a dense reference)."""
        return self.layers[layer][which](x, self.pdl)

    def _all_reduce(self, t):
        if self.tp_size > 1:
            dist.all_reduce(t)
        return t

    def row_parallel(self, layer: int, which: str, x: torch.Tensor) -> torch.Tensor:
        """A row-parallel layer and the all-reduce of its output (vLLM's RowParallelLinear in the reference)."""
        L = self.layers[layer][which]
        if (self.tp_size > 1 and self.peer_ar is not None and len(L.parts) == 1
                and self.peer_ar.fits(x.shape[0], L.n_out, L.group_size)):
            rows, bits, packed, scales = L.parts[0]
            flag = L.flag | (_native.FLAG_PDL if self.pdl else 0)
            return self.peer_ar.matmul(x, packed, scales, rows, L.n_in, bits, L.group_size, flag)
        return self._all_reduce(self.linear(layer, which, x))

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, fp32_logits: bool = True) -> torch.Tensor:
        """tokens [B, S] int64, positions [S] int64 (device) -> logits of the last position [B, vocab]
        (fp32, or the model dtype with ``fp32_logits=False``)."""
        B, S = tokens.shape
        d, H = self.shape.head_dim, self.shape.hidden
        lib = _native.load()
        # the helper kernels take part in programmatic dependent launch: the product behind each of them starts
        # prefetching its weights while the helper still runs
        flag = (_native.FLAG_BF16 if self.dtype == torch.bfloat16 else 0) | (_native.FLAG_PDL if self.pdl else 0)
        stream = torch.cuda.current_stream(self.dev).cuda_stream
        rows = B * S

        def add_norm(x, delta, w, h):
            _native.check(lib.matgptq_b200_add_rmsnorm(x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                                       w.data_ptr(), h.data_ptr(), rows, H, self.shape.eps, flag, stream),
                          "add_rmsnorm")

        x = self.embed[tokens].reshape(rows, H)
        h = torch.empty_like(x)
        q = torch.empty(B, self.h_loc, S, d, dtype=self.dtype, device=self.dev)
        act = torch.empty(rows, self.layers[0]["down"].n_in, dtype=self.dtype, device=self.dev)
        visible = self.key_index[None, :] <= positions[:, None]
        mask = torch.zeros(S, self.max_seq, dtype=self.dtype, device=self.dev).masked_fill_(~visible, float("-inf"))[None, None]
        add_norm(x, None, self.layers[0]["ln1"], h)
        for li, L in enumerate(self.layers):
            qkv = self.linear(li, "qkv", h)
            _native.check(lib.matgptq_b200_rope_kv(qkv.data_ptr(), positions.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(),
                                                   q.data_ptr(), self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(),
                                                   B, S, self.h_loc, self.kv_loc, d, self.max_seq, flag, stream), "rope_kv")
            att = F.scaled_dot_product_attention(q, self.k_cache[li], self.v_cache[li], attn_mask=mask, enable_gqa=True)
            att = att.transpose(1, 2).reshape(rows, self.h_loc * d)
            o = self.row_parallel(li, "o", att)
            add_norm(x, o, L["ln2"], h)
            gu = self.linear(li, "gate_up", h)
            _native.check(lib.matgptq_b200_silu_mul(gu.data_ptr(), act.data_ptr(), rows, act.shape[1], flag, stream), "silu_mul")
            dn = self.row_parallel(li, "down", act)
            nxt = self.layers[li + 1]["ln1"] if li + 1 < len(self.layers) else self.final_norm
            add_norm(x, dn, nxt, h)
        last = h.view(B, S, H)[:, -1]
        logits = F.linear(last, self.lm_head)
        if fp32_logits:
            logits = logits.float()
        if self.tp_size > 1:
            parts = [torch.empty_like(logits) for _ in range(self.tp_size)]
            dist.all_gather(parts, logits)
            logits = torch.cat(parts, dim=-1)
        return logits

    def weight_bytes(self) -> int:
        return sum(L[k].weight_bytes() for L in self.layers for k in ("qkv", "o", "gate_up", "down"))

    # -- generation --------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, new_tokens: int, use_graph: bool = True) -> dict:
        """Greedy decode. Returns generated tokens [B, new_tokens] and device-timed prefill/decode seconds."""
        B, P = prompt.shape
        assert B == self.batch and P + new_tokens <= self.max_seq
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
        logits = self.forward(prompt, torch.arange(P, device=self.dev))
        ev[1].record()
        tok = logits.argmax(-1, keepdim=True)
        out = torch.empty(B, new_tokens, dtype=torch.int64, device=self.dev)
        out[:, 0:1] = tok
        pos = torch.full((1,), P, dtype=torch.int64, device=self.dev)
        step_idx = torch.zeros(1, dtype=torch.int64, device=self.dev)

        lib = _native.load()
        flag = (_native.FLAG_BF16 if self.dtype == torch.bfloat16 else 0) | (_native.FLAG_PDL if self.pdl else 0)
        nxt = torch.empty(B, 1, dtype=torch.int64, device=self.dev)

        def step():
            logits16 = self.forward(tok, pos, fp32_logits=False).contiguous()
            _native.check(lib.matgptq_b200_argmax(logits16.data_ptr(), nxt.data_ptr(), B, logits16.shape[1], flag,
                                                  torch.cuda.current_stream(self.dev).cuda_stream), "argmax")
            tok.copy_(nxt)
            pos.add_(1)
            step_idx.add_(1)
            out.index_copy_(1, step_idx, nxt)

        graph = None
        if use_graph and new_tokens > 2:
            state = (tok.clone(), pos.clone(), step_idx.clone(), out.clone(), [k.clone() for k in self.k_cache], [v.clone() for v in self.v_cache])
            s = torch.cuda.Stream(device=self.dev)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                step()  # warm-up outside capture (loads kernels, NCCL buffers)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=s):
                    step()
            torch.cuda.current_stream().wait_stream(s)
            # rewind everything the two trial steps touched
            tok.copy_(state[0]); pos.copy_(state[1]); step_idx.copy_(state[2]); out.copy_(state[3])
            for k, k0 in zip(self.k_cache, state[4]):
                k.copy_(k0)
            for v, v0 in zip(self.v_cache, state[5]):
                v.copy_(v0)
        torch.cuda.synchronize()
        if self.tp_size > 1:
            dist.barrier()
        ev[2].record()
        for _ in range(new_tokens - 1):
            if graph is not None:
                graph.replay()
            else:
                step()
        ev[3].record()
        torch.cuda.synchronize()
        if graph is not None:
            graph.reset()  # a live graph holding NCCL kernels would block the process group's shutdown
        return {"tokens": out, "prefill_s": ev[0].elapsed_time(ev[1]) * 1e-3,
                "decode_s": ev[2].elapsed_time(ev[3]) * 1e-3, "decode_steps": new_tokens - 1}


def mixed_bitwidths(shape: LlamaShape, mean_bits: float, seed: int = 0) -> dict[str, int]:
    """Seeded heterogeneous per-layer assignment from {2,3,4,6,8} with the given parameter-weighted mean."""
    return synth.bitwidth_assignment(layer_names(shape), mean_bits, seed=seed)
