"""Decode throughput of the ``matgptq_quant`` method inside a vLLM engine on random-init weights.

    python -m matgptq_b200.vllm_bench --arch 8b --batch 1 8 32 --prompt-len 128 --new-tokens 128 --mean-bits 3.0

Stands in for the reference's ``vllm bench throughput`` recipe on a packed checkpoint
(``inference_lib/README.md:85-109``, ``inference_lib/inference_demo_vllm.py:16-30``) where no checkpoint
exists: a directory with only ``config.json`` (Llama-3.1 architecture, ``quantization_config`` of
``pack_quantized_model.py:134-141`` plus a per-layer bitwidth file) is loaded with ``load_format="dummy"``, so
vLLM builds the model, creates ``qweight``/``scales`` through ``MatGPTQLinearMethod.create_weights``, runs
``process_weights_after_loading`` (slice + pack on the GPU) and serves random prompt ids.  Prints one JSON line
per batch size: tokens/s of the whole request (prefill included) and of the decode phase alone (the same
request with one new token subtracted).  CUDA graphs without torch.compile by default (``--eager`` for neither).
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time

os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
os.environ.setdefault("HF_HUB_OFFLINE", "1")
os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def write_config_only_checkpoint(out_dir: str, arch: str, mean_bits: float, layers: int | None = None) -> dict:
    from transformers import LlamaConfig

    from . import decode
    from .bitwidth_config import write_bitwidth_config
    from .checkpoint import quantization_config
    shape = {"8b": decode.LLAMA31_8B, "70b": decode.LLAMA31_70B}[arch]
    if layers:
        shape = decode.LlamaShape(shape.hidden, shape.intermediate, shape.n_heads, shape.n_kv_heads, layers, shape.vocab)
    bits = decode.mixed_bitwidths(shape, mean_bits, seed=0)
    os.makedirs(out_dir, exist_ok=True)
    bits_path = os.path.join(out_dir, "bitwidths.txt")
    write_bitwidth_config(bits_path, bits)
    cfg = LlamaConfig(hidden_size=shape.hidden, intermediate_size=shape.intermediate, num_hidden_layers=shape.n_layers,
                      num_attention_heads=shape.n_heads, num_key_value_heads=shape.n_kv_heads, vocab_size=shape.vocab,
                      max_position_embeddings=8192, rms_norm_eps=shape.eps, rope_theta=shape.rope_theta,
                      tie_word_embeddings=False, torch_dtype="float16", bos_token_id=0, eos_token_id=1)
    d = cfg.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]
    q = quantization_config(128, 8, 4, "float16")
    q["bitwidth_config_path"] = bits_path
    d["quantization_config"] = q
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    names = decode.layer_names(shape)
    return {"mean_bits": sum(bits[n] * names[n] for n in names) / sum(names.values()), "layers": shape.n_layers}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", choices=["8b", "70b"], default="8b")
    ap.add_argument("--layers", type=int, default=0, help="fewer decoder layers than the architecture has (0 = all)")
    ap.add_argument("--batch", type=int, nargs="+", default=[1, 8, 32])
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--mean-bits", type=float, default=3.0)
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs either")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.5)
    args = ap.parse_args()

    import torch
    from vllm import LLM, SamplingParams

    import matgptq_b200.vllm_matgptq  # noqa: F401  registers "matgptq_quant"

    ckpt = tempfile.mkdtemp(prefix="matgptq_vllm_")
    info = write_config_only_checkpoint(ckpt, args.arch, args.mean_bits, args.layers or None)
    kwargs = dict(model=ckpt, load_format="dummy", skip_tokenizer_init=True, dtype=torch.float16,
                  tensor_parallel_size=args.tensor_parallel, max_model_len=args.prompt_len + args.new_tokens + 16,
                  gpu_memory_utilization=args.gpu_memory_utilization, seed=0, enable_prefix_caching=False,
                  max_num_seqs=max(args.batch))
    if args.eager:
        kwargs["enforce_eager"] = True
    else:
        kwargs["compilation_config"] = {"mode": 0, "cudagraph_mode": "FULL_DECODE_ONLY"}
    llm = LLM(**kwargs)
    g = torch.Generator().manual_seed(0)
    for batch in args.batch:
        prompts = [{"prompt_token_ids": torch.randint(2, 100000, (args.prompt_len,), generator=g).tolist()} for _ in range(batch)]

        def run(new_tokens: int) -> float:
            params = SamplingParams(temperature=0.0, max_tokens=new_tokens, detokenize=False, ignore_eos=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = llm.generate(prompts, params, use_tqdm=False)
            torch.cuda.synchronize()
            assert all(len(o.outputs[0].token_ids) == new_tokens for o in outs)
            return time.perf_counter() - t0

        run(8)  # warm-up: graphs, allocator
        t_full = min(run(args.new_tokens) for _ in range(2))
        t_one = min(run(1) for _ in range(2))
        decode_s = max(t_full - t_one, 1e-9)
        print("RESULT " + json.dumps({
            "engine": "vllm", "arch": args.arch, "layers": info["layers"], "mean_bits": round(info["mean_bits"], 3),
            "tp": args.tensor_parallel, "batch": batch, "prompt_len": args.prompt_len, "new_tokens": args.new_tokens,
            "cuda_graphs": not args.eager, "request_tok_per_s": round(batch * args.new_tokens / t_full, 1),
            "decode_tok_per_s": round(batch * (args.new_tokens - 1) / decode_s, 1),
            "decode_ms_per_token": round(decode_s / (args.new_tokens - 1) * 1e3, 4)}), flush=True)


if __name__ == "__main__":
    main()
