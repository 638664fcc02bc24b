"""Helper of tests/test_vllm_engine.py (run as a child process): bring a vLLM engine up on a packed
checkpoint through the ``matgptq_quant`` method and print what it generates as one JSON line.

    python tests/vllm_engine_run.py <packed dir> <tp size> <prompt ids, comma separated> <new tokens>

The plugin module must be imported in the process that builds the model; with
``VLLM_ENABLE_V1_MULTIPROCESSING=0`` that is this process (the reference's demo imports its module at the top
of the script the same way, ``inference_lib/inference_demo_vllm.py:7``).
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
os.environ.setdefault("HF_HUB_OFFLINE", "1")
os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def main() -> None:
    ckpt, tp, prompt, new_tokens = sys.argv[1], int(sys.argv[2]), [int(t) for t in sys.argv[3].split(",")], int(sys.argv[4])
    import torch
    from vllm import LLM, SamplingParams

    import matgptq_b200.vllm_matgptq  # noqa: F401  registers "matgptq_quant"

    llm = LLM(model=ckpt, tensor_parallel_size=tp, dtype=torch.float16, max_model_len=128, enforce_eager=True,
              gpu_memory_utilization=0.05, skip_tokenizer_init=True, seed=0, enable_prefix_caching=False)
    params = SamplingParams(temperature=0.0, max_tokens=new_tokens, logprobs=8, detokenize=False, ignore_eos=True)
    out = llm.generate([{"prompt_token_ids": prompt}], params, use_tqdm=False)[0].outputs[0]
    steps = []
    for lp in out.logprobs:
        steps.append({str(tok): float(v.logprob) for tok, v in lp.items()})
    print("RESULT " + json.dumps({"tokens": list(out.token_ids), "logprobs": steps}), flush=True)


if __name__ == "__main__":
    main()
