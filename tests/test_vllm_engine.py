"""The ``matgptq_quant`` method inside a real vLLM engine, on a checkpoint the reference's packer wrote.

``LLM(model=<packed dir>)`` (``inference_lib/inference_demo_vllm.py:23-30``) finds the method through
``config.json``'s ``quantization_config``, builds the fused qkv / gate_up layers with vLLM's own weight
loaders, runs ``process_weights_after_loading`` and ``apply``.  The generated tokens and their
log-probabilities are compared with the record made from the reference's ``dequantize()``
(tests/golden/packed_tiny_llama/expected.json): uniform 4 bits would not match it, the per-layer
bitwidth file (2 to 8 bits, several bitwidths inside one fused layer) does.
"""
import json
import os
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURE = os.path.join(HERE, "golden", "packed_tiny_llama")


def _run_engine(ckpt: str, tp: int, prompt, new_tokens: int) -> dict:
    cmd = [sys.executable, os.path.join(HERE, "vllm_engine_run.py"), ckpt, str(tp), ",".join(map(str, prompt)), str(new_tokens)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("RESULT ")]
    assert proc.returncode == 0 and lines, f"vLLM engine run failed (rc {proc.returncode}):\n{proc.stdout[-3000:]}\n{proc.stderr[-6000:]}"
    return json.loads(lines[-1][len("RESULT "):])


def test_engine_generates_the_recorded_tokens(tmp_path):
    with open(os.path.join(FIXTURE, "expected.json")) as f:
        expected = json.load(f)
    ckpt = str(tmp_path / "packed")
    shutil.copytree(FIXTURE, ckpt)
    # the addition to the reference's config: a per-layer bitwidth file (the format of evo_quant_search.py:659-671)
    with open(os.path.join(ckpt, "config.json")) as f:
        config = json.load(f)
    config["quantization_config"]["bitwidth_config_path"] = os.path.join(ckpt, "bitwidths.txt")
    with open(os.path.join(ckpt, "config.json"), "w") as f:
        json.dump(config, f)
    got = _run_engine(ckpt, 1, expected["prompt"], len(expected["greedy_tokens"]))
    assert got["tokens"] == expected["greedy_tokens"]
    for step, lp in zip(expected["steps"], got["logprobs"]):
        for tok, logit in zip(step["ids"][:4], step["logits"][:4]):
            want = logit - step["logsumexp"]
            assert str(tok) in lp and abs(lp[str(tok)] - want) <= 5e-2, (tok, lp.get(str(tok)), want)
