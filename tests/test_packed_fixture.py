"""A packed checkpoint written by the reference's own packer (tests/golden/packed_tiny_llama, made by
tests/golden/make_packed_fixture.py from pack_quantized_model.py:33-142) read by this package's checkpoint
reader, per-layer bitwidth reader and HF-transformers path.  expected.json holds the fp32 logits of the model
whose linears are the reference's dequantize() of the same codes at the per-layer bitwidths."""
import json
import os

import pytest
import torch

from matgptq_b200 import bitwidth_config as bc
from matgptq_b200 import checkpoint as ck
from oracle import matgptq_oracle as oracle

FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "packed_tiny_llama")


@pytest.fixture(scope="module")
def expected():
    with open(os.path.join(FIXTURE, "expected.json")) as f:
        return json.load(f)


def test_reference_packed_layout_is_read(expected):
    qcfg = ck.read_checkpoint_config(FIXTURE)
    assert qcfg == {"group_size": 128, "modules_to_not_convert": ["lm_head", "norm"], "master_bitwidth": 8,
                    "inference_bitwidth": 4, "quant_method": "matgptq_quant", "quant_dtype": "float16"}
    names = {k for k, _ in ck.iter_checkpoint_tensors(FIXTURE)}
    bits = bc.read_bitwidth_config(os.path.join(FIXTURE, "bitwidths.txt"))
    assert bits == expected["layer_bits"] and len(bits) == 14
    for layer in bits:
        assert f"{layer}.qweight" in names and f"{layer}.scales" in names and f"{layer}.weight" not in names
        q, s = ck.load_linear(FIXTURE, layer)
        assert q.dtype == torch.uint8 and s.dtype == torch.float16 and s.shape == (q.shape[0], q.shape[1] // 128)
        assert int(q.max()) > 200 and int(q.min()) < 50  # master codes, unsliced
    # what the packer leaves dense
    assert {"lm_head.weight", "model.embed_tokens.weight", "model.norm.weight"} <= names


def _dense_model_from_fixture(bits):
    """transformers Llama in fp32 whose linears are the ORACLE's dequantised weights of the fixture's codes."""
    from transformers import AutoConfig, AutoModelForCausalLM
    config = AutoConfig.from_pretrained(FIXTURE)
    delattr(config, "quantization_config")
    model = AutoModelForCausalLM.from_config(config, torch_dtype=torch.float32)
    state = {k: v.float() for k, v in ck.iter_checkpoint_tensors(FIXTURE) if not k.endswith((".qweight", ".scales"))}
    for layer, b in bits.items():
        q, s = ck.load_linear(FIXTURE, layer)
        state[f"{layer}.weight"] = oracle.dequantize_weight(q, s, torch.full_like(s, 128.0), 8, b).float()
    model.load_state_dict(state, strict=True)
    return model.eval()


def test_oracle_on_reference_packed_checkpoint_reproduces_the_recorded_logits(expected):
    model = _dense_model_from_fixture(expected["layer_bits"])
    with torch.no_grad():
        logits = model(torch.tensor([expected["prompt"]])).logits[0, -1]
    step0 = expected["steps"][0]
    got = logits[torch.tensor(step0["ids"])]
    assert torch.allclose(got, torch.tensor(step0["logits"]), atol=2e-4)
    assert abs(float(torch.logsumexp(logits, 0)) - step0["logsumexp"]) < 2e-4


def _check_logits(logits_last, step, atol):
    got = logits_last.float().cpu()[torch.tensor(step["ids"])]
    assert torch.allclose(got, torch.tensor(step["logits"]), atol=atol), (got, step["logits"])
    assert int(logits_last.argmax()) == step["ids"][0]


@pytest.mark.gpu
def test_hf_path_from_packed_checkpoint(cuda, expected):
    """load -> replace every linear by MatGPTQLinear at its own bitwidth -> logits and greedy tokens of the
    recorded model, eagerly over a StaticCache."""
    from matgptq_b200 import hf_transformers as hf
    from matgptq_b200.matgptq_linear import MatGPTQLinear
    model = hf.load_packed_causal_lm(FIXTURE, os.path.join(FIXTURE, "bitwidths.txt"), cuda)
    replaced = {n: m.bitwidth for n, m in model.named_modules() if isinstance(m, MatGPTQLinear)}
    assert replaced == expected["layer_bits"]
    ids = torch.tensor([expected["prompt"]], device=cuda)
    with torch.no_grad():
        logits = model(ids).logits[0, -1]
    _check_logits(logits, expected["steps"][0], atol=3e-2)  # fp16 model against the fp32 record
    dec = hf.StaticCacheDecoder(model, compile_forward=False)
    tokens = dec.generate(ids, len(expected["greedy_tokens"]))
    assert tokens[0].tolist() == expected["greedy_tokens"]


@pytest.mark.gpu
def test_hf_path_from_quantiser_directories(cuda, expected, tmp_path):
    """The reference's own input format: one directory per layer with data.pt (src/quantizer.py:185-193),
    uniform bitwidth and per-layer file."""
    from matgptq_b200 import hf_transformers as hf
    from transformers import AutoConfig, AutoModelForCausalLM
    for layer in expected["layer_bits"]:
        q, s = ck.load_linear(FIXTURE, layer)
        os.makedirs(tmp_path / layer)
        torch.save({"qweight": q, "scale": s, "zero": torch.full_like(s, 128.0), "perm": None}, tmp_path / layer / "data.pt")
    config = AutoConfig.from_pretrained(FIXTURE)
    delattr(config, "quantization_config")

    def dense():
        model = AutoModelForCausalLM.from_config(config, torch_dtype=torch.float16)
        model.load_state_dict({k: v for k, v in ck.iter_checkpoint_tensors(FIXTURE)
                               if not k.endswith((".qweight", ".scales"))}, strict=False)
        return model.to(cuda).eval()

    ids = torch.tensor([expected["prompt"]], device=cuda)
    mixed = hf.replace_with_matgptq_linear(dense(), str(tmp_path), os.path.join(FIXTURE, "bitwidths.txt"), 8, 8, 128)
    with torch.no_grad():
        _check_logits(mixed(ids).logits[0, -1], expected["steps"][0], atol=3e-2)
    # uniform 8 bits = the master codes themselves: compare with the oracle-weight model in fp32
    uniform = hf.replace_with_matgptq_linear(dense(), str(tmp_path), None, 8, 8, 128)
    ref = _dense_model_from_fixture({k: 8 for k in expected["layer_bits"]})
    with torch.no_grad():
        a = uniform(ids).logits[0, -1].float().cpu()
        b = ref(ids.cpu()).logits[0, -1]
    assert (a - b).abs().max() <= 3e-2 and int(a.argmax()) == int(b.argmax())


@pytest.mark.gpu
def test_operators_are_traceable(cuda, expected):
    """What the reference's compiled decode loop (torch.compile(fullgraph=True, mode="reduce-overhead") over a
    StaticCache, inference_demo_transformers.py:141-173) needs from the operators: a schema that matches what
    they do (no hidden mutation) and a fake implementation whose output metadata equals the real output's.
    torch.library.opcheck runs both and compares; the timing protocol of bench_transformers_e2e.py runs on the
    eager StaticCache loop."""
    from matgptq_b200 import hf_transformers as hf
    from matgptq_b200.matgptq_linear import MatGPTQLinear
    model = hf.load_packed_causal_lm(FIXTURE, os.path.join(FIXTURE, "bitwidths.txt"), cuda)
    lin = next(m for m in model.modules() if isinstance(m, MatGPTQLinear))
    for rows in (1, 40):
        x = torch.randn(rows, lin.n_in_features, dtype=torch.float16, device=cuda)
        args = (x, lin.matgptq_qweight.data, lin.matgptq_scales.data, lin.n_out_features, lin.n_in_features,
                lin.bitwidth, lin.group_size, int(lin.flag))
        torch.library.opcheck(torch.ops.matgptq_cuda.matmul_matgptq.default, args,
                              test_utils=("test_schema", "test_faketensor"))
    x = torch.randn(3, lin.n_in_features, dtype=torch.float16, device=cuda)
    gargs = (x, [lin.matgptq_qweight.data, lin.matgptq_qweight.data], [lin.matgptq_scales.data, lin.matgptq_scales.data],
             [lin.n_out_features, lin.n_out_features], lin.n_in_features, [lin.bitwidth, lin.bitwidth], lin.group_size,
             int(lin.flag))
    torch.library.opcheck(torch.ops.matgptq_cuda.matmul_matgptq_grouped.default, gargs,
                          test_utils=("test_schema", "test_faketensor"))
    ids = torch.tensor([expected["prompt"]], device=cuda)
    times = hf.StaticCacheDecoder(model, compile_forward=False).time_decode(ids, benchmark_runs=2, number_of_runs=16, warmups=16)
    assert len(times) == 2 and all(t > 0 for t in times)


@pytest.mark.gpu
def test_hf_static_cache_decode_under_torch_compile(cuda, expected):
    """The reference's decode loop: torch.compile(fullgraph=True, mode="reduce-overhead") over a StaticCache
    (inference_demo_transformers.py:141-173).  The compiled loop must give the eager loop's tokens.  inductor
    also emits host C++ and builds it with the machine's g++; where that toolchain cannot (no libgomp.spec on
    some boxes) the step is still traced as one full graph with fake tensors, which is what the operator's
    fake registration is for, and the traced graph runs with the ordinary kernels."""
    from matgptq_b200 import hf_transformers as hf
    model = hf.load_packed_causal_lm(FIXTURE, os.path.join(FIXTURE, "bitwidths.txt"), cuda)
    ids = torch.tensor([expected["prompt"]], device=cuda)
    compiled = hf.StaticCacheDecoder(model, compile_forward=True)
    try:
        tokens = compiled.generate(ids, len(expected["greedy_tokens"]))
    except Exception as e:  # noqa: BLE001
        if "CppCompileError" not in repr(e) and "CppCompileError" not in str(e):
            raise
        torch._dynamo.reset()
        compiled = hf.StaticCacheDecoder(model, compile_forward=True, backend="eager")
        tokens = compiled.generate(ids, len(expected["greedy_tokens"]))
    assert tokens[0].tolist() == expected["greedy_tokens"]
