"""Checkpoint layout, per-layer bitwidth files and the vLLM method, as far as they run without a GPU;
the GPU test at the end runs the method's load path and forward against the oracle."""
import json
import os

import pytest
import torch

from matgptq_b200 import bitwidth_config as bc
from matgptq_b200 import checkpoint as ck
from oracle import matgptq_oracle as oracle


def test_bitwidth_file_roundtrip(tmp_path):
    bits = {"model.layers.0.self_attn.q_proj": 2, "model.layers.0.mlp.down_proj": 8, "model.layers.1.mlp.up_proj": 3}
    path = str(tmp_path / "evo-configuration-3.0.txt")
    bc.write_bitwidth_config(path, bits)
    assert open(path).read().splitlines()[0] == "model.layers.0.self_attn.q_proj: 2"
    assert bc.read_bitwidth_config(path) == bits
    with pytest.raises(ValueError):
        bc.write_bitwidth_config(path, {"x": 5})
    (tmp_path / "bad.txt").write_text("model.layers.0.q_proj 4\n")
    with pytest.raises(ValueError):
        bc.read_bitwidth_config(str(tmp_path / "bad.txt"))


def test_resolve_bitwidths_for_fused_layers():
    bits = {"model.layers.0.self_attn.q_proj": 2, "model.layers.0.self_attn.v_proj": 6, "model.layers.0.mlp.up_proj": 3}
    assert bc.resolve_bitwidths("model.layers.0.self_attn.qkv_proj", 3, 4, bits) == [2, 4, 6]
    assert bc.resolve_bitwidths("model.layers.0.mlp.gate_up_proj", 2, 4, bits) == [4, 3]
    assert bc.resolve_bitwidths("model.layers.0.self_attn.o_proj", 1, 4, bits) == [4]
    assert bc.resolve_bitwidths("model.layers.0.self_attn.qkv_proj", 3, 8, None) == [8, 8, 8]


def test_synthetic_checkpoint_layout(tmp_path):
    shapes = ck.llama_linear_shapes(hidden=256, intermediate=512, n_heads=4, n_kv_heads=2, n_layers=2)
    assert len(shapes) == 14 and shapes["model.layers.1.self_attn.k_proj"] == (128, 256)
    dense = {"model.embed_tokens.weight": torch.zeros(32, 256, dtype=torch.float16),
             "model.norm.weight": torch.ones(256, dtype=torch.float16), "lm_head.weight": torch.zeros(32, 256, dtype=torch.float16)}
    bits = {name: (2, 3, 4, 6, 8)[i % 5] for i, name in enumerate(shapes)}
    out = str(tmp_path / "packed")
    ck.write_synthetic_checkpoint(out, shapes, inference_bitwidth=4, quant_dtype="float16", dense_tensors=dense,
                                  layer_bitwidths=bits, base_config={"architectures": ["LlamaForCausalLM"]},
                                  shard_bytes=256 * 1024)
    qcfg = ck.read_checkpoint_config(out)
    assert qcfg["quant_method"] == "matgptq_quant" and qcfg["modules_to_not_convert"] == ["lm_head", "norm"]
    assert set(qcfg) >= {"group_size", "master_bitwidth", "inference_bitwidth", "quant_dtype"}
    index = json.load(open(os.path.join(out, "model.safetensors.index.json")))
    names = set(index["weight_map"])
    assert "model.layers.0.mlp.down_proj.qweight" in names and "model.layers.0.mlp.down_proj.scales" in names
    assert not any(n.endswith("_proj.weight") for n in names) and "lm_head.weight" in names
    q, s = ck.load_linear(out, "model.layers.1.mlp.down_proj")
    assert q.dtype == torch.uint8 and q.shape == (256, 512) and s.shape == (256, 4) and s.dtype == torch.float16
    assert bc.read_bitwidth_config(os.path.join(out, "bitwidths.txt")) == bits
    # master codes are unsliced 8-bit codes and dequantise to something weight-like
    w = oracle.dequantize_weight(q, s, torch.full_like(s, 128.0), 8, 8)
    assert q.max() > 200 and 0.005 < w.float().std() < 0.05
    assert ck.should_skip_quantisation("model.layers.0.input_layernorm") and ck.should_skip_quantisation("lm_head")
    (tmp_path / "plain").mkdir()
    (tmp_path / "plain" / "config.json").write_text("{}")
    with pytest.raises(ValueError):
        ck.read_checkpoint_config(str(tmp_path / "plain"))


@pytest.fixture(scope="module")
def plugin():
    return pytest.importorskip("matgptq_b200.vllm_matgptq", reason="vllm not importable")


def test_vllm_config_surface(plugin, tmp_path):
    from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS, get_quantization_config
    assert "matgptq_quant" in QUANTIZATION_METHODS
    assert get_quantization_config("matgptq_quant") is plugin.MatGPTQConfig
    base = {"group_size": 128, "master_bitwidth": 8, "inference_bitwidth": 3, "quant_dtype": "bfloat16",
            "modules_to_not_convert": ["lm_head", "norm"], "quant_method": "matgptq_quant"}
    cfg = plugin.MatGPTQConfig.from_config(base)
    assert cfg.get_name() == "matgptq_quant" and cfg.inference_bitwidth == 3 and cfg.quant_dtype == torch.bfloat16
    assert cfg.flag == 3 and cfg.layer_bitwidths is None and cfg.get_config_filenames() == []
    for missing in ("group_size", "master_bitwidth", "inference_bitwidth", "quant_dtype", "modules_to_not_convert"):
        with pytest.raises(ValueError):
            plugin.MatGPTQConfig.from_config({k: v for k, v in base.items() if k != missing})
    path = str(tmp_path / "bits.txt")
    bc.write_bitwidth_config(path, {"model.layers.0.self_attn.k_proj": 2})
    cfg = plugin.MatGPTQConfig.from_config({**base, "bitwidth_config_path": path, "layer_bitwidths": {"a.b": 6}})
    assert cfg.layer_bitwidths == {"model.layers.0.self_attn.k_proj": 2, "a.b": 6}
    with pytest.raises(AssertionError):
        plugin.MatGPTQConfig(group_size=64)


class _FakeLinear(torch.nn.Module):
    pass


@pytest.fixture
def single_rank_tp(monkeypatch):
    """vLLM's parameter classes ask the tensor-parallel state for rank and size; stand in for a
    one-rank group so that they can be built outside an engine."""
    import vllm.model_executor.parameter as vp
    monkeypatch.setattr(vp, "get_tensor_model_parallel_rank", lambda: 0)
    monkeypatch.setattr(vp, "get_tensor_model_parallel_world_size", lambda: 1)


def test_vllm_method_create_weights(plugin, single_rank_tp):
    cfg = plugin.MatGPTQConfig(128, 8, 4, "float16", ["lm_head", "norm"], {"model.layers.0.self_attn.k_proj": 2})
    method = plugin.MatGPTQLinearMethod(cfg, "model.layers.0.self_attn.qkv_proj")
    layer = _FakeLinear()
    method.create_weights(layer, 512, [256, 64, 64], 512, 384, torch.float16, weight_loader=lambda *a, **k: None)
    assert layer.qweight.dtype == torch.uint8 and tuple(layer.qweight.shape) == (384, 512)
    assert tuple(layer.scales.shape) == (384, 4) and layer.scales.dtype == torch.float16
    assert layer.matgptq_bits == [4, 2, 4] and layer.matgptq_partitions == [256, 64, 64]
    assert layer.qweight.input_dim == 1 and layer.qweight.output_dim == 0
    with pytest.raises(ValueError):
        method.create_weights(_FakeLinear(), 448, [256], 448, 256, torch.float16, weight_loader=None)
    # layers the config excludes stay unquantised, non-linear layers get no method
    from vllm.model_executor.layers.linear import UnquantizedLinearMethod
    assert isinstance(cfg.get_quant_method(_FakeLinear(), "lm_head"), UnquantizedLinearMethod)
    assert cfg.get_quant_method(_FakeLinear(), "model.layers.0.mlp.act") is None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,qd", [(torch.float16, "float16"), (torch.bfloat16, "bfloat16")])
@pytest.mark.parametrize("m", [1, 7, 40])
def test_vllm_method_load_and_apply(plugin, single_rank_tp, cuda, dtype, qd, m):
    from matgptq_b200 import synth
    cfg = plugin.MatGPTQConfig(128, 8, 4, qd, ["lm_head", "norm"],
                               {"model.layers.0.self_attn.q_proj": 3, "model.layers.0.self_attn.v_proj": 8})
    method = plugin.MatGPTQLinearMethod(cfg, "model.layers.0.self_attn.qkv_proj")
    parts, n_in = [256, 64, 64], 512
    layer = _FakeLinear()
    method.create_weights(layer, n_in, parts, n_in, sum(parts), dtype, weight_loader=lambda *a, **k: None)
    src = synth.make_layer(sum(parts), n_in, 128, seed=5, dtype=dtype)
    layer.qweight.data.copy_(src.qweight)
    layer.scales.data.copy_(src.scales)
    layer.to(cuda)
    method.process_weights_after_loading(layer)
    assert not hasattr(layer, "qweight") and [b for _, b in layer.matgptq_segments] == [3, 4, 8]
    x = synth.make_activations(m, n_in, seed=m, dtype=dtype, device=cuda).reshape(1, m, n_in)
    bias = torch.randn(sum(parts), dtype=dtype, device=cuda)
    y = method.apply(layer, x, bias)
    assert y.shape == (1, m, sum(parts)) and y.dtype == dtype
    rows, w_parts = 0, []
    for p, b in zip(parts, [3, 4, 8]):
        w_parts.append(oracle.dequantize_weight(src.qweight[rows:rows + p], src.scales[rows:rows + p],
                                                src.zeros[rows:rows + p], 8, b))
        rows += p
    y_ref = oracle.linear_fp32_accumulate(x.cpu()[0], torch.cat(w_parts)) + bias.cpu().float()
    assert oracle.rel_err(y.cpu()[0], y_ref) <= 1e-2


def test_checkpoint_with_zero_points(tmp_path):
    shapes = {"model.layers.0.mlp.down_proj": (256, 512)}
    out = str(tmp_path / "asym")
    qcfg = ck.write_synthetic_checkpoint(out, shapes, inference_bitwidth=4, sym=False)
    assert qcfg["zero_points"] is True and ck.read_checkpoint_config(out)["zero_points"] is True
    q, s, z = ck.load_linear(out, "model.layers.0.mlp.down_proj", with_zeros=True)
    assert z is not None and z.shape == s.shape and z.dtype == s.dtype and z.float().min() < 120 < 136 < z.float().max()
    out_sym = str(tmp_path / "sym")
    assert "zero_points" not in ck.write_synthetic_checkpoint(out_sym, shapes, inference_bitwidth=4)
    assert ck.load_linear(out_sym, "model.layers.0.mlp.down_proj", with_zeros=True)[2] is None


@pytest.mark.gpu
def test_vllm_method_with_zero_points(plugin, single_rank_tp, cuda):
    from matgptq_b200 import synth
    cfg = plugin.MatGPTQConfig.from_config({"group_size": 128, "master_bitwidth": 8, "inference_bitwidth": 4,
                                            "quant_dtype": "float16", "modules_to_not_convert": ["lm_head", "norm"],
                                            "zero_points": True})
    assert cfg.zero_points
    method = plugin.MatGPTQLinearMethod(cfg, "model.layers.0.mlp.down_proj")
    n_out, n_in, m = 256, 512, 3
    layer = _FakeLinear()
    method.create_weights(layer, n_in, [n_out], n_in, n_out, torch.float16, weight_loader=lambda *a, **k: None)
    assert tuple(layer.zeros.shape) == (n_out, 4)
    src = synth.make_layer(n_out, n_in, 128, seed=8, sym=False, dtype=torch.float16)
    layer.qweight.data.copy_(src.qweight)
    layer.scales.data.copy_(src.scales)
    layer.zeros.data.copy_(src.zeros)
    layer.to(cuda)
    method.process_weights_after_loading(layer)
    assert not hasattr(layer, "zeros") and len(layer.matgptq_zeros) == 1
    x = synth.make_activations(m, n_in, seed=1, dtype=torch.float16, device=cuda)
    y = method.apply(layer, x)
    w = oracle.dequantize_weight(src.qweight, src.scales, src.zeros, 8, 4)
    assert oracle.rel_err(y.cpu(), oracle.linear_fp32_accumulate(x.cpu(), w)) <= 1e-2
