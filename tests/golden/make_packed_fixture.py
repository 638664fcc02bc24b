"""Builds ``tests/golden/packed_tiny_llama``: a packed checkpoint WRITTEN BY THE REFERENCE'S OWN PACKER.

    python tests/golden/make_packed_fixture.py /path/to/MatGPTQ-checkout

Steps (all on the CPU):
  1. a 2-layer Llama-architecture model (hidden 256, MLP 512, 4 heads / 2 KV heads, vocabulary 256) with
     seeded random weights is saved with ``transformers`` as ``model.safetensors`` + ``config.json``;
  2. every block linear is quantised to 8-bit master codes per group of 128 (symmetric min-max grid and
     round-to-nearest, the grid ``MatryoshkaQuantizer.find_params`` starts from) and stored the way the
     reference's calibration run stores a layer: ``<dir>/<layer name>/data.pt`` holding ``qweight``,
     ``scale``, ``zero`` and ``perm`` (``src/quantizer.py:185-193``);
  3. the reference's ``pack_quantized_model.pack_model`` (``pack_quantized_model.py:33-142``), imported from
     the checkout, turns both into the packed directory;
  4. next to it go a per-layer bitwidth file in the format of ``evo_quant_search.py:659-671`` and
     ``expected.json``: for a fixed prompt, the fp32 logits (top entries) of the model whose linears are the
     reference's ``dequantize()`` of those codes at the per-layer bitwidths, computed with ``transformers``.

The packed directory is what ``matgptq_b200.checkpoint``, the vLLM method and the HF-transformers path
must read; nothing in it was written by this repository's own checkpoint writer.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "packed_tiny_llama")
GROUP = 128
BITS_CYCLE = (4, 2, 8, 3, 6)  # per-layer bitwidths, cycled over the layers in checkpoint order
PROMPT = [3, 17, 42, 99, 128, 200, 7, 64, 255, 1, 33, 150]


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import pack_quantized_model as ref_packer  # the reference's packer
    from src.quant_utils_matgpqt import MatryoshkaQuantizer, dequantize  # the reference's grid and dequantiser
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=256, max_position_embeddings=256, rms_norm_eps=1e-5,
                      rope_theta=10000.0, tie_word_embeddings=False, torch_dtype="float16",
                      bos_token_id=0, eos_token_id=1)
    model = LlamaForCausalLM(cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.copy_(torch.randn_like(p) * (0.08 if "embed" in name or "lm_head" in name else 0.06))
            else:
                p.copy_(1.0 + 0.1 * torch.randn_like(p))
    model = model.half()

    tmp = tempfile.mkdtemp(prefix="matgptq_fixture_")
    dense_dir, quant_dir = os.path.join(tmp, "dense"), os.path.join(tmp, "quant")
    model.save_pretrained(dense_dir, safe_serialization=True)

    layer_bits, dense_weights = {}, {}
    linears = [(n, m) for n, m in model.named_modules()
               if isinstance(m, torch.nn.Linear) and not ref_packer.should_skip_quantisation(n)]
    for i, (name, mod) in enumerate(linears):
        w = mod.weight.detach().float()
        n_out, n_in = w.shape
        quantizer = MatryoshkaQuantizer()
        quantizer.configure(bits=8, perchannel=True, sym=True)
        quantizer.find_params(w.reshape(-1, GROUP), weight=True)
        scale = quantizer.scale.reshape(n_out, n_in // GROUP).half()
        zero = quantizer.zero.reshape(n_out, n_in // GROUP).half()
        q = torch.clamp(torch.round(w.reshape(n_out, -1, GROUP) / scale.float()[..., None] + zero.float()[..., None]), 0, 255)
        q = q.to(torch.uint8).reshape(n_out, n_in)
        os.makedirs(os.path.join(quant_dir, name), exist_ok=True)
        torch.save({"qweight": q, "scale": scale, "zero": zero, "perm": None}, os.path.join(quant_dir, name, "data.pt"))
        bits = BITS_CYCLE[i % len(BITS_CYCLE)]
        layer_bits[name] = bits
        dense_weights[name] = dequantize(q.reshape(n_out, -1, GROUP), scale[..., None], zero[..., None], 8, bits).reshape(n_out, n_in)

    if os.path.isdir(OUT):
        shutil.rmtree(OUT)
    ref_packer.pack_model(model_name_or_path=dense_dir, quantised_dir=quant_dir, output_dir=OUT, group_size=GROUP,
                          master_bitwidth=8, inference_bitwidth=4, quant_dtype="float16")

    with open(os.path.join(OUT, "bitwidths.txt"), "w") as f:  # evo_quant_search.py:659-671
        for name, bits in layer_bits.items():
            f.write(f"{name}: {bits}\n")

    # expected logits: the dense model whose linears are the reference's dequantised weights, fp32 on the CPU
    ref_model = LlamaForCausalLM(cfg).float()
    ref_model.load_state_dict({k: v.float() for k, v in model.state_dict().items()})
    with torch.no_grad():
        for name, mod in ref_model.named_modules():
            if name in dense_weights:
                mod.weight.copy_(dense_weights[name].float())
        ids = torch.tensor([PROMPT])
        steps, tokens, logits_top = 8, [], []
        for _ in range(steps):
            logits = ref_model(ids).logits[0, -1]
            top = torch.topk(logits, 8)
            logits_top.append({"ids": top.indices.tolist(), "logits": [round(float(v), 5) for v in top.values],
                               "logsumexp": round(float(torch.logsumexp(logits, 0)), 5)})
            tokens.append(int(top.indices[0]))
            ids = torch.cat([ids, top.indices[:1][None]], dim=1)
    with open(os.path.join(OUT, "expected.json"), "w") as f:
        json.dump({"prompt": PROMPT, "greedy_tokens": tokens, "steps": logits_top, "layer_bits": layer_bits}, f, indent=1)
    shutil.rmtree(tmp)
    print("wrote", OUT, sorted(os.listdir(OUT)))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
