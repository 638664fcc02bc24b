"""HF-transformers path of the packed linear layer: swap ``nn.Linear`` for ``MatGPTQLinear`` and decode
over a static KV cache.

Mirrors the second serving loop of the reference, ``inference_lib/inference_demo_transformers.py``:
``replace_with_matgptq_linear`` (``:17-57``: per layer ``data.pt`` -> slice -> ``MatGPTQLinear``; per-layer
bitwidths from a ``name: bits`` file, ``:45-49``), ``decode_one_tokens`` (``:60-70``) and the ``StaticCache``
loop compiled with ``torch.compile(fullgraph=True, mode="reduce-overhead")`` (``:141-173``); the timing
protocol is the one of ``inference_lib/bench_transformers_e2e.py:61-76,187-190`` (16 warm-ups, 16 runs of 16
decode steps).  Additions: the layers can also come from a packed checkpoint directory (the layout of
``pack_quantized_model.py``), and slicing is fused into packing on the GPU instead of torch ops on the host.
"""
from __future__ import annotations

import os
import time
from typing import Optional, Union

import torch

from . import checkpoint
from .bitwidth_config import read_bitwidth_config
from .matgptq_linear import MatGPTQLinear


def _set_submodule(model: torch.nn.Module, layer_name: str, new: torch.nn.Module) -> None:
    *parent_path, attr = layer_name.split(".")
    parent = model.get_submodule(".".join(parent_path)) if parent_path else model
    setattr(parent, attr, new)


def replace_with_matgptq_linear(
    model: torch.nn.Module,
    quantized_weights_path: Union[str, os.PathLike],
    quantized_config_path: Optional[str] = None,
    master_bitwidth: int = 8,
    slice_bitwidth: int = 8,
    group_size: int = 128,
    device: Union[str, torch.device] = "cuda",
):
    """Same arguments and behaviour as ``inference_demo_transformers.py:17-57``.

    ``quantized_weights_path`` is either the quantiser's output (one directory per layer holding
    ``data.pt`` with ``qweight`` and ``scale``, ``src/quantizer.py:185-193``) or, as an addition, a packed
    checkpoint directory.  With ``quantized_config_path`` only the layers the file names are replaced,
    each at its own bitwidth; without it every layer found is replaced at ``slice_bitwidth``."""
    path = str(quantized_weights_path)
    packed = os.path.exists(os.path.join(path, "config.json"))
    if packed:
        checkpoint.read_checkpoint_config(path)
        found = sorted({k[:-len(".qweight")] for k, _ in checkpoint.iter_checkpoint_tensors(path) if k.endswith(".qweight")})
    else:
        found = sorted(n for n in os.listdir(path) if os.path.isdir(os.path.join(path, n)))

    def _load(layer_name: str):
        if packed:
            return checkpoint.load_linear(path, layer_name)
        data = torch.load(os.path.join(path, layer_name, "data.pt"), weights_only=True)
        return data["qweight"], data["scale"]

    def _replace(layer_name: str, bitwidth: int) -> None:
        qweight, scale = _load(layer_name)
        _set_submodule(model, layer_name, MatGPTQLinear.from_master(
            qweight.to(device), scale.to(device), master_bitwidth, bitwidth, group_size))

    if quantized_config_path:
        for layer_name, bitwidth in read_bitwidth_config(quantized_config_path).items():
            _replace(layer_name, bitwidth)
    else:
        for layer_name in found:
            _replace(layer_name, slice_bitwidth)
    return model


def load_packed_causal_lm(ckpt_dir: str, quantized_config_path: Optional[str] = None,
                          device: Union[str, torch.device] = "cuda"):
    """Addition: a ``transformers`` causal LM straight from a packed checkpoint directory.  The dense tensors
    (embeddings, norms, ``lm_head``) come from the safetensors, every ``<L>.qweight``/``<L>.scales`` pair becomes
    a ``MatGPTQLinear`` at the bitwidth of ``quantized_config_path`` or the checkpoint's ``inference_bitwidth``."""
    from transformers import AutoConfig, AutoModelForCausalLM
    qcfg = checkpoint.read_checkpoint_config(ckpt_dir)
    config = AutoConfig.from_pretrained(ckpt_dir)
    if hasattr(config, "quantization_config"):
        delattr(config, "quantization_config")  # transformers has no quantiser of that name; the layers are swapped below
    dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16}[qcfg["quant_dtype"]]
    model = AutoModelForCausalLM.from_config(config, torch_dtype=dtype)
    dense = {k: v for k, v in checkpoint.iter_checkpoint_tensors(ckpt_dir)
             if not k.endswith((".qweight", ".scales", ".zeros"))}
    missing, unexpected = model.load_state_dict(dense, strict=False)
    if unexpected:
        raise ValueError(f"{ckpt_dir}: tensors the model does not have: {unexpected[:4]}")
    model = model.to(device).eval()
    replace_with_matgptq_linear(model, ckpt_dir, quantized_config_path, qcfg["master_bitwidth"],
                                qcfg["inference_bitwidth"], qcfg["group_size"], device)
    still_missing = [k for k in missing if k.endswith(".weight") and isinstance(
        model.get_submodule(k[:-len(".weight")]), torch.nn.Linear) and "lm_head" not in k]
    if still_missing:
        raise ValueError(f"{ckpt_dir}: linear layers with neither dense nor packed weights: {still_missing[:4]}")
    return model


def decode_one_tokens(model, cur_token, input_pos, cache_position, past_key_values):
    """One greedy decode step (``inference_demo_transformers.py:60-70``)."""
    logits = model(cur_token, position_ids=input_pos, cache_position=cache_position,
                   past_key_values=past_key_values, return_dict=False, use_cache=True)[0]
    return torch.argmax(logits[:, -1], dim=-1)[:, None]


class StaticCacheDecoder:
    """Prefill + token-by-token greedy decode over a ``StaticCache`` (``inference_demo_transformers.py:141-173``)."""

    def __init__(self, model, compile_forward: bool = True, backend: str = "inductor"):
        """``backend="inductor"`` is the reference's setting (``mode="reduce-overhead"``: generated kernels
        for the model's own elementwise work plus CUDA-graph replay).  Any other dynamo backend name traces
        the same step as one full graph (fake tensors, so the operator's fake registration is exercised)
        without inductor; ``"eager"`` then runs the traced graph with the ordinary kernels, for hosts whose
        C++ toolchain cannot build inductor's host code."""
        self.model = model
        self.compile_forward = compile_forward
        self.backend = backend
        self._decode = None

    def _decode_fn(self):
        if self._decode is None:
            if not self.compile_forward:
                self._decode = decode_one_tokens
            elif self.backend == "inductor":
                torch._dynamo.config.capture_scalar_outputs = True
                self._decode = torch.compile(decode_one_tokens, fullgraph=True, dynamic=True, mode="reduce-overhead")
            else:
                self._decode = torch.compile(decode_one_tokens, fullgraph=True, backend=self.backend)
        return self._decode

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, max_new_tokens: int):
        from transformers import StaticCache
        dev, seq_len = input_ids.device, input_ids.shape[1]
        cache = StaticCache(config=self.model.config, max_cache_len=seq_len + max_new_tokens, max_batch_size=input_ids.shape[0],
                            device=dev, dtype=self.model.dtype)
        cache_position = torch.arange(seq_len, dtype=torch.int64, device=dev)
        logits = self.model(input_ids, cache_position=cache_position, past_key_values=cache, return_dict=False,
                            use_cache=True)[0]
        return logits[:, -1], cache

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        """Returns the ``[B, max_new_tokens]`` greedy continuation."""
        dev, seq_len = input_ids.device, input_ids.shape[1]
        last_logits, cache = self.prefill(input_ids, max_new_tokens)
        next_token = torch.argmax(last_logits, dim=-1)[:, None]
        out = [next_token]
        decode = self._decode_fn()
        cache_position = torch.tensor([seq_len], device=dev)
        for _ in range(1, max_new_tokens):
            next_token = decode(self.model, next_token.clone(), None, cache_position, cache)
            out.append(next_token.clone())
            cache_position += 1
        return torch.cat(out, dim=1)

    @torch.no_grad()
    def time_decode(self, input_ids: torch.Tensor, benchmark_runs: int = 16, number_of_runs: int = 16, warmups: int = 16):
        """Seconds per decode step, one mean per run of ``number_of_runs`` steps (the protocol of
        ``bench_transformers_e2e.py:61-76,187-190``).  The reference re-runs the step at one cache position;
        here the position advances and the cache is sized for every step of the measurement, because newer
        ``transformers`` caches count the tokens they have seen themselves and a step past the end of the
        cache is an out-of-bounds write."""
        dev, seq_len = input_ids.device, input_ids.shape[1]
        total_steps = warmups + benchmark_runs * number_of_runs
        last_logits, cache = self.prefill(input_ids, total_steps + 1)
        next_token = torch.argmax(last_logits, dim=-1)[:, None]
        decode = self._decode_fn()
        cache_position = torch.tensor([seq_len], device=dev)

        def step():
            decode(self.model, next_token.clone(), None, cache_position, cache)
            cache_position.add_(1)

        for _ in range(warmups):
            step()
        torch.cuda.synchronize()
        times = []
        for _ in range(benchmark_runs):
            t1 = time.time()
            for _ in range(number_of_runs):
                step()
            torch.cuda.synchronize()
            times.append((time.time() - t1) / number_of_runs)
        return times
