"""Packed MatGPTQ checkpoints: the on-disk layout written by ``pack_quantized_model.py``.

Layout (``pack_quantized_model.py:33-142``): for every quantised linear ``<L>`` the safetensors hold
``<L>.qweight`` (uint8 ``[N, K]``, 8-bit MASTER codes, unsliced) and ``<L>.scales`` (``[N, K/g]``,
fp16/bf16) instead of ``<L>.weight``; layers whose name contains ``lm_head`` or ``norm`` stay dense
(``:25-30``); a sharded model keeps ``model.safetensors.index.json``; ``config.json`` gains

    "quantization_config": {"group_size", "modules_to_not_convert": ["lm_head", "norm"],
                            "master_bitwidth", "inference_bitwidth", "quant_method": "matgptq_quant",
                            "quant_dtype"}                                     (``:134-141``)

The reference builds such a directory from a calibrated model.  There are no calibrated models here,
so ``write_synthetic_checkpoint`` writes the same layout from seeded random layers
(``matgptq_b200.synth``).  Optional ``<L>.zeros`` tensors (an addition) carry per-group zero points.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Mapping

import torch
from safetensors import safe_open
from safetensors.torch import save_file

from . import synth
from .bitwidth_config import write_bitwidth_config

QUANT_METHOD = "matgptq_quant"
EXCLUDED = ("lm_head", "norm")


def should_skip_quantisation(module_name: str) -> bool:
    """Same rule as ``pack_quantized_model.py:25-30``."""
    return any(excl in module_name for excl in EXCLUDED)


def quantization_config(group_size: int, master_bitwidth: int, inference_bitwidth: int, quant_dtype: str,
                        layer_bitwidths: Mapping[str, int] | None = None, zero_points: bool = False) -> dict:
    cfg = {
        "group_size": group_size,
        "modules_to_not_convert": list(EXCLUDED),
        "master_bitwidth": master_bitwidth,
        "inference_bitwidth": inference_bitwidth,
        "quant_method": QUANT_METHOD,
        "quant_dtype": quant_dtype,
    }
    if layer_bitwidths:
        cfg["layer_bitwidths"] = dict(layer_bitwidths)
    if zero_points:
        cfg["zero_points"] = True  # the checkpoint holds <layer>.zeros (an addition to the reference's layout)
    return cfg


def llama_linear_shapes(hidden: int, intermediate: int, n_heads: int, n_kv_heads: int, n_layers: int) -> Dict[str, tuple]:
    """``name -> (n_out, n_in)`` of every block linear of a Llama-architecture model."""
    head_dim = hidden // n_heads
    shapes: Dict[str, tuple] = {}
    for i in range(n_layers):
        p = f"model.layers.{i}"
        shapes[f"{p}.self_attn.q_proj"] = (hidden, hidden)
        shapes[f"{p}.self_attn.k_proj"] = (n_kv_heads * head_dim, hidden)
        shapes[f"{p}.self_attn.v_proj"] = (n_kv_heads * head_dim, hidden)
        shapes[f"{p}.self_attn.o_proj"] = (hidden, hidden)
        shapes[f"{p}.mlp.gate_proj"] = (intermediate, hidden)
        shapes[f"{p}.mlp.up_proj"] = (intermediate, hidden)
        shapes[f"{p}.mlp.down_proj"] = (hidden, intermediate)
    return shapes


def write_synthetic_checkpoint(out_dir: str, linear_shapes: Mapping[str, tuple], *, group_size: int = 128,
                               inference_bitwidth: int = 4, quant_dtype: str = "float16",
                               dense_tensors: Mapping[str, torch.Tensor] | None = None,
                               layer_bitwidths: Mapping[str, int] | None = None, base_config: dict | None = None,
                               seed: int = 0, shard_bytes: int = 2 << 30, device: str = "cpu", sym: bool = True) -> dict:
    """Write a packed checkpoint directory; returns the ``quantization_config`` it wrote."""
    os.makedirs(out_dir, exist_ok=True)
    dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16}[quant_dtype]
    shards: list[Dict[str, torch.Tensor]] = [{}]
    sizes = [0]

    def put(name: str, t: torch.Tensor) -> None:
        nbytes = t.numel() * t.element_size()
        if sizes[-1] and sizes[-1] + nbytes > shard_bytes:
            shards.append({})
            sizes.append(0)
        shards[-1][name] = t.contiguous().cpu()
        sizes[-1] += nbytes

    for i, (name, (n_out, n_in)) in enumerate(linear_shapes.items()):
        if should_skip_quantisation(name):
            raise ValueError(f"{name} would be skipped by the packer's exclusion rule")
        layer = synth.make_layer(n_out, n_in, group_size, seed=seed + i, sym=sym, dtype=dtype, device=device)
        put(f"{name}.qweight", layer.qweight)
        put(f"{name}.scales", layer.scales)
        if not sym:
            put(f"{name}.zeros", layer.zeros)
    for name, t in (dense_tensors or {}).items():
        put(name, t)

    weight_map: Dict[str, str] = {}
    if len(shards) == 1:
        save_file(shards[0], os.path.join(out_dir, "model.safetensors"))
    else:
        for si, shard in enumerate(shards):
            fname = f"model-{si + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file(shard, os.path.join(out_dir, fname))
            weight_map.update({k: fname for k in shard})
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {}, "weight_map": weight_map}, f)

    qcfg = quantization_config(group_size, 8, inference_bitwidth, quant_dtype, layer_bitwidths, zero_points=not sym)
    config = dict(base_config or {})
    config["quantization_config"] = qcfg
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    if layer_bitwidths:
        write_bitwidth_config(os.path.join(out_dir, "bitwidths.txt"), layer_bitwidths)
    return qcfg


def read_checkpoint_config(ckpt_dir: str) -> dict:
    with open(os.path.join(ckpt_dir, "config.json")) as f:
        config = json.load(f)
    qcfg = config.get("quantization_config")
    if not qcfg or qcfg.get("quant_method") != QUANT_METHOD:
        raise ValueError(f"{ckpt_dir} is not a packed MatGPTQ checkpoint")
    for key in ("group_size", "master_bitwidth", "inference_bitwidth", "quant_dtype", "modules_to_not_convert"):
        if key not in qcfg:
            raise ValueError(f"quantization_config lacks '{key}'")
    return qcfg


def iter_checkpoint_tensors(ckpt_dir: str, names: Iterable[str] | None = None):
    """Yield ``(name, tensor)`` from a single-file or sharded checkpoint directory."""
    index = os.path.join(ckpt_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = ["model.safetensors"]
    wanted = set(names) if names is not None else None
    for fname in files:
        with safe_open(os.path.join(ckpt_dir, fname), framework="pt") as f:
            for key in f.keys():
                if wanted is None or key in wanted:
                    yield key, f.get_tensor(key)


def load_linear(ckpt_dir: str, name: str, with_zeros: bool = False):
    """``(qweight, scales)`` of one quantised linear layer, or ``(qweight, scales, zeros)`` with ``with_zeros``
    (``zeros`` is None when the checkpoint has none: implicit zero point 128)."""
    got = dict(iter_checkpoint_tensors(ckpt_dir, [f"{name}.qweight", f"{name}.scales", f"{name}.zeros"]))
    if f"{name}.qweight" not in got or f"{name}.scales" not in got:
        raise KeyError(f"{name}: qweight/scales not found in {ckpt_dir}")
    q, s = got[f"{name}.qweight"], got[f"{name}.scales"]
    if q.dtype != torch.uint8 or q.dim() != 2 or s.dim() != 2 or s.shape[0] != q.shape[0]:
        raise ValueError(f"{name}: unexpected tensor layout {q.dtype}{tuple(q.shape)} / {s.dtype}{tuple(s.shape)}")
    if not with_zeros:
        return q, s
    z = got.get(f"{name}.zeros")
    if z is not None and (z.shape != s.shape or z.dtype != s.dtype):
        raise ValueError(f"{name}: zeros {z.dtype}{tuple(z.shape)} do not match scales {s.dtype}{tuple(s.shape)}")
    return q, s, z
