"""Per-layer bitwidth files: one ``layer.dotted.name: bits`` per line.

Format of the reference's search output (writer ``evo_quant_search.py:659-671``; readers
``inference_lib/inference_demo_transformers.py:45-49``, ``src/model_utils.py:173-177``).
"""
from __future__ import annotations

from typing import Dict, Iterable, Mapping

ALLOWED_BITS = (2, 3, 4, 6, 8)

# names of the checkpoint layers that vLLM fuses into one linear layer
PACKED_MODULES = {
    "qkv_proj": ("q_proj", "k_proj", "v_proj"),
    "gate_up_proj": ("gate_proj", "up_proj"),
}


def write_bitwidth_config(path: str, bits: Mapping[str, int]) -> None:
    with open(path, "w") as f:
        for name, b in bits.items():
            if int(b) not in ALLOWED_BITS:
                raise ValueError(f"{name}: bitwidth {b} is not one of {ALLOWED_BITS}")
            f.write(f"{name}: {int(b)}\n")


def read_bitwidth_config(path: str) -> Dict[str, int]:
    bits: Dict[str, int] = {}
    with open(path) as f:
        for lineno, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            if ":" not in line:
                raise ValueError(f"{path}:{lineno}: expected 'layer.name: bits', got {line!r}")
            name, value = line.rsplit(":", 1)
            b = int(value.strip())
            if b not in ALLOWED_BITS:
                raise ValueError(f"{path}:{lineno}: bitwidth {b} is not one of {ALLOWED_BITS}")
            bits[name.strip()] = b
    return bits


def shard_names(prefix: str) -> Iterable[str]:
    """Checkpoint layer names behind a (possibly fused) vLLM layer prefix, in partition order."""
    head, _, leaf = prefix.rpartition(".")
    if leaf in PACKED_MODULES:
        return [f"{head}.{s}" if head else s for s in PACKED_MODULES[leaf]]
    return [prefix]


def resolve_bitwidths(prefix: str, n_partitions: int, default_bits: int,
                      layer_bits: Mapping[str, int] | None) -> list[int]:
    """Bitwidth of every output partition of the layer at ``prefix``.

    A fused layer (qkv, gate_up) has one partition per checkpoint layer and each may have its own
    bitwidth; layers the file does not name use ``default_bits`` (the uniform ``inference_bitwidth``)."""
    names = list(shard_names(prefix))
    if len(names) != n_partitions:
        names = [prefix] * n_partitions
    out = []
    for name in names:
        b = default_bits
        if layer_bits:
            b = layer_bits.get(name, layer_bits.get(prefix, default_bits))
        if b not in ALLOWED_BITS:
            raise ValueError(f"{name}: bitwidth {b} is not one of {ALLOWED_BITS}")
        out.append(int(b))
    return out
