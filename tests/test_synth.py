"""Synthetic-layer generator: same grid as the reference's quantiser initialisation."""
import numpy as np
import pytest
import torch

from matgptq_b200 import synth
from oracle import matgptq_oracle as oracle


@pytest.mark.parametrize("sym", [False, True])
def test_make_layer_matches_reference_grid(sym):
    layer = synth.make_layer(32, 512, 128, seed=3, sym=sym, dtype=torch.float16)
    gen = torch.Generator().manual_seed(3)
    w = torch.randn(32, 512, generator=gen) * 0.02
    scale, zero = oracle.minmax_params(w.reshape(-1, 128), 8, sym)
    assert torch.equal(layer.scales, scale.half().reshape(32, 4))
    assert torch.equal(layer.zeros, zero.half().reshape(32, 4))
    codes = oracle.rtn_quantize(w.reshape(-1, 128), scale.half().float(), zero, 255).reshape(32, 512)
    assert torch.equal(layer.qweight, codes)
    if sym:
        assert (layer.zeros == 128).all()
    else:
        assert 60 < layer.zeros.float().mean() < 200


def test_algorithmic_bytes_examples():
    # 4096 x 4096, M = 1, b = 4, group 128, no zeros: 8.39 MB planes + 0.26 MB scales + 16 KB
    assert synth.algorithmic_bytes(4096, 4096, 1, 4, 128) == 4096 * 4096 // 2 + 4096 * 32 * 2 + 8192 + 8192
    assert synth.algorithmic_bytes(4096, 4096, 1, 2, 128) == 4096 * 4096 // 4 + 4096 * 32 * 2 + 8192 + 8192


def test_bitwidth_assignment_hits_mean():
    sizes = {}
    for layer in range(32):
        for name, (k, n) in (("q", (4096, 4096)), ("k", (4096, 1024)), ("v", (4096, 1024)), ("o", (4096, 4096)),
                             ("gate", (4096, 14336)), ("up", (4096, 14336)), ("down", (14336, 4096))):
            sizes[f"model.layers.{layer}.{name}"] = k * n
    bits = synth.bitwidth_assignment(sizes, 3.0, seed=0)
    mean = sum(bits[n] * sizes[n] for n in sizes) / sum(sizes.values())
    assert abs(mean - 3.0) < 0.02
    assert set(bits.values()) <= set(synth.BITWIDTHS) and len(set(bits.values())) >= 3
    assert bits == synth.bitwidth_assignment(sizes, 3.0, seed=0)
