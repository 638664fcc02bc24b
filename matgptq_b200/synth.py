"""Seeded synthetic layers in the shapes and value distributions of the benchmark configurations.

There are no checkpoints or datasets on the machines this runs on, so weights are drawn
``W ~ N(0, 0.02)`` and quantised the way the reference's quantiser initialises its grid:
per group of ``group_size`` along K, min-max scale and zero-point at 8 bits
(``MatryoshkaQuantizer.find_params``, ``src/quant_utils_matgpqt.py:92-151``) and round-to-nearest
codes (``src/quant_utils_gptq.py:23-25``).  Activations are ``x ~ N(0, 1)``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

# (K, N) of the Llama-3-8B linear layers
LLAMA3_8B_SHAPES = {
    "q_o": (4096, 4096),
    "k_v": (4096, 1024),
    "gate_up": (4096, 14336),
    "down": (14336, 4096),
}
BITWIDTHS = (2, 3, 4, 6, 8)


@dataclass
class SynthLayer:
    qweight: torch.Tensor  # uint8 [N, K], 8-bit master codes
    scales: torch.Tensor   # [N, G] fp16 / bf16
    zeros: torch.Tensor    # [N, G] same dtype (128 everywhere when symmetric)
    group_size: int

    @property
    def n_out(self) -> int:
        return self.qweight.shape[0]

    @property
    def n_in(self) -> int:
        return self.qweight.shape[1]


def make_layer(n_out: int, n_in: int, group_size: int = 128, seed: int = 0, sym: bool = True,
               dtype: torch.dtype = torch.float16, device: str | torch.device = "cpu") -> SynthLayer:
    """Master-8-bit codes, scales and zero-points of a random ``[n_out, n_in]`` layer."""
    gen = torch.Generator(device=device).manual_seed(seed)
    gs = n_in if group_size == -1 else group_size
    w = torch.randn(n_out, n_in, generator=gen, device=device, dtype=torch.float32) * 0.02
    wg = w.reshape(-1, gs)
    maxq = 255
    xmin = wg.min(1).values
    xmax = wg.max(1).values
    if sym:
        xmax = torch.maximum(xmin.abs(), xmax)
        xmin = torch.where(xmin < 0, -xmax, xmin)
    same = xmin == xmax
    xmin = torch.where(same, torch.full_like(xmin, -1.0), xmin)
    xmax = torch.where(same, torch.full_like(xmax, 1.0), xmax)
    scale = (xmax - xmin) / maxq
    zero = torch.full_like(scale, (maxq + 1) / 2) if sym else torch.round(-xmin / scale)
    # the codes are drawn against the scale the kernels will see, i.e. after rounding to fp16/bf16
    scale_lp = scale.to(dtype)
    q = torch.clamp(torch.round(wg / scale_lp.float().clamp_min(1e-9).unsqueeze(1) + zero.unsqueeze(1)), 0, maxq)
    return SynthLayer(
        qweight=q.to(torch.uint8).reshape(n_out, n_in),
        scales=scale_lp.reshape(n_out, -1).contiguous(),
        zeros=zero.to(dtype).reshape(n_out, -1).contiguous(),
        group_size=group_size,
    )


def make_activations(m: int, n_in: int, seed: int = 0, dtype: torch.dtype = torch.float16,
                     device: str | torch.device = "cpu") -> torch.Tensor:
    gen = torch.Generator(device=device).manual_seed(seed + 1_000_003)
    return torch.randn(m, n_in, generator=gen, device=device, dtype=torch.float32).to(dtype)


def algorithmic_bytes(n_out: int, n_in: int, m: int, bitwidth: int, group_size: int, has_zeros: bool = False) -> int:
    """Bytes one call must move: packed planes + scales (+ zeros) + activations + output."""
    groups = 1 if group_size == -1 else n_in // group_size
    return (n_out * n_in * bitwidth // 8 + n_out * groups * 2 * (2 if has_zeros else 1)
            + m * n_in * 2 + m * n_out * 2)


def bitwidth_assignment(layer_sizes: dict[str, int], mean_bits: float, seed: int = 0,
                        choices: tuple[int, ...] = BITWIDTHS) -> dict[str, int]:
    """Seeded heterogeneous per-layer bitwidths whose parameter-weighted mean is close to ``mean_bits``.

    Starts from a random draw and greedily moves single layers up or down until the weighted mean
    is within 0.01 bit of the target (or no move helps).
    """
    gen = torch.Generator().manual_seed(seed)
    names = list(layer_sizes)
    total = float(sum(layer_sizes.values()))
    idx = torch.randint(0, len(choices), (len(names),), generator=gen).tolist()
    bits = {n: choices[i] for n, i in zip(names, idx)}

    def mean() -> float:
        return sum(bits[n] * layer_sizes[n] for n in names) / total

    order = torch.randperm(len(names), generator=gen).tolist()
    for _ in range(20 * len(names)):
        cur = mean()
        if abs(cur - mean_bits) <= 0.01:
            break
        moved = False
        for j in order:
            n = names[j]
            pos = choices.index(bits[n])
            new_pos = pos - 1 if cur > mean_bits else pos + 1
            if 0 <= new_pos < len(choices):
                new_mean = cur + (choices[new_pos] - bits[n]) * layer_sizes[n] / total
                if abs(new_mean - mean_bits) < abs(cur - mean_bits):
                    bits[n] = choices[new_pos]
                    moved = True
                    break
        if not moved:
            break
        order = order[1:] + order[:1]
    return bits
