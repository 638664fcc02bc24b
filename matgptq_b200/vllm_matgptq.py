"""vLLM quantisation method ``matgptq_quant`` on the B200 library.

Mirrors ``inference_lib/vllm_matgptq.py:18-200``: same registration name, same config keys
(``group_size``, ``master_bitwidth``, ``inference_bitwidth``, ``quant_dtype``,
``modules_to_not_convert``), same parameters (`qweight` uint8 master codes, `scales`), slicing and
packing after loading, one operator call per forward.

Additions (absent keys give the reference's behaviour):
  * ``layer_bitwidths`` (dict) or ``bitwidth_config_path`` (a ``name: bits`` file, the format of
    ``evo_quant_search.py:659-671``): per-layer inference bitwidths.  The reference's vLLM method has
    one uniform bitwidth; per-layer files only reach its HF-transformers path
    (``inference_lib/inference_demo_transformers.py:45-49``).  vLLM fuses q/k/v and gate/up into one
    layer, so a fused layer may carry several bitwidths: each output partition is packed and run at
    its own bitwidth.
  * ``zero_points`` (bool): the checkpoint also holds ``<layer>.zeros`` (``[N, K/g]``, master units, dtype of
    the scales; ``dequantize`` of ``src/quant_utils_matgpqt.py:19-22`` takes them, the reference's operator and
    packer do not).  The layers then run ``matmul_matgptq_zeros``.
  * slicing is fused into packing on the GPU (the reference slices with torch ops and packs on one
    CPU thread, ``vllm_matgptq.py:150-166``, ``csrc/bindings.cpp:63-83``).
"""
from __future__ import annotations

import torch
from torch.nn.parameter import Parameter
from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase, UnquantizedLinearMethod
from vllm.model_executor.layers.quantization import register_quantization_config
from vllm.model_executor.layers.quantization.base_config import QuantizationConfig, QuantizeMethodBase
from vllm.model_executor.parameter import ModelWeightParameter
from vllm.model_executor.utils import set_weight_attrs

from . import ops  # noqa: F401  registers torch.ops.matgptq_cuda.*
from .bitwidth_config import read_bitwidth_config, resolve_bitwidths
from .matgptq_linear import MatGTPQ_FeatureFlags


@register_quantization_config("matgptq_quant")
class MatGPTQConfig(QuantizationConfig):
    """Quantisation config of packed MatGPTQ checkpoints."""

    def __init__(
        self,
        group_size: int = 128,
        master_bitwidth: int = 8,
        inference_bitwidth: int = 4,
        quant_dtype: str = "float16",
        modules_to_not_convert: list[str] | None = None,
        layer_bitwidths: dict[str, int] | None = None,
        zero_points: bool = False,
    ) -> None:
        super().__init__()
        assert group_size in [-1, 32, 128]
        assert quant_dtype in ["float16", "bfloat16"]
        self.group_size = group_size
        self.master_bitwidth = master_bitwidth
        self.inference_bitwidth = inference_bitwidth
        self.quant_dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16}[quant_dtype]
        self.modules_to_not_convert = modules_to_not_convert
        self.layer_bitwidths = dict(layer_bitwidths) if layer_bitwidths else None
        self.zero_points = bool(zero_points)
        self.flag = MatGTPQ_FeatureFlags.ASYNC + MatGTPQ_FeatureFlags.IS_BF16 * (self.quant_dtype == torch.bfloat16)
        # what the products are launched with: programmatic dependent launch on top, so that launches of this library
        # that follow one another (the segments of a fused layer above 16 rows) prefetch weights behind each other;
        # behind a kernel of the host that does not release its dependents early the launch simply starts when that
        # kernel is done, as it would without the flag
        self.matmul_flag = int(self.flag) | 4

    def get_name(self) -> str:
        return "matgptq_quant"

    def get_supported_act_dtypes(self) -> list:
        return [torch.float16, torch.bfloat16]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100  # the kernels are sm_100a only (the reference says 80)

    @staticmethod
    def get_config_filenames() -> list[str]:
        return []

    @classmethod
    def from_config(cls, config: dict) -> "MatGPTQConfig":
        group_size = cls.get_from_keys(config, ["group_size"])
        master_bitwidth = cls.get_from_keys(config, ["master_bitwidth"])
        inference_bitwidth = cls.get_from_keys(config, ["inference_bitwidth"])
        modules_to_not_convert = cls.get_from_keys(config, ["modules_to_not_convert"])
        quant_dtype = cls.get_from_keys(config, ["quant_dtype"])
        layer_bitwidths = cls.get_from_keys_or(config, ["layer_bitwidths"], None)
        path = cls.get_from_keys_or(config, ["bitwidth_config_path"], None)
        if path:
            layer_bitwidths = {**read_bitwidth_config(path), **(layer_bitwidths or {})}
        zero_points = cls.get_from_keys_or(config, ["zero_points"], False)
        return cls(group_size, master_bitwidth, inference_bitwidth, quant_dtype, modules_to_not_convert,
                   layer_bitwidths, zero_points)

    def get_quant_method(self, layer: torch.nn.Module, prefix: str) -> QuantizeMethodBase | None:
        if self.modules_to_not_convert is not None and any(
                prefix.endswith(module) for module in self.modules_to_not_convert):
            return UnquantizedLinearMethod()
        if isinstance(layer, LinearBase):
            return MatGPTQLinearMethod(self, prefix)
        return None


class MatGPTQLinearMethod(LinearMethodBase):
    """Linear method: uint8 master codes + scales in, packed b-bit weights after loading."""

    def __init__(self, config: MatGPTQConfig, prefix: str = ""):
        super().__init__()
        self.config = config
        self.prefix = prefix

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int,
                       output_partition_sizes: list[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, **extra_weight_attrs):
        gs = self.config.group_size
        if gs != -1 and input_size_per_partition % gs != 0:
            raise ValueError(
                "The input size is not aligned with the quantized weight shape. "
                "This can be caused by too large tensor parallel size.")
        if input_size_per_partition % 128 != 0 or any(p % 16 != 0 for p in output_partition_sizes):
            raise ValueError("matgptq_b200 needs in-features per partition % 128 == 0 and out-features % 16 == 0")
        n_out = sum(output_partition_sizes)
        layer.matgptq_n_out = n_out
        layer.matgptq_n_in = input_size_per_partition
        layer.matgptq_partitions = list(output_partition_sizes)
        layer.matgptq_bits = resolve_bitwidths(self.prefix, len(output_partition_sizes),
                                               self.config.inference_bitwidth, self.config.layer_bitwidths)

        qweight = ModelWeightParameter(
            data=torch.empty(n_out, input_size_per_partition, dtype=torch.uint8),
            input_dim=1, output_dim=0, weight_loader=extra_weight_attrs.get("weight_loader"))
        layer.register_parameter("qweight", qweight)

        groups = 1 if gs == -1 else input_size_per_partition // gs
        scales = Parameter(torch.empty(n_out, groups, dtype=self.config.quant_dtype), requires_grad=False)
        set_weight_attrs(scales, {"input_dim": 1, "output_dim": 0, "packed_dim": 1, "pack_factor": 1}
                         | extra_weight_attrs)
        layer.register_parameter("scales", scales)
        if self.config.zero_points:
            zeros = Parameter(torch.empty(n_out, groups, dtype=self.config.quant_dtype), requires_grad=False)
            set_weight_attrs(zeros, {"input_dim": 1, "output_dim": 0, "packed_dim": 1, "pack_factor": 1}
                             | extra_weight_attrs)
            layer.register_parameter("zeros", zeros)

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        cfg = self.config
        n_in = layer.matgptq_n_in
        # consecutive partitions with the same bitwidth become one packed segment (one launch)
        segments: list[list[int]] = []  # [row0, rows, bits]
        row = 0
        for rows, bits in zip(layer.matgptq_partitions, layer.matgptq_bits):
            if segments and segments[-1][2] == bits:
                segments[-1][1] += rows
            else:
                segments.append([row, rows, bits])
            row += rows
        with torch.no_grad():
            packed, scales, zeros = [], [], []
            for row0, rows, bits in segments:
                q = layer.qweight.data[row0:row0 + rows].contiguous()
                s = layer.scales.data[row0:row0 + rows].contiguous()
                if cfg.zero_points:
                    z = layer.zeros.data[row0:row0 + rows].contiguous()
                    zeros.append(Parameter(torch.ops.matgptq_cuda.reorder_matgptq_scales(z, rows, n_in, cfg.group_size),
                                           requires_grad=False))
                packed.append(Parameter(torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(
                    q, rows, n_in, cfg.master_bitwidth, bits, cfg.group_size, cfg.flag), requires_grad=False))
                scales.append(Parameter(torch.ops.matgptq_cuda.reorder_matgptq_scales(
                    s, rows, n_in, cfg.group_size), requires_grad=False))
            layer.matgptq_segments = [(rows, bits) for _, rows, bits in segments]
            layer.matgptq_weights = torch.nn.ParameterList(packed)
            layer.matgptq_scales = torch.nn.ParameterList(scales)
            del layer.qweight
            del layer.scales
            if cfg.zero_points:
                del layer.zeros
                layer.matgptq_zeros = torch.nn.ParameterList(zeros)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        cfg = self.config
        x2 = x.reshape(-1, x.shape[-1])
        if cfg.zero_points:
            outs = [
                torch.ops.matgptq_cuda.matmul_matgptq_zeros(x2, w, s, z, rows, layer.matgptq_n_in, bits, cfg.group_size,
                                                            cfg.matmul_flag)
                for (rows, bits), w, s, z in zip(layer.matgptq_segments, layer.matgptq_weights, layer.matgptq_scales,
                                                 layer.matgptq_zeros)
            ]
        elif len(layer.matgptq_segments) == 1:
            (rows, bits), = layer.matgptq_segments
            outs = [torch.ops.matgptq_cuda.matmul_matgptq(x2, layer.matgptq_weights[0], layer.matgptq_scales[0], rows,
                                                          layer.matgptq_n_in, bits, cfg.group_size, cfg.matmul_flag)]
        else:
            # a fused layer whose partitions carry different bitwidths: one grouped launch, outputs side by side
            outs = [torch.ops.matgptq_cuda.matmul_matgptq_grouped(
                x2, list(layer.matgptq_weights), list(layer.matgptq_scales), [rows for rows, _ in layer.matgptq_segments],
                layer.matgptq_n_in, [bits for _, bits in layer.matgptq_segments], cfg.group_size, cfg.matmul_flag)]
        y = outs[0] if len(outs) == 1 else torch.cat(outs, dim=-1)
        y = y.view(*x.shape[:-1], y.shape[-1])
        if bias is not None:
            y += bias
        return y
