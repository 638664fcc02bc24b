"""``MatGPTQLinear`` and its feature flags, as in ``inference_lib/matgptq_cuda/matgptq_linear.py:6-59``."""
from enum import IntEnum

import torch

from . import ops  # noqa: F401  (registers torch.ops.matgptq_cuda.*)


class MatGTPQ_FeatureFlags(IntEnum):
    SYNC = 0
    ASYNC = 1
    IS_BF16 = 2
    # addition: programmatic dependent launch (weight prefetch overlaps the previous kernel)
    PDL = 4


# forward() launches with programmatic dependent launch on top of the module's flag (the reference's two bits):
# q, k, v or gate, up of a model that calls one module after the other then prefetch their weights behind each other
_PDL = int(MatGTPQ_FeatureFlags.PDL)


class MatGPTQLinear(torch.nn.Module):
    """Linear layer over packed b-bit weights.

    ``qweight``: uint8 ``[N, K]`` codes already sliced to ``bitwidth`` bits (CPU or CUDA);
    ``scales``: ``[N, K/group_size]`` (``[N, 1]`` for ``group_size == -1``), float16 or bfloat16,
    which also selects the activation and output dtype.
    """

    def __init__(self, qweight: torch.Tensor, scales: torch.Tensor, bitwidth: int, group_size: int):
        super().__init__()
        self.n_out_features: int = qweight.shape[0]
        self.n_in_features: int = qweight.shape[1]
        self.bitwidth: int = bitwidth
        self.group_size: int = group_size

        self.flag: int = MatGTPQ_FeatureFlags.ASYNC + MatGTPQ_FeatureFlags.IS_BF16 * (scales.dtype == torch.bfloat16)

        self.matgptq_qweight = torch.nn.Parameter(
            torch.ops.matgptq_cuda.pack_matgptq_qweights(
                qweight, self.n_out_features, self.n_in_features, self.bitwidth, self.group_size, self.flag),
            requires_grad=False)
        self.matgptq_scales = torch.nn.Parameter(
            torch.ops.matgptq_cuda.reorder_matgptq_scales(
                scales, self.n_out_features, self.n_in_features, self.group_size),
            requires_grad=False)

    @classmethod
    def from_master(cls, qweight_master: torch.Tensor, scales: torch.Tensor, master_bitwidth: int, bitwidth: int,
                    group_size: int, keep_master: bool = False) -> "MatGPTQLinear":
        """Addition: build the layer from UNSLICED master codes; the MSB slicing of
        ``matryoshka_slice`` (``src/quant_utils_matgpqt.py:9-17``) is fused into the GPU packer instead of
        being a separate pass (``inference_demo_transformers.py:30-39``).  With ``keep_master`` the uint8 master
        codes stay resident on the GPU and ``set_bitwidth`` re-slices from them at run time."""
        self = cls.__new__(cls)
        torch.nn.Module.__init__(self)
        self.master_bitwidth = master_bitwidth
        self.register_buffer("master_qweight", qweight_master.contiguous() if keep_master else None, persistent=False)
        self.n_out_features, self.n_in_features = qweight_master.shape
        self.bitwidth, self.group_size = bitwidth, group_size
        self.flag = MatGTPQ_FeatureFlags.ASYNC + MatGTPQ_FeatureFlags.IS_BF16 * (scales.dtype == torch.bfloat16)
        self.matgptq_qweight = torch.nn.Parameter(
            torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(
                qweight_master.contiguous(), self.n_out_features, self.n_in_features, master_bitwidth, bitwidth,
                group_size, self.flag),
            requires_grad=False)
        self.matgptq_scales = torch.nn.Parameter(
            torch.ops.matgptq_cuda.reorder_matgptq_scales(
                scales.contiguous(), self.n_out_features, self.n_in_features, group_size),
            requires_grad=False)
        return self

    @torch.no_grad()
    def set_bitwidth(self, bitwidth: int) -> None:
        """Addition: serve this layer at another bitwidth from the resident master codes (one GPU pass of the
        fused slice + pack kernel; the scales do not depend on the bitwidth).  The reference switches bitwidth by
        re-running slice and host-side pack for the whole model (``vllm_matgptq.py:150-178``)."""
        if getattr(self, "master_qweight", None) is None:
            raise RuntimeError("set_bitwidth needs the master codes: build the layer with from_master(..., keep_master=True)")
        if bitwidth == self.bitwidth:
            return
        self.matgptq_qweight = torch.nn.Parameter(
            torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(
                self.master_qweight, self.n_out_features, self.n_in_features, self.master_bitwidth, bitwidth,
                self.group_size, self.flag),
            requires_grad=False)
        self.bitwidth = bitwidth

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() > 2:
            # The reference hands the tensor to the operator as it is, which reads the last two dimensions
            # only and returns [M, N] (csrc/bindings.cpp:171-174): right for a leading dimension of 1, wrong
            # beyond.  Here every leading dimension counts as rows and the result keeps them.
            y = torch.ops.matgptq_cuda.matmul_matgptq(
                x.reshape(-1, self.n_in_features), self.matgptq_qweight, self.matgptq_scales, self.n_out_features,
                self.n_in_features, self.bitwidth, self.group_size, self.flag | _PDL)
            return y.view(*x.shape[:-1], self.n_out_features)
        return torch.ops.matgptq_cuda.matmul_matgptq(
            x, self.matgptq_qweight, self.matgptq_scales, self.n_out_features, self.n_in_features,
            self.bitwidth, self.group_size, self.flag | _PDL)
