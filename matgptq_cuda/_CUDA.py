"""Stand-in for the reference's pybind extension ``matgptq_cuda._CUDA`` (``csrc/bindings.cpp:214-218``):
the same three callables with the same positional arguments, going straight to the C-ABI library
(no ``torch.library`` dispatch in between, as with the pybind functions)."""
from matgptq_b200 import ops as _ops


def pack_matgptq_qweights(qweights, n_out_features, n_in_features, bitwidth, group_size, feature_flag):
    """``csrc/bindings.cpp:43-84``."""
    return _ops._pack_impl(qweights, n_out_features, n_in_features, bitwidth, group_size, 0)


def reorder_matgptq_scales(scales, m, n, group_size):
    """``csrc/bindings.cpp:86-142``."""
    return _ops._reorder_impl(scales, m, n, group_size)


def matmul_matgptq(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features, bitwidth, group_size,
                   feature_flag):
    """``csrc/bindings.cpp:146-191``."""
    return _ops._matmul_impl(input, matgptq_weights, matgptq_scales, n_out_features, n_in_features,
                                        bitwidth, group_size, feature_flag)
