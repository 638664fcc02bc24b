"""``matgptq_cuda.matgptq_linear`` of the reference (``inference_lib/matgptq_cuda/matgptq_linear.py:6-59``):
the module and the flag enum live in ``matgptq_b200.matgptq_linear``."""
from matgptq_b200.matgptq_linear import MatGPTQLinear, MatGTPQ_FeatureFlags

__all__ = ["MatGPTQLinear", "MatGTPQ_FeatureFlags"]
