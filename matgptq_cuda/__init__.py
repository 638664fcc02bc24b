"""Import name of the reference's operator package, served by the B200 library.

Every caller of the reference does ``import matgptq_cuda`` (``inference_lib/vllm_matgptq.py:15-16``,
``inference_lib/test_matgptq_matmul.py:5``, ``inference_lib/bench_matgptq_matmul.py``,
``inference_lib/inference_demo_transformers.py``) and reaches the three operators either as
``torch.ops.matgptq_cuda.<name>`` (registered by ``inference_lib/matgptq_cuda/__init__.py:5-63``) or as
``matgptq_cuda._CUDA.<name>`` (the pybind module of ``csrc/bindings.cpp:214-218``).  With this directory on
``sys.path`` in place of the reference's build, those imports resolve here and the calls land in
``libmatgptq_b200.so``; nothing else of the caller has to change.
"""
from matgptq_b200 import ops as _ops

from . import _CUDA, matgptq_linear  # noqa: F401

# the Python-level custom ops, under the names the reference module exposes
pack_matgptq_qweights = _ops.pack_matgptq_qweights
reorder_matgptq_scales = _ops.reorder_matgptq_scales
matmul_matgptq = _ops.matmul_matgptq

__all__ = ["pack_matgptq_qweights", "reorder_matgptq_scales", "matmul_matgptq", "matgptq_linear", "_CUDA"]
