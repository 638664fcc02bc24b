"""The import surface every caller of the reference uses (``import matgptq_cuda``, ``matgptq_cuda._CUDA``,
``matgptq_cuda.matgptq_linear``) served by this repository, and the reference's own kernel test run
UNCHANGED against it where a checkout of the reference is available (``MATGPTQ_REFERENCE_DIR``, default
``/root/reference``)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("MATGPTQ_REFERENCE_DIR", "/root/reference")


def test_import_surface():
    import torch

    import matgptq_cuda
    from matgptq_cuda.matgptq_linear import MatGPTQLinear, MatGTPQ_FeatureFlags  # inference_lib/vllm_matgptq.py:15-16
    assert (MatGTPQ_FeatureFlags.SYNC, MatGTPQ_FeatureFlags.ASYNC, MatGTPQ_FeatureFlags.IS_BF16) == (0, 1, 2)
    assert MatGPTQLinear.__module__ == "matgptq_b200.matgptq_linear"
    for name in ("pack_matgptq_qweights", "reorder_matgptq_scales", "matmul_matgptq"):
        assert callable(getattr(matgptq_cuda._CUDA, name))       # csrc/bindings.cpp:214-218
        assert callable(getattr(matgptq_cuda, name))             # matgptq_cuda/__init__.py:5-47
        assert hasattr(torch.ops.matgptq_cuda, name)             # callers' torch.ops.matgptq_cuda.<name>
    # without a GPU the pybind-style entry raises like the operator does (no CPU path)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            matgptq_cuda._CUDA.pack_matgptq_qweights(torch.zeros(16, 128, dtype=torch.uint8), 16, 128, 4, 128, 1)


def _have_reference() -> bool:
    return os.path.exists(os.path.join(REFERENCE, "inference_lib", "test_matgptq_matmul.py"))


@pytest.mark.skipif(not _have_reference(), reason="no checkout of the reference on this machine")
def test_reference_vllm_module_imports_against_the_shim():
    """inference_lib/vllm_matgptq.py, unmodified, imports with this repository first on sys.path (its
    ``import matgptq_cuda`` and ``from matgptq_cuda.matgptq_linear import MatGTPQ_FeatureFlags`` resolve here)."""
    code = ("import sys; sys.path.insert(0, %r); sys.path.insert(0, %r); import vllm_matgptq as m; "
            "import matgptq_cuda; assert matgptq_cuda.__file__.startswith(%r); "
            "c = m.MatGPTQConfig(128, 8, 4, 'bfloat16', ['lm_head']); print('flag', int(c.flag))"
            % (os.path.join(REFERENCE, "inference_lib"), ROOT, ROOT))
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "flag 3" in proc.stdout, proc.stderr[-3000:]


@pytest.mark.gpu
@pytest.mark.skipif(not _have_reference(), reason="no checkout of the reference on this machine")
def test_reference_kernel_test_file_passes_unchanged():
    """pytest on the reference's inference_lib/test_matgptq_matmul.py itself (270 exact-match cases)."""
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-p", "no:cacheprovider",
                           os.path.join(REFERENCE, "inference_lib", "test_matgptq_matmul.py")],
                          capture_output=True, text=True, timeout=1800, env=env, cwd=ROOT)
    assert proc.returncode == 0 and "270 passed" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-2000:]
