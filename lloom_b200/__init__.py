"""lloom_b200: B200-native (sm_100a) backend for lloom's quantized-weight matmul path.

The package holds the CUDA kernels with their C ABI (``csrc/``, ``include/lloom_b200.h``) and the
host-side mirror of the reference's ``GgmlDType`` / ``QTensor`` / ``QMatMul`` / ``QCudaStorage``
interface (``quantized.py``), plus the row-sharded multi-GPU forward (``sharded.py``) and the GGUF
container reader that feeds ``QTensor`` from a file's block bytes (``gguf_file.py``).
"""
from ._lib import LloomError  # noqa: F401
from .quantized import GgmlDType, QCudaStorage, QMatMul, QTensor  # noqa: F401

__all__ = ["GgmlDType", "QCudaStorage", "QMatMul", "QTensor", "LloomError"]
