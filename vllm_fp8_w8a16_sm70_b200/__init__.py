"""B200-native block-scaled FP8 (E4M3) W8A16 linear and MoE engine.

Hand-written sm_100a CUDA kernels behind a C ABI (``include/fp8w8a16_b200.h``), loaded with ctypes;
the Python layer mirrors the vLLM-facing hooks of KumphanartDansiri/vllm-fp8-w8a16-sm70.
"""

from .backend import backend_mode, select_backend  # noqa: F401
from . import ops  # noqa: F401
from . import checkpoint  # noqa: F401
from .linear_method import CompressedTensorsW8A16Fp8, Fp8LinearMethod  # noqa: F401
from .module import FP8W8A16Linear  # noqa: F401
from .moe_method import CompressedTensorsFp8MoEMethod, Fp8MoEMethod  # noqa: F401

__version__ = "0.1.0"
