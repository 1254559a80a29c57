"""B200-native KataGo neural-net backend: Python harness around libkatab200.so.

The product is the CUDA library (katago_b200/csrc, C ABI in include/katab200.h) and the
reference-side backend katago_b200/host/b200backend.cpp.  This package only binds the C ABI
for tests and benchmarks and holds the host-side model-file logic.  There is no CPU fallback:
loading fails loudly when the library has not been built.
"""
from . import modelfile  # noqa: F401
from .capi import (  # noqa: F401
    PRECISION_BF16,
    PRECISION_FP16,
    PRECISION_FP32,
    Handle,
    Model,
    build_library,
    device_count,
    eval_layer,
    library_path,
)
