"""sepal_runner_b200: Sepal-Runner's trunk projection GEMMs for NVIDIA B200 (sm_100a), behind a C ABI.

The product is `libsepal_b200.so` (CUDA kernels + C++ host code, built in-tree by `build.py`); this package is the thin
ctypes binding that tests, the benchmark and Python callers use. PyTorch is used only for device memory and streams.
There is no CPU path: loading fails loudly when the library is missing, and `Context()` fails on a device that is not sm_100.
"""
from .lib import (  # noqa: F401
    ADD,
    AttentionRow,
    AttentionShape,
    attention,
    attention_prepare,
    BF16,
    Checkpoint,
    Model,
    STORE,
    SWIGLU,
    Context,
    DeltaNetRow,
    DeltaNetShape,
    deltanet,
    gemm_f16_noalloc,
    w8g_schedule,
    Provider,
    SepalB200Error,
    Trunk,
    TrunkConfig,
    W8gWeight,
    library,
    library_path,
    pack_gate_up_source,
    write_tensor_file,
)
