"""B200-native replacements for mlx-train-perf's two training hot paths.

Public surface (mirrors src/mlx_train_perf/__init__.py and the modules it re-exports):
`linear_cross_entropy`, `fused_linear_ce`, `DenseHead`, `QuantizedHead`, `tied_head`,
`flash_attention`, `PackedMask`, `enable_flash_attention`, `packed_iterate_batches`,
`plan_fit`.  Every numeric operator is a thin ctypes wrapper over one C-ABI CUDA library
(`csrc/`), and raises `NativeLibraryError` when that library cannot be loaded.
"""
from mlx_train_perf_b200.errors import (  # noqa: F401
    AdapterError, AttentionInputError, DeviceTimeoutError, DoesNotFitError, LossInputError,
    MlxTrainPerfError, NativeLibraryError, PackingError, PlanInputError,
    UnsupportedAttentionError, UnsupportedHeadError,
)

__version__ = "0.1.0"

_LAZY = {
    "linear_cross_entropy": "mlx_train_perf_b200.core.loss",
    "fused_linear_ce": "mlx_train_perf_b200.core.loss",
    "DenseHead": "mlx_train_perf_b200.core.loss",
    "QuantizedHead": "mlx_train_perf_b200.core.loss",
    "tied_head": "mlx_train_perf_b200.core.loss",
    "flash_attention": "mlx_train_perf_b200.attention.api",
    "PackedMask": "mlx_train_perf_b200.attention.segments",
    "enable_flash_attention": "mlx_train_perf_b200.attention.wrapper",
    "packed_iterate_batches": "mlx_train_perf_b200.data.packing",
    "plan_fit": "mlx_train_perf_b200.plan.estimate",
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        return getattr(importlib.import_module(_LAZY[name]), name)
    raise AttributeError(name)
