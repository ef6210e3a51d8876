"""Typed error tree of the operator surface.

Mirrors the reference's convention (src/mlx_train_perf/errors.py:1-76): every refusal is a
typed exception raised BEFORE any launch, naming the alternative; there is no silent
fallback.  Only the classes the B200 surface can raise are kept; `DeviceTimeoutError`
and `NativeLibraryError` are new (a bounded device-side wait that gave up; the CUDA
library missing or failing to load).
"""


class MlxTrainPerfError(Exception):
    """Root of all errors raised by this package."""


class UnsupportedHeadError(MlxTrainPerfError):
    """Head kind/dtype the requested impl cannot serve (no silent fallback)."""


class LossInputError(MlxTrainPerfError):
    """Shape/dtype/target-range validation failure at the loss boundary."""


class UnsupportedAttentionError(MlxTrainPerfError):
    """Attention impl/config combination the kernel cannot serve (dtype, head_dim,
    causal=False, wrapper refusals)."""


class AttentionInputError(MlxTrainPerfError):
    """Shape validation failure at the flash_attention boundary."""


class PackingError(MlxTrainPerfError):
    """Sequence-packing input validation failure."""


class PlanInputError(MlxTrainPerfError):
    """Shape/config validation failure in the fit planner."""


class DoesNotFitError(MlxTrainPerfError):
    """Planner verdict: predicted peak exceeds the memory budget."""


class AdapterError(MlxTrainPerfError):
    """Model cannot be split into trunk + head (unsupported architecture)."""


class DeviceTimeoutError(MlxTrainPerfError):
    """A bounded device-side wait (mbarrier / flag) ran out; the kernel returned early and
    the outputs of that call are invalid.  The CUDA context stays usable."""


class NativeLibraryError(MlxTrainPerfError):
    """The CUDA shared library is missing, failed to load, or reported an internal error."""
