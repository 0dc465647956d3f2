"""B200-native differential attention: `MultiheadDiffAttnKernel` backed by hand-written sm_100a CUDA
(TMA + tcgen05 + TMEM) behind the C ABI of include/diffattn.h.  Importing this package loads
libdiffattn.so and raises if it has not been built; there is no fallback path."""
from .layers import (DiffAttnCore, DiffAttnFunction, MultiheadDiffAttnKernel, device_status,  # noqa: F401
                     lambda_from_reparam)
from .host_pipeline import HostStepPipeline  # noqa: F401
from .shard import shard_range, shard_batch, sum_dlambda_on_host  # noqa: F401

__all__ = ["MultiheadDiffAttnKernel", "DiffAttnFunction", "device_status", "shard_range", "shard_batch",
           "sum_dlambda_on_host", "HostStepPipeline", "lambda_from_reparam", "DiffAttnCore"]
