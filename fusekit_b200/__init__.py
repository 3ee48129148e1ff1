"""fusekit_b200 -- B200-native backend for FuseKit's fused decode path.

The compute lives in ``libfusekit_cuda.so`` (hand-written sm_100a kernels behind the C ABI of
``include/fusekit_cuda.h``); this package is the host-side mirror of the reference's runtime
interface for that path.  Importing it does not need a GPU; using it does.
"""
from .model_spec import CONFIGS, ModelSpec, stream_id  # noqa: F401

__all__ = ["CONFIGS", "ModelSpec", "stream_id"]
