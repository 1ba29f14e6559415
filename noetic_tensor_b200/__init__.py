"""noetic_tensor_b200 — the `nn::rl` token-level hot path of noetic-tensor, fused for B200.

The product is libnrl.so (CUDA, sm_100a) behind the C ABI of include/nrl.h; `capi` declares that
ABI for ctypes and `ops` calls it with torch tensors as device buffers. Importing this package
does not need a GPU; calling any op without libnrl.so or without a CUDA device raises.
"""
from . import capi  # noqa: F401

__all__ = ["capi", "ops"]


def __getattr__(name):
    if name == "ops":
        import importlib

        return importlib.import_module(".ops", __name__)
    raise AttributeError(name)
