"""B200-native backend for Tritium's packed additive-ternary linear layer."""
from . import _lib
from .backend import (B200Backend, DeviceBuffer, DeviceCaps, GemmShape, LinearStack, MpGemm, SaltV2Forward,
                      SaltV2ForwardReceipt, SaltV2ResidentTensor, TernaryFormat)
from .errors import (Backend, BackendError, InvalidInput, NullArg, OutOfMemory, ShapeMismatch, Timeout,
                     UnsupportedFormat)
from .format import SaltV2Codec, SaltV2Tensor, write_salt_v2_package
from .runtime import BACKENDS, BackendEntry, Registry, list_backends

__all__ = [
    "B200Backend", "DeviceBuffer", "DeviceCaps", "GemmShape", "LinearStack", "MpGemm", "SaltV2Forward",
    "SaltV2ForwardReceipt", "SaltV2ResidentTensor", "TernaryFormat", "Backend", "BackendError", "InvalidInput",
    "NullArg", "OutOfMemory", "ShapeMismatch", "Timeout", "UnsupportedFormat", "SaltV2Codec", "SaltV2Tensor",
    "write_salt_v2_package", "BACKENDS", "BackendEntry", "Registry", "list_backends",
]
