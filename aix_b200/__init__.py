"""B200-native compute device for the AIX tensor library: C-ABI library (libaixb200.so) plus the host-side mirror
of the reference's device and tensor-value interfaces used to drive it from Python."""
from ._capi import BF16, F16, F32, F64, I8, I16, I32, I64, U8, DTYPE_NAMES, DTYPE_SIZES
from .device import DeviceB200, DeviceTensorParams, bfloat16_bits_to_float32, float32_to_bfloat16_bits, from_storage, to_storage
from .tensor import TensorValue, scalar_like

__all__ = ["DeviceB200", "DeviceTensorParams", "TensorValue", "scalar_like", "to_storage", "from_storage",
           "float32_to_bfloat16_bits", "bfloat16_bits_to_float32", "DTYPE_NAMES", "DTYPE_SIZES",
           "F64", "F32", "F16", "BF16", "I64", "I32", "I16", "I8", "U8"]
