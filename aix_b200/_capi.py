"""ctypes binding of include/aixb200.h. Loads aix_b200/lib/libaixb200.so and fails loudly when it is missing:
there is no Python or CPU fallback for any device operation."""
import ctypes
import os

MAX_RANK = 8
COMM_ID_BYTES = 128

OK, ERR_INVALID, ERR_RUNTIME, ERR_NOGPU, ERR_TIMEOUT = 0, 1, 2, 3, 4

F64, F32, F16, BF16, I64, I32, I16, I8, U8 = range(9)
DTYPE_NAMES = ["f64", "f32", "f16", "bf16", "i64", "i32", "i16", "i8", "u8"]
DTYPE_SIZES = [8, 4, 2, 2, 8, 4, 2, 1, 1]


class Tensor(ctypes.Structure):
    """aixb200_tensor: POD image of aix::DeviceTensorParams."""
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("offset", ctypes.c_uint64),
        ("size", ctypes.c_uint64),
        ("dtype", ctypes.c_uint32),
        ("rank", ctypes.c_uint32),
        ("shape", ctypes.c_uint64 * MAX_RANK),
        ("strides", ctypes.c_uint64 * MAX_RANK),
    ]


class Config(ctypes.Structure):
    _fields_ = [
        ("ordinal", ctypes.c_int32),
        ("managed_memory", ctypes.c_int32),
        ("flush_threshold", ctypes.c_uint32),
        ("strict_math", ctypes.c_int32),
        ("fusion", ctypes.c_int32),
        ("disk_cache", ctypes.c_int32),
        ("cache_limit_bytes", ctypes.c_uint64),
        ("stream", ctypes.c_void_p),
        ("tf32x3_matmul", ctypes.c_int32),
        ("dry_run", ctypes.c_int32),
        ("inject_alloc_limit_bytes", ctypes.c_uint64),
        ("inject_nvrtc_failures", ctypes.c_int32),
        ("reserved", ctypes.c_int32 * 3),
    ]


class Stats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in (
        "ops_recorded", "flushes", "fused_kernels", "fused_ops", "fills_absorbed", "stores_elided",
        "kernel_cache_hits", "kernel_cache_misses", "nvrtc_compiles")] + [("nvrtc_ms", ctypes.c_double)] + [
        (n, ctypes.c_uint64) for n in (
        "static_kernel_launches", "total_kernel_launches", "bytes_in_use", "bytes_cached", "bytes_reserved",
        "cuda_mallocs", "h2d_bytes", "d2h_bytes", "reductions_fused", "prepared_operand_hits", "prepared_operand_builds", "prepared_operand_max_known", "matmul_consumers_folded")] + [
        ("reserved", ctypes.c_uint64 * 1)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_ if n != "reserved"}


LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libaixb200.so")

# Every symbol include/aixb200.h declares, with its argument types (the return type is int unless given).
_T = ctypes.POINTER(Tensor)
_D = ctypes.c_void_p
_SZ = ctypes.c_size_t
SIGNATURES = {
    "aixb200_default_config": ([ctypes.POINTER(Config)], None),
    "aixb200_create": ([ctypes.c_int, ctypes.POINTER(_D)], ctypes.c_int),
    "aixb200_create_with_config": ([ctypes.POINTER(Config), ctypes.POINTER(_D)], ctypes.c_int),
    "aixb200_destroy": ([_D], None),
    "aixb200_last_error": ([_D], ctypes.c_char_p),
    "aixb200_name": ([_D], ctypes.c_char_p),
    "aixb200_device_count": ([], ctypes.c_int),
    "aixb200_version": ([], ctypes.c_char_p),
    "aixb200_allocate": ([_D, _SZ, ctypes.POINTER(ctypes.c_void_p)], ctypes.c_int),
    "aixb200_allocate_typed": ([_D, _SZ, ctypes.c_uint32, ctypes.POINTER(ctypes.c_void_p)], ctypes.c_int),
    "aixb200_deallocate": ([_D, ctypes.c_void_p], ctypes.c_int),
    "aixb200_empty_cache": ([_D], ctypes.c_int),
    "aixb200_synchronize": ([_D], ctypes.c_int),
    "aixb200_fill": ([_D, ctypes.c_void_p, ctypes.c_uint32, _T], ctypes.c_int),
    "aixb200_fill_min": ([_D, _T], ctypes.c_int),
    "aixb200_matmul": ([_D, _T, _T, _T], ctypes.c_int),
    "aixb200_transpose": ([_D, _T, _T, _SZ, _SZ], ctypes.c_int),
    "aixb200_copy": ([_D, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32, _SZ], ctypes.c_int),
    "aixb200_copy_immediate": ([_D, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32, _SZ], ctypes.c_int),
    "aixb200_argmax_to": ([_D, _T, _T, _SZ], ctypes.c_int),
    "aixb200_argmax_indices_to": ([_D, _T, _T, _SZ], ctypes.c_int),
    "aixb200_slice_set": ([_D, _T, _T, _SZ, _SZ, _SZ, _SZ], ctypes.c_int),
    "aixb200_tril": ([_D, _T, _T, ctypes.c_int64], ctypes.c_int),
    "aixb200_triu": ([_D, _T, _T, ctypes.c_int64], ctypes.c_int),
    "aixb200_index_select": ([_D, _T, _T, _T, _SZ], ctypes.c_int),
    "aixb200_index_add": ([_D, _T, _T, _T, _SZ], ctypes.c_int),
    "aixb200_get_stats": ([_D, ctypes.POINTER(Stats)], ctypes.c_int),
    "aixb200_last_kernel_source": ([_D], ctypes.c_char_p),
    "aixb200_event_create": ([_D, ctypes.POINTER(ctypes.c_void_p)], ctypes.c_int),
    "aixb200_event_record": ([_D, ctypes.c_void_p], ctypes.c_int),
    "aixb200_event_elapsed_ms": ([_D, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)], ctypes.c_int),
    "aixb200_event_destroy": ([_D, ctypes.c_void_p], ctypes.c_int),
    "aixb200_flush_l2": ([_D], ctypes.c_int),
    "aixb200_self_test_bounded_wait": ([_D, ctypes.c_uint64], ctypes.c_int),
    "aixb200_comm_unique_id": ([ctypes.c_void_p], ctypes.c_int),
    "aixb200_comm_init": ([_D, ctypes.c_int, ctypes.c_int, ctypes.c_void_p], ctypes.c_int),
    "aixb200_all_reduce": ([_D, ctypes.c_void_p, _SZ, ctypes.c_uint32, ctypes.c_double], ctypes.c_int),
    "aixb200_all_reduce_async": ([_D, ctypes.c_void_p, _SZ, ctypes.c_uint32, ctypes.c_double], ctypes.c_int),
    "aixb200_reduce_scatter_async": ([_D, ctypes.c_void_p, _SZ, ctypes.c_uint32, ctypes.c_double], ctypes.c_int),
    "aixb200_all_gather_async": ([_D, ctypes.c_void_p, _SZ, ctypes.c_uint32], ctypes.c_int),
    "aixb200_comm_rank": ([_D, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)], ctypes.c_int),
    "aixb200_comm_inject_backend": ([ctypes.c_int, ctypes.c_int], ctypes.c_int),
    "aixb200_comm_injected_counters": ([ctypes.POINTER(ctypes.c_int)] * 3, ctypes.c_int),
    "aixb200_comm_wait": ([_D], ctypes.c_int),
    "aixb200_comm_wait_for": ([_D, ctypes.c_void_p, _SZ], ctypes.c_int),
    "aixb200_comm_destroy": ([_D], ctypes.c_int),
}
for _name in ("add", "sub", "mul", "div", "pow"):
    SIGNATURES["aixb200_" + _name] = ([_D, _T, _T, _T], ctypes.c_int)
for _name in ("unary", "sqrt", "sin", "cos", "tanh", "log", "exp", "sum", "sum_static_scratch", "max", "argmax", "argmax_indices",
              "reduce_to", "max_to", "contiguous"):
    SIGNATURES["aixb200_" + _name] = ([_D, _T, _T], ctypes.c_int)

_lib = None


def load():
    """Returns the loaded library; raises if it has not been built (python -m aix_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m aix_b200.build`; "
                               "the B200 device has no fallback implementation")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
    return _lib
