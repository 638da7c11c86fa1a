"""Loads `libfrink_b200.so` (the C ABI in include/frink_b200.h) through ctypes.

There is no fallback: if the library is missing or does not load, importing
any launch surface of this package raises.  `python -m frink_b200.build`
compiles it in-tree.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FRINK_B200_LIB names another build of the same library (a kernel variant under study)
LIB_PATH = os.environ.get("FRINK_B200_LIB") or os.path.join(_HERE, "libfrink_b200.so")

FK_OK, FK_DRIVER_INIT, FK_KERNEL, FK_LAUNCH, FK_UNSUPPORTED, FK_COMM, FK_INVALID = range(7)

# every symbol include/frink_b200.h declares: (name, restype, argtypes)
_P, _I, _SZ = C.c_void_p, C.c_int, C.c_size_t
SYMBOLS = {
    "fk_init": (_I, [_I, C.POINTER(_P)]),
    "fk_destroy": (None, [_P]),
    "fk_last_error": (C.c_char_p, []),
    "fk_device_info": (_I, [_P, C.c_char_p, _SZ, C.POINTER(_I), C.POINTER(_SZ)]),
    "fk_counters": (_I, [_P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), _I]),
    "fk_device_error": (_I, [_P, C.POINTER(_I), _I]),
    "fk_block_bytes": (_I, [_I]),
    "fk_block_elems": (_I, [_I]),
    "fk_register_weights": (_I, [_P, _P, _SZ, _I, _I, _I, _I, C.POINTER(_P)]),
    "fk_register_weights_dev": (_I, [_P, _P, _SZ, _I, _I, _I, _I, _P, C.POINTER(_P)]),
    "fk_release_weights": (_I, [_P, _P]),
    "fk_weight_shape": (_I, [_P, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I), C.POINTER(_I), C.POINTER(_SZ)]),
    "fk_quantize_q8_1": (_I, [_P, _P, _P, _I, _P]),
    "fk_gemv": (_I, [_P, _P, _P, _I, _P, _I, _P]),
    "fk_gemv_fused": (_I, [_P, _P, _P, _I, _P, _I, _I, _P, _P, C.c_float, _P, _I, _I, _I]),
    "fk_gemv_multi": (_I, [_P, _P, _P, _P, _I, _P, _I, _P]),
    "fk_gemv_multi_glu": (_I, [_P, _P, _P, _P, _I, _P, _P, _I, _I, _P, _P]),
    "fk_gemv_biased": (_I, [_P, _P, _P, _I, _P, _I, _I, _P, _P, C.c_float, _P, _I]),
    "fk_gemv_multi_biased": (_I, [_P, _P, _P, _P, _I, _P, _P, _I, _I, _P, _P]),
    "fk_gemv_multi_gate_up": (_I, [_P, _P, _P, _P, _P, _I, _P, _I, _P, C.c_float, _P, _P, _P]),
    "fk_gemv_multi_active": (_I, [_P, _P, _P, _P, _I, _P, _I, _P, _P]),
    "fk_moe_layer_workspace": (_SZ, [_I, _I, _I, _I, _I]),
    "fk_moe_layer": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _I, _P, _I, _P, _SZ]),
    "fk_moe_layer_biased": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _I, _P, _I, _P, _SZ]),
    "fk_moe_layer_normed": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, C.c_float, _P, _I, _P, _I, _P, _SZ]),
    "fk_moe_local_pairs": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P]),
    "fk_moe_local_slots": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P, _P]),
    "fk_moe_localize": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "fk_gemv_isums": (_I, [_P, _P, _P, _I, _P, _P]),
    "fk_gemm": (_I, [_P, _P, _P, _I, _P, _I, _P]),
    "fk_gemm_isums": (_I, [_P, _P, _P, _I, _P, _I, _P, _P]),
    "fk_gemm_q8k": (_I, [_P, _P, _P, _I, _P, _I, _P]),
    "fk_gemm_q8k_isums": (_I, [_P, _P, _P, _I, _P, _I, _P, _P]),
    "fk_gemm_static": (_I, [_P, _P, _P, _I, _P, _I, _P]),
    "fk_gemm_grouped": (_I, [_P, _P, _P, _P, _P, _P, _I, _P]),
    "fk_moe_route": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "fk_router_logits": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "fk_moe_permute": (_I, [_P, _P, _P, _I, _I, _I, _P, _P, _P]),
    "fk_glu": (_I, [_P, _P, _P, _P, _SZ, _I, _P]),
    "fk_router_route": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _I, _I, _P, _P, _P]),
    "fk_moe_combine": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "fk_moe_combine_add": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "fk_get_rows": (_I, [_P, _P, _P, _I, _P, _I, _P]),
    "fk_rmsnorm": (_I, [_P, _P, _P, _P, _P, _I, _I, C.c_float, _P]),
    "fk_rope": (_I, [_P, _P, _P, _I, _I, _I, _P, C.c_float, _I]),
    "fk_rope_kv": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, C.c_float, _I, _P, _P, _P, _P, C.c_float, _I]),
    "fk_add": (_I, [_P, _P, _P, _P, _SZ]),
    "fk_kv_append": (_I, [_P, _P, _P, _P, _SZ, _I, _P, _I]),
    "fk_attention_rope_kv": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, C.c_float, C.c_float, _I, _P, _P, C.c_float, _P, _I, _I, _P]),
    "fk_attention_rope_kv_seqs": (_I, [_P, _P, _P, _I, _P, _P, _I, _I, _P, _P, _SZ, _I, _I, _I, _I, _P, C.c_float, C.c_float, _I, _P, _P, C.c_float, _P, _I, _I, _P]),
    "fk_attention": (_I, [_P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _P, C.c_float, _P, _I, _I, _P]),
    "fk_reserve_scratch": (_I, [_P, _SZ]),
    "fk_add_bias": (_I, [_P, _P, _P, _P, _P, _I, _I]),
    "fk_argmax": (_I, [_P, _P, _P, _I, _I, _P]),
    "fk_add_int": (_I, [_P, _P, _P, _I]),
    "fk_comm_create": (_I, [_P, _SZ, _I, _I, _P, C.POINTER(_P)]),
    "fk_comm_connect": (_I, [_P, _P]),
    "fk_comm_connect_local": (_I, [_P, C.POINTER(_P)]),
    "fk_comm_arena": (_I, [_P, C.POINTER(_P), C.POINTER(_SZ)]),
    "fk_comm_destroy": (_I, [_P]),
    "fk_comm_channel_bytes": (_SZ, [_I, _I]),
    "fk_allreduce": (_I, [_P, _P, _P, _SZ, _I, _P, _P, _I, _I, _I]),
    "fk_gemv_fused_allreduce": (_I, [_P, _P, _P, _I, _P, _I, _I, _P, _P, C.c_float, _P, _I, _I, _P, _SZ, _I, _I]),
    "fk_launch_matvec": (_I, [_P, _I, _P, _SZ, _P, _I, _I, _I, _P]),
    "fk_quantize_q8_1_host": (_I, [_P, _P, _I, _P]),
    "fk_launch_matvec_multi": (_I, [_P, _P, _I, _P, _I, _P]),
    "fk_launch_dense_ffn_swiglu": (_I, [_P, _P, _P, _P, _P, _I, _P]),
    "fk_launch_mul_mm": (_I, [_P, _I, _P, _SZ, _P, _I, _I, _I, _I, _P]),
    "fk_forget_resident": (_I, [_P]),
}


class CudaError(RuntimeError):
    """Mirror of frink-cuda's `CudaError` (crates/frink-cuda/src/gpu.rs:91-104)."""
    status = FK_LAUNCH


class DriverInit(CudaError):
    status = FK_DRIVER_INIT


class KernelCompile(CudaError):
    status = FK_KERNEL


class Launch(CudaError):
    status = FK_LAUNCH


class Unsupported(CudaError):
    """The caller must use a path that can compute the result, never something else."""
    status = FK_UNSUPPORTED


class Comm(CudaError):
    status = FK_COMM


class Invalid(CudaError, ValueError):
    status = FK_INVALID


_BY_STATUS = {c.status: c for c in (DriverInit, KernelCompile, Launch, Unsupported, Comm, Invalid)}
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise DriverInit(f"{LIB_PATH} is not built (run `python -m frink_b200.build`); there is no fallback path")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)  # AttributeError if the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc):
    if rc != FK_OK:
        msg = lib().fk_last_error().decode("utf-8", "replace")
        raise _BY_STATUS.get(rc, CudaError)(msg)
