"""ctypes binding of libcutile_b200.so (the C ABI in include/cutile_b200.h).

The library is the product; this module only loads it and declares the
signatures.  There is no fallback: if the shared object is missing the import
fails with instructions to build it, and on a machine without an sm_100 GPU
every compute call fails with CtbError(NO_DEVICE).
"""
import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcutile_b200.so")

OK, BAD_ARG, BAD_ALIGN, UNSUPPORTED_TILE, UNSUPPORTED, CUDA_ERROR, NCCL_ERROR, TIMEOUT, NO_DEVICE = range(9)
F32, F16, BF16 = 0, 1, 2


class CtbError(RuntimeError):
    """Raised for every non-zero status; `.status` is the ctb_status code."""

    def __init__(self, status, message):
        super().__init__(f"{status_string(status)}: {message}")
        self.status = status


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing. Build it with `python cutile.jl_b200/csrc/build.py` "
        "(needs nvcc with sm_100a support); there is no CPU fallback.")

lib = C.CDLL(LIB_PATH)

_p, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float
_pp = C.POINTER(C.c_void_p)

EP_MAX_RANKS = 8


class EpBuffers(C.Structure):
    """ctb_ep_buffers: addresses of every rank's receive / output buffers, valid on the calling device."""
    _fields_ = [("world", _i), ("rank", _i), ("recv_rows", _p * EP_MAX_RANKS), ("recv_ids", _p * EP_MAX_RANKS),
                ("recv_gates", _p * EP_MAX_RANKS), ("slot_out", _p * EP_MAX_RANKS), ("flags", _p * EP_MAX_RANKS),
                ("epoch", _p)]


# name -> argument types (return type is int unless listed in _RESTYPES)
SIGNATURES = {
    "ctb_create": [C.POINTER(_p), _i],
    "ctb_destroy": [_p],
    "ctb_last_error": [],
    "ctb_status_string": [_i],
    "ctb_version_info": [C.c_char_p, C.c_size_t],
    "ctb_check_device_status": [_p, _p],
    "ctb_set_flag_wait_limit": [_p, C.c_uint64],
    "ctb_set_tf32_rounding": [_p, _i],
    "ctb_validate_hints": [_i, _i, _i, _i],
    "ctb_softmax": [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _i, _i],
    "ctb_vadd": [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i],
    "ctb_transpose": [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i, _i, _i],
    "ctb_tiled_broadcast": [_p, _p, _p, C.POINTER(_i64), C.POINTER(_p), C.POINTER(_i64), _i, C.POINTER(C.c_int32), _i,
                            C.POINTER(C.c_float), _i, _i],
    "ctb_tiled_compile": [C.POINTER(C.c_int32), _i, _i, _i, C.POINTER(C.c_uint32), C.POINTER(_i)],
    "ctb_tiled_mapreduce": [_p, _p, _p, _p, C.POINTER(_i64), _i, _i, _i, _i],
    "ctb_fft": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i64, _i, _i],
    "ctb_layernorm_fwd": [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i],
    "ctb_layernorm_bwd_dx_partial_dwdb": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64,
                                          _i, _i],
    "ctb_layernorm_bwd_dwdb": [_p, _p, _p, _p, _p, _p, _i64, _i, _i, _i],
    "ctb_gemm": [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i],
    "ctb_gemm_batched": [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i,
                         _i],
    "ctb_fmha_fwd": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f, C.c_int32, _i, _i, _i, _i,
                     _i],
    "ctb_layernorm_bwd_static": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64],
    "ctb_layernorm_bwd_static_status": [_p],
    "ctb_moe_max_blocks": [_i64, _i64, _i64, _i],
    "ctb_moe_router": [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i],
    "ctb_moe_align": [_p, _p, _p, _i, _i64, _i64, _i64, _i, _p, _p, _p, _i64],
    "ctb_moe_fused_gemm": [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _i],
    "ctb_moe_silu_and_mul": [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i],
    "ctb_moe_gather_rows": [_p, _p, _p, _p, _p, _i64, _i64, _i, _i64],
    "ctb_moe_scatter_rows": [_p, _p, _p, _p, _p, _i64, _i64, _i64],
    "ctb_moe_combine": [_p, _p, _p, _p, _i64, _i64, _i64],
    "ctb_moe_ffn": [_p, _p, _p, _p, _p, _p, _p, _i, _p, _i64, _i64, _i64, _i64, _i64, _i, _i, _i],
    "ctb_moe_ep_dispatch": [_p, _p, C.POINTER(EpBuffers), _p, _p, _p, _i64, _i64, _i64, _i64],
    "ctb_moe_ep_barrier": [_p, _p, C.POINTER(EpBuffers)],
    "ctb_moe_ep_experts": [_p, _p, C.POINTER(EpBuffers), _p, _p, _i64, _i64, _i64, _i64, _i, _i, _i],
    "ctb_create_multi": [C.POINTER(_p), C.POINTER(_i), _i],
    "ctb_destroy_multi": [_p],
    "ctb_group_size": [_p],
    "ctb_group_ctx": [_p, _i],
    "ctb_comm_unique_id": [_p],
    "ctb_comm_init_rank": [_p, _p, _i, _i],
    "ctb_comm_abort": [_p],
    "ctb_comm_info": [_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)],
    "ctb_gemm_batched_sharded": [_p, _pp, _pp, _pp, _pp, _i64, _i64, _i64, C.POINTER(_i64), _i64, _i64, _i64, _i64, _i64,
                                 _i64, _i, _i, _i, _i],
    "ctb_fmha_fwd_sharded": [_p, _pp, _pp, _pp, _pp, _pp, _i64, _i64, _i64, _i64, _i64, _i64, C.POINTER(_i64), _f,
                             C.c_int32, _i, _i, _i, _i, _i],
    "ctb_ep_create": [_p, _i, _i, _i64, _i64, _i64, C.POINTER(_p)],
    "ctb_ep_destroy": [_p],
    "ctb_ep_export": [_p, _p],
    "ctb_ep_import": [_p, _i, _p],
    "ctb_ep_connect_local": [_pp, _i],
    "ctb_ep_table": [_p],
    "ctb_moe_ffn_ep": [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i],
    "ctb_moe_ffn_ep_group": [_p, _pp, _pp, _pp, _pp, _pp, _pp, _pp, _pp, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i],
    "ctb_workspace_bytes": [_i, C.POINTER(_i64), _i],
    "ctb_reserve_workspace": [_p, _p, C.c_size_t],
}
_RESTYPES = {"ctb_destroy": None, "ctb_last_error": C.c_char_p, "ctb_status_string": C.c_char_p,
             "ctb_moe_max_blocks": _i64, "ctb_destroy_multi": None, "ctb_ep_destroy": None, "ctb_group_ctx": _p,
             "ctb_ep_table": C.POINTER(EpBuffers), "ctb_workspace_bytes": C.c_size_t}
UNIQUE_ID_BYTES, EP_HANDLE_BYTES = 128, 64
A2A_NCCL, A2A_PEER = 0, 1
OP_MOE_FFN, OP_MOE_EP = 1, 2

for _name, _args in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = header and library disagree
    _fn.argtypes = _args
    _fn.restype = _RESTYPES.get(_name, _i)


def status_string(status):
    return lib.ctb_status_string(int(status)).decode()


def last_error():
    return lib.ctb_last_error().decode()


def check(status):
    if status != OK:
        raise CtbError(status, last_error())


def version_info():
    buf = C.create_string_buffer(256)
    check(lib.ctb_version_info(buf, 256))
    return buf.value.decode()


_ctx_lock = threading.Lock()
_ctxs = {}


def context(device):
    """The per-device context of this process (created on first use)."""
    with _ctx_lock:
        h = _ctxs.get(device)
        if h is None:
            out = _p()
            check(lib.ctb_create(C.byref(out), int(device)))
            h = _ctxs[device] = out
        return h


def check_device_status(device, stream=0):
    check(lib.ctb_check_device_status(context(device), _p(stream)))


def set_tf32_rounding(device, nearest_even):
    """f32 GEMM operands: False = truncated by the tensor core (default), True = rounded to nearest even first, like
    the reference's f32 -> tf32 conversion."""
    check(lib.ctb_set_tf32_rounding(context(device), 1 if nearest_even else 0))


def set_flag_wait_limit(device, nanoseconds):
    """How long kernels of the device's context wait for another rank's flag before they give up (2 s by default)."""
    check(lib.ctb_set_flag_wait_limit(context(device), int(nanoseconds)))
