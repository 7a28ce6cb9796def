"""ctypes view of the C ABI declared in include/rg_b200.h (struct layouts mirror the header one to one).

The library must be present: there is no CPU or eager fallback.  `load()` raises if librg_b200.so is missing.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librg_b200.so")

# rg_status
OK, ERR_NULL, ERR_SHAPE, ERR_DTYPE, ERR_ALIGN, ERR_CUDA, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_LIMIT = range(9)
# rg_dtype (= the reference's DataType codes)
F32, U8, I8, I32, I64, BOOL, FP16, F64, U32, BF16 = 1, 2, 3, 6, 7, 9, 10, 11, 12, 16
U16, I16, U64 = 4, 5, 13


class RmsNormParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rows", C.c_uint32), ("dim", C.c_uint32), ("epsilon", C.c_float),
                ("add_residual", C.c_int32)]


class SoftmaxParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("pre", C.c_uint32), ("mid", C.c_uint32), ("post", C.c_uint32)]


class TopkParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rows", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
                ("softmax", C.c_int32)]


class TopkSampleParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rows", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
                ("temperature", C.c_float), ("seed", C.c_uint64)]


class GatherParams(C.Structure):
    _fields_ = [("prefix", C.c_uint32), ("mid_in", C.c_uint32), ("mid_out", C.c_uint32),
                ("postfix_bytes", C.c_uint64), ("idx_dtype", C.c_int32)]


class BinaryParams(C.Structure):
    _fields_ = [("op", C.c_int32), ("dtype", C.c_int32), ("shape", C.c_uint32 * 4),
                ("a_stride", C.c_uint32 * 4), ("b_stride", C.c_uint32 * 4)]


class UnaryParams(C.Structure):
    _fields_ = [("op", C.c_int32), ("dtype", C.c_int32), ("n", C.c_uint64)]


class WhereParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("shape", C.c_uint32 * 4), ("c_stride", C.c_uint32 * 4),
                ("a_stride", C.c_uint32 * 4), ("b_stride", C.c_uint32 * 4)]


class TransposeParams(C.Structure):
    _fields_ = [("elem_bytes", C.c_uint32), ("rank", C.c_uint32), ("in_shape", C.c_uint32 * 4),
                ("perm", C.c_uint32 * 4)]


class ConcatParams(C.Structure):       # concat and split
    _fields_ = [("elem_bytes", C.c_uint32), ("n_parts", C.c_uint32), ("outer", C.c_uint32), ("inner", C.c_uint32), ("axis_len", C.c_uint32 * 32)]


class SliceParams(C.Structure):
    _fields_ = [("elem_bytes", C.c_uint32), ("rank", C.c_uint32), ("in_shape", C.c_uint32 * 6), ("start", C.c_int64 * 6), ("step", C.c_int64 * 6),
                ("length", C.c_uint32 * 6)]


class ExpandParams(C.Structure):
    _fields_ = [("elem_bytes", C.c_uint32), ("rank", C.c_uint32), ("in_shape", C.c_uint32 * 6), ("out_shape", C.c_uint32 * 6)]


class CastParams(C.Structure):
    _fields_ = [("from_", C.c_int32), ("to", C.c_int32), ("n", C.c_uint64)]


class RopeParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("tokens", C.c_uint32), ("heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("theta", C.c_float)]


class StateUpdateParams(C.Structure):
    _fields_ = [("n", C.c_uint32), ("delta", C.c_int64)]


class MatMulParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
                ("trans_a", C.c_int32), ("trans_b", C.c_int32), ("alpha", C.c_float), ("beta", C.c_float),
                ("batch", C.c_uint32), ("stride_a", C.c_uint64), ("stride_b", C.c_uint64), ("stride_y", C.c_uint64),
                ("has_bias", C.c_int32), ("bias_row_stride", C.c_uint32), ("bias_col_stride", C.c_uint32),
                ("stride_c", C.c_uint64), ("force_kernel", C.c_int32), ("flags", C.c_uint32)]


MM_B_STATIC = 1


class KvLayout(C.Structure):
    _fields_ = [("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("max_seq", C.c_uint32),
                ("page_size", C.c_uint32), ("max_blocks_per_seq", C.c_uint32), ("n_blocks", C.c_uint32)]


class LinearParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
                ("prologue", C.c_int32), ("epilogue", C.c_int32), ("epsilon", C.c_float), ("n_heads", C.c_uint32),
                ("theta", C.c_float), ("kv", KvLayout), ("tokens_per_seq", C.c_uint32)]


class QkvRopeAppendParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("tokens", C.c_uint32), ("n_heads", C.c_uint32), ("theta", C.c_float), ("kv", KvLayout),
                ("tokens_per_seq", C.c_uint32)]


class SwigluParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rows", C.c_uint32), ("f", C.c_uint32)]


class AttentionParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_uint32), ("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32),
                ("seq_len", C.c_uint32), ("head_dim", C.c_uint32), ("max_seq", C.c_uint32), ("has_cache", C.c_int32)]


class AttnPrefillParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_uint32), ("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32),
                ("seq_len", C.c_uint32), ("head_dim", C.c_uint32), ("kv_capacity", C.c_uint32), ("strides", C.c_int64 * 12)]


class AttnDecodeParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_uint32), ("n_heads", C.c_uint32), ("max_len", C.c_uint32),
                ("kv", KvLayout)]


class DecodeStepParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("layers", C.c_uint32), ("hidden", C.c_uint32), ("n_heads", C.c_uint32),
                ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("ffn", C.c_uint32), ("vocab", C.c_uint32),
                ("max_seq", C.c_uint32), ("epsilon", C.c_float), ("theta", C.c_float)]


class AllReduceParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("op", C.c_int32), ("count", C.c_uint64)]


class AllReduceNormParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rows", C.c_uint32), ("dim", C.c_uint32), ("epsilon", C.c_float)]


# name -> params struct, for every op with the (params, ws, in, out, stream) calling shape
OPS = {
    "rms_norm": RmsNormParams, "softmax": SoftmaxParams, "topk": TopkParams, "topk_sample": TopkSampleParams,
    "gather": GatherParams, "binary": BinaryParams, "unary": UnaryParams, "where": WhereParams,
    "transpose": TransposeParams, "rope": RopeParams, "state_update": StateUpdateParams, "mat_mul": MatMulParams, "linear": LinearParams,
    "attention": AttentionParams, "attn_decode": AttnDecodeParams, "qkv_rope_append": QkvRopeAppendParams,
    "swiglu": SwigluParams, "decode_step": DecodeStepParams, "attn_prefill": AttnPrefillParams,
    "concat": ConcatParams, "split": ConcatParams, "slice": SliceParams, "expand": ExpandParams, "cast": CastParams,
}
# every symbol include/rg_b200.h declares
SYMBOLS = (["rg_b200_status_string", "rg_b200_version", "rg_b200_launch_count", "rg_b200_error_state", "rg_b200_error_clear", "rg_b200_attn_decode_static",
            "rg_b200_attn_decode_static_capacity", "rg_b200_decode_step_timeline", "rg_b200_comm_create", "rg_b200_comm_base", "rg_b200_comm_bytes", "rg_b200_comm_connect_ptrs",
            "rg_b200_comm_set_wait_ns",
            "rg_b200_comm_connect", "rg_b200_comm_status", "rg_b200_comm_destroy", "rg_b200_all_reduce", "rg_b200_all_reduce_norm", "rg_b200_all_reduce_recv", "rg_b200_mat_mul_push"]
           + [f"rg_b200_{n}" for n in OPS] + [f"rg_b200_{n}_workspace" for n in OPS])

_lib = None


def load() -> C.CDLL:
    """Load librg_b200.so (built by __graft_entry__.build() / make -C refactorgraph_b200/csrc)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()'). "
                               "There is no fallback path.")
        lib = C.CDLL(LIB_PATH)
        lib.rg_b200_status_string.restype = C.c_char_p
        lib.rg_b200_launch_count.restype = C.c_uint64
        for name, ptype in OPS.items():
            fn = getattr(lib, f"rg_b200_{name}")
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(ptype), C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p]
            ws = getattr(lib, f"rg_b200_{name}_workspace")
            ws.restype = C.c_size_t
            ws.argtypes = [C.POINTER(ptype)]
        lib.rg_b200_attn_decode_static_capacity.restype = C.c_size_t
        lib.rg_b200_attn_decode_static.restype = C.c_int
        lib.rg_b200_attn_decode_static.argtypes = [C.POINTER(AttnDecodeParams), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p]
        lib.rg_b200_decode_step_timeline.restype = C.c_size_t
        lib.rg_b200_decode_step_timeline.argtypes = [C.POINTER(DecodeStepParams), C.c_void_p, C.POINTER(C.c_uint64), C.c_size_t]
        lib.rg_b200_comm_create.argtypes = [C.c_int, C.c_int, C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]
        lib.rg_b200_comm_connect.argtypes = [C.c_void_p, C.c_void_p]
        lib.rg_b200_comm_status.argtypes = [C.c_void_p]
        lib.rg_b200_comm_base.restype = C.c_void_p
        lib.rg_b200_comm_base.argtypes = [C.c_void_p]
        lib.rg_b200_comm_bytes.restype = C.c_size_t
        lib.rg_b200_comm_bytes.argtypes = [C.c_void_p]
        lib.rg_b200_comm_connect_ptrs.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        lib.rg_b200_comm_set_wait_ns.argtypes = [C.c_void_p, C.c_uint64]
        lib.rg_b200_comm_destroy.argtypes = [C.c_void_p]
        lib.rg_b200_all_reduce.argtypes = [C.c_void_p, C.POINTER(AllReduceParams), C.POINTER(C.c_void_p),
                                           C.POINTER(C.c_void_p), C.c_void_p]
        lib.rg_b200_all_reduce_recv.argtypes = [C.c_void_p, C.POINTER(AllReduceParams), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p]
        lib.rg_b200_mat_mul_push.argtypes = [C.c_void_p, C.POINTER(MatMulParams), C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p]
        lib.rg_b200_all_reduce_norm.argtypes = [C.c_void_p, C.POINTER(AllReduceNormParams), C.POINTER(C.c_void_p),
                                                C.POINTER(C.c_void_p), C.c_void_p]
        _lib = lib
    return _lib


class RgError(RuntimeError):
    def __init__(self, op: str, status: int):
        self.status = status
        super().__init__(f"rg_b200_{op}: {load().rg_b200_status_string(status).decode()} (status {status})")


def _ptrs(ptrs):
    arr = (C.c_void_p * max(1, len(ptrs)))()
    for i, p in enumerate(ptrs):
        arr[i] = p if p else None
    return arr


def workspace(op: str, params) -> int:
    return int(getattr(load(), f"rg_b200_{op}_workspace")(C.byref(params)))


def call(op: str, params, inputs, outputs, ws: int = 0, stream: int = 0, check: bool = True) -> int:
    """Invoke rg_b200_<op> with raw device addresses (ints; 0/None = NULL)."""
    rc = getattr(load(), f"rg_b200_{op}")(C.byref(params), ws or None, _ptrs(inputs), _ptrs(outputs), stream or None)
    if check and rc != OK:
        raise RgError(op, rc)
    return rc


def attn_decode_static(params, inputs, outputs, stream: int = 0, check: bool = True) -> int:
    """rg_b200_attn_decode_static: flash-decoding with library-owned scratch (no workspace argument)."""
    rc = load().rg_b200_attn_decode_static(C.byref(params), _ptrs(inputs), _ptrs(outputs), stream or None)
    if check and rc != OK:
        raise RgError("attn_decode_static", rc)
    return rc


class Comm:
    """One rank's NVLink peer-memory communicator (rg_b200_comm_*).  `exchange(handle: bytes) -> list[bytes]` is any
    host transport that returns every rank's 64-byte handle in rank order (e.g. torch.distributed.all_gather_object)."""

    def __init__(self, world: int, rank: int, capacity_bytes: int, exchange=None):
        lib = load()
        self.world, self.rank = world, rank
        self._ptr = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        rc = lib.rg_b200_comm_create(world, rank, capacity_bytes, C.byref(self._ptr), handle)
        if rc != OK:
            raise RgError("comm_create", rc)
        if world > 1 and exchange is not None:
            handles = exchange(bytes(handle))
            blob = (C.c_ubyte * (64 * world)).from_buffer_copy(b"".join(handles))
            rc = lib.rg_b200_comm_connect(self._ptr, blob)
            if rc != OK:
                raise RgError("comm_connect", rc)

    @property
    def address(self) -> int:
        return self._ptr.value

    def connect_ptrs(self, bases):
        arr = (C.c_void_p * self.world)(*bases)
        rc = load().rg_b200_comm_connect_ptrs(self._ptr, arr)
        if rc != OK:
            raise RgError("comm_connect_ptrs", rc)

    def base(self) -> int:
        return load().rg_b200_comm_base(self._ptr)

    def nbytes(self) -> int:
        return load().rg_b200_comm_bytes(self._ptr)

    def set_wait_ns(self, ns: int):
        load().rg_b200_comm_set_wait_ns(self._ptr, ns)

    def all_reduce(self, dtype: int, op: int, count: int, x: int, y: int, residual: int = 0, stream: int = 0, check: bool = True) -> int:
        p = AllReduceParams(dtype, op, count)
        rc = load().rg_b200_all_reduce(self._ptr, C.byref(p), _ptrs([x, residual]), _ptrs([y]), stream or None)
        if check and rc != OK:
            raise RgError("all_reduce", rc)
        return rc

    def mat_mul_push(self, p, a: int, b: int, ws: int = 0, stream: int = 0, check: bool = True) -> int:
        """Row-parallel product whose epilogue writes this rank's all-reduce input into the peers' slots (p: MatMulParams)."""
        rc = load().rg_b200_mat_mul_push(self._ptr, C.byref(p), ws or None, _ptrs([a, b]), stream or None)
        if check and rc != OK:
            raise RgError("mat_mul_push", rc)
        return rc

    def all_reduce_recv(self, dtype: int, count: int, y: int, residual: int = 0, stream: int = 0, check: bool = True) -> int:
        """Receiving half of an all-reduce (Sum) whose input a mat_mul_push has already delivered."""
        p = AllReduceParams(dtype, 0, count)
        rc = load().rg_b200_all_reduce_recv(self._ptr, C.byref(p), _ptrs([residual]), _ptrs([y]), stream or None)
        if check and rc != OK:
            raise RgError("all_reduce_recv", rc)
        return rc

    def all_reduce_norm(self, dtype: int, rows: int, dim: int, eps: float, x: int, w: int, y: int, n: int, residual: int = 0,
                        stream: int = 0, check: bool = True) -> int:
        """y = sum over ranks of x (+ residual), n = rmsnorm(y) * w, in one launch."""
        p = AllReduceNormParams(dtype, rows, dim, eps)
        rc = load().rg_b200_all_reduce_norm(self._ptr, C.byref(p), _ptrs([x, residual, w]), _ptrs([y, n]), stream or None)
        if check and rc != OK:
            raise RgError("all_reduce_norm", rc)
        return rc

    def status(self) -> int:
        return load().rg_b200_comm_status(self._ptr)

    def destroy(self):
        if self._ptr:
            load().rg_b200_comm_destroy(self._ptr)
            self._ptr = C.c_void_p()
