"""ctypes binding of ``include/smelt_cuda.h`` — the only way Python reaches the CUDA kernels.

There is no fallback: if ``libsmelt_cuda.so`` is missing it is built with nvcc, and if that
fails, or no CUDA device is usable, the call raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libsmelt_cuda.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "smelt_cuda.h")

STATUS_NAMES = {
    0: "OK", 1: "BAD_ARGUMENT", 2: "UNKNOWN_PIPELINE", 3: "OUT_OF_RANGE", 4: "CUDA", 5: "ALLOC", 6: "UNSUPPORTED",
    7: "COMM", 8: "DEVICE_TIMEOUT",
}
OK, BAD_ARGUMENT, UNKNOWN_PIPELINE, OUT_OF_RANGE, CUDA, ALLOC, UNSUPPORTED, COMM, DEVICE_TIMEOUT = range(9)

CONST_LITERAL_U32, CONST_LITERAL_F32, CONST_POSITION, CONST_POSITION_PLUS1 = 0, 1, 2, 3
CONST_SKIP_UNLESS_POS1_LT, CONST_SKIP_UNLESS_POS1_GE, CONST_CACHE_SEQ_CAPACITY = 10, 11, 12
SLOT_CUR, SLOT_ALT = -1, -2
TP_ID_BYTES = 128
TP_HANDLE_BYTES = 64
TP_HANDLE_BYTES = 64


class SmeltError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libsmelt_cuda: {STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class BufferRecord(C.Structure):
    _fields_ = [("slot", C.c_int16), ("binding_index", C.c_uint8), ("offset_kind", C.c_uint8), ("_pad", C.c_uint32),
                ("offset", C.c_uint64)]


class ConstantRecord(C.Structure):
    _fields_ = [("kind", C.c_uint8), ("binding_index", C.c_uint8), ("pad", C.c_uint16), ("value", C.c_uint32)]


class DispatchRecord(C.Structure):
    _fields_ = [("op_kind", C.c_uint8), ("_pad0", C.c_uint8), ("pipeline", C.c_uint16), ("style", C.c_uint8),
                ("buffer_count", C.c_uint8), ("constant_count", C.c_uint8), ("_pad1", C.c_uint8),
                ("min_seq_len", C.c_uint16), ("_pad2", C.c_uint16), ("grid", C.c_uint32 * 3),
                ("threadgroup", C.c_uint32 * 3), ("_pad3", C.c_uint32), ("buf", BufferRecord * 16),
                ("con", ConstantRecord * 8)]


class RuntimeConfig(C.Structure):
    _fields_ = [("token_id_slot", C.c_int32), ("position_slot", C.c_int32), ("weights_slot", C.c_int32),
                ("argmax_slot", C.c_int32), ("cur_slot", C.c_int32), ("alt_slot", C.c_int32),
                ("cache_seq_capacity", C.c_uint32), ("context_limit", C.c_uint32), ("vocab_size", C.c_uint32),
                ("batch", C.c_uint32)]


class AffineRef(C.Structure):
    _fields_ = [("packed", C.c_uint64), ("scales", C.c_uint64), ("biases", C.c_uint64)]


class AffineTensor(C.Structure):
    """``smelt_affine_tensor``: one weight tensor and its output for ``affine_multi_matvec``."""

    _fields_ = [("w_dev", C.c_void_p), ("scales_dev", C.c_void_p), ("biases_dev", C.c_void_p), ("y_dev", C.c_void_p),
                ("rows", C.c_int32)]


class LayerRef(C.Structure):
    _fields_ = [("input_norm", C.c_uint64), ("post_norm", C.c_uint64), ("q", AffineRef), ("k", AffineRef),
                ("v", AffineRef), ("o", AffineRef), ("gate", AffineRef), ("up", AffineRef), ("down", AffineRef)]


class DecoderDesc(C.Structure):
    _fields_ = [("layers", C.c_int32), ("hidden", C.c_int32), ("inter", C.c_int32), ("n_q", C.c_int32),
                ("n_kv", C.c_int32), ("head_dim", C.c_int32), ("vocab", C.c_int32), ("group", C.c_int32),
                ("eps", C.c_float), ("rope_theta", C.c_float), ("embedding", C.c_uint64), ("lm_head", C.c_uint64),
                ("final_norm", C.c_uint64), ("tp_world", C.c_int32), ("tp_rank", C.c_int32),
                ("fuse_residual", C.c_int32)]


class DeltaDesc(C.Structure):
    """``smelt_delta_desc``: the linear-attention geometry of a hybrid decoder's DeltaNet layers."""
    _fields_ = [("value_heads", C.c_int32), ("qk_heads", C.c_int32), ("head_dim", C.c_int32), ("conv_kernel", C.c_int32)]


class DeltaRef(C.Structure):
    """``smelt_delta_ref``: one DeltaNet layer's mixer tensors inside the weights image."""
    _fields_ = [("qkv", AffineRef), ("z", AffineRef), ("a", AffineRef), ("b", AffineRef), ("out", AffineRef),
                ("conv_weight", C.c_uint64), ("a_log", C.c_uint64), ("dt_bias", C.c_uint64), ("norm_weight", C.c_uint64)]


class PackageOptions(C.Structure):
    _fields_ = [("context_capacity", C.c_uint32), ("context_limit", C.c_uint32)]


class PackageInfo(C.Structure):
    _fields_ = [("n_records", C.c_uint32), ("n_pipelines", C.c_uint32), ("n_pipelines_used", C.c_uint32), ("n_slots", C.c_uint32),
                ("n_weight_entries", C.c_uint32), ("vocab_size", C.c_uint32), ("hidden_size", C.c_uint32), ("num_layers", C.c_uint32),
                ("cache_seq_capacity", C.c_uint32), ("token_id_slot", C.c_int32), ("position_slot", C.c_int32), ("weights_slot", C.c_int32),
                ("argmax_slot", C.c_int32), ("logits_slot", C.c_int32), ("weights_bytes", C.c_uint64),
                ("n_prefill_records", C.c_uint32), ("_pad", C.c_uint32)]


class KvSlot(C.Structure):
    _fields_ = [("slot", C.c_int32), ("rows", C.c_int32), ("head_dim", C.c_int32)]


class SnapshotInfo(C.Structure):
    _fields_ = [("captured_length", C.c_uint32), ("prompt_length", C.c_uint32), ("next_token", C.c_int32), ("n_slots", C.c_uint32),
                ("byte_count", C.c_uint64), ("blob_bytes", C.c_uint64)]


def _declarations() -> dict[str, list[str]]:
    """name -> parameter type strings, parsed from ``smelt_cuda.h``."""
    with open(HEADER_PATH) as f:
        text = re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)
    out = {}
    for m in re.finditer(r"SMELT_CUDA_API\s+[\w\s\*]+?\b(smelt_cuda_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        params = [" ".join(p.split()) for p in m.group(2).split(",")]
        out[m.group(1)] = [] if params == ["void"] else params
    return out


def declared_symbols() -> list[str]:
    """Every entry point ``smelt_cuda.h`` declares."""
    return sorted(_declarations())


def _ctype_of(param: str):
    if "*" in param or "[" in param:
        return C.c_char_p if param.startswith("const char") else C.c_void_p  # char* out buffers stay void*
    t = param.rsplit(" ", 1)[0].replace("const ", "").strip()
    return {"int": C.c_int, "int32_t": C.c_int32, "uint32_t": C.c_uint32, "size_t": C.c_size_t, "float": C.c_float,
            "uint64_t": C.c_uint64}[t]


_lib = None


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load ``libsmelt_cuda.so`` (building it in-tree if absent).  Needs no GPU."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if not build_if_missing:
            raise FileNotFoundError(LIB_PATH)
        from . import build as _build

        _build.build()
    lib = C.CDLL(LIB_PATH)
    lib.smelt_cuda_last_error.restype = C.c_char_p
    lib.smelt_cuda_stream.restype = C.c_void_p
    lib.smelt_cuda_destroy.restype = None
    for name, params in _declarations().items():
        fn = getattr(lib, name)  # raises AttributeError when the library lacks a declared symbol
        fn.argtypes = [_ctype_of(p) for p in params]
        if name not in ("smelt_cuda_last_error", "smelt_cuda_stream", "smelt_cuda_destroy"):
            fn.restype = C.c_int32
    _lib = lib
    return lib


def _vp(x):
    if isinstance(x, DeviceBuffer):
        return x.ptr
    if isinstance(x, np.ndarray):
        return x.ctypes.data_as(C.c_void_p)
    if isinstance(x, str):
        return x.encode()
    return x


class DeviceBuffer:
    """A device allocation owned through the C ABI."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx, self.nbytes = ctx, int(nbytes)
        p = C.c_void_p()
        ctx._check(ctx.lib.smelt_cuda_malloc(ctx.h, C.c_size_t(self.nbytes), C.byref(p)))
        self.ptr = p.value

    def upload(self, arr: np.ndarray, offset: int = 0) -> "DeviceBuffer":
        arr = np.ascontiguousarray(arr)
        assert offset + arr.nbytes <= self.nbytes
        self.ctx._check(self.ctx.lib.smelt_cuda_memcpy_h2d(self.ctx.h, C.c_void_p(self.ptr + offset), arr.ctypes.data_as(C.c_void_p), C.c_size_t(arr.nbytes)))
        return self

    def download(self, dtype, shape, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert offset + out.nbytes <= self.nbytes
        self.ctx._check(self.ctx.lib.smelt_cuda_memcpy_d2h(self.ctx.h, out.ctypes.data_as(C.c_void_p), C.c_void_p(self.ptr + offset), C.c_size_t(out.nbytes)))
        return out

    def fill(self, byte: int) -> "DeviceBuffer":
        self.ctx._check(self.ctx.lib.smelt_cuda_memset(self.ctx.h, C.c_void_p(self.ptr), int(byte), C.c_size_t(self.nbytes)))
        return self

    def free(self):
        if self.ptr:
            self.ctx.lib.smelt_cuda_free(self.ctx.h, C.c_void_p(self.ptr))
            self.ptr = None

    def at(self, offset: int) -> int:
        return self.ptr + offset


class Context:
    """One device, one stream (SmeltRuntime is single-threaded per instance)."""

    def __init__(self, device: int = 0):
        self.lib = load()
        h = C.c_void_p()
        st = self.lib.smelt_cuda_create(int(device), C.byref(h))
        if st != 0:
            raise SmeltError(st, f"smelt_cuda_create(device={device}) failed: no usable sm_100 CUDA device, and there is no CPU fallback")
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.smelt_cuda_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int):
        if status != 0:
            raise SmeltError(status, (self.lib.smelt_cuda_last_error(self.h) or b"").decode())

    def status_of(self, status: int) -> tuple[int, str]:
        return status, (self.lib.smelt_cuda_last_error(self.h) or b"").decode()

    # memory
    def alloc(self, nbytes: int) -> DeviceBuffer:
        return DeviceBuffer(self, nbytes)

    def to_device(self, arr: np.ndarray) -> DeviceBuffer:
        arr = np.ascontiguousarray(arr)
        return DeviceBuffer(self, max(arr.nbytes, 16)).upload(arr)

    def synchronize(self):
        self._check(self.lib.smelt_cuda_synchronize(self.h))

    def device_error(self) -> int:
        flags = C.c_uint32(0)
        self._check(self.lib.smelt_cuda_device_error(self.h, C.byref(flags)))
        return flags.value

    def device_error_flags(self) -> int:
        """The device error word, read and cleared, without raising when it is non-zero."""
        flags = C.c_uint32(0)
        st = self.lib.smelt_cuda_device_error(self.h, C.byref(flags))
        if st not in (OK, DEVICE_TIMEOUT):
            self._check(st)
        return flags.value

    @property
    def stream(self) -> int:
        return self.lib.smelt_cuda_stream(self.h)

    @property
    def sm_count(self) -> int:
        return self.lib.smelt_cuda_sm_count(self.h)

    def call(self, name: str, *args):
        """Call ``smelt_cuda_<name>(ctx, *args)`` and raise on a non-zero status."""
        self._check(getattr(self.lib, "smelt_cuda_" + name)(self.h, *[_vp(a) for a in args]))

    def call_status(self, name: str, *args) -> int:
        return getattr(self.lib, "smelt_cuda_" + name)(self.h, *[_vp(a) for a in args])

    def last_error(self) -> str:
        return (self.lib.smelt_cuda_last_error(self.h) or b"").decode()
