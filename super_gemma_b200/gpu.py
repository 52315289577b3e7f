"""Host-side mirror of the slice of ``sg-gpu`` that the attention path uses, over the C ABI of
``libsgattn.so`` (``include/sgattn.h``).

Names, argument meaning and error behaviour follow the reference's Rust API
(``crates/sg-gpu/src/lib.rs:20-44``): ``GpuContext`` (``context.rs:103``), ``Buffer`` and
``BufferBinding`` (``buffer.rs:80``), ``Kernel`` / ``load_kernel`` (``kernel.rs:79``),
``dispatch`` / ``dispatch_blocking`` (``graph.rs:203``, ``exec.rs:12``), ``record_graph`` /
``submit_blocking`` (``graph.rs:523-528,640``), ``StepState`` (``graph.rs:29-61``), ``GpuTimer``
(``graph.rs:404-473``) and the ``GpuError`` variants.  There is no fallback of any kind: if the
CUDA library is missing or no B200 is present, construction raises.
"""
from __future__ import annotations

import ctypes as C
import os
import struct
from dataclasses import dataclass
from typing import Callable, Iterable, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsgattn.so")

SGB_OK, SGB_ERR_NO_DEVICE, SGB_ERR_UNKNOWN_KERNEL, SGB_ERR_VALIDATION, SGB_ERR_CUDA, SGB_ERR_TIMEOUT, SGB_ERR_BOUNDS, \
    SGB_ERR_STATE = range(8)


class GpuError(Exception):
    """Base of the error variants (``GpuError`` in crates/sg-gpu/src/lib.rs:30-44)."""

    code = -1


class NoDevice(GpuError):
    code = SGB_ERR_NO_DEVICE


class UnknownKernel(GpuError):
    code = SGB_ERR_UNKNOWN_KERNEL


class Validation(GpuError):
    code = SGB_ERR_VALIDATION


class CudaError(GpuError):
    code = SGB_ERR_CUDA


class Timeout(GpuError):
    code = SGB_ERR_TIMEOUT


class Bounds(GpuError):
    code = SGB_ERR_BOUNDS


class State(GpuError):
    code = SGB_ERR_STATE


_BY_CODE = {c.code: c for c in (NoDevice, UnknownKernel, Validation, CudaError, Timeout, Bounds, State)}


class _KernelInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("workgroup", C.c_uint32 * 3), ("bindings", C.c_uint32), ("push_bytes", C.c_uint32),
                ("signature", C.c_char_p)]


class _Binding(C.Structure):
    _fields_ = [("index", C.c_uint32), ("buffer", C.c_void_p)]


class _Cache2Stats(C.Structure):
    _fields_ = [("page_tokens", C.c_uint32), ("pool_pages", C.c_uint32), ("free_pages", C.c_uint32),
                ("reclaimable_pages", C.c_uint32), ("live_sequences", C.c_uint32), ("reserved", C.c_uint32),
                ("hits", C.c_uint64), ("misses", C.c_uint64), ("evictions", C.c_uint64)]


# Every symbol include/sgattn.h declares: (restype, argtypes).
_vp, _u32, _u64, _sz, _int = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t, C.c_int
_PP = C.POINTER(C.c_void_p)
ABI = {
    "sgb_version": (C.c_char_p, []),
    "sgb_last_error": (C.c_char_p, []),
    "sgb_ctx_create": (_int, [_int, _PP]),
    "sgb_ctx_create_on_stream": (_int, [_int, _vp, _PP]),
    "sgb_ctx_destroy": (None, [_vp]),
    "sgb_ctx_device": (_int, [_vp]),
    "sgb_ctx_stream": (_vp, [_vp]),
    "sgb_ctx_sm_count": (_int, [_vp]),
    "sgb_sync": (_int, [_vp, _u32]),
    "sgb_buffer_create": (_int, [_vp, _sz, _PP]),
    "sgb_buffer_adopt": (_int, [_vp, _vp, _sz, _PP]),
    "sgb_buffer_slice": (_int, [_vp, _sz, _sz, _PP]),
    "sgb_buffer_retain": (None, [_vp]),
    "sgb_buffer_release": (None, [_vp]),
    "sgb_buffer_device_ptr": (_vp, [_vp]),
    "sgb_buffer_bytes": (_sz, [_vp]),
    "sgb_buffer_upload": (_int, [_vp, _sz, _vp, _sz]),
    "sgb_buffer_download": (_int, [_vp, _sz, _vp, _sz]),
    "sgb_buffer_upload_async": (_int, [_vp, _sz, _vp, _sz]),
    "sgb_buffer_download_async": (_int, [_vp, _sz, _vp, _sz]),
    "sgb_buffer_fill_zero": (_int, [_vp]),
    "sgb_host_alloc": (_int, [_sz, _PP]),
    "sgb_host_free": (None, [_vp]),
    "sgb_step_write": (_int, [_vp, _u32, _u32, _u32, _u32]),
    "sgb_kernel_count": (_int, []),
    "sgb_kernel_info_at": (_int, [_int, C.POINTER(_KernelInfo)]),
    "sgb_kernel_get": (_int, [_vp, C.c_char_p, _PP]),
    "sgb_kernel_describe": (_int, [_vp, C.POINTER(_KernelInfo)]),
    "sgb_dispatch": (_int, [_vp, _vp, C.POINTER(_Binding), _u32, _vp, _sz, C.POINTER(_u32)]),
    "sgb_dispatch_blocking": (_int, [_vp, _vp, C.POINTER(_Binding), _u32, _vp, _sz, C.POINTER(_u32)]),
    "sgb_launch_count": (_u64, [_vp]),
    "sgb_decode_paged_splits_hint": (_u32, [_vp, _u32, _u32]),
    "sgb_graph_begin": (_int, [_vp]),
    "sgb_graph_end": (_int, [_vp, _PP]),
    "sgb_graph_launch": (_int, [_vp, _vp]),
    "sgb_graph_destroy": (None, [_vp]),
    "sgb_timer_create": (_int, [_vp, _u32, _PP]),
    "sgb_timer_stamp": (_int, [_vp, _vp, _u32]),
    "sgb_timer_read_ns": (_int, [_vp, C.POINTER(_u64), _u32]),
    "sgb_timer_destroy": (None, [_vp]),
    "sgb_cache2_create": (_int, [_u32, _u32, _PP]),
    "sgb_cache2_destroy": (None, [_vp]),
    "sgb_cache2_lookup": (_int, [_vp, _vp, _u64, C.POINTER(_u64)]),
    "sgb_cache2_acquire": (_int, [_vp, _vp, _u64, _u64, _vp, _u32, C.POINTER(_u32), C.POINTER(_u64), C.POINTER(_u64)]),
    "sgb_cache2_commit": (_int, [_vp, _u64, _vp, _u64]),
    "sgb_cache2_release": (_int, [_vp, _u64]),
    "sgb_cache2_stats": (_int, [_vp, C.POINTER(_Cache2Stats)]),
    "sgb_decode_paged_q8kv_d128_noalloc": (_int, [_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u64, _vp, _vp, _u32, _u32, _u32,
                                                   _u32, _u32, C.c_float]),
}

_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """Load ``libsgattn.so`` (built in-tree by ``super_gemma_b200/build.py``).  Raises if it is
    missing: there is no other implementation to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NoDevice(f"{LIB_PATH} is missing: run `python -m super_gemma_b200.build` (nvcc, sm_100a)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in ABI.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _check(code: int) -> None:
    if code != SGB_OK:
        msg = lib().sgb_last_error().decode()
        raise _BY_CODE.get(code, GpuError)(msg)


@dataclass
class KernelBlob:
    """Registry metadata (``KernelBlob`` in crates/sg-gpu/src/kernel.rs:18-34, minus the SPIR-V)."""

    name: str
    workgroup: tuple
    bindings: int
    push_bytes: int
    signature: str


def kernels() -> list[KernelBlob]:
    """The compiled-in registry (``KERNELS``)."""
    L = lib()
    out = []
    for i in range(L.sgb_kernel_count()):
        info = _KernelInfo()
        _check(L.sgb_kernel_info_at(i, C.byref(info)))
        out.append(KernelBlob(info.name.decode(), tuple(info.workgroup), info.bindings, info.push_bytes, info.signature.decode()))
    return out


def kernel_blob(name: str) -> Optional[KernelBlob]:
    return next((k for k in kernels() if k.name == name), None)


@dataclass
class StepState:
    """Per-step dynamic state read by the kernels from the step buffer (graph.rs:29-48)."""

    pos: int = 0
    kv_len_sliding: int = 0
    kv_len_global: int = 0
    q0: int = 0

    def write_to(self, buf: "Buffer") -> None:
        _check(lib().sgb_step_write(buf._h, self.pos, self.kv_len_sliding, self.kv_len_global, self.q0))


STEP_WORDS = 4


class Buffer:
    """A device buffer view.  ``read``/``write`` copy through the context's stream (the reference
    maps unified memory instead; buffer.rs:132-162)."""

    def __init__(self, ctx: "GpuContext", handle: int, dtype=np.uint8, keep=None):
        self._ctx, self._h, self.dtype, self._keep = ctx, handle, np.dtype(dtype), keep

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.sgb_buffer_release(h)

    @property
    def nbytes(self) -> int:
        return lib().sgb_buffer_bytes(self._h)

    def __len__(self) -> int:
        return self.nbytes // self.dtype.itemsize

    @property
    def device_ptr(self) -> int:
        return lib().sgb_buffer_device_ptr(self._h) or 0

    def slice(self, start: int, stop: int) -> "Buffer":
        """Element range [start, stop) sharing the allocation (Buffer::slice, buffer.rs:112-124)."""
        out = C.c_void_p()
        isz = self.dtype.itemsize
        _check(lib().sgb_buffer_slice(self._h, start * isz, (stop - start) * isz, C.byref(out)))
        return Buffer(self._ctx, out.value, self.dtype, keep=self)

    def write(self, data, offset_elems: int = 0) -> None:
        a = np.ascontiguousarray(data)
        if a.dtype != self.dtype:
            a = a.view(self.dtype) if a.dtype.itemsize == self.dtype.itemsize else a.astype(self.dtype)
        _check(lib().sgb_buffer_upload(self._h, offset_elems * self.dtype.itemsize, a.ctypes.data, a.nbytes))

    def read(self, count: Optional[int] = None, offset_elems: int = 0) -> np.ndarray:
        n = len(self) - offset_elems if count is None else count
        out = np.empty(n, self.dtype)
        _check(lib().sgb_buffer_download(self._h, offset_elems * self.dtype.itemsize, out.ctypes.data, out.nbytes))
        return out

    def zero(self) -> None:
        _check(lib().sgb_buffer_fill_zero(self._h))


@dataclass
class BufferBinding:
    index: int
    buf: Buffer

    @staticmethod
    def buffer(index: int, buf: Buffer) -> "BufferBinding":
        return BufferBinding(index, buf)


class Kernel:
    def __init__(self, handle: int, blob: KernelBlob):
        self._h, self.blob = handle, blob
        self.name, self.workgroup = blob.name, blob.workgroup

    def groups_for(self, n: int) -> list[int]:
        """Workgroup count covering n invocations on x (kernel.rs:56-58)."""
        return [-(-n // self.workgroup[0]), 1, 1]


class CommandGraph:
    def __init__(self, handle: int):
        self._h = handle

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.sgb_graph_destroy(h)


class GpuTimer:
    def __init__(self, ctx: "GpuContext", n: int):
        out = C.c_void_p()
        _check(lib().sgb_timer_create(ctx._h, n, C.byref(out)))
        self._ctx, self._h, self.n = ctx, out.value, n

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.sgb_timer_destroy(h)

    def stamp(self, index: int) -> None:
        _check(lib().sgb_timer_stamp(self._ctx._h, self._h, index))

    def read_ns(self) -> list[int]:
        arr = (C.c_uint64 * self.n)()
        _check(lib().sgb_timer_read_ns(self._h, arr, self.n))
        return list(arr)


def _push_bytes(push) -> bytes:
    if push is None:
        return b""
    if isinstance(push, (bytes, bytearray)):
        return bytes(push)
    if isinstance(push, (int, np.integer)):
        return struct.pack("<I", int(push))
    if isinstance(push, (float, np.floating)):
        return struct.pack("<f", float(push))
    out = b""
    for v in push:  # a tuple of u32 / f32 fields, in declaration order
        out += struct.pack("<f", float(v)) if isinstance(v, (float, np.floating)) else struct.pack("<I", int(v))
    return out


class GpuContext:
    """One CUDA device and one stream (``GpuContext::new``, context.rs:103).  ``stream`` may be a
    ``cudaStream_t`` value owned by the host program (0 = the legacy default stream)."""

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        out = C.c_void_p()
        if stream is None:
            _check(lib().sgb_ctx_create(device, C.byref(out)))
        else:
            _check(lib().sgb_ctx_create_on_stream(device, C.c_void_p(stream), C.byref(out)))
        self._h = out.value
        self.device = device

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.sgb_ctx_destroy(h)

    def __del__(self):
        # Buffers hold a reference to the context object, so they are released first.
        self.close()

    @property
    def sm_count(self) -> int:
        return lib().sgb_ctx_sm_count(self._h)

    @property
    def stream(self) -> int:
        return lib().sgb_ctx_stream(self._h) or 0

    def decode_splits_hint(self, n_kv_heads: int, kv_len: int) -> int:
        """A split count for the paged decode / verify kernels that fills every SM evenly."""
        return lib().sgb_decode_paged_splits_hint(self._h, n_kv_heads, kv_len)

    @property
    def launch_count(self) -> int:
        return lib().sgb_launch_count(self._h)

    # ---- buffers ----------------------------------------------------------------------------------
    def new_buffer(self, length: int, dtype=np.uint8) -> Buffer:
        """Zero-initialised buffer of `length` elements (new_buffer, buffer.rs:257-275)."""
        out = C.c_void_p()
        _check(lib().sgb_buffer_create(self._h, length * np.dtype(dtype).itemsize, C.byref(out)))
        return Buffer(self, out.value, dtype)

    def buffer_from_iter(self, data) -> Buffer:
        """Buffer initialised from host data (buffer_from_iter, buffer.rs:278)."""
        a = np.ascontiguousarray(data)
        if a.dtype == np.float16:
            a = a.view(np.uint16)
        b = self.new_buffer(a.size, a.dtype)
        b.write(a.reshape(-1))
        return b

    def adopt(self, device_ptr: int, nbytes: int, dtype=np.uint8, keep=None) -> Buffer:
        """Bind device memory owned by someone else (e.g. a torch tensor's storage) without copying."""
        out = C.c_void_p()
        _check(lib().sgb_buffer_adopt(self._h, C.c_void_p(device_ptr), nbytes, C.byref(out)))
        return Buffer(self, out.value, dtype, keep=keep)

    def new_step_buffer(self) -> Buffer:
        return self.new_buffer(STEP_WORDS, np.uint32)

    # ---- kernels ----------------------------------------------------------------------------------
    def load_kernel(self, name: str) -> Kernel:
        out = C.c_void_p()
        _check(lib().sgb_kernel_get(self._h, name.encode(), C.byref(out)))
        info = _KernelInfo()
        _check(lib().sgb_kernel_describe(out.value, C.byref(info)))
        return Kernel(out.value, KernelBlob(info.name.decode(), tuple(info.workgroup), info.bindings, info.push_bytes,
                                            info.signature.decode()))

    def _dispatch(self, fn, kernel: Kernel, bindings: Sequence[BufferBinding], push, groups: Sequence[int]) -> None:
        arr = (_Binding * len(bindings))(*[_Binding(b.index, b.buf._h) for b in bindings])
        pb = _push_bytes(push)
        g = (C.c_uint32 * 3)(*(list(groups) + [1, 1, 1])[:3])
        pbuf = C.create_string_buffer(pb, len(pb)) if pb else None
        _check(fn(self._h, kernel._h, arr, len(bindings), C.cast(pbuf, C.c_void_p) if pbuf else None, len(pb), g))

    def dispatch(self, kernel: Kernel, bindings: Sequence[BufferBinding], push, groups: Sequence[int]) -> None:
        """Enqueue (or, while recording, capture) one kernel (GraphRecorder::dispatch, graph.rs:203)."""
        self._dispatch(lib().sgb_dispatch, kernel, bindings, push, groups)

    def dispatch_blocking(self, kernel: Kernel, bindings: Sequence[BufferBinding], push, groups: Sequence[int]) -> None:
        """One-shot dispatch and wait (exec.rs:12-23)."""
        self._dispatch(lib().sgb_dispatch_blocking, kernel, bindings, push, groups)

    def sync(self, timeout_ms: int = 0) -> None:
        _check(lib().sgb_sync(self._h, timeout_ms))

    # ---- record / replay ----------------------------------------------------------------------------
    def record_graph(self, record: Callable[["GpuContext"], None]) -> CommandGraph:
        """Record once (record_graph, graph.rs:523-528): dispatches made by `record` are captured."""
        _check(lib().sgb_graph_begin(self._h))
        try:
            record(self)
        except BaseException:
            out = C.c_void_p()
            if lib().sgb_graph_end(self._h, C.byref(out)) == SGB_OK:
                lib().sgb_graph_destroy(out.value)
            raise
        out = C.c_void_p()
        _check(lib().sgb_graph_end(self._h, C.byref(out)))
        return CommandGraph(out.value)

    def submit(self, graph: CommandGraph) -> None:
        _check(lib().sgb_graph_launch(self._h, graph._h))

    def submit_blocking(self, graph: CommandGraph, timeout_ms: int = 0) -> None:
        """Replay and wait (submit_blocking, graph.rs:640-642), with a finite wait."""
        self.submit(graph)
        self.sync(timeout_ms)

    def new_timer(self, n: int) -> GpuTimer:
        return GpuTimer(self, n)
