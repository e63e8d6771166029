"""Host-side handles over the C ABI: device, buffer, stream, event.

These mirror what fractal.py obtains from its runtime -- ``ti.init`` (fractal.py:5) becomes
:class:`Device`, ``ti.field`` (fractal.py:8) becomes :class:`Buffer` -- with nothing between them
and ``libvrhi.so`` except ctypes.  numpy arrays are used for host memory; torch tensors can be
adopted without a copy through :meth:`Device.wrap_tensor`.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib as L
from ._lib import check, lib


class Device:
    """One opened GPU (``vrhi_device``).  Requires an sm_100 part: the library carries no other code."""

    def __init__(self, ordinal: int = 0):
        h = C.c_void_p()
        check(lib().vrhi_device_create(int(ordinal), C.byref(h)))
        self._h = h
        self.ordinal = int(ordinal)
        p = L.DeviceProps()
        p.size = C.sizeof(L.DeviceProps)
        check(lib().vrhi_device_props_get(self._h, C.byref(p)))
        self.props = p
        self.name = p.name.decode()
        self.sm_count = int(p.sm_count)
        self.sm_clock_khz = int(p.sm_clock_khz)

    @staticmethod
    def count() -> int:
        n = C.c_int()
        check(lib().vrhi_device_count(C.byref(n)))
        return n.value

    def close(self) -> None:
        if self._h:
            lib().vrhi_device_destroy(self._h)
            self._h = None

    def synchronize(self) -> None:
        check(lib().vrhi_device_synchronize(self._h))

    def set_alloc_limit(self, nbytes: int) -> None:
        check(lib().vrhi_device_set_alloc_limit(self._h, int(nbytes)))

    def allocated(self) -> int:
        v = C.c_uint64()
        check(lib().vrhi_device_allocated(self._h, C.byref(v)))
        return v.value

    # -- buffers -------------------------------------------------------------------------------
    def buffer(self, nbytes: int, arg_class: int = L.STORAGE_BUFFER) -> "Buffer":
        h = C.c_void_p()
        check(lib().vrhi_buffer_create(self._h, int(nbytes), int(arg_class), C.byref(h)))
        return Buffer(self, h, int(nbytes), arg_class)

    def from_numpy(self, array: np.ndarray, arg_class: int = L.INPUT, stream: Optional["Stream"] = None) -> "Buffer":
        a = np.ascontiguousarray(array)
        b = self.buffer(max(a.nbytes, 16), arg_class)
        b.dtype, b.shape = a.dtype, a.shape
        if a.nbytes:
            b.upload(a, stream=stream)
        return b

    def empty(self, shape, dtype=np.float32, arg_class: int = L.OUTPUT) -> "Buffer":
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        b = self.buffer(max(n, 16), arg_class)
        b.dtype, b.shape = np.dtype(dtype), shape
        return b

    def wrap_pointer(self, ptr: int, nbytes: int, arg_class: int = L.STORAGE_BUFFER) -> "Buffer":
        h = C.c_void_p()
        check(lib().vrhi_buffer_wrap(self._h, C.c_void_p(int(ptr)), int(nbytes), int(arg_class), C.byref(h)))
        return Buffer(self, h, int(nbytes), arg_class)

    def wrap_tensor(self, tensor, arg_class: int = L.STORAGE_BUFFER) -> "Buffer":
        """Adopt a contiguous CUDA torch tensor without copying; the tensor must outlive the buffer."""
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("wrap_tensor needs a contiguous CUDA tensor")
        if tensor.device.index not in (None, self.ordinal):
            raise ValueError("tensor lives on another device")
        b = self.wrap_pointer(tensor.data_ptr(), tensor.numel() * tensor.element_size(), arg_class)
        b._keepalive = tensor
        b.shape = tuple(tensor.shape)
        return b

    def open_ipc(self, handle: bytes, nbytes: int, arg_class: int = L.STORAGE_BUFFER) -> "Buffer":
        """Map a buffer that another process of this box exported with :meth:`Buffer.ipc_handle`."""
        h = C.c_void_p()
        raw = C.create_string_buffer(bytes(handle), 64)
        check(lib().vrhi_buffer_ipc_open(self._h, raw, int(nbytes), int(arg_class), C.byref(h)))
        return Buffer(self, h, int(nbytes), arg_class)

    # -- streams / events ----------------------------------------------------------------------
    def stream(self) -> "Stream":
        h = C.c_void_p()
        check(lib().vrhi_stream_create(self._h, C.byref(h)))
        return Stream(self, h)

    def wrap_stream(self, cuda_stream: int) -> "Stream":
        """Adopt an existing CUDA stream handle, e.g. ``torch.cuda.current_stream().cuda_stream``."""
        h = C.c_void_p()
        check(lib().vrhi_stream_wrap(self._h, C.c_void_p(int(cuda_stream)), C.byref(h)))
        s = Stream(self, h)
        s.cuda_stream = int(cuda_stream)
        return s

    def event(self) -> "Event":
        h = C.c_void_p()
        check(lib().vrhi_event_create(self._h, C.byref(h)))
        return Event(self, h)


class Buffer:
    """Device storage (``vrhi_buffer``) with an argument class from the vernon.semantic vocabulary."""

    def __init__(self, dev: Device, handle, nbytes: int, arg_class: int):
        self.dev, self._h, self.nbytes, self.arg_class = dev, handle, nbytes, arg_class
        self.dtype, self.shape = np.dtype(np.uint8), (nbytes,)
        self._keepalive = None

    def close(self) -> None:
        if self._h:
            check(lib().vrhi_buffer_destroy(self._h))
            self._h = None

    @property
    def ptr(self) -> int:
        p = C.c_void_p()
        check(lib().vrhi_buffer_device_ptr(self._h, C.byref(p)))
        return int(p.value)

    def upload(self, array: np.ndarray, offset: int = 0, stream: Optional["Stream"] = None) -> None:
        a = np.ascontiguousarray(array)
        check(lib().vrhi_buffer_upload(self._h, int(offset), a.ctypes.data_as(C.c_void_p), a.nbytes,
                                       stream._h if stream else None))

    def download(self, out: Optional[np.ndarray] = None, offset: int = 0, stream: Optional["Stream"] = None,
                 dtype=None, shape=None) -> np.ndarray:
        if out is None:
            out = np.empty(shape if shape is not None else self.shape, dtype=dtype if dtype is not None else self.dtype)
        check(lib().vrhi_buffer_download(self._h, int(offset), out.ctypes.data_as(C.c_void_p), out.nbytes,
                                         stream._h if stream else None))
        return out

    def fill(self, byte: int, offset: int = 0, nbytes: Optional[int] = None, stream: Optional["Stream"] = None) -> None:
        check(lib().vrhi_buffer_fill_u8(self._h, int(offset), int(byte), int(self.nbytes - offset if nbytes is None else nbytes),
                                        stream._h if stream else None))

    def ipc_handle(self) -> bytes:
        """64-byte handle another process of this box can open with :meth:`Device.open_ipc`."""
        raw = C.create_string_buffer(64)
        check(lib().vrhi_buffer_ipc_export(self._h, raw))
        return raw.raw

    def copy_2d_to(self, dst: "Buffer", dst_offset: int, dst_pitch: int, src_offset: int, src_pitch: int, width_bytes: int,
                   rows: int, stream: Optional["Stream"] = None) -> None:
        """Copy `rows` runs of `width_bytes` from this buffer into `dst` (possibly on a peer GPU) with the copy engines."""
        check(lib().vrhi_buffer_copy_2d(dst._h, int(dst_offset), int(dst_pitch), self._h, int(src_offset), int(src_pitch),
                                        int(width_bytes), int(rows), stream._h if stream else None))

    def arg(self, arg_class: Optional[int] = None, offset: int = 0, nbytes: int = 0) -> L.Arg:
        a = L.Arg()
        a.buffer = self._h
        a.offset, a.bytes = int(offset), int(nbytes)
        a.arg_class = self.arg_class if arg_class is None else arg_class
        return a

    def as_tensor(self, dtype=None, shape=None):
        """A torch view of the same device memory (for torch.distributed collectives)."""
        import torch

        np_dtype = np.dtype(dtype if dtype is not None else self.dtype)
        tdt = {np.dtype(np.float32): torch.float32, np.dtype(np.uint32): torch.int32, np.dtype(np.int32): torch.int32,
               np.dtype(np.uint16): torch.int16, np.dtype(np.uint8): torch.uint8}[np_dtype]
        shp = tuple(shape if shape is not None else self.shape)

        class _View:
            pass

        v = _View()
        v.__cuda_array_interface__ = {"shape": shp, "typestr": np.dtype(
            {torch.float32: "<f4", torch.int32: "<i4", torch.int16: "<i2", torch.uint8: "|u1"}[tdt]).str,
            "data": (self.ptr, False), "version": 2}
        t = torch.as_tensor(v, device=f"cuda:{self.dev.ordinal}")
        t._vrhi_owner = self
        return t


class Stream:
    """An ordered queue of kernels and copies (``vrhi_stream``)."""

    def __init__(self, dev: Device, handle):
        self.dev, self._h = dev, handle
        self.cuda_stream = None   # the adopted CUDA stream handle, where this stream wraps one

    def close(self) -> None:
        if self._h:
            check(lib().vrhi_stream_destroy(self._h))
            self._h = None

    def synchronize(self) -> None:
        check(lib().vrhi_stream_synchronize(self._h))

    def check(self) -> None:
        """Synchronise and raise if a kernel recorded a device-side status (e.g. a bounded wait gave up)."""
        check(lib().vrhi_stream_check(self._h))

    def launch_count(self) -> int:
        v = C.c_uint64()
        check(lib().vrhi_stream_launch_count(self._h, C.byref(v)))
        return v.value

    def wait(self, event: "Event") -> None:
        check(lib().vrhi_stream_wait_event(self._h, event._h))

    def record(self, into: Optional["Sequence"] = None) -> "_Recording":
        """``with stream.record() as seq:`` records the launches issued on this stream inside the
        block (``vrhi_sequence_begin/end``) instead of running them; ``seq.launch()`` replays them as
        one submission.  Passing an existing sequence re-targets it in place."""
        return _Recording(self, into)

    def fork_recording(self, side: "Stream") -> None:
        """While this stream records: draw ``side`` into the recording (``vrhi_sequence_fork``).  Launches on
        ``side`` are recorded from here on and may run beside this stream's; they rejoin when the recording ends."""
        check(lib().vrhi_sequence_fork(self._h, side._h))


class Sequence:
    """A recorded run of launches (``vrhi_sequence``), replayed with one submission."""

    def __init__(self, stream: Stream):
        self.stream = stream
        self._h = C.c_void_p()

    def launch(self, stream: Optional[Stream] = None) -> None:
        check(lib().vrhi_sequence_launch(self._h, (stream or self.stream)._h))

    def stats(self) -> dict:
        k, u, r = C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(lib().vrhi_sequence_stats(self._h, C.byref(k), C.byref(u), C.byref(r)))
        return {"kernels": k.value, "retargets": u.value, "rebuilds": r.value}

    def close(self) -> None:
        if self._h:
            lib().vrhi_sequence_destroy(self._h)
            self._h = C.c_void_p()


class _Recording:
    def __init__(self, stream: Stream, into: Optional[Sequence]):
        self.stream, self.seq = stream, into or Sequence(stream)

    def __enter__(self) -> Sequence:
        check(lib().vrhi_sequence_begin(self.stream._h))
        return self.seq

    def __exit__(self, exc_type, exc, tb) -> bool:
        rc = lib().vrhi_sequence_end(self.stream._h, C.byref(self.seq._h))
        if exc_type is None:
            check(rc)
        return False


class Event:
    def __init__(self, dev: Device, handle):
        self.dev, self._h = dev, handle

    def close(self) -> None:
        if self._h:
            lib().vrhi_event_destroy(self._h)
            self._h = None

    def record(self, stream: Optional[Stream] = None) -> None:
        check(lib().vrhi_event_record(self._h, stream._h if stream else None))

    def synchronize(self) -> None:
        check(lib().vrhi_event_synchronize(self._h))

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float()
        check(lib().vrhi_event_elapsed_ms(self._h, stop._h, C.byref(ms)))
        return float(ms.value)


class PinnedArray:
    """Page-locked host memory (``vrhi_host_alloc``) viewed as a numpy array in ``.array``."""

    def __init__(self, shape, dtype=np.float32):
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        count = int(np.prod(shape))
        n = max(count * np.dtype(dtype).itemsize, 16)
        p = C.c_void_p()
        check(lib().vrhi_host_alloc(n, C.byref(p)))
        self._ptr = p.value
        self._raw = (C.c_uint8 * n).from_address(self._ptr)
        self.array = np.frombuffer(self._raw, dtype=dtype, count=count).reshape(shape)

    def close(self) -> None:
        if self._ptr:
            self.array = None
            self._raw = None
            check(lib().vrhi_host_free(C.c_void_p(self._ptr)))
            self._ptr = None
