"""Python mirror of the plugin classes (faiss_metal::MetalIndexFlat and friends,
include/faiss-metal/MetalIndexFlat.h:13-120) over the handle-based C-ABI.

Arrays may be numpy arrays (host) or torch CUDA tensors (device); the C-ABI
detects which from the pointer.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import abi


def device_caps(device: int = -1) -> dict:
    c = abi.Caps()
    abi.check_op(abi.lib().b200f_device_caps(device, ctypes.byref(c)), "device_caps")
    out = {name: getattr(c, name) for name, _ in abi.Caps._fields_}
    out["name"] = c.name.decode()
    return out


def _ptr(a):
    """Raw address of a numpy array or torch tensor (contiguous)."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        if not a.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        return ctypes.c_void_p(a.ctypes.data)
    if hasattr(a, "data_ptr"):
        if not a.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return ctypes.c_void_p(a.data_ptr())
    raise TypeError("expected numpy array or torch tensor")


def _dtype_name(a) -> str:
    return str(a.dtype).replace("torch.", "")


def _check(a, what: str, dtype: str, shape) -> None:
    """The C side reads / writes rows * cols * itemsize bytes behind the pointer: a wrong dtype
    or shape would be an out-of-bounds access there, so it is refused here."""
    if not (isinstance(a, np.ndarray) or hasattr(a, "data_ptr")):
        raise TypeError("%s: expected numpy array or torch tensor" % what)
    if _dtype_name(a) != dtype:
        raise ValueError("%s: expected dtype %s, got %s" % (what, dtype, _dtype_name(a)))
    if tuple(int(v) for v in a.shape) != tuple(shape):
        raise ValueError("%s: expected shape %s, got %s" % (what, tuple(shape), tuple(a.shape)))


def _is_cuda(a) -> bool:
    return hasattr(a, "is_cuda") and bool(a.is_cuda)


class StandardB200Resources:
    """StandardMetalResources (include/faiss-metal/StandardMetalResources.h:9-32)."""

    def __init__(self, device: int = -1):
        h = ctypes.c_void_p()
        abi.check(abi.lib().b200f_resources_create(device, ctypes.byref(h)), "resources")
        self._h = h

    @property
    def device(self) -> int:
        return abi.lib().b200f_resources_device(self._h)

    @property
    def stream(self) -> int:
        return abi.lib().b200f_resources_stream(self._h) or 0

    @property
    def scratch_bytes(self) -> int:
        return abi.lib().b200f_resources_scratch_bytes(self._h)

    def wait_stream(self, producer_stream: int = 0):
        """Orders the resources' stream after everything queued so far on `producer_stream`
        (a cudaStream_t as an integer; 0 = the legacy default stream)."""
        abi.check(abi.lib().b200f_resources_wait_stream(self._h, ctypes.c_void_p(producer_stream)), "wait_stream")

    def _order_after_torch(self, *arrays):
        """The library's stream does not synchronise with torch's streams: a CUDA tensor that
        torch has just produced (or will overwrite) must be ordered explicitly.  Makes the
        resources' stream wait for torch's current stream when any argument is a CUDA tensor."""
        if any(_is_cuda(a) for a in arrays if a is not None):
            import torch
            cur = torch.cuda.current_stream().cuda_stream
            if cur != self.stream:
                self.wait_stream(cur)

    def close(self):
        if getattr(self, "_h", None):
            abi.lib().b200f_resources_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class SearchToken:
    """MetalSearchToken (include/faiss-metal/MetalIndexFlat.h:15-36)."""

    def __init__(self, handle, keepalive):
        self._h = handle
        self._keep = keepalive

    def wait(self):
        if self._h is None:
            raise abi.B200Error(abi.lib().b200f_token_wait(None), "token already consumed")
        abi.check(abi.lib().b200f_token_wait(self._h), "token wait")

    def is_ready(self) -> bool:
        r = ctypes.c_int(0)
        abi.check(abi.lib().b200f_token_is_ready(self._h, ctypes.byref(r)), "token is_ready")
        return bool(r.value)

    def close(self):
        if self._h is not None:
            abi.lib().b200f_token_destroy(self._h)  # waits if never waited
            self._h = None
            self._keep = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class B200IndexFlat:
    """MetalIndexFlat (include/faiss-metal/MetalIndexFlat.h:47-111)."""

    def __init__(self, resources: StandardB200Resources, d: int, metric: int = abi.METRIC_L2,
                 storage: int = abi.STORAGE_F32):
        h = ctypes.c_void_p()
        abi.check(abi.lib().b200f_index_create(resources._h, d, metric, storage, ctypes.byref(h)), "index")
        self._h = h
        self.resources = resources
        self.d = d
        self.metric_type = metric
        self.storage = storage
        self.is_trained = True

    # -- faiss::Index surface ---------------------------------------------------------
    @property
    def ntotal(self) -> int:
        return abi.lib().b200f_index_ntotal(self._h)

    def add(self, x):
        if len(x.shape) != 2:
            raise ValueError("add: expected a 2-d array [n, %d]" % self.d)
        n = int(x.shape[0])
        _check(x, "add: x", "float32", (n, self.d))
        self.resources._order_after_torch(x)
        abi.check(abi.lib().b200f_index_add(self._h, n, _ptr(x) if n else None), "add")

    def reserve(self, n: int):
        abi.check(abi.lib().b200f_index_reserve(self._h, int(n)), "reserve")

    def search(self, x, k: int, distances=None, labels=None):
        """Returns (distances float32 [n,k], labels int64 [n,k]) in the memory space of x
        unless output arrays are given."""
        n = self._check_queries(x, "search")
        if distances is None or labels is None:
            if isinstance(x, np.ndarray):
                distances = np.empty((n, k), dtype=np.float32)
                labels = np.empty((n, k), dtype=np.int64)
            else:
                import torch
                distances = torch.empty((n, k), dtype=torch.float32, device=x.device)
                labels = torch.empty((n, k), dtype=torch.int64, device=x.device)
        self._check_outputs(n, k, distances, labels, "search")
        self.resources._order_after_torch(x, distances, labels)
        abi.check(abi.lib().b200f_index_search(self._h, n, _ptr(x) if n else None, int(k),
                                                _ptr(distances), _ptr(labels)), "search")
        return distances, labels

    def _check_queries(self, x, what: str) -> int:
        if len(x.shape) != 2:
            raise ValueError("%s: expected a 2-d array [n, %d]" % (what, self.d))
        n = int(x.shape[0])
        _check(x, what + ": x", "float32", (n, self.d))
        return n

    def _check_outputs(self, n: int, k: int, distances, labels, what: str) -> None:
        if int(k) >= 1:   # k < 1 is reported by the library with its own status code
            _check(distances, what + ": distances", "float32", (n, int(k)))
            _check(labels, what + ": labels", "int64", (n, int(k)))

    def search_enqueue(self, x, k: int, distances, labels):
        """Device tensors only; queues the search on the resources' stream without waiting.
        The inputs are ordered after torch's current stream; the OUTPUTS are complete only on
        the resources' stream (call synchronize(), or make your stream wait on that one)."""
        n = self._check_queries(x, "search_enqueue")
        self._check_outputs(n, k, distances, labels, "search_enqueue")
        self.resources._order_after_torch(x, distances, labels)
        abi.check(abi.lib().b200f_index_search_enqueue(self._h, n, _ptr(x) if n else None, int(k),
                                                        _ptr(distances), _ptr(labels)), "search_enqueue")

    def synchronize(self):
        abi.check(abi.lib().b200f_index_synchronize(self._h), "synchronize")

    def search_async(self, x, k: int, distances, labels) -> SearchToken:
        n = self._check_queries(x, "search_async")
        self._check_outputs(n, k, distances, labels, "search_async")
        self.resources._order_after_torch(x, distances, labels)
        t = ctypes.c_void_p()
        abi.check(abi.lib().b200f_index_search_async(self._h, n, _ptr(x) if n else None, int(k),
                                                      _ptr(distances), _ptr(labels), ctypes.byref(t)),
                  "search_async")
        return SearchToken(t, (distances, labels))

    def reset(self):
        abi.check(abi.lib().b200f_index_reset(self._h), "reset")

    def reconstruct(self, key: int) -> np.ndarray:
        out = np.empty(self.d, dtype=np.float32)
        abi.check(abi.lib().b200f_index_reconstruct(self._h, int(key), _ptr(out)), "reconstruct")
        return out

    def reconstruct_n(self, first: int, n: int, out=None):
        if out is None:
            out = np.empty((n, self.d), dtype=np.float32)
        _check(out, "reconstruct_n: out", "float32", (int(n), self.d))
        self.resources._order_after_torch(out)
        abi.check(abi.lib().b200f_index_reconstruct_n(self._h, int(first), int(n), _ptr(out)), "reconstruct_n")
        return out

    # -- extras ---------------------------------------------------------------------------
    def set_path(self, path: int):
        abi.check(abi.lib().b200f_index_set_path(self._h, int(path)), "set_path")

    def set_growth_mode(self, mode: int):
        """0: grow in place (default where supported), 1: allocate-copy-free; empty index only."""
        abi.check(abi.lib().b200f_index_set_growth_mode(self._h, int(mode)), "set_growth_mode")

    def set_fp32_planes(self, fmt: int):
        """FP32 storage: abi.PLANES_BF16X3 or abi.PLANES_FP16X2 (default); empty index only."""
        abi.check(abi.lib().b200f_index_set_fp32_planes(self._h, int(fmt)), "set_fp32_planes")

    @property
    def fp32_planes(self) -> int:
        return abi.lib().b200f_index_fp32_planes(self._h)

    def set_use_graphs(self, on: bool):
        abi.check(abi.lib().b200f_index_set_use_graphs(self._h, 1 if on else 0), "set_use_graphs")

    def set_label_base(self, base: int):
        abi.check(abi.lib().b200f_index_set_label_base(self._h, int(base)), "set_label_base")

    def device_rows(self) -> int:
        """Device address of the stored rows (0 for an empty index)."""
        return int(abi.lib().b200f_index_device_rows(self._h) or 0)

    @property
    def last_device_status(self) -> int:
        return abi.lib().b200f_index_last_device_status(self._h)

    def close(self):
        if getattr(self, "_h", None):
            abi.lib().b200f_index_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
