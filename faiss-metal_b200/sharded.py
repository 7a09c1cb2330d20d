"""Row-sharded flat index over the GPUs of one box: Python mirrors of
faiss_b200::B200ShardedIndexFlat (the reference is single-device,
src/StandardMetalResources.mm:17-23, and has no counterpart).

``MultiGpuIndexFlat``   one process drives several GPUs: add() places rows block-cyclically,
                        search() copies the queries up in slices, all-gathers them, searches
                        every shard, all-gathers the candidates and merges.
``ShardedIndexFlat``    one process per GPU (what torchrun launches): each rank holds rows
                        [lo, hi) (``shard_range``) in its own B200IndexFlat with
                        ``label_base = lo``; search is a collective call.

In both the exchange is one ncclAllGather issued by the C++ library on the resources' own stream
between the shard search and the k-way merge kernel; torch.distributed is used for one thing
only, to hand rank 0's NCCL id to the other ranks.

With a CPU process group (``backend="gloo"``) and a ``merge_fn`` the exchange of
``ShardedIndexFlat.search`` runs on CPU tensors through torch.distributed, so the shard / offset /
merge logic can be tested without GPUs.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import abi
from .index import _check, _is_cuda, _ptr


def shard_range(nb: int, rank: int, world: int):
    """Contiguous equal split: rank r owns rows [lo, hi).  Global label = lo + local row."""
    per = (nb + world - 1) // world
    lo = min(nb, rank * per)
    hi = min(nb, lo + per)
    return lo, hi


def pack_candidates(dist, labels):
    """Pack (float32 distance, int64 label) lists [nq, k] into one int32 [nq, k, 3] buffer so
    a single all-gather moves both (CPU process groups)."""
    import torch
    nq, k = dist.shape
    buf = torch.empty((nq, k, 3), dtype=torch.int32, device=dist.device)
    buf[..., 0] = dist.view(torch.int32)
    buf[..., 1:] = labels.view(torch.int32).reshape(nq, k, 2)
    return buf


def unpack_candidates(buf):
    """Inverse of pack_candidates for a gathered buffer [P, nq, k, 3]."""
    import torch
    dist = buf[..., 0].contiguous().view(torch.float32)
    labels = buf[..., 1:].contiguous().view(torch.int64).reshape(buf.shape[:-1])
    return dist, labels


class _ShardedHandle:
    """Calls shared by the two mirrors (a B200FSharded handle)."""

    _h = None
    d = 0
    metric_type = abi.METRIC_L2
    resources = None

    def _search(self, x, k, distances, labels, want_result=True):
        if len(x.shape) != 2:
            raise ValueError("search: expected a 2-d array [n, %d]" % self.d)
        n = int(x.shape[0])
        _check(x, "search: x", "float32", (n, self.d))
        if want_result and (distances is None or labels is None):
            if isinstance(x, np.ndarray):
                distances = np.empty((n, k), dtype=np.float32)
                labels = np.empty((n, k), dtype=np.int64)
            else:
                import torch
                distances = torch.empty((n, k), dtype=torch.float32, device=x.device)
                labels = torch.empty((n, k), dtype=torch.int64, device=x.device)
        if want_result and int(k) >= 1:
            _check(distances, "search: distances", "float32", (n, int(k)))
            _check(labels, "search: labels", "int64", (n, int(k)))
        self.resources._order_after_torch(x, distances, labels)
        abi.check(abi.lib().b200f_sharded_search(self._h, n, _ptr(x) if n else None, int(k),
                                                 _ptr(distances) if want_result else None,
                                                 _ptr(labels) if want_result else None), "sharded search")
        return distances, labels

    def search_enqueue(self, x, k: int, distances=None, labels=None):
        """Device tensors only, one batch; queued on the resources' stream(s), no host wait."""
        n = int(x.shape[0])
        _check(x, "search_enqueue: x", "float32", (n, self.d))
        if distances is not None:
            _check(distances, "search_enqueue: distances", "float32", (n, int(k)))
            _check(labels, "search_enqueue: labels", "int64", (n, int(k)))
        self.resources._order_after_torch(x, distances, labels)
        abi.check(abi.lib().b200f_sharded_search_enqueue(self._h, n, _ptr(x) if n else None, int(k),
                                                         _ptr(distances), _ptr(labels)), "sharded search_enqueue")

    def synchronize(self):
        abi.check(abi.lib().b200f_sharded_synchronize(self._h), "sharded synchronize")

    def set_path(self, path: int):
        abi.check(abi.lib().b200f_sharded_set_path(self._h, int(path)), "sharded set_path")

    def set_use_graphs(self, on: bool):
        abi.check(abi.lib().b200f_sharded_set_use_graphs(self._h, 1 if on else 0), "sharded set_use_graphs")

    def trace(self, on: bool):
        """Start (and clear) or stop the host-side trace of search() calls."""
        abi.check(abi.lib().b200f_sharded_trace(self._h, 1 if on else 0), "sharded trace")

    def read_trace(self):
        """(enqueue_us, wait_us) float32 arrays, one entry per traced search() call."""
        n = abi.lib().b200f_sharded_trace_read(self._h, None, None, 0)
        enq = np.empty(max(n, 0), dtype=np.float32)
        wait = np.empty(max(n, 0), dtype=np.float32)
        if n > 0:
            abi.lib().b200f_sharded_trace_read(self._h, _ptr(enq), _ptr(wait), n)
        return enq, wait

    def close(self):
        if getattr(self, "_h", None):
            abi.lib().b200f_sharded_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MultiGpuIndexFlat(_ShardedHandle):
    """One process, several GPUs (or several shards on one GPU: a single-GPU rehearsal of the
    same code).  ``resources``: one StandardB200Resources per shard."""

    def __init__(self, resources, d: int, metric: int = abi.METRIC_L2, storage: int = abi.STORAGE_F32,
                 block_rows: int = 65536):
        arr = (ctypes.c_void_p * len(resources))(*[r._h for r in resources])
        h = ctypes.c_void_p()
        abi.check(abi.lib().b200f_sharded_create(arr, len(resources), d, metric, storage, int(block_rows),
                                                 ctypes.byref(h)), "sharded create")
        self._h = h
        self._res_list = list(resources)
        self.resources = resources[0]
        self.d = d
        self.metric_type = metric
        self.storage = storage
        self.block_rows = int(block_rows)

    @property
    def ntotal(self) -> int:
        return abi.lib().b200f_sharded_ntotal(self._h)

    @property
    def num_shards(self) -> int:
        return abi.lib().b200f_sharded_num_shards(self._h)

    def add(self, x):
        if len(x.shape) != 2:
            raise ValueError("add: expected a 2-d array [n, %d]" % self.d)
        n = int(x.shape[0])
        _check(x, "add: x", "float32", (n, self.d))
        if _is_cuda(x):
            raise ValueError("add: the several-GPU index takes host rows (each shard uploads its own blocks)")
        abi.check(abi.lib().b200f_sharded_add(self._h, n, _ptr(x) if n else None), "sharded add")

    def search(self, x, k: int, distances=None, labels=None):
        return self._search(x, k, distances, labels)

    def reset(self):
        abi.check(abi.lib().b200f_sharded_reset(self._h), "sharded reset")

    def reconstruct(self, key: int) -> np.ndarray:
        out = np.empty(self.d, dtype=np.float32)
        abi.check(abi.lib().b200f_sharded_reconstruct(self._h, int(key), _ptr(out)), "sharded reconstruct")
        return out


class ShardedIndexFlat(_ShardedHandle):
    """One process per GPU: database rows sharded over the ranks of a process group.

    GPU ranks: ``local_index`` is this rank's B200IndexFlat.  world > 1 needs an initialised
    torch.distributed process group (any backend), used once to broadcast rank 0's NCCL id.
    CPU ranks (tests): ``merge_fn`` given, ``local_index`` any object with ``search`` and
    ``set_label_base``."""

    def __init__(self, local_index, rank: int, world: int, group=None, merge_fn=None):
        self.local = local_index
        self.rank = rank
        self.world = world
        self.group = group
        self.merge_fn = merge_fn
        self.metric_type = local_index.metric_type
        self._bufs = {}
        self._h = None
        if merge_fn is not None:
            return
        self.d = local_index.d
        self.resources = local_index.resources
        ident = ctypes.create_string_buffer(128)
        if world > 1:
            import torch.distributed as dist
            box = [None]
            if rank == 0:
                abi.check(abi.lib().b200f_comm_id_create(ident), "comm id")
                box[0] = ident.raw
            dist.broadcast_object_list(box, src=0, group=group)
            ident = ctypes.create_string_buffer(box[0], 128)
        h = ctypes.c_void_p()
        abi.check(abi.lib().b200f_sharded_create_rank(local_index._h, rank, world, ident, ctypes.byref(h)),
                  "sharded create_rank")
        self._h = h

    def set_shard(self, lo: int):
        self.local.set_label_base(lo)

    def search_device(self, x, k: int, sync: bool = True, want_result: bool = True):
        """x: fp32 CUDA tensor [nq, d] on this rank's GPU, identical on every rank, one batch.
        Shard search, one all-gather of [distances | labels] and the k-way merge are queued back
        to back on the resources' stream.  Returns this rank's merged (distances, labels) device
        tensors, reused by the next call with the same (nq, k); (None, None) with
        want_result=False (the rank takes part in the exchange, merges nothing)."""
        import torch
        nq = int(x.shape[0])
        out = (None, None)
        if want_result:
            out = self._bufs.get((nq, k))
            if out is None:
                out = (torch.empty((nq, k), dtype=torch.float32, device=x.device),
                       torch.empty((nq, k), dtype=torch.int64, device=x.device))
                self._bufs[(nq, k)] = out
        self.search_enqueue(x, k, out[0], out[1])
        if sync:
            self.synchronize()
        return out

    def search(self, x, k: int, distances=None, labels=None, want_result: bool = True):
        """x: fp32 queries [nq, d], identical on every rank: numpy (host) or a CUDA tensor on this
        rank's GPU.  Returns (distances, labels) in the memory space of x; with want_result=False
        the rank only takes part (returns (None, None)).  With a CPU process group and a
        merge_fn: x numpy / CPU tensor, the exchange runs through torch.distributed."""
        if self.merge_fn is None:
            return self._search(x, k, distances, labels, want_result)
        import torch
        import torch.distributed as dist
        d_loc, l_loc = self.local.search(x, k)
        if self.world == 1:
            return d_loc, l_loc
        if isinstance(d_loc, np.ndarray):
            d_loc = torch.from_numpy(d_loc)
            l_loc = torch.from_numpy(l_loc)
        packed = pack_candidates(d_loc, l_loc)
        gathered = torch.empty((self.world,) + tuple(packed.shape), dtype=packed.dtype, device=packed.device)
        dist.all_gather([gathered[r] for r in range(self.world)], packed, group=self.group)
        d_all, l_all = unpack_candidates(gathered)
        return self.merge_fn(self.metric_type, d_all.numpy(), l_all.numpy())
