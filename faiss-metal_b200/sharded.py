"""Row-sharded flat index over the GPUs of one box: one process per GPU.

Each rank holds rows [lo, hi) of the database (``shard_range``) in its own
B200IndexFlat with ``label_base = lo``; a search runs the shard-local search on
every rank, exchanges the per-rank (distance, label) candidate lists with one
all-gather over NCCL (NVLink / NVSwitch) and merges the ``world_size`` sorted
lists per query with the k-way merge kernel (b200f_merge_lists).  The reference
is single-device (src/StandardMetalResources.mm:17-23); this layer has no
counterpart there.

With ``backend="gloo"`` process groups the exchange runs on CPU tensors so the
shard / offset / merge logic can be tested without GPUs (``merge_fn`` must then
be a host merge supplied by the test).
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import abi


def shard_range(nb: int, rank: int, world: int):
    """Contiguous equal split: rank r owns rows [lo, hi).  Global label = lo + local row."""
    per = (nb + world - 1) // world
    lo = min(nb, rank * per)
    hi = min(nb, lo + per)
    return lo, hi


def pack_candidates(dist, labels):
    """Pack (float32 distance, int64 label) lists [nq, k] into one int32 [nq, k, 3] buffer so
    a single all-gather moves both."""
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


class ShardedIndexFlat:
    """Data-parallel flat index: database rows sharded over the ranks of a process group."""

    def __init__(self, local_index, rank: int, world: int, group=None, merge_fn=None):
        self.local = local_index
        self.rank = rank
        self.world = world
        self.group = group
        self.merge_fn = merge_fn
        self.metric_type = local_index.metric_type

    def set_shard(self, lo: int):
        self.local.set_label_base(lo)

    def _merge_device(self, dist_all, labels_all, k, stream):
        import torch
        P, nq, _ = dist_all.shape
        out_d = torch.empty((nq, k), dtype=torch.float32, device=dist_all.device)
        out_l = torch.empty((nq, k), dtype=torch.int64, device=dist_all.device)
        abi.check_op(abi.lib().b200f_merge_lists(
            ctypes.c_void_p(dist_all.data_ptr()), ctypes.c_void_p(labels_all.data_ptr()), P, nq, k,
            self.metric_type, ctypes.c_void_p(out_d.data_ptr()), ctypes.c_void_p(out_l.data_ptr()),
            ctypes.c_void_p(stream)), "merge_lists")
        return out_d, out_l

    # -- device path: no allocation, no host synchronisation between the three steps ------
    def _buffers(self, nq: int, k: int, device):
        import torch
        key = (nq, k)
        b = self._bufs.get(key) if hasattr(self, "_bufs") else None
        if b is None:
            if not hasattr(self, "_bufs"):
                self._bufs = {}
            dist_bytes = (nq * k * 4 + 15) // 16 * 16
            rank_bytes = (dist_bytes + nq * k * 8 + 15) // 16 * 16
            mine = torch.empty(rank_bytes, dtype=torch.uint8, device=device)
            allb = torch.empty(self.world * rank_bytes, dtype=torch.uint8, device=device)
            b = {
                "rank_bytes": rank_bytes, "dist_bytes": dist_bytes, "mine": mine, "all": allb,
                "d_loc": mine[: nq * k * 4].view(torch.float32).view(nq, k),
                "l_loc": mine[dist_bytes: dist_bytes + nq * k * 8].view(torch.int64).view(nq, k),
                "out_d": torch.empty((nq, k), dtype=torch.float32, device=device),
                "out_l": torch.empty((nq, k), dtype=torch.int64, device=device),
            }
            self._bufs[key] = b
        return b

    def search_device(self, x, k: int, sync: bool = True):
        """x: fp32 CUDA tensor [nq, d] on this rank's GPU, identical on every rank; torch's current
        stream must be the resources' stream (wrap it with torch.cuda.ExternalStream).  Shard
        search, one all-gather of [distances | labels] per rank and the k-way merge are queued
        back to back; the returned tensors are reused by the next call with the same (nq, k)."""
        import torch
        import torch.distributed as dist
        nq = int(x.shape[0])
        b = self._buffers(nq, k, x.device)
        if self.world == 1:
            self.local.search_enqueue(x, k, b["out_d"], b["out_l"])
        else:
            self.local.search_enqueue(x, k, b["d_loc"], b["l_loc"])
            dist.all_gather_into_tensor(b["all"], b["mine"], group=self.group)
            base = b["all"].data_ptr()
            abi.check_op(abi.lib().b200f_merge_lists_strided(
                ctypes.c_void_p(base), ctypes.c_void_p(base + b["dist_bytes"]),
                b["rank_bytes"] // 4, b["rank_bytes"] // 8, self.world, nq, k, self.metric_type,
                ctypes.c_void_p(b["out_d"].data_ptr()), ctypes.c_void_p(b["out_l"].data_ptr()),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "merge_lists_strided")
        if sync:
            self.local.synchronize()
        return b["out_d"], b["out_l"]

    def search(self, x, k: int):
        """x: fp32 queries [nq, d], identical on every rank (torch tensor on this rank's GPU,
        or a CPU tensor / numpy array with a gloo group).  Returns the merged
        (distances, labels) on every rank."""
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
        if packed.is_cuda:
            dist.all_gather_into_tensor(gathered, packed, group=self.group)
        else:  # gloo
            dist.all_gather([gathered[r] for r in range(self.world)], packed, group=self.group)
        d_all, l_all = unpack_candidates(gathered)
        if d_all.is_cuda:
            stream = torch.cuda.current_stream().cuda_stream
            return self._merge_device(d_all.contiguous(), l_all.contiguous(), k, stream)
        if self.merge_fn is None:
            raise RuntimeError("CPU process group: a host merge_fn must be supplied (tests only)")
        out_d, out_l = self.merge_fn(self.metric_type, d_all.numpy(), l_all.numpy())
        return out_d, out_l
