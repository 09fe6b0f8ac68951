"""Peer-memory buffers for the sharded decode path: one process per GPU on one node, every rank's gather buffer and
signal words mapped into every process through CUDA IPC (torch's storage sharing), so that a GEMV kernel can store its
result straight into the other GPUs' memory (`dinoml_b200_gguf_gemv_rcr_scatter`) and a small kernel finishes the
collective (`dinoml_b200_peer_exchange`).  The reference is single-GPU; nothing here has a counterpart there.

Only plain peer stores / loads are used: no TMA, no multicast, no multimem.  Every device-side wait is bounded."""
from __future__ import annotations

import ctypes

from . import _native


def _open_peer_tensor(meta, shape, dtype):
    """Maps a tensor another rank exported with `_export_tensor` and returns it (a view of the peer GPU's memory)."""
    import torch
    storage = torch.UntypedStorage._new_shared_cuda(*meta["storage"])
    t = torch.empty(0, dtype=dtype, device=storage.device)
    return t.set_(storage, meta["offset"], shape)


def _export_tensor(t):
    storage = t.untyped_storage()
    return {"storage": storage._share_cuda_(), "offset": t.storage_offset()}


class PeerExchange:
    """`world` slots of `slot_elems` elements on every rank + 8 signal words, all ranks' copies mapped locally.

    slot r of every rank's buffer receives rank r's GEMV result; `finish_gather` / `finish_reduce` complete the
    collective on the current stream.  All ranks must make the same sequence of calls."""

    def __init__(self, slot_elems: int, dtype, group=None):
        import torch
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("peer exchange supports up to 8 ranks")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dtype, self.slot_elems = dtype, int(slot_elems)
        # own allocations (not sub-ranges of a cached block that other tensors share)
        self.slots = torch.zeros(self.world * self.slot_elems, dtype=dtype, device=dev)
        self.signals = torch.zeros(8, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        metas = [None] * self.world
        dist.all_gather_object(metas, {"slots": _export_tensor(self.slots), "signals": _export_tensor(self.signals),
                                       "device": dev.index}, group=group)
        self.peer_slots, self.peer_signals = [], []
        for r, meta in enumerate(metas):
            if r == self.rank:
                self.peer_slots.append(self.slots)
                self.peer_signals.append(self.signals)
                continue
            if not torch.cuda.can_device_access_peer(dev.index, meta["device"]):
                raise RuntimeError(f"GPU {dev.index} cannot access GPU {meta['device']} as a peer")
            self.peer_slots.append(_open_peer_tensor(meta["slots"], (self.world * self.slot_elems,), dtype))
            self.peer_signals.append(_open_peer_tensor(meta["signals"], (8,), torch.int32))
        self._signal_ptrs = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in self.peer_signals])
        esize = self.slots.element_size()
        others = [r for r in range(self.world) if r != self.rank]
        # where THIS rank's result lives in every other rank's buffer
        self._peer_dst = (ctypes.c_void_p * max(1, len(others)))(
            *[self.peer_slots[r].data_ptr() + self.rank * self.slot_elems * esize for r in others])
        self._n_peers = len(others)
        self.epoch = 0
        dist.barrier(group=group)          # every rank has mapped every buffer before anyone writes

    def local_slot(self):
        """[slot_elems] view of this rank's slot in its own buffer: the primary output of the scatter GEMV."""
        return self.slots[self.rank * self.slot_elems:(self.rank + 1) * self.slot_elems]

    def gathered(self):
        """[world, slot_elems] view of the local buffer (valid after `finish_gather`)."""
        return self.slots.view(self.world, self.slot_elems)

    def scatter_gemv(self, a, b_quant, qtype, bias=None):
        """y = a @ dequant(b_quant)^T (M <= 16) stored into slot [rank] of every rank's buffer, by one kernel."""
        import torch

        from .gguf_blocks import qtype_of
        q = qtype_of(qtype)
        m, k = a.shape
        n = b_quant.shape[0]
        if m * n != self.slot_elems:
            raise ValueError(f"result [{m}, {n}] does not fill a slot of {self.slot_elems} elements")
        lib = _native.lib()
        rc = lib.dinoml_b200_gguf_gemv_rcr_scatter(
            a.data_ptr(), b_quant.data_ptr(), bias.data_ptr() if bias is not None else None, self.local_slot().data_ptr(),
            self._peer_dst, self._n_peers, q.value, _native.DINO_DTYPE[str(a.dtype).replace("torch.", "")], m, n, k,
            torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "dinoml_b200_gguf_gemv_rcr_scatter")

    def _exchange(self, out, count):
        import torch
        self.epoch += 1
        lib = _native.lib()
        rc = lib.dinoml_b200_peer_exchange(self._signal_ptrs, self.world, self.rank, self.epoch, self.slots.data_ptr() if count else None,
                                           out.data_ptr() if count else None, count,
                                           _native.DINO_DTYPE[str(self.dtype).replace("torch.", "")],
                                           torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "dinoml_b200_peer_exchange")

    def finish_gather(self):
        """Completes an all-gather: after this kernel every rank's slot in the local buffer is final."""
        self._exchange(None, 0)
        return self.gathered()

    def finish_reduce(self, out):
        """Completes a one-shot all-reduce: out[i] = sum over ranks of slot r [i] (same bits on every rank)."""
        if out.numel() != self.slot_elems:
            raise ValueError("output does not match the slot size")
        self._exchange(out, self.slot_elems)
        return out
