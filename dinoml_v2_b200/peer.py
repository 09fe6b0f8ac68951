"""Peer-memory buffers for the sharded decode path: one process per GPU on one node, every rank's gather buffer and
signal words mapped into every process (torch's symmetric memory: CUDA virtual-memory allocations whose handles the
ranks exchange and map with access for the local GPU), so that a GEMV kernel can store its result straight into the
other GPUs' memory (`dinoml_b200_gguf_gemv_rcr_scatter`) and a small kernel finishes the collective
(`dinoml_b200_peer_exchange`).  The reference is single-GPU; nothing here has a counterpart there.

Only plain peer stores / loads are used on peer memory: no TMA from a peer, no multicast, no multimem.  Every device-side
wait is bounded.

Slot reuse.  The exchange kernel lets a rank go as soon as it has seen every peer's signal and summed its OWN copy of
the slots; nothing tells it that the peers have finished reading theirs.  So each PeerExchange owns TWO slot sets and
alternates them by epoch parity: the results for exchange e+1 are stored into set (e+1) & 1 while a slow peer may still
be summing set e & 1.  The set written for e+1 was last read in exchange e-1, and a rank only signals epoch e after its
own exchange e-1 has completed, so a full barrier always separates a set's readers from its next writer - one
PeerExchange may be used back to back (down_proj_peer in a loop, swiglu_mlp_peer) without a race.

Pull path (prefill-sized results).  `pull_gather` / `pull_all_reduce` leave the GEMM's result in LOCAL memory and move
it with `dinoml_b200_peer_pull` (one CTA per SM, 16-byte loads from the peers' buffers): an all-gather is one kernel, an
all-reduce is two (every rank sums its own slice of all partial results in rank order, then the slices are gathered from
an extra slot of the set), so every rank ends with identical bits.  A collective, not a kernel, advances the slot set."""
from __future__ import annotations

import ctypes
import os

from . import _native

_SIGNAL_BYTES = 256      # 8 signal words, padded so that the slots start on a 256-byte boundary
_QTYPE_VALUE: dict = {}  # qtype (name or enum) -> ggml id, filled on first use


class PeerExchange:
    """Two sets of `world` slots of `slot_elems` elements on every rank + 8 signal words, all ranks' copies mapped locally.

    slot r of every rank's buffer receives rank r's GEMV result; `finish_gather` / `finish_reduce` complete the
    collective on the current stream.  All ranks must make the same sequence of calls."""

    def __init__(self, slot_elems: int, dtype, group=None, device_epoch: bool = False):
        import torch
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("peer exchange supports up to 8 ranks")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dtype, self.slot_elems = dtype, int(slot_elems)
        esize = torch.empty(0, dtype=dtype).element_size()
        # plain peer stores only: keep the allocation off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self._slot_bytes = self.slot_elems * esize
        # one slot set = `world` slots + one more for the reduced result of the pull all-reduce, 256-byte aligned
        self._set_bytes = -(-((self.world + 1) * self._slot_bytes) // 256) * 256
        nbytes = _SIGNAL_BYTES + 2 * self._set_bytes
        self._buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)      # [signals | set 0: slot 0 .. | set 1: slot 0 ..]
        self._buffer.zero_()
        torch.cuda.synchronize()
        self._handle = symm_mem.rendezvous(self._buffer, dist.group.WORLD if group is None else group)
        base = [int(p) for p in self._handle.buffer_ptrs]                           # every rank's buffer, mapped here
        if len(base) != self.world or base[self.rank] != self._buffer.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned an unexpected mapping")
        self.signals = self._buffer[:32].view(torch.int32)
        used = self.world * self.slot_elems * esize
        self._sets = [self._buffer[_SIGNAL_BYTES + p * self._set_bytes:_SIGNAL_BYTES + p * self._set_bytes + used].view(dtype)
                      for p in (0, 1)]
        self._signal_ptrs = (ctypes.c_void_p * self.world)(*base)
        others = [r for r in range(self.world) if r != self.rank]
        # where THIS rank's result lives in every other rank's buffer, per slot set
        self._peer_dst = [(ctypes.c_void_p * max(1, len(others)))(
            *[base[r] + _SIGNAL_BYTES + p * self._set_bytes + self.rank * self.slot_elems * esize for r in others]) for p in (0, 1)]
        self._n_peers = len(others)
        # raw addresses and codes, so that a launch costs one ctypes call and no tensor views (decode steps are a few
        # microseconds of device time: the host side must not be the slower one)
        self._set_ptr = [int(t.data_ptr()) for t in self._sets]
        self._local_ptr = [ptr + self.rank * self.slot_elems * esize for ptr in self._set_ptr]
        self._dtype_code = _native.DINO_DTYPE[str(dtype).replace("torch.", "")]
        self._lib = _native.lib()
        self._auto = _native.variant_code("auto")
        self._buffer_ptrs = (ctypes.c_void_p * self.world)(*base)
        self._set_off = [_SIGNAL_BYTES + p * self._set_bytes for p in (0, 1)]
        self._result = [self._buffer[off + self.world * self._slot_bytes:off + (self.world + 1) * self._slot_bytes].view(dtype)
                        for off in self._set_off]
        # device_epoch: the kernels keep the signal counter in device memory, so a captured CUDA graph of exchanges can be
        # replayed (capture an even number of collectives: the slot-set parity of a replay is then the captured one)
        self._epoch_ctr = torch.zeros(2, dtype=torch.int32, device=dev) if device_epoch else None
        self.epoch = 0          # signal counter: one per exchange KERNEL
        self.round = 0          # collectives completed: its parity picks the slot set
        dist.barrier(group=group)          # every rank has mapped every buffer before anyone writes

    @property
    def slots(self):
        """The slot set of the exchange that completed last (after `finish_*`), [world * slot_elems]."""
        return self._sets[self.round & 1]

    def local_slot(self):
        """[slot_elems] view of this rank's slot in the set the NEXT exchange reads: the primary output of the scatter GEMV."""
        nxt = self._sets[(self.round + 1) & 1]
        return nxt[self.rank * self.slot_elems:(self.rank + 1) * self.slot_elems]

    def gathered(self):
        """[world, slot_elems] view of the local buffer (valid after `finish_gather`, until the exchange after the next)."""
        return self.slots.view(self.world, self.slot_elems)

    def scatter_gemv(self, a, b_quant, qtype, bias=None, variant: str = "auto"):
        """y = a @ dequant(b_quant)^T stored into slot [rank] of every rank's buffer, by one kernel (mma or umma variant)."""
        import torch
        qv = _QTYPE_VALUE.get(qtype)
        if qv is None:
            from .gguf_blocks import qtype_of
            qv = _QTYPE_VALUE[qtype] = qtype_of(qtype).value
        m, k = a.shape
        n = b_quant.shape[0]
        if m * n != self.slot_elems:
            raise ValueError(f"result [{m}, {n}] does not fill a slot of {self.slot_elems} elements")
        if a.dtype != self.dtype:
            raise ValueError("activation dtype differs from the exchange buffers'")
        nxt = (self.round + 1) & 1                    # the set the NEXT exchange reads
        rc = self._lib.dinoml_b200_gguf_gemm_rcr_scatter(
            a.data_ptr(), b_quant.data_ptr(), bias.data_ptr() if bias is not None else None, self._local_ptr[nxt],
            self._peer_dst[nxt], self._n_peers, qv, self._dtype_code, m, n, k,
            self._auto if variant == "auto" else _native.variant_code(variant), torch.cuda.current_stream().cuda_stream)
        if rc:
            _native.check(rc, "dinoml_b200_gguf_gemm_rcr_scatter")

    def _exchange(self, out, count):
        import torch
        self.epoch += 1
        self.round += 1
        if self._epoch_ctr is not None:
            rc = self._lib.dinoml_b200_peer_exchange_ctr(self._signal_ptrs, self.world, self.rank, self._epoch_ctr.data_ptr(),
                                                         self._set_ptr[self.round & 1] if count else None,
                                                         out.data_ptr() if count else None, count, self._dtype_code,
                                                         torch.cuda.current_stream().cuda_stream)
        else:
            rc = self._lib.dinoml_b200_peer_exchange(self._signal_ptrs, self.world, self.rank, self.epoch,
                                                     self._set_ptr[self.round & 1] if count else None,
                                                     out.data_ptr() if count else None, count, self._dtype_code,
                                                     torch.cuda.current_stream().cuda_stream)
        if rc:
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

    # ---- pull path: the GEMM writes local memory only -----------------------------------------------------------------
    def _pull(self, mode: int, off: int, chunk: int, region_stride: int, dst_off: int):
        import torch
        self.epoch += 1
        if self._epoch_ctr is not None:
            rc = self._lib.dinoml_b200_peer_pull_ctr(self._signal_ptrs, self._buffer_ptrs, self.world, self.rank, self._epoch_ctr.data_ptr(), mode,
                                                     off, chunk, region_stride, dst_off, self._dtype_code, torch.cuda.current_stream().cuda_stream)
        else:
            rc = self._lib.dinoml_b200_peer_pull(self._signal_ptrs, self._buffer_ptrs, self.world, self.rank, self.epoch, mode, off, chunk,
                                                 region_stride, dst_off, self._dtype_code, torch.cuda.current_stream().cuda_stream)
        if rc:
            _native.check(rc, "dinoml_b200_peer_pull")

    def pull_gather(self):
        """Completes an all-gather whose shards every rank stored into `local_slot()` of its own buffer: one kernel pulls the
        other ranks' shards over NVLink.  Returns the [world, slot_elems] view."""
        if self._slot_bytes % 16:
            raise ValueError("pull exchanges need slots that are multiples of 16 bytes")
        self.round += 1
        self._pull(0, self._set_off[self.round & 1], self._slot_bytes, 0, 0)
        return self.gathered()

    def pull_all_reduce(self, out=None):
        """Two-shot all-reduce of the partial results every rank stored into `local_slot()`: every rank sums slice `rank` of all
        partial results (rank order, fp32), then the slices are gathered.  Returns the reduced [slot_elems] tensor (a view of
        this rank's buffer, valid until the collective after the next) or copies it into `out`."""
        if self._slot_bytes % (16 * self.world):
            raise ValueError("the pull all-reduce needs slots that split into 16-byte multiples per rank")
        self.round += 1
        s = self.round & 1
        off, res_off, slice_bytes = self._set_off[s], self._set_off[s] + self.world * self._slot_bytes, self._slot_bytes // self.world
        self._pull(1, off, slice_bytes, self._slot_bytes, res_off)       # reduce-scatter: partial of rank r = slot r of ITS buffer
        self._pull(0, res_off, slice_bytes, 0, 0)                        # all-gather of the reduced slices
        res = self._result[s]
        if out is not None:
            out.view(-1).copy_(res)
            return out
        return res
