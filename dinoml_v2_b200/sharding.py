"""Tensor-parallel sharding of GGUF-encoded linears across the GPUs of one node (one process per GPU, NCCL).

The reference has no distributed code at all; this covers the Llama-70B-shaped FFN configuration:
* N-split (gate / up): packed rows are independent and contiguous, so rank r keeps rows [r*N/G, (r+1)*N/G) - a plain
  byte slice - computes y_r[M, N/G] and the ranks all-gather;
* K-split (down): shards are cut at 256-weight super-block granularity; rank r needs blocks [r*nb/G, (r+1)*nb/G) of
  EVERY row, a one-time strided repack at load into a dense [N, nb/G] block matrix, computes a partial [M, N] and the
  ranks all-reduce.  The N-shard of gate/up on rank r is exactly the K-slice rank r needs for down.
Two ways to finish the collectives: torch.distributed (NCCL over NVLink) on the compute stream, or - for decode
and small batches - the peer-memory path of `peer.PeerExchange`, where gate and up are one stacked weight, the GEMV kernels
store their results straight into every GPU's gather buffer and one small kernel per collective does the barrier
(all-gather) or the barrier + sum (all-reduce)."""
from __future__ import annotations

import numpy as np

from .gguf_blocks import qtype_of, row_bytes


def shard_rows(blocks: np.ndarray, rank: int, world: int) -> np.ndarray:
    """N-split: contiguous slice of rows.  blocks: uint8 [N, row_bytes]."""
    n = blocks.shape[0]
    if n % world:
        raise ValueError(f"N={n} is not divisible by world size {world}")
    per = n // world
    return np.ascontiguousarray(blocks[rank * per:(rank + 1) * per])


def shard_k(blocks: np.ndarray, qtype, k: int, rank: int, world: int) -> tuple[np.ndarray, int]:
    """K-split at block granularity.  Returns (uint8 [N, row_bytes(k/world)], k/world)."""
    q = qtype_of(qtype)
    nb = k // q.block_size
    if blocks.shape[1] != row_bytes(q, k):
        raise ValueError("blocks do not match (qtype, k)")
    if nb % world:
        raise ValueError(f"K={k} has {nb} {q.name} blocks per row, not divisible by world size {world}")
    per = nb // world
    if (per * q.block_bytes) % 16:
        raise ValueError(f"a K-shard row of {per} {q.name} blocks is {per * q.block_bytes} B, not 16-byte aligned; "
                         "choose a world size that keeps shard rows 16-byte multiples")
    n = blocks.shape[0]
    shard = blocks.reshape(n, nb, q.block_bytes)[:, rank * per:(rank + 1) * per, :]
    return np.ascontiguousarray(shard).reshape(n, per * q.block_bytes), per * q.block_size


class ShardedFFN:
    """gate / up N-split + all-gather, down K-split + all-reduce, for one rank.  Device tensors are torch tensors."""

    def __init__(self, gate_shard, up_shard, down_shard, qtype, hidden: int, ffn: int, group=None):
        import torch.distributed as dist
        self.gate, self.up, self.down = gate_shard, up_shard, down_shard
        self.qtype, self.hidden, self.ffn = qtype, hidden, ffn
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def gate_up(self, x, out_gate, out_up, gathered_gate, gathered_up):
        """x [M, hidden] replicated.  gathered_* are [world, M, ffn/world] (rank-major, no transpose kernel)."""
        import torch.distributed as dist

        from . import kernels
        kernels.gemm_rcr(x, self.gate, self.qtype, out=out_gate)
        kernels.gemm_rcr(x, self.up, self.qtype, out=out_up)
        if self.world > 1:
            dist.all_gather_into_tensor(gathered_gate.view(-1, out_gate.shape[-1]), out_gate, group=self.group)
            dist.all_gather_into_tensor(gathered_up.view(-1, out_up.shape[-1]), out_up, group=self.group)
        return gathered_gate, gathered_up

    # ---- peer-memory path (decode and small batches; the variant is chosen by shape as for gemm_rcr) ----------------------------------------------------------------------
    def enable_peer_path(self, m: int, dtype, share_with=None, device_epoch: bool = False):
        """Stacks gate and up into one [2 * ffn / world, hidden] weight (one launch, one gather) and maps the exchange
        buffers of all ranks (or reuses those of `share_with`, another ShardedFFN of the same shape that runs on the
        same stream).  Collective call: every rank must make it."""
        import torch

        from .peer import PeerExchange
        self.gate_up_stacked = torch.cat([self.gate, self.up], dim=0).contiguous()
        self.peer_m = int(m)
        if share_with is not None:
            self.xchg_gate_up, self.xchg_down = share_with.xchg_gate_up, share_with.xchg_down
        else:
            self.xchg_gate_up = PeerExchange(self.peer_m * self.gate_up_stacked.shape[0], dtype, self.group, device_epoch=device_epoch)
            self.xchg_down = PeerExchange(self.peer_m * self.hidden, dtype, self.group, device_epoch=device_epoch)

    def gate_up_peer(self, x):
        """Returns [world, M, 2 * ffn / world]: per rank, its gate rows then its up rows."""
        self.xchg_gate_up.scatter_gemv(x, self.gate_up_stacked, self.qtype)
        g = self.xchg_gate_up.finish_gather()
        return g.view(self.world, self.peer_m, self.gate_up_stacked.shape[0])

    def down_proj_peer(self, h_slice, out):
        """out [M, hidden] = sum over ranks of h_slice_r @ down_r^T, identical bits on every rank."""
        self.xchg_down.scatter_gemv(h_slice, self.down, self.qtype)
        self.xchg_down.finish_reduce(out)
        return out

    def gate_up_pull(self, x):
        """The peer path for prefill-sized batches: the GEMM stores its shard locally, one pull kernel gathers the others."""
        from . import kernels
        xg = self.xchg_gate_up
        kernels.gemm_rcr(x, self.gate_up_stacked, self.qtype, out=xg.local_slot().view(self.peer_m, self.gate_up_stacked.shape[0]))
        g = xg.pull_gather()
        return g.view(self.world, self.peer_m, self.gate_up_stacked.shape[0])

    def down_proj_pull(self, h_slice, out=None):
        """Down projection with the two-shot pull all-reduce (identical bits on every rank)."""
        from . import kernels
        xd = self.xchg_down
        kernels.gemm_rcr(h_slice, self.down, self.qtype, out=xd.local_slot().view(self.peer_m, self.hidden))
        return xd.pull_all_reduce(out)

    def swiglu_mlp_peer(self, x, out):
        """The whole gated MLP, out [M, hidden] = (silu(x Wgate^T) * (x Wup^T)) Wdown^T, in three launches and no
        all-gather: rank r's rows of gate / up are exactly the K-slice of down it owns, so the gated activations stay
        local (one dual GEMM on the row-interleaved gate / up shard), and only the down projection's partial sums cross
        NVLink (scatter epilogue + barrier-and-sum kernel).  Needs `enable_peer_path`."""
        from . import kernels
        if not hasattr(self, "gate_up_rows8"):
            self.gate_up_rows8 = kernels.interleave_rows8(self.gate, self.up)
        h = kernels.dual_gemm_rcr(x, self.gate_up_rows8, self.qtype, "silu")
        self.xchg_down.scatter_gemv(h, self.down, self.qtype)
        self.xchg_down.finish_reduce(out)
        return out

    def down_proj(self, h_slice, out):
        """h_slice [M, ffn/world] = this rank's K-slice of the down-projection input; out [M, hidden] is summed in place."""
        import torch.distributed as dist

        from . import kernels
        kernels.gemm_rcr(h_slice, self.down, self.qtype, out=out)
        if self.world > 1:
            dist.all_reduce(out, group=self.group)
        return out
