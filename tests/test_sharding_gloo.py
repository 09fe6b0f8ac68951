"""CPU test of the multi-GPU sharding logic with two gloo ranks: N-split + all-gather and K-split + all-reduce
reassemble exactly what the unsharded CPU oracle computes (the oracle plays the role of the per-rank kernel)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from dinoml_v2_b200 import sharding, synthetic as S
    hidden, ffn, m = 512, 1024, 3
    gate = S.random_blocks("Q4_K", ffn, hidden, 1)
    down = S.random_blocks("Q4_K", hidden, ffn, 2)
    x = S.random_activations(m, hidden, 3, "float32")
    h = S.random_activations(m, ffn, 4, "float32")
    # N-split + all-gather (rank-major [world, M, ffn/world])
    g_shard = sharding.shard_rows(gate, rank, world)
    y_r = torch.from_numpy(oracle.gemm_quant(x, g_shard, "Q4_K", ffn // world, hidden))
    gathered = torch.empty(world, m, ffn // world)
    dist.all_gather_into_tensor(gathered.view(world * m, ffn // world), y_r)
    full = gathered.permute(1, 0, 2).reshape(m, ffn).numpy()
    ref = oracle.gemm_quant(x, gate, "Q4_K", ffn, hidden)
    assert np.array_equal(full, ref)
    # K-split + all-reduce
    d_shard, k_shard = sharding.shard_k(down, "Q4_K", ffn, rank, world)
    assert k_shard == ffn // world and d_shard.shape == (hidden, 144 * (ffn // world // 256))
    part = torch.from_numpy(oracle.gemm_quant(np.ascontiguousarray(h[:, rank * k_shard:(rank + 1) * k_shard]), d_shard, "Q4_K", hidden, k_shard))
    dist.all_reduce(part)
    ref_d = oracle.gemm_quant(h, down, "Q4_K", hidden, ffn)
    _, _, norm = oracle.max_errors(ref_d, part.numpy())
    assert norm < 1e-5, norm          # only the fp32 summation order differs
    # the N-shard of gate on rank r covers exactly the K-slice of down that rank r owns
    assert (ffn // world) == k_shard
    Path(result_dir, f"ok{rank}").write_text("ok")
    dist.destroy_process_group()


def test_two_rank_gloo_sharding(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_validation():
    from dinoml_v2_b200 import sharding, synthetic as S
    b = S.random_blocks("Q6_K", 8, 1024, 1)
    with pytest.raises(ValueError, match="16-byte"):
        sharding.shard_k(b, "Q6_K", 1024, 0, 4)          # 1 block of 210 B per shard row
    with pytest.raises(ValueError, match="divisible"):
        sharding.shard_rows(b, 0, 3)
    s0, k0 = sharding.shard_k(S.random_blocks("Q4_K", 8, 1024, 1), "Q4_K", 1024, 1, 2)
    assert k0 == 512 and s0.shape == (8, 288)


@pytest.mark.parametrize("world", [2, 4])
def test_gated_mlp_needs_no_all_gather(world):
    """The identity behind ShardedFFN.swiglu_mlp_peer: rank r's rows of gate / up are the K-slice of down it owns, so
    sum over ranks of (silu(x gate_r^T) * (x up_r^T)) down_r^T equals the unsharded gated MLP.  Oracle on every 'rank',
    the sum stands in for the all-reduce; also checks the row-interleaved weight the dual GEMM reads."""
    import oracle
    from dinoml_v2_b200 import kernels, sharding, synthetic as S
    hidden, ffn, m = 512, 1024, 2
    gate, up = S.random_blocks("Q4_K", ffn, hidden, 11), S.random_blocks("Q4_K", ffn, hidden, 12)
    down = S.random_blocks("Q4_K", hidden, ffn, 13)
    x = S.random_activations(m, hidden, 14, "float32")
    full_h = oracle.dual_gemm_quant(x, gate, up, "Q4_K", ffn, hidden, "silu")
    want = oracle.gemm_quant(full_h, down, "Q4_K", hidden, ffn)
    total = np.zeros_like(want, dtype=np.float64)
    for r in range(world):
        g_r, u_r = sharding.shard_rows(gate, r, world), sharding.shard_rows(up, r, world)
        d_r, k_r = sharding.shard_k(down, "Q4_K", ffn, r, world)
        fused = kernels.interleave_rows8(g_r, u_r)
        assert np.array_equal(fused[0:8], g_r[0:8]) and np.array_equal(fused[8:16], u_r[0:8])
        h_r = oracle.dual_gemm_quant(x, g_r, u_r, "Q4_K", ffn // world, hidden, "silu")
        assert np.array_equal(h_r, full_h[:, r * k_r:(r + 1) * k_r])
        total += oracle.gemm_quant(h_r, d_r, "Q4_K", hidden, k_r)
    assert np.abs(total - want).max() <= 1e-4 * np.abs(want).max()
