"""Scatter GEMV and peer exchange kernels on ONE GPU: the extra destinations and the "peer" signal arrays are local
buffers, and the signals a peer would send are written beforehand, so nothing waits on another process."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

import oracle                                                  # noqa: E402
from dinoml_v2_b200 import _native, kernels, synthetic as S   # noqa: E402
from dinoml_v2_b200.gguf_blocks import qtype_of                # noqa: E402

pytestmark = pytest.mark.gpu
BF16 = 6


@pytest.mark.parametrize("qtype,k", [("Q4_K", 1024), ("Q6_K", 2048)])
def test_scatter_gemv_writes_every_destination(qtype, k):
    dev = torch.device("cuda:0")
    lib = _native.lib()
    n = 100
    w = torch.from_numpy(S.random_blocks(qtype, n, k, seed=11)).to(dev)
    stream = torch.cuda.current_stream().cuda_stream
    for m in (1, 2, 4, 9, 16):
        x = torch.from_numpy(S.random_activations(m, k, 12 + m, "float32")).to(dev).to(torch.bfloat16)
        want = kernels.gemm_rcr(x, w, qtype, variant="mma")
        dst = [torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(4)]
        peers = (ctypes.c_void_p * 3)(*[t.data_ptr() for t in dst[1:]])
        rc = lib.dinoml_b200_gguf_gemv_rcr_scatter(x.data_ptr(), w.data_ptr(), None, dst[0].data_ptr(), peers, 3, qtype_of(qtype).value,
                                                   BF16, m, n, k, stream)
        assert rc == 0, _native.last_error()
        torch.cuda.synchronize()
        for t in dst:
            assert torch.equal(t.view(torch.int16), want.view(torch.int16)), (qtype, m)
    # more than 8 extra destinations is refused, M > 16 belongs to the other variants
    assert lib.dinoml_b200_gguf_gemv_rcr_scatter(x.data_ptr(), w.data_ptr(), None, dst[0].data_ptr(), peers, 9, qtype_of(qtype).value,
                                                 BF16, 1, n, k, stream) == 8
    assert lib.dinoml_b200_gguf_gemv_rcr_scatter(x.data_ptr(), w.data_ptr(), None, dst[0].data_ptr(), peers, 3, qtype_of(qtype).value,
                                                 BF16, 17, n, k, stream) == 8


def test_scatter_gemv_full_size_shard_shapes():
    """The stacked gate/up shard [2 * 14336, 8192] and the down shard [8192, 14336] of the 2-GPU sharded FFN."""
    dev = torch.device("cuda:0")
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    for (n, k) in ((28672, 8192), (8192, 14336)):
        w = S.random_blocks_torch("Q4_K", n, k, 21, dev)
        for m in (1, 4):
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            want = kernels.gemm_rcr(x, w, "Q4_K", variant="mma")
            dst = [torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(2)]
            peers = (ctypes.c_void_p * 1)(dst[1].data_ptr())
            rc = lib.dinoml_b200_gguf_gemv_rcr_scatter(x.data_ptr(), w.data_ptr(), None, dst[0].data_ptr(), peers, 1, 12, BF16, m, n, k, stream)
            assert rc == 0, _native.last_error()
            torch.cuda.synchronize()
            assert torch.equal(dst[0].view(torch.int16), want.view(torch.int16)) and torch.equal(dst[1].view(torch.int16), want.view(torch.int16))
            # the same shapes through the entry point the sharded FFN uses (variant chosen by shape: the persistent GEMV here),
            # every destination against the CPU oracle on a sample of weight rows
            dst2 = [torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(2)]
            peers2 = (ctypes.c_void_p * 1)(dst2[1].data_ptr())
            rc = lib.dinoml_b200_gguf_gemm_rcr_scatter(x.data_ptr(), w.data_ptr(), None, dst2[0].data_ptr(), peers2, 1, 12, BF16, m, n, k, 0, stream)
            assert rc == 0, _native.last_error()
            torch.cuda.synchronize()
            assert kernels.device_status() == 0
            rows = np.unique(np.r_[0:16, n // 2:n // 2 + 16, n - 16:n, np.random.default_rng(5).choice(n, 80, replace=False)])
            ridx = torch.from_numpy(rows).to(dev)
            ref = oracle.gemm_quant(x.float().cpu().numpy(), w[ridx].cpu().numpy(), "Q4_K", len(rows), k)
            for t in (dst[0], dst2[0], dst2[1]):
                _, rel, norm = oracle.max_errors(ref, t[:, ridx].float().cpu().numpy())
                assert rel <= 2e-2 and norm <= 2e-2, (n, k, m, rel, norm)


def test_scatter_gemm_umma_writes_every_destination():
    """The tcgen05 kernel's scatter epilogue (finished tiles, including tiles finished after a stream-K reduction)."""
    dev = torch.device("cuda:0")
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    for (qtype, m, n, k) in (("Q4_K", 16, 2048, 2048), ("Q4_K", 64, 384, 4096), ("Q6_K", 200, 130, 2048)):
        w = torch.from_numpy(S.random_blocks(qtype, n, k, seed=31)).to(dev)
        x = torch.from_numpy(S.random_activations(m, k, 32, "float32")).to(dev).to(torch.bfloat16)
        want = kernels.gemm_rcr(x, w, qtype, variant="umma")
        dst = [torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(3)]
        peers = (ctypes.c_void_p * 2)(dst[1].data_ptr(), dst[2].data_ptr())
        rc = lib.dinoml_b200_gguf_gemm_rcr_scatter(x.data_ptr(), w.data_ptr(), None, dst[0].data_ptr(), peers, 2, qtype_of(qtype).value, BF16,
                                                   m, n, k, 0, stream)
        assert rc == 0, _native.last_error()
        torch.cuda.synchronize()
        assert kernels.device_status() == 0
        for t in dst:
            assert torch.equal(t.view(torch.int16), want.view(torch.int16)), (qtype, m, n, k)
    # a shape only the simt variant serves has no scatter epilogue
    w8 = torch.from_numpy(S.random_blocks("Q8_0", 64, 256, seed=1)).to(dev)
    x8 = torch.zeros(1, 256, device=dev, dtype=torch.bfloat16)
    y8 = torch.zeros(1, 64, device=dev, dtype=torch.bfloat16)
    assert lib.dinoml_b200_gguf_gemm_rcr_scatter(x8.data_ptr(), w8.data_ptr(), None, y8.data_ptr(), peers, 2, 8, BF16, 1, 64, 256, 0, stream) == 8


def test_peer_exchange_barrier_and_sum_single_process():
    dev = torch.device("cuda:0")
    lib = _native.lib()
    world, rank, epoch, count = 3, 1, 7, 5000
    local = torch.zeros(8, dtype=torch.int32, device=dev)
    local[0], local[2] = epoch, epoch + 1                 # what ranks 0 and 2 would have stored (later epochs count too)
    fake = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(2)]
    sig = (ctypes.c_void_p * 3)(fake[0].data_ptr(), local.data_ptr(), fake[1].data_ptr())
    slots = torch.randn(world, count, device=dev).to(torch.bfloat16)
    out = torch.empty(count, device=dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.dinoml_b200_peer_exchange(sig, world, rank, epoch, slots.data_ptr(), out.data_ptr(), count, BF16, stream)
    assert rc == 0, _native.last_error()
    torch.cuda.synchronize()
    assert kernels.device_status() == 0
    want = (slots[0].float() + slots[1].float() + slots[2].float()).to(torch.bfloat16)     # same order, fp32 accumulation
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    for f in fake:                                         # this rank's signal landed in word [rank] of both peers
        assert f.cpu().tolist() == [0, epoch, 0, 0, 0, 0, 0, 0]
    # barrier only (count = 0), and argument checks
    assert lib.dinoml_b200_peer_exchange(sig, world, rank, epoch, None, None, 0, BF16, stream) == 0
    assert lib.dinoml_b200_peer_exchange(sig, 9, rank, epoch, None, None, 0, BF16, stream) == 8
    torch.cuda.synchronize()
    assert kernels.device_status() == 0


def test_peer_exchange_bounded_wait_runs_out():
    """A peer that never signals: the kernel's poll limit runs out, the call returns, and the device status reads 6 once.
    One process on one GPU, the "peer" is a signal word that nothing writes; the limit is lowered to a few thousand polls
    so the wait lasts about a millisecond."""
    dev = torch.device("cuda:0")
    lib = _native.lib()
    lib.dinoml_b200_peer_exchange_set_poll_limit.argtypes = [ctypes.c_uint]
    lib.dinoml_b200_peer_exchange_set_poll_limit.restype = ctypes.c_uint
    before = lib.dinoml_b200_peer_exchange_set_poll_limit(4000)
    try:
        world, rank, epoch, count = 2, 0, 3, 256
        local = torch.zeros(8, dtype=torch.int32, device=dev)          # word [1] stays below the epoch: rank 1 never arrives
        local[1] = epoch - 1
        fake = torch.zeros(8, dtype=torch.int32, device=dev)
        sig = (ctypes.c_void_p * 2)(local.data_ptr(), fake.data_ptr())
        slots = torch.ones(world, count, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(count, device=dev, dtype=torch.bfloat16)
        stream = torch.cuda.current_stream().cuda_stream
        assert lib.dinoml_b200_peer_exchange(sig, world, rank, epoch, slots.data_ptr(), out.data_ptr(), count, BF16, stream) == 0
        torch.cuda.synchronize()                                        # the kernel came back by itself
        assert kernels.device_status() == 6
        assert kernels.device_status() == 0                             # reading clears the word
        assert fake.cpu().tolist()[0] == epoch                          # its own signal still went out
    finally:
        assert lib.dinoml_b200_peer_exchange_set_poll_limit(before) == 4000


def test_peer_pull_gather_and_reduce_single_process():
    """The pull exchanges with three "ranks" that are local buffers (signals pre-written): gather copies every other rank's
    shard into place, reduce-slice sums this rank's slice of all partial results in rank order with fp32 accumulation."""
    dev = torch.device("cuda:0")
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    world, rank, epoch = 3, 1, 5
    slot_elems = 3 * 8 * 1000                              # divisible into 16-byte multiples per rank
    slot_bytes = slot_elems * 2
    region = (world + 1) * slot_bytes
    bufs = [torch.zeros(256 + region, dtype=torch.uint8, device=dev) for _ in range(world)]
    sigs = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(world)]
    sigs[rank][0], sigs[rank][2] = epoch, epoch + 3        # what ranks 0 and 2 would have stored by now
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    shards = [torch.randn(slot_elems, device=dev, generator=gen).to(torch.bfloat16) for _ in range(world)]
    for r in range(world):                                 # rank r's shard sits in slot r of ITS buffer
        bufs[r][256 + r * slot_bytes:256 + (r + 1) * slot_bytes].view(torch.bfloat16).copy_(shards[r])
    sig_ptrs = (ctypes.c_void_p * world)(*[s.data_ptr() for s in sigs])
    buf_ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    lib.dinoml_b200_peer_pull.restype = ctypes.c_int
    rc = lib.dinoml_b200_peer_pull(sig_ptrs, buf_ptrs, world, rank, epoch, 0, 256, slot_bytes, 0, 0, BF16, stream)
    assert rc == 0, _native.last_error()
    torch.cuda.synchronize()
    assert kernels.device_status() == 0
    mine = bufs[rank][256:256 + world * slot_bytes].view(torch.bfloat16).view(world, slot_elems)
    for r in range(world):
        assert torch.equal(mine[r], shards[r]), r
    # reduce-slice: partial of rank r = slot r of rank r's buffer; this rank's slice of the sum lands in its result slot
    slice_elems = slot_elems // world
    rc = lib.dinoml_b200_peer_pull(sig_ptrs, buf_ptrs, world, rank, epoch, 1, 256, slot_bytes // world, slot_bytes, 256 + world * slot_bytes,
                                   BF16, stream)
    assert rc == 0, _native.last_error()
    torch.cuda.synchronize()
    want = sum(s[rank * slice_elems:(rank + 1) * slice_elems].float() for s in shards).to(torch.bfloat16)
    res = bufs[rank][256 + world * slot_bytes:256 + (world + 1) * slot_bytes].view(torch.bfloat16)
    assert torch.equal(res[rank * slice_elems:(rank + 1) * slice_elems], want)
    assert int(res[:rank * slice_elems].float().abs().sum()) == 0      # other slices are the other ranks' business
    # argument checks
    assert lib.dinoml_b200_peer_pull(sig_ptrs, buf_ptrs, world, rank, epoch, 0, 256, slot_bytes + 8, 0, 0, BF16, stream) == 7
    assert lib.dinoml_b200_peer_pull(sig_ptrs, buf_ptrs, world, rank, epoch, 2, 256, slot_bytes, 0, 0, BF16, stream) == 8
    assert lib.dinoml_b200_peer_pull(sig_ptrs, buf_ptrs, 9, rank, epoch, 0, 256, slot_bytes, 0, 0, BF16, stream) == 8
    assert kernels.device_status() == 0


def test_peer_exchange_device_epoch_in_a_replayed_graph():
    """Exchanges captured in a CUDA graph keep their epoch in device memory: every replay signals the next value, the last
    block out stores it back; the "peers" here are local signal arrays pre-written far ahead."""
    dev = torch.device("cuda:0")
    lib = _native.lib()
    world, rank, count = 3, 1, 5000
    local = torch.full((8,), 1000, dtype=torch.int32, device=dev)      # ranks 0 and 2 are "far ahead": every wait passes
    fakes = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(2)]
    sig = (ctypes.c_void_p * world)(fakes[0].data_ptr(), local.data_ptr(), fakes[1].data_ptr())
    ctr = torch.zeros(2, dtype=torch.int32, device=dev)
    slots = torch.randn(world, count, device=dev).to(torch.bfloat16)
    out = torch.zeros(count, device=dev, dtype=torch.bfloat16)
    side = torch.cuda.Stream(device=dev)

    def two_exchanges():
        s = torch.cuda.current_stream().cuda_stream
        assert lib.dinoml_b200_peer_exchange_ctr(sig, world, rank, ctr.data_ptr(), None, None, 0, BF16, s) == 0, _native.last_error()
        assert lib.dinoml_b200_peer_exchange_ctr(sig, world, rank, ctr.data_ptr(), slots.data_ptr(), out.data_ptr(), count, BF16, s) == 0

    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        two_exchanges()                                   # epochs 1, 2
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            two_exchanges()
    torch.cuda.synchronize()
    assert ctr.cpu().tolist() == [2, 0] and fakes[0].cpu().tolist()[rank] == 2
    for replay in range(3):
        graph.replay()
        torch.cuda.synchronize()
        assert ctr.cpu().tolist() == [4 + 2 * replay, 0]
        for f in fakes:
            assert f.cpu().tolist()[rank] == 4 + 2 * replay               # the signal of the last exchange of the replay
    want = slots.float().sum(dim=0).to(torch.bfloat16)
    assert torch.equal(out, want) and kernels.device_status() == 0
    assert lib.dinoml_b200_peer_exchange_ctr(sig, world, rank, None, None, None, 0, BF16, None) == 1      # null counter
