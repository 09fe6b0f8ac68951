"""GPU test of the allocation-free prefill GEMM entry point (collected last on purpose).

`dinoml_b200_gguf_gemm_rcr_prealloc` exists for hosts that forbid device allocation calls - everything it needs
beyond the caller's own tensors sits in a fixed array inside the library.  The test drives it straight through
the C ABI with ctypes and checks it against the ordinary entry point on two consecutive calls of different
sizes (the second call finds the first call's leftovers in the shared scratch), then checks that a problem
whose partial sums exceed the built-in scratch is refused with a message instead of being run."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from dinoml_v2_b200 import _native, synthetic as S
from dinoml_v2_b200.gguf_blocks import qtype_of

pytestmark = pytest.mark.gpu

UMMA, BF16 = 3, 6


def _entry_points():
    lib = _native.lib()
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.dinoml_b200_gguf_gemm_rcr_prealloc.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]
    lib.dinoml_b200_gguf_gemm_rcr_prealloc.restype = ci
    lib.dinoml_b200_gguf_prealloc_scratch_bytes.restype = ctypes.c_size_t
    lib.dinoml_b200_gguf_gemm_rcr_workspace.restype = ctypes.c_size_t
    return lib


def _run_pair(lib, qtype, m, n, k, seed, bias):
    dev = torch.device("cuda:0")
    q = qtype_of(qtype)
    blocks = S.random_blocks(qtype, n, k, seed)
    w = torch.from_numpy(blocks).to(dev)
    x = torch.from_numpy(S.random_activations(m, k, seed + 1, "float32")).to(dev).to(torch.bfloat16)
    b = torch.randn(n, device=dev).to(torch.bfloat16) if bias else None
    want = torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16)
    got = torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    bp = b.data_ptr() if b is not None else None
    assert lib.dinoml_b200_gguf_gemm_rcr(x.data_ptr(), w.data_ptr(), bp, want.data_ptr(), q.value, BF16, m, n, k, UMMA, stream) == 0
    torch.cuda.synchronize()
    # "allocates nothing": the driver's free-memory figure is the same before and after the call, although this shape
    # needs partial-tile scratch (the ordinary entry point grows a cudaMalloc'ed workspace for it)
    need = lib.dinoml_b200_gguf_gemm_rcr_workspace(q.value, BF16, m, n, k, UMMA)
    assert need > 0
    # the first call on a device makes the driver place the library's device image (kernel code, the static scratch) on the GPU -
    # lazy module loading, which the documentation tells callers to get over with at start-up: warm up, then measure
    assert lib.dinoml_b200_gguf_gemm_rcr_prealloc(x.data_ptr(), w.data_ptr(), bp, got.data_ptr(), q.value, BF16, m, n, k, stream) == 0
    torch.cuda.synchronize()
    got.fill_(float("nan"))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.dinoml_b200_gguf_gemm_rcr_prealloc(x.data_ptr(), w.data_ptr(), bp, got.data_ptr(), q.value, BF16, m, n, k, stream)
    assert rc == 0, _native.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert lib.dinoml_b200_gguf_device_status() == 0
    # against the CPU oracle too, not only against the sibling entry point
    ref = oracle.gemm_quant(x.float().cpu().numpy(), blocks, qtype, n, k)
    if b is not None:
        ref = ref + b.float().cpu().numpy()
    _, _, norm_oracle = oracle.max_errors(ref, got.float().cpu().numpy())
    assert norm_oracle <= 2e-2, (qtype, m, n, k, norm_oracle)
    a, e = got.float().cpu().numpy(), want.float().cpu().numpy()
    assert np.isfinite(a).all() and np.isfinite(e).all()
    norm = float(np.abs(a - e).max() / max(np.abs(e).max(), 1e-30))
    assert norm <= 2e-2, (qtype, m, n, k, norm)       # the bar the other matmul tests use; same kernel, so in practice 0
    return norm


def test_prealloc_entry_matches_regular_entry_twice_in_a_row():
    lib = _entry_points()
    assert lib.dinoml_b200_gguf_prealloc_scratch_bytes() == 16 << 20
    # both shapes have few output tiles and a long K, so their tiles are cut between SMs: they really use the scratch
    first = _run_pair(lib, "Q4_K", 96, 256, 4096, 31, bias=False)
    second = _run_pair(lib, "Q6_K", 40, 384, 8192, 47, bias=True)
    assert first == 0.0 and second == 0.0            # identical kernel and summation order


def test_prealloc_entry_refuses_problems_beyond_its_scratch():
    lib = _entry_points()
    dev = torch.device("cuda:0")
    m, n, k = 512, 4608, 2048                         # one 256 x 128 fp32 partial tile per SM: 148 x 128 KiB > 16 MiB
    w = torch.from_numpy(S.random_blocks("Q4_K", n, k, 5)).to(dev)
    x = torch.zeros(m, k, device=dev, dtype=torch.bfloat16)
    y = torch.zeros(m, n, device=dev, dtype=torch.bfloat16)
    rc = lib.dinoml_b200_gguf_gemm_rcr_prealloc(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 12, BF16, m, n, k, None)
    assert rc == 8
    msg = _native.last_error()
    lib.dinoml_b200_gguf_gemm_rcr_workspace.restype = ctypes.c_size_t
    need = lib.dinoml_b200_gguf_gemm_rcr_workspace(12, BF16, m, n, k, UMMA)
    assert need > (16 << 20) and str(need) in msg and str(16 << 20) in msg, msg
    # small-M problems belong to the GEMV kernels, not to this entry point
    assert lib.dinoml_b200_gguf_gemm_rcr_prealloc(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 12, BF16, 4, n, k, None) != 0
