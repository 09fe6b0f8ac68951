"""GPU parity tests (run on the B200 box): every CUDA kernel, called through the C ABI, against the
CPU oracle and the committed golden fixtures.

Bars: dequantization bit-exact; matmul max relative error <= 1e-3 for float32/float16 outputs and
<= 2e-2 for bfloat16 outputs, measured with the reference's own metric |d| / max(1, |expected|)
(tools/bench_ck_gguf_q8_gemm.hip:798-808) AND normalised by max|expected|."""
import numpy as np
import pytest
import torch

import oracle
from dinoml_v2_b200 import kernels, manifest as mf, synthetic as S
from dinoml_v2_b200.gguf_blocks import qtype_of

pytestmark = pytest.mark.gpu

QT = ("Q8_0", "Q4_K", "Q6_K")
QT_MORE = ("Q4_0", "Q5_K", "Q2_K", "Q3_K", "MXFP4", "NVFP4")     # decoded by the dequantizer and the CUDA-core gemm variant
TOL = {"float32": 1e-3, "float16": 1e-3, "bfloat16": 2e-2}
TDT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need the CUDA device"
    return torch.device("cuda:0")


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.float32:
        return t.cpu().numpy().view(np.uint32)
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("qtype", QT + QT_MORE)
def test_dequant_golden_bit_exact(dev, golden_dir, qtype):
    kat = np.load(golden_dir / "gguf_dequant_kat.npz")
    blocks = torch.from_numpy(kat[f"{qtype}_blocks"]).to(dev)
    k = int(kat[f"{qtype}_n_per_row"])
    for dtype, key in (("float32", "f32_bits"), ("float16", "f16_bits"), ("bfloat16", "bf16_bits")):
        got = kernels.dequantize_rows(blocks, qtype, k, dtype)
        assert np.array_equal(_bits(got), kat[f"{qtype}_{key}"]), (qtype, dtype)


@pytest.mark.parametrize("qtype", QT + QT_MORE)
@pytest.mark.parametrize("rows,nblk", [(1, 1), (3, 5), (257, 7), (64, 16)])
def test_dequant_random_bit_exact(dev, qtype, rows, nblk):
    k = nblk * qtype_of(qtype).block_size
    blocks = S.random_blocks(qtype, rows, k, seed=100 + rows + nblk)
    got = kernels.dequantize_rows(torch.from_numpy(blocks).to(dev), qtype, k, "float32")
    assert np.array_equal(_bits(got), oracle.dequantize(blocks, qtype, k).view(np.uint32))
    got16 = kernels.dequantize_rows(torch.from_numpy(blocks).to(dev), qtype, k, "bfloat16")
    assert np.array_equal(_bits(got16), oracle.dequantize(blocks, qtype, k, "bfloat16"))


def test_dequant_full_size_checksum(dev):
    """Config-2 sized tensor (Q4_K 11008x4096): compare a sampled set of rows bit for bit and an
    order-independent checksum of all output bit patterns against the oracle on those rows."""
    n, k = 11008, 4096
    blocks = S.random_blocks("Q4_K", n, k, seed=2000)
    got = kernels.dequantize_rows(torch.from_numpy(blocks).to(dev), "Q4_K", k, "float32")
    rows = np.r_[0:8, 5000:5008, n - 8:n]
    want = oracle.dequantize(blocks[rows], "Q4_K", k)
    assert np.array_equal(_bits(got[torch.from_numpy(rows).to(dev)]), want.view(np.uint32))
    # idempotence / determinism: second call gives identical bits
    again = kernels.dequantize_rows(torch.from_numpy(blocks).to(dev), "Q4_K", k, "float32")
    assert torch.equal(got.view(torch.int32), again.view(torch.int32))
    want_all = oracle.dequantize(blocks, "Q4_K", k)
    assert int(got.view(torch.int32).to(torch.int64).sum().item()) == int(want_all.view(np.int32).astype(np.int64).sum())


@pytest.mark.parametrize("qtype", QT_MORE)
def test_dequant_random_bytes_bit_exact(dev, qtype):
    """Blocks of uniformly random BYTES: every scale bit pattern (NaN, Inf, subnormals) and every packed field value;
    compared as bit patterns, at an odd device address for the types that need no alignment."""
    q = qtype_of(qtype)
    k = 5 * q.block_size
    raw = np.random.default_rng(31).integers(0, 256, (37, 5 * q.block_bytes), dtype=np.uint8)
    want = oracle.dequantize(raw, qtype, k)
    got = kernels.dequantize_rows(torch.from_numpy(raw).to(dev), qtype, k, "float32")
    a, b = _bits(got), want.view(np.uint32)
    nan = np.isnan(want)
    assert np.array_equal(a[~nan], b[~nan]) and np.isnan(got.cpu().numpy()[nan]).all(), qtype
    if qtype == "MXFP4":                                 # 17-byte blocks: any byte address is legal
        pad = torch.zeros(raw.size + 1, dtype=torch.uint8, device=dev)
        pad[1:] = torch.from_numpy(raw.reshape(-1)).to(dev)
        got2 = kernels.dequantize_rows(pad[1:].view(37, -1), qtype, k, "float32")
        assert torch.equal(got2.view(torch.int32), got.view(torch.int32))


@pytest.mark.parametrize("qtype", QT_MORE)
@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
def test_gemm_further_qtypes(dev, qtype, dtype):
    """Fused gemm on the six further types (CUDA-core variant, every dtype, small and mid M, with bias) against the oracle."""
    q = qtype_of(qtype)
    for (m, n, k) in [(1, 16, 256), (1, 1000, 1024), (3, 33, 512), (4, 64, 2048), (17, 24, 768), (64, 40, 512)]:
        # AUTO: the CUDA-core kernel, or (16-bit dtypes, 16-byte rows) the persistent GEMV up to M = 8 and the tcgen05 GEMM above
        allowed = ("simt",) if dtype == "float32" else ("simt", "stream") if m <= 8 else ("simt", "umma") if qtype in mf.UMMA_MORE_QTYPES else ("simt",)
        assert kernels.select_variant(qtype, dtype, m, n, k) in allowed
        blocks = S.random_blocks(qtype, n, k, seed=3100 + m + n)
        x, xf = _activations(m, k, 3200 + m, dtype, dev)
        bias = torch.randn(n, device=dev).to(TDT[dtype])
        ref = oracle.gemm_quant(xf, blocks, qtype, n, k) + bias.float().cpu().numpy()
        for variant in ("auto", "simt"):
            y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), qtype, bias, variant=variant)
            if variant == "auto" and kernels.select_variant(qtype, dtype, m, n, k) == "umma":
                # 16-bit weight operands: the normalised bar, and element-wise the harness metric above the operands' noise floor
                got = y.float().cpu().numpy()
                assert oracle.max_errors(ref, got)[2] <= TOL[dtype], (qtype, dtype, m, n, k)
                assert oracle.within_operand_noise(ref, got, oracle.dot_noise(xf, blocks, qtype, k), dtype, TOL[dtype]), (qtype, dtype, m, n, k)
            else:
                _check(y, ref, dtype, (qtype, dtype, variant, m, n, k))
    with pytest.raises(RuntimeError):                   # no mma.sync tile kernel for these types
        kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), qtype, variant="mma")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("qtype", ["MXFP4", "NVFP4"])
def test_fp4_scale_codes_across_their_range(dev, qtype, dtype):
    """The tensor-core paths build their operands from the scale CODES: e8m0 exponents from the subnormal codes 0 / 1 up to
    large ones; ue4m3 zero, subnormals (exponent field 0), the largest values, 0x7f (decodes to 0) and codes with the unused
    top bit set.  One class of codes per weight row, checked row by row (a whole-matrix norm would only see the large rows);
    rows whose results lie below the output type's normal range are only required to be finite."""
    q = qtype_of(qtype)
    n, k = 64, 2048
    rng = np.random.Generator(np.random.PCG64(4101))
    blocks = S.random_blocks(qtype, n, k, seed=4100).reshape(n, -1, q.block_bytes).copy()
    if qtype == "MXFP4":
        classes = [[0], [1], [2, 3], [30, 31], [90, 91], [108, 110], [117, 119, 122], [127, 128], [131, 132]]
        for r in range(n):
            blocks[r, :, 0] = rng.choice(classes[r % len(classes)], size=blocks.shape[1])
    else:
        classes = [[0x00], [1, 2, 3, 4, 5, 6, 7], [8, 9, 15], [0x30, 0x33, 0x38], [0x70, 0x77, 0x7e], [0x7f], [0x7f, 0x38], [0xb0, 0xb8, 0x80, 0xff]]
        for r in range(n):
            blocks[r, :, 0:4] = rng.choice(classes[r % len(classes)], size=(blocks.shape[1], 4))
    blocks = np.ascontiguousarray(blocks.reshape(n, -1))
    floor = 1e-30 if dtype == "bfloat16" else 1e-3
    tol = 2e-2 if dtype == "bfloat16" else 2e-3
    bq = torch.from_numpy(blocks).to(dev)
    for (m, variant) in [(3, "simt"), (3, "stream"), (1, "stream"), (8, "stream:2"), (20, "umma"), (200, "umma"), (20, "auto")]:
        xf = (S.random_activations(m, k, 4200 + m, "float32") * 0.05).astype(np.float32)
        x = torch.from_numpy(xf).to(dev).to(TDT[dtype])
        ref = oracle.gemm_quant(x.float().cpu().numpy(), blocks, qtype, n, k)
        got = kernels.gemm_rcr(x, bq, qtype, variant=variant).float().cpu().numpy()
        assert kernels.device_status() == 0
        assert np.isfinite(got).all(), (qtype, dtype, variant, m)
        checked = 0
        for r in range(n):
            top = float(np.abs(ref[:, r]).max())
            if top < floor:
                continue
            checked += 1
            err = float(np.abs(got[:, r] - ref[:, r]).max())
            assert err <= tol * top, (qtype, dtype, variant, m, r, err, top)
        assert checked >= n // 4, (qtype, dtype, variant, checked)


def _activations(m, k, seed, dtype, dev):
    x = S.random_activations(m, k, seed, "float32")
    xt = torch.from_numpy(x).to(dev).to(TDT[dtype])
    return xt, xt.float().cpu().numpy()          # device tensor and its exact float32 value


def _check(y: torch.Tensor, ref: np.ndarray, dtype: str, what):
    got = y.float().cpu().numpy()
    _, rel, norm = oracle.max_errors(ref, got)
    assert rel <= TOL[dtype] and norm <= TOL[dtype], (what, rel, norm)
    return rel, norm


SHAPES = [  # (m, n, k-blocks)
    (1, 16, 1), (1, 48, 4), (2, 33, 2), (3, 17, 3), (4, 64, 8), (5, 100, 2), (8, 40, 4), (9, 31, 1), (16, 64, 4), (17, 24, 2),
]


@pytest.mark.parametrize("qtype", QT)
@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("variant", ["simt", "auto"])
def test_gemm_small_shapes(dev, qtype, dtype, variant):
    q = qtype_of(qtype)
    for (m, n, kb) in SHAPES:
        k = kb * 256
        blocks = S.random_blocks(qtype, n, k, seed=300 + m * 7 + n)
        x, xf = _activations(m, k, 400 + m + n, dtype, dev)
        ref = oracle.gemm_quant(xf, blocks, qtype, n, k)
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), qtype, variant=variant)
        assert y.shape == (m, n) and y.dtype == TDT[dtype]
        if kernels.select_variant(qtype, dtype, m, n, k) == "umma" and variant == "auto":
            # 16-bit operand tiles (weights rounded like the reference CPU path rounds them): normalised bar only
            _, _, norm = oracle.max_errors(ref, y.float().cpu().numpy())
            assert norm <= TOL[dtype], (qtype, dtype, variant, m, n, k, norm)
        else:
            _check(y, ref, dtype, (qtype, dtype, variant, m, n, k))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_gemv_mma_q4k(dev, dtype):
    for (m, n, k) in [(1, 16, 256), (1, 1000, 1024), (2, 50, 512), (4, 128, 4096), (7, 33, 768), (8, 64, 2048),
                      (9, 48, 512), (13, 17, 1024), (16, 160, 4096)]:
        blocks = S.random_blocks("Q4_K", n, k, seed=500 + m + n)
        x, xf = _activations(m, k, 600 + m, dtype, dev)
        ref = oracle.gemm_quant(xf, blocks, "Q4_K", n, k)
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), "Q4_K", variant="mma")
        # the tensor-core path keeps integer products exact: hold it to the fp32 bar before output rounding
        got = y.float().cpu().numpy()
        _, rel, norm = oracle.max_errors(ref, got)
        bound = 4e-3 if dtype == "bfloat16" else 6e-4     # output rounding of bf16 (2^-9) / fp16 (2^-11)
        assert norm <= bound, (dtype, m, n, k, rel, norm)
        _check(y, ref, dtype, ("mma", m, n, k))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_gemv_mma_q6k(dev, dtype):
    """Q6_K decode GEMV on mma.sync: K % 2048 == 0 (16-byte rows); ragged N, every M bucket, odd and even blocks."""
    for (m, n, k) in [(1, 16, 2048), (1, 1000, 4096), (2, 50, 2048), (3, 129, 6144), (4, 128, 4096), (7, 33, 2048), (8, 64, 8192),
                      (9, 48, 2048), (13, 17, 4096), (16, 160, 4096)]:
        blocks = S.random_blocks("Q6_K", n, k, seed=520 + m + n)
        x, xf = _activations(m, k, 620 + m, dtype, dev)
        ref = oracle.gemm_quant(xf, blocks, "Q6_K", n, k)
        assert kernels.select_variant("Q6_K", dtype, m, n, k) in ("mma", "stream")      # both decode kernels serve K % 2048 == 0
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), "Q6_K", variant="mma")
        got = y.float().cpu().numpy()
        _, rel, norm = oracle.max_errors(ref, got)
        bound = 4e-3 if dtype == "bfloat16" else 6e-4     # output rounding of bf16 (2^-9) / fp16 (2^-11)
        assert norm <= bound, (dtype, m, n, k, rel, norm)
        _check(y, ref, dtype, ("mma q6k", m, n, k))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_gemv_mma_q6k_ragged_k(dev, dtype):
    """Any K % 256 == 0: weight rows of 210 * K / 256 bytes that are not 16-byte (or even 4-byte) multiples, last stage
    with fewer than 4 super-blocks, last row ending right at the end of the buffer."""
    for (m, n, k) in [(1, 16, 256), (1, 33, 768), (2, 50, 1024), (1, 100, 2816), (4, 47, 1280), (8, 64, 3328), (16, 40, 1792),
                      (1, 256, 11008), (3, 17, 4352)]:
        blocks = S.random_blocks("Q6_K", n, k, seed=540 + m + n)
        x, xf = _activations(m, k, 640 + m, dtype, dev)
        ref = oracle.gemm_quant(xf, blocks, "Q6_K", n, k)
        assert kernels.select_variant("Q6_K", dtype, m, n, k) == "mma"
        # an exact-size device buffer: the kernel must not read past the last row
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev).clone(), "Q6_K", variant="mma")
        got = y.float().cpu().numpy()
        _, rel, norm = oracle.max_errors(ref, got)
        bound = 4e-3 if dtype == "bfloat16" else 6e-4
        assert norm <= bound, (dtype, m, n, k, rel, norm)
        _check(y, ref, dtype, ("mma q6k ragged", m, n, k))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_gemv_mma_q8_0(dev, dtype):
    """Q8_0 decode GEMV on mma.sync (int8 split into two exact nibble operands): every M bucket, ragged N, whole and
    partial K stages, extreme quants (-128 / 127) included by the synthetic distribution's tails plus a forced block."""
    for (m, n, k) in [(1, 16, 256), (1, 1000, 4096), (2, 50, 512), (3, 129, 1536), (4, 128, 4096), (7, 33, 768), (8, 64, 2048),
                      (9, 48, 1280), (13, 17, 1024), (16, 160, 4096)]:
        blocks = S.random_blocks("Q8_0", n, k, seed=560 + m + n)
        blocks[0, 2:34] = np.frombuffer(np.array([-128, 127] * 16, dtype=np.int8).tobytes(), dtype=np.uint8)   # first block of row 0
        x, xf = _activations(m, k, 660 + m, dtype, dev)
        ref = oracle.gemm_quant(xf, blocks, "Q8_0", n, k)
        assert kernels.select_variant("Q8_0", dtype, m, n, k) == "mma"
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), "Q8_0", variant="mma")
        got = y.float().cpu().numpy()
        _, rel, norm = oracle.max_errors(ref, got)
        bound = 4e-3 if dtype == "bfloat16" else 6e-4     # output rounding of bf16 (2^-9) / fp16 (2^-11)
        assert norm <= bound, (dtype, m, n, k, rel, norm)
        _check(y, ref, dtype, ("mma q8_0", m, n, k))
    # K that is not a multiple of 256 stays with the simt variant
    assert kernels.select_variant("Q8_0", dtype, 1, 64, 96) == "simt"


UMMA_SHAPES = [  # (m, n, k)
    (17, 128, 256), (64, 256, 512), (100, 200, 1024), (128, 384, 768), (200, 130, 512), (256, 128, 2048),
    (300, 512, 4096), (513, 256, 1024), (150, 256, 6144),
]


def _umma_k(qtype, k):
    """The umma variant needs 16-byte weight rows: K % 2048 == 0 for Q6_K and Q3_K (210 / 110 bytes per 256 weights), K % 1024 == 0
    for Q2_K (84), K % 512 == 0 for MXFP4 (136), any K % 256 == 0 for the others."""
    step = {"Q6_K": 2048, "Q3_K": 2048, "Q2_K": 1024, "MXFP4": 512}.get(qtype, 256)
    return -(-k // step) * step


@pytest.mark.parametrize("qtype", ["Q4_K", "Q6_K", "Q8_0", "Q5_K", "Q4_0", "MXFP4", "NVFP4", "Q2_K", "Q3_K"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_gemm_umma(dev, qtype, dtype):
    """tcgen05 / TMEM prefill GEMM against the oracle (fp32 weights, fp32 accumulation)."""
    for (m, n, k) in UMMA_SHAPES:
        k = _umma_k(qtype, k)
        blocks = S.random_blocks(qtype, n, k, seed=800 + m + n)
        x, xf = _activations(m, k, 900 + m, dtype, dev)
        ref = oracle.gemm_quant(xf, blocks, qtype, n, k)
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), qtype, variant="umma")
        assert kernels.device_status() == 0, "a bounded device-side wait gave up"
        got = y.float().cpu().numpy()
        max_abs, rel, norm = oracle.max_errors(ref, got)
        # operands are 16-bit (weights rounded like the reference CPU path rounds them): the stated bars on the normalised
        # error (2e-2 bfloat16, 1e-3 float16), and element-wise the reference harness metric above the operands' noise floor
        assert norm <= TOL[dtype], (qtype, dtype, m, n, k, norm)
        noise = oracle.dot_noise(xf, blocks, qtype, k)
        assert oracle.within_operand_noise(ref, got, noise, dtype, TOL[dtype]), (qtype, dtype, m, n, k, max_abs, rel)
        # against bf16/f16-rounded weights (what the reference CPU path multiplies) the agreement is tighter
        code = {"float16": 1, "bfloat16": 2}[dtype]
        ref_r = oracle.gemm_quant(xf, blocks, qtype, n, k, round_w=code)
        _, _, norm_r = oracle.max_errors(ref_r, got)
        assert norm_r <= (8e-3 if dtype == "bfloat16" else 2e-3), (qtype, dtype, m, n, k, norm_r)


def test_gemm_umma_bias_and_auto_dispatch(dev):
    n, k, m = 256, 2048, 96
    blocks = S.random_blocks("Q6_K", n, k, seed=990)
    x, xf = _activations(m, k, 991, "bfloat16", dev)
    bias = torch.randn(n, device=dev, dtype=torch.bfloat16)
    ref = oracle.gemm_quant(xf, blocks, "Q6_K", n, k) + bias.float().cpu().numpy()
    assert kernels.select_variant("Q6_K", "bfloat16", m, n, k) == "umma"
    y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), "Q6_K", bias)
    _, _, norm = oracle.max_errors(ref, y.float().cpu().numpy())
    assert norm <= 2e-2, norm
    assert kernels.device_status() == 0
    # Q6_K rows that are not 16-byte multiples are outside the umma variant: dispatch avoids it, asking for it fails
    assert kernels.select_variant("Q6_K", "bfloat16", m, n, 1024) == "simt"
    with pytest.raises(RuntimeError, match="alignment"):
        kernels.gemm_rcr(x[:, :1024].contiguous(), torch.from_numpy(S.random_blocks("Q6_K", n, 1024, seed=1)).to(dev), "Q6_K",
                         variant="umma")


def test_gemm_umma_on_two_streams_at_once(dev):
    """Each stream has its own partial-tile workspace and flags: launches that overlap on the GPU do not disturb each
    other (shapes whose tiles are cut between SMs, so the workspace is really used)."""
    cases = [("Q4_K", 96, 256, 4096), ("Q6_K", 40, 384, 8192)]
    work = []
    for i, (qtype, m, n, k) in enumerate(cases):
        w = torch.from_numpy(S.random_blocks(qtype, n, k, seed=1200 + i)).to(dev)
        x, _ = _activations(m, k, 1300 + i, "bfloat16", dev)
        want = kernels.gemm_rcr(x, w, qtype, variant="umma")
        work.append((qtype, w, x, want, torch.cuda.Stream(), [torch.empty_like(want) for _ in range(8)]))
    torch.cuda.synchronize()
    for it in range(8):
        for (qtype, w, x, want, stream, outs) in work:
            with torch.cuda.stream(stream):
                kernels.gemm_rcr(x, w, qtype, variant="umma", out=outs[it])
    torch.cuda.synchronize()
    assert kernels.device_status() == 0
    for (qtype, w, x, want, stream, outs) in work:
        for o in outs:
            assert torch.equal(o.view(torch.int16), want.view(torch.int16)), qtype


@pytest.mark.parametrize("qtype", ["Q4_K", "Q6_K"])
@pytest.mark.parametrize("activation", ["silu", "fast_gelu"])
def test_dual_gemm_gated_epilogue(dev, qtype, activation):
    """act(a B0^T) * (a B1^T) in one launch on row-interleaved weights, mma GEMV (plain and cluster-sliced shapes) and
    tcgen05 kernel (whole tiles and tiles finished after a stream-K reduction), against the oracle."""
    k = 2048
    for (m, n) in [(1, 8), (1, 104), (2, 64), (4, 200), (8, 48), (16, 64), (16, 2048), (40, 136), (300, 264)]:
        b0 = S.random_blocks(qtype, n, k, seed=1400 + n)
        b1 = S.random_blocks(qtype, n, k, seed=1500 + n)
        x, xf = _activations(m, k, 1600 + m, "bfloat16", dev)
        ref = oracle.dual_gemm_quant(xf, b0, b1, qtype, n, k, activation)
        w = kernels.interleave_rows8(torch.from_numpy(b0).to(dev), torch.from_numpy(b1).to(dev))
        assert np.array_equal(w.cpu().numpy(), kernels.interleave_rows8(b0, b1))
        y = kernels.dual_gemm_rcr(x, w, qtype, activation)
        assert y.shape == (m, n) and kernels.device_status() == 0
        _, _, norm = oracle.max_errors(ref, y.float().cpu().numpy())
        assert norm <= 2e-2, (qtype, activation, m, n, norm)
        # the same numbers as two plain launches combined in fp32 (bf16 rounding of the intermediates aside)
        if m <= 8:
            g = kernels.gemm_rcr(x, torch.from_numpy(b0).to(dev), qtype, variant="mma").float()
            u = kernels.gemm_rcr(x, torch.from_numpy(b1).to(dev), qtype, variant="mma").float()
            two = (torch.nn.functional.silu(g) if activation == "silu" else torch.nn.functional.gelu(g, approximate="tanh")) * u
            assert float((two - y.float()).abs().max()) <= 3e-2 * float(two.abs().max())
    with pytest.raises(ValueError):
        kernels.dual_gemm_rcr(x, w[:-8], qtype, activation)             # 2N must be a multiple of 16
    with pytest.raises(RuntimeError):
        kernels.dual_gemm_rcr(x.float(), w, qtype, activation)         # fp32 activations have no tensor-core variant


@pytest.mark.parametrize("qtype", ["Q4_K", "Q6_K", "Q8_0", "Q5_K", "Q4_0", "MXFP4", "NVFP4", "Q2_K", "Q3_K"])
@pytest.mark.parametrize("activation", ["silu", "fast_gelu"])
def test_dual_gemm_bias_and_b1_broadcast(dev, qtype, activation):
    """The reference's _bias_ forms and its B1 [1, K] broadcast: act(a B0^T + bias0) * (a B1^T + bias1) on every kernel that has
    the gated epilogue (persistent GEMV, tile GEMV, tcgen05 kernel), against the oracle."""
    k = 2048
    rng = np.random.Generator(np.random.PCG64(77))
    for (m, n) in [(1, 104), (4, 200), (8, 48), (16, 64), (40, 136), (300, 264)]:
        for b1_rows in (n, 1):
            b0 = S.random_blocks(qtype, n, k, seed=2400 + n)
            b1 = S.random_blocks(qtype, b1_rows, k, seed=2500 + n)
            bias0 = rng.standard_normal(n).astype(np.float32)
            bias1 = rng.standard_normal(b1_rows).astype(np.float32)
            x, xf = _activations(m, k, 2600 + m, "bfloat16", dev)
            bias0_t, bias1_t = (torch.from_numpy(v).to(dev).to(torch.bfloat16) for v in (bias0, bias1))
            ref = oracle.dual_gemm_quant(xf, b0, b1, qtype, n, k, activation, bias0_t.float().cpu().numpy(), bias1_t.float().cpu().numpy())
            w = kernels.interleave_rows8(torch.from_numpy(b0).to(dev), torch.from_numpy(b1).to(dev))
            bias = kernels.interleave_bias8(bias0_t, bias1_t)
            assert w.shape[0] == 2 * n and bias.numel() == 2 * n
            variants = ["auto"] + [v for v in ("stream", "mma", "umma") if mf.variant_supports(v, m, qtype=qtype, dtype="bfloat16", n=2 * n, k=k)
                                   and not (qtype == "Q8_0" and v == "mma")]
            for variant in variants:
                y = kernels.dual_gemm_rcr(x, w, qtype, activation, bias01_interleaved=bias, variant=variant)
                assert y.shape == (m, n) and kernels.device_status() == 0
                _, _, norm = oracle.max_errors(ref, y.float().cpu().numpy())
                assert norm <= 2e-2, (qtype, activation, variant, m, n, b1_rows, norm)
    with pytest.raises(ValueError):
        kernels.dual_gemm_rcr(x, w, qtype, activation, bias01_interleaved=bias[:-1])


def test_dual_gemm_q8_0_runs_on_the_tcgen05_kernel_only(dev):
    """Q8_0 has the gated epilogue on the tcgen05 kernel only; AUTO sends every M there (the activation tile is zero-filled past M)."""
    k = 1024
    for (m, n) in [(1, 64), (4, 136), (9, 64), (16, 2048), (40, 136), (300, 264)]:
        b0 = S.random_blocks("Q8_0", n, k, seed=1700 + n)
        b1 = S.random_blocks("Q8_0", n, k, seed=1800 + n)
        x, xf = _activations(m, k, 1900 + m, "bfloat16", dev)
        ref = oracle.dual_gemm_quant(xf, b0, b1, "Q8_0", n, k, "silu")
        w = kernels.interleave_rows8(torch.from_numpy(b0).to(dev), torch.from_numpy(b1).to(dev))
        y = kernels.dual_gemm_rcr(x, w, "Q8_0", "silu")
        assert y.shape == (m, n) and kernels.device_status() == 0
        _, _, norm = oracle.max_errors(ref, y.float().cpu().numpy())
        assert norm <= 2e-2, (m, n, norm)
    with pytest.raises(RuntimeError):
        kernels.dual_gemm_rcr(x[:4].contiguous(), w, "Q8_0", "silu", variant="mma")       # its tile GEMV has no gated epilogue


def test_gemm_bias_and_batch_dims(dev):
    n, k = 48, 512
    blocks = S.random_blocks("Q4_K", n, k, seed=700)
    x = torch.randn(2, 3, k, device=dev, dtype=torch.bfloat16)
    bias = torch.randn(n, device=dev, dtype=torch.bfloat16)
    ref = oracle.gemm_quant(x.float().cpu().numpy().reshape(6, k), blocks, "Q4_K", n, k) + bias.float().cpu().numpy()
    for variant in ("simt", "mma"):
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), "Q4_K", bias, variant=variant)
        assert y.shape == (2, 3, n)
        _check(y.reshape(6, n), ref, "bfloat16", variant)


def test_gemm_matches_reference_cpu_artifact_outputs(dev, golden_dir):
    """Same seeded inputs the reference's CPU artifact was run on (fixtures made by tests/golden/make_golden.py).

    For 16-bit dtypes the reference CPU path first rounds the dequantized weights to the storage dtype
    (src/dinoml/constant_sources.py:72) and both sides round the output, the fused kernels keep the weights in
    fp32: an element may land on the neighbouring 16-bit output value.  Bars: normalised max error <= TOL; element
    wise, float32 within 1e-3 (reference metric), 16-bit within two output ulps plus the weight-rounding noise floor."""
    g = np.load(golden_dir / "gemm_rcr_reference_cpu.npz")
    for i, case in enumerate(g["cases"]):
        qtype, dtype, m, n, k = str(case).split("|")
        m, n, k = int(m), int(n), int(k)
        x = torch.from_numpy(g[f"case{i}_x_f32"]).to(dev).to(TDT[dtype])
        y = kernels.gemm_rcr(x, torch.from_numpy(g[f"case{i}_blocks"]).to(dev), qtype)
        ref = np.asarray(g[f"case{i}_y"], dtype=np.float32)
        got = y.float().cpu().numpy()
        max_abs, rel, norm = oracle.max_errors(ref, got)
        assert norm <= TOL[dtype], (i, qtype, dtype, norm)
        if dtype == "float32":
            assert rel <= 1e-3, (i, rel)
        else:
            # noise of rounding each weight to the storage dtype grows like sqrt(K); the constants are ~2x what the
            # CPU oracle (fp32 weights) itself shows against these fixtures
            ulp, floor = (2.0 ** -8, 0.015 * k ** 0.5) if dtype == "bfloat16" else (2.0 ** -11, 0.001 * k ** 0.5)
            assert np.all(np.abs(got - ref) <= 2 * ulp * np.abs(ref) + floor), (i, qtype, dtype, max_abs, rel)


def test_gemv_full_size_config2(dev):
    """Config 2 (Q4_K 11008x4096, bf16, M in {1,4,16}) against the oracle on the full output."""
    n, k = 11008, 4096
    blocks = S.random_blocks("Q4_K", n, k, seed=2000)
    bq = torch.from_numpy(blocks).to(dev)
    for m in (1, 4, 16):
        x, xf = _activations(m, k, 2001 + m, "bfloat16", dev)
        ref = oracle.gemm_quant(xf, blocks, "Q4_K", n, k)
        for variant in ("mma", "simt"):
            y = kernels.gemm_rcr(x, bq, "Q4_K", variant=variant)
            _check(y, ref, "bfloat16", (variant, m))
    # linearity (size-independent property): f(x1 + x2) == f(x1) + f(x2) within rounding, float16 to keep sums exact-ish
    x1 = torch.randn(1, k, device=dev, dtype=torch.float32)
    x2 = torch.randn(1, k, device=dev, dtype=torch.float32)
    f = lambda t: kernels.gemm_rcr(t, bq, "Q4_K", variant="simt").double()
    lhs, rhs = f(x1 + x2), f(x1) + f(x2)
    assert float((lhs - rhs).abs().max() / rhs.abs().max()) < 1e-5


def test_error_paths(dev):
    blocks = torch.from_numpy(S.random_blocks("Q4_K", 16, 256, seed=1)).to(dev)
    x = torch.randn(1, 256, device=dev, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        kernels.gemm_rcr(x.cpu(), blocks, "Q4_K")
    with pytest.raises(ValueError):
        kernels.gemm_rcr(x[:, :128].contiguous(), blocks, "Q4_K")
    with pytest.raises(RuntimeError, match="shape outside"):
        kernels.gemm_rcr(torch.randn(17, 256, device=dev, dtype=torch.bfloat16), blocks, "Q4_K", variant="mma")
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        kernels.gemm_rcr(x.float(), blocks, "Q4_K", variant="mma")


def test_umma_refuses_k_that_is_not_a_multiple_of_256(dev):
    """Q8_0 only needs K % 32 == 0, but the tcgen05 kernel walks whole 256-weight super-blocks: asking for it explicitly with
    K = 288 or 896 is refused (alignment code), not computed wrongly; so are the per-candidate symbol and the allocation-free
    entry; the profiler's predicate says the same, and AUTO serves the shape on another variant."""
    import ctypes

    from dinoml_v2_b200 import _native, manifest as mf
    lib = _native.lib()
    for k in (288, 896):
        m, n = 32, 64
        bq = torch.from_numpy(S.random_blocks("Q8_0", n, k, seed=k)).to(dev)
        x, xf = _activations(m, k, k + 1, "bfloat16", dev)
        with pytest.raises(RuntimeError, match="alignment"):
            kernels.gemm_rcr(x, bq, "Q8_0", variant="umma")
        y = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        sym = _native.candidate_symbol("q8_0", "bfloat16", "umma")
        assert sym(x.data_ptr(), bq.data_ptr(), y.data_ptr(), m, n, k, None) == 7
        lib.dinoml_b200_gguf_gemm_rcr_prealloc.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 5 + [ctypes.c_void_p]
        assert lib.dinoml_b200_gguf_gemm_rcr_prealloc(x.data_ptr(), bq.data_ptr(), None, y.data_ptr(), 8, 6, m, n, k, None) == 7
        assert not mf.variant_supports("umma", m, qtype="Q8_0", dtype="bfloat16", n=n, k=k)
        assert kernels.select_variant("Q8_0", "bfloat16", m, n, k) == "simt"
        got = kernels.gemm_rcr(x, bq, "Q8_0")
        _check(got, oracle.gemm_quant(xf, bq.cpu().numpy(), "Q8_0", n, k), "bfloat16", ("auto", k))
