"""Seeded synthetic GGUF weights with the value distributions of the benchmark configs.

No real `.gguf` checkpoint is needed: every generator packs independently drawn
quantized fields into the exact GGUF block bytes, so the tensors have the shapes,
sizes and per-field distributions of the Llama-shaped configurations:

* Q8_0: ``d = fp16(|N(0,1)| * 0.01)``, ``qs ~ U{-127..127}``
* Q4_K: ``d, dmin = fp16(|N(0,1)| * 0.005)``, 8 sub-block scales and 8 mins ``~ U{0..63}``
  packed into the 12 scale bytes (inverse of the 6-bit unpack in
  kernels/rocm/src/ck_gguf_q8_gemm.hip:143-155), nibbles ``~ U{0..15}``
* Q6_K: 6-bit quants ``~ U{0..63}`` split into ``ql``/``qh`` per the index map of
  kernels/rocm/src/ck_gguf_q8_gemm.hip:924-938, ``scales ~ U{-64..63}``,
  ``d = fp16(|N(0,1)| * 0.002)``

* Q4_0, Q5_K, Q2_K, Q3_K, MXFP4, NVFP4 (not in the benchmark configurations): every packed field uniform random bytes, as
  the reference's bench tool fills them (tools/bench_ck_gguf_q8_gemm.hip:2191-2345), fp16 scales ``fp16(|N(0,1)| * c)``,
  the MXFP4 exponent byte ``~ U{117..122}`` and the NVFP4 ue4m3 scale bytes ``~ U{32..48}`` (the tool's ranges)

`pack_*` take explicit field arrays (used by tests for edge cases), `random_*`
draw them from ``numpy.random.Generator(PCG64(seed))``.  `random_blocks_torch`
produces the same distributions directly on a CUDA device for multi-GB cases.
"""
from __future__ import annotations

import numpy as np

from .gguf_blocks import Q4_K, Q6_K, Q8_0, qtype_of, row_bytes

D_SCALE = {"Q8_0": 0.01, "Q4_K": 0.005, "Q6_K": 0.002, "Q4_0": 0.01, "Q5_K": 0.003, "Q2_K": 0.005, "Q3_K": 0.005}
# byte offsets of the fp16 scale fields (d, then dmin where the layout has one) inside a block of the further types
_HALF_FIELDS = {"Q4_0": (0,), "Q5_K": (0, 2), "Q2_K": (80, 82), "Q3_K": (108,)}


def _rng(seed) -> np.random.Generator:
    return seed if isinstance(seed, np.random.Generator) else np.random.Generator(np.random.PCG64(seed))


def _half_scale(rng: np.random.Generator, shape, scale: float) -> np.ndarray:
    return (np.abs(rng.standard_normal(shape, dtype=np.float32)) * np.float32(scale)).astype(np.float16)


# ----------------------------------------------------------------------------- packers
def pack_q8_0(d: np.ndarray, qs: np.ndarray) -> np.ndarray:
    """d: float16 [...]; qs: int8 [..., 32] -> uint8 [..., 34]."""
    d = np.asarray(d, dtype=np.float16)
    qs = np.asarray(qs, dtype=np.int8)
    out = np.empty(d.shape + (34,), dtype=np.uint8)
    out[..., 0:2] = d[..., None].view(np.uint8)
    out[..., 2:34] = qs.view(np.uint8)
    return out


def pack_k4_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """8 six-bit scales + 8 six-bit mins [..., 8] -> the 12 packed bytes [..., 12]."""
    sc = np.asarray(sc, dtype=np.uint8)
    mn = np.asarray(mn, dtype=np.uint8)
    q = np.empty(sc.shape[:-1] + (12,), dtype=np.uint8)
    q[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    q[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    q[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((mn[..., 4:8] & 0x0F) << 4)
    return q


def pack_q4_k(d, dmin, sc, mn, q) -> np.ndarray:
    """d,dmin float16 [...]; sc,mn uint8 [...,8] (0..63); q uint8 [...,256] (0..15) -> uint8 [...,144]."""
    d = np.asarray(d, dtype=np.float16)
    dmin = np.asarray(dmin, dtype=np.float16)
    q = np.asarray(q, dtype=np.uint8)
    out = np.empty(d.shape + (144,), dtype=np.uint8)
    out[..., 0:2] = d[..., None].view(np.uint8)
    out[..., 2:4] = dmin[..., None].view(np.uint8)
    out[..., 4:16] = pack_k4_scales(sc, mn)
    g = q.reshape(q.shape[:-1] + (4, 2, 32))           # [group64, nibble half, 32]
    out[..., 16:144] = ((g[..., 0, :] & 0x0F) | (g[..., 1, :] << 4)).reshape(q.shape[:-1] + (128,))
    return out


def pack_q6_k(d, scales, q) -> np.ndarray:
    """d float16 [...]; scales int8 [...,16]; q uint8 [...,256] (0..63) -> uint8 [...,210]."""
    d = np.asarray(d, dtype=np.float16)
    scales = np.asarray(scales, dtype=np.int8)
    q = np.asarray(q, dtype=np.uint8)
    out = np.empty(d.shape + (210,), dtype=np.uint8)
    v = q.reshape(q.shape[:-1] + (2, 4, 32))            # [half_block, quad, l]
    lo, hi = v & 0x0F, v >> 4
    ql = np.empty(q.shape[:-1] + (2, 2, 32), dtype=np.uint8)
    ql[..., 0, :] = lo[..., 0, :] | (lo[..., 2, :] << 4)   # quads 0 / 2 share bytes 0..31
    ql[..., 1, :] = lo[..., 1, :] | (lo[..., 3, :] << 4)   # quads 1 / 3 share bytes 32..63
    qh = hi[..., 0, :] | (hi[..., 1, :] << 2) | (hi[..., 2, :] << 4) | (hi[..., 3, :] << 6)
    out[..., 0:128] = ql.reshape(q.shape[:-1] + (128,))
    out[..., 128:192] = qh.reshape(q.shape[:-1] + (64,))
    out[..., 192:208] = scales.view(np.uint8)
    out[..., 208:210] = d[..., None].view(np.uint8)
    return out


# ----------------------------------------------------------------------------- random tensors
def random_blocks(qtype, rows: int, n_per_row: int, seed) -> np.ndarray:
    """uint8 [rows, row_bytes] of GGUF blocks drawn from the benchmark distributions."""
    q = qtype_of(qtype)
    rng = _rng(seed)
    nb = n_per_row // q.block_size
    rb = row_bytes(q, n_per_row)
    shape = (rows, nb)
    if q is Q8_0:
        blocks = pack_q8_0(_half_scale(rng, shape, D_SCALE["Q8_0"]),
                           rng.integers(-127, 128, size=shape + (32,), dtype=np.int8))
    elif q is Q4_K:
        blocks = pack_q4_k(_half_scale(rng, shape, D_SCALE["Q4_K"]), _half_scale(rng, shape, D_SCALE["Q4_K"]),
                           rng.integers(0, 64, size=shape + (8,), dtype=np.uint8),
                           rng.integers(0, 64, size=shape + (8,), dtype=np.uint8),
                           rng.integers(0, 16, size=shape + (256,), dtype=np.uint8))
    elif q is Q6_K:
        blocks = pack_q6_k(_half_scale(rng, shape, D_SCALE["Q6_K"]),
                           rng.integers(-64, 64, size=shape + (16,), dtype=np.int8),
                           rng.integers(0, 64, size=shape + (256,), dtype=np.uint8))
    else:
        blocks = rng.integers(0, 256, size=shape + (q.block_bytes,), dtype=np.uint8)
        if q.name == "MXFP4":
            blocks[..., 0] = rng.integers(117, 123, size=shape, dtype=np.uint8)
        elif q.name == "NVFP4":
            blocks[..., 0:4] = rng.integers(32, 49, size=shape + (4,), dtype=np.uint8)
        else:
            for off in _HALF_FIELDS[q.name]:
                blocks[..., off:off + 2] = _half_scale(rng, shape, D_SCALE[q.name])[..., None].view(np.uint8)
    return np.ascontiguousarray(blocks.reshape(rows, rb))


def random_activations(m: int, k: int, seed, dtype: str = "bfloat16") -> np.ndarray:
    """N(0,1) activations.  float32 -> float32 array; bfloat16 -> uint16 storage (RNE); float16 -> float16."""
    x = _rng(seed).standard_normal((m, k), dtype=np.float32)
    if dtype == "float32":
        return x
    if dtype == "float16":
        return x.astype(np.float16)
    if dtype == "bfloat16":
        return float32_to_bf16_bits(x)
    raise ValueError(dtype)


def float32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 storage, as src/dinoml/ir.py:68-73."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    return ((bits + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_float32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def random_blocks_torch(qtype, rows: int, n_per_row: int, seed: int, device):
    """Same per-field distributions as `random_blocks`, generated on `device` by torch.

    For these layouts uniform quantized fields are exactly uniform packed bytes
    (the 12 Q4_K scale bytes are a bijection of sixteen 6-bit values; ql/qh are a
    bijection of 256 six-bit values), so only d/dmin and the Q6_K int8 scales need
    shaping.  Returns a uint8 tensor [rows, row_bytes].
    """
    import torch

    q = qtype_of(qtype)
    nb = n_per_row // q.block_size
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    blocks = torch.randint(0, 256, (rows, nb, q.block_bytes), dtype=torch.uint8, device=device, generator=g)

    def half_bytes(scale):
        d = (torch.randn((rows, nb), device=device, generator=g).abs() * scale).to(torch.float16)
        return d.view(torch.uint8).reshape(rows, nb, 2)

    if q is Q8_0:
        blocks[..., 0:2] = half_bytes(D_SCALE["Q8_0"])
        qs = blocks[..., 2:34]
        qs[qs == 128] = 129                      # -128 is outside U{-127..127}
    elif q is Q4_K:
        blocks[..., 0:2] = half_bytes(D_SCALE["Q4_K"])
        blocks[..., 2:4] = half_bytes(D_SCALE["Q4_K"])
    elif q.name == "MXFP4":
        blocks[..., 0] = torch.randint(117, 123, (rows, nb), dtype=torch.uint8, device=device, generator=g)
    elif q.name == "NVFP4":
        blocks[..., 0:4] = torch.randint(32, 49, (rows, nb, 4), dtype=torch.uint8, device=device, generator=g)
    elif q.name in _HALF_FIELDS:
        for off in _HALF_FIELDS[q.name]:
            blocks[..., off:off + 2] = half_bytes(D_SCALE[q.name])
    else:
        sc = torch.randint(-64, 64, (rows, nb, 16), dtype=torch.int8, device=device, generator=g)
        blocks[..., 192:208] = sc.view(torch.uint8)
        blocks[..., 208:210] = half_bytes(D_SCALE["Q6_K"])
    return blocks.reshape(rows, nb * q.block_bytes).contiguous()
