"""Guards the code generation of the kernels the headline numbers are measured on: `ptxas -v` figures recorded by
`python -m dinoml_v2_b200.build` (build/ptxas_<source>.log).  A source change far away from the inner loop has flipped the
register allocation of the decode GEMV before (78 registers -> 48 with spills, 10 % slower); this catches that at build
time, without a GPU."""
import re
from pathlib import Path

import pytest

BUILD = Path(__file__).resolve().parents[1] / "dinoml_v2_b200" / "build"
ENTRY = re.compile(r"Compiling entry function '(\S+)'.*?\n.*?\n\s*(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads\n"
                   r"ptxas info\s*: Used (\d+) registers")

# (log, mangled-name fragment, threads per CTA, CTAs per SM the launch configuration counts on, spill bytes tolerated)
HOT = [
    ("ptxas_gemv_mma.log", "gemv_q4k_mma_kernelI13__nv_bfloat16Li1ELi8ELi4ELb0ELb0E", 256, 3, 0),        # BASELINE config 2, M = 1
    ("ptxas_gemv_q6k_mma.log", "gemv_q6k_mma_kernelI13__nv_bfloat16Li1ELi8ELi6ELb0ELb0ELb0E", 256, 2, 0),
    ("ptxas_gemv_stream.log", "gemv_stream_kernelILi12E13__nv_bfloat16Li1ELi1ELi4ELb0E", 320, 2, 0),      # persistent GEMV, Q4_K, configuration 4
    ("ptxas_gemv_stream.log", "gemv_stream_kernelILi14E13__nv_bfloat16Li1ELi1ELi3ELb0E", 320, 2, 0),      # persistent GEMV, Q6_K
    ("ptxas_umma_gemm_q6_k.log", "gemm_umma_kernelILi14E13__nv_bfloat16Li256ELb0E", 608, 1, 64),                # BASELINE config 3, M = 512
    ("ptxas_umma_gemm_q4_k.log", "gemm_umma_kernelILi12E13__nv_bfloat16Li64ELb0E", 608, 1, 64),
]


def _entries(log: Path) -> dict:
    return {m.group(1): (int(m.group(5)), int(m.group(3)), int(m.group(4))) for m in ENTRY.finditer(log.read_text())}


@pytest.mark.parametrize("log,fragment,threads,ctas_per_sm,spill_ok", HOT)
def test_hot_kernels_keep_their_registers(log, fragment, threads, ctas_per_sm, spill_ok):
    path = BUILD / log
    if not path.exists():
        pytest.skip("no ptxas log: the library was not built in this tree")
    hits = {k: v for k, v in _entries(path).items() if fragment in k}
    assert hits, f"{fragment} not found in {log}"
    for name, (regs, spill_st, spill_ld) in hits.items():
        assert spill_st <= spill_ok and spill_ld <= spill_ok, (name, regs, spill_st, spill_ld)   # the tcgen05 GEMM sits at its 96-register cap: a few spilled words in the epilogue
        assert regs * threads * ctas_per_sm <= 65536, (name, regs)
        assert regs >= 56, (name, regs)        # a much smaller count means ptxas traded registers for local memory or occupancy heuristics
