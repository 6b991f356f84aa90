"""No GPU needed: the C-ABI library loads and exports every symbol the header declares."""
import os
import re

from tests._util import capi
from __graft_entry__ import ROOT


def test_library_loads_and_exports_header_symbols():
    c = capi()
    L = c.lib()
    header = open(os.path.join(ROOT, "include", "cccc_cuda_b200.h")).read()
    declared = set(re.findall(r"C_EXPORT\s+[\w\s\*]+?\b(cuda_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(c.SYMBOLS), declared ^ set(c.SYMBOLS)
    for name in declared:
        assert getattr(L, name) is not None
    assert "sm_100a" in c.version()


def test_plan_needs_no_gpu():
    c = capi()
    # aligned decode shapes -> GEMV kernel; misaligned -> plain kernel
    assert c.gemm_wq_bf16_plan(c.FP8_E5M2, 0x1000, None, 0x2000, 0x3000, 4096, 1, 4096) == c.PLAN_DECODE
    assert c.gemm_wq_bf16_plan(c.FP8_E5M2, 0x1001, None, 0x2000, 0x3000, 4096, 1, 4096) == c.PLAN_PLAIN
    assert c.gemm_wq_bf16_plan(c.FP8_E5M2, 0x1000, None, 0x2000, 0x3000, 4096, 1, 4100) == c.PLAN_PLAIN
    assert c.gemm_wq_bf16_plan(c.FP4_E2M1, 0x1000, 0x4000, 0x2000, 0x3000, 4096, 8, 4096) == c.PLAN_DECODE
    assert c.gemm_wq_bf16_plan(c.FP4_E2M1, 0x1000, None, 0x2000, 0x3000, 4096, 8, 4096) == c.PLAN_PLAIN
    assert c.gemm_wq_bf16_plan(3, 0x1000, None, 0x2000, 0x3000, 4096, 8, 4096) == -1


def test_host_layer_library_loads():
    from __graft_entry__ import load_package

    h = load_package().hostapi
    L = h.lib()
    for name in h.SYMBOLS:
        assert getattr(L, name) is not None
