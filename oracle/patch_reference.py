"""Applies the call-site change this library asks of a cccc maintainer to a COPY of the reference's
cccc/cublas_real.h, so that the claim "Cublas::gemm lands in cuda_gemm_wq_bf16" is compiled and run,
not only described.

    python oracle/patch_reference.py <reference root> <output dir>

writes <output dir>/cublas_real.h: the reference's file with (1) an include of cccc_cuda_b200.h and
(2) one inserted block in front of each of the two W8A16 / W4A16 BF16 branches of Cublas::gemm (weight
as A, cccc/cublas_real.h:943; weight as B, :1066).  Everything else is the reference's text, untouched.
The output is a build product for oracle/_ref/ (git-ignored); nothing of the reference enters the
repository.  Test infrastructure only.
"""
from __future__ import annotations

import os
import sys

INCLUDE_ANCHOR = '#include "cuda_functions.h"\n'

WEIGHT_IS_A = '''            // ---- cccc-cuda-b200: the fused W8A16 / W4A16 linear, weight as A ----
            if (typeB == DataType::BFLOAT16 && typeC == DataType::BFLOAT16
                && TransA == MATRIX_TRANS && TransB == MATRIX_NO_TRANS && cuda_gemm_wq_bf16)
            {
                if (cuda_gemm_wq_bf16((int)typeA, A, blk_scA, invScaleA, B, C,
                        /*N_out*/ M, /*M_tokens*/ N, K, /*ldw*/ lda, /*ldx*/ ldb, /*ldy_m*/ ldc, /*ldy_n*/ 1,
                        alpha, beta, /*stream*/ nullptr, /*flags*/ 0) == 0)
                {
                    cuda_check_error("gemm_wq_bf16");
                    return;
                }
            }
'''

WEIGHT_IS_B = '''            // ---- cccc-cuda-b200: the fused W8A16 / W4A16 linear, weight as B ----
            if (typeA == DataType::BFLOAT16 && typeC == DataType::BFLOAT16
                && TransA == MATRIX_TRANS && TransB == MATRIX_NO_TRANS && cuda_gemm_wq_bf16)
            {
                if (cuda_gemm_wq_bf16((int)typeB, B, blk_scB, invScaleB, A, C,
                        /*N_out*/ N, /*M_tokens*/ M, K, /*ldw*/ ldb, /*ldx*/ lda, /*ldy_m*/ 1, /*ldy_n*/ ldc,
                        alpha, beta, nullptr, 0) == 0)
                {
                    cuda_check_error("gemm_wq_bf16");
                    return;
                }
            }
'''

# (text that identifies the branch body, the `if` line that opens the branch, the block to put in front of it)
SITES = [
    ("                int szA = lda * (TransA == MATRIX_NO_TRANS ? K : M);\n                ensureWS(&ws_A_, &ws_A_cap_, (size_t)szA * sizeof(bfloat16));",
     "            if (typeB == DataType::BFLOAT16 && typeC == DataType::BFLOAT16)\n", WEIGHT_IS_A),
    ("                ensureWS(&ws_A_, &ws_A_cap_, (size_t)szB2 * sizeof(bfloat16));",
     "            if (typeA == DataType::BFLOAT16 && typeC == DataType::BFLOAT16)\n", WEIGHT_IS_B),
]


def patch(text: str) -> str:
    if text.count(INCLUDE_ANCHOR) != 1:
        raise SystemExit("patch_reference: the include anchor is not unique in cublas_real.h")
    text = text.replace(INCLUDE_ANCHOR, INCLUDE_ANCHOR + '#include "cccc_cuda_b200.h"\n')
    for body, opener, block in SITES:
        if text.count(body) != 1:
            raise SystemExit(f"patch_reference: branch body not found exactly once: {body}")
        at = text.rfind(opener, 0, text.index(body))
        if at < 0:
            raise SystemExit(f"patch_reference: branch opener not found before: {body}")
        text = text[:at] + block + text[at:]
    return text


def main() -> None:
    ref, out = sys.argv[1], sys.argv[2]
    with open(os.path.join(ref, "cccc", "cublas_real.h"), encoding="utf-8") as f:
        src = f.read()
    os.makedirs(out, exist_ok=True)
    with open(os.path.join(out, "cublas_real.h"), "w", encoding="utf-8") as f:
        f.write(patch(src))


if __name__ == "__main__":
    main()
