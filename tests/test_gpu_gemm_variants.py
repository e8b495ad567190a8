"""The tensor-core matmul has switches that select its fallback and experimental paths (single-CTA kernel, 2-D TMA boxes,
row-per-thread epilogue, remainder wave shared along K, the TF32 + bf16 form of the f32 product, tiles dealt out at run time,
products launched by their own call). They are read once per process, so each variant runs in a child
process on the same parity shapes (ragged M/N/K, transposed operands, bf16 and f32)."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

VARIANTS = {
    "default": {},
    "single_cta": {"AIXB200_GEMM_PAIR": "0"},
    "boxes_2d": {"AIXB200_GEMM_BOX3D": "0"},
    "direct_epilogue": {"AIXB200_GEMM_TMA_STORE": "0"},
    "shared_remainder_wave": {"AIXB200_GEMM_SPLITK": "1"},
    "narrow_tiles": {"AIXB200_GEMM_BLOCKN": "128"},
    "f32_tf32_hybrid": {"AIXB200_GEMM_F32": "hybrid"},
    "tiles_dealt_at_run_time": {"AIXB200_GEMM_DYNAMIC": "1"},
    "no_folded_epilogue": {"AIXB200_GEMM_EPILOGUE": "0"},
}


@pytest.mark.parametrize("variant", list(VARIANTS), ids=list(VARIANTS))
def test_matmul_parity_under_switch(variant):
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_gemm_variant_worker.py")
    env = dict(os.environ, **VARIANTS[variant])
    out = subprocess.run([sys.executable, worker], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    result = json.loads(out.stdout.strip().splitlines()[-1])
    assert result["repeatable"], "two runs of the same product differ"
    assert result["worst"]["bf16"] <= 1e-2, result          # bf16 result rounding dominates (2^-9)
    assert result["worst"]["f32"] <= 1e-5, result
