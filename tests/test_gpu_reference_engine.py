"""The reference's own engine (scheduler, block manager, model runner, attention, sampler: the
staged, unmodified copy under oracle/_ref/reference_python) generating with this library's MoE
layer installed by ``install_into_reference()``: a two-layer random-init Mixtral on one GPU, and
the same model split tensor-parallel over two GPUs where the box has them.  The full-size
configuration (32 layers, 100 requests) is a measurement, not a test: ``oracle/reference_engine.py``.
Skipped where the reference's Python package was never staged."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("tp", [1, 2])
def test_reference_engine_generates_with_this_layer(tp):
    if not (REPO / "oracle" / "_ref" / "reference_python" / "electrock_infer").is_dir():
        pytest.skip("the reference's Python package is not staged under oracle/_ref")
    if torch.cuda.device_count() < tp:
        pytest.skip(f"needs {tp} GPUs")
    proc = subprocess.run(
        [sys.executable, str(REPO / "oracle" / "reference_engine.py"), "--tp", str(tp), "--layers", "2",
         "--requests", "6", "--max-input", "300", "--max-output", "24", "--min-len", "12",
         "--gpu-memory-utilization", "0.3"],
        capture_output=True, text=True, timeout=900)
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert proc.returncode == 0 and lines, (proc.stdout[-500:], proc.stderr[-1500:])
    res = json.loads(lines[-1])
    assert "failed" not in res, res
    assert res["moe_layer"] == "electrock_infer_b200.FusedMoE" and res["tensor_parallel"] == tp
    # Two layers, one FusedMoE.forward per layer and engine step; every request got its tokens.
    assert res["output_tokens"] > 0 and res["moe_forward_calls"] >= 2 * 12
    assert res["moe_forward_calls"] % 2 == 0 and res["output_tokens_per_s"] > 0
