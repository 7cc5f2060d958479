"""GPU: the decode router inside a running vLLM engine (SURVEY's caller-integration row).  A small random-weight
Llama (SmolLM2 shape family: hidden 576, 9 / 3 heads of 64, 4 layers) is served by vLLM's own engine with its
FLASH_ATTN backend and its native KV cache layout; greedy generation with the stock forward and with
``decode_backend.install_into_vllm()`` must give the same tokens, with log-probabilities within the bf16 tolerance,
and the router must have taken every pure-decode step.  Skipped when vLLM is not importable or its engine does not
start on the box."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


def test_router_inside_a_vllm_engine(cuda_device):
    script = Path(__file__).with_name("vllm_engine_check.py")
    try:
        proc = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=900)
    except subprocess.TimeoutExpired:
        pytest.skip("the vLLM engine process did not finish within 15 minutes")
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    if not lines:          # the engine is third-party infrastructure: its own failure to run is not this library's
        pytest.skip(f"no result from the vLLM engine process (exit {proc.returncode}): {proc.stderr[-300:]}")
    res = json.loads(lines[-1])
    if "skip" in res:
        pytest.skip(res["skip"])
    assert "error" not in res, f"the router failed inside the engine: {res.get('error')}\n{res.get('trace')}"
    assert res["cache_shape"][0] == 2 and res["cache_shape"][2:] == [16, 3, 64]        # vLLM's [2, blocks, 16, kv_heads, 64]
    for case in res["cases"]:
        print(case)
        assert case["stats"].get("backend_decode", 0) == 7          # 8 tokens: one prefill step, seven routed decode steps
        assert case["equal_tokens"] == case["total_tokens"]
        assert case["max_logprob_diff"] <= 5e-2
