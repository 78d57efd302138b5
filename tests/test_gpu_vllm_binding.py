"""The reader bound into the installed vLLM: a two-layer model of the Qwen3-30B-A3B layer
shape decodes with the stock blocks and with the readers, in a child process (the engine
keeps its memory pool until the process ends)."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_two_layer_decode_study():
    pytest.importorskip("vllm")
    env = dict(os.environ, VLLM_LOGGING_LEVEL="WARNING", PYTHONPATH=str(ROOT))
    run = subprocess.run(
        [sys.executable, "-m", "cfm_b200.runtime.vllm_binding", "--layers", "2", "--batch", "4",
         "--prompt-tokens", "64", "--decode-tokens", "8", "--memory-fraction", "0.2"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=900,
    )
    assert run.returncode == 0, run.stderr[-3000:]
    report = json.loads([line for line in run.stdout.splitlines() if line.startswith("{")][-1])
    # every decode row of every step went through the reader: 7 decode steps of 4 rows
    assert report["decode_steps"] == 7
    assert report["sparse_rows_per_layer"] == 4 * 7
    assert report["tokens_forced_to_stock"] is True
    assert report["prefill_step_kl"] == 0.0  # the prefill step runs the stock blocks
    assert 0.0 <= report["kl_stock_to_sparse_mean"] < 0.05
    assert 0.0 < report["read_fraction_layer0"] < 0.5
