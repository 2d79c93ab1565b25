"""There is no CPU execution path: everything that would run the model says so at once (no GPU needed)."""

import subprocess
import sys
from pathlib import Path

import pytest
import torch

import ondeviceinfer_b200 as odi
import plain_qwen3 as plain
from helpers import write_model_folder
from ondeviceinfer_b200.kernels import ops

ROOT = Path(__file__).resolve().parent.parent


def test_loading_a_model_onto_the_cpu_is_refused(tmp_path):
    folder = write_model_folder(tmp_path / "model", plain.TINY_A, plain.random_weights(plain.TINY_A, 0))
    with pytest.raises(RuntimeError, match="no CPU path"):
        odi.load_resident_model(folder, device="cpu", dtype="float32")


def test_kernels_refuse_host_tensors():
    x = torch.zeros(2, 8)
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.rmsnorm(x, torch.ones(8), 1e-6, torch.empty(2, 8))


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a GPU")
def test_the_programs_say_that_they_need_a_gpu(tmp_path):
    folder = write_model_folder(tmp_path / "model", plain.TINY_A, plain.random_weights(plain.TINY_A, 0))
    replay = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                             "--out", str(tmp_path / "out"), "--max-tokens", "64"], input="", text=True,
                            capture_output=True, timeout=300)
    assert replay.returncode != 0 and "no CUDA device" in replay.stderr
    generate = subprocess.run([sys.executable, "-m", "ondeviceinfer_b200", "generate", "--model", str(folder),
                               "--prompt-ids", "1,2,3", "--max-new-tokens", "2"], cwd=ROOT, text=True,
                              capture_output=True, timeout=300)
    assert generate.returncode != 0 and "CUDA is required" in generate.stderr
