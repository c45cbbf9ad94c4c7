"""There is no CPU fallback: without a CUDA device the engine, the replay program and the kernel wrappers
refuse loudly instead of computing something slowly or wrongly."""
import os
import subprocess
import sys

import pytest
import torch

from tiny_configs import TINY, make_folder

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
no_gpu = pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a CUDA device")


@no_gpu
def test_engine_refuses_without_cuda(tmp_path):
    from qwen_decoder_b200.config import Qwen2Config
    from qwen_decoder_b200.engine import Engine, ModelRunner
    folder = make_folder("A", str(tmp_path))
    with pytest.raises(RuntimeError, match="no CPU path"):
        ModelRunner.from_folder(folder, dtype="float32", num_pages=4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine(config=Qwen2Config.from_dict(TINY["A"]), random_seed=0, num_pages=4)


@no_gpu
def test_trace_run_exits_with_an_error_without_cuda(tmp_path):
    folder = make_folder("A", str(tmp_path))
    step = '{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [2]}], "end": []}\n'
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(tmp_path / "out"), "--max-tokens", "64"], input=step, capture_output=True, text=True)
    assert p.returncode != 0 and "no CPU path" in p.stderr and "done 0" not in p.stdout


def test_kernel_wrappers_refuse_cpu_tensors():
    from qwen_decoder_b200 import kernels
    x = torch.zeros(2, 8)
    with pytest.raises(kernels.KernelError, match="CUDA"):
        kernels._ptr(x)
    from qwen_decoder_b200.parts import matmul_backend
    with pytest.raises(kernels.KernelError, match="no CPU path"):
        matmul_backend.linear(x, torch.zeros(4, 8), None, torch.zeros(2, 4))
