"""The entry point where there is no GPU: it says so, with the reference's error
code for a failure that is not the caller's, and does nothing else."""
import subprocess
import sys
import os

import pytest
import torch

from helpers import model_dir

pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="a CUDA device is there")


def test_open_without_a_device_fails_loudly():
    import janas_b200
    with pytest.raises(janas_b200.LLMError) as e:
        janas_b200.open(model_dir("A"))
    assert e.value.code == janas_b200.EFAIL and "CUDA" in str(e.value)
    with pytest.raises(janas_b200.LLMError) as e:
        janas_b200.open("/nonexistent/model")
    assert e.value.code == janas_b200.EOPEN or e.value.code == janas_b200.EFAIL


def test_cli_without_a_device_says_so():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "janas-b200"), model_dir("A"),
                        "--tokens", "1 2 3", "--max", "2"], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 2 and r.stdout == ""
    assert "needs a CUDA device" in r.stderr and "Traceback" not in r.stderr
