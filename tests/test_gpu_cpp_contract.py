"""Runs the C++ contract test binary (tests/cpp/contract_test.cpp) on the GPU."""
import os
import subprocess

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(REPO, "tests", "_build", "contract_test")


@pytest.mark.gpu
def test_cpp_contract_binary():
    assert os.path.exists(BINARY), "run __graft_entry__.build() first"
    r = subprocess.run([BINARY], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:]
    assert "ALL PASS" in r.stdout


def test_cpp_contract_binary_fails_loudly_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    if not os.path.exists(BINARY):
        pytest.skip("binary not built")
    r = subprocess.run([BINARY], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=60)
    assert r.returncode == 77 and "no CPU fallback" in r.stdout
