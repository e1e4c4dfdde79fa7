"""Runs the C++ operator layer's own test programs (nano-vllm-cpp_b200/host/tests/*.cpp).

``test_host_cpu`` needs no GPU: tensor views, the step context, the metadata builders against the arrays the
reference's tests expect, the KV-cache plan.  ``test_host_gpu`` repeats the reference's known-answer cases through
the ``Attention`` layer and the operator wrappers on a B200.
"""
import os
import subprocess

import pytest

from util import ROOT, entry

BUILD_DIR = os.path.join(ROOT, "nano-vllm-cpp_b200", "build")


def _run(name):
    entry.build()
    exe = os.path.join(BUILD_DIR, name)
    assert os.path.exists(exe), f"{exe} was not built"
    return subprocess.run([exe], capture_output=True, text=True, timeout=300)


def test_host_logic_without_a_gpu():
    res = _run("test_host_cpu")
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout


@pytest.mark.gpu
def test_operator_layer_known_answers_on_gpu():
    res = _run("test_host_gpu")
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout
