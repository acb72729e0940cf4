"""The C++ operator classes (SdpaOp, PagedAttentionOp, KvBlockManager, registry) through their own test program."""
import subprocess

import pytest

from openvino_contrib_b200.build import build_host_tests


def _run(args):
    exe = build_host_tests()
    r = subprocess.run([exe, *args], capture_output=True, text=True, timeout=600)
    print(r.stdout[-4000:], r.stderr[-2000:])
    return r


def test_registry_and_block_manager_cpu():
    r = _run(["--cpu"])
    assert r.returncode == 0, r.stdout
    assert "0 failed" in r.stdout


@pytest.mark.gpu
def test_operators_on_gpu():
    r = _run([])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failed" in r.stdout and "test_paged_op_decode_with_block_manager" in r.stdout
