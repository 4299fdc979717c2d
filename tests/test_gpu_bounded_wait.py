"""A bounded wait that runs out, in the form that leaves the GPU alone: a test-only kernel
(tests/csrc/bounded_wait_probe.cu, compiled here, not part of the package) calls the package's
``kl::mbar_wait`` with a short limit on a barrier nobody arrives at.  The device's status word
must take the code and ``ops.check_status`` / ``ops.check_device_words`` must raise and clear it."""
from __future__ import annotations

import ctypes
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    from kuiperllama_b200.csrc import build
    out = str(tmp_path_factory.mktemp("probe") / "bounded_wait_probe.so")
    cmd = [build.find_nvcc()] + build.NVCC_FLAGS + ["-I", build.CSRC, "-o", out, os.path.join(HERE, "csrc", "bounded_wait_probe.cu")]
    done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert done.returncode == 0, done.stdout
    return ctypes.CDLL(out)


def test_a_wait_that_runs_out_sets_the_status_word_and_the_host_raises(probe):
    from kuiperllama_b200.csrc import ops
    dev = torch.device("cuda:0")
    ops.check_device_words(dev)                                   # clean before
    status = ops.status_word(dev)
    result = torch.full((3,), -1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for where, check in ((2, ops.check_status), (3, ops.check_device_words)):
        rc = probe.kl_test_bounded_wait(ctypes.c_void_p(status.data_ptr()), where, ctypes.c_void_p(result.data_ptr()), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert result.tolist() == [0, 1, 0]                       # gave up, raised the flag; the second wait stopped at once
        assert int(status.item()) == where                        # the first code stays
        with pytest.raises(ops.KernelError, match=f"code {where}"):
            check(dev)
        assert int(status.item()) == 0                            # raised once and cleared
        check(dev)
    # the context is as usable as before
    x = torch.arange(8, device=dev, dtype=torch.float32)
    assert float(x.sum()) == 28.0
