"""Drop-in proof: the reference's unmodified C++ front end (aix::Tensor, autograd, nn::Sequential, optim::Adam) running
on aix::DeviceB200 - the adapter a maintainer would add (aix_b200/adapter/aixDeviceB200.hpp) - against the same
program on aix::DeviceCPU. The binary is built from the reference headers by oracle/build_ref.py."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
BINARY = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "adapter_check")


def test_reference_front_end_runs_on_the_b200_device():
    if not os.path.isfile(BINARY):
        pytest.skip("oracle/_ref/adapter_check not built (reference headers absent)")
    run = subprocess.run([BINARY], capture_output=True, text=True, timeout=600)
    print(run.stdout, run.stderr)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "ALL OK" in run.stdout and "B200" in run.stdout
