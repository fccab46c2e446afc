"""The C++ host mirror of the reference interface (ml-drift_b200/host) builds and its own test
program passes: CPU-only checks here, the device checks under -m gpu."""
import importlib.util
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build():
    spec = importlib.util.spec_from_file_location("mld_build", os.path.join(ROOT, "ml-drift_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build_host_test()


def test_host_mirror_cpu_checks():
    exe = _build()
    out = subprocess.run([exe, "--cpu"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "PASSED" in out.stdout


@pytest.mark.gpu
def test_host_mirror_device_checks():
    exe = os.path.join(ROOT, "ml-drift_b200", "build", "host_test")
    if not os.path.exists(exe):
        exe = _build()
    fixture = os.path.join(ROOT, "tests", "golden", "loader_fixture", "int4_block32") + os.sep
    out = subprocess.run([exe, "--fixture", fixture], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "PASSED" in out.stdout and "file loader" in out.stdout
