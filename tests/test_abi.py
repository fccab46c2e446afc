"""The C-ABI library builds, loads and exports every symbol the header declares.
No compute is called here (there is no GPU on the CPU test box)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def mld():
    import __graft_entry__ as g
    g.build()
    return g.import_package()


def _declared():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", fn)).read()
        names += re.findall(r"MLD_API\s+[^;(]*?\b(mld_\w+)\s*\(", text)
    return names


def test_header_declares_entry_points():
    names = _declared()
    for must in ("mld_pack_weights", "mld_pack_scales", "mld_fc_plan_create", "mld_fc_run",
                 "mld_fc_plan_destroy", "mld_packed_size_bytes", "mld_status_string"):
        assert must in names


def test_library_exports_every_declared_symbol(mld):
    lib = mld.binding.lib()
    for name in _declared():
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_library_exports_nothing_the_header_does_not_declare(mld):
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", mld.binding.LIB_PATH], capture_output=True, text=True, check=True)
    exported = {ln.split()[-1] for ln in out.stdout.splitlines() if " T " in ln}
    assert exported == set(_declared()), exported ^ set(_declared())


def test_status_strings_and_sizes(mld):
    lib = mld.binding.lib()
    assert lib.mld_status_string(0) == b"OK"
    assert lib.mld_status_string(2) == b"UNIMPLEMENTED"
    # GetTotalElementsCountForLayout (weights_conversion.cc:1015-1027)
    assert mld.packed_size_bytes(533, 171, 8) == 536 * 172
    assert mld.packed_size_bytes(533, 171, 4) == 536 * 172 // 2
    assert mld.packed_size_bytes(16, 8, 4, h=2, group=2) == 16 * 8 * 2 // 2


def test_argument_errors_do_not_need_a_gpu(mld):
    lib = mld.binding.lib()
    d = mld.binding.PackDesc(4, 1, 1, 4, 5, 0, 0, 0, 8)       # bits = 5
    assert lib.mld_pack_weights(ctypes.byref(d), None, None, None, 0, None) == mld.INVALID_ARGUMENT
    assert b"bits" in lib.mld_last_error()
    assert lib.mld_fc_plan_create(None, None) == mld.INVALID_ARGUMENT
    assert lib.mld_fc_is_gemv_recommended(mld.F16, 16) == 1    # fully_connected.cc:981-1011
    assert lib.mld_fc_is_gemv_recommended(mld.F16, 17) == 0
    assert lib.mld_fc_is_gemv_recommended(mld.F32F16, 8) == 1
    assert lib.mld_fc_is_gemv_recommended(mld.F32, 9) == 0


def test_no_oracle_in_product():
    """The shipped package must not reach into oracle/."""
    pkg = os.path.join(ROOT, "ml-drift_b200")
    for base, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h", ".cc", ".cpp")):
                text = open(os.path.join(base, fn), errors="ignore").read()
                assert "oracle" not in text.lower(), f"{fn} mentions the oracle"
