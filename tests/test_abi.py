"""The C ABI library loads without a GPU and exports every function include/msx.h declares."""
import os
import re

import modelspec_b200 as M

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "msx.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(msx_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_function_is_exported_and_bound():
    names = declared_functions()
    assert len(names) >= 40
    L = M.lib()
    for name in names:
        assert hasattr(L, name), "%s is declared in include/msx.h but not exported" % name
        assert name in M.SIGNATURES, "%s has no ctypes signature" % name


def test_no_device_is_a_status_not_a_crash():
    try:
        d = M.Device(99)
    except M.MsxError as e:
        assert e.status == M.NO_DEVICE
    else:
        d.close()
        raise AssertionError("device 99 opened")


def test_null_handles_are_bad_arguments():
    L = M.lib()
    assert L.msx_run(None) == M.BAD_ARGUMENT
    assert L.msx_plan_input_count(None) == 0
    assert L.msx_set_input(None, b"x", None, 0) == M.BAD_ARGUMENT
    assert L.msx_training_steps(None) == 0
