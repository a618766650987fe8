"""CPU-only checks of the boundary: both libraries load, every function declared in include/onemodel_b200.h is
exported, and creating a context without a GPU fails loudly (there is no CPU path)."""
import ctypes
import os
import re

import pytest

import om_binding as omb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "onemodel_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bint32_t\s+(om_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert len(names) > 60 and "om_linear_bwd" in names and "om_optim_adam_step" in names


def test_every_declared_symbol_is_exported():
    lib = omb.kernel_lib()
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_host_library_loads():
    host = omb.host_lib()
    for n in ("omh_init", "omh_call", "omh_backward", "omh_optim_step", "omh_trainer_create", "omh_trainer_step"):
        assert hasattr(host, n), n


def test_no_cpu_path():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(omb.OmError) as e:
        omb.Context(0, 0)
    assert "no CPU path" in str(e.value)


def test_product_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "onemodel-csharp_b200")
    for dirpath, _, files in os.walk(pkg):
        if "build" in dirpath:
            continue
        for f in files:
            if f.endswith((".cu", ".cuh", ".cpp", ".hpp", ".py", "Makefile")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "oracle" not in text.lower() or f == "om_binding.py" and "oracle" not in text.lower(), os.path.join(dirpath, f)
