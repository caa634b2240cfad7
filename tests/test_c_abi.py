"""The shared library loads, exports every function include/etb200_sampler.h declares, and
refuses to work without a GPU instead of falling back to anything."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "etb200_sampler.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(etb200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_bindings_agree():
    from executorch_b200 import _lib
    names = declared_functions()
    assert len(names) >= 10
    assert sorted(_lib.SYMBOLS) == names


def test_library_exports_every_declared_symbol():
    from executorch_b200 import _lib
    from executorch_b200.build import build
    build()
    lib = _lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert lib.etb200_sampler_abi_version() == 1


def test_header_cites_the_reference_interface():
    text = open(HEADER).read()
    for cite in ("sampler.h:37-83", "sampler.cpp:173-181", "sampler.cpp:183-187", "sampler.h:48-53",
                 "sampler.h:58-60", "sampler.cpp:222-251", "util.h:25-55", "error.h:29-100",
                 "scalar_type.h:98-125"):
        assert cite in text, cite


def test_argument_checks_do_not_need_a_device():
    from executorch_b200 import _lib
    lib = _lib.load()
    assert lib.etb200_sampler_create(100, 0.5, 0.9, 1, 0, None) == _lib.INVALID_ARGUMENT
    h = C.c_void_p()
    assert lib.etb200_sampler_create(0, 0.5, 0.9, 1, 0, C.byref(h)) == _lib.INVALID_ARGUMENT
    assert lib.etb200_sampler_set_temperature(None, 0.5) == _lib.INVALID_ARGUMENT
    assert lib.etb200_sampler_sample_rows(None, None, 6, 1, 0, None, None, None) == _lib.INVALID_ARGUMENT
    assert b"null" in lib.etb200_last_error_message()
    assert lib.etb200_sampler_destroy(None) == _lib.OK


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_gpu_means_an_error_not_a_fallback():
    from executorch_b200 import _lib
    lib = _lib.load()
    h = C.c_void_p()
    code = lib.etb200_sampler_create(100, 0.5, 0.9, 1, 0, C.byref(h))
    assert code == _lib.INTERNAL and not h.value
    assert b"no CPU path" in lib.etb200_last_error_message()
    from executorch_b200 import Sampler
    with pytest.raises(RuntimeError):
        Sampler(100, 0.5, 0.9, 1)


def test_product_code_never_touches_the_oracle():
    """The oracle is a checker: nothing in the package may import, load or link it."""
    pkg = os.path.join(ROOT, "executorch_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in src and "from oracle" not in src, f
                assert "liboracle" not in src and "libref_sampler" not in src, f
