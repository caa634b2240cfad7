"""The C++ face (include/etb200_sampler.hpp) and the pybind11 module built from it."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "executorch_b200", "lib")

PROGRAM = r"""
#include <cstdio>
#include "etb200_sampler.hpp"
using executorch_b200::Error;
using executorch_b200::ScalarType;
using executorch_b200::ScalarTypeOf;
using executorch_b200::extension::llm::Sampler;
int main() {
  static_assert(static_cast<int>(ScalarTypeOf<float>::value) == 6, "Float");
  static_assert(static_cast<int>(ScalarTypeOf<executorch_b200::Half>::value) == 5, "Half");
  static_assert(static_cast<int>(ScalarTypeOf<executorch_b200::BFloat16>::value) == 15, "BFloat16");
  static_assert(static_cast<int>(ScalarTypeOf<uint16_t>::value) == 27, "UInt16");
  static_assert(executorch_b200::extension::llm::kTopp == 0.9f, "kTopp");
  Sampler four(32000, 0.8f, 0.9f, 42ull);   // the reference's 4-argument constructor
  Sampler two(32000, 0.8f);                 // and its 2-argument one
  Sampler moved(std::move(two));
  moved.set_temperature(-1.0f);
  moved.set_topk(40);
  Sampler bad(0, 0.8f, 0.9f, 1ull);
  std::printf("%u %u %u\n", (unsigned)four.status(), (unsigned)moved.status(), (unsigned)bad.status());
  return 0;
}
"""


def test_cpp_header_compiles_links_and_reports_status():
    from executorch_b200.build import build
    build()
    d = tempfile.mkdtemp(prefix="etb200_cpp_")
    src, exe = os.path.join(d, "t.cpp"), os.path.join(d, "t")
    open(src, "w").write(PROGRAM)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"), src,
                    "-L" + LIBDIR, "-letb200_sampler", "-Wl,-rpath," + LIBDIR, "-o", exe], check=True)
    out = subprocess.run([exe], check=True, capture_output=True, text=True).stdout.split()
    four, moved, bad = (int(v) for v in out)
    assert bad == 0x12  # InvalidArgument: vocab_size 0
    if torch.cuda.is_available():
        assert four == 0 and moved == 0
    else:
        assert four == 0x01 and moved == 0x01  # Internal: no device, and no CPU path to fall back to


def test_pybind_module_builds_and_raises_like_the_runner_bindings():
    from executorch_b200.build import build, build_pybind
    build()
    build_pybind()
    sys.path.insert(0, LIBDIR)
    try:
        import _sampler_pybind as m
    finally:
        sys.path.remove(LIBDIR)
    assert abs(m.kTopp - 0.9) < 1e-7
    with pytest.raises(RuntimeError):
        m.Sampler(0, 0.5, 0.9, 1)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU path"):
            m.Sampler(100, 0.5, 0.9, 1)
