"""The drop-in translation unit (executorch_b200/csrc/reference_sampler_dropin.cpp) built
inside the reference's own header tree: the reference's unmodified sampler.h, util.h and
portable Tensor, with the B200 sampler behind `executorch::extension::llm::Sampler`. The
check program (oracle/dropin_check.cpp) is compiled by oracle/Makefile where the reference
checkout is at hand and travels with the tree; here it is run on the GPU. It replays the
fixtures of the reference's own tests (argmax 396, {0.1, 0.2, 0.8, 0.4} -> 2 in three dtypes,
rank-3 last position, injected sampler with set_temperature / set_topk) with device-resident
logits, and the batched tensor entry point."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "oracle", "_ref", "dropin_check")


def test_reference_headers_with_the_dropin_sampler(cuda_device):
    if not os.path.exists(BINARY):
        pytest.skip("oracle/_ref/dropin_check has not been built (needs the reference checkout: "
                    "make -f oracle/Makefile ref REF=<checkout>)")
    res = subprocess.run([BINARY], capture_output=True, text=True, timeout=300)
    print(res.stdout)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = res.stdout.strip().splitlines()
    assert lines[-1] == "ALL PASS"
    assert sum(1 for ln in lines if ln.startswith("PASS")) >= 14
    assert not any(ln.startswith("FAIL") for ln in lines)
