"""The reference's own Python front-end and its two acceptance scripts, unmodified, executed on
the GPU against this library.

`make -C oracle frontend` copies ilang-python/{ilang.py, flash-attn.py, test.py} from the reference
checkout into baseline/_ref/ilang-python/ (git-ignored).  Each script runs in a child process with
ILANG_CORE_LIB pointing at i_b200/lib/libi_core.so, which is how the reference selects its core
library (ilang-python/ilang.py:6-9); nothing of this repository's Python is on the child's path.
"""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FRONT = os.path.join(ROOT, "baseline", "_ref", "ilang-python")


def run_script(ilang, name):
    path = os.path.join(FRONT, name)
    if not os.path.exists(path):
        pytest.fail("%s is missing: run `make -C oracle frontend` where the reference checkout is present" % path)
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    env["ILANG_CORE_LIB"] = ilang.DEFAULT_LIB
    return subprocess.run([sys.executable, name], cwd=FRONT, env=env, capture_output=True, text=True,
                          timeout=600)


def test_reference_flash_attention_demo_passes_its_own_tolerance(ilang):
    # flash-attn.py:31-77: fused and naive schedules of a 32 x 32 x 2048 attention against NumPy,
    # rtol 3e-4 / atol 5e-5, asserted by the script itself.
    out = run_script(ilang, "flash-attn.py")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "FlashAttention output matches NumPy reference" in out.stdout
    assert "Naive Attention output matches NumPy reference" in out.stdout


def test_reference_test_script_cases(ilang):
    # test.py:130-150 runs six cases and prints ok / fail per case.  Its `mlp` case fails in the
    # reference itself: it builds the component with `@`, an operator ilang.py does not define
    # (test.py:93-98), so the script exits non-zero there too.  Every other case must pass.
    out = run_script(ilang, "test.py")
    text = re.sub(r"\x1b\[[0-9;]*m", "", out.stdout)
    results = {name: verdict for verdict, name in re.findall(r"^(ok|fail): (\w+)", text, re.M)}
    assert set(results) == {"matmul", "attention", "mlp", "rowmax", "rowmin", "rowaccum"}, out.stdout + out.stderr
    for name in ("matmul", "attention", "rowmax", "rowmin", "rowaccum"):
        assert results[name] == "ok", text
