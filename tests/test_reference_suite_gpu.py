"""The reference's OWN test files, run unmodified against this package on the GPU.

The files come from `baseline/_ref/tests` (staged from a reference checkout by
`oracle/stage_reference.py`; never committed).  They run in a child pytest process with the reference's
import paths aliased onto `worldattention_b200` and the default device set to CUDA
(`tests/refsuite_plugin.py`).  Every forward-only test must pass.  Left out, by name:
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, "baseline", "_ref", "tests")

# Training is outside what this package replaces: the CUDA forward builds no autograd graph.
EXCLUDED = {
    "test_hsa_attention.py::test_gradients_reach_the_hsa_parameters": "backward through the HSA forward",
    "test_hsa_attention.py::test_a_saturated_gate_starves_the_gate_gradient": "backward through the HSA forward",
    "test_hsa_attention.py::test_distillation_records_one_loss_per_forward": "distillation losses carry gradients",
    "test_training_stage.py": "training-stage helpers (trainable sets, distillation collection)",
}
__doc__ += "".join(f"\n  {name}: {why}" for name, why in EXCLUDED.items())


def test_forward_only_reference_tests_pass_against_the_drop_in():
    if not os.path.isdir(STAGED):
        pytest.skip("baseline/_ref is not staged (run `python oracle/stage_reference.py` where a reference checkout exists)")
    cmd = [sys.executable, "-m", "pytest", "-p", "tests.refsuite_plugin", "-q", "--no-header", "-p", "no:cacheprovider",
           STAGED]
    for name in EXCLUDED:
        flag = "--deselect" if "::" in name else "--ignore"
        cmd += [flag, os.path.join(STAGED, name)]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    tail = (res.stdout + res.stderr)[-6000:]
    log_dir = os.environ.get("WA_TEST_LOG_DIR")
    if log_dir:
        os.makedirs(log_dir, exist_ok=True)
        with open(os.path.join(log_dir, "reference_suite.log"), "w") as f:
            f.write(res.stdout + res.stderr)
    assert res.returncode == 0, tail
    assert " passed" in res.stdout and "failed" not in res.stdout, tail
    passed = int(res.stdout.rsplit(" passed", 1)[0].split()[-1])
    assert passed >= 60, tail     # 79 tests in the suite, 16 of them left out above
