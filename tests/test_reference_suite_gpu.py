"""The reference's OWN test files, run unmodified against this package on the GPU.

The files come from `baseline/_ref/tests` (staged from a reference checkout by
`oracle/stage_reference.py`; never committed).  They run in child pytest processes with the reference's
import paths aliased onto `worldattention_b200` (`tests/refsuite_plugin.py`) and, except for the file
that is about host memory, with the default device set to CUDA, so that the tensors those tests create
land where the kernels run.  Every forward-only test must pass.  Left out, by name:
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join("baseline", "_ref", "tests")

EXCLUDED = {
    # training is outside what this package replaces: the CUDA forward builds no autograd graph
    "test_hsa_attention.py::test_gradients_reach_the_hsa_parameters": "backward through the HSA forward",
    "test_hsa_attention.py::test_a_saturated_gate_starves_the_gate_gradient": "backward through the HSA forward",
    "test_hsa_attention.py::test_distillation_records_one_loss_per_forward": "distillation losses carry gradients",
    "test_training_stage.py": "training-stage helpers (trainable sets, distillation collection)",
    # not runnable under a CUDA default device by ANY implementation, the reference's included: the test re-rotates a
    # chunk fetched from the host tier (a CPU tensor, `store` moves chunks to the host) and compares it with the device cache
    "test_hkv_cache.py::test_apply_reropes_keys_to_their_new_positions": "compares a host-tier tensor with a device tensor",
}
ON_HOST = ["test_hkv_tiering.py"]      # the tier manager's own tests: host tensors by design ("CPU only" in their header)
__doc__ += "".join(f"\n  {name}: {why}" for name, why in EXCLUDED.items())


def _run(files, device, extra):
    cmd = [sys.executable, "-m", "pytest", "-p", "tests.refsuite_plugin", "-q", "--no-header", "-p", "no:cacheprovider", *files, *extra]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), WA_REFSUITE_DEVICE=device)
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    log_dir = os.environ.get("WA_TEST_LOG_DIR")
    if log_dir:
        os.makedirs(log_dir, exist_ok=True)
        with open(os.path.join(log_dir, f"reference_suite_{device}.log"), "w") as f:
            f.write(res.stdout + res.stderr)
    tail = (res.stdout + res.stderr)[-6000:]
    assert res.returncode == 0, tail
    assert " passed" in res.stdout and "failed" not in res.stdout, tail
    return int(res.stdout.rsplit(" passed", 1)[0].split()[-1])


def test_forward_only_reference_tests_pass_against_the_drop_in():
    if not os.path.isdir(os.path.join(ROOT, STAGED)):
        pytest.skip("baseline/_ref is not staged (run `python oracle/stage_reference.py` where a reference checkout exists)")
    extra = []
    for name in list(EXCLUDED) + ON_HOST:
        extra += ["--deselect" if "::" in name else "--ignore", os.path.join(STAGED, name)]
    on_device = _run([STAGED], "cuda", extra)
    on_host = _run([os.path.join(STAGED, name) for name in ON_HOST], "cpu", [])
    # 79 tests in the reference's suite: 12 training-stage + 4 named above are left out
    assert on_device + on_host == 79 - 12 - 4, (on_device, on_host)
