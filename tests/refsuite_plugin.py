"""pytest plugin for running the REFERENCE project's own test files against this package.

Loaded with `-p tests.refsuite_plugin` by tests/test_reference_suite_gpu.py (in a child process): the
reference's import paths (`wan.modules.hsa`, `pipeline.hkv`, `trainer.hsa_stage`) are aliased onto
`worldattention_b200` before any test module is imported, and the default device becomes CUDA, so the
tensors and modules those tests create without naming a device land on the GPU, where the kernels run
(`WA_REFSUITE_DEVICE=cpu` keeps the default device for test files that are about host memory).
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from worldattention_b200 import compat  # noqa: E402

compat.install_reference_aliases()
torch.set_default_device(os.environ.get("WA_REFSUITE_DEVICE", "cuda"))
