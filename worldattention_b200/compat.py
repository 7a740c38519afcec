"""Make the reference's import paths resolve to this package.

After `install_reference_aliases()`:

    from wan.modules.hsa import HSAAttention            -> worldattention_b200.hsa
    from wan.modules.hsa.routing import ...             -> worldattention_b200.hsa.routing
    from pipeline.hkv import HKVCache                   -> worldattention_b200.hkv
    from trainer.hsa_stage import init_hsa_parameters   -> worldattention_b200.hsa_stage

Parent packages (`wan`, `wan.modules`, `pipeline`, `trainer`) that are not importable are created
as empty namespace modules; parents that already exist are left alone and only gain the
sub-module attribute.
"""
from __future__ import annotations

import importlib
import sys
import types

_ALIASES = {
    "wan.modules.hsa": "worldattention_b200.hsa",
    "wan.modules.hsa.attention": "worldattention_b200.hsa.attention",
    "wan.modules.hsa.routing": "worldattention_b200.hsa.routing",
    "wan.modules.hsa.distill": "worldattention_b200.hsa.distill",
    "wan.modules.hsa.block_sparse_torch": "worldattention_b200.hsa.block_sparse_torch",
    "wan.modules.hsa.block_sparse_triton": "worldattention_b200.hsa.block_sparse_triton",
    "pipeline.hkv": "worldattention_b200.hkv",
    "pipeline.hkv.cache": "worldattention_b200.hkv.cache",
    "pipeline.hkv.retrieval": "worldattention_b200.hkv.retrieval",
    "pipeline.hkv.rope": "worldattention_b200.hkv.rope",
    "pipeline.hkv.tiering": "worldattention_b200.hkv.tiering",
    "trainer.hsa_stage": "worldattention_b200.hsa_stage",
}


def _ensure_parent(name: str) -> types.ModuleType:
    if name in sys.modules:
        return sys.modules[name]
    module = types.ModuleType(name)
    module.__path__ = []  # namespace-like: sub-modules come from sys.modules
    sys.modules[name] = module
    if "." in name:
        parent, _, leaf = name.rpartition(".")
        setattr(_ensure_parent(parent), leaf, module)
    return module


def install_reference_aliases() -> None:
    for alias, target in _ALIASES.items():
        module = importlib.import_module(target)
        sys.modules[alias] = module
        parent, _, leaf = alias.rpartition(".")
        setattr(_ensure_parent(parent), leaf, module)
