"""Packed routed-expert forward backend.

Presents the same three names as ``bitsmoe.algorithms`` (bitsmoe/algorithms/__init__.py:28-46):
``mlp_forward_cuda`` (an object with ``moe_packed_forward``), ``_HAS_MLP_FORWARD_CUDA`` and
``_MLP_FORWARD_BACKEND``.  The op is served by the sm_100a library through the C ABI; when the
library is absent the flag is False, the object is None and the blocks raise at forward, as the
reference does (bitsmoe/models/base_block.py:428-438).
"""
from __future__ import annotations

import torch


def get_cuda_device_name() -> str:
    if not torch.cuda.is_available():
        return "cpu"
    p = torch.cuda.get_device_properties(torch.cuda.current_device())
    return f"{p.name.strip()} ({round(p.total_memory / 1024 ** 3)}GB)"


try:
    from bitsmoe_b200 import capi as _capi
    _capi.lib()
    from bitsmoe_b200.algorithms import _mlp_forward as mlp_forward_cuda

    _HAS_MLP_FORWARD_CUDA = True
    _MLP_FORWARD_BACKEND = get_cuda_device_name()
except Exception:  # library not built
    mlp_forward_cuda = None
    _HAS_MLP_FORWARD_CUDA = False
    _MLP_FORWARD_BACKEND = "None"

__all__ = ["mlp_forward_cuda", "_HAS_MLP_FORWARD_CUDA", "_MLP_FORWARD_BACKEND", "get_cuda_device_name"]
