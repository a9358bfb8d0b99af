"""``torch.ops.anemoi_sm100.*``: the library's entry points registered as torch operators, the way
the reference registers its own (``TORCH_LIBRARY_FRAGMENT`` in
csrc/attention/cuda/sm120/bindings.cpp:9-237).  ``load()`` builds the small host-side shim if
needed (``csrc/torch_ops.cpp``, linked against the C-ABI library) and loads it; after that

    torch.ops.anemoi_sm100.draft_probability(q_pool, k_pool, None, None, 0.0, 128)
    torch.ops.anemoi_sm100.route(probability, n16, n8, n4, prefix_phase, query_block, prefix_tokens, head_dim)
    torch.ops.anemoi_sm100.qknorm_rope_(x, weight, cos, sin, eps)

call the same kernels as the ctypes layer in ``native.py``.  The Python package itself keeps
using ctypes: the operators exist for hosts that want the torch dispatcher in between (operator
tracing, ``torch.library`` tooling).
"""

from __future__ import annotations

import torch

_LOADED = False


def load() -> None:
    global _LOADED
    if _LOADED:
        return
    from .build import build_torch_ops

    torch.ops.load_library(str(build_torch_ops()))
    _LOADED = True


__all__ = ["load"]
