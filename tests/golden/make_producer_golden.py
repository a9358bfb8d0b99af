"""Generates ``tests/golden/reference_producer.npz``: outputs of the reference's own fused
qk-norm + partial-rotary function.

Test infrastructure.  The reference's function is a Triton kernel
(anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/fusions.py:208-274); Triton's
interpreter (``TRITON_INTERPRET=1``) executes it on CPU tensors, so the fixtures can be made
without a GPU wherever the reference checkout is present.  The interpreter has no 16-bit float
types of its own (its bfloat16 store truncates instead of rounding), so the kernel is given the
16-bit inputs widened to float32 and its float32 results are stored: the fixture then holds the
reference's arithmetic up to, and not including, the final rounding to the caller's type, which
``tests/test_producer.py`` applies itself.  The inputs are rebuilt from seeds there (same
``_case`` helper).

Run:  TRITON_INTERPRET=1 python tests/golden/make_producer_golden.py
"""

from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.test_producer import _case  # noqa: E402

# name: tokens, heads, D, rotary channels, dtype
CASES = {
    "bf16_d128_r64": (29, 3, 128, 64, torch.bfloat16),
    "f16_d128_r64": (29, 3, 128, 64, torch.float16),
    "bf16_d128_r128": (17, 2, 128, 128, torch.bfloat16),
    "f16_d64_r32": (23, 4, 64, 32, torch.float16),
    "bf16_d64_r16": (11, 5, 64, 16, torch.bfloat16),
}
EPS = 1e-6


def load_reference():
    if os.environ.get("TRITON_INTERPRET") != "1":
        raise SystemExit("run with TRITON_INTERPRET=1 (the reference's kernel is executed on CPU)")
    root = Path(os.environ.get("ANEMOI_REFERENCE_ROOT", ROOT.parent / "reference"))
    path = root / "anemoi/models/minimax_h3/solengine/models/minimax_h3/optimized/fusions.py"
    spec = importlib.util.spec_from_file_location("reference_fusions", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    if not module.HAVE_TRITON:
        raise SystemExit("the reference's fused path needs triton")
    return module.fused_qknorm_rope


def main() -> None:
    fused = load_reference()
    out = {}
    for name, (tokens, heads, d, rotary, dtype) in CASES.items():
        x, w, cos, sin = _case(tokens, heads, d, rotary, dtype, seed=tokens + heads)
        y = fused(x[None].float(), w, cos, sin, EPS)[0]
        out[name] = y.contiguous().numpy().astype(np.float32)
    path = ROOT / "tests" / "golden" / "reference_producer.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size} bytes, {len(out)} cases)")


if __name__ == "__main__":
    main()
