"""Source compatibility for the reference's ahead-of-time tooling.

The reference JIT-compiles Triton kernels and offers ``aot_compile_spaces`` (reference
python/triton_dist/tools/compile_aot.py:61-77) to pre-build chosen signatures into a C library. Here every kernel
is compiled ahead of time by nvcc into ``libtdist.so`` and the "space" is the template instantiation table of each
``.cu`` file (flash decode: dtype x head_dim; GEMM: mode x CTA tiling), so the decorator only records what was asked
for, which ``aot_spaces()`` lists.
"""
from __future__ import annotations

from typing import Callable, Dict

_SPACES: Dict[str, dict] = {}


def aot_compile_spaces(spaces: dict) -> Callable:
    def decor(fn):
        for name, spec in spaces.items():
            _SPACES[name] = dict(spec, function=getattr(fn, "__name__", str(fn)))
        return fn
    return decor


def aot_spaces() -> Dict[str, dict]:
    return dict(_SPACES)


def get_triton_combine_kv_algo_info(num_q_heads: int, head_dim: int, *a, **kw) -> dict:
    """What the reference returns to pick a compiled variant of its combine kernel (flash_decode.py): the fixed
    configuration of the merge stage here (a warp per query head, 4 columns per lane)."""
    return {"num_warps": 4, "num_stages": 1, "BLOCK_DV": head_dim, "heads_per_cta": min(16, num_q_heads)}
