"""Compatibility module for code written against ``megablocks.grouped_gemm_util``.

The reference wraps an optional import of the external ``grouped_gemm`` package
(megablocks/grouped_gemm_util.py:1-26).  Here the grouped GEMM is built in, so
``ops`` / ``backend`` always resolve to this library's implementation.
"""

from megablocks_b200.ops import gg as _gg


def grouped_gemm_is_available() -> bool:
    return True


def assert_grouped_gemm_is_available() -> None:
    return None


class _Ops:
    gmm = staticmethod(_gg.gmm)


ops = _Ops()
backend = _gg.backend
