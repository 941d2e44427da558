"""Stand-in for the ``grouped_gemm`` pip package, used ONLY by the reference arm of bench.py.

The reference imports ``grouped_gemm`` (setup.py:71-73 of the reference) and it is
not installable offline.  This module reproduces the package's default build: a
loop of one library (cuBLAS) matmul per expert over row counts held on the host.
It is not product code and nothing under ``megablocks_b200`` imports it.
"""

from grouped_gemm import backend, ops  # noqa: F401
