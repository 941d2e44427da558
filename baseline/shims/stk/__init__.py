"""Import-level stand-in for ``stanford-stk``, used ONLY by the reference arm of bench.py.

The reference imports ``stk`` unconditionally (megablocks/layers/mlp.py:6-8 of the
reference); the package is not installable offline and its Triton kernels refuse
triton >= 3.2 anyway.  Only what the reference's *grouped* path touches at import
time is provided: the ``Matrix`` container and the autocast decorators.  The
block-sparse products raise.  Not product code.
"""

from stk import backend, ops, random  # noqa: F401
from stk.matrix import Matrix  # noqa: F401
