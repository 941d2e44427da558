"""Import-name compatibility: make ``import megablocks`` resolve to this library.

Code written against the reference (``import megablocks``, ``megablocks.layers.dmoe.dMoE``,
``megablocks.ops.gather`` ...) keeps working after one call::

    import megablocks_b200.compat
    megablocks_b200.compat.install_alias()

The alias is registered in ``sys.modules`` only (no files named ``megablocks`` are
shipped), so it cannot shadow a real installation of the reference unless asked to.
"""

import importlib
import sys

_SUBMODULES = [
    'layers', 'layers.arguments', 'layers.common', 'layers.mpu', 'layers.router', 'layers.moe', 'layers.dmoe',
    'layers.mlp', 'layers.glu', 'layers.gelu', 'layers.activation_fn', 'layers.all_to_all',
    'layers.dmlp_registry', 'layers.sharedexpert_registry', 'ops', 'benchmark_util', 'grouped_gemm_util',
]


def install_alias(name: str = 'megablocks', force: bool = False) -> None:
    if name in sys.modules and not force:
        existing = sys.modules[name]
        if getattr(existing, '__name__', '') != 'megablocks_b200':
            raise RuntimeError(f'a different module named {name!r} is already imported; pass force=True to replace')
        return
    root = importlib.import_module('megablocks_b200')
    sys.modules[name] = root
    for sub in _SUBMODULES:
        sys.modules[f'{name}.{sub}'] = importlib.import_module(f'megablocks_b200.{sub}')
