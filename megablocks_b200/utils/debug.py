"""Debug-mode range checks for every index the kernels consume.

``compute-sanitizer`` is not available where this library is developed, so the stand-in is a
switch, ``MB200_DEBUG_BOUNDS=1`` (or :func:`enable`), under which the ops validate their routing
metadata on the device before each launch: copy ids inside ``[0, copies)``, expert ids inside
``[0, experts)``, prefix sums non-decreasing and inside the buffers they address, destination rows
inside the output.  A violation raises :class:`BoundsError` naming the tensor and the offending
value instead of letting a kernel read or write outside its operands.  Each check costs a small
reduction and a host synchronisation, so the switch is for tests and debugging, not for training.
"""

import os
from typing import Optional

import torch

_enabled = os.environ.get('MB200_DEBUG_BOUNDS', '0') == '1'


class BoundsError(IndexError):
    """An index tensor would have made a kernel leave its operands."""


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


def _range(name: str, t: Optional[torch.Tensor], lo: int, hi: int) -> None:
    """Every element of ``t`` in ``[lo, hi)``."""
    if t is None or t.numel() == 0:
        return
    mn, mx = int(t.min()), int(t.max())
    if mn < lo or mx >= hi:
        raise BoundsError(f'{name}: values span [{mn}, {mx}] but must lie in [{lo}, {hi})')


def _prefix(name: str, t: Optional[torch.Tensor], limit: int) -> None:
    """``t`` is a non-decreasing, non-negative prefix sum that ends at or below ``limit``."""
    if t is None or t.numel() == 0:
        return
    v = t.to(torch.int64)
    if int(v[0]) < 0 or (v.numel() > 1 and bool((v[1:] < v[:-1]).any())):
        raise BoundsError(f'{name}: not a non-decreasing prefix sum')
    if int(v[-1]) > limit:
        raise BoundsError(f'{name}: ends at {int(v[-1])}, beyond the {limit} rows it addresses')


def check_routing(indices, bin_ids, bins, padded_bins, top_k: int, tokens: int, out_rows: Optional[int] = None) -> None:
    """Routing metadata of the permutation ops against ``tokens`` source rows (``tokens * top_k``
    copies) and, for the gather forms, ``out_rows`` destination rows."""
    if not _enabled:
        return
    copies = tokens * top_k
    if indices.numel() > copies:
        raise BoundsError(f'indices: {indices.numel()} sorted positions for {copies} copies')
    _range('indices', indices, 0, copies)
    experts = bins.numel()
    _range('bin_ids', bin_ids, 0, experts)
    _prefix('bins', bins, indices.numel())
    if padded_bins is not None:
        _prefix('padded_bins', padded_bins, out_rows if out_rows is not None else 2**31 - 1)
        if padded_bins is not bins and bool((padded_bins.to(torch.int64) < bins.to(torch.int64)).any()):
            raise BoundsError('padded_bins: smaller than bins for some expert')


def check_groups(bins: torch.Tensor, rows: int, what: str = 'bins') -> None:
    """Group ends of a grouped GEMM against the rows of its operand."""
    if _enabled:
        _prefix(what, bins, rows)


def check_topology(row_indices, column_indices, offsets, shape, blocking: int) -> None:
    """BCSR metadata against the block grid of the matrix."""
    if not _enabled:
        return
    block_rows, block_cols = shape[0] // blocking, shape[1] // blocking
    _range('row_indices', row_indices, 0, block_rows)
    _range('column_indices', column_indices, 0, block_cols)
    _prefix('offsets', offsets, int(column_indices.numel()))
    if offsets.numel() != block_rows + 1:
        raise BoundsError(f'offsets: {offsets.numel()} entries for {block_rows} block rows')
