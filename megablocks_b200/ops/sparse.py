"""Block-sparse matrices (BCSR, square blocks) and their products.

This module takes the place of the external ``stk`` package used by the
reference (call sites: megablocks/layers/dmoe.py:102-129, mlp.py:212-300,
392-394, glu.py:57-63).  ``Matrix`` stores the nonzero ``B x B`` blocks of a
matrix in row-major block order together with the metadata of its transpose,
so that products with the transposed matrix need no re-sorting.

Products:

* ``sdd(a, b, topo)``  dense x dense sampled at the nonzero blocks of ``topo``;
* ``dsd(s, b)``        sparse x dense  -> dense;
* ``dds(a, s)``        dense x sparse  -> dense;
* ``mul(a, b)``        elementwise product of two matrices with equal topology.

All are differentiable with respect to their dense operands and the block
values.  A matrix whose topology was produced by the dropless-MoE layer is
block-diagonal per expert; it carries ``padded_bins`` and the expert MLPs then
run the tcgen05 grouped kernel directly on it.  Any other topology with 128 x 128
blocks and 16-bit CUDA operands runs the BCSR-driven tcgen05 kernel of
``csrc/bsmm_kernel.cuh`` (transposed dense operands and transposed topologies are
read in place, as K-major or MN-major tiles).  Everything else - CPU tensors,
fp32, other block sizes - runs the gather-blocks + batched-matmul formulation
below, which is also the oracle of the tests.
"""

from typing import Any, Optional, Tuple

import torch

from megablocks_b200._ext import ext
from megablocks_b200.utils import debug

_KERNEL_BLOCK = 128
_MODE_SDD, _MODE_DSD, _MODE_DDS = 0, 1, 2


class Matrix:
    """BCSR matrix with square blocks.

    ``data`` is ``[nnz, B, B]``; ``row_indices`` / ``column_indices`` give each
    stored block's block-row / block-column; ``offsets`` (length rows/B + 1)
    delimits block-rows.  ``column_indices_t`` (block-row id of every block in
    transposed order), ``offsets_t`` and ``block_offsets_t`` (position in
    ``data`` of every block in transposed order) describe the transpose.
    """

    def __init__(self, size, data, row_indices, column_indices, offsets, column_indices_t=None, offsets_t=None,
                 block_offsets_t=None, transposed: bool = False):
        self._size = tuple(int(s) for s in size)
        self.data = data
        self.row_indices = row_indices
        self.column_indices = column_indices
        self.offsets = offsets
        if column_indices_t is None or offsets_t is None or block_offsets_t is None:
            column_indices_t, offsets_t, block_offsets_t = _transpose_metadata(
                self._size, int(data.shape[1]), row_indices, column_indices)
        self.column_indices_t = column_indices_t
        self.offsets_t = offsets_t
        self.block_offsets_t = block_offsets_t
        self._transposed = transposed
        # Set by the dropless-MoE layer for block-diagonal expert topologies.
        self.padded_bins: Optional[torch.Tensor] = None

    # -- shape protocol -------------------------------------------------------
    @property
    def blocking(self) -> int:
        return int(self.data.shape[1])

    @property
    def nnz(self) -> int:
        return int(self.data.numel())

    @property
    def is_transposed(self) -> bool:
        return self._transposed

    def size(self, dim: Optional[int] = None):
        shape = (self._size[1], self._size[0]) if self._transposed else self._size
        return shape if dim is None else shape[dim]

    @property
    def shape(self):
        return self.size()

    def dim(self) -> int:
        return 2

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def device(self):
        return self.data.device

    def t(self) -> 'Matrix':
        out = with_data(self, self.data)
        out._transposed = not self._transposed
        return out

    def contiguous(self) -> 'Matrix':
        return with_data(self, self.data.contiguous())

    def to(self, *args, **kwargs) -> 'Matrix':
        return with_data(self, self.data.to(*args, **kwargs))

    def to_dense(self) -> torch.Tensor:
        return to_dense(self)


def with_data(m: Matrix, data: torch.Tensor) -> Matrix:
    """A matrix with the topology of ``m`` and new block values."""
    out = Matrix(m._size, data, m.row_indices, m.column_indices, m.offsets, m.column_indices_t, m.offsets_t,
                 m.block_offsets_t, m._transposed)
    out.padded_bins = m.padded_bins
    return out


def _transpose_metadata(size, blocking, row_indices, column_indices):
    block_cols = size[1] // blocking
    cols = column_indices.to(torch.int64)
    order = torch.argsort(cols, stable=True)
    column_indices_t = row_indices.to(torch.int64)[order].to(row_indices.dtype)
    block_offsets_t = order.to(torch.int32)
    counts = torch.bincount(cols, minlength=block_cols)
    offsets_t = torch.cat([counts.new_zeros(1), torch.cumsum(counts, 0)]).to(torch.int32)
    return column_indices_t, offsets_t, block_offsets_t


def row_indices(shape, data, offsets, column_indices) -> torch.Tensor:
    """Expand CSR ``offsets`` into the block-row id of every stored block."""
    counts = (offsets[1:] - offsets[:-1]).to(torch.int64)
    rows = torch.arange(counts.numel(), device=offsets.device, dtype=column_indices.dtype)
    return torch.repeat_interleave(rows, counts, output_size=int(column_indices.numel()))


def to_dense(m: Matrix) -> torch.Tensor:
    b = m.blocking
    rows, cols = m._size
    out = m.data.new_zeros(rows // b, cols // b, b, b)
    out[m.row_indices.to(torch.int64), m.column_indices.to(torch.int64)] = m.data
    dense = out.permute(0, 2, 1, 3).reshape(rows, cols)
    return dense.t() if m._transposed else dense


def to_sparse(x: torch.Tensor, blocking: int = 128) -> Matrix:
    """Keep every ``blocking``-square block of ``x`` that has a nonzero entry."""
    rows, cols = x.shape
    if rows % blocking or cols % blocking:
        raise ValueError('matrix dimensions must be multiples of the block size')
    blocks = x.view(rows // blocking, blocking, cols // blocking, blocking).permute(0, 2, 1, 3)
    mask = (blocks != 0).any(dim=-1).any(dim=-1)
    r, c = torch.nonzero(mask, as_tuple=True)
    counts = torch.bincount(r, minlength=rows // blocking)
    offsets = torch.cat([counts.new_zeros(1), torch.cumsum(counts, 0)]).to(torch.int32)
    return Matrix((rows, cols), blocks[r, c].contiguous(), r.to(torch.int16), c.to(torch.int16), offsets)


def random_mask(rows: int, cols: int, sparsity: float, blocking: int = 128, device=None,
                dtype=torch.float16) -> Matrix:
    """Random topology with all-ones blocks; ``sparsity`` 0 keeps every block."""
    keep = torch.rand(rows // blocking, cols // blocking) >= sparsity
    dense = keep.to(dtype).repeat_interleave(blocking, 0).repeat_interleave(blocking, 1)
    return to_sparse(dense.to(device) if device is not None else dense, blocking)


# ----------------------------------------------------------------------------
# tcgen05 route (CUDA, 16-bit, 128 x 128 blocks)
# ----------------------------------------------------------------------------
def _stored(x: torch.Tensor):
    """``(storage, transposed)``: a contiguous row-major tensor that is ``x`` or ``x.t()``, without a copy if possible."""
    if x.is_contiguous():
        return x, False
    if x.dim() == 2 and x.t().is_contiguous():
        return x.t(), True
    return x.contiguous(), False


def _kernel_ok(blocking: int, *tensors: torch.Tensor) -> bool:
    if blocking != _KERNEL_BLOCK:
        return False
    first = tensors[0]
    for t in tensors:
        if not (t.is_cuda and t.dtype == first.dtype and t.dtype in (torch.bfloat16, torch.float16)):
            return False
        stored, _ = _stored(t)
        if stored.shape[-1] % 8 or stored.data_ptr() % 16:
            return False
    return True


def _i32(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.int32 and t.is_contiguous() else t.to(torch.int32).contiguous()


def _segments(s: Matrix, transposed_list: bool):
    """Segment list ``(offsets, block position or None, k-block)`` of the rows of ``s`` or of ``s^T``."""
    if transposed_list:
        return _i32(s.offsets_t), _i32(s.block_offsets_t), _i32(s.column_indices_t)
    return _i32(s.offsets), None, _i32(s.column_indices)


def _sdd_kernel(a: torch.Tensor, b: torch.Tensor, topo: Matrix) -> torch.Tensor:
    debug.check_topology(topo.row_indices, topo.column_indices, topo.offsets, topo._size, topo.blocking)
    sa, a_t = _stored(a)
    sb, b_t = _stored(b)
    # a is [M, K]: stored transposed = MN-major.  b is [K, N]: stored as given = MN-major.
    return ext().bsmm(_MODE_SDD, sa, a_t, sb, not b_t, _i32(topo.row_indices), _i32(topo.column_indices), None, 0, 0)


def _dsd_kernel(s: Matrix, data: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    debug.check_topology(s.row_indices, s.column_indices, s.offsets, s._size, s.blocking)
    sb, b_t = _stored(b)
    offsets, block, kblock = _segments(s, s.is_transposed)
    return ext().bsmm(_MODE_DSD, data.contiguous(), s.is_transposed, sb, not b_t, offsets, block, kblock, s.size(0),
                      b.shape[1])


def _dds_kernel(a: torch.Tensor, s: Matrix, data: torch.Tensor) -> torch.Tensor:
    debug.check_topology(s.row_indices, s.column_indices, s.offsets, s._size, s.blocking)
    sa, a_t = _stored(a)
    # Columns of s are the rows of its transpose: a plain topology needs the transposed list.
    offsets, block, kblock = _segments(s, not s.is_transposed)
    return ext().bsmm(_MODE_DDS, sa, a_t, data.contiguous(), not s.is_transposed, offsets, block, kblock, a.shape[0],
                      s.size(1))


# ----------------------------------------------------------------------------
# Products on raw block arrays.  (r, c) index blocks of the *stored* matrix.
# ----------------------------------------------------------------------------
def _rc(m: Matrix):
    return m.row_indices.to(torch.int64), m.column_indices.to(torch.int64)


def _sdd_blocks(a: torch.Tensor, b: torch.Tensor, topo: Matrix) -> torch.Tensor:
    """Blocks of ``a @ b`` at the nonzero positions of ``topo`` (not transposed)."""
    if _kernel_ok(topo.blocking, a, b):
        return _sdd_kernel(a, b, topo)
    blk = topo.blocking
    r, c = _rc(topo)
    a_rows = a.reshape(a.shape[0] // blk, blk, a.shape[1])[r]
    b_cols = b.reshape(b.shape[0], b.shape[1] // blk, blk).permute(1, 0, 2)[c]
    return torch.bmm(a_rows, b_cols)


def _dsd_dense(s: Matrix, data: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``op(s) @ b`` where ``op`` transposes when ``s`` is flagged transposed."""
    if _kernel_ok(s.blocking, data, b):
        return _dsd_kernel(s, data, b)
    blk = s.blocking
    r, c = _rc(s)
    out_rows = s.size(0)
    if s.is_transposed:
        lhs, out_idx, in_idx = data.transpose(1, 2), c, r
    else:
        lhs, out_idx, in_idx = data, r, c
    prod = torch.bmm(lhs, b.reshape(b.shape[0] // blk, blk, b.shape[1])[in_idx])
    out = torch.zeros(out_rows // blk, blk, b.shape[1], dtype=torch.float32, device=b.device)
    out.index_add_(0, out_idx, prod.float())
    return out.reshape(out_rows, b.shape[1]).to(b.dtype)


def _dds_dense(a: torch.Tensor, s: Matrix, data: torch.Tensor) -> torch.Tensor:
    """``a @ op(s)``."""
    if _kernel_ok(s.blocking, a, data):
        return _dds_kernel(a, s, data)
    blk = s.blocking
    r, c = _rc(s)
    out_cols = s.size(1)
    if s.is_transposed:
        rhs, in_idx, out_idx = data.transpose(1, 2), c, r
    else:
        rhs, in_idx, out_idx = data, r, c
    a_cols = a.reshape(a.shape[0], a.shape[1] // blk, blk).permute(1, 0, 2)[in_idx]
    prod = torch.bmm(a_cols, rhs)
    out = torch.zeros(out_cols // blk, a.shape[0], blk, dtype=torch.float32, device=a.device)
    out.index_add_(0, out_idx, prod.float())
    return out.permute(1, 0, 2).reshape(a.shape[0], out_cols).to(a.dtype)


class _SDD(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, a, b, topo: Matrix):
        ctx.save_for_backward(a, b)
        ctx.topo = topo
        return _sdd_blocks(a, b, topo)

    @staticmethod
    def backward(ctx: Any, dblocks):
        a, b = ctx.saved_tensors
        topo = ctx.topo
        da = db = None
        if ctx.needs_input_grad[0]:
            da = _dsd_dense(topo, dblocks, b.t())
        if ctx.needs_input_grad[1]:
            db = _dsd_dense(topo.t(), dblocks, a).t()
        return da, db, None


class _DSD(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, data, b, s: Matrix):
        ctx.save_for_backward(data, b)
        ctx.s = s
        return _dsd_dense(s, data, b)

    @staticmethod
    def backward(ctx: Any, dout):
        data, b = ctx.saved_tensors
        s = ctx.s
        ddata = db = None
        if ctx.needs_input_grad[0]:
            if s.is_transposed:
                # out = S^T b  =>  dS = b dout^T sampled at S's topology.
                ddata = _sdd_blocks(b, dout.t(), s.t())
            else:
                ddata = _sdd_blocks(dout, b.t(), s)
        if ctx.needs_input_grad[1]:
            db = _dsd_dense(s.t(), data, dout)
        return ddata, db, None


class _DDS(torch.autograd.Function):

    @staticmethod
    def forward(ctx: Any, a, data, s: Matrix):
        ctx.save_for_backward(a, data)
        ctx.s = s
        return _dds_dense(a, s, data)

    @staticmethod
    def backward(ctx: Any, dout):
        a, data = ctx.saved_tensors
        s = ctx.s
        da = ddata = None
        if ctx.needs_input_grad[0]:
            da = _dds_dense(dout, s.t(), data)
        if ctx.needs_input_grad[1]:
            if s.is_transposed:
                ddata = _sdd_blocks(dout.t(), a, s.t())
            else:
                ddata = _sdd_blocks(a.t(), dout, s)
        return da, ddata, None


def sdd(a: torch.Tensor, b: torch.Tensor, topo: Matrix) -> Matrix:
    """``(a @ b)`` restricted to the nonzero blocks of ``topo``."""
    if topo.is_transposed:
        raise ValueError('sdd expects a non-transposed topology')
    return with_data(topo, _SDD.apply(a, b, topo))


def dsd(s: Matrix, b: torch.Tensor) -> torch.Tensor:
    """``s @ b`` (``s`` may be a transposed view)."""
    return _DSD.apply(s.data, b, s)


def dds(a: torch.Tensor, s: Matrix) -> torch.Tensor:
    """``a @ s`` (``s`` may be a transposed view)."""
    return _DDS.apply(a, s.data, s)


def mul(a: Matrix, b: Matrix) -> Matrix:
    """Elementwise product of two matrices that share a topology."""
    if a.data.shape != b.data.shape:
        raise ValueError('mul expects matrices with identical topology')
    return with_data(a, a.data * b.data)
