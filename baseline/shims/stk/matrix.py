class Matrix:
    """Plain container with the constructor signature of ``stk.Matrix``."""

    def __init__(self, size, data, row_indices, column_indices, offsets, column_indices_t=None, offsets_t=None,
                 block_offsets_t=None):
        self._size = tuple(size)
        self.data = data
        self.row_indices = row_indices
        self.column_indices = column_indices
        self.offsets = offsets
        self.column_indices_t = column_indices_t
        self.offsets_t = offsets_t
        self.block_offsets_t = block_offsets_t

    def size(self):
        return self._size

    @property
    def shape(self):
        return self._size
