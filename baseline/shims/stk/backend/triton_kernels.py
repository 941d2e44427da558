def _unavailable(*args, **kwargs):
    raise NotImplementedError('block-sparse stk kernels are not available offline; use mlp_impl="grouped"')


sdd = dsd = dds = _unavailable
