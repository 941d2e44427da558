def mask(*args, **kwargs):
    raise NotImplementedError('stk.random.mask is not available offline')
