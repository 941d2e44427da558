from stk.backend import autocast, triton_kernels  # noqa: F401
