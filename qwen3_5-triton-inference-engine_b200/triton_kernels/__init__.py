"""Drop-in package for the reference engine's `triton_kernels` imports.

The reference's `engine/runner.py`, `engine/cache.py` and `engine/paging.py` import their operators with
`from triton_kernels.<module> import <symbol>`.  Putting this directory's parent first on `sys.path` makes
those imports resolve to the sm_100a CUDA operators of `b200attn` instead; module and symbol names are the
reference's (there is no Triton code here).
"""
