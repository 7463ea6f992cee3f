"""CPU oracle for the warpy-kernels hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under ``warpy_kernels_b200/`` or ``warpy_kernels/`` imports this package.  It is used by ``tests/``, by
``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline / reference legs, as the checker and the timed CPU
baseline, never as a compute path of the product.
"""
