"""Global constants of the SparseCore path.

Mirrors jax_tpu_embedding/sparsecore/lib/core/constants.py:17 of the reference.
"""

# Padding value of the CSR-wrapped COO buffers (ids and sample ids); padded gains are NaN.
PADDING_VALUE = 2**31 - 1
