"""CPU oracle of the SparseCore hot path.  TEST INFRASTRUCTURE - NOT THE PRODUCT.

Only tests/, the smoke test of __graft_entry__ and the CPU-baseline legs of
bench.py may import this package.
"""
