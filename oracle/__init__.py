"""CPU oracle of the aiehlc matmul hot path -- test infrastructure, not part of the product.

Only tests/, __graft_entry__.smoke() and the CPU legs of bench.py import this package.
"""
