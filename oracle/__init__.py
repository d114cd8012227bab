"""CPU oracle of the packed W2/W3/W4 linear path: test infrastructure, not part of the product.

``cb_oracle`` is the numpy restatement, ``cb_oracle_c`` the ctypes front end of the C
restatement (``cb_oracle.c``).  Only tests, the smoke entry point and the benchmark's CPU-baseline
leg may import this package.
"""
