"""Checker side of the repository (test infrastructure, never a product path).

``oracle.cpu``  - ctypes view of the CPU restatement in ``tcec_oracle.c``.
``oracle.ref``  - ctypes view of the reference itself built for sm_100a (``_ref/``).
"""
