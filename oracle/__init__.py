"""CPU oracle for the SBLocal attention forward.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package may import this directory: it exists so that
tests, the smoke check and the CPU-baseline leg of the benchmark have an
independent statement of the reference's arithmetic to compare the CUDA path
against.  Parity status: PINNED -- `oracle/ref_bridge.py` runs the reference's
own `SBLocalAttention` (with `oracle/local_product.py` standing in for the two
third-party window functions the reference imports) and the restatement in
`oracle/sblocal_oracle.py` is checked against it and against committed golden
vectors produced by `tests/golden/make_golden.py`.
"""
