"""CPU oracle for the MoE expert hot path (test infrastructure, not product code).

Everything in this package is a numpy/torch restatement of the reference's CPU
golden algorithms for router top-K, token-to-block grouping, MXFP8 block
quantisation and the blockwise expert MLP.  It exists so the CUDA path can be
checked against it; only the tests, the smoke check and the benchmark's CPU
baseline legs are allowed to import it.  The shipped package never does.
"""
