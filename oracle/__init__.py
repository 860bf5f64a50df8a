"""CPU oracle for the LSVD decode hot paths.

TEST INFRASTRUCTURE ONLY.  This package restates, on the CPU and in plain
torch / numpy, the arithmetic of the reference implementation (SAI-Lab-NYU/LSVD)
for the latent KV-cache append, the int8 latent flash-decoding attention and the
hybrid SVD/RTN FFN.  It exists so that the CUDA kernels can be checked against it.
Nothing in the shipped package imports it: only the tests, the smoke check and
the CPU-baseline leg of the benchmark do.

How the restatement is pinned to the reference
----------------------------------------------
The reference is pure Python.  ``tests/golden/make_golden.py`` imports the
reference's own functions (its PyTorch quantisers, ``HybridSVDQuantFFN``,
``matmul_hadU_cuda``, and its Triton kernels run by Triton's CPU interpreter)
and stores their outputs on small seeded inputs under ``tests/golden/``; the
CPU test-suite checks every oracle function against those stored outputs.  The
reference ships no golden vectors of its own for these paths.

The one mode that has no counterpart in the reference is the ``absorb``
attention (query folded into the K up-factor, no rotary embedding): it is pinned
indirectly, through its algebraic equality with the reconstruct-then-dot form
whose rotary variant is checked against the reference kernel.
"""
