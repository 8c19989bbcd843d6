"""CPU oracle for the two-stage sparse-attention forward path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by the test-suite, by the smoke check and by the CPU
baseline leg of the benchmark as the checker / timed CPU arm.

Pinning: the reference holds no golden vectors of its own, so the restatements
here are pinned against outputs of the reference itself (its pure-torch
``compute_mask_slow`` and its Triton kernels run under the Triton CPU
interpreter).  The vectors and the script that produced them live in
``tests/golden``.
"""
