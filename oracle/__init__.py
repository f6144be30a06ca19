"""CPU oracle for the MoE decode hot path.  TEST INFRASTRUCTURE ONLY.

This package restates, on the CPU, the arithmetic that the reference (ZMLX
v0.8.5 on MLX) performs for router top-k -> gather_qmm_swiglu -> down
projection -> weighted combine.  It exists so that the CUDA kernels can be
checked and so that a host-CPU timing can be printed beside the GPU number.
Nothing in the shipped package imports it: only the tests, the smoke check and
the CPU-baseline leg of the benchmark do.

Parity status
-------------
The arithmetic of ``mx.gather_qmm``, ``mx.quantize``, ``mx.argpartition`` and
the mxfp4 mode lives in MLX (pinned by the reference at commit
185b06d9efc1c869540eccfb5baff853fff3659d, i.e. v0.30.6), which is a third-party
dependency that is not vendored in the reference tree and cannot be imported on
this platform.  The oracle therefore follows the reference's own in-tree
statements of that arithmetic (cited per function) and is pinned against the
known-answer cases the reference's tests contain (zero-logit tie-break,
boosted-bias selection, group-limited selection, one-hot / K=1 combine
identities, the top-2 hand-written rows).  Bit-level accumulation order of
MLX's CPU ``gather_qmm``, ``argpartition`` tie order, ``mx.quantize`` rounding
and the whole mxfp4 mode are **parity unpinned**: no golden vector for them
exists in the reference.
"""
