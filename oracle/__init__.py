"""CPU oracle for the sphconv hot path (rule generation + rule-driven sparse convolution).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this directory: it is
used by ``tests/``, by ``__graft_entry__.smoke()`` as the checker, and by ``bench.py`` for the
timed CPU baseline.  The product path is the CUDA library behind ``include/sphconv_b200.h``
and fails loudly when that library is missing.

What it restates (paths are relative to the reference project):

* ``rules_loops``  - literal, loop-for-loop restatement of ``src/sphconv/rules.cu`` (small cases).
* ``rules_np``     - vectorised numpy restatement of the same algorithm (any size).
* ``conv_np``      - "sum over pairs" forward / dgrad / wgrad of
                     ``include/sphconv/rule_conv_kernel.cu.h:91-153`` and ``src/sphconv/rule_conv.cu:469-597``.
* ``dense_ref``    - the dense ``torch.nn.functional.conv3d`` construction the reference's own tests use
                     as their ground truth (``test/test_rules.py:14-60``, ``test/test_grad.py:7-36``).

Pinning.  The reference holds no golden vectors or known-answer files for this path (its tests
compute every expectation at run time with spconv 1.x or dense torch conv3d) and has no CPU
implementation.  The oracle is pinned two ways: (1) ``tests/test_oracle.py`` checks it against the
dense-conv3d construction of the reference's tests, on CPU, for occupancy, forward, dgrad and wgrad;
(2) ``tests/test_golden.py`` checks it against outputs of the reference's own CUDA kernels
(``oracle/_ref``, built from the unmodified reference sources by ``oracle/build_ref.py``) recorded on a
B200 into ``tests/golden/`` by ``tests/golden/make_golden.py``: rule sizes, pair sets, output indices,
and fp32 forward / dgrad / wgrad.
"""
