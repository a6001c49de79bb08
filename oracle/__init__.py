"""CPU oracle of the decode-monokernel hot path.  TEST INFRASTRUCTURE ONLY.

A numpy / torch-CPU restatement of the arithmetic the reference's own torch
goldens define for each stage (each function cites the reference file:line it
follows).  Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU
baseline legs may import this package, and only as the checker or as the timed
CPU baseline; the product package never imports it and has no CPU fallback.

Pinning: the quantisation helpers, the radix key and the walk plan are checked
against the reference's importable Python (``tests/golden/make_golden.py`` ran
them and stored the vectors under ``tests/golden/``) and against the
known-answer values in the reference's unit tests.  The stage compositions
(whole MoE block, whole layer) have no stored golden in the reference; their
rules are the reference's torch goldens restated here.
"""
