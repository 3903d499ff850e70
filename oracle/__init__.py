"""CPU oracle for the Muon + AdamW hybrid optimizer step.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark do, and there only as the checker or the timed CPU arm.

Every function restates, in plain numpy float32 arithmetic, one piece of the
reference optimizer and cites the reference file:line it follows.

Parity status
-------------
* AdamW update, bf16 round-to-nearest-even, Muon momentum / update formulas,
  the fp32 Newton-Schulz and the Polar-Express coefficient table are PINNED:
  ``tests/golden/make_golden.py`` imports the reference's own Python modules
  and records their outputs on seeded inputs; ``tests/test_oracle_golden.py``
  checks this oracle against those files.
* The stochastic-rounding stream (Philox4x32-10) has no counterpart in the
  reference, which dithers with a coordinate hash.  Only the bit rule
  ``(f32_bits + dither16) >> 16`` is the reference's; the dither source is
  defined here and pinned by the published Philox known-answer vectors.
  For that stream: parity unpinned by the reference.
"""
