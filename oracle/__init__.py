"""CPU oracle for the FlashMLA attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory.  It is imported by ``tests/``, by ``__graft_entry__.smoke()`` and by
the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the checker
and as the timed CPU baseline, never as the product path.

Every function restates, in plain torch/numpy on the CPU, what the reference
computes for this path, and cites the reference file:line it follows.  Parity is
PINNED: ``tests/golden/make_golden.py`` imports the reference's own Python
(tests/test_flash_mla_decoding.py, tests/test_flash_mla_prefill.py,
tests/test_fmha_sm100.py, tests/quant.py, flash_mla/flash_mla_interface.py) and
stores its outputs on seeded inputs as fixtures; ``tests/test_oracle_golden.py``
checks each oracle function against those fixtures.  The integer scheduler is
pinned against a line-by-line trace of csrc/smxx/get_mla_metadata.cu (the CUDA
source cannot be executed on a CPU), by invariants and by hand-worked vectors.
"""
