"""CPU restatement (PyTorch fp32 on the host) of the DiT-step arithmetic of DiffSynth-Engine v0.1.1.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this; it is used by ``tests/``,
by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of ``bench.py`` as the checker / the
timed CPU arm.  Each function cites the reference file:line it restates.

Parity status: pinned.  ``tests/golden/make_golden.py`` executes the reference's own modules
(imported from its source tree) on seeded inputs and stores their outputs as fixtures;
``tests/test_oracle_golden.py`` checks every oracle function against them, and against the two
fixtures the reference's own test-suite ships for the flow-match sampler and scheduler.
"""
