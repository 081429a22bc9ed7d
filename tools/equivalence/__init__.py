"""Equivalence gates: frozen fingerprints of what must not change silently (wire formats, oracle execution digests,
checkpoint bytes, import closures) plus a mutation self-test of the gates themselves.

    python -m tools.equivalence.driver check            # compare against tests/golden/data/*.json
    python -m tools.equivalence.driver update           # rewrite the goldens after an intended change
    python -m tools.equivalence.driver selftest         # every mutant must change at least one digest
    python -m tools.equivalence.compare_run RUN_A RUN_B # token-stream identity of two real runs

Gate names follow the reference's (``tools/equivalence/README.md:69-132``): G1 the launch programs (``programs.py``: the ordered
launch list of a decode step and a prefill chunk per configuration; recorded and checked on a GPU), G2 production defaults (``defaults.py``:
every limit, cap, default and choice that is relied on without being named), G3 execution digests, G4 checkpoint identity,
G6 import closures (may only shrink), G7 the set of functions a fixed CPU scenario executes (``executed.py``), G9 wire formats, G14
mutation self-test.  There is no compiler here, so the reference's G1/G2 (StableHLO fingerprints of compiled programs) become one gate
over the static launch list.
"""
