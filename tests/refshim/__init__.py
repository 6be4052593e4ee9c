"""Stand-ins that let the reference's own source files run in this container.  TEST INFRASTRUCTURE ONLY.

Used by ``tests/golden/make_reference_fixtures.py`` (which writes the committed ``ref_*.npz`` fixtures) and by the live
half of ``tests/test_oracle_vs_reference_sources.py``; nothing in the product imports this package.
"""
