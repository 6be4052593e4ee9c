"""CPU oracle for the TACE energy+force path.  TEST INFRASTRUCTURE ONLY.

This package is a plain PyTorch / numpy restatement of the reference
(xvzemin/tace) energy, conservative-force and virial evaluation path, used to
check the CUDA kernels in ``tace_b200``.  Nothing in the shipped product path
imports it: only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` do.

PINNED against the reference's own source files, UNPINNED at the e3nn
boundary.  ``tests/golden/make_reference_fixtures.py`` imports the reference's
``tace.models`` package from its source tree (third-party packages replaced by
the stand-ins of ``tests/refshim``) and stores what the reference's code
computes for seven model cases (cgtp, TECE, LAMMPS ghost mode, ZBL, density,
multi-fidelity, correlation 3, ...) and for single components (edge frame,
Wigner rows, segment softmax, radial basis, radial MLP);
``tests/test_oracle_vs_reference_sources.py`` requires the oracle to reproduce
those numbers to fp64 round-off.  What the stand-in for the third-party
package ``e3nn`` (``pyproject.toml:21``, unpinned, absent from the reference
tree, not installable offline) supplies comes from ``oracle/o3.py`` and is
therefore NOT pinned by that comparison: Wigner-3j symbols, spherical
harmonics, ``o3.TensorProduct`` / ``o3.Linear`` normalisation, the activation
second-moment constants (the last are pinned separately by
``tace/models/mlp.py:34,43,52``).  The neighbour list follows matscipy's
documented semantics (``tace/dataset/neighbour_list.py:240-247``); matscipy is
absent too, so the edge set is checked against brute-force image enumeration.
"""
