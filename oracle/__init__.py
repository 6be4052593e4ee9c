"""CPU oracle for the TACE energy+force path.  TEST INFRASTRUCTURE ONLY.

This package is a plain PyTorch / numpy restatement of the reference
(xvzemin/tace) energy, conservative-force and virial evaluation path, used to
check the CUDA kernels in ``tace_b200``.  Nothing in the shipped product path
imports it: only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` do.

PARITY UNPINNED at the e3nn boundary: the reference delegates Wigner-3j
symbols, spherical harmonics, tensor-product and linear normalisation and the
gate slot order to the third-party package ``e3nn`` (``pyproject.toml:21``,
unpinned), which is not vendored in the reference tree and is not installable
offline.  The reference's own tests hold no energy / force / neighbour-list
golden value for this path.  ``oracle/o3.py`` therefore restates e3nn's
published algorithms; the only reference-held known answers that pin it are
the three activation second-moment constants (``tace/models/mlp.py:34,43,52``,
pinned by ``tests/test_o2.py:352-376``), which ``tests/test_oracle_o3.py``
reproduces.
"""
