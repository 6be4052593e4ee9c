"""Simulation-driver entry points: the ASE calculator and the LAMMPS ML-IAP object
(``tace/interface/ase/calculator.py``, ``tace/interface/lammps/mliap.py`` in the reference)."""

from .ase_calculator import TACEAseCalc  # noqa: F401
from .lammps_mliap import EdgeForcesWrapper, TACELammpsCalc  # noqa: F401
