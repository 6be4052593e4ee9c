"""Simulation-driver entry points: the ASE calculator, the LAMMPS ML-IAP object and the TorchSim model
(``tace/interface/ase/calculator.py``, ``tace/interface/lammps/mliap.py``, ``tace/interface/torchsim/torchsim.py``
in the reference)."""

from .ase_calculator import TACEAseCalc  # noqa: F401
from .lammps_mliap import TACELammpsCalc  # noqa: F401
from .torchsim import TACETorchSimCalc, tace_b200_nl  # noqa: F401
