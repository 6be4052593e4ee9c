"""tace_b200: TACE energy / force / stress evaluation as hand-written CUDA for sm_100a.

``tace_b200.models`` mirrors ``tace.models`` (``e3nnTACE``, ``cartTACE``, ``TensorModel``);
``tace_b200.neighbour_list`` mirrors ``tace.dataset.neighbour_list``; ``tace_b200.interface``
holds the ASE calculator and the LAMMPS ML-IAP object.
"""

from . import models  # noqa: F401
from .models import TensorModel, cartTACE, create_model, e3nnTACE  # noqa: F401

__all__ = ["models", "e3nnTACE", "cartTACE", "TensorModel", "create_model"]
