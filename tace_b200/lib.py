"""ctypes binding of ``libtace_b200.so`` (declarations in ``include/tace_b200.h``).

There is no CPU fallback: if the shared library is missing, or was built without the
entry points the header declares, importing callers fail loudly here.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_int, c_int32, c_int64, c_size_t, c_uint8, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtace_b200.so")

TACE_F32, TACE_F64 = 0, 1

EXPORTS = [
    "tace_status_string", "tace_create", "tace_destroy", "tace_weight_count", "tace_weight_info", "tace_set_weight",
    "tace_workspace_bytes", "tace_forward", "tace_debug_read", "tace_nl_count", "tace_nl_fill", "tace_nl_workspace_bytes",
    "tace_launch_count", "tace_profile_enable", "tace_profile_count", "tace_profile_read", "tace_tc_gemm_f32", "tace_tc_gemm_set_test_mode",
    "tace_device_error", "tace_set_exchange", "tace_nl_build_noalloc", "tace_md_kick_drift", "tace_md_kinetic_energy",
    "tace_edge_vectors", "tace_edges_within", "tace_edges_scan_workspace_bytes", "tace_edges_scan", "tace_edges_compact", "tace_rows_gather", "tace_rows_scatter_add", "tace_set_graph_mode", "tace_graph_replays", "tace_set_exchange_sync", "tace_set_exchange_stream",
    "tace_set_chunk_edges", "tace_md_langevin",
]


class TaceConfig(ctypes.Structure):
    _fields_ = [
        ("dtype", c_int), ("L", c_int), ("num_layers", c_int), ("num_channel", c_int), ("num_elements", c_int),
        ("correlation", c_int), ("num_bessel", c_int), ("mlp_hidden", c_int), ("envelope_p", c_int),
        ("readout_hidden", c_int), ("cutoff", c_double), ("avg_num_neighbors", c_double), ("Lnode", c_int),
        ("use_alllayer", c_int), ("gate_m0_off", c_int), ("mlp_layers", c_int), ("mlp_bias", c_int), ("env_after_mlp", c_int),
        ("edge_update_element2", c_int), ("num_fidelities", c_int), ("zbl", c_int), ("scatter_norm_density", c_int), ("resnet_identity", c_int), ("product_bilinear", c_int), ("tece_layers", c_int), ("mmax", c_int),
        ("num_head", c_int), ("edge_ace_hidden", c_int), ("edge_act", c_int), ("radial_table", c_int),
    ]


class TaceBatch(ctypes.Structure):
    _fields_ = [
        ("n_atoms", c_int64), ("n_local", c_int64), ("n_edges", c_int64), ("n_graphs", c_int32),
        ("positions", c_void_p), ("lattice", c_void_p), ("species", c_void_p), ("graph_ptr", c_void_p),
        ("edge_index", c_void_p), ("edge_shifts", c_void_p), ("edge_vector", c_void_p), ("fidelity", c_void_p),
    ]


class TaceOutputs(ctypes.Structure):
    _fields_ = [
        ("energy", c_void_p), ("node_energy", c_void_p), ("forces", c_void_p), ("virials", c_void_p),
        ("stress", c_void_p), ("edge_forces", c_void_p),
    ]


class TaceError(RuntimeError):
    pass


EXCHANGE_FN = ctypes.CFUNCTYPE(c_int, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int32)

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once and declare argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TaceError(
            f"{LIB_PATH} is missing: build it with `python -m tace_b200.build` (needs nvcc); "
            "tace_b200 has no CPU or PyTorch fallback"
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise TaceError(f"{LIB_PATH} does not export {name}")
    lib.tace_status_string.restype = c_char_p
    lib.tace_status_string.argtypes = [c_int]
    lib.tace_create.argtypes = [POINTER(TaceConfig), POINTER(c_void_p)]
    lib.tace_destroy.argtypes = [c_void_p]
    lib.tace_destroy.restype = None
    lib.tace_weight_count.argtypes = [c_void_p]
    lib.tace_weight_info.argtypes = [c_void_p, c_int, POINTER(c_char_p), POINTER(c_int64)]
    lib.tace_set_weight.argtypes = [c_void_p, c_char_p, c_void_p, c_int64]
    lib.tace_workspace_bytes.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_int32, POINTER(c_size_t)]
    lib.tace_forward.argtypes = [c_void_p, POINTER(TaceBatch), POINTER(TaceOutputs), c_void_p, c_size_t, c_void_p]
    lib.tace_debug_read.argtypes = [c_void_p, c_char_p, c_void_p, c_int64, c_void_p]
    lib.tace_debug_read.restype = c_int64
    lib.tace_launch_count.argtypes = [c_void_p]
    lib.tace_launch_count.restype = c_int64
    lib.tace_profile_enable.argtypes = [c_void_p, c_int]
    lib.tace_profile_count.argtypes = [c_void_p]
    lib.tace_profile_read.argtypes = [c_void_p, c_int, POINTER(c_char_p), POINTER(ctypes.c_float)]
    lib.tace_tc_gemm_f32.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32,
                                     c_void_p, c_void_p]
    lib.tace_device_error.argtypes = [c_void_p, POINTER(c_int32)]
    lib.tace_nl_build_noalloc.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_double, c_int64, c_void_p,
                                          c_void_p, c_void_p, c_void_p]
    lib.tace_set_exchange.argtypes = [c_void_p, EXCHANGE_FN, c_void_p]
    lib.tace_set_exchange_sync.argtypes = [c_void_p, c_int]
    lib.tace_set_exchange_stream.argtypes = [c_void_p, c_void_p]
    lib.tace_tc_gemm_set_test_mode.argtypes = [ctypes.c_uint32, ctypes.c_uint32]
    lib.tace_nl_workspace_bytes.argtypes = [c_int64, c_int32, POINTER(ctypes.c_size_t)]
    lib.tace_nl_count.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_double, c_void_p, c_void_p,
                                  ctypes.c_size_t, c_void_p]
    lib.tace_nl_fill.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_double, c_void_p, c_int64,
                                 c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_void_p]
    lib.tace_set_graph_mode.argtypes = [c_void_p, c_int]
    lib.tace_set_chunk_edges.argtypes = [c_void_p, c_int64]
    lib.tace_graph_replays.argtypes = [c_void_p]
    lib.tace_graph_replays.restype = c_int64
    lib.tace_md_kick_drift.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_double, c_double, c_void_p]
    lib.tace_md_langevin.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_double, c_double, ctypes.c_uint64, ctypes.c_uint64,
                                     c_void_p]
    lib.tace_md_kinetic_energy.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]
    lib.tace_edge_vectors.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_int32, c_void_p]
    lib.tace_edges_within.argtypes = [c_void_p, c_void_p, c_int64, ctypes.c_double, c_void_p, c_void_p]
    lib.tace_edges_scan_workspace_bytes.argtypes = [c_int64, POINTER(c_size_t)]
    lib.tace_edges_scan.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
    lib.tace_edges_compact.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int32, c_void_p]
    lib.tace_rows_gather.argtypes = [c_void_p, c_void_p, c_int64, c_int32, c_int32, c_void_p, c_void_p]
    lib.tace_rows_scatter_add.argtypes = [c_void_p, c_void_p, c_int64, c_int32, c_int32, c_void_p, c_void_p]
    _lib = lib
    return lib


def dtype_code(dtype) -> int:
    import torch
    if dtype == torch.float32:
        return TACE_F32
    if dtype == torch.float64:
        return TACE_F64
    raise TaceError(f"unsupported dtype {dtype}")


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().tace_status_string(int(status)).decode()
        raise TaceError(f"{what}: {msg} (status {status})")
