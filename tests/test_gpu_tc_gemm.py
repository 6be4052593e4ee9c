"""tcgen05 3xTF32 GEMM (through the C ABI) against an fp64 product: fp32-level accuracy is required
because its output feeds the energy at the 1e-5 eV/atom tolerance."""
import numpy as np
import pytest
import torch

from tace_b200 import lib as _lib
from tace_b200.pack import split_tf32

pytestmark = pytest.mark.gpu


def run(M, N, K, lda=None, seed=0):
    lib = _lib.load()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    lda = lda or K
    A_full = torch.randn(M, lda, generator=g, dtype=torch.float32)
    B = torch.randn(N, K, generator=g, dtype=torch.float32)
    hi, lo = split_tf32(B.numpy())
    A_d, hi_d, lo_d = A_full.to(dev), torch.from_numpy(hi).to(dev), torch.from_numpy(lo).to(dev)
    C = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    st = lib.tace_tc_gemm_f32(A_d.data_ptr(), lda, hi_d.data_ptr(), lo_d.data_ptr(), C.data_ptr(), N, M, N, K,
                              err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 0, f"kernel reported a bounded-wait expiry (code {int(err.item())})"
    ref = A_full[:, :K].double() @ B.double().T
    scale = ref.abs().max().item()
    diff = (C.cpu().double() - ref).abs().max().item()
    assert diff <= 2e-6 * scale * max(1.0, (K / 64) ** 0.5), f"M={M} N={N} K={K}: max diff {diff} at scale {scale}"


def test_radial_forward_shape():
    run(1000, 2944, 64)          # edges x (paths*channels), K = hidden width


def test_radial_backward_shape():
    run(777, 64, 2944)           # long K loop, narrow N (BN = 64)


def test_single_row_and_exact_tiles():
    run(1, 128, 32)
    run(128, 128, 64)
    run(129, 64, 96)


def test_strided_A_and_many_tiles_per_cta():
    run(40000, 256, 64, lda=96)  # more tiles than SMs: exercises the ring across tile boundaries


def test_an_expired_wait_is_reported_and_leaves_the_device_usable():
    """Failure path of the bounded waits, provoked without any fault: in the test mode every load barrier expects 16
    bytes more than its loads deliver, so it never completes; each role of the kernel gives up after its (shortened)
    poll limit, the kernel records which wait ran out, waits for the loads it has issued, frees its tensor memory and
    returns.  The context stays usable: the same GEMM in normal mode is correct afterwards."""
    lib = _lib.load()
    dev = torch.device("cuda:0")
    M, N, K = 256, 128, 64
    A = torch.randn(M, K, device=dev)
    B = torch.randn(N, K)
    hi, lo = split_tf32(B.numpy())
    hi_d, lo_d = torch.from_numpy(hi).to(dev), torch.from_numpy(lo).to(dev)
    C = torch.zeros(M, N, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.tace_tc_gemm_set_test_mode(4096, 16) == 0
    try:
        st = lib.tace_tc_gemm_f32(A.data_ptr(), K, hi_d.data_ptr(), lo_d.data_ptr(), C.data_ptr(), N, M, N, K, err.data_ptr(), stream)
        assert st == 0
        torch.cuda.synchronize()
    finally:
        assert lib.tace_tc_gemm_set_test_mode(0, 0) == 0
    assert int(err.item()) in (1, 2, 3, 4, 5), "no wait reported its expiry"
    err.zero_()
    st = lib.tace_tc_gemm_f32(A.data_ptr(), K, hi_d.data_ptr(), lo_d.data_ptr(), C.data_ptr(), N, M, N, K, err.data_ptr(), stream)
    assert st == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = A.double().cpu() @ B.double().T
    assert (C.cpu().double() - ref).abs().max().item() <= 2e-6 * ref.abs().max().item()
