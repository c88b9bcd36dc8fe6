"""GPU check of the sm_100a building blocks (TMA swizzled loads, shared-memory operand
descriptors in both majors, a 16-bit operand in tensor memory) against a plain matmul."""
import pytest
import torch

from flash_trittention import _native

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_selftest_matches_matmul(dtype):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    A = (torch.randn(128, 128, generator=g) * 0.25).to(dtype).to(dev)
    Bm = (torch.randn(128, 128, generator=g) * 0.25).to(dtype).to(dev)
    V = torch.randn(128, 128, generator=g).to(dtype).to(dev)
    C = torch.full((128, 128), float("nan"), device=dev)
    C2 = torch.full((128, 128), float("nan"), device=dev)
    st = _native.status_word(dev)
    rc = _native.lib().tritt_selftest_umma(A.data_ptr(), Bm.data_ptr(), V.data_ptr(), C.data_ptr(), C2.data_ptr(),
                                           _native.dtype_code(dtype), st.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _native.lib().tritt_last_error()
    torch.cuda.synchronize()
    assert _native.read_status(dev) == 0, "a bounded barrier wait ran out"
    ref = A.float() @ Bm.float().t()
    torch.testing.assert_close(C, ref, rtol=1e-4, atol=1e-4)
    ref2 = C.to(dtype).float() @ V.float()
    torch.testing.assert_close(C2, ref2, rtol=1e-3, atol=1e-3)
