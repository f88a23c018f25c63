"""The allocation-free GEMM entry point, called through its exported C symbol.

Some callers of the library cannot allocate device memory at the point where they need a
GEMM (an RPC handler inside a serving loop, code running under a host framework's memory
accounting). `eux_gemm_bf16_noalloc` serves them: its scratch is a static array inside the
library. This test checks it against the ordinary entry point on two calls in a row; the
second call finds the static array as the first one left it."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [512, 384])   # 512: the CTA-pair kernel (M % 256 == 0); 384: one CTA per tile
def test_noalloc_gemm_matches_regular_entry_point(cuda_device, m):
    from execution_ucx_b200.ops import _native
    from execution_ucx_b200.ops.remote_gemm import RemoteGemm
    lib = _native.load()
    fn = getattr(lib, "eux_gemm_bf16_noalloc")          # the exported C symbol itself
    n, k = 768, 1024
    torch.manual_seed(11)
    w = (torch.randn(k, n, device=cuda_device) * 0.02).to(torch.bfloat16)
    regular = RemoteGemm(w, m)
    w_t = regular.w_t
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(3):
        x = torch.randn(m, k, device=cuda_device).to(torch.bfloat16)   # fresh input per call
        want = torch.zeros(m, n, dtype=torch.bfloat16, device=cuda_device)
        got = torch.zeros(m, n, dtype=torch.bfloat16, device=cuda_device)
        regular(x.data_ptr(), m, want.data_ptr(), x_is_local=True)
        torch.cuda.synchronize()
        # what the driver itself reports as free: an allocation made inside the library (which torch's
        # own counters cannot see) would show here. The first call may load the kernels' module, so the
        # comparison starts with the second.
        free_before, _ = torch.cuda.mem_get_info()
        rc = fn(C.c_void_p(x.data_ptr()), C.c_void_p(w_t.data_ptr()), C.c_void_p(got.data_ptr()), m, n, k,
                C.c_void_p(status.data_ptr()), 2_000_000_000, stream)
        assert rc == 0, _native.load().eux_error_string(rc).decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call > 0:
            assert free_after == free_before
        assert int(status.item()) == 0
        regular.check_status()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(got.float(), x.float() @ w.float(), rtol=2e-2, atol=2e-2)
    # beyond the static array's capacity the call is refused, and says why
    rc = fn(C.c_void_p(x.data_ptr()), C.c_void_p(w_t.data_ptr()), C.c_void_p(got.data_ptr()), 131072 + 128, n, k,
            C.c_void_p(status.data_ptr()), 0, stream)
    assert rc == 100002
    assert b"maximum" in lib.eux_error_string(rc)
    # a shape the kernels do not take is refused before anything is put on the stream
    rc = fn(C.c_void_p(x.data_ptr()), C.c_void_p(w_t.data_ptr()), C.c_void_p(got.data_ptr()), m + 64, n, k,
            C.c_void_p(status.data_ptr()), 0, stream)
    assert rc == 100001
