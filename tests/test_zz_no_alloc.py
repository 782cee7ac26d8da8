r"""The allocation-free bias-gradient entry point, called through its exported C symbol.

Some callers of this library cannot ask for device memory at the moment they need a result —
a stream capture in progress, a runtime with a fixed memory plan, a host that only speaks the
C ABI.  ``fmoe_bias_grad_noalloc`` serves them with an accumulation buffer that is part of the
library.  It must agree with the regular (allocating) entry point, and because every call
shares that buffer, a second call right after the first must not see the first call's sums.

The file name sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from fastmoe_b200.ops import native
    native.get()
    lib = ctypes.CDLL(native.so_path())
    lib.fmoe_bias_grad_noalloc.restype = ctypes.c_int
    lib.fmoe_bias_grad_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                           ctypes.c_long, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_void_p, ctypes.c_void_p]
    lib.fmoe_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _call(lib, x, offs, out):
    code = 0 if x.dtype == torch.bfloat16 else 1
    stream = torch.cuda.current_stream().cuda_stream
    return lib.fmoe_bias_grad_noalloc(x.data_ptr(), offs.data_ptr(), offs.numel() - 1, x.shape[0],
                                      x.shape[1], code, out.data_ptr(), stream)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_noalloc_matches_regular_entry_twice(dtype):
    from fastmoe_b200.ops import grouped_gemm as gg
    lib = _lib()
    dev = "cuda"
    torch.manual_seed(0)
    counts = [300, 0, 129, 71]
    offs = torch.zeros(len(counts) + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(torch.tensor(counts), 0)
    offs = offs.to(dev)
    n = 512
    for call in range(2):
        # different data on the second call: stale sums in the shared array would show
        x = (torch.randn(sum(counts) + 5, n, device=dev) * (1 + 3 * call)).to(dtype)
        out = torch.full((len(counts), n), float("nan"), device=dev, dtype=dtype)
        rc = _call(lib, x, offs, out)
        assert rc == 0, lib.fmoe_noalloc_last_error()
        ref = gg.bias_grad(x, offs)
        torch.cuda.synchronize()
        assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2), \
            float((out.float() - ref.float()).abs().max())
        assert float(out[1].abs().max()) == 0.0  # the empty expert
        # and against plain fp32 sums of the segments (an oracle that shares no kernel with it)
        base = 0
        for e, cnt in enumerate(counts):
            want = x[base:base + cnt].float().sum(0)
            tol = 2e-2 * float(want.abs().max()) + 1e-2     # one rounding of the 16-bit result
            assert float((out[e].float() - want).abs().max()) <= tol, e
            base += cnt


def test_noalloc_rejects_bad_pointers_and_follows_no_offsets_past_the_matrix():
    lib = _lib()
    dev = "cuda"
    x = torch.ones(64, 64, device=dev, dtype=torch.bfloat16)
    offs = torch.tensor([0, 64], dtype=torch.int32, device=dev)
    out = torch.zeros(1, 64, device=dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    # host-side rejection only: nothing is launched for a misaligned x
    rc = lib.fmoe_bias_grad_noalloc(x.data_ptr() + 2, offs.data_ptr(), 1, 63, 64, 0, out.data_ptr(), stream)
    assert rc == -1 and b"aligned" in lib.fmoe_noalloc_last_error()
    # offsets that claim more rows than the matrix has: the extra rows are not read
    big = torch.tensor([0, 1000], dtype=torch.int32, device=dev)
    assert lib.fmoe_bias_grad_noalloc(x.data_ptr(), big.data_ptr(), 1, 64, 64, 0, out.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(out.float(), torch.full((1, 64), 64.0, device=dev))


def test_noalloc_rejects_oversize():
    lib = _lib()
    dev = "cuda"
    x = torch.zeros(8, 8192, device=dev, dtype=torch.bfloat16)
    offs = torch.zeros(17, dtype=torch.int32, device=dev)  # 16 groups * 8192 > 65536
    out = torch.zeros(16, 8192, device=dev, dtype=torch.bfloat16)
    assert _call(lib, x, offs, out) == -2
    assert b"exceeds" in lib.fmoe_noalloc_last_error()
