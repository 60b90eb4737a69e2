"""llmb_gemm_skinny_static: the decode product for callers that cannot allocate.

Some callers of the kernels hold no device memory of their own and may not ask for
any (they run where cudaMalloc is forbidden or would stall the device, or through a
binding that can launch but not allocate), so they cannot hand the split-K product
its scratch. For them the library exports one entry point whose scratch lives in
the library's own `static __device__` arrays. This test calls that entry point
through its exported C symbol, as such a caller would, and checks its output against
the existing entry point (which takes the caller's scratch), on two calls in a row:
the second call finds what the first one left in the shared arrays.

The file is named to be collected last, so that a run that stops at the first
failure has already run every other test. It passes alone in a fresh process and
after the other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F32, BF16 = 0, 1


def _library():
    from llm_b200.ops.build import compile_library
    lib = ctypes.CDLL(str(compile_library("gemm_skinny")))
    lib.llmb_gemm_skinny_scratch_bytes.restype = ctypes.c_longlong
    lib.llmb_gemm_skinny_last_error.restype = ctypes.c_char_p
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _with_callers_scratch(lib, x, w, bias, out, residual, m, n, k):
    need = lib.llmb_gemm_skinny_scratch_bytes(m, n, k)
    partials = torch.empty(max(need // 4, 1), dtype=torch.float32, device=DEV)
    counters = torch.zeros((n + 15) // 16, dtype=torch.int32, device=DEV)
    code = lib.llmb_gemm_skinny(_p(x), x.stride(0), _p(w), _p(bias), _p(out), F32, _p(residual),
                                _p(partials), ctypes.c_longlong(partials.numel() * 4), _p(counters),
                                counters.numel(), m, n, k, n, _stream())
    assert code == 0, lib.llmb_gemm_skinny_last_error()


def _without_allocating(lib, x, w, bias, out, residual, m, n, k):
    code = lib.llmb_gemm_skinny_static(_p(x), x.stride(0), _p(w), _p(bias), _p(out), F32,
                                       _p(residual), m, n, k, n, _stream())
    assert code == 0, lib.llmb_gemm_skinny_last_error()


@pytest.mark.parametrize("m,n,k", [(8, 4096, 4096), (3, 1000, 1032), (1, 6144, 14336)])
def test_static_scratch_entry_point_equals_the_existing_one(m, n, k):
    lib = _library()
    gen = torch.Generator().manual_seed(m + n + k)
    expected_calls = []
    for call in range(2):                      # two calls in a row share the built-in scratch
        x = torch.randn(m, k, generator=gen).to(torch.bfloat16).to(DEV)
        w = (torch.randn(n, k, generator=gen) * 0.05).to(torch.bfloat16).to(DEV)
        bias = torch.randn(n, generator=gen).to(DEV)
        want = torch.empty(m, n, dtype=torch.float32, device=DEV)
        got = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        _with_callers_scratch(lib, x, w, bias, want, None, m, n, k)
        _without_allocating(lib, x, w, bias, got, None, m, n, k)
        torch.cuda.synchronize()
        # the same kernel, the same split and order of additions: equal to the bit, and
        # within the tolerance the other kernel tests use against the plain product
        assert torch.equal(got, want), call
        plain = x.float() @ w.float().T + bias
        assert float((got - plain).abs().max()) <= 2e-3 * float(plain.abs().max())
        # adding into a residual stream, the second way to take the result
        residual_a = torch.randn(m, n, generator=gen).to(DEV)
        residual_b = residual_a.clone()
        _with_callers_scratch(lib, x, w, None, None, residual_a, m, n, k)
        _without_allocating(lib, x, w, None, None, residual_b, m, n, k)
        torch.cuda.synchronize()
        assert torch.equal(residual_a, residual_b), call


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _library()
    m, n, k = 64, 28672, 4096                  # partial sums beyond the built-in 4 MiB
    assert lib.llmb_gemm_skinny_scratch_bytes(m, n, k) > (1 << 22)
    x = torch.zeros(m, k, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(n, k, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    code = lib.llmb_gemm_skinny_static(_p(x), k, _p(w), None, _p(out), F32, None, m, n, k, n, _stream())
    assert code == 1
    text = lib.llmb_gemm_skinny_last_error().decode()
    assert "built-in" in text and "bytes" in text
