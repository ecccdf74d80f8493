"""The allocation-free entry point, fuelq_qmatmul_static_scratch.

It exists for hosts that can hand this library device pointers but cannot give it memory of
their own choosing at call time (no allocator in a plug-in sandbox; memory fixed before a
latency-critical loop started). Its scratch is an array inside the library, so the checks here
are: same bits as the ordinary entry point, on two calls in a row (the array is reused and is
not cleared in between), with different inputs so stale contents would show; and a clean
refusal when the problem does not fit. Collected last on purpose.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_static_scratch_matches_workspace_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import GgmlDType as T, _lib, ops
    L = _lib.lib
    stream = torch.cuda.current_stream().cuda_stream
    limit = L.fuelq_static_scratch_bytes()
    assert limit >= 1 << 20
    for dtype, n, k, ms in ((T.Q4K, 512, 4096, (1, 3)), (T.Q6K, 96, 1024, (5, 2)), (T.Q8_0, 200, 1056, (16, 1))):
        g = torch.Generator(device="cuda")
        g.manual_seed(int(dtype))
        w = ops.quantize_weights(dtype, torch.randn(n, k, generator=g, device="cuda") * 0.02)
        for call, m in enumerate(ms):  # two calls in a row, different batch and values
            x = torch.randn(m, k, generator=g, device="cuda") * (1.0 + call)
            want = ops.qmatmul(dtype, w, n, x)
            got = torch.full((m, n), float("nan"), device="cuda")
            _lib.check(L.fuelq_qmatmul_static_scratch(int(dtype), m, n, k, w.data_ptr(), x.data_ptr(), got.data_ptr(), stream),
                       "fuelq_qmatmul_static_scratch")
            torch.cuda.synchronize()
            assert torch.equal(got, want), (dtype, m)   # tolerance of the other GPU tests is met with equality
    # too large for the built-in scratch: refused with the workspace status, output untouched
    m, k, n = 300, 4096, 8
    assert L.fuelq_act_packed_bytes(int(T.Q4K), m, k) > limit
    w = torch.zeros(n * (k // 256) * 144, dtype=torch.uint8, device="cuda")
    x = torch.zeros(m, k, device="cuda")
    y = torch.full((m, n), 7.0, device="cuda")
    st = L.fuelq_qmatmul_static_scratch(int(T.Q4K), m, n, k, w.data_ptr(), x.data_ptr(), y.data_ptr(), stream)
    assert st == _lib.WORKSPACE
    torch.cuda.synchronize()
    assert bool((y == 7.0).all())
    assert ops.device_error() == 0


def test_static_scratch_runs_tensor_core_problems_without_a_slab():
    """Above the crossover the ordinary entry point wants a slab of dequantized weight rows in its workspace; the built-in
    array has no room for one. Q4_K / Q6_K / Q8_0 then run the one-kernel form (bit-identical to the ordinary entry under
    FUELQ_OPT_PREFILL_ONE_KERNEL), the other formats the integer kernels (bit-identical to the ordinary entry with the
    crossover raised)."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import GgmlDType as T, _lib, ops
    L = _lib.lib
    stream = torch.cuda.current_stream().cuda_stream
    limit = L.fuelq_static_scratch_bytes()
    g = torch.Generator(device="cuda")
    for dtype, m, n, k, opt, val in ((T.Q4K, 100, 4096, 1024, _lib.OPT_PREFILL_ONE_KERNEL, 1),
                                     (T.Q6K, 80, 2048, 512, _lib.OPT_PREFILL_ONE_KERNEL, 1),
                                     (T.Q5K, 70, 2048, 1024, _lib.OPT_DECODE_MAX_M, 1 << 20),
                                     (T.Q4_0, 33, 1024, 2048, _lib.OPT_DECODE_MAX_M, 1 << 20)):
        g.manual_seed(int(dtype) + m)
        w = ops.quantize_weights(dtype, torch.randn(n, k, generator=g, device="cuda") * 0.02)
        x = torch.randn(m, k, generator=g, device="cuda")
        assert L.fuelq_qmatmul_numerics(int(dtype), m, n, k) == _lib.NUMERICS_F16
        assert L.fuelq_qmatmul_workspace_bytes(int(dtype), m, n, k) > limit
        got = torch.full((m, n), float("nan"), device="cuda")
        _lib.check(L.fuelq_qmatmul_static_scratch(int(dtype), m, n, k, w.data_ptr(), x.data_ptr(), got.data_ptr(), stream),
                   "fuelq_qmatmul_static_scratch")
        try:
            _lib.check(L.fuelq_set_option(opt, val), "set_option")
            want = ops.qmatmul(dtype, w, n, x)
        finally:
            L.fuelq_set_option(opt, 0)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (dtype, m)
    assert ops.device_error() == 0
