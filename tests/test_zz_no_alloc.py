"""The allocation-free attention backward, called through its exported C symbol.

Some hosts of this library may not allocate device memory (a memory budget fixed at
start-up, a device allocator owned by another framework, a loop that cannot afford the
device-wide synchronisation of a driver allocation): they call
`bux_attn_bwd_static`, which keeps its one scratch table inside the library. The test
hands it raw pointers of tensors allocated up front and checks it against the regular
entry point, twice in a row (the scratch keeps the previous call's contents).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, q, k, v, o, do, lse, sinks, dq, dk, dv, dsinks, window):
    b, t, h, d = q.shape
    s, g = k.shape[1], k.shape[2]
    msg = ctypes.c_char_p()
    ptr = lambda x: ctypes.c_void_p(0 if x is None else x.data_ptr())  # noqa: E731
    rc = lib.bux_attn_bwd_static(
        ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(dq), ptr(dk), ptr(dv), ptr(sinks),
        ptr(dsinks), b, t, s, h, g, d, ctypes.c_float(d ** -0.5), 1, window,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.byref(msg))
    return rc, (msg.value or b"").decode()


def test_static_entry_matches_the_regular_one(cuda):
    from bux_b200.ops import _build
    from bux_b200.ops import kernels as K

    lib = ctypes.CDLL(str(_build.build()))
    lib.bux_attn_bwd_static.restype = ctypes.c_int
    torch.manual_seed(0)
    for call, (t, window, with_sinks) in enumerate([(384, 0, False), (300, 128, True)]):
        q = torch.randn(2, t, 4, 128, device=cuda).bfloat16()
        k = torch.randn(2, t, 2, 128, device=cuda).bfloat16()
        v = torch.randn(2, t, 2, 128, device=cuda).bfloat16()
        do = torch.randn_like(q)
        sinks = torch.randn(4, device=cuda) if with_sinks else None
        o, lse = K.attn_fwd(q, k, v, causal=True, window=window, sinks=sinks)
        want = K.attn_bwd(q, k, v, o, do, lse, causal=True, window=window, sinks=sinks)
        # everything the entry point touches is allocated here, before the call
        dq = torch.full(q.shape, 7.0, dtype=torch.float32, device=cuda)
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        dsinks = torch.full((4,), 7.0, device=cuda) if with_sinks else None
        if call == 0:
            # the first call on a device resolves the scratch address; later calls must not
            # change what the driver reports as free either (a cudaMalloc inside the library
            # would not show in torch's own counter)
            rc, msg = _call(lib, q, k, v, o, do, lse, sinks, dq, dk, dv, dsinks, window)
            torch.cuda.synchronize()
            assert rc == 0, msg
        before = torch.cuda.memory_allocated(cuda)
        free_before = torch.cuda.mem_get_info(cuda)[0]
        rc, msg = _call(lib, q, k, v, o, do, lse, sinks, dq, dk, dv, dsinks, window)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.cuda.memory_allocated(cuda) == before
        assert torch.cuda.mem_get_info(cuda)[0] == free_before
        code, count = ctypes.c_uint(7), ctypes.c_uint(7)
        assert lib.bux_attn_bwd_static_status(ctypes.byref(code), ctypes.byref(count), 1) == 0
        assert (code.value, count.value) == (0, 0)  # no bounded wait ran out
        for got, ref in zip((dq, dk, dv), want[:3]):
            err = ((got.float() - ref.float()).norm() / ref.float().norm()).item()
            assert err < 2e-2, (call, err)
        if with_sinks:
            assert torch.allclose(dsinks, want[3], rtol=2e-2, atol=1e-3)


def test_static_entry_rejects_oversized_problems(cuda):
    from bux_b200.ops import _build

    lib = ctypes.CDLL(str(_build.build()))
    lib.bux_attn_bwd_static.restype = ctypes.c_int
    msg = ctypes.c_char_p()
    null = ctypes.c_void_p(0)
    rc = lib.bux_attn_bwd_static(null, null, null, null, null, null, null, null, null, null, null,
                                 64, 8192, 8192, 32, 4, 128, ctypes.c_float(0.1), 1, 0, null,
                                 ctypes.byref(msg))
    assert rc == 1 and b"exceeds" in msg.value
