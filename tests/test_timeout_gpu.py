"""The time-out path of the tcgen05 kernels, exercised without faulting anything: the wait limit is set to a
few milliseconds and a test hook makes one CTA of the forward skip the request for its first K tile, so the
waits behind that tile run out. The CTA must record a code, drain its copies, free its tensor memory and return;
the host must see SLA_ERR_TIMEOUT; and after clearing the word the same call must give correct results."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_reports_and_recovers():
    from sla_b200 import _lib, ops
    from sla_b200._lib import lib
    g = torch.Generator().manual_seed(21)
    B, H, L, D = 1, 2, 1024, 128
    q, k, v = (torch.randn(B, H, L, D, generator=g).bfloat16().cuda() for _ in range(3))
    bm = ops.block_map(q, k, 0.25, 64, 64)
    shape = ops.make_shape(B, H, L, D, 64, 64, bm.topk, torch.bfloat16, flags=_lib.FLAG_SPARSE_ONLY)
    lse = torch.empty(B, H, L, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def run():
        o = torch.zeros_like(q)
        _lib.check(lib.sla_sparse_fwd(C.byref(shape), q.data_ptr(), k.data_ptr(), v.data_ptr(), bm.lut.data_ptr(),
                                      o.data_ptr(), lse.data_ptr(), stream))
        return o

    good = run()
    assert _lib.poll_device_error() == 0
    try:
        _lib.check(lib.sla_debug_set_wait_limit_ns(3_000_000))          # 3 ms
        _lib.check(lib.sla_debug_drop_first_k_tile(1))
        run()
        code = C.c_int(0)
        rc = lib.sla_poll_device_error(C.byref(code), 0)
        assert rc == -8 and lib.sla_status_string(rc).decode().startswith("bounded device-side wait")
        assert 101 <= code.value <= 111, code.value                     # a wait of the forward kernel
        with pytest.raises(_lib.SlaError):
            _lib.raise_on_device_error()                                 # what SLA_B200_CHECK=1 does; clears the word
    finally:
        _lib.check(lib.sla_debug_drop_first_k_tile(0))
        _lib.check(lib.sla_debug_set_wait_limit_ns(0))
        _lib.poll_device_error(clear=True)
    again = run()
    assert _lib.poll_device_error() == 0
    assert torch.equal(again, good)
