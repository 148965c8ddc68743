"""CPU-side checks of the C-ABI boundary: the library loads, exports exactly what the header
declares, and its host-only helpers agree with the reference's host arithmetic. No GPU needed."""
import ctypes as C
import os
import re

import pytest

from sla_b200 import _lib
from sla_b200._lib import SlaShape, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "sla_b200.h")).read()
    return sorted(set(re.findall(r"SLA_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)))


def test_header_and_library_agree():
    names = _declared()
    assert names == sorted(_lib.EXPORTS)
    raw = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/sla_b200.h but not exported"


def test_version_and_status_strings():
    assert lib.sla_version() >= 100
    for s in range(0, -11, -1):
        assert lib.sla_status_string(s)
    assert b"unknown" in lib.sla_status_string(-99)


@pytest.mark.parametrize("n,ratio", [(16, 0.25), (64, 0.2), (512, 0.05), (1182, 0.05), (2048, 0.05),
                                     (2048, 0.1), (2048, 0.2), (4, 0.3), (7, 1.0), (7, 1.5), (3, 0.1)])
def test_topk_count_matches_python(n, ratio):
    assert _lib.topk_count(n, ratio) == min(n, int(ratio * n))  # utils.py:61-62


def test_workspace_sizes_are_aligned_and_monotone():
    prev = 0
    for L in (1024, 4096, 32760):
        s = SlaShape(1, 4, L, 128, 64, 64, 4, 0, 0, 0, 0.0)
        for op in (_lib.OP_BLOCK_MAP, _lib.OP_FWD, _lib.OP_BWD, _lib.OP_LINEAR_STATE, _lib.OP_SAGE_FWD):
            n = lib.sla_workspace_bytes(C.byref(s), op)
            assert n > 0 and n % 256 == 0
        n = lib.sla_workspace_bytes(C.byref(s), _lib.OP_BLOCK_MAP)
        assert n >= prev
        prev = n
    assert lib.sla_workspace_bytes(None, 0) == 0


def test_argument_errors_need_no_gpu():
    s = SlaShape(1, 1, 128, 128, 64, 64, 1, 0, 0, 0, 0.0)
    # NULL pointers are rejected before any CUDA call
    assert lib.sla_sparse_fwd(C.byref(s), None, None, None, None, None, None, None) == -9
    assert lib.sla_block_map(C.byref(s), 0, None, None, None, None, None, None, None, 0, None) == -9
    bad = SlaShape(1, 1, 128, 96, 64, 64, 1, 0, 0, 0, 0.0)   # D = 96
    one = C.c_void_p(16)
    assert lib.sla_sparse_fwd(C.byref(bad), one, one, one, one, one, one, None) == -1
    bad = SlaShape(1, 1, 128, 128, 32, 64, 1, 0, 0, 0, 0.0)  # BLKQ = 32 (kernel.py:247)
    assert lib.sla_sparse_fwd(C.byref(bad), one, one, one, one, one, one, None) == -1
    bad = SlaShape(1, 1, 128, 128, 64, 64, 0, 0, 0, 0, 0.0)  # topk = 0: the reference divides 0/0
    assert lib.sla_sparse_fwd(C.byref(bad), one, one, one, one, one, one, None) == -4


def test_module_surface_matches_reference():
    import torch
    import sla_b200
    m = sla_b200.SparseLinearAttention(head_dim=64, topk=0.2, feature_map="elu", BLKQ=128, BLKK=64)
    sd = m.state_dict()
    assert list(sd) == ["proj_l.weight", "proj_l.bias"]            # core.py:41
    assert sd["proj_l.weight"].dtype == torch.float32 and sd["proj_l.weight"].shape == (64, 64)
    assert float(sd["proj_l.weight"].abs().sum()) == 0 and float(sd["proj_l.bias"].abs().sum()) == 0  # core.py:64-67
    with pytest.raises(NotImplementedError):
        sla_b200.SparseLinearAttention(64, 0.2, feature_map="hedgehog")  # core.py:57
    with pytest.raises(RuntimeError):
        m(torch.zeros(1, 1, 64, 64), torch.zeros(1, 1, 64, 64), torch.zeros(1, 1, 64, 64))  # no CPU path
    s = sla_b200.SageSparseLinearAttention(128, 0.05)
    assert list(s.state_dict()) == ["proj_l.weight", "proj_l.bias"]
    sla_b200.install_aliases()
    from sparse_linear_attention import SparseLinearAttention as A
    from sparse_linear_attention.utils import get_block_map  # noqa: F401
    from sparse_linear_attention.kernel import _attention  # noqa: F401
    from SageSLA import SageSparseLinearAttention as B
    assert A is sla_b200.SparseLinearAttention and B is sla_b200.SageSparseLinearAttention
