"""The C-ABI library on a machine without a GPU: it loads, exports every
symbol the header declares, and validates arguments before touching a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    with open(os.path.join(ROOT, 'include', 'sblocal_b200.h')) as fh:
        text = fh.read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(sbl_\w+)\s*\(', text)))


def test_header_symbols_are_exported_and_bound(sbl_lib):
    from fly_b200 import _cabi
    declared = _declared_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(sbl_lib, name), f'{name} declared in the header but not exported'
    assert sorted(_cabi.EXPORTS) == declared


def test_version_and_struct_size(sbl_lib):
    from fly_b200 import _cabi
    assert sbl_lib.sbl_version() == _cabi.ABI_VERSION
    # 11 int32/float + 4 x (ptr + 3 int64) + 2 ptr + 3 int64 + 6 int32, with C alignment
    assert ctypes.sizeof(_cabi.SblParams) == 240


def _params(**over):
    from fly_b200 import _cabi
    p = _cabi.SblParams()
    p.dtype = _cabi.SBL_DTYPE_F32
    p.B, p.H, p.T, p.S, p.E, p.D, p.r, p.w = 2, 3, 100, 100, 64, 64, 128, 32
    p.softmax_temp = 0.125
    for nm in ('q', 'k', 'v', 'out', 'W'):
        setattr(p, nm, 4096)
    p.q_stride_t = p.k_stride_s = p.v_stride_s = p.o_stride_t = 192
    p.S_total, p.sum_lo, p.sum_hi = 100, 0, 100
    for k, v in over.items():
        setattr(p, k, v)
    return p


def _bytes(lib, p):
    n = ctypes.c_size_t(0)
    rc = lib.sbl_workspace_bytes(ctypes.byref(p), ctypes.byref(n))
    return rc, n.value


def test_workspace_size_is_reported(sbl_lib):
    rc, n = _bytes(sbl_lib, _params())
    assert rc == 0
    # at least phi(K) and phi(Q) in fp32
    assert n >= 2 * 2 * 3 * 100 * 256 * 4
    rc2, n2 = _bytes(sbl_lib, _params(T=200))
    assert rc2 == 0 and n2 > n


@pytest.mark.parametrize('over,code,fragment', [
    (dict(dtype=7), -1, 'dtype'),
    (dict(B=0), -1, 'positive'),
    (dict(r=0), -1, 'projection rows'),
    (dict(w=0), -1, 'local_context'),
    (dict(softmax_temp=0.0), -1, 'softmax_temp'),
    (dict(q=None), -1, 'non-null'),
    (dict(D=200), -2, 'D=200'),
    (dict(sum_hi=101), -1, 'summary rows'),
    (dict(k_pos0=10, S_total=200), -1, 'halo'),
    (dict(S_total=50), -1, 'exceed S_total'),
    (dict(flags=6), -1, 'flag'),
])
def test_bad_arguments_are_rejected_with_a_message(sbl_lib, over, code, fragment):
    rc, _ = _bytes(sbl_lib, _params(**over))
    assert rc == code
    assert fragment in sbl_lib.sbl_last_error().decode()


def test_python_exceptions_follow_status(sbl_lib):
    from fly_b200 import _cabi
    rc, _ = _bytes(sbl_lib, _params(w=0))
    with pytest.raises(ValueError):
        _cabi.check(rc)
    rc, _ = _bytes(sbl_lib, _params(D=200))
    with pytest.raises(NotImplementedError):
        _cabi.check(rc)


def test_null_workspace_is_an_error_not_a_crash(sbl_lib):
    from fly_b200 import _cabi
    p = _params()
    rc = sbl_lib.sbl_forward(ctypes.byref(p), None, 0, None)
    assert rc == _cabi.SBL_ERR_WORKSPACE
    rc = sbl_lib.sbl_key_logscale_static(ctypes.byref(_params(k=None)), 4096, None)
    assert rc == _cabi.SBL_ERR_INVALID_ARGUMENT
