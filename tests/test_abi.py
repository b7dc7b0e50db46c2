"""The C-ABI library loads and exports every symbol declared in include/clt_b200.h (no GPU needed)."""
import ctypes

from crosslayer_transcoder_b200 import _lib


def test_header_parses():
    protos = _lib.parse_header()
    assert "clt_encoder_fwd_act" in protos and "clt_adam_step" in protos
    assert len(protos) >= 18
    ret, args = protos["clt_adam_step"]
    assert ret is ctypes.c_int and len(args) == 14


def test_library_exports_every_declared_symbol():
    L = _lib.lib()                      # raises if a declared symbol is missing
    assert L.cdll.clt_version() >= 1
    for name in L.protos:
        assert hasattr(L.cdll, name)


def test_argument_errors_do_not_launch():
    L = _lib.lib()
    # bad dims are rejected before anything touches a device
    rc = L.cdll.clt_encoder_fwd_store(None, None, None, 0, 1, 1, 1, 0, None, None)
    assert rc != 0 and "bad dims" in L.last_error()
