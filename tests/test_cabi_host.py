"""C ABI checks that need no GPU: the library loads, exports every function the header
declares, and rejects bad arguments on the host before touching CUDA."""

import ctypes
import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "tq_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    from turboquant_b200 import _lib

    names = declared_functions()
    assert len(names) >= 14
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} declared in tq_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_version_and_error_text():
    from turboquant_b200 import _lib

    assert _lib.version() >= 100
    st = _lib.lib.tq_pack_bits(None, 4, 128, 9, None, None)
    assert st == 1 and "bit width" in _lib.last_error()


@pytest.mark.parametrize("d,bits", [(96, 3), (128, 5), (128, 1), (0, 3)])
def test_compress_rejects_bad_config(d, bits):
    from turboquant_b200 import _lib

    st = _lib.lib.tq_compress_keys(None, 1, 1, 1, 8, d, 0, 0, d, None, None, None, None, bits,
                                   None, None, None, None, 1, None)
    assert st == 1
    assert ("head_dim" in _lib.last_error()) or ("bits" in _lib.last_error())


def test_null_and_misaligned_pointers_rejected():
    from turboquant_b200 import _lib

    buf = ctypes.create_string_buffer(4096)
    base = ctypes.addressof(buf)
    aligned = (base + 15) & ~15
    # NULL input with a non-empty problem
    assert _lib.lib.tq_compress_values(None, 1, 1, 1, 8, 128, 0, 0, 128, None, None, 3, None, None, 1, None) == 1
    # misaligned base pointer / stride that breaks 16-byte rows: rejected before any launch
    assert _lib.lib.tq_compress_values(aligned + 2, 1, 1, 1, 8, 128, 0, 0, 128, aligned, aligned, 3,
                                       aligned, aligned, 1, None) == 1
    assert "aligned" in _lib.last_error()
    assert _lib.lib.tq_compress_values(aligned, 1, 1, 1, 8, 128, 0, 0, 132, aligned, aligned, 3,
                                       aligned, aligned, 1, None) == 1
    # empty problems succeed without touching the device
    assert _lib.lib.tq_compress_values(None, 1, 0, 4, 8, 128, 0, 0, 128, None, None, 3, None, None, 1, None) == 0
    assert _lib.lib.tq_pack_bits(None, 0, 128, 3, None, None) == 0


def test_attention_argument_checks():
    from turboquant_b200 import _lib

    buf = ctypes.create_string_buffer(1 << 16)
    p = (ctypes.addressof(buf) + 255) & ~255
    args = dict(B=1, Hq=6, Sq=4, d=128, Hkv=4, Sk=4)

    def call(Hq=6, Hkv=4, Sq=4, Sk=4, ws=p, ws_bytes=0, causal=1):
        return _lib.lib.tq_attention_fwd(p, 1, 1, Hq, Sq, 128, Hq * Sq * 128, Sq * 128, 128, Hkv, Sk,
                                         p, p, p, p, p, p, p, p, p, p, p, 3, 0.1, causal, None, 0, 0,
                                         p, Hq * Sq * 128, Sq * 128, 128, ws, ws_bytes, 1, None)

    assert call() == 1 and "multiple" in _lib.last_error()          # 6 query heads over 4 KV heads
    assert call(Hq=8, Sq=8, Sk=4) == 1 and "causal" in _lib.last_error()
    assert call(Hq=8) == 4 and "workspace" in _lib.last_error()       # TQ_ERR_WORKSPACE
    need = _lib.lib.tq_attention_workspace_bytes(1, 8, 4, 128, 1)
    assert need >= 8 * 4 * 128 * 2 * 3 and need % 256 == 0
    assert _lib.lib.tq_attention_workspace_bytes(0, 8, 4, 128, 1) == 0


def test_cached_attention_argument_checks():
    """tq_attention_fwd_cached refuses a capacity below the keys in use and shapes the split-KV kernel does not
    serve, before anything is launched."""
    from turboquant_b200 import _lib

    buf = ctypes.create_string_buffer(1 << 16)
    p = (ctypes.addressof(buf) + 255) & ~255

    def call(Hq=8, Hkv=2, Sq=1, Sk=64, cap=128, d=128):
        return _lib.lib.tq_attention_fwd_cached(p, 1, 1, Hq, Sq, d, Hq * Sq * d, Sq * d, d, Hkv, Sk, cap,
                                                p, p, p, p, p, p, p, p, p, p, p, 3, 0.1, 1, None, 0, 0,
                                                p, Hq * Sq * d, Sq * d, d, p, 0, None)

    assert call(cap=32) == 1 and "capacity" in _lib.last_error()
    assert call(Sq=8) == 1 and "query rows" in _lib.last_error()        # 4 heads per KV head x 8 positions > 16
    assert call(d=64) == 1
    assert call() == 4 and "workspace" in _lib.last_error()             # passes the shape checks


def test_append_argument_checks():
    """tq_append_keys / tq_append_values refuse tokens that do not fit behind the ones stored."""
    from turboquant_b200 import _lib

    buf = ctypes.create_string_buffer(1 << 16)
    p = (ctypes.addressof(buf) + 255) & ~255
    st = _lib.lib.tq_append_keys(p, 1, 1, 2, 8, 128, 2048, 1024, 128, p, p, p, p, 3, p, p, p, p, 64, 60, 1, None)
    assert st == 1 and "do not fit" in _lib.last_error()
    st = _lib.lib.tq_append_values(p, 1, 1, 2, 8, 128, 2048, 1024, 128, p, p, 3, p, p, 64, -1, 1, None)
    assert st == 1 and "do not fit" in _lib.last_error()
    assert _lib.lib.tq_append_values(None, 1, 1, 2, 0, 128, 0, 0, 128, None, None, 3, None, None, 64, 64, 1, None) == 0
