"""The scratch-free attention entry point, for callers that are not allowed to allocate device
memory (a plugin inside someone else's serving process, code that only holds borrowed buffers).

tq_attention_fwd_static must give the same output as tq_attention_fwd, which gets its scratch
from the caller, on two calls in a row that share the library's built-in scratch array; the
second call uses different data and a different shape, so anything left behind by the first
would show.  Collected last on purpose: a failure here cannot hide other results."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(L, kc, vc, q, ck, cv, mode):
    B, Hq, Sq, D = q.shape
    _, Hkv, Sk, _ = ck["shape"]
    dt = {torch.float32: L.TQ_F32, torch.bfloat16: L.TQ_BF16}[q.dtype]
    stream = torch.cuda.current_stream().cuda_stream
    common = (q.data_ptr(), dt, B, Hq, Sq, D, q.stride(0), q.stride(1), q.stride(2), Hkv, Sk,
              ck["packed_key_indices"].data_ptr(), ck["packed_qjl_signs"].data_ptr(), ck["vec_norms"].data_ptr(),
              ck["residual_norm"].data_ptr(), cv["packed_indices"].data_ptr(), cv["vec_norms"].data_ptr(),
              kc.Pi.data_ptr(), kc.S_eff.data_ptr(), kc.centroids.data_ptr(), vc.Pi.data_ptr(),
              vc.centroids.data_ptr(), kc.bits, 1.0 / math.sqrt(D), 1, None, 0, 0)
    ref = torch.empty_like(q)
    need = L.lib.tq_attention_workspace_bytes(B, Hq, Sq, D, mode)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    L.check(L.lib.tq_attention_fwd(*common, ref.data_ptr(), ref.stride(0), ref.stride(1), ref.stride(2),
                                   ws.data_ptr(), ws.numel(), mode, stream))
    out = torch.full_like(q, float("nan"))
    L.check(L.lib.tq_attention_fwd_static(*common, out.data_ptr(), out.stride(0), out.stride(1), out.stride(2),
                                          mode, stream))
    torch.cuda.synchronize()
    return out, ref


@pytest.mark.parametrize("mode_name", ["bf16", "fp32"])
def test_static_scratch_matches_workspace_variant(mode_name):
    import turboquant_b200 as tq
    from turboquant_b200 import _lib as L

    mode = L.TQ_MODE_BF16 if mode_name == "bf16" else L.TQ_MODE_FP32
    dtype = torch.bfloat16 if mode_name == "bf16" else torch.float32
    tol = 1e-2 if mode_name == "bf16" else 1e-4          # the tolerances of the parity tests
    kc = tq.TurboQuantCompressorV2(128, 3, 42, device="cuda", mode=mode_name)
    vc = tq.TurboQuantCompressorMSE(128, 3, 10042, device="cuda", mode=mode_name)
    g = torch.Generator(device="cuda").manual_seed(0)
    for B, Hq, Hkv, S in ((1, 4, 2, 300), (2, 2, 2, 129)):   # two calls in a row, different data and shape
        q = torch.randn(B, Hq, S, 128, generator=g, device="cuda").to(dtype)
        k = torch.randn(B, Hkv, S, 128, generator=g, device="cuda").to(dtype)
        v = torch.randn(B, Hkv, S, 128, generator=g, device="cuda").to(dtype)
        ck, cv = kc.compress(k), vc.compress(v)
        out, ref = _run_both(L, kc, vc, q, ck, cv, mode)
        assert torch.isfinite(out.float()).all()
        err = float((out.float() - ref.float()).norm() / ref.float().norm())
        assert err <= tol, err
        assert torch.equal(out, ref)  # same kernels, same inputs: in fact bit-identical


def test_static_scratch_rejects_oversized_problem():
    from turboquant_b200 import _lib as L

    cap = L.lib.tq_static_scratch_bytes()
    assert cap == 32 << 20
    B, Hq, Sq, D = 1, 32, 8192, 128                       # needs ~200 MB of scratch
    assert L.lib.tq_attention_workspace_bytes(B, Hq, Sq, D, L.TQ_MODE_BF16) > cap
    x = torch.zeros(1024, device="cuda")
    p = x.data_ptr()
    st = L.lib.tq_attention_fwd_static(p, L.TQ_BF16, B, Hq, Sq, D, Hq * Sq * D, Sq * D, D, 8, Sq, p, p, p, p, p, p,
                                       p, p, p, p, p, 3, 0.1, 1, None, 0, 0, p, Hq * Sq * D, Sq * D, D,
                                       L.TQ_MODE_BF16, None)
    assert st == 4 and "built-in array" in L.last_error()
