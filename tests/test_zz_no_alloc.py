"""GPU: ``skb_decode_noalloc`` -- the decode entry point for hosts that may not allocate device
memory (pre-planned memory pools, plugin enqueue hooks, loops that cannot afford cudaMalloc's
device-wide synchronisation).  It must give the same answer as ``skb_decode`` while taking its
split-KV scratch from the array built into the library.

Collected last on purpose: a failure here cannot hide the result of any other test when the
suite stops at the first failure.  The test passes on its own in a fresh process and after the
rest of the suite.
"""
import ctypes

import pytest
import torch

from _cases import TOL

pytestmark = pytest.mark.gpu


def _decode_both(lib, _lib, q, k, v, lens, splits):
    """Run skb_decode (caller-provided workspace) and skb_decode_noalloc on the same inputs."""
    B, Hq, _, D = q.shape
    Hkv, cap = k.shape[1], k.shape[2]
    dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[q.dtype]
    scale = 1.0 / D ** 0.5
    lens_p = None if lens is None else lens.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for noalloc in (False, True):
        o = torch.full_like(q, float("nan"))
        lse = torch.full((B, Hq, 1), float("nan"), dtype=torch.float32, device=q.device)
        if noalloc:
            rc = lib.skb_decode_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens_p, o.data_ptr(), lse.data_ptr(),
                                        B, Hq, Hkv, cap, D, dt, scale, splits, stream)
        else:
            ws_bytes = lib.skb_decode_workspace_bytes(B, Hq, Hkv, cap, D, dt, splits)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
            rc = lib.skb_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens_p, o.data_ptr(), lse.data_ptr(),
                                B, Hq, Hkv, cap, D, dt, scale, splits, 0, ws.data_ptr(), ws_bytes, stream)
        assert rc == _lib.SKB_OK, _lib.status_string(rc) + " " + _lib.last_cuda_error()
        torch.cuda.synchronize()
        outs.append((o, lse))
    return outs


def test_noalloc_decode_matches_decode_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from stackkernels_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.manual_seed(77)
    # two different problems back to back: the second call finds the first call's partials in the scratch
    problems = [
        dict(B=3, Hq=8, Hkv=2, cap=3000, D=128, dtype=torch.bfloat16, lens=[3000, 17, 1501], splits=5),
        dict(B=2, Hq=4, Hkv=4, cap=1000, D=64, dtype=torch.float16, lens=None, splits=2),
    ]
    for p in problems:
        q = torch.randn(p["B"], p["Hq"], 1, p["D"]).to(p["dtype"]).to(dev)
        k = torch.randn(p["B"], p["Hkv"], p["cap"], p["D"]).to(p["dtype"]).to(dev)
        v = torch.randn(p["B"], p["Hkv"], p["cap"], p["D"]).to(p["dtype"]).to(dev)
        lens = None if p["lens"] is None else torch.tensor(p["lens"], dtype=torch.int32, device=dev)
        (o_ref, lse_ref), (o_new, lse_new) = _decode_both(lib, _lib, q, k, v, lens, p["splits"])
        tol = TOL["bf16" if p["dtype"] == torch.bfloat16 else "fp16"]
        assert torch.isfinite(o_new.float()).all() and torch.isfinite(lse_new).all()
        assert (o_new.float() - o_ref.float()).abs().max().item() <= tol
        assert (lse_new - lse_ref).abs().max().item() <= tol


def test_noalloc_decode_rejects_problems_beyond_its_scratch():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from stackkernels_b200 import _lib
    lib = _lib.load()
    p = ctypes.c_void_p(1 << 20)     # never dereferenced: the size check comes before any launch
    B, Hq, Hkv, cap, D, splits = 64, 32, 8, 32768, 128, 16
    assert lib.skb_decode_workspace_bytes(B, Hq, Hkv, cap, D, 2, splits) > _lib.DECODE_NOALLOC_SCRATCH_BYTES
    rc = lib.skb_decode_noalloc(p, p, p, None, p, None, B, Hq, Hkv, cap, D, 2, 0.088, splits, None)
    assert rc == _lib.SKB_ERR_TOO_LARGE
