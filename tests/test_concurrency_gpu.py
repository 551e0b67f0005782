"""Host threads, each on its own CUDA stream, call the library at the same time.

The reference's launchers are re-entrant Python functions that launch on torch's current stream
(``src/stackkernels/_core/attention/flash_fwd.py:182-264``); the C ABI behind this package keeps that contract: no
global state besides cached driver entry points, every buffer owned by the caller, launches on the stream passed
in.  Forward and decode must give the bits of a serial run; the backward adds fp32 partial sums of dQ in an order
that varies from run to run, so its results are compared within one 16-bit ulp."""
import threading

import pytest
import torch

pytestmark = pytest.mark.gpu

N_THREADS = 4
N_ITERS = 6


def _inputs(seed):
    g = torch.Generator(device="cuda").manual_seed(seed)

    def rnd(*shape):
        return (torch.randn(*shape, device="cuda", generator=g) * 0.7).to(torch.bfloat16)
    B, Hq, Hkv, S, D = 2, 8, 4, 1024, 128
    prefill = dict(q=rnd(B, Hq, S, D), k=rnd(B, Hkv, S, D), v=rnd(B, Hkv, S, D), do=rnd(B, Hq, S, D))
    cap = 4096
    decode = dict(q=rnd(4, 32, 1, D), k=rnd(4, 8, cap, D), v=rnd(4, 8, cap, D),
                  lens=torch.tensor([cap, 1, 2500 + seed, 0], dtype=torch.int32, device="cuda"))
    return prefill, decode


def _run(prefill, decode):
    from stackkernels_b200.launchers import flash_attn_bwd, flash_attn_fwd, flash_decode
    o, lse = flash_attn_fwd(prefill["q"], prefill["k"], prefill["v"], is_causal=True)
    dq, dk, dv = flash_attn_bwd(prefill["do"], prefill["q"], prefill["k"], prefill["v"], o, lse, is_causal=True)
    od, ld = flash_decode(decode["q"], decode["k"], decode["v"], cache_seqlens=decode["lens"], return_lse=True)
    return dict(o=o, lse=lse, dq=dq, dk=dk, dv=dv, od=od, ld=ld)


def test_threads_on_their_own_streams_match_a_serial_run():
    from stackkernels_b200 import _lib
    data = [_inputs(100 + i) for i in range(N_THREADS)]
    serial = [_run(*d) for d in data]
    torch.cuda.synchronize()
    results, errors = [None] * N_THREADS, []
    start = threading.Barrier(N_THREADS)

    def worker(i):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            start.wait(timeout=60)
            with torch.cuda.stream(stream):
                for _ in range(N_ITERS):
                    out = _run(*data[i])
            stream.synchronize()
            results[i] = out
        except Exception as exc:       # surfaced in the main thread below
            errors.append((i, repr(exc)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(N_THREADS)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    assert all(r is not None for r in results)
    assert _lib.device_status() == 0
    for i in range(N_THREADS):
        for name in ("o", "lse", "od", "ld"):
            assert torch.equal(results[i][name], serial[i][name]), f"thread {i}: {name} differs from the serial run"
        for name in ("dq", "dk", "dv"):
            torch.testing.assert_close(results[i][name].float(), serial[i][name].float(), rtol=2.0 ** -7, atol=1e-3,
                                       msg=lambda m, n=name, i=i: f"thread {i}: {n}: {m}")
