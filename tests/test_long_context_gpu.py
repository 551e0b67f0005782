"""Long contexts: 128K-token causal prefill, a 32K-token backward and decode over a one-million-token cache.

The reference materialises the (S_q, S_k) score matrix (``src/stackkernels/_reference/torch/attention.py:52-70``), which
does not fit at these lengths, so the forward is checked on 128-row windows of queries (start, middle, end of the
sequence) against the same formula evaluated in fp32 on the device, the backward against the library's fp32
CUDA-core kernels, and decode against the formula on the whole cache.  Bars: 2e-2 (bf16) on O and gradients, 2e-3
on LSE."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape):
    return (torch.randn(*shape, device="cuda") * 0.7).to(torch.bfloat16)


def test_prefill_128k_tokens_on_query_windows():
    from stackkernels_b200 import _lib
    from stackkernels_b200.launchers import flash_attn_fwd
    torch.manual_seed(0)
    S, D, group = 131072, 128, 2
    q, k, v = _rand(1, 4, S, D), _rand(1, 2, S, D), _rand(1, 2, S, D)
    o, lse = flash_attn_fwd(q, k, v, is_causal=True, impl="sm100")
    for r0 in (0, S // 2 - 64, S - 128):
        keys = r0 + 128                                  # later keys are masked for every row of the window
        kk = k[:, :, :keys].float().repeat_interleave(group, 1)
        vv = v[:, :, :keys].float().repeat_interleave(group, 1)
        s = q[:, :, r0:r0 + 128].float() @ kk.transpose(-1, -2) * D ** -0.5
        hidden = torch.arange(keys, device="cuda")[None, :] > torch.arange(128, device="cuda")[:, None] + r0
        s = s.masked_fill(hidden, float("-inf"))
        assert (o[:, :, r0:r0 + 128].float() - torch.softmax(s, -1) @ vv).abs().max().item() <= 2e-2
        assert (lse[:, :, r0:r0 + 128] - torch.logsumexp(s, -1)).abs().max().item() <= 2e-3
    assert _lib.device_status() == 0


def test_backward_32k_tokens_against_the_fp32_kernels():
    from stackkernels_b200 import _lib
    from stackkernels_b200.launchers import flash_attn_bwd, flash_attn_fwd
    torch.manual_seed(1)
    S, D = 32768, 128
    q, k, v, do = _rand(1, 4, S, D), _rand(1, 2, S, D), _rand(1, 2, S, D), _rand(1, 4, S, D)
    o, lse = flash_attn_fwd(q, k, v, is_causal=True, impl="sm100")
    fast = flash_attn_bwd(do, q, k, v, o, lse, is_causal=True, impl="sm100")
    exact = flash_attn_bwd(do, q, k, v, o, lse, is_causal=True, impl="general")
    for name, a, b in zip(("dQ", "dK", "dV"), fast, exact):
        err = (a.float() - b.float()).abs()
        allowed = torch.clamp(b.float().abs() * 2.0 ** -7, min=2e-2)     # one bf16 ulp above the bar's range
        assert (err - allowed).max().item() <= 0, f"{name}: max abs err {err.max().item():.3e}"
    assert _lib.device_status() == 0


def test_decode_over_a_million_tokens():
    from stackkernels_b200 import _lib
    from stackkernels_b200.launchers import flash_decode
    torch.manual_seed(2)
    cap, D = 1 << 20, 128
    q, kc, vc = _rand(1, 32, 1, D), _rand(1, 8, cap, D), _rand(1, 8, cap, D)
    o, lse = flash_decode(q, kc, vc, return_lse=True)
    s = (q.float().view(1, 8, 4, D) @ kc.float().transpose(-1, -2)) * D ** -0.5
    ref = (torch.softmax(s, -1) @ vc.float()).view(1, 32, 1, D)
    assert (o.float() - ref).abs().max().item() <= 2e-2
    assert (lse.view(1, 8, 4) - torch.logsumexp(s, -1)).abs().max().item() <= 2e-3
    assert _lib.device_status() == 0
