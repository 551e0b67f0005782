"""Host-buffer entry point: attention on tensors that live in (pinned) host memory.

``flash_attention_host`` streams a batch through the GPU in chunks of whole batch rows -- units of
(batch, kv head) never interact, so a chunk is a self-contained problem -- overlapping the
host-to-device copy of chunk i+1, the kernel of chunk i and the device-to-host copy of chunk i-1 on
three CUDA streams with double-buffered device staging.  The PCIe link, not the kernel, bounds this path;
the pipeline keeps both directions of the link and the GPU busy at the same time.
The reference has no such call (its tensors are wherever the caller put them); this is the end-to-end
path `bench.py` times under ``e2e``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .launchers import flash_attn_fwd, validate_attention_layout


class _Staging:
    """Two sets of device buffers for (q, k, v, o) chunks plus the events that order their reuse."""

    def __init__(self, q, k, v, rows, device):
        def buf(t):
            return torch.empty((rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=device)
        self.sets = [dict(q=buf(q), k=buf(k), v=buf(v), o=None, lse=None,
                          loaded=torch.cuda.Event(), computed=torch.cuda.Event(), drained=torch.cuda.Event())
                     for _ in range(2)]


def flash_attention_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None, *,
                         causal: bool = False, softmax_scale: Optional[float] = None, device=None,
                         chunk_rows: Optional[int] = None, return_lse: bool = False):
    """q ``(B,H_q,S_q,D)``, k/v ``(B,H_kv,S_k,D)`` in host memory (pinned for full copy speed).

    Returns ``out`` (host tensor like q; allocated pinned if not given) and, with ``return_lse``, the fp32 LSE
    ``(B,H_q,S_q)`` on the host.  ``chunk_rows`` = batch rows per chunk (default: about eight chunks).
    """
    B, H_q, H_kv, S_q, S_k, D = validate_attention_layout(q, k, v)
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("flash_attention_host expects host tensors; use flash_attention for device tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(D)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    lse_host = torch.empty((B, H_q, S_q), dtype=torch.float32).pin_memory() if return_lse else None
    rows = chunk_rows or max(1, B // 8)
    rows = min(rows, B)
    with torch.cuda.device(dev):
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        st = _Staging(q, k, v, rows, dev)
        caller = torch.cuda.current_stream()
        for s in (s_in, s_run, s_out):
            s.wait_stream(caller)
        for i, b0 in enumerate(range(0, B, rows)):
            n = min(rows, B - b0)
            cur = st.sets[i & 1]
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(cur["computed"])      # the kernel two chunks ago has consumed these inputs
                cur["q"][:n].copy_(q[b0:b0 + n], non_blocking=True)
                cur["k"][:n].copy_(k[b0:b0 + n], non_blocking=True)
                cur["v"][:n].copy_(v[b0:b0 + n], non_blocking=True)
                cur["loaded"].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(cur["loaded"])
                if i >= 2:
                    s_run.wait_event(cur["drained"])      # its previous output has left the staging buffer
                o_d, lse_d = flash_attn_fwd(cur["q"][:n], cur["k"][:n], cur["v"][:n], is_causal=causal,
                                            sm_scale=softmax_scale)
                cur["o"], cur["lse"] = o_d, lse_d
                cur["computed"].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(cur["computed"])
                out[b0:b0 + n].copy_(cur["o"], non_blocking=True)
                if lse_host is not None:
                    lse_host[b0:b0 + n].copy_(cur["lse"], non_blocking=True)
                cur["o"].record_stream(s_out)
                cur["lse"].record_stream(s_out)
                cur["drained"].record(s_out)
        caller.wait_stream(s_out)
        caller.wait_stream(s_run)
    return (out, lse_host) if return_lse else out
