"""CPU oracle for the attention hot path -- TEST INFRASTRUCTURE, not product code.

This is a fresh restatement, in plain torch-CPU tensor algebra, of what the
reference computes on its CPU path:

* forward  : ``attention_reference``  (reference file
  ``src/stackkernels/_reference/torch/attention.py:17-76``)
* GQA map  : ``repeat_kv``            (same file, ``:10-14``)
* backward : autograd through the forward, as the reference's CPU branch does
  (``src/stackkernels/torch/attention.py:82-102``); restated here as the closed
  form  dV = P^T dO, dP = dO V^T, dS = P*(dP - rowsum(dO*O)), dQ = dS K * scale,
  dK = dS^T Q * scale  (the same algebra the reference's GPU kernels use,
  ``src/stackkernels/_core/attention/flash_bwd.py:155-185,306-342``).
* decode   : ``attention_reference(..., is_causal=False)`` on a single query
  token (``src/stackkernels/torch/attention.py:134-155``); per-sequence
  ``cache_seqlens`` is emulated by slicing the cache to ``[:len_b]``.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the unmodified
reference in the build container and stores its outputs; ``tests/test_oracle.py``
checks this file against those stored outputs and against the config-1
checksums recorded from the reference.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py``
may import this module.  The product path never does.
"""
from __future__ import annotations

import math

import torch


def expand_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """(B, H_kv, S, D) -> (B, H_kv*n_rep, S, D); q head h uses kv head h // n_rep."""
    if n_rep == 1:
        return x
    b, h, s, d = x.shape
    return x[:, :, None].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)


def _scores(q, k, causal, scale):
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    if k.shape[3] != d:
        raise AssertionError(f"Head dimensions must match: {d} != {k.shape[3]}")
    if hq % hkv:
        raise AssertionError(f"Query heads {hq} must be divisible by KV heads {hkv}")
    kf = expand_kv(k, hq // hkv).float()
    s = torch.matmul(q.float(), kf.transpose(-2, -1)) * scale
    if causal:
        # key j visible to query i  iff  j <= i + (S_k - S_q)   (bottom-right aligned)
        qi = torch.arange(sq).unsqueeze(1)
        kj = torch.arange(sk).unsqueeze(0)
        s = s.masked_fill((kj > qi + (sk - sq))[None, None], float("-inf"))
    return s


def attention_forward(q, k, v, causal=False, scale=None):
    """Returns (O in q.dtype, LSE fp32).  Fully masked rows give O=0, LSE=-inf."""
    d = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    s = _scores(q, k, causal, scale)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
    vf = expand_kv(v, q.shape[1] // v.shape[1]).float()
    return torch.matmul(p, vf).to(q.dtype), lse


def attention_backward(do, q, k, v, causal=False, scale=None):
    """Returns (dQ, dK, dV) in the input dtypes; all arithmetic in fp32."""
    b, hq, sq, d = q.shape
    hkv, sk = k.shape[1], k.shape[2]
    g = hq // hkv
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    s = _scores(q, k, causal, scale)
    p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
    kf = expand_kv(k, g).float()
    vf = expand_kv(v, g).float()
    dof = do.float()
    o = torch.matmul(p, vf)
    dv_full = torch.matmul(p.transpose(-2, -1), dof)
    dp = torch.matmul(dof, vf.transpose(-2, -1))
    delta = (dof * o).sum(-1, keepdim=True)
    ds = p * (dp - delta)
    dq = torch.matmul(ds, kf) * scale
    dk_full = torch.matmul(ds.transpose(-2, -1), q.float()) * scale
    dk = dk_full.reshape(b, hkv, g, sk, d).sum(2)
    dv = dv_full.reshape(b, hkv, g, sk, d).sum(2)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def decode_forward(q, k_cache, v_cache, cache_seqlens=None, scale=None):
    """Single-token decode. Returns (O (B,Hq,1,D) in q.dtype, LSE (B,Hq,1) fp32).

    With ``cache_seqlens`` None the whole cache is attended (the reference's
    behaviour); otherwise sequence b attends to cache rows [0, cache_seqlens[b]).
    """
    assert q.shape[2] == 1, f"flash_decode requires q_len == 1, got {q.shape[2]}"
    if cache_seqlens is None:
        return attention_forward(q, k_cache, v_cache, causal=False, scale=scale)
    outs, lses = [], []
    for b in range(q.shape[0]):
        n = int(cache_seqlens[b])
        o, l = attention_forward(q[b:b + 1], k_cache[b:b + 1, :, :n], v_cache[b:b + 1, :, :n],
                                 causal=False, scale=scale)
        outs.append(o)
        lses.append(l)
    return torch.cat(outs), torch.cat(lses)


def decode_paged_forward(q, k_pages, v_pages, block_table, cache_seqlens, scale=None):
    """Decode over a paged cache: gather each sequence's pages into a dense cache, then ``decode_forward``.

    ``k_pages`` / ``v_pages`` ``(num_pages, Hkv, page_size, D)``; ``block_table`` ``(B, max_pages)``.  The reference
    only reserves this op (src/stackkernels/_core/attention/paged.py:1-3); its meaning here is "decode on the
    cache the block table describes", so the oracle is the gather followed by the pinned decode oracle."""
    bsz, page = q.shape[0], k_pages.shape[2]
    outs, lses = [], []
    for b in range(bsz):
        n = int(cache_seqlens[b])
        npg = (n + page - 1) // page
        idx = block_table[b, :npg].long()
        kb = k_pages[idx].permute(1, 0, 2, 3).reshape(1, k_pages.shape[1], npg * page, k_pages.shape[3])[:, :, :n]
        vb = v_pages[idx].permute(1, 0, 2, 3).reshape(1, v_pages.shape[1], npg * page, v_pages.shape[3])[:, :, :n]
        o, l = attention_forward(q[b:b + 1], kb, vb, causal=False, scale=scale)
        outs.append(o)
        lses.append(l)
    return torch.cat(outs), torch.cat(lses)


def varlen_forward(q, k, v, cu_q, cu_k, causal=False, scale=None):
    """Packed variable-length attention: ``attention_forward`` on every sequence by itself.

    ``q`` ``(total_q, Hq, D)``, ``k`` / ``v`` ``(total_k, Hkv, D)``, ``cu_*`` ``(B+1,)`` prefix sums.  Returns
    (O ``(total_q, Hq, D)`` in q.dtype, LSE ``(Hq, total_q)`` fp32).  The reference only reserves this op
    (src/stackkernels/_core/attention/varlen.py:1-3); its meaning here is "each sequence as a batch of one"."""
    outs, lses = [], []
    for b in range(len(cu_q) - 1):
        qb = q[int(cu_q[b]):int(cu_q[b + 1])].transpose(0, 1).unsqueeze(0)
        kb = k[int(cu_k[b]):int(cu_k[b + 1])].transpose(0, 1).unsqueeze(0)
        vb = v[int(cu_k[b]):int(cu_k[b + 1])].transpose(0, 1).unsqueeze(0)
        if qb.shape[2] == 0:
            continue
        o, l = attention_forward(qb, kb, vb, causal=causal, scale=scale)
        outs.append(o[0].transpose(0, 1))
        lses.append(l[0])
    return torch.cat(outs, 0), torch.cat(lses, 1)


def varlen_backward(do, q, k, v, cu_q, cu_k, causal=False, scale=None):
    """Gradients of ``varlen_forward``: ``attention_backward`` on every sequence by itself."""
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    for b in range(len(cu_q) - 1):
        q0, q1, k0, k1 = int(cu_q[b]), int(cu_q[b + 1]), int(cu_k[b]), int(cu_k[b + 1])
        if q1 == q0 or k1 == k0:
            continue
        sl = lambda t, a, e: t[a:e].transpose(0, 1).unsqueeze(0)
        gq, gk, gv = attention_backward(sl(do, q0, q1), sl(q, q0, q1), sl(k, k0, k1), sl(v, k0, k1), causal=causal,
                                        scale=scale)
        dq[q0:q1], dk[k0:k1], dv[k0:k1] = gq[0].transpose(0, 1), gk[0].transpose(0, 1), gv[0].transpose(0, 1)
    return dq, dk, dv


def forward_sliced(q, k, v, causal=False, scale=None, units=None):
    """Evaluate ``attention_forward`` one (batch, kv-head) unit at a time.

    Exact, because attention never couples two units; needed because the full
    score tensor of the large configurations does not fit in host memory.
    ``units`` is an iterable of (b, h_kv) pairs; None = all.  Yields
    (b, h_kv, O_slice (1,G,Sq,D), LSE_slice (1,G,Sq)).
    """
    bsz, hq = q.shape[0], q.shape[1]
    hkv = k.shape[1]
    g = hq // hkv
    if units is None:
        units = [(b, h) for b in range(bsz) for h in range(hkv)]
    for b, h in units:
        o, l = attention_forward(q[b:b + 1, h * g:(h + 1) * g], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1],
                                 causal=causal, scale=scale)
        yield b, h, o, l


def backward_sliced(do, q, k, v, causal=False, scale=None, units=None):
    """Per-unit ``attention_backward``; yields (b, h_kv, dQ_slice, dK_slice, dV_slice)."""
    bsz, hq = q.shape[0], q.shape[1]
    hkv = k.shape[1]
    g = hq // hkv
    if units is None:
        units = [(b, h) for b in range(bsz) for h in range(hkv)]
    for b, h in units:
        sl = slice(h * g, (h + 1) * g)
        dq, dk, dv = attention_backward(do[b:b + 1, sl], q[b:b + 1, sl], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1],
                                        causal=causal, scale=scale)
        yield b, h, dq, dk, dv
