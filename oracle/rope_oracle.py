"""CPU oracle for RoPE and the KV-cache append -- TEST INFRASTRUCTURE, not product code.

RoPE restates ``src/stackkernels/_reference/torch/rope.py:6-59`` (tables, ``rotate_half``, forward in fp32) and
the backward formula of ``src/stackkernels/torch/embedding.py:46-64``.  Parity status: PINNED against outputs of
the unmodified reference stored in ``tests/golden/rope.npz`` (``tests/golden/make_golden.py``).
The KV-cache append has no reference implementation (``_core/cache/kv_update.py`` is a stub); its oracle is the
index assignment it is defined as -- parity unpinned by construction, there is nothing to pin it to.
"""
import torch


def precompute_freqs(dim, max_seq_len=4096, base=10000.0, dtype=torch.float32):
    half = dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) / half))
    freqs = torch.outer(torch.arange(max_seq_len, dtype=torch.float32), inv_freq)
    c, s = torch.cos(freqs), torch.sin(freqs)
    return torch.cat([c, c], -1).to(dtype), torch.cat([s, s], -1).to(dtype)


def _rot(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def rope_forward(x, cos, sin, start_pos=0):
    """x (B,S,H,D) -> same shape/dtype; positions start_pos .. start_pos+S-1."""
    s = x.shape[1]
    c = cos[start_pos:start_pos + s].float()[None, :, None, :]
    sn = sin[start_pos:start_pos + s].float()[None, :, None, :]
    xf = x.float()
    return (xf * c + _rot(xf) * sn).to(x.dtype)


def rope_backward(dy, cos, sin, start_pos=0):
    s = dy.shape[1]
    c = cos[start_pos:start_pos + s].float()[None, :, None, :]
    sn = sin[start_pos:start_pos + s].float()[None, :, None, :]
    df = dy.float()
    return (df * c - _rot(df) * sn).to(dy.dtype)


def kv_append(k_cache, v_cache, k_new, v_new, lens):
    """Returns updated copies (k_cache, v_cache, lens): rows past the capacity are dropped, lens clamp to it."""
    k_cache, v_cache = k_cache.clone(), v_cache.clone()
    cap, t_new = k_cache.shape[2], k_new.shape[2]
    out_lens = []
    for b in range(k_cache.shape[0]):
        n = min(max(int(lens[b]), 0), cap)
        m = min(t_new, cap - n)
        k_cache[b, :, n:n + m] = k_new[b, :, :m]
        v_cache[b, :, n:n + m] = v_new[b, :, :m]
        out_lens.append(min(n + t_new, cap))
    return k_cache, v_cache, torch.tensor(out_lens, dtype=torch.int32)
