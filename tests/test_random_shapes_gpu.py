"""Randomised shapes through every entry point (dense, strided, packed, decode, paged) against a plain fp32
evaluation on the device: ``softmax(q k^T * scale + mask) v`` and autograd through it, the formula of
``src/stackkernels/_reference/torch/attention.py:43-76``.  The oracle-based tests pin chosen cases; this one sweeps
head dims 32..256, group sizes 1..64, ragged and empty lengths, page sizes 8..256 and sequence lengths around the
tile sizes, with fixed seeds.  Bar: 1e-2 fp16 / 2e-2 bf16 with the one-ulp allowance of ``tests/_parity.py``."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {torch.float16: 1e-2, torch.bfloat16: 2e-2}
ULP = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


def fp32_attention(q, k, v, causal):
    """(O, LSE) of (B,H,S,D) tensors in fp32 on their device; fully masked rows give O = 0, LSE = -inf."""
    group = q.shape[1] // k.shape[1]
    kk = k.float().repeat_interleave(group, 1)
    vv = v.float().repeat_interleave(group, 1)
    s = q.float() @ kk.transpose(-1, -2) * q.shape[-1] ** -0.5
    s_q, s_k = q.shape[2], k.shape[2]
    if causal:
        hidden = torch.arange(s_k, device=q.device)[None, :] > torch.arange(s_q, device=q.device)[:, None] + (s_k - s_q)
        s = s.masked_fill(hidden, float("-inf"))
    return torch.softmax(s, -1).nan_to_num(0.0) @ vv, torch.logsumexp(s, -1)


def mismatch(what, ours, ref, dtype):
    """None if ``ours`` meets the bar against ``ref``, else a short description."""
    fin = torch.isfinite(ref)
    if not torch.equal(torch.isfinite(ours), fin):
        return f"{what}: non-finite pattern differs"
    if fin.any():
        err = (ours[fin].float() - ref[fin].float()).abs()
        allowed = torch.clamp(ref[fin].float().abs() * ULP[dtype], min=TOL[dtype])
        if (err - allowed).max().item() > 0:
            return f"{what}: max abs err {err.max().item():.3e}"
    return None


def rand(shape, dtype):
    return (torch.randn(*shape, device="cuda") * 0.7).to(dtype)


def prefill_case(dtype, B, Hq, Hkv, D, causal, strided):
    from stackkernels_b200.launchers import flash_attn_bwd, flash_attn_fwd
    s_q = random.choice([1, 37, 128, 129, 200, 256, 300, 513])
    s_k = random.choice([64, 128, 130, 257, 400, 640])
    if strided:      # (B,S,H,D) storage seen through transpose(1, 2)
        q, k, v = (rand((B, s, h, D), dtype).transpose(1, 2) for s, h in ((s_q, Hq), (s_k, Hkv), (s_k, Hkv)))
    else:
        q, k, v = (rand((B, h, s, D), dtype) for s, h in ((s_q, Hq), (s_k, Hkv), (s_k, Hkv)))
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    eo, el = fp32_attention(qr, kr, vr, causal)
    o, lse = flash_attn_fwd(q, k, v, is_causal=causal)
    do = rand((B, Hq, s_q, D), dtype)
    eo.backward(do.float())
    dq, dk, dv = flash_attn_bwd(do, q, k, v, o, lse, is_causal=causal)
    return f"Sq{s_q} Sk{s_k}", [mismatch("O", o, eo.detach(), dtype), mismatch("LSE", lse, el.detach(), dtype),
                                mismatch("dQ", dq, qr.grad, dtype), mismatch("dK", dk, kr.grad, dtype),
                                mismatch("dV", dv, vr.grad, dtype)]


def decode_case(dtype, B, Hq, Hkv, D, paged):
    import stackkernels_b200 as skb
    from stackkernels_b200.launchers import flash_decode
    cap = random.choice([64, 300, 1024, 2100])
    lens = torch.tensor([random.choice([0, 1, cap // 2, cap - 1, cap]) for _ in range(B)], dtype=torch.int32,
                        device="cuda")
    q, k, v = rand((B, Hq, 1, D), dtype), rand((B, Hkv, cap, D), dtype), rand((B, Hkv, cap, D), dtype)
    outs, lses = [], []
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            outs.append(torch.zeros(1, Hq, 1, D, device="cuda"))
            lses.append(torch.full((1, Hq, 1), float("-inf"), device="cuda"))
        else:
            o_b, l_b = fp32_attention(q[b:b + 1], k[b:b + 1, :, :n], v[b:b + 1, :, :n], False)
            outs.append(o_b)
            lses.append(l_b)
    eo, el = torch.cat(outs), torch.cat(lses)
    tag = f"cap{cap} lens{lens.tolist()}"
    if not paged:
        o, lse = flash_decode(q, k, v, cache_seqlens=lens, return_lse=True, num_splits=random.choice([0, 1, 3]))
    else:
        page = random.choice([8, 16, 64, 256])
        cap_p = (cap + page - 1) // page * page
        n_pages = B * cap_p // page

        def to_pool(t, perm):        # (B,Hkv,cap,D) -> pages in a random order
            padded = torch.zeros(B, Hkv, cap_p, D, device="cuda", dtype=dtype)
            padded[:, :, :cap] = t
            pages = padded.view(B, Hkv, cap_p // page, page, D).permute(0, 2, 1, 3, 4).reshape(n_pages, Hkv, page, D)
            pool = torch.empty_like(pages)
            pool[perm] = pages
            return pool
        perm = torch.randperm(n_pages, device="cuda")
        table = perm.view(B, cap_p // page).to(torch.int32)
        o, lse = skb.flash_decode_paged(q, to_pool(k, perm), to_pool(v, perm), table, lens, return_lse=True)
        tag += f" page{page}"
    return tag, [mismatch("O", o, eo, dtype), mismatch("LSE", lse, el, dtype)]


def varlen_case(dtype, Hq, Hkv, D, causal):
    import stackkernels_b200 as skb
    n_seq = random.randint(1, 4)
    len_q = [random.choice([0, 1, 64, 129, 200, 300]) for _ in range(n_seq)]
    len_k = [0 if a == 0 else random.choice([a, 64, 257, 400]) for a in len_q]
    if sum(len_q) == 0:
        len_q[0] = len_k[0] = 130
    cu_q = torch.tensor([0] + list(torch.tensor(len_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(len_k).cumsum(0)), dtype=torch.int32, device="cuda")
    q, k, v = rand((sum(len_q), Hq, D), dtype), rand((sum(len_k), Hkv, D), dtype), rand((sum(len_k), Hkv, D), dtype)
    o, lse = skb.flash_attention_varlen(q, k, v, cu_q, cu_k, max(len_q), max(len_k), is_causal=causal,
                                        return_lse=True)
    problems = []
    for s in range(n_seq):
        q0, q1, k0, k1 = int(cu_q[s]), int(cu_q[s + 1]), int(cu_k[s]), int(cu_k[s + 1])
        if q1 == q0:
            continue
        as_batch = lambda t, a, e: t[a:e].transpose(0, 1).unsqueeze(0)
        eo, el = fp32_attention(as_batch(q, q0, q1), as_batch(k, k0, k1), as_batch(v, k0, k1), causal)
        problems += [mismatch(f"O[{s}]", as_batch(o, q0, q1), eo, dtype),
                     mismatch(f"LSE[{s}]", lse[:, q0:q1].unsqueeze(0), el, dtype)]
    return f"len_q{len_q} len_k{len_k}", problems


@pytest.mark.parametrize("seed", [11, 12])
def test_random_shapes_against_fp32_evaluation(seed):
    from stackkernels_b200 import _lib
    random.seed(seed)
    torch.manual_seed(seed)
    failures = []
    for it in range(120):
        dtype = random.choice([torch.float16, torch.bfloat16])
        B, Hkv, group = random.randint(1, 3), random.choice([1, 2, 3]), random.choice([1, 2, 4, 8, 24, 64])
        D = random.choice([32, 64, 80, 96, 128, 160, 256])
        mode = random.choice(["prefill", "prefill", "strided", "decode", "paged", "varlen"])
        causal = random.random() < 0.6
        if mode in ("prefill", "strided", "varlen"):
            group = min(group, 8)
        desc = f"#{it} {mode} {dtype} B{B} Hq{Hkv * group} Hkv{Hkv} D{D} causal={causal}"
        if mode in ("prefill", "strided"):
            tag, problems = prefill_case(dtype, B, Hkv * group, Hkv, D, causal, mode == "strided")
        elif mode in ("decode", "paged"):
            tag, problems = decode_case(dtype, B, Hkv * group, Hkv, D, mode == "paged")
        else:
            tag, problems = varlen_case(dtype, Hkv * group, Hkv, D, causal)
        torch.cuda.synchronize()
        problems = [p for p in problems if p]
        if problems or _lib.device_status() != 0:
            failures.append((desc + " " + tag, problems, _lib.device_status()))
    assert not failures, failures[:5]
