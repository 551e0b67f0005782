"""A decode step (KV-cache append, then split-KV decode) captured once in a CUDA graph and replayed.

A serving loop is launch-bound at small batch, so the step has to be capturable: no host synchronisation, no
host read of device data, workspace taken from the capturing allocator.  Lengths live on the device
(``cache_seqlens``), so one captured graph serves every step while the sequences grow; each replay must give the
bits of the same step run eagerly."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (64, 1, 128), (16, 16, 64), (32, 8, 256)])
def test_decode_step_replays_from_a_cuda_graph(Hq, Hkv, D):
    import stackkernels_b200 as skb
    from stackkernels_b200 import _lib
    B, cap, steps = 4, 2048, 6
    dt = torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(7)

    def rnd(*shape):
        return (torch.randn(*shape, device="cuda", generator=g) * 0.7).to(dt)
    start = torch.tensor([100, 0, 1500, cap - steps], dtype=torch.int32, device="cuda")
    k0, v0 = rnd(B, Hkv, cap, D), rnd(B, Hkv, cap, D)
    feed = [(rnd(B, Hq, 1, D), rnd(B, Hkv, 1, D), rnd(B, Hkv, 1, D)) for _ in range(steps)]

    # eager run of all steps
    kc, vc, lens = k0.clone(), v0.clone(), start.clone()
    eager = []
    for q, kn, vn in feed:
        skb.kv_cache_append(kc, vc, kn, vn, lens)
        eager.append(skb.flash_decode(q, kc, vc, cache_seqlens=lens).clone())
    eager_lens = lens.clone()

    # the same steps from one captured graph with static input buffers
    kc, vc, lens = k0.clone(), v0.clone(), start.clone()
    q_s, kn_s, vn_s = (torch.empty_like(t) for t in feed[0])
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                       # warm-up outside capture, on scratch state
        kw, vw, lw = k0.clone(), v0.clone(), start.clone()
        for _ in range(2):
            skb.kv_cache_append(kw, vw, feed[0][1], feed[0][2], lw)
            skb.flash_decode(feed[0][0], kw, vw, cache_seqlens=lw)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        skb.kv_cache_append(kc, vc, kn_s, vn_s, lens)
        out_s = skb.flash_decode(q_s, kc, vc, cache_seqlens=lens)
    # capture runs nothing: restore nothing, just replay step by step
    for i, (q, kn, vn) in enumerate(feed):
        q_s.copy_(q)
        kn_s.copy_(kn)
        vn_s.copy_(vn)
        graph.replay()
        assert torch.equal(out_s, eager[i]), f"step {i}: replay differs from the eager step"
    torch.cuda.synchronize()
    assert torch.equal(lens, eager_lens)
    assert _lib.device_status() == 0
