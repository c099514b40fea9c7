"""tcgen05 flash forward for head_dim 256 and sliding windows (third form of csrc/kernels/flash_tc.cu) against
the fp32 eager attention, and the backward that consumes its log-sum-exp.  Reference behaviour: the gated
GQA core of crates/ferrl/src/qwen35.rs:1240-1313 (head_dim 256) and Gemma's sliding layers
(crates/ferrl/src/gemma4.rs:898-991, window 1024, score scale 1)."""
import pytest
import torch

from _numerics import close

pytestmark = pytest.mark.gpu


def _qkv(B, S, Hq, Hkv, D, seed, amp=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = (torch.randn(B, S, Hq, D, device="cuda", generator=g) * amp).bfloat16()
    k = (torch.randn(B, S, Hkv, D, device="cuda", generator=g) * amp).bfloat16()
    v = torch.randn(B, S, Hkv, D, device="cuda", generator=g).bfloat16()
    return q, k, v


@pytest.mark.parametrize("B,S,Hq,Hkv,D,window,scale", [
    (2, 300, 4, 2, 128, 100, 128 ** -0.5),      # window cuts inside tiles, ragged length
    (1, 1536, 8, 4, 128, 1024, 1.0),            # Gemma: window 1024, no 1/sqrt(d)
    (2, 257, 4, 4, 128, 64, 128 ** -0.5),       # window smaller than a tile
    (1, 200, 4, 2, 128, 4096, 128 ** -0.5),     # window longer than the sequence
    (2, 333, 8, 1, 256, 0, 256 ** -0.5),        # head_dim 256, 64-key tiles
    (1, 1536, 16, 2, 256, 0, 256 ** -0.5),      # Qwen3.5 gated GQA geometry
    (1, 700, 4, 2, 256, 150, 256 ** -0.5),      # head_dim 256 with a window
    (1, 1, 2, 1, 256, 0, 256 ** -0.5),          # a single token
])
def test_tcgen05_flash_window_and_head_dim_256(B, S, Hq, Hkv, D, window, scale):
    from ferrl_b200.ops import cuda as C, eager
    amp = 0.25 if scale == 1.0 else 1.0          # unscaled scores: keep the logits in a sane range
    q, k, v = _qkv(B, S, Hq, Hkv, D, S + D + window, amp)
    ref = eager.attention(q.float(), k.float(), v.float(), scale=scale, causal=True, window=window)
    out = C.attention(q, k, v, scale=scale, causal=True, window=window)            # tcgen05
    warp = C.attention(q, k, v, scale=scale, causal=True, window=window, variant=1)  # warp-level kernel
    assert C.kernel_status() == 0
    close(out.float(), ref, 1.2e-2)
    close(out.float(), warp.float(), 1.2e-2)


# head dim 128 with a window runs the tcgen05 backward kernels too (window masks in both of them);
# head dim 256 takes the warp-level backward
@pytest.mark.parametrize("S,Hq,Hkv,D,window", [(300, 4, 2, 128, 100), (333, 4, 1, 256, 0), (1536, 8, 4, 128, 1024),
                                               (257, 4, 4, 128, 64), (200, 4, 2, 128, 4096), (700, 6, 2, 128, 129)])
def test_backward_through_the_tcgen05_forward(S, Hq, Hkv, D, window):
    from ferrl_b200.ops import cuda as C, eager
    scale = D ** -0.5
    q, k, v = _qkv(2, S, Hq, Hkv, D, 7)
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    out = C.attention(*leaves, scale=scale, causal=True, window=window)
    do = torch.randn_like(out)
    out.backward(do)
    refs = [t.float().requires_grad_() for t in (q, k, v)]
    eager.attention(*refs, scale=scale, causal=True, window=window).backward(do.float())
    for a, r in zip(leaves, refs):
        close(a.grad.float(), r.grad, 2e-2)
    if D == 128:        # and the two backward implementations agree with each other
        o2, lse2 = C.lib().flash_fwd(q, k, v, scale, True, window, 0, 1)
        warp = C.lib().flash_bwd(q, k, v, o2, lse2, do.contiguous(), scale, True, window, 0, 1, None)
        for a, w in zip(leaves, warp):
            close(a.grad.float(), w.float(), 2e-2)
        assert C.kernel_status() == 0
