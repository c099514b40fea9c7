"""Language-model head log-probabilities taken in the GEMM epilogue (no logits tensor), forward and backward,
against the eager chunked log-softmax gather.  Reference behaviour: crates/ferrl/src/model.rs:523-559."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(N, H, V, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    h = (torch.randn(N, H, device="cuda", generator=g) * 0.7).bfloat16()
    w = (torch.randn(V, H, device="cuda", generator=g) * 0.05).bfloat16()
    t = torch.randint(0, V, (N,), device="cuda", generator=g)
    return h, w, t


@pytest.mark.parametrize("N,H,V,temperature,softcap", [
    (300, 256, 1000, 1.0, 0.0),          # one-SM kernel, ragged rows and a ragged last vocabulary tile
    (1536, 512, 4104, 0.7, 0.0),         # two-SM kernel
    (1100, 256, 2048, 1.0, 30.0),        # softcap (Gemma)
])
def test_head_logprob_matches_eager(N, H, V, temperature, softcap):
    from ferrl_b200.ops import cuda as C, eager
    h, w, t = _case(N, H, V)
    hs = h.clone().requires_grad_()
    lp = C.logprob_gather(hs, w, t, temperature, softcap)
    dlp = torch.randn(N, device="cuda")
    lp.backward(dlp)
    hr = h.float().requires_grad_()
    ref = eager.logprob_gather(hr, w.float(), t, temperature, softcap)
    ref.backward(dlp)
    assert lp.dtype == torch.float32 and lp.shape == (N,)
    assert (lp - ref).abs().max().item() < 2e-3 * max(1.0, ref.abs().max().item())
    rel = ((hs.grad.float() - hr.grad).norm() / hr.grad.norm()).item()
    assert rel < 1.5e-2, rel
    # elementwise: bf16 rounding of the gradient tile and of the result
    tol = 0.03 * hr.grad.abs() + 0.02 * hr.grad.pow(2).mean().sqrt()
    assert ((hs.grad.float() - hr.grad).abs() <= tol).float().mean().item() > 0.999


@pytest.mark.no_canary
def test_head_logprob_forward_allocates_nothing_of_vocabulary_width():
    from ferrl_b200.ops import cuda as C
    N, H, V = 4096, 256, 32768
    h, w, t = _case(N, H, V, 1)
    C.logprob_gather(h, w, t)          # warm-up: library handles, workspaces
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    with torch.no_grad():
        lp = C.logprob_gather(h, w, t)
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    assert torch.isfinite(lp).all()
    # a bf16 [N, V] tensor would be 256 MiB; the statistics workspace is N * V / 256 * 8 bytes = 4 MiB
    assert peak < 16 * 2 ** 20, peak


@pytest.mark.no_canary
def test_head_logprob_backward_is_bounded_by_the_row_chunk(monkeypatch):
    from ferrl_b200.ops import cuda as C
    N, H, V = 4096, 256, 32768
    h, w, t = _case(N, H, V, 2)
    monkeypatch.setattr(C, "LOGPROB_CHUNK_BYTES", 32 * 2 ** 20)     # 512 rows of the vocabulary per chunk
    hs = h.clone().requires_grad_()
    lp = C.logprob_gather(hs, w, t)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    lp.backward(torch.ones_like(lp))
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    assert peak < 96 * 2 ** 20, peak          # [N, V] bf16 would be 256 MiB
    hs2 = h.clone().requires_grad_()
    monkeypatch.setattr(C, "LOGPROB_CHUNK_BYTES", 1 << 30)
    C.logprob_gather(hs2, w, t).backward(torch.ones(N, device="cuda"))
    # chunking the rows only changes which kernel variant runs, never the mathematics
    assert ((hs.grad.float() - hs2.grad.float()).norm() / hs2.grad.float().norm()).item() < 1e-2
