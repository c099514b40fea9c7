"""Model-level GPU checks: the bf16 kernel path against the same model evaluated eagerly in fp32 on the CPU."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _models(remat=False):
    from ferrl_b200.models import DenseGradModel, DenseSpec, LoraSpec
    spec = DenseSpec(vocab_size=1024, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=64, intermediate_size=512, max_position_embeddings=256)
    cpu = DenseGradModel(copy.deepcopy(spec), LoraSpec(8, 16.0), dtype=torch.float32)
    cpu.init_random(1, 0.05)
    gpu = DenseGradModel(copy.deepcopy(spec), LoraSpec(8, 16.0), dtype=torch.bfloat16, device="cuda", remat=remat)
    with torch.no_grad():
        gpu.embed.copy_(cpu.embed)
        gpu.lm_head.copy_(cpu.lm_head)
        gpu.final_norm.copy_(cpu.final_norm)
        for lc, lg in zip(cpu.layers, gpu.layers):
            for pc, pg in zip(lc.projections(), lg.projections()):
                pg.set_weight(pc.weight.to(torch.bfloat16).cuda())
                for a, b in zip(pc.adapter_params(), pg.adapter_params()):
                    b.copy_(a)
                    if a.shape[1] == 8:  # give B a non-zero value so the LoRA path matters
                        a.add_(0.05)
                        b.add_(0.05)
            for n in ("input_norm", "post_norm", "q_norm", "k_norm"):
                getattr(lg, n).copy_(getattr(lc, n))
            # the CPU oracle uses the bf16-rounded base weights too
            for pc in lc.projections():
                pc.weight.copy_(pc.weight.to(torch.bfloat16).float())
        cpu.embed.copy_(cpu.embed.to(torch.bfloat16).float())
        cpu.lm_head.copy_(cpu.lm_head.to(torch.bfloat16).float())
        gpu.refresh_head()
    return cpu, gpu


@pytest.mark.parametrize("remat", [False, True])
def test_token_logprobs_and_grads_match_cpu(remat):
    _need_gpu()
    cpu, gpu = _models(remat)
    ids = torch.randint(0, 1024, (3, 40))
    start = torch.tensor([9, 14, 19])
    targets = torch.randint(0, 1024, (3, 16))
    from test_model_families_gpu import _check_against_yardstick, _eager_bf16
    w = torch.randn(3, 16)

    def run(model, dev):
        for p in model.trainable_params():
            p.grad = None
        lp = model.token_logprobs(ids.to(dev), start.to(dev), targets.to(dev), 1.0)
        (lp * w.to(dev)).sum().backward()
        for p in model.trainable_params():
            assert p.grad is not None and torch.isfinite(p.grad).all()
        return lp.detach().float().cpu(), torch.cat([p.grad.float().cpu().reshape(-1) for p in model.trainable_params()])
    lp_c, g_c = run(cpu, "cpu")
    lp_g, g_g = run(gpu, "cuda")
    with _eager_bf16():
        lp_e, g_e = run(gpu, "cuda")
    # The yardstick is PyTorch's own bf16 evaluation of the same GPU model: bf16 activations carry 8 bits of
    # mantissa through two layers and a 1024-way softmax, so neither path can match fp32 to better than a few
    # 1e-2 in log-prob; what the kernels owe is to be as close to fp32 as the library's bf16 path is.
    _check_against_yardstick(lp_g, lp_e, lp_c, "dense logprobs")
    _check_against_yardstick(g_g, g_e, g_c, "dense adapter grads", slack=2.0, floor=1e-2)
    assert (lp_c - lp_g).abs().max().item() < 0.15          # and an absolute ceiling on top


def test_cached_decode_matches_full_forward_on_gpu():
    _need_gpu()
    _, gpu = _models()
    gpu.merge_adapters()
    ids = torch.randint(0, 1024, (4, 24), device="cuda")
    with torch.no_grad():
        full = gpu(ids)
        dec = gpu.new_decoder(4, 32)
        lg = dec.prefill(ids[:, :10], torch.full((4,), 10, device="cuda"))
        errs = [(lg - full[:, 9]).abs().max().item()]
        for t in range(10, 24):
            lg = dec.decode(ids[:, t])
            errs.append((lg - full[:, t]).abs().max().item())
    assert max(errs) < 0.25


def test_trainer_step_on_gpu():
    _need_gpu()
    from ferrl_b200.config import TrainerConfig
    from ferrl_b200.lm_policy import LmPolicy
    from ferrl_b200.rewards import FnReward, Sample
    from ferrl_b200.sampler import GrpoSampler
    from ferrl_b200.tokenizer import SyntheticTokenizer
    from ferrl_b200.trainer import Trainer
    _, gpu = _models(True)
    pol = LmPolicy(gpu, GrpoSampler(5, 1.0))
    tok = SyntheticTokenizer(1024, 8, 20)
    samples = [Sample(f"prompt {i}", i) for i in range(8)]
    cfg = TrainerConfig(steps=2, group_size=4, max_new_tokens=12, beta=0.04, lr=1e-3, prompts_per_item=4,
                        truncation_masking=False, top_p=0.95)
    tr = Trainer(pol, tok, FnReward(lambda s, c: float(len(c) % 5)), samples, cfg)
    before = [p.detach().clone() for p in tr.params]
    m0 = tr.step(0)
    m1 = tr.step(1)
    assert m0.grad_norm > 0 and m1.grad_norm > 0
    assert any(not torch.equal(a, b.detach()) for a, b in zip(before, tr.params))
    from ferrl_b200.ops import cuda as C
    assert C.launches() > 0 and C.kernel_status() == 0


@pytest.mark.parametrize("lens", [[5, 64, 70, 129], [1, 1, 1, 1], [200, 63, 128, 65]])
def test_paged_decoder_with_shared_prompt_pages_matches_contiguous(lens):
    """Grouped rollout through the paged cache (prompt pages stored once per group, block table,
    paged append and paged decode attention) must give the logits of the contiguous cache."""
    _need_gpu()
    _, gpu = _models()
    gpu.merge_adapters()
    P, G, steps = len(lens), 3, 5
    L = max(lens)
    gen = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 1024, (P, L), generator=gen).cuda()
    lens_t = torch.tensor(lens).cuda()
    with torch.no_grad():
        a = gpu.new_decoder(P * G, 256, group=G, paged=False)
        b = gpu.new_decoder(P * G, 256, group=G, paged=True)
        la = a.prefill(ids, lens_t)
        a.broadcast_groups(G)
        lb = b.prefill(ids, lens_t)
        b.broadcast_groups(G)
        assert torch.equal(la, lb)
        assert torch.equal(a.kv_len, b.kv_len)
        tok = torch.randint(0, 1024, (steps, P * G), generator=gen).cuda()
        for s in range(steps):
            xa, xb = a.decode(tok[s]), b.decode(tok[s])
            assert float((xa - xb).abs().max()) <= 2e-2 * float(xa.abs().max()), s
    assert b.cache_bytes() > 0
