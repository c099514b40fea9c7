"""Model-level GPU checks for the hybrid (GatedDeltaNet + gated GQA, dense and sparse-MoE) and
Gemma-style families: the committed tiny checkpoints loaded in bf16 on CUDA, through this package's
kernels, against the same checkpoint evaluated in fp32 on the CPU (whose logits are pinned to the
HF goldens by the CPU oracle tests).  Also: retired rows in the graphed decode loop.

Tolerances: the models have hidden width 32-64 and logits of order one; bf16 weights and
activations give relative errors of about 2^-8 per matmul, a few of which stack per layer, so the
full-logit check allows 6e-2 absolute, an order of magnitude below the negative-control floor of
the oracle tests' perturbations scaled to bf16 (wrong RoPE base, eps, window: > 0.3 here)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
FAMILIES = ["hybrid", "hybrid_d256", "hybrid_moe", "gemma", "llama"]


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _build(name, dtype, device, remat=False):
    """Small random models with kernel-friendly geometry (head dims 64/128/256, GatedDeltaNet heads of
    128, hidden 256), so that the bf16 CUDA path really runs this package's kernels."""
    from ferrl_b200.models import DenseGradModel, LoraSpec
    from ferrl_b200.models.gemma4 import Gemma4GradModel, Gemma4Spec
    from ferrl_b200.models.llama import llama_spec
    from ferrl_b200.models.qwen35 import MoeDims, Qwen35GradModel, Qwen35Spec
    lora = LoraSpec(8, 16.0)
    kw = dict(dtype=dtype, device=device, remat=remat)
    if name.startswith("hybrid"):
        spec = Qwen35Spec(vocab_size=1024, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=256 if name == "hybrid_d256" else 128, intermediate_size=512,
                          layer_types=["linear_attention"] * 3 + ["full_attention"], max_position_embeddings=256,
                          lin_k_heads=2, lin_v_heads=4, lin_k_dim=128, lin_v_dim=128,
                          moe=MoeDims(8, 2, 128, 128) if name == "hybrid_moe" else None)
        return Qwen35GradModel(spec, lora, **kw)
    if name == "gemma":
        spec = Gemma4Spec(vocab_size=1024, hidden_size=256, num_hidden_layers=6, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=128, global_head_dim=128, num_global_key_value_heads=2,
                          intermediate_size=512, layer_types=["sliding_attention"] * 5 + ["full_attention"],
                          sliding_window=16, max_position_embeddings=256)
        m = Gemma4GradModel(spec, lora, **kw)
        with torch.no_grad():           # scores are q.k without 1/sqrt(d): keep them of order ten, as trained norms do
            for l in m.layers:
                l.q_norm.fill_(0.3)
                l.k_norm.fill_(0.3)
        return m
    cfg = {"vocab_size": 1024, "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
           "num_key_value_heads": 2, "intermediate_size": 512, "max_position_embeddings": 256, "rms_norm_eps": 1e-5,
           "rope_theta": 10000.0, "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                   "high_freq_factor": 4.0, "original_max_position_embeddings": 64}}
    return DenseGradModel(llama_spec(cfg), lora, **kw)


def _pair(name, remat=False):
    """The same random model twice: fp32 on the CPU (frozen tensors rounded to bf16 first, so both hold
    the same values) and bf16 on CUDA."""
    cpu = _build(name, torch.float32, "cpu")
    cpu.init_random(11, 0.05)
    gpu = _build(name, torch.bfloat16, "cuda", remat)
    cn = dict(list(cpu.named_parameters()) + list(cpu.named_buffers()))
    with torch.no_grad():
        for n, tg in list(gpu.named_parameters()) + list(gpu.named_buffers()):
            tc = cn.get(n)
            if tc is None or tc.shape != tg.shape:
                continue
            if tg.dtype == torch.bfloat16:
                tc.copy_(tc.to(torch.bfloat16).float())
            tg.copy_(tc.to(tg.dtype))
        for a, b in zip(cpu.trainable_params(), gpu.trainable_params()):
            if a.shape[1] == 8:          # B matrices start at zero: give the adapter path a signal
                a.add_(0.02)
            b.copy_(a)
        for m in (cpu, gpu):
            for l in m.layers:
                for pr in l.projections():
                    if getattr(pr, "weight_t", None) is not None:
                        pr.weight_t.copy_(pr.weight.t())
            m.refresh_head()
    return cpu, gpu


def _rel(a, b):
    return float((a - b).norm() / b.norm().clamp(min=1e-12))


class _eager_bf16:
    """Run the same CUDA bf16 model through PyTorch's own kernels (the library-baseline switch): the
    yardstick for what bf16 storage with fp32 arithmetic costs on this model, independent of our kernels."""

    def __enter__(self):
        from ferrl_b200 import ops
        ops.use_library_kernels(True)

    def __exit__(self, *exc):
        from ferrl_b200 import ops
        ops.use_library_kernels(False)
        return False


def _check_against_yardstick(kernel, eager, ref, what, slack=1.6, floor=4e-3):
    """The kernel path must be about as close to the fp32 reference as PyTorch's bf16 path is (within
    ``slack``, plus a small floor), in norm and in the worst element; and the two bf16 paths must agree
    with each other far better than either agrees with a wrong model."""
    rk, re_ = _rel(kernel, ref), _rel(eager, ref)
    assert rk <= slack * re_ + floor, (what, "norm", rk, re_)
    mk, me = float((kernel - ref).abs().max()), float((eager - ref).abs().max())
    assert mk <= 2.5 * me + 10 * floor * float(ref.abs().max()), (what, "max", mk, me)


@pytest.mark.parametrize("name", FAMILIES)
def test_family_logits_on_gpu_match_cpu_fp32(name):
    _need_gpu()
    from ferrl_b200.ops import cuda as C
    cpu, gpu = _pair(name)
    ids = torch.randint(0, 1024, (2, 40), generator=torch.Generator().manual_seed(1))
    before = C.launches()
    with torch.no_grad():
        ref = cpu(ids)
        got = gpu(ids.cuda()).float().cpu()
        assert C.launches() > before                      # this package's kernels ran
        with _eager_bf16():
            yard = gpu(ids.cuda()).float().cpu()
        wrong = cpu(torch.roll(ids, 1, dims=1))
    _check_against_yardstick(got, yard, ref, name)
    assert _rel(got, ref) < 0.25 * _rel(wrong, ref)       # negative control: a wrong model is far away


@pytest.mark.parametrize("name", FAMILIES)
@pytest.mark.parametrize("remat", [False, True])
def test_family_token_logprobs_and_adapter_grads_on_gpu_match_cpu(name, remat):
    _need_gpu()
    cpu, gpu = _pair(name, remat)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 1024, (3, 48), generator=g)
    start = torch.tensor([5, 9, 2])
    targets = torch.randint(0, 1024, (3, 24), generator=g)
    w = torch.randn(3, 24, generator=g)

    def run(model, dev):
        for p in model.trainable_params():
            p.grad = None
        lp = model.token_logprobs(ids.to(dev), start.to(dev), targets.to(dev), 1.0)
        (lp * w.to(dev)).sum().backward()
        return lp.detach().float().cpu(), torch.cat([p.grad.float().cpu().reshape(-1) for p in model.trainable_params()])
    lp_ref, g_ref = run(cpu, "cpu")
    lp_k, g_k = run(gpu, "cuda")
    with _eager_bf16():
        lp_e, g_e = run(gpu, "cuda")
    assert torch.isfinite(g_k).all()
    _check_against_yardstick(lp_k, lp_e, lp_ref, name + " logprobs")
    _check_against_yardstick(g_k, g_e, g_ref, name + " adapter grads", slack=2.0, floor=1e-2)


@pytest.mark.parametrize("name", FAMILIES)
def test_family_cached_decode_on_gpu_matches_full_forward(name):
    _need_gpu()
    _, gpu = _pair(name)
    gpu.merge_adapters()
    ids = torch.randint(0, 1024, (4, 36), generator=torch.Generator().manual_seed(4)).cuda()

    def run():
        full = gpu(ids).float()
        dec = gpu.new_decoder(4, 64)
        outs = [dec.prefill(ids[:, :11], torch.full((4,), 11, device="cuda")).float()]
        for t in range(11, 36):
            outs.append(dec.decode(ids[:, t]).float())
        return full[:, 10:], torch.stack(outs, 1)
    with torch.no_grad():
        full_k, dec_k = run()
        with _eager_bf16():
            full_e, dec_e = run()
    # cached decode vs full forward of the same path: as consistent as PyTorch's own bf16 path is
    rk, re_ = _rel(dec_k, full_k), _rel(dec_e, full_e)
    assert rk <= 1.6 * re_ + 1e-2, (name, rk, re_)
    assert _rel(dec_k, full_e) < 0.2                      # and the two paths describe the same model


def test_graphed_decode_retires_finished_rows_and_leaves_live_rows_bit_identical():
    """Half of the rows emit EOS at step 8 of a 40-token rollout.  With retirement those rows' KV is not
    read from then on: the attention lengths summed over the decode steps (what the kernels are told to
    read) drop by more than 1.6x against the same rollout without an EOS id, while the tokens and
    behaviour log-probs of the rows that keep going are bit-identical."""
    _need_gpu()
    from ferrl_b200.lm_policy import GraphedDecodeStep
    from ferrl_b200.models import DenseGradModel, DenseSpec
    spec = DenseSpec(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                     head_dim=64, intermediate_size=512, max_position_embeddings=256)
    model = DenseGradModel(spec, None, dtype=torch.bfloat16, device="cuda")
    model.init_random(5, 0.3)
    model.merge_adapters()
    B, N, EOS = 8, 40, 511
    ids = torch.randint(0, 400, (B, 6), generator=torch.Generator().manual_seed(6)).cuda()
    lens = torch.full((B,), 6, device="cuda")
    stop = torch.arange(B, device="cuda") % 2 == 1

    class ScriptedSampler:
        """Greedy, except that the odd rows emit EOS at draw 8 (the draw index is a device counter)."""

        def sample(self, logits, rows, draw, temperature, top_p, draw_dev=None):
            lf = logits.float().clone()
            lf[:, EOS] = -1e30                      # nobody reaches EOS on their own
            tok = lf.argmax(-1)
            d = draw_dev if draw_dev is not None else torch.full((1,), draw, device=logits.device, dtype=torch.int32)
            tok = torch.where(stop & (d == 8), torch.full_like(tok, EOS), tok)
            return tok, torch.log_softmax(lf, -1).gather(-1, tok.clamp(max=EOS - 1)[:, None]).squeeze(-1)

    outs = {}
    for eos in (EOS, None):
        dec = model.new_decoder(B, 64)
        logits = dec.prefill(ids, lens)
        step = GraphedDecodeStep(dec, ScriptedSampler(), B, 1.0, None, eos, 0)
        tok, lp, clen = step.run(logits, torch.arange(B, device="cuda"), N, early_exit_every=0)
        outs[eos] = (tok.cpu(), lp.cpu(), clen.cpu(), int(step.kv_tokens_read) if eos is not None else None, dec.kv_len.cpu())
    tok_r, lp_r, clen_r, read_r, kvlen_r = outs[EOS]
    tok_n, lp_n, clen_n, _, kvlen_n = outs[None]
    live = ~stop.cpu()
    assert torch.equal(tok_r[live], tok_n[live]) and torch.equal(lp_r[live], lp_n[live])
    assert clen_r[~live].tolist() == [9] * int((~live).sum()) and clen_r[live].tolist() == [N] * int(live.sum())
    assert torch.all(tok_r[~live][:, 9:] == 0)
    # attention lengths handed to the kernels over the N-1 decode steps, per layer
    read_all = sum(int((6 + t + 1) * B) for t in range(N - 1))
    assert read_r is not None and read_all / read_r > 1.6, (read_all, read_r)
    assert kvlen_r[~live].max() < kvlen_n[~live].min()        # retired rows' caches stopped growing
