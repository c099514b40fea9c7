"""Model oracles: full-position logits of every family match the committed HF-transformers
goldens, the cached (prefill + decode) path equals the uncached forward, and deliberately
wrong hyper-parameters move the logits by far more than the tolerance (negative controls)."""
import copy
import json
import os

import pytest
import torch

from ferrl_b200.models.loader import LoaderOpts, load_auto_policy, load_llama

FIX = os.path.join(os.path.dirname(__file__), "fixtures")
ORACLE_TOL = 5e-4
PERTURBATION_FLOOR = 1e-2


def _golden(name):
    return json.load(open(os.path.join(FIX, name, "golden.json")))["cases"]


def _load(name, **kw):
    fn = load_llama if name == "tiny_llama" else load_auto_policy
    return fn(os.path.join(FIX, name), LoaderOpts(**kw))[0]


def _max_err(model, case):
    ids = torch.tensor(case["input_ids"])
    ref = torch.tensor(case["logits"]).view(case["shape"])
    with torch.no_grad():
        return (model(ids) - ref).abs().max().item()


@pytest.mark.parametrize("name", ["tiny_qwen3", "tiny_llama", "tiny_qwen35", "tiny_qwen35_moe", "tiny_gemma4"])
def test_full_logits_match_hf_golden(name):
    m = _load(name)
    g = _golden(name)
    for c in ("full_b1", "full_b2"):
        assert _max_err(m, g[c]) < ORACLE_TOL


@pytest.mark.parametrize("name", ["tiny_qwen3", "tiny_llama", "tiny_gemma4"])
def test_cached_decode_equals_uncached(name):
    m = _load(name)
    ids = torch.tensor(_golden(name)["full_b2"]["input_ids"])
    B, S = ids.shape
    m.merge_adapters()
    with torch.no_grad():
        full = m(ids)
    dec = m.new_decoder(B, S + 1)
    lg = dec.prefill(ids[:, :3], torch.full((B,), 3))
    errs = [(lg - full[:, 2]).abs().max().item()]
    for t in range(3, S):
        errs.append((dec.decode(ids[:, t]) - full[:, t]).abs().max().item())
    assert max(errs) < ORACLE_TOL


@pytest.mark.parametrize("name", ["tiny_qwen35", "tiny_qwen35_moe"])
def test_hybrid_cached_split_matches_golden(name):
    m = _load(name)
    c = _golden(name)["cached_split"]
    ids = torch.tensor(c["input_ids"])
    P, S, V = c["prefill_len"], len(c["input_ids"][0]), m.spec.vocab_size
    unc = torch.tensor(c["uncached_logits"]).view(1, S, V)
    m.merge_adapters()
    dec = m.new_decoder(1, S + 1)
    errs = [(dec.prefill(ids[:, :P], torch.tensor([P])) - unc[:, P - 1]).abs().max().item()]
    for t in range(P, S):
        errs.append((dec.decode(ids[:, t]) - unc[:, t]).abs().max().item())
    assert max(errs) < ORACLE_TOL
    # a right-padded prefill must leave every row's recurrent state exactly as the unpadded one
    dec2 = m.new_decoder(2, S + 4)
    padded = torch.cat([ids[:, :P], torch.zeros(1, 3, dtype=torch.long)], 1).repeat(2, 1)
    lg = dec2.prefill(padded, torch.tensor([P, P]))
    e2 = [(lg[0] - unc[0, P - 1]).abs().max().item()]
    for t in range(P, S):
        e2.append((dec2.decode(ids[:, t].repeat(2))[1] - unc[0, t]).abs().max().item())
    assert max(e2) < ORACLE_TOL


def test_negative_controls_qwen3():
    g = _golden("tiny_qwen3")["full_b2"]
    m = _load("tiny_qwen3")
    bad = copy.deepcopy(m)
    from ferrl_b200 import ops
    cos, sin = ops.rope_tables(ops.default_inv_freq(m.spec.head_dim, 10000.0), m.spec.max_position_embeddings)
    bad.cos, bad.sin = cos, sin                      # wrong RoPE theta
    assert _max_err(bad, g) > PERTURBATION_FLOOR
    bad = copy.deepcopy(m)
    for l in bad.layers:
        l.eps = 1e-1                                  # wrong RMSNorm epsilon
    assert _max_err(bad, g) > PERTURBATION_FLOOR


def test_negative_controls_gemma_and_moe():
    g = _golden("tiny_gemma4")["full_b2"]
    m = _load("tiny_gemma4")
    bad = copy.deepcopy(m)
    for l in bad.layers:
        if l.window:
            l.window = 1                              # wrong sliding window
    assert _max_err(bad, g) > PERTURBATION_FLOOR
    g = _golden("tiny_qwen35_moe")["full_b2"]
    m = _load("tiny_qwen35_moe")
    import dataclasses
    bad = copy.deepcopy(m)
    bad_moe = dataclasses.replace(m.spec.moe, top_k=1)   # wrong top-k
    for l in bad.layers:
        l.spec = dataclasses.replace(l.spec, moe=bad_moe)
    assert _max_err(bad, g) > PERTURBATION_FLOOR


def test_lora_zero_b_is_identity_and_merge_matches_side_path():
    m = _load("tiny_qwen3")
    ids = torch.tensor(_golden("tiny_qwen3")["full_b2"]["input_ids"])
    with torch.no_grad():
        base = m(ids)
        for p in m.trainable_params():
            if p.shape[1] == m.lora.rank:
                p.add_(0.05)
        side = m(ids)
        assert (side - base).abs().max().item() > 1e-3
        m.merge_adapters()
        h = m.forward_hidden(ids, merged=True)
        from ferrl_b200 import ops
        merged = torch.nn.functional.linear(ops.rmsnorm(h, m.final_norm, m.spec.rms_norm_eps), m.head_weight())
        assert (merged - side).abs().max().item() < 1e-4
        m.set_adapter_enabled(False)
        assert (m(ids) - base).abs().max().item() < 1e-6


@pytest.mark.parametrize("sequence_parallel,remat", [(False, False), (True, False), (True, True)])
def test_tensor_parallel_matches_single_rank(sequence_parallel, remat):
    """Two thread-ranks with column/row sharded weights reproduce the unsharded logits and the
    replicated-adapter gradients sum to the unsharded gradients, with the residual stream replicated or
    sharded over the token rows."""
    from ferrl_b200.comm import run_ranks
    single = _load("tiny_qwen3")
    ids = torch.tensor(_golden("tiny_qwen3")["full_b2"]["input_ids"])
    for p in single.trainable_params():
        if p.shape[1] == single.lora.rank:
            with torch.no_grad():
                p.add_(0.03)
    want = single(ids)
    want.pow(2).sum().backward()
    ref_grads = [p.grad.clone() for p in single.trainable_params()]

    def body(comm):
        m = _load("tiny_qwen3", tp=(comm.rank, comm.world_size), remat=remat)
        m.sequence_parallel = sequence_parallel
        with torch.no_grad():
            for a, b in zip(m.trainable_params(), single.trainable_params()):
                a.copy_(b)
        out = m(ids, comm)
        out.pow(2).sum().backward()
        grads = [p.grad.contiguous() for p in m.trainable_params()]
        comm.all_reduce_sum(grads)
        return out.detach(), grads
    res = run_ranks(2, body)
    for out, grads in res:
        assert (out - want.detach()).abs().max().item() < 1e-4
        for g, r in zip(grads, ref_grads):
            assert (g - r).abs().max().item() < 1e-3 * max(1.0, r.abs().max().item())


def test_remat_gradients_equal_plain():
    a, b = _load("tiny_qwen35"), _load("tiny_qwen35", remat=True)
    ids = torch.tensor(_golden("tiny_qwen35")["full_b2"]["input_ids"])
    for m in (a, b):
        with torch.no_grad():
            for p in m.trainable_params():
                if p.shape[1] == m.lora.rank:
                    p.add_(0.02)
        m(ids).pow(2).mean().backward()
    for p, q in zip(a.trainable_params(), b.trainable_params()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6)


def test_paged_decoder_block_table_matches_contiguous_cache():
    """Block-table logic of the paged cache (shared full prompt pages, private tail and generated
    pages) on CPU: logits equal the contiguous cache's for ragged prompts over several steps."""
    import torch
    from ferrl_b200.models import DenseGradModel, DenseSpec, LoraSpec
    spec = DenseSpec(vocab_size=64, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=8, intermediate_size=64, max_position_embeddings=512)
    m = DenseGradModel(spec, LoraSpec(4, 8.0), dtype=torch.float32)
    m.init_random(3, 0.3)
    m.merge_adapters()
    lens = [5, 64, 70, 129, 1]
    P, G, steps = len(lens), 3, 4
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 64, (P, max(lens)), generator=g)
    lens_t = torch.tensor(lens)
    with torch.no_grad():
        a = m.new_decoder(P * G, 256, group=G, paged=False)
        b = m.new_decoder(P * G, 256, group=G, paged=True)
        la = a.prefill(ids, lens_t)
        a.broadcast_groups(G)
        lb = b.prefill(ids, lens_t)
        b.broadcast_groups(G)
        assert torch.allclose(la, lb)
        tok = torch.randint(0, 64, (steps, P * G), generator=g)
        for s in range(steps):
            xa, xb = a.decode(tok[s]), b.decode(tok[s])
            assert torch.allclose(xa, xb, atol=1e-5), s
    # rows of one prompt share its full pages and nothing else
    t = b.table
    assert torch.equal(t[3 * G, :2], t[3 * G + 1, :2]) and t[3 * G, 2] != t[3 * G + 1, 2]


def make_ckpt(d):
    """A random Gemma 4 checkpoint in HF naming with 4 query / 2 kv heads, so that it shards over two ranks."""
    from safetensors.torch import save_file
    cfg = json.load(open(os.path.join(FIX, "tiny_gemma4", "config.json")))
    t = cfg["text_config"]
    t.update(num_attention_heads=4, num_key_value_heads=2, num_global_key_value_heads=2, hidden_size=16, intermediate_size=32)
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    g = torch.Generator().manual_seed(5)
    H, F, D, GD, V = 16, 32, t["head_dim"], t["global_head_dim"], t["vocab_size"]
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.2
    w = {"model.embed_tokens.weight": rnd(V, H), "model.norm.weight": 1 + 0.1 * rnd(H)}
    for i, kind in enumerate(t["layer_types"]):
        b = f"model.layers.{i}."
        d_ = D if kind == "sliding_attention" else GD
        hkv = 2
        w[b + "self_attn.q_proj.weight"] = rnd(4 * d_, H)
        w[b + "self_attn.k_proj.weight"] = rnd(hkv * d_, H)
        if kind == "sliding_attention" or not t["attention_k_eq_v"]:
            w[b + "self_attn.v_proj.weight"] = rnd(hkv * d_, H)
        w[b + "self_attn.o_proj.weight"] = rnd(H, 4 * d_)
        w[b + "mlp.gate_proj.weight"] = rnd(F, H); w[b + "mlp.up_proj.weight"] = rnd(F, H); w[b + "mlp.down_proj.weight"] = rnd(H, F)
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            w[b + n + ".weight"] = 1 + 0.1 * rnd(H)
        w[b + "self_attn.q_norm.weight"] = 1 + 0.1 * rnd(d_); w[b + "self_attn.k_norm.weight"] = 1 + 0.1 * rnd(d_)
        w[b + "layer_scalar"] = torch.tensor([0.7 + 0.1 * i])
    save_file(w, os.path.join(d, "model.safetensors"))
    return t


@pytest.mark.parametrize("sequence_parallel", [False, True])
@pytest.mark.parametrize("remat", [False, True])
def test_gemma4_tensor_parallel_training_matches_single_rank(tmp_path, remat, sequence_parallel):
    """Gemma 4 is the family the reference trains tensor-parallel (with activation checkpointing):
    two thread ranks that stream only their own rows/columns of a checkpoint reproduce the
    unsharded logits, and their replicated-adapter gradients sum to the unsharded gradients."""
    from ferrl_b200.comm import run_ranks
    d = str(tmp_path)
    t = make_ckpt(d)
    ids = torch.randint(0, t["vocab_size"], (2, 10), generator=torch.Generator().manual_seed(1))
    single = load_auto_policy(d, LoaderOpts())[0]
    for p in single.trainable_params():
        if p.shape[1] == single.lora.rank:
            with torch.no_grad():
                p.add_(0.03)
    want = single(ids)
    want.pow(2).sum().backward()
    ref = [p.grad.clone() for p in single.trainable_params()]

    def body(comm):
        m = load_auto_policy(d, LoaderOpts(tp=(comm.rank, comm.world_size), remat=remat))[0]
        assert m.layers[0].qkv.weight.shape[0] * 2 == single.layers[0].qkv.weight.shape[0]      # a real shard
        m.sequence_parallel = sequence_parallel          # residual stream sharded over the token rows between projections
        with torch.no_grad():
            for a, b in zip(m.trainable_params(), single.trainable_params()):
                a.copy_(b)
        out = m(ids, comm)
        out.pow(2).sum().backward()
        grads = [p.grad.contiguous() for p in m.trainable_params()]
        comm.all_reduce_sum(grads)
        return out.detach(), grads
    for out, grads in run_ranks(2, body, timeout=120):
        assert (out - want.detach()).abs().max().item() < 1e-4
        for g, r in zip(grads, ref):
            assert (g - r).abs().max().item() < 1e-3 * max(1.0, r.abs().max().item())


def test_tensor_parallel_plan_divides_evenly_or_refuses():
    from ferrl_b200.comm import CommConfigError
    from ferrl_b200.parallel.tp import TensorParallelPlan
    p = TensorParallelPlan.new(1, 4, 32, 8, 12288)
    assert (p.local_heads, p.local_kv_heads, p.local_intermediate) == (8, 2, 3072)
    s = p.shard(4096)
    assert (s.start, s.len, s.end) == (1024, 1024, 2048)
    for args, msg in (((0, 3, 32, 8, 12288), "attention heads"), ((0, 16, 32, 8, 12288), "kv heads"),
                      ((0, 5, 40, 40, 12288), "intermediate size"), ((4, 4, 32, 8, 12288), "outside world")):
        with pytest.raises(CommConfigError, match=msg):
            TensorParallelPlan.new(*args)


def test_retired_rows_read_no_kv_and_live_rows_are_unchanged():
    """Rows that have emitted EOS stay in the fixed-shape decode batch but attend to nothing: the
    lengths handed to decode attention drop to zero for them and their cache length freezes, while
    the live rows' logits are bit-identical to a run without retirement (reference retires rows in
    lm_policy.rs:736-743)."""
    from ferrl_b200.models import DenseGradModel, DenseSpec
    spec = DenseSpec(vocab_size=97, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=8, intermediate_size=64, max_position_embeddings=64)
    m = DenseGradModel(spec, None, dtype=torch.float32)
    m.init_random(3, 0.2)
    m.merge_adapters()
    B, L = 4, 6
    ids = torch.randint(0, 97, (B, L), generator=torch.Generator().manual_seed(1))
    lens = torch.tensor([6, 4, 5, 6])
    a, b = m.new_decoder(B, 32), m.new_decoder(B, 32)
    a.prefill(ids, lens)
    b.prefill(ids, lens)
    active = torch.tensor([True, False, True, False])
    tok = torch.tensor([3, 0, 5, 0])
    before = b.kv_len.clone()
    assert int(b.kv_tokens_read(active)) == int(((before + 1) * active).sum()) < int(a.kv_tokens_read())
    for _ in range(3):
        la = a.decode(tok)
        lb = b.decode(tok, active)
        assert torch.equal(la[active], lb[active])
        assert torch.isfinite(lb).all()
    assert torch.equal(b.kv_len[active], before[active] + 3) and torch.equal(b.kv_len[~active], before[~active])


def test_gemma_sliding_layers_retain_only_their_window_and_decode_matches_uncached():
    """Sliding-attention layers keep a ring of ``sliding_window`` slots instead of the whole sequence
    (reference gemma4.rs:2327-2394): the cache of those layers does not grow with ``max_len``, and a
    ragged-prefill + long decode through the ring reproduces the uncached forward exactly."""
    model = _load("tiny_gemma4")
    model.merge_adapters()
    W = model.spec.sliding_window
    sliding = [l.window > 0 for l in model.layers]
    assert any(sliding) and not all(sliding)
    dec = model.new_decoder(2, 24)
    for s, n in zip(sliding, dec.slots):
        assert n == (W if s else 24)
    assert dec.retained_bytes() < dec.dense_bytes()
    g = torch.Generator().manual_seed(0)
    V = model.spec.vocab_size
    ids = torch.randint(0, V, (2, 16), generator=g)
    lens = torch.tensor([7, 2])                          # one prompt longer than the window, one shorter
    prompt = ids[:, :7].clone()
    logits = dec.prefill(prompt, lens)
    seqs = [ids[0, :7].tolist(), ids[1, :2].tolist()]
    for step in range(9):
        for b in range(2):
            with torch.no_grad():
                ref = model(torch.tensor([seqs[b]]))[0, -1]
            assert torch.allclose(logits[b], ref, atol=2e-4), (step, b, float((logits[b] - ref).abs().max()))
        nxt = torch.tensor([int(ids[0, 7 + step]), int(ids[1, 2 + step])])
        for b in range(2):
            seqs[b].append(int(nxt[b]))
        logits = dec.decode(nxt)


def test_policy_identity_binds_the_execution_recipe_but_no_rank_or_stream_position():
    """crates/ferrl/src/loader.rs:1358-1450 as golden cases: every option that changes what the policy computes
    changes the identity a checkpoint is bound to; the rank inside a tensor-parallel group and the adapter seed
    (which only positions a random stream) do not; the same directory loads to the same identity twice."""
    import dataclasses

    from ferrl_b200.models.lora import BaseQuantization, LoraSpec
    d = os.path.join(FIX, "tiny_qwen3")
    base = LoaderOpts()
    want = load_auto_policy(d, base)[1].digest()
    assert load_auto_policy(d, LoaderOpts())[1].digest() == want
    changed = {"LoRA rank": dataclasses.replace(base, lora=LoraSpec(base.lora.rank + 1, base.lora.alpha)),
               "LoRA alpha": dataclasses.replace(base, lora=LoraSpec(base.lora.rank, base.lora.alpha + 1.0)),
               "base dtype": dataclasses.replace(base, dtype=torch.bfloat16),
               "activation checkpointing": dataclasses.replace(base, remat=True),
               "tensor-parallel world": dataclasses.replace(base, tp=(0, 2))}
    for label, opts in changed.items():
        assert load_auto_policy(d, opts)[1].digest() != want, label
    # (the tiny fixture's widths are no multiple of the Q8_0 block, so that option is checked on the recipe itself)
    from ferrl_b200.models.loader import execution_recipe
    assert execution_recipe(dataclasses.replace(base, quantization=BaseQuantization.Q8_0)) != execution_recipe(base)
    assert load_auto_policy(d, dataclasses.replace(base, adapter_seed=base.adapter_seed + 1))[1].digest() == want
    rank0 = load_auto_policy(d, dataclasses.replace(base, tp=(0, 2)))[1].digest()
    rank1 = load_auto_policy(d, dataclasses.replace(base, tp=(1, 2)))[1].digest()
    assert rank0 == rank1                      # the rank must not split one logical policy identity


def test_hybrid_lora_target_recipes_follow_the_reference_spellings():
    """crates/ferrl/src/qwen35.rs:3524-3600: canonical recipe strings (they are written into checkpoint manifests),
    the five GatedDeltaNet projections of the all-linear recipe, and the refusal of a recipe that selects nothing."""
    from ferrl_b200.models.lora import LoraSpec
    from ferrl_b200.models.qwen35 import Qwen35GradModel, Qwen35LoraTargets as T
    assert T().canonical() == "attn:qkvo|mlp:gud|gdn:-"
    assert T.all_linear().canonical() == "attn:qkvo|mlp:gud|gdn:qzbao" == T.parse("all_linear").canonical()
    assert T("", "", "").canonical() == "attn:-|mlp:-|gdn:-" and not T("", "", "").any()
    assert T.parse("attn:qv|mlp:-|gdn:zo").canonical() == "attn:qv|mlp:-|gdn:zo"
    assert T("qkvo", "gud", "io").canonical() == "attn:qkvo|mlp:gud|gdn:qzo"          # "i" abbreviates q and z
    with pytest.raises(ValueError):
        T.parse("attn:qx|mlp:-|gdn:-")
    base = _load("tiny_qwen35")
    linear_layers = sum(1 for l in base.layers if l.kind != "full_attention")
    wide = Qwen35GradModel(base.spec, LoraSpec(2, 4.0), T.all_linear())
    assert len(wide.trainable_params()) == len(base.trainable_params()) + 2 * 5 * linear_layers
    with pytest.raises(ValueError, match="would train nothing"):
        Qwen35GradModel(base.spec, LoraSpec(2, 4.0), T("", "", ""))


def test_configured_lora_targets_reach_the_hybrid_family():
    """``policy.lora_targets`` names the dense recipe and, for the hybrid families, the GatedDeltaNet projections;
    the loader builds exactly those adapters and binds the recipe into the policy identity."""
    from ferrl_b200.models.lora import DenseLoraTargets, LoraSpec
    d = os.path.join(FIX, "tiny_qwen35")
    default, wide = load_auto_policy(d, LoaderOpts()), load_auto_policy(d, LoaderOpts(gdn_targets="qzbao"))
    narrow = load_auto_policy(d, LoaderOpts(lora=LoraSpec(4, 8.0, DenseLoraTargets.legacy())))
    assert default[0].targets.canonical() == "attn:qkvo|mlp:gud|gdn:-"
    assert wide[0].targets.canonical() == "attn:qkvo|mlp:gud|gdn:qzbao" and narrow[0].targets.canonical() == "attn:qv|mlp:-|gdn:-"
    assert len(narrow[0].trainable_params()) < len(default[0].trainable_params()) < len(wide[0].trainable_params())
    assert len({default[1].digest(), wide[1].digest(), narrow[1].digest()}) == 3
    assert "gdn:qzbao" in wide[0].lora_recipe()


def test_gemma4_config_rejections_follow_the_reference():
    """crates/ferrl/src/gemma4.rs:5752-5810: other text model types, MoE fields and per-layer embeddings are refused
    before any weight is read; an unknown top-level model type never reaches a family loader."""
    import copy

    from ferrl_b200.models.gemma4 import gemma4_spec
    cfg = json.load(open(os.path.join(FIX, "tiny_gemma4", "config.json")))
    gemma4_spec(cfg)
    for change, msg in ((dict(model_type="gemma4_unified_audio"), "model_type"), (dict(enable_moe_block=True, num_experts=128), "MoE"),
                        (dict(hidden_size_per_layer_input=128), "per-layer")):
        bad = copy.deepcopy(cfg)
        bad["text_config"].update(change)
        with pytest.raises(ValueError, match=msg):
            gemma4_spec(bad)
    unified = copy.deepcopy(cfg)
    unified["text_config"]["model_type"] = "gemma4_unified_text"
    gemma4_spec(unified)
