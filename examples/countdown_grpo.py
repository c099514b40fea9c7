"""LoRA-GRPO on synthetic countdown tasks with a tiny random-init Qwen3-architecture policy.

    python examples/countdown_grpo.py [--steps 5] [--device cpu|cuda] [--out runs/]

World size 1: 8 prompts x group 4, 32 new tokens, temperature 1.0, exact-arithmetic verifier,
clip 0.2, KL beta 0.04, AdamW lr 1e-4 on LoRA r8/alpha16 adapters of q and v.  The policy is a
2-layer, hidden-64 decoder (4 q / 2 kv heads of 16, SwiGLU 128, vocab 512, RoPE theta 1e6) in fp32,
so the whole loop runs in seconds on a CPU.  Counterpart of the reference's
``crates/ferrl/examples/countdown_grpo.rs``.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrl_b200.config import TrainerConfig  # noqa: E402
from ferrl_b200.lm_policy import LmPolicy  # noqa: E402
from ferrl_b200.models import DenseGradModel, DenseLoraTargets, DenseSpec, LoraSpec  # noqa: E402
from ferrl_b200.rewards import Sample  # noqa: E402
from ferrl_b200.rewards.countdown import CountdownConfig, CountdownReward, build_prompt, generate_dataset  # noqa: E402
from ferrl_b200.sampler import GrpoSampler  # noqa: E402
from ferrl_b200.telemetry import RunDir  # noqa: E402
from ferrl_b200.tokenizer import SyntheticTokenizer  # noqa: E402
from ferrl_b200.trainer import Trainer  # noqa: E402


def build(device="cpu", seed=0, vocab=512):
    spec = DenseSpec(vocab_size=vocab, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=16, intermediate_size=128, rope_theta=1e6,
                     max_position_embeddings=256)
    lora = LoraSpec(8, 16.0, DenseLoraTargets.legacy())
    model = DenseGradModel(spec, lora, dtype=torch.float32, device=device)
    model.init_random(seed, 0.05)
    return LmPolicy(model, GrpoSampler(seed + 1, 1.0)), spec


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    policy, spec = build(args.device)
    problems = generate_dataset(7, 64, CountdownConfig())
    samples = [Sample(build_prompt(p), p) for p in problems]
    tok = SyntheticTokenizer(spec.vocab_size, 24, 48)       # prompt tokens: uniform draws with a fixed seed
    cfg = TrainerConfig(steps=args.steps, group_size=4, prompts_per_item=8, max_new_tokens=32, temperature=1.0,
                        clip_eps=0.2, beta=0.04, lr=1e-4, truncation_masking=False, eos_token_id=spec.vocab_size - 1)
    run_dir = RunDir.create(args.out, "countdown-grpo") if args.out else None
    trainer = Trainer(policy, tok, CountdownReward(), samples, cfg, run_dir=run_dir)
    stop = trainer.train()
    for m in trainer.history:
        print(f"step {m.step:3d} reward {m.reward_mean:.3f} loss {m.loss:+.5f} kl {m.kl:.5f} grad_norm {m.grad_norm:.4f} "
              f"tokens/s {m.tokens_per_sec:.0f}")
    print("stopped:", stop.name)
    return 0


if __name__ == "__main__":
    sys.exit(main())
