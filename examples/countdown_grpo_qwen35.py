"""LoRA-GRPO with a tiny hybrid GatedDeltaNet + gated-attention (Qwen3.5-style) policy.

    python examples/countdown_grpo_qwen35.py [--steps 3] [--moe] [--device cpu|cuda]

Three linear-attention layers to one full-attention layer, optional sparse-MoE feed-forward.
Counterpart of ``crates/ferrl/examples/countdown_grpo_qwen35.rs``.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrl_b200.config import TrainerConfig  # noqa: E402
from ferrl_b200.lm_policy import LmPolicy  # noqa: E402
from ferrl_b200.models import LoraSpec  # noqa: E402
from ferrl_b200.models.qwen35 import MoeDims, Qwen35GradModel, Qwen35Spec  # noqa: E402
from ferrl_b200.rewards import Sample  # noqa: E402
from ferrl_b200.rewards.countdown import CountdownConfig, CountdownReward, build_prompt, generate_dataset  # noqa: E402
from ferrl_b200.sampler import GrpoSampler  # noqa: E402
from ferrl_b200.tokenizer import SyntheticTokenizer  # noqa: E402
from ferrl_b200.trainer import Trainer  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--moe", action="store_true")
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args(argv)
    spec = Qwen35Spec(vocab_size=512, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=16, intermediate_size=128, max_position_embeddings=256,
                      layer_types=["linear_attention"] * 3 + ["full_attention"],
                      lin_k_dim=16, lin_k_heads=2, lin_v_heads=4, lin_v_dim=16,
                      moe=MoeDims(num_experts=8, top_k=2, moe_intermediate=32, shared_intermediate=32) if args.moe else None)
    dtype = torch.bfloat16 if args.device == "cuda" else torch.float32
    model = Qwen35GradModel(spec, LoraSpec(8, 16.0), dtype=dtype, device=args.device)
    model.init_random(3, 0.05)
    policy = LmPolicy(model, GrpoSampler(5, 1.0))
    samples = [Sample(build_prompt(p), p) for p in generate_dataset(7, 32, CountdownConfig())]
    tok = SyntheticTokenizer(spec.vocab_size, 16, 32)
    cfg = TrainerConfig(steps=args.steps, group_size=4, prompts_per_item=4, max_new_tokens=16, beta=0.04, lr=1e-4,
                        truncation_masking=False, eos_token_id=spec.vocab_size - 1)
    trainer = Trainer(policy, tok, CountdownReward(), samples, cfg)
    trainer.train()
    for m in trainer.history:
        print(f"step {m.step} reward {m.reward_mean:.3f} loss {m.loss:+.5f} grad_norm {m.grad_norm:.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
