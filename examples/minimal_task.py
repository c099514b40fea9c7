"""The smallest custom task: a reward function, a handful of samples, a byte-level policy.

    python examples/minimal_task.py

Shows the three seams a task author touches: ``Sample`` (prompt + target), a ``RewardFn`` (here
``FnReward`` around a plain function) and ``TrainerConfig``.  Counterpart of
``crates/ferrl/examples/minimal_task.rs``.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrl_b200.config import TrainerConfig  # noqa: E402
from ferrl_b200.lm_policy import LmPolicy  # noqa: E402
from ferrl_b200.models import DenseGradModel, DenseSpec, LoraSpec  # noqa: E402
from ferrl_b200.rewards import FnReward, Sample  # noqa: E402
from ferrl_b200.sampler import GrpoSampler  # noqa: E402
from ferrl_b200.tokenizer import ByteTokenizer  # noqa: E402
from ferrl_b200.trainer import Trainer  # noqa: E402


def vowel_reward(sample, completion: str) -> float:
    """Fraction of completion bytes that are the sample's target vowel."""
    return completion.count(sample.target) / max(len(completion), 1)


def main():
    tok = ByteTokenizer()
    spec = DenseSpec(vocab_size=tok.vocab_size(), hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, intermediate_size=64, max_position_embeddings=128)
    model = DenseGradModel(spec, LoraSpec(4, 8.0), dtype=torch.float32)
    model.init_random(0, 0.3)
    policy = LmPolicy(model, GrpoSampler(1, 1.0))
    samples = [Sample(f"say {v}: ", v) for v in "aeiou"]
    cfg = TrainerConfig(steps=10, group_size=6, prompts_per_item=2, max_new_tokens=8, lr=1e-2, beta=0.0,
                        truncation_masking=False, eos_token_id=ByteTokenizer.EOS)
    trainer = Trainer(policy, tok, FnReward(vowel_reward), samples, cfg)
    trainer.train()
    print("reward per step:", " ".join(f"{m.reward_mean:.3f}" for m in trainer.history))


if __name__ == "__main__":
    main()
