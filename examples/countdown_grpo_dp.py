"""Data-parallel LoRA-GRPO: one process per rank, bitwise lockstep across ranks.

    # two CPU ranks over gloo
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/countdown_grpo_dp.py --steps 3
    # one rank per GPU over NCCL + the fused peer-memory gradient step
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/countdown_grpo_dp.py --steps 3 --device cuda

Every rank holds the same adapters, draws a disjoint slice of the prompt window, and after the
reduced update all ranks must hold bit-identical parameters (checked with ``require_consensus``).
Counterpart of ``crates/ferrl/examples/countdown_grpo_dp.rs``.
"""
import argparse
import hashlib
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from examples.countdown_grpo import build  # noqa: E402
from ferrl_b200.comm import TorchDistComm  # noqa: E402
from ferrl_b200.config import TrainerConfig  # noqa: E402
from ferrl_b200.rewards import Sample  # noqa: E402
from ferrl_b200.rewards.countdown import CountdownConfig, CountdownReward, build_prompt, generate_dataset  # noqa: E402
from ferrl_b200.tokenizer import SyntheticTokenizer  # noqa: E402
from ferrl_b200.trainer import Trainer  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    args = ap.parse_args(argv)
    comm = TorchDistComm.bootstrap(backend="nccl" if args.device == "cuda" else "gloo", timeout_s=300.0)
    device = comm.device if args.device == "cuda" else torch.device("cpu")
    policy, spec = build(device)
    samples = [Sample(build_prompt(p), p) for p in generate_dataset(7, 64, CountdownConfig())]
    tok = SyntheticTokenizer(spec.vocab_size, 24, 48)
    cfg = TrainerConfig(steps=args.steps, group_size=4, prompts_per_item=4, max_new_tokens=32, beta=0.04, lr=1e-4,
                        truncation_masking=False, eos_token_id=spec.vocab_size - 1)
    fused = None
    if args.device == "cuda" and comm.world_size > 1:
        from ferrl_b200.parallel.dp import FusedDpStep
        fused = FusedDpStep.create(comm, policy.trainable_params(), device)
    trainer = Trainer(policy, tok, CountdownReward(), samples, cfg, comm=comm, fused_dp_step=fused)
    trainer.train()
    digest = hashlib.sha256(b"".join(p.detach().cpu().numpy().tobytes() for p in policy.trainable_params())).digest()
    comm.require_consensus(digest, "adapter parameters after training")
    if comm.rank == 0:
        for m in trainer.history:
            print(f"step {m.step} reward {m.reward_mean:.3f} grad_norm {m.grad_norm:.4f}")
        print(f"{comm.world_size} ranks hold identical adapters: {digest.hex()[:16]}")
    comm.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
