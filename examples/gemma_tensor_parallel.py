"""Tensor-parallel LoRA-GRPO on a Gemma-style policy.

    # two CPU ranks over gloo
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/gemma_tensor_parallel.py --steps 2
    # one rank per GPU: fused GEMM -> all-reduce projections over the symmetric heap
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        examples/gemma_tensor_parallel.py --steps 2 --device cuda
    # the same with the residual stream sharded over the token rows between the projections
    # (all-gather -> GEMM in front of the column-parallel ones, GEMM -> reduce-scatter behind the row-parallel ones)
    ... examples/gemma_tensor_parallel.py --steps 2 --device cuda --sequence-parallel

All ranks form one tensor-parallel group: they stream their own rows / columns of the checkpoint, work on the
same prompts, and hold replicated adapters whose gradients are summed once per step; after training every rank
must hold bit-identical adapters.  The checkpoint is a random Gemma 4 text model in Hugging Face naming (4 query /
2 key-value heads, so that it shards over two ranks) written to a temporary directory by rank 0; the reward is a
synthetic one that varies inside a group (the share of even token ids in the completion), so that the steps carry
gradients.  A run configuration with ``"tensor_parallel": {"enabled": true, "rank": r, "world_size": n,
"sequence_parallel": true}`` makes ``python -m ferrl_b200.cli train`` build the same objects.  The reference trains
this family tensor-parallel with activation checkpointing (``crates/ferrl/src/gemma4.rs:1929-1984``); it has no
sequence-sharded layout.
"""
import argparse
import hashlib
import json
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrl_b200.comm import TorchDistComm  # noqa: E402
from ferrl_b200.config import TrainerConfig  # noqa: E402
from ferrl_b200.lm_policy import LmPolicy  # noqa: E402
from ferrl_b200.models.loader import LoaderOpts, load_auto_policy  # noqa: E402
from ferrl_b200.models.lora import LoraSpec  # noqa: E402
from ferrl_b200.parallel.runtime import ParallelRuntime  # noqa: E402
from ferrl_b200.rewards import FnReward, Sample  # noqa: E402
from ferrl_b200.sampler import GrpoSampler  # noqa: E402
from ferrl_b200.tokenizer import SyntheticTokenizer  # noqa: E402
from ferrl_b200.trainer import Trainer  # noqa: E402

VOCAB, HIDDEN, FFN, HEADS, KV_HEADS, HEAD_DIM, GLOBAL_HEAD_DIM = 64, 32, 64, 4, 2, 8, 16
LAYER_TYPES = ["sliding_attention", "full_attention"]


def write_random_checkpoint(path: str) -> None:
    """``config.json`` + ``model.safetensors`` of a two-layer Gemma 4 text model with random weights."""
    from safetensors.torch import save_file
    text = {"model_type": "gemma4_text", "vocab_size": VOCAB, "hidden_size": HIDDEN, "intermediate_size": FFN,
            "num_hidden_layers": len(LAYER_TYPES), "num_attention_heads": HEADS, "num_key_value_heads": KV_HEADS,
            "num_global_key_value_heads": KV_HEADS, "head_dim": HEAD_DIM, "global_head_dim": GLOBAL_HEAD_DIM,
            "layer_types": LAYER_TYPES, "sliding_window": 16, "max_position_embeddings": 128, "rms_norm_eps": 1e-6,
            "attention_k_eq_v": True, "final_logit_softcapping": 30.0, "hidden_activation": "gelu_pytorch_tanh",
            "tie_word_embeddings": True, "eos_token_id": 1, "bos_token_id": 2, "pad_token_id": 0,
            "rope_parameters": {"full_attention": {"partial_rotary_factor": 0.5, "rope_theta": 1e6, "rope_type": "proportional"},
                                "sliding_attention": {"rope_theta": 1e4, "rope_type": "default"}}}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump({"model_type": "gemma4", "text_config": text}, f)
    g = torch.Generator().manual_seed(5)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.2  # noqa: E731
    w = {"model.embed_tokens.weight": rnd(VOCAB, HIDDEN), "model.norm.weight": 1 + 0.1 * rnd(HIDDEN)}
    for i, kind in enumerate(LAYER_TYPES):
        b, d = f"model.layers.{i}.", (HEAD_DIM if kind == "sliding_attention" else GLOBAL_HEAD_DIM)
        w[b + "self_attn.q_proj.weight"] = rnd(HEADS * d, HIDDEN)
        w[b + "self_attn.k_proj.weight"] = rnd(KV_HEADS * d, HIDDEN)
        if kind == "sliding_attention":                    # global layers use K as V
            w[b + "self_attn.v_proj.weight"] = rnd(KV_HEADS * d, HIDDEN)
        w[b + "self_attn.o_proj.weight"] = rnd(HIDDEN, HEADS * d)
        w[b + "mlp.gate_proj.weight"], w[b + "mlp.up_proj.weight"] = rnd(FFN, HIDDEN), rnd(FFN, HIDDEN)
        w[b + "mlp.down_proj.weight"] = rnd(HIDDEN, FFN)
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            w[b + n + ".weight"] = 1 + 0.1 * rnd(HIDDEN)
        w[b + "self_attn.q_norm.weight"], w[b + "self_attn.k_norm.weight"] = 1 + 0.1 * rnd(d), 1 + 0.1 * rnd(d)
        w[b + "layer_scalar"] = torch.tensor([0.8])
    save_file(w, os.path.join(path, "model.safetensors"))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--sequence-parallel", action="store_true")
    ap.add_argument("--out", default=None, help="run directory root (default: a temporary directory)")
    args = ap.parse_args(argv)
    comm = TorchDistComm.bootstrap(backend="nccl" if args.device == "cuda" else "gloo", timeout_s=300.0)
    root = comm.broadcast_bytes((args.out or tempfile.mkdtemp(prefix="ferrl_b200_tp_")).encode() if comm.rank == 0 else None,
                                0).decode()
    ckpt = os.path.join(root, "checkpoint")
    if comm.rank == 0:
        os.makedirs(ckpt, exist_ok=True)
        write_random_checkpoint(ckpt)
    comm.barrier()
    device = comm.device if args.device == "cuda" else torch.device("cpu")
    opts = LoaderOpts(dtype=torch.bfloat16 if args.device == "cuda" else torch.float32, device=str(device),
                      lora=LoraSpec(4, 8.0), remat=True, tp=(comm.rank, comm.world_size), adapter_seed=11)
    model, _ = load_auto_policy(ckpt, opts)
    model.sequence_parallel = bool(args.sequence_parallel)
    with torch.no_grad():                                  # non-zero B factors: both adapter halves get gradients
        for i, p in enumerate(model.trainable_params()):
            if p.shape[1] == 4:
                p.copy_(torch.randn(p.shape, generator=torch.Generator().manual_seed(100 + i)) * 0.02)
    cfg = TrainerConfig(steps=args.steps, group_size=4, prompts_per_item=2, max_new_tokens=8, beta=0.0, lr=1e-3,
                        truncation_masking=False, eos_token_id=None)
    # peer-memory runtime of the tensor-parallel group (GPUs: symmetric heap, fused projection kernels, row
    # collectives; CPU ranks: nothing to build, the collectives go through the communicator)
    runtime = ParallelRuntime.create(comm, device, tensor_parallel=True, hidden=HIDDEN,
                                     max_rows=cfg.group_size * cfg.prompts_per_item * 32,
                                     sequence_parallel=bool(args.sequence_parallel))
    policy = LmPolicy(model, GrpoSampler(7, 1.0), comm)
    samples = [Sample(f"prompt {i}", None) for i in range(16)]
    reward = FnReward(lambda sample, text: sum(1 for t in text.split() if t.isdigit() and int(t) % 2 == 0) / 8.0)
    trainer = Trainer(policy, SyntheticTokenizer(VOCAB, 4, 8), reward, samples, cfg, comm=comm, topology="tp",
                      parallel_runtime=runtime)
    trainer.train()
    digest = hashlib.sha256(b"".join(p.detach().float().cpu().numpy().tobytes() for p in policy.trainable_params())).digest()
    comm.require_consensus(digest, "adapter parameters after training")
    runtime.close()
    if comm.rank == 0:
        for m in trainer.history:
            print(f"step {m.step} reward {m.reward_mean:.3f} loss {m.loss:+.5f} grad_norm {m.grad_norm:.4f}")
        print(f"tensor-parallel world {comm.world_size}, sequence_parallel={bool(args.sequence_parallel)}: "
              f"all ranks hold identical adapters {digest.hex()[:16]}")
    comm.barrier()


if __name__ == "__main__":
    sys.exit(main())
