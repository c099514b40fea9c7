"""Headline benchmark: GRPO step tokens/s (rollout + score + update) for Qwen3-8B LoRA.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference ...                     # the unmodified reference (if installable)

Workload (data-parallel, weak scaling): every rank runs 16 prompts x group 8 = 128
sequences per step; prompt lengths uniform in [128, 512] (synthetic token ids), completions up
to 1024 tokens sampled with the KV-cached decoder at top-p 0.95; rewards are Bernoulli(0.5)
synthetic verifier outcomes; LoRA rank 16 on all seven linear projections of every layer of a
random-init Qwen3-8B (36 layers, hidden 4096, 32q/8kv heads, head_dim 128, FFN 12288, vocab
151936) in bf16 with float32 adapters; one optimizer step per rollout including the
data-parallel LoRA gradient all-reduce, global-norm clip and AdamW.

Two timed regions of K steps each, both through ``Trainer.step`` (the public API):
  value  CUDA events around the K steps (max over ranks), barrier + synchronize on both sides
  e2e    host wall clock around K more steps; every step copies its prompt ids and scoring
         inputs from pinned host memory and reads rollout tokens, loss and metrics back
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_VALUE = None  # the reference publishes no throughput number


def reference_arm(args):
    why = ("reference is a Rust crate (no setup.py/pyproject.toml; pip: 'Neither setup.py nor pyproject.toml found') "
           "and this image has no cargo/rustc, so it cannot be installed or run here")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (read-only query)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact child we started
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_trainer(args, comm, device):
    import torch
    from ferrl_b200.config import TrainerConfig
    from ferrl_b200.lm_policy import LmPolicy
    from ferrl_b200.models import DenseGradModel, DenseSpec, LoraSpec, qwen3_8b_spec
    from ferrl_b200.rewards import RewardFn, Sample
    from ferrl_b200.sampler import GrpoSampler
    from ferrl_b200.tokenizer import SyntheticTokenizer
    from ferrl_b200.trainer import Trainer

    max_pos = (args.prompt_hi + args.max_new + 127) // 128 * 128 + 128
    if args.model == "qwen3-8b":
        spec = qwen3_8b_spec(max_pos)
    else:  # reduced geometry for bring-up only; never used for a reported number
        spec = DenseSpec(vocab_size=32768, hidden_size=1024, num_hidden_layers=4, num_attention_heads=8,
                         num_key_value_heads=2, head_dim=128, intermediate_size=3072, max_position_embeddings=max_pos)
    model = DenseGradModel(spec, LoraSpec(16, 32.0), dtype=torch.bfloat16, device=device, remat=bool(args.remat))
    model.init_random(seed=1234, std=0.02)
    # non-zero B so the adapter path carries signal from the first step (same on every rank)
    g = torch.Generator().manual_seed(99)
    with torch.no_grad():
        for p in model.trainable_params():
            if p.shape[1] == 16:
                p.copy_((torch.randn(p.shape, generator=g) * 0.01).to(p.device))
    policy = LmPolicy(model, GrpoSampler(args.seed, 1.0), score_microbatch=args.microbatch, early_exit_every=64)
    if args.no_graph:
        policy.use_cuda_graph = False

    class BernoulliVerifier(RewardFn):
        """Synthetic verifier: reward 1 with probability 1/2, a pure function of the completion text."""

        def reward(self, sample, completion):
            return float(hashlib.blake2b(completion.encode(), digest_size=1).digest()[0] & 1)

    tok = SyntheticTokenizer(spec.vocab_size, args.prompt_lo, args.prompt_hi)
    samples = [Sample(f"synthetic prompt #{i}", i) for i in range(4096)]
    cfg = TrainerConfig(steps=10 ** 6, group_size=args.group, max_new_tokens=args.max_new, temperature=1.0, mu=1,
                        beta=0.0, clip_eps=0.2, lr=1e-5, max_grad_norm=1.0, truncation_masking=False,
                        loss_type="dapo", grad_accum_steps=1, prompts_per_item=args.prompts,
                        backward_microbatch_size=args.microbatch, eos_token_id=spec.vocab_size - 1, top_p=0.95)
    fused = None
    if comm.world_size > 1 and not args.nccl_baseline:
        from ferrl_b200.parallel.dp import FusedDpStep
        fused = FusedDpStep.create(comm, policy.trainable_params(), device)
    trainer = Trainer(policy, tok, BernoulliVerifier(), samples, cfg, comm=comm, fused_dp_step=fused)
    return trainer, policy, spec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch-baseline"],
                    help="torch-baseline: the same trainer on PyTorch library kernels (eager ops, no CUDA graph, "
                         "per-tensor NCCL all-reduce) - a stand-in for the reference's execution shape")
    ap.add_argument("--model", default="qwen3-8b", choices=["qwen3-8b", "bringup"])
    ap.add_argument("--prompts", type=int, default=16)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--max-new", type=int, default=1024)
    ap.add_argument("--prompt-lo", type=int, default=128)
    ap.add_argument("--prompt-hi", type=int, default=512)
    ap.add_argument("--microbatch", type=int, default=8, help="rows per scoring/backward micro-batch")
    ap.add_argument("--remat", type=int, default=0, help="1 = recompute layer activations in backward (less memory)")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--no-graph", action="store_true", help="run decode steps eagerly (for per-kernel profiling)")
    ap.add_argument("--nccl-baseline", action="store_true", help="use per-tensor NCCL all-reduce instead of the fused DP step")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        print("warning: fewer than 3 warm-up steps", file=sys.stderr)

    import torch
    from ferrl_b200.comm import SoloComm, TorchDistComm
    from ferrl_b200.ops import cuda as C
    if args.impl == "torch-baseline":
        # stand-in comparator (the reference itself cannot be built here): the same trainer and models on
        # library kernels - cuBLAS GEMMs with the LoRA side path as separate matmuls, PyTorch SDPA for
        # scoring/backward, flash-attn's KV-cache kernel for decode, eager norms / RoPE / GLU / log-softmax,
        # host-seeded eager sampler, no CUDA graph, no paged cache, one NCCL all-reduce per gradient tensor
        from ferrl_b200 import ops as _ops
        _ops.use_library_kernels(True)
        args.no_graph = True
        args.nccl_baseline = True
        args.remat = 1          # eager ops keep fp32 intermediates alive: recompute per layer
        args.microbatch = min(args.microbatch, 4)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        comm = TorchDistComm.bootstrap(timeout_s=1800.0)
        device = comm.device
    else:
        comm = SoloComm()
        device = torch.device("cuda", 0)
        torch.cuda.set_device(device)
    if args.gpus != comm.world_size and comm.rank == 0:
        print(f"warning: --gpus {args.gpus} but world size is {comm.world_size}", file=sys.stderr)
    rank = comm.rank

    trainer, policy, spec = build_trainer(args, comm, device)
    step_idx = 0

    def barrier():
        torch.cuda.synchronize()
        comm.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        trainer.step(step_idx)
        step_idx += 1

    tokens_local = 0
    local_idx = device.index if device.index is not None else 0
    clocks = ClockSampler(local_idx)
    barrier()
    clocks.start()
    l0 = C.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    phase = {}
    for _ in range(args.steps):
        m = trainer.step(step_idx)
        step_idx += 1
        tokens_local += int(round(m.completion_len * args.prompts * args.group))
        for k, v in m.phase_ms.items():
            phase[k] = phase.get(k, 0.0) + v
    e1.record()
    barrier()
    launches = C.launches() - l0
    clk = clocks.stop()
    ms = e0.elapsed_time(e1)
    vals = comm.all_gather_bytes(json.dumps({"ms": ms, "tok": tokens_local, "rollout_ms": phase.get("rollout", 0.0)}).encode())
    vals = [json.loads(v.decode()) for v in vals]
    ms_max = max(v["ms"] for v in vals)
    tok_total = sum(v["tok"] for v in vals)
    value = tok_total / (ms_max / 1e3)
    # decode throughput: completion tokens of all ranks over the slowest rank's rollout phase (prefill included)
    rollout_ms_max = max(v["rollout_ms"] for v in vals)
    decode_tok_s = tok_total / (rollout_ms_max / 1e3) if rollout_ms_max > 0 else None

    # end-to-end pass: host wall clock, explicit H2D/D2H accounting
    policy.h2d_bytes = policy.d2h_bytes = 0
    barrier()
    t0 = time.perf_counter()
    tok2 = 0
    for _ in range(args.steps):
        m = trainer.step(step_idx)
        step_idx += 1
        tok2 += int(round(m.completion_len * args.prompts * args.group))
        _ = float(m.loss)  # loss was read back from the device inside the step
    barrier()
    wall = time.perf_counter() - t0
    vals2 = [json.loads(v.decode()) for v in comm.all_gather_bytes(json.dumps({"s": wall, "tok": tok2}).encode())]
    e2e = sum(v["tok"] for v in vals2) / max(v["s"] for v in vals2)

    if rank == 0:
        out = {
            "metric": "GRPO step tok/s (rollout+score+update) Qwen3-8B LoRA", "value": value, "unit": "tokens/s",
            "n_gpus": comm.world_size, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_VALUE) if BASELINE_VALUE else None, "dtype": "bf16",
            "data": "synthetic prompts (uniform random token ids), random-init weights, Bernoulli(0.5) rewards",
            "impl": args.impl,
            "config": {"model": "Qwen3-8B (36L, h4096, 32q/8kv, d128, ffn12288, vocab151936)" if args.model == "qwen3-8b"
                       else "bringup (NOT the named config)",
                       "global_batch": args.prompts * args.group * comm.world_size, "prompts_per_rank": args.prompts,
                       "group_size": args.group, "seq_len": f"prompt U[{args.prompt_lo},{args.prompt_hi}] + {args.max_new} new",
                       "lora": "r16 all-linear", "top_p": 0.95, "parallelism": f"dp{comm.world_size}",
                       "l2_policy": "inputs larger than L2 (16 GB of weights stream every step)",
                       "dp_step": ("single rank" if comm.world_size == 1 else
                                   "nccl per tensor" if args.nccl_baseline else "fused-peer-memory"),
                       "tokens_counted": "completion tokens"},
            "clocks": clk,
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": policy.h2d_bytes // args.steps,
                    "d2h_bytes_per_step": (policy.d2h_bytes + 64) // args.steps},
            "decode_tok_s": decode_tok_s,
            "rollout_ms_per_token": round(rollout_ms_max / args.steps / args.max_new, 4),   # one decode step of the whole batch
            "gpu_launches": int(launches),
            "phase_ms_per_step": {k: round(v / args.steps, 2) for k, v in phase.items()},
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
            "peak_reserved_gb": round(torch.cuda.max_memory_reserved() / 2 ** 30, 1),
            "alloc_retries": int(torch.cuda.memory_stats().get("num_alloc_retries", 0)),
            "remat": bool(args.remat), "microbatch_rows": args.microbatch,
        }
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
