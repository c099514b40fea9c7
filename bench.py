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


# ---------------------------------------------------------------------------------------------
# Benchmark configurations.  "qwen3-dp" is the headline (default); the other three time the
# remaining model families / parallel layouts at their named geometries (random weights).
CONFIGS = {
    "qwen3-dp": dict(label="Qwen3-8B (36L, h4096, 32q/8kv, d128, ffn12288, vocab151936)", lora="r16 all-linear",
                     prompts=16, group=8, max_new=1024, prompt_lo=128, prompt_hi=512, microbatch=8, remat=0, beta=0.0,
                     parallelism="dp", rank_lora=16),
    "gemma-tp": dict(label="Gemma-style dense (62L, h5376, 32q/16kv, d128, GeGLU 21504, vocab262144, window 1024 at 5:1)",
                     lora="r16 attention+MLP", prompts=64, group=8, max_new=2048, prompt_lo=256, prompt_hi=256, microbatch=2,
                     remat=1, beta=0.0, parallelism="tp", rank_lora=16),
    "moe-ep": dict(label="Qwen3.5-style hybrid MoE (48L, h2048, GDN:GQA 3:1, 16q/2kv d256, GDN 16x128, 128 experts top-8 "
                         "ffn768 + shared, vocab151936)", lora="r8 attention+shared expert", prompts=16, group=8, max_new=1024,
                   prompt_lo=512, prompt_hi=512, microbatch=4, remat=1, beta=0.0, parallelism="ep", rank_lora=8),
    "hybrid27b-dp": dict(label="Qwen3.6-27B-class dense hybrid (64L, h5120, GDN:GQA 3:1, 24q/4kv d256, ffn17408, vocab151936)",
                         lora="r32 attn:qkvo|mlp:gud|gdn:qzo", prompts=4, group=16, max_new=4096, prompt_lo=1024, prompt_hi=1024, microbatch=1,
                         remat=1, beta=0.04, parallelism="dp", rank_lora=32),
}


def _build_model(args, comm, device):
    import torch
    from ferrl_b200.models import DenseGradModel, DenseSpec, LoraSpec, qwen3_8b_spec
    cfg = CONFIGS[args.config]
    max_pos = (args.prompt_hi + args.max_new + 127) // 128 * 128 + 128
    lora = LoraSpec(cfg["rank_lora"], 2.0 * cfg["rank_lora"])
    kw = dict(dtype=torch.bfloat16, device=device, remat=bool(args.remat))
    if args.config == "qwen3-dp":
        if args.model == "qwen3-8b":
            spec = qwen3_8b_spec(max_pos)
        else:  # reduced geometry for bring-up only; never used for a reported number
            spec = DenseSpec(vocab_size=32768, hidden_size=1024, num_hidden_layers=4, num_attention_heads=8,
                             num_key_value_heads=2, head_dim=128, intermediate_size=3072, max_position_embeddings=max_pos)
        return DenseGradModel(spec, lora, **kw), spec
    small = args.model == "bringup"
    if args.config == "gemma-tp":
        from ferrl_b200.models.gemma4 import Gemma4GradModel, Gemma4Spec
        from ferrl_b200.parallel.tp import TensorParallelPlan
        L = 6 if small else 62
        spec = Gemma4Spec(vocab_size=8192 if small else 262144, hidden_size=512 if small else 5376, num_hidden_layers=L,
                          num_attention_heads=32, num_key_value_heads=16, head_dim=128, global_head_dim=128,
                          num_global_key_value_heads=16, intermediate_size=2048 if small else 21504,
                          layer_types=["full_attention" if i % 6 == 5 else "sliding_attention" for i in range(L)],
                          sliding_window=1024, max_position_embeddings=max_pos)
        tp = TensorParallelPlan.new(comm.rank, comm.world_size, 32, 16, spec.intermediate_size) if comm.world_size > 1 else None
        # the frozen base is kept once (no resident transpose): 27B parameters leave no room for a second copy
        return Gemma4GradModel(spec, lora, tp=tp, keep_transpose=False,
                               sequence_parallel=bool(args.sequence_parallel and tp is not None), **kw), spec
    from ferrl_b200.models.qwen35 import MoeDims, Qwen35GradModel, Qwen35LoraTargets, Qwen35Spec
    if args.config == "moe-ep":
        L = 4 if small else 48
        spec = Qwen35Spec(vocab_size=8192 if small else 151936, hidden_size=512 if small else 2048, num_hidden_layers=L,
                          num_attention_heads=16, num_key_value_heads=2, head_dim=256, intermediate_size=768,
                          layer_types=["full_attention" if i % 4 == 3 else "linear_attention" for i in range(L)],
                          max_position_embeddings=max_pos, lin_k_heads=16, lin_v_heads=16, lin_k_dim=128, lin_v_dim=128,
                          moe=MoeDims(16 if small else 128, 8, 768, 768))
        ep = (comm.rank, comm.world_size) if comm.world_size > 1 else None
        return Qwen35GradModel(spec, lora, Qwen35LoraTargets("qkvo", "gud", ""), ep=ep, **kw), spec
    L = 4 if small else 64
    spec = Qwen35Spec(vocab_size=8192 if small else 151936, hidden_size=512 if small else 5120, num_hidden_layers=L,
                      num_attention_heads=24, num_key_value_heads=4, head_dim=256, intermediate_size=1024 if small else 17408,
                      layer_types=["full_attention" if i % 4 == 3 else "linear_attention" for i in range(L)],
                      max_position_embeddings=max_pos, lin_k_heads=16, lin_v_heads=48, lin_k_dim=128, lin_v_dim=128)
    return Qwen35GradModel(spec, lora, Qwen35LoraTargets("qkvo", "gud", "io"), keep_transpose=False, **kw), spec


def build_trainer(args, comm, device):
    import torch
    from ferrl_b200.config import TrainerConfig
    from ferrl_b200.lm_policy import LmPolicy
    from ferrl_b200.rewards import RewardFn, Sample
    from ferrl_b200.sampler import GrpoSampler
    from ferrl_b200.tokenizer import SyntheticTokenizer
    from ferrl_b200.trainer import Trainer

    cfg = CONFIGS[args.config]
    model, spec = _build_model(args, comm, device)
    model.init_random(seed=1234, std=0.02)
    # non-zero B so the adapter path carries signal from the first step (same on every rank)
    g = torch.Generator().manual_seed(99)
    r = cfg["rank_lora"]
    with torch.no_grad():
        for p in model.trainable_params():
            if p.shape[1] == r:
                p.copy_((torch.randn(p.shape, generator=g) * 0.01).to(p.device))
    topology = "tp" if cfg["parallelism"] == "tp" and comm.world_size > 1 else "dp"
    policy = LmPolicy(model, GrpoSampler(args.seed, 1.0), comm if topology == "tp" else None,
                      score_microbatch=args.microbatch, early_exit_every=0 if cfg["parallelism"] == "ep" else 64)
    if args.no_graph:
        policy.use_cuda_graph = False

    class BernoulliVerifier(RewardFn):
        """Synthetic verifier: reward 1 with probability 1/2, a pure function of the completion text."""

        def reward(self, sample, completion):
            return float(hashlib.blake2b(completion.encode(), digest_size=1).digest()[0] & 1)

    tok = SyntheticTokenizer(spec.vocab_size, args.prompt_lo, args.prompt_hi)
    samples = [Sample(f"synthetic prompt #{i}", i) for i in range(4096)]
    tcfg = TrainerConfig(steps=10 ** 6, group_size=args.group, max_new_tokens=args.max_new, temperature=1.0, mu=1,
                         beta=cfg["beta"], clip_eps=0.2, lr=1e-5, max_grad_norm=1.0, truncation_masking=False,
                         loss_type="dapo", grad_accum_steps=1, prompts_per_item=args.prompts,
                         backward_microbatch_size=args.microbatch, eos_token_id=spec.vocab_size - 1, top_p=0.95)
    fused = None
    runtime = None
    if comm.world_size > 1:
        from ferrl_b200.parallel.runtime import ParallelRuntime
        rows = args.microbatch * (args.prompt_hi + args.max_new)
        if topology == "tp":
            runtime = ParallelRuntime.create(comm, device, tensor_parallel=True, hidden=spec.hidden_size,
                                             max_rows=max(rows, args.prompts * args.group),
                                             sequence_parallel=args.sequence_parallel)
        elif cfg["parallelism"] == "ep":
            runtime = ParallelRuntime.create(comm, device, expert_parallel={
                "num_experts": spec.moe.num_experts, "hidden": spec.hidden_size, "top_k": spec.moe.top_k,
                "max_tokens": max(rows, args.prompts * args.group, args.prompts * args.prompt_hi), "capacity_factor": 2.0})
    if topology == "dp" and not args.nccl_baseline:
        # one kernel for reduce (a no-op at world 1), clip and AdamW at every world size
        from ferrl_b200.parallel.dp import FusedDpStep
        fused = FusedDpStep.create(comm, policy.trainable_params(), device)
    trainer = Trainer(policy, tok, BernoulliVerifier(), samples, tcfg, comm=comm, topology=topology, fused_dp_step=fused,
                      parallel_runtime=runtime, lockstep_model_calls=cfg["parallelism"] == "ep" and comm.world_size > 1)
    return trainer, policy, spec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch-baseline"],
                    help="torch-baseline: the same trainer on PyTorch library kernels (eager ops, no CUDA graph, "
                         "per-tensor NCCL all-reduce) - a stand-in for the reference's execution shape")
    ap.add_argument("--config", default="qwen3-dp", choices=sorted(CONFIGS),
                    help="qwen3-dp: the headline benchmark (default); gemma-tp / moe-ep / hybrid27b-dp: the other model "
                         "families at their named geometries (tensor-parallel, expert-parallel, data-parallel with a KL reference)")
    ap.add_argument("--model", default="qwen3-8b", choices=["qwen3-8b", "bringup"],
                    help="bringup: a reduced geometry of the chosen config, for plumbing checks only")
    ap.add_argument("--prompts", type=int, default=None, help="prompts per rank (per tensor-parallel group for gemma-tp)")
    ap.add_argument("--group", type=int, default=None)
    ap.add_argument("--max-new", type=int, default=None)
    ap.add_argument("--prompt-lo", type=int, default=None)
    ap.add_argument("--prompt-hi", type=int, default=None)
    ap.add_argument("--microbatch", type=int, default=None, help="rows per scoring/backward micro-batch")
    ap.add_argument("--remat", type=int, default=None, help="1 = recompute layer activations in backward (less memory)")
    ap.add_argument("--sequence-parallel", action="store_true",
                    help="gemma-tp: keep the residual stream sharded over the token rows between the projections")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--no-graph", action="store_true", help="run decode steps eagerly (for per-kernel profiling)")
    ap.add_argument("--nccl-baseline", action="store_true", help="use per-tensor NCCL all-reduce instead of the fused DP step")
    args = ap.parse_args()
    for k in ("prompts", "group", "max_new", "prompt_lo", "prompt_hi", "microbatch", "remat"):
        if getattr(args, k) is None:
            setattr(args, k, CONFIGS[args.config][k])
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
    shared_batch = CONFIGS[args.config]["parallelism"] == "tp"      # tensor-parallel ranks work on ONE batch together
    tok_total = vals[0]["tok"] if shared_batch else sum(v["tok"] for v in vals)
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
    e2e = (vals2[0]["tok"] if shared_batch else sum(v["tok"] for v in vals2)) / max(v["s"] for v in vals2)

    if rank == 0:
        out = {
            "metric": "GRPO step tok/s (rollout+score+update) " + ("Qwen3-8B LoRA" if args.config == "qwen3-dp" else args.config + " LoRA"),
            "value": value, "unit": "tokens/s",
            "n_gpus": comm.world_size, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_VALUE) if BASELINE_VALUE else None, "dtype": "bf16",
            "data": "synthetic prompts (uniform random token ids), random-init weights, Bernoulli(0.5) rewards",
            "impl": args.impl,
            "config": {"name": args.config,
                       "model": CONFIGS[args.config]["label"] if args.model == "qwen3-8b" else "bringup (NOT the named config)",
                       "global_batch": args.prompts * args.group * (1 if CONFIGS[args.config]["parallelism"] == "tp" else comm.world_size),
                       "prompts_per_rank": args.prompts,
                       "group_size": args.group, "seq_len": f"prompt U[{args.prompt_lo},{args.prompt_hi}] + {args.max_new} new",
                       "lora": CONFIGS[args.config]["lora"], "top_p": 0.95,
                       "parallelism": f"{CONFIGS[args.config]['parallelism']}{comm.world_size}",
                       "kl_beta": CONFIGS[args.config]["beta"],
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
