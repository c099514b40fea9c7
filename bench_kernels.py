"""Per-kernel timings at the headline model's shapes, against the measured roofline.

    python bench_kernels.py [--only gemm,attn,...] [--iters 20] [--json out.json]
    python bench_kernels.py --profile-case gemm|gemm_2cta_256|gemm_lora|gemm_decode|decode_attn|sample|flash|flash_tc1|flash_tc2|flash_bwd|rmsnorm|swiglu|qk_norm_rope|logprob|lora_grad|moe_grouped|gdn_decode|gdn_chunk|gdn_tc_fwd|gdn_tc_bwd|flash_tc3_d256|flash_tc3_window|decode_attn_group|logprob_head   # small, for a profiler

Every kernel is timed with CUDA events on the launching stream after warm-up, with a buffer
larger than L2 written between iterations (cold L2), and reported as achieved bytes/s or FLOP/s
over the measured peaks in ``MEASURED_PEAKS.json`` (fallback 6.65 TB/s, 1.59 PFLOP/s when the
file is absent).  Shapes follow Qwen3-8B: hidden 4096, 32q/8kv heads of 128, FFN 12288, vocab
151936; decode batch 128, training micro-batch 16 x 1536 tokens.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


class Timer:
    def __init__(self, iters, flush_bytes=256 << 20):
        self.iters = iters
        self.flush = torch.empty(flush_bytes, dtype=torch.uint8, device="cuda")

    def __call__(self, fn, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            self.flush.zero_()                     # evict L2 (126 MB) between timed iterations
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2] * 1e-3            # median seconds


def profile_case(name, C):
    """A small fixed workload per kernel (inputs above the 126 MB L2, well under 2 GB on the
    device, 2 warm-up + 3 measured launches) meant to be run under a profiler that replays
    every launch many times."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    bf = torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g).to(bf)
    if name == "gemm":
        a, b = rnd(8192, 4096), rnd(8192, 4096)
        fn = lambda: C.gemm(a, b)
    elif name in ("gemm_2cta_128", "gemm_2cta_256"):
        a, b = rnd(8192, 4096), rnd(8192, 4096)
        fn = lambda: C.gemm(a, b, two_cta=int(name.rsplit("_", 1)[1]))
    elif name == "gemm_streamk":
        a, b = rnd(128, 4096), rnd(6144, 4096)
        fn = lambda: C.gemm(a, b, stream_k=1)
    elif name == "gemm_decode":
        a, b = rnd(128, 4096), rnd(24576, 4096)
        fn = lambda: C.gemm(a, b)
    elif name == "decode_attn":
        q, k, v = rnd(128, 32, 128), rnd(128, 1536, 8, 128), rnd(128, 1536, 8, 128)
        lens = torch.full((128,), 832, device=dev, dtype=torch.int32)
        fn = lambda: C.decode_attention(q, k, v, lens, scale=128 ** -0.5)
    elif name == "sample":
        logits = rnd(512, 151936)
        rows = torch.arange(512, device=dev)
        fn = lambda: C.sample_top_p(logits, 1, rows, 0, 1.0, 0.95)
    elif name == "flash":
        q, k, v = rnd(8, 1536, 32, 128), rnd(8, 1536, 8, 128), rnd(8, 1536, 8, 128)
        fn = lambda: C.attention(q, k, v, scale=128 ** -0.5, causal=True)
    elif name == "flash_warp":
        q, k, v = rnd(8, 1536, 32, 128), rnd(8, 1536, 8, 128), rnd(8, 1536, 8, 128)
        fn = lambda: C.attention(q, k, v, scale=128 ** -0.5, causal=True, variant=1)
    elif name == "rmsnorm":
        x, r, w = rnd(24576, 4096), rnd(24576, 4096), torch.ones(4096, device=dev, dtype=bf)
        fn = lambda: C.add_rmsnorm(x, r, w, 1e-6)
    elif name == "swiglu":
        gu = rnd(12288, 24576)
        fn = lambda: C.swiglu(gu)
    elif name == "qk_norm_rope":
        from ferrl_b200 import ops
        qq, kk = rnd(8, 1536, 32, 128), rnd(8, 1536, 8, 128)
        wq, wk = torch.ones(128, device=dev, dtype=bf), torch.ones(128, device=dev, dtype=bf)
        cos, sin = ops.rope_tables(ops.default_inv_freq(128, 1e6), 2048)
        cos, sin, pos = cos.to(dev), sin.to(dev), torch.arange(1536, device=dev)
        fn = lambda: C.qk_norm_rope(qq, kk, wq, wk, 1e-6, cos, sin, pos)
    elif name == "logprob":
        lg = rnd(2048, 151936)
        tg = torch.randint(0, 151936, (2048,), device=dev)
        fn = lambda: C.lib().logprob_rows(lg, tg, 1.0, 0.0)
    elif name == "gemm_lora":
        a, b, a2, b2 = rnd(8192, 4096), rnd(6144, 4096), rnd(8192, 48), rnd(6144, 48)
        fn = lambda: C.gemm(a, b, a2, b2)
    elif name == "moe_grouped":
        T_, E_, k_, H_, I_ = 8192, 64, 8, 2048, 768
        x = rnd(T_, H_)
        gate_up, down = rnd(E_, 2 * I_, H_), rnd(E_, H_, I_)
        scores, idx, counts, _ = C.moe_route(torch.randn(T_, E_, device=dev, generator=g), k_, True)
        fn = lambda: C.moe_experts(x, scores, idx, counts, gate_up, down, "silu")
    elif name == "gdn_decode":
        B_, Hk_, Hv_ = 128, 16, 32
        qd, kd, vd = rnd(B_, Hk_ * 128), rnd(B_, Hk_ * 128), rnd(B_, Hv_ * 128)
        gg = -torch.rand(B_, Hv_, device=dev)
        bb = torch.rand(B_, Hv_, device=dev)
        S = torch.zeros(B_, Hv_, 128, 128, device=dev)
        fn = lambda: C.gdn_decode_step(qd, kd, vd, gg, bb, S, True, 1e-6)
    elif name == "gdn_chunk":
        B_, T_, Hk_, Hv_ = 8, 1536, 16, 32
        qc, kc_, vc_ = rnd(B_, T_, Hk_, 128), rnd(B_, T_, Hk_, 128), rnd(B_, T_, Hv_, 128)
        gc = -torch.rand(B_, T_, Hv_, device=dev)
        bc = torch.rand(B_, T_, Hv_, device=dev)
        fn = lambda: C.gdn_chunk_fwd(qc, kc_, vc_, gc, bc)
    elif name in ("gdn_tc_fwd", "gdn_tc_bwd"):
        B_, T_, Hk_, Hv_ = 4, 1024, 16, 32
        f32 = lambda *sh: torch.randn(*sh, device=dev, generator=g)  # noqa: E731
        qn = torch.nn.functional.normalize(f32(B_, T_, Hk_, 128), dim=-1) * 128 ** -0.5
        kn = torch.nn.functional.normalize(f32(B_, T_, Hk_, 128), dim=-1)
        vv = f32(B_, T_, Hv_, 128)
        gc = -torch.rand(B_, T_, Hv_, device=dev) * 0.3
        bc = torch.rand(B_, T_, Hv_, device=dev)
        if name == "gdn_tc_fwd":
            fn = lambda: C.lib().gdn_tc_fwd(qn, kn, vv, gc, bc, None)
        else:
            saved_ = C.lib().gdn_tc_fwd(qn, kn, vv, gc, bc, None)[2:]
            dO_ = f32(B_, T_, Hv_, 128)
            fn = lambda: C.lib().gdn_tc_bwd(qn, kn, vv, bc, *saved_, dO_, None)
    elif name in ("flash_tc3_d256", "flash_tc3_window"):
        if name == "flash_tc3_d256":
            q, k, v = rnd(8, 1536, 16, 256), rnd(8, 1536, 2, 256), rnd(8, 1536, 2, 256)
            fn = lambda: C.attention(q, k, v, scale=1.0 / 16, causal=True)
        else:
            q, k, v = rnd(8, 1536, 32, 128), rnd(8, 1536, 8, 128), rnd(8, 1536, 8, 128)
            fn = lambda: C.attention(q, k, v, scale=1.0 / 16, causal=True, window=1024)
    elif name == "decode_attn_group":
        # 16 groups of 8 rows, 448 shared prompt tokens (7 pages of 64) + 384 private tokens per row, Qwen3-8B heads
        P_, G_, page_, ppr_ = 16, 8, 64, 14
        B_ = P_ * G_
        n_pages = (P_ + B_) * ppr_
        kp, vp = rnd(n_pages, page_, 8, 128), rnd(n_pages, page_, 8, 128)
        qd = rnd(B_, 32, 128)
        jj = torch.arange(ppr_, device=dev)[None, :]
        grp = torch.arange(P_, device=dev).repeat_interleave(G_)
        shared = grp[:, None] * ppr_ + jj
        private = P_ * ppr_ + torch.arange(B_, device=dev)[:, None] * ppr_ + (jj - 7).clamp(min=0)
        table = torch.where(jj < 7, shared, private).to(torch.int32).contiguous()
        prefix = torch.full((P_,), 7 * page_, device=dev, dtype=torch.int32)
        lens = torch.full((B_,), 832, device=dev, dtype=torch.int32)
        fn = lambda: C.decode_attention(qd, kp, vp, lens, scale=128 ** -0.5, block_table=table, prefix_len=prefix, group=G_)
    elif name == "logprob_head":
        hh, ww = rnd(4096, 4096), rnd(32768, 4096) * 0.02
        tg = torch.randint(0, 32768, (4096,), device=dev)
        fn = lambda: C.lib().logprob_head_fwd(hh, ww, tg, 1.0, 0.0)
    elif name == "lora_grad":
        u, xx = rnd(24576, 48), rnd(24576, 4096)
        fn = lambda: C.lib().lora_grad(u, xx)
    elif name == "flash_bwd":
        q, k, v = rnd(8, 1536, 32, 128), rnd(8, 1536, 8, 128), rnd(8, 1536, 8, 128)
        dd = rnd(8, 1536, 32, 128)
        o_, lse_ = C.lib().flash_fwd(q, k, v, 128 ** -0.5, True, 0, 0, 1)
        fn = lambda: C.lib().flash_bwd(q, k, v, o_, lse_, dd, 128 ** -0.5, True, 0, 0, 0)
    elif name == "flash_tc2":   # the default form (output and P in TMEM); "flash_tc1" is the first form
        q, k, v = rnd(8, 1536, 32, 128), rnd(8, 1536, 8, 128), rnd(8, 1536, 8, 128)
        fn = lambda: C.attention(q, k, v, scale=128 ** -0.5, causal=True, variant=0)
    elif name == "flash_tc1":
        q, k, v = rnd(8, 1536, 32, 128), rnd(8, 1536, 8, 128), rnd(8, 1536, 8, 128)
        fn = lambda: C.attention(q, k, v, scale=128 ** -0.5, causal=True, variant=2)
    else:
        raise SystemExit(f"unknown profile case {name!r}")
    evs = []
    with torch.no_grad():
        for i in range(5):
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_.record()
            fn()
            b_.record()
            evs.append((a_, b_))
    torch.cuda.synchronize()
    print(f"profile case {name}: " + " ".join(f"{x.elapsed_time(y) * 1e3:.1f}us" for x, y in evs), flush=True)
    if C.kernel_status() != 0:
        raise SystemExit(f"kernel status {C.kernel_status()}")
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=15)
    ap.add_argument("--json", default="")
    ap.add_argument("--profile-case", default="", help="run one kernel a few times on a small case and exit")
    args = ap.parse_args()
    from ferrl_b200.ops import cuda as C
    if args.profile_case:
        return profile_case(args.profile_case, C)
    only = set(filter(None, args.only.split(",")))
    want = lambda k: not only or k in only  # noqa: E731
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, flops_peak, src = peaks()
    T = Timer(args.iters)
    rows = []
    bf = torch.bfloat16

    def report(name, secs, bytes_=0, flops=0, note=""):
        bw = bytes_ / secs if bytes_ else 0
        fl = flops / secs if flops else 0
        frac = max(bw / hbm, fl / flops_peak)
        bound = "mem" if bw / hbm >= fl / flops_peak else "math"
        rows.append({"kernel": name, "us": secs * 1e6, "GBps": bw / 1e9, "TFLOPs": fl / 1e12,
                     f"frac_of_{src}": frac, "bound": bound, "note": note})
        print(f"{name:46s} {secs * 1e6:10.1f} us  {bw / 1e9:8.0f} GB/s  {fl / 1e12:8.1f} TFLOP/s  "
              f"{100 * frac:5.1f}% of {src} ({bound}) {note}", flush=True)

    H, F, V, D, HQ, HKV = 4096, 12288, 151936, 128, 32, 8
    if want("gemm"):
        shapes = [("decode qkv", 128, 6144, H), ("decode o", 128, H, H), ("decode gate_up", 128, 2 * F, H),
                  ("decode down", 128, H, F), ("decode lm_head", 128, V, H),
                  ("train qkv", 24576, 6144, H), ("train o", 24576, H, H), ("train gate_up", 24576, 2 * F, H),
                  ("train down", 24576, H, F), ("square 8192", 8192, 8192, 8192)]
        for name, M, N, K in shapes:
            a = torch.randn(M, K, device=dev, dtype=bf)
            b = torch.randn(N, K, device=dev, dtype=bf) * 0.02
            for bn in ([0] if M > 128 else [0, 64, 128]):
                s = T(lambda: C.gemm(a, b, force_bn=bn))
                report(f"gemm {name} M{M} N{N} K{K} bn{bn or 'auto'}", s, 2 * (M * K + N * K + M * N), 2 * M * N * K)
            if M <= 128:
                s = T(lambda: C.lib().decode_gemm(a, b, None, -1, 0, False))
                report(f"gemm {name} resident-activation cluster kernel", s, 2 * (M * K + N * K + M * N), 2 * M * N * K)
                s = T(lambda: C.gemm(a, b, stream_k=1))
                report(f"gemm {name} stream-k", s, 2 * (M * K + N * K + M * N), 2 * M * N * K)
                s = T(lambda: C.gemm(a, b, stream_k=-1))
                report(f"gemm {name} planner without stream-k", s, 2 * (M * K + N * K + M * N), 2 * M * N * K)
                for bn, cl in ((128, 2), (128, 4)):
                    s = T(lambda: C.gemm(a, b, force_bn=bn, cluster_k=cl))
                    report(f"gemm {name} cluster split-k bn{bn} x{cl}", s, 2 * (M * K + N * K + M * N), 2 * M * N * K)
            else:
                s = T(lambda: C.gemm(a, b, two_cta=-1))
                report(f"gemm {name} one-SM kernel", s, 2 * (M * K + N * K + M * N), 2 * M * N * K)
            s = T(lambda: torch.matmul(a, b.t()))
            report(f"  cuBLAS same shape (library reference)", s, 2 * (M * K + N * K + M * N), 2 * M * N * K)
            del a, b
        M, N, K, R = 24576, 6144, H, 48
        a = torch.randn(M, K, device=dev, dtype=bf)
        b = torch.randn(N, K, device=dev, dtype=bf) * 0.02
        a2, b2 = torch.randn(M, R, device=dev, dtype=bf), torch.randn(N, R, device=dev, dtype=bf)
        s = T(lambda: C.gemm(a, b, a2, b2))
        report("gemm train qkv + LoRA k-slab (R=48)", s, 2 * (M * K + N * K + M * N), 2 * M * N * (K + R))
        del a, b, a2, b2
    if want("gdn"):
        from ferrl_b200.models import gdn as G
        B_, T_, Hk_, Hv_ = 8, 1536, 16, 32
        qc, kc_, vc_ = (torch.randn(B_, T_, h, 128, device=dev, dtype=bf) for h in (Hk_, Hk_, Hv_))
        gc = -torch.rand(B_, T_, Hv_, device=dev) * 0.3
        bc = torch.rand(B_, T_, Hv_, device=dev)
        fl = B_ * Hv_ * (T_ // 64) * 2 * (64 * 64 * 128 * 2 + 64 * 128 * 64 * 3 + 64 * 128 * 128 * 3)
        with torch.no_grad():
            s = T(lambda: C.gdn_chunk_fwd(qc, kc_, vc_, gc, bc))
            report("gdn chunk scan fwd B8 T1536 Hv32, CUDA-core kernel", s, 0, fl)
            s = T(lambda: C.gdn_chunk_tc(qc, kc_, vc_, gc, bc))
            report("gdn chunk fwd B8 T1536 Hv32, tensor-core kernels (incl. l2norm, casts)", s, 0, fl)
            qn = torch.nn.functional.normalize(qc.float(), dim=-1) * 128 ** -0.5
            kn = torch.nn.functional.normalize(kc_.float(), dim=-1)
            vf = vc_.float()
            s = T(lambda: C.lib().gdn_tc_fwd(qn, kn, vf, gc, bc, None))
            report("gdn chunk fwd B8 T1536 Hv32, tensor-core kernels only", s, 0, fl)
        saved = C.lib().gdn_tc_fwd(qn, kn, vf, gc, bc, None)[2:]
        dO_ = torch.randn_like(vf)
        s = T(lambda: C.lib().gdn_tc_bwd(qn, kn, vf, bc, *saved, dO_, None))
        report("gdn chunk bwd B8 T1536 Hv32, tensor-core kernels only", s, 0, 3 * fl)
        del saved

        def train(fn_):
            leaves = [t.clone().requires_grad_() for t in (qc, kc_, vc_)]
            o, _ = fn_(*leaves)
            o.backward(torch.ones_like(o))
        rep_ = Hv_ // Hk_
        s = T(lambda: train(lambda a, b_, c: C.gdn_chunk_tc(a, b_, c, gc, bc)))
        report("gdn chunk fwd+bwd B8 T1536 Hv32, tensor-core kernels via autograd", s, 0, 4 * fl)
        s = T(lambda: train(lambda a, b_, c: G.gated_delta_rule_chunked(a.repeat_interleave(rep_, 2), b_.repeat_interleave(rep_, 2),
                                                                        c, gc, bc, None, use_qk_l2norm=True)))
        report("gdn chunk fwd+bwd B8 T1536 Hv32, eager chunk loop (the former training path)", s, 0, 4 * fl)
        # one decode token: the 128 x 128 fp32 state of every (row, value head) is read and written once
        for Bd, Hkd, Hvd in ((64, 16, 48), (128, 16, 16)):
            qd, kd, vd = (torch.randn(Bd, h * 128, device=dev, dtype=bf) for h in (Hkd, Hkd, Hvd))
            gg, bb = -torch.rand(Bd, Hvd, device=dev), torch.rand(Bd, Hvd, device=dev)
            Sd = torch.randn(Bd, Hvd, 128, 128, device=dev) * 0.05
            s = T(lambda: C.gdn_decode_step(qd, kd, vd, gg, bb, Sd, True, 1e-6))
            report(f"gdn decode step B{Bd} Hv{Hvd} (state in registers, 16-byte accesses)", s, 2 * Sd.numel() * 4, 0)
    if "hybrid_decode" in only:
        # one decode step of a 4-layer slice (3 GatedDeltaNet layers + 1 attention layer + final norm and head) of the two
        # hybrid geometries, replayed from a CUDA graph at cache length prompt + 2048; only on request (builds a model)
        from ferrl_b200.models.lora import LoraSpec
        from ferrl_b200.models.qwen35 import MoeDims, Qwen35GradModel, Qwen35LoraTargets, Qwen35Spec
        kinds = ["full_attention" if i % 4 == 3 else "linear_attention" for i in range(4)]
        for label, Bd, Pd, Gd, kw, lora, tg in (
                ("27B-class dense hybrid, 64 rows", 64, 1024, 16,
                 dict(hidden_size=5120, num_attention_heads=24, num_key_value_heads=4, intermediate_size=17408, lin_v_heads=48),
                 LoraSpec(rank=32, alpha=64.0), Qwen35LoraTargets("qkvo", "gud", "io")),
                ("hybrid MoE 128 experts top-8, 128 rows", 128, 512, 8,
                 dict(hidden_size=2048, num_attention_heads=16, num_key_value_heads=2, intermediate_size=768, lin_v_heads=16,
                      moe=MoeDims(128, 8, 768, 768)),
                 LoraSpec(rank=8, alpha=16.0), Qwen35LoraTargets("qkvo", "gud", ""))):
            spec = Qwen35Spec(vocab_size=V, num_hidden_layers=4, head_dim=256, layer_types=kinds, max_position_embeddings=6144,
                              lin_k_heads=16, lin_k_dim=128, lin_v_dim=128, **kw)
            model = Qwen35GradModel(spec, lora, tg, keep_transpose=False, dtype=bf, device=dev)
            model.init_random(seed=1)
            model.merge_adapters()
            dec = model.new_decoder(Bd, Pd + 3072, None)
            with torch.no_grad():
                dec.prefill(torch.randint(0, 1000, (Bd // Gd, Pd), device=dev), torch.full((Bd // Gd,), Pd, device=dev))
                dec.broadcast_groups(Gd)
                dec.kv_len += 2048
                tok = torch.randint(0, 1000, (Bd,), device=dev)
                for _ in range(3):
                    dec.decode(tok)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    dec.decode(tok)
                s = T(graph.replay)
            report(f"decode step, 4-layer slice: {label}", s, 0, 0)
            del graph, dec, model
    if want("slab"):
        # cost of the adapter k-slab as a function of its width (the k-block is 64 wide whatever R is)
        M, N, K = 24576, 6144, H
        a = torch.randn(M, K, device=dev, dtype=bf)
        b = torch.randn(N, K, device=dev, dtype=bf) * 0.02
        s = T(lambda: C.gemm(a, b))
        report("gemm train qkv, no slab", s, 2 * (M * K + N * K + M * N), 2 * M * N * K)
        for R in (16, 48, 64):
            a2, b2 = torch.randn(M, R, device=dev, dtype=bf), torch.randn(N, R, device=dev, dtype=bf)
            s = T(lambda: C.gemm(a, b, a2, b2))
            report(f"gemm train qkv + LoRA k-slab R={R}", s, 2 * (M * K + N * K + M * N), 2 * M * N * (K + R))
        del a, b, a2, b2
    if want("chain"):
        # The four projections of a decode step over LAYERS distinct weight sets, back to back in one
        # CUDA graph: what a decode step's GEMMs cost with the L2 state a real step leaves (clean
        # weight lines of the previous layer, no dirty flush buffer).  Inputs (LAYERS x 444 MB) are
        # far larger than L2, so no flush between iterations.
        LAYERS, Bd = 8, 128
        ws = [[torch.randn(n, k, device=dev, dtype=bf) * 0.02 for n, k in ((6144, H), (H, H), (2 * F, H), (H, F))]
              for _ in range(LAYERS)]
        x = torch.randn(Bd, H, device=dev, dtype=bf)
        xo = torch.randn(Bd, H, device=dev, dtype=bf)
        xf = torch.randn(Bd, F, device=dev, dtype=bf)
        wbytes = sum(w.numel() * 2 for w in ws[0])

        def chain(mm):
            for wq, wo, wg, wd in ws:
                mm(x, wq)
                mm(xo, wo)
                mm(x, wg)
                mm(xf, wd)

        def planner_pdl(a, b):
            return C.gemm(a, b, static_b=True)

        for label, mm in (("tcgen05 planner", lambda a, b: C.gemm(a, b)),
                          ("tcgen05 planner, weights prefetched under the previous kernel (dependent launch)", planner_pdl),
                          ("tcgen05 resident-activation cluster kernel (dependent launch)",
                           lambda a, b: C.lib().decode_gemm(a, b, None, -1, 0, True)),
                          ("tcgen05 resident-activation cluster kernel, no dependent launch",
                           lambda a, b: C.lib().decode_gemm(a, b, None, -1, 0, False)),
                          ("cuBLAS (library reference)", lambda a, b: torch.matmul(a, b.t()))):
            chain(mm)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                chain(mm)
            for _ in range(3):
                gr.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(args.iters):
                gr.replay()
            e1.record()
            torch.cuda.synchronize()
            s = e0.elapsed_time(e1) * 1e-3 / (args.iters * LAYERS)
            report(f"decode GEMM chain per layer B{Bd}, {label}", s, wbytes, 2 * Bd * wbytes / 2,
                   f"{LAYERS} layers per graph, inputs > L2")
        del ws
    if want("attn"):
        B, S = 16, 1536
        q = torch.randn(B, S, HQ, D, device=dev, dtype=bf, requires_grad=True)
        k = torch.randn(B, S, HKV, D, device=dev, dtype=bf, requires_grad=True)
        v = torch.randn(B, S, HKV, D, device=dev, dtype=bf, requires_grad=True)
        fl = 4 * B * HQ * S * S * D / 2
        with torch.no_grad():
            s = T(lambda: C.attention(q, k, v, scale=D ** -0.5, causal=True))
        report(f"flash fwd B{B} S{S} causal (tcgen05, output and P in TMEM, lazy rescale)", s, 2 * B * S * (2 * HQ + 2 * HKV) * D, fl)
        with torch.no_grad():
            s = T(lambda: C.attention(q, k, v, scale=D ** -0.5, causal=True, variant=2))
        report(f"flash fwd B{B} S{S} causal (tcgen05, first form: output in registers)", s, 2 * B * S * (2 * HQ + 2 * HKV) * D, fl)
        with torch.no_grad():
            s = T(lambda: C.attention(q, k, v, scale=D ** -0.5, causal=True, variant=3))
        report(f"flash fwd B{B} S{S} causal (tcgen05, output in TMEM, P through shared memory)", s, 2 * B * S * (2 * HQ + 2 * HKV) * D, fl)
        with torch.no_grad():
            s = T(lambda: C.attention(q, k, v, scale=D ** -0.5, causal=True, variant=1))
        report(f"flash fwd B{B} S{S} causal (warp-level mma.sync)", s, 2 * B * S * (2 * HQ + 2 * HKV) * D, fl)
        o = C.attention(q, k, v, scale=D ** -0.5, causal=True)
        do = torch.randn_like(o)
        s = T(lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True))
        report(f"flash bwd B{B} S{S} causal (tcgen05, dQ + dK/dV kernels)", s, 0, 2.5 * fl, "5 matmuls of the algorithm counted (the two kernels run 7)")
        with torch.no_grad():
            o2, lse2 = C.lib().flash_fwd(q, k, v, D ** -0.5, True, 0, 0, 1)
            s = T(lambda: C.lib().flash_bwd(q, k, v, o2, lse2, do, D ** -0.5, True, 0, 0, 1))
        report(f"flash bwd B{B} S{S} causal (warp-level mma.sync)", s, 0, 2.5 * fl, "5 matmuls")
        with torch.no_grad():
            W_ = 1024
            flw = 4 * B * HQ * D * (S * W_ - W_ * W_ / 2)          # visible (query, key) pairs with a 1024-key window
            s = T(lambda: C.attention(q, k, v, scale=1.0 / 16, causal=True, window=W_))
            report(f"flash fwd B{B} S{S} window {W_} (tcgen05, third form)", s, 0, flw)
            s = T(lambda: C.attention(q, k, v, scale=1.0 / 16, causal=True, window=W_, variant=1))
            report(f"flash fwd B{B} S{S} window {W_} (warp-level mma.sync)", s, 0, flw)
            ow, lsew = C.lib().flash_fwd(q, k, v, 1.0 / 16, True, W_, 0, 0)
            s = T(lambda: C.lib().flash_bwd(q, k, v, ow, lsew, do, 1.0 / 16, True, W_, 0, 0, None))
            report(f"flash bwd B{B} S{S} window {W_} (tcgen05, dQ + dK/dV kernels)", s, 0, 2.5 * flw, "5 matmuls")
            s = T(lambda: C.lib().flash_bwd(q, k, v, ow, lsew, do, 1.0 / 16, True, W_, 0, 1, None))
            report(f"flash bwd B{B} S{S} window {W_} (warp-level mma.sync)", s, 0, 2.5 * flw, "5 matmuls")
            q2 = torch.randn(B, S, 16, 256, device=dev, dtype=bf)
            k2 = torch.randn(B, S, 2, 256, device=dev, dtype=bf)
            v2 = torch.randn(B, S, 2, 256, device=dev, dtype=bf)
            fl2 = 4 * B * 16 * S * S * 256 / 2
            s = T(lambda: C.attention(q2, k2, v2, scale=1.0 / 16, causal=True))
            report(f"flash fwd B{B} S{S} 16q/2kv head_dim 256 (tcgen05, third form, 64-key tiles)", s, 0, fl2)
            s = T(lambda: C.attention(q2, k2, v2, scale=1.0 / 16, causal=True, variant=1))
            report(f"flash fwd B{B} S{S} 16q/2kv head_dim 256 (warp-level mma.sync)", s, 0, fl2)
            del q2, k2, v2
        Bd, Smax = 128, 1536
        qd = torch.randn(Bd, HQ, D, device=dev, dtype=bf)
        kc = torch.randn(Bd, Smax, HKV, D, device=dev, dtype=bf)
        vc = torch.randn(Bd, Smax, HKV, D, device=dev, dtype=bf)
        lens = torch.full((Bd,), 832, device=dev, dtype=torch.int32)
        s = T(lambda: C.decode_attention(qd, kc, vc, lens, scale=D ** -0.5))
        report("decode attention B128 len832 (tensor-core pipeline)", s, 2 * Bd * 832 * HKV * D * 2, 4 * Bd * HQ * 832 * D)
        s = T(lambda: C.decode_attention(qd, kc, vc, lens, scale=D ** -0.5, variant=2))
        report("decode attention B128 len832 (scalar pipeline)", s, 2 * Bd * 832 * HKV * D * 2, 4 * Bd * HQ * 832 * D)
        s = T(lambda: C.decode_attention(qd, kc, vc, lens, scale=D ** -0.5, variant=1))
        report("decode attention B128 len832 (register kernel)", s, 2 * Bd * 832 * HKV * D * 2, 4 * Bd * HQ * 832 * D)
        lens2 = torch.full((Bd,), 1500, device=dev, dtype=torch.int32)
        s = T(lambda: C.decode_attention(qd, kc, vc, lens2, scale=D ** -0.5))
        report("decode attention B128 len1500 (tensor-core pipeline)", s, 2 * Bd * 1500 * HKV * D * 2, 4 * Bd * HQ * 1500 * D)
    if want("rows"):
        x = torch.randn(24576, H, device=dev, dtype=bf)
        r = torch.randn(24576, H, device=dev, dtype=bf)
        w = torch.ones(H, device=dev, dtype=bf)
        with torch.no_grad():
            s = T(lambda: C.rmsnorm(x, w, 1e-6))
            report("rmsnorm 24576x4096", s, 2 * x.numel() * 2)
            s = T(lambda: C.add_rmsnorm(x, r, w, 1e-6))
            report("add_rmsnorm 24576x4096", s, 4 * x.numel() * 2)
            gu = torch.randn(24576, 2 * F, device=dev, dtype=bf)
            s = T(lambda: C.swiglu(gu))
            report("swiglu 24576x24576", s, 3 * 24576 * F * 2)
            del gu
            xd = torch.randn(128, H, device=dev, dtype=bf)
            s = T(lambda: C.rmsnorm(xd, w, 1e-6))
            report("rmsnorm decode 128x4096 (launch bound)", s, 2 * xd.numel() * 2)
    if want("vocab"):
        logits = torch.randn(128, V, device=dev, dtype=bf)
        rows_ = torch.arange(128, device=dev)
        s = T(lambda: C.sample_top_p(logits, 1, rows_, 0, 1.0, 0.95))
        report("sample top-p 128 x 151936", s, logits.numel() * 2)
        s = T(lambda: C.sample_top_p(logits, 1, rows_, 0, 1.0, None))
        report("sample (no nucleus) 128 x 151936", s, logits.numel() * 2)
        N = 4096
        lg = torch.randn(N, V, device=dev, dtype=bf)
        tg = torch.randint(0, V, (N,), device=dev)
        s = T(lambda: C.lib().logprob_rows(lg, tg, 1.0, 0.0))
        report("logprob rows 4096 x 151936", s, lg.numel() * 2)
    if want("opt"):
        shapes = [(16, 4096)] * 252 + [(4096, 16)] * 252
        p = [torch.randn(s_, device=dev) for s_ in shapes]
        g = [torch.randn(s_, device=dev) for s_ in shapes]
        m = [torch.zeros(s_, device=dev) for s_ in shapes]
        v = [torch.zeros(s_, device=dev) for s_ in shapes]
        n = sum(t.numel() for t in p)
        s = T(lambda: C.adamw_step(p, g, m, v, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1,
                                   max_norm=1.0, compute_norm=True))
        report(f"adamw + norm + clip, {len(p)} tensors {n / 1e6:.1f}M", s, n * 4 * 8)
        from ferrl_b200.grpo import LossConfig, grpo_loss
        G, L = 128, 1024
        lp = (-torch.rand(G, L, device=dev)).requires_grad_(True)
        lo, lr_ = lp.detach() + 0.1 * torch.randn(G, L, device=dev), lp.detach() + 0.1 * torch.randn(G, L, device=dev)
        adv, mask = torch.randn(G, device=dev), (torch.rand(G, L, device=dev) > 0.2).float()
        cfg = LossConfig(0.2, 0.28, 0.04)

        def loss_fb():
            lp.grad = None
            grpo_loss(lp, lo, lr_, adv, mask, cfg).backward()

        s = T(loss_fb)
        report(f"GRPO loss forward + backward {G} x {L} (one kernel + row scaling)", s, G * L * 4 * 6)
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"peaks": {"hbm_Bps": hbm, "bf16_flops": flops_peak, "source": src}, "rows": rows}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
