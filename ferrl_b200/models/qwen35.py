"""Qwen3.5 / Qwen3.6 hybrid decoder: GatedDeltaNet linear-attention layers
interleaved with gated GQA full-attention layers, dense or sparse-MoE MLPs.

Reference: ``crates/ferrl/src/qwen35.rs`` - config ``:178-272``, ``MoeDims``
``:277``, LoRA targets (attn qkvo, mlp gud, gdn opt-in) with canonical string
``attn:..|mlp:..|gdn:..`` ``:735-887``, GDN layer ``:1062-1161``, gated GQA
core (q_proj emits ``[query | gate]`` per head, zero-centred QK-norm, partial
RoPE, fp32 softmax, sigmoid output gate) ``:1240-1313``, sparse MoE layer
``:1502-1619``, chunked norm+head+logprob tail ``:2059-2101``, remat
``:2110-2137``, merged decoder with conv / recurrent / KV state
``:2522-2637``.  Tensor parallelism is not offered for this family, as in the
reference.

B200 layout: per layer ONE fused input projection (full attention:
``[query | gate | k | v]`` with the per-head interleave of the checkpoint
undone at load time so heads are packed; GDN: ``[qkv | z | b | a]``), one
fused gate|up projection, LoRA deltas as extra k-tiles.  Padded prompt
positions are neutralised inside the delta rule (``beta = 0, g = 0``) so a
right-padded batch of unequal prompts prefills in one pass and every row's
recurrent state is exact.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..comm import Comm, SoloComm
from ..remat import remat_segment
from . import gdn as G
from . import moe as M
from .lora import BaseQuantization, FusedLoraLinear, LoraSpec


@dataclass(frozen=True)
class MoeDims:
    num_experts: int
    top_k: int
    moe_intermediate: int
    shared_intermediate: int
    norm_topk_prob: bool = True


@dataclass(frozen=True)
class Qwen35LoraTargets:
    attn: str = "qkvo"
    mlp: str = "gud"
    # opt-in GatedDeltaNet projections, the reference's letters (crates/ferrl/src/qwen35.rs:735-887): q = in_proj_qkv,
    # z = in_proj_z, b = in_proj_b, a = in_proj_a, o = out_proj; "i" is shorthand for "qz"
    gdn: str = ""

    def gdn_letters(self) -> str:
        want = set(self.gdn.replace("i", "qz"))
        return "".join(c for c in "qzbao" if c in want)

    def canonical(self) -> str:
        return f"attn:{self.attn or '-'}|mlp:{self.mlp or '-'}|gdn:{self.gdn_letters() or '-'}"

    def any(self) -> bool:
        return bool(self.attn or self.mlp or self.gdn)

    @staticmethod
    def all_linear() -> "Qwen35LoraTargets":
        return Qwen35LoraTargets("qkvo", "gud", "qzbao")

    @staticmethod
    def parse(s: str) -> "Qwen35LoraTargets":
        if s in ("industrial", "all"):
            return Qwen35LoraTargets()
        if s == "all_linear":
            return Qwen35LoraTargets.all_linear()
        if s == "attention_shared":
            return Qwen35LoraTargets("qkvo", "gud", "")
        parts = dict(p.split(":") for p in s.split("|"))
        clean = lambda v: "" if v == "-" else v  # noqa: E731
        t = Qwen35LoraTargets(clean(parts.get("attn", "-")), clean(parts.get("mlp", "-")), clean(parts.get("gdn", "-")))
        if set(t.attn) - set("qkvo") or set(t.mlp) - set("gud") or set(t.gdn) - set("qzbaoi"):
            raise ValueError(f"bad LoRA target string {s!r}")
        return t


@dataclass
class Qwen35Spec:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    layer_types: list
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = True
    rope_theta: float = 1e7
    partial_rotary_factor: float = 0.25
    max_position_embeddings: int = 4096
    conv_kernel: int = 4
    lin_k_dim: int = 128
    lin_k_heads: int = 16
    lin_v_heads: int = 32
    lin_v_dim: int = 128
    activation: str = "silu"
    moe: Optional[MoeDims] = None

    @property
    def rot_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor) // 2 * 2

    def validate(self) -> None:
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types must list every layer")
        if any(t not in ("linear_attention", "full_attention") for t in self.layer_types):
            raise ValueError("unknown layer type")
        if self.num_attention_heads % self.num_key_value_heads or self.lin_v_heads % self.lin_k_heads:
            raise ValueError("head counts must divide")
        if self.moe and self.moe.top_k > self.moe.num_experts:
            raise ValueError("top_k exceeds num_experts")


def qwen35_spec(cfg: Mapping[str, Any]) -> Qwen35Spec:
    t = cfg.get("text_config", cfg)
    rope = t.get("rope_parameters") or {}
    L = int(t["num_hidden_layers"])
    types = t.get("layer_types")
    if types is None:
        every = int(t.get("full_attention_interval", 4))
        types = ["full_attention" if (i + 1) % every == 0 else "linear_attention" for i in range(L)]
    moe = None
    if int(t.get("num_experts", 0) or 0) > 0:
        moe = MoeDims(int(t["num_experts"]), int(t["num_experts_per_tok"]), int(t["moe_intermediate_size"]),
                      int(t.get("shared_expert_intermediate_size", 0)), bool(t.get("norm_topk_prob", True)))
    heads = int(t["num_attention_heads"])
    spec = Qwen35Spec(
        vocab_size=int(t["vocab_size"]), hidden_size=int(t["hidden_size"]), num_hidden_layers=L,
        num_attention_heads=heads, num_key_value_heads=int(t.get("num_key_value_heads", heads)),
        head_dim=int(t.get("head_dim") or int(t["hidden_size"]) // heads),
        intermediate_size=int(t.get("intermediate_size", 0) or 0), layer_types=list(types),
        rms_norm_eps=float(t.get("rms_norm_eps", 1e-6)),
        tie_word_embeddings=bool(t.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False))),
        rope_theta=float(rope.get("rope_theta", t.get("rope_theta", 1e7))),
        partial_rotary_factor=float(rope.get("partial_rotary_factor", t.get("partial_rotary_factor", 0.25))),
        max_position_embeddings=int(t.get("max_position_embeddings", 4096)),
        conv_kernel=int(t.get("linear_conv_kernel_dim", 4)), lin_k_dim=int(t.get("linear_key_head_dim", 128)),
        lin_k_heads=int(t.get("linear_num_key_heads", 16)), lin_v_heads=int(t.get("linear_num_value_heads", 32)),
        lin_v_dim=int(t.get("linear_value_head_dim", 128)), activation=str(t.get("hidden_act", "silu")), moe=moe)
    spec.validate()
    return spec


class _Mlp(nn.Module):
    def __init__(self, hidden, inter, lora, tg: Qwen35LoraTargets, kw, act):
        super().__init__()
        self.gate_up = FusedLoraLinear(hidden, [inter, inter], ("gate", "up"), ("g" in tg.mlp, "u" in tg.mlp), lora, **kw)
        self.down = FusedLoraLinear(inter, [hidden], ("down",), ("d" in tg.mlp,), lora, **kw)
        self.act = act

    def forward(self, x, merged=False, residual=None):
        """``residual`` (the layer's stream) is added in the down projection's GEMM epilogue."""
        if merged:
            return self.down.forward_merged(ops.swiglu(self.gate_up.forward_merged(x), self.act), residual)
        return self.down(ops.swiglu(self.gate_up(x), self.act), residual)

    def projections(self):
        return (self.gate_up, self.down)


class Qwen35Layer(nn.Module):
    def __init__(self, spec: Qwen35Spec, kind: str, lora: Optional[LoraSpec], tg: Qwen35LoraTargets, dtype, device,
                 keep_transpose, quant, trainable_base=False, ep_world: int = 1):
        super().__init__()
        self.spec, self.kind = spec, kind
        H, D = spec.hidden_size, spec.head_dim
        kw = dict(dtype=dtype, device=device, keep_transpose=keep_transpose, quant=quant, trainable_base=trainable_base)
        buf = (lambda n, v=0.0: nn.Parameter(torch.full((n,), v, dtype=dtype, device=device)) if trainable_base
               else torch.full((n,), v, dtype=dtype, device=device))

        def reg(name, t):
            if isinstance(t, nn.Parameter):
                setattr(self, name, t)
            else:
                self.register_buffer(name, t, persistent=False)
        reg("input_norm", buf(H))
        reg("post_norm", buf(H))
        if kind == "full_attention":
            hq, hkv = spec.num_attention_heads, spec.num_key_value_heads
            self.hq, self.hkv, self.D = hq, hkv, D
            self.inp = FusedLoraLinear(H, [2 * hq * D, hkv * D, hkv * D], ("q", "k", "v"),
                                       ("q" in tg.attn, "k" in tg.attn, "v" in tg.attn), lora, **kw)
            self.out = FusedLoraLinear(hq * D, [H], ("o",), ("o" in tg.attn,), lora, **kw)
            reg("q_norm", buf(D))
            reg("k_norm", buf(D))
            self.scale = D ** -0.5
        else:
            self.kh, self.vh, self.kd, self.vd = spec.lin_k_heads, spec.lin_v_heads, spec.lin_k_dim, spec.lin_v_dim
            self.key_dim, self.value_dim = self.kh * self.kd, self.vh * self.vd
            self.conv_dim = 2 * self.key_dim + self.value_dim
            g = tg.gdn_letters()
            self.inp = FusedLoraLinear(H, [self.conv_dim, self.value_dim, self.vh, self.vh], ("qkv", "z", "b", "a"),
                                       ("q" in g, "z" in g, "b" in g, "a" in g), lora, **kw)
            self.out = FusedLoraLinear(self.value_dim, [H], ("out",), ("o" in g,), lora, **kw)
            reg("conv_w", torch.zeros(self.conv_dim, spec.conv_kernel, dtype=dtype, device=device))
            reg("A_log", torch.zeros(self.vh, dtype=torch.float32, device=device))
            reg("dt_bias", torch.ones(self.vh, dtype=torch.float32, device=device))
            reg("gdn_norm", buf(self.vd, 1.0))
        if spec.moe is None:
            self.mlp = _Mlp(H, spec.intermediate_size, lora, tg, kw, spec.activation)
            self.shared = None
        else:
            m = spec.moe
            self.mlp = None
            self.shared = _Mlp(H, m.shared_intermediate, lora, tg, kw, spec.activation) if m.shared_intermediate else None
            reg("router", torch.zeros(m.num_experts, H, dtype=dtype, device=device))
            e_local = m.num_experts // ep_world          # expert parallelism: this rank's contiguous block of experts
            reg("experts_gate_up", torch.zeros(e_local, 2 * m.moe_intermediate, H, dtype=dtype, device=device))
            reg("experts_down", torch.zeros(e_local, H, m.moe_intermediate, dtype=dtype, device=device))
            reg("shared_gate", torch.zeros(1, H, dtype=dtype, device=device))
        self.eps = spec.rms_norm_eps

    def projections(self):
        ps = [self.inp, self.out]
        for m in (self.mlp, self.shared):
            if m is not None:
                ps += list(m.projections())
        return ps

    def adapter_params(self):
        out = []
        for p in self.projections():
            out += p.adapter_params()
        return out

    # ------------------------------------------------------------------ mixers
    def _attn(self, x, positions, cos, sin, merged, cache=None, kv_len=None):
        B, S, _ = x.shape
        f = (lambda m, z: m.forward_merged(z)) if merged else (lambda m, z: m(z))
        hq, hkv, D = self.hq, self.hkv, self.D
        p = f(self.inp, x)
        q, gate, k, v = p.split([hq * D, hq * D, hkv * D, hkv * D], dim=-1)
        q, k, v = q.reshape(B, S, hq, D), k.reshape(B, S, hkv, D), v.reshape(B, S, hkv, D)
        q, k = ops.qk_norm_rope(q, k, self.q_norm, self.k_norm, self.eps, cos, sin, positions, zero_centered=True)
        if cache is None:
            a = ops.attention(q, k, v, scale=self.scale, causal=True, softmax_fp32=True)
        elif kv_len is None:                     # prefill: record K/V, attend causally
            cache[0][:, :S].copy_(k)
            cache[1][:, :S].copy_(v)
            a = ops.attention(q, k, v, scale=self.scale, causal=True, softmax_fp32=True)
        else:                                    # one-token decode against the cache
            from .dense import ops_cache_write
            ops_cache_write(cache[0], cache[1], k[:, 0], v[:, 0], kv_len)
            a = ops.decode_attention(q[:, 0], cache[0], cache[1], kv_len + 1, scale=self.scale).unsqueeze(1)
        a = a.reshape(B, S, hq * D) * torch.sigmoid(gate.float()).to(a.dtype)
        return f(self.out, a)

    def _gdn(self, x, merged, state=None, valid=None, decode=False):
        """``state`` = (conv_state [B,C,K-1], S [B,Hv,kd,vd]) or None. Returns (out, new_state)."""
        B, S_, _ = x.shape
        f = (lambda m, z: m.forward_merged(z)) if merged else (lambda m, z: m(z))
        p = f(self.inp, x)
        mixed, z, b, a = p.split([self.conv_dim, self.value_dim, self.vh, self.vh], dim=-1)
        left = None if state is None else state[0]
        fast = (ops.native(x) and mixed.dtype == torch.bfloat16 and not self.conv_w.requires_grad
                and self.kd in (16, 32, 64, 128))
        if fast and decode and state is not None and S_ == 1 and state[0].dtype == torch.bfloat16 \
                and state[1].dtype == torch.float32 and state[0].is_contiguous() and state[1].is_contiguous():
            # one-token path: two kernels, both states updated in place
            from ..ops import cuda as C
            y = C.gdn_conv_step(mixed[:, 0], self.conv_w, state[0], True)
            if self.A_log.dtype == torch.float32 and self.dt_bias.dtype == torch.float32:
                core = C.gdn_decode_step_raw(y[:, :self.key_dim], y[:, self.key_dim:2 * self.key_dim], y[:, 2 * self.key_dim:],
                                             a[:, 0], b[:, 0], self.A_log, self.dt_bias, state[1], True, 1e-6)
            else:
                beta = torch.sigmoid(b[:, 0].float())
                g = -self.A_log.float().exp() * F.softplus(a[:, 0].float() + self.dt_bias.float())
                core = C.gdn_decode_step(y[:, :self.key_dim], y[:, self.key_dim:2 * self.key_dim], y[:, 2 * self.key_dim:],
                                         g, beta, state[1], True, 1e-6)
            core = ops.rmsnorm_gated(core.reshape(-1, self.vd), z.reshape(-1, self.vd), self.gdn_norm, self.eps)
            return f(self.out, core.reshape(B, S_, self.value_dim)), (state[0], state[1])
        y = None
        if fast:
            from ..ops import cuda as C
            y = C.gdn_conv(mixed, self.conv_w, left, True)
        if y is not None:
            K1 = self.conv_w.shape[-1] - 1
            ctx = mixed if left is None else torch.cat([left.transpose(1, 2).to(mixed.dtype), mixed], dim=1)
            if ctx.shape[1] < K1:
                ctx = F.pad(ctx, (0, 0, K1 - ctx.shape[1], 0))
            new_left = ctx[:, ctx.shape[1] - K1:].transpose(1, 2).detach()
        else:
            y, new_left = G.causal_depthwise_conv1d(mixed.transpose(1, 2), self.conv_w, left, activation=True)
            y = y.transpose(1, 2)
        if valid is not None and state is not None:
            # conv context must be the last K-1 *real* inputs of every row
            K1 = self.conv_w.shape[-1] - 1
            xx = torch.cat([mixed.new_zeros(B, K1, self.conv_dim) if left is None else left.transpose(1, 2).to(mixed.dtype),
                            mixed], dim=1)
            lens = valid.sum(1).long()
            idx = (lens[:, None] + torch.arange(K1, device=x.device)[None, :]).clamp(max=xx.shape[1] - 1)
            new_left = torch.gather(xx, 1, idx[:, :, None].expand(B, K1, self.conv_dim)).transpose(1, 2)
        q, k, v = y.split([self.key_dim, self.key_dim, self.value_dim], dim=-1)
        q, k = q.reshape(B, S_, self.kh, self.kd), k.reshape(B, S_, self.kh, self.kd)
        v = v.reshape(B, S_, self.vh, self.vd)
        beta = torch.sigmoid(b.float())
        g = -self.A_log.float().exp() * F.softplus(a.float() + self.dt_bias.float())
        if valid is not None:
            beta = beta * valid[:, :, None]
            g = g * valid[:, :, None]
        S0 = None if state is None else state[1]
        if fast and not decode and not torch.is_grad_enabled() and self.kd == 128 and self.vd == 128:
            # grad-free scoring and prefill: the whole chunked scan is one kernel with the state in shared memory
            from ..ops import cuda as C
            res = C.gdn_chunk_fwd(q, k, v, g, beta, S0, True, 1e-6)
            if res is not None:
                core, S1 = res
                core = ops.rmsnorm_gated(core.reshape(-1, self.vd), z.reshape(-1, self.vd), self.gdn_norm, self.eps)
                return f(self.out, core.reshape(B, S_, self.value_dim)), (new_left, S1)
        if fast and not decode and self.kd == 128 and self.vd == 128:
            # training: tensor-core chunk kernels with a hand-written backward
            from ..ops import cuda as C
            res = C.gdn_chunk_tc(q, k, v, g, beta, S0, 1e-6)
            if res is not None:
                core, S1 = res
                core = ops.rmsnorm_gated(core.reshape(-1, self.vd), z.reshape(-1, self.vd), self.gdn_norm, self.eps)
                return f(self.out, core.reshape(B, S_, self.value_dim)), (new_left, S1)
        rep = self.vh // self.kh
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
        if decode:
            core, S1 = G.gated_delta_rule_recurrent(q, k, v, g, beta, S0, use_qk_l2norm=True)
        else:
            core, S1 = G.gated_delta_rule_chunked(q, k, v, g, beta, S0, use_qk_l2norm=True)
        core = ops.rmsnorm_gated(core.reshape(-1, self.vd), z.reshape(-1, self.vd), self.gdn_norm, self.eps)
        return f(self.out, core.reshape(B, S_, self.value_dim)), (new_left, S1)

    def _ffn(self, x, merged):
        if self.spec.moe is None:
            return self.mlp(x, merged)
        m = self.spec.moe
        shared = (lambda z: self.shared(z, merged)) if self.shared is not None else None
        from ..parallel import ep
        return ep.sparse_moe(x, self.router, self.experts_gate_up, self.experts_down, m.top_k, shared,
                             self.shared_gate, self.spec.activation)

    def forward(self, h, positions, cos, sin, merged=False, cache=None, kv_len=None, valid=None, decode=False):
        x = ops.rmsnorm(h, self.input_norm, self.eps, True)
        new_state = None
        if self.kind == "full_attention":
            o = self._attn(x, positions, cos, sin, merged, cache, kv_len)
        else:
            o, new_state = self._gdn(x, merged, cache, valid, decode)
        x, h = ops.add_rmsnorm(o, h, self.post_norm, self.eps, True)
        if self.spec.moe is None:
            return self.mlp(x, merged, residual=h), new_state
        return h + self._ffn(x, merged), new_state


class Qwen35GradModel(nn.Module):
    def __init__(self, spec: Qwen35Spec, lora: Optional[LoraSpec] = None, targets: Optional[Qwen35LoraTargets] = None, *,
                 dtype=torch.float32, device=None, keep_transpose: Optional[bool] = None,
                 quant: BaseQuantization = BaseQuantization.NONE, remat: bool = False, full_ft: bool = False,
                 ep: Optional[tuple] = None):
        """``ep = (rank, world)``: hold only this rank's ``E / world`` routed experts (expert
        parallelism, see ``ferrl_b200.parallel.ep``); everything else is replicated."""
        super().__init__()
        spec.validate()
        self.spec, self.lora, self.remat, self.full_ft, self.dtype = spec, lora, remat, full_ft, dtype
        self.ep = ep if ep is not None and ep[1] > 1 else None
        if self.ep is not None:
            if spec.moe is None:
                raise ValueError("expert parallelism needs a sparse-MoE model")
            if spec.moe.num_experts % self.ep[1] or not 0 <= self.ep[0] < self.ep[1]:
                raise ValueError(f"{spec.moe.num_experts} experts do not split over expert-parallel world {self.ep[1]}")
            if full_ft:
                raise ValueError("expert parallelism keeps the routed experts frozen: not available with full fine-tuning")
        self.targets = targets or Qwen35LoraTargets()
        if lora is not None and not full_ft and not self.targets.any():
            # the reference refuses a load whose recipe selects nothing (crates/ferrl/src/qwen35.rs:3546-3560)
            raise ValueError("the LoRA target recipe selects no projection: the model would train nothing")
        dev = torch.device(device) if device is not None else torch.device("cpu")
        if keep_transpose is None:
            keep_transpose = dev.type == "cuda" and not full_ft
        self.keep_transpose = keep_transpose
        emb = torch.zeros(spec.vocab_size, spec.hidden_size, dtype=dtype, device=dev)
        fn = torch.zeros(spec.hidden_size, dtype=dtype, device=dev)
        if full_ft:
            self.embed, self.final_norm = nn.Parameter(emb), nn.Parameter(fn)
        else:
            self.register_buffer("embed", emb, persistent=False)
            self.register_buffer("final_norm", fn, persistent=False)
        if spec.tie_word_embeddings:
            self.lm_head = None
        elif full_ft:
            self.lm_head = nn.Parameter(torch.zeros_like(emb))
        else:
            self.register_buffer("lm_head", torch.zeros_like(emb), persistent=False)
        self.register_buffer("head_t", None, persistent=False)
        self.layers = nn.ModuleList([Qwen35Layer(spec, k, None if full_ft else lora, self.targets, dtype, dev,
                                                 keep_transpose, quant, full_ft,
                                                 ep_world=self.ep[1] if self.ep else 1) for k in spec.layer_types])
        cos, sin = ops.rope_tables(ops.default_inv_freq(spec.rot_dim, spec.rope_theta), spec.max_position_embeddings)
        self.register_buffer("cos", cos.to(dev), persistent=False)
        self.register_buffer("sin", sin.to(dev), persistent=False)

    # ------------------------------------------------------------ plumbing
    def head_weight(self):
        return self.embed if self.lm_head is None else self.lm_head

    @torch.no_grad()
    def refresh_head(self):
        if self.keep_transpose:
            self.head_t = self.head_weight().t().contiguous()

    def trainable_params(self):
        if self.full_ft:
            return [p for p in self.parameters()]
        out = []
        for l in self.layers:
            out += l.adapter_params()
        return out

    def set_adapter_enabled(self, on: bool):
        for l in self.layers:
            for p in l.projections():
                p.enabled = on

    def lora_recipe(self) -> str:
        if self.full_ft:
            return "full_ft"
        return f"lora:r{self.lora.rank}:a{self.lora.alpha:g}:{self.targets.canonical()}" if self.lora else "none"

    @torch.no_grad()
    def merge_adapters(self):
        for l in self.layers:
            for p in l.projections():
                p.merge()

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        dev = self.embed.device

        def rnd(shape, s=std):
            return (torch.randn(shape, generator=g) * s).to(self.dtype).to(dev)
        if dev.type == "cuda":
            gg = torch.Generator(device=dev).manual_seed(seed)

            def rnd(shape, s=std):  # noqa: F811 - device-side generation for the large synthetic benchmarks
                return (torch.randn(shape, generator=gg, device=dev, dtype=torch.float32) * s).to(self.dtype)
        self.embed.copy_(rnd(self.embed.shape))
        if self.lm_head is not None:
            self.lm_head.copy_(rnd(self.lm_head.shape))
        for li, l in enumerate(self.layers):
            for p in l.projections():
                p.set_weight(rnd(p.weight.shape))
                p.init_adapters(g)
            if l.kind == "linear_attention":
                l.conv_w.copy_(rnd(l.conv_w.shape, 0.3))
                l.A_log.copy_(torch.log(torch.rand(l.A_log.shape, generator=g) * 15 + 1).to(dev))
            if self.spec.moe is not None:
                l.router.copy_(rnd(l.router.shape, 1.0))          # N(0,1) router logits scale with the input norm
                self._init_experts(l, li, seed, std, rnd)
                l.shared_gate.copy_(rnd(l.shared_gate.shape))
        self.refresh_head()

    def _init_experts(self, l, li: int, seed: int, std: float, rnd):
        """Random experts.  Each expert's values are a pure function of (seed, layer, expert), drawn on
        the parameter's device, so an expert-parallel rank generates exactly its own block and the
        world as a whole holds the same experts as a single rank would."""
        E = self.spec.moe.num_experts
        if self.ep is None and l.experts_gate_up.device.type == "cpu":
            l.experts_gate_up.copy_(rnd(l.experts_gate_up.shape))
            l.experts_down.copy_(rnd(l.experts_down.shape))
            return
        e_local = l.experts_gate_up.shape[0]
        first = (self.ep[0] * e_local) if self.ep else 0
        dev = l.experts_gate_up.device
        for j in range(e_local):
            gg = torch.Generator(device=dev).manual_seed((seed * 1000003 + li * 4099 + first + j) & 0x7fffffff)
            l.experts_gate_up[j].copy_((torch.randn(l.experts_gate_up.shape[1:], generator=gg, device=dev) * std).to(self.dtype))
            l.experts_down[j].copy_((torch.randn(l.experts_down.shape[1:], generator=gg, device=dev) * std).to(self.dtype))
        del E

    # ------------------------------------------------------------- forward
    def forward_hidden(self, ids, comm: Optional[Comm] = None, merged=False, detached=False):
        B, S = ids.shape
        positions = torch.arange(S, device=ids.device)
        h = ops.embedding(ids, self.embed)
        for layer in self.layers:
            if self.remat and torch.is_grad_enabled() and not detached:
                fn = (lambda x, layer=layer: layer(x, positions, self.cos, self.sin, merged)[0])
                h = remat_segment(fn, h, layer.adapter_params() if not self.full_ft else list(layer.parameters()))
            else:
                h, _ = layer(h, positions, self.cos, self.sin, merged)
        return h

    def forward(self, ids, comm: Optional[Comm] = None):
        h = ops.rmsnorm(self.forward_hidden(ids), self.final_norm, self.spec.rms_norm_eps, True)
        return F.linear(h, self.head_weight()).float()

    def token_logprobs(self, ids, win_start, targets, temperature=1.0, comm: Optional[Comm] = None):
        h = self.forward_hidden(ids, detached=not torch.is_grad_enabled())
        B, L = targets.shape
        idx = (win_start.view(B, 1).long() + torch.arange(L, device=ids.device)[None, :]).clamp(max=ids.shape[1] - 1)
        hw = torch.gather(h, 1, idx[:, :, None].expand(B, L, h.shape[-1]))
        hw = ops.rmsnorm(hw, self.final_norm, self.spec.rms_norm_eps, True)
        return ops.logprob_gather(hw.reshape(B * L, -1), self.head_weight(), targets.reshape(-1), temperature, 0.0,
                                  head_wt=self.head_t).view(B, L)

    def new_decoder(self, batch: int, max_len: int, comm: Optional[Comm] = None):
        return Qwen35CachedDecoder(self, batch, max_len)


class Qwen35CachedDecoder:
    """Rollout twin with KV caches for the full-attention layers and (conv, recurrent)
    state for the GatedDeltaNet layers."""

    def __init__(self, model: Qwen35GradModel, batch: int, max_len: int):
        self.m, self.batch, self.max_len = model, batch, max_len
        spec, dev, dt = model.spec, model.embed.device, model.dtype
        self.state = []
        for l in model.layers:
            if l.kind == "full_attention":
                self.state.append([torch.zeros(batch, max_len, l.hkv, l.D, dtype=dt, device=dev),
                                   torch.zeros(batch, max_len, l.hkv, l.D, dtype=dt, device=dev)])
            else:
                self.state.append([torch.zeros(batch, l.conv_dim, spec.conv_kernel - 1, dtype=dt, device=dev),
                                   torch.zeros(batch, l.vh, l.kd, l.vd, dtype=torch.float32, device=dev)])
        self.kv_len = torch.zeros(batch, dtype=torch.int32, device=dev)

    def cache_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for s in self.state for t in s)

    @torch.no_grad()
    def prefill(self, ids, lens, rows=None):
        m = self.m
        P, L = ids.shape
        rows = torch.arange(P, device=ids.device) if rows is None else rows
        positions = torch.arange(L, device=ids.device)
        valid = (positions[None, :] < lens[:, None]).float()
        h = ops.embedding(ids, m.embed)
        for l, st in zip(m.layers, self.state):
            if l.kind == "full_attention":
                tmp = [torch.empty(P, L, l.hkv, l.D, dtype=m.dtype, device=ids.device) for _ in range(2)]
                h, _ = l(h, positions, m.cos, m.sin, True, cache=tmp)
                st[0][rows, :L] = tmp[0]
                st[1][rows, :L] = tmp[1]
            else:
                zero = [torch.zeros(P, l.conv_dim, m.spec.conv_kernel - 1, dtype=m.dtype, device=ids.device),
                        torch.zeros(P, l.vh, l.kd, l.vd, dtype=torch.float32, device=ids.device)]
                h, ns = l(h, positions, m.cos, m.sin, True, cache=zero, valid=valid)
                st[0][rows] = ns[0].to(st[0].dtype)
                st[1][rows] = ns[1]
        self.kv_len[rows] = lens.to(torch.int32)
        last = h[torch.arange(P, device=ids.device), (lens - 1).long()]
        last = ops.rmsnorm(last, m.final_norm, m.spec.rms_norm_eps, True)
        return ops.lora_linear(last, m.head_weight(), None, None).float()

    @torch.no_grad()
    def broadcast_groups(self, group: int):
        P = self.batch // group
        src = torch.arange(P, device=self.kv_len.device).repeat_interleave(group)
        for st in self.state:
            st[0].copy_(st[0][src])
            st[1].copy_(st[1][src])
        self.kv_len.copy_(self.kv_len[src])

    @torch.no_grad()
    def decode(self, tokens):
        m = self.m
        h = ops.embedding(tokens, m.embed).unsqueeze(1)
        pos = self.kv_len[:, None].long()
        for l, st in zip(m.layers, self.state):
            if l.kind == "full_attention":
                h, _ = l(h, pos, m.cos, m.sin, True, cache=st, kv_len=self.kv_len)
            else:
                h, ns = l(h, pos, m.cos, m.sin, True, cache=st, decode=True)
                st[0].copy_(ns[0])
                st[1].copy_(ns[1])
        self.kv_len += 1
        h = ops.rmsnorm(h[:, 0], m.final_norm, m.spec.rms_norm_eps, True)
        return ops.lora_linear(h, m.head_weight(), None, None).float()


@torch.no_grad()
def load_qwen35_weights(model: Qwen35GradModel, src) -> None:
    """HF names -> fused layout. q_proj rows are stored per head as ``[query | gate]``;
    they are regrouped to ``[all queries | all gates]`` so heads are packed."""
    spec = model.spec
    p = next(pre for pre in ("model.language_model.", "model.", "language_model.model.")
             if src.has(pre + "embed_tokens.weight"))
    to = lambda t: t.to(model.dtype)  # noqa: E731
    model.embed.copy_(to(src.get(p + "embed_tokens.weight")))
    model.final_norm.copy_(to(src.get(p + "norm.weight")))
    if model.lm_head is not None:
        model.lm_head.copy_(to(src.get("lm_head.weight")))
    D, hq = spec.head_dim, spec.num_attention_heads
    for i, l in enumerate(model.layers):
        b = f"{p}layers.{i}."
        l.input_norm.copy_(to(src.get(b + "input_layernorm.weight")))
        l.post_norm.copy_(to(src.get(b + "post_attention_layernorm.weight")))
        if l.kind == "full_attention":
            qw = src.get(b + "self_attn.q_proj.weight").view(hq, 2, D, spec.hidden_size)
            q = torch.cat([qw[:, 0].reshape(hq * D, -1), qw[:, 1].reshape(hq * D, -1)], 0)
            l.inp.set_weight(to(torch.cat([q, src.get(b + "self_attn.k_proj.weight"),
                                           src.get(b + "self_attn.v_proj.weight")], 0)))
            l.out.set_weight(to(src.get(b + "self_attn.o_proj.weight")))
            l.q_norm.copy_(to(src.get(b + "self_attn.q_norm.weight")))
            l.k_norm.copy_(to(src.get(b + "self_attn.k_norm.weight")))
        else:
            a = b + "linear_attn."
            l.inp.set_weight(to(torch.cat([src.get(a + "in_proj_qkv.weight"), src.get(a + "in_proj_z.weight"),
                                           src.get(a + "in_proj_b.weight"), src.get(a + "in_proj_a.weight")], 0)))
            l.out.set_weight(to(src.get(a + "out_proj.weight")))
            l.conv_w.copy_(to(src.get(a + "conv1d.weight").squeeze(1)))
            l.A_log.copy_(src.get(a + "A_log").float())
            l.dt_bias.copy_(src.get(a + "dt_bias").float())
            l.gdn_norm.copy_(to(src.get(a + "norm.weight")))
        if spec.moe is None:
            l.mlp.gate_up.set_weight(to(torch.cat([src.get(b + "mlp.gate_proj.weight"), src.get(b + "mlp.up_proj.weight")], 0)))
            l.mlp.down.set_weight(to(src.get(b + "mlp.down_proj.weight")))
        else:
            l.router.copy_(to(src.get(b + "mlp.gate.weight")))
            e_local = l.experts_gate_up.shape[0]
            first = model.ep[0] * e_local if model.ep else 0      # expert parallelism: read this rank's experts only
            if src.has(b + "mlp.experts.gate_up_proj"):        # fused 3-D layout
                l.experts_gate_up.copy_(to(src.get(b + "mlp.experts.gate_up_proj")[first:first + e_local]))
                l.experts_down.copy_(to(src.get(b + "mlp.experts.down_proj")[first:first + e_local]))
            else:                                               # one tensor per expert and projection
                for j in range(e_local):
                    eb = f"{b}mlp.experts.{first + j}."
                    l.experts_gate_up[j].copy_(to(torch.cat([src.get(eb + "gate_proj.weight"),
                                                             src.get(eb + "up_proj.weight")], 0)))
                    l.experts_down[j].copy_(to(src.get(eb + "down_proj.weight")))
            l.shared_gate.copy_(to(src.get(b + "mlp.shared_expert_gate.weight")))
            if l.shared is not None:
                l.shared.gate_up.set_weight(to(torch.cat([src.get(b + "mlp.shared_expert.gate_proj.weight"),
                                                          src.get(b + "mlp.shared_expert.up_proj.weight")], 0)))
                l.shared.down.set_weight(to(src.get(b + "mlp.shared_expert.down_proj.weight")))
    model.refresh_head()


def load_qwen35(model_dir: str, opts):
    from .loader import TensorSource, _identity, read_config
    cfg = read_config(model_dir)
    spec = qwen35_spec(cfg)
    if opts.max_position_embeddings:
        spec.max_position_embeddings = opts.max_position_embeddings
    if opts.tp is not None:
        raise ValueError("tensor parallelism is not supported for the Qwen3.5 family")
    targets = None
    if opts.lora is not None and not opts.full_ft:
        # the dense recipe names the attention and MLP projections; the GatedDeltaNet letters come beside it
        targets = Qwen35LoraTargets.parse(opts.lora.targets.canonical() + "|gdn:" + (opts.gdn_targets or "-"))
    model = Qwen35GradModel(spec, None if opts.full_ft else opts.lora, targets, dtype=opts.dtype, device=opts.device,
                            quant=opts.quantization, remat=opts.remat, full_ft=opts.full_ft, ep=opts.ep)
    src = TensorSource(model_dir)
    load_qwen35_weights(model, src)
    g = torch.Generator().manual_seed(opts.adapter_seed)
    for l in model.layers:
        for pr in l.projections():
            pr.init_adapters(g)
    return model, _identity(model_dir, cfg, src, opts)
