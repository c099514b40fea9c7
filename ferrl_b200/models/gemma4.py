"""Dense Gemma 4 text decoder (LoRA, remat, tensor parallel training, cached rollout).

Reference: ``crates/ferrl/src/gemma4.rs`` - config ``:354-430`` and validation
``:519-720``; two RoPE tables (sliding layers: default theta over the whole
head; full layers: "proportional" - only the first ``partial_rotary_factor``
share of the frequency pairs rotate, the rest have zero frequency) ``:818-881``;
sliding / full causal masks ``:898-991``; attention with q/k RMS norms, an
unscaled v norm, **no 1/sqrt(d) score scale**, K = V on full layers, fp32
softmax ``:1090-1150``; GeGLU (``gelu_pytorch_tanh``) MLP ``:1188-1265``; four
norms and a ``layer_scalar`` per layer ``:1290-1432``; embeddings scaled by
sqrt(hidden) ``:1621``; tied head with ``cap * tanh(x / cap)`` ``:1796-1804``;
tensor-parallel remat forward with two segments per layer ``:1929-1984`` and
backward with boundary cotangent all-reduce ``:2033-2170``; windowed KV cache
``:2327-2394``.

Here the masks are index arithmetic inside the flash / decode kernels
(``window`` argument), the softcap is applied inside the fused log-prob kernel,
and under TP the row-parallel partial sums go through ``reduce_from_tp`` (fused
GEMM + peer all-reduce on GPUs).  Each layer is two remat segments (attention
half, MLP half) so the boundary cotangents reduced in backward are exactly the
residual-stream tensors, as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..comm import Comm, SoloComm
from ..parallel.tp import TensorParallelPlan, copy_to_tp
from ..remat import remat_segment
from .dense import ops_cache_write
from .lora import BaseQuantization, DenseLoraTargets, FusedLoraLinear, LoraSpec, Shard


@dataclass
class Gemma4Spec:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    global_head_dim: int
    num_global_key_value_heads: int
    intermediate_size: int
    layer_types: list
    sliding_window: int
    rms_norm_eps: float = 1e-6
    attention_k_eq_v: bool = True
    final_logit_softcapping: float = 30.0
    rope_theta_sliding: float = 1e4
    rope_theta_full: float = 1e6
    full_partial_rotary_factor: float = 1.0
    full_rope_proportional: bool = True
    max_position_embeddings: int = 4096
    activation: str = "gelu_pytorch_tanh"
    tie_word_embeddings: bool = True

    def validate(self):
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types must list every layer")
        if any(t not in ("sliding_attention", "full_attention") for t in self.layer_types):
            raise ValueError("unknown Gemma layer type")
        if self.sliding_window <= 0:
            raise ValueError("sliding_window must be > 0")
        if self.num_attention_heads % self.num_key_value_heads or self.num_attention_heads % self.num_global_key_value_heads:
            raise ValueError("query heads must be a multiple of kv heads")

    def full_inv_freq(self) -> torch.Tensor:
        D = self.global_head_dim
        if not self.full_rope_proportional:
            return ops.default_inv_freq(D, self.rope_theta_full)
        angles = int(self.full_partial_rotary_factor * D // 2)
        i = torch.arange(0, 2 * angles, 2, dtype=torch.float64)
        rot = (1.0 / (self.rope_theta_full ** (i / D))).float()
        return torch.cat([rot, torch.zeros(D // 2 - angles)])


def gemma4_spec(cfg: Mapping[str, Any]) -> Gemma4Spec:
    t = cfg.get("text_config", cfg)
    if t.get("model_type") is not None and t["model_type"] not in ("gemma4_text", "gemma4_unified_text"):
        # the multimodal wrappers carry audio / vision towers under other text model types (gemma4.rs:519-532)
        raise ValueError(f"gemma4 config: text_config.model_type {t['model_type']!r}, expected \"gemma4_text\" or "
                         "\"gemma4_unified_text\"")
    for key, why in (("hidden_size_per_layer_input", "per-layer inputs"), ("num_kv_shared_layers", "kv-shared layers")):
        if int(t.get(key, 0) or 0) != 0:
            raise ValueError(f"Gemma 4 checkpoints with {why} are not supported (dense text decoder only)")
    if t.get("enable_moe_block"):
        raise ValueError("Gemma 4 MoE checkpoints are not supported (dense text decoder only)")
    if t.get("attention_bias"):
        raise ValueError("Gemma 4 with attention_bias is not supported")
    rp = t.get("rope_parameters") or {}
    full, slide = rp.get("full_attention", {}), rp.get("sliding_attention", {})
    L = int(t["num_hidden_layers"])
    types = t.get("layer_types") or [("full_attention" if (i + 1) % 6 == 0 else "sliding_attention") for i in range(L)]
    heads = int(t["num_attention_heads"])
    hd = int(t.get("head_dim") or int(t["hidden_size"]) // heads)
    spec = Gemma4Spec(
        vocab_size=int(t["vocab_size"]), hidden_size=int(t["hidden_size"]), num_hidden_layers=L,
        num_attention_heads=heads, num_key_value_heads=int(t.get("num_key_value_heads", heads)), head_dim=hd,
        global_head_dim=int(t.get("global_head_dim") or hd),
        num_global_key_value_heads=int(t.get("num_global_key_value_heads") or t.get("num_key_value_heads", heads)),
        intermediate_size=int(t["intermediate_size"]), layer_types=list(types),
        sliding_window=int(t.get("sliding_window", 1024)), rms_norm_eps=float(t.get("rms_norm_eps", 1e-6)),
        attention_k_eq_v=bool(t.get("attention_k_eq_v", False)),
        final_logit_softcapping=float(t.get("final_logit_softcapping") or 0.0),
        rope_theta_sliding=float(slide.get("rope_theta", 1e4)), rope_theta_full=float(full.get("rope_theta", 1e6)),
        full_partial_rotary_factor=float(full.get("partial_rotary_factor", 1.0)),
        full_rope_proportional=full.get("rope_type", "default") == "proportional",
        max_position_embeddings=int(t.get("max_position_embeddings", 4096)),
        activation=str(t.get("hidden_activation", "gelu_pytorch_tanh")),
        tie_word_embeddings=bool(t.get("tie_word_embeddings", cfg.get("tie_word_embeddings", True))))
    spec.validate()
    return spec


class Gemma4Layer(nn.Module):
    def __init__(self, spec: Gemma4Spec, kind: str, lora, dtype, device, tp, keep_transpose, quant, trainable_base=False):
        super().__init__()
        self.kind = kind
        sliding = kind == "sliding_attention"
        H, Fd = spec.hidden_size, spec.intermediate_size
        D = spec.head_dim if sliding else spec.global_head_dim
        hq = spec.num_attention_heads
        self.k_eq_v = spec.attention_k_eq_v and not sliding
        hkv = spec.num_key_value_heads if not self.k_eq_v else spec.num_global_key_value_heads
        if not sliding and not self.k_eq_v:
            hkv = spec.num_key_value_heads
        w = tp.world if tp else 1
        r = tp.rank if tp else 0
        if hq % w or hkv % w or Fd % w:
            raise ValueError("Gemma heads / kv heads / intermediate size must divide the tensor-parallel world")
        t = lora.targets if lora else DenseLoraTargets(*(False,) * 7)
        col = Shard("column", r, w) if w > 1 else None
        row = Shard("row", r, w) if w > 1 else None
        kw = dict(dtype=dtype, device=device, keep_transpose=keep_transpose, quant=quant, trainable_base=trainable_base)
        self.hq, self.hkv, self.D = hq // w, hkv // w, D
        self.window = spec.sliding_window if sliding else 0
        if self.k_eq_v:
            self.qkv = FusedLoraLinear(H, [hq * D // w, hkv * D // w], ("q", "k"), (t.attn_q, t.attn_k), lora, shard=col,
                                       full_out_sizes=[hq * D, hkv * D], **kw)
        else:
            self.qkv = FusedLoraLinear(H, [hq * D // w, hkv * D // w, hkv * D // w], ("q", "k", "v"),
                                       (t.attn_q, t.attn_k, t.attn_v), lora, shard=col,
                                       full_out_sizes=[hq * D, hkv * D, hkv * D], **kw)
        self.o = FusedLoraLinear(hq * D // w, [H], ("o",), (t.attn_o,), lora, shard=row, full_in=hq * D, **kw)
        self.gate_up = FusedLoraLinear(H, [Fd // w, Fd // w], ("gate", "up"), (t.mlp_gate, t.mlp_up), lora, shard=col,
                                       full_out_sizes=[Fd, Fd], **kw)
        self.down = FusedLoraLinear(Fd // w, [H], ("down",), (t.mlp_down,), lora, shard=row, full_in=Fd, **kw)
        for name, n in (("input_norm", H), ("post_attn_norm", H), ("pre_ffn_norm", H), ("post_ffn_norm", H),
                        ("q_norm", D), ("k_norm", D)):
            v = torch.ones(n, dtype=dtype, device=device)
            if trainable_base:
                setattr(self, name, nn.Parameter(v))
            else:
                self.register_buffer(name, v, persistent=False)
        self.register_buffer("layer_scalar", torch.ones(1, dtype=dtype, device=device), persistent=False)
        self.eps, self.act = spec.rms_norm_eps, spec.activation

    def projections(self):
        return (self.qkv, self.o, self.gate_up, self.down)

    def adapter_params(self):
        out = []
        for p in self.projections():
            out += p.adapter_params()
        return out

    def _qkv(self, x, positions, cos, sin, lin):
        return self._split_qkv(lin(self.qkv, x), positions, cos, sin)

    def _split_qkv(self, p, positions, cos, sin):
        B, S, _ = p.shape
        if self.k_eq_v:
            q, k = p.split([self.hq * self.D, self.hkv * self.D], dim=-1)
            v_raw = k
        else:
            q, k, v_raw = p.split([self.hq * self.D, self.hkv * self.D, self.hkv * self.D], dim=-1)
        q = q.reshape(B, S, self.hq, self.D)
        k = k.reshape(B, S, self.hkv, self.D)
        v = ops.rmsnorm(v_raw.reshape(B, S, self.hkv, self.D).contiguous(), None, self.eps)   # scale-free v norm
        q, k = ops.qk_norm_rope(q, k, self.q_norm, self.k_norm, self.eps, cos, sin, positions)
        return q, k, v

    def attn_half(self, h, positions, cos, sin, comm, merged=False, kv_out=None):
        B, S, _ = h.shape
        lin = (lambda m, z: m.forward_merged(z)) if merged else (lambda m, z: m(z))
        x = copy_to_tp(ops.rmsnorm(h, self.input_norm, self.eps), comm)
        q, k, v = self._qkv(x, positions, cos, sin, lin)
        if kv_out is not None:
            kv_out[0][:, :S].copy_(k)
            kv_out[1][:, :S].copy_(v)
        a = ops.attention(q, k, v, scale=1.0, causal=True, window=self.window, softmax_fp32=True)
        # row-parallel projection and its tensor-parallel sum: one fused GEMM -> all-reduce kernel where a
        # reducer is registered for ``comm`` (the residual joins after the post-norm, so none rides along)
        o = self.o.forward_reduce(a.reshape(B, S, self.hq * self.D), comm, merged)
        return h + ops.rmsnorm(o, self.post_attn_norm, self.eps)

    # ---- sequence-sharded forms: ``hs`` holds this rank's block of the flattened [B * S, H] token rows
    def attn_half_sp(self, hs, B, S, positions, cos, sin, comm, merged=False):
        # the column-parallel projection gathers the normalised rows; its backward reduce-scatters inside the GEMM
        p = self.qkv.forward_gathered(ops.rmsnorm(hs, self.input_norm, self.eps), comm, merged).view(B, S, -1)
        q, k, v = self._split_qkv(p, positions, cos, sin)
        a = ops.attention(q, k, v, scale=1.0, causal=True, window=self.window, softmax_fp32=True)
        o = self.o.forward_reduce_scatter(a.reshape(B * S, self.hq * self.D), comm, merged)   # this rank's rows of the sum
        return hs + ops.rmsnorm(o, self.post_attn_norm, self.eps)

    def mlp_half_sp(self, hs, comm, merged=False):
        gu = self.gate_up.forward_gathered(ops.rmsnorm(hs, self.pre_ffn_norm, self.eps), comm, merged)
        d = self.down.forward_reduce_scatter(ops.swiglu(gu, self.act), comm, merged)
        return (hs + ops.rmsnorm(d, self.post_ffn_norm, self.eps)) * self.layer_scalar

    def mlp_half(self, h, comm, merged=False):
        lin = (lambda m, z: m.forward_merged(z)) if merged else (lambda m, z: m(z))
        x = copy_to_tp(ops.rmsnorm(h, self.pre_ffn_norm, self.eps), comm)
        d = self.down.forward_reduce(ops.swiglu(lin(self.gate_up, x), self.act), comm, merged)
        return (h + ops.rmsnorm(d, self.post_ffn_norm, self.eps)) * self.layer_scalar

    def decode(self, h, kv_len, cos, sin, k_cache, v_cache, comm):
        """One token against the cache.  A sliding layer's cache is a ring of ``window`` slots (token ``p``
        lives in slot ``p % window``): the new token overwrites the one that just left the window and
        attention runs over the ``min(p + 1, window)`` occupied slots - keys carry their RoPE phase, so the
        slot order does not matter.  Full-attention layers keep the whole sequence."""
        B = h.shape[0]
        lin = lambda m, z: m.forward_merged(z)  # noqa: E731
        x = ops.rmsnorm(h, self.input_norm, self.eps).unsqueeze(1)
        q, k, v = self._qkv(x, kv_len[:, None].long(), cos, sin, lin)
        slots = k_cache.shape[1]
        if self.window and slots <= self.window:
            ops_cache_write(k_cache, v_cache, k[:, 0], v[:, 0], kv_len % slots)
            a = ops.decode_attention(q[:, 0], k_cache, v_cache, (kv_len + 1).clamp(max=slots), scale=1.0)
        else:
            ops_cache_write(k_cache, v_cache, k[:, 0], v[:, 0], kv_len)
            a = ops.decode_attention(q[:, 0], k_cache, v_cache, kv_len + 1, scale=1.0, window=self.window)
        o = self.o.forward_reduce(a.reshape(B, self.hq * self.D), comm, True)
        h = h + ops.rmsnorm(o, self.post_attn_norm, self.eps)
        return self.mlp_half(h, comm, merged=True)


class Gemma4GradModel(nn.Module):
    def __init__(self, spec: Gemma4Spec, lora: Optional[LoraSpec] = None, *, dtype=torch.float32, device=None,
                 tp: Optional[TensorParallelPlan] = None, keep_transpose: Optional[bool] = None,
                 quant: BaseQuantization = BaseQuantization.NONE, remat: bool = False, full_ft: bool = False,
                 sequence_parallel: bool = False):
        super().__init__()
        spec.validate()
        self.spec, self.lora, self.tp, self.remat, self.full_ft, self.dtype = spec, lora, tp, remat, full_ft, dtype
        # training / scoring forward with the residual stream sharded over the token rows (``parallel/sp.py``)
        self.sequence_parallel = bool(sequence_parallel)
        dev = torch.device(device) if device is not None else torch.device("cpu")
        if keep_transpose is None:
            keep_transpose = dev.type == "cuda" and not full_ft
        self.keep_transpose = keep_transpose
        emb = torch.zeros(spec.vocab_size, spec.hidden_size, dtype=dtype, device=dev)
        fn = torch.ones(spec.hidden_size, dtype=dtype, device=dev)
        if full_ft:
            self.embed, self.final_norm = nn.Parameter(emb), nn.Parameter(fn)
        else:
            self.register_buffer("embed", emb, persistent=False)
            self.register_buffer("final_norm", fn, persistent=False)
        self.register_buffer("head_t", None, persistent=False)
        self.layers = nn.ModuleList([Gemma4Layer(spec, k, None if full_ft else lora, dtype, dev, tp, keep_transpose,
                                                 quant, full_ft) for k in spec.layer_types])
        cs, ss = ops.rope_tables(ops.default_inv_freq(spec.head_dim, spec.rope_theta_sliding), spec.max_position_embeddings)
        cf, sf = ops.rope_tables(spec.full_inv_freq(), spec.max_position_embeddings)
        for n, t in (("cos_s", cs), ("sin_s", ss), ("cos_f", cf), ("sin_f", sf)):
            self.register_buffer(n, t.to(dev), persistent=False)
        self.embed_scale = math.sqrt(spec.hidden_size)

    def _tables(self, layer):
        return (self.cos_s, self.sin_s) if layer.kind == "sliding_attention" else (self.cos_f, self.sin_f)

    def head_weight(self):
        return self.embed

    @torch.no_grad()
    def refresh_head(self):
        if self.keep_transpose:
            self.head_t = self.embed.t().contiguous()

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

    def lora_recipe(self):
        if self.full_ft:
            return "full_ft"
        return self.lora.recipe() if self.lora else "none"

    @torch.no_grad()
    def merge_adapters(self):
        for l in self.layers:
            for p in l.projections():
                p.merge()

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator().manual_seed(seed)
        dev = self.embed.device
        rnd = lambda shape: (torch.randn(shape, generator=g) * std).to(self.dtype).to(dev)  # noqa: E731
        if dev.type == "cuda":          # device-side generation for the large synthetic benchmarks
            gg = torch.Generator(device=dev).manual_seed(seed)
            rnd = lambda shape: (torch.randn(shape, generator=gg, device=dev, dtype=torch.float32) * std).to(self.dtype)  # noqa: E731
        self.embed.copy_(rnd(self.embed.shape))
        for l in self.layers:
            for p in l.projections():
                p.set_weight(rnd(p.weight.shape))
                p.init_adapters(g)
        self.refresh_head()

    def forward_hidden(self, ids, comm: Optional[Comm] = None, merged=False, kv_out=None, detached=False):
        comm = comm or SoloComm()
        B, S = ids.shape
        positions = torch.arange(S, device=ids.device)
        h = ops.embedding(ids, self.embed, self.embed_scale)
        use_remat = self.remat and torch.is_grad_enabled() and not detached
        if self.sequence_parallel and comm.world_size > 1 and kv_out is None and (B * S) % comm.world_size == 0:
            from ..parallel import sp
            hs = sp.shard_rows(h.reshape(B * S, -1), comm)
            for layer in self.layers:
                cos, sin = self._tables(layer)
                params = layer.adapter_params() if not self.full_ft else list(layer.parameters())
                if use_remat:
                    hs = remat_segment(lambda x, l=layer, c=cos, s=sin: l.attn_half_sp(x, B, S, positions, c, s, comm, merged), hs, params)
                    hs = remat_segment(lambda x, l=layer: l.mlp_half_sp(x, comm, merged), hs, params)
                else:
                    hs = layer.attn_half_sp(hs, B, S, positions, cos, sin, comm, merged)
                    hs = layer.mlp_half_sp(hs, comm, merged)
            return sp.gather_rows_replicated(hs, comm).view(B, S, -1)
        for i, layer in enumerate(self.layers):
            cos, sin = self._tables(layer)
            params = layer.adapter_params() if not self.full_ft else list(layer.parameters())
            if use_remat:
                h = remat_segment(lambda x, l=layer, c=cos, s=sin: l.attn_half(x, positions, c, s, comm, merged), h, params)
                h = remat_segment(lambda x, l=layer: l.mlp_half(x, comm, merged), h, params)
            else:
                h = layer.attn_half(h, positions, cos, sin, comm, merged, None if kv_out is None else kv_out[i])
                h = layer.mlp_half(h, comm, merged)
        return h

    def _softcap(self, logits):
        c = self.spec.final_logit_softcapping
        return c * torch.tanh(logits / c) if c and c > 0 else logits

    def forward(self, ids, comm: Optional[Comm] = None):
        h = ops.rmsnorm(self.forward_hidden(ids, comm), self.final_norm, self.spec.rms_norm_eps)
        return self._softcap(F.linear(h, self.embed).float())

    def token_logprobs(self, ids, win_start, targets, temperature=1.0, comm: Optional[Comm] = None):
        h = self.forward_hidden(ids, comm, detached=not torch.is_grad_enabled())
        B, L = targets.shape
        idx = (win_start.view(B, 1).long() + torch.arange(L, device=ids.device)[None, :]).clamp(max=ids.shape[1] - 1)
        hw = torch.gather(h, 1, idx[:, :, None].expand(B, L, h.shape[-1]))
        hw = ops.rmsnorm(hw, self.final_norm, self.spec.rms_norm_eps)
        if comm is not None and comm.world_size > 1 and self.tp is not None and not self.full_ft:
            # tensor parallelism: every rank scores 1 / world of the (tied, replicated) vocabulary and the ranks
            # exchange three floats per row instead of each evaluating the whole 262144-row head
            from ..parallel.tp import sharded_logprob_gather
            lp = sharded_logprob_gather(hw.reshape(B * L, -1), self.embed, targets.reshape(-1), temperature,
                                        self.spec.final_logit_softcapping, comm)
            if lp is not None:
                return lp.view(B, L)
        return ops.logprob_gather(hw.reshape(B * L, -1), self.embed, targets.reshape(-1), temperature,
                                  self.spec.final_logit_softcapping, head_wt=self.head_t).view(B, L)

    def new_decoder(self, batch: int, max_len: int, comm: Optional[Comm] = None):
        return Gemma4CachedDecoder(self, batch, max_len, comm or SoloComm())


class Gemma4CachedDecoder:
    """Cached rollout twin with windowed retention: a sliding layer keeps only the last
    ``sliding_window`` tokens of every row, in a ring of that many slots, so its cache does not grow
    with the sequence (reference gemma4.rs:2327-2394); full-attention layers keep ``max_len`` tokens.
    ``retained_bytes`` is what is actually allocated, as the reference's cache telemetry reports
    (gemma4.rs:2960-2977); ``dense_bytes`` is what a cache without retention would take."""

    def __init__(self, model: Gemma4GradModel, batch: int, max_len: int, comm: Comm):
        self.m, self.comm, self.batch, self.max_len = model, comm, batch, max_len
        dev, dt = model.embed.device, model.dtype
        self.slots = [min(max_len, l.window) if l.window else max_len for l in model.layers]
        self.k = [torch.zeros(batch, n, l.hkv, l.D, dtype=dt, device=dev) for l, n in zip(model.layers, self.slots)]
        self.v = [torch.zeros(batch, n, l.hkv, l.D, dtype=dt, device=dev) for l, n in zip(model.layers, self.slots)]
        self.kv_len = torch.zeros(batch, dtype=torch.int32, device=dev)

    def cache_bytes(self):
        return sum(t.numel() * t.element_size() for t in self.k + self.v)

    def retained_bytes(self):
        return self.cache_bytes()

    def dense_bytes(self):
        return sum(2 * k.shape[0] * self.max_len * k.shape[2] * k.shape[3] * k.element_size() for k in self.k)

    @torch.no_grad()
    def prefill(self, ids, lens, rows=None):
        m = self.m
        P, L = ids.shape
        rows = torch.arange(P, device=ids.device) if rows is None else rows
        tmp = [(torch.empty(P, L, l.hkv, l.D, dtype=m.dtype, device=ids.device),
                torch.empty(P, L, l.hkv, l.D, dtype=m.dtype, device=ids.device)) for l in m.layers]
        h = m.forward_hidden(ids, self.comm, merged=True, kv_out=tmp, detached=True)
        lens64 = lens.to(ids.device).long()
        for i, n in enumerate(self.slots):
            if n >= L:
                self.k[i][rows, :L] = tmp[i][0]
                self.v[i][rows, :L] = tmp[i][1]
                continue
            # ring: slot s of a row holds its newest token p < len with p % n == s
            s_idx = torch.arange(n, device=ids.device)[None, :]
            pos = (s_idx + n * ((lens64[:, None] - 1 - s_idx).clamp(min=0) // n)).clamp(max=L - 1)     # [P, n]
            gi = pos[:, :, None, None].expand(P, n, tmp[i][0].shape[2], tmp[i][0].shape[3])
            self.k[i][rows] = torch.gather(tmp[i][0], 1, gi)
            self.v[i][rows] = torch.gather(tmp[i][1], 1, gi)
        self.kv_len[rows] = lens.to(torch.int32)
        last = h[torch.arange(P, device=ids.device), (lens - 1).long()]
        last = ops.rmsnorm(last, m.final_norm, m.spec.rms_norm_eps)
        return m._softcap(ops.lora_linear(last, m.embed, None, None).float())

    @torch.no_grad()
    def broadcast_groups(self, group: int):
        P = self.batch // group
        src = torch.arange(P, device=self.kv_len.device).repeat_interleave(group)
        for i in range(len(self.k)):
            self.k[i].copy_(self.k[i][src])
            self.v[i].copy_(self.v[i][src])
        self.kv_len.copy_(self.kv_len[src])

    @torch.no_grad()
    def decode(self, tokens):
        m = self.m
        h = ops.embedding(tokens, m.embed, m.embed_scale)
        for i, l in enumerate(m.layers):
            cos, sin = m._tables(l)
            h = l.decode(h, self.kv_len, cos, sin, self.k[i], self.v[i], self.comm)
        self.kv_len += 1
        h = ops.rmsnorm(h, m.final_norm, m.spec.rms_norm_eps)
        return m._softcap(ops.lora_linear(h, m.embed, None, None).float())


@torch.no_grad()
def load_gemma4_weights(model: Gemma4GradModel, src) -> None:
    spec, tp = model.spec, model.tp
    p = next(pre for pre in ("model.language_model.", "model.", "language_model.model.")
             if src.has(pre + "embed_tokens.weight"))
    to = lambda t: t.to(model.dtype)  # noqa: E731
    model.embed.copy_(to(src.get(p + "embed_tokens.weight")))
    model.final_norm.copy_(to(src.get(p + "norm.weight")))
    w = tp.world if tp else 1
    r = tp.rank if tp else 0
    for i, l in enumerate(model.layers):
        b = f"{p}layers.{i}."

        def col(name):
            t = src.get(b + name)
            per = t.shape[0] // w
            return src.rows(b + name, r * per, per) if w > 1 else t

        def row(name):
            t = src.get(b + name)
            per = t.shape[1] // w
            return src.cols(b + name, r * per, per) if w > 1 else t
        parts = [col("self_attn.q_proj.weight"), col("self_attn.k_proj.weight")]
        if not l.k_eq_v:
            parts.append(col("self_attn.v_proj.weight"))
        l.qkv.set_weight(to(torch.cat(parts, 0)))
        l.o.set_weight(to(row("self_attn.o_proj.weight")))
        l.gate_up.set_weight(to(torch.cat([col("mlp.gate_proj.weight"), col("mlp.up_proj.weight")], 0)))
        l.down.set_weight(to(row("mlp.down_proj.weight")))
        for mine, theirs in (("input_norm", "input_layernorm"), ("post_attn_norm", "post_attention_layernorm"),
                             ("pre_ffn_norm", "pre_feedforward_layernorm"), ("post_ffn_norm", "post_feedforward_layernorm")):
            getattr(l, mine).copy_(to(src.get(b + theirs + ".weight")))
        l.q_norm.copy_(to(src.get(b + "self_attn.q_norm.weight")))
        l.k_norm.copy_(to(src.get(b + "self_attn.k_norm.weight")))
        if src.has(b + "layer_scalar"):
            l.layer_scalar.copy_(to(src.get(b + "layer_scalar")))
    model.refresh_head()


def load_gemma4(model_dir: str, opts):
    from .loader import TensorSource, _identity, read_config
    cfg = read_config(model_dir)
    spec = gemma4_spec(cfg)
    if opts.max_position_embeddings:
        spec.max_position_embeddings = opts.max_position_embeddings
    tp = None
    if opts.tp is not None:
        tp = TensorParallelPlan.new(opts.tp[0], opts.tp[1], spec.num_attention_heads,
                                    math.gcd(spec.num_key_value_heads, spec.num_global_key_value_heads),
                                    spec.intermediate_size)
    model = Gemma4GradModel(spec, None if opts.full_ft else opts.lora, dtype=opts.dtype, device=opts.device, tp=tp,
                            quant=opts.quantization, remat=opts.remat, full_ft=opts.full_ft)
    src = TensorSource(model_dir)
    load_gemma4_weights(model, src)
    g = torch.Generator().manual_seed(opts.adapter_seed)
    for l in model.layers:
        for pr in l.projections():
            pr.init_adapters(g)
    return model, _identity(model_dir, cfg, src, opts)
