"""Shared dense decoder backbone (Qwen3 and Llama-3.x) with LoRA, activation
rematerialisation, tensor parallelism and a KV-cached rollout twin.

What the reference does (``crates/ferrl/src/dense.rs``): pre-norm RMSNorm +
GQA attention + SwiGLU residual stack (``:276-566``); the variation between
the two families is data on the spec (per-head QK-norm, fp32 softmax, head_dim
rule, RoPE frequencies; knob table ``:9-17``); an uncached grad-bearing forward
whose hidden state is narrowed to the completion window *before* the final
norm and LM head (``:802-815``, ``:929-935``); a remat forward (``:941-955``);
and a grad-free cached decoder over merged weights (``:1635-1828``).

How it is laid out here for B200:

* q|k|v and gate|up are single fused projections (one GEMM each, LoRA deltas
  as extra k-tiles, see ``models.lora``); a transposed copy of every frozen
  weight stays resident so backward GEMMs also stream K-major tiles.
* attention goes through ``ops.attention`` (flash kernel, GQA native, causal
  mask in-kernel) and ``ops.decode_attention`` (KV-cached, GQA groups share the
  K/V loads) - no ``repeat_kv`` copies, no mask tensors, no cache ``cat``.
* rollout keeps its KV cache preallocated ``[B, Smax, Hkv, D]`` per layer and
  all per-row state (lengths, finished flags) on the device, so a decode step
  has fixed shapes and can be replayed as a CUDA graph.
* the group's shared prompt is prefilled once and its KV rows are broadcast to
  the G completions instead of prefilling G identical copies.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn

from .. import ops
from ..comm import Comm, SoloComm
from ..parallel.tp import TensorParallelPlan, copy_to_tp
from ..remat import remat_segment
from .lora import BaseQuantization, DenseLoraTargets, FusedLoraLinear, LoraSpec, Shard


@dataclass
class DenseSpec:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    qk_norm: bool = True
    sdpa_f32: bool = False
    activation: str = "silu"
    rope_theta: float = 1e6
    max_position_embeddings: int = 4096
    inv_freq: Optional[torch.Tensor] = None  # overrides rope_theta (llama3 smoothing)
    family: str = "qwen3"

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("query heads must be a multiple of kv heads")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for RoPE")
        for n in ("vocab_size", "hidden_size", "num_hidden_layers", "intermediate_size"):
            if getattr(self, n) <= 0:
                raise ValueError(f"{n} must be > 0")

    def rope_inv_freq(self) -> torch.Tensor:
        return self.inv_freq if self.inv_freq is not None else ops.default_inv_freq(self.head_dim, self.rope_theta)


class DenseLayer(nn.Module):
    def __init__(self, spec: DenseSpec, lora: Optional[LoraSpec], dtype, device,
                 tp: Optional[TensorParallelPlan], keep_transpose: bool, quant: BaseQuantization,
                 trainable_base: bool = False):
        super().__init__()
        H, D = spec.hidden_size, spec.head_dim
        hq, hkv, F = spec.num_attention_heads, spec.num_key_value_heads, spec.intermediate_size
        w = tp.world if tp else 1
        r = tp.rank if tp else 0
        t = lora.targets if lora else DenseLoraTargets(*(False,) * 7)
        col = Shard("column", r, w) if tp and w > 1 else None
        row = Shard("row", r, w) if tp and w > 1 else None
        kw = dict(dtype=dtype, device=device, keep_transpose=keep_transpose, quant=quant,
                  trainable_base=trainable_base)
        self.hq, self.hkv, self.D = hq // w, hkv // w, D
        self.qkv = FusedLoraLinear(H, [hq * D // w, hkv * D // w, hkv * D // w], ("q", "k", "v"),
                                   (t.attn_q, t.attn_k, t.attn_v), lora, shard=col,
                                   full_out_sizes=[hq * D, hkv * D, hkv * D], **kw)
        self.o = FusedLoraLinear(hq * D // w, [H], ("o",), (t.attn_o,), lora, shard=row,
                                 full_in=hq * D, **kw)
        self.gate_up = FusedLoraLinear(H, [F // w, F // w], ("gate", "up"), (t.mlp_gate, t.mlp_up), lora,
                                       shard=col, full_out_sizes=[F, F], **kw)
        self.gate_up.enable_glu_layout()      # rollout snapshot interleaved for the GEMM's GLU epilogue
        self.down = FusedLoraLinear(F // w, [H], ("down",), (t.mlp_down,), lora, shard=row, full_in=F, **kw)
        mk = (lambda n: nn.Parameter(torch.ones(n, dtype=dtype, device=device))) if trainable_base else None
        for name, n in (("input_norm", H), ("post_norm", H)) + ((("q_norm", D), ("k_norm", D)) if spec.qk_norm else ()):
            if trainable_base:
                setattr(self, name, mk(n))
            else:
                self.register_buffer(name, torch.ones(n, dtype=dtype, device=device), persistent=False)
        if not spec.qk_norm:
            self.q_norm = None
            self.k_norm = None
        self.eps = spec.rms_norm_eps
        self.scale = 1.0 / math.sqrt(D)
        self.act = spec.activation
        self.sdpa_f32 = spec.sdpa_f32

    def projections(self):
        return (self.qkv, self.o, self.gate_up, self.down)

    def adapter_params(self):
        out = []
        for p in self.projections():
            out += p.adapter_params()
        return out

    # full-sequence forward (training / scoring / prefill)
    def forward(self, h, positions, cos, sin, comm: Comm, merged: bool = False, kv_out=None):
        B, S, _ = h.shape
        lin = (lambda m, x: m.forward_merged(x)) if merged else (lambda m, x: m(x))
        x = ops.rmsnorm(h, self.input_norm, self.eps)
        x = copy_to_tp(x, comm)
        qkv = lin(self.qkv, x)
        q, k, v = qkv.split([self.hq * self.D, self.hkv * self.D, self.hkv * self.D], dim=-1)
        q = q.reshape(B, S, self.hq, self.D)
        k = k.reshape(B, S, self.hkv, self.D)
        v = v.reshape(B, S, self.hkv, self.D)
        q, k = ops.qk_norm_rope(q, k, self.q_norm, self.k_norm, self.eps, cos, sin, positions)
        if kv_out is not None:
            kv_out[0][:, :S].copy_(k)
            kv_out[1][:, :S].copy_(v)
        a = ops.attention(q, k, v, scale=self.scale, causal=True, softmax_fp32=True)
        o = self.o.forward_reduce(a.reshape(B, S, self.hq * self.D), comm, merged)
        x, h = ops.add_rmsnorm(o, h, self.post_norm, self.eps)
        x = copy_to_tp(x, comm)
        mid = self.gate_up.forward_merged_glu(x, self.act) if merged else ops.swiglu(self.gate_up(x), self.act)
        return self.down.forward_reduce(mid, comm, merged, residual=h)

    def forward_sp(self, hs, B, S, positions, cos, sin, comm: Comm, merged: bool = False):
        """Sequence-sharded form: ``hs`` holds this rank's block of the flattened ``[B * S, H]`` token rows.  The
        column-parallel projections gather the normalised rows (their backward reduce-scatters inside its GEMM),
        the row-parallel ones keep this rank's rows of the tensor-parallel sum; norms and residual adds run on the
        shard."""
        p = self.qkv.forward_gathered(ops.rmsnorm(hs, self.input_norm, self.eps), comm, merged).view(B, S, -1)
        q, k, v = p.split([self.hq * self.D, self.hkv * self.D, self.hkv * self.D], dim=-1)
        q = q.reshape(B, S, self.hq, self.D)
        k = k.reshape(B, S, self.hkv, self.D)
        v = v.reshape(B, S, self.hkv, self.D)
        q, k = ops.qk_norm_rope(q, k, self.q_norm, self.k_norm, self.eps, cos, sin, positions)
        a = ops.attention(q, k, v, scale=self.scale, causal=True, softmax_fp32=True)
        o = self.o.forward_reduce_scatter(a.reshape(B * S, self.hq * self.D), comm, merged)
        x, hs = ops.add_rmsnorm(o, hs, self.post_norm, self.eps)
        mid = ops.swiglu(self.gate_up.forward_gathered(x, comm, merged), self.act)
        return hs + self.down.forward_reduce_scatter(mid, comm, merged)

    # one-token forward against the cache (rollout; merged weights)
    def decode_fused(self, h, ss, kv_len, cos, sin, k_cache, v_cache, kv_next, pos, table=None, prefix=None):
        """One decode step of the layer in six kernels.  The two RMSNorms are folded around the
        projections: ``ss`` ``[parts, B]`` holds partial row sums of squares of ``h`` (written by the
        epilogue of the projection that produced ``h``), the QKV and gate/up projections scale their
        rows by the resulting ``rstd`` and read snapshots whose columns carry the norm weights, and the
        output and down projections add the residual and emit the statistics of the new ``h``.
        Returns ``(h_next, ss_next)``."""
        from ..ops import cuda as _c
        B = h.shape[0]
        qkv, _ = _c.gemm_norm(h, self.qkv.weight_decode, None, ss, self.eps)
        q, k, v = qkv.split([self.hq * self.D, self.hkv * self.D, self.hkv * self.D], dim=-1)
        qr = _c.qk_norm_rope_append(q.unflatten(-1, (self.hq, self.D)), k.unflatten(-1, (self.hkv, self.D)),
                                    v.unflatten(-1, (self.hkv, self.D)), self.q_norm, self.k_norm, self.eps, cos, sin,
                                    pos, k_cache, v_cache, kv_len, table)
        if qr is None:
            q4, k4 = ops.qk_norm_rope(q.reshape(B, 1, self.hq, self.D), k.reshape(B, 1, self.hkv, self.D), self.q_norm,
                                      self.k_norm, self.eps, cos, sin, pos)
            if table is not None:
                _c.kv_append_paged(k_cache, v_cache, k4[:, 0].contiguous(), v.reshape(B, self.hkv, self.D), kv_len, table)
            else:
                ops_cache_write(k_cache, v_cache, k4[:, 0], v.reshape(B, self.hkv, self.D), kv_len)
            qr = q4[:, 0]
        a = _c.decode_attention(qr, k_cache, v_cache, kv_next, scale=self.scale, block_table=table, **_prefix_kw(prefix))
        wo = self.o.weight_merged if self.o.weight_merged is not None else self.o.weight
        h2, ss2 = _c.gemm_norm(a.reshape(B, self.hq * self.D), wo, h, None, 0.0, None, True)
        mid, _ = _c.gemm_norm(h2, self.gate_up.weight_decode, None, ss2, self.eps, self.act)
        wd = self.down.weight_merged if self.down.weight_merged is not None else self.down.weight
        return _c.gemm_norm(mid, wd, h2, None, 0.0, None, True)

    def decode(self, h, kv_len, cos, sin, k_cache, v_cache, comm: Comm, kv_next=None, pos=None, table=None, prefix=None):
        B = h.shape[0]
        x = ops.rmsnorm(h, self.input_norm, self.eps)
        qkv = self.qkv.forward_merged(x)
        q, k, v = qkv.split([self.hq * self.D, self.hkv * self.D, self.hkv * self.D], dim=-1)
        if ops.native(qkv) and cos.dtype == torch.float32 and (table is not None or k_cache.dim() == 4):
            # one kernel: QK-norm, RoPE and the cache write of this token's K and V
            from ..ops import cuda as _c
            qr = _c.qk_norm_rope_append(q.unflatten(-1, (self.hq, self.D)), k.unflatten(-1, (self.hkv, self.D)),
                                        v.unflatten(-1, (self.hkv, self.D)), self.q_norm, self.k_norm, self.eps, cos, sin,
                                        pos if pos is not None else kv_len[:, None].long(), k_cache, v_cache, kv_len, table)
            if qr is not None:
                a = _c.decode_attention(qr, k_cache, v_cache, kv_next if kv_next is not None else kv_len + 1,
                                        scale=self.scale, block_table=table, **_prefix_kw(prefix))
                o = self.o.forward_reduce(a.reshape(B, self.hq * self.D), comm, merged=True)
                x, h = ops.add_rmsnorm(o, h, self.post_norm, self.eps)
                return self.down.forward_reduce(self.gate_up.forward_merged_glu(x, self.act), comm, merged=True,
                                                residual=h)
        q = q.reshape(B, 1, self.hq, self.D)
        k = k.reshape(B, 1, self.hkv, self.D)
        v = v.reshape(B, 1, self.hkv, self.D)
        q, k = ops.qk_norm_rope(q, k, self.q_norm, self.k_norm, self.eps, cos, sin,
                                pos if pos is not None else kv_len[:, None].long())
        if table is not None and ops.native(k_cache):
            from ..ops import cuda as _c
            _c.kv_append_paged(k_cache, v_cache, k[:, 0].contiguous(), v[:, 0], kv_len, table)
            a = _c.decode_attention(q[:, 0], k_cache, v_cache, kv_next if kv_next is not None else kv_len + 1,
                                    scale=self.scale, block_table=table, **_prefix_kw(prefix))
        elif table is not None:
            # eager restatement of the paged path (CPU tests of the block-table logic)
            page = k_cache.shape[1]
            t = kv_len.long()
            rows = torch.arange(B, device=h.device)
            slot_page = table[rows, t // page].long()
            k_cache[slot_page, t % page] = k[:, 0]
            v_cache[slot_page, t % page] = v[:, 0]
            kc = k_cache[table.long()].reshape(B, -1, self.hkv, self.D)       # [B, max_pages*page, Hkv, D]
            vc = v_cache[table.long()].reshape(B, -1, self.hkv, self.D)
            a = ops.decode_attention(q[:, 0], kc, vc, kv_next if kv_next is not None else kv_len + 1, scale=self.scale)
        else:
            ops_cache_write(k_cache, v_cache, k[:, 0], v[:, 0], kv_len)
            a = ops.decode_attention(q[:, 0], k_cache, v_cache, kv_next if kv_next is not None else kv_len + 1,
                                     scale=self.scale)
        o = self.o.forward_reduce(a.reshape(B, self.hq * self.D), comm, merged=True)
        x, h = ops.add_rmsnorm(o, h, self.post_norm, self.eps)
        return self.down.forward_reduce(self.gate_up.forward_merged_glu(x, self.act), comm, merged=True,
                                        residual=h)


def _prefix_kw(prefix) -> dict:
    """``prefix = (prefix_len [P] int32, group)`` of a paged grouped cache -> keyword arguments of
    ``decode_attention`` (empty when the cache has no shared prefix)."""
    return {} if prefix is None else {"prefix_len": prefix[0], "group": prefix[1]}


# Opt-in (FERRL_DECODE_FOLD=1): on the Qwen3-8B benchmark the folded chain launches 37 % fewer kernels
# per decode step and shortens rollout by 1.5 %, but its extra snapshots (9 GB) slow the training
# phases of the same step by more than that, so the default decode step keeps the two RMSNorm
# kernels per layer.
_DECODE_FOLD = os.environ.get("FERRL_DECODE_FOLD", "0") == "1"


def _decode_fused_ok(layers, h, comm) -> bool:
    """The decode chain with folded norms needs bf16 CUDA tensors, one rank and the folded snapshots."""
    if comm.world_size != 1 or not ops.native(h) or h.dtype != torch.bfloat16 or not _DECODE_FOLD:
        return False
    for l in layers:
        if l.qkv.weight_decode is None or l.gate_up.weight_decode is None or l.act not in ("silu", "gelu_pytorch_tanh",
                                                                                            "gelu_tanh"):
            return False
    return True


def ops_cache_write(k_cache, v_cache, k, v, kv_len):
    """Write one token's K/V per row at that row's current length."""
    if ops.native(k) and k.dtype == torch.bfloat16:
        from ..ops import cuda as _c
        _c.kv_append(k_cache, v_cache, k.contiguous(), v, kv_len)
        return
    idx = kv_len.long()
    rows = torch.arange(k.shape[0], device=k.device)
    k_cache[rows, idx] = k
    v_cache[rows, idx] = v


class DenseGradModel(nn.Module):
    """Policy network: grad-bearing scoring forward plus the cached decoder."""

    def __init__(self, spec: DenseSpec, lora: Optional[LoraSpec] = None, *, dtype=torch.float32,
                 device=None, tp: Optional[TensorParallelPlan] = None, keep_transpose: Optional[bool] = None,
                 quant: BaseQuantization = BaseQuantization.NONE, remat: bool = False,
                 full_ft: bool = False, sequence_parallel: bool = False):
        super().__init__()
        spec.validate()
        if tp is not None and (tp.num_heads != spec.num_attention_heads or tp.num_kv_heads != spec.num_key_value_heads):
            raise ValueError("tensor-parallel plan does not match the model's head counts")
        self.spec = spec
        self.lora = lora
        self.tp = tp
        # tensor parallelism with the residual stream sharded over the token rows (training and scoring passes)
        self.sequence_parallel = bool(sequence_parallel)
        self.remat = remat
        self.full_ft = full_ft
        dev = torch.device(device) if device is not None else torch.device("cpu")
        if keep_transpose is None:
            keep_transpose = dev.type == "cuda" and not full_ft
        self.dtype = dtype
        emb = torch.zeros(spec.vocab_size, spec.hidden_size, dtype=dtype, device=dev)
        if full_ft:
            self.embed = nn.Parameter(emb)
            self.final_norm = nn.Parameter(torch.ones(spec.hidden_size, dtype=dtype, device=dev))
        else:
            self.register_buffer("embed", emb, persistent=False)
            self.register_buffer("final_norm", torch.ones(spec.hidden_size, dtype=dtype, device=dev), persistent=False)
        if spec.tie_word_embeddings:
            self.lm_head = None
        elif full_ft:
            self.lm_head = nn.Parameter(torch.zeros(spec.vocab_size, spec.hidden_size, dtype=dtype, device=dev))
        else:
            self.register_buffer("lm_head", torch.zeros(spec.vocab_size, spec.hidden_size, dtype=dtype, device=dev),
                                 persistent=False)
        self.register_buffer("head_t", None, persistent=False)
        self.layers = nn.ModuleList([DenseLayer(spec, lora, dtype, dev, tp, keep_transpose, quant, full_ft)
                                     for _ in range(spec.num_hidden_layers)])
        cos, sin = ops.rope_tables(spec.rope_inv_freq(), spec.max_position_embeddings)
        self.register_buffer("cos", cos.to(dev), persistent=False)
        self.register_buffer("sin", sin.to(dev), persistent=False)
        self.keep_transpose = keep_transpose

    # ------------------------------------------------------------ weights
    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02):
        """Random-init base weights (synthetic benchmarks) and LoRA adapters."""
        g = torch.Generator().manual_seed(seed)
        dev = self.embed.device

        def rnd(shape):
            # generate on the host in chunks to bound peak host memory
            out = torch.empty(shape, dtype=self.dtype, device=dev)
            flat = out.view(-1)
            step = 1 << 24
            for s in range(0, flat.numel(), step):
                n = min(step, flat.numel() - s)
                flat[s:s + n] = (torch.randn(n, generator=g) * std).to(self.dtype).to(dev)
            return out

        fast = dev.type == "cuda"
        if fast:
            gg = torch.Generator(device=dev).manual_seed(seed)

            def rnd(shape):  # noqa: F811 - device-side generation for the 8B-class benchmarks
                return (torch.randn(shape, generator=gg, device=dev, dtype=torch.float32) * std).to(self.dtype)
        self.embed.copy_(rnd(self.embed.shape))
        if self.lm_head is not None:
            self.lm_head.copy_(rnd(self.lm_head.shape))
        for l in self.layers:
            for p in l.projections():
                p.set_weight(rnd(p.weight.shape))
                p.init_adapters(g)
        self.refresh_head()

    @torch.no_grad()
    def refresh_head(self):
        if self.keep_transpose:
            self.head_t = self.head_weight().t().contiguous()

    def head_weight(self) -> torch.Tensor:
        return self.embed if self.lm_head is None else self.lm_head

    def trainable_params(self) -> list[nn.Parameter]:
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
        return self.lora.recipe() if self.lora else "none"

    @torch.no_grad()
    def merge_adapters(self):
        for l in self.layers:
            if _DECODE_FOLD and l.qkv.shard is None and l.gate_up.shard is None:
                # second rollout snapshot with the RMSNorm weights folded in: the decode chain then needs
                # no normalisation kernels (see DenseLayer.decode_fused)
                l.qkv.enable_decode_fold(l.input_norm)
                l.gate_up.enable_decode_fold(l.post_norm, glu=True)
            for p in l.projections():
                p.merge()

    # ------------------------------------------------------------- forward
    def forward_hidden(self, ids: torch.Tensor, comm: Optional[Comm] = None, merged: bool = False,
                       kv_out=None, detached: bool = False) -> torch.Tensor:
        comm = comm or SoloComm()
        B, S = ids.shape
        if S > self.cos.shape[0]:
            raise ValueError(f"sequence length {S} exceeds max_position_embeddings {self.cos.shape[0]}")
        positions = torch.arange(S, device=ids.device)
        h = ops.embedding(ids, self.embed)
        if self.sequence_parallel and comm.world_size > 1 and kv_out is None and (B * S) % comm.world_size == 0:
            from ..parallel import sp
            hs = sp.shard_rows(h.reshape(B * S, -1), comm)
            for layer in self.layers:
                fn = (lambda x, layer=layer: layer.forward_sp(x, B, S, positions, self.cos, self.sin, comm, merged))
                if self.remat and torch.is_grad_enabled() and not detached:
                    hs = remat_segment(fn, hs, layer.adapter_params() if not self.full_ft else list(layer.parameters()), None)
                else:
                    hs = fn(hs)
            return sp.gather_rows_replicated(hs, comm).view(B, S, -1)
        cot = (lambda g: g)  # boundary cotangents are already reduced by copy_to_tp's backward
        for i, layer in enumerate(self.layers):
            kv = None if kv_out is None else kv_out[i]
            if self.remat and torch.is_grad_enabled() and not detached:
                fn = (lambda x, layer=layer: layer(x, positions, self.cos, self.sin, comm, merged, None))
                h = remat_segment(fn, h, layer.adapter_params() if not self.full_ft else list(layer.parameters()), None)
            else:
                h = layer(h, positions, self.cos, self.sin, comm, merged, kv)
        del cot
        return h

    def forward(self, ids: torch.Tensor, comm: Optional[Comm] = None) -> torch.Tensor:
        """Full-position logits ``[B, S, V]`` in float32 (oracle/test surface)."""
        h = self.forward_hidden(ids, comm)
        h = ops.rmsnorm(h, self.final_norm, self.spec.rms_norm_eps)
        return torch.nn.functional.linear(h, self.head_weight()).float()

    def token_logprobs(self, ids: torch.Tensor, win_start: torch.Tensor, targets: torch.Tensor,
                       temperature: float = 1.0, comm: Optional[Comm] = None) -> torch.Tensor:
        """Log-probs of ``targets[b, t]`` predicted at position ``win_start[b]+t``.
        The hidden state is narrowed to the window before the final norm and the
        head, and ``[.., V]`` logits never outlive a chunk."""
        h = self.forward_hidden(ids, comm, detached=not torch.is_grad_enabled())
        B, L = targets.shape
        idx = (win_start.view(B, 1).long() + torch.arange(L, device=ids.device)[None, :]).clamp(max=ids.shape[1] - 1)
        hw = torch.gather(h, 1, idx[:, :, None].expand(B, L, h.shape[-1]))
        hw = ops.rmsnorm(hw, self.final_norm, self.spec.rms_norm_eps)
        lp = ops.logprob_gather(hw.reshape(B * L, -1), self.head_weight(), targets.reshape(-1), temperature,
                                0.0, head_wt=self.head_t)
        return lp.view(B, L)

    # ------------------------------------------------------------- rollout
    def new_decoder(self, batch: int, max_len: int, comm: Optional[Comm] = None, group: int = 1,
                    paged: Optional[bool] = None) -> "DenseCachedDecoder":
        """``group`` > 1 on a GPU selects the paged cache whose prompt pages are shared by the
        ``group`` rows of a prompt (rows are prompt-major: row ``p*group + g``)."""
        comm = comm or SoloComm()
        if paged is None:
            paged = (ops.native(self.embed) and self.dtype == torch.bfloat16 and group > 1 and batch % group == 0
                     and self.spec.head_dim % 8 == 0)
        if paged:
            return DensePagedDecoder(self, batch, max_len, comm, group)
        return DenseCachedDecoder(self, batch, max_len, comm)


class DenseCachedDecoder:
    """KV-cached, grad-free twin over merged weights. ``kv_len[b]`` tokens of row
    ``b`` are cached; a decode step must be fed position ``kv_len[b]`` exactly
    (the reference guards the same invariant, dense.rs:1708-1717)."""

    def __init__(self, model: DenseGradModel, batch: int, max_len: int, comm: Comm):
        self.m = model
        self.comm = comm
        spec = model.spec
        if max_len > spec.max_position_embeddings:
            raise ValueError("cache longer than the RoPE table")
        dev, dt = model.embed.device, model.dtype
        hkv = model.layers[0].hkv
        self.k = [torch.zeros(batch, max_len, hkv, spec.head_dim, dtype=dt, device=dev) for _ in model.layers]
        self.v = [torch.zeros(batch, max_len, hkv, spec.head_dim, dtype=dt, device=dev) for _ in model.layers]
        self.kv_len = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.max_len = max_len
        self.batch = batch

    def cache_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, lens: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Prefill ``ids`` ``[P, L]`` (right-padded, true lengths ``lens``) into
        cache rows ``rows`` (default ``0..P``); returns last-token logits ``[P, V]``."""
        m = self.m
        P, L = ids.shape
        rows = torch.arange(P, device=ids.device) if rows is None else rows
        tmp = [(torch.empty(P, L, self.k[0].shape[2], self.k[0].shape[3], dtype=m.dtype, device=ids.device),
                torch.empty(P, L, self.k[0].shape[2], self.k[0].shape[3], dtype=m.dtype, device=ids.device))
               for _ in m.layers]
        h = m.forward_hidden(ids, self.comm, merged=True, kv_out=tmp, detached=True)
        for i in range(len(m.layers)):
            self.k[i][rows, :L] = tmp[i][0]
            self.v[i][rows, :L] = tmp[i][1]
        self.kv_len[rows] = lens.to(torch.int32)
        last = h[torch.arange(P, device=ids.device), (lens - 1).long()]
        last = ops.rmsnorm(last, m.final_norm, m.spec.rms_norm_eps)
        return ops.lora_linear(last, m.head_weight(), None, None).float()

    @torch.no_grad()
    def broadcast_groups(self, group: int):
        """Rows ``0..P`` hold one prefilled prompt each; replicate so that row
        ``p*group + g`` holds prompt ``p`` (the group shares its prompt's KV)."""
        P = self.batch // group
        src = torch.arange(P, device=self.kv_len.device).repeat_interleave(group)
        for i in range(len(self.k)):
            self.k[i].copy_(self.k[i][src])
            self.v[i].copy_(self.v[i][src])
        self.kv_len.copy_(self.kv_len[src])

    supports_retirement = True      # ``decode(tokens, active)``: see ``_step_lengths``

    def _step_lengths(self, active: Optional[torch.Tensor]):
        """Attention length of every row for this token and the length increment afterwards.
        A retired row (``active[b]`` false: it has emitted EOS) attends to nothing, so the decode
        attention kernels read none of its KV, and its cache length stays frozen (its pad token is
        written over the same slot every step).  The reference drops such rows from the batch
        (lm_policy.rs:736-743); here the batch keeps its shape, so a captured CUDA graph stays valid,
        and the projections, whose cost is the weight stream, do not care about the row count."""
        if active is None:
            return self.kv_len + 1, None
        inc = active.to(torch.int32)
        return (self.kv_len + 1) * inc, inc

    def kv_tokens_read(self, active: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Tokens of KV that the next ``decode`` call's attention reads per layer (sum of the lengths
        handed to the kernel): the quantity row retirement shrinks."""
        return self._step_lengths(active)[0].sum()

    @torch.no_grad()
    def decode(self, tokens: torch.Tensor, active: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Feed one token per row; returns next-token logits ``[B, V]`` float32."""
        return self.decode_native(tokens, active).float()

    @torch.no_grad()
    def decode_native(self, tokens: torch.Tensor, active: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``decode`` with the logits left in the head GEMM's output dtype (bf16 for a bf16 model): the
        device sampler reads them as they are, which saves the fp32 copy of ``[B, V]`` every token."""
        m = self.m
        h = ops.embedding(tokens, m.embed)
        kv_next, inc = self._step_lengths(active)  # shared by every layer: computed once per token
        pos = self.kv_len[:, None].long()
        if _decode_fused_ok(m.layers, h, self.comm) and m.cos.dtype == torch.float32:
            from ..ops import cuda as _c
            ss = _c.row_sumsq(h)
            for i, layer in enumerate(m.layers):
                h, ss = layer.decode_fused(h, ss, self.kv_len, m.cos, m.sin, self.k[i], self.v[i], kv_next, pos)
        else:
            for i, layer in enumerate(m.layers):
                h = layer.decode(h, self.kv_len, m.cos, m.sin, self.k[i], self.v[i], self.comm, kv_next, pos)
        self.kv_len += 1 if inc is None else inc
        h = ops.rmsnorm(h, m.final_norm, m.spec.rms_norm_eps)
        return ops.lora_linear(h, m.head_weight(), None, None)


class DensePagedDecoder(DenseCachedDecoder):
    """Paged twin of ``DenseCachedDecoder`` for grouped rollouts.

    K/V live in a per-layer pool ``[n_pages, PAGE, Hkv, D]`` addressed through one block table
    ``[B, max_pages]`` shared by all layers.  The full pages of a prompt are stored once and
    referenced by all ``group`` rows of that prompt, so decode attention reads them from HBM once
    per group (the other rows hit L2) and prefill needs no per-row copy of the prompt; the
    prompt's ragged tail and everything generated go to row-private pages.  The reference keeps
    one contiguous cache per row (``crates/ferrl/src/dense.rs`` cached decoder)."""

    PAGE = 64

    def __init__(self, model: DenseGradModel, batch: int, max_len: int, comm: Comm, group: int):
        self.m, self.comm = model, comm
        spec = model.spec
        if max_len > spec.max_position_embeddings:
            raise ValueError("cache longer than the RoPE table")
        if batch % group:
            raise ValueError("batch must be a multiple of the group size")
        dev, dt = model.embed.device, model.dtype
        hkv, D, page = model.layers[0].hkv, spec.head_dim, self.PAGE
        self.group, self.batch, self.max_len = group, batch, max_len
        self.prompts = batch // group
        self.pages_per_row = (max_len + page - 1) // page
        self.shared_pages = self.prompts * self.pages_per_row          # upper bound: a prompt as long as the cache
        n_pages = self.shared_pages + batch * self.pages_per_row
        self.k = [torch.zeros(n_pages, page, hkv, D, dtype=dt, device=dev) for _ in model.layers]
        self.v = [torch.zeros(n_pages, page, hkv, D, dtype=dt, device=dev) for _ in model.layers]
        self.table = torch.zeros(batch, self.pages_per_row, dtype=torch.int32, device=dev)
        self.kv_len = torch.zeros(batch, dtype=torch.int32, device=dev)
        # tokens of each prompt that live in shared pages: decode attention streams them once per group
        self.prefix_len = torch.zeros(self.prompts, dtype=torch.int32, device=dev)
        from ..ops import cuda as _c
        self.share_prefix = (os.environ.get("FERRL_PREFIX_ATTN", "1") != "0" and ops.native(self.k[0])
                             and _c.prefix_attention_supported(D, model.layers[0].hq // hkv, group))

    def _prefix(self):
        return (self.prefix_len, self.group) if self.share_prefix else None

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, lens: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Prefill the ``P = batch // group`` prompts; afterwards every row ``p*group + g`` sees its
        prompt (``broadcast_groups`` has nothing left to copy)."""
        if rows is not None:
            raise ValueError("the paged decoder prefills all prompts at once")
        m, page, G = self.m, self.PAGE, self.group
        P, L = ids.shape
        if P != self.prompts:
            raise ValueError(f"expected {self.prompts} prompts, got {P}")
        dev = ids.device
        hkv, D = self.k[0].shape[2], self.k[0].shape[3]
        tmp = [(torch.empty(P, L, hkv, D, dtype=m.dtype, device=dev), torch.empty(P, L, hkv, D, dtype=m.dtype, device=dev))
               for _ in m.layers]
        h = m.forward_hidden(ids, self.comm, merged=True, kv_out=tmp, detached=True)
        ppr = self.pages_per_row
        full = (lens // page).to(torch.int64)                                  # shared (full) pages per prompt
        # block table: shared page ids first, then the row's private pages
        j = torch.arange(ppr, device=dev)[None, :]
        p_of_row = torch.arange(P, device=dev).repeat_interleave(G)
        full_r = full[p_of_row][:, None]
        shared_id = p_of_row[:, None] * ppr + j
        private_id = self.shared_pages + torch.arange(self.batch, device=dev)[:, None] * ppr + (j - full_r).clamp(min=0)
        self.table.copy_(torch.where(j < full_r, shared_id, private_id).to(torch.int32))
        self.prefix_len.copy_((full * page).to(torch.int32))
        # tail of every prompt (< PAGE tokens) goes to the first private page of each of its rows
        tail_idx = (full[:, None] * page + torch.arange(page, device=dev)[None, :]).clamp(max=L - 1)     # [P, PAGE]
        first_private = (self.shared_pages + torch.arange(self.batch, device=dev) * ppr).long()
        Lp = min(L, ppr * page)
        for i in range(len(m.layers)):
            for pool, src in ((self.k[i], tmp[i][0]), (self.v[i], tmp[i][1])):
                pool[:self.shared_pages].view(P, ppr * page, hkv, D)[:, :Lp] = src[:, :Lp]
                tail = torch.gather(src, 1, tail_idx[:, :, None, None].expand(P, page, hkv, D))
                pool[first_private] = tail.repeat_interleave(G, dim=0)
        self.kv_len.copy_(lens.to(torch.int32).repeat_interleave(G))
        last = h[torch.arange(P, device=dev), (lens - 1).long()]
        last = ops.rmsnorm(last, m.final_norm, m.spec.rms_norm_eps)
        return ops.lora_linear(last, m.head_weight(), None, None).float()

    @torch.no_grad()
    def broadcast_groups(self, group: int):
        if group != self.group:
            raise ValueError("group size differs from the one this cache was built for")

    @torch.no_grad()
    def decode_native(self, tokens: torch.Tensor, active: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = self.m
        h = ops.embedding(tokens, m.embed)
        kv_next, inc = self._step_lengths(active)
        pos = self.kv_len[:, None].long()
        if _decode_fused_ok(m.layers, h, self.comm) and m.cos.dtype == torch.float32:
            from ..ops import cuda as _c
            ss = _c.row_sumsq(h)
            for i, layer in enumerate(m.layers):
                h, ss = layer.decode_fused(h, ss, self.kv_len, m.cos, m.sin, self.k[i], self.v[i], kv_next, pos, self.table,
                                            self._prefix())
        else:
            for i, layer in enumerate(m.layers):
                h = layer.decode(h, self.kv_len, m.cos, m.sin, self.k[i], self.v[i], self.comm, kv_next, pos, self.table,
                                 self._prefix())
        self.kv_len += 1 if inc is None else inc
        h = ops.rmsnorm(h, m.final_norm, m.spec.rms_norm_eps)
        return ops.lora_linear(h, m.head_weight(), None, None)
