"""LoRA over frozen linear projections, grouped by shared input.

A ``FusedLoraLinear`` owns one frozen weight whose rows are the concatenation
of several logical projections that read the same activation (q|k|v, gate|up)
or a single projection (o, down).  Each adapted projection ``i`` has float32
master adapters ``A_i [r, in]`` (normal, std 0.02) and ``B_i [out_i, r]``
(zeros) with scale ``alpha / r`` over a bf16 (or fp32) frozen base, as in the
reference (``crates/ferrl/src/lora.rs:1044-1406``).

B200 layout: the group is evaluated as ONE GEMM whose K dimension is extended
by the stacked LoRA width, ``y = [x | x A_stackᵀ] · [W | s·B_blockdiag]ᵀ``,
so the LoRA delta is extra k-tiles of the same tcgen05 tile loop instead of
three more matmuls and an add.  ``x A_stackᵀ`` is one skinny GEMM for the whole
group.  The stacks are rebuilt from the masters each call with differentiable
torch ops, so autograd delivers per-projection gradients in master layout and
checkpoints keep one tensor per adapter.

Rollout does not run the side path at all: ``merged_weight`` folds ``W+s·B·A``
into a second resident copy of the weights (HBM3e has room), rebuilt once per
policy update (reference lora.rs:1335-1350 rebuilds per ``generate`` call).

Tensor parallelism follows the reference's slicing-at-use rule
(``lora.rs:1245-1304``): adapters stay replicated; a column-parallel shard uses
the matching rows of ``B``, a row-parallel shard the matching columns of ``A``.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
from torch import nn

from .. import ops


class BaseQuantization(str, enum.Enum):
    NONE = "none"
    Q8_0 = "q8_0"


# closed ranges of finite, positive values of the 16-bit compute dtypes (smallest subnormal .. largest finite)
_SCALE_RANGE = {torch.float16: (5.960464477539063e-08, 65504.0),
                torch.bfloat16: (9.183549615799121e-41, 3.3895313892515355e38)}
_DTYPE_NAME = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16"}


def validated_lora_scale(rank: int, alpha: float, compute_dtype: Optional[torch.dtype] = None) -> float:
    """``alpha / rank``, which must stay finite and nonzero when narrowed to the dtype the base weight computes in
    (``None``: float64).  Reference: crates/ferrl/src/lora.rs:1072-1100."""
    if rank <= 0:
        raise ValueError("lora rank must be > 0")
    if not math.isfinite(alpha) or alpha <= 0:
        raise ValueError("lora alpha must be finite and > 0")
    s = alpha / rank
    dt = compute_dtype or torch.float64
    if dt == torch.float64:
        ok = math.isfinite(s) and s > 0
    elif dt == torch.float32:
        narrowed = float(torch.tensor(s, dtype=torch.float64).to(torch.float32))
        ok = math.isfinite(narrowed) and narrowed > 0
    elif dt in _SCALE_RANGE:
        ok = _SCALE_RANGE[dt][0] <= s <= _SCALE_RANGE[dt][1]
    else:
        ok = False
    if not ok:
        raise ValueError(f"lora scale alpha/rank = {s} must be finite and nonzero in compute dtype "
                         f"{_DTYPE_NAME.get(dt, str(dt))}")
    return s


@dataclass(frozen=True)
class DenseLoraTargets:
    """Which of the seven dense projections carry adapters (reference
    lora.rs:635-735). ``canonical()`` is part of the checkpoint recipe."""

    attn_q: bool = True
    attn_k: bool = True
    attn_v: bool = True
    attn_o: bool = True
    mlp_gate: bool = True
    mlp_up: bool = True
    mlp_down: bool = True

    @staticmethod
    def industrial() -> "DenseLoraTargets":
        return DenseLoraTargets()

    @staticmethod
    def legacy() -> "DenseLoraTargets":
        return DenseLoraTargets(True, False, True, False, False, False, False)

    @staticmethod
    def attention_only() -> "DenseLoraTargets":
        return DenseLoraTargets(True, True, True, True, False, False, False)

    def any(self) -> bool:
        return any((self.attn_q, self.attn_k, self.attn_v, self.attn_o,
                    self.mlp_gate, self.mlp_up, self.mlp_down))

    def canonical(self) -> str:
        def pick(pairs):
            s = "".join(c for on, c in pairs if on)
            return s or "-"
        return "attn:{}|mlp:{}".format(
            pick([(self.attn_q, "q"), (self.attn_k, "k"), (self.attn_v, "v"), (self.attn_o, "o")]),
            pick([(self.mlp_gate, "g"), (self.mlp_up, "u"), (self.mlp_down, "d")]))

    @staticmethod
    def parse(s: str) -> "DenseLoraTargets":
        if s in ("industrial", "all"):
            return DenseLoraTargets.industrial()
        if s in ("legacy", "qv"):
            return DenseLoraTargets.legacy()
        try:
            parts = dict(p.split(":") for p in s.split("|"))
            a, m = parts.get("attn", "-"), parts.get("mlp", "-")
        except ValueError as e:
            raise ValueError(f"bad LoRA target string {s!r}") from e
        if set(a) - set("qkvo-") or set(m) - set("gud-"):
            raise ValueError(f"bad LoRA target string {s!r}")
        return DenseLoraTargets("q" in a, "k" in a, "v" in a, "o" in a, "g" in m, "u" in m, "d" in m)


@dataclass
class LoraSpec:
    rank: int = 8
    alpha: float = 16.0
    targets: DenseLoraTargets = field(default_factory=DenseLoraTargets)

    @property
    def scale(self) -> float:
        return validated_lora_scale(self.rank, self.alpha)

    def recipe(self) -> str:
        return f"lora:r{self.rank}:a{self.alpha:g}:{self.targets.canonical()}"


@dataclass(frozen=True)
class Shard:
    """Tensor-parallel placement of a projection group. ``kind`` is ``column``
    (output rows split) or ``row`` (input columns split)."""

    kind: str
    rank: int
    world: int


def q8_0_quantize(w: torch.Tensor):
    """GGML-style Q8_0: blocks of 32 along the input dim, one fp16 scale each."""
    out, inn = w.shape
    if inn % 32:
        raise ValueError("Q8_0 needs the input dim to be a multiple of 32")
    blocks = w.float().reshape(out, inn // 32, 32)
    d = blocks.abs().amax(-1, keepdim=True) / 127.0
    q = torch.where(d > 0, blocks / d.clamp(min=1e-30), torch.zeros_like(blocks)).round().clamp(-127, 127)
    return q.to(torch.int8).reshape(out, inn), d.squeeze(-1).half()


def q8_0_dequantize(q: torch.Tensor, d: torch.Tensor, dtype) -> torch.Tensor:
    out, inn = q.shape
    return (q.reshape(out, inn // 32, 32).float() * d.float().unsqueeze(-1)).reshape(out, inn).to(dtype)


class FusedLoraLinear(nn.Module):
    """Frozen ``[sum(out_sizes), in]`` weight + optional adapters per logical
    projection.  ``names`` label the projections (``("q","k","v")``)."""

    def __init__(self, in_features: int, out_sizes: Sequence[int], names: Sequence[str],
                 adapted: Sequence[bool], lora: Optional[LoraSpec], *, dtype=torch.float32,
                 device=None, shard: Optional[Shard] = None, full_in: Optional[int] = None,
                 full_out_sizes: Optional[Sequence[int]] = None, keep_transpose: bool = False,
                 quant: BaseQuantization = BaseQuantization.NONE, trainable_base: bool = False):
        super().__init__()
        self.in_features = in_features
        self.out_sizes = list(out_sizes)
        self.names = list(names)
        self.shard = shard
        # adapters are replicated at FULL size under TP and sliced at use
        self.full_in = full_in if full_in is not None else in_features
        self.full_out_sizes = list(full_out_sizes) if full_out_sizes is not None else list(out_sizes)
        self.quant = BaseQuantization(quant)
        self.keep_transpose = keep_transpose
        self.enabled = True
        w = torch.empty(sum(out_sizes), in_features, dtype=dtype, device=device)
        if trainable_base:
            self.weight = nn.Parameter(w)
        else:
            self.register_buffer("weight", w, persistent=False)
        self.register_buffer("weight_t", None, persistent=False)
        self.register_buffer("weight_merged", None, persistent=False)
        self.weight_decode = None               # see enable_decode_fold()
        self._q = None
        # the scale multiplies values of the base weight's dtype: it must survive the narrowing
        self.scale = validated_lora_scale(lora.rank, lora.alpha, dtype) if lora is not None else 0.0
        self.rank = lora.rank if lora is not None else 0
        self.lora_A = nn.ParameterList()
        self.lora_B = nn.ParameterList()
        self.adapted_idx: list[int] = []
        if lora is not None:
            for i, on in enumerate(adapted):
                if not on:
                    continue
                self.adapted_idx.append(i)
                a = torch.empty(lora.rank, self.full_in, dtype=torch.float32, device=device)
                self.lora_A.append(nn.Parameter(a))
                self.lora_B.append(nn.Parameter(torch.zeros(self.full_out_sizes[i], lora.rank,
                                                            dtype=torch.float32, device=device)))

    # ---------------------------------------------------------------- init
    @torch.no_grad()
    def init_adapters(self, generator: Optional[torch.Generator] = None):
        for a in self.lora_A:
            a.copy_(torch.randn(a.shape, generator=generator, dtype=torch.float32) * 0.02)
        for b in self.lora_B:
            b.zero_()

    @torch.no_grad()
    def set_weight(self, w: torch.Tensor):
        """Install the (local shard of the) frozen weight and derived copies."""
        assert tuple(w.shape) == tuple(self.weight.shape), (w.shape, self.weight.shape)
        if self.quant is BaseQuantization.Q8_0:
            q, d = q8_0_quantize(w)
            self._q = (q.to(self.weight.device), d.to(self.weight.device))
            w = q8_0_dequantize(q, d, self.weight.dtype)
        self.weight.copy_(w)
        self.refresh_derived()

    @torch.no_grad()
    def refresh_derived(self):
        if self.keep_transpose:
            self.weight_t = self.weight.t().contiguous()
        self.weight_merged = None
        self.weight_decode = None

    # ------------------------------------------------------------- adapters
    def has_adapters(self) -> bool:
        return len(self.adapted_idx) > 0

    def _stacks(self):
        """Differentiable ``(A_stack [n*r, in_local], B_stack [out_local, n*r])``
        with the LoRA scale folded into ``B_stack`` and TP slicing applied."""
        if not self.has_adapters() or not self.enabled:
            return None, None
        r = self.rank
        A = torch.cat(list(self.lora_A), dim=0)  # [n*r, full_in]
        offs = 0
        starts = []
        for o in self.out_sizes:
            starts.append(offs)
            offs += o
        pieces = []
        for j, i in enumerate(self.adapted_idx):
            b = self.lora_B[j]
            if self.shard is not None and self.shard.kind == "column":
                per = self.full_out_sizes[i] // self.shard.world
                b = b[self.shard.rank * per:(self.shard.rank + 1) * per]
            pieces.append((starts[i], j, b))
        # block placement via padding keeps autograd simple and cheap
        rows = []
        cur = 0
        for start, j, b in sorted(pieces, key=lambda p: p[0]):
            if start > cur:
                rows.append(A.new_zeros(start - cur, r * len(self.adapted_idx)))
            left = A.new_zeros(b.shape[0], j * r)
            right = A.new_zeros(b.shape[0], (len(self.adapted_idx) - j - 1) * r)
            rows.append(torch.cat([left, b * self.scale, right], dim=1))
            cur = start + b.shape[0]
        if cur < sum(self.out_sizes):
            rows.append(A.new_zeros(sum(self.out_sizes) - cur, r * len(self.adapted_idx)))
        B = torch.cat(rows, dim=0)
        if self.shard is not None and self.shard.kind == "row":
            per = self.full_in // self.shard.world
            A = A[:, self.shard.rank * per:(self.shard.rank + 1) * per]
        return A, B

    # --------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        a, b = self._stacks()
        return ops.lora_linear(x, self.weight, a, b, wt=self.weight_t, residual=residual)

    def forward_reduce(self, x: torch.Tensor, comm, merged: bool = False, residual=None) -> torch.Tensor:
        """Row-parallel use: the projection, its tensor-parallel sum over ``comm`` and an
        optional residual add.  On GPUs with a registered ``GemmAllReducer`` all three happen
        in the GEMM kernel; otherwise the projection is followed by ``reduce_from_tp``."""
        from ..parallel.tp import reduce_from_tp
        if comm.world_size > 1 and x.is_cuda:
            from ..parallel.symm import gemm_all_reducer
            red = gemm_all_reducer(comm)
            if red is not None:
                from ..ops import cuda as _c
                if merged:
                    w = self.weight_merged if self.weight_merged is not None else self.weight
                    y = _c.lora_linear_reduce(x, w, None, None, None, red, residual)
                else:
                    a, b = self._stacks()
                    y = _c.lora_linear_reduce(x, self.weight, a, b, self.weight_t, red, residual)
                if y is not None:
                    return y
        if comm.world_size == 1:
            # no reduction to wait for: the residual rides in the GEMM epilogue
            return self.forward_merged(x, residual) if merged else self.forward(x, residual)
        y = reduce_from_tp(self.forward_merged(x) if merged else self.forward(x), comm)
        return y if residual is None else residual + y

    def forward_gathered(self, xs: torch.Tensor, comm, merged: bool = False) -> torch.Tensor:
        """Column-parallel use under sequence sharding: ``xs`` is this rank's ``[rows / world, in]`` block of the
        input and the result covers all rows.  On GPUs the gather runs over the symmetric heap and the backward's
        reduce-scatter of the input gradient happens inside its GEMM."""
        from ..parallel import sp
        if comm.world_size > 1 and xs.is_cuda and xs.dim() == 2:
            from ..parallel.symm import gemm_all_reducer
            from ..ops import cuda as _c
            gather = lambda z: sp.all_gather_rows_value(z, comm)            # noqa: E731
            scatter = lambda z: sp.reduce_scatter_rows_value(z, comm)       # noqa: E731
            if merged:
                w = self.weight_merged if self.weight_merged is not None else self.weight
                y = None if self._glu_rows() is not None else \
                    _c.gather_lora_linear(xs, w, None, None, None, gather, scatter, gemm_all_reducer(comm))
            else:
                a, b = self._stacks()
                y = _c.gather_lora_linear(xs, self.weight, a, b, self.weight_t, gather, scatter, gemm_all_reducer(comm))
            if y is not None:
                return y
        x = sp.gather_rows_tp(xs, comm)
        return self.forward_merged(x) if merged else self.forward(x)

    def forward_reduce_scatter(self, x: torch.Tensor, comm, merged: bool = False) -> torch.Tensor:
        """Row-parallel use under sequence sharding: ``x`` is ``[rows, in_local]`` and the result is this rank's
        ``rows / world`` rows of the tensor-parallel sum.  On GPUs with a registered ``GemmAllReducer`` the sum and
        the scatter happen in the GEMM kernel; otherwise the projection is followed by ``scatter_rows_sum``."""
        from ..parallel import sp
        if comm.world_size > 1 and x.is_cuda and x.dim() == 2:
            from ..parallel.symm import gemm_all_reducer
            red = gemm_all_reducer(comm)
            if red is not None:
                from ..ops import cuda as _c
                gather = lambda g: sp.all_gather_rows_value(g, comm)  # noqa: E731
                if merged:
                    w = self.weight_merged if self.weight_merged is not None else self.weight
                    y = _c.lora_linear_reduce_scatter(x, w, None, None, None, red, gather)
                else:
                    a, b = self._stacks()
                    y = _c.lora_linear_reduce_scatter(x, self.weight, a, b, self.weight_t, red, gather)
                if y is not None:
                    return y
        return sp.scatter_rows_sum(self.forward_merged(x) if merged else self.forward(x), comm)

    def forward_merged(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        """Rollout path over the merged snapshot (no adapter side path)."""
        w = self.weight_merged if self.weight_merged is not None else self.weight
        y = ops.lora_linear(x, w, None, None, residual=None if self._glu_rows() is not None else residual)
        if self._glu_rows() is not None:      # snapshot rows are interleaved for the fused GLU: undo it for plain use
            y = y.index_select(-1, self._glu_inverse)
            if residual is not None:
                y = residual + y
        return y

    # ------------------------------------------------------------ gate/up projections
    def enable_glu_layout(self):
        """For a fused [gate | up] projection: keep the merged snapshot with its rows interleaved in
        groups of 16 (8 gate rows, then the 8 up rows of the same features), the layout the GEMM's
        GLU epilogue reads, so that rollout computes ``act(gate) * up`` inside the projection.
        Takes effect at the next ``merge()`` on a bf16 CUDA weight; a plain snapshot otherwise."""
        self._glu_requested = True

    def _glu_rows(self):
        """Row permutation of the interleaved snapshot, or ``None`` when the snapshot is plain."""
        if not getattr(self, "_glu_active", False) or self.weight_merged is None:
            return None
        return self._glu_perm

    @staticmethod
    def glu_row_order(half: int, device=None) -> torch.Tensor:
        """Row order of an interleaved [gate | up] weight: groups of 16 rows, the 8 gate rows of features
        ``8q .. 8q+7`` followed by their 8 up rows (``half`` = number of features, a multiple of 8)."""
        g = torch.arange(half, device=device).view(-1, 8)
        return torch.stack([g, g + half], dim=1).reshape(-1)

    def _glu_prepare(self) -> bool:
        w = self.weight
        ok = getattr(self, "_glu_requested", False) and w.is_cuda and w.dtype == torch.bfloat16 and \
            w.shape[0] % 16 == 0 and (w.shape[0] // 2) % 8 == 0
        if ok and (getattr(self, "_glu_perm", None) is None or self._glu_perm.device != w.device):
            self._glu_perm = self.glu_row_order(w.shape[0] // 2, w.device)
            self._glu_inverse = torch.argsort(self._glu_perm)
        self._glu_active = bool(ok)
        return self._glu_active

    def enable_decode_fold(self, norm_weight, zero_centered: bool = False, glu: bool = False):
        """Keep a second rollout snapshot ``weight_decode`` whose columns carry the weight of the
        RMSNorm in front of this projection (and whose rows are interleaved for the GLU epilogue when
        ``glu``): the decode chain then applies the norm as a per-row scale in the GEMM epilogue
        (``ops.cuda.gemm_norm``) and needs no normalisation kernel.  Built by ``merge()`` on bf16
        CUDA weights."""
        self._fold_src = [norm_weight]          # in a list: not registered as this module's parameter
        self._fold_zc = bool(zero_centered)
        self._fold_glu = bool(glu)

    @torch.no_grad()
    def _refresh_decode_snapshot(self, plain: torch.Tensor):
        """``plain``: the merged (or frozen) weight in its natural row order."""
        src = getattr(self, "_fold_src", None)
        if src is None or not plain.is_cuda or plain.dtype != torch.bfloat16:
            self.weight_decode = None
            return
        scale = src[0].detach().float()
        if self._fold_zc:
            scale = scale + 1.0
        wd = (plain.float() * scale[None, :]).to(plain.dtype)
        if self._fold_glu:
            half = plain.shape[0] // 2
            if plain.shape[0] % 16 or half % 8:
                self.weight_decode = None
                return
            wd = wd.index_select(0, self.glu_row_order(half, plain.device))
        cur = getattr(self, "weight_decode", None)
        if cur is not None and cur.shape == wd.shape:
            cur.copy_(wd)                        # stable address for captured decode graphs
        else:
            self.weight_decode = wd

    def forward_merged_glu(self, x: torch.Tensor, act: str) -> torch.Tensor:
        """``act(x Wg^T) * (x Wu^T)`` over the merged snapshot; one kernel where the snapshot is
        interleaved, projection + GLU kernel otherwise."""
        if self._glu_rows() is not None and ops.native(x) and x.dtype == torch.bfloat16 and act in ("silu", "gelu_pytorch_tanh",
                                                                                                    "gelu_tanh"):
            from ..ops import cuda as _c
            return _c.gemm_glu(x, self.weight_merged, act)
        return ops.swiglu(self.forward_merged(x), act)

    @torch.no_grad()
    def merge(self):
        """Refresh the merged snapshot ``W + s·B·A`` (call after each update)."""
        a, b = self._stacks()
        if a is None:
            self.weight_merged = None
            self._glu_active = False
            self._refresh_decode_snapshot(self.weight)
            return
        new = ops.lora_merge(self.weight, a.detach(), b.detach())
        self._refresh_decode_snapshot(new)
        if self._glu_prepare():
            new = new.index_select(0, self._glu_perm)
        if self.weight_merged is not None and self.weight_merged.shape == new.shape:
            self.weight_merged.copy_(new)  # keep the address stable: captured decode graphs point at it
        else:
            self.weight_merged = new

    def merged_weight(self) -> torch.Tensor:
        a, b = self._stacks()
        return ops.lora_merge(self.weight, None if a is None else a.detach(),
                              None if b is None else b.detach())

    def adapter_params(self) -> list[nn.Parameter]:
        out = []
        for a, b in zip(self.lora_A, self.lora_B):
            out += [a, b]
        return out
