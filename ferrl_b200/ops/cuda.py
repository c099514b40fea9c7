"""CUDA side of ``ferrl_b200.ops``: loads the in-tree native library and wraps
each sm_100a kernel as an autograd-aware function.

bf16 is the production dtype: the tcgen05 GEMM, flash attention and decode
attention accept bf16 only.  float32 CUDA tensors (a debugging configuration)
run the eager restatement for those three ops and the native kernels for the
rest.  A missing library raises ``ExtensionMissing`` - nothing falls back
silently.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from . import eager

_LIB = None
_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")


def lib():
    global _LIB
    if _LIB is None:
        from . import ExtensionMissing
        if not os.path.exists(_SO):
            raise ExtensionMissing(f"native library {_SO} is not built; run `python -m ferrl_b200._build`")
        try:
            torch.ops.load_library(_SO)
        except OSError as e:
            raise ExtensionMissing(f"cannot load {_SO}: {e}") from e
        _LIB = torch.ops.ferrl_b200
    return _LIB


def launches() -> int:
    return int(lib().launches())


def kernel_status() -> int:
    return int(lib().kernel_status())


def _bf16(t):
    return t is not None and t.dtype == torch.bfloat16


# ----------------------------------------------------------------- GEMM
def gemm(a, b, a2=None, b2=None, residual=None, out_f32=False, force_bn=0, force_split=0, two_cta=0, debug=None,
         cluster_k=0, stream_k=0, static_b=False):
    """``a [M,K] @ b[N,K]^T (+ a2 @ b2^T) (+ residual)`` on the tcgen05 kernel.
    Tile width and k-split are planned from the shape unless forced; ``two_cta`` (128 or 256)
    selects the two-SM kernel with 256 x ``two_cta`` tiles; ``cluster_k`` (with ``force_bn``) the
    cluster split-k kernel (``-1`` keeps the planner away from it); ``stream_k`` 1 forces and -1
    forbids the stream-k kernel for decode shapes (0: planner decides).  ``static_b``: ``b`` is a
    weight that no kernel earlier in the stream writes; a decode-shaped call (M <= 256) is then
    launched as a programmatic dependent and streams its first weight tiles while the previous
    kernel is still running."""
    return lib().gemm(a, b, a2, b2, residual, out_f32, force_bn, force_split, two_cta, debug, cluster_k, stream_k,
                      bool(static_b))


def gemm_glu(x, w_interleaved, act="silu"):
    """``act(x Wg^T) * (x Wu^T)`` with ``w_interleaved`` ``[2F, K]`` holding gate and up rows in groups of
    16 (8 gate, 8 up): the GLU runs in the GEMM epilogue (``[..., F]`` out, no ``[..., 2F]`` round trip)."""
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = lib().gemm_glu(x2, w_interleaved, _ACT[act], True)
    return y.view(*x.shape[:-1], w_interleaved.shape[0] // 2)


def gemm_norm(x, w, residual=None, ss_in=None, eps=1e-6, glu_act=None, want_ss=False):
    """Decode-chain projection with an RMSNorm folded around it: with ``ss_in`` ``[parts, M]`` (partial row
    sums of squares of ``x``) the result rows are scaled by ``rsqrt(sum / K + eps)`` in the epilogue (the
    norm weight must already be folded into ``w``'s columns); ``want_ss`` also returns the partial row sums
    of squares of the stored output for the next projection; ``glu_act`` runs the GLU in the epilogue
    (``w`` interleaved as for ``gemm_glu``).  ``x`` ``[M, K]``; returns ``(y, ss_or_None)``."""
    y, ss = lib().gemm_norm(x, w, residual, ss_in, float(eps), -1 if glu_act is None else _ACT[glu_act], bool(want_ss), True)
    return y, (ss if want_ss else None)


def row_sumsq(x):
    """``[1, M]`` float32 sums of squares of the bf16 rows of ``x`` ``[M, H]``."""
    return lib().row_sumsq(x)


def _pad8(t, dim):
    n = t.shape[dim]
    if n % 8 == 0:
        return t
    pad = [0, 0] * t.dim()
    pad[2 * (t.dim() - 1 - dim) + 1] = 8 - n % 8
    return torch.nn.functional.pad(t, pad)


def _lora_grad(u, x):
    """``uᵀ x`` in fp32 for ``u`` ``[M, R]`` (R a multiple of 8, <= 128) and ``x`` ``[M, C]`` bf16."""
    if u.shape[1] > 128 or x.shape[1] % 8 or x.stride(0) % 8 or u.stride(0) % 8:
        return torch.matmul(u.t().float(), x.float())
    return lib().lora_grad(u, x)


class _LoraLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, wt, a_stack, b_stack, residual=None):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        t = a16 = b16 = None
        if a_stack is not None:
            a16 = _pad8(a_stack.detach().to(torch.bfloat16), 0).contiguous()   # [R, K]
            b16 = _pad8(b_stack.detach().to(torch.bfloat16), 1).contiguous()   # [N, R]
            t = gemm(x2, a16)                                                  # [M, R]
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, w.shape[0])
            if res2.stride(-1) != 1:
                res2 = res2.contiguous()
        y = gemm(x2, w, t, b16, res2, static_b=a_stack is None)   # no adapter slab: a frozen (or merged) weight
        ctx.save_for_backward(x2, w, wt, a_stack, b_stack, t, a16, b16)
        ctx.x_shape = x.shape
        ctx.x_grad = x.requires_grad
        ctx.res_grad = residual is not None and residual.requires_grad
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, wt, a_stack, b_stack, t, a16, b16 = ctx.saved_tensors
        N = w.shape[0]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = da = db = None
        u = None
        if a_stack is not None:
            u = gemm(dy2, b16.t().contiguous())                                # [M, R] = dy @ B
        if ctx.x_grad:
            wt_ = wt if wt is not None else w.t().contiguous()
            if u is not None:
                dx = gemm(dy2, wt_, u, a16.t().contiguous())
            else:
                dx = gemm(dy2, wt_)
            dx = dx.view(ctx.x_shape)
        if a_stack is not None:
            R = a_stack.shape[0]
            # adapter gradients: tall-skinny reductions over the token dimension
            # adapter gradients: reductions over the token dimension (csrc/kernels/lora_grad.cu)
            da = _lora_grad(u, x2)[:R] if a_stack.requires_grad else None
            db = _lora_grad(t, dy2)[:R].t().contiguous() if b_stack.requires_grad else None
        return dx, None, None, da, db, (dy if getattr(ctx, "res_grad", False) else None)


class _LoraLinearReduce(torch.autograd.Function):
    """Row-parallel projection whose tensor-parallel sum happens inside the GEMM kernel.
    Backward is the local one: the cotangent of an all-reduced value is already replicated."""

    @staticmethod
    def forward(ctx, x, w, wt, a_stack, b_stack, residual, reducer):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        t = a16 = b16 = None
        if a_stack is not None:
            a16 = _pad8(a_stack.detach().to(torch.bfloat16), 0).contiguous()
            b16 = _pad8(b_stack.detach().to(torch.bfloat16), 1).contiguous()
            t = gemm(x2, a16)
        res2 = None
        if residual is not None:
            res2 = residual.reshape(-1, w.shape[0])
            if not res2.is_contiguous():
                res2 = res2.contiguous()
        y = reducer(x2, w, t, b16, res2)
        ctx.save_for_backward(x2, w, wt, a_stack, b_stack, t, a16, b16)
        ctx.x_shape = x.shape
        ctx.x_grad = x.requires_grad
        ctx.res_grad = residual is not None and residual.requires_grad
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        dx, _, _, da, db, dres = _LoraLinear.backward(ctx, dy)
        return dx, None, None, da, db, dres, None


class _LoraLinearReduceScatter(torch.autograd.Function):
    """Row-parallel projection whose tensor-parallel sum is reduce-scattered over the token rows inside the GEMM
    kernel: the result is this rank's ``rows / world`` rows.  Backward all-gathers the row shards of the cotangent
    (``gather``: shard -> all rows) and then runs the local backward of the projection."""

    @staticmethod
    def forward(ctx, x, w, wt, a_stack, b_stack, reducer, gather):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        t = a16 = b16 = None
        if a_stack is not None:
            a16 = _pad8(a_stack.detach().to(torch.bfloat16), 0).contiguous()
            b16 = _pad8(b_stack.detach().to(torch.bfloat16), 1).contiguous()
            t = gemm(x2, a16)
        y = reducer.reduce_scatter(x2, w, t, b16)
        ctx.save_for_backward(x2, w, wt, a_stack, b_stack, t, a16, b16)
        ctx.x_shape = x.shape
        ctx.x_grad = x.requires_grad
        ctx.res_grad = False
        ctx.gather = gather
        return y

    @staticmethod
    def backward(ctx, dy):
        dx, _, _, da, db, _ = _LoraLinear.backward(ctx, ctx.gather(dy.contiguous()))
        return dx, None, None, da, db, None, None


class _GatherLoraLinear(torch.autograd.Function):
    """Column-parallel projection of an all-gathered row shard: ``y = gather(xs) Wᵀ + (gather(xs) Aᵀ) Bᵀ``.
    Backward: the input gradient of rank r is ``dy_r W_r + (dy_r B_r) A``, and the shard of ``xs`` wants the sum of
    those over the ranks for its own rows: one fused GEMM -> reduce-scatter launch (the cotangent path of the
    reference's column-parallel layers sums full activations, ``crates/ferrl/src/gemma4.rs:2136-2169``)."""

    @staticmethod
    def forward(ctx, xs, w, wt, a_stack, b_stack, gather, scatter_sum, reducer):
        xs2 = xs.reshape(-1, xs.shape[-1]).contiguous()
        t = a16 = b16 = None
        if a_stack is not None:
            a16 = _pad8(a_stack.detach().to(torch.bfloat16), 0).contiguous()
            b16 = _pad8(b_stack.detach().to(torch.bfloat16), 1).contiguous()
        if reducer is not None and reducer.fits_gather(xs2.shape[0] * reducer.heap.world, xs2.shape[1]):
            # one launch gathers and projects; the rank-r factor of the adapter path is gathered from its row shards
            if a_stack is not None:
                t = gather(gemm(xs2, a16))
            y, x2 = reducer.gather_gemm(xs2, w, t, b16)
            if a_stack is not None and ctx.needs_input_grad[3]:
                x2 = x2.clone()             # the buffer is reused two calls later; the adapter gradient wants these rows
        else:
            x2 = gather(xs2)
            if a_stack is not None:
                t = gemm(x2, a16)
            y = gemm(x2, w, t, b16, None, static_b=a_stack is None)
        ctx.save_for_backward(x2, w, wt, a_stack, b_stack, t, a16, b16)
        ctx.x_grad = xs.requires_grad
        ctx.scatter_sum, ctx.reducer = scatter_sum, reducer
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w, wt, a_stack, b_stack, t, a16, b16 = ctx.saved_tensors
        dy2 = dy.reshape(-1, w.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dxs = da = db = None
        u = gemm(dy2, b16.t().contiguous()) if a_stack is not None else None
        if ctx.x_grad:
            wt_ = wt if wt is not None else w.t().contiguous()
            a16t = a16.t().contiguous() if u is not None else None
            red = ctx.reducer
            if red is not None and red.fits_scatter(dy2.shape[0], wt_.shape[0]):
                dxs = red.reduce_scatter(dy2, wt_, u, a16t)
            else:
                dxs = ctx.scatter_sum(gemm(dy2, wt_, u, a16t))
        if a_stack is not None:
            R = a_stack.shape[0]
            da = _lora_grad(u, x2)[:R] if a_stack.requires_grad else None
            db = _lora_grad(t, dy2)[:R].t().contiguous() if b_stack.requires_grad else None
        return dxs, None, None, da, db, None, None, None


def gather_lora_linear(xs, w, a_stack, b_stack, wt, gather, scatter_sum, reducer):
    """``lora_linear(all_gather_rows(xs))`` for a ``[rows / world, in]`` shard, with the reduce-scatter of the input
    gradient fused into its GEMM; ``None`` when the operands are not the bf16 frozen-weight case."""
    if not (_bf16(xs) and _bf16(w)) or w.requires_grad or xs.shape[-1] % 8 or xs.dim() != 2:
        return None
    return _GatherLoraLinear.apply(xs, w, wt, a_stack, b_stack, gather, scatter_sum, reducer)


def lora_linear_reduce_scatter(x, w, a_stack, b_stack, wt, reducer, gather):
    """This rank's rows of ``sum_r (x_r W_rᵀ + (x_r A_rᵀ) Bᵀ)``, ``[rows / world, out]``, in one kernel per rank;
    ``None`` when the shapes do not fit (the caller then projects and reduce-scatters separately)."""
    if not (_bf16(x) and _bf16(w)) or w.requires_grad or x.shape[-1] % 8:
        return None
    rows = x.numel() // x.shape[-1]
    if not reducer.fits_scatter(rows, w.shape[0]):
        return None
    return _LoraLinearReduceScatter.apply(x, w, wt, a_stack, b_stack, reducer, gather)


def lora_linear_reduce(x, w, a_stack, b_stack, wt, reducer, residual=None):
    """``all_reduce(x Wᵀ + (x Aᵀ) Bᵀ) (+ residual)`` in one kernel per rank; ``None`` when the
    shapes do not fit the reducer's symmetric buffers (the caller then reduces separately)."""
    if not (_bf16(x) and _bf16(w)) or w.requires_grad or x.shape[-1] % 8:
        return None
    rows = x.numel() // x.shape[-1]
    if not reducer.fits(rows, w.shape[0]):
        return None
    return _LoraLinearReduce.apply(x, w, wt, a_stack, b_stack, residual, reducer)


def lora_linear(x, w, a_stack, b_stack, wt=None, bias=None, residual=None):
    """``x Wᵀ + (x Aᵀ) Bᵀ (+ residual)``; the residual add happens in the GEMM epilogue."""
    if not (_bf16(x) and _bf16(w)) or bias is not None or w.requires_grad or x.shape[-1] % 8:
        y = eager.lora_linear(x, w, a_stack, b_stack, bias)
        return y if residual is None else residual + y
    if residual is not None and residual.dtype != torch.bfloat16:
        return residual + _LoraLinear.apply(x, w, wt, a_stack, b_stack)
    return _LoraLinear.apply(x, w, wt, a_stack, b_stack, residual)


def lora_merge(w, a_stack, b_stack):
    if a_stack is None:
        return w
    return lib().lora_merge(w.contiguous(), a_stack.float().contiguous(), b_stack.float().contiguous())


# ----------------------------------------------------------------- norms
class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, zc):
        xc = x.contiguous()
        y, _ = lib().rmsnorm(xc, None, w, None, eps, zc)
        ctx.save_for_backward(xc, w)
        ctx.eps, ctx.zc = eps, zc
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        return lib().rmsnorm_bwd(x, w, dy.contiguous(), ctx.eps, ctx.zc), None, None, None


def rmsnorm(x, weight, eps, zero_centered=False):
    if weight is not None and (weight.requires_grad or weight.dtype != x.dtype):
        return eager.rmsnorm(x, weight, eps, zero_centered)
    return _RmsNorm.apply(x, weight, eps, zero_centered)


class _AddRmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, eps, zc):
        y, h = lib().rmsnorm(x.contiguous(), res.contiguous(), w, None, eps, zc)
        ctx.save_for_backward(h, w)
        ctx.eps, ctx.zc = eps, zc
        return y, h

    @staticmethod
    def backward(ctx, dy, dh):
        h, w = ctx.saved_tensors
        g = lib().rmsnorm_bwd(h, w, dy.contiguous(), ctx.eps, ctx.zc)
        if dh is not None:
            g = g + dh
        return g, g, None, None, None


def add_rmsnorm(x, residual, weight, eps, zero_centered=False):
    if weight is not None and (weight.requires_grad or weight.dtype != x.dtype):
        return eager.add_rmsnorm(x, residual, weight, eps, zero_centered)
    return _AddRmsNorm.apply(x, residual, weight, eps, zero_centered)


class _RmsNormGated(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, w, eps):
        y, _ = lib().rmsnorm(x, None, w, gate, eps, False)
        ctx.save_for_backward(x, gate, w)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gate, w = ctx.saved_tensors
        dx, dg = lib().rmsnorm_gated_bwd(x, gate, w, dy.contiguous(), ctx.eps)
        return dx, dg, None, None


def rmsnorm_gated(x, gate, weight, eps):
    if weight.requires_grad or gate.dtype != x.dtype:
        return eager.rmsnorm_gated(x, gate, weight, eps)
    w = weight.to(x.dtype).contiguous()
    if torch.is_grad_enabled() and (x.requires_grad or gate.requires_grad):
        return _RmsNormGated.apply(x.contiguous(), gate.contiguous(), w, eps)
    y, _ = lib().rmsnorm(x.contiguous(), None, w, gate.contiguous(), eps, False)
    return y


class _QkNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, qw, kw, eps, cos, sin, pos, pos_div, zc):
        B, S, Hq, D = q.shape
        Hkv = k.shape[2]
        ts = (lambda t: t.stride(1) if S > 1 else t.stride(0))  # token stride (a size-1 dim has an arbitrary stride)
        q3 = q.reshape(B * S, Hq, D) if q.is_contiguous() else q.as_strided((B * S, Hq, D), (ts(q), D, 1), q.storage_offset())
        k3 = k.reshape(B * S, Hkv, D) if k.is_contiguous() else k.as_strided((B * S, Hkv, D), (ts(k), D, 1), k.storage_offset())
        qo, ko = lib().qk_norm_rope_fwd(q3, k3, qw, kw, cos, sin, pos, pos_div, eps, zc)
        ctx.save_for_backward(q3, k3, qw, kw, cos, sin, pos)
        ctx.meta = (B, S, Hq, Hkv, D, pos_div, eps, zc)
        return qo.view(B, S, Hq, D), ko.view(B, S, Hkv, D)

    @staticmethod
    def backward(ctx, dq, dk):
        q3, k3, qw, kw, cos, sin, pos = ctx.saved_tensors
        B, S, Hq, Hkv, D, pos_div, eps, zc = ctx.meta
        dqi = torch.empty(B * S, Hq, D, dtype=q3.dtype, device=q3.device)
        dki = torch.empty(B * S, Hkv, D, dtype=k3.dtype, device=k3.device)
        lib().qk_norm_rope_bwd(q3, k3, qw, kw, cos, sin, pos, pos_div, eps, zc, dq.contiguous().view(B * S, Hq, D),
                               dk.contiguous().view(B * S, Hkv, D), dqi, dki)
        return dqi.view(B, S, Hq, D), dki.view(B, S, Hkv, D), None, None, None, None, None, None, None, None


def _strided_ok(t):
    # [B,S,H,D] with packed heads and batch stride == S * token stride (so tokens form one strided 2-D matrix)
    B, S, H, D = t.shape
    return t.stride(3) == 1 and t.stride(2) == D and (B == 1 or S == 1 or t.stride(0) == S * t.stride(1))


def qk_norm_rope(q, k, q_w, k_w, eps, cos, sin, positions, zero_centered=False):
    if (q_w is not None and q_w.requires_grad) or not (_strided_ok(q) and _strided_ok(k)):
        return eager.qk_norm_rope(q, k, q_w, k_w, eps, cos, sin, positions, zero_centered)
    B, S = q.shape[:2]
    if positions.dim() == 1:          # [S], shared by every batch row -> position of token t is pos[t % S]
        pos = positions.repeat(B) if B > 1 else positions
    else:
        pos = positions.reshape(-1)
    pos = pos.contiguous()
    if pos.dtype not in (torch.int64, torch.int32):
        pos = pos.long()
    qw = None if q_w is None else q_w.to(q.dtype)
    kw = None if k_w is None else k_w.to(k.dtype)
    return _QkNormRope.apply(q, k, qw, kw, eps, cos.float(), sin.float(), pos, 1, zero_centered)


def qk_norm_rope_append(q, k, v, q_w, k_w, eps, cos, sin, positions, k_cache, v_cache, kv_len, table=None,
                        zero_centered=False):
    """Decode form of ``qk_norm_rope`` fused with the KV-cache write: ``q, k, v`` ``[B, H, D]`` (one
    token per row, views into the fused projection are fine), the rotated keys and the values go to
    cache row ``kv_len[b]`` (dense ``[B, Smax, Hkv, D]`` caches, or paged pools behind ``table``).
    Returns the rotated ``q`` ``[B, Hq, D]``, or ``None`` outside the kernel's domain."""
    D = q.shape[-1]
    if not (_bf16(q) and _bf16(k) and _bf16(v) and _bf16(k_cache)) or D not in (128, 256) or kv_len.dtype != torch.int32:
        return None
    if (q_w is not None and q_w.dtype != q.dtype) or (k_w is not None and k_w.dtype != k.dtype):
        return None
    for t in (q, k, v):
        if t.dim() != 3 or t.stride(2) != 1 or t.stride(1) != D or t.stride(0) % 8:
            return None
    pos = positions.reshape(-1)
    if pos.dtype not in (torch.int64, torch.int32):
        pos = pos.long()
    return lib().qk_norm_rope_append(q, k, v, q_w, k_w, cos, sin, pos.contiguous(), float(eps), bool(zero_centered),
                                     k_cache, v_cache, kv_len, table)


# ------------------------------------------------------------- attention
class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, window, q_offset, variant=0):
        o, lse = lib().flash_fwd(q, k, v, scale, causal, window, q_offset, variant)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (scale, causal, window, q_offset, 1 if variant == 1 else 0)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = lib().flash_bwd(q, k, v, o, lse, do.contiguous(), *ctx.meta)
        return dq, dk, dv, None, None, None, None, None


def _packed(t):
    return t if (t.stride(3) == 1 and t.stride(2) == t.shape[3]) else t.contiguous()


def attention(q, k, v, *, scale, causal=True, window=0, q_offset=0, kv_len=None, variant=0):
    """Flash attention.  Causal self-attention with head_dim 128 runs the tcgen05 forward
    (``csrc/kernels/flash_tc.cu``); ``variant=1`` forces the warp-level kernel everywhere."""
    if not _bf16(q) or q.shape[-1] not in (64, 128, 256) or kv_len is not None:
        return eager.attention(q, k, v, scale=scale, causal=causal, window=window, q_offset=q_offset, kv_len=kv_len)
    return _Flash.apply(_packed(q), _packed(k), _packed(v), float(scale), bool(causal), int(window or 0), int(q_offset),
                        int(variant))


_PREFIX_SHAPES = {(128, 4, 8), (128, 4, 4), (128, 8, 4), (128, 8, 2), (128, 2, 8), (64, 4, 8), (64, 4, 4), (128, 2, 16)}


def prefix_attention_supported(head_dim: int, q_per_kv: int, group: int) -> bool:
    """Whether ``decode_attention(..., prefix_len=...)`` has a kernel for this (head_dim, query heads
    per KV head, rows per group) triple."""
    return (head_dim, q_per_kv, group) in _PREFIX_SHAPES


def decode_attention(q, k_cache, v_cache, kv_len, *, scale, window=0, n_splits=0, variant=0, block_table=None,
                     prefix_len=None, group=1, prefix_splits=0):
    """``variant`` 0 picks the tensor-core pipelined kernel where it applies, 2 the scalar pipelined
    one, 1 the register-resident one (both kept for uncovered head shapes and as cross-checks).
    ``prefix_len`` ``[B / group]`` int32 (paged cache only): the first ``prefix_len[b // group]`` keys of
    row ``b`` are shared by the ``group`` rows of its group (same pages in ``block_table``); they are
    streamed once per group by a kernel that applies them to all the group's queries, each row's
    remaining keys by the per-row kernel, and a combine kernel merges the two partial results."""
    if not _bf16(q) or q.shape[-1] % 8 or q.shape[-1] > 256:
        return eager.decode_attention(q, k_cache, v_cache, kv_len, scale=scale, window=window)
    if block_table is not None and prefix_len is not None and not window:
        B = q.shape[0]
        if int(prefix_splits):
            ps = int(prefix_splits)
        elif (q.shape[-1], q.shape[1] // k_cache.shape[2], group) == (128, 4, 8):
            ps = 1          # the whole-group kernel: prefix and private keys in one launch
        else:
            ps = max(1, min(4, 296 // max(1, (B // group) * k_cache.shape[2])))   # about two prefix CTAs per SM
        return lib().decode_attn(q.contiguous(), k_cache, v_cache, kv_len.to(torch.int32), float(scale), 0, 1, block_table,
                                 k_cache.shape[1], 0, prefix_len, int(group), ps)
    if block_table is not None:
        # paged pool [n_pages, page, Hkv, D]; row b's token t is in page block_table[b, t // page]
        return lib().decode_attn(q.contiguous(), k_cache, v_cache, kv_len.to(torch.int32), float(scale), int(window or 0),
                                 int(n_splits) or 1, block_table, k_cache.shape[1], int(variant))
    return lib().decode_attn(q.contiguous(), k_cache, v_cache, kv_len.to(torch.int32), float(scale), int(window or 0),
                             int(n_splits), None, 0, int(variant))


def kv_append_paged(k_pool, v_pool, k, v, kv_len, table):
    """Paged form of ``kv_append``: pools ``[n_pages, page, Hkv, D]``, ``table`` ``[B, max_pages]`` int32."""
    B = k.shape[0]
    lib().kv_append_paged(k.reshape(B, -1), v.reshape(B, -1) if v.is_contiguous() else v.as_strided(
        (B, v.shape[-2] * v.shape[-1]), (v.stride(0), 1), v.storage_offset()), k_pool, v_pool, kv_len, table)


def kv_append(k_cache, v_cache, k, v, kv_len):
    """Write one token's K/V per row at ``kv_len[b]`` (``k`` contiguous [B,Hkv,D], ``v`` may be a strided view)."""
    B = k.shape[0]
    lib().kv_append(k.reshape(B, -1), v.reshape(B, -1) if v.is_contiguous() else v.as_strided(
        (B, v.shape[-2] * v.shape[-1]), (v.stride(0), 1), v.storage_offset()), k_cache, v_cache, kv_len)


# ------------------------------------------------------------------ mlp
_ACT = {"silu": 0, "gelu_pytorch_tanh": 1, "gelu_tanh": 1}


class _Glu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, act):
        guc = gu.contiguous()
        ctx.save_for_backward(guc)
        ctx.act = act
        return lib().glu_fwd(guc, act)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        return lib().glu_bwd(gu, dout.contiguous(), ctx.act), None


def swiglu(gate_up, act="silu"):
    if act not in _ACT:
        return eager.swiglu(gate_up, act)
    return _Glu.apply(gate_up, _ACT[act])


# ------------------------------------------------------------------ GatedDeltaNet
class _GdnConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, left, act):
        ctx.save_for_backward(x, w, left)
        ctx.act = act
        return lib().gdn_conv_fwd(x, w, left, act)

    @staticmethod
    def backward(ctx, dy):
        x, w, left = ctx.saved_tensors
        return lib().gdn_conv_bwd(x, w, left, dy.contiguous(), ctx.act), None, None, None


def gdn_conv(x, w, left=None, activation=True):
    """Causal depthwise conv (+SiLU) over ``x`` ``[B, L, C]`` with frozen ``w`` ``[C, K]`` and
    left context ``[B, C, K-1]``; ``None`` outside the kernel's domain."""
    if not (_bf16(x) and _bf16(w)) or w.requires_grad or w.shape[-1] > 8 or x.dim() != 3:
        return None
    if x.stride(2) != 1 or x.stride(0) != x.shape[1] * x.stride(1):
        x = x.contiguous()
    if left is not None:
        left = left.to(torch.bfloat16).contiguous()
    return _GdnConv.apply(x, w.contiguous(), left, bool(activation))


def gdn_conv_step(x, w, state, activation=True):
    """One-token conv against ``state`` ``[B, C, K-1]`` (updated in place)."""
    return lib().gdn_conv_step(x, w.contiguous(), state, bool(activation))


def gdn_chunk_fwd(q, k, v, g, beta, S0=None, l2norm=True, eps=1e-6):
    """Chunked gated delta rule, forward only (no autograd): ``q,k`` ``[B,T,Hk,128]``, ``v``
    ``[B,T,Hv,128]`` bf16, ``g,beta`` ``[B,T,Hv]`` f32 -> ``(out [B,T,Hv,128] bf16, S [B,Hv,128,128] f32)``;
    ``None`` outside the kernel's domain."""
    if not (_bf16(q) and _bf16(k) and _bf16(v)) or q.shape[-1] != 128 or v.shape[-1] != 128:
        return None
    fix = lambda t: t if (t.stride(3) == 1 and t.stride(2) == t.shape[3]) else t.contiguous()  # noqa: E731
    return lib().gdn_chunk_fwd(fix(q), fix(k), fix(v), g.float().contiguous(), beta.float().contiguous(), S0,
                               bool(l2norm), float(eps))


class _GdnTc(torch.autograd.Function):
    """Tensor-core chunked gated delta rule with its hand-written backward (``csrc/kernels/gdn_tc.cu``)."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, S0):
        out, S1, *saved = lib().gdn_tc_fwd(q, k, v, g, beta, S0)
        if any(ctx.needs_input_grad):
            ctx.save_for_backward(q, k, v, beta, *saved)
        ctx.set_materialize_grads(False)
        return out, S1

    @staticmethod
    def backward(ctx, dO, dS1):
        q, k, v, beta, Gc, gl, Tm, Wn, Kd, Vn, Sin = ctx.saved_tensors
        dO = torch.zeros_like(v) if dO is None else dO.contiguous()
        dq, dk, dv, dbeta, dG, dS0 = lib().gdn_tc_bwd(q, k, v, beta, Gc, gl, Tm, Wn, Kd, Vn, Sin, dO,
                                                      None if dS1 is None else dS1.contiguous())
        B, T, Hv, D = dq.shape
        Hk = q.shape[2]
        if Hv != Hk:      # several value heads share one key head
            dq = dq.view(B, T, Hk, Hv // Hk, D).sum(3)
            dk = dk.view(B, T, Hk, Hv // Hk, D).sum(3)
        # dG is the gradient of the cumulative log decay inside each chunk: g_j reaches every G_i with i >= j
        dg = dG.view(B, T // 64, 64, Hv).flip(2).cumsum(2).flip(2).reshape(B, T, Hv)
        return dq, dk, dv, dg, dbeta, (dS0 if ctx.needs_input_grad[5] else None)


def gdn_chunk_tc(q, k, v, g, beta, S0=None, eps=1e-6):
    """Chunked gated delta rule on the tensor cores with autograd: ``q,k`` ``[B,T,Hk,128]`` (raw; they are
    L2-normalised here and q is scaled by 1/sqrt(128)), ``v`` ``[B,T,Hv,128]``, ``g,beta`` ``[B,T,Hv]``, ``S0``
    ``[B,Hv,128,128]`` f32 -> ``(out [B,T,Hv,128] in v's dtype, S [B,Hv,128,128] f32)``; ``None`` outside the
    kernels' domain (head dims other than 128)."""
    if q.shape[-1] != 128 or v.shape[-1] != 128 or v.shape[2] % q.shape[2]:
        return None
    T = q.shape[1]
    qf = eager.l2norm(q.float(), eps) * (128 ** -0.5)
    kf = eager.l2norm(k.float(), eps)
    vf, gf, bf = v.float(), g.float(), beta.float()
    pad = (-T) % 64
    if pad:
        # beta = 0 and g = 0 leave the state untouched on the padded tokens
        qf, kf, vf = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (qf, kf, vf))
        gf, bf = F.pad(gf, (0, 0, 0, pad)), F.pad(bf, (0, 0, 0, pad))
    out, S1 = _GdnTc.apply(qf.contiguous(), kf.contiguous(), vf.contiguous(), gf.contiguous(), bf.contiguous(),
                           None if S0 is None else S0.float().contiguous())
    return out[:, :T].to(v.dtype), S1


def gdn_decode_step(q, k, v, g, beta, S, l2norm=True, eps=1e-6):
    """Single-token gated delta rule; ``S`` ``[B,Hv,KD,VD]`` float32 is updated in place."""
    return lib().gdn_decode_step(q, k, v, g.contiguous(), beta.contiguous(), S, bool(l2norm), float(eps))


def gdn_decode_step_raw(q, k, v, a, b, A_log, dt_bias, S, l2norm=True, eps=1e-6):
    """The same step with the gates formed in the kernel from the projection's ``a`` and ``b`` columns
    (``g = -exp(A_log) softplus(a + dt_bias)``, ``beta = sigmoid(b)``): ten small launches fewer per layer."""
    return lib().gdn_decode_step_raw(q, k, v, a, b, A_log, dt_bias, S, bool(l2norm), float(eps))


# ------------------------------------------------------------------ MoE
class _MoeRoute(torch.autograd.Function):
    """fp32 softmax over the router logits, top-k and renormalisation in one kernel; the
    backward is the closed form of softmax -> gather -> normalise on the small [T, E] table."""

    @staticmethod
    def forward(ctx, logits, k, renorm):
        probs, scores, idx, counts = lib().moe_route(logits.contiguous(), k, renorm)
        ctx.save_for_backward(probs, scores, idx)
        ctx.renorm = renorm
        ctx.mark_non_differentiable(idx, counts)
        return scores, idx, counts, probs.detach()

    @staticmethod
    def backward(ctx, ds, _di, _dc, _dp):
        probs, scores, idx = ctx.saved_tensors
        li = idx.long()
        if ctx.renorm:
            top = probs.gather(1, li).sum(-1, keepdim=True)
            ds = (ds - (ds * scores).sum(-1, keepdim=True)) / top
        dp = torch.zeros_like(probs).scatter_(1, li, ds)
        return probs * (dp - (dp * probs).sum(-1, keepdim=True)), None, None


def moe_route(logits_f32, k, renorm=True):
    """``(scores [T,k] f32, idx [T,k] i32, counts [E] i32, probs [T,E] f32)``."""
    return _MoeRoute.apply(logits_f32, int(k), bool(renorm))


class _MoeExperts(torch.autograd.Function):
    """Routed frozen experts: plan -> gather -> grouped GEMM -> SwiGLU -> grouped GEMM -> combine,
    with no host synchronisation; gradients flow to the tokens and to the routing scores."""

    @staticmethod
    def forward(ctx, x, scores, idx, counts, gate_up, down, gate_up_t, down_t, act):
        L = lib()
        T, k = idx.shape
        row_of, token_of, tile_expert, _ = L.moe_plan(idx.contiguous(), counts)
        xs = L.moe_gather(x.contiguous(), token_of, None, row_of)
        # rows of unused tiles are never written and never read back (the combine reads routed rows only); the
        # zero fill of the outputs is kept for training, where the padded rows are saved for the backward pass
        train = any(ctx.needs_input_grad)
        o1 = None if train else torch.empty(xs.shape[0], gate_up.shape[1], dtype=xs.dtype, device=xs.device)
        gu = L.moe_grouped_gemm(xs, gate_up, tile_expert, o1)
        del xs
        h = L.glu_fwd(gu, act)
        o2 = None if train else torch.empty(h.shape[0], down.shape[1], dtype=h.dtype, device=h.device)
        ys = L.moe_grouped_gemm(h, down, tile_expert, o2)
        del h
        sc = scores.float().contiguous()
        out = L.moe_combine(ys, row_of, sc, T, k)
        ctx.save_for_backward(gu, ys, sc, row_of, token_of, tile_expert, gate_up, down, gate_up_t, down_t)
        ctx.act, ctx.k = act, k
        ctx.score_dtype = scores.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        L = lib()
        gu, ys, sc, row_of, token_of, tile_expert, gate_up, down, gate_up_t, down_t = ctx.saved_tensors
        dout = dout.contiguous()
        T = dout.shape[0]
        dsc = L.moe_pair_dot(dout, ys, row_of, ctx.k).to(ctx.score_dtype)
        dys = L.moe_gather(dout, token_of, sc.view(-1), row_of)
        if down_t is None:
            down_t = down.transpose(1, 2).contiguous()
        dh = L.moe_grouped_gemm(dys, down_t, tile_expert)
        del dys
        dgu = L.glu_bwd(gu, dh, ctx.act)
        del dh
        if gate_up_t is None:
            gate_up_t = gate_up.transpose(1, 2).contiguous()
        dxs = L.moe_grouped_gemm(dgu, gate_up_t, tile_expert)
        dx = L.moe_combine(dxs, row_of, None, T, ctx.k)
        return dx, dsc, None, None, None, None, None, None, None


def moe_experts(x, scores, idx, counts, gate_up, down, act="silu", gate_up_t=None, down_t=None):
    """``x`` ``[T,H]`` bf16; ``gate_up`` ``[E,2I,H]``, ``down`` ``[E,H,I]`` frozen bf16; optional
    resident transposes for the backward GEMMs.  ``None`` when the shapes are outside the kernels'
    domain (caller falls back to the eager plan)."""
    if not (_bf16(x) and _bf16(gate_up) and _bf16(down)) or act not in _ACT or gate_up.requires_grad or down.requires_grad:
        return None
    H, I = x.shape[-1], down.shape[-1]
    if H % 8 or I % 8 or not (gate_up.is_contiguous() and down.is_contiguous()):
        return None
    return _MoeExperts.apply(x, scores, idx, counts, gate_up, down, gate_up_t, down_t, _ACT[act])


def embedding(ids, table, scale=1.0):
    if table.requires_grad:
        return eager.embedding(ids, table, scale)
    return lib().embedding(ids, table, float(scale))


# -------------------------------------------------------------- logprob
LOGPROB_CHUNK_BYTES = 1 << 30


class _LogprobGather(torch.autograd.Function):
    """``log_softmax(softcap(h Wᵀ) / T)[target]`` with the row statistics taken in the head GEMM's epilogue
    (``csrc/gemm/tcgen05_gemm.cu``, ``lp_mode``): the forward allocates nothing of vocabulary width.  The
    backward recomputes the logits tile by tile and writes the softmax gradient straight from the epilogue,
    one bounded row chunk at a time, then multiplies by the weight again.  Reference: the chunked
    log-softmax gather of crates/ferrl/src/model.rs:523-559, which materialises ``[chunk, V]`` logits."""

    @staticmethod
    def forward(ctx, hidden, head_w, head_wt, targets, temperature, softcap):
        h = hidden.contiguous()
        t = targets.contiguous()
        lp, lse = lib().logprob_head_fwd(h, head_w, t, temperature, softcap)
        ctx.save_for_backward(h, head_w, head_wt, t, lse)
        ctx.meta = (temperature, softcap)
        return lp

    @staticmethod
    def backward(ctx, dlp):
        h, head_w, head_wt, t, lse = ctx.saved_tensors
        temperature, softcap = ctx.meta
        N, V = h.shape[0], head_w.shape[0]
        chunk = max(256, min(N, (LOGPROB_CHUNK_BYTES // (2 * V)) // 256 * 256)) if N else 1
        wt = head_wt if head_wt is not None else head_w.t().contiguous()
        dh = torch.empty_like(h)
        coef = (-dlp).contiguous().float()
        for s in range(0, N, chunk):
            dl = lib().logprob_head_dlogits(h[s:s + chunk], head_w, t[s:s + chunk], lse[s:s + chunk], coef[s:s + chunk],
                                            temperature, softcap, 0)
            dh[s:s + chunk] = gemm(dl, wt)
            del dl
        return dh, None, None, None, None, None


def logprob_gather(hidden, head_w, targets, temperature=1.0, softcap=0.0, head_wt=None):
    if not (_bf16(hidden) and _bf16(head_w)) or head_w.requires_grad or head_w.shape[0] % 8 or hidden.shape[-1] % 8:
        return eager.logprob_gather(hidden, head_w, targets, temperature, softcap)
    return _LogprobGather.apply(hidden, head_w, head_wt, targets.long(), float(temperature), float(softcap or 0.0))


# -------------------------------------------------------------- sampling
def _s64(x: int) -> int:
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


def sample_top_p(logits, base_seed, global_rows, draw, temperature, top_p, draw_dev=None):
    lg = logits if logits.stride(-1) == 1 else logits.contiguous()
    return lib().sample_rows(lg, global_rows.long().contiguous(), _s64(int(base_seed)), draw_dev, int(draw),
                             float(temperature), float(top_p) if top_p is not None else 0.0)


# ----------------------------------------------------------------- loss
class _GrpoLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp, logp_old, logp_ref, adv, mask, tis_w, eps_lo, eps_hi, beta, seq_level, loss_type,
                dapo_norm, scale):
        G, L = logp.shape
        want = logp.requires_grad
        row_sum, row_cnt, dl = lib().grpo_loss_rows(logp.contiguous(), logp_old.contiguous(),
                                                    None if logp_ref is None else logp_ref.contiguous(),
                                                    adv.reshape(-1).float().contiguous(), mask.contiguous(),
                                                    None if tis_w is None else tis_w.contiguous(), eps_lo, eps_hi,
                                                    beta, seq_level, want)
        if loss_type == "grpo":
            row_scale = 1.0 / (row_cnt.clamp(min=1.0) * G)
        elif loss_type == "dr_grpo":
            row_scale = torch.full_like(row_cnt, 1.0 / (G * L))
        else:
            norm = row_cnt.sum().clamp(min=1.0) if dapo_norm is None else torch.full((), max(dapo_norm, 1.0),
                                                                                    device=logp.device)
            row_scale = torch.ones_like(row_cnt) / norm
        row_scale = row_scale * scale
        loss = -(row_sum * row_scale).sum()
        if want:
            ctx.save_for_backward(dl, row_scale)
        return loss

    @staticmethod
    def backward(ctx, g):
        dl, row_scale = ctx.saved_tensors
        out = dl.clone()
        lib().grpo_scale_rows(out, (-g * row_scale).contiguous())
        return (out,) + (None,) * 12


def grpo_loss(logp, logp_old, logp_ref, advantages, mask, cfg, tis_w=None):
    from ..grpo import ImportanceSamplingLevel, LossType
    if logp.dtype != torch.float32:
        from ..grpo import grpo_loss_eager
        return grpo_loss_eager(logp, logp_old, logp_ref, advantages, mask, cfg, tis_w)
    return _GrpoLoss.apply(logp, logp_old.float(), None if logp_ref is None else logp_ref.float(), advantages,
                           mask.float(), None if tis_w is None else tis_w.float(), float(cfg.clip_eps_low),
                           float(cfg.clip_eps_high), float(cfg.beta),
                           ImportanceSamplingLevel(cfg.is_level) is ImportanceSamplingLevel.SEQUENCE,
                           LossType(cfg.loss_type).value, cfg.dapo_norm, float(cfg.scale))


# ---------------------------------------------------------------- adamw
def adamw_step(params, grads, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
               max_norm: float = 0.0, compute_norm: bool = False):
    """Multi-tensor AdamW. With ``compute_norm`` the kernel also derives the global
    gradient norm and clip factor on the device; returns the norm tensor."""
    if not params:
        return None
    if any(p.dtype != torch.float32 for p in params):
        return eager.adamw_step(params, grads, m, v, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                                weight_decay=weight_decay, step=step, grad_scale=grad_scale)
    return lib().adamw_step(list(params), [g.contiguous() for g in grads], list(m), list(v), lr, beta1, beta2, eps,
                            weight_decay, step, max_norm, grad_scale, compute_norm)
