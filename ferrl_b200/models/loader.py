"""Checkpoint loading: HF-layout safetensors -> fused, (optionally) rank-local
weights, plus the policy identity digest.

Reference behaviour (``crates/ferrl/src/loader.rs``): ``LoaderOpts`` ``:51-97``;
dispatch on ``config.json``'s ``model_type`` into Qwen3 / Qwen3.5 / Gemma 4
``:987-1010`` (Llama is library-only); a frozen-policy digest over config and
weight bytes ``:269-307`` that checkpoints bind to.  Rank-local streaming reads
only the bytes of this rank's shard (``sharded_safetensors.rs:644-750``); here
that is done by the native range reader (``ferrl_b200.native.SafetensorsFile``:
threaded positional reads into pinned host memory); ``safetensors`` slicing is the
fallback when the helper library cannot be built.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..parallel.tp import TensorParallelPlan
from .dense import DenseGradModel, DenseSpec
from .lora import BaseQuantization, DenseLoraTargets, LoraSpec


@dataclass
class LoaderOpts:
    dtype: torch.dtype = torch.float32
    device: str = "cpu"
    lora: Optional[LoraSpec] = field(default_factory=LoraSpec)
    quantization: BaseQuantization = BaseQuantization.NONE
    remat: bool = False
    tp: Optional[tuple[int, int]] = None  # (rank, world)
    ep: Optional[tuple[int, int]] = None  # (rank, world): expert parallelism, sparse-MoE families only
    full_ft: bool = False
    adapter_seed: int = 0
    max_position_embeddings: Optional[int] = None
    gdn_targets: str = ""     # hybrid families: adapted GatedDeltaNet projections, letters of q z b a o (see qwen35.py)


@dataclass(frozen=True)
class PolicyLoadIdentity:
    """What a checkpoint is bound to: the checkpoint's bytes and the recipe the policy executes under (adapter rank
    and alpha, base and adapter dtypes, base quantisation, activation checkpointing, full fine-tuning, the
    tensor- and expert-parallel world sizes), but neither the rank inside such a group nor anything that only
    positions a random stream (reference: ``checkpoint_policy_digest``, crates/ferrl/src/loader.rs:269-307)."""
    model_type: str
    config_sha256: str
    weights_sha256: str
    recipe: str = ""

    def digest(self) -> str:
        h = hashlib.sha256(b"ferrl-b200/policy-identity/v2\0")
        for part in (self.model_type, self.config_sha256, self.weights_sha256, self.recipe):
            h.update(part.encode() + b"\0")
        return h.hexdigest()


def execution_recipe(opts: "LoaderOpts") -> str:
    """Canonical JSON of the options that change what the loaded policy computes."""
    import struct
    lora = None if (opts.lora is None or opts.full_ft) else opts.lora
    return json.dumps({
        "lora_rank": lora.rank if lora else 0,
        "lora_alpha_bits": struct.unpack("<Q", struct.pack("<d", float(lora.alpha)))[0] if lora else 0,
        "lora_targets": (lora.targets.canonical() + ("|gdn:" + opts.gdn_targets if opts.gdn_targets else ""))
        if lora and getattr(lora, "targets", None) is not None else "",
        "base_dtype": str(opts.dtype).replace("torch.", ""),
        "adapter_dtype": "float32",
        "base_quantization": BaseQuantization(opts.quantization).value,
        "activation_checkpointing": bool(opts.remat),
        "full_fine_tuning": bool(opts.full_ft),
        "tensor_parallel_world_size": opts.tp[1] if opts.tp is not None else 1,
        "expert_parallel_world_size": opts.ep[1] if opts.ep is not None else 1,
    }, sort_keys=True, separators=(",", ":"))


class _SafeOpenFile:
    """The ``safetensors`` library behind the same three calls as the native reader."""

    def __init__(self, handle):
        self.h = handle

    def keys(self):
        return list(self.h.keys())

    def get(self, name):
        return self.h.get_tensor(name)

    def rows(self, name, start, n):
        return self.h.get_slice(name)[start:start + n]

    def cols(self, name, start, n):
        return self.h.get_slice(name)[:, start:start + n]


class TensorSource:
    """Name -> tensor access over one or many safetensors files, with row/column
    range reads so a TP rank never materialises a full matrix."""

    def __init__(self, model_dir: str, native: bool = True):
        self.dir = model_dir
        idx = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self.weight_map = json.load(f)["weight_map"]
            self.files = sorted(set(self.weight_map.values()))
        else:
            self.files = ["model.safetensors"]
            self.weight_map = None
        self._open = {f: self._open_file(os.path.join(model_dir, f), native) for f in self.files}
        if self.weight_map is None:
            self.weight_map = {k: "model.safetensors" for k in self._open["model.safetensors"].keys()}

    @staticmethod
    def _open_file(path: str, native: bool):
        if native:
            try:
                from ..native import SafetensorsFile
                return SafetensorsFile(path)
            except (OSError, RuntimeError):   # helper library missing and no compiler: library fallback
                pass
        from safetensors import safe_open
        return _SafeOpenFile(safe_open(path, framework="pt"))

    def names(self):
        return list(self.weight_map.keys())

    def has(self, name: str) -> bool:
        return name in self.weight_map

    def get(self, name: str) -> torch.Tensor:
        return self._open[self.weight_map[name]].get(name)

    def rows(self, name: str, start: int, n: int) -> torch.Tensor:
        return self._open[self.weight_map[name]].rows(name, start, n)

    def cols(self, name: str, start: int, n: int) -> torch.Tensor:
        return self._open[self.weight_map[name]].cols(name, start, n)

    def files_sha256(self) -> str:
        h = hashlib.sha256()
        for f in self.files:
            with open(os.path.join(self.dir, f), "rb") as fh:
                while True:
                    chunk = fh.read(1 << 20)
                    if not chunk:
                        break
                    h.update(chunk)
        return h.hexdigest()


def _strip_prefix(src: TensorSource) -> str:
    for p in ("model.language_model.", "model.", "language_model.model."):
        if src.has(p + "embed_tokens.weight"):
            return p
    raise ValueError("cannot find embed_tokens.weight in the checkpoint")


@torch.no_grad()
def load_dense_weights(model: DenseGradModel, src: TensorSource) -> None:
    """HF names -> fused layout; TP ranks read only their rows/columns."""
    spec, tp = model.spec, model.tp
    p = _strip_prefix(src)
    D = spec.head_dim
    to = lambda t: t.to(model.dtype)  # noqa: E731
    model.embed.copy_(to(src.get(p + "embed_tokens.weight")))
    model.final_norm.copy_(to(src.get(p + "norm.weight")))
    if model.lm_head is not None:
        model.lm_head.copy_(to(src.get("lm_head.weight")))
    w = tp.world if tp else 1
    r = tp.rank if tp else 0
    for i, layer in enumerate(model.layers):
        b = f"{p}layers.{i}."

        def colshard(name, total):
            per = total // w
            return src.rows(b + name, r * per, per) if w > 1 else src.get(b + name)

        def rowshard(name, total):
            per = total // w
            return src.cols(b + name, r * per, per) if w > 1 else src.get(b + name)

        qkv = torch.cat([colshard("self_attn.q_proj.weight", spec.num_attention_heads * D),
                         colshard("self_attn.k_proj.weight", spec.num_key_value_heads * D),
                         colshard("self_attn.v_proj.weight", spec.num_key_value_heads * D)], 0)
        layer.qkv.set_weight(to(qkv))
        layer.o.set_weight(to(rowshard("self_attn.o_proj.weight", spec.num_attention_heads * D)))
        gu = torch.cat([colshard("mlp.gate_proj.weight", spec.intermediate_size),
                        colshard("mlp.up_proj.weight", spec.intermediate_size)], 0)
        layer.gate_up.set_weight(to(gu))
        layer.down.set_weight(to(rowshard("mlp.down_proj.weight", spec.intermediate_size)))
        layer.input_norm.copy_(to(src.get(b + "input_layernorm.weight")))
        layer.post_norm.copy_(to(src.get(b + "post_attention_layernorm.weight")))
        if spec.qk_norm:
            layer.q_norm.copy_(to(src.get(b + "self_attn.q_norm.weight")))
            layer.k_norm.copy_(to(src.get(b + "self_attn.k_norm.weight")))
    model.refresh_head()


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def _identity(model_dir: str, cfg: dict, src: TensorSource, opts: Optional["LoaderOpts"] = None) -> PolicyLoadIdentity:
    with open(os.path.join(model_dir, "config.json"), "rb") as f:
        csha = hashlib.sha256(f.read()).hexdigest()
    return PolicyLoadIdentity(str(cfg.get("model_type")), csha, src.files_sha256(),
                              execution_recipe(opts) if opts is not None else "")


def load_dense(model_dir: str, spec_fn: Callable[[dict], DenseSpec], opts: LoaderOpts):
    cfg = read_config(model_dir)
    spec = spec_fn(cfg)
    if opts.max_position_embeddings:
        spec.max_position_embeddings = opts.max_position_embeddings
    tp = None
    if opts.tp is not None:
        tp = TensorParallelPlan.new(opts.tp[0], opts.tp[1], spec.num_attention_heads,
                                    spec.num_key_value_heads, spec.intermediate_size)
    model = DenseGradModel(spec, None if opts.full_ft else opts.lora, dtype=opts.dtype, device=opts.device,
                           tp=tp, quant=opts.quantization, remat=opts.remat, full_ft=opts.full_ft)
    src = TensorSource(model_dir)
    load_dense_weights(model, src)
    g = torch.Generator().manual_seed(opts.adapter_seed)
    for l in model.layers:
        for pr in l.projections():
            pr.init_adapters(g)
    return model, _identity(model_dir, cfg, src, opts)


def load_auto_policy(model_dir: str, opts: Optional[LoaderOpts] = None):
    """Build the right model family from ``config.json`` and return
    ``(model, PolicyLoadIdentity)``.  ``model_type`` dispatch: ``qwen3`` ->
    dense Qwen3, ``qwen3_5``/``qwen3_5_text``/``qwen3_5_moe`` -> hybrid,
    ``gemma4``/``gemma4_text`` -> Gemma.  Llama must be loaded explicitly with
    ``load_llama`` (library API only)."""
    opts = opts or LoaderOpts()
    cfg = read_config(model_dir)
    mt = cfg.get("model_type")
    if mt == "qwen3":
        from .qwen3 import qwen3_spec
        return load_dense(model_dir, qwen3_spec, opts)
    if mt in ("qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text"):
        from .qwen35 import load_qwen35
        return load_qwen35(model_dir, opts)
    if mt in ("gemma4", "gemma4_text", "gemma4_uni"):
        from .gemma4 import load_gemma4
        return load_gemma4(model_dir, opts)
    raise ValueError(f"unsupported model_type {mt!r} (supported: qwen3, qwen3_5[_moe], gemma4)")


def load_llama(model_dir: str, opts: Optional[LoaderOpts] = None):
    from .llama import llama_spec
    return load_dense(model_dir, llama_spec, opts or LoaderOpts())
