"""HF checkpoint helpers: EOS resolution, EOS consensus, ChatML prompt shaping.

Reference ``crates/ferrl/src/hf.rs``: the checkpoint's ``eos_token_id`` (under
``text_config`` first) may be missing, a single id or a list (``:190-257``).
Selection modes: *checkpoint default* (needs exactly one declared id),
*explicit* (must be a member when several are declared), *disabled*.  The
selected id must be inside the model vocab and known to the tokenizer.  All
ranks must resolve the same id (``:267-305``); ``chatml`` ``:369-379``.
"""
from __future__ import annotations

import json
import os
from typing import Optional, Union

from .comm import Comm


class HfError(ValueError):
    pass


def _read_config(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, encoding="utf-8") as f:
            return json.load(f)
    except OSError as e:
        raise HfError(f"cannot read {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise HfError(f"{path} is not valid JSON: {e}") from e


def _preferred(cfg: dict, field: str):
    tc = cfg.get("text_config")
    if isinstance(tc, dict) and field in tc:
        return tc[field]
    return cfg.get(field)


def _token_id(raw) -> Optional[int]:
    if isinstance(raw, bool) or not isinstance(raw, int):
        return None
    return raw if 0 <= raw < 2 ** 32 else None


def model_vocab_size(cfg: dict) -> int:
    """The model's vocabulary bound (nested ``text_config`` first): a positive integer, or the checkpoint is refused
    (crates/ferrl/src/hf.rs ``vocab_size_from_json``)."""
    raw = _preferred(cfg, "vocab_size")
    if isinstance(raw, bool) or not isinstance(raw, int) or raw <= 0:
        raise HfError(f"config vocab_size {raw!r} must be a positive integer")
    return raw


def checkpoint_eos(model_dir: str) -> Union[None, int, list]:
    """``None`` (missing), one id, or the declared list."""
    raw = _preferred(_read_config(model_dir), "eos_token_id")
    if raw is None:
        return None
    if isinstance(raw, list):
        ids = [_token_id(x) for x in raw]
        if not ids or any(i is None for i in ids):
            raise HfError(f"eos_token_id list {raw!r} must hold unsigned integers")
        return ids[0] if len(ids) == 1 else ids
    i = _token_id(raw)
    if i is None:
        raise HfError(f"eos_token_id {raw!r} must be an unsigned integer or a list of them")
    return i


def resolve_eos(model_dir: str, selection: str, explicit: Optional[int], tokenizer) -> Optional[int]:
    """``selection`` is ``checkpoint`` | ``explicit`` | ``disabled``."""
    if selection == "disabled":
        return None
    declared = checkpoint_eos(model_dir)
    if selection == "checkpoint":
        if declared is None:
            raise HfError("checkpoint declares no eos_token_id; select one explicit id or disable EOS explicitly")
        if isinstance(declared, list):
            raise HfError(f"checkpoint declares multiple EOS ids {declared}; select one declared id explicitly "
                          "or disable EOS explicitly")
        chosen = declared
    elif selection == "explicit":
        if explicit is None:
            raise HfError("explicit EOS selection lost its token id")
        if isinstance(declared, list) and explicit not in declared:
            raise HfError(f"explicit EOS id {explicit} is not a member of the checkpoint's declared EOS ids {declared}")
        chosen = explicit
    else:
        raise HfError(f"unknown EOS selection {selection!r}")
    vocab = model_vocab_size(_read_config(model_dir))
    if chosen >= vocab:
        raise HfError(f"EOS id {chosen} is outside model vocab_size {vocab}")
    if tokenizer is not None and not tokenizer.contains_id(chosen):
        raise HfError(f"EOS id {chosen} is not present in the loaded tokenizer vocabulary")
    return chosen


def validate_resolved_eos_consensus(eos: Optional[int], comm: Comm) -> None:
    if comm.world_size <= 1:
        return
    blob = b"\x00" if eos is None else b"\x01" + int(eos).to_bytes(4, "little")
    try:
        comm.require_consensus(blob, "resolved EOS token")
    except Exception as e:  # noqa: BLE001
        raise HfError(f"ranks resolved different EOS token semantics: {e}") from e


def chatml(system: Optional[str], user: str) -> str:
    out = ""
    if system is not None:
        out += f"<|im_start|>system\n{system}<|im_end|>\n"
    return out + f"<|im_start|>user\n{user}<|im_end|>\n<|im_start|>assistant\n"
