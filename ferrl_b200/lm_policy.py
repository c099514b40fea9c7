"""``LmPolicy``: rollout and scoring for any model family behind the ``Policy`` seam.

Reference: ``crates/ferrl/src/lm_policy.rs`` - ``batched_group_decode``
``:626-798`` (prefill, per-row sampling, EOS retire, pad), scoring window
``:331-349``, ``token_logprobs`` ``:826-845``.  There, sampling copies a
``[vocab]`` row to the host per row per token and the merged weights are
rebuilt on every ``generate`` call.

Here the decode loop never leaves the device: logits, sampling (counter RNG
keyed by global row and draw index), EOS retirement, completion lengths and
behaviour log-probs are device tensors with fixed shapes, one host sync at the
end of the rollout (plus an optional early-exit poll).  All prompts of a
window decode as ONE batch; a prompt is prefilled once and its KV is shared
by its group.  Merged weights are refreshed only after an optimizer step.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .comm import Comm, SoloComm
from .policy import GenConfig, Policy, Rollout
from .sampler import GrpoSampler, validate_temperature, validate_top_p

SCORING_CHUNK = 128


class LmPolicy(Policy):
    def __init__(self, model, sampler: GrpoSampler, comm: Optional[Comm] = None, *,
                 pad_token_id: int = 0, score_microbatch: int = 0, early_exit_every: int = 32):
        self.model = model
        self.sampler = sampler
        self.comm = comm or SoloComm()  # tensor-parallel group communicator (Solo when unsharded)
        self.pad_token_id = pad_token_id
        self.score_microbatch = score_microbatch
        self.early_exit_every = early_exit_every
        self._adapter_on = True
        self._merged_fresh = False
        self.last_cache_bytes = 0

    # ------------------------------------------------------------ plumbing
    def device(self):
        return self.model.embed.device if hasattr(self.model, "embed") else next(self.model.buffers()).device

    def trainable_params(self):
        return self.model.trainable_params()

    def set_adapter_enabled(self, on: bool):
        self._adapter_on = bool(on)
        self.model.set_adapter_enabled(on)
        self._merged_fresh = False

    def adapter_enabled(self) -> bool:
        return self._adapter_on

    def on_params_updated(self):
        self._merged_fresh = False

    def lora_recipe(self):
        return self.model.lora_recipe()

    def sampler_state(self) -> bytes:
        return self.sampler.state_bytes()

    def validate_sampler_state(self, state: bytes) -> None:
        GrpoSampler.from_state_bytes(state)

    def restore_sampler_state(self, state: bytes) -> None:
        self.sampler.load_state_bytes(state)

    def _resolve_sampling(self, cfg: GenConfig):
        """Training rolls out at the sampler's baked temperature; only the eval
        harness may override temperature / top-p (reference lm_policy.rs:481-512)."""
        if cfg.eval_sampling is not None:
            return validate_temperature(cfg.eval_sampling.temperature), validate_top_p(cfg.eval_sampling.top_p)
        if abs(cfg.temperature - self.sampler.temperature) > 0:
            raise ValueError(f"GenConfig temperature {cfg.temperature} differs from the sampler's baked "
                             f"temperature {self.sampler.temperature}")
        return self.sampler.temperature, validate_top_p(cfg.top_p)

    # ------------------------------------------------------------- rollout
    @torch.no_grad()
    def generate_batch(self, prompts: Sequence[Sequence[int]], cfg: GenConfig,
                       global_row_bases: Sequence[int]) -> list[Rollout]:
        if len(prompts) == 0:
            return []
        if any(len(p) == 0 for p in prompts):
            raise ValueError("empty prompt")
        if cfg.group_size < 1 or cfg.max_new_tokens < 1:
            raise ValueError("group_size and max_new_tokens must be >= 1")
        temperature, top_p = self._resolve_sampling(cfg)
        dev = self.device()
        P, G, N = len(prompts), cfg.group_size, cfg.max_new_tokens
        B = P * G
        lens_host = torch.tensor([len(p) for p in prompts], dtype=torch.int64)
        Lmax = int(lens_host.max())
        ids_host = torch.full((P, Lmax), self.pad_token_id, dtype=torch.int64)
        for i, p in enumerate(prompts):
            ids_host[i, :len(p)] = torch.as_tensor(list(p), dtype=torch.int64)
        if dev.type == "cuda":
            ids_host, lens_host = ids_host.pin_memory(), lens_host.pin_memory()
        ids = ids_host.to(dev, non_blocking=True)
        lens = lens_host.to(dev, non_blocking=True)
        rows = (torch.as_tensor(list(global_row_bases), dtype=torch.int64).repeat_interleave(G)
                + torch.arange(G, dtype=torch.int64).repeat(P)).to(dev)
        if not self._merged_fresh:
            self.model.merge_adapters()
            self._merged_fresh = True
        dec = self.model.new_decoder(B, Lmax + N, self.comm)
        self.last_cache_bytes = dec.cache_bytes()
        logits = dec.prefill(ids, lens)
        dec.broadcast_groups(G)
        logits = logits.repeat_interleave(G, dim=0)
        eos = cfg.eos_token_id
        pad = eos if eos is not None else self.pad_token_id
        out_tok, out_lp, comp_len = run_decode_loop(dec, self.sampler, logits, rows, N, temperature, top_p,
                                                    eos, pad, self.early_exit_every)
        out_tok, out_lp, comp_len = out_tok.cpu(), out_lp.cpu(), comp_len.cpu()
        res = []
        for i, p in enumerate(prompts):
            pl = len(p)
            prompt_part = torch.as_tensor(list(p), dtype=torch.int64)[None].expand(G, pl)
            toks = torch.cat([prompt_part, out_tok[i * G:(i + 1) * G]], dim=1)
            res.append(Rollout(toks, pl, comp_len[i * G:(i + 1) * G].tolist(), out_lp[i * G:(i + 1) * G].clone()))
        return res

    # ------------------------------------------------------------- scoring
    def _pack(self, rollouts: Sequence[Rollout]):
        """Rows of all rollouts, left-aligned, right-padded to the widest."""
        N = rollouts[0].width
        if any(r.width != N for r in rollouts):
            raise ValueError("rollouts of one scoring call must share max_new_tokens")
        W = max(r.token_ids.shape[1] for r in rollouts)
        R = sum(len(r) for r in rollouts)
        ids = torch.full((R, W), self.pad_token_id, dtype=torch.int64)
        targets = torch.empty((R, N), dtype=torch.int64)
        start = torch.empty(R, dtype=torch.int64)
        o = 0
        for r in rollouts:
            g = len(r)
            ids[o:o + g, :r.token_ids.shape[1]] = r.token_ids
            targets[o:o + g] = r.token_ids[:, r.prompt_len:]
            start[o:o + g] = r.prompt_len - 1
            o += g
        return ids, start, targets

    def token_logprobs(self, rollouts) -> torch.Tensor:
        if isinstance(rollouts, Rollout):
            rollouts = [rollouts]
        ids, start, targets = self._pack(rollouts)
        dev = self.device()
        if dev.type == "cuda":
            ids, start, targets = ids.pin_memory(), start.pin_memory(), targets.pin_memory()
        ids, start, targets = (t.to(dev, non_blocking=True) for t in (ids, start, targets))
        inp = ids[:, :-1]
        mb = self.score_microbatch if self.score_microbatch > 0 else inp.shape[0]
        outs = []
        for s in range(0, inp.shape[0], mb):
            outs.append(self.model.token_logprobs(inp[s:s + mb], start[s:s + mb], targets[s:s + mb],
                                                  self.sampler.temperature, self.comm))
        return torch.cat(outs, dim=0)


@torch.no_grad()
def run_decode_loop(dec, sampler: GrpoSampler, logits, rows, N: int, temperature: float,
                    top_p: Optional[float], eos: Optional[int], pad: int, early_exit_every: int = 32):
    """Device-resident sampling loop shared by every family's cached decoder.
    Returns ``(tokens [B,N] int64, behaviour_logprobs [B,N] f32, completion_len [B] int64)``."""
    dev = logits.device
    B = logits.shape[0]
    finished = torch.zeros(B, dtype=torch.bool, device=dev)
    comp_len = torch.zeros(B, dtype=torch.int64, device=dev)
    out_tok = torch.full((B, N), pad, dtype=torch.int64, device=dev)
    out_lp = torch.zeros((B, N), dtype=torch.float32, device=dev)
    pad_t = torch.full((B,), pad, dtype=torch.int64, device=dev)
    for t in range(N):
        tok, lp = sampler.sample(logits, rows, t, temperature, top_p)
        tok = torch.where(finished, pad_t, tok)
        out_tok[:, t] = tok
        out_lp[:, t] = torch.where(finished, torch.zeros_like(lp), lp)
        comp_len += (~finished).to(torch.int64)
        if eos is not None:
            finished = finished | (tok == eos)
        if t == N - 1:
            break
        if eos is not None and early_exit_every > 0 and (t + 1) % early_exit_every == 0 and bool(finished.all()):
            break
        logits = dec.decode(tok)
    return out_tok, out_lp, comp_len
