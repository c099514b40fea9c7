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
        self.use_cuda_graph = True
        self._decoders: dict = {}      # (batch, max_len) -> cached decoder (KV buffers are reused across rollouts)
        self._graphs: dict = {}        # (batch, max_len, sampling) -> GraphedDecodeStep
        self.h2d_bytes = 0             # bytes copied host->device / device->host since the last reset
        self.d2h_bytes = 0

    # ------------------------------------------------------------ plumbing
    def device(self):
        return self.model.embed.device if hasattr(self.model, "embed") else next(self.model.buffers()).device

    def trainable_params(self):
        return self.model.trainable_params()

    def set_adapter_enabled(self, on: bool):
        self._adapter_on = bool(on)
        self.model.set_adapter_enabled(on)
        self._merged_fresh = False
        self._graphs.clear()  # merged-weight addresses may change with the adapter state

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
        self.h2d_bytes += ids_host.numel() * 8 + lens_host.numel() * 8 + B * 8
        rows = (torch.as_tensor(list(global_row_bases), dtype=torch.int64).repeat_interleave(G)
                + torch.arange(G, dtype=torch.int64).repeat(P)).to(dev)
        if not self._merged_fresh:
            self.model.merge_adapters()
            self._merged_fresh = True
        max_len = Lmax + N
        if dev.type == "cuda":
            max_len = (max_len + 127) // 128 * 128  # bucket the cache length so decoders and graphs are reused
        dkey = (B, max_len, G)
        dec = self._decoders.get(dkey)
        if dec is None:
            self._decoders.clear()
            self._graphs.clear()
            try:
                dec = self.model.new_decoder(B, max_len, self.comm, group=G)
            except TypeError:       # model families whose decoder takes no group argument
                dec = self.model.new_decoder(B, max_len, self.comm)
            self._decoders[dkey] = dec
        self.last_cache_bytes = dec.cache_bytes()
        logits = dec.prefill(ids, lens)
        dec.broadcast_groups(G)
        logits = logits.repeat_interleave(G, dim=0)
        eos = cfg.eos_token_id
        pad = eos if eos is not None else self.pad_token_id
        if dev.type == "cuda" and self.use_cuda_graph and N > 2:
            gkey = (B, max_len, temperature, top_p, eos, pad)
            step = self._graphs.get(gkey)
            if step is None:
                step = GraphedDecodeStep(dec, self.sampler, B, temperature, top_p, eos, pad)
                self._graphs[gkey] = step
            out_tok, out_lp, comp_len = step.run(logits, rows, N, self.early_exit_every)
        else:
            out_tok, out_lp, comp_len = run_decode_loop(dec, self.sampler, logits, rows, N, temperature, top_p,
                                                        eos, pad, self.early_exit_every)
        self.d2h_bytes += out_tok.numel() * 8 + out_lp.numel() * 4 + comp_len.numel() * 8
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
        self.h2d_bytes += (ids.numel() + start.numel() + targets.numel()) * 8
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
        # rows that have emitted EOS are retired: their attention reads no KV from here on
        if eos is not None and getattr(dec, "supports_retirement", False):
            logits = dec.decode(tok, ~finished)
        else:
            logits = dec.decode(tok)
    return out_tok, out_lp, comp_len


class GraphedDecodeStep:
    """One decode step (sample -> bookkeeping -> model decode) captured as a CUDA
    graph over static buffers, replayed once per generated token.  The draw
    index is a device counter that the graph itself advances, so replays need
    no host-side parameters and the host never synchronises inside the loop
    (except for the optional every-k early-exit poll)."""

    def __init__(self, dec, sampler: GrpoSampler, B: int, temperature, top_p, eos, pad):
        self.dec, self.sampler = dec, sampler
        self.B, self.temperature, self.top_p, self.eos, self.pad = B, temperature, top_p, eos, pad
        self.graph = None
        self.launches_per_replay = 0
        self.N = 0

    def _alloc(self, logits, rows, N):
        dev = logits.device
        B = self.B
        self.N = N
        # logits stay in the head GEMM's dtype inside the loop where the decoder offers that (the
        # sampler upcasts element by element, so the draw is the same as from an fp32 copy)
        self._decode = getattr(self.dec, "decode_native", None) or self.dec.decode
        dt = logits.dtype
        if self._decode is not self.dec.decode and logits.is_cuda:
            dt = self.dec.m.head_weight().dtype
        self.logits = torch.empty(logits.shape, dtype=dt, device=dev)
        self.rows = rows.clone()
        self.draw = torch.zeros(1, dtype=torch.int32, device=dev)
        self.finished = torch.zeros(B, dtype=torch.bool, device=dev)
        self.comp_len = torch.zeros(B, dtype=torch.int64, device=dev)
        self.out_tok = torch.full((B, N), self.pad, dtype=torch.int64, device=dev)
        self.out_lp = torch.zeros((B, N), dtype=torch.float32, device=dev)
        self.pad_t = torch.full((B,), self.pad, dtype=torch.int64, device=dev)
        self.kv_tokens_read = torch.zeros((), dtype=torch.int64, device=dev)   # per layer, summed over steps

    def _body(self):
        tok, lp = self.sampler.sample(self.logits, self.rows, 0, self.temperature, self.top_p, draw_dev=self.draw)
        tok = torch.where(self.finished, self.pad_t, tok)
        col = self.draw.to(torch.int64).clamp(max=self.N - 1).view(1, 1).expand(self.B, 1)
        self.out_tok.scatter_(1, col, tok[:, None])
        self.out_lp.scatter_(1, col, torch.where(self.finished, torch.zeros_like(lp), lp)[:, None])
        self.comp_len += (~self.finished).to(torch.int64)
        if self.eos is not None:
            self.finished |= tok == self.eos
        if self.eos is not None and getattr(self.dec, "supports_retirement", False):
            # retired rows stay in the fixed-shape batch but attend to nothing (see _step_lengths)
            self.kv_tokens_read += self.dec.kv_tokens_read(~self.finished).to(torch.int64)
            self.logits.copy_(self._decode(tok, ~self.finished))
        else:
            self.logits.copy_(self._decode(tok))
        self.draw += 1

    @torch.no_grad()
    def run(self, logits, rows, N, early_exit_every=32):
        from .ops import cuda as C
        if self.graph is None or N != self.N:
            self._alloc(logits, rows, N)
            self.graph = None
        self.logits.copy_(logits)
        self.rows.copy_(rows)
        self.draw.zero_()
        self.finished.zero_()
        self.comp_len.zero_()
        self.out_tok.fill_(self.pad)
        self.out_lp.zero_()
        self.kv_tokens_read.zero_()
        kv0 = self.dec.kv_len.clone()
        if self.graph is None:
            # one eager step warms every kernel (and lazy one-time allocations) before capture; its
            # effects are rolled back so the captured graph starts from the same state
            snap = (self.logits.clone(),)
            self._body()
            torch.cuda.synchronize()
            self.dec.kv_len.copy_(kv0)
            self.logits.copy_(snap[0])
            self.draw.zero_()
            self.finished.zero_()
            self.comp_len.zero_()
            self.out_tok.fill_(self.pad)
            self.out_lp.zero_()
            self.kv_tokens_read.zero_()
            before = C.launches()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._body()
            self.launches_per_replay = C.launches() - before
            self.graph = g
        steps = 0
        # N-1 full steps, then a final sample-only step handled eagerly below
        for t in range(N - 1):
            self.graph.replay()
            steps += 1
            if self.eos is not None and early_exit_every > 0 and (t + 1) % early_exit_every == 0 \
                    and bool(self.finished.all()):
                break
        C.lib().add_launches(self.launches_per_replay * steps)
        if steps == N - 1:
            tok, lp = self.sampler.sample(self.logits, self.rows, N - 1, self.temperature, self.top_p)
            tok = torch.where(self.finished, self.pad_t, tok)
            self.out_tok[:, N - 1] = tok
            self.out_lp[:, N - 1] = torch.where(self.finished, torch.zeros_like(lp), lp)
            self.comp_len += (~self.finished).to(torch.int64)
        return self.out_tok.clone(), self.out_lp.clone(), self.comp_len.clone()
