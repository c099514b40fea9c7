"""``torch.distributed`` communicator: one OS process per GPU.

Rank discovery accepts both launchers: ``torchrun`` (``RANK``/``WORLD_SIZE``/
``LOCAL_RANK``/``MASTER_ADDR``/``MASTER_PORT``) and Slurm ``srun``
(``SLURM_PROCID``/``SLURM_NTASKS``/``SLURM_LOCALID`` with the rendezvous file
named by ``FERRL_NCCL_RENDEZVOUS``), the reference's launch contract
(``crates/ferrl/src/comm/nccl.rs:93-128``, ``:184-220``).  Unlike the
reference's NCCL bridge, which has no timeout or abort path
(``comm/nccl.rs:30-36``), the process group is created with a finite timeout so
a dead peer ends the next collective with ``CommTimeout`` instead of a hang.

Tensor all-reduce keeps the reference's dtype gate (f32/f64, contiguous) and
is the *baseline* data plane; the product data plane is ``SymmComm``.
"""
from __future__ import annotations

import datetime
import time
import os
from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from . import Comm, CommConfigError, CommError, CommMismatch, CommPoisoned, CommTimeout

RENDEZVOUS_ENV = "FERRL_NCCL_RENDEZVOUS"


@dataclass(frozen=True)
class NcclConfig:
    rank: int
    world_size: int
    local_rank: int
    init_method: str

    @staticmethod
    def from_env(env: Optional[Mapping[str, str]] = None) -> Optional["NcclConfig"]:
        """``None`` when no distributed launch is described by the environment."""
        env = os.environ if env is None else env

        def geti(name: str) -> int:
            try:
                v = int(env[name])
            except KeyError:
                raise CommConfigError(f"{name} is not set") from None
            except ValueError:
                raise CommConfigError(f"{name}={env[name]!r} is not an integer") from None
            if v < 0:
                raise CommConfigError(f"{name} must be >= 0")
            return v

        if "RANK" in env and "WORLD_SIZE" in env:
            rank, world = geti("RANK"), geti("WORLD_SIZE")
            local = geti("LOCAL_RANK") if "LOCAL_RANK" in env else rank
            addr = env.get("MASTER_ADDR", "127.0.0.1")
            port = env.get("MASTER_PORT", "29500")
            init = f"tcp://{addr}:{port}"
        elif RENDEZVOUS_ENV in env:
            rank, world, local = geti("SLURM_PROCID"), geti("SLURM_NTASKS"), geti("SLURM_LOCALID")
            path = env[RENDEZVOUS_ENV]
            if not path:
                raise CommConfigError(f"{RENDEZVOUS_ENV} is empty")
            init = f"file://{os.path.abspath(path)}"
        else:
            return None
        if world < 1 or rank >= world:
            raise CommConfigError(f"rank {rank} outside world of {world}")
        return NcclConfig(rank, world, local, init)


class TorchDistComm(Comm):
    def __init__(self, group=None, device: Optional[torch.device] = None):
        import torch.distributed as dist
        self._dist = dist
        self._group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.device = device if device is not None else torch.device("cpu")
        self._poison: Optional[str] = None
        self.collective_calls = 0

    @classmethod
    def bootstrap(cls, cfg: Optional[NcclConfig] = None, backend: Optional[str] = None,
                  timeout_s: float = 300.0) -> "TorchDistComm":
        import torch.distributed as dist
        cfg = cfg or NcclConfig.from_env()
        if cfg is None:
            raise CommConfigError("no distributed launch environment (RANK/WORLD_SIZE or "
                                  f"{RENDEZVOUS_ENV}+SLURM_*)")
        use_cuda = torch.cuda.is_available()
        backend = backend or ("nccl" if use_cuda else "gloo")
        device = torch.device("cpu")
        if backend == "nccl":
            if cfg.local_rank >= torch.cuda.device_count():
                raise CommConfigError(f"local rank {cfg.local_rank} has no GPU "
                                      f"({torch.cuda.device_count()} visible)")
            torch.cuda.set_device(cfg.local_rank)
            device = torch.device("cuda", cfg.local_rank)
        if not dist.is_initialized():
            kw = dict(backend=backend, init_method=cfg.init_method, rank=cfg.rank,
                      world_size=cfg.world_size, timeout=datetime.timedelta(seconds=timeout_s))
            if backend == "nccl":
                kw["device_id"] = device
            dist.init_process_group(**kw)
        return cls(None, device)

    def _guard(self):
        if self._poison is not None:
            raise CommPoisoned(self._poison)

    def _wrap(self, fn):
        self._guard()
        t0 = time.perf_counter()
        try:
            self.collective_calls += 1
            return fn()
        except CommError:
            raise
        except RuntimeError as e:
            msg = str(e)
            self._poison = msg
            if "imeout" in msg or "timed out" in msg:
                raise CommTimeout(msg) from e
            raise CommError(msg) from e
        finally:
            # host-blocking time only: a collective on device tensors returns when it is enqueued, the control-plane
            # exchanges (scalars, byte blobs, barriers) return when every rank has arrived
            self.wait_s += time.perf_counter() - t0

    def all_reduce_sum(self, tensors):
        self.validate_all_reduce_sum(tensors)
        if self.world_size == 1:
            return tensors
        dist = self._dist

        def go():
            if self.device.type == "cuda" and len(tensors) > 1:
                # NCCL baseline: coalesce same-dtype tensors into one flat launch
                by = {}
                for t in tensors:
                    by.setdefault(t.dtype, []).append(t)
                for ts in by.values():
                    flat = torch.cat([t.reshape(-1) for t in ts])
                    dist.all_reduce(flat, group=self._group)
                    off = 0
                    for t in ts:
                        t.copy_(flat[off:off + t.numel()].view_as(t))
                        off += t.numel()
            else:
                for t in tensors:
                    dist.all_reduce(t, group=self._group)
            return tensors

        return self._wrap(go)

    def all_reduce_scalar_sum(self, value):
        if self.world_size == 1:
            return float(value)
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device)

        def go():
            self._dist.all_reduce(t, group=self._group)
            return float(t.item())          # the read-back is where the host waits for the slowest rank
        return self._wrap(go)

    def all_gather_bytes(self, blob):
        if self.world_size == 1:
            return [blob]
        out = [None] * self.world_size
        self._wrap(lambda: self._dist.all_gather_object(out, bytes(blob), group=self._group))
        return out

    def barrier(self):
        if self.world_size > 1:
            self._wrap(lambda: self._dist.barrier(group=self._group))

    def validate_all_reduce_sum(self, tensors):
        super().validate_all_reduce_sum(tensors)
        for t in tensors:
            if t.device.type != self.device.type:
                raise CommMismatch(f"tensor on {t.device}, communicator on {self.device}")
