"""Communicator seam.

Every distributed call site receives a ``Comm`` explicitly (never ambient), as
in the reference (``crates/ferrl/src/comm.rs:127-175``).  Implementations:

* ``SoloComm``      world of one, zero collective calls.
* ``ThreadComm``    ranks are threads of this process; fixed rank-order sums,
                    barrier timeouts and a shared poison cell.  CPU stand-in for
                    lockstep tests (reference ``LocalComm``, comm.rs:414-498).
* ``TorchDistComm`` one process per rank over ``torch.distributed`` (``nccl``
                    on GPUs, ``gloo`` on CPU) - bootstrap, control plane and the
                    measured NCCL baseline.
* ``SymmComm``      (``ferrl_b200.parallel.symm``) peer-memory data plane whose
                    collectives run inside our own sm_100a kernels.

Beyond the reference's single sum all-reduce the seam also offers
``all_gather_bytes`` so consensus checks cost one exchange instead of one
scalar all-reduce per digest word.
"""
from __future__ import annotations

import hashlib
import struct
import threading
import time
from typing import Callable, Optional, Sequence

import torch

DEFAULT_COLLECTIVE_TIMEOUT = 300.0


class CommError(RuntimeError):
    """Base class; ``kind`` mirrors the reference's CommError variants."""

    kind = "backend"


class CommMismatch(CommError):
    kind = "mismatch"


class CommTimeout(CommError):
    kind = "timeout"


class CommPoisoned(CommError):
    kind = "poisoned"


class CommConfigError(CommError):
    kind = "config"


class Comm:
    """Abstract communicator. All tensors are summed in fixed rank order so every
    rank observes identical bits."""

    rank: int = 0
    world_size: int = 1
    # seconds this rank's host thread has spent blocked inside collectives (waiting for slower peers plus the
    # exchange itself); the trainer reports the per-step difference as the ``comm_wait`` phase
    wait_s: float = 0.0

    def validate_all_reduce_sum(self, tensors: Sequence[torch.Tensor]) -> None:
        for t in tensors:
            if t.dtype not in (torch.float32, torch.float64):
                raise CommMismatch(f"all_reduce_sum supports f32/f64 tensors, got {t.dtype}")
            if not t.is_contiguous():
                raise CommMismatch("all_reduce_sum requires contiguous tensors")

    def all_reduce_sum(self, tensors: list[torch.Tensor]) -> list[torch.Tensor]:
        raise NotImplementedError

    def all_reduce_scalar_sum(self, value: float) -> float:
        raise NotImplementedError

    def all_gather_bytes(self, blob: bytes) -> list[bytes]:
        raise NotImplementedError

    # ---- derived helpers used all over the trainer ----
    def all_reduce_scalars_sum(self, values: Sequence[float]) -> list[float]:
        """Several control scalars in one exchange (window token count, live
        groups, kl/clip sums ... are packed rather than sent one by one)."""
        if self.world_size == 1:
            return [float(v) for v in values]
        blobs = self.all_gather_bytes(struct.pack(f"<{len(values)}d", *values))
        cols = [struct.unpack(f"<{len(values)}d", b) for b in blobs]
        return [sum(c[i] for c in cols) for i in range(len(values))]

    def barrier(self) -> None:
        self.all_reduce_scalar_sum(0.0)

    def broadcast_bytes(self, blob: Optional[bytes], root: int = 0) -> bytes:
        return self.all_gather_bytes(blob if self.rank == root and blob is not None else b"")[root]

    def require_consensus(self, blob: bytes, what: str) -> None:
        """Every rank must hold the same bytes (compared by SHA-256), else all
        ranks raise ``CommMismatch`` together (reference trainer.rs:4415-4445)."""
        if self.world_size == 1:
            return
        digests = self.all_gather_bytes(hashlib.sha256(blob).digest())
        if any(d != digests[0] for d in digests):
            bad = [i for i, d in enumerate(digests) if d != digests[0]]
            raise CommMismatch(f"ranks disagree on {what}: ranks {bad} differ from rank 0")

    def coordinate(self, fn: Callable[[], object], what: str = "local call"):
        """Status rendezvous: run ``fn`` locally, agree on failure across ranks so
        all ranks take the same branch without waiting for a collective timeout
        (reference tensor_parallel.rs:31-61, trainer.rs:4342-4366)."""
        err: Optional[BaseException] = None
        out = None
        try:
            out = fn()
        except CommError:
            raise  # a communicator failure is terminal: never enter another collective
        except Exception as e:  # noqa: BLE001 - converted to a flag on purpose
            err = e
        failures = self.all_reduce_scalar_sum(0.0 if err is None else 1.0)
        if failures > 0:
            if err is not None:
                raise PeerFailure(f"{what} failed on this rank: {err!r}", local=err)
            raise PeerFailure(f"{what} failed on {int(failures)} peer rank(s)", local=None)
        return out


class PeerFailure(RuntimeError):
    """A coordinated failure: at least one rank failed; every rank raises this."""

    def __init__(self, msg: str, local: Optional[BaseException]):
        super().__init__(msg)
        self.local = local


class SoloComm(Comm):
    rank = 0
    world_size = 1

    def all_reduce_sum(self, tensors):
        return tensors

    def all_reduce_scalar_sum(self, value):
        return float(value)

    def all_gather_bytes(self, blob):
        return [blob]


# --------------------------------------------------------------------------
# ThreadComm: in-process world for lockstep tests
# --------------------------------------------------------------------------

class _World:
    def __init__(self, n: int, timeout: float):
        self.n = n
        self.timeout = timeout
        self.cv = threading.Condition()
        self.generation = 0
        self.arrived = 0
        self.slots: list = [None] * n
        self.result = None
        self.poison: Optional[str] = None
        self.calls = 0


class ThreadComm(Comm):
    """One instance per rank, sharing a ``_World``. A collective is: deposit,
    wait for all, rank 0 of the generation reduces in rank order, all read."""

    def __init__(self, world: _World, rank: int):
        self._w = world
        self.rank = rank
        self.world_size = world.n

    @staticmethod
    def world(n: int, timeout: float = DEFAULT_COLLECTIVE_TIMEOUT) -> list["ThreadComm"]:
        if n < 1:
            raise CommConfigError("world size must be >= 1")
        w = _World(n, timeout)
        return [ThreadComm(w, r) for r in range(n)]

    @property
    def collective_calls(self) -> int:
        return self._w.calls

    def poison(self, why: str) -> None:
        with self._w.cv:
            if self._w.poison is None:
                self._w.poison = why
            self._w.cv.notify_all()

    def _exchange(self, payload, reduce_fn):
        t0 = time.perf_counter()
        try:
            return self._exchange_inner(payload, reduce_fn)
        finally:
            self.wait_s += time.perf_counter() - t0

    def _exchange_inner(self, payload, reduce_fn):
        w = self._w
        deadline = time.monotonic() + w.timeout
        with w.cv:
            if w.poison is not None:
                raise CommPoisoned(w.poison)
            gen = w.generation
            w.slots[self.rank] = payload
            w.arrived += 1
            if w.arrived == w.n:
                try:
                    w.result = reduce_fn(list(w.slots))
                except CommError as e:
                    w.poison = str(e)
                    w.result = e
                w.arrived = 0
                w.slots = [None] * w.n
                w.generation += 1
                w.calls += 1
                w.cv.notify_all()
            else:
                while w.generation == gen and w.poison is None:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        w.poison = f"rank {self.rank} timed out after {w.timeout}s waiting for peers"
                        w.cv.notify_all()
                        raise CommTimeout(w.poison)
                    w.cv.wait(left)
                if w.generation == gen and w.poison is not None:
                    raise CommPoisoned(w.poison)
            res = w.result
        if isinstance(res, CommError):
            raise type(res)(str(res))
        return res

    def all_reduce_sum(self, tensors):
        self.validate_all_reduce_sum(tensors)
        if self.world_size == 1:
            return tensors

        def reduce(slots):
            sig0 = [(tuple(t.shape), t.dtype) for t in slots[0]]
            for r, s in enumerate(slots):
                if [(tuple(t.shape), t.dtype) for t in s] != sig0:
                    raise CommMismatch(f"rank {r} deposited a different tensor signature than rank 0")
            out = []
            for i in range(len(sig0)):
                acc = slots[0][i].clone()
                for r in range(1, len(slots)):
                    acc = acc + slots[r][i]
                out.append(acc)
            return out

        res = self._exchange([t.detach().clone() for t in tensors], reduce)
        for t, r in zip(tensors, res):
            t.copy_(r)
        return tensors

    def all_reduce_scalar_sum(self, value):
        if self.world_size == 1:
            return float(value)

        def reduce(slots):
            acc = 0.0
            for v in slots:
                acc += v
            return acc

        return self._exchange(float(value), reduce)

    def all_gather_bytes(self, blob):
        if self.world_size == 1:
            return [blob]
        return self._exchange(bytes(blob), lambda slots: list(slots))


def run_ranks(n: int, fn: Callable[[Comm], object], timeout: float = 20.0) -> list:
    """Run ``fn(comm)`` on ``n`` ThreadComm ranks; returns results (or raises the
    first rank's exception after all threads ended)."""
    comms = ThreadComm.world(n, timeout)
    out: list = [None] * n
    errs: list = [None] * n

    def body(r):
        try:
            out[r] = fn(comms[r])
        except BaseException as e:  # noqa: BLE001
            errs[r] = e
            comms[r].poison(f"rank {r} raised {e!r}")

    ts = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout * 4)
    for e in errs:
        if e is not None and not isinstance(e, CommPoisoned):
            raise e
    for e in errs:
        if e is not None:
            raise e
    return out


from .dist import TorchDistComm, NcclConfig  # noqa: E402,F401
