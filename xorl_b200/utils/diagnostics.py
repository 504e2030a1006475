"""Run-time diagnostics of the trainer: NVTX ranges, CUDA memory history, a non-finite gradient
scan, a host-side rank watchdog and the metrics sink.

* ``nvtx_range(name)``: NVTX push/pop on CUDA, nothing on CPU.
* ``MemoryHistory``: ``XORL_MEMHIST=1`` records allocator history from start-up and dumps a
  snapshot pickle into ``XORL_MEMHIST_DIR`` after step ``XORL_MEMHIST_DUMP_STEP`` and on an
  out-of-memory error (src/xorl/trainers/trainer.py:1464, :2133).
* ``nonfinite_gradient_report(engine)``: with ``XORL_DEBUG_NONFINITE_GRAD_SCAN=1`` the trainer lists
  the parameters whose gradient shard holds inf / nan after the reduction
  (src/xorl/trainers/trainer.py:1898).
* ``RankWatchdog``: every rank publishes a heartbeat counter in the rendezvous key-value store from
  a host thread and watches its peers'; a rank whose counter stops for ``timeout_s`` or that
  publishes a failure makes ``check()`` raise ``RankFailure`` on the others *before their next
  launch*, so nobody enters a collective with a dead peer.  The process then exits with
  ``RANK_FAILURE_EXIT_CODE`` and the job restarts from the last checkpoint (the reference is
  fail-closed in the same way: src/xorl/utils/device.py:25-51 bounds every collective, the server
  workers exchange heartbeats every 5 s, src/xorl/server/runner/utils/rank0_protocol.py:282-297).
* ``MetricsSink``: Weights & Biases when the package is importable and ``use_wandb`` is set, else a
  JSON-lines file ``metrics.jsonl`` in the output directory (src/xorl/trainers/trainer.py:409-423).
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from typing import Dict, List, Optional

import torch

RANK_FAILURE_EXIT_CODE = 75


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class MemoryHistory:
    def __init__(self, rank: int = 0, env=os.environ):
        self.enabled = env.get("XORL_MEMHIST", "0") not in ("0", "", "false") and torch.cuda.is_available()
        self.dir = env.get("XORL_MEMHIST_DIR", "./memhist")
        self.dump_step = int(env.get("XORL_MEMHIST_DUMP_STEP", "2"))
        self.rank = rank
        self.dumped: List[str] = []
        if self.enabled:
            torch.cuda.memory._record_memory_history(max_entries=200_000)

    def _dump(self, tag: str) -> Optional[str]:
        if not self.enabled:
            return None
        os.makedirs(self.dir, exist_ok=True)
        path = os.path.join(self.dir, f"memhist_rank{self.rank}_{tag}.pickle")
        torch.cuda.memory._dump_snapshot(path)
        self.dumped.append(path)
        return path

    def after_step(self, step: int) -> Optional[str]:
        return self._dump(f"step{step}") if step == self.dump_step else None

    def on_oom(self) -> Optional[str]:
        return self._dump("oom")

    def close(self) -> None:
        if self.enabled:
            torch.cuda.memory._record_memory_history(enabled=None)
            self.enabled = False


def nonfinite_scan_enabled(env=os.environ) -> bool:
    return env.get("XORL_DEBUG_NONFINITE_GRAD_SCAN", "0") not in ("0", "", "false")


def nonfinite_gradient_report(engine) -> List[str]:
    """Names of the parameters (``unit/group:param``) whose slice of this rank's gradient shard is
    not finite, plus ``.../<gap>`` when the bad values sit between parameters."""
    bad: List[str] = []
    for unit in engine.units:
        for g in unit.groups:
            gs = getattr(g, "grad_shard", None)
            if gs is None or bool(torch.isfinite(gs).all()):
                continue
            covered = torch.zeros(gs.numel(), dtype=torch.bool, device=gs.device)
            for i, a, b in g.param_segments_in_shard():
                covered[a:b] = True
                if not bool(torch.isfinite(gs[a:b]).all()):
                    bad.append(f"{unit.name}/{g.name}:{g.named_params[i][0]}")
            if not bool(torch.isfinite(gs[~covered]).all()):
                bad.append(f"{unit.name}/{g.name}:<gap>")
    return bad


class RankFailure(RuntimeError):
    """Another rank stopped answering or reported a failure."""


class RankWatchdog:
    """Heartbeats over a ``torch.distributed`` store (TCPStore / HashStore / FileStore).

    ``start()`` launches one daemon thread that bumps ``hb/<rank>`` every ``interval_s`` and reads
    the peers' counters.  ``check()`` is called by the training loop between steps."""

    def __init__(self, store, rank: int, world: int, interval_s: float = 5.0, timeout_s: float = 60.0,
                 prefix: str = "xorl_wd"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._failure: Optional[str] = None
        self._beat = 0
        self._seen: Dict[int, tuple] = {}

    def _key(self, kind: str, r: int) -> str:
        return f"{self.prefix}/{kind}/{r}"

    def _read(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:  # noqa: BLE001  (store gone: treated like a silent peer)
            return None

    def _tick(self) -> None:
        self._beat += 1
        try:
            self.store.set(self._key("hb", self.rank), str(self._beat))
        except Exception as e:  # noqa: BLE001
            self._failure = f"rank {self.rank}: heartbeat store unreachable ({e})"
            return
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            msg = self._read(self._key("fail", r))
            if msg is not None:
                self._failure = f"rank {r} reported: {msg}"
                return
            val = self._read(self._key("hb", r))
            last = self._seen.get(r)
            if last is None or last[0] != val:
                self._seen[r] = (val, now)
            elif now - last[1] > self.timeout_s:
                self._failure = f"rank {r} sent no heartbeat for {now - last[1]:.1f} s"
                return

    def _loop(self) -> None:
        while not self._stop.is_set() and self._failure is None:
            self._tick()
            self._stop.wait(self.interval_s)

    def start(self) -> "RankWatchdog":
        self._tick()
        self._thread = threading.Thread(target=self._loop, name="xorl-rank-watchdog", daemon=True)
        self._thread.start()
        return self

    def report_failure(self, message: str) -> None:
        """Tell the peers that this rank is going down (called from the trainer's exception path)."""
        try:
            self.store.set(self._key("fail", self.rank), message[:500])
        except Exception:  # noqa: BLE001
            pass

    def check(self) -> None:
        if self._failure is not None:
            raise RankFailure(self._failure)

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)


class MetricsSink:
    def __init__(self, train_args, rank: int, config: Optional[dict] = None):
        self.rank = rank
        self.interval = max(1, int(getattr(train_args, "wandb_log_interval", 1)))
        self.run = None
        self.file = None
        if rank != 0:
            return
        if getattr(train_args, "use_wandb", False):
            try:
                import wandb  # type: ignore
                self.run = wandb.init(project=train_args.wandb_project, name=train_args.wandb_name,
                                      tags=train_args.wandb_tags, config=config or {})
            except Exception:  # noqa: BLE001  (package or network missing: fall back to the file)
                self.run = None
        if self.run is None:
            os.makedirs(train_args.output_dir, exist_ok=True)
            self.file = open(os.path.join(train_args.output_dir, "metrics.jsonl"), "a")

    def log(self, metrics: Dict[str, float], step: int) -> None:
        if self.rank != 0 or step % self.interval:
            return
        if self.run is not None:
            self.run.log(metrics, step=step)
        elif self.file is not None:
            self.file.write(json.dumps({"step": step, **{k: float(v) for k, v in metrics.items()
                                                         if isinstance(v, (int, float))}}) + "\n")
            self.file.flush()

    def close(self) -> None:
        if self.run is not None:
            self.run.finish()
        if self.file is not None:
            self.file.close()
            self.file = None
