"""Process supervisor of the training service.

``launcher --mode launch`` starts the service as separate processes, the way the reference's
launcher does (src/xorl/server/launcher.py:1111 ``_launch_workers_with_torchrun``, :1426-1458
wait / stop): a ``torchrun`` fleet of workers whose rank 0 serves commands over ZMQ
(``--mode worker``) and one API process (``--mode connect``) that owns the REST server and the
orchestrator.  The supervisor

* starts every child in its own process group (so that a whole ``torchrun`` tree can be signalled),
* waits until each reports ready (a callable per child, polled; a child that exits first is an error),
* then watches them: when any child exits, or a readiness / liveness probe keeps failing for
  ``liveness_timeout`` seconds, every other child is sent SIGTERM, then SIGKILL after a grace period,
  and ``run()`` returns the exit code of the first child that ended (non-zero for a probe failure),
* forwards SIGTERM / SIGINT received by itself to the children and tears everything down.

Nothing here touches a GPU; failures are process exits and unanswered probes on the host.
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence


@dataclass
class ChildSpec:
    name: str
    argv: Sequence[str]
    env: Optional[Dict[str, str]] = None
    ready: Optional[Callable[[], bool]] = None       # polled until True
    alive: Optional[Callable[[], bool]] = None       # polled after start-up (None: process exit only)
    ready_timeout: float = 600.0


@dataclass
class _Child:
    spec: ChildSpec
    proc: subprocess.Popen
    ready: bool = False
    last_alive: float = field(default_factory=time.monotonic)


class Supervisor:
    def __init__(self, children: Sequence[ChildSpec], poll_interval: float = 0.2, grace: float = 10.0,
                 liveness_timeout: float = 60.0, log: Callable[[str], None] = None):
        self.specs = list(children)
        self.poll, self.grace, self.liveness_timeout = poll_interval, grace, liveness_timeout
        self.children: List[_Child] = []
        self._stop = threading.Event()
        self.events: List[str] = []
        self._log = log or (lambda m: print(f"[supervisor] {m}", file=sys.stderr, flush=True))
        self.first_exit: Optional[str] = None

    # ---- lifecycle -----------------------------------------------------------------------------
    def start(self) -> None:
        for spec in self.specs:
            env = dict(os.environ)
            env.update(spec.env or {})
            proc = subprocess.Popen(list(spec.argv), env=env, start_new_session=True)
            self.children.append(_Child(spec, proc))
            self._note(f"started {spec.name} (pid {proc.pid})")

    def _note(self, msg: str) -> None:
        self.events.append(msg)
        self._log(msg)

    def request_stop(self, *_args) -> None:
        self._stop.set()

    def _signal_group(self, c: _Child, sig: int) -> None:
        try:
            os.killpg(c.proc.pid, sig)          # the child leads its own session / process group
        except (ProcessLookupError, PermissionError):
            pass

    def stop_all(self) -> None:
        live = [c for c in self.children if c.proc.poll() is None]
        for c in live:
            self._signal_group(c, signal.SIGTERM)
        deadline = time.monotonic() + self.grace
        while time.monotonic() < deadline and any(c.proc.poll() is None for c in live):
            time.sleep(self.poll)
        for c in live:
            if c.proc.poll() is None:
                self._note(f"{c.spec.name} ignored SIGTERM for {self.grace:.0f}s: SIGKILL")
                self._signal_group(c, signal.SIGKILL)
        for c in live:
            try:
                c.proc.wait(timeout=self.grace)
            except subprocess.TimeoutExpired:
                pass

    def run(self, install_signal_handlers: bool = True) -> int:
        """Starts, waits for readiness, supervises.  Returns the service's exit code."""
        if install_signal_handlers and threading.current_thread() is threading.main_thread():
            signal.signal(signal.SIGTERM, self.request_stop)
            signal.signal(signal.SIGINT, self.request_stop)
        self.start()
        code = 0
        t0 = time.monotonic()
        try:
            while not self._stop.is_set():
                now = time.monotonic()
                for c in self.children:
                    rc = c.proc.poll()
                    if rc is not None:
                        self.first_exit = c.spec.name
                        self._note(f"{c.spec.name} exited with code {rc}: stopping the service")
                        code = rc if rc != 0 else (0 if all(x.proc.poll() == 0 for x in self.children) else 1)
                        if rc == 0 and any(x.proc.poll() is None for x in self.children):
                            code = 1                      # a service member may not leave on its own
                        return code
                    if not c.ready:
                        if c.spec.ready is None or self._probe(c.spec.ready):
                            c.ready = True
                            c.last_alive = now
                            self._note(f"{c.spec.name} ready after {now - t0:.1f}s")
                        elif now - t0 > c.spec.ready_timeout:
                            self.first_exit = c.spec.name
                            self._note(f"{c.spec.name} not ready after {c.spec.ready_timeout:.0f}s: stopping")
                            return 1
                    elif c.spec.alive is not None:
                        if self._probe(c.spec.alive):
                            c.last_alive = now
                        elif now - c.last_alive > self.liveness_timeout:
                            self.first_exit = c.spec.name
                            self._note(f"{c.spec.name} unresponsive for {self.liveness_timeout:.0f}s: stopping")
                            return 1
                time.sleep(self.poll)
            self._note("stop requested")
            return 0
        finally:
            self.stop_all()

    @staticmethod
    def _probe(fn: Callable[[], bool]) -> bool:
        try:
            return bool(fn())
        except Exception:  # noqa: BLE001
            return False

    def all_ready(self) -> bool:
        return bool(self.children) and all(c.ready for c in self.children)


# ---- probes -----------------------------------------------------------------------------------
def http_ready(url: str, timeout: float = 2.0) -> Callable[[], bool]:
    def probe() -> bool:
        import urllib.request
        with urllib.request.urlopen(url, timeout=timeout) as r:      # noqa: S310  (loopback URL built by the launcher)
            return 200 <= r.status < 300
    return probe


def zmq_health(address: str, timeout_ms: int = 2000) -> Callable[[], bool]:
    """Heartbeat of the worker fleet: rank 0 answers ``{"op": "health"}`` on its command socket."""
    def probe() -> bool:
        import msgpack
        import zmq
        ctx = zmq.Context.instance()
        s = ctx.socket(zmq.REQ)
        s.setsockopt(zmq.LINGER, 0)
        s.setsockopt(zmq.RCVTIMEO, timeout_ms)
        s.setsockopt(zmq.SNDTIMEO, timeout_ms)
        try:
            s.connect(address)
            s.send(msgpack.packb({"op": "health"}, use_bin_type=True))
            return "result" in msgpack.unpackb(s.recv(), raw=False)
        finally:
            s.close()
    return probe


def service_children(config: str, nproc: int, api_host: str, api_port: int, worker_address: str,
                     master_port: int = 29400) -> List[ChildSpec]:
    """The two members of a single-node service: the torchrun worker fleet and the API process."""
    py = sys.executable
    workers = [py, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(master_port),
               "-m", "xorl_b200.server.launcher", "--mode", "worker", "--config", config,
               "--worker-address", worker_address]
    api = [py, "-m", "xorl_b200.server.launcher", "--mode", "connect", "--config", config,
           "--api-host", api_host, "--api-port", str(api_port), "--worker-address", worker_address]
    connect = worker_address.replace("*", "127.0.0.1").replace("0.0.0.0", "127.0.0.1")
    return [ChildSpec("workers", workers, ready=zmq_health(connect), alive=None),
            ChildSpec("api", api, ready=http_ready(f"http://127.0.0.1:{api_port}/health"))]
