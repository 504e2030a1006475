"""Self-launching distributed tests: under pytest a test calls ``run_distributed(__file__, n)``
which starts ``torch.distributed.run`` with n CPU (gloo) or GPU (nccl) ranks executing the same
file as ``__main__``."""
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_distributed(script: str, nproc: int, *args: str, timeout: int = 600, env=None) -> str:
    e = dict(os.environ)
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    e.setdefault("OMP_NUM_THREADS", "1")
    e.setdefault("XORL_PROCESS_GROUP_TIMEOUT_MINUTES", "5")
    if env:
        e.update(env)
    # A port found free can be taken by another process before the rendezvous binds it, and a
    # loaded box can miss the store's connect window: such launches fail before any test code
    # runs, so they are retried once on a new port.  Failures of the test itself are not retried.
    transient = ("Address already in use", "EADDRINUSE", "address already in use", "The server socket has failed",
                 "RendezvousConnectionError", "Connection refused", "Connection reset by peer",
                 "failed to connect", "Timed out waiting for clients")
    for attempt in range(2):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), script, *args]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)
        if r.returncode == 0 or attempt == 1 or not any(t in r.stderr for t in transient):
            break
    if r.returncode != 0:
        raise AssertionError(f"distributed run failed ({r.returncode})\nSTDOUT:\n{r.stdout[-4000:]}\n"
                             f"STDERR:\n{r.stderr[-6000:]}")
    return r.stdout
