"""Pipeline schedules as explicit per-rank action lists.

An action is ``(op, microbatch, chunk)`` with ``op`` in
  F  forward of one model chunk          B  full backward (input + weight gradients)
  I  backward for inputs only            W  deferred weight-gradient work of (microbatch, chunk)
``chunk`` is the index of the local model chunk (virtual stage) on that rank.  Communication is
implied: a chunk's F receives from the previous global stage and sends to the next, B/I the other
way round.  Six schedules, as in the reference (src/xorl/distributed/pipeline_parallel.py:107-130):
gpipe, 1f1b, interleaved1f1b, interleavedzerobubble (loop placement: global stage g lives on rank
g % P) and zbvzerobubble, dualpipev (V placement: rank r holds stages r and 2P-1-r).

The generators only decide *order*; ``simulate`` checks an order for dead-lock freedom and gives
the bubble fraction for unit costs (cf. src/xorl/distributed/pp_profiling.py).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

Action = Tuple[str, int, int]
SCHEDULES = ("gpipe", "1f1b", "interleaved1f1b", "interleavedzerobubble", "zbvzerobubble", "dualpipev")


def placement(schedule: str) -> str:
    return "v" if schedule in ("zbvzerobubble", "dualpipev") else "loop"


def num_chunks(schedule: str, virtual_stages: int) -> int:
    if placement(schedule) == "v":
        return 2
    if schedule in ("gpipe", "1f1b"):
        return 1
    return max(2, virtual_stages)


def global_stage(rank: int, chunk: int, pp: int, schedule: str) -> int:
    if placement(schedule) == "v":
        return rank if chunk == 0 else 2 * pp - 1 - rank
    return chunk * pp + rank


def stage_owner(stage: int, pp: int, schedule: str) -> Tuple[int, int]:
    """global stage -> (rank, local chunk)."""
    if placement(schedule) == "v":
        return (stage, 0) if stage < pp else (2 * pp - 1 - stage, 1)
    return stage % pp, stage // pp


# --------------------------------------------------------------------------------------------
def _gpipe(rank, pp, n_mb, chunks):
    return [("F", m, 0) for m in range(n_mb)] + [("B", m, 0) for m in range(n_mb)]


def _1f1b(rank, pp, n_mb, chunks):
    warm = min(pp - 1 - rank, n_mb)
    acts: List[Action] = [("F", m, 0) for m in range(warm)]
    f, b = warm, 0
    while f < n_mb:
        acts.append(("F", f, 0)); f += 1
        acts.append(("B", b, 0)); b += 1
    while b < n_mb:
        acts.append(("B", b, 0)); b += 1
    return acts


def _interleaved(rank, pp, n_mb, chunks, zero_bubble=False):
    """Megatron-style interleaved 1F1B: micro-batches advance in groups of ``pp`` through the local
    chunks; with ``zero_bubble`` the backward is split and W work fills the tail."""
    total = n_mb * chunks

    def f_item(i):  # i-th forward on this rank -> (mb, chunk)
        grp, pos = divmod(i, pp * chunks)
        return grp * pp + pos % pp, pos // pp

    def b_item(i):
        grp, pos = divmod(i, pp * chunks)
        return grp * pp + pos % pp, chunks - 1 - pos // pp

    valid_f = [f_item(i) for i in range(total + pp * chunks) if f_item(i)[0] < n_mb][:total]
    valid_b = [b_item(i) for i in range(total + pp * chunks) if b_item(i)[0] < n_mb][:total]
    warm = min((pp - rank - 1) * 2 + (chunks - 1) * pp, total)
    acts: List[Action] = [("F",) + valid_f[i] for i in range(warm)]
    fi, bi = warm, 0
    bop = "I" if zero_bubble else "B"
    pending_w: List[Tuple[int, int]] = []
    while fi < total:
        acts.append(("F",) + valid_f[fi]); fi += 1
        acts.append((bop,) + valid_b[bi])
        if zero_bubble:
            pending_w.append(valid_b[bi])
            if len(pending_w) > rank:      # later ranks can afford to defer more weight work
                acts.append(("W",) + pending_w.pop(0))
        bi += 1
    while bi < total:
        acts.append((bop,) + valid_b[bi])
        if zero_bubble:
            pending_w.append(valid_b[bi])
            acts.append(("W",) + pending_w.pop(0))
        bi += 1
    for w in pending_w:
        acts.append(("W",) + w)
    return acts


def _greedy_v(pp: int, n_mb: int, dual: bool) -> List[List[Action]]:
    """List scheduling for the V placement with split backward.  Every rank, whenever it is free,
    runs the ready action of highest priority: input-gradient work first (it unblocks the
    neighbour), then a forward while the number of micro-batches in flight on that rank is below
    its cap, then deferred weight-gradient work; a rank with nothing ready waits for its next
    dependency.  ZB-V caps in-flight forwards at 2P per rank, the DualPipe-V flavour at 2P+1 and
    prefers alternating forward / backward once both are ready."""
    chunks, n_stages = 2, 2 * pp
    cost = {"F": 1.0, "I": 1.0, "W": 1.0}
    done: Dict[Tuple[str, int, int], float] = {}
    clock = [0.0] * pp
    acts: List[List[Action]] = [[] for _ in range(pp)]
    nf = [[0, 0] for _ in range(pp)]       # next forward micro-batch per chunk
    ni = [[0, 0] for _ in range(pp)]       # next input-backward micro-batch per chunk
    pend_w: List[List[Tuple[int, int]]] = [[] for _ in range(pp)]
    last_op = [""] * pp
    cap = 2 * pp + (1 if dual else 0)
    total = pp * n_mb * chunks * 3
    emitted = 0

    def stage(r, c):
        return r if c == 0 else 2 * pp - 1 - r

    def ready_time(r, op, m, c):
        g = stage(r, c)
        deps = []
        if op == "F":
            if g > 0:
                deps.append(("F", m, g - 1))
        elif op == "I":
            deps.append(("F", m, g))
            if g < n_stages - 1:
                deps.append(("I", m, g + 1))
        if not all(d in done for d in deps):
            return None
        return max([0.0] + [done[d] for d in deps])

    guard = 0
    while emitted < total:
        guard += 1
        if guard > 20 * total + 1000:
            raise RuntimeError("greedy V scheduler did not converge")
        # the rank that is free earliest acts next
        order = sorted(range(pp), key=lambda r: clock[r])
        acted = False
        for r in order:
            cands = []
            for c in (1, 0):
                if ni[r][c] < n_mb:
                    t = ready_time(r, "I", ni[r][c], c)
                    if t is not None:
                        cands.append((t, 0 if not (dual and last_op[r] == "I") else 2, "I", ni[r][c], c))
            inflight = (nf[r][0] - ni[r][0]) + (nf[r][1] - ni[r][1])
            for c in (1, 0):
                if nf[r][c] < n_mb and (c == 1 or inflight < cap):
                    t = ready_time(r, "F", nf[r][c], c)
                    if t is not None:
                        cands.append((t, 1, "F", nf[r][c], c))
            now = [x for x in cands if x[0] <= clock[r] + 1e-9]
            if now:
                _, _, op, m, c = min(now, key=lambda x: (x[1], x[0]))
            elif pend_w[r]:
                m, c = pend_w[r].pop(0)
                op = "W"
            elif cands:
                t, _, op, m, c = min(cands, key=lambda x: (x[0], x[1]))
                clock[r] = t
            else:
                continue
            end = clock[r] + cost[op]
            if op == "F":
                nf[r][c] += 1
                done[("F", m, stage(r, c))] = end
            elif op == "I":
                ni[r][c] += 1
                done[("I", m, stage(r, c))] = end
                pend_w[r].append((m, c))
            acts[r].append((op, m, c))
            last_op[r] = op
            clock[r] = end
            emitted += 1
            acted = True
            break
        if not acted:
            raise RuntimeError("greedy V scheduler stalled")
    return acts


def build_schedule(schedule: str, pp: int, n_mb: int, virtual_stages: int = 1) -> List[List[Action]]:
    """Per-rank action lists for one optimizer step."""
    s = schedule.lower()
    if s not in SCHEDULES:
        raise ValueError(f"unknown pipeline schedule {schedule!r}; choose from {SCHEDULES}")
    chunks = num_chunks(s, virtual_stages)
    if placement(s) == "v":
        return _greedy_v(pp, n_mb, dual=(s == "dualpipev"))
    out = []
    for r in range(pp):
        if s == "gpipe":
            a = _gpipe(r, pp, n_mb, chunks)
        elif s == "1f1b":
            a = _1f1b(r, pp, n_mb, chunks)
        elif s == "interleaved1f1b":
            a = _interleaved(r, pp, n_mb, chunks, False)
        else:
            a = _interleaved(r, pp, n_mb, chunks, True)
        out.append(a)
    return out


# --------------------------------------------------------------------------------------------
def simulate(actions: List[List[Action]], schedule: str, pp: int, n_mb: int, virtual_stages: int = 1,
             cost: Optional[Dict[str, float]] = None) -> Dict[str, float]:
    """Event simulation with blocking receives.  Raises RuntimeError on dead-lock or on a missing /
    duplicated action; returns makespan, per-rank busy time and the bubble fraction."""
    s = schedule.lower()
    chunks = num_chunks(s, virtual_stages)
    n_stages = pp * chunks
    cost = cost or {"F": 1.0, "B": 2.0, "I": 1.0, "W": 1.0}
    done: Dict[Tuple[str, int, int], float] = {}    # (op, mb, global stage) -> finish time
    ptr = [0] * pp
    clock = [0.0] * pp
    busy = [0.0] * pp
    progressed = True
    while progressed:
        progressed = False
        for r in range(pp):
            while ptr[r] < len(actions[r]):
                op, m, c = actions[r][ptr[r]]
                g = global_stage(r, c, pp, s)
                deps = []
                if op == "F":
                    if g > 0:
                        deps.append(("F", m, g - 1))
                elif op in ("B", "I"):
                    deps.append(("F", m, g))
                    if g < n_stages - 1:
                        deps.append(("BI", m, g + 1))
                else:
                    deps.append(("BI", m, g))
                if not all(d in done for d in deps):
                    break
                start = max([clock[r]] + [done[d] for d in deps])
                end = start + cost[op]
                key = ("BI", m, g) if op in ("B", "I") else (op, m, g)
                if key in done:
                    raise RuntimeError(f"duplicate action {actions[r][ptr[r]]} on rank {r}")
                done[key] = end
                if op == "B":
                    done[("W", m, g)] = end
                clock[r] = end
                busy[r] += cost[op]
                ptr[r] += 1
                progressed = True
    if any(ptr[r] < len(actions[r]) for r in range(pp)):
        stuck = {r: actions[r][ptr[r]] for r in range(pp) if ptr[r] < len(actions[r])}
        raise RuntimeError(f"schedule dead-locks at {stuck}")
    for m in range(n_mb):
        for g in range(n_stages):
            for k in (("F", m, g), ("BI", m, g), ("W", m, g)):
                if k not in done:
                    raise RuntimeError(f"schedule never runs {k}")
    makespan = max(clock)
    return {"makespan": makespan, "busy": busy,
            "bubble_fraction": 1.0 - sum(busy) / (pp * makespan)}


def analytic_bubble_fraction(schedule: str, pp: int, n_mb: int, virtual_stages: int = 1) -> float:
    """Closed-form estimates: (P-1)/(M+P-1) for gpipe/1f1b, divided by the number of chunks when
    interleaved; zero-bubble variants approach 0 as weight work fills the tail."""
    s = schedule.lower()
    chunks = num_chunks(s, virtual_stages)
    base = (pp - 1) / (n_mb + pp - 1)
    if s in ("gpipe", "1f1b"):
        return base
    if s == "interleaved1f1b":
        return (pp - 1) / (chunks * n_mb + pp - 1)
    return max(0.0, (pp - 1) / (3 * chunks * n_mb + pp - 1))


def estimate_p2p_bytes_per_step(pp: int, n_mb: int, tokens: int, hidden: int, chunks: int = 1,
                                bytes_per_el: int = 2, tensors: int = 2) -> int:
    """Activations forward + gradients backward over every stage boundary."""
    boundaries = pp * chunks - 1
    return 2 * boundaries * n_mb * tokens * hidden * bytes_per_el * tensors
