"""A host-side model of the device barrier over per-rank flag words, small enough to check exhaustively.

The kernels' hand-overs (``csrc/comm.cu``: ``barrier_kernel``; callers in ``ops/fused_comm.py`` and
``parallel/symm_mem.py``) follow one protocol: every rank owns an array of ``n`` 64-bit flags; a barrier with epoch
``e`` stores ``e`` into slot ``my_rank`` of every rank's array, then waits until every slot of its own array is
``>= e``; epochs only grow; a wait that runs out of its clock budget sets a status word and lets the kernel return.
An exchange through the symmetric heap is bracketed by two such barriers: one after the writes ("data ready"), one
after the reads ("buffers free").

:func:`explore` walks every interleaving of a few ranks running a few such exchanges (sequentially consistent memory:
the kernels put ``__threadfence_system`` around the flag accesses) and reports violations of the two properties the
callers rely on:

* a rank that passed the "data ready" barrier of exchange ``k`` reads version ``k`` of every peer's buffer, never an
  older or a newer one;
* no interleaving deadlocks; with a rank that never arrives, every waiting rank leaves through the timeout with its
  status word set, and any stale read it makes afterwards is one the status word has already announced.

The reference has no counterpart (all its collectives are library calls); this exists because a protocol of flags and
epochs is easy to get subtly wrong and costs nothing to check on the host.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class Program:
    """What every rank runs: ``exchanges`` rounds of write -> barrier -> read all peers -> (barrier) -> next."""
    ranks: int
    exchanges: int
    second_barrier: bool = True          # the "buffers free" barrier after the reads
    absent: Optional[int] = None         # a rank that never starts (its peers must time out, not hang)
    spurious_timeouts: bool = False      # any blocked wait may give up at any moment (a peer that is only slow)


def _ops(p: Program, rank: int) -> List[Tuple]:
    """The rank's straight-line program as atomic steps."""
    ops: List[Tuple] = []
    epoch = 0
    for k in range(1, p.exchanges + 1):
        ops.append(("write", k))                               # own buffer <- version k
        epoch += 1
        ops += [("publish", epoch, t) for t in range(p.ranks)]
        ops += [("wait", epoch, t) for t in range(p.ranks)]
        ops += [("read", k, t) for t in range(p.ranks) if t != rank]
        if p.second_barrier:
            epoch += 1
            ops += [("publish", epoch, t) for t in range(p.ranks)]
            ops += [("wait", epoch, t) for t in range(p.ranks)]
    return ops


@dataclass
class Result:
    states: int
    violations: List[str]
    timeouts: int                         # interleavings' wait steps that had to leave through the timeout


def explore(p: Program, max_states: int = 2_000_000) -> Result:
    """Depth-first over all interleavings with memoisation on the global state."""
    n = p.ranks
    progs = [_ops(p, r) for r in range(n)]
    violations: List[str] = []
    seen = set()
    timeouts = 0
    # state: pcs, flags[r][s], data[r], status[r]
    start = (tuple(len(progs[r]) if r == p.absent else 0 for r in range(n)), tuple((0,) * n for _ in range(n)), (0,) * n,
             (False,) * n)
    stack = [start]
    while stack:
        state = stack.pop()
        if state in seen:
            continue
        seen.add(state)
        if len(seen) > max_states:
            violations.append("state space larger than the limit")
            break
        pcs, flags, data, status = state
        enabled = []
        blocked = []
        for r in range(n):
            if pcs[r] >= len(progs[r]):
                continue
            op = progs[r][pcs[r]]
            if op[0] == "wait" and flags[r][op[2]] < op[1]:
                blocked.append(r)
            else:
                enabled.append(r)
        if p.spurious_timeouts:
            for r in blocked:                                   # the clock budget may run out while the peer is only slow
                st = list(status)
                st[r] = True
                pc = list(pcs)
                pc[r] += 1
                stack.append((tuple(pc), flags, data, tuple(st)))
        if not enabled:
            if not blocked:
                continue                                        # every rank finished
            if p.spurious_timeouts:
                continue                                        # the timeout transitions above cover it
            # nothing can move: on the device the clock budget runs out; every blocked wait leaves with its status set
            if p.absent is None:
                violations.append(f"deadlock at pcs {pcs}")
                continue
            timeouts += 1
            r = blocked[0]
            st = list(status)
            st[r] = True
            pc = list(pcs)
            pc[r] += 1
            stack.append((tuple(pc), flags, data, tuple(st)))
            continue
        for r in enabled:
            op = progs[r][pcs[r]]
            fl, da = flags, data
            if op[0] == "write":
                d = list(data)
                d[r] = op[1]
                da = tuple(d)
            elif op[0] == "publish":
                f = [list(row) for row in flags]
                f[op[2]][r] = max(f[op[2]][r], op[1])
                fl = tuple(tuple(row) for row in f)
            elif op[0] == "read":
                got = data[op[2]]
                # a stale read is acceptable only if a status word already announces the broken hand-over: the reader's own
                # (it gave up on a wait), or with spurious timeouts any rank's (the per-step check reduces them over ranks)
                announced = status[r] or (p.spurious_timeouts and any(status))
                if got != op[1] and not announced:
                    violations.append(f"rank {r} read version {got} of rank {op[2]}'s buffer in exchange {op[1]}")
            pc = list(pcs)
            pc[r] += 1
            stack.append((tuple(pc), fl, da, status))
    return Result(states=len(seen), violations=sorted(set(violations)), timeouts=timeouts)


def summary(results: Dict[str, Result]) -> str:
    return "\n".join(f"{name}: {r.states} states, {len(r.violations)} violations, {r.timeouts} timeouts" for name, r in results.items())
