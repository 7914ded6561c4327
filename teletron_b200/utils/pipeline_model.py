"""A host-side model of the one-pass attention backward's warp-role pipeline (``csrc/attn_bwd_tcgen05.cu``,
``attn_bwd_fused_kernel``), small enough to walk every interleaving of its roles for a few query chunks.

The kernel has five kinds of actors that only meet at mbarriers: the TMA-issuing thread, the MMA-issuing thread, the
softmax warps (modelled as two groups of eight: column groups 0, 1 and 2, 3), the thread that issues and awaits the dQ
reductions, and the two asynchronous units they feed - the tensor core, which executes what it is given in issue order
and signals through commits, and the TMA unit, whose pending copies may complete in any order.  Buffers are reused
aggressively: T1 holds S, T2 holds dP, then bf16 P / dS, then dQ; the dS tile and each chunk's dO slot double as staging
buffers for the reductions.  The model gives every buffer a content tag and the set of readers that still need it, and
reports

* a read that finds something else than the tag it expects,
* a write over a content that still has readers,
* a state in which nothing can move before every role has finished (a deadlock; on the device a bounded wait would
  expire and the kernel would report a timeout).

An mbarrier is modelled with its arrival count and a phase counter; ``wait(parity)`` passes exactly when the
barrier's current phase has the other parity, as ``mbarrier.try_wait.parity`` does, so a waiter that could fall two
phases behind shows up as a deadlock.

The programs below are transcribed from the kernel; a change of the kernel's synchronisation has to be mirrored here.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

RING = 2            # slots of the streamed Q and dO rings


@dataclass(frozen=True)
class Variant:
    """Switches that re-introduce hazards the kernel's synchronisation exists to prevent (to show the model sees them)."""
    wait_stage_done: bool = True        # softmax warps wait for the staged dQ half to leave the dS tile before storing dS
    release_slot_after_reduce: bool = True   # the dO slot is handed back only after the staged half has been read
    wait_dq_read: bool = True           # dP(c+1) is issued only after dQ(c) has been read out of T2


# ------------------------------------------------------------------------------------------------ effects of async ops
# each effect: reads = [(buffer, expected tag, reader id)], writes = [(buffer, tag, readers)], arrives = [(barrier, weight)]

def _tc_effect(op: Tuple, n: int):
    kind, c = op[0], op[1]
    if kind == "commit":
        return ([], [], [(op[1], 1)])
    s = c % RING
    if kind == "S":
        return ([("KV", "KV", None), (f"q{s}", ("Q", c), "S")], [("T1a", ("S", c), {"smA"}), ("T1b", ("S", c), {"smB"})], [])
    if kind == "dP":
        return ([("KV", "KV", None), (f"do{s}", ("dO", c), "dP")], [("T2a", ("dP", c), {"smA"}), ("T2b", ("dP", c), {"smB"})], [])
    if kind == "dK":
        return ([("T2a", ("PdS", c), "dK"), ("T2b", ("PdS", c), "dK"), (f"q{s}", ("Q", c), "dK")], [], [])
    if kind == "dV":
        return ([("T2a", ("PdS", c), "dV"), ("T2b", ("PdS", c), "dV"), (f"do{s}", ("dO", c), "dV")], [], [])
    if kind == "dQ":
        return ([("dsA", ("dS", c), "dQ"), ("dsB", ("dS", c), "dQ"), ("KV", "KV", None)],
                [("T2a", ("dQ", c), {"smA"}), ("T2b", ("dQ", c), {"smB"})], [])
    raise ValueError(op)


def _tma_effect(op: Tuple):
    kind, c = op[0], op[1]
    s = c % RING if isinstance(c, int) else 0
    if kind == "loadKV":
        return ([], [("KV", "KV", set())], [("a_full", 1)])
    if kind == "loadQ":
        return ([], [(f"q{s}", ("Q", c), {"S", "dK"})], [(f"b1_full{s}", 1)])
    if kind == "loadDO":
        return ([], [(f"do{s}", ("dO", c), {"dP", "dV"})], [(f"b2_full{s}", 1)])
    if kind == "redA":
        return ([("dsA", ("stage", c), "redA"), ("dsB", ("stage", c), "redA")], [], [])
    if kind == "redB":
        return ([(f"do{s}", ("stage", c), "redB")], [], [])
    raise ValueError(op)


# ------------------------------------------------------------------------------------------------ the roles' programs

def _producer(n: int) -> List[Tuple]:
    ops: List[Tuple] = [("tma", ("loadKV", 0))]
    for c in range(n):
        s, wpar = c % RING, ((c // RING) & 1) ^ 1
        ops += [("wait", f"b1_empty{s}", wpar), ("tma", ("loadQ", c)), ("wait", f"b2_empty{s}", wpar), ("tma", ("loadDO", c))]
    return ops


def _mma(n: int, v: Variant) -> List[Tuple]:
    ops: List[Tuple] = [("wait", "a_full", 0), ("wait", "b1_full0", 0), ("tc", ("S", 0)), ("tc", ("commit", "s_full")),
                        ("wait", "b2_full0", 0), ("tc", ("dP", 0)), ("tc", ("commit", "dp_full"))]
    for c in range(n):
        par, more = c & 1, c + 1 < n
        s, ns, npar = c % RING, (c + 1) % RING, ((c + 1) // RING) & 1
        ops.append(("wait", "p_ready", par))
        if more:
            ops += [("wait", f"b1_full{ns}", npar), ("tc", ("S", c + 1)), ("tc", ("commit", "s_full"))]
        ops += [("wait", "ds_ready", par), ("tc", ("dK", c)), ("tc", ("commit", f"b1_empty{s}")), ("tc", ("dV", c)),
                ("tc", ("commit", f"b2_empty{s}")), ("tc", ("dQ", c)), ("tc", ("commit", "dq_full"))]
        if more:
            if v.wait_dq_read:
                ops.append(("wait", "dq_read", par))
            ops += [("wait", f"b2_full{ns}", npar), ("tc", ("dP", c + 1)), ("tc", ("commit", "dp_full"))]
    ops.append(("tc", ("commit", "acc_final")))
    return ops


def _softmax(n: int, g: str, v: Variant) -> List[Tuple]:
    """Group ``g`` in {"A", "B"}: eight warps; every arrival of the group counts eight."""
    me, t1, t2, ds = "sm" + g, "T1" + g.lower(), "T2" + g.lower(), "ds" + g

    def p_pass(c):
        return [("wait", "s_full", c & 1), ("read", t1, ("S", c), me), ("arrive", "p_ready", 8)]

    ops: List[Tuple] = p_pass(0)
    for c in range(n):
        par = c & 1
        ops += [("wait", "dp_full", par), ("read", t2, ("dP", c), me), ("write", t2, ("PdS", c), ("dK", "dV"))]
        if c > 0 and v.wait_stage_done:
            ops.append(("wait", "stage_done", (c - 1) & 1))
        ops += [("write", ds, ("dS", c), ("dQ",)), ("arrive", "ds_ready", 8)]
        if c + 1 < n:
            ops += p_pass(c + 1)
        ops += [("wait", "dq_full", par), ("read", t2, ("dQ", c), me), ("arrive", "dq_read", 8)]
        if g == "A":       # column groups 0, 1 stage in the dS tile (all of it), groups 2, 3 in chunk c's dO slot
            ops += [("write", "dsA", ("stage", c), ("redA",)), ("write", "dsB", ("stage", c), ("redA",)), ("arrive", "staged_a", 8)]
        else:
            ops += [("write", f"do{c % RING}", ("stage", c), ("redB",)), ("arrive", "staged_b", 8)]
    ops.append(("wait", "acc_final", 0))
    return ops


def _reducer(n: int, v: Variant) -> List[Tuple]:
    ops: List[Tuple] = []
    for c in range(n):
        par, s = c & 1, c % RING
        ops += [("wait", "staged_a", par), ("tma", ("redA", c)), ("wait", "staged_b", par), ("tma", ("redB", c)),
                ("tma_done", ("redA", c)), ("arrive", "stage_done", 1)]
        if v.release_slot_after_reduce:
            ops.append(("tma_done", ("redB", c)))
        ops.append(("arrive", f"b2_empty{s}", 1))
    return ops


def _barriers() -> Dict[str, int]:
    b = {"a_full": 1, "s_full": 1, "dp_full": 1, "p_ready": 16, "ds_ready": 16, "dq_full": 1, "dq_read": 16, "acc_final": 1,
         "stage_done": 1, "staged_a": 8, "staged_b": 8}
    for s in range(RING):
        b.update({f"b1_full{s}": 1, f"b1_empty{s}": 1, f"b2_full{s}": 1, f"b2_empty{s}": 2})
    return b


@dataclass
class Result:
    states: int
    violations: List[str] = field(default_factory=list)


def explore(chunks: int = 3, variant: Variant = Variant(), max_states: int = 3_000_000) -> Result:
    """Every interleaving of the four thread roles, the in-order tensor core and the any-order TMA unit."""
    n = chunks
    progs = [_producer(n), _mma(n, variant), _softmax(n, "A", variant), _softmax(n, "B", variant), _reducer(n, variant)]
    names = ["producer", "mma", "softmax A", "softmax B", "reducer"]
    counts = _barriers()
    bar_names = sorted(counts)
    bidx = {b: i for i, b in enumerate(bar_names)}
    buf_names = ["KV", "T1a", "T1b", "T2a", "T2b", "dsA", "dsB"] + [f"q{s}" for s in range(RING)] + [f"do{s}" for s in range(RING)]
    fidx = {b: i for i, b in enumerate(buf_names)}
    violations = set()

    def apply(bufs, bars, done, reads, writes, arrives, who):
        bufs = list(bufs)
        for name, expect, reader in reads:
            tag, left = bufs[fidx[name]]
            if tag != expect:
                violations.add(f"{who} read {name} expecting {expect}, found {tag}")
            elif reader is not None:
                bufs[fidx[name]] = (tag, left - {reader})
        for name, tag, readers in writes:
            old, left = bufs[fidx[name]]
            if left:
                violations.add(f"{who} overwrote {name} = {old} while {sorted(left)} had not read it")
            bufs[fidx[name]] = (tag, frozenset(readers))
        bars = list(bars)
        for name, w in arrives:
            pending, phase = bars[bidx[name]]
            pending -= w
            if pending < 0:
                violations.add(f"{who} arrived on {name} beyond its count")
                pending = 0
            if pending == 0:
                pending, phase = counts[name], phase + 1
            bars[bidx[name]] = (pending, phase)
        return tuple(bufs), tuple(bars), done

    start = (tuple(0 for _ in progs), tuple((counts[b], 0) for b in bar_names), tuple((None, frozenset()) for _ in buf_names),
             (), (), frozenset())
    seen = set()
    stack = [start]
    while stack:
        st = stack.pop()
        if st in seen:
            continue
        seen.add(st)
        if len(seen) > max_states:
            violations.add("state space larger than the limit")
            break
        pcs, bars, bufs, tcq, tmaq, done = st
        moved = False
        # thread roles
        for r, prog in enumerate(progs):
            if pcs[r] >= len(prog):
                continue
            op = prog[pcs[r]]
            nb, nbuf, ntc, ntma, nd = bars, bufs, tcq, tmaq, done
            if op[0] == "wait":
                if (bars[bidx[op[1]]][1] & 1) == op[2]:
                    continue
            elif op[0] == "tma_done":
                if op[1] not in done:
                    continue
            elif op[0] == "tc":
                ntc = tcq + (op[1],)
            elif op[0] == "tma":
                ntma = tmaq + (op[1],)
            elif op[0] == "arrive":
                nbuf, nb, nd = apply(bufs, bars, done, [], [], [(op[1], op[2])], names[r])
            elif op[0] == "read":
                nbuf, nb, nd = apply(bufs, bars, done, [(op[1], op[2], op[3])], [], [], names[r])
            elif op[0] == "write":
                nbuf, nb, nd = apply(bufs, bars, done, [], [(op[1], op[2], set(op[3]))], [], names[r])
            moved = True
            npc = pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:]
            stack.append((npc, nb, nbuf, ntc, ntma, nd))
        # tensor core: strictly in issue order
        if tcq:
            reads, writes, arrives = _tc_effect(tcq[0], n)
            nbuf, nb, nd = apply(bufs, bars, done, reads, writes, arrives, f"tensor core {tcq[0]}")
            stack.append((pcs, nb, nbuf, tcq[1:], tmaq, nd))
            moved = True
        # TMA unit: any pending copy may complete next
        for i, op in enumerate(tmaq):
            reads, writes, arrives = _tma_effect(op)
            nbuf, nb, nd = apply(bufs, bars, done, reads, writes, arrives, f"TMA {op}")
            stack.append((pcs, nb, nbuf, tcq, tmaq[:i] + tmaq[i + 1:], done | {op} if op[0].startswith("red") else done))
            moved = True
        if not moved and any(pcs[r] < len(progs[r]) for r in range(len(progs))):
            where = ", ".join(f"{names[r]} at {progs[r][pcs[r]]}" for r in range(len(progs)) if pcs[r] < len(progs[r]))
            violations.add(f"deadlock: {where}")
    return Result(states=len(seen), violations=sorted(violations))
