"""Tick-level model of the deadlock-free daemon: bounded waits + preemption.

The reference's simulator only *counts* how often the baseline execution
models deadlock (simulator/simulator.py:599-648); it has no model of its own
remedy.  This module adds one: every GPU runs a daemon that owns a task queue
of submitted collectives and executes each as the step program the device
engine uses

    post-arrival -> wait-all-arrived -> move data -> post-done -> wait-all-done

where the two waits are *bounded*: after ``spin_budget`` unsuccessful polls
the daemon parks the collective (its cursor is two integers) and visits the
next entry of its queue — the behaviour of the reference's ``waitPeer`` budget
(src/collectives_ofccl/device/ofccl_prims_simple.h:118-140) and task-queue
traversal (src/collectives_ofccl/device/enqueue_ofccl_dev.cu:922-1023).  With
``preemptive=False`` the same machine models a stream-ordered library: a wait
never gives up, so incompatible issue orders hang, which the model reports
together with the wait-for cycle that explains it.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from .waitgraph import build_fifo_wait_for_graph, find_cycle

# phases of one collective on one GPU
P_NEW, P_ARRIVE_WAIT, P_DATA, P_DONE_WAIT, P_FINISHED = -1, 0, 1, 2, 3


@dataclass
class CollSpec:
    coll_id: int
    kind: str                  # "allreduce" | "allgather" | "reducescatter" | "broadcast" | "reduce"
    nbytes: int
    members: Sequence[int]

    def wire_bytes(self) -> int:
        """Bytes one GPU moves over the fabric for the direct (switch) schedules."""
        n = len(self.members)
        if n <= 1:
            return 0
        if self.kind == "allreduce":
            return 2 * self.nbytes * (n - 1) // n
        if self.kind in ("allgather", "reducescatter"):
            return self.nbytes * (n - 1)
        return self.nbytes


@dataclass
class DaemonParams:
    preemptive: bool = True
    spin_budget: int = 80            # polls before a wait gives up (reference BASE_CTX_SWITCH_THRESHOLD)
    head_tries: int = 5              # budget multiplier for the queue head (reference NUM_TRY_TASKQ_HEAD)
    tick_us: float = 0.25            # duration of one poll
    ctx_switch_ticks: int = 4        # cost of parking one collective and loading another
    link_gbs: float = 770.0          # per-direction fabric bandwidth per GPU
    submit_gap_ticks: int = 8        # host time between two submissions of one GPU
    max_ticks: int = 50_000_000


@dataclass
class DaemonResult:
    completed: bool
    ticks: int
    time_us: float
    ctx_switches: int
    completion_order: Dict[int, List[int]]
    stalled_colls: Dict[int, List[int]] = field(default_factory=dict)
    fifo_cycle: Optional[list] = None      # cycle among collectives under the in-order model, if any


class _Gpu:
    def __init__(self, gid: int, order: Sequence[int]) -> None:
        self.gid = gid
        self.to_submit = list(order)
        self.queue: List[int] = []           # active collectives, head first
        self.cur = 0                         # index in queue being visited
        self.spins = 0
        self.busy = 0                        # remaining ticks of data movement / ctx switch
        self.phase: Dict[int, int] = {}
        self.next_submit_tick = 0
        self.done_order: List[int] = []
        self.switches = 0
        self.tries = 0


def simulate_daemon(colls: Sequence[CollSpec], issue_order: Dict[int, Sequence[int]],
                    params: Optional[DaemonParams] = None) -> DaemonResult:
    """Run every GPU's daemon until all collectives completed (or nothing can
    ever progress).  ``issue_order[g]`` is the order GPU ``g`` submits in."""
    p = params or DaemonParams()
    spec = {c.coll_id: c for c in colls}
    gpus = {g: _Gpu(g, order) for g, order in issue_order.items()}
    arrived = {c.coll_id: set() for c in colls}     # GPUs that posted their arrival flag
    finished = {c.coll_id: set() for c in colls}    # GPUs that posted their done flag
    total = sum(len(o) for o in issue_order.values())
    completed = 0
    tick = 0
    idle_streak = 0
    fifo_cycle = find_cycle(build_fifo_wait_for_graph(issue_order))

    def data_ticks(c: CollSpec) -> int:
        us = c.wire_bytes() / (p.link_gbs * 1e3)     # bytes / (GB/s) -> us
        return max(1, int(us / p.tick_us))

    while completed < total and tick < p.max_ticks:
        tick += 1
        any_progress = False
        for g in gpus.values():
            # host side: one submission every submit_gap_ticks
            if g.to_submit and tick >= g.next_submit_tick:
                c = g.to_submit.pop(0)
                g.queue.append(c)
                g.phase[c] = P_NEW
                g.next_submit_tick = tick + p.submit_gap_ticks
                any_progress = True
            if g.busy > 0:
                g.busy -= 1
                any_progress = True
                continue
            if not g.queue:
                continue
            if not p.preemptive:
                g.cur = 0                            # in-order: only the head may run
            g.cur %= len(g.queue)
            c = g.queue[g.cur]
            s = spec[c]
            ph = g.phase[c]
            if ph == P_NEW:                          # first visit: post the arrival flag to the peers
                arrived[c].add(g.gid)
                g.phase[c] = ph = P_ARRIVE_WAIT
                any_progress = True
            if ph == P_ARRIVE_WAIT:
                ready = arrived[c] >= set(s.members)
            elif ph == P_DONE_WAIT:
                ready = finished[c] >= set(s.members)
            else:
                ready = True
            if ready:
                any_progress = True
                g.spins = 0
                g.tries = 0
                if ph == P_ARRIVE_WAIT:
                    g.phase[c] = P_DATA
                    g.busy = data_ticks(s)
                elif ph == P_DATA:
                    finished[c].add(g.gid)
                    g.phase[c] = P_DONE_WAIT
                elif ph == P_DONE_WAIT:
                    g.phase[c] = P_FINISHED
                    g.queue.pop(g.cur)
                    g.done_order.append(c)
                    completed += 1
                continue
            # unsuccessful poll
            g.spins += 1
            budget = p.spin_budget * (min(g.tries + 1, p.head_tries) if g.cur == 0 else 1)
            if p.preemptive and g.spins >= budget and len(g.queue) > 1:
                g.spins = 0
                g.tries = g.tries + 1 if g.cur == 0 else 0
                g.cur = (g.cur + 1) % len(g.queue)
                g.busy = p.ctx_switch_ticks
                g.switches += 1
        idle_streak = 0 if any_progress else idle_streak + 1
        # nothing moved for longer than any budget and nobody has work to submit: dead
        if idle_streak > 4 * p.spin_budget * p.head_tries + p.submit_gap_ticks:
            if not any(g.to_submit for g in gpus.values()):
                break

    return DaemonResult(
        completed=completed == total, ticks=tick, time_us=tick * p.tick_us,
        ctx_switches=sum(g.switches for g in gpus.values()),
        completion_order={g.gid: g.done_order for g in gpus.values()},
        stalled_colls={g.gid: list(g.queue) for g in gpus.values() if g.queue},
        fifo_cycle=fifo_cycle)


def run_round_daemon(w, rng: random.Random, params: Optional[DaemonParams] = None,
                     nbytes: int = 4 << 20) -> DaemonResult:
    """One round of a :class:`~dfccl_b200.simulator.model.Workload` under the
    daemon model: every GPU draws its issue order with ``disorder_prob`` and
    the daemons run to completion."""
    from .model import draw_issue_order
    colls = [CollSpec(c, "allreduce", nbytes, w.members(c)) for c in sorted(w.coll_2_group)]
    order = {g: draw_issue_order(w.coll_per_gpu.get(g, ()), w.disorder_prob, rng)
             for g in range(w.gpu_num)}
    return simulate_daemon(colls, order, params)


def baseline_config_1(seed: int = 0, n_ranks: int = 4, n_colls: int = 8,
                      nbytes: int = 4 << 20):
    """The CPU headline workload: ``n_ranks`` ranks, ``n_colls`` collectives
    (alternating allreduce / allgather of ``nbytes`` fp32 data) over groups of
    2 or 4 ranks, each rank issuing its collectives in its own seeded random
    permutation.  Returns ``(colls, issue_order)``."""
    rng = random.Random(seed)
    pairs = [[0, 1], [2, 3], [0, 2], [1, 3]]
    colls: List[CollSpec] = []
    for c in range(n_colls):
        members = list(range(n_ranks)) if c % 2 == 0 else pairs[(c // 2) % len(pairs)]
        members = [m for m in members if m < n_ranks]
        colls.append(CollSpec(c, "allreduce" if c % 4 < 2 else "allgather", nbytes, members))
    order: Dict[int, List[int]] = {}
    for g in range(n_ranks):
        mine = [c.coll_id for c in colls if g in c.members]
        rng.shuffle(mine)
        order[g] = mine
    return colls, order
