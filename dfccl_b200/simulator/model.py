"""Monte-Carlo deadlock models for collectives issued in different orders.

What is modelled (same behaviour as the reference's simulator/simulator.py,
re-written as small data classes driven by one ``random.Random`` instance so
that every run is reproducible from its seed):

* ``Single`` — every communication group owns ONE in-order queue.  Each GPU
  of the group pushes the collective it decided to launch; the group is
  deadlocked as soon as two different collective ids coexist in the queue
  (reference: simulator/simulator.py:200-218).
* ``StreamWithSync`` — a GPU either submits its next collective or, with
  probability ``sync_prob``, issues a stream synchronisation.  A sync with
  submitted-but-undone collectives hangs the GPU until they all finish.  A
  deadlock is a cycle among hung GPUs, found either with the cheap
  set-intersection test (reference :322-343) or with the wait-for graph and a
  cycle detector (reference :345-385); an optional resource limit declares a
  group dead once all its members hold ``resource_limit`` outstanding
  collectives (reference :303-319).
* ``disorder_prob`` — when choosing what to launch next a GPU skips the head
  of its remaining list with this probability, repeatedly (reference :61-81).
* grouping policies ``Megatron`` (tp x dp x pp, reference :434-493) and
  ``Arbitrary`` (explicit member lists, reference :495-522), and the
  round-robin interleave that gives each GPU its expected order
  (reference :535-578).

The daemon-preemption model that runs the same workloads to completion lives
in ``daemon_model.py``.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set, Tuple

from .waitgraph import build_wait_for_graph, find_cycle

SINGLE_MODEL = "Single"
STREAM_WITH_SYNC_MODEL = "StreamWithSync"
DAEMON_MODEL = "Daemon"
MEGATRON_GROUPING_POLICY = "Megatron"
ARBITRARY_GROUPING_POLICY = "Arbitrary"

OK, DEADLOCK = 0, -1


# --------------------------------------------------------------------------- config

@dataclass
class Workload:
    """Static description of one simulated job."""
    gpu_num: int
    gpu_per_group: List[List[int]]
    coll_per_group: List[List[int]]
    total_rounds: int = 100
    disorder_prob: float = 0.0
    sync_prob: float = 0.0
    model: str = STREAM_WITH_SYNC_MODEL
    grouping_policy: str = ARBITRARY_GROUPING_POLICY
    resource_limit: int = -1
    deadlock_test: str = "intersection"       # or "graph"
    seed: Optional[int] = None
    num_process: int = 1
    coll_2_group: Dict[int, int] = field(default_factory=dict)
    coll_per_gpu: Dict[int, List[int]] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not self.coll_2_group:
            for gid, colls in enumerate(self.coll_per_group):
                for c in colls:
                    self.coll_2_group[c] = gid
        if not self.coll_per_gpu:
            self.coll_per_gpu = interleave_expected_order(self.gpu_per_group, self.coll_per_group)

    @property
    def coll_num(self) -> int:
        return len(self.coll_2_group)

    def members(self, coll: int) -> List[int]:
        return self.gpu_per_group[self.coll_2_group[coll]]


def megatron_groups(tp: int, dp: int, pp: int, colls_per_tp: int, colls_per_dp: int
                    ) -> Tuple[int, List[List[int]], List[List[int]]]:
    """GPU groups of a tp x dp x pp job.  Within each pipeline stage there are
    ``dp`` tensor-parallel groups of ``tp`` consecutive GPUs and ``tp``
    data-parallel groups (the transpose); collective ids are handed out
    contiguously, group after group."""
    gpu_per_group: List[List[int]] = []
    coll_per_group: List[List[int]] = []
    next_gpu = next_coll = 0
    for _stage in range(pp):
        tp_groups = []
        for _ in range(dp):
            members = list(range(next_gpu, next_gpu + tp))
            next_gpu += tp
            tp_groups.append(members)
            gpu_per_group.append(members)
            coll_per_group.append(list(range(next_coll, next_coll + colls_per_tp)))
            next_coll += colls_per_tp
        for k in range(tp):
            gpu_per_group.append([grp[k] for grp in tp_groups])
            coll_per_group.append(list(range(next_coll, next_coll + colls_per_dp)))
            next_coll += colls_per_dp
    return tp * dp * pp, gpu_per_group, coll_per_group


def interleave_expected_order(gpu_per_group: Sequence[Sequence[int]],
                              coll_per_group: Sequence[Sequence[int]]) -> Dict[int, List[int]]:
    """Expected (program) order of each GPU: round-robin over the groups it
    belongs to, one collective of each per turn."""
    lists: Dict[int, List[Sequence[int]]] = {}
    for members, colls in zip(gpu_per_group, coll_per_group):
        for g in members:
            lists.setdefault(g, []).append(colls)
    out: Dict[int, List[int]] = {}
    for g, per_group in lists.items():
        depth = max(len(l) for l in per_group)
        out[g] = [l[i] for i in range(depth) for l in per_group if i < len(l)]
    return out


def parse_config(cfg: dict) -> Workload:
    """Build a :class:`Workload` from the reference's JSON schema
    (simulator/arbitrary_example.json, simulator/megatron_example.json) plus
    the optional keys ``seed`` and ``deadlock_test``."""
    policy = cfg["grouping_policy"]
    if policy == MEGATRON_GROUPING_POLICY:
        gpu_num, gpg, cpg = megatron_groups(
            cfg["tp_group_size"], cfg["dp_group_size"], cfg["pp_group_size"],
            cfg["coll_cnt_per_tp_group"], cfg["coll_cnt_per_dp_group"])
    elif policy == ARBITRARY_GROUPING_POLICY:
        gpu_num = cfg["gpu_num"]
        gpg = [list(m) for m in cfg["gpu_per_group"]]
        if len(gpg) != cfg["group_num"]:
            raise ValueError("group_num does not match gpu_per_group")
        used = set().union(*map(set, gpg))
        if used != set(range(gpu_num)):
            raise ValueError(f"groups must cover GPUs 0..{gpu_num - 1} exactly, got {sorted(used)}")
        counts = cfg["coll_cnt_per_group"]
        if len(counts) != len(gpg):
            raise ValueError("coll_cnt_per_group does not match gpu_per_group")
        cpg, nxt = [], 0
        for n in counts:
            cpg.append(list(range(nxt, nxt + n)))
            nxt += n
    else:
        raise ValueError(f"unknown grouping_policy {policy!r}")
    seed = cfg.get("seed")
    if seed is None and cfg.get("fix_seed", 0) == 1:
        seed = 2023
    return Workload(
        gpu_num=gpu_num, gpu_per_group=gpg, coll_per_group=cpg,
        total_rounds=cfg.get("total_rounds", 100),
        disorder_prob=cfg.get("disorder_prob", 0.0),
        sync_prob=cfg.get("sync_prob", 0.0),
        model=cfg.get("model", STREAM_WITH_SYNC_MODEL),
        grouping_policy=policy,
        resource_limit=cfg.get("resource_limit", -1),
        deadlock_test=cfg.get("deadlock_test", "intersection"),
        seed=seed, num_process=cfg.get("num_process", 1))


# --------------------------------------------------------------------------- issue order

def pick_next(remaining: List[int], disorder_prob: float, rng: random.Random) -> int:
    """Pop and return the collective a GPU launches next.  Starting at the
    head of ``remaining`` each candidate is skipped with ``disorder_prob``;
    the last one is always taken."""
    i = 0
    while i < len(remaining) - 1 and rng.random() < disorder_prob:
        i += 1
    return remaining.pop(i)


def draw_issue_order(expected: Sequence[int], disorder_prob: float, rng: random.Random) -> List[int]:
    rem = list(expected)
    return [pick_next(rem, disorder_prob, rng) for _ in range(len(rem))]


# --------------------------------------------------------------------------- baseline models

class GlobalState:
    """Who has submitted what (StreamWithSync bookkeeping)."""

    def __init__(self, w: Workload) -> None:
        self.w = w
        self.reset()

    def reset(self) -> None:
        w = self.w
        self.submitted_undone: Dict[int, Set[int]] = {g: set() for g in range(w.gpu_num)}
        self.unsubmitted: Dict[int, Set[int]] = {g: set(w.coll_per_gpu.get(g, ())) for g in range(w.gpu_num)}
        self.hung: Set[int] = set()
        self.pending: Dict[int, int] = {c: len(w.members(c)) for c in w.coll_2_group}

    def submit(self, gpu: int, coll: int) -> None:
        self.submitted_undone[gpu].add(coll)
        self.unsubmitted[gpu].discard(coll)
        self.pending[coll] -= 1
        if self.pending[coll] == 0:                  # everybody is in: it runs and completes
            for g in self.w.members(coll):
                self.submitted_undone[g].discard(coll)
            self.hung = {g for g in self.hung if self.submitted_undone[g]}

    def sync(self, gpu: int) -> bool:
        """Stream-sync on ``gpu``; True if the GPU hangs."""
        if self.submitted_undone[gpu]:
            self.hung.add(gpu)
            return True
        return False

    def resource_deadlock(self) -> bool:
        lim = self.w.resource_limit
        if lim <= 0:
            return False
        return any(all(len(self.submitted_undone[g]) >= lim for g in members)
                   for members in self.w.gpu_per_group)

    def deadlock_by_intersection(self, new_hung: int) -> bool:
        if len(self.hung) < 2:
            return False
        s_new, u_new = self.submitted_undone[new_hung], self.unsubmitted[new_hung]
        s_oth: Set[int] = set()
        u_oth: Set[int] = set()
        for g in self.hung:
            if g != new_hung:
                s_oth |= self.submitted_undone[g]
                u_oth |= self.unsubmitted[g]
        return bool(s_new & u_oth) and bool(u_new & s_oth)

    def deadlock_by_graph(self) -> Optional[list]:
        if len(self.hung) < 2:
            return None
        return find_cycle(build_wait_for_graph(self.hung, self.submitted_undone, self.unsubmitted))


@dataclass
class RoundResult:
    deadlock: bool
    reason: str = ""
    cycle: Optional[list] = None


def run_round_single(w: Workload, rng: random.Random) -> RoundResult:
    """One round of the ``Single`` model."""
    remaining = {g: list(w.coll_per_gpu.get(g, ())) for g in range(w.gpu_num)}
    queue: Dict[int, List[int]] = {gid: [] for gid in range(len(w.gpu_per_group))}
    in_queue: Dict[int, Set[int]] = {gid: set() for gid in range(len(w.gpu_per_group))}
    while any(remaining.values()):
        moved = False
        for g in range(w.gpu_num):
            if not remaining[g]:
                continue
            # peek the decision, but only commit if the GPU may push to that group now
            save = list(remaining[g])
            c = pick_next(remaining[g], w.disorder_prob, rng)
            gid = w.coll_2_group[c]
            if g in in_queue[gid]:
                remaining[g] = save          # its previous push has not executed yet
                continue
            moved = True
            queue[gid].append(c)
            in_queue[gid].add(g)
            if len(set(queue[gid])) > 1:
                return RoundResult(True, f"group {gid} queue holds {sorted(set(queue[gid]))}")
            if len(queue[gid]) == len(w.gpu_per_group[gid]):
                queue[gid].clear()
                in_queue[gid].clear()
        if not moved:
            return RoundResult(True, "no GPU can push")
    return RoundResult(False)


def run_round_stream_with_sync(w: Workload, rng: random.Random) -> RoundResult:
    """One round of the ``StreamWithSync`` model."""
    st = GlobalState(w)
    remaining = {g: list(w.coll_per_gpu.get(g, ())) for g in range(w.gpu_num)}
    while any(remaining.values()):
        progressed = False
        for g in range(w.gpu_num):
            if not remaining[g] or g in st.hung:
                continue
            progressed = True
            if rng.random() < w.sync_prob:
                if st.sync(g):
                    if w.deadlock_test == "graph":
                        cyc = st.deadlock_by_graph()
                        if cyc:
                            return RoundResult(True, "wait-for cycle", cyc)
                    elif st.deadlock_by_intersection(g):
                        return RoundResult(True, "hung sets intersect")
            else:
                st.submit(g, pick_next(remaining[g], w.disorder_prob, rng))
                if st.resource_deadlock():
                    return RoundResult(True, "resource limit")
        if not progressed:                   # everybody with work left is hung
            cyc = st.deadlock_by_graph()
            return RoundResult(True, "all runnable GPUs hung", cyc)
    return RoundResult(False)


def run_rounds(w: Workload, rounds: Optional[int] = None, seed: Optional[int] = None) -> Tuple[int, int]:
    """Run ``rounds`` rounds of ``w.model``; returns ``(deadlocked, rounds)``."""
    from .daemon_model import run_round_daemon
    rng = random.Random(w.seed if seed is None else seed)
    n = w.total_rounds if rounds is None else rounds
    bad = 0
    for _ in range(n):
        if w.model == SINGLE_MODEL:
            r = run_round_single(w, rng)
        elif w.model == STREAM_WITH_SYNC_MODEL:
            r = run_round_stream_with_sync(w, rng)
        elif w.model == DAEMON_MODEL:
            r = RoundResult(not run_round_daemon(w, rng).completed)
        else:
            raise ValueError(f"unknown model {w.model!r}")
        bad += r.deadlock
    return bad, n
