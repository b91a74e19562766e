"""Wait-for graphs over (gpu, collective) pairs and cycle detection.

Parity: the reference keeps a recursive DFS with list-based visited/trace sets
(simulator/detect_ring.py:28-81) and builds the graph inline in
simulator/simulator.py:345-373.  Here the graph builder and the detector are
separate, the DFS is iterative with three colours (O(V+E), no recursion limit)
and the detector returns the cycle it found instead of printing it.

Node naming follows the reference so that dumps are comparable:
``"<gpu>-<coll>-S"`` is a collective that ``gpu`` has submitted and that is not
done, ``"<gpu>-<coll>-U"`` one that it has not submitted yet.
"""
from __future__ import annotations

from typing import Dict, Hashable, Iterable, List, Mapping, Optional, Sequence, Set

Graph = Dict[Hashable, List[Hashable]]

WHITE, GREY, BLACK = 0, 1, 2


def find_cycle(graph: Mapping[Hashable, Sequence[Hashable]]) -> Optional[List[Hashable]]:
    """Return one directed cycle as a list of nodes (first == last) or None.

    Successors that are not keys of ``graph`` are treated as sink nodes.
    """
    colour: Dict[Hashable, int] = {}
    for root in graph:
        if colour.get(root, WHITE) != WHITE:
            continue
        # stack of (node, iterator over successors); `path` mirrors the grey chain
        path: List[Hashable] = [root]
        iters = [iter(graph.get(root, ()))]
        colour[root] = GREY
        while iters:
            try:
                nxt = next(iters[-1])
            except StopIteration:
                colour[path.pop()] = BLACK
                iters.pop()
                continue
            c = colour.get(nxt, WHITE)
            if c == GREY:
                i = path.index(nxt)
                return path[i:] + [nxt]
            if c == WHITE:
                colour[nxt] = GREY
                path.append(nxt)
                iters.append(iter(graph.get(nxt, ())))
    return None


class RingDetector:
    """Object form of :func:`find_cycle` with the reference's method name
    (simulator/detect_ring.py:61 ``detect_ring(graph) -> bool``)."""

    def __init__(self) -> None:
        self.cycle: Optional[List[Hashable]] = None

    def reset(self) -> None:
        self.cycle = None

    def detect_ring(self, graph: Mapping[Hashable, Sequence[Hashable]]) -> bool:
        self.cycle = find_cycle(graph)
        return self.cycle is not None


def node(gpu: int, coll: int, submitted: bool) -> str:
    return f"{gpu}-{coll}-{'S' if submitted else 'U'}"


def build_wait_for_graph(
    hung_gpus: Iterable[int],
    submitted_undone: Mapping[int, Set[int]],
    unsubmitted: Mapping[int, Set[int]],
) -> Graph:
    """Wait-for graph among GPUs that are blocked (stream-synchronising).

    Edges (same rule as simulator/simulator.py:345-373 of the reference):

    * ``g-c-S -> h-c-U`` for every other hung GPU ``h`` that has not submitted
      ``c``: the submitted collective cannot finish before ``h`` joins it;
    * ``g-c-U -> g-x-S`` for every submitted-undone ``x`` on the same GPU: a
      hung GPU submits nothing new until everything it submitted is done.

    A cycle in this graph is a deadlock: no member of the cycle can make the
    move another member is waiting for.
    """
    hung = sorted(set(hung_gpus))
    g: Graph = {}
    for gpu in hung:
        for c in sorted(submitted_undone[gpu]):
            edges = g.setdefault(node(gpu, c, True), [])
            for other in hung:
                if other != gpu and c in unsubmitted[other]:
                    edges.append(node(other, c, False))
        for c in sorted(unsubmitted[gpu]):
            g.setdefault(node(gpu, c, False), []).extend(
                node(gpu, x, True) for x in sorted(submitted_undone[gpu])
            )
    return g


def build_fifo_wait_for_graph(issue_order: Mapping[int, Sequence[int]]) -> Graph:
    """Wait-for graph of the *single in-order queue per GPU* execution model
    (what a stream-ordered library does when every rank launches blocking
    collectives in its own order).

    ``issue_order[g]`` is the order in which GPU ``g`` launches its
    collectives.  Nodes are collective ids.  Collective ``c`` cannot start on
    GPU ``g`` before the collective queued just before it on ``g`` has
    finished, and it cannot finish before it has started on every member, so
    ``c -> prev_g(c)`` for every member ``g``.  A cycle means the launch orders
    are incompatible: without preemption the job hangs.
    """
    g: Graph = {}
    for gpu in sorted(issue_order):
        prev = None
        for c in issue_order[gpu]:
            edges = g.setdefault(c, [])
            if prev is not None and prev not in edges:
                edges.append(prev)
            prev = c
    return g
