"""Deadlock simulator: models, cycle detector, daemon-preemption model."""
import json
import random
from pathlib import Path

import pytest

from dfccl_b200 import simulator as sim

CFG = Path(sim.__file__).parent / "configs"


def test_cycle_detector_on_hand_built_graphs():
    assert sim.find_cycle({"a": ["b"], "b": ["c"], "c": []}) is None
    cyc = sim.find_cycle({"a": ["b"], "b": ["c"], "c": ["a"]})
    assert cyc[0] == cyc[-1] and set(cyc) == {"a", "b", "c"}
    assert sim.find_cycle({1: [1]}) == [1, 1]
    # successors that are not keys are sinks; deep chains do not hit the recursion limit
    deep = {i: [i + 1] for i in range(50000)}
    assert sim.find_cycle(deep) is None
    d = sim.RingDetector()
    assert d.detect_ring({"x": ["y"], "y": ["x"]}) and d.cycle is not None


def test_wait_for_graph_of_two_hung_gpus():
    # gpu0 submitted 0 and waits at a sync, gpu1 submitted 1: classic crossed order
    g = sim.build_wait_for_graph({0, 1}, {0: {0}, 1: {1}}, {0: {1}, 1: {0}})
    assert sim.find_cycle(g) is not None
    g = sim.build_wait_for_graph({0, 1}, {0: {0}, 1: {0}}, {0: {1}, 1: {1}})
    assert sim.find_cycle(g) is None


def test_fifo_graph_detects_incompatible_orders():
    assert sim.find_cycle(sim.build_fifo_wait_for_graph({0: [0, 1], 1: [1, 0]})) is not None
    assert sim.find_cycle(sim.build_fifo_wait_for_graph({0: [0, 1, 2], 1: [0, 1, 2]})) is None


def test_megatron_grouping_matches_layout():
    n, gpg, cpg = sim.megatron_groups(2, 2, 2, 3, 2)
    assert n == 8
    assert gpg[:4] == [[0, 1], [2, 3], [0, 2], [1, 3]]
    assert gpg[4:] == [[4, 5], [6, 7], [4, 6], [5, 7]]
    assert cpg[0] == [0, 1, 2] and cpg[2] == [6, 7]
    order = sim.interleave_expected_order(gpg, cpg)
    assert order[0] == [0, 6, 1, 7, 2]


@pytest.mark.parametrize("name", ["arbitrary", "megatron"])
def test_configs_are_deterministic(name):
    cfg = json.loads((CFG / f"{name}.json").read_text())
    a = sim.run_config(cfg, processes=1)
    b = sim.run_config(cfg, processes=1)
    assert a == b and a[1] == cfg["total_rounds"]


def test_no_disorder_means_no_deadlock():
    cfg = json.loads((CFG / "megatron.json").read_text())
    cfg.update(disorder_prob=0.0, sync_prob=0.2, total_rounds=30)
    for model in ("Single", "StreamWithSync", "Daemon"):
        cfg["model"] = model
        bad, total = sim.run_config(cfg, processes=1)
        assert bad == 0 and total == 30


def test_graph_test_agrees_with_intersection_test_on_direction():
    cfg = json.loads((CFG / "arbitrary.json").read_text())
    cfg.update(total_rounds=60, resource_limit=-1)
    inter = sim.run_config(dict(cfg, deadlock_test="intersection"), processes=1)[0]
    graph = sim.run_config(dict(cfg, deadlock_test="graph"), processes=1)[0]
    assert inter > 0 and graph > 0
    # every cycle implies intersecting sets, never the other way round
    assert graph <= inter


def test_multiprocess_runner_sums_rounds():
    cfg = json.loads((CFG / "megatron.json").read_text())
    cfg.update(total_rounds=10, num_process=2)
    bad, total = sim.run_config(cfg)
    assert total == 20 and 0 <= bad <= 20


@pytest.mark.parametrize("seed", range(8))
def test_headline_config_daemon_completes_where_in_order_hangs(seed):
    """4 ranks, 8 collectives (allreduce / allgather, 4 MB fp32, groups of 2 or 4),
    every rank issues in its own seeded permutation."""
    colls, order = sim.baseline_config_1(seed)
    assert len(colls) == 8 and all(c.nbytes == 4 << 20 for c in colls)
    assert {len(c.members) for c in colls} == {2, 4}
    daemon = sim.simulate_daemon(colls, order)
    assert daemon.completed and not daemon.stalled_colls
    assert all(sorted(v) == sorted(order[g]) for g, v in daemon.completion_order.items())
    inorder = sim.simulate_daemon(colls, order, sim.DaemonParams(preemptive=False))
    # the in-order machine hangs exactly when the launch orders contain a cycle
    assert inorder.completed == (daemon.fifo_cycle is None)
    if daemon.fifo_cycle is not None:
        assert daemon.ctx_switches > 0


def test_daemon_model_identical_orders_need_no_preemption():
    colls = [sim.CollSpec(c, "allreduce", 1 << 20, [0, 1, 2, 3]) for c in range(6)]
    order = {g: list(range(6)) for g in range(4)}
    r = sim.simulate_daemon(colls, order, sim.DaemonParams(submit_gap_ticks=0))
    assert r.completed and r.fifo_cycle is None


def test_pick_next_respects_disorder_probability():
    rng = random.Random(1)
    assert sim.draw_issue_order([1, 2, 3, 4], 0.0, rng) == [1, 2, 3, 4]
    shuffled = [sim.draw_issue_order(list(range(10)), 0.5, rng) for _ in range(20)]
    assert any(s != list(range(10)) for s in shuffled)
    assert all(sorted(s) == list(range(10)) for s in shuffled)


def test_cli(tmp_path, capsys):
    p = tmp_path / "c.json"
    cfg = json.loads((CFG / "megatron_daemon.json").read_text())
    cfg["total_rounds"] = 3
    p.write_text(json.dumps(cfg))
    assert sim.main(["-f", str(p)]) == 0
    assert "#Deadlock round / rounds: 0 / 3" in capsys.readouterr().out
