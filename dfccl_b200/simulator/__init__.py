"""Deadlock simulator: baseline Monte-Carlo models, wait-for-graph cycle
detection and the daemon-preemption model (reference: simulator/)."""
from .waitgraph import RingDetector, find_cycle, build_wait_for_graph, build_fifo_wait_for_graph
from .model import (Workload, parse_config, megatron_groups, interleave_expected_order,
                    pick_next, draw_issue_order, run_round_single, run_round_stream_with_sync,
                    run_rounds, GlobalState, SINGLE_MODEL, STREAM_WITH_SYNC_MODEL, DAEMON_MODEL)
from .daemon_model import (CollSpec, DaemonParams, DaemonResult, simulate_daemon,
                           run_round_daemon, baseline_config_1)
from .cli import main, run_config
