"""One OS process per rank: TCP bootstrap with a unique id, peer memory across processes
(POSIX shm on the host backend, CUDA IPC on GPUs), daemon and stream-ordered interfaces."""
import pytest

import mp_worker


@pytest.mark.parametrize("world", [2, 4])
def test_host_processes_daemon(world):
    res = mp_worker.launch(world, "host", "daemon")
    assert all(s["cqesDelivered"] == 48 and s["waitTimeouts"] == 0 and s["transport"] == "peer" for s in res.values())


def test_host_processes_stream_interface():
    mp_worker.launch(3, "host", "stream")


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_processes_daemon():
    import torch
    world = min(torch.cuda.device_count(), 4)
    res = mp_worker.launch(world, "cuda", "daemon")
    assert all(s["cqesDelivered"] == 48 for s in res.values())


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_processes_shared_memory_heap(monkeypatch):
    """Two GPUs in two processes that may not map one another's memory (NCCL_P2P_DISABLE=1) pick the heap in registered
    host shared memory together; the daemon's mixed, disordered collectives run on it unchanged."""
    monkeypatch.setenv("NCCL_P2P_DISABLE", "1")
    res = mp_worker.launch(2, "cuda", "daemon")
    assert all(s["cqesDelivered"] == 48 and s["transport"] == "shm" for s in res.values()), res


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_processes_stream_interface():
    import torch
    mp_worker.launch(min(torch.cuda.device_count(), 4), "cuda", "stream")


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fused_tensor_parallel_gemms():
    import torch
    mp_worker.launch(2 if torch.cuda.device_count() < 4 else 4, "cuda", "fused_tp", timeout=300)


@pytest.mark.parametrize("layout,world", [("tp2", 2), ("tp2pp2", 4), ("pp2dp2", 4), ("pp3", 3), ("tp2pp2dp2", 8)])
def test_host_gpt2_hybrid_parallel(layout, world):
    """Tensor x pipeline x data parallel GPT-2 steps on CPU ranks match the unsharded model."""
    res = mp_worker.launch(world, "host", "gpt_" + layout, timeout=300)
    assert all(r["cqes"] > 0 for r in res.values())
    losses = [tuple(round(x, 3) for x in r["losses"]) for r in res.values()]
    assert len(set(losses)) == 1, losses                     # every rank reports the same global loss


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_fused_operators_among_shuffled_gradient_buckets():
    """Registered fused tensor-parallel operators and daemon all-reduces of the overlapping data-parallel group, issued
    in per-rank shuffled interleavings (tp2 x dp2 on four GPUs, tp2 x dp1 on two)."""
    import torch
    world = 4 if torch.cuda.device_count() >= 4 else 2
    res = mp_worker.launch(world, "cuda", "tp_dp_shuffle", timeout=300)
    assert all(r["fused"] == 8 and r["cqes"] == 20 for r in res.values()), res


def test_host_pipeline_schedules_agree_and_1f1b_holds_fewer_activations():
    """Three pipeline stages, four micro-batches: GPipe and 1F1B train identically (same losses as the unsharded
    model, checked inside the scenario); 1F1B holds at most pp - stage micro-batches of activations, GPipe all."""
    a = mp_worker.launch(3, "host", "gpt_pp3_gpipe", timeout=300)
    b = mp_worker.launch(3, "host", "gpt_pp3_1f1b", timeout=300)
    for r in a.values():
        assert r["peak_live"] == 4
    for r in b.values():
        assert r["peak_live"] == min(3 - r["pp_rank"], 4)
    la = [round(x, 3) for x in next(iter(a.values()))["losses"]]
    lb = [round(x, 3) for x in next(iter(b.values()))["losses"]]
    assert la == lb, (la, lb)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_gpt2_hybrid_parallel():
    import torch
    n = torch.cuda.device_count()
    layout, world = ("tp2pp2dp2", 8) if n >= 8 else ("tp2pp2", 4) if n >= 4 else ("tp2", 2)
    mp_worker.launch(world, "cuda", "gpt_" + layout, timeout=600)


def test_host_processes_nvls_schedule():
    res = mp_worker.launch(2, "host", "nvls", timeout=200)
    assert all(r["available"] and r["daemon"] == 4 for r in res.values())


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_nvls_allreduce():
    """multimem.ld_reduce / multimem.st all-reduce; skipped by the library itself (available = False) on
    machines whose devices or driver cannot create a multicast object."""
    import torch
    res = mp_worker.launch(min(torch.cuda.device_count(), 4), "cuda", "nvls", timeout=300)
    if not all(r["available"] for r in res.values()):
        pytest.skip("no NVLink-switch multicast on this machine")


def test_host_processes_nvls_reducescatter_allgather():
    res = mp_worker.launch(2, "host", "nvls_rsag", timeout=200)
    assert all(r["available"] for r in res.values())


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_nvls_reducescatter_allgather():
    """multimem.ld_reduce into local memory (reduce-scatter) and multimem.st of the local piece (all-gather)."""
    res = mp_worker.launch(2, "cuda", "nvls_rsag", timeout=200)
    if not all(r["available"] for r in res.values()):
        pytest.skip("no NVLink-switch multicast on this machine")


def test_host_processes_network_path(monkeypatch):
    """Ranks in separate processes forced through the network path (TCP rings, host-staged collectives)."""
    monkeypatch.setenv("DFCCL_FORCE_NET", "1")
    res = mp_worker.launch(3, "host", "net_path", timeout=200)
    assert all(r["ok"] for r in res.values())


@pytest.mark.gpu
@pytest.mark.multigpu
def test_gpu_network_path(monkeypatch):
    """The same path on device buffers: operands staged through host memory around the TCP rings."""
    monkeypatch.setenv("DFCCL_FORCE_NET", "1")
    res = mp_worker.launch(2, "cuda", "net_path", timeout=200)
    assert all(r["ok"] for r in res.values())
