"""Data-parallel wrapper on the host backend: flat buckets, gradient views in the symmetric
heap, fused scale / cast in the all-reduce, randomized bucket order, optimizer arithmetic."""
import copy

import numpy as np
import pytest
import torch
import torch.nn as nn

from helpers import run_ranks


def _mlp():
    torch.manual_seed(5)
    return nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, 8))


@pytest.mark.parametrize("world", [1, 2, 4])
def test_ddp_matches_single_process_sgd(host_backend, world):
    nv = host_backend
    from dfccl_b200.parallel import DaemonDDP, Dist
    comms = nv.Comm.init_loopback(world)
    steps, lr, mu, wd = 4, 0.05, 0.9, 1e-3
    xs = [[torch.randn(16, 32, generator=torch.Generator().manual_seed(10 * s + r)) for r in range(world)] for s in range(steps)]
    ys = [[torch.randn(16, 8, generator=torch.Generator().manual_seed(99 + 10 * s + r)) for r in range(world)] for s in range(steps)]

    # reference: one process, gradients averaged over the per-rank batches, classic momentum SGD
    ref = _mlp()
    bufs = [torch.zeros_like(p) for p in ref.parameters()]
    for s in range(steps):
        grads = [torch.zeros_like(p) for p in ref.parameters()]
        for r in range(world):
            ref.zero_grad()
            nn.functional.mse_loss(ref(xs[s][r]), ys[s][r]).backward()
            for g, p in zip(grads, ref.parameters()):
                g += p.grad / world
        with torch.no_grad():
            for p, g, m in zip(ref.parameters(), grads, bufs):
                g = g + wd * p
                m.mul_(mu if s > 0 else 0.0).add_(g)
                p.sub_(lr * m)

    finals = {}
    nets = [_mlp() for _ in range(world)]       # built here: the global RNG is not thread safe

    def body(r):
        d = Dist(r, world, 0, torch.device("cpu"), comms[r], False)
        net = nets[r]
        ddp = DaemonDDP(net, d, bucket_mb=0.004, lr=lr, momentum=mu, weight_decay=wd, randomize_order=True, window=2, seed=3)
        assert len(ddp.buckets) >= 3                      # several buckets so that orders really differ
        for s in range(steps):
            nn.functional.mse_loss(net(xs[s][r]), ys[s][r]).backward()
            ddp.finish_backward()
            assert ddp.ctx.wait_all(30000) == nv.SUCCESS
            ddp.step()
        finals[r] = [p.detach().clone() for p in net.parameters()]
        st = ddp.stats()
        assert st["cqesDelivered"] == steps * len(ddp.buckets)
        ddp.close()

    run_ranks(world, body)
    for c in comms:
        c.destroy()
    for r in range(world):
        for got, exp in zip(finals[r], ref.parameters()):
            torch.testing.assert_close(got, exp.detach(), rtol=1e-5, atol=1e-6)


def test_parameters_and_gradients_are_views_of_flat_buckets(host_backend):
    nv = host_backend
    from dfccl_b200.parallel import DaemonDDP, Dist
    (c,) = nv.Comm.init_loopback(1)
    net = _mlp()
    ddp = DaemonDDP(net, Dist(0, 1, 0, torch.device("cpu"), c, False), bucket_mb=1.0)
    base, nbytes, _ = c.heap_info()
    for b in ddp.buckets:
        assert base <= b.grad.data_ptr() < base + nbytes and base <= b.grad32.data_ptr() < base + nbytes
        for p, off in zip(b.params, b.offsets):
            assert p.data_ptr() == b.flat_param.data_ptr() + off * p.element_size()
            assert p.grad.data_ptr() == b.grad.data_ptr() + off * p.element_size()
            assert off % 8 == 0
    ddp.close()
    c.destroy()


def test_parameter_groups_reduce_over_their_own_communicators(host_backend):
    """Two groups of parameters on one daemon: the first is averaged over pairs of ranks (a split
    communicator), the second summed over all four ranks."""
    nv = host_backend
    from dfccl_b200.parallel import DaemonDDP, Dist
    world = 4
    comms = nv.Comm.init_loopback(world)
    out = {}
    nets = []
    for r in range(world):
        torch.manual_seed(1)
        nets.append(nn.Sequential(nn.Linear(8, 8, bias=False), nn.Linear(8, 4, bias=False)))

    def body(r):
        pair = comms[r].split(r // 2, r)
        d = Dist(r, world, 0, torch.device("cpu"), comms[r], False)
        net = nets[r]
        groups = [{"params": [net[0].weight], "comm": pair, "scale": 0.5},
                  {"params": [net[1].weight], "comm": comms[r], "scale": 1.0}]
        ddp = DaemonDDP(net, d, lr=1.0, momentum=0.0, weight_decay=0.0, param_groups=groups, seed=r)
        w0, w1 = net[0].weight.detach().clone(), net[1].weight.detach().clone()
        net[0].weight.grad.fill_(float(r + 1))             # gradients are views of the flat buckets
        net[1].weight.grad.fill_(float(10 * (r + 1)))
        ddp.submit_all()
        ddp.finish_backward()
        assert ddp.ctx.wait_all(30000) == nv.SUCCESS
        ddp.step()
        out[r] = ((w0 - net[0].weight.detach()).mean().item(), (w1 - net[1].weight.detach()).mean().item())
        ddp.close()
        pair.destroy()

    run_ranks(world, body)
    for c in comms:
        c.destroy()
    for r in range(world):
        mate = r ^ 1
        assert abs(out[r][0] - ((r + 1) + (mate + 1)) / 2) < 1e-5, out      # lr 1, no momentum: the update is the reduced gradient
        assert abs(out[r][1] - 10 * (1 + 2 + 3 + 4)) < 1e-4, out


def test_gradient_buckets_in_the_multicast_arena(host_backend):
    """``nvls=True`` places the buckets' gradient arrays in the communicator's multicast arena and registers their
    all-reduces on the multimem schedule (bf16 in, fp32 out, 1/N scale); the training trajectory is the one of the
    heap-resident buckets.  Buckets whose size is not a 16-byte multiple keep the peer schedule."""
    nv = host_backend
    from dfccl_b200.parallel import DaemonDDP, Dist
    world, steps = 3, 3
    xs = [[torch.randn(8, 32, generator=torch.Generator().manual_seed(7 * s + r)) for r in range(world)] for s in range(steps)]
    finals = {}
    for mode in (False, True):
        comms = nv.Comm.init_loopback(world)
        nets = [_mlp() for _ in range(world)]
        paths = {}

        def body(r):
            d = Dist(r, world, 0, torch.device("cpu"), comms[r], False)
            ddp = DaemonDDP(nets[r], d, bucket_mb=0.004, lr=0.05, momentum=0.9, weight_decay=0.0, seed=5, nvls=mode)
            for s in range(steps):
                nets[r](xs[s][r]).square().mean().backward()
                ddp.finish_backward()
                assert ddp.ctx.wait_all(30000) == nv.SUCCESS
                ddp.step()
            paths[r] = (ddp.gradient_path(), [b.nvls for b in ddp.buckets])
            finals[(mode, r)] = [p.detach().clone() for p in nets[r].parameters()]
            ddp.close()

        run_ranks(world, body)
        for c in comms:
            c.destroy()
        if mode:
            assert all("multimem" in p[0] and any(p[1]) for p in paths.values()), paths
        else:
            assert all(p[0] == "peer loads/stores" for p in paths.values()), paths
    for r in range(world):
        for a, b in zip(finals[(False, r)], finals[(True, r)]):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)


def test_stress_orders_deadlock_an_inorder_library():
    from dfccl_b200.benchmarks.stress import inorder_verdict
    v = inorder_verdict(64, 20, 8, 2024)
    assert v["iterations_with_incompatible_orders"] == 20 and v["first"]["iteration"] == 0
    assert inorder_verdict(16, 5, 1, 7)["iterations_with_incompatible_orders"] == 0     # one rank cannot disagree with itself


def test_checkpoint_resume_continues_the_same_trajectory(host_backend, tmp_path):
    """Save after two steps, rebuild the wrapper from scratch, load, continue: same weights as an uninterrupted run."""
    nv = host_backend
    from dfccl_b200.parallel import DaemonDDP, Dist
    xs = [torch.randn(16, 32, generator=torch.Generator().manual_seed(s)) for s in range(4)]
    ys = [torch.randn(16, 8, generator=torch.Generator().manual_seed(50 + s)) for s in range(4)]

    def run(steps, state=None):
        (c,) = nv.Comm.init_loopback(1)
        d = Dist(0, 1, 0, torch.device("cpu"), c, False)
        net = _mlp()
        ddp = DaemonDDP(net, d, bucket_mb=0.004, lr=0.05, momentum=0.9, weight_decay=1e-3)
        if state is not None:
            ddp.load_state_dict(torch.load(state, weights_only=False))
        for s in steps:
            nn.functional.mse_loss(net(xs[s]), ys[s]).backward()
            ddp.finish_backward()
            assert ddp.ctx.wait_all(30000) == nv.SUCCESS
            ddp.step()
        out = [p.detach().clone() for p in net.parameters()]
        sd = ddp.state_dict()
        ddp.close()
        c.destroy()
        return out, sd

    full, _ = run([0, 1, 2, 3])
    _, sd = run([0, 1])
    path = tmp_path / "ckpt.pt"
    torch.save(sd, path)
    resumed, _ = run([2, 3], state=path)
    for a, b in zip(full, resumed):
        torch.testing.assert_close(a, b, rtol=0, atol=0)


def test_adamw_matches_torch_optim(host_backend):
    """AdamW over the flat buckets (host arithmetic of the fused kernel) against torch.optim.AdamW, two ranks."""
    nv = host_backend
    from dfccl_b200.parallel import DaemonDDP, Dist
    world, steps = 2, 4
    comms = nv.Comm.init_loopback(world)
    xs = [[torch.randn(16, 32, generator=torch.Generator().manual_seed(10 * s + r)) for r in range(world)] for s in range(steps)]
    ys = [[torch.randn(16, 8, generator=torch.Generator().manual_seed(99 + 10 * s + r)) for r in range(world)] for s in range(steps)]
    ref = _mlp()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for s in range(steps):
        opt.zero_grad()
        for r in range(world):
            (nn.functional.mse_loss(ref(xs[s][r]), ys[s][r]) / world).backward()
        opt.step()
    finals = {}
    nets = [_mlp() for _ in range(world)]

    def body(r):
        d = Dist(r, world, 0, torch.device("cpu"), comms[r], False)
        ddp = DaemonDDP(nets[r], d, bucket_mb=0.004, lr=1e-2, weight_decay=0.1, optimizer="adamw", betas=(0.9, 0.95), eps=1e-8)
        for s in range(steps):
            nn.functional.mse_loss(nets[r](xs[s][r]), ys[s][r]).backward()
            ddp.finish_backward()
            assert ddp.ctx.wait_all(30000) == nv.SUCCESS
            ddp.step()
        finals[r] = [p.detach().clone() for p in nets[r].parameters()]
        ddp.close()

    run_ranks(world, body)
    for c in comms:
        c.destroy()
    for r in range(world):
        for got, exp in zip(finals[r], ref.parameters()):
            torch.testing.assert_close(got, exp.detach(), rtol=1e-4, atol=1e-6)
