"""Worker body for multi-process tests: one OS process per rank, rendezvous through this
library's own TCP bootstrap (the unique id travels over a multiprocessing queue), memory
shared through POSIX shm (host backend) or CUDA IPC (cuda backend)."""
import ctypes as C
import os
import random
import sys
import traceback

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _view(nv, backend, ptr, n, npdt, tdt=None, dev=0):
    if backend == "host":
        from helpers import host_array
        return host_array(ptr, n, npdt)
    import torch
    from dfccl_b200.utils import tensor_from_ptr
    return tensor_from_ptr(ptr, (n,), tdt, f"cuda:{dev}")


def worker(rank, world, backend, uid_q, res_q, scenario):
    try:
        os.environ.setdefault("DFCCL_WAIT_TIMEOUT_MS", "20000")
        from dfccl_b200 import native as nv
        nv.set_backend(backend)
        if backend == "cuda":
            import torch
            torch.cuda.set_device(rank)
        if rank == 0:
            uid = nv.get_unique_id()
            for _ in range(world - 1):
                uid_q.put(uid)
        else:
            uid = uid_q.get(timeout=60)
        comm = nv.Comm.init_rank(world, uid, rank)
        assert comm.rank == rank and comm.nranks == world
        out = globals()["scenario_" + scenario](nv, comm, rank, world, backend)
        comm.destroy()
        res_q.put((rank, "ok", out))
    except BaseException:
        res_q.put((rank, "fail", traceback.format_exc()))


def _fill(v, value, backend):
    if backend == "host":
        v[:] = value
    else:
        v.fill_(value)


def _all_equal(v, value, backend):
    if backend == "host":
        return bool(np.all(v == value))
    return bool((v == value).all())


def scenario_daemon(nv, comm, rank, world, backend):
    """Register-then-submit across processes: mixed kinds, per-rank random order, several rounds."""
    tdt = None
    if backend == "cuda":
        import torch
        tdt = torch.float32
    ncolls, iters = 12, 4
    rng = random.Random(11)
    kinds = [rng.choice([nv.ALLREDUCE, nv.ALLGATHER, nv.REDUCESCATTER, nv.BROADCAST, nv.REDUCE]) for _ in range(ncolls)]
    counts = [rng.choice([32, 1000, 65536, 300001]) for _ in range(ncolls)]
    ctx = nv.RankCtx(rank, rank if backend == "cuda" else -1)
    bufs = []
    for i in range(ncolls):
        ctx.prepare(i, comm, kinds[i], counts[i], nv.FLOAT32, root=i % world)
        sn = counts[i] * (world if kinds[i] == nv.REDUCESCATTER else 1)
        rn = counts[i] * (world if kinds[i] == nv.ALLGATHER else 1)
        sp, rp = comm.alloc(sn * 4), comm.alloc(rn * 4)
        bufs.append((sp, rp, _view(nv, backend, sp, sn, np.float32, tdt, rank), _view(nv, backend, rp, rn, np.float32, tdt, rank)))
    ctx.finalize()
    orng = random.Random(1000 + rank)
    for it in range(iters):
        for i in range(ncolls):
            _fill(bufs[i][2], float((rank + 1) * (i + 1) + it), backend)
        if backend == "cuda":
            import torch
            torch.cuda.synchronize()
        order = list(range(ncolls))
        orng.shuffle(order)
        for i in order:
            ctx.run(i, bufs[i][0], bufs[i][1])
        rc = ctx.wait_all(120000)
        assert rc == nv.SUCCESS, rc
        for i in range(ncolls):
            vals = [float((q + 1) * (i + 1) + it) for q in range(world)]
            out = bufs[i][3]
            root = i % world
            if kinds[i] in (nv.ALLREDUCE, nv.REDUCESCATTER):
                assert _all_equal(out, sum(vals), backend), (i, kinds[i])
            elif kinds[i] == nv.REDUCE:
                if rank == root:
                    assert _all_equal(out, sum(vals), backend), (i, "reduce")
            elif kinds[i] == nv.BROADCAST:
                assert _all_equal(out, vals[root], backend), (i, "bcast")
            else:
                for q in range(world):
                    assert _all_equal(out[q * counts[i]:(q + 1) * counts[i]], vals[q], backend), (i, "ag", q)
    import time
    time.sleep(0.05)
    st = ctx.stats()
    st["transport"] = comm.transport()
    ctx.destroy()
    return st


def scenario_stream(nv, comm, rank, world, backend):
    """Stream-ordered nccl* interface across processes, plus send / recv."""
    L = nv.lib()
    vp = C.c_void_p
    n = 100003
    if backend == "cuda":
        import torch
        x = torch.full((n,), float(rank + 1), device=f"cuda:{rank}")
        y = torch.zeros(n, device=f"cuda:{rank}")
        st = vp(torch.cuda.current_stream().cuda_stream)
        xp, yp = x.data_ptr(), y.data_ptr()
        sync = torch.cuda.synchronize
    else:
        x = np.full(n, float(rank + 1), np.float32)
        y = np.zeros(n, np.float32)
        st, xp, yp, sync = None, x.ctypes.data, y.ctypes.data, (lambda: None)
    tot = world * (world + 1) / 2
    for _ in range(3):
        nv.check(L.ncclAllReduce(vp(xp), vp(yp), n, nv.FLOAT32, nv.SUM, comm.handle, st))
        sync()
        assert _all_equal(y, tot, backend)
    nv.check(L.ncclAllReduce(vp(yp), vp(yp), n, nv.FLOAT32, nv.AVG, comm.handle, st))   # in place
    sync()
    assert _all_equal(y, tot, backend)
    nv.check(L.ncclBcast(vp(yp), n, nv.FLOAT32, world - 1, comm.handle, st))
    sync()
    # heap-resident buffers take the zero-copy path
    hp = comm.alloc(4 * n)
    hv = _view(nv, backend, hp, n, np.float32, None if backend == "host" else __import__("torch").float32, rank)
    _fill(hv, float(rank), backend)
    sync()
    nv.check(L.ncclAllReduce(vp(hp), vp(hp), n, nv.FLOAT32, nv.MAX, comm.handle, st))
    sync()
    assert _all_equal(hv, world - 1, backend)
    # ring send / recv
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    _fill(x, float(rank), backend)
    sync()
    nv.check(L.ncclGroupStart())
    nv.check(L.ncclSend(vp(xp), n, nv.FLOAT32, nxt, comm.handle, st))
    nv.check(L.ncclRecv(vp(yp), n, nv.FLOAT32, prv, comm.handle, st))
    nv.check(L.ncclGroupEnd())
    sync()
    assert _all_equal(y, prv, backend)
    assert comm.async_error() == nv.SUCCESS
    return {}


def launch(world, backend, scenario, timeout=240):
    """Spawn `world` ranks, return their results; raises on any failure or timeout."""
    import multiprocessing as mp
    import socket
    # a fresh rendezvous port for whatever the scenario sets up with torch.distributed: a fixed one can still be
    # in TIME_WAIT from the previous run of the same test
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        os.environ["MASTER_PORT"] = str(s.getsockname()[1])
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    ctx = mp.get_context("spawn")
    uid_q, res_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, backend, uid_q, res_q, scenario), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            r, status, payload = res_q.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {r} failed:\n{payload}")
            results[r] = payload
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.terminate()       # the exact children started above
    return results


def scenario_fused_tp(nv, comm, rank, world, backend):
    """all-gather -> GEMM and GEMM -> reduce-scatter fused kernels against PyTorch fp32 references."""
    import torch
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from dfccl_b200.ops.fused_linear import AllGatherGemm, GemmReduceScatter, TpGroup
    from dfccl_b200.ops import gemm
    dev = torch.device("cuda", rank)
    tp = TpGroup(comm, dist.group.WORLD, dev)
    out = {}
    for rows, k, n_out in ((256, 1024, 1536), (1024, 1024, 2048)):
        g = torch.Generator(device="cpu").manual_seed(5)
        x_full = torch.randn(rows * world, k, generator=g).to(torch.bfloat16)
        w = torch.randn(n_out, k, generator=torch.Generator().manual_seed(100 + rank)).to(torch.bfloat16).to(dev)
        op = AllGatherGemm(tp, rows, k, n_out)
        for it in range(3):
            xs = (x_full[rank * rows:(rank + 1) * rows] * (it + 1)).to(dev)
            y = op(xs, w)
            torch.cuda.synchronize()
            ref = (x_full.to(dev).float() * (it + 1)) @ w.float().t()
            err = (y.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
            assert err < 1e-2, ("ag-gemm", rows, k, n_out, it, err)
        # row-parallel: every rank holds a K-slice of x and w, output rows are scattered
        m = rows * world
        kl = k // world
        xr = torch.randn(m, k, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16)
        wr = torch.randn(n_out, k, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
        op2 = GemmReduceScatter(tp, m, kl, n_out)
        for it in range(3):
            xl = (xr[:, rank * kl:(rank + 1) * kl] * (it + 1)).contiguous().to(dev)
            wl = wr[:, rank * kl:(rank + 1) * kl].contiguous().to(dev)
            ys = op2(xl, wl)
            torch.cuda.synchronize()
            # reference with the same rounding points: per-rank partial products in bf16, summed in fp32
            parts = [((xr[:, q * kl:(q + 1) * kl].to(dev).float() * (it + 1)) @ wr[:, q * kl:(q + 1) * kl].to(dev).float().t()).to(torch.bfloat16).float() for q in range(world)]
            ref = sum(parts)[rank * rows:(rank + 1) * rows]
            err = (ys.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
            assert err < 1e-2, ("gemm-rs", rows, k, n_out, it, err)
        assert gemm.check_kernels()
    dist.barrier()
    dist.destroy_process_group()
    return out


def scenario_tp_dp_shuffle(nv, comm, rank, world, backend):
    """Fused tensor-parallel operators (registered with the rank context) and data-parallel gradient all-reduces of the
    overlapping group, one context per rank: operators in model order, all-reduces in a per-rank shuffled order in
    between, on one stream.  tp = 2, dp = world / 2.  Results against fp32 references."""
    import torch
    from dfccl_b200.utils import tensor_from_ptr
    dev = torch.device("cuda", rank)
    tp_comm = comm.split(rank // 2, rank)
    dp_comm = comm.split(rank % 2, rank)
    dp = world // 2
    rows, k, n = 256, 512, 512
    ctx = nv.RankCtx(rank, rank)
    ctx.set_daemon_geometry(4, 0)
    ctx.prepare_fused(0, tp_comm, nv.FUSED_ALLGATHER_GEMM, rows, k, n)
    ctx.prepare_fused(1, tp_comm, nv.FUSED_GEMM_REDUCESCATTER, rows, k, n)
    counts = [3000, 1 << 20, 517, 70000, 1 << 18]
    bufs = []
    for i, cnt in enumerate(counts):
        ctx.prepare(2 + i, dp_comm, nv.ALLREDUCE, cnt, nv.FLOAT32)
        p = dp_comm.alloc(cnt * 4)
        bufs.append((p, tensor_from_ptr(p, (cnt,), torch.float32, dev)))
    ctx.finalize()
    g = torch.Generator().manual_seed(77)
    tpg = rank // 2                                   # my tensor-parallel group
    xs = torch.randn(world, rows, k, generator=g).to(torch.bfloat16)
    ws = torch.randn(world, n, k, generator=g).to(torch.bfloat16)
    x2 = torch.randn(world, 2 * rows, k, generator=g).to(torch.bfloat16)
    x_d, w_d, x2_d = xs[rank].to(dev), ws[rank].to(dev), x2[rank].to(dev)
    out_ag = torch.empty(2 * rows, n, dtype=torch.bfloat16, device=dev)
    out_rs = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    rng = random.Random(31 + rank)
    for it in range(4):
        dpart = list(range(len(counts)))
        rng.shuffle(dpart)
        cut = sorted(rng.sample(range(len(dpart) + 1), 2))
        seq = [("d", i) for i in dpart[:cut[0]]] + [("f", 0)] + [("d", i) for i in dpart[cut[0]:cut[1]]] + [("f", 1)] + [("d", i) for i in dpart[cut[1]:]]
        for kind, i in seq:
            if kind == "d":
                bufs[i][1].fill_(float((rank + 1) * (i + 1) + it))
                ctx.run_on_stream(2 + i, bufs[i][0], bufs[i][0], st)
            elif i == 0:
                ctx.run_fused(0, x_d.data_ptr(), w_d.data_ptr(), out_ag.data_ptr(), st)
            else:
                ctx.run_fused(1, x2_d.data_ptr(), w_d.data_ptr(), out_rs.data_ptr(), st)
        for i in range(len(counts)):
            ctx.stream_wait(2 + i, st)
        torch.cuda.synchronize()
        assert ctx.wait_all(60000) == nv.SUCCESS
        lo, hi = 2 * tpg, 2 * tpg + 1
        ref = torch.cat([xs[lo], xs[hi]]).to(dev).float() @ ws[rank].to(dev).float().t()
        err = (out_ag.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
        assert err < 1e-2, ("ag-gemm", it, err)
        parts = [(x2[q].to(dev).float() @ ws[q].to(dev).float().t()).to(torch.bfloat16).float() for q in (lo, hi)]
        ref2 = sum(parts)[(rank % 2) * rows:(rank % 2 + 1) * rows]
        err2 = (out_rs.float() - ref2).abs().max().item() / (ref2.abs().max().item() + 1e-6)
        assert err2 < 1e-2, ("gemm-rs", it, err2)
        for i in range(len(counts)):
            want = sum((q + 1) * (i + 1) + it for q in range(rank % 2, world, 2))
            assert bool((bufs[i][1] == float(want)).all()), ("bucket", i, it)
    stats = ctx.stats()
    assert ctx.async_error() == nv.SUCCESS
    ctx.destroy()
    tp_comm.destroy()
    dp_comm.destroy()
    return {"fused": stats["fusedLaunches"], "cqes": stats["cqesDelivered"], "dp": dp}


def _gpt_hybrid(nv, comm, rank, world, backend, tp, pp, dp, port, schedule="1f1b", n_micro=2):
    """Hybrid tp x pp x dp training of a small GPT-2 against the same model on one rank: the loss of
    every step must agree (the second and third steps depend on the gradients and the update)."""
    import torch
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(port))
    cuda = backend == "cuda"
    dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world, device_id=dev if cuda else None)
    from dfccl_b200.models.gpt2 import GPT2Config, GPT2Stage
    from dfccl_b200.parallel.groups import Dist
    from dfccl_b200.parallel.hybrid import HybridTrainer, build_mesh
    cfg = GPT2Config(n_layer=4, d_model=512, n_head=8, seq_len=128, vocab=512) if cuda else \
        GPT2Config(n_layer=2 if pp < 3 else pp, d_model=64, n_head=4, seq_len=32, vocab=96)
    micro_batch, steps = 2, 3
    d = Dist(rank, world, rank if cuda else 0, dev, comm, True)
    mesh = build_mesh(d, tp, pp, dp)
    stage = GPT2Stage(cfg, mesh.tp_group, mesh.pp_rank, pp, micro_batch)
    tr = HybridTrainer(d, mesh, stage, n_micro=n_micro, lr=0.3, bucket_mb=0.25, seed=3, schedule=schedule)
    g = torch.Generator().manual_seed(11)
    data = torch.randint(0, cfg.vocab, (dp, n_micro, micro_batch, cfg.seq_len + 1), generator=g)
    tok, tgt = data[mesh.dp_rank, ..., :-1].to(dev), data[mesh.dp_rank, ..., 1:].to(dev)
    losses = []
    for _ in range(steps):
        losses.append(float(tr.step(tok, tgt)))
    if cuda:
        torch.cuda.synchronize()
        bad = C.c_int(0)
        nv.check(nv.lib().dfcclGemmCheck(C.byref(bad)))
        assert bad.value == 0, "a fused GEMM kernel gave up on a wait"
    st = tr.ddp.stats()
    peak = tr.peak_live_microbatches
    graphed = None
    tr.close()
    if cuda and pp == 1:
        # the same step captured in a CUDA graph: it must really be captured and replayed, and keep training.  A rank
        # context is finalized once, so the second trainer gets a mesh (and a context) of its own.
        mesh2 = build_mesh(d, tp, pp, dp)
        tg = HybridTrainer(d, mesh2, GPT2Stage(cfg, mesh2.tp_group, mesh2.pp_rank, pp, micro_batch), n_micro=n_micro, lr=0.3,
                           bucket_mb=0.25, seed=3, use_graph=True, schedule=schedule)
        gl = [float(tg.step(tok, tgt)) for _ in range(3)]
        torch.cuda.synchronize()
        assert tg._graph is not None, "use_graph=True did not capture a graph"
        assert abs(gl[0] - losses[0]) < 3e-2 * max(1.0, abs(losses[0])), (gl, losses)
        assert gl[-1] < gl[0], gl
        graphed = gl
        tg.close()
    if rank == 0:                                           # the same model, unsharded, on this rank alone
        (c1,) = nv.Comm.init_loopback(1, rank if cuda else 0)
        d1 = Dist(0, 1, rank if cuda else 0, dev, c1, False)
        m1 = build_mesh(d1, 1, 1, 1)
        s1 = GPT2Stage(cfg, m1.tp_group, 0, 1, micro_batch)
        t1 = HybridTrainer(d1, m1, s1, n_micro=n_micro * dp, lr=0.3, bucket_mb=0.25, seed=3)
        flat = data.reshape(dp * n_micro, micro_batch, cfg.seq_len + 1)
        ref = [float(t1.step(flat[..., :-1].to(dev), flat[..., 1:].to(dev))) for _ in range(steps)]
        t1.close()
        for a, b in zip(losses, ref):
            assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (losses, ref)
        assert ref[-1] < ref[0] - 0.05, ref
    dist.barrier()
    dist.destroy_process_group()
    return {"losses": losses, "cqes": st["cqesDelivered"], "peak_live": peak, "pp_rank": mesh.pp_rank, "graphed": graphed}


def scenario_gpt_pp3_gpipe(nv, comm, rank, world, backend):
    return _gpt_hybrid(nv, comm, rank, world, backend, 1, 3, 1, 29586, schedule="gpipe", n_micro=4)


def scenario_gpt_pp3_1f1b(nv, comm, rank, world, backend):
    return _gpt_hybrid(nv, comm, rank, world, backend, 1, 3, 1, 29587, schedule="1f1b", n_micro=4)


def scenario_gpt_tp2(nv, comm, rank, world, backend):
    return _gpt_hybrid(nv, comm, rank, world, backend, 2, 1, 1, 29581)


def scenario_gpt_tp2pp2(nv, comm, rank, world, backend):
    return _gpt_hybrid(nv, comm, rank, world, backend, 2, 2, 1, 29582)


def scenario_gpt_pp2dp2(nv, comm, rank, world, backend):
    return _gpt_hybrid(nv, comm, rank, world, backend, 1, 2, 2, 29583)


def scenario_gpt_pp3(nv, comm, rank, world, backend):
    return _gpt_hybrid(nv, comm, rank, world, backend, 1, 3, 1, 29585)


def scenario_gpt_tp2pp2dp2(nv, comm, rank, world, backend):
    return _gpt_hybrid(nv, comm, rank, world, backend, 2, 2, 2, 29584)


def scenario_nvls(nv, comm, rank, world, backend):
    """All-reduce through the switch-multicast arena: daemon (fused scale + cast, arena-resident and staged
    buffers) and the stream-ordered entry point (in place in the arena, and staged in pieces)."""
    os.environ["DFCCL_NVLS_MIN_BYTES"] = "4096"
    small = backend == "host"                               # the shared-memory heap of the CPU runs is small
    if small:
        os.environ["DFCCL_NVLS_STREAM_BYTES"] = str(8 << 20)
    arena = (48 << 20) if small else (256 << 20)
    if not comm.nvls_init(arena):
        return {"available": False}
    uc, mc, nbytes, used = comm.nvls_info()
    assert uc and nbytes >= arena and (backend == "host" or mc)
    import torch
    cuda = backend == "cuda"
    dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
    from dfccl_b200.utils import tensor_from_ptr
    out = {"available": True}
    ctx = nv.RankCtx(rank, rank if cuda else -1)
    count = (256 * 1024 if small else 3 * 1024 * 1024) + 4096
    ctx.prepare(1, comm, nv.ALLREDUCE, count, nv.BFLOAT16, out_dtype=nv.FLOAT32, op=nv.SUM, scale=1.0 / world, algo=nv.ALGO_NVLS)
    ctx.prepare(2, comm, nv.ALLREDUCE, count, nv.FLOAT32, op=nv.SUM, algo=nv.ALGO_NVLS)
    ctx.finalize()
    g = torch.Generator().manual_seed(9)
    full = torch.rand(world, count, generator=g) * 2 - 1
    # 1: bf16 gradients averaged into fp32, buffers in the arena (zero copy)
    sp, rp = comm.nvls_alloc(count * 2), comm.nvls_alloc(count * 4)
    s, r = tensor_from_ptr(sp, (count,), torch.bfloat16, dev), tensor_from_ptr(rp, (count,), torch.float32, dev)
    ref = full.to(torch.bfloat16).float().sum(0) / world
    for it in range(3):
        s.copy_(full[rank].to(torch.bfloat16))
        r.zero_()
        if cuda:
            torch.cuda.synchronize()
        ctx.run(1, sp, rp)
        assert ctx.wait(1, 30000) == nv.SUCCESS
        err = (r.cpu() - ref).abs().max().item()
        assert err < 2e-2, ("nvls bf16->f32", it, err)
    # 2: fp32 sum, ordinary device tensors (staged through the arena slots)
    a = full[rank].to(dev).contiguous()
    b = torch.zeros(count, device=dev)
    if cuda:
        torch.cuda.synchronize()
    ctx.run(2, a.data_ptr(), b.data_ptr())
    assert ctx.wait(2, 30000) == nv.SUCCESS
    err = (b.cpu() - full.sum(0)).abs().max().item()
    assert err < 1e-4, ("nvls f32 staged", err)
    out["daemon"] = ctx.stats()["cqesDelivered"]
    ctx.destroy()
    # stream-ordered: a tensor larger than the staging front of the arena goes through it in pieces
    n2 = (3 if small else 24) * 1024 * 1024
    x = torch.full((n2,), float(rank + 1), device=dev)
    stream = torch.cuda.current_stream().cuda_stream if cuda else None
    nv.check(nv.lib().ncclAllReduce(x.data_ptr(), x.data_ptr(), n2, nv.FLOAT32, nv.SUM, comm.handle, stream))
    if cuda:
        torch.cuda.synchronize()
    want = world * (world + 1) / 2
    assert float(x.min()) == want and float(x.max()) == want, (float(x.min()), float(x.max()), want)
    return out


def scenario_nvls_rsag(nv, comm, rank, world, backend):
    """Reduce-scatter and all-gather on the multimem schedule (pinned at registration), arena-resident shared side."""
    arena = (24 << 20) if backend == "host" else (128 << 20)
    if not comm.nvls_init(arena):
        return {"available": False}
    import torch
    cuda = backend == "cuda"
    dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
    from dfccl_b200.utils import tensor_from_ptr
    count = 64 * 1024 if backend == "host" else 1024 * 1024
    ctx = nv.RankCtx(rank, rank if cuda else -1)
    ctx.prepare(1, comm, nv.REDUCESCATTER, count, nv.BFLOAT16, out_dtype=nv.FLOAT32, op=nv.SUM, scale=0.5, algo=nv.ALGO_NVLS)
    ctx.prepare(2, comm, nv.ALLGATHER, count, nv.FLOAT32, algo=nv.ALGO_NVLS)
    ctx.prepare(3, comm, nv.BROADCAST, count, nv.FLOAT32, root=world - 1, algo=nv.ALGO_NVLS)
    ctx.finalize()
    g = torch.Generator().manual_seed(4)
    full = (torch.rand(world, world * count, generator=g) * 2 - 1).to(torch.bfloat16)
    sp = comm.nvls_alloc(world * count * 2)                       # what the switch reads: in the arena
    s = tensor_from_ptr(sp, (world * count,), torch.bfloat16, dev)
    r = torch.zeros(count, dtype=torch.float32, device=dev)      # the result stays local: an ordinary tensor
    ref = 0.5 * full.float().sum(0)[rank * count:(rank + 1) * count]
    for it in range(2):
        s.copy_(full[rank])
        r.zero_()
        if cuda:
            torch.cuda.synchronize()
        ctx.run(1, sp, r.data_ptr())
        assert ctx.wait(1, 30000) == nv.SUCCESS
        err = (r.cpu() - ref).abs().max().item()
        assert err < 3e-2, ("nvls reduce-scatter", it, err)
    x = torch.full((count,), float(rank + 1), device=dev)         # local input: an ordinary tensor
    op = comm.nvls_alloc(world * count * 4)                       # what the switch writes: in the arena
    o = tensor_from_ptr(op, (world * count,), torch.float32, dev)
    o.zero_()
    if cuda:
        torch.cuda.synchronize()
    ctx.run(2, x.data_ptr(), op)
    assert ctx.wait(2, 30000) == nv.SUCCESS
    got = o.view(world, count).cpu()
    assert all(float(got[j].min()) == j + 1 and float(got[j].max()) == j + 1 for j in range(world)), "nvls all-gather"
    # broadcast: the root's multicast stores fill every member's output (an ordinary tensor here: staged through the
    # collective's arena slot), twice with different data
    b = torch.zeros(count, device=dev)
    for it in range(2):
        src = torch.arange(count, dtype=torch.float32, device=dev) + 7 * it + 100 * rank
        b.fill_(-1)
        if cuda:
            torch.cuda.synchronize()
        ctx.run(3, src.data_ptr() if rank == world - 1 else 0, b.data_ptr())
        assert ctx.wait(3, 30000) == nv.SUCCESS
        want = torch.arange(count, dtype=torch.float32) + 7 * it + 100 * (world - 1)
        assert torch.equal(b.cpu(), want), ("nvls broadcast", it)
    ctx.destroy()
    return {"available": True}


def scenario_net_path(nv, comm, rank, world, backend):
    """Network path (set DFCCL_FORCE_NET=1 before launching): the stream-ordered entry point and a registered
    collective on buffers of the backend's memory (device tensors on the cuda backend: staged through the host)."""
    import torch
    cuda = backend == "cuda"
    dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
    n = 100003
    x = torch.full((n,), float(rank + 1), device=dev)
    stream = torch.cuda.current_stream().cuda_stream if cuda else None
    nv.check(nv.lib().ncclAllReduce(x.data_ptr(), x.data_ptr(), n, nv.FLOAT32, nv.SUM, comm.handle, stream))
    want = world * (world + 1) / 2
    assert float(x.min()) == want and float(x.max()) == want
    ctx = nv.RankCtx(rank, rank if cuda else -1)
    ctx.prepare(0, comm, nv.ALLREDUCE, n, nv.BFLOAT16, out_dtype=nv.FLOAT32, op=nv.SUM, scale=0.5)
    ctx.finalize()
    a = torch.full((n,), float(rank + 1), device=dev, dtype=torch.bfloat16)
    b = torch.zeros(n, device=dev)
    if cuda:
        torch.cuda.synchronize()
    ctx.run(0, a.data_ptr(), b.data_ptr())
    assert ctx.wait(0, 60000) == nv.SUCCESS
    assert float(b.min()) == 0.5 * want and float(b.max()) == 0.5 * want
    ctx.destroy()
    # send / recv on this path: messages over the communicator's out-of-band connections, staged through the host.
    # Everybody sends two messages to the next rank and receives two from the previous one inside one group.
    L, nxt, prv = nv.lib(), (rank + 1) % world, (rank - 1) % world
    m = 70001
    s1 = torch.full((m,), float(10 * rank + 1), device=dev)
    s2 = torch.full((3,), float(10 * rank + 2), device=dev)
    r1, r2 = torch.zeros(m, device=dev), torch.zeros(3, device=dev)
    nv.check(L.ncclGroupStart())
    nv.check(L.ncclSend(s1.data_ptr(), m, nv.FLOAT32, nxt, comm.handle, stream))
    nv.check(L.ncclSend(s2.data_ptr(), 3, nv.FLOAT32, nxt, comm.handle, stream))
    nv.check(L.ncclRecv(r1.data_ptr(), m, nv.FLOAT32, prv, comm.handle, stream))
    nv.check(L.ncclRecv(r2.data_ptr(), 3, nv.FLOAT32, prv, comm.handle, stream))
    nv.check(L.ncclGroupEnd())
    if cuda:
        torch.cuda.synchronize()
    assert float(r1.min()) == float(r1.max()) == 10 * prv + 1 and float(r2.min()) == float(r2.max()) == 10 * prv + 2
    return {"ok": True}
