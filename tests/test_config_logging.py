"""Configuration (environment prefixes, conf files, size suffixes) and logging (levels, subsystem masks, log files):
each case runs in a process of its own, because conf files and the log set-up are read once per process."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(code: str, env: dict, tmp_path) -> str:
    full = dict(os.environ)
    for k in list(full):
        if k.startswith(("DFCCL_", "NCCL_")):
            del full[k]
    full.update({"HOME": str(tmp_path), "PYTHONPATH": ROOT}, **env)
    p = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], env=full, capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert p.returncode == 0, p.stdout + p.stderr
    return p.stdout + p.stderr


def test_parameter_sources_and_precedence(tmp_path):
    (tmp_path / ".dfccl.conf").write_text("# a comment\nDFCCL_IDLE_QUIT_US=1234\nDFCCL_HEAP_BYTES=1G\n")
    (tmp_path / ".nccl.conf").write_text("NCCL_WAIT_TIMEOUT_MS=777\nDFCCL_IDLE_QUIT_US=9999\n")
    out = _run("""
        from dfccl_b200 import native as nv
        print("idle", nv.param("IDLE_QUIT_US", 1))              # ~/.dfccl.conf is read before ~/.nccl.conf: first one wins
        print("wait", nv.param("WAIT_TIMEOUT_MS", 1))           # the reference's prefix, from its conf file
        print("heap", nv.param("HEAP_BYTES", 1))                # the environment beats the file; size suffix
        print("blocks", nv.param("DAEMON_BLOCKS", 5))           # both prefixes set: DFCCL_ wins
        print("factor", nv.param("RECV_SUCCESS_FACTOR", 1))     # the reference's unprefixed scheduler knob
        print("bad", nv.param("SLICE_BYTES", 42))               # not a number: the default
        print("unset", nv.param("NO_SUCH_PARAMETER", -3))
        print("hex", nv.param("STALL_QUIT_US", 0))
    """, {"DFCCL_HEAP_BYTES": "64M", "DFCCL_DAEMON_BLOCKS": "12", "NCCL_DAEMON_BLOCKS": "3", "RECV_SUCCESS_FACTOR": "7",
          "DFCCL_SLICE_BYTES": "lots", "NCCL_STALL_QUIT_US": "0x10"}, tmp_path)
    got = dict(line.split() for line in out.splitlines() if line and line.split()[0] in
               ("idle", "wait", "heap", "blocks", "factor", "bad", "unset", "hex"))
    assert got == {"idle": "1234", "wait": "777", "heap": str(64 << 20), "blocks": "12", "factor": "7", "bad": "42",
                   "unset": "-3", "hex": "16"}, out


def test_log_levels_subsystems_and_file(tmp_path):
    code = """
        import glob, os
        from dfccl_b200 import native as nv
        nv.set_backend("host")
        comms = nv.Comm.init_loopback(2)
        rc = nv.lib().ncclAllReduce(None, None, 8, nv.FLOAT32, nv.SUM, comms[0].handle, None)   # null buffers: a warning
        assert rc != nv.SUCCESS
        print("LAST", nv.last_error())
        for c in comms:
            c.destroy()
    """
    # INFO + INIT subsystem into a per-process file: communicator creation is logged there, nothing on stdout
    out = _run(code, {"DFCCL_DEBUG": "INFO", "DFCCL_DEBUG_SUBSYS": "INIT", "DFCCL_DEBUG_FILE": str(tmp_path / "log.%p.txt")}, tmp_path)
    files = list(tmp_path.glob("log.*.txt"))
    assert len(files) == 1 and files[0].name != "log.%p.txt"
    text = files[0].read_text()
    assert "DFCCL INFO" in text and "comm " in text and "rank 0/2" in text and "DFCCL WARN" in text and "null buffer" in text
    assert "DFCCL INFO" not in out and "LAST null buffer" in out
    # the mask can be inverted: everything but INIT leaves the creation lines out
    out = _run(code, {"NCCL_DEBUG": "INFO", "NCCL_DEBUG_SUBSYS": "^INIT"}, tmp_path)
    assert "rank 0/2" not in out and "DFCCL WARN" in out
    # WARN level: warnings only; no level: silence, but the text of the last warning stays available to the caller
    out = _run(code, {"DFCCL_DEBUG": "WARN"}, tmp_path)
    assert "DFCCL WARN" in out and "DFCCL INFO" not in out
    out = _run(code, {}, tmp_path)
    assert "DFCCL WARN" not in out and "LAST null buffer" in out


def test_rendezvous_by_comm_id_without_exchanging_a_unique_id(tmp_path):
    """``NCCL_COMM_ID=host:port`` (the reference's knob): every rank derives the same unique id from the environment
    and rank 0 serves the rendezvous there, so nothing has to be passed between the processes."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    code = """
        import sys
        import numpy as np
        from dfccl_b200 import native as nv
        rank, world = int(sys.argv[1]), 3
        nv.set_backend("host")
        comm = nv.Comm.init_rank(world, nv.get_unique_id(), rank)
        x = np.full(1000, float(rank + 1), np.float32)
        nv.check(nv.lib().ncclAllReduce(x.ctypes.data, x.ctypes.data, x.size, nv.FLOAT32, nv.SUM, comm.handle, None))
        assert float(x.min()) == float(x.max()) == 6.0, x[:4]
        comm.destroy()
        print("RANK_OK", rank)
    """
    env = dict(os.environ, NCCL_COMM_ID=f"127.0.0.1:{port}", HOME=str(tmp_path), PYTHONPATH=ROOT)
    procs = [subprocess.Popen([sys.executable, "-c", textwrap.dedent(code), str(r)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True, cwd=ROOT) for r in range(3)]
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=120)
            outs.append((p.returncode, out))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()                     # the exact children started above
    assert all(rc == 0 and "RANK_OK" in out for rc, out in outs), outs


def test_ranks_that_report_different_hosts_take_the_network_path(tmp_path):
    """``NCCL_HOSTID`` (the reference's knob for pretending to be on other hardware) gives two processes of this machine
    different host identities: they cannot map one another's memory, so the communicator selects the network
    transport by itself and the collectives still give the right answer."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    code = """
        import sys
        import numpy as np
        from dfccl_b200 import native as nv
        rank, world = int(sys.argv[1]), 2
        nv.set_backend("host")
        comm = nv.Comm.init_rank(world, nv.get_unique_id(), rank)
        assert comm.transport() == "net", comm.transport()
        x = (np.arange(5003, dtype=np.float32) % 13) + rank
        nv.check(nv.lib().ncclAllReduce(x.ctypes.data, x.ctypes.data, x.size, nv.FLOAT32, nv.SUM, comm.handle, None))
        assert np.array_equal(x, 2 * (np.arange(5003, dtype=np.float32) % 13) + 1)
        comm.destroy()
        print("RANK_OK", rank)
    """
    procs = []
    for r in range(2):
        env = dict(os.environ, NCCL_COMM_ID=f"127.0.0.1:{port}", NCCL_HOSTID=f"machine-{r}", HOME=str(tmp_path), PYTHONPATH=ROOT)
        env.pop("DFCCL_FORCE_NET", None)
        procs.append(subprocess.Popen([sys.executable, "-c", textwrap.dedent(code), str(r)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True, cwd=ROOT))
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=120)
            outs.append((p.returncode, out))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()                     # the exact children started above
    assert all(rc == 0 and "RANK_OK" in out for rc, out in outs), outs
