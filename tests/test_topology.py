"""Topology (injection, dump, path policy) and the size -> schedule tuner, without a GPU: a fake system comes in
through DFCCL_TOPO_FILE, as the reference's NCCL_TOPO_FILE does for its graph search."""
import pytest

FAKE = """<system nvswitch="1" link_gbs="770" hbm_gbs="6500" block_gbs="28" hop_us="1.8">
  <gpu dev="0" name="NVIDIA B200" busid="0000:1b:00.0" sm="100" sms="148" mem="191000000000" l2="132120576" multicast="1" nvlinks="18"/>
  <gpu dev="1" name="NVIDIA B200" busid="0000:43:00.0" sm="100" sms="148" mem="191000000000" l2="132120576" multicast="1" nvlinks="18"/>
  <gpu dev="2" name="NVIDIA B200" busid="0000:52:00.0" sm="100" sms="148" mem="191000000000" l2="132120576" multicast="1" nvlinks="18"/>
  <gpu dev="3" name="NVIDIA L4" busid="0000:61:00.0" sm="89" sms="58" mem="24000000000" l2="50331648" multicast="0" nvlinks="0"/>
  <p2p a="0" b="1" type="NVL"/>
  <p2p a="0" b="2" type="NVL"/>
  <p2p a="1" b="2" type="NVL"/>
  <p2p a="0" b="3" type="PCI"/>
</system>
"""


@pytest.fixture
def fake_system(native, tmp_path, monkeypatch):
    path = tmp_path / "system.xml"
    path.write_text(FAKE)
    monkeypatch.setenv("DFCCL_TOPO_FILE", str(path))
    native.topo_reset()
    yield native
    monkeypatch.delenv("DFCCL_TOPO_FILE")
    native.topo_reset()


def test_injected_topology_round_trips(fake_system, tmp_path, monkeypatch):
    nv = fake_system
    assert nv.topo_gpu_count() == 4
    xml = nv.topo_xml()
    assert 'name="NVIDIA L4"' in xml and xml.count("<p2p ") == 4 and 'type="PCI"' in xml
    # what the library dumps is what it reads back: inject the dump and compare
    dump = tmp_path / "dump.xml"
    monkeypatch.setenv("DFCCL_TOPO_DUMP_FILE", str(dump))
    nv.topo_reset()
    assert nv.topo_gpu_count() == 4
    monkeypatch.delenv("DFCCL_TOPO_DUMP_FILE")
    monkeypatch.setenv("DFCCL_TOPO_FILE", str(dump))
    nv.topo_reset()
    assert nv.topo_xml() == xml


def test_path_policy(fake_system, monkeypatch):
    nv = fake_system
    assert nv.topo_p2p_allowed(0, 1) and nv.topo_p2p_allowed(0, 3) and nv.topo_p2p_allowed(2, 2)
    assert not nv.topo_p2p_allowed(1, 3)                       # no peer path between the two at all
    monkeypatch.setenv("NCCL_P2P_LEVEL", "NVL")                # the reference's knob: NVLink only
    assert nv.topo_p2p_allowed(0, 1) and not nv.topo_p2p_allowed(0, 3)
    monkeypatch.setenv("NCCL_P2P_LEVEL", "LOC")
    assert nv.topo_p2p_allowed(1, 1) and not nv.topo_p2p_allowed(0, 1)
    monkeypatch.setenv("NCCL_P2P_LEVEL", "PHB")
    assert nv.topo_p2p_allowed(0, 3)
    monkeypatch.setenv("NCCL_P2P_DISABLE", "1")
    assert not nv.topo_p2p_allowed(0, 1)
    monkeypatch.delenv("NCCL_P2P_DISABLE")
    monkeypatch.delenv("NCCL_P2P_LEVEL")
    assert nv.topo_p2p_allowed(7, 9)                           # devices the file does not know: left to the mapping attempt


def test_tuner_blocks_and_schedules(fake_system):
    nv = fake_system
    # small messages take one block, large ones as many as they may; the prediction grows with the size
    algo, nb, us_small = nv.tuner_choose(nv.ALLREDUCE, 4096, 8, 64)
    assert nb == 1 and algo in (nv.ALGO_ONESHOT, nv.ALGO_TWOSHOT)
    algo, nb, us_big = nv.tuner_choose(nv.ALLREDUCE, 256 << 20, 8, 64)
    assert nb == 64 and algo == nv.ALGO_TWOSHOT and us_big > us_small
    # the multimem schedule where the fabric has it and the message is large enough; never for tiny messages
    assert nv.tuner_choose(nv.ALLREDUCE, 256 << 20, 8, 64, nvls=True)[0] == nv.ALGO_NVLS
    assert nv.tuner_choose(nv.ALLREDUCE, 4096, 8, 64, nvls=True)[0] != nv.ALGO_NVLS
    # a pinned schedule is kept; kinds without a one-shot form fall back to the one they have
    assert nv.tuner_choose(nv.ALLREDUCE, 256 << 20, 8, 64, pinned_algo=nv.ALGO_ONESHOT)[0] == nv.ALGO_ONESHOT
    assert nv.tuner_choose(nv.ALLGATHER, 1 << 20, 8, 64, pinned_algo=nv.ALGO_ONESHOT)[0] == nv.ALGO_TWOSHOT
    # more blocks never make the model slower for a bandwidth-bound message, and two-shot moves less per link than one-shot
    t8 = nv.tuner_predict_us(nv.ALLREDUCE, nv.ALGO_TWOSHOT, 64 << 20, 8, 8)
    t64 = nv.tuner_predict_us(nv.ALLREDUCE, nv.ALGO_TWOSHOT, 64 << 20, 8, 64)
    assert t64 <= t8
    assert nv.tuner_predict_us(nv.ALLREDUCE, nv.ALGO_TWOSHOT, 64 << 20, 8, 64) < nv.tuner_predict_us(nv.ALLREDUCE, nv.ALGO_ONESHOT, 64 << 20, 8, 64)
