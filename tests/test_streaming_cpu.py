"""Host-side placement helpers of the host-streamed path (no GPU): the GPU's host socket is read from a
sysfs tree, and the binding is put back after the allocation."""
import os
import types

import pytest

from artifact_b200 import streaming


def fake_sysfs(tmp_path, node, cpulist, bdf="0000:1b:00.0"):
    d = tmp_path / "bus" / "pci" / "devices" / bdf
    d.mkdir(parents=True)
    (d / "numa_node").write_text(f"{node}\n")
    if node >= 0:
        n = tmp_path / "devices" / "system" / "node" / f"node{node}"
        n.mkdir(parents=True)
        (n / "cpulist").write_text(cpulist + "\n")
    return str(tmp_path)


@pytest.fixture
def one_gpu(monkeypatch):
    props = types.SimpleNamespace(pci_domain_id=0, pci_bus_id=0x1b, pci_device_id=0)
    monkeypatch.setattr(streaming.torch.cuda, "get_device_properties", lambda i: props)


def test_cpulist_forms():
    assert streaming._cpulist("0-3,8,10-11") == {0, 1, 2, 3, 8, 10, 11}
    assert streaming._cpulist("") == set()
    assert streaming._cpulist("5") == {5}


def test_host_node_from_sysfs(tmp_path, one_gpu):
    root = fake_sysfs(tmp_path, 1, "4-7,12-15")
    assert streaming.device_host_node(0, root) == (1, {4, 5, 6, 7, 12, 13, 14, 15})


def test_host_node_unknown(tmp_path, one_gpu):
    assert streaming.device_host_node(0, fake_sysfs(tmp_path, -1, "")) == (None, set())
    assert streaming.device_host_node(0, str(tmp_path / "nothing")) == (None, set())


def test_near_device_binds_and_restores(tmp_path, one_gpu):
    mine = os.sched_getaffinity(0)
    if len(mine) < 2:
        pytest.skip("one core: nothing to narrow")
    keep = sorted(mine)[: len(mine) // 2]
    root = fake_sysfs(tmp_path, 0, ",".join(str(c) for c in keep))
    with streaming.near_device(0, root) as node:
        assert node == 0
        assert os.sched_getaffinity(0) == set(keep)
    assert os.sched_getaffinity(0) == mine


def test_near_device_without_common_cores(tmp_path, one_gpu):
    mine = os.sched_getaffinity(0)
    root = fake_sysfs(tmp_path, 0, str(max(mine) + 1000))
    with streaming.near_device(0, root) as node:
        assert node is None and os.sched_getaffinity(0) == mine
    assert os.sched_getaffinity(0) == mine
