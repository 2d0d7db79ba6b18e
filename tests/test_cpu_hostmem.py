"""Host-side placement helper of the host-buffer path: parsing and planning against a fake sysfs tree."""
from miroxen_b200 import hostmem as hm


def fake_sysfs(tmp_path, node, cpulists):
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text(f"{node}\n")
    for n, text in cpulists.items():
        d = tmp_path / "devices" / "system" / "node" / f"node{n}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(text + "\n")
    return tmp_path


def test_parse_cpulist():
    assert hm.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert hm.parse_cpulist("5") == [5]
    assert hm.parse_cpulist("") == []


def test_pci_address_format():
    assert hm.pci_address(0, 0x1b, 0) == "0000:1b:00.0"
    assert hm.pci_address(1, 0xa, 0x1f) == "0001:0a:1f.0"


def test_plan_binds_to_the_devices_node_within_the_allowed_set(tmp_path):
    root = fake_sysfs(tmp_path, 1, {0: "0-3", 1: "4-7"})
    plan = hm.plan_binding("0000:1b:00.0", {0, 1, 4, 5, 6}, root)
    assert plan["node"] == 1 and plan["cpus"] == [4, 5, 6] and plan["why"] == "bound"


def test_plan_does_nothing_without_a_numa_answer(tmp_path):
    root = fake_sysfs(tmp_path, -1, {0: "0-7"})
    plan = hm.plan_binding("0000:1b:00.0", set(range(8)), root)
    assert plan["node"] is None and plan["cpus"] == []
    plan = hm.plan_binding("0000:ff:00.0", set(range(8)), root)      # unknown device
    assert plan["node"] is None and plan["cpus"] == []


def test_plan_never_widens_the_allowed_set(tmp_path):
    root = fake_sysfs(tmp_path, 1, {0: "0-3", 1: "4-7"})
    plan = hm.plan_binding("0000:1b:00.0", {0, 1}, root)             # the node's CPUs are all outside the cgroup
    assert plan["node"] == 1 and plan["cpus"] == [] and "available" in plan["why"]
