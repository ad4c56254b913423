"""Provider probing and adapter / GID / port selection against a fake sysfs tree.

The machine has no adapter, so the tree the kernel would publish is built under a
temporary directory: two mlx5 functions behind different PCI switches (one
InfiniBand, one RoCE with a GID table), an EFA function, and two GPUs.  Provider
libraries are stand-ins that export only the marker symbol.
"""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

from aboleth_b200 import runtime
from aboleth_b200.runtime import Provider


def _hca(root: Path, name: str, pci: str, driver: str):
    function = root / "devices" / pci
    function.mkdir(parents=True, exist_ok=True)
    drivers = root / "bus" / "pci" / "drivers" / driver
    drivers.mkdir(parents=True, exist_ok=True)
    if not (function / "driver").exists():
        os.symlink(drivers, function / "driver")
    node = root / "class" / "infiniband" / name
    node.mkdir(parents=True)
    os.symlink(function, node / "device")
    return node


def _port(node: Path, port: int, link_layer: str, lid: str, gids: dict, netdev: str = ""):
    base = node / "ports" / str(port)
    (base / "gids").mkdir(parents=True)
    (base / "gid_attrs" / "types").mkdir(parents=True)
    (base / "gid_attrs" / "ndevs").mkdir(parents=True)
    (base / "link_layer").write_text(link_layer + "\n")
    (base / "lid").write_text(lid + "\n")
    for index, (gid, kind) in gids.items():
        (base / "gids" / str(index)).write_text(gid + "\n")
        (base / "gid_attrs" / "types" / str(index)).write_text(kind + "\n")
        if netdev:
            (base / "gid_attrs" / "ndevs" / str(index)).write_text(netdev + "\n")


@pytest.fixture
def sysfs(tmp_path, monkeypatch):
    root = tmp_path / "sys"
    # Two PCI switches under two root ports; a GPU and an adapter behind each.
    a = "pci0000:10/0000:10:01.0/0000:11:00.0"
    b = "pci0000:80/0000:80:01.0/0000:81:00.0"
    ib = _hca(root, "mlx5_0", f"{a}/0000:12:00.0/0000:13:00.0", "mlx5_core")
    roce = _hca(root, "mlx5_1", f"{b}/0000:82:00.0/0000:83:00.0", "mlx5_core")
    _hca(root, "rdmap16s27", "pci0000:00/0000:00:1b.0", "efa")
    _port(ib, 1, "InfiniBand", "0x002a", {0: ("fe80:0000:0000:0000:0002:c903:00ab:cdef", "IB/RoCE v1")})
    zero = "0000:0000:0000:0000:0000:0000:0000:0000"
    _port(roce, 1, "Ethernet", "0x0000", {
        0: ("fe80:0000:0000:0000:0ac0:ebff:fe12:3456", "IB/RoCE v1"),
        1: ("fe80:0000:0000:0000:0ac0:ebff:fe12:3456", "RoCE v2"),
        2: ("0000:0000:0000:0000:0000:ffff:0a00:0105", "IB/RoCE v1"),
        3: ("0000:0000:0000:0000:0000:ffff:0a00:0105", "RoCE v2"),
        4: (zero, "RoCE v2")}, netdev="eth7")
    (root / "class" / "net" / "eth7").mkdir(parents=True)
    (root / "class" / "net" / "eth7" / "mtu").write_text("9000\n")
    devices = root / "bus" / "pci" / "devices"
    devices.mkdir(parents=True, exist_ok=True)
    for bus_id, path in (("0000:14:00.0", f"{a}/0000:12:01.0/0000:14:00.0"),
                         ("0000:84:00.0", f"{b}/0000:82:01.0/0000:84:00.0")):
        (root / "devices" / path).mkdir(parents=True)
        os.symlink(root / "devices" / path, devices / bus_id)
    monkeypatch.setenv("ABOLETH_SYSFS_ROOT", str(root))
    monkeypatch.setenv("ABOLETH_GPU_PCI_BUS_IDS", "0000:14:00.0,0000:84:00.0")
    for name in ("ABOLETH_HCA", "ABOLETH_PORT", "ABOLETH_GID_INDEX", "ABOLETH_PATH_MTU"):
        monkeypatch.delenv(name, raising=False)
    return root


def test_nearest_adapter_follows_the_pci_path(sysfs, monkeypatch):
    assert runtime.select_device(0) == "mlx5_0"
    assert runtime.select_device(1) == "mlx5_1"
    assert runtime.select_device(-1) == "mlx5_0"  # topology-free default: first in name order
    monkeypatch.setenv("ABOLETH_HCA", "mlx5_1")
    assert runtime.select_device(0) == "mlx5_1"
    monkeypatch.setenv("ABOLETH_HCA", "mlx5_9")
    with pytest.raises(RuntimeError, match="ABOLETH_HCA names 'mlx5_9'"):
        runtime.select_device(0)
    monkeypatch.delenv("ABOLETH_HCA")
    with pytest.raises(RuntimeError, match="no bus id for CUDA ordinal 5"):
        runtime.select_device(5)


def test_gid_choice_and_port_address(sysfs, monkeypatch):
    assert runtime.select_gid_index("mlx5_0") == 0  # InfiniBand
    assert runtime.select_gid_index("mlx5_1") == 3  # RoCE v2, IPv4-mapped entry first
    assert runtime.select_gid_index() == 0  # default adapter
    ib = runtime.query_port_address("mlx5_0")
    assert (ib.lid, ib.link_layer, ib.gid_index, ib.path_mtu, ib.is_global) == (0x2a, 1, 0, 5, False)
    assert ib.gid.hex() == "fe800000000000000002c90300abcdef"
    roce = runtime.query_port_address("mlx5_1", 1)
    assert (roce.lid, roce.link_layer, roce.gid_index, roce.is_global) == (0, 2, 3, True)
    assert roce.gid.hex() == "00000000000000000000ffff0a000105"
    assert roce.path_mtu == 5 and roce.path_mtu_bytes == 4096  # a 9000-byte netdev carries 4096
    monkeypatch.setenv("ABOLETH_PATH_MTU", "1024")
    assert runtime.query_port_address("mlx5_1").path_mtu == 3
    monkeypatch.setenv("ABOLETH_PATH_MTU", "1000")
    with pytest.raises(RuntimeError, match="ABOLETH_PATH_MTU must be"):
        runtime.query_port_address("mlx5_1")
    monkeypatch.delenv("ABOLETH_PATH_MTU")
    monkeypatch.setenv("ABOLETH_GID_INDEX", "1")
    assert runtime.query_port_address("mlx5_1").gid_index == 1
    monkeypatch.delenv("ABOLETH_GID_INDEX")
    (sysfs / "class" / "net" / "eth7" / "mtu").write_text("1500\n")
    assert runtime.query_port_address("mlx5_1").path_mtu == 3  # 1500 - headers -> 1024
    with pytest.raises(RuntimeError, match="has no port 2"):
        runtime.select_gid_index("mlx5_0", 2)
    with pytest.raises(RuntimeError, match="adapter 'mlx5_7' is not present"):
        runtime.select_gid_index("mlx5_7")


def test_probe_needs_both_the_library_and_a_device(sysfs, tmp_path, monkeypatch):
    if shutil.which("gcc") is None:
        pytest.skip("needs gcc for the stand-in libraries")
    for name in ("IBVERBS", "MLX5", "EFA", "FABRIC"):  # whatever the machine has installed stays out of it
        monkeypatch.setenv(f"ABOLETH_DL_{name}", str(tmp_path / "absent.so"))
    assert runtime.probe_providers() & (Provider.VERBS | Provider.MLX5 | Provider.EFA) == 0  # no libraries

    def stand_in(name: str, symbol: str) -> str:
        src = tmp_path / f"{name}.c"
        src.write_text(f"int {symbol}(void) {{ return 0; }}\n")
        out = tmp_path / f"lib{name}.so"
        subprocess.run(["gcc", "-shared", "-fPIC", str(src), "-o", str(out)], check=True)
        return str(out)

    monkeypatch.setenv("ABOLETH_DL_IBVERBS", stand_in("ibverbs", "ibv_get_device_list"))
    assert runtime.probe_providers() & (Provider.VERBS | Provider.MLX5) == Provider.VERBS
    monkeypatch.setenv("ABOLETH_DL_MLX5", stand_in("mlx5", "mlx5dv_init_obj"))
    monkeypatch.setenv("ABOLETH_DL_EFA", stand_in("efa", "some_other_symbol"))  # resolves, wrong library
    bits = runtime.probe_providers()
    assert bits & Provider.MLX5 and not bits & Provider.EFA
    # What the build can drive does not change: adapters are served through the ring.
    assert runtime.provider_caps() & (Provider.VERBS | Provider.MLX5) == 0
    # Without devices the libraries alone report nothing.
    shutil.rmtree(sysfs / "class" / "infiniband")
    assert runtime.probe_providers() & (Provider.VERBS | Provider.MLX5) == 0


def test_no_provider_library_is_a_link_time_dependency():
    from aboleth_b200 import _native

    if shutil.which("readelf") is None:
        pytest.skip("needs readelf")
    for name in ("runtime", "kernels", "spec"):
        dynamic = subprocess.run(["readelf", "-d", str(_native.library_path(name))],
                                 capture_output=True, text=True, check=True).stdout
        needed = [line for line in dynamic.splitlines() if "(NEEDED)" in line]
        for provider in ("ibverbs", "mlx5", "libefa", "libfabric", "libcuda.so", "amdhip", "nccl", "nvshmem"):
            assert not any(provider in line for line in needed), (name, provider, needed)
