"""What this node has for bridges between hosts: one small text file per subject in a directory.

    python -m gpubridge_b200.kit.node_report DIR

``kernel.txt``    kernel release, distribution, the dma-buf / PCI peer-to-peer options of its config;
``modules.txt``   GPU and RDMA kernel modules that are loaded (nvidia, nvidia_peermem, ib_core,
                  mlx5_core, ...), and the driver version;
``rdma.txt``      RDMA devices under /sys/class/infiniband: ports, state, rate, link layer, and
                  whether libibverbs is installed and can register dma-bufs (``ibv_reg_dmabuf_mr``);
``net.txt``       network interfaces: state, MTU, speed, addresses - what ``kit.preflight`` chooses from;
``gpus.txt``      ``nvidia-smi -L`` and the NVLink / NVSwitch matrix (``nvidia-smi topo -m``);
``ucx.txt``       whether libucp is installed (``ucx_info -v`` when the tool is there);
``report.json``   the same facts as data, for ``kit.summarize`` and the tables.

Something that is not there leaves a one-line note instead; the program never fails and changes
nothing on the node (it only reads).  The roots of /sys, /proc, /boot and /etc can be pointed
elsewhere (tests do).  Reference: scripts/gpu/rdma_report.sh, scripts/gpu/net_report.sh.
"""
from __future__ import annotations

import argparse
import ctypes
import ctypes.util
import json
import os
import platform
import shutil
import subprocess
import sys
from pathlib import Path

MODULES = ("nvidia", "nvidia_uvm", "nvidia_peermem", "nv_peer_mem", "gdrdrv", "ib_core", "ib_uverbs",
           "mlx5_core", "mlx5_ib", "rdma_ucm", "rdma_cm")
CONFIG_OPTIONS = ("CONFIG_DMA_SHARED_BUFFER", "CONFIG_DMABUF_MOVE_NOTIFY", "CONFIG_PCI_P2PDMA",
                  "CONFIG_INFINIBAND_USER_MEM", "CONFIG_INFINIBAND_ON_DEMAND_PAGING")


def _read(path: Path) -> str | None:
    try:
        return path.read_text(errors="replace").strip()
    except OSError:
        return None


def _tool(*cmd: str, limit: float = 20.0) -> str | None:
    if shutil.which(cmd[0]) is None:
        return None
    try:
        done = subprocess.run(cmd, capture_output=True, text=True, timeout=limit)
    except (OSError, subprocess.SubprocessError):
        return None
    return (done.stdout or done.stderr).strip()


def kernel(root: Path) -> dict:
    release = platform.release()
    config = _read(root / "boot" / f"config-{release}")
    options = {}
    if config is not None:
        for line in config.splitlines():
            for name in CONFIG_OPTIONS:
                if line.startswith(name + "=") or line == f"# {name} is not set":
                    options[name] = line.split("=", 1)[1] if "=" in line else "not set"
    pretty = None
    for line in (_read(root / "etc" / "os-release") or "").splitlines():
        if line.startswith("PRETTY_NAME="):
            pretty = line.split("=", 1)[1].strip('"')
    return {"release": release, "distribution": pretty,
            "config": options if config is not None else "this kernel's config is not in /boot"}


def modules(root: Path) -> dict:
    loaded = {}
    for line in (_read(root / "proc" / "modules") or "").splitlines():
        fields = line.split()
        if fields and fields[0] in MODULES:
            loaded[fields[0]] = {"size": int(fields[1]), "users": int(fields[2])}
    version = _read(root / "proc" / "driver" / "nvidia" / "version")
    return {"loaded": loaded, "missing": [m for m in MODULES if m not in loaded],
            "nvidia_driver": version.splitlines()[0] if version else None}


def rdma(root: Path, find_library=ctypes.util.find_library) -> dict:
    devices = {}
    base = root / "sys" / "class" / "infiniband"
    if base.is_dir():
        for device in sorted(base.iterdir()):
            ports = {}
            for port in sorted((device / "ports").iterdir()) if (device / "ports").is_dir() else []:
                ports[port.name] = {key: _read(port / key) for key in ("state", "rate", "link_layer", "phys_state")}
            devices[device.name] = {"node_type": _read(device / "node_type"), "fw_ver": _read(device / "fw_ver"),
                                    "ports": ports}
    library = find_library("ibverbs")
    dmabuf = None
    if library:
        try:
            dmabuf = hasattr(ctypes.CDLL(library), "ibv_reg_dmabuf_mr")
        except OSError:
            dmabuf = None
    return {"devices": devices, "libibverbs": library, "ibv_reg_dmabuf_mr": dmabuf,
            "verbs_header": (root / "usr" / "include" / "infiniband" / "verbs.h").exists()}


def net(root: Path) -> dict:
    interfaces = {}
    base = root / "sys" / "class" / "net"
    if base.is_dir():
        for nic in sorted(base.iterdir()):
            speed = _read(nic / "speed")
            interfaces[nic.name] = {"state": _read(nic / "operstate"), "mtu": _read(nic / "mtu"),
                                    "speed_mbps": int(speed) if speed and speed.lstrip("-").isdigit() else None,
                                    "address": _read(nic / "address")}
    return {"interfaces": interfaces, "addresses": (_tool("ip", "-o", "addr") or "").splitlines() or None}


def gpus() -> dict:
    listing = _tool("nvidia-smi", "-L")
    return {"devices": listing.splitlines() if listing else None, "topology": _tool("nvidia-smi", "topo", "-m")}


def ucx(find_library=ctypes.util.find_library) -> dict:
    return {"libucp": find_library("ucp"), "ucx_info": _tool("ucx_info", "-v")}


def _text(title: str, value, indent: int = 0) -> list[str]:
    pad = "  " * indent
    if value is None or value == {} or value == []:
        return [f"{pad}{title}: not found on this node"]
    if isinstance(value, dict):
        lines = [f"{pad}{title}:"]
        for key, inner in value.items():
            lines += _text(str(key), inner, indent + 1)
        return lines
    if isinstance(value, list):
        return [f"{pad}{title}:"] + [f"{pad}  {item}" for item in value]
    text = str(value)
    if "\n" in text:
        return [f"{pad}{title}:"] + [f"{pad}  {line}" for line in text.splitlines()]
    return [f"{pad}{title}: {text}"]


def report(root: Path = Path("/"), find_library=ctypes.util.find_library) -> dict:
    """Everything, as data.  Never raises: a subject that cannot be read says so."""
    out = {}
    for name, fn in (("kernel", lambda: kernel(root)), ("modules", lambda: modules(root)),
                     ("rdma", lambda: rdma(root, find_library)), ("net", lambda: net(root)),
                     ("gpus", gpus), ("ucx", lambda: ucx(find_library))):
        try:
            out[name] = fn()
        except Exception as failure:  # noqa: BLE001 - the report never fails
            out[name] = {"error": f"{type(failure).__name__}: {failure}"}
    return out


def write(directory: Path, facts: dict) -> None:
    directory.mkdir(parents=True, exist_ok=True)
    for name, value in facts.items():
        (directory / f"{name}.txt").write_text("\n".join(_text(name, value)) + "\n")
    (directory / "report.json").write_text(json.dumps({"schema": "gpubridge_b200.node_report/1", **facts}, indent=1))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("directory", type=Path)
    ap.add_argument("--root", type=Path, default=Path("/"), help="where /sys, /proc, /boot and /etc are read from")
    args = ap.parse_args(argv)
    try:
        write(args.directory, report(args.root))
        print(args.directory)
    except OSError as failure:                     # a directory that cannot be written: say so, still exit 0
        print(f"node report not written: {failure}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
