"""Single-process environment probe: what this machine offers before any job starts.

    python -m gpubridge_b200.kit.probe --out results/probe [--allow-no-gpu]

Stages, each recorded in ``probe.json``: GPUs visible to PyTorch; every GPU is a Blackwell
part the native library is built for (compute capability 10.x); the native library exists
(or builds) and loads; its struct layouts match the bindings; the import resolves to this
checkout; every pair of GPUs can address each other's memory (what the fused kernels need);
what NVML reports of the NVLink side (links per GPU, whether they end at an NVSwitch);
``CUDA_VISIBLE_DEVICES`` selects the GPU it names (a child that sees only the last GPU must
find that GPU's PCI address at ``cuda:0`` - one process per GPU depends on it).
A failed stage prints one line on stderr and the exit code is 1.  Same role as the
reference's ``scripts/gpu/probe.py``, ``import_check.py`` and ``device_map.py``.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

from gpubridge_b200.kit import Journal

CHILD = ("import torch; p = torch.cuda.get_device_properties(0) if torch.cuda.device_count() else None; "
         "print('pci=' + (f'{p.pci_bus_id:02x}:{p.pci_device_id:02x}' if p else 'none'))")


def child_pci(visible: str, run=None) -> str:
    """PCI address of ``cuda:0`` in a fresh process that sees only ``visible``."""
    import os
    import subprocess
    run = run or subprocess.run
    done = run([sys.executable, "-c", CHILD], env=dict(os.environ, CUDA_VISIBLE_DEVICES=visible),
               capture_output=True, text=True, timeout=300)
    for line in done.stdout.splitlines():
        if line.startswith("pci="):
            return line[4:]
    raise RuntimeError(f"the child printed no address (exit code {done.returncode}): {done.stderr[-300:]}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", type=Path, required=True)
    ap.add_argument("--allow-no-gpu", action="store_true")
    args = ap.parse_args(argv)
    journal = Journal(args.out / "probe.json", "gpubridge_b200.kit.probe", hang_dump_seconds=0)
    env = journal.data["environment"]
    count = env["device_count"]

    def fail(entry, message):
        entry["ok"] = False
        entry["error"] = message
        print(f"probe: {entry['name']}: {message}", file=sys.stderr)

    with journal.stage("gpus_visible") as e:
        e["device_count"] = count
        if count == 0 and not args.allow_no_gpu:
            fail(e, "no GPU visible to PyTorch (check the GPU request and the driver)")
    with journal.stage("blackwell") as e:
        other = [d for d in env["devices"] if d and not d["capability"].startswith("10.")]
        e["devices"] = [d["name"] for d in env["devices"] if d]
        if other:
            fail(e, f"the native library targets sm_100a; found {[d['name'] for d in other]}")
    with journal.stage("native_library") as e:
        try:
            from gpubridge_b200.ops import _build, _lib
            e["path"] = _build.LIB
            e["prebuilt"] = _lib.available()
            if count or _lib.available():
                handle = _lib.lib()
                e["sizeof"] = {"team": handle.gb_sizeof_team(), "args": handle.gb_sizeof_args(),
                               "ctrl": handle.gb_sizeof_ctrl()}
            else:
                e["skipped"] = "no GPU and no built library"
        except Exception as exc:  # noqa: BLE001
            fail(e, f"{type(exc).__name__}: {exc}")
    with journal.stage("cpp_front_end") as e:
        try:
            from gpubridge_b200.ops import _build_c10d
            e["path"], e["stale"] = _build_c10d.OUT, _build_c10d.stale()
            if e["stale"]:
                e["skipped"] = "not built for these sources (python -m gpubridge_b200.ops._build_c10d)"
            else:
                e["loaded"] = hasattr(_build_c10d.load(), "GbBackend")
                if not e["loaded"]:
                    fail(e, "gb_c10d.so loaded without its backend class")
        except Exception as exc:  # noqa: BLE001
            fail(e, f"{type(exc).__name__}: {exc}")
    with journal.stage("import") as e:
        import gpubridge_b200
        here = Path(__file__).resolve().parents[1]
        e["imported_from"] = str(Path(gpubridge_b200.__file__).resolve().parent)
        if Path(gpubridge_b200.__file__).resolve().parent != here:
            fail(e, f"import gpubridge_b200 resolved outside this checkout ({here})")
    with journal.stage("peer_access") as e:
        if count >= 2:
            import torch
            blocked = [(a, b) for a in range(count) for b in range(count)
                       if a != b and not torch.cuda.can_device_access_peer(a, b)]
            e["pairs_checked"] = count * (count - 1)
            if blocked:
                fail(e, f"GPU pairs without peer access: {blocked[:8]} - the fused kernels need it")
        else:
            e["skipped"] = "fewer than two GPUs"
    with journal.stage("nvlink") as e:
        from gpubridge_b200.utils.links import link_layout
        layout = link_layout() if count else None
        if layout is None:
            e["skipped"] = "no GPU or no NVML"
        else:
            e.update(layout)
            # reported, never a failure: peer access (above) is what decides whether the fused
            # kernels can run; this says what kind of box the numbers come from
            if count >= 2 and layout["fabric"] == "none":
                e["warning"] = "NVML reports no active NVLink: peer traffic would cross PCIe"
            elif layout["links_uneven"]:
                e["warning"] = ("GPUs report different numbers of active NVLink links: "
                                f"{[g['links_active'] for g in layout['gpus']]}")
    with journal.stage("device_map") as e:
        if count >= 2:
            import os
            names = os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")
            last = names[count - 1] if len(names) == count and names[0] else str(count - 1)
            want = env["devices"][count - 1]["pci_bus_id"]
            e["selected"], e["expected_pci"] = last, want
            try:
                e["child_pci"] = child_pci(last)
                if e["child_pci"] != want:
                    fail(e, f"CUDA_VISIBLE_DEVICES={last} gave the child the GPU at {e['child_pci']}, "
                            f"not the one at {want}: ranks would not sit on the GPUs they are given")
            except Exception as exc:  # noqa: BLE001
                fail(e, f"{type(exc).__name__}: {exc}")
        else:
            e["skipped"] = "fewer than two GPUs"
    return journal.close()


if __name__ == "__main__":
    sys.exit(main())
