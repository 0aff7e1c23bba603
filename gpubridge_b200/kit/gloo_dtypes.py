"""Which element types Gloo's all_reduce (SUM) and broadcast really handle in this torch build.

    python -m gpubridge_b200.kit.gloo_dtypes [OUT.json]

This is what stands behind :data:`gpubridge_b200.collectives.SUPPORTED_DTYPES`: a type is
supported by the library only if it works on every path, and Gloo - the world group, the bridge
of CPU simulation, the cross-node fallback - is the narrowest.  Two CPU processes contribute
small integers, so a correct sum is exact; the broadcast is checked from rank 1.  A type Gloo
rejects is recorded with its message, one it gets WRONG (bool's sum is a logical OR) with what
came out.  Run it in every torch version the package is to support; the exit code is 1 when a
type the library promises fails here.  (Reference: scripts/gloo_dtypes.py.)
"""
from __future__ import annotations

import json
import sys
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

EXTRAS = ("bool", "int16", "uint16", "uint32", "complex64", "float8_e4m3fn")


def candidates() -> list[str]:
    from gpubridge_b200.collectives import SUPPORTED_DTYPES
    return [str(d).removeprefix("torch.") for d in SUPPORTED_DTYPES] + [n for n in EXTRAS if hasattr(torch, n)]


def values(dtype: torch.dtype, rank: int) -> torch.Tensor:
    if dtype == torch.bool:
        return torch.tensor([True, rank == 0, False, rank == 1])
    return (torch.arange(6) % 3 + rank + 1).to(dtype)


def same(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.dtype == b.dtype and torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def _member(rank: int, path: str, names: list[str], out) -> None:
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=2)
    rows = {}
    for name in names:
        dtype = getattr(torch, name)
        row = {}
        for op in ("all_reduce", "broadcast"):
            try:
                mine = values(dtype, rank)
                if op == "all_reduce":
                    dist.all_reduce(mine)
                    if dtype == torch.bool:
                        want = values(dtype, 0) | values(dtype, 1)
                    else:
                        want = (values(torch.float64, 0) + values(torch.float64, 1)).to(dtype)
                else:
                    dist.broadcast(mine, 1)
                    want = values(dtype, 1)
                row[op] = "ok" if same(mine, want) else f"WRONG: got {mine.tolist()}, want {want.tolist()}"
            except Exception as failure:  # noqa: BLE001 - the answer we are after
                row[op] = f"refused: {type(failure).__name__}: {str(failure).splitlines()[0][:120]}"
        rows[name] = row
    if rank == 0:
        out.put(rows)
    dist.barrier()
    dist.destroy_process_group()


def survey(names: list[str] | None = None) -> dict:
    names = names or candidates()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    with tempfile.TemporaryDirectory() as scratch:
        members = [ctx.Process(target=_member, args=(r, f"{scratch}/rdzv", names, out)) for r in (0, 1)]
        for m in members:
            m.start()
        rows = out.get(timeout=120)
        for m in members:
            m.join(30)
    return {"torch": torch.__version__, "rows": rows}


def verdict(found: dict) -> list[str]:
    """The promised types that do not work here (empty: the table holds)."""
    from gpubridge_b200.collectives import SUPPORTED_DTYPES
    promised = [str(d).removeprefix("torch.") for d in SUPPORTED_DTYPES]
    return [name for name in promised
            if any(found["rows"].get(name, {}).get(op) != "ok" for op in ("all_reduce", "broadcast"))]


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if argv and argv[0].startswith("-"):
        print(__doc__)
        return 0 if argv[0] in ("-h", "--help") else 2
    found = survey()
    width = max(len(n) for n in found["rows"])
    print(f"torch {found['torch']}")
    for name, row in found["rows"].items():
        print(f"  {name:<{width}}  all_reduce: {row['all_reduce']:<12.60}  broadcast: {row['broadcast']:.60}")
    broken = verdict(found)
    found["promised_but_failing"] = broken
    if argv:
        with open(argv[0], "w") as fh:
            json.dump(found, fh, indent=1)
    print("the supported-types table holds here" if not broken else f"PROMISED BUT FAILING: {', '.join(broken)}")
    return 1 if broken else 0


if __name__ == "__main__":
    sys.exit(main())
