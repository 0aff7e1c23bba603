"""TEST ONLY: give a one-vendor job several islands by relabelling ranks.

The ranks keep their GPU, NCCL and true build; only the island layout changes, which is
how one 8xB200 box exercises islands, leaders and the bridge (reference:
src/gpubridge/split_test.py:28-79).  B200 addition: :func:`island_labels` makes any number
of islands from explicit sizes (``GPUBRIDGE_ISLANDS=2,2,2,2``).
"""
from __future__ import annotations

from collections.abc import Sequence

from gpubridge_b200.config import ISLANDS_ENV, SPLIT_TEST_ENV, SPLIT_TEST_MODES


class SplitTestWarning(UserWarning):
    """Raised as a warning on every rank of a relabelled run."""


def _other(vendor: str) -> str:
    return "amd" if vendor == "nvidia" else "nvidia"


def split_labels(vendors: Sequence[str], hostnames: Sequence[str], mode: str) -> list[str]:
    """Island label per rank: ``half`` flips the upper half, ``alternate`` the odd ranks,
    ``node`` every second host (hosts ordered by their lowest rank)."""
    if mode not in SPLIT_TEST_MODES:
        raise ValueError(f"unknown split-test mode {mode!r}")
    world = len(vendors)
    if world < 2:
        raise RuntimeError(f"{SPLIT_TEST_ENV} needs at least 2 ranks, got {world}")
    present = sorted(set(vendors))
    if len(present) != 1:
        raise RuntimeError(f"{SPLIT_TEST_ENV} only splits a single-vendor job, but this job "
                           f"already has {' and '.join(present)} ranks. Unset it for a real "
                           "mixed-vendor run.")
    if mode == "half":
        flip = [r >= (world + 1) // 2 for r in range(world)]
    elif mode == "alternate":
        flip = [r % 2 == 1 for r in range(world)]
    else:
        order = list(dict.fromkeys(hostnames))
        if len(order) < 2:
            raise RuntimeError(f"{SPLIT_TEST_ENV}=node splits islands by machine but every "
                               f"rank runs on {order[0]}. Use half or alternate on one machine.")
        flip = [order.index(h) % 2 == 1 for h in hostnames]
    return [_other(v) if f else v for v, f in zip(vendors, flip)]


def island_labels(vendors: Sequence[str], sizes: Sequence[int]) -> list[str]:
    """Labels for explicit island sizes: consecutive ranks, island i labelled
    ``<vendor>`` (i = 0), ``<other vendor>`` (i = 1), then ``<vendor>#i``."""
    world = len(vendors)
    if sum(sizes) != world:
        raise RuntimeError(f"{ISLANDS_ENV}={','.join(map(str, sizes))} names {sum(sizes)} "
                           f"ranks but the job has {world}")
    if len(set(vendors)) != 1:
        raise RuntimeError(f"{ISLANDS_ENV} only relabels a single-vendor job")
    vendor = vendors[0]
    names = [vendor, _other(vendor)] + [f"{vendor}#{i}" for i in range(2, len(sizes))]
    return [names[i] for i, n in enumerate(sizes) for _ in range(n)]


def banner(mode: str, vendors: Sequence[str], labels: Sequence[str]) -> str:
    moved = [r for r, (v, l) in enumerate(zip(vendors, labels)) if v != l]
    return (f"{SPLIT_TEST_ENV}={mode}: TEST-ONLY split of a single-vendor job. Ranks {moved} run "
            f"{vendors[0]} builds but carry other island labels to exercise islands and the "
            "bridge. This is NOT a mixed-vendor run; do not report its results as one.")
