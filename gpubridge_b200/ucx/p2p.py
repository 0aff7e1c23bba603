"""Cross-island point-to-point over UCX: the wire of the P2P engine when the bridge is ``ucx``.

The engine (:mod:`gpubridge_b200.p2p`) does everything that is not the wire - matching, payload
checks, chunking, pinned slots for device tensors, deadlines; a link only has to move one host
buffer per :meth:`UcxLink.post`.  The collective bridge's worker belongs to the island leaders
and to one call at a time, so the link has workers of its own: one two-member worker per PEER,
made when the first message with that peer is posted (both ends do so after the engine has
matched them through the store, so neither waits long for the other's address).  Requests are
waited for by polling, which holds the worker only for the length of a progress call: a slow
transfer on one tag never keeps the engine from posting the next one to the same peer, and
another peer has another worker altogether.  (Reference: src/gpubridge/ucx/p2p.py, one worker
per (source, destination, tag) lane.)
"""
from __future__ import annotations

import base64
import threading
import time
from datetime import timedelta

import torch

from gpubridge_b200 import ucx as _ucx
from gpubridge_b200.tagged import wait_for_keys


class _Request:
    """What the engine's wire pool waits on."""

    def __init__(self, pair: "_Pair", identifier: int, buffer: torch.Tensor) -> None:
        self.pair, self.identifier, self.buffer = pair, identifier, buffer       # the buffer stays alive

    def wait(self, timeout: timedelta) -> None:
        deadline = time.monotonic() + timeout.total_seconds()
        pause = 20e-6
        while not self.pair.poll(self.identifier):
            if time.monotonic() > deadline:
                self.pair.fail()
                raise TimeoutError("a UCX point-to-point message was still in flight at its deadline")
            time.sleep(pause)
            pause = min(pause * 2, 2e-3)


class _Pair:
    """This rank's worker for one peer."""

    def __init__(self, worker: "_ucx.Worker", other: int) -> None:
        self.worker, self.other = worker, other
        self.lock = threading.Lock()
        self.closed = False

    def post(self, buffer: torch.Tensor, tag: int, sending: bool) -> _Request:
        nbytes = buffer.numel() * buffer.element_size()
        with self.lock:
            if self.closed:
                raise RuntimeError("the UCX point-to-point link was closed")
            if sending:
                identifier = self.worker.send(self.other, buffer.data_ptr(), nbytes, tag & (2 ** 64 - 1))
            else:
                identifier = self.worker.recv(self.other, buffer.data_ptr(), nbytes, tag & (2 ** 64 - 1))
        return _Request(self, identifier, buffer)

    def poll(self, identifier: int) -> bool:
        with self.lock:
            if self.closed:
                raise RuntimeError("the UCX point-to-point link was closed")
            return self.worker.poll([identifier])

    def fail(self) -> None:
        with self.lock:
            if not self.closed:
                self.worker.abort()

    def close(self) -> None:
        with self.lock:
            if not self.closed:
                self.closed = True
                self.worker.close(0.5)


class UcxLink:
    """``post(buffer, peer, tag, sending)`` for the engine; host buffers only (the engine stages
    device tensors through pinned slots)."""

    def __init__(self, rank: int, store, timeout: timedelta) -> None:
        self.rank, self.store, self.timeout = rank, store, timeout.total_seconds()
        self.pairs: dict[int, _Pair] = {}
        self.making: dict[int, threading.Lock] = {}
        self.lock = threading.Lock()
        self.closed = False

    def _connect(self, peer: int) -> _Pair:
        low, high = min(self.rank, peer), max(self.rank, peer)
        index = 0 if self.rank == low else 1
        worker = _ucx.Worker(2, index)
        try:
            major, minor, patch = _ucx.version()
            mine = f"{major}.{minor}.{patch}|{base64.b64encode(worker.address()).decode()}"
            self.store.set(f"gb/ucx-p2p/{low}-{high}/{self.rank}", mine)
            told, = wait_for_keys(self.store, [f"gb/ucx-p2p/{low}-{high}/{peer}"],
                                  time.monotonic() + self.timeout, f"rank {peer}'s UCX address")
            version, address = told.split("|", 1)
            if version.split(".")[:2] != [str(major), str(minor)]:
                raise RuntimeError(f"ranks {self.rank} and {peer} run different UCX versions "
                                   f"({major}.{minor} and {version})")
            worker.connect(1 - index, base64.b64decode(address))
            return _Pair(worker, 1 - index)
        except BaseException:
            worker.close(0.5)
            raise

    def _pair(self, peer: int) -> _Pair:
        with self.lock:
            if self.closed:
                raise RuntimeError("the UCX point-to-point link was closed")
            pair = self.pairs.get(peer)
            if pair is not None:
                return pair
            gate = self.making.setdefault(peer, threading.Lock())
        with gate:                                  # one maker per peer; other peers are not held up
            with self.lock:
                pair = self.pairs.get(peer)
            if pair is None:
                pair = self._connect(peer)
                with self.lock:
                    if self.closed:
                        pair.close()
                        raise RuntimeError("the UCX point-to-point link was closed while connecting")
                    self.pairs[peer] = pair
        return pair

    def post(self, buffer: torch.Tensor, peer: int, tag: int, sending: bool) -> _Request:
        if buffer.device.type != "cpu":
            raise ValueError("the UCX point-to-point link carries host buffers")
        return self._pair(peer).post(buffer, tag, sending)

    def close(self) -> None:
        with self.lock:
            if self.closed:
                return
            self.closed = True
            pairs, self.pairs = list(self.pairs.values()), {}
        for pair in pairs:
            pair.close()
