"""The registrar of device memory for direct adapter access (``csrc/gb_direct.cpp``) over pretend
device memory and a pretend adapter: which method is chosen and why not, every reason when none
works, the cache's identity (allocation, not address), rounding inside the allocation, eviction
that spares what is in use, invalidation now or at the last release, descriptors closed exactly
once, and one-receive windows.  (Reference: the unit tests of the verbs crate's direct.rs.)"""
import pytest

from gpubridge_b200.ops import _lib

pytestmark = pytest.mark.skipif(not _lib.available() or not hasattr(_lib.lib(), "gb_direct_new"),
                                reason="the native library is not built")
MB = 1 << 20


@pytest.fixture
def modules(tmp_path):
    def write(*names):
        (tmp_path / "proc").mkdir(exist_ok=True)
        (tmp_path / "proc" / "modules").write_text("".join(f"{n} 16384 0 - Live 0x0\n" for n in names))
        return str(tmp_path)
    return write


@pytest.fixture
def registrar(modules):
    from gpubridge_b200.rdma_direct import Registrar
    made = Registrar.pretend(modules("nvidia", "nvidia_peermem"), capacity=3)
    yield made
    made.close()


def test_dma_buf_first_then_peer_memory_then_every_reason(registrar):
    from gpubridge_b200.rdma_direct import NotDirect
    a = registrar.alloc(8 * MB)
    with registrar.acquire(a, MB) as region:
        assert region.method == "dma-buf" and region.lo == a and region.hi == a + 2 * MB
    assert "dma-buf: yes; peer memory: yes (nvidia_peermem)" == registrar.capabilities()
    registrar.invalidate(a, 8 * MB)
    registrar.fail("device dma-buf", "needs the open kernel modules")
    with registrar.acquire(a, MB) as region:
        assert region.method == "peer memory"
    assert registrar.capabilities().startswith("dma-buf: no (needs the open kernel modules)")
    registrar.invalidate(a, 8 * MB)
    registrar.fail("adapter pointer", "ibv_reg_mr: Bad address")
    with pytest.raises(NotDirect) as caught:
        registrar.take(a, MB)
    assert str(caught.value) == "dma-buf: needs the open kernel modules; peer memory: ibv_reg_mr: Bad address"
    registrar.fail("device dma-buf")                               # switched back on
    registrar.fail("export", "out of descriptors")
    with pytest.raises(NotDirect, match="dma-buf: out of descriptors; peer memory: ibv_reg_mr"):
        registrar.take(a, MB)
    registrar.fail("export")
    registrar.fail("adapter dma-buf", "ibv_reg_dmabuf_mr: Operation not supported")
    with pytest.raises(NotDirect, match="Operation not supported"):
        registrar.take(a, MB)
    counts = registrar.counts()
    assert counts["descriptors_open"] == 0 and counts["descriptors_closed_twice"] == 0     # the refused export was closed


def test_without_a_peer_memory_module_only_dma_buf_can_work(modules):
    from gpubridge_b200.rdma_direct import NotDirect, Registrar
    registrar = Registrar.pretend(modules("nvidia", "mlx5_core"))
    try:
        a = registrar.alloc(4 * MB)
        with registrar.acquire(a, 100) as region:
            assert region.method == "dma-buf"
        registrar.invalidate(a, 4 * MB)
        registrar.fail("device dma-buf", "not exported here")
        with pytest.raises(NotDirect, match="peer memory: neither nvidia_peermem nor nv_peer_mem is loaded"):
            registrar.take(a, 100)
        assert "peer memory: no (no peer-memory module is loaded)" in registrar.capabilities()
    finally:
        registrar.close()
    older = Registrar.pretend(modules("nv_peer_mem"))              # the older module's name counts too
    try:
        older.fail("device dma-buf", "no")
        with older.acquire(older.alloc(MB), 10) as region:
            assert region.method == "peer memory"
    finally:
        older.close()


def test_what_is_not_one_allocation_is_refused(registrar):
    from gpubridge_b200.rdma_direct import NotDirect
    a = registrar.alloc(MB)
    with pytest.raises(NotDirect, match="not device memory"):
        registrar.take(0x1234, 16)
    with pytest.raises(NotDirect, match="spans more than one"):
        registrar.take(a + MB - 8, 16)
    with pytest.raises(NotDirect, match="empty range"):
        registrar.take(a, 0)
    registrar.free(a)
    with pytest.raises(NotDirect, match="not device memory"):
        registrar.take(a, 16)


def test_neighbouring_tensors_of_one_allocation_share_a_registration(registrar):
    a = registrar.alloc(16 * MB)
    first = registrar.take(a + 100, 1000)
    second = registrar.take(a + MB, 1000)                          # inside the same 2 MiB
    third = registrar.take(a + 3 * MB, 10)                         # another 2 MiB of the same allocation
    assert first.key == second.key != third.key
    assert (first.lo, first.hi) == (a, a + 2 * MB) and (third.lo, third.hi) == (a + 2 * MB, a + 4 * MB)
    told = registrar.telemetry()
    assert told["hits"] == 1 and told["misses"] == 2 and told["cached"] == 2 and told["held"] == 2
    for region in (first, second, third):
        registrar.give_back(region)
    with pytest.raises(ValueError, match="given back already"):
        registrar.give_back(first)
    assert registrar.telemetry()["held"] == 0
    small = registrar.alloc(1000)                                  # rounding never leaves the allocation
    with registrar.acquire(small + 10, 100) as region:
        assert (region.lo, region.hi) == (small, small + 1000)


def test_the_same_address_in_a_later_allocation_is_another_owner(registrar):
    from gpubridge_b200.rdma_direct import NotDirect
    a = registrar.alloc(4 * MB)
    with registrar.acquire(a, MB) as old:
        pass
    registrar.free(a)
    again = registrar.alloc(4 * MB, at=a)                          # the allocator hands the address out again
    assert again == a
    with registrar.acquire(a, MB) as new:
        assert new.key != old.key                                  # not the stale registration
    told = registrar.telemetry()
    assert told["stale_dropped"] == 1 and told["misses"] == 2 and told["hits"] == 0
    # ... and while posted work still holds the old one, the new owner is refused rather than mixed up
    held = registrar.take(a, MB)
    registrar.free(a)
    registrar.alloc(4 * MB, at=a)
    with pytest.raises(NotDirect, match="still held by posted work"):
        registrar.take(a, MB)
    registrar.give_back(held)
    with registrar.acquire(a, MB):
        pass
    assert registrar.telemetry()["refusals"] == 1


def test_eviction_spares_what_is_in_use_and_closes_descriptors_once(registrar):
    allocations = [registrar.alloc(2 * MB) for _ in range(6)]
    held = registrar.take(allocations[0], 100)                     # the oldest, but in use
    for a in allocations[1:]:
        with registrar.acquire(a, 100):
            pass
    told = registrar.telemetry()
    assert told["cached"] == 3 and told["evictions"] == 3          # capacity 3, six made
    with registrar.acquire(allocations[0], 100) as same:
        assert same.key == held.key                                # it survived every eviction
    registrar.give_back(held)
    counts = registrar.counts()
    assert counts["exports"] == 6 and counts["descriptors_open"] == 3 and counts["descriptors_closed_twice"] == 0
    assert counts["registrations_alive"] == 3 and counts["registrations_released"] == 3


def test_invalidation_is_immediate_when_idle_and_deferred_while_held(registrar):
    a = registrar.alloc(8 * MB)
    with registrar.acquire(a, 100):
        pass
    assert registrar.invalidate(a + 50, 10) == 1 and registrar.telemetry()["cached"] == 0
    assert registrar.invalidate(a, 8 * MB) == 0
    held = registrar.take(a, 100)
    assert registrar.invalidate(a, 8 * MB) == 1
    assert registrar.counts()["registrations_alive"] == 1          # still there: work is posted with it
    fresh = registrar.take(a, 100)                                 # but nobody new gets the doomed one
    assert fresh.key != held.key
    registrar.give_back(held)
    assert registrar.counts()["registrations_alive"] == 1          # the doomed one went with its last holder
    registrar.give_back(fresh)
    assert registrar.telemetry()["cached"] == 1


def test_a_window_is_exactly_one_receive_and_never_cached(registrar):
    from gpubridge_b200.rdma_direct import NotDirect
    a = registrar.alloc(8 * MB)
    with registrar.acquire(a, 8 * MB) as cached:
        window, key = registrar.expose(a + 4096, 65536)
        other, other_key = registrar.expose(a + 4096, 65536)       # the same bytes again: another window, another key
        assert key != cached.key and other_key not in (key, cached.key)
        told = registrar.telemetry()
        assert told["windows_open"] == 2 and told["windows_made"] == 2 and told["cached"] == 1
        registrar.close_window(window)
        registrar.close_window(other)
        with pytest.raises(ValueError, match="no such window"):
            registrar.close_window(window)
    told = registrar.telemetry()
    assert told["windows_open"] == 0 and told["write_window_register_ns"] > 0 and told["write_window_release_ns"] > 0
    with pytest.raises(NotDirect, match="inside one allocation"):
        registrar.expose(a + 8 * MB - 10, 100)
    registrar.fail("device dma-buf", "no")
    registrar.fail("device peer memory", "GPUDirect RDMA is off")
    with pytest.raises(NotDirect, match="dma-buf: no; peer memory: GPUDirect RDMA is off"):
        registrar.expose(a, 100)


def test_closing_the_registrar_releases_everything(modules):
    from gpubridge_b200.rdma_direct import Registrar
    registrar = Registrar.pretend(modules("nvidia_peermem"))
    a = registrar.alloc(4 * MB)
    registrar.take(a, 100)
    registrar.expose(a, 100)
    assert registrar.counts()["registrations_alive"] == 2
    registrar.close()
    registrar.close()                                              # twice is fine


def test_on_a_machine_without_the_driver_every_reason_names_it():
    from gpubridge_b200.rdma_direct import NotDirect, Registrar
    import ctypes.util
    if ctypes.util.find_library("cuda"):
        pytest.skip("this machine has the CUDA driver")
    registrar = Registrar.on_this_machine()
    try:
        with pytest.raises(NotDirect, match="libcuda.so.1 cannot be loaded"):
            registrar.take(0x7000_0000, 4096)
        assert "libcuda.so.1 cannot be loaded" in registrar.capabilities()
    finally:
        registrar.close()


def test_the_router_asks_the_registrar_and_passes_its_reasons_on(registrar):
    """A device tensor goes in place only when its own range can be registered; otherwise the
    route is ``bounce`` and says why in the registrar's words."""
    from types import SimpleNamespace

    from gpubridge_b200 import gdr
    from gpubridge_b200.rdma_transport import Router

    ordered = lambda device: gdr.FlushPlan(device, True, False, "completed writes are ordered: no flush")   # noqa: E731
    router = Router(direct_min_bytes=1024, flush_plans=ordered, registrar=registrar)
    a = registrar.alloc(4 * MB)

    def tensor(pointer, nbytes, contiguous=True):
        return SimpleNamespace(device=SimpleNamespace(type="cuda", index=0), nbytes=nbytes,
                               is_contiguous=lambda: contiguous, data_ptr=lambda: pointer)

    route = router.route(tensor(a, MB))
    assert route.how == "in-place" and route.why.startswith("registered through dma-buf")
    assert router.route(tensor(a, 100)).how == "bounce"                            # too small to be worth it
    assert router.route(tensor(a, MB, contiguous=False)).how == "bounce"
    stray = router.route(tensor(0x5000, MB))
    assert stray.how == "bounce" and "not device memory" in stray.why
    registrar.invalidate(a, 4 * MB)
    registrar.fail("device dma-buf", "closed driver")
    registrar.fail("device peer memory", "not allowed")
    refused = router.route(tensor(a, MB))
    assert refused.how == "bounce" and "dma-buf: closed driver; peer memory: not allowed" in refused.why
    assert router.counts == {"in-place": 1, "bounce": 4}
    assert registrar.telemetry()["held"] == 0                                      # deciding holds nothing


def test_a_method_can_be_switched_off_by_the_user(modules, monkeypatch):
    from gpubridge_b200.rdma_direct import NotDirect, Registrar
    monkeypatch.setenv("GPUBRIDGE_VERBS_DMABUF", "0")
    registrar = Registrar.pretend(modules("nvidia_peermem"))
    try:
        a = registrar.alloc(4 * MB)
        with registrar.acquire(a, MB) as region:
            assert region.method == "peer memory"
        assert registrar.capabilities().startswith("dma-buf: no (switched off by GPUBRIDGE_VERBS_DMABUF)")
        assert registrar.counts()["exports"] == 0                  # not even tried
        registrar.invalidate(a, 4 * MB)
        registrar.switch_off("peer memory", "not on this cluster")
        with pytest.raises(NotDirect, match="dma-buf: switched off by GPUBRIDGE_VERBS_DMABUF; peer memory: not on this cluster"):
            registrar.take(a, MB)
        registrar.switch_off("dma-buf", "")                         # back on
        with registrar.acquire(a, MB) as region:
            assert region.method == "dma-buf"
    finally:
        registrar.close()
    monkeypatch.setenv("GPUBRIDGE_VERBS_DMABUF", "perhaps")
    with pytest.raises(ValueError, match="GPUBRIDGE_VERBS_DMABUF"):
        Registrar.pretend(modules("nvidia_peermem"))


def test_many_threads_share_the_registrar(modules):
    """Acquire, expose, invalidate and release from eight threads at once: every registration that
    was made is released again, no descriptor is closed twice and the counts add up."""
    import threading

    from gpubridge_b200.rdma_direct import NotDirect, Registrar
    registrar = Registrar.pretend(modules("nvidia_peermem"), capacity=4)
    allocations = [registrar.alloc(8 * MB) for _ in range(6)]
    errors = []

    def work(seed):
        try:
            for step in range(300):
                a = allocations[(seed + step) % len(allocations)]
                offset = ((seed * 7 + step) % 4) * 2 * MB
                try:
                    with registrar.acquire(a + offset, 1000) as region:
                        assert region.lo <= a + offset and a + offset + 1000 <= region.hi
                        if step % 5 == 0:
                            window, _ = registrar.expose(a + offset, 512)
                            registrar.close_window(window)
                except NotDirect as refused:
                    assert "still held" in str(refused)
                if step % 37 == 0:
                    registrar.invalidate(a, 8 * MB)
        except BaseException as failure:  # noqa: BLE001
            errors.append(repr(failure))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors, errors[:3]
    told, counts = registrar.telemetry(), registrar.counts()
    assert told["held"] == 0 and told["windows_open"] == 0 and told["cached"] <= 4
    assert told["hits"] + told["misses"] + told["refusals"] == 8 * 300
    assert counts["descriptors_closed_twice"] == 0 and counts["registrations_alive"] == told["cached"]
    assert counts["descriptors_open"] == told["cached"]
    assert counts["registrations_made"] - counts["registrations_released"] == told["cached"]
    registrar.close()
