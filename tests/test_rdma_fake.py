"""RDMA executor against the in-process loopback fabric: handshake, transfers, injected faults.

Host only: the "heaps" are CPU tensors, the transport is a fake, failures are injected through
the fabric (error completions, dropped requests, delays), never on a device.
"""

import pytest
import torch

from pccl_b200 import engine


@pytest.fixture()
def rdma():
    return engine.load_native().rdma


def _pair(rdma, world=2, size=1 << 16):
    fabric = rdma.LoopbackFabric(world)
    mems = [torch.zeros(size, dtype=torch.uint8) for _ in range(world)]
    proxies = [rdma.Proxy(fabric, r, mems[r]) for r in range(world)]
    # two-step handshake: everybody prepares a queue pair per peer, then connects with the peer's info
    info = {(r, p): proxies[r].prepare(p) for r in range(world) for p in range(world) if p != r}
    for r in range(world):
        for p in range(world):
            if p != r:
                assert proxies[r].connect(p, info[(p, r)]) == rdma.Status.OK
    return fabric, mems, proxies


def test_write_and_read_move_bytes(rdma):
    fabric, mems, proxies = _pair(rdma)
    mems[0][:4096] = torch.arange(4096, dtype=torch.int64).to(torch.uint8)
    t = proxies[0].write(1, 0, 8192, 4096)
    assert proxies[0].wait(t) == rdma.Status.OK
    assert torch.equal(mems[1][8192:8192 + 4096], mems[0][:4096])
    t = proxies[1].read(0, 100, 0, 1000)
    assert proxies[1].wait(t) == rdma.Status.OK
    assert torch.equal(mems[1][100:1100], mems[0][:1000])
    assert proxies[0].completed() == 1 and proxies[1].completed() == 1
    for p in proxies:
        p.stop()


def test_connect_requires_the_peers_queue_pair(rdma):
    fabric = rdma.LoopbackFabric(2)
    mems = [torch.zeros(1024, dtype=torch.uint8) for _ in range(2)]
    proxies = [rdma.Proxy(fabric, r, mems[r]) for r in range(2)]
    mine = proxies[0].prepare(1)
    assert proxies[0].connect(1, mine) == rdma.Status.NOT_CONNECTED      # peer has not prepared anything
    theirs = proxies[1].prepare(0)
    assert proxies[0].connect(1, theirs) == rdma.Status.OK
    # an unconnected direction refuses work instead of hanging
    t = proxies[1].write(0, 0, 0, 16)
    assert proxies[1].wait(t) == rdma.Status.NOT_CONNECTED
    for p in proxies:
        p.stop()


def test_out_of_range_and_injected_errors_are_reported(rdma):
    fabric, mems, proxies = _pair(rdma, size=4096)
    t = proxies[0].write(1, 0, 4000, 1000)                               # runs past the peer's registration
    assert proxies[0].wait(t) == rdma.Status.REMOTE_ACCESS_ERROR
    fabric.fail_next(0, 2, rdma.Status.TRANSPORT_ERROR)
    tickets = [proxies[0].write(1, 0, 0, 64) for _ in range(3)]
    assert [proxies[0].wait(t) for t in tickets] == [rdma.Status.TRANSPORT_ERROR, rdma.Status.TRANSPORT_ERROR,
                                                     rdma.Status.OK]
    for p in proxies:
        p.stop()


def test_dropped_request_times_out_and_proxy_stays_usable(rdma):
    fabric, mems, proxies = _pair(rdma)
    fabric.set_drop(0, True)
    lost = proxies[0].write(1, 0, 0, 64)
    assert proxies[0].wait(lost, timeout_ms=50) == rdma.Status.TIMEOUT
    fabric.set_drop(0, False)
    mems[0][:64] = 7
    ok = proxies[0].write(1, 0, 128, 64)
    assert proxies[0].wait(ok) == rdma.Status.OK
    assert int(mems[1][128:192].sum()) == 7 * 64
    assert proxies[0].drain(timeout_ms=50) == rdma.Status.TIMEOUT        # the lost request is still outstanding
    for p in proxies:
        p.stop()


def test_many_outstanding_requests_in_order_with_delay(rdma):
    fabric, mems, proxies = _pair(rdma, world=4, size=1 << 20)
    fabric.set_delay_us(2, 200)
    src = torch.randint(0, 255, (1 << 18,), dtype=torch.uint8)
    mems[2][:1 << 18] = src
    tickets = [proxies[2].write((2 + 1 + i % 3) % 4, i * 1024, (1 << 19) + i * 1024, 1024) for i in range(256)]
    assert proxies[2].drain(timeout_ms=5000) == rdma.Status.OK
    assert len(set(tickets)) == 256
    for i in range(256):
        peer = (2 + 1 + i % 3) % 4
        assert torch.equal(mems[peer][(1 << 19) + i * 1024:(1 << 19) + (i + 1) * 1024], src[i * 1024:(i + 1) * 1024])
    for p in proxies:
        p.stop()


def test_verbs_transport_is_optional(rdma):
    # The default build carries no verbs dependency; the flag only reports how it was compiled.
    assert rdma.verbs_compiled() in (True, False)
