"""The virtual-memory arena's host side: descriptor exchange between ranks (threads here), argument handling, and the
answer of the driver-backed calls on a machine without a driver."""
import os
import threading

import pytest
import torch

from arctic_platform_b200.parallel import vmm


def _exchange(world, tmp_path, payloads=None, timeout=20.0):
    barrier = threading.Barrier(world)
    pipes = [os.pipe() for _ in range(world)]            # rank r shares the WRITE end of its pipe
    results, errors = {}, []

    def rank(r):
        try:
            results[r] = vmm.exchange_fds(r, world, pipes[r][1], str(tmp_path), barrier.wait, timeout,
                                          payload=(payloads or [0] * world)[r])
        except BaseException as exc:
            errors.append(exc)

    threads = [threading.Thread(target=rank, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout + 10)
    return pipes, results, errors


def test_every_rank_receives_every_peers_descriptor(tmp_path):
    world = 4
    pipes, results, errors = _exchange(world, tmp_path, payloads=[100 + r for r in range(world)])
    assert not errors and set(results) == set(range(world))
    for r in range(world):
        assert set(results[r]) == set(range(world)) - {r}
        for peer, (fd, payload) in results[r].items():
            assert payload == 100 + peer and fd not in (pipes[peer][1],)         # a new descriptor of the same pipe
            os.write(fd, bytes([r, peer]))
            assert os.read(pipes[peer][0], 2) == bytes([r, peer])
            os.close(fd)
    assert os.listdir(tmp_path) == []                                            # the sockets are gone
    for rd, wr in pipes:
        os.close(rd)
        os.close(wr)


def test_single_rank_and_missing_peer(tmp_path):
    assert vmm.exchange_fds(0, 1, 0, str(tmp_path), lambda: None) == {}
    rd, wr = os.pipe()
    with pytest.raises(TimeoutError, match="not listening"):
        vmm.exchange_fds(0, 2, wr, str(tmp_path), lambda: None, timeout=0.3)     # rank 1 never shows up
    os.close(rd)
    os.close(wr)


def test_driver_calls_report_the_missing_driver_and_bad_arguments():
    if torch.cuda.is_available():
        pytest.skip("this case is about machines without a driver")
    with pytest.raises(vmm.VmmError) as e:
        vmm.granularity(0)
    assert e.value.code == vmm.NO_DRIVER and "no CUDA driver" in str(e.value)
    with pytest.raises(vmm.VmmError):
        vmm.VmmBuffer(0, 1 << 20)
    with pytest.raises(ValueError):
        vmm.VmmBuffer(0, 0)
    with pytest.raises(vmm.VmmError):
        vmm.ImportedBuffer(0, 3, 1 << 21)


def test_tensor_view_checks_sizes(monkeypatch):
    with pytest.raises(ValueError, match="need 4096 bytes"):
        vmm.view_as_tensor(0x1000, 1024, torch.float32, 1024, 0)
    with pytest.raises(TypeError):
        vmm.view_as_tensor(0x1000, 1 << 20, torch.complex64, 4, 0)
    monkeypatch.setenv("MASTER_PORT", "29511")
    monkeypatch.setenv("APB_VMM_SOCK_DIR", "/tmp/x")
    assert vmm.default_sock_dir() == "/tmp/x/29511"
