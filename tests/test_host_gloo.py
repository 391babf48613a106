"""CPU, two gloo ranks: the host-side logic of the N > 1 path — configuration agreement, collective
error propagation, IPC-handle exchange order, and the collective close protocol — with a fake
native object in place of the CUDA runtime (the reference simulates its multi-rank host logic
in-process the same way, tests/test_notify_dispatch.cpp with HostFakeCountExchange)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from weftmoe_b200.runtime import TensorRuntime, _Collectives, agree_on_preparation, exchange_handles


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class FakeNative:
    """Records the order of lifecycle calls; plays the native object's part on CPU."""

    def __init__(self, col, *args):
        self.col, self.args, self.calls, self.tapes = col, args, [], 0
        self.stream = args[6]

    def drain_training(self):
        self.calls.append("drain_training")

    def drain_eager_inference(self):
        self.calls.append("drain_eager")

    def usage(self):
        return dict(notify_slots_in_use=self.tapes)

    def retire_peer_mappings(self):
        self.calls.append("retire")

    def destroy(self):
        self.calls.append("destroy")


def make_runtime(group, hidden=256, factory=FakeNative):
    return TensorRuntime(group=group, experts=8, top_k=2, hidden=hidden, intermediate=128, max_tokens=16,
                         max_rows=64, training=True, stream=object(), _native_factory=factory)


def worker(rank, world, port, scenario, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    group = dist.group.WORLD
    out = "ok"
    try:
        if scenario == "agree":
            rt = make_runtime(group)
            assert (rt.rank, rt.world, rt.nodes) == (rank, world, 1)
            assert rt.native.args[:4] == (8, 2, 256, 128) and rt.native.col.world == world
        elif scenario == "mismatch":
            try:
                make_runtime(group, hidden=256 if rank == 0 else 512)
                out = "no error"
            except ValueError as e:
                out = "ValueError" if "incompatible" in str(e) else f"other {e}"
        elif scenario == "one rank fails":
            col = _Collectives(group)
            try:
                agree_on_preparation(col, None if rank == 0 else "RuntimeError: out of memory")
                out = "no error"
            except RuntimeError as e:
                out = "RuntimeError" if "out of memory" in str(e) else f"other {e}"
            try:
                agree_on_preparation(col, "ValueError: bad shape" if rank == 0 else None)
                out += " / no error"
            except ValueError:
                out += " / ValueError"
        elif scenario == "handles":
            col = _Collectives(group)
            blob = exchange_handles(col, bytes([rank + 1]) * 64)
            assert blob == bytes([1]) * 64 + bytes([2]) * 64   # rank-major, what wm_runtime_import_peers expects
            try:
                exchange_handles(col, bytes(64 if rank == 0 else 32))
                out = "no error"
            except RuntimeError:
                pass
        elif scenario == "close":
            rt = make_runtime(group)
            native = rt.native
            native.tapes = 1 if rank == 0 else 0
            if rank == 0:
                try:
                    # a live tape blocks close before any barrier: peers are not left hanging
                    torch.cuda.synchronize = lambda: None
                    rt.close()
                    out = "no error"
                except RuntimeError as e:
                    assert "Live backward tapes" in str(e)
                native.tapes = 0
            torch.cuda.synchronize = lambda: None
            rt.close()
            assert native.calls[-2:] == ["retire", "destroy"] and rt.native is None
            rt.close()  # idempotent
    except Exception as e:  # noqa: BLE001
        out = f"{type(e).__name__}: {e}"
    results[rank] = out
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("scenario,expected", [
    ("agree", "ok"), ("mismatch", "ValueError"), ("one rank fails", "RuntimeError / ValueError"),
    ("handles", "ok"), ("close", "ok")])
def test_two_gloo_ranks(scenario, expected):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), scenario, results), nprocs=world, join=True)
    assert dict(results) == {0: expected, 1: expected}
