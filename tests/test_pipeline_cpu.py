"""CPU checks of the multi-GPU host logic: the stage split, and the ring wiring run as two gloo
ranks (the handle exchange that precedes qw3_stage_connect), with fake handles since there is no GPU."""
import multiprocessing as mp
import os
import socket

import pytest


def test_stage_split_matches_the_pipeline_contract(pkg):
    import importlib
    pipeline = importlib.import_module("qw3awq_b200.pipeline")
    cabi = pkg.cabi
    want = {1: [36], 2: [18, 18], 4: [9, 9, 9, 9], 8: [5, 5, 5, 5, 4, 4, 4, 4], 3: [12, 12, 12], 5: [8, 7, 7, 7, 7]}
    for n, counts in want.items():
        cfg = cabi.default_config(n_stages=n)
        got = [pipeline.stage_layers(cfg, s) for s in range(n)]
        assert [c for _, c in got] == counts
        assert [f for f, _ in got] == [sum(counts[:s]) for s in range(n)]
    cfg = cabi.default_config(n_stages=2, first_layer=[0, 30, 36])      # explicit split
    assert pipeline.stage_layers(cfg, 1) == (30, 6)
    with pytest.raises(cabi.Qw3Error):
        pipeline.stage_layers(cabi.default_config(n_stages=2), 2)
    assert pipeline.ring_neighbours(0, 4) == (1, 3) and pipeline.ring_neighbours(3, 4) == (0, 2)
    assert pipeline.ring_neighbours(1, 2) == (0, 0)


def _rank_main(rank, world, port, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import torch.distributed as dist
    from conftest import load_package
    load_package()
    import importlib
    pipeline = importlib.import_module("qw3awq_b200.pipeline")
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = bytes([rank + 1]) * 64                        # a fake 64-byte handle that names its owner
        handles = pipeline.exchange_handles(mine, dist)
        nxt, prv = pipeline.ring_neighbours(rank, world)
        ids = pipeline.broadcast_ids([7, 8, 9] if rank == world - 1 else [], 3, dist)
        q.put((rank, handles[nxt][0], handles[prv][0], len(handles), ids))
    finally:
        dist.destroy_process_group()


def test_ring_wiring_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, 2, 2, 2, [7, 8, 9]), (1, 1, 1, 2, [7, 8, 9])]


def test_multiprocess_handle_requires_matching_stage_count(pkg, tmp_path):
    import ctypes as C
    cabi = pkg.cabi
    h = C.c_void_p()
    cfg = cabi.default_config(world=2, rank=0, n_stages=4)
    assert cabi.lib().qw3_create(str(tmp_path).encode(), C.byref(cfg), C.byref(h)) == cabi.QW3_ERR_ARG
    assert cabi.lib().qw3_stage_export(None, None) == cabi.QW3_ERR_ARG
    assert cabi.lib().qw3_stage_connect(None, None, None) == cabi.QW3_ERR_ARG


class _FakeTpLib:
    """Stands in for the C library in connect_all: hands out a handle that names its rank, records what is connected."""
    def __init__(self, rank):
        self.rank, self.connected = rank, None

    def qw3_tp_export(self, h, buf):
        for i in range(64):
            buf[i] = self.rank + 1
        return 0

    def qw3_tp_connect(self, h, flat):
        self.connected = bytes(flat)
        return 0


def _tp_rank_main(rank, world, port, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import torch.distributed as dist
    from conftest import load_package
    pkg = load_package()
    import importlib
    pipeline = importlib.import_module("qw3awq_b200.pipeline")
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fake = _FakeTpLib(rank)
        pkg.cabi.lib = lambda: fake                      # connect_all goes through cabi.lib()

        class Infer:
            _h = None
        pipeline.connect_all(Infer(), dist)
        q.put((rank, fake.connected))
    finally:
        dist.destroy_process_group()


def test_row_split_wiring_two_gloo_ranks():
    """connect_all hands qw3_tp_connect the handles of ALL ranks, rank-major, 64 bytes each (the rank's own included),
    and every rank gets the same table."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world = 2
    procs = [ctx.Process(target=_tp_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        got = sorted(q.get(timeout=120) for _ in range(world))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join()
    table = bytes([1]) * 64 + bytes([2]) * 64
    assert got == [(0, table), (1, table)]
    assert pkg_null_checks()


def pkg_null_checks():
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from conftest import load_package
    cabi = load_package().cabi
    return cabi.lib().qw3_tp_export(None, None) == cabi.QW3_ERR_ARG and cabi.lib().qw3_tp_connect(None, None) == cabi.QW3_ERR_ARG
