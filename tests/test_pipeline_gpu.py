"""Two stages in two processes on two GPUs: the hidden state and the sampled id cross NVLink by peer
stores into CUDA-IPC mailboxes (by hand-off launches, or by the token-pass kernels themselves); the ids must equal the single-GPU run and the oracle's golden ids.
Needs two visible GPUs (skipped otherwise).  gloo carries the handle exchange."""
import datetime
import json
import multiprocessing as mp
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
SMALL = dict(hidden=512, inter=1536, heads=4, head_dim=128, layers=4, vocab=2176, max_pos=64, rope_base=10000.0)


def _rank_main(rank, world, port, wdir, prompt, q, sample_first, chained):
    import sys
    sys.path.insert(0, HERE)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from conftest import load_package
    pkg = load_package()
    import importlib
    pipeline = importlib.import_module("qw3awq_b200.pipeline")
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    try:
        torch.cuda.set_device(rank)
        inf = pkg.QWen3AWQInfer(wdir, n_stages=world, world=world, rank=rank, device=list(range(world)),
                                sample_first=sample_first, keep_logits=1 if rank == world - 1 else 0, **SMALL)
        pipeline.connect_ring(inf, dist)
        inf.set_chained_decode(bool(chained))
        dist.barrier()
        ids = inf.generateResponse(prompt, 6)
        more = inf.decode_more(4)
        logits = inf.last_logits() if rank == world - 1 else None   # of the tenth step, on the stage that samples
        dist.barrier()
        ids = pipeline.broadcast_ids(ids + more if rank == world - 1 else [], 10, dist)
        q.put((rank, ids, logits))
        inf.close()
    finally:
        dist.destroy_process_group()


# chained = 1: from the second decode step on the stages hand over inside the token-pass kernels (tagged words stored
# into the next GPU's mailbox); chained = 0: mailbox send / receive launches for every step
@pytest.mark.parametrize("world,sample_first,chained", [(2, 0, 1), (2, 1, 1), (4, 0, 1), (2, 0, 0)])
def test_one_process_per_gpu_matches_golden(orc, cuda, tmp_path, world, sample_first, chained):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    golden = json.load(open(os.path.join(HERE, "golden", "golden.json")))
    want = golden["small_model_sample_first" if sample_first else "small_model"]["ids"]
    seed = golden["small_model"]["seed"]
    wdir = str(tmp_path)
    orc.write_weight_dir(orc.default_config(**SMALL), seed, wdir)
    prompt = [int(t) for t in orc.gen_tokens(seed, orc.TOKENS, 6, SMALL["vocab"])]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, wdir, prompt, q, sample_first, chained)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        got = sorted((q.get(timeout=300) for _ in range(world)), key=lambda t: t[0])
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:   # a rank that died must not leave the others waiting in a barrier with their GPUs held
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join()
    g = golden["small_model_sample_first" if sample_first else "small_model"]
    for rank, ids, logits in got:
        assert ids == want, (rank, ids, want)
        if rank == world - 1:   # not the ids only: the last step's eight largest logits of the oracle, within the logits tolerance
            top = np.array(g["last_logits_top8_idx"])
            ref = np.array(g["last_logits_top8"], np.float32)
            assert (np.abs(logits[top] - ref) <= 2e-2 * np.abs(ref) + 2e-2 * np.abs(ref).mean()).all()


def _rank_main_batched(rank, world, port, wdir, prompt, q, max_pos):
    import sys
    sys.path.insert(0, HERE)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from conftest import load_package
    pkg = load_package()
    import importlib
    pipeline = importlib.import_module("qw3awq_b200.pipeline")
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    try:
        torch.cuda.set_device(rank)
        cfg = dict(SMALL, max_pos=max_pos)
        inf = pkg.QWen3AWQInfer(wdir, n_stages=world, world=world, rank=rank, device=list(range(world)), **cfg)
        pipeline.connect_ring(inf, dist)
        inf.set_batched_prefill(True)
        dist.barrier()
        ids = inf.generateResponse(prompt, 8)
        ids2 = inf.generateResponse(prompt, 8)      # the block counters carry on into a second sequence
        dist.barrier()
        last = rank == world - 1
        ids = pipeline.broadcast_ids(ids if last else [], 8, dist)
        ids2 = pipeline.broadcast_ids(ids2 if last else [], 8, dist)
        q.put((rank, ids, ids2))
        inf.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_prompt", [(2, 6), (2, 5000), (4, 5000)])
def test_one_process_per_gpu_batched_prompt(pkg, orc, cuda, tmp_path, world, n_prompt):
    """Prompt in blocks of up to 2048 rows handed from stage to stage through the mailboxes' block inboxes (5000 rows:
    three blocks over two acknowledged slots): same ids as the single-GPU run with the same blocks."""
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    seed = json.load(open(os.path.join(HERE, "golden", "golden.json")))["small_model"]["seed"]
    wdir = str(tmp_path)
    orc.write_weight_dir(orc.default_config(**SMALL), seed, wdir)
    prompt = [int(t) for t in orc.gen_tokens(seed, orc.TOKENS, n_prompt, SMALL["vocab"])]
    max_pos = n_prompt + 24
    one = pkg.QWen3AWQInfer(wdir, **dict(SMALL, max_pos=max_pos))
    one.set_batched_prefill(True)
    want = one.generateResponse(prompt, 8)
    one.close()
    if n_prompt == 6:
        golden = json.load(open(os.path.join(HERE, "golden", "golden.json")))
        assert want == golden["small_model"]["ids"][:8]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main_batched, args=(r, world, port, wdir, prompt, q, max_pos)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        got = sorted(q.get(timeout=300) for _ in range(world))
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join()
    for rank, ids, ids2 in got:
        assert ids == want and ids2 == want, (rank, ids, ids2, want)
