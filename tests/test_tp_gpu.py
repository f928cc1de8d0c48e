"""Row-split tensor parallelism: one process per GPU, every matrix split over the GPUs, partial sums and the gathered
hidden state crossing NVLink as tagged words inside the fused pass kernel.  The ids of every rank must equal the
oracle's golden ids (so also the single-GPU run), and the logits -- every rank holds its own blocks -- must meet the
stated tolerance once merged.  Needs as many visible GPUs as ranks (skipped otherwise).  gloo carries the handle exchange."""
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


def _rank_main(rank, world, port, wdir, prompt, q, batched):
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
        # one case also splits the attention over the CTAs of a head group from the fourth position on (the default keeps
        # contexts this short whole)
        inf = pkg.QWen3AWQInfer(wdir, world=world, rank=rank, tensor_parallel=1, device=[rank], keep_logits=1,
                                attn_split_min=3 if (world == 2 and not batched) else 0, **SMALL)
        pipeline.connect_all(inf, dist)
        inf.set_batched_prefill(bool(batched))
        ids = inf.generateResponse(prompt, 6)
        ids += inf.decode_more(4)
        logits = inf.last_logits()
        again = inf.generateResponse(prompt, 10)      # the handle is reusable; the generation counter moves the tags on
        dist.barrier()                                # nobody frees its exchange buffer while another rank still stores into it
        q.put((rank, ids, again, logits))
        inf.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,batched", [(2, 0), (2, 1), (4, 0), (8, 0)])
def test_row_split_matches_golden(orc, cuda, tmp_path, world, batched):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    golden = json.load(open(os.path.join(HERE, "golden", "golden.json")))["small_model"]
    if SMALL["heads"] % world:
        pytest.skip("the small model has 4 heads")
    wdir = str(tmp_path)
    orc.write_weight_dir(orc.default_config(**SMALL), golden["seed"], wdir)
    prompt = [int(t) for t in orc.gen_tokens(golden["seed"], orc.TOKENS, 6, SMALL["vocab"])]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, wdir, prompt, q, batched)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        got = sorted((q.get(timeout=90) for _ in range(world)), key=lambda t: t[0])
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join()
    merged = np.full(SMALL["vocab"], np.nan, np.float32)
    for rank, ids, again, logits in got:
        assert ids == golden["ids"], (rank, ids, golden["ids"])
        assert again == golden["ids"], (rank, again)
        own = ~np.isnan(logits)
        assert not (own & ~np.isnan(merged)).any()      # every block of the vocabulary belongs to exactly one rank
        merged[own] = logits[own]
    assert not np.isnan(merged).any()
    top = np.array(golden["last_logits_top8_idx"])
    want = np.array(golden["last_logits_top8"], np.float32)
    assert (np.abs(merged[top] - want) <= 2e-2 * np.abs(want) + 2e-2 * np.abs(want).mean()).all()
