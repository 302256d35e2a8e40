"""Host logic of the multi-GPU path on CPU: two gloo ranks shard the rows, each produces its
slice of y (the oracle stands in for the kernel here -- test only), and the product's all-gather
assembles the full vector."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_pkg


def test_shard_rows_cover_everything_once():
    sh = load_pkg("sharding")
    for rows, world in ((14336, 8), (14336, 1), (10, 4), (7, 8), (4096, 3)):
        spans = [sh.shard_rows(rows, world, r) for r in range(world)]
        assert spans[0][0] == 0 and sum(c for _b, c in spans) == rows
        for (b0, c0), (b1, _c1) in zip(spans, spans[1:]):
            assert b0 + c0 == b1
        assert max(c for _b, c in spans) - min(c for _b, c in spans) <= 1
    assert sh.shard_byte_range(14336, 16, 144, 8, 3) == (3 * 1792 * 2304, 1792 * 2304)
    with pytest.raises(ValueError):
        sh.shard_rows(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, rows_list, n_sb, out_dir):
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        sh = load_pkg("sharding")
        synth = load_pkg("synth")
        for rows in rows_list:   # even and ragged split
            q = synth.q4k_weights(rows, n_sb, 123)
            x = synth.activations(n_sb * 256, 124)
            off, ln = sh.shard_byte_range(rows, n_sb, 144, world, rank)
            _b, count = sh.shard_rows(rows, world, rank)
            y_local = torch.from_numpy(oracle.matvec_rows("q4k", q[off:off + ln], x, count, n_sb, threads=1))
            y = sh.all_gather_rows(y_local, rows)
            y_full = oracle.matvec_rows("q4k", q, x, rows, n_sb, threads=1)
            assert (y.numpy().view(np.uint32) == y_full.view(np.uint32)).all()
            with pytest.raises(ValueError):
                sh.all_gather_rows(y_local[:-1], rows)
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_all_gather_rows_two_gloo_ranks(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, [64, 37], 2, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))
