"""The multi-GPU data path on two GPUs (skipped where fewer are visible): the fused all-gather of the
row-sharded matvec and the decode sweep built on it, one process per GPU, every rank checking
EVERY rank's slice of what it assembled against the CPU oracle.

NCCL serves the rendezvous and host-side barriers only (in-switch reduction off); the data moves
by the kernels' own peer stores.  All device-side waits are bounded and report through a status
word, so a failure here is an assertion, not a hang.
"""
import os
import socket
import time

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _setup(rank, world, port):
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import datetime
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    return dist


def _gather_worker(rank, world, port, out_dir):
    dist = _setup(rank, world, port)
    try:
        import oracle
        from conftest import load_pkg
        coll, ops, synth, sh = load_pkg("collective"), load_pkg("ops"), load_pkg("synth"), load_pkg("sharding")
        dev = torch.device("cuda", rank)
        rows, n_sb, slots, steps = 1536, 16, 3, 6
        pg = coll.PeerGather(rows, slots, dev)
        assert (pg.world, pg.rank) == (world, rank)
        st = ops.new_status(dev)
        # the global matrices (same seeds on every rank); this rank keeps only its rows on the GPU
        q_full = [synth.q4k_weights(rows, n_sb, 600 + s) for s in range(slots)]
        off, ln = sh.shard_byte_range(rows, n_sb, 144, world, rank)
        q_dev = [torch.from_numpy(q[off:off + ln].copy()).to(dev) for q in q_full]
        for step in range(steps):
            # x differs per step and per slot: a value of another step in a vector is an error
            xs = [synth.activations(n_sb * 256, 700 + 10 * step + s) for s in range(slots)]
            for s in range(slots):
                pg.matvec(q_dev[s], torch.from_numpy(xs[s]).to(dev), n_sb, s, status=st,
                          tuning=ops.make_tuning(pdl=3 if s else 2))
            pg.finish(st, let_next_start=bool(step % 2))
            torch.cuda.synchronize(dev)
            assert int(st.item()) == 0, f"rank {rank} step {step}: status {int(st.item())}"
            for s in range(slots):
                got = pg.vector(s).cpu().numpy()
                y_ref = oracle.matvec_rows("q4k", q_full[s], xs[s], rows, n_sb)
                _y64, mag = oracle.matvec_rows_f64("q4k", q_full[s], xs[s], rows, n_sb)
                err = np.abs(got - y_ref) / mag
                for r in range(world):      # every rank's slice, named in the message
                    b, c = sh.shard_rows(rows, world, r)
                    assert err[b:b + c].max() <= 1e-5, f"rank {rank} step {step} slot {s}: slice of rank {r}"
            assert int(pg.epoch.item()) == step + 2
            # no host barrier between steps; one rank dawdles, so the other runs its next step's
            # matvec (stores into this rank's memory) while this one has not even begun
            if rank == 1:
                time.sleep(0.05)
        # Steps back to back with nothing between them: every launch declared independent and the
        # finish launches letting the next step's matvecs start while they still wait, so steps
        # overlap on the GPU.  x differs per step; only the last step's vectors are read.
        burst = 5
        xs_dev = [[torch.from_numpy(synth.activations(n_sb * 256, 900 + 10 * t + s)).to(dev) for s in range(slots)]
                  for t in range(burst)]
        torch.cuda.synchronize(dev)
        e0 = int(pg.epoch.item())
        for t in range(burst):
            for s in range(slots):
                pg.matvec(q_dev[s], xs_dev[t][s], n_sb, s, status=st, tuning=ops.make_tuning(pdl=3))
            pg.finish(st, let_next_start=True)
        torch.cuda.synchronize(dev)
        assert int(st.item()) == 0, f"rank {rank} burst: status {int(st.item())}"
        assert int(pg.epoch.item()) == e0 + burst
        for s in range(slots):
            x_last = synth.activations(n_sb * 256, 900 + 10 * (burst - 1) + s)
            y_ref = oracle.matvec_rows("q4k", q_full[s], x_last, rows, n_sb)
            _y64, mag = oracle.matvec_rows_f64("q4k", q_full[s], x_last, rows, n_sb)
            assert (np.abs(pg.vector(s).cpu().numpy() - y_ref) / mag).max() <= 1e-5, f"rank {rank} burst slot {s}"
        open(os.path.join(out_dir, f"gather_ok{rank}"), "w").write("ok")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _decode_worker(rank, world, port, out_dir):
    dist = _setup(rank, world, port)
    try:
        import oracle
        from conftest import load_pkg
        decode = load_pkg("decode")
        dev = torch.device("cuda", rank)
        shape = decode.SweepShape(hidden=512, kv=128, ffn=1024, layers=3)
        for mode in ("fused", "prepared", "mixed", "poll", "paired"):
            if mode not in decode.MODES:
                continue
            sweep = decode.DecodeSweep(shape, dev, seed=4242, mode=mode)
            assert sweep.world == world
            # the full matrices from the seeds (each rank holds only its row or column shard)
            weights = [tuple(decode.full_matrix(shape, sweep.seed, layer, j, dev).cpu().numpy() for j in range(4))
                       for layer in range(shape.layers)]
            h0 = np.random.default_rng(5).standard_normal(shape.hidden).astype(np.float32)
            sweep.h.copy_(torch.from_numpy(h0).to(dev))
            sweep.token(normalise_input=False)
            torch.cuda.synchronize(dev)
            assert int(sweep.status.item()) == 0, (mode, int(sweep.status.item()))
            outs, d, h1, ksum = oracle.decode_token(weights, shape.hidden, shape.kv, shape.ffn, h0,
                                                    normalise_input=False)
            _y64, mag = oracle.matvec_rows_f64("q4k", weights[0][0], h0, shape.hidden + 2 * shape.kv, shape.hidden // 256)
            if mode == "paired":
                # this rank's rows of q, k, v (the per-kernel bar) ...
                hq, hk, _hf = sweep.slices
                hid, kv = shape.hidden, shape.kv
                idx = np.concatenate([np.arange(rank * hq, (rank + 1) * hq), hid + np.arange(rank * hk, (rank + 1) * hk),
                                      hid + kv + np.arange(rank * hk, (rank + 1) * hk)])
                got0 = sweep.local_output(0, 0).cpu().numpy()
                assert (np.abs(got0 - outs[0][0][idx]) / mag[idx]).max() <= 1e-5, mode
                # ... and the sum of EVERY rank's partial products: o before its input's unit-RMS scale
                q_full = outs[0][0][:hid]
                o_raw = oracle.matvec_rows("q4k", weights[0][1], q_full, hid, hid // 256)
                _o64, omag = oracle.matvec_rows_f64("q4k", weights[0][1], q_full, hid, hid // 256)
                got1 = sweep.local_output(0, 1).cpu().numpy()
                assert (np.abs(got1 - o_raw) / omag).max() <= 2e-5, mode
            else:
                got0 = sweep.output(0, 0).cpu().numpy()
                assert (np.abs(got0 - outs[0][0]) / mag).max() <= 1e-5, mode   # every rank's slice of the first linear
            for layer in range(shape.layers):
                for j in sweep.checkable_outputs:
                    got, ref = sweep.output(layer, j).cpu().numpy(), outs[layer][j]
                    assert np.abs(got - ref).max() <= 1e-3 * np.sqrt(np.mean(ref.astype(np.float64) ** 2)), (mode, layer, j)
            assert np.abs(sweep.hidden_out().cpu().numpy() - h1).max() <= 1e-3, mode
            assert abs(float(sweep.kv_checksum().item()) - ksum) <= 1e-3 * max(1.0, abs(ksum)), mode
            # two more tokens: the stores alternate between the two copies of the word storage
            for _ in range(2):
                sweep.advance()
                sweep.token()
                _o, d, h1, _k = oracle.decode_token(weights, shape.hidden, shape.kv, shape.ffn, d, normalise_input=True)
            torch.cuda.synchronize(dev)
            assert int(sweep.status.item()) == 0, mode
            assert np.abs(sweep.hidden_out().cpu().numpy() - h1).max() <= 3e-3, mode
            dist.barrier()
        open(os.path.join(out_dir, f"decode_ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def _run(worker, tmp_path, tag):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    world, port = 2, _free_port()
    mp.spawn(worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"{tag}_ok{r}") for r in range(world))


def test_fused_allgather_two_ranks_with_a_slow_rank(tmp_path):
    _run(_gather_worker, tmp_path, "gather")


def test_decode_sweep_two_ranks_matches_oracle(tmp_path):
    _run(_decode_worker, tmp_path, "decode")
