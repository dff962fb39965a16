"""Expert-parallel planning and exchange on CPU ranks (gloo, world size 2 and 4): every pair is computed on exactly
one rank, and the rank-ordered sum of the ranks' partial layer outputs equals the single-rank combine.  The oracle
stands in for the GPU kernels (this is host logic; the GPU path is tested under -m gpu)."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import ROOT, rel_err

H, I, E, S, R, LAYERS = 256, 256, 4, 3, 5, 3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    from glmflash_b200 import ep, synth
    O = entry.load_oracle()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        worst = 0.0
        # (rows, handle capacity): a verify window (shared expert owned by one rank per layer) and a prefill-sized
        # handle (capacity above 16 rows: the shared expert is split by rows)
        for layer, (R, cap) in enumerate([(5, None), (5, None), (5, None), (21, 21), (18, 40)]):
            bank = synth.expert_bank(50 + layer, H, I, E, svh_scale=True)
            x = synth.activations_bf16(60 + layer, R, H)
            picks, rw = synth.route(70 + layer, R, E, S - 1)
            Y = O.experts_run_rows(bank, H, I, E + 1, S, x, picks, mode=1, threads=1)
            full = O.combine(Y, rw, R, S, H)
            mine = ep.computed_here(picks, rank, world, E, layer, max_rows=cap)
            wmask = np.where(mine, np.concatenate([rw[:, :-1], np.ones((R, 1), np.float32)], 1), 0).astype(np.float32)
            # partial combine of this rank: masked pairs contribute nothing (their Y rows are never computed on a GPU rank)
            Ym = np.where(np.repeat(mine.reshape(-1, 1), H, 1), Y, 0).astype(np.float32)
            part = (wmask.reshape(R, S, 1) * Ym.reshape(R, S, H)).sum(1).astype(np.float32)
            gathered = torch.empty((world, R, H), dtype=torch.float32)
            out = torch.empty((R, H), dtype=torch.float32)
            ep.exchange(torch.from_numpy(part), gathered, out)
            # every rank holds the same bytes, and they are the single-rank result up to fp32 re-association
            chk = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(chk, out)
            assert all(torch.equal(chk[0], c) for c in chk)
            worst = max(worst, rel_err(out.numpy(), full)[0])
            owners = torch.zeros((R, S), dtype=torch.int32) + torch.from_numpy(mine.astype(np.int32))
            dist.all_reduce(owners)
            assert (owners == 1).all(), "a pair must be computed on exactly one rank"
        q.put((rank, worst))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ep_exchange_gloo(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    res = [q.get(timeout=5) for _ in range(world)]
    assert sorted(r for r, _ in res) == list(range(world))
    assert max(w for _, w in res) < 1e-5


def test_windows(pkg):
    from glmflash_b200 import ep
    for world in (1, 2, 4, 8):
        wins = [ep.expert_window(r, world, 64) for r in range(world)]
        assert wins[0][0] == 0 and wins[-1][1] == 64 and all(a[1] == b[0] for a, b in zip(wins, wins[1:]))
        assert sorted(ep.shared_owner(l, world) for l in range(world)) == list(range(world))
    with pytest.raises(ValueError):
        ep.expert_window(0, 3, 64)
    with pytest.raises(ValueError):
        ep.expert_window(2, 2, 64)


def _failing_worker(rank, world, port, store_port, mode, q):
    """mode 'absent': rank 1 raises before exchange 2 and says nothing; 'withdraw': it tells the peers; 'collective': its
    all-gather closure reports an error code.  Nobody may hang: every rank ends with a result or an ExchangeError."""
    sys.path.insert(0, ROOT)
    import datetime
    import time
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    from glmflash_b200 import ep
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    store = dist.TCPStore("127.0.0.1", store_port, world, rank == 0, timeout=datetime.timedelta(seconds=20))
    log = []
    try:
        for step in range(4):
            part = torch.full((3, 8), float(rank + 1 + step))
            gathered, out = torch.empty((world, 3, 8)), torch.empty((3, 8))
            t0 = time.monotonic()
            try:
                if rank == 1 and step == 2 and mode in ("absent", "withdraw"):
                    if mode == "withdraw":
                        ep.withdraw(store, step, rank, "device status word 4")
                    raise RuntimeError("rank 1 lost its GPU work before the exchange")
                ep.arrive(store, step, rank, world, timeout_s=2.0)
                inject = None
                if mode == "collective" and step == 2:
                    def inject(dst, src):
                        raise RuntimeError("ncclSystemError (2)")
                ep.exchange(part, gathered, out, all_gather=inject)
                log.append((step, "ok", float(out[0, 0])))
            except ep.ExchangeError as ex:
                log.append((step, "exchange-error", str(ex), time.monotonic() - t0))
                break
            except RuntimeError as ex:
                log.append((step, "local-failure", str(ex)))
                break
        q.put((rank, log))
        q.close()
        q.join_thread()
    finally:
        os._exit(0)                      # a rank that failed leaves without a collective tear-down


@pytest.mark.parametrize("mode", ["absent", "withdraw", "collective"])
def test_a_failing_rank_gives_its_peers_an_error_not_a_hang(mode):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, store_port = _free_port(), _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, store_port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    want_sum = lambda step: float(1 + step) + float(2 + step)
    for rank in (0, 1):
        assert [e[:2] for e in res[rank][:2]] == [(0, "ok"), (1, "ok")]
        assert res[rank][0][2] == want_sum(0) and res[rank][1][2] == want_sum(1)
    if mode == "collective":
        for rank in (0, 1):
            assert res[rank][2][1] == "exchange-error" and "all-gather" in res[rank][2][2] and "ncclSystemError" in res[rank][2][2]
    else:
        assert res[1][2][1] == "local-failure"
        step, kind, msg, waited = res[0][2]
        assert kind == "exchange-error" and "rank 1" in msg
        if mode == "withdraw":
            assert "withdrew" in msg and "status word 4" in msg and waited < 1.5      # told at once, not after the time-out
        else:
            assert "did not reach exchange 2" in msg and waited < 10
