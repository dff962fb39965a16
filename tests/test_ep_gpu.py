"""Expert-parallel layer on 2 GPUs (NCCL over NVLink): every rank ends with the bytes of the rank-ordered sum, and
they equal the single-GPU layer output within fp32 re-association.  Skipped with fewer than 2 GPUs."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import ROOT, rel_err

pytestmark = pytest.mark.gpu

H, I, E, S = 2048, 1536, 64, 5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows_list, q):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load_package()
    from glmflash_b200 import ep, synth
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        res = []
        for rows, launches in [(r, k) for r in rows_list for k in ((3, 1) if r <= 16 else (3,))]:
            # launches = 1: the one-launch layer kernel with the exchange inside; 3: expert kernels, then the exchange kernel
            os.environ["GLMFLASH_LAYER_KERNELS"] = str(launches)
            # three launches, windows of <= 16 rows: also with the shared expert's owner decided per window on the device
            # (every second layer set); the one-launch kernel serves the round-robin rule only
            dyn = launches == 3 and rows == 16
            layer = ep.EpMoe(pkg, rank, world, rows, H, I, E, S, device=dev, exchange="nvlink", dynamic_shared=dyn)
            base = ep.EpMoe(pkg, rank, world, rows, H, I, E, S, device=dev, exchange="nccl", dynamic_shared=dyn)
            single = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=rows))
            for l in range(2):
                bank = synth.device_bank(300 + l, H, I, E, dev)
                x = torch.from_numpy(synth.activations_bf16(310 + l, rows, H).view(np.int16)).to(dev).view(torch.bfloat16)
                picks, rw = synth.route(320 + l, rows, E, S - 1, shared_bias=rows <= 16, uniform=rows > 16)
                pd, wd = torch.from_numpy(picks).to(dev), torch.from_numpy(rw).to(dev)
                out = layer.run(l, bank, x, pd, wd, rows).clone()
                for _ in range(3):                                  # epochs advance in lockstep, buffers alternate
                    again = layer.run(l, bank, x, pd, wd, rows).clone()
                nccl = base.run(l, bank, x, pd, wd, rows).clone()
                single.run(bank, x, pd, wd, rows)
                torch.cuda.synchronize()
                assert int(layer.ep.status.cpu()[0]) == 0, "a bounded peer wait gave up"
                layer.check()
                assert torch.equal(out, again) and torch.equal(out, nccl), "fused NVLink exchange != NCCL all-gather + ordered sum"
                ref = single.output[:rows].clone()
                chk = [torch.empty_like(out) for _ in range(world)]
                dist.all_gather(chk, out)
                same = all(torch.equal(chk[0], c) for c in chk)
                res.append((rows, l, same, rel_err(out.cpu().numpy(), ref.cpu().numpy())[0]))
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_ep_two_gpus(cuda):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    world = 2
    procs = [ctx.Process(target=_worker, args=(r, world, port, [1, 16, 300], q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
        assert p.exitcode == 0
    for _ in range(world):
        rank, res = q.get(timeout=5)
        for rows, l, same, err in res:
            assert same, (rank, rows, l, "ranks disagree")
            assert err < 1e-5, (rank, rows, l, err)


def test_peer_that_never_arrives_times_out(pkg, synth, cuda):
    """Failure detection without a fault: two owners (ranks 0 and 1 of a world of 2) live on ONE GPU and are connected
    by pointers; only rank 0 calls the exchange, so its wait for rank 1's flag runs out after the (shortened) poll
    limit.  The kernel returns, the status word says PEER_TIMEOUT, and the context stays usable: once rank 1 does
    arrive for that epoch, a later pair of calls completes and gives the sum."""
    import torch
    rows = 2
    cfgs = [pkg.make_config(H, I, E, S, max_rows=rows, shared_exl3=0, expert_lo=r * 32, expert_hi=(r + 1) * 32, pdl=0) for r in (0, 1)]
    eps = [pkg.EpCombine(cfgs[r], r, 2, None) for r in (0, 1)]
    bases = [e.local_base for e in eps]
    for e in eps:
        e.connect_ptrs(bases)
        e.set_wait_limit(20000)
    picks, rw = synth.route(5, rows, E, S - 1)
    pd, wd = torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda)
    Y = torch.randn((rows * S, H), dtype=torch.float32, device=cuda)
    eps[0].combine(C_void(Y), pd, wd, rows, True)
    torch.cuda.synchronize()
    assert int(eps[0].status.cpu()[0]) == 4                     # GF_STATUS_PEER_TIMEOUT
    # the context is alive and the protocol recovers: rank 1 delivers the missed epoch, then both run a fresh one
    eps[1].combine(C_void(Y), pd, wd, rows, False)
    torch.cuda.synchronize()
    eps[0].clear_status()                                       # the host has dealt with the failure
    eps[0].set_wait_limit(2000000)
    eps[1].set_wait_limit(20000)
    eps[1].combine(C_void(Y), pd, wd, rows, False)               # rank 1 pushes epoch 2 (its own wait for rank 0 runs out)
    eps[0].combine(C_void(Y), pd, wd, rows, True)                # rank 0 finds rank 1's epoch-2 partial already there
    torch.cuda.synchronize()
    assert int(eps[0].status.cpu()[0]) == 0
    y = Y.view(rows, S, H)
    want = (wd[:, :, None] * y).sum(1)
    assert torch.allclose(eps[0].output[:rows], want, rtol=1e-5, atol=1e-5)


def test_connect_rejects_a_peer_built_with_another_configuration(pkg, cuda):
    """The handle blob carries a hash of the exchange's layout; a rank whose hidden size, row limit or world differs is
    named at connect time, before any peer memory is mapped, instead of being indexed with the wrong strides."""
    import ctypes
    from glmflash_b200 import lib
    mk = lambda **kw: pkg.make_config(H, I, E, S, shared_exl3=0, expert_lo=32, expert_hi=64, pdl=0, **kw)
    for other in (mk(max_rows=8), pkg.make_config(H // 2, I, E, S, max_rows=4, shared_exl3=0, expert_lo=32, expert_hi=64, pdl=0)):
        peer = pkg.EpCombine(other, 1, 2, None)
        blob = ctypes.create_string_buffer(lib().glmflash_ep_handle_bytes())
        assert lib().glmflash_ep_get_handle(peer._h, blob) == 0
        with pytest.raises(RuntimeError, match="rank 1 was built with a different configuration"):
            pkg.EpCombine(mk(max_rows=4), 0, 2, lambda mine: [mine, bytes(blob.raw)])


@pytest.mark.parametrize("bf16", [False, True])
def test_two_step_exchange_of_a_large_window_on_one_gpu(pkg, synth, cuda, bf16):
    """Windows of more than 16 rows: every chunk of 8 rows has an owner rank that adds the ranks' partials in rank order
    and hands the finished rows to everybody.  Two owners on ONE GPU, connected by pointers, called one after the other
    with short wait limits (nothing hangs): rank 1 delivers its partials and gives up waiting; rank 0 then finds them and
    finishes the chunks it owns (rows 0..31 of 64).  fp32 mode: the bytes of the plain rank-ordered sum; bf16 mode: every
    partial rounded to bf16 once, then the fp32 sum in rank order (the reference's prefill exchange, src/batch.rs:651-658)."""
    import torch
    rows = 64
    cfgs = [pkg.make_config(H, I, E, S, max_rows=rows, shared_exl3=0, expert_lo=r * 32, expert_hi=(r + 1) * 32, pdl=0) for r in (0, 1)]
    eps = [pkg.EpCombine(cfgs[r], r, 2, None) for r in (0, 1)]
    bases = [e.local_base for e in eps]
    for e in eps:
        e.connect_ptrs(bases)
        e.set_wait_limit(20000)
        e.set_exchange_bf16(bf16)
    picks, rw = synth.route(15, rows, E, S - 1, uniform=True)
    pd, wd = torch.from_numpy(picks).to(cuda), torch.from_numpy(rw).to(cuda)
    Y = torch.randn((rows * S, H), dtype=torch.float32, device=cuda)
    for step in range(2):                                        # the receive buffers alternate with the epoch
        eps[1].combine(C_void(Y), pd, wd, rows, False)
        torch.cuda.synchronize()
        assert int(eps[1].status.cpu()[0]) == 4                  # rank 1's own chunks never got rank 0's partials
        eps[1].clear_status()
        got = eps[0].combine(C_void(Y), pd, wd, rows, True).clone()
        torch.cuda.synchronize()
        assert int(eps[0].status.cpu()[0]) == 4                  # ... and rank 0 waited in vain for rank 1's finished chunks
        eps[0].clear_status()
        y = Y.view(rows, S, H)
        parts = []
        for r in (0, 1):
            mine = ((pd >= r * 32) & (pd < (r + 1) * 32)).float()
            mine[:, S - 1] = 0.0
            part = torch.zeros((rows, H), dtype=torch.float32, device=cuda)
            for s_ in range(S - 1):                              # ascending slots, as the kernel adds them
                part += (mine[:, s_] * wd[:, s_])[:, None] * y[:, s_]
            if r == 0:
                part += y[:, S - 1]                              # the shared expert's pair, weight 1, on rank 0
            parts.append(part.bfloat16().float() if bf16 else part)
        want = parts[0] + parts[1]
        diff = (got[:32] - want[:32]).abs()
        if not bf16:
            assert float(diff.max()) < 2e-6, step                # fused vs separate multiply-add: an fp32 ulp
        else:
            # an fp32 ulp in a partial can flip its bf16 rounding: a handful of elements differ by one bf16 step
            assert float((diff > 2e-6).float().mean()) < 1e-3 and float(diff.max()) < 0.1, step
        if bf16:
            plain = ((y[:, :S - 1] * wd[:, :S - 1, None]).sum(1) + y[:, S - 1])
            assert not torch.allclose(got[:32], plain[:32], rtol=0, atol=1e-4)       # the rounding really happened


def C_void(t):
    import ctypes
    return ctypes.c_void_p(t.data_ptr())
