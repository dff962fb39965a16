"""Generates tests/golden/ref_sm100.npz from the REFERENCE's own CUDA kernels (compiled unmodified for sm_100a into
oracle/_ref/*.cubin by oracle/Makefile) run on a B200.  The inputs are regenerated from seeds by the tests
(glm-flash-rs_b200/synth.py is numpy PCG64, identical on every machine); the file holds only reference outputs:

  decode_w      fp16 [256][128]   the reference's decoded weights of a seeded 256 x 128 trellis matrix, obtained by
                                  running its grouped GEMV kernel on one-hot activation rows (1.0 * w accumulates
                                  exactly in fp32), i.e. the reference's device decode, not a restatement of it
  y, xd         fp32 / fp16       reference decode-path outputs (exl3_grouped_8_4 pipeline) of a small window
  y_prefill     fp32              reference prefill-path outputs (fast_gu_separate / fast_down) of the same window
  group_*       int32             reference grouping kernels (fixed upstream sizes E = 289, slots = 9)

Run on a GPU box:   python tests/golden/make_golden.py <output.npz>
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

H, I, E, S, ROWS = 512, 256, 4, 3, 5          # small shapes: the fixture stays a few tens of KB
SEED = 4242


def inputs():
    import __graft_entry__ as entry
    entry.load_package()
    from glmflash_b200 import synth
    bank = synth.expert_bank(SEED, H, I, E, svh_scale=True)
    x = synth.activations_bf16(SEED + 1, ROWS, H)
    picks, rw = synth.route(SEED + 2, ROWS, E, S - 1)
    g = synth.rng(SEED + 3)
    words = g.integers(0, 1 << 32, size=(16, 8, 32), dtype=np.uint64).astype(np.uint32)     # K = 256, N = 128
    gp = np.stack([np.concatenate([(np.arange(8) * 37 + 11 * r) % 288, [288]]) for r in range(40)]).astype(np.int32)
    return bank, x, picks, rw, words, gp


def main(out_path):
    import torch
    import ref_gpu
    import __graft_entry__ as entry
    entry.load_package()
    O = entry.load_oracle()
    from glmflash_b200 import synth
    bank, x, picks, rw, words, gp = inputs()
    dev = torch.device("cuda:0")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a.view(np.int32) if a.dtype == np.uint32 else a)).to(dev)

    # ---- decode through the reference GEMV: X = identity (256 one-hot rows), one "expert", 256 members, SK = 1
    K, N = 256, 128
    eye = torch.eye(K, dtype=torch.float16, device=dev)
    ids = t(np.array([0], np.int32)); count = t(np.array([1], np.int32))
    m = ref_gpu.module("exl3")
    p = lambda a: a.data_ptr()
    # slots = 2 so that slot 0 is a routed slot (the reference never computes the last slot); pair index = row * 2
    members2 = t((np.arange(K, dtype=np.int32) * 32).reshape(1, K))
    x2 = torch.zeros((2 * K, K), dtype=torch.float16, device=dev)
    x2[0::2] = eye
    z2 = torch.zeros((2 * K, N), dtype=torch.float32, device=dev)
    m.launch("exl3_grouped_8_4", (1, N // 128, 1 * 1 * (K // 16)), 128,
             [p(x2), p(x2), p(t(words)), p(t(words)), p(ids), p(count), p(members2), p(z2), K, N, 2 * K, 1, K, 2, 1])
    torch.cuda.synchronize()
    decode_w = z2[0::2].cpu().numpy()
    assert (decode_w == decode_w.astype(np.float16).astype(np.float32)).all()

    # ---- decode-path and prefill-path pipelines (one extra trailing slot so that the shared expert is computed)
    wd = synth.to_device(bank, dev)
    S1 = S + 1
    picks1 = np.concatenate([picks, np.full((ROWS, 1), E + 1, np.int32)], 1)
    gi, gc, gm = O.grouping(picks, ROWS, S, E + 1, 16)
    xb = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16)
    y, xd = ref_gpu.experts_run_rows(wd, xb, t(picks1), t(gi), t(np.array([gc], np.int32)), t(gm), ROWS, 16, H, I, E + 1, S1)
    yp, _ = ref_gpu.fast_experts_run(wd, xb, t(picks1), t(gi), t(np.array([gc], np.int32)), t(gm), ROWS, 16, H, I, E + 1, S1)
    torch.cuda.synchronize()
    sel = lambda a, w: a.cpu().numpy().reshape(ROWS, S1, w)[:, :S].reshape(ROWS * S, w)

    # ---- grouping (upstream sizes)
    rid, rcount, rmem = ref_gpu.grouping_run(t(gp), gp.shape[0], 64)
    torch.cuda.synchronize()
    np.savez_compressed(out_path, decode_w=decode_w.astype(np.float16), y=sel(y, H), xd=sel(xd, I), y_prefill=sel(yp, H),
                        group_ids=rid.cpu().numpy()[: int(rcount.cpu()[0])], group_count=rcount.cpu().numpy(),
                        group_members=rmem.cpu().numpy())
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
