#!/usr/bin/env python
"""Benchmark of the EXL3 MoE expert path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rows R] [--layers L] [--impl reference]

Workload (N = 1, default): benchmark config 2 -- the MoE layer decoding ONE token (hidden 2048, 64 routed
experts + 1 shared, top-4, SwiGLU experts 2048 -> 1536 -> 2048, all EXL3 4 bpw) -- walked over a stack of 47
layers with distinct random weights (config 5's stack, 14.4 GB), so that every packed word comes from HBM
(one layer's touched weights, 23.7 MB, would otherwise sit in the 126 MB L2).  One step = the token through
all 47 layers (each layer with its own input row and routing table, as the stack is "experts only").
    value   = layer-tokens per second = rows * layers / step time, inputs resident in HBM, the step replayed
              as one CUDA graph, CUDA-event timed.
    e2e     = the same through the host-buffer C-ABI call (glmflash_moe_run_host) per layer: pinned host
              activations / picks / routing weights copied in, the layer output copied back, every step.
    roofline= the dominant kernel (gate/up grouped GEMV + SwiGLU epilogue), launched alone over the stack and
              timed with CUDA events: algorithmic bytes per launch / average duration / measured HBM peak.
N > 1: the 64 routed experts are split evenly over the ranks (expert parallel), the shared expert goes round
robin over the layers; each rank computes a partial layer output, NCCL all-gathers the partials over NVLink and
every rank adds them in rank order (the reference's fixed-order sum after its all-gather).  Total work is fixed:
"scaling": "strong".
--impl reference: the reference's CPU path for the op (its scalar oracle restated in oracle/exl3_oracle.c; the
Rust original cannot be built here) on all host threads, bounded samples of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

H, I, E, S = 2048, 1536, 64, 5
MAT_BYTES = H * I // 2                                     # packed bytes of one matrix
W_E = 3 * MAT_BYTES + (2 * H + 2 * I + I + H) * 2          # 4,740,096 B: one expert's matrices + its six scale vectors
GATEUP_BYTES_E = 2 * MAT_BYTES + (2 * H + 3 * I) * 2       # what the gate/up kernel reads per expert (algorithmic)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "25",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def host_layer_inputs(synth, layers, rows, seed0=5000):
    xs, ps, ws = [], [], []
    for l in range(layers):
        xs.append(synth.activations_bf16(seed0 + 3 * l, rows, H))
        p, w = synth.route(seed0 + 3 * l + 1, rows, E, S - 1, shared_bias=rows > 1)
        ps.append(p); ws.append(w)
    return np.stack(xs), np.stack(ps), np.stack(ws)


def cpu_sample(O, synth, rows, budget_s=12.0):
    """The CPU baseline: the oracle's whole-layer path (unpack every touched matrix, fp32 dot products in the
    reference's split/warp order, epilogues, combine) on all host threads, on layers of the same workload."""
    threads = O.max_threads()
    bank = synth.expert_bank(1000, H, I, E)
    t0, n = time.time(), 0
    while True:
        x = synth.activations_bf16(7000 + n, rows, H)
        picks, rw = synth.route(7100 + n, rows, E, S - 1, shared_bias=rows > 1)
        Y = O.experts_run_rows(bank, H, I, E + 1, S, x, picks, mode=0, sk_gu=4, sk_dn=1, threads=threads)
        O.combine(Y, rw, rows, S, H)
        n += 1
        if time.time() - t0 > budget_s or n >= 64:
            break
    dt = time.time() - t0
    return rows * n / dt, threads, f"{n} layer passes of {rows} token(s), {dt:.1f} s"


def run_reference(args, rank):
    if rank != 0:
        return
    O = entry.load_oracle()
    entry.load_package()
    from glmflash_b200 import synth
    threads = O.max_threads()
    bank = synth.expert_bank(1000, H, I, E)
    times = []
    for i in range(args.warmup + args.steps):
        x = synth.activations_bf16(7000 + i, args.rows, H)
        picks, rw = synth.route(7100 + i, args.rows, E, S - 1, shared_bias=args.rows > 1)
        t0 = time.time()
        Y = O.experts_run_rows(bank, H, I, E + 1, S, x, picks, mode=0, sk_gu=4, sk_dn=1, threads=threads)
        O.combine(Y, rw, args.rows, S, H)
        if i >= args.warmup:
            times.append(time.time() - t0)
    ms = 1e3 * float(np.mean(times))
    v = args.rows / (ms / 1e3)
    sample = f"each step = 1 layer pass of {args.rows} token(s) of the {args.layers}-layer workload"
    print(json.dumps({
        "impl": "reference", "metric": "EXL3-4bpw MoE layer tok/s", "value": v, "unit": "layer-tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": v, "unit": "layer-tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "layer-tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(args):
    if args.workload == "prefill":
        return {"workload": f"moe_layer_prefill_{args.rows}tok (config 4): uniform random top-4 routing, alternating over "
                            f"{args.layers} layers of distinct weights", "hidden": H, "intermediate": I, "experts": E,
                "shared_experts": 1, "top_k": S - 1, "bits_per_weight": 4, "rows": args.rows, "layers": args.layers,
                "l2": "one layer's bank (308 MB) plus rotated activations exceed L2", "parallelism": f"ep{args.gpus}"}
    return {"workload": f"moe_layer_decode_bs{args.rows} (config 2{'/3' if args.rows > 1 else ''}) over a {args.layers}-layer stack of distinct "
                        "weights (config 5 stack)", "hidden": H, "intermediate": I, "experts": E, "shared_experts": 1, "top_k": S - 1,
            "bits_per_weight": 4, "rows": args.rows, "layers": args.layers,
            "l2": f"weights of a step ({args.layers} layers) exceed L2; every layer has its own weights",
            "parallelism": f"ep{args.gpus}"}


def run_prefill(args, pkg, synth, torch, dist, dev, rank, world, local):
    """Config 4: one step = one prefill chunk of `rows` tokens through one MoE layer (alternating layers)."""
    R, L, G = args.rows, args.layers, world
    banks = [synth.device_bank(1000 * l + 1, H, I, E, dev) for l in range(L)]
    structs = [pkg.weights_struct(b) for b in banks]
    xs = np.stack([synth.activations_bf16(9000 + l, R, H) for l in range(L)])
    routes = [synth.route(9100 + l, R, E, S - 1, uniform=True) for l in range(L)]
    ps, ws = np.stack([r[0] for r in routes]), np.stack([r[1] for r in routes])
    x_d = torch.from_numpy(xs.view(np.int16)).to(dev).view(torch.bfloat16)
    p_d, w_d = torch.from_numpy(ps).to(dev), torch.from_numpy(ws).to(dev)
    # the shared expert's rows go to one rank per layer (round robin)
    from glmflash_b200 import ep
    epm = ep.EpMoe(pkg, rank, G, R, H, I, E, S, device=dev, exchange=args.exchange)
    owner = epm.owner
    stream = torch.cuda.Stream()
    state = {"i": 0}

    def step():
        l = state["i"] % L
        state["i"] += 1
        epm.run(l, structs[l], x_d[l], p_d[l], w_d[l], R)

    def timed(fn, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(step, args.steps, args.warmup)
    flops = R * S * 3 * 2 * H * I                                  # all pairs incl. the shared expert, three matrices
    xh = torch.from_numpy(xs.view(np.int16)).pin_memory()
    ph, wh = torch.from_numpy(ps).pin_memory(), torch.from_numpy(ws).pin_memory()
    oh = torch.empty((R, H), dtype=torch.float32).pin_memory()

    x_stage = torch.empty((R, H), dtype=torch.bfloat16, device=dev)
    p_stage = torch.empty((R, S), dtype=torch.int32, device=dev)
    w_stage = torch.empty((R, S), dtype=torch.float32, device=dev)

    def step_e2e():
        l = state["i"] % L
        state["i"] += 1
        if G == 1:
            owner(l).run_host(structs[l], xh[l], ph[l], wh[l], R, oh, stream=stream)
        else:
            x_stage.view(torch.int16).copy_(xh[l], non_blocking=True)
            p_stage.copy_(ph[l], non_blocking=True)
            w_stage.copy_(wh[l], non_blocking=True)
            res = epm.run(l, structs[l], x_stage, p_stage, w_stage, R)
            oh.copy_(res, non_blocking=True)
            stream.synchronize()
    ms_e2e = timed(step_e2e, max(3, args.steps // 2), 3)
    e2e = {"value": R / (ms_e2e / 1e3), "unit": "layer-tokens/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": R * H * 2 + 2 * R * S * 4, "d2h_bytes_per_step": R * H * 4,
           "call": "glmflash_moe_run_host (pinned host input / picks / weights in, output out, sync)"}
    roofline = upstream = None
    if G == 1:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
        peak, how = (float(peaks["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)") if peaks else (1590.0, "fallback")
        # the dominant kernel alone: the gate/up grouped GEMM (2/3 of the flops)
        fe = pkg.FastExperts(pkg.make_config(H, I, E, S, max_rows=R))
        O = entry.load_oracle()
        lay = []
        for l in range(L):
            ids, count, members = O.grouping(ps[l], R, S, E + 1, R)
            t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
            lay.append((t(ids), t(np.array([count], np.int32)), t(members)))

        def fe_step():
            l = state["i"] % L
            state["i"] += 1
            fe.run(structs[l], x_d[l], p_d[l], *lay[l], R, R)
        timed(fe_step, L, 1)
        fe.set_phases(4)
        ms_gu = timed(fe_step, max(5, args.steps), 3)
        fe.set_phases(8)
        ms_dn = timed(fe_step, max(5, args.steps), 3)
        fe.set_phases(15)
        gu_flops = R * S * 2 * 2 * H * I
        ach = gu_flops / (ms_gu * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "fast_gemm_kernel<2> (gate/up grouped GEMM: tcgen05 + in-kernel trellis decode + SwiGLU epilogue)",
                    "achieved": ach, "peak": peak, "peak_source": how, "unit": "TFLOP/s", "frac": ach / peak, "ms_per_launch": ms_gu,
                    "algorithmic_flops_per_launch": gu_flops,
                    # dram bytes of one launch from the capture in profiles/fast_gemm_prefill_4096.md (500.6 MB + 65.4 MB)
                    "traffic": 566022912.0 if R == 4096 else None,
                    "down_kernel": {"ms_per_launch": ms_dn, "tflops": R * S * 2 * H * I / (ms_dn * 1e-3) / 1e12},
                    "layer": {"tflops": flops / (ms_step * 1e-3) / 1e12, "frac": flops / (ms_step * 1e-3) / 1e12 / peak}}
        # the reference's own CUDA kernels, recompiled unmodified for sm_100a, on the same tensors (comparison only)
        try:
            sys.path.insert(0, os.path.join(ROOT, "oracle"))
            import ref_gpu
            if ref_gpu.available():
                S6 = S + 1
                l = 0
                picks6 = torch.from_numpy(np.concatenate([ps[l], np.full((R, 1), E + 1, np.int32)], 1)).to(dev)

                def up_step():
                    ref_gpu.fast_experts_run(banks[l], x_d[l], picks6, *lay[l], R, R, H, I, E + 1, S6, stream=stream)
                ms_up = timed(up_step, 3, 1)
                upstream = {"what": "reference prefill kernels (mma.sync) compiled unmodified for sm_100a, experts only (no grouping/combine)",
                            "ms_per_step": ms_up, "layer_tokens_per_s": R / (ms_up / 1e3), "tflops": flops / (ms_up * 1e-3) / 1e12}
        except Exception as ex:
            upstream = {"error": repr(ex)}
    clocks = sampler.stop() if rank == 0 else None       # sampled over every timed region above
    cpu = None
    if rank == 0 and G == 1 and not args.no_cpu_baseline:
        O = entry.load_oracle()
        bank = synth.expert_bank(1000, H, I, E)
        n = 32                                                     # a 32-token slice of the chunk, all host threads
        t0 = time.time()
        O.experts_run_rows(bank, H, I, E + 1, S, xs[0][:n], ps[0][:n], mode=0, sk_gu=4, sk_dn=1)
        dt = time.time() - t0
        cpu = {"value": n / dt, "unit": "layer-tokens/s", "cores": O.max_threads(), "kind": "port",
               "sample": f"{n} of the {R} tokens of one chunk ({dt:.1f} s); every touched expert is unpacked once per slice"}
    if rank == 0:
        print(json.dumps({"metric": "EXL3-4bpw MoE layer tok/s", "value": R / (ms_step / 1e3), "unit": "layer-tokens/s", "n_gpus": G,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
                          "config": workload_config(args), "tflops": flops / (ms_step * 1e-3) / 1e12, "clocks": clocks, "e2e": e2e,
                          "exchange": epm.exchange,
                          "gpu_launches": 6 * args.steps, "roofline": roofline, "upstream_kernels_sm100a": upstream, "cpu_baseline": cpu}))
    finish(world, dist)


def finish(world, dist):
    """Leave without tearing the process group down (destroy_process_group can block after graph-captured
    collectives); every rank has passed the final barrier of its last timed region by now."""
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        try:
            dist.barrier()
        except Exception:
            pass
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--layers", type=int, default=47)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill"])
    ap.add_argument("--exchange", default="nvlink", choices=["nvlink", "nccl"],
                    help="N > 1: fused combine + NVLink push + ordered sum kernel, or NCCL all-gather + ordered sum")
    ap.add_argument("--router", action="store_true",
                    help="decode: produce the routing table on the device inside the timed layer (router matvec + sigmoid "
                         "top-k kernels ahead of the expert kernels) instead of taking it as an input")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload == "prefill":
        if args.rows == 1:
            args.rows = 4096
        if args.layers == 47:
            args.layers = 2
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    pkg = entry.load_package()
    from glmflash_b200 import synth
    pkg.lib()                                                   # fails loudly when the CUDA library is missing
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node N for --gpus N"
    G = world
    R, L = args.rows, args.layers
    assert E % G == 0
    if args.workload == "prefill":
        return run_prefill(args, pkg, synth, torch, dist, dev, rank, world, local)

    # ---- weights: one bank per layer, generated on the device (identical on every rank)
    banks = [synth.device_bank(1000 * l + 1, H, I, E, dev) for l in range(L)]
    structs = [pkg.weights_struct(b) for b in banks]
    xs, ps, ws = host_layer_inputs(synth, L, R)
    x_d = torch.from_numpy(xs.view(np.int16)).to(dev).view(torch.bfloat16)      # [L][R][H]
    p_d = torch.from_numpy(ps).to(dev)
    w_d = torch.from_numpy(ws).to(dev)

    # ---- owners: expert window per rank; the shared expert goes round robin over the layers
    from glmflash_b200 import ep
    epm = ep.EpMoe(pkg, rank, G, max(R, 1), H, I, E, S, device=dev, exchange=args.exchange)
    owner = epm.owner
    moes = epm.moes
    if G > 1:
        final = torch.empty((L, R, H), dtype=torch.float32, device=dev)

    if args.router:
        # router matrices scaled so that the logits are ~N(0,1) as the workload defines them; the table is then made
        # on the device, per layer, by the library's router kernels
        gen = torch.Generator(device=dev).manual_seed(4242)
        wr_d = (torch.randn((L, E, H), generator=gen, device=dev) / (H ** 0.5)).to(torch.bfloat16)
        logit_d = torch.empty((L, R, E), dtype=torch.float32, device=dev)
        p_d = torch.empty_like(p_d)
        w_d = torch.empty_like(w_d)

    def route(l):
        if args.router:
            pkg.route(x_d[l], wr_d[l], logit_d[l], p_d[l], w_d[l])

    def layer(l):
        route(l)
        if G == 1:
            epm.run(l, structs[l], x_d[l], p_d[l], w_d[l], R)
        else:
            epm.run(l, structs[l], x_d[l], p_d[l], w_d[l], R, out=final[l])

    def step_eager():
        for l in range(L):
            layer(l)

    stream = torch.cuda.Stream()
    graph = None
    with torch.cuda.stream(stream):
        step_eager()
        stream.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step_eager()
            graph = g
        except Exception as ex:                                  # NCCL capture can be refused: time eager launches
            if rank == 0:
                print(f"graph capture failed ({type(ex).__name__}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
    step = (lambda: graph.replay()) if graph is not None else step_eager

    def timed(fn, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(step, args.steps, args.warmup)
    value = R * L / (ms_step / 1e3)

    # ---- end to end: every step copies the step's inputs (all layers' activations, routing tables, routing weights)
    #      from pinned host memory, runs the 47 layer calls of the public API on them, and reads all layer outputs back
    xh = torch.from_numpy(xs.view(np.int16)).pin_memory()
    ph, wh = torch.from_numpy(ps).pin_memory(), torch.from_numpy(ws).pin_memory()
    oh = torch.empty((L, R, H), dtype=torch.float32).pin_memory()
    out_all = torch.empty((L, R, H), dtype=torch.float32, device=dev)

    def layers_with_outputs():
        for l in range(L):
            route(l)
            if G == 1:
                out_all[l].copy_(epm.run(l, structs[l], x_d[l], p_d[l], w_d[l], R))
            else:
                epm.run(l, structs[l], x_d[l], p_d[l], w_d[l], R, out=out_all[l])
    graph_e2e = None
    with torch.cuda.stream(stream):
        layers_with_outputs()
        stream.synchronize()
        try:
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=stream):
                layers_with_outputs()
            graph_e2e = g2
        except Exception:
            torch.cuda.synchronize()

    def step_e2e():
        x_d.view(torch.int16).copy_(xh, non_blocking=True)
        if not args.router:
            p_d.copy_(ph, non_blocking=True)
            w_d.copy_(wh, non_blocking=True)
        if graph_e2e is not None:
            graph_e2e.replay()
        else:
            layers_with_outputs()
        oh.copy_(out_all, non_blocking=True)
        stream.synchronize()
    ms_e2e = timed(step_e2e, max(5, args.steps), 3)
    e2e = {"value": R * L / (ms_e2e / 1e3), "unit": "layer-tokens/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": L * (R * H * 2 + (0 if args.router else 2 * R * S * 4)), "d2h_bytes_per_step": L * R * H * 4,
           "call": "per step: pinned host inputs of all layers -> device, glmflash_moe_run per layer (graph replay), all layer "
                   "outputs -> pinned host, one synchronize"}
    # the same through the synchronous per-layer host-buffer entry point (glmflash_moe_run_host), N = 1 only
    if G == 1:
        def step_layer_calls():
            for l in range(L):
                owner(l).run_host(structs[l], xh[l], ph[l], wh[l], R, oh[l], stream=stream)
        ms_lc = timed(step_layer_calls, max(3, args.steps // 4), 3)
        e2e["per_layer_host_call"] = {"value": R * L / (ms_lc / 1e3), "ms_per_step": ms_lc,
                                      "call": "glmflash_moe_run_host per layer: copy in, run, copy out, synchronize"}

    # ---- roofline of the dominant kernel: gate/up GEMV alone, every layer, back to back (N = 1 only)
    roofline = None
    if G == 1:
        m = moes[1]
        peak, how = measured_peaks()
        distinct = [len(np.unique(ps[l])) for l in range(L)]     # experts touched incl. the shared one
        m.set_phases(4)                                          # gate/up only (scratch of the last step stays in place)

        def gateup_pass_eager():
            for l in range(L):
                m.run(structs[l], x_d[l], p_d[l], w_d[l], R)
        with torch.cuda.stream(stream):
            gateup_pass_eager()
            stream.synchronize()
            gg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gg, stream=stream):
                gateup_pass_eager()
        ms_pass = timed(lambda: gg.replay(), max(5, args.steps), 3)
        m.set_phases(31)
        bytes_per_launch = float(np.mean(distinct)) * GATEUP_BYTES_E + R * H * 2 * 2
        achieved = bytes_per_launch / (ms_pass / L * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "gemv_kernel<2,*> (gate/up grouped GEMV + SwiGLU epilogue)", "achieved": achieved,
                    "peak": peak, "peak_source": how + " (MEASURED_PEAKS.json hbm_gbs)" if how == "measured" else how,
                    "unit": "GB/s", "frac": achieved / peak, "us_per_launch": ms_pass / L * 1e3,
                    "algorithmic_bytes_per_launch": bytes_per_launch,
                    # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised in
                    # profiles/gemv_decode_bs1.md (1 token: 15.88 MB read, 0 written); other row counts were not captured
                    "traffic": 15880192.0 if R == 1 else None,
                    "layer": {"algorithmic_bytes": float(np.mean(distinct)) * W_E + R * H * 6, "us": ms_step / L * 1e3,
                              "gbs": (float(np.mean(distinct)) * W_E + R * H * 6) / (ms_step / L * 1e-3) / 1e9}}
        roofline["layer"]["frac"] = roofline["layer"]["gbs"] / peak

    clocks = sampler.stop() if rank == 0 else None       # sampled over every timed region above
    cpu = None
    if rank == 0 and G == 1 and not args.no_cpu_baseline:
        O = entry.load_oracle()
        v, cores, sample = cpu_sample(O, synth, R)
        cpu = {"value": v, "unit": "layer-tokens/s", "cores": cores, "kind": "port", "sample": sample}

    if rank == 0:
        out = {"metric": "EXL3-4bpw MoE layer tok/s", "value": value, "unit": "layer-tokens/s", "n_gpus": G, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
               "dtype": "f16xf16->f32", "data": "synthetic", "config": workload_config(args),
               "stack_tokens_per_s": R / (ms_step / 1e3), "graph": graph is not None,
               "clocks": clocks, "e2e": e2e, "exchange": epm.exchange,
               "gpu_launches": ((3 if G == 1 or epm.exchange == "nvlink" else 4) + ((1 if R <= 16 else 2) if args.router else 0)) * L * args.steps,
               "router": "on device, inside the timed layer" if args.router else "routing table is an input",
               "roofline": roofline, "cpu_baseline": cpu}
        print(json.dumps(out))
    finish(world, dist)


if __name__ == "__main__":
    main()
