#!/usr/bin/env python
"""Benchmark of the EXL3 MoE expert path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rows R] [--layers L] [--impl reference]

Headline workload (every N): benchmark config 2 -- the MoE layer decoding ONE token (hidden 2048, 64 routed experts +
1 shared, top-4, SwiGLU experts 2048 -> 1536 -> 2048, all EXL3 4 bpw) -- walked over a stack of 47 layers with distinct
random weights (config 5's stack, 14.4 GB), so that every packed word comes from HBM (one layer's touched weights,
23.7 MB, would otherwise sit in the 126 MB L2).  One step = the token through all 47 layers (each layer with its own
input row and routing table, as the stack is "experts only").
    value    = layer-tokens per second = rows * layers / step time, inputs resident in HBM, the step replayed as one
               CUDA graph, CUDA-event timed.
    e2e      = the same through the public C-ABI calls with HOST buffers: per step the pinned host inputs of all layers
               are copied in, the layer calls run, all layer outputs are copied back, one synchronise; the blocking
               per-layer host-buffer call (glmflash_moe_run_host) is reported beside it as e2e_per_layer_host_call.
    roofline = the dominant kernel (windows of <= 16 rows: the gate/up grouped GEMV; prefill: the gate/up grouped
               GEMM) timed with CUDA events: algorithmic bytes (or flops) per launch / average duration / measured peak.
    workloads= the other benchmark configs in the same line: decode / verify windows of 4, 8 and 16 tokens (config 3
               routing: one bias vector shared by the tokens of a window) and the 4096-token prefill chunk (config 4),
               each with ms_per_step, value, e2e and its own roofline.
N > 1: the 64 routed experts are split evenly over the ranks (expert parallel), the shared expert goes round robin over
the layers (prefill: split by rows); every rank computes a partial layer output, and the ranks' partials are exchanged
over NVLink and added in rank order (the reference's fixed-order sum after its all-gather) by the exchange kernel.
Total work is fixed: "scaling": "strong".  phases_us_per_layer splits a layer into the rank's own kernels and the exchange;
outside the timed region every rank also runs the whole window on its own and compares (ep_check); a failed check or a
non-zero device status word makes the run exit non-zero, and a status word that is set after the first step stops the run
there.  Prefill at N > 1 also reports the exchange with bf16 partial rows (exchange_bf16, checked at a bf16 tolerance).
roofline.traffic comes from profiles/traffic.json, which `bench.py --record-traffic NCU_CSV KEY KERNEL_REGEX COMMAND` writes
from an ncu --csv log; it is null when the kernel source has changed since that capture.
--impl reference: the reference's CPU path for the op (its scalar oracle restated in oracle/exl3_oracle.c; the Rust
original cannot be built here) on all host threads, bounded samples of the same workload.
"""
import argparse
import hashlib
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
INSTRUCTION_CEILING_GBS = 3800.0                           # packed bytes/s at one decode instruction per cycle and scheduler


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_threads():
    """Threads the CPU arm may use: the cores this process may run on (torchrun pins OMP_NUM_THREADS to 1, which says
    nothing about the machine)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def recorded_traffic(key, path=None):
    """DRAM bytes of one launch of the dominant kernel from the last ncu capture (profiles/traffic.json), or None when
    the kernel source has changed since that capture."""
    p = path or os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(p):
        return None
    rec = json.load(open(p)).get(key)
    if not rec:
        return None
    src = os.path.join(ROOT, rec["source"])
    if not os.path.exists(src) or hashlib.sha256(open(src, "rb").read()).hexdigest() != rec["source_sha256"]:
        return None
    return float(rec["traffic_bytes"])


TRAFFIC_SOURCES = {"gemv": "glm-flash-rs_b200/csrc/gemv.cuh", "window": "glm-flash-rs_b200/csrc/window.cu",
                   "fast": "glm-flash-rs_b200/csrc/fast_experts.cu"}


def record_traffic(csv_path, key, kernel_regex, command, out=None):
    """Summary step of an ncu capture: read the `--csv` log of a run that collected dram__bytes_read.sum and
    dram__bytes_write.sum, average read + write per launch over the kernels whose name matches, and store the figure in
    profiles/traffic.json under `key`, with the hash of the kernel source it was measured on and the capture's command.
    recorded_traffic() hands the figure to the roofline only while that source is unchanged."""
    import csv
    import re
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}
    lines = [ln for ln in open(csv_path, newline="") if ln.startswith('"')]
    rows = list(csv.DictReader(lines))
    per = {}
    for r in rows:
        if r.get("Metric Name") in ("dram__bytes_read.sum", "dram__bytes_write.sum") and re.search(kernel_regex, r["Kernel Name"]):
            v = float(r["Metric Value"].replace(",", "")) * scale[r["Metric Unit"]]
            per.setdefault(r["ID"], {})[r["Metric Name"]] = v
    full = [d for d in per.values() if len(d) == 2]
    if not full:
        sys.exit(f"no launch of /{kernel_regex}/ with both DRAM counters in {csv_path}")
    rd = sum(d["dram__bytes_read.sum"] for d in full) / len(full)
    wr = sum(d["dram__bytes_write.sum"] for d in full) / len(full)
    source = TRAFFIC_SOURCES[key.split("_")[0]]
    out = out or os.path.join(ROOT, "profiles", "traffic.json")
    table = json.load(open(out)) if os.path.exists(out) else {}
    table[key] = {"traffic_bytes": round(rd + wr), "dram_read_bytes": round(rd), "dram_write_bytes": round(wr), "launches": len(full),
                  "kernel": kernel_regex, "source": source,
                  "source_sha256": hashlib.sha256(open(os.path.join(ROOT, source), "rb").read()).hexdigest(), "command": command}
    json.dump(table, open(out, "w"), indent=1, sort_keys=True)
    print(json.dumps({key: table[key]}))


class ClockSampler:
    """nvidia-smi clock / throttle samples while the timed regions run."""
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
        busy = [s for s in sm if s > 0.6 * max(mx)] if mx else sm
        return {"sm_mhz": float(np.median(busy or sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_layers(O, synth, rows, threads, budget_s, max_layers=64):
    """The CPU arm: the oracle's whole-layer path (unpack every touched matrix, fp32 dot products in the reference's
    split/warp order, epilogues, combine) on `threads` host threads, on layers of the same workload."""
    bank = synth.expert_bank(1000, H, I, E)
    t0, n = time.time(), 0
    while True:
        x = synth.activations_bf16(7000 + n, rows, H)
        picks, rw = synth.route(7100 + n, rows, E, S - 1, shared_bias=rows > 1)
        Y = O.experts_run_rows(bank, H, I, E + 1, S, x, picks, mode=0, sk_gu=4, sk_dn=1, threads=threads)
        O.combine(Y, rw, rows, S, H)
        n += 1
        if time.time() - t0 > budget_s or n >= max_layers:
            break
    dt = time.time() - t0
    return rows * n / dt, f"{n} layer passes of {rows} token(s), {dt:.1f} s"


def decode_config(rows, layers, gpus):
    return {"workload": f"moe_layer_decode_bs{rows} (config 2{'/3' if rows > 1 else ''}) over a {layers}-layer stack of distinct weights "
                        "(config 5 stack)", "hidden": H, "intermediate": I, "experts": E, "shared_experts": 1, "top_k": S - 1,
            "bits_per_weight": 4, "rows": rows, "layers": layers,
            "l2": f"weights of a step ({layers} layers) exceed L2; every layer has its own weights", "parallelism": f"ep{gpus}"}


def prefill_config(rows, layers, gpus):
    return {"workload": f"moe_layer_prefill_{rows}tok (config 4): uniform random top-4 routing, alternating over {layers} layers of "
                        "distinct weights", "hidden": H, "intermediate": I, "experts": E, "shared_experts": 1, "top_k": S - 1,
            "bits_per_weight": 4, "rows": rows, "layers": layers,
            "l2": "one layer's bank (308 MB) plus rotated activations exceed L2", "parallelism": f"ep{gpus}"}


def run_reference(args, rank):
    if rank != 0:
        return
    O = entry.load_oracle()
    entry.load_package()
    from glmflash_b200 import synth
    threads = host_threads()
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
    single, single_sample = cpu_layers(O, synth, args.rows, 1, 4.0, max_layers=4)
    sample = f"each step = 1 layer pass of {args.rows} token(s) of the {args.layers}-layer workload"
    print(json.dumps({
        "impl": "reference", "metric": "EXL3-4bpw MoE layer tok/s", "value": v, "unit": "layer-tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
        "config": decode_config(args.rows, args.layers, args.gpus),
        "cpu_baseline": {"value": v, "unit": "layer-tokens/s", "cores": threads, "kind": "port", "sample": sample,
                         "single_thread": {"value": single, "cores": 1, "sample": single_sample}},
        "e2e": {"value": v, "unit": "layer-tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


class Bench:
    """Device state shared by the workloads of one run: the layer stack, the timing helpers, the status checks."""

    def __init__(self, args, pkg, synth, torch, dist, dev, rank, world, local):
        self.args, self.pkg, self.synth, self.torch, self.dist = args, pkg, synth, torch, dist
        self.dev, self.rank, self.world, self.local = dev, rank, world, local
        self.stream = torch.cuda.Stream()
        self.banks = [synth.device_bank(1000 * l + 1, H, I, E, dev) for l in range(args.layers)]
        self.structs = [pkg.weights_struct(b) for b in self.banks]
        self.peaks = peaks()
        self.failures = []

    # ---- timing: K steps between CUDA events on the launching stream, barrier + synchronise on both sides, max over ranks
    def timed(self, fn, steps, warmup, guard=None):
        """guard: an owner with check() (EpMoe).  A device status word that is set after the first warm-up step means every
        further step would sit out its bounded waits (seconds each): the run stops there instead of timing garbage."""
        torch, dist = self.torch, self.dist
        with torch.cuda.stream(self.stream):
            for k in range(warmup):
                fn()
                if k == 0 and guard is not None:
                    self.stream.synchronize()
                    try:
                        guard.check()
                    except self.pkg.GlmFlashError as ex:
                        print(f"bench: rank {self.rank}: {ex} after the first step; stopping", file=sys.stderr, flush=True)
                        os._exit(3)
            self.stream.synchronize()
            if self.world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(steps):
                fn()
            e1.record(self.stream)
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier()
        ms = e0.elapsed_time(e1)
        if self.world > 1:
            t = torch.tensor([ms], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    def graph_of(self, fn):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            fn()
            self.stream.synchronize()
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    fn()
                return g
            except Exception as ex:
                if self.rank == 0:
                    print(f"graph capture failed ({type(ex).__name__}); timing eager launches", file=sys.stderr)
                torch.cuda.synchronize()
                return None

    def check_status(self, epm, what):
        try:
            epm.check()
        except self.pkg.GlmFlashError as ex:
            self.failures.append(f"{what}: {ex}")

    # ---- expert-parallel self-check, outside every timed region
    def ep_check(self, epm, layers, x_d, p_d, w_d, rows, max_rows, tol=1e-5):
        torch, dist, pkg = self.torch, self.dist, self.pkg
        single = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=max_rows))
        worst, same = 0.0, True
        for l in layers:
            got = epm.run(l, self.structs[l], x_d[l], p_d[l], w_d[l], rows).clone()
            single.run(self.structs[l], x_d[l], p_d[l], w_d[l], rows)
            torch.cuda.synchronize()
            ref = single.output[:rows]
            worst = max(worst, float((got - ref).abs().max() / ref.abs().max()))
            if self.world > 1:
                all_ = [torch.empty_like(got) for _ in range(self.world)]
                dist.all_gather(all_, got)
                same = same and all(torch.equal(all_[0], a) for a in all_)
        ok = worst < tol and same and int(single.status.cpu()[0]) == 0
        res = {"layers": list(layers), "max_rel_diff_vs_single_rank_layer": worst, "tolerance": tol, "ranks_hold_identical_bytes": same, "ok": ok}
        if self.world > 1:
            t = torch.tensor([0.0 if ok else 1.0], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res["ok"] = float(t.item()) == 0.0
        if not res["ok"]:
            self.failures.append(f"ep_check rows={rows}: {res}")
        return res

    # ---- decode / verify windows over the layer stack
    def decode(self, rows, steps, warmup, headline=False, cpu=False):
        torch, pkg, synth, args = self.torch, self.pkg, self.synth, self.args
        G, L, dev = self.world, args.layers, self.dev
        from glmflash_b200 import ep
        xs = np.stack([synth.activations_bf16(5000 + 3 * l, rows, H) for l in range(L)])
        rts = [synth.route(5001 + 3 * l, rows, E, S - 1, shared_bias=rows > 1) for l in range(L)]
        ps, ws = np.stack([r[0] for r in rts]), np.stack([r[1] for r in rts])
        x_d = torch.from_numpy(xs.view(np.int16)).to(dev).view(torch.bfloat16)
        p_d, w_d = torch.from_numpy(ps).to(dev), torch.from_numpy(ws).to(dev)
        epm = ep.EpMoe(pkg, self.rank, G, rows, H, I, E, S, device=dev, exchange=args.exchange)
        out_all = torch.empty((L, rows, H), dtype=torch.float32, device=dev)
        wr_d = logit_d = None
        if args.router and headline:
            gen = torch.Generator(device=dev).manual_seed(4242)
            wr_d = (torch.randn((L, E, H), generator=gen, device=dev) / (H ** 0.5)).to(torch.bfloat16)
            logit_d = torch.empty((L, rows, E), dtype=torch.float32, device=dev)
            p_d, w_d = torch.empty_like(p_d), torch.empty_like(w_d)

        def layer(l, keep):
            if wr_d is not None:
                pkg.route(x_d[l], wr_d[l], logit_d[l], p_d[l], w_d[l])
            res = epm.run(l, self.structs[l], x_d[l], p_d[l], w_d[l], rows)
            if keep:
                out_all[l].copy_(res)

        def step_eager():
            for l in range(L):
                layer(l, False)

        def step_keep():
            for l in range(L):
                layer(l, True)
        g = self.graph_of(step_eager)
        ms_step = self.timed((lambda: g.replay()) if g is not None else step_eager, steps, warmup, guard=epm)
        self.check_status(epm, f"decode rows={rows}")
        value = rows * L / (ms_step / 1e3)

        # end to end: pinned host inputs of all layers in, the layer calls, all outputs back, one synchronise
        xh = torch.from_numpy(xs.view(np.int16)).pin_memory()
        ph, wh = torch.from_numpy(ps).pin_memory(), torch.from_numpy(ws).pin_memory()
        oh = torch.empty((L, rows, H), dtype=torch.float32).pin_memory()
        g2 = self.graph_of(step_keep)

        def step_e2e():
            x_d.view(torch.int16).copy_(xh, non_blocking=True)
            if wr_d is None:
                p_d.copy_(ph, non_blocking=True)
                w_d.copy_(wh, non_blocking=True)
            if g2 is not None:
                g2.replay()
            else:
                step_keep()
            oh.copy_(out_all, non_blocking=True)
            self.stream.synchronize()
        ms_e2e = self.timed(step_e2e, max(5, steps), 3)
        e2e = {"value": rows * L / (ms_e2e / 1e3), "unit": "layer-tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": L * (rows * H * 2 + (0 if wr_d is not None else 2 * rows * S * 4)), "d2h_bytes_per_step": L * rows * H * 4,
               "call": "per step: pinned host inputs of all layers -> device, one layer call per layer (graph replay), all layer "
                       "outputs -> pinned host, one synchronize"}
        res = {"rows": rows, "ms_per_step": ms_step, "us_per_layer": ms_step / L * 1e3, "value": value, "unit": "layer-tokens/s",
               "stack_tokens_per_s": rows / (ms_step / 1e3), "graph": g is not None, "e2e": e2e}
        if G == 1:
            def step_layer_calls():
                for l in range(L):
                    epm.owner(l).run_host(self.structs[l], xh[l], ph[l], wh[l], rows, oh[l], stream=self.stream)
            ms_lc = self.timed(step_layer_calls, max(3, steps // 4), 3)
            res["e2e_per_layer_host_call"] = {"value": rows * L / (ms_lc / 1e3), "unit": "layer-tokens/s", "ms_per_step": ms_lc,
                                              "call": "glmflash_moe_run_host per layer: copy in, run, copy out, synchronize"}
        # roofline: the layer is one launch of the layer kernel; its time is the step's time per layer
        distinct = float(np.mean([len(np.unique(ps[l])) for l in range(L)]))          # experts touched incl. the shared one
        layer_bytes = distinct * W_E + rows * H * 6
        one_launch = os.environ.get("GLMFLASH_LAYER_KERNELS", "") == "1"
        if G == 1 and one_launch:
            gbs = layer_bytes / (ms_step / L * 1e-3) / 1e9
            res["roofline"] = {"bound": "hbm", "kernel": "window_kernel (grouping, input rotation, gate/up and down GEMV, SwiGLU and output "
                               "epilogues, combine: the whole layer in one launch)",
                               "achieved": gbs, "peak": self.peaks["hbm_gbs"], "peak_source": self.peaks["source"] + " hbm_gbs", "unit": "GB/s",
                               "frac": gbs / self.peaks["hbm_gbs"], "us_per_launch": ms_step / L * 1e3, "algorithmic_bytes_per_launch": layer_bytes,
                               "distinct_experts_per_layer": distinct, "traffic": recorded_traffic(f"window_kernel_rows{rows}"),
                               "instruction_ceiling_gbs": INSTRUCTION_CEILING_GBS, "frac_of_instruction_ceiling": gbs / INSTRUCTION_CEILING_GBS}
        elif G == 1:
            # the dominant kernel alone: the gate/up GEMV (with grouping, input rotation and the SwiGLU epilogue inside), every
            # layer back to back
            m = epm.owner(0)
            m.set_phases(4)                                          # gate/up only (scratch of the last step stays in place)

            def gateup_pass():
                for l in range(L):
                    m.run(self.structs[l], x_d[l], p_d[l], w_d[l], rows)
            gg = self.graph_of(gateup_pass)
            ms_pass = self.timed((lambda: gg.replay()) if gg is not None else gateup_pass, max(5, steps), 3)
            m.set_phases(31)
            gu_bytes = distinct * GATEUP_BYTES_E + rows * H * 2 * 2
            gbs = gu_bytes / (ms_pass / L * 1e-3) / 1e9
            lgbs = layer_bytes / (ms_step / L * 1e-3) / 1e9
            res["roofline"] = {"bound": "hbm", "kernel": "gemv_kernel<2,*> (gate/up grouped GEMV + grouping + input rotation + SwiGLU epilogue)",
                               "achieved": gbs, "peak": self.peaks["hbm_gbs"], "peak_source": self.peaks["source"] + " hbm_gbs", "unit": "GB/s",
                               "frac": gbs / self.peaks["hbm_gbs"], "us_per_launch": ms_pass / L * 1e3, "algorithmic_bytes_per_launch": gu_bytes,
                               "distinct_experts_per_layer": distinct, "traffic": recorded_traffic(f"gemv_gateup_rows{rows}"),
                               "instruction_ceiling_gbs": INSTRUCTION_CEILING_GBS, "frac_of_instruction_ceiling": gbs / INSTRUCTION_CEILING_GBS,
                               "layer": {"algorithmic_bytes": layer_bytes, "us": ms_step / L * 1e3, "gbs": lgbs, "frac": lgbs / self.peaks["hbm_gbs"],
                                         "frac_of_instruction_ceiling": lgbs / INSTRUCTION_CEILING_GBS}}
        else:
            res["distinct_experts_per_layer"] = distinct
            # per-phase split of one layer: this rank's share without the exchange, and with it
            solo = pkg.Moe(pkg.make_config(H, I, E, S, max_rows=rows, expert_lo=epm.window[0], expert_hi=epm.window[1],
                                           shared_exl3=2 if epm.dynamic else 1))

            def step_solo():
                for l in range(L):
                    solo.run(self.structs[l], x_d[l], p_d[l], w_d[l], rows)
            gs = self.graph_of(step_solo)
            ms_solo = self.timed((lambda: gs.replay()) if gs is not None else step_solo, max(3, steps // 2), 3)
            res["phases_us_per_layer"] = {"rank_share_without_exchange": ms_solo / L * 1e3, "with_exchange": ms_step / L * 1e3,
                                          "exchange_and_imbalance": (ms_step - ms_solo) / L * 1e3}
            res["ep_check"] = self.ep_check(epm, (0, L - 1), x_d, p_d, w_d, rows, rows)
            self.check_status(epm, f"decode rows={rows} after ep_check")
        if cpu and self.rank == 0 and not args.no_cpu_baseline:
            O = entry.load_oracle()
            v, sample = cpu_layers(O, synth, rows, host_threads(), 12.0)
            v1, sample1 = cpu_layers(O, synth, rows, 1, 4.0, max_layers=4)
            res["cpu_baseline"] = {"value": v, "unit": "layer-tokens/s", "cores": host_threads(), "kind": "port", "sample": sample,
                                   "single_thread": {"value": v1, "cores": 1, "sample": sample1}}
        # one layer against the oracle before anything is reported (N = 1: the whole layer; N > 1: ep_check covers it)
        if headline and G == 1 and self.rank == 0 and not args.no_cpu_baseline and wr_d is None:
            O = entry.load_oracle()
            bank = {k: (v.cpu().numpy().view(np.uint32) if v.dtype == torch.int32 else v.cpu().numpy()) for k, v in self.banks[0].items()}
            want = O.combine(O.experts_run_rows(bank, H, I, E + 1, S, xs[0], ps[0], mode=1, threads=host_threads()), ws[0], rows, S, H)
            epm.run(0, self.structs[0], x_d[0], p_d[0], w_d[0], rows)
            torch.cuda.synchronize()
            got = epm.owner(0).output[:rows].cpu().numpy()
            err = float(np.abs(got - want).max() / np.abs(want).max())
            res["oracle_check"] = {"layer": 0, "max_rel_err": err, "ok": err < 1e-3}
            if not err < 1e-3:
                self.failures.append(f"oracle check: {err}")
        return res

    # ---- prefill chunks (config 4)
    def prefill(self, rows, steps, warmup, cpu=False):
        torch, pkg, synth, args = self.torch, self.pkg, self.synth, self.args
        G, dev = self.world, self.dev
        L = min(2, args.layers)
        from glmflash_b200 import ep
        xs = np.stack([synth.activations_bf16(9000 + l, rows, H) for l in range(L)])
        routes = [synth.route(9100 + l, rows, E, S - 1, uniform=True) for l in range(L)]
        ps, ws = np.stack([r[0] for r in routes]), np.stack([r[1] for r in routes])
        x_d = torch.from_numpy(xs.view(np.int16)).to(dev).view(torch.bfloat16)
        p_d, w_d = torch.from_numpy(ps).to(dev), torch.from_numpy(ws).to(dev)
        epm = ep.EpMoe(pkg, self.rank, G, rows, H, I, E, S, device=dev, exchange=args.exchange)
        state = {"i": 0}

        def step():
            l = state["i"] % L
            state["i"] += 1
            epm.run(l, self.structs[l], x_d[l], p_d[l], w_d[l], rows)
        ms_step = self.timed(step, steps, warmup, guard=epm)
        self.check_status(epm, f"prefill rows={rows}")
        flops = rows * S * 3 * 2 * H * I                               # all pairs incl. the shared expert, three matrices
        xh = torch.from_numpy(xs.view(np.int16)).pin_memory()
        ph, wh = torch.from_numpy(ps).pin_memory(), torch.from_numpy(ws).pin_memory()
        oh = torch.empty((rows, H), dtype=torch.float32).pin_memory()
        x_stage = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
        p_stage = torch.empty((rows, S), dtype=torch.int32, device=dev)
        w_stage = torch.empty((rows, S), dtype=torch.float32, device=dev)

        def step_e2e():
            l = state["i"] % L
            state["i"] += 1
            if G == 1:
                epm.owner(l).run_host(self.structs[l], xh[l], ph[l], wh[l], rows, oh, stream=self.stream)
            else:
                x_stage.view(torch.int16).copy_(xh[l], non_blocking=True)
                p_stage.copy_(ph[l], non_blocking=True)
                w_stage.copy_(wh[l], non_blocking=True)
                oh.copy_(epm.run(l, self.structs[l], x_stage, p_stage, w_stage, rows), non_blocking=True)
                self.stream.synchronize()
        ms_e2e = self.timed(step_e2e, max(3, steps // 2), 3)
        res = {"rows": rows, "ms_per_step": ms_step, "value": rows / (ms_step / 1e3), "unit": "layer-tokens/s",
               "tflops": flops / (ms_step * 1e-3) / 1e12,
               "e2e": {"value": rows / (ms_e2e / 1e3), "unit": "layer-tokens/s", "ms_per_step": ms_e2e,
                       "h2d_bytes_per_step": rows * H * 2 + 2 * rows * S * 4, "d2h_bytes_per_step": rows * H * 4,
                       "call": "glmflash_moe_run_host (pinned host input / picks / weights in, output out, sync)" if G == 1 else
                               "pinned host inputs -> device, glmflash_moe_run_ep, output -> pinned host, sync"}}
        if G == 1:
            # the dominant kernel alone (the gate/up grouped GEMM, 2/3 of the flops), fed by the library's own grouping
            fe = pkg.FastExperts(pkg.make_config(H, I, E, S, max_rows=rows))
            groupings = []
            for l in range(L):
                gr = pkg.Grouping(pkg.make_config(H, I, E, S, max_rows=rows))
                gr.run(p_d[l], rows, stream=self.stream)
                groupings.append(gr)
            self.stream.synchronize()

            def fe_step():
                l = state["i"] % L
                state["i"] += 1
                gr = groupings[l]
                fe.run(self.structs[l], x_d[l], p_d[l], gr.ids, gr.count, gr.members, rows, rows, stream=self.stream)
            self.timed(fe_step, L, 1)
            fe.set_phases(4)
            ms_gu = self.timed(fe_step, max(5, steps), 3)
            fe.set_phases(8)
            ms_dn = self.timed(fe_step, max(5, steps), 3)
            fe.set_phases(15)
            if int(fe.status.cpu()[0]) != 0:
                self.failures.append("prefill roofline leg: device status word set")
            gu_flops = rows * S * 2 * 2 * H * I
            ach = gu_flops / (ms_gu * 1e-3) / 1e12
            layer_tf = flops / (ms_step * 1e-3) / 1e12
            res["roofline"] = {"bound": "tensor", "kernel": "fast_gemm_kernel<2> (gate/up grouped GEMM: tcgen05 + in-kernel trellis decode + SwiGLU epilogue)",
                               "achieved": ach, "peak": self.peaks["bf16_tflops"], "peak_source": self.peaks["source"] + " bf16_tflops (burst)",
                               "unit": "TFLOP/s", "frac": ach / self.peaks["bf16_tflops"], "ms_per_launch": ms_gu, "algorithmic_flops_per_launch": gu_flops,
                               "traffic": recorded_traffic(f"fast_gemm_gateup_rows{rows}"),
                               "down_kernel": {"ms_per_launch": ms_dn, "tflops": rows * S * 2 * H * I / (ms_dn * 1e-3) / 1e12},
                               "layer": {"tflops": layer_tf, "frac_of_burst": layer_tf / self.peaks["bf16_tflops"],
                                         "frac_of_sustained": layer_tf / self.peaks["bf16_tflops_sustained"]}}
            # the reference's own CUDA kernels, recompiled unmodified for sm_100a, on the same tensors (comparison only)
            try:
                sys.path.insert(0, os.path.join(ROOT, "oracle"))
                import ref_gpu
                if ref_gpu.available():
                    picks6 = torch.from_numpy(np.concatenate([ps[0], np.full((rows, 1), E + 1, np.int32)], 1)).to(dev)
                    gr = groupings[0]

                    def up_step():
                        ref_gpu.fast_experts_run(self.banks[0], x_d[0], picks6, gr.ids, gr.count, gr.members, rows, rows, H, I, E + 1, S + 1,
                                                 stream=self.stream)
                    ms_up = self.timed(up_step, 3, 1)
                    res["upstream_kernels_sm100a"] = {"what": "reference prefill kernels (mma.sync) compiled unmodified for sm_100a, experts only "
                                                      "(no grouping / combine)", "ms_per_step": ms_up, "tflops": flops / (ms_up * 1e-3) / 1e12}
            except Exception as ex:
                res["upstream_kernels_sm100a"] = {"error": repr(ex)}
            if cpu and self.rank == 0 and not args.no_cpu_baseline:
                O = entry.load_oracle()
                bank = synth.expert_bank(1000, H, I, E)
                n = 32                                                 # a 32-token slice of the chunk, all host threads
                t0 = time.time()
                O.experts_run_rows(bank, H, I, E + 1, S, xs[0][:n], ps[0][:n], mode=0, sk_gu=4, sk_dn=1, threads=host_threads())
                dt = time.time() - t0
                res["cpu_baseline"] = {"value": n / dt, "unit": "layer-tokens/s", "cores": host_threads(), "kind": "port",
                                       "sample": f"{n} of the {rows} tokens of one chunk ({dt:.1f} s); every touched expert is unpacked once per slice"}
        else:
            # per-phase split of one chunk: this rank's share with a local combine and no exchange; the whole call; and the
            # exchange kernel alone (combine of this rank's pairs + NVLink push + ordered sum) on the pair buffer left in place
            m = epm.owner(0)

            def solo():
                l = state["i"] % L
                state["i"] += 1
                m.run(self.structs[l], x_d[l], p_d[l], w_d[l], rows, stream=self.stream)
            ms_solo = self.timed(solo, max(3, steps // 2), 3)
            res["phases_us_per_layer"] = {"rank_share_with_local_combine": ms_solo * 1e3, "with_exchange": ms_step * 1e3}
            if args.exchange == "nvlink":
                def xonly():
                    epm.ep.combine(m.pairs_ptr, p_d[0], w_d[0], rows, True, stream=self.stream)
                ms_x = self.timed(xonly, max(3, steps // 2), 3)
                res["phases_us_per_layer"]["exchange_kernel_alone"] = ms_x * 1e3
                res["phases_us_per_layer"]["exchange_bytes_out_per_rank"] = int(2 * rows * H * 4 * (G - 1) / G)
            res["ep_check"] = self.ep_check(epm, range(L), x_d, p_d, w_d, rows, rows)
            self.check_status(epm, f"prefill rows={rows} after ep_check")
            if args.exchange == "nvlink":
                # the same chunk with the partial rows crossing NVLink as bf16 (the reference's prefill exchange format);
                # not the headline: its result is not the fp32 all-gather's, so it is checked at a bf16 tolerance
                epm.ep.set_exchange_bf16(True)
                ms_b = self.timed(step, max(3, steps // 2), 3)
                res["exchange_bf16"] = {"ms_per_step": ms_b, "value": rows / (ms_b / 1e3), "unit": "layer-tokens/s",
                                        "ep_check": self.ep_check(epm, range(L), x_d, p_d, w_d, rows, rows, tol=2e-2)}
                self.check_status(epm, f"prefill rows={rows}, bf16 exchange")
                epm.ep.set_exchange_bf16(False)
        return res


def finish(world, dist, code):
    """Leave without tearing the process group down (destroy_process_group can block after graph-captured
    collectives); every rank has passed the final barrier of its last timed region by now."""
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        try:
            dist.barrier()
        except Exception:
            pass
        os._exit(code)
    sys.exit(code)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rows", type=int, default=1, help="rows of the headline decode window (1 = config 2)")
    ap.add_argument("--layers", type=int, default=47)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="all", choices=["all", "decode", "prefill"],
                    help="all: the headline and every other config as `workloads`; decode / prefill: only that one as the headline")
    ap.add_argument("--exchange", default="nvlink", choices=["nvlink", "nccl"],
                    help="N > 1: exchange fused into the layer kernel (NVLink peer stores + ordered sum), or NCCL all-gather + ordered sum")
    ap.add_argument("--router", action="store_true",
                    help="headline decode: produce the routing table on the device inside the timed layer (router matvec + sigmoid "
                         "top-k kernels ahead of the layer kernel) instead of taking it as an input")
    ap.add_argument("--layer-kernels", type=int, default=3, choices=[1, 3],
                    help="windows of <= 16 rows: 3 = gate/up, down, combine (default); 1 = the one-launch layer kernel (comparison runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--record-traffic", nargs=4, metavar=("NCU_CSV", "KEY", "KERNEL_REGEX", "COMMAND"),
                    help="no benchmark: store the per-launch DRAM traffic of an ncu --csv log in profiles/traffic.json (needs no GPU)")
    args = ap.parse_args()
    if args.record_traffic:
        record_traffic(*args.record_traffic)
        return
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    os.environ["GLMFLASH_LAYER_KERNELS"] = str(args.layer_kernels)

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
    assert E % world == 0
    if args.workload == "prefill" and args.rows == 1:
        args.rows = 4096
    b = Bench(args, pkg, synth, torch, dist, dev, rank, world, local)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    workloads = {}
    if args.workload == "prefill":
        head = b.prefill(args.rows, args.steps, args.warmup, cpu=True)
        config = prefill_config(args.rows, min(2, args.layers), world)
        launches = 6 * args.steps
    else:
        head = b.decode(args.rows, args.steps, args.warmup, headline=True, cpu=True)
        config = decode_config(args.rows, args.layers, world)
        per_layer = (1 if args.layer_kernels == 1 else 3) + (1 if args.router else 0)
        launches = per_layer * args.layers * args.steps
        if args.workload == "all":
            for r in ((4, 8, 16) if world == 1 else (16,)):
                if r != args.rows:
                    workloads[f"decode_bs{r}"] = b.decode(r, max(5, args.steps // 2), 3)
            workloads["prefill_4096"] = b.prefill(4096, max(5, args.steps // 2), 3)
    clocks = sampler.stop() if rank == 0 else None              # sampled over every timed region above
    if rank == 0:
        out = {"metric": "EXL3-4bpw MoE layer tok/s", "value": head["value"], "unit": "layer-tokens/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
               "dtype": "f16xf16->f32", "data": "synthetic", "config": config, "clocks": clocks, "e2e": head["e2e"],
               "gpu_launches": launches, "exchange": args.exchange if world > 1 else "none",
               "router": "on device, inside the timed layer" if args.router else "routing table is an input",
               "layer_kernels": args.layer_kernels}
        for k in ("us_per_layer", "stack_tokens_per_s", "graph", "tflops", "e2e_per_layer_host_call", "roofline", "cpu_baseline", "oracle_check",
                  "phases_us_per_layer", "ep_check", "exchange_bf16", "distinct_experts_per_layer", "upstream_kernels_sm100a"):
            if k in head:
                out[k] = head[k]
        out.setdefault("roofline", None)
        out.setdefault("cpu_baseline", None)
        if workloads:
            out["workloads"] = workloads
        if b.failures:
            out["failures"] = b.failures
        print(json.dumps(out))
    code = 0
    if world > 1:
        t = torch.tensor([1.0 if b.failures else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        code = 1 if float(t.item()) else 0
    elif b.failures:
        code = 1
    if code and rank == 0:
        print("bench: " + "; ".join(b.failures), file=sys.stderr)
    finish(world, dist, code)


if __name__ == "__main__":
    main()
