"""GPU-side reference: the upstream CUDA kernels, compiled UNMODIFIED for sm_100a into oracle/_ref/*.cubin
(see oracle/Makefile), loaded with the CUDA driver API and launched exactly as the upstream Rust host
launches them (src/experts.rs:447-563, src/grouping.rs:51-111, src/fast_experts.rs:91-208: one 64-bit
little-endian word per parameter, block (threads,1,1)).  TEST INFRASTRUCTURE ONLY: the parity tests and the
benchmark's comparison leg use it as the checker / baseline; the shipped library never touches it.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")

_cu = None


def _driver():
    global _cu
    if _cu is None:
        _cu = C.CDLL("libcuda.so.1")
    return _cu


def available():
    return all(os.path.exists(os.path.join(REF_DIR, f + ".cubin")) for f in ("exl3", "grouping", "exl3_prefill"))


class Module:
    def __init__(self, name):
        import torch
        torch.cuda.init()
        torch.zeros(1, device="cuda")                 # make sure the primary context is current
        self.mod = C.c_void_p()
        path = os.path.join(REF_DIR, name + ".cubin").encode()
        rc = _driver().cuModuleLoad(C.byref(self.mod), path)
        if rc != 0:
            raise RuntimeError(f"cuModuleLoad({name}) failed: {rc}")
        self.fns = {}

    def fn(self, symbol, smem=0):
        if symbol not in self.fns:
            f = C.c_void_p()
            rc = _driver().cuModuleGetFunction(C.byref(f), self.mod, symbol.encode())
            if rc != 0:
                raise RuntimeError(f"cuModuleGetFunction({symbol}) failed: {rc}")
            if smem > 0:                              # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8
                rc = _driver().cuFuncSetAttribute(f, 8, smem)
                if rc != 0:
                    raise RuntimeError(f"cuFuncSetAttribute({symbol}) failed: {rc}")
            self.fns[symbol] = f
        return self.fns[symbol]

    def launch(self, symbol, grid, threads, words, smem=0, stream=None):
        """words: python ints (pointers, ints) or floats (passed as their fp32 bit pattern)."""
        import struct
        import torch
        vals = []
        for w in words:
            if isinstance(w, float):
                w = struct.unpack("<I", struct.pack("<f", w))[0]
            vals.append(C.c_uint64(int(w) & 0xFFFFFFFFFFFFFFFF))
        params = (C.c_void_p * len(vals))(*[C.cast(C.byref(v), C.c_void_p) for v in vals])
        s = stream if stream is not None else torch.cuda.current_stream()
        rc = _driver().cuLaunchKernel(self.fn(symbol, smem), C.c_uint(grid[0]), C.c_uint(grid[1]), C.c_uint(grid[2]),
                                      C.c_uint(threads), C.c_uint(1), C.c_uint(1), C.c_uint(smem),
                                      C.c_void_p(s.cuda_stream), params, None)
        if rc != 0:
            raise RuntimeError(f"cuLaunchKernel({symbol}) failed: {rc}")


_mods = {}
_fast_scratch = {}


def module(name):
    if name not in _mods:
        _mods[name] = Module(name)
    return _mods[name]


def experts_run_rows(w, x, picks, ids, count, members, rows, maxm, H, I, E, slots, grouped="exl3_grouped_8_4"):
    """The upstream decode / verify pipeline (src/experts.rs:447-563) on CUDA tensors.

    Upstream never computes the last slot of a row (its shared expert is not EXL3).  To obtain the shared
    expert's EXL3 result from the unmodified kernels the caller passes picks / members built with one extra,
    unused trailing slot (slots = real slots + 1) and E = number of EXL3 experts including the shared one.
    Returns Y fp32 [rows*slots][H] and Xd fp16 [rows*slots][I].  SK = 4 for gate/up and 1 for down, as upstream.
    """
    import torch
    m = module("expert_loads" if grouped == "exl3_load_nc_8_1" else "exl3")
    base = module("exl3")
    P = rows * slots
    dev = x.device
    xg = torch.zeros((P, H), dtype=torch.float16, device=dev)
    xu = torch.zeros((P, H), dtype=torch.float16, device=dev)
    xd = torch.zeros((P, I), dtype=torch.float16, device=dev)
    z = torch.zeros(2 * 4 * P * max(H, I), dtype=torch.float32, device=dev)
    y = torch.zeros((P, H), dtype=torch.float32, device=dev)
    distinct = min(rows * (slots - 1) + 1, E + 1)
    mt = (maxm + 15) // 16
    p = lambda t: t.data_ptr()
    base.launch("rot_in_kernel", (P, H // 128, 2), 32,
                [p(x), x.stride(0), p(picks), p(w["suh_g"]), p(w["suh_u"]), p(xg), p(xu), H, slots])
    m.launch(grouped, (distinct, I // 128, 2 * 4 * mt), 128,
             [p(xg), p(xu), p(w["gt"]), p(w["ut"]), p(ids), p(count), p(members), p(z), H, I, P, 4, maxm, slots, E])
    base.launch("gateup_epilogue_kernel", (P, I // 128, 1), 32,
                [p(z), p(picks), p(w["svh_g"]), p(w["svh_u"]), p(w["suh_d"]), p(xd), P, I, 4, slots, 10.0, 0])
    m.launch(grouped, (distinct, H // 128, 1 * 1 * mt), 128,
             [p(xd), p(xd), p(w["dt"]), p(w["dt"]), p(ids), p(count), p(members), p(z), I, H, P, 1, maxm, slots, E])
    base.launch("down_epilogue_kernel", (P, H // 128, 1), 32, [p(z), p(picks), p(w["svh_d"]), p(y), P, H, 1, slots, 0])
    return y, xd


def grouping_run(picks, rows, max_rows):
    """Upstream Grouping::run (src/grouping.rs:51-111); fixed upstream sizes E = 289, slots = 9.
    Returns ids [289], count [1], members [289][max_rows] (int32 CUDA tensors)."""
    import torch
    E = 289
    g = module("grouping")
    dev = picks.device
    ids = torch.full((E,), -77, dtype=torch.int32, device=dev)
    count = torch.zeros(1, dtype=torch.int32, device=dev)
    members = torch.full((E, max_rows), 12345, dtype=torch.int32, device=dev)
    p = lambda t: t.data_ptr()
    if rows <= 32 and max_rows <= 32:
        g.launch("group_small", (1, 1, 1), 512, [p(picks), rows, p(ids), p(count), p(members), max_rows])
        return ids, count, members
    bits = torch.zeros(E * 256, dtype=torch.int32, device=dev)
    prefix = torch.zeros(E * 256, dtype=torch.int32, device=dev)
    counts = torch.zeros(E, dtype=torch.int32, device=dev)
    place = torch.zeros(E, dtype=torch.int32, device=dev)
    g.launch("group_clear", (E, 1, 1), 256, [p(bits)])
    g.launch("group_mark", ((rows + 255) // 256, 1, 1), 256, [p(picks), p(bits), rows])
    g.launch("group_prefix", (E, 1, 1), 256, [p(bits), p(prefix), p(counts)])
    g.launch("group_ids", (1, 1, 1), 512, [p(counts), p(place), p(ids), p(count)])
    g.launch("group_scatter", (E, 1, 1), 256,
             [p(picks), p(bits), p(prefix), p(counts), p(place), p(count), p(members), max_rows])
    return ids, count, members


def fast_experts_run(w, x, picks, ids, count, members, rows, maxm, H, I, E, slots, shared_x=False, stream=None):
    """Upstream FastExperts::run (src/fast_experts.rs:91-208).  Same trailing-slot convention as
    experts_run_rows.  Returns output fp32 [rows*slots][H], xd fp16 [rows*slots][I]."""
    import torch
    pf = module("exl3_prefill")
    base = module("exl3")
    dev = x.device
    P = rows * slots
    maxu = E + 1
    key = (P, H, I, maxu, bool(shared_x), str(dev))
    if stream is not None and key in _fast_scratch:           # timing mode: scratch is allocated once, as upstream's owner does
        xg, xu, xd, out, plan = _fast_scratch[key]
    else:
        xg = torch.zeros((P, H), dtype=torch.float16, device=dev)
        xu = xg if shared_x else torch.zeros((P, H), dtype=torch.float16, device=dev)
        xd = torch.zeros((P, I), dtype=torch.float16, device=dev)
        out = torch.zeros((P, H), dtype=torch.float32, device=dev)
        plan = torch.zeros(maxu + 3, dtype=torch.int32, device=dev)
        if stream is not None:
            torch.cuda.synchronize()
            _fast_scratch[key] = (xg, xu, xd, out, plan)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    p = lambda t: t.data_ptr()
    if shared_x:
        items = P * (H // 128)
        pf.launch("fast_rot_in", ((items + 7) // 8, 1, 1), 256, [p(x), x.stride(0), p(picks), p(w["suh_g"]), p(xg), H, slots, items], stream=stream)
    else:
        base.launch("rot_in_kernel", (P, H // 128, 2), 32,
                    [p(x), x.stride(0), p(picks), p(w["suh_g"]), p(w["suh_u"]), p(xg), p(xu), H, slots], stream=stream)
    ticket = p(plan) + (maxu + 2) * 4
    pf.launch("fast_expert_plan", (1, 1, 1), 1024, [p(ids), p(count), p(members), maxu, maxm, E, 64, p(plan)], stream=stream)
    gu, smem, occ = ("fast_gu_shared", 49152, 2) if shared_x else ("fast_gu_separate", 73728, 1)
    pf.launch(gu, (sms * occ, 1, 1), 256,
              [p(xg), p(xu), p(w["gt"]), p(w["ut"]), p(ids), p(members), p(plan), ticket, H, I, maxm, slots, maxu,
               p(w["svh_g"]), p(w["svh_u"]), p(w["suh_d"]), p(xd), 0, 10.0], smem=smem, stream=stream)
    large = maxm >= 4096
    pf.launch("fast_expert_plan", (1, 1, 1), 1024, [p(ids), p(count), p(members), maxu, maxm, E, 128 if large else 64, p(plan)], stream=stream)
    dn, smem = ("fast_down_large", 33792) if large else ("fast_down", 36864)
    pf.launch(dn, (sms * 2, 1, 1), 128,
              [p(xd), p(xd), p(w["dt"]), p(w["dt"]), p(ids), p(members), p(plan), ticket, I, H, maxm, slots, maxu,
               p(w["svh_d"]), p(w["svh_d"]), p(w["svh_d"]), 0, p(out), 0.0], smem=smem, stream=stream)
    return out, xd
