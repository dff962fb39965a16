"""Host-side mirror of the reference operator surface over the C ABI (include/glmflash_b200.h).

The reference's owners are Rust structs (`ExpertGpu` src/experts.rs:365, `FastExperts`
src/fast_experts.rs:27, `Grouping` src/grouping.rs:12, `Moe` src/moe.rs:11); no Rust toolchain exists in this
build environment, so the owners live in C++ behind the C ABI and this module binds them with ctypes for the
tests and the benchmark.  torch is used only for device memory and streams.  There is no CPU fallback: every
constructor raises when the CUDA library is missing or no GPU is present.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.environ.get("GLMFLASH_B200_SO") or os.path.join(_HERE, "libglmflash_b200.so")


class Config(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("inter", C.c_int32), ("experts", C.c_int32), ("slots", C.c_int32),
                ("max_rows", C.c_int32), ("shared_exl3", C.c_int32), ("expert_lo", C.c_int32),
                ("expert_hi", C.c_int32), ("limit", C.c_float), ("pdl", C.c_int32), ("shared_row_lo", C.c_int32),
                ("shared_row_hi", C.c_int32), ("reserved", C.c_int32 * 4)]


class Weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("gt", "ut", "dt", "suh_g", "suh_u", "suh_d", "svh_g", "svh_u", "svh_d")]


WEIGHT_NAMES = [n for n, _ in Weights._fields_]

# every symbol include/glmflash_b200.h declares: name -> (restype, argtypes)
_P, _I, _Z = C.c_void_p, C.c_int, C.c_size_t
SYMBOLS = {
    "glmflash_abi_version": (_I, []),
    "glmflash_config_bytes": (_Z, []),
    "glmflash_weights_bytes": (_Z, []),
    "glmflash_error": (C.c_char_p, []),
    "glmflash_exl3_decode": (_I, [_P, _P, C.c_int64, _P]),
    "glmflash_exl3_linear_scratch_bytes": (_Z, [_I, _I]),
    "glmflash_exl3_linear": (_I, [_P, _P, _I, _P, _P, _P, _I, _I, _P, _P]),
    "glmflash_exl3_linear_static_max_bytes": (_Z, []),
    "glmflash_exl3_linear_static": (_I, [_P, _P, _I, _P, _P, _P, _I, _I, _P]),
    "glmflash_grouping_new": (_I, [_P, _Z, _P]),
    "glmflash_grouping_free": (None, [_P]),
    "glmflash_grouping_run": (_I, [_P, _P, _P, _I]),
    "glmflash_grouping_ids": (_P, [_P]),
    "glmflash_grouping_count": (_P, [_P]),
    "glmflash_grouping_members": (_P, [_P]),
    "glmflash_experts_new": (_I, [_P, _Z, _P]),
    "glmflash_experts_free": (None, [_P]),
    "glmflash_experts_run_rows": (_I, [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I]),
    "glmflash_experts_y": (_P, [_P]),
    "glmflash_experts_xd": (_P, [_P]),
    "glmflash_experts_status": (_P, [_P]),
    "glmflash_experts_set_phases": (_I, [_P, _I]),
    "glmflash_experts_clear_status": (_I, [_P, _P]),
    "glmflash_fast_experts_clear_status": (_I, [_P, _P]),
    "glmflash_moe_status": (_P, [_P]),
    "glmflash_moe_clear_status": (_I, [_P, _P]),
    "glmflash_moe_run_ep": (_I, [_P, _P, _P, _P, _P, _I, _P, _P, _I, _I]),
    "glmflash_ep_clear_status": (_I, [_P, _P]),
    "glmflash_fast_experts_new": (_I, [_P, _Z, _P]),
    "glmflash_fast_experts_free": (None, [_P]),
    "glmflash_fast_experts_run": (_I, [_P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I]),
    "glmflash_fast_experts_output": (_P, [_P]),
    "glmflash_fast_experts_xd": (_P, [_P]),
    "glmflash_fast_experts_row_pairs": (_P, [_P]),
    "glmflash_fast_experts_plan": (_P, [_P]),
    "glmflash_fast_experts_status": (_P, [_P]),
    "glmflash_fast_experts_set_phases": (_I, [_P, _I]),
    "glmflash_moe_new": (_I, [_P, _Z, _P]),
    "glmflash_moe_free": (None, [_P]),
    "glmflash_moe_run": (_I, [_P, _P, _P, _P, _I, _P, _P, _I]),
    "glmflash_moe_output": (_P, [_P]),
    "glmflash_moe_pairs": (_P, [_P]),
    "glmflash_moe_set_phases": (_I, [_P, _I]),
    "glmflash_moe_run_host": (_I, [_P, _P, _P, _P, _I, _P, _P, _I, _P]),
    "glmflash_rank_sum": (_I, [_P, _P, _I, _I, _I, _P]),
    "glmflash_ep_handle_bytes": (_Z, []),
    "glmflash_ep_new": (_I, [_P, _Z, _I, _I, _P]),
    "glmflash_ep_free": (None, [_P]),
    "glmflash_ep_get_handle": (_I, [_P, _P]),
    "glmflash_ep_connect": (_I, [_P, _P]),
    "glmflash_ep_combine": (_I, [_P, _P, _P, _P, _P, _I, _I]),
    "glmflash_ep_output": (_P, [_P]),
    "glmflash_router_logits": (_I, [_P, _P, _I, _P, _I, _I, _I, _P, _I]),
    "glmflash_topk": (_I, [_P, _P, _I, _I, _I, _P, _P, _I]),
    "glmflash_route": (_I, [_P, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P, _I]),
    "glmflash_ep_status": (_P, [_P]),
    "glmflash_ep_set_wait_limit": (_I, [_P, C.c_uint32]),
    "glmflash_ep_set_exchange_bf16": (_I, [_P, _I]),
    "glmflash_ep_local_base": (_P, [_P]),
    "glmflash_ep_connect_ptrs": (_I, [_P, _P]),
    "glmflash_prepared_open": (_I, [C.c_char_p, _P]),
    "glmflash_prepared_close": (None, [_P]),
    "glmflash_prepared_key_int": (_I, [_P, C.c_char_p, _P]),
    "glmflash_prepared_tensor_count": (_I, [_P]),
    "glmflash_prepared_tensor_name": (C.c_char_p, [_P, _I]),
    "glmflash_prepared_tensor": (_I, [_P, C.c_char_p, _P]),
    "glmflash_prepared_verify": (_I, [_P]),
    "glmflash_prepared_load": (_I, [_P, _P, _I]),
    "glmflash_expert_bank_from_tp": (_I, [_P, _I, C.c_char_p, _I, _I, _P, _P]),
    "glmflash_expert_bank_weights": (_I, [_P, _P, _P, _P]),
    "glmflash_expert_bank_free": (None, [_P]),
    "glmflash_graph_policy_default": (_I, [_I, _P]),
    "glmflash_graph_cache_new": (_I, [_P, _P]),
    "glmflash_graph_cache_free": (None, [_P]),
    "glmflash_graph_cache_action": (_I, [_P, C.c_uint64]),
    "glmflash_graph_cache_insert": (_I, [_P, C.c_uint64, C.c_uint64, _P]),
    "glmflash_graph_cache_get": (_P, [_P, C.c_uint64]),
    "glmflash_graph_cache_stats": (_I, [_P, _P]),
    "glmflash_graph_cache_run": (_I, [_P, C.c_uint64, _P, _P, _P]),
}


class GraphPolicy(C.Structure):
    _fields_ = [("bounded", C.c_int32), ("entries", C.c_uint32), ("nodes", C.c_uint64), ("sightings", C.c_uint32), ("after", C.c_uint32)]


class GraphStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("hits", "eager", "captures", "evictions", "oversized", "retained_graphs", "retained_nodes",
                                          "peak_graphs", "peak_nodes", "largest_graph_nodes", "tracked_sightings")]


ENQUEUE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p)
REPLAY, EAGER, CAPTURE = 0, 1, 2


class GraphCache:
    """Cache::{action, insert} of the reference's verify-window graph cache (src/verifier_graph_cache.rs) and the capture /
    replay step built on it.  The policy part needs no GPU."""

    def __init__(self, policy=None, bounded=True):
        if policy is None:
            policy = GraphPolicy()
            _check(lib().glmflash_graph_policy_default(int(bounded), C.byref(policy)))
        self.policy = policy
        self._h = C.c_void_p()
        _check(lib().glmflash_graph_cache_new(C.byref(policy), C.byref(self._h)))
        self._keep = []

    def action(self, key):
        return lib().glmflash_graph_cache_action(self._h, key)

    def insert(self, key, nodes, graph_exec=None):
        return lib().glmflash_graph_cache_insert(self._h, key, nodes, graph_exec)

    def contains(self, key):
        return bool(lib().glmflash_graph_cache_get(self._h, key)) or key in self._null_keys()

    def _null_keys(self):
        return ()

    def stats(self):
        st = GraphStats()
        _check(lib().glmflash_graph_cache_stats(self._h, C.byref(st)))
        return {n: getattr(st, n) for n, _ in GraphStats._fields_}

    def run(self, key, fn, stream=None):
        """fn(): enqueue the window's work on the current torch stream (it is made current for the call)."""
        torch = _torch()
        st = stream if stream is not None else torch.cuda.current_stream()
        err = []

        def tramp(_user, _stream):
            try:
                with torch.cuda.stream(st):
                    fn()
                return 0
            except Exception as ex:          # noqa: BLE001 -- nothing may cross the C boundary
                err.append(ex)
                return -1
        cb = ENQUEUE_FN(tramp)
        rc = lib().glmflash_graph_cache_run(self._h, key, C.c_void_p(st.cuda_stream), cb, None)
        if err:
            raise err[0]
        _check(rc)

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().glmflash_graph_cache_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TensorInfo(C.Structure):
    _fields_ = [("dtype", C.c_char * 16), ("rank", C.c_int32), ("on_device", C.c_int32), ("contiguous", C.c_int32),
                ("reserved", C.c_int32), ("shape", C.c_int64 * 8), ("stride", C.c_int64 * 8), ("nbytes", C.c_int64), ("ptr", C.c_void_p)]


class Prepared:
    """Prepared::{open, tensor, load_selected} + Loaded::pointer (reference src/prepared.rs:151-377).  Opening and
    verifying need no GPU."""

    def __init__(self, manifest_path):
        self._h = C.c_void_p()
        _check(lib().glmflash_prepared_open(str(manifest_path).encode(), C.byref(self._h)))

    def key_int(self, name):
        v = C.c_int64()
        _check(lib().glmflash_prepared_key_int(self._h, name.encode(), C.byref(v)))
        return v.value

    def names(self):
        L = lib()
        return [L.glmflash_prepared_tensor_name(self._h, i).decode() for i in range(L.glmflash_prepared_tensor_count(self._h))]

    def tensor(self, name):
        info = TensorInfo()
        _check(lib().glmflash_prepared_tensor(self._h, name.encode(), C.byref(info)))
        return {"dtype": info.dtype.decode(), "shape": list(info.shape[: info.rank]), "stride": list(info.stride[: info.rank]),
                "nbytes": info.nbytes, "on_device": bool(info.on_device), "contiguous": bool(info.contiguous), "ptr": info.ptr}

    def verify(self):
        _check(lib().glmflash_prepared_verify(self._h))

    def load(self, prefixes=()):
        arr = (C.c_char_p * max(1, len(prefixes)))(*[p.encode() for p in prefixes])
        _check(lib().glmflash_prepared_load(self._h, arr, len(prefixes)))

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().glmflash_prepared_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ExpertBank:
    """Whole experts [e_lo, e_hi) assembled from the tensor-parallel shards of `stem` (glmflash_expert_bank_from_tp)."""

    def __init__(self, shards, stem, e_lo, e_hi, stream=None):
        arr = (C.c_void_p * len(shards))(*[s._h for s in shards])
        self._h = C.c_void_p()
        _check(lib().glmflash_expert_bank_from_tp(arr, len(shards), stem.encode(), e_lo, e_hi, _stream_ptr(stream), C.byref(self._h)))
        self.weights = Weights()
        h, i = C.c_int32(), C.c_int32()
        _check(lib().glmflash_expert_bank_weights(self._h, C.byref(self.weights), C.byref(h), C.byref(i)))
        self.hidden, self.inter = h.value, i.value

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().glmflash_expert_bank_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

_lib = None


class GlmFlashError(RuntimeError):
    pass


def lib():
    """The loaded C-ABI library.  Raises when it has not been built: there is no other path."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise GlmFlashError(f"{SO_PATH} is missing: build it (python -c 'import __graft_entry__ as g; g.build()')")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in SYMBOLS.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        if L.glmflash_abi_version() != 1 or L.glmflash_config_bytes() != C.sizeof(Config) or \
                L.glmflash_weights_bytes() != C.sizeof(Weights):
            raise GlmFlashError("ABI mismatch between the python binding and libglmflash_b200.so")
        _lib = L
    return _lib


def _check(rc):
    if rc != 0:
        raise GlmFlashError(lib().glmflash_error().decode())


def make_config(hidden=2048, inter=1536, experts=64, slots=5, max_rows=1, shared_exl3=1, expert_lo=0,
                expert_hi=None, limit=10.0, pdl=1, shared_rows=(0, 0)):
    return Config(hidden, inter, experts, slots, max_rows, shared_exl3, expert_lo,
                  experts if expert_hi is None else expert_hi, limit, pdl, shared_rows[0], shared_rows[1])


def _torch():
    import torch
    if not torch.cuda.is_available():
        raise GlmFlashError("no CUDA device: this library has no CPU path")
    return torch


def _stream_ptr(stream=None):
    torch = _torch()
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def weights_struct(w):
    """w: mapping name -> CUDA torch tensor (gt/ut/dt int32, scales float16).  Keeps nothing alive."""
    return Weights(**{n: w[n].data_ptr() for n in WEIGHT_NAMES})


def _view(ptr, shape, dtype):
    """A torch view of library-owned device memory (valid while the owner lives)."""
    torch = _torch()
    import numpy as np
    n = int(np.prod(shape))
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (n * itemsize,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}
    return torch.as_tensor(h, device="cuda").view(dtype).view(*shape)


def exl3_decode(words, stream=None):
    """words: int32/uint32-bit CUDA tensor [tiles][32] -> float16 [tiles][16][16] (k, n)."""
    torch = _torch()
    tiles = words.numel() // 32
    out = torch.empty((tiles, 16, 16), dtype=torch.float16, device=words.device)
    _check(lib().glmflash_exl3_decode(_stream_ptr(stream), words.data_ptr(), tiles, out.data_ptr()))
    return out


def exl3_linear(x, words, suh, svh, K, N, stream=None):
    """x fp16 [rows][K] (rows <= 16) -> fp16 [rows][N]."""
    torch = _torch()
    rows = x.shape[0]
    nbytes = lib().glmflash_exl3_linear_scratch_bytes(K, N)
    if nbytes == 0:
        raise GlmFlashError("unsupported linear shape")
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    y = torch.empty((rows, N), dtype=torch.float16, device=x.device)
    _check(lib().glmflash_exl3_linear(_stream_ptr(stream), x.data_ptr(), rows, words.data_ptr(), suh.data_ptr(),
                                      svh.data_ptr(), K, N, y.data_ptr(), scratch.data_ptr()))
    torch.cuda.current_stream().synchronize()      # scratch is freed on return
    return y


def exl3_linear_static(x, words, suh, svh, K, N, stream=None):
    """exl3_linear without any allocation inside the library: the scratch is the library's built-in array
    (K <= 4096).  Calls that overlap on the GPU share that array and must be ordered by the caller."""
    torch = _torch()
    rows = x.shape[0]
    y = torch.empty((rows, N), dtype=torch.float16, device=x.device)
    _check(lib().glmflash_exl3_linear_static(_stream_ptr(stream), x.data_ptr(), rows, words.data_ptr(), suh.data_ptr(),
                                             svh.data_ptr(), K, N, y.data_ptr()))
    return y


class _Owner:
    _new = _free = None

    def __init__(self, cfg):
        _torch()
        self.cfg = cfg
        self._h = C.c_void_p()
        _check(getattr(lib(), self._new)(C.byref(cfg), C.sizeof(cfg), C.byref(self._h)))

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            getattr(lib(), self._free)(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Grouping(_Owner):
    """Grouping::{new,run} + ids/count/members (reference src/grouping.rs:29-111)."""
    _new, _free = "glmflash_grouping_new", "glmflash_grouping_free"

    def run(self, picks, rows, stream=None):
        _check(lib().glmflash_grouping_run(self._h, _stream_ptr(stream), picks.data_ptr(), rows))

    @property
    def ids(self):
        import torch
        return _view(lib().glmflash_grouping_ids(self._h), (self.cfg.experts + 1,), torch.int32)

    @property
    def count(self):
        import torch
        return _view(lib().glmflash_grouping_count(self._h), (1,), torch.int32)

    @property
    def members(self):
        import torch
        return _view(lib().glmflash_grouping_members(self._h), (self.cfg.experts + 1, self.cfg.max_rows), torch.int32)


class ExpertGpu(_Owner):
    """ExpertGpu::{new_rows,run_rows,y} (reference src/experts.rs:382-563)."""
    _new, _free = "glmflash_experts_new", "glmflash_experts_free"

    def run_rows(self, w, x, picks, ids, count, members, rows, maxm, x_stride=None, stream=None):
        ws = w if isinstance(w, Weights) else weights_struct(w)
        _check(lib().glmflash_experts_run_rows(self._h, _stream_ptr(stream), C.byref(ws), x.data_ptr(),
                                               x_stride or x.stride(0), picks.data_ptr(), ids.data_ptr(),
                                               count.data_ptr(), members.data_ptr(), rows, maxm))

    @property
    def y(self):
        import torch
        return _view(lib().glmflash_experts_y(self._h), (self.cfg.max_rows * self.cfg.slots, self.cfg.hidden),
                     torch.float32)

    @property
    def xd(self):
        import torch
        return _view(lib().glmflash_experts_xd(self._h), (self.cfg.max_rows * self.cfg.slots, self.cfg.inter),
                     torch.float16)

    @property
    def status(self):
        import torch
        return _view(lib().glmflash_experts_status(self._h), (1,), torch.int32)


class FastExperts(_Owner):
    """FastExperts::{new,run,output} (reference src/fast_experts.rs:43-208)."""
    _new, _free = "glmflash_fast_experts_new", "glmflash_fast_experts_free"

    def run(self, w, x, picks, ids, count, members, rows, maxm, shared_x=False, x_stride=None, stream=None):
        ws = w if isinstance(w, Weights) else weights_struct(w)
        _check(lib().glmflash_fast_experts_run(self._h, _stream_ptr(stream), C.byref(ws), x.data_ptr(),
                                               x_stride or x.stride(0), picks.data_ptr(), ids.data_ptr(),
                                               count.data_ptr(), members.data_ptr(), rows, maxm, int(shared_x)))

    @property
    def output(self):
        import torch
        return _view(lib().glmflash_fast_experts_output(self._h),
                     (self.cfg.max_rows * self.cfg.slots, self.cfg.hidden), torch.float32)

    @property
    def xd(self):
        """fp16 [grouped rows][I]; grouped row j is pair row_pairs[j] (valid rows: plan[1])."""
        import torch
        return _view(lib().glmflash_fast_experts_xd(self._h), (self.cfg.max_rows * self.cfg.slots, self.cfg.inter),
                     torch.float16)

    def set_phases(self, mask):
        _check(lib().glmflash_fast_experts_set_phases(self._h, mask))

    @property
    def row_pairs(self):
        import torch
        return _view(lib().glmflash_fast_experts_row_pairs(self._h), (self.cfg.max_rows * self.cfg.slots,), torch.int32)

    @property
    def plan(self):
        import torch
        return _view(lib().glmflash_fast_experts_plan(self._h), (2,), torch.int32)

    @property
    def status(self):
        import torch
        return _view(lib().glmflash_fast_experts_status(self._h), (1,), torch.int32)


class Moe(_Owner):
    """Moe::{new,run,output}: grouping -> experts -> combine (reference src/moe.rs:28-182)."""
    _new, _free = "glmflash_moe_new", "glmflash_moe_free"

    def run(self, w, x, picks, route_w, rows, x_stride=None, stream=None):
        ws = w if isinstance(w, Weights) else weights_struct(w)
        _check(lib().glmflash_moe_run(self._h, _stream_ptr(stream), C.byref(ws), x.data_ptr(),
                                      x_stride or x.stride(0), picks.data_ptr(), route_w.data_ptr(), rows))

    def run_host(self, w, x_host, picks_host, route_w_host, rows, out_host, stream=None):
        """Host (pinned) buffers in, host buffer out; synchronises.  The end-to-end entry point."""
        ws = w if isinstance(w, Weights) else weights_struct(w)
        _check(lib().glmflash_moe_run_host(self._h, _stream_ptr(stream), C.byref(ws), x_host.data_ptr(),
                                           self.cfg.hidden, picks_host.data_ptr(), route_w_host.data_ptr(), rows,
                                           out_host.data_ptr()))

    def set_phases(self, mask):
        _check(lib().glmflash_moe_set_phases(self._h, mask))

    def run_ep(self, ep, w, x, picks, route_w, rows, shared_here=-1, x_stride=None, stream=None):
        """The layer and its cross-GPU exchange (glmflash_moe_run_ep); result: ep.output[:rows]."""
        ws = w if isinstance(w, Weights) else weights_struct(w)
        _check(lib().glmflash_moe_run_ep(self._h, ep._h, _stream_ptr(stream), C.byref(ws), x.data_ptr(),
                                         x_stride or x.stride(0), picks.data_ptr(), route_w.data_ptr(), rows, int(shared_here)))
        return ep.output[:rows]

    @property
    def status(self):
        import torch
        return _view(lib().glmflash_moe_status(self._h), (1,), torch.int32)

    def clear_status(self, stream=None):
        _check(lib().glmflash_moe_clear_status(self._h, _stream_ptr(stream)))

    @property
    def pairs_ptr(self):
        """Device address of the pair results Y fp32 [rows*slots][H] of the last run."""
        return C.c_void_p(lib().glmflash_moe_pairs(self._h))

    @property
    def output(self):
        import torch
        return _view(lib().glmflash_moe_output(self._h), (self.cfg.max_rows, self.cfg.hidden), torch.float32)


def router_logits(x, wr, logits, stream=None, pdl=1):
    """logits[r][e] = x[r] . wr[e]  (x bf16 [rows][H], wr bf16 [E][H], logits fp32 [rows][E]; CUDA tensors)."""
    rows, E = logits.shape
    _check(lib().glmflash_router_logits(_stream_ptr(stream), x.data_ptr(), x.stride(0), wr.data_ptr(), rows, wr.shape[1], E,
                                        logits.data_ptr(), pdl))
    return logits


def topk(logits, picks, weights, stream=None, pdl=1):
    """Sigmoid top-k of logits fp32 [rows][E] into picks int32 / weights fp32 [rows][k + 1] (shared expert last)."""
    rows, E = logits.shape
    _check(lib().glmflash_topk(_stream_ptr(stream), logits.data_ptr(), rows, E, picks.shape[1] - 1, picks.data_ptr(),
                               weights.data_ptr(), pdl))
    return picks, weights


def route(x, wr, logits, picks, weights, stream=None, pdl=1):
    """router_logits + topk; one launch for windows of <= 16 rows."""
    rows, E = logits.shape
    _check(lib().glmflash_route(_stream_ptr(stream), x.data_ptr(), x.stride(0), wr.data_ptr(), rows, wr.shape[1], E,
                                picks.shape[1] - 1, logits.data_ptr(), picks.data_ptr(), weights.data_ptr(), pdl))
    return picks, weights


def rank_sum(gathered, out, stream=None):
    """out[r] = sum over ranks in ascending order of gathered[rank][r] (fp32 [world][rows][H])."""
    world, rows, H = gathered.shape
    _check(lib().glmflash_rank_sum(_stream_ptr(stream), gathered.data_ptr(), world, rows, H, out.data_ptr()))
    return out


class EpCombine:
    """glmflash_ep_*: combine fused with the cross-GPU exchange over NVLink (one owner per rank).
    `exchange_handles(local_bytes) -> list of every rank's bytes in rank order` is the host's bootstrap channel
    (torch.distributed.all_gather_object in the tests and the benchmark)."""

    def __init__(self, cfg, rank, world, exchange_handles):
        _torch()
        self.cfg, self.rank, self.world = cfg, rank, world
        self._h = C.c_void_p()
        _check(lib().glmflash_ep_new(C.byref(cfg), C.sizeof(cfg), rank, world, C.byref(self._h)))
        if world > 1 and exchange_handles is not None:
            n = lib().glmflash_ep_handle_bytes()
            buf = C.create_string_buffer(n)
            _check(lib().glmflash_ep_get_handle(self._h, buf))
            allh = exchange_handles(bytes(buf.raw))
            assert len(allh) == world and all(len(b) == n for b in allh)
            _check(lib().glmflash_ep_connect(self._h, C.create_string_buffer(b"".join(allh), n * world)))

    def combine(self, Y_ptr, picks, route_w, rows, shared_here, stream=None):
        _check(lib().glmflash_ep_combine(self._h, _stream_ptr(stream), Y_ptr, picks.data_ptr(), route_w.data_ptr(), rows,
                                         int(shared_here)))
        return self.output[:rows]

    @property
    def output(self):
        import torch
        return _view(lib().glmflash_ep_output(self._h), (self.cfg.max_rows, self.cfg.hidden), torch.float32)

    @property
    def status(self):
        import torch
        return _view(lib().glmflash_ep_status(self._h), (1,), torch.int32)

    @property
    def local_base(self):
        return lib().glmflash_ep_local_base(self._h)

    def connect_ptrs(self, bases):
        """Same-process peers: `bases[k]` = local_base of rank k's owner."""
        arr = (C.c_void_p * self.world)(*[C.c_void_p(b) for b in bases])
        _check(lib().glmflash_ep_connect_ptrs(self._h, arr))

    def clear_status(self, stream=None):
        _check(lib().glmflash_ep_clear_status(self._h, _stream_ptr(stream)))

    def set_exchange_bf16(self, on):
        """Windows of more than 16 rows: partial rows cross NVLink as bf16 (every rank must choose the same)."""
        _check(lib().glmflash_ep_set_exchange_bf16(self._h, int(bool(on))))

    def set_wait_limit(self, polls):
        _check(lib().glmflash_ep_set_wait_limit(self._h, polls))

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            lib().glmflash_ep_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
