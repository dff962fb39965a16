"""ctypes binding of the CPU oracle (oracle/exl3_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this module; the shipped
library never does.  Every function cites the reference lines it follows in exl3_oracle.c.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libexl3_oracle.so")


def build(force=False):
    """Compile the oracle (and, when the upstream sources are present, the upstream kernels' cubins)."""
    src = os.path.join(_HERE, "exl3_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "all"], stdout=subprocess.DEVNULL)
    return _SO


class Weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("gt", "ut", "dt", "suh_g", "suh_u", "suh_d", "svh_g", "svh_u", "svh_d")]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.gfo_codebook.restype = C.c_uint16
        L.gfo_codebook.argtypes = [C.c_uint32]
        L.gfo_codeword.restype = C.c_uint32
        L.gfo_codeword.argtypes = [C.c_uint32]
        L.gfo_f32_to_f16.restype = C.c_uint16
        L.gfo_f32_to_f16.argtypes = [C.c_float]
        L.gfo_f16_to_f32.restype = C.c_float
        L.gfo_f16_to_f32.argtypes = [C.c_uint16]
        L.gfo_bf.restype = C.c_float
        L.gfo_bf.argtypes = [C.c_float]
        L.gfo_hf.restype = C.c_float
        L.gfo_hf.argtypes = [C.c_float]
        L.gfo_max_threads.restype = C.c_int
        L.gfo_grouping.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    assert a.dtype == dt, (a.dtype, dt)
    return a


def codebook_all():
    """fp16 bits of all 65536 states."""
    L = lib()
    return np.array([L.gfo_codebook(s) for s in range(65536)], dtype=np.uint16)


def decode_tiles(words, form="stream"):
    """words [T][32] u32 -> [T][16][16] fp16 (rows k, columns n)."""
    words = _c(words, np.uint32).reshape(-1, 32)
    out = np.empty((words.shape[0], 256), np.uint16)
    f = lib().gfo_decode_tile_stream if form == "stream" else lib().gfo_decode_tile_lanes
    for i in range(words.shape[0]):
        f(_p(words[i]), _p(out[i]))
    return out.view(np.float16).reshape(-1, 16, 16)


def tile_states(words):
    words = _c(words, np.uint32).reshape(-1, 32)
    out = np.empty((words.shape[0], 256), np.uint16)
    for i in range(words.shape[0]):
        lib().gfo_tile_states(_p(words[i]), _p(out[i]))
    return out


def unpack(words, K, N):
    """words [K/16][N/16][32] u32 -> [K][N] fp16."""
    words = _c(words, np.uint32)
    out = np.empty((K, N), np.uint16)
    lib().gfo_unpack_f16(_p(words), C.c_int(K), C.c_int(N), _p(out))
    return out.view(np.float16)


def had128(x):
    y = np.array(x, dtype=np.float32, copy=True).reshape(-1)
    assert y.size % 128 == 0
    lib().gfo_had128(_p(y), C.c_int(y.size))
    return y.reshape(np.shape(x))


def matmul(x, w, sk=1, mode=0):
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    K, N = w.shape
    y = np.empty(N, np.float32)
    lib().gfo_matmul(_p(x), _p(w), C.c_int(K), C.c_int(N), C.c_int(sk), C.c_int(mode), _p(y))
    return y


def linear_f16(x, words, suh, svh, K, N, sk=4, mode=1):
    """x [rows][K] fp16 -> (y fp16 [rows][N], y fp32 before the final rounding)."""
    x = _c(x, np.float16).reshape(-1, K)
    rows = x.shape[0]
    y = np.empty((rows, N), np.uint16)
    y32 = np.empty((rows, N), np.float32)
    lib().gfo_linear_f16(_p(x), C.c_int(rows), _p(_c(words, np.uint32)), _p(_c(suh, np.float16)),
                         _p(_c(svh, np.float16)), C.c_int(K), C.c_int(N), C.c_int(sk), C.c_int(mode), _p(y), _p(y32))
    return y.view(np.float16), y32


def _weights_struct(w):
    keep = {name: np.ascontiguousarray(w[name]) for name, _ in Weights._fields_}
    s = Weights(**{k: v.ctypes.data for k, v in keep.items()})
    return s, keep


def experts_run_rows(w, H, I, E1, slots, x_bf16, picks, skip_ge=None, limit=10.0, sk_gu=4, sk_dn=1, mode=1,
                     threads=None, want_xd=False):
    """Every pair of a window through its expert.  x_bf16: uint16 [rows][H] (bf16 bits); picks int32
    [rows][slots].  Returns Y fp32 [rows*slots][H] (rows of skipped experts stay NaN) and optionally Xd."""
    x = _c(x_bf16, np.uint16)
    rows = x.shape[0]
    picks = _c(picks, np.int32).reshape(rows, slots)
    s, keep = _weights_struct(w)
    Y = np.full((rows * slots, H), np.nan, np.float32)
    xd = np.full((rows * slots, I), np.nan, np.float32) if want_xd else None
    if threads is None:
        threads = lib().gfo_max_threads()
    lib().gfo_experts_run_rows(C.byref(s), C.c_int(H), C.c_int(I), C.c_int(E1), C.c_int(slots), _p(x),
                               C.c_int(x.shape[1]), _p(picks), C.c_int(rows),
                               C.c_int(E1 if skip_ge is None else skip_ge), C.c_float(limit), C.c_int(sk_gu),
                               C.c_int(sk_dn), C.c_int(mode), C.c_int(threads), _p(Y),
                               _p(xd) if want_xd else None)
    del keep
    return (Y, xd) if want_xd else Y


def combine(Y, weights, rows, slots, H):
    Y = _c(Y, np.float32)
    weights = _c(weights, np.float32)
    out = np.empty((rows, H), np.float32)
    lib().gfo_combine(_p(Y), _p(weights), C.c_int(rows), C.c_int(slots), C.c_int(H), _p(out))
    return out


def grouping(picks, rows, slots, E1, maxm):
    """-> (ids [E1] (first count valid), count, members [E1][maxm])."""
    picks = _c(picks, np.int32).reshape(rows, slots)
    ids = np.full(E1, -1, np.int32)
    count = np.zeros(1, np.int32)
    members = np.empty((E1, maxm), np.int32)
    rc = lib().gfo_grouping(_p(picks), C.c_int(rows), C.c_int(slots), C.c_int(E1), C.c_int(maxm), _p(ids),
                            _p(count), _p(members))
    if rc != 0:
        raise ValueError("grouping: pick out of range or more than maxm members")
    return ids, int(count[0]), members


def router_logits(x_bf16_bits, wr_bf16_bits, rows, H, E):
    """x [rows][H], wr [E][H] as uint16 bf16 bit patterns -> logits fp32 [rows][E] (double accumulation)."""
    x = _c(x_bf16_bits, np.uint16)
    wr = _c(wr_bf16_bits, np.uint16)
    out = np.empty((rows, E), np.float32)
    lib().gfo_router_logits(_p(x), C.c_int(H), _p(wr), C.c_int(rows), C.c_int(H), C.c_int(E), _p(out))
    return out


def topk(logits, rows, E, k):
    """-> picks int32 [rows][k+1], weights fp32 [rows][k+1] (shared expert id E, weight 1, in the last slot)."""
    logits = _c(logits, np.float32)
    picks = np.empty((rows, k + 1), np.int32)
    weights = np.empty((rows, k + 1), np.float32)
    lib().gfo_topk(_p(logits), C.c_int(rows), C.c_int(E), C.c_int(k), _p(picks), _p(weights))
    return picks, weights


def max_threads():
    return lib().gfo_max_threads()
