"""ctypes view of the CPU oracle (oracle/libmlxs_oracle.so).  Test infrastructure: only the tests, the smoke check
and the benchmark's CPU-baseline leg import this."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
_LIB = None

SCORE_SQRTSOFTPLUS, SCORE_SIGMOID, SCORE_SOFTMAX = 0, 1, 2
BANK_EXL3, BANK_MXFP4, BANK_NVFP4, BANK_EXL3_K2 = 0, 1, 2, 3


class Geom(C.Structure):
    _fields_ = [("off", C.c_uint64 * 9), ("len", C.c_uint64 * 9), ("logical_bytes", C.c_uint64),
                ("record_bytes", C.c_uint64)]


class LayerCfg(C.Structure):
    _fields_ = [("bank", C.c_int), ("hidden", C.c_uint64), ("inter", C.c_uint64), ("n_experts", C.c_uint64),
                ("top_k", C.c_uint64), ("limit", C.c_double), ("chain_rounding", C.c_int),
                ("shared_bf16_add", C.c_int)]


def build():
    subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)


def lib():
    global _LIB
    if _LIB is None:
        so = ORACLE_DIR / "libmlxs_oracle.so"
        src = ORACLE_DIR / "mlxs_oracle.c"
        if not so.exists() or (src.exists() and so.stat().st_mtime < src.stat().st_mtime):
            build()
        L = C.CDLL(str(so))
        L.orc_splitmix64.restype = C.c_uint64
        L.orc_mul1_decode.restype = C.c_uint16
        L.orc_h2f.restype = C.c_float
        L.orc_f2h.restype = C.c_uint16
        L.orc_f2h.argtypes = [C.c_double]
        L.orc_bf16_round.restype = C.c_float
        L.orc_bf16_round.argtypes = [C.c_float]
        L.orc_swiglu_clamped.restype = C.c_double
        L.orc_swiglu_clamped.argtypes = [C.c_double, C.c_double, C.c_double]
        for n in ("orc_e2m1_value", "orc_e4m3_kernel", "orc_e4m3_value", "orc_e8m0_value", "orc_mxfp4_scale_ref"):
            getattr(L, n).restype = C.c_float
        L.orc_e4m3_kernel.argtypes = [C.c_uint8]
        L.orc_e4m3_value.argtypes = [C.c_uint8]
        L.orc_e2m1_halfbits.restype = C.c_uint16
        for n in ("orc_nvfp4_weight", "orc_nvfp4_kernel_weight"):
            getattr(L, n).restype = C.c_float
            getattr(L, n).argtypes = [C.c_uint8, C.c_uint32, C.c_float]
        L.orc_silu_mul_ref.restype = C.c_float
        L.orc_silu_mul_ref.argtypes = [C.c_float, C.c_float]
        L.orc_silu_mul_clamped_ref.restype = C.c_float
        L.orc_silu_mul_clamped_ref.argtypes = [C.c_float, C.c_float, C.c_float]
        L.orc_det_expf.restype = C.c_float
        L.orc_det_expf.argtypes = [C.c_float]
        L.orc_det_logf.restype = C.c_float
        L.orc_det_logf.argtypes = [C.c_float]
        L.orc_mxfp4_record_bytes.restype = C.c_uint64
        L.orc_nvfp4_record_bytes.restype = C.c_uint64
        L.orc_fill_scales.argtypes = [C.c_uint64, C.c_double, C.c_void_p, C.c_size_t]
        L.orc_fill_code.argtypes = [C.c_uint64, C.c_void_p, C.c_size_t]
        L.orc_fill_x_bf16.argtypes = [C.c_uint64, C.c_void_p, C.c_size_t]
        L.orc_exl3_synth_record.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_double, C.c_double, C.c_void_p]
        L.orc_exl3_synth_record_k.argtypes = [C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_double, C.c_double, C.c_void_p]
        L.orc_mxfp4_synth_record.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_double, C.c_void_p]
        L.orc_nvfp4_synth_record.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_double, C.c_void_p]
        L.orc_exl3_expert_f64.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_double, C.c_void_p, C.c_size_t,
                                          C.c_void_p, C.c_void_p]
        L.orc_exl3_expert_f32chain.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_size_t,
                                               C.c_void_p, C.c_void_p]
        L.orc_reconstruct.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p,
                                      C.c_void_p]
        L.orc_tile_states.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        for n in ("orc_route_libm", "orc_route_det"):
            getattr(L, n).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_int,
                                      C.c_float, C.c_void_p, C.c_void_p]
        L.orc_dispatch.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p]
        L.orc_layer.argtypes = [C.POINTER(LayerCfg), C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p,
                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_layer_fast.argtypes = [C.POINTER(LayerCfg), C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_mxfp4_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.orc_nvfp4_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_size_t, C.c_size_t, C.c_void_p]
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ---- numpy-level helpers -------------------------------------------------------------------------------------

def mul1_table():
    t = np.empty(65536, np.uint16)
    lib().orc_mul1_table(_p(t))
    return t


def fill_code(seed, n):
    out = np.empty(n, np.int16)
    lib().orc_fill_code(seed, _p(out), n)
    return out


def fill_scales(seed, scale, n):
    out = np.empty(n, np.uint16)
    lib().orc_fill_scales(seed, scale, _p(out), n)
    return out


def fill_x_bf16(seed, n):
    out = np.empty(n, np.float32)
    lib().orc_fill_x_bf16(seed, _p(out), n)
    return out


def reconstruct(code, n_i, n_j, K, table=None, want_states=False):
    table = mul1_table() if table is None else table
    w = np.empty((n_i * 16, n_j * 16), np.uint16)
    st = np.empty_like(w) if want_states else None
    lib().orc_reconstruct(_p(code), n_i, n_j, K, _p(table), _p(w), _p(st))
    return (w, st) if want_states else w


def exl3_geometry(hidden, inter, K=3):
    g = Geom()
    rc = lib().orc_exl3_geometry(K, C.c_uint64(hidden), C.c_uint64(inter), C.byref(g))
    if rc:
        raise ValueError("bad EXL3 geometry")
    return g


def exl3_synth_record(seed, hidden, inter, suh_scale=1.0, svh_scale=0.02, K=3):
    g = exl3_geometry(hidden, inter, K)
    rec = np.zeros(g.record_bytes, np.uint8)
    lib().orc_exl3_synth_record_k(K, seed, hidden, inter, suh_scale, svh_scale, _p(rec))
    return rec


def mxfp4_record_bytes(hidden, inter):
    off = (C.c_uint64 * 6)()
    n = lib().orc_mxfp4_record_bytes(C.c_uint64(hidden), C.c_uint64(inter), off)
    return int(n), [int(x) for x in off]


def nvfp4_record_bytes(hidden, inter):
    off = (C.c_uint64 * 9)()
    n = lib().orc_nvfp4_record_bytes(C.c_uint64(hidden), C.c_uint64(inter), off)
    return int(n), [int(x) for x in off]


def mxfp4_synth_record(seed, hidden, inter, sigma=0.02):
    n, _ = mxfp4_record_bytes(hidden, inter)
    rec = np.zeros(n, np.uint8)
    lib().orc_mxfp4_synth_record(seed, hidden, inter, sigma, _p(rec))
    return rec


def nvfp4_synth_record(seed, hidden, inter, sigma=0.02):
    n, _ = nvfp4_record_bytes(hidden, inter)
    rec = np.zeros(n, np.uint8)
    lib().orc_nvfp4_synth_record(seed, hidden, inter, sigma, _p(rec))
    return rec


def exl3_expert_f64(rec, hidden, inter, x, limit=10.0):
    x = np.ascontiguousarray(x, np.float64).reshape(-1, hidden)
    rows = x.shape[0]
    h = np.empty((rows, inter), np.float64)
    y = np.empty((rows, hidden), np.float64)
    rc = lib().orc_exl3_expert_f64(_p(rec), hidden, inter, limit, _p(x), rows, _p(h), _p(y))
    assert rc == 0, rc
    return h, y


def exl3_expert_f32chain(rec, hidden, inter, x):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, hidden)
    rows = x.shape[0]
    h = np.empty((rows, inter), np.float32)
    y = np.empty((rows, hidden), np.float32)
    rc = lib().orc_exl3_expert_f32chain(_p(rec), hidden, inter, _p(x), rows, _p(h), _p(y))
    assert rc == 0, rc
    return h, y


def route(logits, bias, k, scoring, norm=True, scale=1.0, det=True):
    logits = np.ascontiguousarray(logits, np.float32)
    T, E = logits.shape
    ids = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    fn = lib().orc_route_det if det else lib().orc_route_libm
    rc = fn(_p(logits), _p(b), T, E, k, scoring, int(norm), scale, _p(ids), _p(w))
    assert rc == 0, rc
    return ids, w


def dispatch(slot, n_slots):
    slot = np.ascontiguousarray(slot, np.int32).reshape(-1)
    n = slot.size
    order = np.empty(n, np.uint32)
    sorted_slot = np.empty(n, np.uint32)
    inv = np.empty(n, np.uint32)
    offs = np.empty(n_slots + 1, np.uint32)
    lib().orc_dispatch(_p(slot), n, n_slots, _p(order), _p(sorted_slot), _p(inv), _p(offs))
    return order, sorted_slot, inv, offs


def _records_array(records, n_experts):
    arr = (C.c_void_p * n_experts)()
    for e in range(n_experts):
        r = records.get(e) if isinstance(records, dict) else records[e]
        arr[e] = None if r is None else r.ctypes.data
    return arr


def layer(bank, hidden, inter, n_experts, top_k, records, x, ids, weights, shared=None, limit=10.0,
          chain_rounding=False, shared_bf16_add=False, want_ro=False):
    """f64 layer oracle.  records: dict/list expert -> uint8 record (reference layout); x: f32 holding bf16 values."""
    cfg = LayerCfg(bank, hidden, inter, n_experts, top_k, limit, int(chain_rounding), int(shared_bf16_add))
    x = np.ascontiguousarray(x, np.float32)
    T = x.shape[0]
    ids = np.ascontiguousarray(ids, np.int32)
    weights = np.ascontiguousarray(weights, np.float32)
    y = np.empty((T, hidden), np.float64)
    ro = np.empty((T, top_k, hidden), np.float64) if want_ro else None
    recs = _records_array(records, n_experts)
    sh = [None, None, None] if shared is None else [np.ascontiguousarray(s, np.uint16) for s in shared]
    rc = lib().orc_layer(C.byref(cfg), recs, _p(x), T, _p(ids), _p(weights), _p(sh[0]), _p(sh[1]), _p(sh[2]), _p(y),
                         _p(ro))
    assert rc == 0, rc
    return (y, ro) if want_ro else y


def layer_fast(hidden, inter, n_experts, top_k, records, x, ids, weights, shared=None, limit=10.0, threads=0):
    cfg = LayerCfg(BANK_EXL3, hidden, inter, n_experts, top_k, limit, 0, 0)
    x = np.ascontiguousarray(x, np.float32)
    T = x.shape[0]
    ids = np.ascontiguousarray(ids, np.int32)
    weights = np.ascontiguousarray(weights, np.float32)
    y = np.empty((T, hidden), np.float32)
    recs = _records_array(records, n_experts)
    sh = [None, None, None] if shared is None else [np.ascontiguousarray(s, np.uint16) for s in shared]
    rc = lib().orc_layer_fast(C.byref(cfg), recs, _p(x), T, _p(ids), _p(weights), _p(sh[0]), _p(sh[1]), _p(sh[2]),
                              _p(y), threads)
    assert rc == 0, rc
    return y


def max_threads():
    return int(lib().orc_max_threads())


def f32_to_bf16_bits(a):
    a = np.ascontiguousarray(a, np.float32)
    b = a.view(np.uint32)
    r = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)
