"""Host-side Python view of libmlxs_moe.so (ctypes over the C ABI in include/mlxs_moe.h).

The product is the shared library; this module only mirrors the reference's seam names so the parity tests and the
benchmark read like the reference's own callers:
  MoE.route    = Gate.__call__'s tail            (src/arch/deepseek_v41/graph.zig:2041-2051)
  MoE.routed   = Hook.routed                     (src/arch/deepseek_v41/experts.zig:1214-1223)
  MoE.experts  = Source.forward / forwardShared  (src/arch/glm5_next/experts.zig:566-595, 639-653)
  MoE.forward  = Tr.moe from the logits on       (src/arch/deepseek_v41/graph.zig:2196-2240)
Pointers are plain integers (device or host addresses); nothing here touches torch.  There is no CPU fallback: if
the library is missing or the machine has no CUDA device the calls raise.
"""
import ctypes as C
from pathlib import Path  # noqa: E402

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libmlxs_moe.so"
ABI = 2026112602

BANK_EXL3_K3_MUL1, BANK_MXFP4, BANK_NVFP4, BANK_EXL3_K2_MUL1 = 0, 1, 2, 3
SCORE_SQRTSOFTPLUS, SCORE_SIGMOID, SCORE_SOFTMAX = 0, 1, 2
ACT_SWIGLU, ACT_SWIGLU_CLAMPED = 0, 1
COMBINE_F32, COMBINE_CHAIN = 0, 1
# return codes (include/mlxs_moe.h)
(E_ARG, E_CONFIG, E_CUDA, E_BANK, E_NOT_LOADED, E_TOO_MANY_TOKENS, E_DEVICE_STATUS, E_MANIFEST, E_EP) = range(-1, -10, -1)

EXPORTS = [
    "mlxs_moe_abi", "mlxs_moe_last_error", "mlxs_moe_create", "mlxs_moe_destroy", "mlxs_moe_record_bytes",
    "mlxs_moe_load_expert", "mlxs_moe_load_bank", "mlxs_moe_bank_peek", "mlxs_moe_bank_peek_text", "mlxs_moe_set_router_bias", "mlxs_moe_set_shared", "mlxs_moe_route",
    "mlxs_moe_routed", "mlxs_moe_experts", "mlxs_moe_forward", "mlxs_moe_forward_host", "mlxs_moe_exl3_gemv",
    "mlxs_moe_exl3_gemv_noalloc",
    "mlxs_moe_stats_get", "mlxs_moe_profile_enable", "mlxs_moe_profile_read", "mlxs_moe_ep_unique_id", "mlxs_moe_ep_init", "mlxs_moe_ep_plan",
    "mlxs_moe_set_placement", "mlxs_moe_set_router_weight", "mlxs_moe_logits", "mlxs_moe_forward_x",
    "mlxs_moe_set_layer_bits", "mlxs_moe_layer_record_bytes", "mlxs_moe_bank_layer_bits_text",
    "mlxs_moe_ep_window_bytes", "mlxs_moe_ep_overloaded_rank",
    "mlxs_moe_status_clear", "mlxs_moe_sort_rows", "mlxs_moe_debug_wait", "mlxs_moe_exl3_decode_rate", "mlxs_moe_fp4_native_probe", "mlxs_moe_mma_rate",
    "mlxs_moe_bank_verify", "mlxs_moe_usage_enable", "mlxs_moe_usage_add", "mlxs_moe_usage_read", "mlxs_moe_usage_reset", "mlxs_moe_plan_placement",
]


class Config(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("hidden", C.c_uint32), ("inter", C.c_uint32), ("n_experts", C.c_uint32),
                ("top_k", C.c_uint32), ("n_layers", C.c_uint32), ("bank_kind", C.c_uint32), ("act", C.c_uint32),
                ("act_limit", C.c_float), ("scoring", C.c_uint32), ("norm_topk", C.c_uint32),
                ("routed_scale", C.c_float), ("shared_expert", C.c_uint32), ("combine", C.c_uint32),
                ("max_tokens", C.c_uint32), ("device", C.c_int32), ("ep_world", C.c_uint32), ("ep_rank", C.c_uint32)]


class Stats(C.Structure):
    _fields_ = [("route_calls", C.c_uint64), ("expert_calls", C.c_uint64), ("tokens", C.c_uint64),
                ("assignments", C.c_uint64), ("distinct_experts_last", C.c_uint64), ("weight_bytes_last", C.c_uint64),
                ("a2a_bytes_sent", C.c_uint64), ("a2a_bytes_recv", C.c_uint64), ("resident_bytes", C.c_uint64),
                ("device_status", C.c_uint32), ("ep_transport", C.c_uint32)]


STAGES = ["router", "dispatch", "prep", "gate_up", "down", "shared", "combine", "exchange", "tensor_lane"]


class Profile(C.Structure):
    _fields_ = [("ms", C.c_double * len(STAGES)), ("launches", C.c_uint64 * len(STAGES))]


class BankInfo(C.Structure):
    _fields_ = [("bank_kind", C.c_uint32), ("has_sha256", C.c_uint32), ("hidden", C.c_uint64), ("inter", C.c_uint64),
                ("n_experts", C.c_uint64), ("n_layers", C.c_uint64), ("first_layer", C.c_uint64),
                ("logical_bytes", C.c_uint64), ("record_stride", C.c_uint64), ("data_bytes", C.c_uint64),
                ("data_file", C.c_char * 64), ("bits_min", C.c_uint32), ("bits_max", C.c_uint32)]


class Fp4NativeResult(C.Structure):
    _fields_ = [("rel_l2_hi_lo", C.c_double), ("rel_l2_hi_only", C.c_double), ("tflops_f16", C.c_double),
                ("tflops_mxf8f6f4", C.c_double), ("tflops_hi_lo_effective", C.c_double)]


class MlxsError(RuntimeError):
    def __init__(self, rc, msg):
        super().__init__(f"mlxs_moe rc={rc}: {msg}")
        self.rc = rc
        self.msg = msg


_lib = None


def lib():
    """The loaded library.  Raises if it has not been built (python mlx-stream_b200/build.py)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(f"{LIB_PATH} is missing: run `python mlx-stream_b200/build.py` (needs nvcc)")
        L = C.CDLL(str(LIB_PATH))
        L.mlxs_moe_abi.restype = C.c_int32
        L.mlxs_moe_last_error.restype = C.c_char_p
        L.mlxs_moe_create.argtypes = [C.POINTER(Config), C.POINTER(C.c_void_p)]
        L.mlxs_moe_destroy.argtypes = [C.c_void_p]
        L.mlxs_moe_destroy.restype = None
        L.mlxs_moe_record_bytes.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        L.mlxs_moe_load_expert.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64, C.c_int]
        L.mlxs_moe_set_layer_bits.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32]
        L.mlxs_moe_usage_enable.argtypes = [C.c_void_p, C.c_int]
        L.mlxs_moe_usage_add.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p]
        L.mlxs_moe_usage_read.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(C.c_uint64), C.c_int]
        L.mlxs_moe_usage_reset.argtypes = [C.c_void_p]
        L.mlxs_moe_plan_placement.argtypes = [C.POINTER(C.c_uint64), C.c_uint32, C.c_uint32, C.POINTER(C.c_uint16)]
        L.mlxs_moe_layer_record_bytes.argtypes = [C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        L.mlxs_moe_bank_layer_bits_text.argtypes = [C.c_char_p, C.POINTER(C.c_uint32), C.c_uint32, C.POINTER(C.c_uint32)]
        L.mlxs_moe_load_bank.argtypes = [C.c_void_p, C.c_char_p]
        L.mlxs_moe_bank_peek.argtypes = [C.c_char_p, C.POINTER(BankInfo)]
        L.mlxs_moe_bank_peek_text.argtypes = [C.c_char_p, C.POINTER(BankInfo)]
        L.mlxs_moe_bank_verify.argtypes = [C.c_char_p, C.POINTER(BankInfo), C.c_int]
        L.mlxs_moe_set_router_bias.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p]
        L.mlxs_moe_set_shared.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.mlxs_moe_route.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
        L.mlxs_moe_routed.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.mlxs_moe_experts.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32,
                                       C.c_void_p, C.c_void_p]
        L.mlxs_moe_forward.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.mlxs_moe_forward_host.argtypes = L.mlxs_moe_forward.argtypes
        L.mlxs_moe_exl3_gemv.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32,
                                         C.c_void_p, C.c_void_p]
        L.mlxs_moe_exl3_gemv_noalloc.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p,
                                                 C.c_void_p]
        L.mlxs_moe_stats_get.argtypes = [C.c_void_p, C.POINTER(Stats)]
        L.mlxs_moe_profile_enable.argtypes = [C.c_void_p, C.c_int]
        L.mlxs_moe_profile_read.argtypes = [C.c_void_p, C.POINTER(Profile)]
        L.mlxs_moe_ep_unique_id.argtypes = [C.c_void_p]
        L.mlxs_moe_ep_init.argtypes = [C.c_void_p, C.c_void_p]
        L.mlxs_moe_ep_plan.argtypes = [C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p]
        L.mlxs_moe_set_placement.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p]
        L.mlxs_moe_set_router_weight.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_int]
        L.mlxs_moe_logits.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.mlxs_moe_forward_x.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.mlxs_moe_fp4_native_probe.argtypes = [C.c_int32, C.c_uint32, C.POINTER(Fp4NativeResult)]
        L.mlxs_moe_mma_rate.argtypes = [C.c_int32, C.c_uint32, C.c_int, C.c_uint32, C.POINTER(C.c_double)]
        L.mlxs_moe_exl3_decode_rate.argtypes = [C.c_int32, C.c_uint32, C.c_int, C.c_uint32, C.POINTER(C.c_double)]
        L.mlxs_moe_ep_window_bytes.restype = C.c_uint64
        L.mlxs_moe_ep_window_bytes.argtypes = [C.c_uint32] * 5
        L.mlxs_moe_ep_overloaded_rank.restype = C.c_int32
        L.mlxs_moe_ep_overloaded_rank.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64]
        L.mlxs_moe_status_clear.argtypes = [C.c_void_p]
        L.mlxs_moe_sort_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]
        L.mlxs_moe_debug_wait.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32]
        if L.mlxs_moe_abi() != ABI:
            raise RuntimeError(f"libmlxs_moe.so ABI {L.mlxs_moe_abi()} != binding ABI {ABI}")
        _lib = L
    return _lib


def last_error():
    return lib().mlxs_moe_last_error().decode()


def _check(rc):
    if rc != 0:
        raise MlxsError(rc, last_error())


def make_config(hidden, inter, n_experts, top_k, n_layers=1, bank_kind=BANK_EXL3_K3_MUL1, act=ACT_SWIGLU_CLAMPED,
                act_limit=10.0, scoring=SCORE_SQRTSOFTPLUS, norm_topk=True, routed_scale=1.0, shared_expert=False,
                combine=COMBINE_F32, max_tokens=64, device=0, ep_world=1, ep_rank=0):
    return Config(C.sizeof(Config), hidden, inter, n_experts, top_k, n_layers, bank_kind, act, act_limit, scoring,
                  int(norm_topk), routed_scale, int(shared_expert), combine, max_tokens, device, ep_world, ep_rank)


def bank_peek(directory=None, text=None):
    """Parses and checks a bank manifest (the directory's, or a manifest text) without a device."""
    info = BankInfo()
    if text is not None:
        _check(lib().mlxs_moe_bank_peek_text(text.encode() if isinstance(text, str) else text, C.byref(info)))
    else:
        _check(lib().mlxs_moe_bank_peek(str(directory).encode(), C.byref(info)))
    return info


def bank_verify(directory, verify_sha256=True):
    """Opens a bank as the load does, without a device: manifests (EXL3: v2 and the v1 runtime manifest), sidecar,
    and on request every record's digests."""
    info = BankInfo()
    _check(lib().mlxs_moe_bank_verify(str(directory).encode(), C.byref(info), int(verify_sha256)))
    return info


def plan_placement(counts, world):
    """Route counts per expert -> the rank of every expert (most used first, dealt to the ranks in snake order)."""
    n = len(counts)
    cin = (C.c_uint64 * n)(*[int(c) for c in counts])
    out = (C.c_uint16 * n)()
    _check(lib().mlxs_moe_plan_placement(cin, n, world, out))
    return list(out)


def bank_layer_bits(text):
    """K of every layer of an EXL3 manifest text."""
    raw = text.encode() if isinstance(text, str) else text
    n = C.c_uint32()
    _check(lib().mlxs_moe_bank_layer_bits_text(raw, None, 0, C.byref(n)))
    out = (C.c_uint32 * n.value)()
    _check(lib().mlxs_moe_bank_layer_bits_text(raw, out, n.value, C.byref(n)))
    return list(out)


def exl3_decode_rate(device=0, bits=3, with_mma=True, tiles_per_warp=1 << 16):
    """Tiles per second of the EXL3 in-register decode alone (operands from registers): the decode's own ceiling."""
    out = C.c_double()
    _check(lib().mlxs_moe_exl3_decode_rate(device, bits, int(with_mma), tiles_per_warp, C.byref(out)))
    return out.value


def mma_rate(device=0, n=256, a_from_tmem=False, mmas=20000):
    """Nanoseconds per tcgen05.mma (M 128 x n x K 16, bf16) issued back to back on every SM."""
    out = C.c_double()
    _check(lib().mlxs_moe_mma_rate(device, n, int(a_from_tmem), mmas, C.byref(out)))
    return out.value


def fp4_native_probe(device=0, rate_mmas=20000):
    """The native block-scaled FP4 MMA measured: numerics of the e2m1 x (e4m3 hi + lo) product and the issue rates."""
    out = Fp4NativeResult()
    _check(lib().mlxs_moe_fp4_native_probe(device, rate_mmas, C.byref(out)))
    return {k: getattr(out, k) for k, _ in Fp4NativeResult._fields_}


def exl3_gemv_noalloc(code, in_dim, out_dim, xh, rows, z, stream=None):
    """z = xh . W_hat of one code plane with no handle and no allocation (fixed scratch inside the library)."""
    _check(lib().mlxs_moe_exl3_gemv_noalloc(code, in_dim, out_dim, xh, rows, z, stream))


class MoE:
    """One handle = one rank's routed-MoE layers (weights resident in HBM)."""

    def __init__(self, cfg: Config):
        self.cfg = cfg
        self._h = C.c_void_p()
        _check(lib().mlxs_moe_create(C.byref(cfg), C.byref(self._h)))

    def close(self):
        if self._h:
            lib().mlxs_moe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def record_bytes(self):
        a, b = C.c_uint64(), C.c_uint64()
        _check(lib().mlxs_moe_record_bytes(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def usage_enable(self, on=True):
        """While on, every route / forward call adds its ids to the layer's device-side route counts."""
        _check(lib().mlxs_moe_usage_enable(self._h, int(on)))

    def usage_add(self, layer, ids_ptr, n_ids, stream=None):
        _check(lib().mlxs_moe_usage_add(self._h, layer, ids_ptr, n_ids, stream))

    def usage_read(self, layer, all_ranks=False):
        out = (C.c_uint64 * self.cfg.n_experts)()
        _check(lib().mlxs_moe_usage_read(self._h, layer, out, int(all_ranks)))
        return list(out)

    def usage_reset(self):
        _check(lib().mlxs_moe_usage_reset(self._h))

    def set_layer_bits(self, layer, bits):
        """EXL3 banks of mixed width: this layer's bits per weight (2 or 3), before its experts are loaded."""
        _check(lib().mlxs_moe_set_layer_bits(self._h, layer, bits))

    def layer_record_bytes(self, layer):
        k, a, b = C.c_uint32(), C.c_uint64(), C.c_uint64()
        _check(lib().mlxs_moe_layer_record_bytes(self._h, layer, C.byref(k), C.byref(a), C.byref(b)))
        return k.value, a.value, b.value

    def load_expert(self, layer, expert, record_ptr, nbytes, on_device=False):
        _check(lib().mlxs_moe_load_expert(self._h, layer, expert, record_ptr, nbytes, int(on_device)))

    def load_bank(self, directory):
        _check(lib().mlxs_moe_load_bank(self._h, str(directory).encode()))

    def set_placement(self, layer, rank_of_expert_u16_ptr):
        _check(lib().mlxs_moe_set_placement(self._h, layer, rank_of_expert_u16_ptr))

    def set_router_weight(self, layer, w_ptr, on_device=False):
        _check(lib().mlxs_moe_set_router_weight(self._h, layer, w_ptr, int(on_device)))

    def logits(self, layer, x, T, out, stream=None):
        _check(lib().mlxs_moe_logits(self._h, layer, x, T, out, stream))

    def forward_x(self, layer, x, T, y, stream=None):
        _check(lib().mlxs_moe_forward_x(self._h, layer, x, T, y, stream))

    def set_router_bias(self, layer, bias_host_ptr):
        _check(lib().mlxs_moe_set_router_bias(self._h, layer, bias_host_ptr))

    def set_shared(self, layer, w1, w3, w2, on_device=False):
        _check(lib().mlxs_moe_set_shared(self._h, layer, w1, w3, w2, int(on_device)))

    def route(self, layer, logits, T, ids, weights, stream=None):
        _check(lib().mlxs_moe_route(self._h, layer, logits, T, ids, weights, stream))

    def routed(self, layer, x, ids, T, out, stream=None):
        _check(lib().mlxs_moe_routed(self._h, layer, x, ids, T, out, stream))

    def experts(self, layer, x, ids, weights, T, y, stream=None):
        _check(lib().mlxs_moe_experts(self._h, layer, x, ids, weights, T, y, stream))

    def forward(self, layer, x, logits, T, y, stream=None):
        _check(lib().mlxs_moe_forward(self._h, layer, x, logits, T, y, stream))

    def forward_host(self, layer, x_host, logits_host, T, y_host, stream=None):
        _check(lib().mlxs_moe_forward_host(self._h, layer, x_host, logits_host, T, y_host, stream))

    def exl3_gemv(self, layer, expert, proj, xh, rows, z, stream=None):
        _check(lib().mlxs_moe_exl3_gemv(self._h, layer, expert, proj, xh, rows, z, stream))

    def status_clear(self):
        """Acknowledges a recorded device error: the sticky status word is cleared."""
        _check(lib().mlxs_moe_status_clear(self._h))

    def sort_rows(self, slot, n, n_slots, order, offsets, stream=None):
        """The dispatch permutation alone: slot ids -> order (sorted position -> row) and per-slot offsets."""
        _check(lib().mlxs_moe_sort_rows(self._h, slot, n, n_slots, order, offsets, stream))

    def debug_wait(self, poll_limit=0, withhold_stage=0):
        """Self-test hook of the bounded waits: a short poll limit and one withheld ring stage."""
        _check(lib().mlxs_moe_debug_wait(self._h, poll_limit, withhold_stage))

    def profile_enable(self, on=True):
        _check(lib().mlxs_moe_profile_enable(self._h, int(on)))

    def profile_read(self):
        p = Profile()
        _check(lib().mlxs_moe_profile_read(self._h, C.byref(p)))
        return {STAGES[i]: (p.ms[i], p.launches[i]) for i in range(len(STAGES))}

    def stats(self):
        s = Stats()
        _check(lib().mlxs_moe_stats_get(self._h, C.byref(s)))
        return s
