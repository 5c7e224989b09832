//! extern-fn view of include/mlxs_moe.h for the Zig host (source only: this image has no Zig compiler; the C header
//! is the compiled, tested statement of the same ABI).  One declaration per C entry point, same order.
const std = @import("std");

pub const abi_expected: i32 = 2026112602;

pub const Moe = opaque {};

pub const BankKind = enum(u32) { exl3_k3_mul1 = 0, mxfp4 = 1, nvfp4 = 2, exl3_k2_mul1 = 3 };
pub const Scoring = enum(u32) { sqrtsoftplus = 0, sigmoid = 1, softmax = 2 };
pub const Act = enum(u32) { swiglu = 0, swiglu_clamped = 1 };
pub const Combine = enum(u32) { f32 = 0, chain = 1 };

pub const Config = extern struct {
    struct_size: u32 = @sizeOf(Config),
    hidden: u32,
    inter: u32,
    n_experts: u32,
    top_k: u32,
    n_layers: u32,
    bank_kind: u32,
    act: u32,
    act_limit: f32,
    scoring: u32,
    norm_topk: u32,
    routed_scale: f32,
    shared_expert: u32,
    combine: u32,
    max_tokens: u32,
    device: i32,
    ep_world: u32 = 1,
    ep_rank: u32 = 0,
};

pub const Stats = extern struct {
    route_calls: u64,
    expert_calls: u64,
    tokens: u64,
    assignments: u64,
    distinct_experts_last: u64,
    weight_bytes_last: u64,
    a2a_bytes_sent: u64,
    a2a_bytes_recv: u64,
    resident_bytes: u64,
    device_status: u32,
    ep_transport: u32,
};

pub extern fn mlxs_moe_abi() i32;
pub extern fn mlxs_moe_last_error() [*:0]const u8;
pub extern fn mlxs_moe_create(cfg: *const Config, out: **Moe) c_int;
pub extern fn mlxs_moe_destroy(h: ?*Moe) void;
pub extern fn mlxs_moe_record_bytes(h: *const Moe, logical: ?*u64, stride: ?*u64) c_int;
pub extern fn mlxs_moe_set_layer_bits(h: *Moe, layer: u32, bits: u32) c_int;
pub extern fn mlxs_moe_layer_record_bytes(h: *const Moe, layer: u32, bits: ?*u32, logical: ?*u64, stride: ?*u64) c_int;
pub extern fn mlxs_moe_load_expert(h: *Moe, layer: u32, expert: u32, record: *const anyopaque, nbytes: u64, on_device: c_int) c_int;
pub extern fn mlxs_moe_load_bank(h: *Moe, dir: [*:0]const u8) c_int;
pub const BankInfo = extern struct {
    bank_kind: u32,
    has_sha256: u32,
    hidden: u64,
    inter: u64,
    n_experts: u64,
    n_layers: u64,
    first_layer: u64,
    logical_bytes: u64,
    record_stride: u64,
    data_bytes: u64,
    data_file: [64]u8,
    bits_min: u32,
    bits_max: u32,
};
pub extern fn mlxs_moe_bank_peek(dir: [*:0]const u8, out: *BankInfo) c_int;
pub extern fn mlxs_moe_bank_peek_text(manifest_json: [*:0]const u8, out: *BankInfo) c_int;
pub extern fn mlxs_moe_bank_verify(dir: [*:0]const u8, out: ?*BankInfo, verify_sha256: c_int) c_int;
pub extern fn mlxs_moe_bank_layer_bits_text(manifest_json: [*:0]const u8, bits_out: ?[*]u32, cap: u32, n_layers_out: *u32) c_int;
pub extern fn mlxs_moe_set_router_bias(h: *Moe, layer: u32, bias_host: ?[*]const f32) c_int;
pub extern fn mlxs_moe_set_router_weight(h: *Moe, layer: u32, w_gate_bf16: *const anyopaque, on_device: c_int) c_int;
pub extern fn mlxs_moe_logits(h: *Moe, layer: u32, x_dev: *const anyopaque, t: u32, logits_dev: [*]f32, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_forward_x(h: *Moe, layer: u32, x_dev: *const anyopaque, t: u32, y_dev: *anyopaque, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_set_shared(h: *Moe, layer: u32, w1: *const anyopaque, w3: *const anyopaque, w2: *const anyopaque, on_device: c_int) c_int;
pub extern fn mlxs_moe_route(h: *Moe, layer: u32, logits_dev: *const anyopaque, t: u32, ids_dev: *anyopaque, weights_dev: *anyopaque, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_routed(h: *Moe, layer: u32, x_dev: *const anyopaque, ids_dev: *const anyopaque, t: u32, out_dev: *anyopaque, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_experts(h: *Moe, layer: u32, x_dev: *const anyopaque, ids_dev: *const anyopaque, weights_dev: *const anyopaque, t: u32, y_dev: *anyopaque, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_forward(h: *Moe, layer: u32, x_dev: *const anyopaque, logits_dev: *const anyopaque, t: u32, y_dev: *anyopaque, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_forward_host(h: *Moe, layer: u32, x_host: *const anyopaque, logits_host: [*]const f32, t: u32, y_host: *anyopaque, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_exl3_gemv(h: *Moe, layer: u32, expert: u32, proj: u32, xh_dev: *const anyopaque, rows: u32, z_dev: *anyopaque, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_exl3_gemv_noalloc(code_dev: *const anyopaque, in_dim: u32, out_dim: u32, xh_dev: *const anyopaque, rows: u32, z_dev: *anyopaque, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_stats_get(h: *Moe, out: *Stats) c_int;
/// bytes of the per-rank window of the peer-store transport
pub extern fn mlxs_moe_ep_window_bytes(world: u32, max_tokens: u32, top_k: u32, n_experts: u32, hidden: u32) u64;
/// all-ranks capacity check of the NCCL transport (pure): lowest overloaded rank or -1
pub extern fn mlxs_moe_ep_overloaded_rank(counts: [*]const i32, world: u32, stride: u32, rows_cap: u64) i32;
/// acknowledges a recorded device error (the status word is sticky)
pub extern fn mlxs_moe_status_clear(h: *Moe) c_int;
/// the dispatch permutation alone (src/sdk_ext/quant.zig:269-301): slot ids -> order, offsets
pub extern fn mlxs_moe_sort_rows(h: *Moe, slot_dev: ?*const i32, n: u32, n_slots: u32, order_dev: ?*u32, offsets_dev: *u32, stream: ?*anyopaque) c_int;
/// measured ceiling of the in-register EXL3 decode (tiles per second, operands from registers)
pub extern fn mlxs_moe_exl3_decode_rate(device: i32, bits: u32, with_mma: c_int, tiles_per_warp: u32, tiles_per_s: *f64) c_int;
pub const Fp4NativeResult = extern struct { rel_l2_hi_lo: f64, rel_l2_hi_only: f64, tflops_f16: f64, tflops_mxf8f6f4: f64, tflops_hi_lo_effective: f64 };
/// the native block-scaled FP4 MMA measured (numerics of the hi / lo split, issue rates)
pub extern fn mlxs_moe_fp4_native_probe(device: i32, rate_mmas: u32, out: *Fp4NativeResult) c_int;
/// nanoseconds per tcgen05.mma (M 128 x n x K 16) issued back to back on every SM, A in shared or tensor memory
pub extern fn mlxs_moe_mma_rate(device: i32, n: u32, a_from_tmem: c_int, mmas: u32, ns_per_mma: *f64) c_int;
/// self-test hook of the bounded waits
pub extern fn mlxs_moe_debug_wait(h: *Moe, poll_limit: u32, withhold_stage: u32) c_int;

/// stage order of the profile arrays (include/mlxs_moe.h MLXS_STAGE_*)
pub const Stage = enum(u32) { router, dispatch, prep, gate_up, down, shared, combine, exchange, tensor_lane };
pub const stage_count = 9;
pub const Profile = extern struct { ms: [stage_count]f64, launches: [stage_count]u64 };
pub extern fn mlxs_moe_profile_enable(h: *Moe, on: c_int) c_int;
pub extern fn mlxs_moe_profile_read(h: *Moe, out: *Profile) c_int;

// expert parallel: one process per GPU, rank 0 makes the id, the host hands it to every rank
pub extern fn mlxs_moe_ep_unique_id(id128_out: *[128]u8) c_int;
pub extern fn mlxs_moe_ep_init(h: *Moe, id128: *const [128]u8) c_int;
pub extern fn mlxs_moe_ep_plan(ids: [*]const i32, n: u64, n_experts: u32, world: u32, send_counts: [*]u64) c_int;
pub extern fn mlxs_moe_usage_enable(h: *Moe, on: c_int) c_int;
pub extern fn mlxs_moe_usage_add(h: *Moe, layer: u32, ids_dev: *const anyopaque, n_ids: u64, stream: ?*anyopaque) c_int;
pub extern fn mlxs_moe_usage_read(h: *Moe, layer: u32, counts_host: [*]u64, all_ranks: c_int) c_int;
pub extern fn mlxs_moe_usage_reset(h: *Moe) c_int;
pub extern fn mlxs_moe_plan_placement(counts: [*]const u64, n_experts: u32, world: u32, rank_of_expert: [*]u16) c_int;
pub extern fn mlxs_moe_set_placement(h: *Moe, layer: u32, rank_of_expert: [*]const u16) c_int;

pub const Error = error{ Arg, Config, Cuda, Bank, NotLoaded, TooManyTokens, DeviceStatus, Manifest, Ep };

/// rc -> Zig error, the message left at mlxs_moe_last_error() (the reference's Diag carries the same kind of text,
/// sdk/peek.zig:15-27).
pub fn check(rc: c_int) Error!void {
    return switch (rc) {
        0 => {},
        -1 => error.Arg,
        -2 => error.Config,
        -3 => error.Cuda,
        -4 => error.Bank,
        -5 => error.NotLoaded,
        -6 => error.TooManyTokens,
        -7 => error.DeviceStatus,
        -8 => error.Manifest,
        else => error.Ep,
    };
}

/// Refuse a library built against another ABI, as the reference does for its read pool
/// (src/sdk_ext/expert/io.zig:62-69).
pub fn negotiate() Error!void {
    if (mlxs_moe_abi() != abi_expected) return error.Config;
}
