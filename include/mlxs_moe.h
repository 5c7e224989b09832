/*
 * mlxs_moe.h: C ABI of the B200 routed-MoE layer (router -> dispatch -> grouped expert gate/up/down with in-register
 * weight decode -> SwiGLU -> weighted combine), the drop-in for mlx-stream's routed-expert hot path.
 *
 * Conventions follow the reference's own native boundary (csrc/q3_lookahead4.h:44-98, csrc/mlx_alloc_shim.h:14-17,
 * src/sdk_ext/expert/io.zig:62-69): every call returns an int (0 = ok, negative = a named refusal), the message of
 * the last refusal on the calling thread is at mlxs_moe_last_error(), the caller compares mlxs_moe_abi() with the
 * value it was built against and refuses a mismatch, buffers are caller-owned, there are no callbacks.
 * One caller thread per handle (the reference's single inference thread, sdk/arch.zig:100-105).  All device work is
 * queued on the stream the caller passes (a cudaStream_t as void*, NULL = the default stream).
 * Pointers named *_dev are device pointers on the handle's device; *_host are host pointers.
 * There is no CPU fallback: without a CUDA device every compute entry refuses with MLXS_E_CUDA.
 */
#ifndef MLXS_MOE_H
#define MLXS_MOE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define MLXS_MOE_ABI 2026112602

/* refusals (the names mirror the reference's refusal sets: src/sdk_ext/quant.zig:94-111, src/expert/bank.zig:79-101) */
enum {
    MLXS_OK = 0,
    MLXS_E_ARG = -1,          /* null / out-of-range argument */
    MLXS_E_CONFIG = -2,       /* a config field is not implemented (named in the message) */
    MLXS_E_CUDA = -3,         /* a CUDA runtime call failed (message carries the CUDA error) */
    MLXS_E_BANK = -4,         /* record bytes / geometry do not match the bank kind */
    MLXS_E_NOT_LOADED = -5,   /* a routed expert (or the shared expert / router bias) was never loaded */
    MLXS_E_TOO_MANY_TOKENS = -6,
    MLXS_E_DEVICE_STATUS = -7, /* a kernel recorded an error word (bad id, bounded wait ran out) */
    MLXS_E_MANIFEST = -8,     /* manifest field mismatch (named) */
    MLXS_E_EP = -9            /* expert-parallel exchange not initialised / failed */
};

/* bank kinds: the record layouts are the reference's own.
 *  EXL3_K3_MUL1: nine segments gate/up/down x {code I16 [in/16,out/16,48], rout F16 [out], rin F16 [in]}
 *                (src/expert/bank.zig:116-141)
 *  MXFP4:        six parts gate/up/down x {weight U32 [out,in/8], scales U8 E8M0 [out,in/32]}
 *                (src/arch/mimo_v2/bank.zig:13-27, 341-345)
 *  NVFP4:        nine parts gate/up/down x {weight U32 [out,in/8], scales U8 E4M3 [out,in/16], global F32}
 *                (src/arch/glm5_next/bank.zig:5-13)
 *  EXL3_K2_MUL1: the EXL3 record at 2 bits per weight, code I16 [in/16,out/16,32] (the reference's K = 2 layers,
 *                src/exl3/kernels.zig:163-177; a model that mixes K = 2 and K = 3 layers uses one handle per width) */
enum { MLXS_BANK_EXL3_K3_MUL1 = 0, MLXS_BANK_MXFP4 = 1, MLXS_BANK_NVFP4 = 2, MLXS_BANK_EXL3_K2_MUL1 = 3 };
/* router scoring: sqrt(softplus) = DeepSeek-V4.1 (src/arch/deepseek_v41/graph.zig:2032-2051), sigmoid = MiMo / GLM
 * (src/arch/mimo_v2/kernels/mimo_glue_top8.metal, src/arch/glm5_next/kernels/glm5n_glue_top8.metal); softmax has no
 * counterpart in the reference (every arch refuses it) and is provided for the MiMo-shaped benchmark config. */
enum { MLXS_SCORE_SQRTSOFTPLUS = 0, MLXS_SCORE_SIGMOID = 1, MLXS_SCORE_SOFTMAX = 2 };
/* activation between gate/up and down (src/sdk_ext/quant.zig:54-61) */
enum { MLXS_ACT_SWIGLU = 0, MLXS_ACT_SWIGLU_CLAMPED = 1 };
/* combine arithmetic:
 *  F32:   sum_k f32(row_k) w_k + shared in f32, one rounding to bf16 (src/arch/deepseek_v41/graph.zig:2182-2184)
 *  CHAIN: rows stored bf16, each product rounded, folded k = 0..top_k-1, bf16 once, then a bf16 add of the shared row
 *         (src/arch/mimo_v2/kernels/mimo_moe_combine.metal, src/arch/glm5_next/kernels/glm5n_moe_combine.metal) */
enum { MLXS_COMBINE_F32 = 0, MLXS_COMBINE_CHAIN = 1 };

typedef struct mlxs_moe mlxs_moe; /* opaque */

typedef struct {
    uint32_t struct_size; /* sizeof(mlxs_moe_config): the version gate of the struct */
    uint32_t hidden, inter, n_experts, top_k, n_layers;
    uint32_t bank_kind;
    uint32_t act;
    float act_limit; /* for MLXS_ACT_SWIGLU_CLAMPED */
    uint32_t scoring;
    uint32_t norm_topk;   /* weights / (sum + 1e-20) */
    float routed_scale;   /* x routed_scaling_factor */
    uint32_t shared_expert; /* 1: a bf16 dense shared expert is added (src/arch/deepseek_v41/graph.zig:2162-2172) */
    uint32_t combine;
    uint32_t max_tokens; /* largest T of one call (the reference's call bound is 16,384 rows: README.md:181-195) */
    int32_t device;      /* CUDA ordinal */
    uint32_t ep_world, ep_rank; /* expert parallel: this rank owns experts [rank E/world, (rank+1) E/world) */
} mlxs_moe_config;

typedef struct {
    uint64_t route_calls, expert_calls, tokens, assignments;
    uint64_t distinct_experts_last; /* distinct routed experts of the last call on this rank */
    uint64_t weight_bytes_last;     /* algorithmic weight bytes of the last call: distinct x bytes per expert */
    uint64_t a2a_bytes_sent, a2a_bytes_recv;
    uint64_t resident_bytes;        /* HBM held by the handle */
    uint32_t device_status;         /* sticky error word written by kernels (0 = none) */
    uint32_t ep_transport;          /* expert parallel: 0 none, 1 NCCL send/recv, 2 stores into the peers' windows */
} mlxs_moe_stats;

/* version gate and error text (csrc/q3_lookahead4.h:91, csrc/mlx_alloc_shim.h:14-17) */
int32_t mlxs_moe_abi(void);
const char *mlxs_moe_last_error(void);

/* Module.init's quant accept: every field checked once, refusals by name (src/exl3/quant.zig:202-212,
 * src/sdk_ext/quant.zig:94-111).  Allocates the resident bank and the workspaces for max_tokens. */
int mlxs_moe_create(const mlxs_moe_config *cfg, mlxs_moe **out);
void mlxs_moe_destroy(mlxs_moe *h);

/* the bank kind's record size at the handle's dims (src/expert/bank.zig:116-141): logical bytes and the 4096-padded
 * stride records have in an experts.bin */
int mlxs_moe_record_bytes(const mlxs_moe *h, uint64_t *logical_bytes, uint64_t *record_stride);

/* An EXL3 bank may mix layer widths (the reference's 2.9 bpw DeepSeek bank keeps layers 18-22 at K = 2 inside a K = 3
 * bank, src/exl3/quant.zig:39-41, 73; src/expert/bank.zig:288-298): the handle's bank kind names the default width,
 * this call gives one layer its own (bits = 2 or 3) before any of its experts is loaded and re-sizes the layer's HBM
 * arrays.  mlxs_moe_load_bank applies the manifest's per-layer K by itself. */
int mlxs_moe_set_layer_bits(mlxs_moe *h, uint32_t layer, uint32_t bits);
/* one layer's width and record size (equal to mlxs_moe_record_bytes unless the layer's width was changed) */
int mlxs_moe_layer_record_bytes(const mlxs_moe *h, uint32_t layer, uint32_t *bits, uint64_t *logical_bytes,
                                uint64_t *record_stride);

/* Replaces the expert source's fill of a slot row (src/sdk_ext/expert.zig:226-264; csrc/q3_lookahead4_exl3.c): one
 * expert's record, in the reference's layout, becomes HBM resident.  `record` is a host pointer (on_device = 0) or a
 * device pointer (1); nbytes >= logical bytes.  Experts outside this rank's shard are accepted and ignored. */
int mlxs_moe_load_expert(mlxs_moe *h, uint32_t layer, uint32_t expert, const void *record, uint64_t nbytes,
                         int on_device);
/* Bank.open + stream fill (src/expert/bank.zig:208-324, src/arch/mimo_v2/bank.zig:172-260,
 * src/arch/glm5_next/bank.zig:29-48): reads <dir>/expert-manifest*.json + experts.bin in the reference's formats,
 * verifies geometry (and record sha256 when the manifest carries it) and loads this rank's experts. */
int mlxs_moe_load_bank(mlxs_moe *h, const char *dir);

/* Peek (src/expert/bank.zig:686-690, src/arch/glm5_next/bank.zig:395): the manifest of the bank at `dir`, or a manifest
 * text, parsed and checked field by field without any device; refusals name the field (MLXS_E_MANIFEST). */
typedef struct {
    uint32_t bank_kind, has_sha256;
    uint64_t hidden, inter, n_experts, n_layers, first_layer;
    uint64_t logical_bytes, record_stride, data_bytes;
    char data_file[64];
    /* EXL3: narrowest and widest layer of the bank; bank_kind, logical_bytes and record_stride are the widest layer's.
     * 0 for the FP4 banks. */
    uint32_t bits_min, bits_max;
} mlxs_bank_info;
int mlxs_moe_bank_peek(const char *dir, mlxs_bank_info *out);
int mlxs_moe_bank_peek_text(const char *manifest_json, mlxs_bank_info *out);
/* Bank.open without a device (src/expert/bank.zig:228-251, 326-400): the manifests of the bank at `dir` (for an EXL3
 * bank both of them: the v2 geometry and the v1 runtime manifest expert-manifest.json, which must describe exactly the
 * v2 records), the sidecar file (present, not a symbolic link, at least the manifest's size) and, with verify_sha256,
 * every record's digests (v2: the padded record, v1: its logical bytes).  mlxs_moe_load_bank runs the same checks. */
int mlxs_moe_bank_verify(const char *dir, mlxs_bank_info *out, int verify_sha256);
/* K of every layer of an EXL3 manifest text (v2 peek, src/expert/bank.zig:641-662): writes min(n_layers, cap) widths
 * and the layer count */
int mlxs_moe_bank_layer_bits_text(const char *manifest_json, uint32_t *bits_out, uint32_t cap, uint32_t *n_layers_out);

/* the router's noaux_tc correction bias, f32 [n_experts] host, NULL = zeros (src/arch/deepseek_v41/graph.zig:2035) */
int mlxs_moe_set_router_bias(mlxs_moe *h, uint32_t layer, const float *bias_host);
/* Router weight W_g bf16 [n_experts, hidden] (src/arch/deepseek_v41/graph.zig:2033): with it the layer can start from x. */
int mlxs_moe_set_router_weight(mlxs_moe *h, uint32_t layer, const void *w_gate_bf16, int on_device);
/* logits[T, n_experts] f32 = f32(x) . f32(W_g)^T, f32 accumulate in a fixed order (own kernel up to 64 tokens, one
 * library GEMM above) */
int mlxs_moe_logits(mlxs_moe *h, uint32_t layer, const void *x_dev, uint32_t T, float *logits_dev, void *stream);
/* mlxs_moe_logits into the handle's workspace, then mlxs_moe_forward: the whole layer from x
 * (Source.forward's real caller, src/arch/glm5_next/experts.zig:566-595) */
int mlxs_moe_forward_x(mlxs_moe *h, uint32_t layer, const void *x_dev, uint32_t T, void *y_dev, void *stream);
/* the shared expert's bf16 linears: w1 (gate) [inter, hidden], w3 (up) [inter, hidden], w2 (down) [hidden, inter]
 * (src/arch/deepseek_v41/graph.zig:2162-2172 sh_w1 / sh_w3 / sh_w2) */
int mlxs_moe_set_shared(mlxs_moe *h, uint32_t layer, const void *w1, const void *w3, const void *w2, int on_device);

/* Gate.__call__'s tail (src/arch/deepseek_v41/graph.zig:2041-2051, src/kernels/exl3/q3rc_router_tail.metal:12-40,
 * src/arch/mimo_v2/kernels/mimo_glue_top8.metal): logits f32 [T, n_experts] -> ids i32 [T, top_k] in rank order
 * (score + bias descending, ties to the lower index, NaN last), weights f32 [T, top_k]. */
int mlxs_moe_route(mlxs_moe *h, uint32_t layer, const float *logits_dev, uint32_t T, int32_t *ids_dev,
                   float *weights_dev, void *stream);
/* Hook.routed (src/arch/deepseek_v41/experts.zig:1214-1223): x bf16 [T, hidden], ids [T, top_k] -> the unweighted
 * expert outputs f32 [T, top_k, hidden] in router order. */
int mlxs_moe_routed(mlxs_moe *h, uint32_t layer, const void *x_dev, const int32_t *ids_dev, uint32_t T,
                    float *out_dev, void *stream);
/* Source.forward + forwardShared (src/arch/glm5_next/experts.zig:566-595, 639-653): x bf16 [T, hidden], ids, weights
 * -> y bf16 [T, hidden] (routed experts, weighted combine, + shared expert when configured).
 * Everything is ordered on `stream`: the handle's own side streams (the shared expert beside the routed kernels, the
 * tensor-core lane beside the streaming lane) fork from it by an event and join it before the result is written, so
 * the caller sees one stream, and a call can be captured into a CUDA graph (one GPU). */
int mlxs_moe_experts(mlxs_moe *h, uint32_t layer, const void *x_dev, const int32_t *ids_dev,
                     const float *weights_dev, uint32_t T, void *y_dev, void *stream);
/* Tr.moe (src/arch/deepseek_v41/graph.zig:2196-2240) from the router's logits on: route + experts in one call; the
 * ids never visit the host (the reference's routing barrier, experts.zig:1576-1587, is gone). */
int mlxs_moe_forward(mlxs_moe *h, uint32_t layer, const void *x_dev, const float *logits_dev, uint32_t T, void *y_dev,
                     void *stream);
/* the same through host buffers (what arch.step / arch.prefill's caller holds): copies x and logits in, runs,
 * copies y out and synchronises the stream. */
int mlxs_moe_forward_host(mlxs_moe *h, uint32_t layer, const void *x_host, const float *logits_host, uint32_t T,
                          void *y_host, void *stream);

/* quant seam, one projection without the rotations: z f32 [rows, out] = xh f32 [rows, in] . W_hat of
 * (layer, expert, proj 0 gate / 1 up / 2 down) through the same in-register decode as the layer path.  One-hot rows
 * give W_hat's rows bit for bit: the reference's decode_table self-check (src/exl3/selfcheck.zig:848-901). */
int mlxs_moe_exl3_gemv(mlxs_moe *h, uint32_t layer, uint32_t expert, uint32_t proj, const float *xh_dev,
                       uint32_t rows, float *z_dev, void *stream);

/* The same projection for callers that may not allocate device memory: z f32 [rows, out_dim] = xh f32 [rows, in_dim]
 * . W_hat of the code plane at code_dev (I16 [in_dim/16, out_dim/16, 48], the bank file's order; K = 3 planes only,
 * a K = 2 plane has 32 values per tile and is not accepted here).  xh_dev must be 16-byte aligned, code_dev and z_dev
 * 4-byte aligned (refused by name otherwise).  It has no counterpart in the reference.  It needs no handle and calls no allocator: a host that fixes its device-memory
 * budget at load time, or code running while a stream is being captured (where cudaMalloc is not allowed), can still
 * use it.  Its scratch is a fixed 1 MiB array inside the library, which limits a call to rows <= 32 and
 * in_dim <= 8192 (a multiple of 128; out_dim a multiple of 16); larger sizes are refused.  The first call on a device
 * looks up the array's address (make that call before any stream capture).  All calls share the array: calls that
 * overlap on the GPU race, so keep them on one stream or order them yourself. */
int mlxs_moe_exl3_gemv_noalloc(const void *code_dev, uint32_t in_dim, uint32_t out_dim, const float *xh_dev,
                               uint32_t rows, float *z_dev, void *stream);

/* Measured ceiling of the EXL3 in-register decode on this GPU (the reference's kernel bench has the same role for its
 * lanes, src/arch/glm5_next/exl3_kbench.zig:1-23): the streaming kernel's decode statements alone, operands from
 * registers, no loads, with (with_mma != 0) or without the one mma per tile, at the streaming kernel's residency.
 * tiles_per_s x 32 bits bytes per tile (96 at K = 3, 64 at K = 2) is the code rate the decode can consume whatever
 * the memory system delivers.  Allocates 16 bytes for the duration of the call; needs no handle. */
int mlxs_moe_exl3_decode_rate(int32_t device, uint32_t bits, int with_mma, uint32_t tiles_per_warp, double *tiles_per_s);

/* The native block-scaled FP4 tensor-core instruction, measured (no counterpart in the reference, whose FP4 prefill is a
 * sorted quantised GEMM of its array library, src/arch/mimo_v2/math.zig:426-447): tcgen05.mma.kind::mxf8f6f4.block_scale
 * with A = MXFP4 codes and E8M0 block scales as the bank stores them and B = bf16 rows split into an E4M3 high and low
 * part with UE8M0 block scales.  rel_l2_*: the product over one 128 x 64 x 128 tile against the exact product of the
 * bf16 rows (hi + lo, and hi alone); tflops_*: issue rates of the two instruction streams on shared-memory operands
 * (M 128, N 256, rate_mmas instructions per SM; 0 skips the timing); the hi / lo pair needs two 8-bit-rate MMAs per 32
 * inputs, so its useful rate is tflops_mxf8f6f4 / 2. */
typedef struct {
    double rel_l2_hi_lo, rel_l2_hi_only;
    double tflops_f16, tflops_mxf8f6f4, tflops_hi_lo_effective;
} mlxs_fp4_native_result;
int mlxs_moe_fp4_native_probe(int32_t device, uint32_t rate_mmas, mlxs_fp4_native_result *out);

/* Time of one tcgen05.mma.kind::f16 (M 128 x N x K 16, bf16) issued back to back by one thread per SM on all SMs, with the
 * A operand in shared memory (a_from_tmem = 0) or in tensor memory: what the tensor-core lanes' tile shapes are chosen
 * by (no counterpart in the reference).  n: 16 .. 256, a multiple of 16; mmas instructions per SM.  ns_per_mma: the
 * measured time; the rate is 2 x 128 x n x 16 / ns_per_mma per SM.  Needs no handle. */
int mlxs_moe_mma_rate(int32_t device, uint32_t n, int a_from_tmem, uint32_t mmas, double *ns_per_mma);

int mlxs_moe_stats_get(mlxs_moe *h, mlxs_moe_stats *out);
/* The device status word is sticky (a host must see a fault it did not poll for): once a kernel has recorded an error
 * every mlxs_moe_forward_host returns MLXS_E_DEVICE_STATUS until the host acknowledges it here.  Synchronises the
 * device, clears the word and the streaming kernels' arrival counters a call that gave up may have left behind.
 * No counterpart in the reference (its kernels have no device-side error word). */
int mlxs_moe_status_clear(mlxs_moe *h);
/* The dispatch permutation by itself (src/sdk_ext/quant.zig:269-301 counting sort; src/arch/glm5_next/exl3_math.zig:
 * 192-225): rows with slot ids slot_dev[n] in [0, n_slots) -> order_dev[n] (sorted position -> row, rows of one slot
 * keep their order) and offsets_dev[n_slots + 1] (first sorted position of every slot).  It runs the layer path's own
 * dispatch kernels (one CTA up to 2048 rows, count / scan / place above) on the handle's tables and copies the two
 * arrays out; n_slots <= n_experts, n <= the handle's row capacity. */
int mlxs_moe_sort_rows(mlxs_moe *h, const int32_t *slot_dev, uint32_t n, uint32_t n_slots, uint32_t *order_dev,
                       uint32_t *offsets_dev, void *stream);
/* Self-test of the bounded waits (no counterpart in the reference).  Every wait inside a kernel gives up after a
 * number of polls, records MLXS_E_DEVICE_STATUS's word and lets the CTA return; poll_limit sets that number for the
 * EXL3 streaming kernels (0 = the default, 2^20).  withhold_stage = n > 0 makes every gate/up producer leave out the
 * copies of its n-th ring stage, so the wait for that stage runs out: the call completes, the status word reads
 * "a bounded wait ran out", nothing faults and nothing is left in flight.  (0, 0) restores normal operation. */
int mlxs_moe_debug_wait(mlxs_moe *h, uint32_t poll_limit, uint32_t withhold_stage);

/* per-stage device timing with CUDA events on the caller's stream, off by default (the reference's comptime profile
 * hooks and kernel bench: src/sdk_ext/profile.zig:1-60, src/arch/glm5_next/exl3_kbench.zig:1-23).  `read` synchronises
 * the pending events, returns the sums since the last read and clears them. */
enum { MLXS_STAGE_ROUTER = 0, MLXS_STAGE_DISPATCH, MLXS_STAGE_PREP, MLXS_STAGE_GATE_UP, MLXS_STAGE_DOWN,
       MLXS_STAGE_SHARED, MLXS_STAGE_COMBINE, MLXS_STAGE_EXCHANGE,
       MLXS_STAGE_TENSOR_LANE, /* gate/up + down of the experts that took the tensor-core lane */
       MLXS_STAGE_COUNT };
typedef struct {
    double ms[MLXS_STAGE_COUNT];
    uint64_t launches[MLXS_STAGE_COUNT];
} mlxs_moe_profile;
int mlxs_moe_profile_enable(mlxs_moe *h, int on);
int mlxs_moe_profile_read(mlxs_moe *h, mlxs_moe_profile *out);

/* ---- expert parallel (no counterpart in the reference: it pages experts from SSD on one GPU; here they are HBM
 * resident and sharded, with a dispatch and a combine all-to-all per layer) ---- */
/* 128-byte NCCL unique id made on rank 0 and handed to every rank by the host */
int mlxs_moe_ep_unique_id(void *id128_out);
/* Joins the ranks: the NCCL communicator, then one window of device memory per rank that the other ranks map through
 * CUDA IPC (mlxs_moe_ep_window_bytes says how large).  With the windows mapped a layer call exchanges rows by plain
 * stores into the peers' windows: no host synchronisation and no collective inside the call (stats.ep_transport = 2).
 * If any rank cannot map a window all ranks fall back to NCCL send/recv with a host-read count exchange (= 1).
 * Capacity: a rank's workspace holds min(world, 4) x max_tokens x top_k received rows; a call that sends a rank more
 * is not executed on that rank, which records MLXS_E_DEVICE_STATUS ("expert parallel: more rows than the workspace
 * holds"), while every rank still completes the call: nobody is left waiting.  Every rank must make the same sequence
 * of layer calls (a rank without tokens calls with T = 0).  Waits for a peer are bounded (MLXS_EP_WAIT_MS, 20 s by
 * default) and report through the status word.  Expert-parallel calls cannot be captured into a CUDA graph. */
int mlxs_moe_ep_init(mlxs_moe *h, const void *id128);
/* bytes of the window mlxs_moe_ep_init allocates per rank (pure arithmetic) */
uint64_t mlxs_moe_ep_window_bytes(uint32_t world, uint32_t max_tokens, uint32_t top_k, uint32_t n_experts, uint32_t hidden);
/* The all-ranks capacity check of the NCCL transport as a pure function: counts[(s * world + d) * stride] = rows rank s
 * sends to rank d; returns the lowest rank that would receive more than rows_cap rows, or -1.  Every rank evaluates it
 * on the same matrix and refuses the call together, before any send or receive is queued. */
int32_t mlxs_moe_ep_overloaded_rank(const int32_t *counts, uint32_t world, uint32_t stride, uint64_t rows_cap);
/* Where a layer's experts live: rank_of_expert[e] in [0, ep_world), every rank exactly n_experts / ep_world of them;
 * an expert's local slot is its order among the rank's experts.  Default: contiguous blocks.  Call on every rank with
 * the same table before the layer's experts are loaded.  (The reference keeps a usage tally per expert for its
 * residency policy, src/sdk_ext/expert/usage.zig; here the same histogram can balance the ranks' load.) */
int mlxs_moe_set_placement(mlxs_moe *h, uint32_t layer, const uint16_t *rank_of_expert);
/* host-side plan of one exchange (pure function, also used by the CPU tests): for `n` assignments with expert ids
 * `ids`, counts per destination rank */
int mlxs_moe_ep_plan(const int32_t *ids, uint64_t n, uint32_t n_experts, uint32_t world, uint64_t *send_counts);

/* Usage tally (src/sdk_ext/expert/usage.zig:202-224 keeps per-layer per-expert route counts to seed residency; here
 * the same counts decide which rank holds which expert).  While enabled, every mlxs_moe_route (and so every
 * mlxs_moe_forward*) adds its ids to the layer's device-side counts: one small kernel per call, nothing read back.
 * A host that routes elsewhere adds its ids with mlxs_moe_usage_add.  usage_read copies a layer's counts to the host;
 * with all_ranks != 0 on an expert-parallel handle the ranks' counts are summed first (every rank must call it). */
int mlxs_moe_usage_enable(mlxs_moe *h, int on);
int mlxs_moe_usage_add(mlxs_moe *h, uint32_t layer, const void *ids_dev, uint64_t n_ids, void *stream);
int mlxs_moe_usage_read(mlxs_moe *h, uint32_t layer, uint64_t *counts_host, int all_ranks);
int mlxs_moe_usage_reset(mlxs_moe *h);
/* counts -> placement: experts in order of use (most used first, ties to the lower id: Profile.order,
 * src/sdk_ext/expert/usage.zig:352-366) dealt to the ranks in snake order, n_experts / world per rank, so the ranks'
 * expected rows come out even under skewed routing.  Pure host arithmetic; feed the result to mlxs_moe_set_placement. */
int mlxs_moe_plan_placement(const uint64_t *counts, uint32_t n_experts, uint32_t world, uint16_t *rank_of_expert);

#ifdef __cplusplus
}
#endif
#endif
