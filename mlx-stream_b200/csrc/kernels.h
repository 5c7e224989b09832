// Host-visible launchers of the routed-MoE kernels (internal to the library; the public surface is include/mlxs_moe.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mlxs {

// Rows of one expert are processed in chunks of 4 (one mma n-tile of 8 token slots: 4 rows as f16 hi + the same
// 4 rows as f16 lo) and a work item carries up to GROUP_CHUNKS chunks of one expert.
constexpr int CHUNK_ROWS = 4;
constexpr int GROUP_CHUNKS = 4;

// Device-side dispatch tables (all uint32), rebuilt by every call.
struct DispatchTables {
    uint32_t* header;        // [16]: 0 n_chunks, 1 n_groups, 2 counter gate/up, 3 counter down, 4 distinct experts,
                             //       5 counter aux
    uint32_t* offsets;       // [E + 1] sorted-row offsets per expert
    uint32_t* order;         // [A] sorted row -> assignment index (stable)
    uint32_t* chunk_expert;  // [max_chunks]
    uint32_t* chunk_row0;    // [max_chunks] first sorted row
    uint32_t* chunk_rows;    // [max_chunks] valid rows (1..8)
    uint32_t* group_chunk0;  // [max_chunks]
    uint32_t* group_mc;      // [max_chunks]
    uint32_t max_chunks;
    const uint32_t* xrow;    // optional [A]: row of x an assignment reads (null: assignment / top_k)
};
// the row of x behind assignment a
__host__ __device__ inline uint32_t x_row_of(const DispatchTables& t, uint32_t a, uint32_t top_k) {
    return t.xrow ? t.xrow[a] : a / top_k;
}
enum { HDR_NCHUNKS = 0, HDR_NGROUPS = 1, HDR_CTR_GU = 2, HDR_CTR_DOWN = 3, HDR_DISTINCT = 4, HDR_CTR_AUX = 5 };

// logits[T, E] = f32(x) . f32(W)^T for decode-sized batches (larger ones: launch_dense_logits)
cudaError_t launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* w, uint32_t T, uint32_t E, uint32_t H,
                                 float* logits, cudaStream_t st);
cudaError_t launch_router(const float* logits, const float* bias, int T, int E, int K, int scoring, int norm,
                          float scale, int32_t* ids, float* weights, cudaStream_t st);

// The front of a decode-sized call in one cooperative launch (front.cu): [logits from x] -> route -> dispatch -> row
// staging for the streaming lane.  bar: two zeroed words (the grid barrier).
struct FrontArgs {
    const __nv_bfloat16* w_router;  // [E, H] bf16: phase 0 computes the logits into logits_out; null: `logits` is given
    float* logits_out;
    const float* logits;
    const float* bias;
    int E, K, scoring, norm;
    float scale;
    int32_t* ids;
    float* weights;
    uint32_t T;
    const uint8_t* loaded;
    DispatchTables t;
    uint32_t chunk_rows, group_chunks;
    uint32_t heavy;                 // rows from which an expert leaves the streaming lane (0: never)
    uint32_t* status;
    const __nv_bfloat16* x;
    uint32_t H;
    int bank_exl3;
    const __half* scales;           // EXL3: the layer's sign / scale vectors
    size_t scales_stride;
    uint32_t* xa;
    uint32_t* bar;
    int sm_count;
};
cudaError_t launch_front(const FrontArgs& a, cudaStream_t st);

// ids [A] (A = T*k) -> tables; expert ids outside [0, E) set *status and are treated as expert 0.
// loaded: optional [E] bytes, 0 = expert not resident -> *status = ST_NOT_LOADED.
// chunk_rows / group_chunks: rows per chunk and chunks per work item of the bank's kernels (EXL3 4 x 4, FP4 8 x 2).
// heavy > 0: experts with that many rows or more get no chunks (the tensor-core lane serves them from `offsets`).
// A_dev (optional): the row count lives on the device (at most A, the bound the launch is sized for)
cudaError_t launch_dispatch(const int32_t* ids, uint32_t A, uint32_t E, const uint8_t* loaded, DispatchTables t,
                            uint32_t chunk_rows, uint32_t group_chunks, uint32_t heavy, uint32_t* status, cudaStream_t st,
                            const uint32_t* A_dev = nullptr);

// the same over several CTAs for prefill-sized calls; blk_cnt: scratch [ceil(A/1024)][E]
cudaError_t launch_dispatch_large(const int32_t* ids, uint32_t A, uint32_t E, const uint8_t* loaded, DispatchTables t,
                                  uint32_t chunk_rows, uint32_t group_chunks, uint32_t heavy, uint32_t* blk_cnt,
                                  uint32_t* status, cudaStream_t st, const uint32_t* A_dev = nullptr);

// usage tally: usage[e] += number of ids equal to e
cudaError_t launch_usage_count(const int32_t* ids, uint64_t n, uint32_t E, unsigned long long* usage, cudaStream_t st);

// ---- EXL3 ----
struct Exl3Layer {            // one layer's resident bank, in the kernels' layout
    const uint32_t* gu_code;  // [E][I/128][H/16][2][192] u32: per 128-wide output block, per k-tile, gate | up tiles
    const uint32_t* d_code;   // [E][H/128][I/16][192] u32
    const __half* scales;     // [E][2H + 2I + I + H]: suh_g, suh_u [H] | svh_g, svh_u [I] | suh_d [I] | svh_d [H]
};
struct Exl3Dims { uint32_t H, I, K; };   // K = bits per weight of the trellis code (3 or 2): a 16x16 tile is 8 K words
static inline size_t exl3_scales_per_expert(Exl3Dims d) { return (size_t)3 * d.H + 3 * d.I; }
static inline uint32_t exl3_tile_words(Exl3Dims d) { return 8u * d.K; }
static inline size_t exl3_code_words(Exl3Dims d) { return (size_t)(d.H / 16) * (d.I / 16) * exl3_tile_words(d); }

// record (device, reference v2 layout) -> the expert's slices of the three arrays
cudaError_t launch_exl3_repack(const uint8_t* record_dev, Exl3Dims d, uint32_t* gu_code_e, uint32_t* d_code_e,
                               __half* scales_e, cudaStream_t st);

// activation staging in mma B-fragment order: [chunk][proj][k-tile][32 lanes][2] u32 (256 B per k-tile)
// gate/up inputs: xg = H128(x * suh_g) * 128^-0.5 and xu likewise, f16 hi/lo
cudaError_t launch_exl3_prep_in(const __nv_bfloat16* x, uint32_t top_k, Exl3Layer L, Exl3Dims d, DispatchTables t,
                                uint32_t* xa_gu, cudaStream_t st);
// raw rows (no rotation) into the same order, one projection: xh f32 [rows, in]
cudaError_t launch_exl3_prep_raw(const float* xh, uint32_t in_dim, DispatchTables t, uint32_t* xa, cudaStream_t st);

struct Exl3GemvArgs {
    Exl3Layer L;
    Exl3Dims d;
    DispatchTables t;
    const uint32_t* xa_gu;  // [chunk][2][H/16][64] u32
    uint32_t* xa_d;         // [chunk][I/16][64] u32 (written by gate/up, read by down)
    float* ro;              // [A, H] f32 routed outputs in assignment order (CHAIN combine: bf16 [A, H])
    int ro_bf16;
    float limit;            // > 0: clamped SwiGLU
    uint32_t* status;
    int sm_count;
    float* ks_scratch;      // optional K-split workspace: exl3_ksplit_scratch_bytes(sm_count) bytes
    uint32_t* ks_count;     // [ksplit_count_words(sm_count)] zeroed once
    uint32_t poll_limit;    // polls after which a wait gives up (0: the default, 2^20)
    uint32_t withhold;      // self-test: the gate/up producers leave out their n-th ring stage (0: off)
};
// The fold's workspace: 12 slots per SM of the largest staging array (2 projections x 16 rows x 132 floats), and as many
// arrival counters.  A kernel whose staging array is zs_bytes and whose sums have up to 4 parts can split this many items:
static inline size_t exl3_ksplit_scratch_bytes(int sm_count) { return (size_t)12 * sm_count * 2 * 16 * 132 * 4; }
static inline size_t ksplit_count_words(int sm_count) { return (size_t)12 * sm_count; }
static inline uint32_t ksplit_cap_items(int sm_count, size_t zs_bytes) {
    const size_t by_slots = exl3_ksplit_scratch_bytes(sm_count) / zs_bytes / 4, by_count = ksplit_count_words(sm_count);
    return (uint32_t)(by_slots < by_count ? by_slots : by_count);
}
cudaError_t launch_exl3_gate_up(const Exl3GemvArgs& a, cudaStream_t st);
cudaError_t launch_exl3_down(const Exl3GemvArgs& a, cudaStream_t st);
// raw projection: z [rows, out] = xa . W_hat(code); `code` in the single-projection block layout with a k-tile
// stride of `ktile_stride_words` and the projection at `proj_off_words` (at K = 3: 192/0 for down, 384/{0,192} for
// gate/up; at K = 2: 128/0 and 256/{0,128}); kbits = bits per weight
cudaError_t launch_exl3_raw(const uint32_t* code_e, uint32_t in_dim, uint32_t out_dim, uint32_t ktile_stride_words,
                            uint32_t proj_off_words, int kbits, DispatchTables t, const uint32_t* xa, float* z,
                            uint32_t* status, int sm_count, cudaStream_t st);

// prefill-sized batches: tcgen05 MMA over trellis tiles decoded to f16 in tensor memory (exl3_prefill.cu)
constexpr int PREFILL_TILE_ROWS = 128;
// An expert's lane in a call: the tensor-core lane when it has `min_rows` rows or more, unless its entry of the
// per-expert table (1 = resident, bit 1 = its weights are outside that lane's exact range) says otherwise.
__host__ __device__ inline bool takes_tensor_lane(uint32_t rows, uint32_t min_rows, const uint8_t* flags, uint32_t e) {
    return min_rows && rows >= min_rows && !(flags && (flags[e] & 2u));
}
// Row tiles of the experts that take the tensor-core lane.  tiles[0], tiles[1] = tiles of list 0 (experts with up to
// cap0 rows; with cap1 = 0 all experts, in tiles of up to cap0 rows) and list 1 (the others, tiles of up to cap1 rows);
// entries {expert, first sorted row, rows, first staging row}, list 1 from entry max_tiles.  The table holds
// prefill_tile_words(max_tiles) words.
__host__ __device__ inline size_t prefill_tile_words(uint32_t max_tiles) { return 2 + 8 * (size_t)max_tiles; }
__host__ __device__ inline uint32_t* prefill_tile(uint32_t* tiles, int list, uint32_t max_tiles, uint32_t i) {
    return tiles + 2 + 4 * ((size_t)(list ? max_tiles : 0) + i);
}
__host__ __device__ inline const uint32_t* prefill_tile(const uint32_t* tiles, int list, uint32_t max_tiles, uint32_t i) {
    return tiles + 2 + 4 * ((size_t)(list ? max_tiles : 0) + i);
}
cudaError_t launch_prefill_plan(DispatchTables t, uint32_t n_experts, const uint8_t* lane_flags, uint32_t min_rows,
                                uint32_t cap0, uint32_t cap1, uint32_t max_tiles, uint32_t* tiles, uint32_t* status,
                                cudaStream_t st);
struct Exl3PrefillArgs {
    Exl3Layer L;
    Exl3Dims d;
    DispatchTables t;
    uint32_t n_experts;      // experts the dispatch ran over
    uint32_t min_rows;       // only experts with at least this many rows take this lane
    const __nv_bfloat16* x;  // [tokens, H]
    uint32_t top_k;
    uint32_t* tiles;         // [prefill_tile_words(max_tiles)] row-tile table (device scratch)
    uint32_t max_tiles;
    __half* xa;              // [2 projections][staging rows][H] f16: rotated rows in the MMA's B-operand order
    __half* xd;              // [staging rows][I] f16
    uint32_t rows_cap;       // assignment rows the staging was sized for
    float* ro;               // [A, H]
    float limit;
    uint32_t* status;
    int sm_count;
    // optional: a stream for the kernels of the large tiles (they touch other experts than the small-tile kernels), with
    // the two events that fork it from and join it into the call's stream; null: one stream
    cudaStream_t side = nullptr;
    cudaEvent_t side_fork = nullptr, side_join = nullptr;
};
// staging rows: every tile's rows padded to 16, tiles in sorted order
static inline size_t exl3_prefill_staging_rows(size_t rows_cap, uint32_t max_tiles) { return rows_cap + 16 * (size_t)(2 * max_tiles + 1); }
static inline size_t exl3_prefill_xa_bytes(Exl3Dims d, size_t rows_cap, uint32_t max_tiles) { return 2 * exl3_prefill_staging_rows(rows_cap, max_tiles) * d.H * 2; }
static inline size_t exl3_prefill_xd_bytes(Exl3Dims d, size_t rows_cap, uint32_t max_tiles) { return exl3_prefill_staging_rows(rows_cap, max_tiles) * d.I * 2; }
cudaError_t launch_exl3_prefill(const Exl3PrefillArgs& a, cudaStream_t st);
bool exl3_prefill_supported(Exl3Dims d);  // the lane groups 2 (gate/up) and 4 (down) column blocks per CTA

// ---- MXFP4 / NVFP4 ----
constexpr int FP4_CHUNK_ROWS = 8;
constexpr int FP4_GROUP_CHUNKS = 2;
static inline size_t fp4_stream_bytes_per_expert(uint32_t H, uint32_t I, int nv, int down) {
    const size_t per_stage = (size_t)(down ? 1 : 2) * (8192 + (nv ? 1024 : 512));
    return (size_t)(H / 128) * (I / 128) * per_stage;
}
// record (device, reference layout) -> the expert's slices of the gate/up stream, the down stream and the global scales
// lane_flag: the expert's entry of the per-expert table; set to 3 when an MXFP4 block scale exceeds 2^1
cudaError_t launch_fp4_repack(const uint8_t* record_dev, uint32_t H, uint32_t I, int nv, uint8_t* gu_e, uint8_t* dn_e,
                              float* gscale_e, uint8_t* lane_flag, cudaStream_t st);
// x bf16 [T, H] -> f16 rows in the kernels' B-fragment order: [chunk][H/32][128] u32
cudaError_t launch_fp4_prep(const __nv_bfloat16* x, uint32_t top_k, uint32_t H, DispatchTables t, uint32_t* xa,
                            cudaStream_t st);
struct Fp4GemvArgs {
    const uint8_t* gu;      // layer base, [E] x fp4_stream_bytes_per_expert(.., 0)
    const uint8_t* dn;      // layer base, [E] x fp4_stream_bytes_per_expert(.., 1)
    const float* gscale;    // NVFP4: [E][3], else null
    int nv;
    uint32_t H, I;
    DispatchTables t;
    const uint32_t* xa;     // [chunk][H/32][128]
    uint32_t* xa_d;         // [chunk][I/32][128]
    void* ro;               // [A, H] bf16 (chain combine) or f32
    int ro_bf16;
    float limit;
    uint32_t* status;
    int sm_count;
    float* ks_scratch;      // optional K-split workspace, exl3_ksplit_scratch_bytes(sm_count) bytes
    uint32_t* ks_count;     // [ksplit_count_words(sm_count)] zeroed once
};
cudaError_t launch_fp4_gemv(const Fp4GemvArgs& a, int down, cudaStream_t st);
// experts with many rows: tcgen05 MMA over codes decoded to 16-bit operands in tensor memory (fp4_prefill.cu)
struct Fp4PrefillArgs {
    const uint8_t* gu;       // the streams of Fp4GemvArgs
    const uint8_t* dn;
    const float* gscale;
    int nv;
    uint32_t H, I;
    DispatchTables t;
    uint32_t n_experts;      // experts the dispatch ran over
    const uint8_t* lane_flags;  // [n_experts] per-expert table of takes_tensor_lane
    uint32_t min_rows;
    const __nv_bfloat16* x;  // [tokens, H]
    uint32_t top_k;
    uint32_t* tiles;         // [prefill_tile_words(max_tiles)]
    uint32_t max_tiles;
    uint16_t* xa;            // [staging rows][H] rows in the MMA's B-operand order (bf16 MXFP4, f16 NVFP4; the block-scaled
                             // MXFP4 lane keeps E4M3 high / low parts and scale bytes here, mxfp4_native_xa_bytes)
    uint16_t* xd;            // [staging rows][I], the same for the down product
    uint32_t rows_cap;       // assignment rows the staging was sized for
    void* ro;                // [A, H] bf16 (chain combine) or f32
    int ro_bf16;
    float limit;
    uint32_t* status;
    int sm_count;
    // optional: a stream for the kernels of the large tiles, with the events that fork it from and join it into the
    // call's stream (as in Exl3PrefillArgs); null: one stream
    cudaStream_t side = nullptr;
    cudaEvent_t side_fork = nullptr, side_join = nullptr;
};
// the large-tile kernels beside the small-tile ones: fork before, join after (always, also after a refused launch)
template <class F>
static inline cudaError_t prefill_lists_side_by_side(cudaStream_t st, cudaStream_t side, cudaEvent_t fork_ev, cudaEvent_t join_ev, F&& launches) {
    cudaError_t e = cudaSuccess;
    if (side && ((e = cudaEventRecord(fork_ev, st)) != cudaSuccess || (e = cudaStreamWaitEvent(side, fork_ev, 0)) != cudaSuccess)) return e;
    e = launches(side ? side : st);
    if (side) {
        const cudaError_t j1 = cudaEventRecord(join_ev, side);
        const cudaError_t j2 = j1 == cudaSuccess ? cudaStreamWaitEvent(st, join_ev, 0) : j1;
        if (e == cudaSuccess) e = j2;
    }
    return e;
}
// staging rows: every tile's rows padded to 16
static inline size_t fp4_prefill_xa_bytes(uint32_t width, size_t rows_cap, uint32_t max_tiles) {
    return (rows_cap + 16 * (size_t)(2 * max_tiles + 1)) * width * 2;
}
cudaError_t launch_fp4_prefill(const Fp4PrefillArgs& a, cudaStream_t st);
// MXFP4 on the block-scaled tensor-core kind (fp4_native.cu): the same arguments; xa / xd hold the rows split into E4M3
// high and low parts with their block scales, 132 bytes per row per 64 inputs
static inline size_t mxfp4_native_xa_bytes(uint32_t width, size_t rows_cap, uint32_t max_tiles) {
    return (rows_cap + 16 * (size_t)(2 * max_tiles + 1)) * (width / 64) * 132;
}
cudaError_t launch_mxfp4_native(const Fp4PrefillArgs& a, cudaStream_t st);
bool fp4_prefill_supported(uint32_t H, uint32_t I);

// ---- shared expert (bf16 dense) + combine ----
cudaError_t launch_shared_expert(const __nv_bfloat16* x, const __nv_bfloat16* w1, const __nv_bfloat16* w3,
                                 const __nv_bfloat16* w2, uint32_t T, uint32_t H, uint32_t I, float limit,
                                 __nv_bfloat16* h_ws, float* out, cudaStream_t st);
// ---- dense bf16 products on tcgen05 (dense_gemm.cu): the shared expert at every batch size, the router's logits ----
// weights re-tiled at load: w_gu = [I/128][H/64] stages of gate and up interleaved, w_d = [H/128][I/64]; see the file
struct DenseSharedArgs {
    const __nv_bfloat16* x;  // [T, H]
    const void* w_gu;        // re-tiled gate + up, 2 * H * I bf16
    const void* w_d;         // re-tiled down, H * I bf16
    uint32_t T, H, I;
    float limit;
    uint16_t* xb;            // [T rounded to 16, H] rows in the MMA's B-operand order (scratch)
    uint16_t* hb;            // [T rounded to 16, I] h in the same order (scratch)
    float* out;              // [T, H] f32
    float* part_scratch;     // dense_gemm_scratch_bytes(sm_count), or null: never split the reduction
    uint32_t* part_count;    // [sm_count] zeroed once
    uint32_t* status;
    int sm_count;
};
size_t dense_gemm_scratch_bytes(int sm_count);
bool dense_gemm_supported(uint32_t n_out, uint32_t K, int two_blocks);
// W[n_out, K] row-major bf16 (w1 = a second matrix interleaved per 8-row group, or null) -> the tiled order
cudaError_t launch_dense_retile(const __nv_bfloat16* w0, const __nv_bfloat16* w1, uint32_t n_out, uint32_t K, void* dst,
                                cudaStream_t st);
cudaError_t launch_dense_shared_expert(const DenseSharedArgs& a, cudaStream_t st);
// logits[T, E] f32 = x . W_g^T with W_g re-tiled (single projection); E a multiple of 256
cudaError_t launch_dense_logits(const __nv_bfloat16* x, const void* w_tiled, uint32_t T, uint32_t E, uint32_t H, uint16_t* xb,
                                float* logits, float* part_scratch, uint32_t* part_count, uint32_t* status, int sm_count,
                                cudaStream_t st);
// y[t] = sum_k ro[t,k] w[t,k] (+ shared[t]) -> bf16
cudaError_t launch_combine(const void* ro, int ro_bf16, const float* weights, const float* shared, uint32_t T,
                           uint32_t K, uint32_t H, int chain, __nv_bfloat16* y, cudaStream_t st);

}  // namespace mlxs
