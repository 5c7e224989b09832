// The handle behind include/mlxs_moe.h (internal).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <vector>

#include "../../include/mlxs_moe.h"
#include "kernels.h"

using namespace mlxs;

int mlxs_fail(int rc, const char* fmt, ...);  // sets the thread's last-error text, returns rc

struct EpState;  // expert-parallel exchange (ep.cu)

struct LayerBank {
    uint32_t* gu_code = nullptr;
    uint32_t* d_code = nullptr;
    __half* scales = nullptr;
    uint8_t *f4_gu = nullptr, *f4_dn = nullptr;  // FP4 banks: the two streams
    float* f4_gscale = nullptr;                  // NVFP4 [E_local][3]
    uint8_t* loaded_dev = nullptr;  // [E_local] per local slot: 1 = loaded (bit 1: see takes_tensor_lane)
    std::vector<uint8_t> loaded;    // [E] by expert id, host copy
    // EXL3: this layer's bits per weight and record size (a bank may mix widths; mlxs_moe_set_layer_bits)
    uint32_t kbits = 3;
    uint64_t logical_bytes = 0, record_stride = 0;
    // where each expert lives: rank and local slot (contiguous blocks unless mlxs_moe_set_placement changed it)
    std::vector<uint16_t> place_rank, place_slot;
    uint32_t* place_dev = nullptr;  // [E] rank << 16 | slot
    bool placement_custom = false;
    unsigned long long* usage = nullptr;  // [E] route counts (mlxs_moe_usage_enable), or null
    float* bias = nullptr;          // [E] or null
    __nv_bfloat16* router_w = nullptr;  // [E, H] bf16 or null (logits supplied by the caller)
    __nv_bfloat16 *sh_w1 = nullptr, *sh_w3 = nullptr, *sh_w2 = nullptr;
    // the same weights re-tiled for the tensor-core products (dense_gemm.cu): gate + up interleaved, down
    void *sh_gu_t = nullptr, *sh_d_t = nullptr;
    void* router_w_t = nullptr;         // router weight re-tiled (n_experts a multiple of 256), or null
};

struct mlxs_moe {
    mlxs_moe_config cfg{};
    int sm_count = 0;
    uint32_t e_local = 0, e_first = 0;
    uint64_t logical_bytes = 0, record_stride = 0;
    bool usage_on = false;
    uint64_t last_logical = 0;  // record size of the layer the last expert call ran
    std::vector<LayerBank> layers;
    std::vector<void*> allocs;
    uint64_t resident = 0;
    // workspaces
    int32_t* ids_ws = nullptr;
    float* w_ws = nullptr;
    DispatchTables tabs{};
    uint32_t* blk_cnt = nullptr;  // per-block histograms of the multi-CTA dispatch
    uint32_t* xa_gu = nullptr;
    uint32_t* xa_d = nullptr;
    float* ro = nullptr;
    // prefill lane (EXL3): row-tile table and operand staging, allocated when the handle can see prefill-sized calls
    uint32_t* pf_tiles = nullptr;
    __half *pf_xa = nullptr, *pf_xd = nullptr;
    uint32_t pf_max_tiles = 0;
    uint32_t pf_min_rows = 0;   // experts with at least this many rows of a call take the tensor-core lane (0: lane off)
    uint32_t chunk_rows = CHUNK_ROWS, group_chunks = GROUP_CHUNKS;
    __nv_bfloat16* sh_h = nullptr;
    // dense tensor-core products (shared expert, router logits): rows / h in the MMA's B-operand order, the scratch of
    // the split reduction
    uint16_t *dg_xb = nullptr, *dg_hb = nullptr;
    float* dg_scratch = nullptr;
    uint32_t* dg_count = nullptr;
    // small batches: the shared expert runs beside the routed kernels on a second stream (they leave SMs free)
    float* logits_ws = nullptr;       // [max_tokens, E] logits of mlxs_moe_forward_x
    float* ks_scratch = nullptr;      // K-split workspace of the streaming kernels (exl3.cu)
    uint32_t* ks_count = nullptr;
    cudaStream_t aux_stream = nullptr;
    cudaEvent_t aux_fork = nullptr, aux_join = nullptr;
    // the tensor-core lane runs on a stream of its own beside the streaming lane
    cudaStream_t lane_stream = nullptr;
    cudaEvent_t lane_fork = nullptr, lane_join = nullptr;
    cudaStream_t lane2_stream = nullptr;   // the tensor-core lane's large-tile kernels beside its small-tile kernels
    cudaEvent_t lane2_fork = nullptr, lane2_join = nullptr;
    float* sh_out = nullptr;
    uint32_t* status = nullptr;
    uint8_t* staging = nullptr;
    void *x_io = nullptr, *y_io = nullptr;
    float* logits_io = nullptr;
    mlxs_moe_stats stats{};
    EpState* ep = nullptr;
    uint32_t* front_bar = nullptr;    // grid barrier of the fused front kernel (two words)
    bool front_done = false;          // the fused front kernel of this call has built the tables and staged the rows
    bool mxfp4_native = true;         // MXFP4 tensor-core lane on the block-scaled kind (MLXS_MXFP4_NATIVE=0 at create: the decoded-operand lane)
    bool front_off = false;           // a cooperative launch was refused once: separate kernels from then on
    uint32_t dbg_poll_limit = 0, dbg_withhold = 0;  // mlxs_moe_debug_wait (self-test of the bounded waits)
    uint32_t rows_cap = 0;  // rows the expert kernels' workspaces hold (assignments of one call, or received rows)
    // per-stage timing (off by default)
    bool prof_on = false;
    struct Span { int stage; cudaEvent_t a, b; };
    std::vector<Span> spans;
    std::vector<cudaEvent_t> ev_pool;
    mlxs_moe_profile prof{};
    cudaEvent_t ev_get() {
        if (!ev_pool.empty()) { cudaEvent_t e = ev_pool.back(); ev_pool.pop_back(); return e; }
        cudaEvent_t e = nullptr;
        cudaEventCreate(&e);
        return e;
    }

    template <class T>
    int alloc(T** p, size_t n_bytes) {
        void* q = nullptr;
        cudaError_t e = cudaMalloc(&q, n_bytes ? n_bytes : 16);
        if (e != cudaSuccess) return mlxs_fail(MLXS_E_CUDA, "cudaMalloc(%zu): %s", n_bytes, cudaGetErrorString(e));
        allocs.push_back(q);
        resident += n_bytes;
        *p = static_cast<T*>(q);
        return 0;
    }
    // gives back one allocation of alloc() (a layer whose width changed before its load)
    template <class T>
    void release(T** p, size_t n_bytes) {
        if (!*p) return;
        for (size_t i = 0; i < allocs.size(); ++i)
            if (allocs[i] == static_cast<void*>(*p)) { allocs[i] = allocs.back(); allocs.pop_back(); break; }
        cudaFree(*p);
        resident -= n_bytes;
        *p = nullptr;
    }
};


// brackets one stage's launches with events when profiling is on
struct StageTimer {
    mlxs_moe* h; cudaStream_t st; cudaEvent_t a = nullptr, b = nullptr; int stage;
    StageTimer(mlxs_moe* h_, int stage_, cudaStream_t st_) : h(h_), st(st_), stage(stage_) {
        if (h->prof_on) { a = h->ev_get(); b = h->ev_get(); cudaEventRecord(a, st); }
    }
    ~StageTimer() {
        if (a) { cudaEventRecord(b, st); h->spans.push_back({stage, a, b}); }
    }
};

// dispatch + the bank's expert kernels over `rows` = n_tok * top_k assignment rows with ids in [0, n_exp) indexing this
// rank's resident experts from `first`: unweighted rows in assignment order into ro (api.cu)
// n_rows_dev (optional): the row count lives on the device; n_tok * top_k is then the bound the launches are sized for
int mlxs_run_routed(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, uint32_t n_tok,
                    uint32_t top_k, uint32_t n_exp, uint32_t first, void* ro, int ro_bf16, cudaStream_t st,
                    const uint32_t* n_rows_dev = nullptr);
// the expert-parallel form of the same (ep.cu): dispatch all-to-all, local experts, combine all-to-all
int mlxs_ep_routed(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, uint32_t T, void* ro,
                   int ro_bf16, cudaStream_t st);
// the layer form with the f32 combine folded in: a token's row travels once per destination rank, weighted partial rows
// come back; y = bf16(sum of partials + shared row)
int mlxs_ep_combined(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, const float* weights_dev,
                     uint32_t T, const float* shared, void* y_dev, cudaStream_t st);
void mlxs_ep_destroy(mlxs_moe* h);
int mlxs_ep_transport(const mlxs_moe* h);                         // 0 none, 1 NCCL send/recv, 2 stores into peers' windows
void mlxs_ep_bytes(mlxs_moe* h, uint64_t* sent, uint64_t* recv);  // adds the peer-store transport's device-side byte counts
// sum of a u64 array over the ranks, in place (expert-parallel handles)
int mlxs_ep_allreduce_u64(mlxs_moe* h, unsigned long long* buf_dev, size_t n, cudaStream_t st);
