// The C ABI (include/mlxs_moe.h): handle, resident bank, workspaces, and the per-call kernel sequence.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <algorithm>
#include <vector>

#include "../../include/mlxs_moe.h"
#include "common.cuh"
#include "kernels.h"

using namespace mlxs;

static thread_local std::string g_err;

static int fail(int rc, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return rc;
}
// the same error channel for the library's other translation units
int mlxs_fail(int rc, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return rc;
}
#define CU(call)                                                                                          \
    do {                                                                                                  \
        cudaError_t e__ = (call);                                                                         \
        if (e__ != cudaSuccess) return fail(MLXS_E_CUDA, "%s: %s", #call, cudaGetErrorString(e__));     \
    } while (0)

#include "handle.h"

extern "C" int32_t mlxs_moe_abi(void) { return MLXS_MOE_ABI; }
extern "C" const char* mlxs_moe_last_error(void) { return g_err.c_str(); }

static uint64_t exl3_logical(uint64_t H, uint64_t I, uint64_t K) { return 3 * ((H / 16) * (I / 16) * 32 * K) + 6 * H + 6 * I; }
static inline bool is_exl3(uint32_t kind) { return kind == MLXS_BANK_EXL3_K3_MUL1 || kind == MLXS_BANK_EXL3_K2_MUL1; }
static inline uint32_t exl3_bits(uint32_t kind) { return kind == MLXS_BANK_EXL3_K2_MUL1 ? 2u : 3u; }
static uint64_t mxfp4_logical(uint64_t H, uint64_t I) { return 3 * (H * I / 2 + H * I / 32); }
static uint64_t nvfp4_logical(uint64_t H, uint64_t I) { return 3 * (H * I / 2 + H * I / 16 + 4); }

extern "C" int mlxs_moe_create(const mlxs_moe_config* c, mlxs_moe** out) {
    if (!c || !out) return fail(MLXS_E_ARG, "create: null argument");
    *out = nullptr;
    if (c->struct_size != sizeof(mlxs_moe_config))
        return fail(MLXS_E_CONFIG, "create: struct_size %u, this library has %zu", c->struct_size, sizeof(mlxs_moe_config));
    // refusals by name, once, at construction (src/exl3/quant.zig:202-212; src/sdk_ext/quant.zig:94-111)
    if (c->hidden == 0 || c->hidden % 128) return fail(MLXS_E_CONFIG, "create: hidden %u is not a multiple of 128", c->hidden);
    if (c->inter == 0 || c->inter % 128) return fail(MLXS_E_CONFIG, "create: inter %u is not a multiple of 128", c->inter);
    if (c->n_experts == 0 || c->n_experts > 1024) return fail(MLXS_E_CONFIG, "create: n_experts %u outside 1..1024", c->n_experts);
    if (c->top_k == 0 || c->top_k > 64 || c->top_k > c->n_experts)
        return fail(MLXS_E_CONFIG, "create: top_k %u outside 1..min(64, n_experts)", c->top_k);
    if (c->n_layers == 0) return fail(MLXS_E_CONFIG, "create: n_layers is 0");
    if (c->bank_kind > MLXS_BANK_EXL3_K2_MUL1) return fail(MLXS_E_CONFIG, "create: bank_kind %u unknown", c->bank_kind);
    if (c->act > MLXS_ACT_SWIGLU_CLAMPED) return fail(MLXS_E_CONFIG, "create: act %u unknown (ActivationUnsupported)", c->act);
    if (c->act == MLXS_ACT_SWIGLU_CLAMPED && !(c->act_limit > 0.f))
        return fail(MLXS_E_CONFIG, "create: act_limit must be > 0 for the clamped SwiGLU");
    if (c->scoring > MLXS_SCORE_SOFTMAX) return fail(MLXS_E_CONFIG, "create: scoring %u unknown", c->scoring);
    if (c->combine > MLXS_COMBINE_CHAIN) return fail(MLXS_E_CONFIG, "create: combine %u unknown", c->combine);
    if (c->max_tokens == 0 || c->max_tokens > 65536) return fail(MLXS_E_CONFIG, "create: max_tokens %u outside 1..65536", c->max_tokens);
    if (c->ep_world == 0 || c->ep_rank >= c->ep_world || c->n_experts % c->ep_world)
        return fail(MLXS_E_CONFIG, "create: ep_world %u / ep_rank %u do not shard %u experts", c->ep_world, c->ep_rank, c->n_experts);
    if (is_exl3(c->bank_kind) && c->combine != MLXS_COMBINE_F32)
        return fail(MLXS_E_CONFIG, "create: the EXL3 bank's routed rows are f32; combine must be MLXS_COMBINE_F32");
    int ndev = 0;
    cudaError_t ce = cudaGetDeviceCount(&ndev);
    if (ce != cudaSuccess || ndev == 0)
        return fail(MLXS_E_CUDA, "create: no CUDA device (%s); this library has no CPU path", cudaGetErrorString(ce));
    if (c->device < 0 || c->device >= ndev) return fail(MLXS_E_ARG, "create: device %d of %d", c->device, ndev);
    CU(cudaSetDevice(c->device));
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, c->device));
    if (prop.major != 10) return fail(MLXS_E_CUDA, "create: device is sm_%d%d; the kernels are built for sm_100a only", prop.major, prop.minor);

    mlxs_moe* h = new (std::nothrow) mlxs_moe();
    if (!h) return fail(MLXS_E_ARG, "create: out of host memory");
    h->cfg = *c;
    h->sm_count = prop.multiProcessorCount;
    h->e_local = c->n_experts / c->ep_world;
    h->e_first = c->ep_rank * h->e_local;
    const uint64_t H = c->hidden, I = c->inter;
    h->logical_bytes = is_exl3(c->bank_kind)               ? exl3_logical(H, I, exl3_bits(c->bank_kind))
                       : c->bank_kind == MLXS_BANK_MXFP4      ? mxfp4_logical(H, I)
                                                              : nvfp4_logical(H, I);
    h->record_stride = (h->logical_bytes + 4095) / 4096 * 4096;
    h->layers.resize(c->n_layers);
    int rc = 0;
    auto bail = [&](int r) { mlxs_moe_destroy(h); return r; };
    const Exl3Dims d{c->hidden, c->inter, exl3_bits(c->bank_kind)};
    for (auto& L : h->layers) {
        L.loaded.assign(c->n_experts, 0);
        if ((rc = h->alloc(&L.loaded_dev, c->n_experts)) || (rc = h->alloc(&L.place_dev, (size_t)c->n_experts * 4))) return bail(rc);
        if (cudaMemset(L.loaded_dev, 0, c->n_experts) != cudaSuccess) return bail(fail(MLXS_E_CUDA, "create: cudaMemset failed"));
        L.place_rank.resize(c->n_experts);
        L.place_slot.resize(c->n_experts);
        std::vector<uint32_t> packed(c->n_experts);
        for (uint32_t e = 0; e < c->n_experts; ++e) {
            L.place_rank[e] = (uint16_t)(e / h->e_local);
            L.place_slot[e] = (uint16_t)(e % h->e_local);
            packed[e] = ((uint32_t)L.place_rank[e] << 16) | L.place_slot[e];
        }
        if (cudaMemcpy(L.place_dev, packed.data(), packed.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess)
            return bail(fail(MLXS_E_CUDA, "create: cudaMemcpy of the placement table failed"));
        L.logical_bytes = h->logical_bytes;
        L.record_stride = h->record_stride;
        if (is_exl3(c->bank_kind)) {
            L.kbits = d.K;
            if ((rc = h->alloc(&L.gu_code, (size_t)h->e_local * 2 * exl3_code_words(d) * 4))) return bail(rc);
            if ((rc = h->alloc(&L.d_code, (size_t)h->e_local * exl3_code_words(d) * 4))) return bail(rc);
            if ((rc = h->alloc(&L.scales, (size_t)h->e_local * exl3_scales_per_expert(d) * 2))) return bail(rc);
        } else {
            const int nv = c->bank_kind == MLXS_BANK_NVFP4;
            if ((rc = h->alloc(&L.f4_gu, (size_t)h->e_local * fp4_stream_bytes_per_expert(c->hidden, c->inter, nv, 0)))) return bail(rc);
            if ((rc = h->alloc(&L.f4_dn, (size_t)h->e_local * fp4_stream_bytes_per_expert(c->hidden, c->inter, nv, 1)))) return bail(rc);
            if ((rc = h->alloc(&L.f4_gscale, (size_t)h->e_local * 3 * 4))) return bail(rc);
        }
    }
    const size_t T = c->max_tokens, A_call = T * c->top_k;
    // with expert parallelism a rank may receive more rows than it routes: workspaces hold up to 4 x (or world x) its own
    const size_t A = c->ep_world == 1 ? A_call : A_call * (c->ep_world < 4 ? c->ep_world : 4);
    h->rows_cap = (uint32_t)A;
    if (!is_exl3(c->bank_kind)) { h->chunk_rows = FP4_CHUNK_ROWS; h->group_chunks = FP4_GROUP_CHUNKS; }
    const uint32_t max_chunks = (uint32_t)(A / h->chunk_rows + (A < c->n_experts ? A : c->n_experts) + 1);
    h->tabs.max_chunks = max_chunks;
    if ((rc = h->alloc(&h->ids_ws, A * 4)) || (rc = h->alloc(&h->w_ws, A * 4)) || (rc = h->alloc(&h->tabs.header, 64)) ||
        (rc = h->alloc(&h->tabs.offsets, (c->n_experts + 1) * 4)) || (rc = h->alloc(&h->tabs.order, A * 4)) ||
        (rc = h->alloc(&h->tabs.chunk_expert, max_chunks * 4)) || (rc = h->alloc(&h->tabs.chunk_row0, max_chunks * 4)) ||
        (rc = h->alloc(&h->tabs.chunk_rows, max_chunks * 4)) || (rc = h->alloc(&h->tabs.group_chunk0, max_chunks * 4)) ||
        (rc = h->alloc(&h->tabs.group_mc, max_chunks * 4)) || (rc = h->alloc(&h->status, 16)) ||
        (rc = h->alloc(&h->front_bar, 16)) ||
        (rc = h->alloc(&h->blk_cnt, (A / 1024 + 1) * (size_t)c->n_experts * 4)) ||
        (rc = h->alloc(&h->staging, is_exl3(c->bank_kind) ? exl3_logical(H, I, 3) : h->logical_bytes)) ||
        (rc = h->alloc(&h->x_io, T * H * 2)) ||
        (rc = h->alloc(&h->y_io, T * H * 2)) || (rc = h->alloc(&h->logits_io, T * c->n_experts * 4)))
        return bail(rc);
    if (cudaMemset(h->status, 0, 16) != cudaSuccess || cudaMemset(h->tabs.header, 0, 64) != cudaSuccess ||
        cudaMemset(h->front_bar, 0, 16) != cudaSuccess)
        return bail(fail(MLXS_E_CUDA, "create: cudaMemset failed"));
    if (is_exl3(c->bank_kind)) {
        const size_t kmax = (H > I ? H : I) / 16;
        if ((rc = h->alloc(&h->xa_gu, (size_t)max_chunks * 2 * kmax * 256)) ||
            (rc = h->alloc(&h->xa_d, (size_t)max_chunks * kmax * 256)) || (rc = h->alloc(&h->ro, A * (H > I ? H : I) * 4)))
            return bail(rc);
        if ((rc = h->alloc(&h->ks_scratch, exl3_ksplit_scratch_bytes(h->sm_count))) || (rc = h->alloc(&h->ks_count, ksplit_count_words(h->sm_count) * 4)))
            return bail(rc);
        if (cudaMemset(h->ks_count, 0, ksplit_count_words(h->sm_count) * 4) != cudaSuccess) return bail(fail(MLXS_E_CUDA, "create: cudaMemset failed"));
    } else {
        if ((rc = h->alloc(&h->xa_gu, (size_t)max_chunks * (H / 32) * 512)) ||
            (rc = h->alloc(&h->xa_d, (size_t)max_chunks * (I / 32) * 512)) || (rc = h->alloc(&h->ro, A * H * 4)))
            return bail(rc);
        if ((rc = h->alloc(&h->ks_scratch, exl3_ksplit_scratch_bytes(h->sm_count))) || (rc = h->alloc(&h->ks_count, ksplit_count_words(h->sm_count) * 4)))
            return bail(rc);
        if (cudaMemset(h->ks_count, 0, ksplit_count_words(h->sm_count) * 4) != cudaSuccess) return bail(fail(MLXS_E_CUDA, "create: cudaMemset failed"));
    }
    {
        // Staging for the tensor-core lane.  One decode pass of the streaming lane serves 16 rows, one of the
        // tensor-core lane up to 192; the two lanes run side by side, so the row count from which an expert takes the
        // tensor-core lane is the one that evens them out.
        const bool exl3 = is_exl3(c->bank_kind);
        if (const char* nv = getenv("MLXS_MXFP4_NATIVE")) h->mxfp4_native = atoi(nv) != 0;
        // measured (24-layer Zipf stack at 64 tokens, EXL3: 9 rows 14.20, 13 rows 14.28, 17 rows 14.79, 21 rows 15.42 ms;
        // FP4 banks are within 1.5 % either way between 13 and 17)
        const char* ev = getenv("MLXS_PREFILL_MIN_ROWS");
        const int min_rows = ev ? atoi(ev) : (exl3 ? 13 : 17);
        const bool supported = exl3 ? exl3_prefill_supported(d) : fp4_prefill_supported(c->hidden, c->inter);
        if (min_rows > 0 && A >= (size_t)min_rows && supported) {
            h->pf_min_rows = (uint32_t)min_rows;
            const size_t heavy_max = A / (size_t)min_rows < h->e_local ? A / (size_t)min_rows : h->e_local;
            h->pf_max_tiles = (uint32_t)(A / PREFILL_TILE_ROWS + heavy_max + 1);
            size_t xa_bytes = exl3 ? exl3_prefill_xa_bytes(d, A, h->pf_max_tiles) : fp4_prefill_xa_bytes(c->hidden, A, h->pf_max_tiles);
            size_t xd_bytes = exl3 ? exl3_prefill_xd_bytes(d, A, h->pf_max_tiles) : fp4_prefill_xa_bytes(c->inter, A, h->pf_max_tiles);
            if (c->bank_kind == MLXS_BANK_MXFP4) {   // the block-scaled lane stages 132 bytes per row per 64 inputs
                xa_bytes = std::max(xa_bytes, mxfp4_native_xa_bytes(c->hidden, A, h->pf_max_tiles));
                xd_bytes = std::max(xd_bytes, mxfp4_native_xa_bytes(c->inter, A, h->pf_max_tiles));
            }
            if ((rc = h->alloc(&h->pf_tiles, prefill_tile_words(h->pf_max_tiles) * 4)) || (rc = h->alloc(&h->pf_xa, xa_bytes)) ||
                (rc = h->alloc(&h->pf_xd, xd_bytes)))
                return bail(rc);
        }
    }
    if (c->shared_expert) {
        if ((rc = h->alloc(&h->sh_h, T * I * 2)) || (rc = h->alloc(&h->sh_out, T * H * 4))) return bail(rc);
        const size_t T16 = (T + 15) / 16 * 16;
        if ((rc = h->alloc(&h->dg_hb, T16 * I * 2))) return bail(rc);
    }
    if (c->shared_expert || h->pf_tiles) {
        if (cudaStreamCreateWithFlags(&h->aux_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&h->aux_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&h->aux_join, cudaEventDisableTiming) != cudaSuccess ||
            cudaStreamCreateWithFlags(&h->lane_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&h->lane_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&h->lane_join, cudaEventDisableTiming) != cudaSuccess ||
            cudaStreamCreateWithFlags(&h->lane2_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&h->lane2_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&h->lane2_join, cudaEventDisableTiming) != cudaSuccess)
            return bail(fail(MLXS_E_CUDA, "create: second stream"));
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return bail(fail(MLXS_E_CUDA, "create: device synchronize failed"));
    *out = h;
    return MLXS_OK;
}

extern "C" void mlxs_moe_destroy(mlxs_moe* h) {
    if (!h) return;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    mlxs_ep_destroy(h);
    if (h->lane_fork) cudaEventDestroy(h->lane_fork);
    if (h->lane_join) cudaEventDestroy(h->lane_join);
    if (h->lane2_fork) cudaEventDestroy(h->lane2_fork);
    if (h->lane2_join) cudaEventDestroy(h->lane2_join);
    if (h->lane2_stream) cudaStreamDestroy(h->lane2_stream);
    if (h->aux_fork) cudaEventDestroy(h->aux_fork);
    if (h->aux_join) cudaEventDestroy(h->aux_join);
    if (h->aux_stream) cudaStreamDestroy(h->aux_stream);
    if (h->lane_stream) cudaStreamDestroy(h->lane_stream);
    for (void* p : h->allocs) cudaFree(p);
    for (auto& s : h->spans) { cudaEventDestroy(s.a); cudaEventDestroy(s.b); }
    for (auto e : h->ev_pool) cudaEventDestroy(e);
    delete h;
}

extern "C" int mlxs_moe_record_bytes(const mlxs_moe* h, uint64_t* logical_bytes, uint64_t* record_stride) {
    if (!h) return fail(MLXS_E_ARG, "record_bytes: null handle");
    if (logical_bytes) *logical_bytes = h->logical_bytes;
    if (record_stride) *record_stride = h->record_stride;
    return MLXS_OK;
}

extern "C" int mlxs_moe_layer_record_bytes(const mlxs_moe* h, uint32_t layer, uint32_t* bits, uint64_t* logical_bytes,
                                           uint64_t* record_stride) {
    if (!h) return fail(MLXS_E_ARG, "layer_record_bytes: null handle");
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "layer_record_bytes: layer %u of %u", layer, h->cfg.n_layers);
    const LayerBank& L = h->layers[layer];
    if (bits) *bits = is_exl3(h->cfg.bank_kind) ? L.kbits : 4u;
    if (logical_bytes) *logical_bytes = L.logical_bytes;
    if (record_stride) *record_stride = L.record_stride;
    return MLXS_OK;
}

extern "C" int mlxs_moe_set_layer_bits(mlxs_moe* h, uint32_t layer, uint32_t bits) {
    if (!h) return fail(MLXS_E_ARG, "set_layer_bits: null handle");
    const mlxs_moe_config& c = h->cfg;
    if (layer >= c.n_layers) return fail(MLXS_E_ARG, "set_layer_bits: layer %u of %u", layer, c.n_layers);
    if (!is_exl3(c.bank_kind)) return fail(MLXS_E_CONFIG, "set_layer_bits: the handle's bank is not EXL3");
    if (bits != 2 && bits != 3) return fail(MLXS_E_CONFIG, "set_layer_bits: K=%u not implemented by the installed lanes (KNotImplemented)", bits);
    LayerBank& L = h->layers[layer];
    if (L.kbits == bits) return MLXS_OK;
    for (uint32_t e = 0; e < c.n_experts; ++e)
        if (L.loaded[e]) return fail(MLXS_E_CONFIG, "set_layer_bits: layer %u already holds experts; set the width before loading", layer);
    CU(cudaSetDevice(c.device));
    CU(cudaDeviceSynchronize());
    const Exl3Dims was{c.hidden, c.inter, L.kbits}, now{c.hidden, c.inter, bits};
    h->release(&L.gu_code, (size_t)h->e_local * 2 * exl3_code_words(was) * 4);
    h->release(&L.d_code, (size_t)h->e_local * exl3_code_words(was) * 4);
    int rc;
    if ((rc = h->alloc(&L.gu_code, (size_t)h->e_local * 2 * exl3_code_words(now) * 4)) ||
        (rc = h->alloc(&L.d_code, (size_t)h->e_local * exl3_code_words(now) * 4)))
        return rc;
    L.kbits = bits;
    L.logical_bytes = exl3_logical(c.hidden, c.inter, bits);
    L.record_stride = (L.logical_bytes + 4095) / 4096 * 4096;
    return MLXS_OK;
}

extern "C" int mlxs_moe_load_expert(mlxs_moe* h, uint32_t layer, uint32_t expert, const void* record, uint64_t nbytes,
                                    int on_device) {
    if (!h || !record) return fail(MLXS_E_ARG, "load_expert: null argument");
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "load_expert: layer %u of %u", layer, h->cfg.n_layers);
    if (expert >= h->cfg.n_experts) return fail(MLXS_E_ARG, "load_expert: expert %u of %u", expert, h->cfg.n_experts);
    LayerBank& L = h->layers[layer];
    if (nbytes < L.logical_bytes)
        return fail(MLXS_E_BANK, "load_expert: record has %llu bytes, the layer's record is %llu (RecordGeometry)",
                    (unsigned long long)nbytes, (unsigned long long)L.logical_bytes);
    if (L.place_rank[expert] != h->cfg.ep_rank) return MLXS_OK;  // another rank's shard
    CU(cudaSetDevice(h->cfg.device));
    const uint32_t le = L.place_slot[expert];
    const uint8_t* src = static_cast<const uint8_t*>(record);
    if (!on_device) {
        CU(cudaMemcpyAsync(h->staging, record, L.logical_bytes, cudaMemcpyHostToDevice, 0));
        src = h->staging;
    }
    // the expert's entry of the per-expert table: 1 = resident; the FP4 repack may raise it to 3 (see takes_tensor_lane)
    const uint8_t one = 1;
    CU(cudaMemcpyAsync(L.loaded_dev + le, &one, 1, cudaMemcpyHostToDevice, 0));
    if (is_exl3(h->cfg.bank_kind)) {
        const Exl3Dims d{h->cfg.hidden, h->cfg.inter, L.kbits};
        CU(launch_exl3_repack(src, d, L.gu_code + (size_t)le * 2 * exl3_code_words(d),
                              L.d_code + (size_t)le * exl3_code_words(d), L.scales + (size_t)le * exl3_scales_per_expert(d), 0));
    } else {
        const int nv = h->cfg.bank_kind == MLXS_BANK_NVFP4;
        CU(launch_fp4_repack(src, h->cfg.hidden, h->cfg.inter, nv,
                             L.f4_gu + (size_t)le * fp4_stream_bytes_per_expert(h->cfg.hidden, h->cfg.inter, nv, 0),
                             L.f4_dn + (size_t)le * fp4_stream_bytes_per_expert(h->cfg.hidden, h->cfg.inter, nv, 1),
                             L.f4_gscale + (size_t)le * 3, L.loaded_dev + le, 0));
    }
    CU(cudaStreamSynchronize(0));
    L.loaded[expert] = 1;
    return MLXS_OK;
}

// what a fused front launch needs beyond the experts call's own arguments (null: ids and weights are given)
struct FrontCall {
    const float* logits;   // the router's logits, or null when the layer starts from x (the layer's router weight)
};

// Can this call take the fused front kernel (front.cu)?  One rank, a decode-sized batch, no route tally to feed.  MLXS_FRONT_MAX moves the batch limit (0: never).
static bool front_applies(const mlxs_moe* h, uint32_t T) {
    static const uint32_t front_max = getenv("MLXS_FRONT_MAX") ? (uint32_t)atoi(getenv("MLXS_FRONT_MAX")) : 16u;
    if (T == 0 || T > front_max || h->cfg.ep_world != 1 || h->usage_on || h->front_off) return false;
    if (T * h->cfg.top_k > 2048) return false;
    return true;
}

static int experts_impl(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, const float* weights_dev,
                        uint32_t T, void* y_dev, void* stream, const FrontCall* front);

int mlxs_bank_for_each_record(const char* dir, uint32_t bank_kind, uint64_t H, uint64_t I, uint64_t E, uint64_t n_layers,
                              uint32_t e_first, uint32_t e_count, int (*layer_begin)(void* ctx, uint32_t layer, uint32_t bits),
                              int (*sink)(void* ctx, uint32_t layer, uint32_t expert, const void* rec, uint64_t n), void* ctx);

extern "C" int mlxs_moe_set_placement(mlxs_moe* h, uint32_t layer, const uint16_t* rank_of_expert) {
    if (!h || !rank_of_expert) return fail(MLXS_E_ARG, "set_placement: null argument");
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "set_placement: layer %u of %u", layer, h->cfg.n_layers);
    LayerBank& L = h->layers[layer];
    const uint32_t E = h->cfg.n_experts, W = h->cfg.ep_world;
    for (uint32_t e = 0; e < E; ++e)
        if (L.loaded[e]) return fail(MLXS_E_CONFIG, "set_placement: layer %u already holds experts; place before loading", layer);
    std::vector<uint32_t> fill(W, 0), packed(E);
    for (uint32_t e = 0; e < E; ++e) {
        const uint32_t r = rank_of_expert[e];
        if (r >= W) return fail(MLXS_E_CONFIG, "set_placement: expert %u on rank %u of %u", e, r, W);
        if (fill[r] >= h->e_local)
            return fail(MLXS_E_CONFIG, "set_placement: rank %u would hold more than %u experts (every rank holds n_experts / ep_world)", r, h->e_local);
        packed[e] = (r << 16) | fill[r]++;
    }
    CU(cudaSetDevice(h->cfg.device));
    CU(cudaMemcpy(L.place_dev, packed.data(), (size_t)E * 4, cudaMemcpyHostToDevice));
    for (uint32_t e = 0; e < E; ++e) { L.place_rank[e] = (uint16_t)(packed[e] >> 16); L.place_slot[e] = (uint16_t)(packed[e] & 0xFFFFu); }
    L.placement_custom = true;
    return MLXS_OK;
}

extern "C" int mlxs_moe_load_bank(mlxs_moe* h, const char* dir) {
    if (!h || !dir) return fail(MLXS_E_ARG, "load_bank: null argument");
    const mlxs_moe_config& c = h->cfg;
    auto sink = [](void* ctx, uint32_t layer, uint32_t expert, const void* rec, uint64_t n) -> int {
        return mlxs_moe_load_expert(static_cast<mlxs_moe*>(ctx), layer, expert, rec, n, 0);
    };
    auto layer_begin = [](void* ctx, uint32_t layer, uint32_t bits) -> int {
        return mlxs_moe_set_layer_bits(static_cast<mlxs_moe*>(ctx), layer, bits);
    };
    // with the default placement only this rank's block of records is read; a custom placement scatters a rank's experts
    // over the file, so every record is visited and load_expert keeps the local ones
    bool custom = false;
    for (const LayerBank& L : h->layers) custom = custom || L.placement_custom;
    return mlxs_bank_for_each_record(dir, c.bank_kind, c.hidden, c.inter, c.n_experts, c.n_layers, custom ? 0 : h->e_first,
                                     custom ? c.n_experts : h->e_local, layer_begin, sink, h);
}

extern "C" int mlxs_moe_set_router_bias(mlxs_moe* h, uint32_t layer, const float* bias_host) {
    if (!h) return fail(MLXS_E_ARG, "set_router_bias: null handle");
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "set_router_bias: layer %u of %u", layer, h->cfg.n_layers);
    CU(cudaSetDevice(h->cfg.device));
    LayerBank& L = h->layers[layer];
    if (!bias_host) { L.bias = nullptr; return MLXS_OK; }
    if (!L.bias) { int rc = h->alloc(&L.bias, h->cfg.n_experts * 4); if (rc) return rc; }
    CU(cudaMemcpy(L.bias, bias_host, h->cfg.n_experts * 4, cudaMemcpyHostToDevice));
    return MLXS_OK;
}

// batches of this many tokens or more take the tcgen05 form of the shared expert (dense_gemm.cu), smaller ones the
// skinny streaming kernel (MLXS_SHARED_DENSE_MIN moves the limit)
static uint32_t shared_dense_min() {
    static const uint32_t v = getenv("MLXS_SHARED_DENSE_MIN") ? (uint32_t)atoi(getenv("MLXS_SHARED_DENSE_MIN")) : 65u;
    return v;
}
// scratch of the dense tensor-core products, allocated with the first weights that need them
static int dense_workspace(mlxs_moe* h) {
    int rc;
    const size_t T16 = ((size_t)h->cfg.max_tokens + 15) / 16 * 16;
    if (!h->dg_xb && (rc = h->alloc(&h->dg_xb, T16 * h->cfg.hidden * 2))) return rc;
    if (!h->dg_scratch) {
        if ((rc = h->alloc(&h->dg_scratch, dense_gemm_scratch_bytes(h->sm_count))) || (rc = h->alloc(&h->dg_count, (size_t)h->sm_count * 4))) return rc;
        CU(cudaMemset(h->dg_count, 0, (size_t)h->sm_count * 4));
    }
    return 0;
}

extern "C" int mlxs_moe_set_shared(mlxs_moe* h, uint32_t layer, const void* w1, const void* w3, const void* w2, int on_device) {
    if (!h || !w1 || !w3 || !w2) return fail(MLXS_E_ARG, "set_shared: null argument");
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "set_shared: layer %u of %u", layer, h->cfg.n_layers);
    if (!h->cfg.shared_expert) return fail(MLXS_E_CONFIG, "set_shared: the handle was created without a shared expert");
    CU(cudaSetDevice(h->cfg.device));
    LayerBank& L = h->layers[layer];
    const size_t n = (size_t)h->cfg.hidden * h->cfg.inter * 2;
    int rc;
    if (!L.sh_w1 && ((rc = h->alloc(&L.sh_w1, n)) || (rc = h->alloc(&L.sh_w3, n)) || (rc = h->alloc(&L.sh_w2, n)))) return rc;
    const cudaMemcpyKind k = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    CU(cudaMemcpy(L.sh_w1, w1, n, k));
    CU(cudaMemcpy(L.sh_w3, w3, n, k));
    CU(cudaMemcpy(L.sh_w2, w2, n, k));
    // the tensor-core form of the same weights, when the handle can see batches that take it
    if (h->cfg.max_tokens < shared_dense_min() || !dense_gemm_supported(h->cfg.inter, h->cfg.hidden, 0) ||
        !dense_gemm_supported(h->cfg.hidden, h->cfg.inter, 1))
        return MLXS_OK;
    if ((rc = dense_workspace(h))) return rc;
    if (!L.sh_gu_t && ((rc = h->alloc(&L.sh_gu_t, 2 * n)) || (rc = h->alloc(&L.sh_d_t, n)))) return rc;
    CU(launch_dense_retile(L.sh_w1, L.sh_w3, h->cfg.inter, h->cfg.hidden, L.sh_gu_t, 0));
    CU(launch_dense_retile(L.sh_w2, nullptr, h->cfg.hidden, h->cfg.inter, L.sh_d_t, 0));
    CU(cudaStreamSynchronize(0));
    return MLXS_OK;
}

static int check_call(mlxs_moe* h, uint32_t layer, uint32_t T, const char* who) {
    if (!h) return fail(MLXS_E_ARG, "%s: null handle", who);
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "%s: layer %u of %u", who, layer, h->cfg.n_layers);
    if (T > h->cfg.max_tokens) return fail(MLXS_E_TOO_MANY_TOKENS, "%s: %u tokens, the handle was created for %u", who, T, h->cfg.max_tokens);
    cudaError_t e = cudaSetDevice(h->cfg.device);
    if (e != cudaSuccess) return fail(MLXS_E_CUDA, "%s: cudaSetDevice: %s", who, cudaGetErrorString(e));
    return 0;
}

// Rows are read and written as 16-byte vectors, ids / weights / logits as 4-byte words: a misaligned base pointer would
// fault on the device, so it is refused by name here.
static int check_aligned(const void* p, uintptr_t align, const char* who, const char* what) {
    if (reinterpret_cast<uintptr_t>(p) & (align - 1))
        return fail(MLXS_E_ARG, "%s: %s must be %u-byte aligned", who, what, (unsigned)align);
    return 0;
}

// Joins the handle's side streams back into the caller's stream on every way out of a layer call (also the refusals
// after a fork): the caller's stream then always orders after the side work, and a stream capture never ends with an
// unjoined fork.
struct ForkGuard {
    cudaStream_t st;
    cudaStream_t side = nullptr;
    cudaEvent_t join = nullptr;
    bool armed = false;
    explicit ForkGuard(cudaStream_t s) : st(s) {}
    void arm(cudaStream_t side_, cudaEvent_t join_) { side = side_; join = join_; armed = true; }
    // the normal path: the side stream's work is recorded here, the wait may come later (wait_now) or at scope exit
    cudaError_t record() { return cudaEventRecord(join, side); }
    cudaError_t wait_now() { armed = false; return cudaStreamWaitEvent(st, join, 0); }
    ~ForkGuard() {
        if (!armed) return;
        cudaEventRecord(join, side);
        cudaStreamWaitEvent(st, join, 0);
    }
};

extern "C" int mlxs_moe_route(mlxs_moe* h, uint32_t layer, const float* logits_dev, uint32_t T, int32_t* ids_dev,
                              float* weights_dev, void* stream) {
    int rc = check_call(h, layer, T, "route");
    if (rc) return rc;
    if (T && (!logits_dev || !ids_dev || !weights_dev)) return fail(MLXS_E_ARG, "route: null buffer");
    if ((rc = check_aligned(logits_dev, 4, "route", "logits_dev")) || (rc = check_aligned(ids_dev, 4, "route", "ids_dev")) ||
        (rc = check_aligned(weights_dev, 4, "route", "weights_dev")))
        return rc;
    const mlxs_moe_config& c = h->cfg;
    StageTimer tm(h, MLXS_STAGE_ROUTER, (cudaStream_t)stream);
    CU(launch_router(logits_dev, h->layers[layer].bias, (int)T, (int)c.n_experts, (int)c.top_k, (int)c.scoring,
                     (int)c.norm_topk, c.routed_scale, ids_dev, weights_dev, (cudaStream_t)stream));
    h->stats.route_calls += 1;
    if (h->usage_on && T)
        CU(launch_usage_count(ids_dev, (uint64_t)T * c.top_k, c.n_experts, h->layers[layer].usage, (cudaStream_t)stream));
    return MLXS_OK;
}

extern "C" int mlxs_moe_usage_enable(mlxs_moe* h, int on) {
    if (!h) return fail(MLXS_E_ARG, "usage_enable: null handle");
    CU(cudaSetDevice(h->cfg.device));
    if (on)
        for (LayerBank& L : h->layers)
            if (!L.usage) {
                int rc = h->alloc(&L.usage, (size_t)h->cfg.n_experts * 8);
                if (rc) return rc;
                CU(cudaMemset(L.usage, 0, (size_t)h->cfg.n_experts * 8));
            }
    h->usage_on = on != 0;
    return MLXS_OK;
}

extern "C" int mlxs_moe_usage_add(mlxs_moe* h, uint32_t layer, const void* ids_dev, uint64_t n_ids, void* stream) {
    if (!h || (n_ids && !ids_dev)) return fail(MLXS_E_ARG, "usage_add: null argument");
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "usage_add: layer %u of %u", layer, h->cfg.n_layers);
    if (!h->layers[layer].usage) return fail(MLXS_E_CONFIG, "usage_add: the tally is off (mlxs_moe_usage_enable)");
    CU(cudaSetDevice(h->cfg.device));
    CU(launch_usage_count(static_cast<const int32_t*>(ids_dev), n_ids, h->cfg.n_experts, h->layers[layer].usage, (cudaStream_t)stream));
    return MLXS_OK;
}

extern "C" int mlxs_moe_usage_read(mlxs_moe* h, uint32_t layer, uint64_t* counts_host, int all_ranks) {
    if (!h || !counts_host) return fail(MLXS_E_ARG, "usage_read: null argument");
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "usage_read: layer %u of %u", layer, h->cfg.n_layers);
    LayerBank& L = h->layers[layer];
    if (!L.usage) return fail(MLXS_E_CONFIG, "usage_read: the tally is off (mlxs_moe_usage_enable)");
    CU(cudaSetDevice(h->cfg.device));
    CU(cudaDeviceSynchronize());
    const size_t n = h->cfg.n_experts;
    if (all_ranks && h->cfg.ep_world > 1) {
        // the sum goes through a scratch copy, so this rank's own counts keep counting from where they were
        unsigned long long* tmp = nullptr;
        CU(cudaMalloc(&tmp, n * 8));
        cudaMemcpy(tmp, L.usage, n * 8, cudaMemcpyDeviceToDevice);
        int rc = mlxs_ep_allreduce_u64(h, tmp, n, 0);
        cudaError_t ce = cudaStreamSynchronize(0);
        if (!rc && ce == cudaSuccess) ce = cudaMemcpy(counts_host, tmp, n * 8, cudaMemcpyDeviceToHost);
        cudaFree(tmp);
        if (rc) return rc;
        CU(ce);
        return MLXS_OK;
    }
    CU(cudaMemcpy(counts_host, L.usage, n * 8, cudaMemcpyDeviceToHost));
    return MLXS_OK;
}

extern "C" int mlxs_moe_usage_reset(mlxs_moe* h) {
    if (!h) return fail(MLXS_E_ARG, "usage_reset: null handle");
    CU(cudaSetDevice(h->cfg.device));
    CU(cudaDeviceSynchronize());
    for (LayerBank& L : h->layers)
        if (L.usage) CU(cudaMemset(L.usage, 0, (size_t)h->cfg.n_experts * 8));
    return MLXS_OK;
}

extern "C" int mlxs_moe_plan_placement(const uint64_t* counts, uint32_t n_experts, uint32_t world, uint16_t* rank_of_expert) {
    if (!counts || !rank_of_expert) return fail(MLXS_E_ARG, "plan_placement: null argument");
    if (world == 0 || n_experts == 0 || n_experts % world || world > 65535)
        return fail(MLXS_E_CONFIG, "plan_placement: %u ranks do not shard %u experts", world, n_experts);
    std::vector<uint32_t> order(n_experts);
    for (uint32_t e = 0; e < n_experts; ++e) order[e] = e;
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return counts[a] > counts[b]; });
    // snake deal: ranks 0..W-1, then W-1..0, ...: each rank takes one expert of every band of W, alternating ends
    for (uint32_t i = 0; i < n_experts; ++i) {
        const uint32_t band = i / world, pos = i % world;
        rank_of_expert[order[i]] = (uint16_t)((band & 1u) ? world - 1 - pos : pos);
    }
    return MLXS_OK;
}

extern "C" int mlxs_moe_set_router_weight(mlxs_moe* h, uint32_t layer, const void* w_gate_bf16, int on_device) {
    if (!h || !w_gate_bf16) return fail(MLXS_E_ARG, "set_router_weight: null argument");
    if (layer >= h->cfg.n_layers) return fail(MLXS_E_ARG, "set_router_weight: layer %u of %u", layer, h->cfg.n_layers);
    CU(cudaSetDevice(h->cfg.device));
    LayerBank& L = h->layers[layer];
    const size_t n = (size_t)h->cfg.n_experts * h->cfg.hidden * 2;
    int rc;
    if (!L.router_w && (rc = h->alloc(&L.router_w, n))) return rc;
    if (!h->logits_ws && (rc = h->alloc(&h->logits_ws, (size_t)h->cfg.max_tokens * h->cfg.n_experts * 4))) return rc;
    CU(cudaMemcpy(L.router_w, w_gate_bf16, n, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    if (h->cfg.max_tokens > 64 && dense_gemm_supported(h->cfg.n_experts, h->cfg.hidden, 1)) {
        if ((rc = dense_workspace(h))) return rc;
        if (!L.router_w_t && (rc = h->alloc(&L.router_w_t, n))) return rc;
        CU(launch_dense_retile(L.router_w, nullptr, h->cfg.n_experts, h->cfg.hidden, L.router_w_t, 0));
        CU(cudaStreamSynchronize(0));
    }
    return MLXS_OK;
}

extern "C" int mlxs_moe_logits(mlxs_moe* h, uint32_t layer, const void* x_dev, uint32_t T, float* logits_dev, void* stream) {
    int rc = check_call(h, layer, T, "logits");
    if (rc) return rc;
    if (T == 0) return MLXS_OK;
    if (!x_dev || !logits_dev) return fail(MLXS_E_ARG, "logits: null buffer");
    const mlxs_moe_config& c = h->cfg;
    LayerBank& L = h->layers[layer];
    if (!L.router_w) return fail(MLXS_E_NOT_LOADED, "logits: layer %u has no router weight (mlxs_moe_set_router_weight)", layer);
    cudaStream_t st = (cudaStream_t)stream;
    StageTimer tm(h, MLXS_STAGE_ROUTER, st);
    if (T > 64 && L.router_w_t) {
        CU(launch_dense_logits(static_cast<const __nv_bfloat16*>(x_dev), L.router_w_t, T, c.n_experts, c.hidden, h->dg_xb, logits_dev,
                               h->dg_scratch, h->dg_count, h->status, h->sm_count, st));
    } else {
        CU(launch_router_logits(static_cast<const __nv_bfloat16*>(x_dev), L.router_w, T, c.n_experts, c.hidden, logits_dev, st));
    }
    return MLXS_OK;
}

extern "C" int mlxs_moe_forward_x(mlxs_moe* h, uint32_t layer, const void* x_dev, uint32_t T, void* y_dev, void* stream) {
    if (!h) return fail(MLXS_E_ARG, "forward_x: null handle");
    if (!h->logits_ws) return fail(MLXS_E_NOT_LOADED, "forward_x: no router weight was set (mlxs_moe_set_router_weight)");
    if (layer < h->cfg.n_layers && front_applies(h, T)) {
        // decode-sized: the logits product is the first phase of the fused front kernel (no [T, E] round trip, no launch)
        if (!h->layers[layer].router_w) return fail(MLXS_E_NOT_LOADED, "forward_x: layer %u has no router weight (mlxs_moe_set_router_weight)", layer);
        const FrontCall fc{nullptr};
        return experts_impl(h, layer, x_dev, h->ids_ws, h->w_ws, T, y_dev, stream, &fc);
    }
    int rc = mlxs_moe_logits(h, layer, x_dev, T, h->logits_ws, stream);
    if (rc) return rc;
    return mlxs_moe_forward(h, layer, x_dev, h->logits_ws, T, y_dev, stream);
}

// dispatch + the bank's expert kernels -> ro (unweighted rows in assignment order)
int mlxs_run_routed(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, uint32_t T, uint32_t top_k,
                    uint32_t n_exp, uint32_t first, void* ro, int ro_bf16, cudaStream_t st, const uint32_t* n_rows_dev) {
    const mlxs_moe_config& c = h->cfg;
    LayerBank& L = h->layers[layer];
    const uint32_t A = T * top_k;
    if (A > h->rows_cap) return fail(MLXS_E_TOO_MANY_TOKENS, "experts: %u rows exceed the workspace's %u", A, h->rows_cap);
    // Lane choice per expert by its row count, as the reference decides on logical M (src/sdk_ext/quant.zig:5-6,
    // src/arch/deepseek_v41/experts.zig:1545-1547): experts with `heavy` rows or more go to the tensor-core lane, which
    // amortises one decode over up to 128 rows; the others stream through the decode-batch lane.
    // a token's experts are distinct, so no expert has more rows than the call has tokens
    const bool two_lanes = h->pf_tiles && T >= h->pf_min_rows;
    const uint32_t heavy = two_lanes ? h->pf_min_rows : 0u;
    h->last_logical = L.logical_bytes;
    const bool front_done = h->front_done;   // the fused front kernel has sorted the rows and staged them already
    h->front_done = false;
    if (!front_done) {
        StageTimer tm(h, MLXS_STAGE_DISPATCH, st);
        if (A > 2048)
            CU(launch_dispatch_large(ids_dev, A, n_exp, L.loaded_dev + first, h->tabs, h->chunk_rows, h->group_chunks, heavy,
                                     h->blk_cnt, h->status, st, n_rows_dev));
        else
            CU(launch_dispatch(ids_dev, A, n_exp, L.loaded_dev + first, h->tabs, h->chunk_rows, h->group_chunks, heavy,
                               h->status, st, n_rows_dev));
    }
    // The two lanes serve disjoint experts from separate staging buffers: the tensor-core lane (tile plan, row prep and
    // its two kernels) is queued on a stream of its own beside the streaming lane, forked after the dispatch
    // and joined before the rows are read.  Its launches, most of all the ones that find no heavy expert and return at
    // once, then cost the step nothing, and the lanes' tails overlap.
    // Prefill-sized calls (nearly every expert in the tensor-core lane, nothing to overlap) keep one stream: with two,
    // C4 at 16384 tokens went from 13.0 to 14.4 ms.  MLXS_LANES_ASIDE_MAX moves the limit (0: always one stream).
    static const uint32_t lanes_aside_max = getenv("MLXS_LANES_ASIDE_MAX") ? (uint32_t)atoi(getenv("MLXS_LANES_ASIDE_MAX")) : 2048u;
    const bool lane_aside = two_lanes && h->lane_stream && T <= lanes_aside_max;
    const cudaStream_t tl = lane_aside ? h->lane_stream : st;
    ForkGuard lane_guard(st);
    if (lane_aside) {
        CU(cudaEventRecord(h->lane_fork, st));
        CU(cudaStreamWaitEvent(h->lane_stream, h->lane_fork, 0));
        lane_guard.arm(h->lane_stream, h->lane_join);
    }
    const float limit = c.act == MLXS_ACT_SWIGLU_CLAMPED ? c.act_limit : 0.f;
    if (is_exl3(c.bank_kind)) {
        const Exl3Dims d{c.hidden, c.inter, L.kbits};
        Exl3Layer EL{L.gu_code, L.d_code, L.scales};
        if (two_lanes) {
            Exl3PrefillArgs pa{};
            pa.L = EL; pa.d = d; pa.t = h->tabs; pa.n_experts = n_exp; pa.min_rows = heavy;
            pa.x = static_cast<const __nv_bfloat16*>(x_dev); pa.top_k = top_k; pa.tiles = h->pf_tiles; pa.max_tiles = h->pf_max_tiles;
            pa.xa = h->pf_xa; pa.xd = h->pf_xd; pa.rows_cap = h->rows_cap; pa.ro = static_cast<float*>(ro);
            pa.limit = limit; pa.status = h->status; pa.sm_count = h->sm_count;
            // side by side with the streaming lane: the large-tile kernels also beside the small-tile ones
            if (lane_aside) { pa.side = h->lane2_stream; pa.side_fork = h->lane2_fork; pa.side_join = h->lane2_join; }
            StageTimer tm(h, MLXS_STAGE_TENSOR_LANE, tl);
            CU(launch_exl3_prefill(pa, tl));
        }
        if (!front_done) {
            StageTimer tm(h, MLXS_STAGE_PREP, st);
            CU(launch_exl3_prep_in(static_cast<const __nv_bfloat16*>(x_dev), top_k, EL, d, h->tabs, h->xa_gu, st));
        }
        Exl3GemvArgs a{};
        a.L = EL; a.d = d; a.t = h->tabs; a.xa_gu = h->xa_gu; a.xa_d = h->xa_d; a.ro = static_cast<float*>(ro); a.ro_bf16 = 0;
        a.limit = limit;
        a.status = h->status; a.sm_count = h->sm_count; a.ks_scratch = h->ks_scratch; a.ks_count = h->ks_count;
        a.poll_limit = h->dbg_poll_limit; a.withhold = h->dbg_withhold;
        {
            StageTimer tm(h, MLXS_STAGE_GATE_UP, st);
            CU(launch_exl3_gate_up(a, st));
        }
        {
            StageTimer tm(h, MLXS_STAGE_DOWN, st);
            CU(launch_exl3_down(a, st));
        }
    } else {
        if (two_lanes) {
            Fp4PrefillArgs pa{};
            pa.gu = L.f4_gu; pa.dn = L.f4_dn; pa.nv = c.bank_kind == MLXS_BANK_NVFP4; pa.gscale = pa.nv ? L.f4_gscale : nullptr;
            pa.H = c.hidden; pa.I = c.inter; pa.t = h->tabs;
            pa.n_experts = n_exp; pa.lane_flags = L.loaded_dev + first; pa.min_rows = heavy;
            pa.x = static_cast<const __nv_bfloat16*>(x_dev); pa.top_k = top_k; pa.tiles = h->pf_tiles; pa.max_tiles = h->pf_max_tiles;
            pa.xa = reinterpret_cast<uint16_t*>(h->pf_xa); pa.xd = reinterpret_cast<uint16_t*>(h->pf_xd);
            pa.ro = ro; pa.ro_bf16 = ro_bf16; pa.limit = limit; pa.status = h->status; pa.sm_count = h->sm_count;
            if (lane_aside) { pa.side = h->lane2_stream; pa.side_fork = h->lane2_fork; pa.side_join = h->lane2_join; }
            StageTimer tm(h, MLXS_STAGE_TENSOR_LANE, tl);
            // MXFP4: the block-scaled tensor-core kind on the codes as stored, unless the handle was created with MLXS_MXFP4_NATIVE=0
            if (!pa.nv && h->mxfp4_native) CU(launch_mxfp4_native(pa, tl));
            else CU(launch_fp4_prefill(pa, tl));
        }
        if (!front_done) {
            StageTimer tm(h, MLXS_STAGE_PREP, st);
            CU(launch_fp4_prep(static_cast<const __nv_bfloat16*>(x_dev), top_k, c.hidden, h->tabs, h->xa_gu, st));
        }
        Fp4GemvArgs a{};
        a.gu = L.f4_gu; a.dn = L.f4_dn; a.nv = c.bank_kind == MLXS_BANK_NVFP4; a.gscale = a.nv ? L.f4_gscale : nullptr;
        a.H = c.hidden; a.I = c.inter; a.t = h->tabs; a.xa = h->xa_gu; a.xa_d = h->xa_d; a.ro = ro;
        a.ro_bf16 = ro_bf16; a.limit = limit;
        a.status = h->status; a.sm_count = h->sm_count; a.ks_scratch = h->ks_scratch; a.ks_count = h->ks_count;
        {
            StageTimer tm(h, MLXS_STAGE_GATE_UP, st);
            CU(launch_fp4_gemv(a, 0, st));
        }
        {
            StageTimer tm(h, MLXS_STAGE_DOWN, st);
            CU(launch_fp4_gemv(a, 1, st));
        }
    }
    if (lane_aside) {
        CU(lane_guard.record());
        CU(lane_guard.wait_now());
    }
    h->stats.expert_calls += 1;
    h->stats.assignments += A;
    return MLXS_OK;
}

// the routed rows of a call: local when the handle is one rank, through the exchange otherwise
static int run_routed(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, uint32_t T, void* ro,
                      int ro_bf16, cudaStream_t st) {
    h->stats.tokens += T;
    if (h->cfg.ep_world == 1)
        return mlxs_run_routed(h, layer, x_dev, ids_dev, T, h->cfg.top_k, h->cfg.n_experts, 0, ro, ro_bf16, st);
    return mlxs_ep_routed(h, layer, x_dev, ids_dev, T, ro, ro_bf16, st);
}

extern "C" int mlxs_moe_routed(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, uint32_t T,
                               float* out_dev, void* stream) {
    int rc = check_call(h, layer, T, "routed");
    if (rc) return rc;
    if (T == 0 && h->cfg.ep_world == 1) return MLXS_OK;  // with expert parallelism an empty rank still serves its peers
    if (T && (!x_dev || !ids_dev || !out_dev)) return fail(MLXS_E_ARG, "routed: null buffer");
    if ((rc = check_aligned(x_dev, 16, "routed", "x_dev")) || (rc = check_aligned(ids_dev, 4, "routed", "ids_dev")) ||
        (rc = check_aligned(out_dev, 16, "routed", "out_dev")))
        return rc;
    return run_routed(h, layer, x_dev, ids_dev, T, out_dev, 0, (cudaStream_t)stream);
}

static int experts_impl(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev, const float* weights_dev,
                        uint32_t T, void* y_dev, void* stream, const FrontCall* front) {
    int rc = check_call(h, layer, T, "experts");
    if (rc) return rc;
    if (T == 0 && h->cfg.ep_world == 1) return MLXS_OK;  // with expert parallelism an empty rank still serves its peers
    if (T && (!x_dev || !ids_dev || !weights_dev || !y_dev)) return fail(MLXS_E_ARG, "experts: null buffer");
    if ((rc = check_aligned(x_dev, 16, "experts", "x_dev")) || (rc = check_aligned(y_dev, 16, "experts", "y_dev")) ||
        (rc = check_aligned(ids_dev, 4, "experts", "ids_dev")) || (rc = check_aligned(weights_dev, 4, "experts", "weights_dev")))
        return rc;
    const mlxs_moe_config& c = h->cfg;
    LayerBank& L = h->layers[layer];
    cudaStream_t st = (cudaStream_t)stream;
    if (c.shared_expert && !L.sh_w1) return fail(MLXS_E_NOT_LOADED, "experts: layer %u has no shared expert weights", layer);
    // FP4 banks with the chain combine keep the routed rows in bf16, as the reference's down texts store them
    const int ro_bf16 = !is_exl3(c.bank_kind) && c.combine == MLXS_COMBINE_CHAIN;
    // expert parallel with the f32 combine: the exchange carries each token once per rank and brings weighted partial
    // rows back (ep.cu); the chain combine needs every assignment's row in k order and keeps the per-assignment form
    static const bool per_assignment = getenv("MLXS_EP_PER_ASSIGNMENT") != nullptr;
    const bool ep_fused = c.ep_world > 1 && c.combine != MLXS_COMBINE_CHAIN && !per_assignment;
    // The shared expert only reads x: it runs beside the routed kernels on the handle's second stream.  Decode-sized
    // batches leave SMs idle in the routed kernels (T = 1: 144 work items for 296 CTA slots); larger ones still have
    // the dispatch and the staging of the rows at their start, about as long as the shared expert itself.
    // Prefill-sized calls keep it on the caller's stream after the routed kernels: its library GEMMs are full-GPU
    // kernels, and running them among the tensor-core lane's persistent CTAs stretched that lane (C4 at 16384 tokens:
    // 12.9 -> 14.6 ms).  MLXS_SHARED_ASIDE_MAX moves the limit (0: never aside).
    static const uint32_t aside_max = getenv("MLXS_SHARED_ASIDE_MAX") ? (uint32_t)atoi(getenv("MLXS_SHARED_ASIDE_MAX")) : 64u;
    const bool shared_aside = c.shared_expert && h->aux_stream && T <= aside_max;
    const float* shared = nullptr;
    auto run_shared = [&](cudaStream_t s) -> int {
        const float lim = c.act == MLXS_ACT_SWIGLU_CLAMPED ? c.act_limit : 0.f;
        if (T >= shared_dense_min() && L.sh_gu_t) {
            DenseSharedArgs da{};
            da.x = static_cast<const __nv_bfloat16*>(x_dev); da.w_gu = L.sh_gu_t; da.w_d = L.sh_d_t;
            da.T = T; da.H = c.hidden; da.I = c.inter; da.limit = lim; da.xb = h->dg_xb; da.hb = h->dg_hb; da.out = h->sh_out;
            da.part_scratch = h->dg_scratch; da.part_count = h->dg_count; da.status = h->status; da.sm_count = h->sm_count;
            CU(launch_dense_shared_expert(da, s));
        } else {
            CU(launch_shared_expert(static_cast<const __nv_bfloat16*>(x_dev), L.sh_w1, L.sh_w3, L.sh_w2, T, c.hidden, c.inter,
                                    lim, h->sh_h, h->sh_out, s));
        }
        return MLXS_OK;
    };
    ForkGuard aux_guard(st);
    if (shared_aside) {
        CU(cudaEventRecord(h->aux_fork, st));
        CU(cudaStreamWaitEvent(h->aux_stream, h->aux_fork, 0));
        aux_guard.arm(h->aux_stream, h->aux_join);
        {
            StageTimer tm(h, MLXS_STAGE_SHARED, h->aux_stream);
            if ((rc = run_shared(h->aux_stream))) return rc;
        }
        CU(aux_guard.record());
        shared = h->sh_out;
    }
    if (front) {
        // route (from the logits, or from x through the layer's router weight), sort and stage in one launch; the
        // shared expert is already running beside it
        FrontArgs fa{};
        fa.w_router = front->logits ? nullptr : L.router_w; fa.logits_out = h->logits_ws; fa.logits = front->logits; fa.bias = L.bias;
        fa.E = (int)c.n_experts; fa.K = (int)c.top_k; fa.scoring = (int)c.scoring; fa.norm = (int)c.norm_topk; fa.scale = c.routed_scale;
        fa.ids = h->ids_ws; fa.weights = h->w_ws; fa.T = T; fa.loaded = L.loaded_dev; fa.t = h->tabs;
        fa.chunk_rows = h->chunk_rows; fa.group_chunks = h->group_chunks; fa.status = h->status; fa.sm_count = h->sm_count;
        fa.heavy = (h->pf_tiles && T >= h->pf_min_rows) ? h->pf_min_rows : 0u;   // the lane choice of mlxs_run_routed
        fa.x = static_cast<const __nv_bfloat16*>(x_dev); fa.H = c.hidden; fa.bank_exl3 = is_exl3(c.bank_kind) ? 1 : 0;
        fa.scales = L.scales; fa.scales_stride = is_exl3(c.bank_kind) ? exl3_scales_per_expert(Exl3Dims{c.hidden, c.inter, L.kbits}) : 0;
        fa.xa = h->xa_gu; fa.bar = h->front_bar;
        StageTimer tm(h, MLXS_STAGE_ROUTER, st);
        const cudaError_t fe = launch_front(fa, st);
        h->stats.route_calls += 1;
        if (fe == cudaSuccess) {
            h->front_done = true;
        } else {
            // the cooperative launch was refused (no room for all of its CTAs at once): the same work as separate
            // kernels, now and from here on
            cudaGetLastError();
            h->front_off = true;
            const float* lg = front->logits;
            if (!lg) {
                CU(launch_router_logits(fa.x, L.router_w, T, c.n_experts, c.hidden, h->logits_ws, st));
                lg = h->logits_ws;
            }
            CU(launch_router(lg, L.bias, (int)T, (int)c.n_experts, (int)c.top_k, (int)c.scoring, (int)c.norm_topk, c.routed_scale,
                             h->ids_ws, h->w_ws, st));
        }
    }
    if (!ep_fused && (rc = run_routed(h, layer, x_dev, ids_dev, T, h->ro, ro_bf16, st))) { h->front_done = false; return rc; }
    if (c.shared_expert && !shared_aside) {
        StageTimer tm(h, MLXS_STAGE_SHARED, st);
        if ((rc = run_shared(st))) return rc;
        shared = h->sh_out;
    }
    if (shared_aside) CU(aux_guard.wait_now());  // before the combine (or the exchange's final sum) reads the row
    if (ep_fused) {
        h->stats.tokens += T;
        return mlxs_ep_combined(h, layer, x_dev, ids_dev, weights_dev, T, shared, y_dev, st);
    }
    StageTimer tm(h, MLXS_STAGE_COMBINE, st);
    CU(launch_combine(h->ro, ro_bf16, weights_dev, shared, T, c.top_k, c.hidden, c.combine == MLXS_COMBINE_CHAIN,
                      static_cast<__nv_bfloat16*>(y_dev), st));
    return MLXS_OK;
}

extern "C" int mlxs_moe_experts(mlxs_moe* h, uint32_t layer, const void* x_dev, const int32_t* ids_dev,
                                const float* weights_dev, uint32_t T, void* y_dev, void* stream) {
    return experts_impl(h, layer, x_dev, ids_dev, weights_dev, T, y_dev, stream, nullptr);
}

extern "C" int mlxs_moe_forward(mlxs_moe* h, uint32_t layer, const void* x_dev, const float* logits_dev, uint32_t T,
                                void* y_dev, void* stream) {
    if (h && layer < h->cfg.n_layers && front_applies(h, T)) {
        if (!logits_dev) return fail(MLXS_E_ARG, "forward: null buffer");
        int rc = check_aligned(logits_dev, 4, "forward", "logits_dev");
        if (rc) return rc;
        const FrontCall fc{logits_dev};
        return experts_impl(h, layer, x_dev, h->ids_ws, h->w_ws, T, y_dev, stream, &fc);
    }
    int rc = mlxs_moe_route(h, layer, logits_dev, T, h ? h->ids_ws : nullptr, h ? h->w_ws : nullptr, stream);
    if (rc) return rc;
    return mlxs_moe_experts(h, layer, x_dev, h->ids_ws, h->w_ws, T, y_dev, stream);
}

static int read_status(mlxs_moe* h, cudaStream_t st) {
    uint32_t s = 0;
    CU(cudaMemcpyAsync(&s, h->status, 4, cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    h->stats.device_status = s;
    if (s) return fail(MLXS_E_DEVICE_STATUS, "device status %u (%s)", s,
                       s == ST_BAD_EXPERT_ID ? "expert id out of range" : s == ST_NOT_LOADED ? "a routed expert is not resident"
                       : s == ST_WORKLIST_OVERFLOW ? "work list overflow"
                       : s == ST_EP_OVERFLOW ? "expert parallel: a rank received more rows than the workspace holds"
                       : s == ST_EP_TIMEOUT ? "expert parallel: a peer's signal did not arrive within the bound"
                                            : "a bounded wait ran out");
    return MLXS_OK;
}

extern "C" int mlxs_moe_forward_host(mlxs_moe* h, uint32_t layer, const void* x_host, const float* logits_host, uint32_t T,
                                     void* y_host, void* stream) {
    int rc = check_call(h, layer, T, "forward_host");
    if (rc) return rc;
    if (T == 0 && h->cfg.ep_world == 1) return MLXS_OK;  // with expert parallelism an empty rank still serves its peers
    if (T && (!x_host || !logits_host || !y_host)) return fail(MLXS_E_ARG, "forward_host: null buffer");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t xb = (size_t)T * h->cfg.hidden * 2;
    if (T) {
        CU(cudaMemcpyAsync(h->x_io, x_host, xb, cudaMemcpyHostToDevice, st));
        CU(cudaMemcpyAsync(h->logits_io, logits_host, (size_t)T * h->cfg.n_experts * 4, cudaMemcpyHostToDevice, st));
    }
    if ((rc = mlxs_moe_forward(h, layer, h->x_io, h->logits_io, T, h->y_io, stream))) return rc;
    if (T) CU(cudaMemcpyAsync(y_host, h->y_io, xb, cudaMemcpyDeviceToHost, st));
    return read_status(h, st);
}

extern "C" int mlxs_moe_exl3_gemv(mlxs_moe* h, uint32_t layer, uint32_t expert, uint32_t proj, const float* xh_dev,
                                  uint32_t rows, float* z_dev, void* stream) {
    if (!h || !xh_dev || !z_dev) return fail(MLXS_E_ARG, "exl3_gemv: null argument");
    const mlxs_moe_config& c = h->cfg;
    if (!is_exl3(c.bank_kind)) return fail(MLXS_E_CONFIG, "exl3_gemv: the handle's bank is not EXL3");
    if (layer >= c.n_layers || expert >= c.n_experts || proj > 2) return fail(MLXS_E_ARG, "exl3_gemv: layer/expert/proj out of range");
    if (h->layers[layer].place_rank[expert] != c.ep_rank || !h->layers[layer].loaded[expert])
        return fail(MLXS_E_NOT_LOADED, "exl3_gemv: expert %u of layer %u is not resident on this rank", expert, layer);
    if (rows == 0) return MLXS_OK;
    if (rows > h->rows_cap) return fail(MLXS_E_TOO_MANY_TOKENS, "exl3_gemv: %u rows exceed the workspace", rows);
    CU(cudaSetDevice(c.device));
    cudaStream_t st = (cudaStream_t)stream;
    LayerBank& L = h->layers[layer];
    const Exl3Dims d{c.hidden, c.inter, L.kbits};
    const uint32_t le = h->layers[layer].place_slot[expert];
    // rows all belong to one pseudo expert 0 of a one-expert dispatch
    CU(cudaMemsetAsync(h->ids_ws, 0, (size_t)rows * 4, st));
    CU(launch_dispatch(h->ids_ws, rows, 1, nullptr, h->tabs, CHUNK_ROWS, GROUP_CHUNKS, 0, h->status, st));
    const uint32_t in_dim = proj == 2 ? c.inter : c.hidden, out_dim = proj == 2 ? c.hidden : c.inter;
    CU(launch_exl3_prep_raw(xh_dev, in_dim, h->tabs, h->xa_gu, st));
    const uint32_t* code = proj == 2 ? L.d_code + (size_t)le * exl3_code_words(d) : L.gu_code + (size_t)le * 2 * exl3_code_words(d);
    const uint32_t tw8 = 8u * exl3_tile_words(d);   // words of one projection's eight tiles of a k-tile
    CU(launch_exl3_raw(code, in_dim, out_dim, proj == 2 ? tw8 : 2u * tw8, proj == 1 ? tw8 : 0u, (int)d.K, h->tabs, h->xa_gu, z_dev,
                       h->status, h->sm_count, st));
    return MLXS_OK;
}

extern "C" int mlxs_moe_status_clear(mlxs_moe* h) {
    if (!h) return fail(MLXS_E_ARG, "status_clear: null handle");
    CU(cudaSetDevice(h->cfg.device));
    CU(cudaDeviceSynchronize());
    CU(cudaMemset(h->status, 0, 16));
    // a call that gave up may have left arrivals of the K-split fold behind
    if (h->ks_count) CU(cudaMemset(h->ks_count, 0, ksplit_count_words(h->sm_count) * 4));
    if (h->dg_count) CU(cudaMemset(h->dg_count, 0, (size_t)h->sm_count * 4));
    CU(cudaMemset(h->front_bar, 0, 16));
    h->stats.device_status = 0;
    return MLXS_OK;
}

extern "C" int mlxs_moe_debug_wait(mlxs_moe* h, uint32_t poll_limit, uint32_t withhold_stage) {
    if (!h) return fail(MLXS_E_ARG, "debug_wait: null handle");
    if (withhold_stage && (poll_limit == 0 || poll_limit > 4096))
        return fail(MLXS_E_ARG, "debug_wait: a withheld stage needs a poll limit of 1..4096 (the wait must run out quickly)");
    h->dbg_poll_limit = poll_limit;
    h->dbg_withhold = withhold_stage;
    return MLXS_OK;
}

extern "C" int mlxs_moe_sort_rows(mlxs_moe* h, const int32_t* slot_dev, uint32_t n, uint32_t n_slots, uint32_t* order_dev,
                                  uint32_t* offsets_dev, void* stream) {
    if (!h || (n && (!slot_dev || !order_dev)) || !offsets_dev) return fail(MLXS_E_ARG, "sort_rows: null argument");
    if (n_slots == 0 || n_slots > h->cfg.n_experts) return fail(MLXS_E_ARG, "sort_rows: %u slots, the handle's tables hold %u", n_slots, h->cfg.n_experts);
    if (n > h->rows_cap) return fail(MLXS_E_TOO_MANY_TOKENS, "sort_rows: %u rows exceed the workspace's %u", n, h->rows_cap);
    CU(cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    // the layer path's own dispatch: one CTA up to 2048 rows, count / scan / place over several CTAs above
    if (n > 2048)
        CU(launch_dispatch_large(slot_dev, n, n_slots, nullptr, h->tabs, h->chunk_rows, h->group_chunks, 0, h->blk_cnt, h->status, st));
    else
        CU(launch_dispatch(slot_dev, n, n_slots, nullptr, h->tabs, h->chunk_rows, h->group_chunks, 0, h->status, st));
    if (n) CU(cudaMemcpyAsync(order_dev, h->tabs.order, (size_t)n * 4, cudaMemcpyDeviceToDevice, st));
    CU(cudaMemcpyAsync(offsets_dev, h->tabs.offsets, ((size_t)n_slots + 1) * 4, cudaMemcpyDeviceToDevice, st));
    return MLXS_OK;
}

extern "C" int mlxs_moe_stats_get(mlxs_moe* h, mlxs_moe_stats* out) {
    if (!h || !out) return fail(MLXS_E_ARG, "stats: null argument");
    CU(cudaSetDevice(h->cfg.device));
    uint32_t hdr[8] = {0}, s = 0;
    CU(cudaDeviceSynchronize());
    CU(cudaMemcpy(hdr, h->tabs.header, sizeof hdr, cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(&s, h->status, 4, cudaMemcpyDeviceToHost));
    h->stats.device_status = s;
    h->stats.distinct_experts_last = hdr[HDR_DISTINCT];
    h->stats.weight_bytes_last = (uint64_t)hdr[HDR_DISTINCT] * (h->last_logical ? h->last_logical : h->logical_bytes);
    h->stats.resident_bytes = h->resident;
    h->stats.ep_transport = (uint32_t)mlxs_ep_transport(h);
    mlxs_ep_bytes(h, &h->stats.a2a_bytes_sent, &h->stats.a2a_bytes_recv);
    *out = h->stats;
    return MLXS_OK;
}

extern "C" int mlxs_moe_profile_enable(mlxs_moe* h, int on) {
    if (!h) return fail(MLXS_E_ARG, "profile_enable: null handle");
    h->prof_on = on != 0;
    return MLXS_OK;
}
extern "C" int mlxs_moe_profile_read(mlxs_moe* h, mlxs_moe_profile* out) {
    if (!h || !out) return fail(MLXS_E_ARG, "profile_read: null argument");
    CU(cudaSetDevice(h->cfg.device));
    for (auto& s : h->spans) {
        CU(cudaEventSynchronize(s.b));
        float ms = 0.f;
        CU(cudaEventElapsedTime(&ms, s.a, s.b));
        h->prof.ms[s.stage] += ms;
        h->prof.launches[s.stage] += 1;
        h->ev_pool.push_back(s.a);
        h->ev_pool.push_back(s.b);
    }
    h->spans.clear();
    *out = h->prof;
    h->prof = mlxs_moe_profile{};
    return MLXS_OK;
}

// ---- expert parallel ----
extern "C" int mlxs_moe_ep_plan(const int32_t* ids, uint64_t n, uint32_t n_experts, uint32_t world, uint64_t* send_counts) {
    if (!ids || !send_counts || world == 0 || n_experts == 0 || n_experts % world) return fail(MLXS_E_ARG, "ep_plan: bad argument");
    const uint32_t per = n_experts / world;
    for (uint32_t r = 0; r < world; ++r) send_counts[r] = 0;
    for (uint64_t i = 0; i < n; ++i) {
        if (ids[i] < 0 || (uint32_t)ids[i] >= n_experts) return fail(MLXS_E_ARG, "ep_plan: id %d at %llu outside 0..%u", ids[i], (unsigned long long)i, n_experts);
        send_counts[(uint32_t)ids[i] / per] += 1;
    }
    return MLXS_OK;
}
