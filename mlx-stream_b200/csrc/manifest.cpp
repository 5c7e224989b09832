// Expert-bank manifests in the reference's own formats, and the bank load built on them.
//   EXL3:  <dir>/expert-manifest-v2.json "mtplx-expert-manifest-v2" + sidecar (src/expert/bank.zig:103-155, 253-324)
//   MXFP4: <dir>/expert-manifest.json "mlx-stream-mxfp4-expert-bank-v1" + experts.bin (src/arch/mimo_v2/bank.zig:172-260)
//   NVFP4: <dir>/expert-manifest.json "mlx-stream-nvfp4-expert-bank-v1", layout "nvfp4-gud-9part"
//          (src/arch/glm5_next/bank.zig:29-48, 262-300)
// Every field the reference checks is checked here and refused by name (src/exl3/quant.zig:174-197).  Host only.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cctype>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/mlxs_moe.h"

int mlxs_fail(int rc, const char* fmt, ...);

namespace {

// ---- a small JSON reader (objects, arrays, strings, numbers, true/false/null) ----
struct JVal {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    uint64_t u = 0;
    bool is_uint = false;
    std::string str;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;
    const JVal* get(const char* key) const {
        if (kind != Obj) return nullptr;
        for (auto& kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
};
struct JParser {
    const char* p;
    const char* end;
    bool ok = true;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool lit(const char* s) {
        size_t n = strlen(s);
        if ((size_t)(end - p) >= n && !memcmp(p, s, n)) { p += n; return true; }
        return false;
    }
    JVal value(int depth = 0) {
        JVal v;
        ws();
        if (p >= end || depth > 64) { ok = false; return v; }
        if (*p == '{') {
            ++p; v.kind = JVal::Obj; ws();
            if (p < end && *p == '}') { ++p; return v; }
            while (ok) {
                ws();
                JVal k = value(depth + 1);
                if (!ok || k.kind != JVal::Str) { ok = false; break; }
                ws();
                if (p >= end || *p != ':') { ok = false; break; }
                ++p;
                v.obj.emplace_back(k.str, value(depth + 1));
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; break; }
                ok = false;
            }
        } else if (*p == '[') {
            ++p; v.kind = JVal::Arr; ws();
            if (p < end && *p == ']') { ++p; return v; }
            while (ok) {
                v.arr.push_back(value(depth + 1));
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; break; }
                ok = false;
            }
        } else if (*p == '"') {
            ++p; v.kind = JVal::Str;
            while (p < end && *p != '"') {
                if (*p == '\\' && p + 1 < end) {
                    ++p;
                    switch (*p) {
                        case 'n': v.str += '\n'; break;
                        case 't': v.str += '\t'; break;
                        case 'u': v.str += '?'; p += (end - p > 4) ? 4 : 0; break;
                        default: v.str += *p;
                    }
                    ++p;
                } else v.str += *p++;
            }
            if (p >= end) ok = false; else ++p;
        } else if (lit("true")) { v.kind = JVal::Bool; v.b = true; }
        else if (lit("false")) { v.kind = JVal::Bool; }
        else if (lit("null")) {}
        else {
            const char* s = p;
            bool integral = true;
            if (p < end && *p == '-') { ++p; integral = false; }
            while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) {
                if (*p < '0' || *p > '9') integral = false;
                ++p;
            }
            if (p == s) { ok = false; return v; }
            std::string t(s, p);
            v.kind = JVal::Num;
            v.num = strtod(t.c_str(), nullptr);
            if (integral && t.size() <= 19) { v.u = strtoull(t.c_str(), nullptr, 10); v.is_uint = true; }
        }
        return v;
    }
};

bool read_file(const std::string& path, std::string& out) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    char buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) out.append(buf, n);
    fclose(f);
    return true;
}
bool geti(const JVal* o, const char* k, uint64_t& out) {
    const JVal* v = o ? o->get(k) : nullptr;
    if (!v || v->kind != JVal::Num || !v->is_uint) return false;
    out = v->u;
    return true;
}
std::string gets(const JVal* o, const char* k) {
    const JVal* v = o ? o->get(k) : nullptr;
    return v && v->kind == JVal::Str ? v->str : std::string();
}
bool lower_hex64(const std::string& h);   // 64 lowercase hex digits (the reference decodes lowercase hex only: src/expert/bank.zig:432-466)
bool plain_name(const std::string& s) {
    if (s.empty() || s == "." || s == "..") return false;
    for (char c : s) if (c == '/' || c == '\\' || c == 0) return false;
    return true;
}

// ---- sha256 (records may carry their digest; verified on request) ----
struct Sha256 {
    uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    uint8_t buf[64];
    uint64_t len = 0;
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const uint8_t* p) {
        static const uint32_t K[64] = {
            0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
            0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
            0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
            0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
            0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
            0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
            0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
        uint32_t w[64];
        for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
        for (int i = 16; i < 64; ++i) {
            uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3), s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; ++i) {
            uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g), t1 = hh + S1 + ch + K[i] + w[i];
            uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c), t2 = S0 + mj;
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const uint8_t* p, size_t n) {
        size_t fill = len % 64;
        len += n;
        if (fill) {
            size_t take = 64 - fill < n ? 64 - fill : n;
            memcpy(buf + fill, p, take);
            p += take; n -= take;
            if (fill + take < 64) return;
            block(buf);
        }
        while (n >= 64) { block(p); p += 64; n -= 64; }
        if (n) memcpy(buf, p, n);
    }
    std::string hex() {
        uint64_t bits = len * 8;
        uint8_t pad[72] = {0x80};
        size_t padn = (len % 64 < 56 ? 56 : 120) - len % 64;
        update(pad, padn);
        uint8_t lb[8];
        for (int i = 0; i < 8; ++i) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(lb, 8);
        char out[65];
        for (int i = 0; i < 8; ++i) snprintf(out + 8 * i, 9, "%08x", h[i]);
        return std::string(out, 64);
    }
};

struct Record { uint64_t offset = 0; std::string sha256; std::string sha256_logical; bool present = false; };
struct Bank {
    mlxs_bank_info info{};
    std::vector<Record> records;  // [layer][expert]
    // EXL3 only: every layer's K, record size and place in the sidecar (a bank may mix widths)
    std::vector<uint32_t> layer_bits;
    std::vector<uint64_t> layer_logical, layer_stride, layer_base;
};

// src/expert/bank.zig:116-141: three code planes of 16x16 tiles at 32 K bytes each, six f16 scale vectors
uint64_t exl3_logical(uint64_t H, uint64_t I, uint64_t K) { return 3 * ((H / 16) * (I / 16) * 32 * K) + 6 * H + 6 * I; }

int parse_exl3(const JVal& m, Bank& b) {
    // src/exl3/quant.zig:174-197 (claims) and src/expert/bank.zig:253-324 (adoptV2), field by field
    const JVal* q = m.get("quantization");
    if (!q) return mlxs_fail(MLXS_E_MANIFEST, "v2: no quantization");
    if (gets(q, "mode") != "exl3") return mlxs_fail(MLXS_E_MANIFEST, "v2: quantization.mode \"%s\"", gets(q, "mode").c_str());
    if (gets(q, "codebook") != "mul1") return mlxs_fail(MLXS_E_MANIFEST, "v2: quantization.codebook \"%s\" not implemented", gets(q, "codebook").c_str());
    uint64_t mult = 0;
    if (!geti(q, "codebook_multiplier", mult) || mult != 0x83DCD12Dull) return mlxs_fail(MLXS_E_MANIFEST, "v2: codebook_multiplier %llu != 2212286765", (unsigned long long)mult);
    const JVal* tile = q->get("tile");
    uint64_t tsz = 0;
    if (!geti(tile, "size", tsz) || tsz != 16 || gets(tile, "layout") != "exl3-tensor-core" || gets(tile, "bitstream") != "msb-first-swap16")
        return mlxs_fail(MLXS_E_MANIFEST, "v2: quantization.tile %llu / %s / %s", (unsigned long long)tsz, gets(tile, "layout").c_str(), gets(tile, "bitstream").c_str());
    const JVal* had = q->get("hadamard");
    uint64_t hsz = 0;
    if (!geti(had, "size", hsz) || hsz != 128 || gets(had, "order") != "sylvester-natural" || gets(had, "scale") != "1/sqrt(128)")
        return mlxs_fail(MLXS_E_MANIFEST, "v2: quantization.hadamard %llu / %s", (unsigned long long)hsz, gets(had, "order").c_str());
    const JVal* sc = q->get("scales");
    if (gets(sc, "rin") != "exl3.suh" || gets(sc, "rout") != "exl3.svh")
        return mlxs_fail(MLXS_E_MANIFEST, "v2: quantization.scales rin %s rout %s", gets(sc, "rin").c_str(), gets(sc, "rout").c_str());
    const JVal* d = m.get("dims");
    uint64_t H = 0, I = 0, E = 0, L = 0;
    if (!geti(d, "hidden", H) || !geti(d, "inter", I) || !geti(d, "n_experts", E) || !geti(d, "n_layers", L) || !H || !I || !E || !L ||
        H % 16 || I % 16 || L > 4096 || E > 65536)
        return mlxs_fail(MLXS_E_MANIFEST, "v2: dims hidden=%llu inter=%llu n_experts=%llu n_layers=%llu", (unsigned long long)H,
                         (unsigned long long)I, (unsigned long long)E, (unsigned long long)L);
    const JVal* layers = m.get("layers");
    if (!layers || layers->kind != JVal::Arr || layers->arr.size() != L)
        return mlxs_fail(MLXS_E_MANIFEST, "v2: %zu layer entries != dims.n_layers %llu", layers ? layers->arr.size() : 0, (unsigned long long)L);
    static const char* proj[3] = {"gate_proj", "up_proj", "down_proj"};
    static const char* part[3] = {"code", "rout", "rin"};
    uint64_t base = 0;
    for (size_t li = 0; li < layers->arr.size(); ++li) {
        const JVal& t = layers->arr[li];
        uint64_t ln = 0, K = 0, rb = 0, lb = 0, bo = 0;
        if (!geti(&t, "layer", ln) || ln != li) return mlxs_fail(MLXS_E_MANIFEST, "v2: layer entry %zu names layer %llu", li, (unsigned long long)ln);
        if (!geti(&t, "K", K) || (K != 3 && K != 2)) return mlxs_fail(MLXS_E_MANIFEST, "v2: layer %zu K %llu not implemented by the installed lanes", li, (unsigned long long)K);
        const uint64_t logical = exl3_logical(H, I, K), stride = (logical + 4095) / 4096 * 4096;
        const JVal* segs = t.get("segments");
        if (!segs || segs->kind != JVal::Arr || segs->arr.size() != 9) return mlxs_fail(MLXS_E_MANIFEST, "v2: layer %zu has no 9-segment table", li);
        uint64_t off = 0;
        for (int p = 0; p < 3; ++p) {
            const uint64_t in = p == 2 ? I : H, out = p == 2 ? H : I;
            for (int j = 0; j < 3; ++j) {
                const JVal& s = segs->arr[p * 3 + j];
                const std::string want = std::string(proj[p]) + "." + part[j], got = gets(&s, "component");
                if (got != want) {
                    const size_t dot = got.find('.');
                    const std::string gp = got.substr(0, dot), gt = dot == std::string::npos ? "" : got.substr(dot + 1);
                    bool known_p = false, known_t = false;
                    for (auto n : proj) known_p |= gp == n;
                    for (auto n : part) known_t |= gt == n;
                    return mlxs_fail(MLXS_E_MANIFEST, "v2: segment %s: %s", got.c_str(),
                                     !known_p ? "an unknown projection" : !known_t ? "an unknown tensor" : "out of order");
                }
                const uint64_t len = j == 0 ? (in / 16) * (out / 16) * 32 * K : (j == 1 ? out * 2 : in * 2);
                if (gets(&s, "dtype") != (j == 0 ? "I16" : "F16")) return mlxs_fail(MLXS_E_MANIFEST, "v2: segment %s: its dtype", want.c_str());
                const JVal* shp = s.get("shape");
                bool shape_ok = shp && shp->kind == JVal::Arr;
                if (shape_ok) {
                    if (j == 0) shape_ok = shp->arr.size() == 3 && shp->arr[0].u == in / 16 && shp->arr[1].u == out / 16 && shp->arr[2].u == 16 * K;
                    else shape_ok = shp->arr.size() == 1 && shp->arr[0].u == (j == 1 ? out : in);
                }
                if (!shape_ok) return mlxs_fail(MLXS_E_MANIFEST, "v2: segment %s: its shape", want.c_str());
                uint64_t so = 0, sl = 0;
                if (!geti(&s, "offset", so) || !geti(&s, "length", sl) || so != off || sl != len)
                    return mlxs_fail(MLXS_E_MANIFEST, "v2: segment %s: its place (offset %llu length %llu)", want.c_str(), (unsigned long long)so, (unsigned long long)sl);
                off += len;
            }
        }
        if (!geti(&t, "record_bytes", rb) || !geti(&t, "logical_bytes", lb) || rb != stride || lb != logical)
            return mlxs_fail(MLXS_E_MANIFEST, "v2: layer %zu segment table / record size differs from the v2 geometry for K=%llu", li, (unsigned long long)K);
        if (!geti(&t, "base_offset", bo) || bo != base) return mlxs_fail(MLXS_E_MANIFEST, "v2: layer %zu base_offset %llu != %llu", li, (unsigned long long)bo, (unsigned long long)base);
        b.layer_bits.push_back((uint32_t)K);
        b.layer_logical.push_back(logical);
        b.layer_stride.push_back(stride);
        b.layer_base.push_back(base);
        base += E * stride;
    }
    uint32_t kmin = 8, kmax = 0;
    for (uint32_t k : b.layer_bits) { kmin = k < kmin ? k : kmin; kmax = k > kmax ? k : kmax; }
    b.info.bank_kind = kmax == 3 ? MLXS_BANK_EXL3_K3_MUL1 : MLXS_BANK_EXL3_K2_MUL1;
    b.info.bits_min = kmin; b.info.bits_max = kmax;
    b.info.hidden = H; b.info.inter = I; b.info.n_experts = E; b.info.n_layers = L; b.info.first_layer = 0;
    b.info.logical_bytes = exl3_logical(H, I, kmax); b.info.record_stride = (b.info.logical_bytes + 4095) / 4096 * 4096;
    b.info.data_bytes = base;
    // sidecar / records / parity: required for a load, absent from a trimmed description
    const JVal* scd = m.get("sidecar");
    if (scd) {
        uint64_t sz = 0, al = 0;
        const std::string file = gets(scd, "file");
        if (!geti(scd, "size", sz) || sz != base) return mlxs_fail(MLXS_E_MANIFEST, "v2: sidecar.size %llu != %llu", (unsigned long long)sz, (unsigned long long)base);
        if (!geti(scd, "alignment", al) || al != 4096) return mlxs_fail(MLXS_E_MANIFEST, "v2: sidecar alignment %llu != 4096", (unsigned long long)al);
        if (!plain_name(file) || file.size() >= sizeof b.info.data_file) return mlxs_fail(MLXS_E_MANIFEST, "v2: sidecar file \"%s\" is not a plain file name", file.c_str());
        snprintf(b.info.data_file, sizeof b.info.data_file, "%s", file.c_str());
    }
    const JVal* recs = m.get("records");
    if (recs) {
        if (recs->kind != JVal::Arr || recs->arr.size() != L * E)
            return mlxs_fail(MLXS_E_MANIFEST, "v2: %zu records != %llu x %llu", recs->arr.size(), (unsigned long long)L, (unsigned long long)E);
        b.records.assign(L * E, Record{});
        for (const JVal& r : recs->arr) {
            uint64_t rl = 0, re = 0, so = 0, rb = 0, lb = 0;
            if (!geti(&r, "layer", rl) || !geti(&r, "expert", re) || rl >= L || re >= E) return mlxs_fail(MLXS_E_MANIFEST, "v2: record (%llu,%llu) out of range", (unsigned long long)rl, (unsigned long long)re);
            Record& dst = b.records[rl * E + re];
            if (dst.present) return mlxs_fail(MLXS_E_MANIFEST, "v2: record (%llu,%llu) duplicated", (unsigned long long)rl, (unsigned long long)re);
            if (!geti(&r, "sidecar_offset", so) || !geti(&r, "record_bytes", rb) || !geti(&r, "logical_bytes", lb) ||
                so != b.layer_base[rl] + re * b.layer_stride[rl] || rb != b.layer_stride[rl] || lb != b.layer_logical[rl])
                return mlxs_fail(MLXS_E_MANIFEST, "v2: record (%llu,%llu) offset/size differs from its layer geometry", (unsigned long long)rl, (unsigned long long)re);
            dst.sha256 = gets(&r, "sha256");
            if (!lower_hex64(dst.sha256)) return mlxs_fail(MLXS_E_MANIFEST, "v2: record (%llu,%llu) has no sha256 (RecordSha256)", (unsigned long long)rl, (unsigned long long)re);
            dst.offset = so;
            dst.present = true;
        }
        b.info.has_sha256 = 1;
        const JVal* par = m.get("parity");
        const JVal* ap = par ? par->get("all_pass") : nullptr;
        if (!ap || ap->kind != JVal::Bool || !ap->b) return mlxs_fail(MLXS_E_MANIFEST, "v2: parity.all_pass is not true");
    }
    return MLXS_OK;
}

int parse_fp4(const JVal& m, Bank& b, bool nv) {
    // src/arch/mimo_v2/bank.zig:202-260, src/arch/glm5_next/bank.zig:262-300
    const char* tag = nv ? "nvfp4" : "mxfp4";
    if (gets(&m, "data_file") != "experts.bin") return mlxs_fail(MLXS_E_MANIFEST, "%s: data_file \"%s\"", tag, gets(&m, "data_file").c_str());
    if (nv && gets(&m, "layout") != "nvfp4-gud-9part") return mlxs_fail(MLXS_E_MANIFEST, "nvfp4: layout \"%s\"", gets(&m, "layout").c_str());
    const JVal* q = m.get("quantization");
    uint64_t bits = 0, gs = 0;
    if (gets(q, "mode") != tag || !geti(q, "bits", bits) || bits != 4 || !geti(q, "group_size", gs) || gs != (nv ? 16u : 32u))
        return mlxs_fail(MLXS_E_MANIFEST, "%s: quantization mode \"%s\" bits %llu group_size %llu (InvalidQuantization)", tag, gets(q, "mode").c_str(), (unsigned long long)bits, (unsigned long long)gs);
    uint64_t H = 0, I = 0, E = 0, first = 0, L = 0, rb = 0, gub = 0;
    if (!geti(&m, "hidden_size", H) || !geti(&m, "intermediate_size", I) || !geti(&m, "num_experts", E) || !geti(&m, "first_moe_layer", first) ||
        !geti(&m, "num_moe_layers", L) || !H || !I || !E || !L || H % 32 || I % 32)
        return mlxs_fail(MLXS_E_MANIFEST, "%s: topology hidden=%llu inter=%llu experts=%llu layers=%llu", tag, (unsigned long long)H, (unsigned long long)I, (unsigned long long)E, (unsigned long long)L);
    const uint64_t blk = nv ? 16 : 32, tail = nv ? 4 : 0;
    const uint64_t part = H * I / 2 + H * I / blk + tail, logical = 3 * part;
    uint64_t stride = logical;
    if (nv) {
        uint64_t al = 0, rs = 0, db = 0;
        if (!geti(&m, "alignment", al) || al != 4096) return mlxs_fail(MLXS_E_MANIFEST, "nvfp4: alignment %llu != 4096", (unsigned long long)al);
        stride = (logical + 4095) / 4096 * 4096;
        if (!geti(&m, "record_stride", rs) || rs != stride) return mlxs_fail(MLXS_E_MANIFEST, "nvfp4: record_stride %llu != %llu", (unsigned long long)rs, (unsigned long long)stride);
        if (!geti(&m, "down_bytes", db) || db != part) return mlxs_fail(MLXS_E_MANIFEST, "nvfp4: down_bytes %llu != %llu", (unsigned long long)db, (unsigned long long)part);
    }
    if (!geti(&m, "record_bytes", rb) || rb != logical) return mlxs_fail(MLXS_E_MANIFEST, "%s: record_bytes %llu != %llu (InvalidGeometry)", tag, (unsigned long long)rb, (unsigned long long)logical);
    if (!geti(&m, "gate_up_bytes", gub) || gub != 2 * part) return mlxs_fail(MLXS_E_MANIFEST, "%s: gate_up_bytes %llu != %llu (InvalidGeometry)", tag, (unsigned long long)gub, (unsigned long long)(2 * part));
    const JVal* segs = m.get(nv ? "parts" : "segments");
    const size_t nseg = nv ? 9 : 6;
    if (!segs || segs->kind != JVal::Arr || segs->arr.size() != nseg) return mlxs_fail(MLXS_E_MANIFEST, "%s: no %zu-part table (InvalidSegment)", tag, nseg);
    static const char* proj[3] = {"gate_proj", "up_proj", "down_proj"};
    uint64_t off = 0;
    for (int p = 0; p < 3; ++p) {
        const uint64_t rows = p == 2 ? H : I, cols = p == 2 ? I : H;
        const char* names[3] = {"weight", "scales", "global_scale"};
        const char* dts[3] = {"U32", "U8", "F32"};
        const uint64_t lens[3] = {rows * cols / 2, rows * cols / blk, 4};
        for (int j = 0; j < (nv ? 3 : 2); ++j) {
            const JVal& s = segs->arr[p * (nv ? 3 : 2) + j];
            const std::string want = std::string(proj[p]) + "." + names[j];
            uint64_t so = 0, sl = 0;
            if (gets(&s, "name") != want || gets(&s, "dtype") != dts[j] || !geti(&s, "offset", so) || !geti(&s, "length", sl) || so != off || sl != lens[j])
                return mlxs_fail(MLXS_E_MANIFEST, "%s: part %s: its name, dtype or place (InvalidSegment)", tag, want.c_str());
            const JVal* shp = s.get("shape");
            bool shape_ok = shp && shp->kind == JVal::Arr;
            if (shape_ok) {
                if (j == 0) shape_ok = shp->arr.size() == 2 && shp->arr[0].u == rows && shp->arr[1].u == cols / 8;
                else if (j == 1) shape_ok = shp->arr.size() == 2 && shp->arr[0].u == rows && shp->arr[1].u == cols / blk;
                else shape_ok = shp->arr.empty();
            }
            if (!shape_ok) return mlxs_fail(MLXS_E_MANIFEST, "%s: part %s: its shape (InvalidSegment)", tag, want.c_str());
            off += lens[j];
        }
    }
    const JVal* src = m.get("source");
    bool rev_hex = true;
    for (char ch : gets(src, "revision")) rev_hex = rev_hex && isxdigit((unsigned char)ch);
    if (gets(src, "repository").empty() || gets(src, "revision").size() != 40 || !rev_hex) return mlxs_fail(MLXS_E_MANIFEST, "%s: source repository / revision (InvalidSource)", tag);
    const JVal* recs = m.get("records");
    if (!recs || recs->kind != JVal::Arr || recs->arr.size() != L * E) return mlxs_fail(MLXS_E_MANIFEST, "%s: %zu records != %llu (InvalidRecord)", tag, recs ? recs->arr.size() : 0, (unsigned long long)(L * E));
    b.records.assign(L * E, Record{});
    for (size_t i = 0; i < recs->arr.size(); ++i) {
        const JVal& r = recs->arr[i];
        uint64_t rl = 0, re = 0, ro = 0, rlen = 0;
        if (!geti(&r, "layer", rl) || !geti(&r, "expert", re) || !geti(&r, "offset", ro) || !geti(&r, "length", rlen) ||
            rl != first + i / E || re != i % E || ro != i * stride || rlen != logical)
            return mlxs_fail(MLXS_E_MANIFEST, "%s: record %zu: its layer, expert or place (InvalidRecord)", tag, i);
        b.records[i].sha256 = gets(&r, "sha256");
        if (!lower_hex64(b.records[i].sha256)) return mlxs_fail(MLXS_E_MANIFEST, "%s: record %zu has no sha256 (InvalidDigest)", tag, i);
        b.records[i].offset = ro;
        b.records[i].present = true;
    }
    const JVal* of = m.get("output_files");
    const JVal* eb = of ? of->get("experts.bin") : nullptr;
    uint64_t sz = 0;
    const uint64_t total = nv ? L * E * stride : L * E * logical;
    if (eb && !lower_hex64(gets(eb, "sha256")))
        return mlxs_fail(MLXS_E_MANIFEST, "%s: output_files experts.bin has no sha256 (InvalidDigest)", tag);
    if (!eb || !geti(eb, "size", sz) || sz != total)
        return mlxs_fail(MLXS_E_MANIFEST, "%s: output_files experts.bin size %llu != %llu (InvalidOutputFile)", tag, (unsigned long long)sz, (unsigned long long)total);
    b.info.bank_kind = nv ? MLXS_BANK_NVFP4 : MLXS_BANK_MXFP4;
    b.info.hidden = H; b.info.inter = I; b.info.n_experts = E; b.info.n_layers = L; b.info.first_layer = first;
    b.info.logical_bytes = logical; b.info.record_stride = stride; b.info.data_bytes = total; b.info.has_sha256 = 1;
    snprintf(b.info.data_file, sizeof b.info.data_file, "experts.bin");
    return MLXS_OK;
}

int parse_text(const std::string& text, const char* name, Bank& b) {
    JParser jp{text.data(), text.data() + text.size()};
    JVal m = jp.value();
    jp.ws();
    if (!jp.ok || m.kind != JVal::Obj) return mlxs_fail(MLXS_E_MANIFEST, "%s: not a JSON object", name);
    const std::string fmt = gets(&m, "format");
    if (fmt == "mtplx-expert-manifest-v2") return parse_exl3(m, b);
    if (fmt == "mlx-stream-mxfp4-expert-bank-v1") return parse_fp4(m, b, false);
    if (fmt == "mlx-stream-nvfp4-expert-bank-v1") return parse_fp4(m, b, true);
    if (fmt == "mtplx-expert-manifest-v1")
        return mlxs_fail(MLXS_E_MANIFEST, "%s is the v1 runtime manifest of an EXL3 bank; its expert-manifest-v2.json cannot be read (ManifestMissing)", name);
    return mlxs_fail(MLXS_E_MANIFEST, "%s: format \"%s\" is none of the three bank formats", name, fmt.c_str());
}

int open_bank(const char* dir, Bank& b) {
    std::string text;
    const std::string d(dir);
    if (read_file(d + "/expert-manifest-v2.json", text)) return parse_text(text, "expert-manifest-v2.json", b);
    if (read_file(d + "/expert-manifest.json", text)) return parse_text(text, "expert-manifest.json", b);
    return mlxs_fail(MLXS_E_MANIFEST, "%s: neither expert-manifest-v2.json nor expert-manifest.json can be read", dir);
}

bool lower_hex64(const std::string& h) {
    if (h.size() != 64) return false;
    for (char ch : h) if (!((ch >= '0' && ch <= '9') || (ch >= 'a' && ch <= 'f'))) return false;
    return true;
}

// An EXL3 bank carries two manifests: the v2 geometry and the v1 runtime manifest <dir>/expert-manifest.json, which must
// describe exactly the v2 records: same offsets, logical sizes and segment table (absolute offsets), every record once,
// the same sidecar (src/expert/bank.zig:326-400, refusals :1064-1072).  Keeps each record's logical-bytes digest.
int check_v1(const std::string& dir, Bank& b) {
    static const char* name = "expert-manifest.json";
    std::string text;
    if (!read_file(dir + "/" + name, text))
        return mlxs_fail(MLXS_E_MANIFEST, "%s: the v1 runtime manifest cannot be read (ManifestMissing)", name);
    JParser jp{text.data(), text.data() + text.size()};
    JVal m = jp.value();
    jp.ws();
    if (!jp.ok || m.kind != JVal::Obj || jp.p != jp.end) return mlxs_fail(MLXS_E_MANIFEST, "%s: not a JSON object (ManifestSyntax)", name);
    const std::string fmt = gets(&m, "format");
    if (fmt != "mtplx-expert-manifest-v1") return mlxs_fail(MLXS_E_MANIFEST, "%s: format \"%s\" is not mtplx-expert-manifest-v1 (ManifestFormat)", name, fmt.c_str());
    const std::string mode = gets(m.get("quantization"), "mode");
    if (mode != "exl3-mul1") return mlxs_fail(MLXS_E_MANIFEST, "%s: quantization.mode \"%s\" is not exl3-mul1 (RuntimeModeNotExl3)", name, mode.c_str());
    const mlxs_bank_info& bi = b.info;
    const uint64_t H = bi.hidden, I = bi.inter, E = bi.n_experts, L = bi.n_layers;
    const JVal* recs = m.get("records");
    if (!recs || recs->kind != JVal::Arr || recs->arr.size() != L * E)
        return mlxs_fail(MLXS_E_MANIFEST, "%s: %zu records != %llu (RecordCount)", name, recs && recs->kind == JVal::Arr ? recs->arr.size() : (size_t)0,
                         (unsigned long long)(L * E));
    static const char* proj[3] = {"gate_proj", "up_proj", "down_proj"};
    static const char* part[3] = {"code", "rout", "rin"};
    std::vector<bool> seen(L * E, false);
    for (const JVal& r : recs->arr) {
        uint64_t rl = 0, re = 0, lb = 0, so = 0, sl = 0;
        if (!geti(&r, "layer", rl) || !geti(&r, "expert", re) || rl >= L || re >= E)
            return mlxs_fail(MLXS_E_MANIFEST, "v1: record (%llu,%llu) is not in the v2 bank (RuntimeRecordMismatch)", (unsigned long long)rl, (unsigned long long)re);
        const size_t i = rl * E + re;
        if (seen[i]) return mlxs_fail(MLXS_E_MANIFEST, "v1: record (%llu,%llu) duplicated (RecordDuplicate)", (unsigned long long)rl, (unsigned long long)re);
        seen[i] = true;
        const uint64_t off = b.layer_base[rl] + re * b.layer_stride[rl], logical = b.layer_logical[rl], K = b.layer_bits[rl];
        if (!geti(&r, "logical_bytes", lb) || !geti(&r, "sidecar_offset", so) || !geti(&r, "sidecar_length", sl) || so != off || lb != logical || sl != logical)
            return mlxs_fail(MLXS_E_MANIFEST, "v1: record (%llu,%llu) offset/length differs from the v2 manifest (RuntimeRecordMismatch)", (unsigned long long)rl, (unsigned long long)re);
        const JVal* segs = r.get("segments");
        if (!segs || segs->kind != JVal::Arr || segs->arr.size() != 9)
            return mlxs_fail(MLXS_E_MANIFEST, "v1: record (%llu,%llu) has %zu segments (RuntimeRecordMismatch)", (unsigned long long)rl, (unsigned long long)re,
                             segs && segs->kind == JVal::Arr ? segs->arr.size() : (size_t)0);
        for (const JVal& sg : segs->arr)
            if (gets(&sg, "shard") != bi.data_file)
                return mlxs_fail(MLXS_E_MANIFEST, "v1: record (%llu,%llu) reads shard \"%s\" (RuntimeRecordMismatch)", (unsigned long long)rl, (unsigned long long)re, gets(&sg, "shard").c_str());
        // absolute offsets equal to the record's offset + the v2 table: contiguous, in record order
        uint64_t rel = 0;
        bool match = true;
        for (int p = 0; p < 3 && match; ++p) {
            const uint64_t in = p == 2 ? I : H, out = p == 2 ? H : I;
            for (int j = 0; j < 3 && match; ++j) {
                const JVal& sg = segs->arr[p * 3 + j];
                const uint64_t len = j == 0 ? (in / 16) * (out / 16) * 32 * K : (j == 1 ? out * 2 : in * 2);
                uint64_t go = 0, gl = 0;
                const JVal* shp = sg.get("shape");
                match = gets(&sg, "component") == std::string(proj[p]) + "." + part[j] && gets(&sg, "dtype") == (j == 0 ? "I16" : "F16") &&
                        geti(&sg, "offset", go) && geti(&sg, "length", gl) && go == off + rel && gl == len && shp && shp->kind == JVal::Arr;
                if (match) {
                    if (j == 0) match = shp->arr.size() == 3 && shp->arr[0].u == in / 16 && shp->arr[1].u == out / 16 && shp->arr[2].u == 16 * K;
                    else match = shp->arr.size() == 1 && shp->arr[0].u == (j == 1 ? out : in);
                }
                rel += len;
            }
        }
        if (!match)
            return mlxs_fail(MLXS_E_MANIFEST, "v1: record (%llu,%llu) segments differ from the v2 layer table (order, offsets, lengths, dtype, shape) (RuntimeRecordMismatch)",
                             (unsigned long long)rl, (unsigned long long)re);
        const std::string sha = gets(&r, "sha256");
        if (!lower_hex64(sha)) return mlxs_fail(MLXS_E_MANIFEST, "v1: record (%llu,%llu) has no sha256 (RecordSha256)", (unsigned long long)rl, (unsigned long long)re);
        b.records[i].sha256_logical = sha;
    }
    const JVal* sc = m.get("sidecar");
    uint64_t sz = 0, al = 0;
    if (!sc) return mlxs_fail(MLXS_E_MANIFEST, "%s: no sidecar (ManifestSyntax)", name);
    if (gets(sc, "file") != bi.data_file || !geti(sc, "size", sz) || sz != bi.data_bytes || !geti(sc, "alignment", al) || al != 4096)
        return mlxs_fail(MLXS_E_MANIFEST, "%s: sidecar %s (%llu B, align %llu) differs from the v2 manifest (SidecarGeometry)", name, gets(sc, "file").c_str(),
                         (unsigned long long)sz, (unsigned long long)al);
    return MLXS_OK;
}

// Bank.open without a device (src/expert/bank.zig:228-251): the manifests, the v1 cross-check of an EXL3 bank, the
// sidecar (a plain file of at least the manifest's size; a symbolic link is refused).  Returns the open descriptor.
int open_checked(const char* dir, Bank& b, int& fd_out) {
    int rc = open_bank(dir, b);
    if (rc) return rc;
    const mlxs_bank_info& bi = b.info;
    if (!bi.data_file[0] || b.records.empty()) return mlxs_fail(MLXS_E_MANIFEST, "load_bank: the manifest names no sidecar / records");
    if (!b.layer_bits.empty() && (rc = check_v1(dir, b))) return rc;
    const std::string path = std::string(dir) + "/" + bi.data_file;
    const int fd = open(path.c_str(), O_RDONLY | O_NOFOLLOW);
    if (fd < 0) return mlxs_fail(MLXS_E_MANIFEST, "load_bank: cannot open %s (SidecarMissing / SidecarOpen)", path.c_str());
    struct stat st;
    if (fstat(fd, &st) || (uint64_t)st.st_size < bi.data_bytes) {
        close(fd);
        return mlxs_fail(MLXS_E_MANIFEST, "load_bank: %s is shorter than the manifest's %llu bytes (SidecarGeometry)", path.c_str(), (unsigned long long)bi.data_bytes);
    }
    fd_out = fd;
    return MLXS_OK;
}

// one record into buf (the padded record of an EXL3 bank, the record's own bytes otherwise), digests checked on request
int read_record(int fd, const Bank& b, uint64_t l, uint64_t e, bool verify, std::vector<uint8_t>& buf) {
    const bool exl3 = !b.layer_bits.empty();
    const Record& r = b.records[l * b.info.n_experts + e];
    if (!r.present) return mlxs_fail(MLXS_E_MANIFEST, "load_bank: record (%llu,%llu) missing", (unsigned long long)l, (unsigned long long)e);
    buf.resize(exl3 ? b.layer_stride[l] : b.info.logical_bytes);
    size_t got = 0;
    while (got < buf.size()) {
        const ssize_t n = pread(fd, buf.data() + got, buf.size() - got, (off_t)(r.offset + got));
        if (n <= 0) break;
        got += (size_t)n;
    }
    if (got != buf.size()) return mlxs_fail(MLXS_E_MANIFEST, "load_bank: short read of record (%llu,%llu)", (unsigned long long)l, (unsigned long long)e);
    if (verify) {
        // the v2 (EXL3) digests cover the padded record, the v1 ones its logical bytes; the FP4 banks' the record's own bytes
        Sha256 s;
        s.update(buf.data(), buf.size());
        if (s.hex() != r.sha256) return mlxs_fail(MLXS_E_MANIFEST, "load_bank: record (%llu,%llu) sha256 mismatch (RecordSha256)", (unsigned long long)l, (unsigned long long)e);
        if (exl3 && !r.sha256_logical.empty()) {
            Sha256 s1;
            s1.update(buf.data(), b.layer_logical[l]);
            if (s1.hex() != r.sha256_logical)
                return mlxs_fail(MLXS_E_MANIFEST, "load_bank: record (%llu,%llu) differs from its v1 sha256 (RecordSha256)", (unsigned long long)l, (unsigned long long)e);
        }
    }
    return MLXS_OK;
}

}  // namespace

extern "C" int mlxs_moe_bank_peek_text(const char* manifest_json, mlxs_bank_info* out) {
    if (!manifest_json || !out) return mlxs_fail(MLXS_E_ARG, "bank_peek_text: null argument");
    Bank b;
    int rc = parse_text(manifest_json, "manifest", b);
    if (rc) return rc;
    *out = b.info;
    return MLXS_OK;
}

extern "C" int mlxs_moe_bank_peek(const char* dir, mlxs_bank_info* out) {
    if (!dir || !out) return mlxs_fail(MLXS_E_ARG, "bank_peek: null argument");
    Bank b;
    int rc = open_bank(dir, b);
    if (rc) return rc;
    *out = b.info;
    return MLXS_OK;
}

extern "C" int mlxs_moe_bank_layer_bits_text(const char* manifest_json, uint32_t* bits_out, uint32_t cap, uint32_t* n_layers_out) {
    if (!manifest_json || !n_layers_out || (cap && !bits_out)) return mlxs_fail(MLXS_E_ARG, "bank_layer_bits_text: null argument");
    Bank b;
    int rc = parse_text(manifest_json, "manifest", b);
    if (rc) return rc;
    if (b.layer_bits.empty()) return mlxs_fail(MLXS_E_MANIFEST, "bank_layer_bits_text: not an EXL3 manifest");
    *n_layers_out = (uint32_t)b.layer_bits.size();
    for (uint32_t i = 0; i < cap && i < b.layer_bits.size(); ++i) bits_out[i] = b.layer_bits[i];
    return MLXS_OK;
}

// mlxs_moe_load_bank's host half: opens the bank, checks it against the handle's shape and hands every record of
// layers [0, n_layers) to `sink` (the caller keeps only its shard).  For an EXL3 bank `layer_begin` hears every
// layer's K before the layer's first record.
int mlxs_bank_for_each_record(const char* dir, uint32_t bank_kind, uint64_t H, uint64_t I, uint64_t E, uint64_t n_layers,
                              uint32_t e_first, uint32_t e_count, int (*layer_begin)(void* ctx, uint32_t layer, uint32_t bits),
                              int (*sink)(void* ctx, uint32_t layer, uint32_t expert, const void* rec, uint64_t n), void* ctx) {
    Bank b;
    int fd = -1;
    int rc = open_checked(dir, b, fd);
    if (rc) return rc;
    const mlxs_bank_info& bi = b.info;
    const bool exl3 = !b.layer_bits.empty();
    const bool handle_exl3 = bank_kind == MLXS_BANK_EXL3_K3_MUL1 || bank_kind == MLXS_BANK_EXL3_K2_MUL1;
    if (exl3 ? !handle_exl3 : bi.bank_kind != bank_kind) {
        close(fd);
        return mlxs_fail(MLXS_E_MANIFEST, "load_bank: the bank at %s is kind %u, the handle is kind %u", dir, bi.bank_kind, bank_kind);
    }
    if (bi.hidden != H || bi.inter != I || bi.n_experts != E || bi.n_layers != n_layers) {
        close(fd);
        return mlxs_fail(MLXS_E_MANIFEST, "load_bank: dims %llu/%llu/%llu experts/%llu layers != the handle's %llu/%llu/%llu/%llu (DimsNotImplemented)",
                         (unsigned long long)bi.hidden, (unsigned long long)bi.inter, (unsigned long long)bi.n_experts, (unsigned long long)bi.n_layers,
                         (unsigned long long)H, (unsigned long long)I, (unsigned long long)E, (unsigned long long)n_layers);
    }
    const char* vs = getenv("MLXS_VERIFY_SHA256");
    const bool verify = vs ? atoi(vs) != 0 : bi.data_bytes <= (1ull << 30);  // small banks always, large ones on request
    std::vector<uint8_t> buf;
    for (uint64_t l = 0; l < n_layers && !rc; ++l) {
        const uint64_t logical = exl3 ? b.layer_logical[l] : bi.logical_bytes;
        if (exl3 && layer_begin && (rc = layer_begin(ctx, (uint32_t)l, b.layer_bits[l]))) break;
        for (uint64_t e = e_first; e < (uint64_t)e_first + e_count && !rc; ++e) {
            if ((rc = read_record(fd, b, l, e, verify, buf))) break;
            rc = sink(ctx, (uint32_t)l, (uint32_t)e, buf.data(), logical);
        }
    }
    close(fd);
    return rc;
}

// Bank.open for a host that only wants the check (src/expert/bank.zig:228-251): both manifests, the sidecar, and with
// verify_sha256 every record's digests; no device involved.
extern "C" int mlxs_moe_bank_verify(const char* dir, mlxs_bank_info* out, int verify_sha256) {
    if (!dir) return mlxs_fail(MLXS_E_ARG, "bank_verify: null argument");
    Bank b;
    int fd = -1;
    int rc = open_checked(dir, b, fd);
    if (rc) return rc;
    std::vector<uint8_t> buf;
    if (verify_sha256)
        for (uint64_t l = 0; l < b.info.n_layers && !rc; ++l)
            for (uint64_t e = 0; e < b.info.n_experts && !rc; ++e) rc = read_record(fd, b, l, e, true, buf);
    close(fd);
    if (!rc && out) *out = b.info;
    return rc;
}
