// Reader of the reference's `.cimage` container (src/quantization/cimage.rs):
//   "TRB_CIMG" | u64 LE header length | JSON header | payloads at 16 KB-aligned offsets
// header = {"tensors": {name: {"tensor_type": "Palettized4Bit"|"StandardFP16"|"Blob",
//                              "offset": u64, "size": u64, "dim_m": u32, "dim_n": u32}, ...},
//           "execution_plan": null | "<json string>"}      (cimage.rs:33-60, serde_json)
// PrismEngine::load (src/lut/engine_impl.rs:597-676) copies every palettized
// payload out of the file; here each one is re-laid straight into HBM, or,
// with the cache of the re-laid image, copied in its device layout.  The
// execution plan is parsed and kept (prism_cuda_cimage_plan); a missing or
// unparseable one is tolerated, as the reference does (`.ok()` at
// engine_impl.rs:638-641).  The reference stores the plan and never reads it
// again (engine_impl.rs:506-507, 670), so nothing here dispatches on it.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>

#include "common.cuh"

namespace prism {

struct CImageRecord {
    std::string type;
    uint64_t offset = 0, size = 0;
    uint32_t dim_m = 0, dim_n = 0;
};

// Minimal JSON reader: enough for the header serde_json writes.
struct Json {
    const char *p, *end;
    bool ok = true;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool eat(char c) { ws(); if (p < end && *p == c) { p++; return true; } return false; }
    std::string str() {
        std::string s;
        ws();
        if (p >= end || *p != '"') { ok = false; return s; }
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                p++;
                switch (*p) {
                case 'n': s += '\n'; break;
                case 't': s += '\t'; break;
                case 'r': s += '\r'; break;
                case 'b': s += '\b'; break;
                case 'f': s += '\f'; break;
                case 'u': {  // keep BMP code points below 0x80 exact, others as '?': keys are ASCII
                    unsigned v = 0;
                    for (int i = 0; i < 4 && p + 1 < end; i++) {
                        p++;
                        char ch = *p;
                        v = v * 16 + (ch >= '0' && ch <= '9' ? ch - '0' : (ch | 32) >= 'a' && (ch | 32) <= 'f' ? (ch | 32) - 'a' + 10 : 0);
                    }
                    s += v < 0x80 ? (char)v : '?';
                    break;
                }
                default: s += *p;
                }
                p++;
            } else {
                s += *p++;
            }
        }
        if (p >= end) { ok = false; return s; }
        p++;
        return s;
    }
    uint64_t num() {
        ws();
        uint64_t v = 0;
        bool any = false;
        while (p < end && *p >= '0' && *p <= '9') { v = v * 10 + (uint64_t)(*p - '0'); p++; any = true; }
        if (!any) ok = false;
        // tolerate a fractional/exponent tail (not produced for integer fields)
        while (p < end && (*p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-' || (*p >= '0' && *p <= '9'))) p++;
        return v;
    }
    void skip() {  // any value
        ws();
        if (p >= end) { ok = false; return; }
        if (*p == '"') { str(); return; }
        if (*p == '{' || *p == '[') {
            char open = *p, close = open == '{' ? '}' : ']';
            p++;
            ws();
            if (p < end && *p == close) { p++; return; }
            while (ok && p < end) {
                if (open == '{') { str(); if (!eat(':')) { ok = false; return; } }
                skip();
                if (eat(',')) continue;
                if (eat(close)) return;
                ok = false;
                return;
            }
            ok = false;
            return;
        }
        while (p < end && *p != ',' && *p != '}' && *p != ']') p++;  // number / true / false / null
    }
};

// The plan string of the header is itself JSON: ExecutionPlan of src/lut/graph.rs:552-589 as serde
// writes it -- {"version":1,"architecture":"...","num_layers":N,"node_backends":["MetalGemm",...],
// "kv_cache":"Fp16"|"Int8","attention_strategy":"...","lm_head_backend":"..."}.  Anything else (the
// plan schema of compute-core's writer, a truncated string) leaves version 0, as the reference's
// `.ok()` does (engine_impl.rs:638-641).
static void parse_plan(const std::string &plan_json, prism_cuda_ctx::PlanInfo &out) {
    prism_cuda_ctx::PlanInfo pi;
    Json j{plan_json.data(), plan_json.data() + plan_json.size()};
    bool have_version = false, have_nodes = false;
    if (!j.eat('{')) return;
    if (!j.eat('}')) {
        while (j.ok) {
            const std::string key = j.str();
            if (!j.eat(':')) { j.ok = false; break; }
            if (key == "version") { pi.version = (uint32_t)j.num(); have_version = true; }
            else if (key == "num_layers") pi.num_layers = (uint32_t)j.num();
            else if (key == "architecture") pi.architecture = j.str();
            else if (key == "attention_strategy") pi.attention_strategy = j.str();
            else if (key == "lm_head_backend") pi.lm_head_backend = j.str();
            else if (key == "kv_cache") {
                const std::string v = j.str();
                pi.kv_fp16 = v == "Fp16" ? 1 : v == "Int8" ? 0 : -1;
            } else if (key == "node_backends") {
                if (!j.eat('[')) { j.ok = false; break; }
                have_nodes = true;
                if (!j.eat(']')) {
                    while (j.ok) {
                        const std::string v = j.str();
                        pi.n_nodes++;
                        if (v == "MetalGemm" || v == "CpuGemm") pi.n_gemm_nodes++;
                        if (j.eat(',')) continue;
                        if (j.eat(']')) break;
                        j.ok = false;
                    }
                }
            } else {
                j.skip();
            }
            if (j.eat(',')) continue;
            if (j.eat('}')) break;
            j.ok = false;
        }
    }
    if (j.ok && have_version && have_nodes && pi.version != 0) out = pi;
}

static bool parse_header(const std::string &json, std::map<std::string, CImageRecord> &out, std::string &plan,
                         std::string &err) {
    Json j{json.data(), json.data() + json.size()};
    plan.clear();
    if (!j.eat('{')) { err = "parse header: not an object"; return false; }
    if (j.eat('}')) return true;
    while (j.ok) {
        std::string key = j.str();
        if (!j.eat(':')) { j.ok = false; break; }
        if (key == "tensors") {
            if (!j.eat('{')) { j.ok = false; break; }
            if (!j.eat('}')) {
                while (j.ok) {
                    std::string name = j.str();
                    if (!j.eat(':') || !j.eat('{')) { j.ok = false; break; }
                    CImageRecord r;
                    if (!j.eat('}')) {
                        while (j.ok) {
                            std::string f = j.str();
                            if (!j.eat(':')) { j.ok = false; break; }
                            if (f == "tensor_type") r.type = j.str();
                            else if (f == "offset") r.offset = j.num();
                            else if (f == "size") r.size = j.num();
                            else if (f == "dim_m") r.dim_m = (uint32_t)j.num();
                            else if (f == "dim_n") r.dim_n = (uint32_t)j.num();
                            else j.skip();
                            if (j.eat(',')) continue;
                            if (j.eat('}')) break;
                            j.ok = false;
                        }
                    }
                    out[name] = r;
                    if (j.eat(',')) continue;
                    if (j.eat('}')) break;
                    j.ok = false;
                }
            }
        } else if (key == "execution_plan") {
            j.ws();
            if (j.p < j.end && *j.p == '"') plan = j.str();  // Option<String>: a JSON string holding JSON
            else j.skip();                                    // null
        } else {
            j.skip();  // anything newer
        }
        if (j.eat(',')) continue;
        if (j.eat('}')) break;
        j.ok = false;
    }
    if (!j.ok) { err = "parse header: malformed JSON"; return false; }
    return true;
}

// ---- the file -------------------------------------------------------------------------------------------
struct CImageFile {
    FILE *f = nullptr;
    std::string json, plan;
    std::map<std::string, CImageRecord> recs;
    uint64_t fsize = 0;
    ~CImageFile() { if (f) fclose(f); }
};

static int open_cimage(prism_cuda_ctx *ctx, const char *path, CImageFile &c) {
    c.f = fopen(path, "rb");
    if (!c.f) return fail(ctx, PRISM_E_IO, std::string("open .cimage: ") + path);
    char magic[8];
    uint8_t szb[8];
    if (fread(magic, 1, 8, c.f) != 8) return fail(ctx, PRISM_E_IO, "read magic: short file");
    if (memcmp(magic, "TRB_CIMG", 8) != 0) return fail(ctx, PRISM_E_IO, "Invalid magic: expected TRB_CIMG");
    if (fread(szb, 1, 8, c.f) != 8) return fail(ctx, PRISM_E_IO, "read header size: short file");
    uint64_t hsz = 0;
    for (int i = 7; i >= 0; i--) hsz = (hsz << 8) | szb[i];
    if (hsz > (1ull << 30)) return fail(ctx, PRISM_E_IO, "read header: implausible header size");
    c.json.assign(hsz, '\0');
    if (hsz && fread(&c.json[0], 1, hsz, c.f) != hsz) return fail(ctx, PRISM_E_IO, "read header: short file");
    std::string err;
    if (!parse_header(c.json, c.recs, c.plan, err)) return fail(ctx, PRISM_E_IO, err);
    fseek(c.f, 0, SEEK_END);
    c.fsize = (uint64_t)ftell(c.f);
    ctx->plan = prism_cuda_ctx::PlanInfo{};
    if (!c.plan.empty()) parse_plan(c.plan, ctx->plan);
    return PRISM_OK;
}

static int upload_from_file(prism_cuda_ctx *ctx, CImageFile &c, uint32_t *n_out) {
    uint32_t n = 0;
    std::vector<uint8_t> buf;
    for (auto &kv : c.recs) {
        const CImageRecord &r = kv.second;
        if (r.type != "Palettized4Bit") continue;
        const uint64_t need = (uint64_t)r.dim_m * 32 + (uint64_t)r.dim_m * (r.dim_n / 2);
        if (r.size < need || r.offset + r.size > c.fsize)
            return fail(ctx, PRISM_E_IO, "tensor " + kv.first + ": payload outside the file or shorter than its dims");
        buf.resize(r.size);
        if (fseek(c.f, (long)r.offset, SEEK_SET) != 0 || fread(buf.data(), 1, r.size, c.f) != r.size)
            return fail(ctx, PRISM_E_IO, "tensor " + kv.first + ": short read");
        int32_t h;
        PRISM_TRY(prism_cuda_upload_palettized(ctx, kv.first.c_str(), buf.data(), buf.size(), r.dim_m, r.dim_n, 4, &h));
        n++;
    }
    if (n_out) *n_out = n;
    return PRISM_OK;
}

// ---- cache of the re-laid image ------------------------------------------------------------------------
// The device layout of every palettized tensor of a .cimage, written next to it after the first
// load, so that later loads skip the payload read and the re-lay kernels: one host-to-device copy
// of the index array and one of the palettes per tensor.  Layout (little endian):
//   "PRB2RLAY" | u32 version = 1 | u32 n_tensors | u64 key |
//   n_tensors x { u32 name_len | name | u32 dim_m | u32 dim_n | u32 bits | u64 idx_bytes | u64 pal_bytes } |
//   per tensor, in the same order: pal bytes, idx bytes.
// key = FNV-1a-64 over the container's header JSON and its file size: the header names every
// tensor's offset, size and dims, so any re-compilation of the model changes it.
constexpr char RELAY_MAGIC[8] = {'P', 'R', 'B', '2', 'R', 'L', 'A', 'Y'};

static uint64_t cimage_key(const CImageFile &c) {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](const uint8_t *p, size_t n) { for (size_t i = 0; i < n; i++) { h ^= p[i]; h *= 1099511628211ull; } };
    mix(reinterpret_cast<const uint8_t *>(c.json.data()), c.json.size());
    uint8_t sz[8];
    for (int i = 0; i < 8; i++) sz[i] = (uint8_t)(c.fsize >> (8 * i));
    mix(sz, 8);
    return h;
}

struct RelayEntry { std::string name; uint32_t m, k, bits; uint64_t idx_bytes, pal_bytes; };

static bool rd(FILE *f, void *p, size_t n) { return fread(p, 1, n, f) == n; }
static bool wr(FILE *f, const void *p, size_t n) { return fwrite(p, 1, n, f) == n; }

// 1: loaded from the cache, 0: no usable cache (nothing uploaded), < 0: error after uploads began
static int load_relay_cache(prism_cuda_ctx *ctx, const std::string &cache_path, uint64_t key, uint32_t *n_out) {
    FILE *f = fopen(cache_path.c_str(), "rb");
    if (!f) return 0;
    struct Closer { FILE *f; ~Closer() { fclose(f); } } closer{f};
    char magic[8];
    uint32_t ver = 0, n = 0;
    uint64_t k = 0;
    if (!rd(f, magic, 8) || memcmp(magic, RELAY_MAGIC, 8) != 0 || !rd(f, &ver, 4) || ver != 1 || !rd(f, &n, 4) || !rd(f, &k, 8) ||
        k != key || n > (1u << 20))
        return 0;
    std::vector<RelayEntry> ents(n);
    for (auto &e : ents) {
        uint32_t nl = 0;
        if (!rd(f, &nl, 4) || nl > 4096) return 0;
        e.name.assign(nl, '\0');
        if ((nl && !rd(f, &e.name[0], nl)) || !rd(f, &e.m, 4) || !rd(f, &e.k, 4) || !rd(f, &e.bits, 4) || !rd(f, &e.idx_bytes, 8) ||
            !rd(f, &e.pal_bytes, 8))
            return 0;
    }
    std::vector<uint8_t> buf;
    std::vector<int32_t> made;
    auto undo = [&]() { for (int32_t h : made) prism_cuda_free_tensor(ctx, h); };
    for (auto &e : ents) {
        int32_t h;
        int rc = alloc_tensor(ctx, e.name.c_str(), e.m, e.k, e.bits, &h);
        if (rc != PRISM_OK) { undo(); return rc; }
        made.push_back(h);
        const LutTensor &t = ctx->tensors[h];
        if (t.idx_bytes != e.idx_bytes || t.pal_bytes != e.pal_bytes) { undo(); return 0; }  // written by another layout version
        buf.resize(std::max(e.idx_bytes, e.pal_bytes));
        if (!rd(f, buf.data(), e.pal_bytes)) { undo(); return 0; }
        if (cudaMemcpy(t.pal, buf.data(), e.pal_bytes, cudaMemcpyHostToDevice) != cudaSuccess) { undo(); return cuda_fail(ctx, cudaGetLastError(), "cudaMemcpy(palettes)"); }
        if (!rd(f, buf.data(), e.idx_bytes)) { undo(); return 0; }
        if (cudaMemcpy(t.idx, buf.data(), e.idx_bytes, cudaMemcpyHostToDevice) != cudaSuccess) { undo(); return cuda_fail(ctx, cudaGetLastError(), "cudaMemcpy(indices)"); }
    }
    if (n_out) *n_out = n;
    return 1;
}

static int write_relay_cache(prism_cuda_ctx *ctx, const CImageFile &c, const std::string &cache_path, uint64_t key) {
    std::vector<int32_t> hs;
    for (auto &kv : c.recs) {
        if (kv.second.type != "Palettized4Bit") continue;
        auto it = ctx->by_name.find(kv.first);
        if (it == ctx->by_name.end()) return fail(ctx, PRISM_E_STATE, "relay cache: tensor " + kv.first + " is not on the device");
        hs.push_back(it->second);
    }
    const std::string tmp = cache_path + ".tmp";
    FILE *f = fopen(tmp.c_str(), "wb");
    if (!f) return fail(ctx, PRISM_E_IO, "relay cache: cannot create " + tmp);
    bool ok = true;
    const uint32_t ver = 1, n = (uint32_t)hs.size();
    ok = ok && wr(f, RELAY_MAGIC, 8) && wr(f, &ver, 4) && wr(f, &n, 4) && wr(f, &key, 8);
    for (int32_t h : hs) {
        const LutTensor &t = ctx->tensors[h];
        const uint32_t nl = (uint32_t)t.name.size();
        const uint64_t ib = t.idx_bytes, pb = t.pal_bytes;
        ok = ok && wr(f, &nl, 4) && wr(f, t.name.data(), nl) && wr(f, &t.m, 4) && wr(f, &t.k, 4) && wr(f, &t.bits, 4) && wr(f, &ib, 8) &&
             wr(f, &pb, 8);
    }
    std::vector<uint8_t> buf;
    cudaError_t ce = cudaStreamSynchronize(ctx->stream);
    for (int32_t h : hs) {
        if (!ok || ce != cudaSuccess) break;
        const LutTensor &t = ctx->tensors[h];
        buf.resize(std::max(t.idx_bytes, t.pal_bytes));
        ce = cudaMemcpy(buf.data(), t.pal, t.pal_bytes, cudaMemcpyDeviceToHost);
        ok = ok && ce == cudaSuccess && wr(f, buf.data(), t.pal_bytes);
        if (!ok) break;
        ce = cudaMemcpy(buf.data(), t.idx, t.idx_bytes, cudaMemcpyDeviceToHost);
        ok = ok && ce == cudaSuccess && wr(f, buf.data(), t.idx_bytes);
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok || ce != cudaSuccess || rename(tmp.c_str(), cache_path.c_str()) != 0) {
        remove(tmp.c_str());
        if (ce != cudaSuccess) return cuda_fail(ctx, ce, "relay cache: device read-back");
        return fail(ctx, PRISM_E_IO, "relay cache: write to " + cache_path + " failed");
    }
    return PRISM_OK;
}

}  // namespace prism

using namespace prism;

extern "C" int prism_cuda_engine_load_cimage(prism_cuda_engine *eng, const char *path, const char *key_prefix);

// Uploads every Palettized4Bit tensor of a .cimage file into the context.
// Returns the number of tensors uploaded through *n_out.
extern "C" int prism_cuda_load_cimage(prism_cuda_ctx *ctx, const char *path, uint32_t *n_out) {
    if (!ctx || !path) return fail(ctx, PRISM_E_NULL, "null argument");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    CImageFile c;
    PRISM_TRY(open_cimage(ctx, path, c));
    return upload_from_file(ctx, c, n_out);
}

extern "C" int prism_cuda_load_cimage_cached(prism_cuda_ctx *ctx, const char *path, const char *cache_path, uint32_t *n_out,
                                             int *hit_out) {
    if (!ctx || !path) return fail(ctx, PRISM_E_NULL, "null argument");
    if (hit_out) *hit_out = 0;
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    CImageFile c;
    PRISM_TRY(open_cimage(ctx, path, c));
    const std::string cp = (cache_path && *cache_path) ? std::string(cache_path) : std::string(path) + ".b200relay";
    const uint64_t key = cimage_key(c);
    const int got = load_relay_cache(ctx, cp, key, n_out);
    if (got < 0) return got;
    if (got == 1) {
        if (hit_out) *hit_out = 1;
        return PRISM_OK;
    }
    PRISM_TRY(upload_from_file(ctx, c, n_out));
    return write_relay_cache(ctx, c, cp, key);
}

extern "C" int prism_cuda_cimage_plan(prism_cuda_ctx *ctx, prism_cimage_plan *out) {
    if (!ctx || !out) return fail(ctx, PRISM_E_NULL, "null argument");
    memset(out, 0, sizeof *out);
    const prism_cuda_ctx::PlanInfo &p = ctx->plan;
    out->version = p.version; out->num_layers = p.num_layers; out->n_nodes = p.n_nodes; out->n_gemm_nodes = p.n_gemm_nodes;
    out->kv_fp16 = p.kv_fp16;
    snprintf(out->architecture, sizeof out->architecture, "%s", p.architecture.c_str());
    snprintf(out->attention_strategy, sizeof out->attention_strategy, "%s", p.attention_strategy.c_str());
    snprintf(out->lm_head_backend, sizeof out->lm_head_backend, "%s", p.lm_head_backend.c_str());
    return PRISM_OK;
}

extern "C" prism_cuda_ctx *prism_cuda_engine_ctx(prism_cuda_engine *eng);

extern "C" int prism_cuda_engine_load_cimage(prism_cuda_engine *eng, const char *path, const char *key_prefix) {
    if (!eng) return PRISM_E_NULL;
    prism_cuda_ctx *ctx = prism_cuda_engine_ctx(eng);
    uint32_t n = 0;
    if (ctx->cimage_cache) PRISM_TRY(prism_cuda_load_cimage_cached(ctx, path, nullptr, &n, nullptr));
    else PRISM_TRY(prism_cuda_load_cimage(ctx, path, &n));
    return prism_cuda_engine_bind_by_keys(eng, key_prefix);
}
