// Reader of the reference's `.cimage` container (src/quantization/cimage.rs):
//   "TRB_CIMG" | u64 LE header length | JSON header | payloads at 16 KB-aligned offsets
// header = {"tensors": {name: {"tensor_type": "Palettized4Bit"|"StandardFP16"|"Blob",
//                              "offset": u64, "size": u64, "dim_m": u32, "dim_n": u32}, ...},
//           "execution_plan": null | "<json string>"}      (cimage.rs:33-60, serde_json)
// PrismEngine::load (src/lut/engine_impl.rs:597-676) copies every palettized
// payload out of the file; here each one is re-laid straight into HBM.  A
// missing or unparseable execution plan is tolerated, as the reference does
// (`.ok()` at engine_impl.rs:638-641).
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

static bool parse_header(const std::string &json, std::map<std::string, CImageRecord> &out, std::string &err) {
    Json j{json.data(), json.data() + json.size()};
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
        } else {
            j.skip();  // execution_plan and anything newer
        }
        if (j.eat(',')) continue;
        if (j.eat('}')) break;
        j.ok = false;
    }
    if (!j.ok) { err = "parse header: malformed JSON"; return false; }
    return true;
}

}  // namespace prism

using namespace prism;

extern "C" int prism_cuda_engine_load_cimage(prism_cuda_engine *eng, const char *path, const char *key_prefix);

// Uploads every Palettized4Bit tensor of a .cimage file into the context.
// Returns the number of tensors uploaded through *n_out.
extern "C" int prism_cuda_load_cimage(prism_cuda_ctx *ctx, const char *path, uint32_t *n_out) {
    if (!ctx || !path) return fail(ctx, PRISM_E_NULL, "null argument");
    FILE *f = fopen(path, "rb");
    if (!f) return fail(ctx, PRISM_E_IO, std::string("open .cimage: ") + path);
    auto bail = [&](int code, const std::string &m) { fclose(f); return fail(ctx, code, m); };
    char magic[8];
    uint8_t szb[8];
    if (fread(magic, 1, 8, f) != 8) return bail(PRISM_E_IO, "read magic: short file");
    if (memcmp(magic, "TRB_CIMG", 8) != 0) return bail(PRISM_E_IO, "Invalid magic: expected TRB_CIMG");
    if (fread(szb, 1, 8, f) != 8) return bail(PRISM_E_IO, "read header size: short file");
    uint64_t hsz = 0;
    for (int i = 7; i >= 0; i--) hsz = (hsz << 8) | szb[i];
    if (hsz > (1ull << 30)) return bail(PRISM_E_IO, "read header: implausible header size");
    std::string json(hsz, '\0');
    if (hsz && fread(&json[0], 1, hsz, f) != hsz) return bail(PRISM_E_IO, "read header: short file");
    std::map<std::string, CImageRecord> recs;
    std::string err;
    if (!parse_header(json, recs, err)) return bail(PRISM_E_IO, err);
    fseek(f, 0, SEEK_END);
    const uint64_t fsize = (uint64_t)ftell(f);
    uint32_t n = 0;
    std::vector<uint8_t> buf;
    for (auto &kv : recs) {
        const CImageRecord &r = kv.second;
        if (r.type != "Palettized4Bit") continue;
        const uint64_t need = (uint64_t)r.dim_m * 32 + (uint64_t)r.dim_m * (r.dim_n / 2);
        if (r.size < need || r.offset + r.size > fsize)
            return bail(PRISM_E_IO, "tensor " + kv.first + ": payload outside the file or shorter than its dims");
        buf.resize(r.size);
        if (fseek(f, (long)r.offset, SEEK_SET) != 0 || fread(buf.data(), 1, r.size, f) != r.size)
            return bail(PRISM_E_IO, "tensor " + kv.first + ": short read");
        int32_t h;
        int rc = prism_cuda_upload_palettized(ctx, kv.first.c_str(), buf.data(), buf.size(), r.dim_m, r.dim_n, 4, &h);
        if (rc != PRISM_OK) { fclose(f); return rc; }
        n++;
    }
    fclose(f);
    if (n_out) *n_out = n;
    return PRISM_OK;
}

extern "C" prism_cuda_ctx *prism_cuda_engine_ctx(prism_cuda_engine *eng);

extern "C" int prism_cuda_engine_load_cimage(prism_cuda_engine *eng, const char *path, const char *key_prefix) {
    if (!eng) return PRISM_E_NULL;
    uint32_t n = 0;
    PRISM_TRY(prism_cuda_load_cimage(prism_cuda_engine_ctx(eng), path, &n));
    return prism_cuda_engine_bind_by_keys(eng, key_prefix);
}
