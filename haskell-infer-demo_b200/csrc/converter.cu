/*
 * converter.cu - the offline converter: a BF16 safetensors checkpoint + a model descriptor ->
 * `weights.manifest.json` and the raw artifacts under `artifacts/`, in the wire format the strict
 * reader (sidecar.cu; the reference's csrc/quant_manifest.c) accepts.
 *
 * Replaces scripts/quantize_weights.py `convert` (scripts/quantize_weights.py:155-325).  The reference
 * hands every tensor to its CPU quantizer through a subprocess and temporary files (1705 s for the
 * 27B checkpoint by its own account); here a tensor is widened to FP32, uploaded, quantized by
 * ffn_quantize_int4 (quantize.cu, byte-identical to the reference's arithmetic) and dequantized on the
 * GPU for the error figures the manifest carries.  Everything else is what the reference's converter
 * does, in its order: only BF16 sources and 2-D weights are admitted; the requested roles on layers
 * whose feed-forward is dense; one `<role>_layer<L>.packed/.scales` pair of files per tensor; the
 * gate||up pair by byte concatenation of its members; a precision map over every role of every
 * layer; the source files hashed before and after; keys sorted, two-space indent, final newline.
 */
#include <dirent.h>
#include <errno.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>

#include <algorithm>
#include <charconv>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"
#include "host_util.h"
#include "kernels.h"

namespace ffn {

/* ------------------------------------------------------------------------------------------- */
/* JSON output the way Python's json.dump(indent=2, sort_keys=True) writes it                      */
/* ------------------------------------------------------------------------------------------- */
struct JOut {
    enum Kind { Int, Real, Str, Arr, Obj } kind = Int;
    long long i = 0;
    double d = 0.0;
    std::string s;
    std::vector<JOut> a;
    std::map<std::string, JOut> o; /* byte order of the keys = Python's order for ASCII keys */
    static JOut integer(long long v) { JOut j; j.kind = Int; j.i = v; return j; }
    static JOut real(double v) { JOut j; j.kind = Real; j.d = v; return j; }
    static JOut str(const std::string &v) { JOut j; j.kind = Str; j.s = v; return j; }
    static JOut arr() { JOut j; j.kind = Arr; return j; }
    static JOut obj() { JOut j; j.kind = Obj; return j; }
    JOut &operator[](const char *key) { return o[key]; }
};

/* repr(float): the shortest digits that read back as the same double, fixed notation for decimal
 * exponents in [-4, 16), exponent notation (at least two exponent digits) otherwise */
static std::string py_float_repr(double v) {
    if (v != v) return "NaN";
    if (isinf(v)) return v > 0 ? "Infinity" : "-Infinity";
    if (v == 0.0) return signbit(v) ? "-0.0" : "0.0";
    char buf[64];
    /* shortest digits that read back as v, and among those the closest to v: std::to_chars guarantees both
     * (trying printf precisions does not: near a power of two the rounded candidate can miss) */
    const std::to_chars_result r = std::to_chars(buf, buf + sizeof(buf) - 1, v, std::chars_format::scientific);
    *r.ptr = '\0';
    /* buf = [-]d[.ddd]e[+-]XX */
    std::string text(buf);
    const bool neg = text[0] == '-';
    if (neg) text.erase(0, 1);
    const size_t epos = text.find('e');
    std::string digits = text.substr(0, epos);
    const int exp10 = atoi(text.c_str() + epos + 1);
    digits.erase(std::remove(digits.begin(), digits.end(), '.'), digits.end());
    while (digits.size() > 1 && digits.back() == '0') digits.pop_back();
    std::string out;
    if (exp10 >= -4 && exp10 < 16) {
        if (exp10 < 0) {
            out = "0." + std::string((size_t)(-exp10 - 1), '0') + digits;
        } else if ((int)digits.size() <= exp10 + 1) {
            out = digits + std::string((size_t)(exp10 + 1 - (int)digits.size()), '0') + ".0";
        } else {
            out = digits.substr(0, (size_t)exp10 + 1) + "." + digits.substr((size_t)exp10 + 1);
        }
    } else {
        out = digits.substr(0, 1);
        if (digits.size() > 1) out += "." + digits.substr(1);
        char e[16];
        snprintf(e, sizeof(e), "e%c%02d", exp10 < 0 ? '-' : '+', abs(exp10));
        out += e;
    }
    return neg ? "-" + out : out;
}

/* ensure_ascii=True: everything outside printable ASCII becomes \uXXXX (UTF-16 units) */
static void json_escape(const std::string &s, std::string &out) {
    out.push_back('"');
    for (size_t i = 0; i < s.size();) {
        const unsigned char c = (unsigned char)s[i];
        if (c < 0x80) {
            ++i;
            switch (c) {
                case '"': out += "\\\""; break;
                case '\\': out += "\\\\"; break;
                case '\n': out += "\\n"; break;
                case '\r': out += "\\r"; break;
                case '\t': out += "\\t"; break;
                case '\b': out += "\\b"; break;
                case '\f': out += "\\f"; break;
                default:
                    if (c < 0x20 || c == 0x7F) { char u[8]; snprintf(u, sizeof(u), "\\u%04x", c); out += u; }
                    else out.push_back((char)c);
            }
            continue;
        }
        /* decode one UTF-8 sequence; malformed bytes are written as U+FFFD */
        uint32_t cp = 0xFFFD;
        int len = c >= 0xF0 ? 4 : c >= 0xE0 ? 3 : c >= 0xC0 ? 2 : 1;
        if (len > 1 && i + (size_t)len <= s.size()) {
            cp = c & (0xFFu >> (len + 1));
            for (int k = 1; k < len; ++k) cp = (cp << 6) | ((unsigned char)s[i + k] & 0x3Fu);
        } else {
            len = 1;
        }
        i += (size_t)len;
        char u[16];
        if (cp >= 0x10000) {
            cp -= 0x10000;
            snprintf(u, sizeof(u), "\\u%04x\\u%04x", 0xD800 + (cp >> 10), 0xDC00 + (cp & 0x3FF));
        } else {
            snprintf(u, sizeof(u), "\\u%04x", cp);
        }
        out += u;
    }
    out.push_back('"');
}

static void json_write(const JOut &j, int level, std::string &out) {
    const std::string pad((size_t)(level + 1) * 2, ' '), close_pad((size_t)level * 2, ' ');
    switch (j.kind) {
        case JOut::Int: out += std::to_string(j.i); break;
        case JOut::Real: out += py_float_repr(j.d); break;
        case JOut::Str: json_escape(j.s, out); break;
        case JOut::Arr: {
            if (j.a.empty()) { out += "[]"; break; }
            out += "[\n";
            for (size_t k = 0; k < j.a.size(); ++k) {
                out += pad;
                json_write(j.a[k], level + 1, out);
                out += k + 1 < j.a.size() ? ",\n" : "\n";
            }
            out += close_pad + "]";
            break;
        }
        case JOut::Obj: {
            if (j.o.empty()) { out += "{}"; break; }
            out += "{\n";
            size_t k = 0;
            for (const auto &kv : j.o) {
                out += pad;
                json_escape(kv.first, out);
                out += ": ";
                json_write(kv.second, level + 1, out);
                out += ++k < j.o.size() ? ",\n" : "\n";
            }
            out += close_pad + "}";
            break;
        }
    }
}

/* ------------------------------------------------------------------------------------------- */
/* Files                                                                                          */
/* ------------------------------------------------------------------------------------------- */
static bool read_whole_file(const std::string &path, std::vector<uint8_t> &out) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    bool ok = fseek(f, 0, SEEK_END) == 0;
    const long size = ok ? ftell(f) : -1;
    ok = ok && size >= 0 && fseek(f, 0, SEEK_SET) == 0;
    if (ok) {
        out.resize((size_t)size);
        ok = size == 0 || fread(out.data(), 1, (size_t)size, f) == (size_t)size;
    }
    fclose(f);
    return ok;
}

static bool write_whole_file(const std::string &path, const void *data, size_t bytes) {
    FILE *f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const bool ok = bytes == 0 || fwrite(data, 1, bytes, f) == bytes;
    return fclose(f) == 0 && ok;
}

/* size and SHA-256 of a file, streamed in 1 MiB blocks (sources are gigabytes) */
static bool hash_file(const std::string &path, long long *bytes, std::string *hex) {
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return false;
    Sha256 sha;
    std::vector<uint8_t> block(1 << 20);
    long long total = 0;
    size_t got;
    while ((got = fread(block.data(), 1, block.size(), f)) > 0) {
        sha.update(block.data(), got);
        total += (long long)got;
    }
    const bool ok = !ferror(f);
    fclose(f);
    if (!ok) return false;
    char digest[65];
    sha.finish(digest);
    *bytes = total;
    *hex = digest;
    return true;
}

static std::string sha_hex_of(const void *data, size_t bytes) {
    Sha256 sha;
    sha.update((const uint8_t *)data, bytes);
    char digest[65];
    sha.finish(digest);
    return digest;
}

static std::string absolute_path(const char *path) {
    char buf[4096];
    if (realpath(path, buf)) return buf;
    return path; /* os.path.abspath would not fail either; the reader does not interpret it */
}

/* ------------------------------------------------------------------------------------------- */
/* The checkpoint: every *.safetensors shard of a directory, name -> where its bytes are          */
/* (scripts/quantize_weights.py:68-91: 8-byte little-endian header length, JSON header,           */
/* data_offsets relative to the end of the header)                                                */
/* ------------------------------------------------------------------------------------------- */
struct TensorInfo {
    std::string file, dtype;
    std::vector<long long> shape;
    long long start = 0, stop = 0; /* absolute byte offsets in the file */
};

static int index_checkpoint(const char *model_dir, std::vector<std::string> &shards, std::map<std::string, TensorInfo> &index) {
    DIR *dir = opendir(model_dir);
    if (!dir) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: cannot open %s: %s", model_dir, strerror(errno));
    while (struct dirent *e = readdir(dir)) {
        const std::string name = e->d_name;
        if (name.size() > 12 && name.compare(name.size() - 12, 12, ".safetensors") == 0) shards.push_back(name);
    }
    closedir(dir);
    std::sort(shards.begin(), shards.end());
    for (const std::string &name : shards) {
        const std::string path = std::string(model_dir) + "/" + name;
        FILE *f = fopen(path.c_str(), "rb");
        if (!f) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: cannot open %s", path.c_str());
        uint8_t len8[8];
        unsigned long long header_len = 0;
        bool ok = fread(len8, 1, 8, f) == 8;
        for (int b = 7; ok && b >= 0; --b) header_len = (header_len << 8) | len8[b];
        ok = ok && header_len > 0 && header_len < (1ull << 31);
        std::string header;
        if (ok) {
            header.resize((size_t)header_len);
            ok = fread(&header[0], 1, (size_t)header_len, f) == (size_t)header_len;
        }
        fclose(f);
        if (!ok) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: %s has no readable safetensors header", path.c_str());
        JsonReader reader(header.c_str());
        Json doc;
        if (!reader.value(doc) || doc.kind != Json::Obj)
            return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: the header of %s is not a JSON object", path.c_str());
        const long long data_start = 8 + (long long)header_len;
        for (const auto &kv : doc.o) {
            if (kv.first == "__metadata__") continue;
            const Json *dtype = kv.second.get("dtype"), *shape = kv.second.get("shape"), *offs = kv.second.get("data_offsets");
            if (!dtype || dtype->kind != Json::Str || !shape || shape->kind != Json::Arr || !offs || offs->kind != Json::Arr ||
                offs->a.size() != 2 || offs->a[0].kind != Json::Int || offs->a[1].kind != Json::Int)
                return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: %s describes %s incompletely", path.c_str(), kv.first.c_str());
            if (index.count(kv.first)) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: %s appears in two shards", kv.first.c_str());
            TensorInfo t;
            t.file = path; t.dtype = dtype->s;
            for (const Json &d : shape->a) {
                if (d.kind != Json::Int) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: %s has a non-integer extent", kv.first.c_str());
                t.shape.push_back(d.i);
            }
            t.start = data_start + offs->a[0].i; t.stop = data_start + offs->a[1].i;
            index[kv.first] = t;
        }
    }
    return FFN_OK;
}

/* A BF16 tensor widened to FP32 (exact): the quantizer consumes FP32 source values. */
static int read_tensor_f32(const std::string &name, const TensorInfo &t, std::vector<float> &out) {
    if (t.dtype != "BF16") return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: only BF16 sources are admitted, got %s", t.dtype.c_str());
    if (t.shape.size() != 2) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: %s is not a 2-D weight", name.c_str());
    const long long elems = t.shape[0] * t.shape[1];
    if (t.shape[0] <= 0 || t.shape[1] <= 0 || t.stop - t.start != elems * 2)
        return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: %s holds %lld bytes, its shape needs %lld", name.c_str(),
                     t.stop - t.start, elems * 2);
    std::vector<uint16_t> raw((size_t)elems);
    FILE *f = fopen(t.file.c_str(), "rb");
    bool ok = f && fseek(f, (long)t.start, SEEK_SET) == 0 && fread(raw.data(), 2, (size_t)elems, f) == (size_t)elems;
    if (f) fclose(f);
    if (!ok) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: cannot read %s from %s", name.c_str(), t.file.c_str());
    out.resize((size_t)elems);
    for (long long i = 0; i < elems; ++i) {
        const uint32_t bits = (uint32_t)raw[(size_t)i] << 16;
        memcpy(&out[(size_t)i], &bits, 4);
    }
    return FFN_OK;
}

/* "model.layers.%d.mlp.up_proj.weight" % layer */
static std::string tensor_name(const std::string &templ, int layer) {
    const size_t at = templ.find("%d");
    if (at == std::string::npos) return templ;
    return templ.substr(0, at) + std::to_string(layer) + templ.substr(at + 2);
}

/* ------------------------------------------------------------------------------------------- */
/* One tensor through the GPU: quantize, and measure what the artifact implies                    */
/* ------------------------------------------------------------------------------------------- */
struct DeviceBuffers { /* grown on demand, freed when the conversion ends */
    float *w = nullptr, *deq = nullptr;
    uint8_t *packed = nullptr;
    uint16_t *scales = nullptr;
    int *bad = nullptr;
    size_t elems = 0;
    ~DeviceBuffers() { release(); }
    void release() {
        if (w) cudaFree(w);
        if (deq) cudaFree(deq);
        if (packed) cudaFree(packed);
        if (scales) cudaFree(scales);
        if (bad) cudaFree(bad);
        w = deq = nullptr; packed = nullptr; scales = nullptr; bad = nullptr; elems = 0;
    }
    int reserve(size_t n) {
        if (n <= elems) return FFN_OK;
        release();
        if (cudaMalloc(&w, n * 4) != cudaSuccess || cudaMalloc(&deq, n * 4) != cudaSuccess ||
            cudaMalloc(&packed, n / 2) != cudaSuccess || cudaMalloc(&scales, n / FFN_INT4_GROUP * 2) != cudaSuccess ||
            cudaMalloc(&bad, sizeof(int)) != cudaSuccess) {
            const cudaError_t e = cudaGetLastError();
            release();
            return fail(e == cudaErrorMemoryAllocation ? FFN_ERR_ALLOC : FFN_ERR_CUDA,
                        "ffn_convert_checkpoint: cannot get device memory for a tensor of %zu elements: %s", n, cudaGetErrorString(e));
        }
        elems = n;
        return FFN_OK;
    }
};

extern "C" int ffn_quantize_int4(const void *weights, void *packed, void *scales, long long n, long long k, void *stream);

struct ErrorStats {
    double max_abs = 0.0, sum_sq = 0.0;
    long long count = 0;
};

static int quantize_tensor(DeviceBuffers &dev, const std::vector<float> &src, long long n, long long k,
                           std::vector<uint8_t> &packed, std::vector<uint8_t> &scales, ErrorStats &err) {
    const size_t elems = (size_t)(n * k);
    int st = dev.reserve(elems);
    if (st) return st;
    FFN_CUDA_TRY(cudaMemcpy(dev.w, src.data(), elems * 4, cudaMemcpyHostToDevice), "ffn_convert_checkpoint: upload");
    st = ffn_quantize_int4(dev.w, dev.packed, dev.scales, n, k, nullptr);
    if (st) return st; /* the quantizer's own message names the element or group */
    packed.resize(elems / 2);
    scales.resize(elems / FFN_INT4_GROUP * 2);
    FFN_CUDA_TRY(cudaMemcpy(packed.data(), dev.packed, packed.size(), cudaMemcpyDeviceToHost), "ffn_convert_checkpoint: download");
    FFN_CUDA_TRY(cudaMemcpy(scales.data(), dev.scales, scales.size(), cudaMemcpyDeviceToHost), "ffn_convert_checkpoint: download");
    /* the error the artifact implies against the source values, per element */
    FFN_CUDA_TRY(cudaMemset(dev.bad, 0, sizeof(int)), "ffn_convert_checkpoint: memset");
    st = dequantize_int4(dev.deq, dev.packed, dev.scales, (int)n, (int)k, dev.bad, nullptr);
    if (st) return st;
    std::vector<float> deq(elems);
    FFN_CUDA_TRY(cudaMemcpy(deq.data(), dev.deq, elems * 4, cudaMemcpyDeviceToHost), "ffn_convert_checkpoint: download");
    for (size_t i = 0; i < elems; ++i) {
        const float diff = fabsf(src[i] - deq[i]);
        if ((double)diff > err.max_abs) err.max_abs = (double)diff;
        err.sum_sq += (double)diff * (double)diff;
    }
    err.count += (long long)elems;
    return FFN_OK;
}

static JOut artifact_json(const std::string &file, const char *dtype, const std::vector<uint8_t> &bytes, bool is_scales) {
    JOut a = JOut::obj();
    a["file"] = JOut::str(file);
    a["dtype"] = JOut::str(dtype);
    a["bytes"] = JOut::integer((long long)bytes.size());
    a["sha256"] = JOut::str(sha_hex_of(bytes.data(), bytes.size()));
    if (is_scales) a["count"] = JOut::integer((long long)bytes.size() / 2);
    return a;
}

}  // namespace ffn

static const char kFormatArithmetic[] = "csrc/linear_weight.cpp (the Q0 reference)";

using namespace ffn;

extern "C" int ffn_convert_checkpoint(const char *model_dir, const char *descriptor_path, const char *out_dir,
                                      const char *const *roles, int num_roles, int limit_layers) {
    clear_error();
    if (!model_dir || !descriptor_path || !out_dir) return fail(FFN_ERR_CONFIG, "ffn_convert_checkpoint: null argument");
    static const char *const kDefaultRoles[] = {"mlpGate", "mlpUp", "mlpDown"};
    if (!roles || num_roles <= 0) { roles = kDefaultRoles; num_roles = 3; }

    /* ---- the descriptor: which tensors are the requested roles of the dense layers */
    std::vector<uint8_t> desc_bytes;
    if (!read_whole_file(descriptor_path, desc_bytes)) return fail(FFN_ERR_CONFIG, "ffn_convert_checkpoint: cannot read %s", descriptor_path);
    const std::string desc_text(desc_bytes.begin(), desc_bytes.end());
    JsonReader reader(desc_text.c_str());
    Json desc;
    if (!reader.value(desc) || desc.kind != Json::Obj) return fail(FFN_ERR_CONFIG, "ffn_convert_checkpoint: %s is not a JSON object", descriptor_path);
    const Json *jl = desc.get("num_layers"), *jf = desc.get("layer_ffns"), *jn = desc.get("role_names"), *jt = desc.get("role_templates");
    if (!jl || jl->kind != Json::Int || !jf || jf->kind != Json::Arr || !jn || jn->kind != Json::Arr || !jt || jt->kind != Json::Arr)
        return fail(FFN_ERR_CONFIG, "ffn_convert_checkpoint: the descriptor lacks num_layers / layer_ffns / role_names / role_templates");
    if (jn->a.size() != jt->a.size()) return fail(FFN_ERR_CONFIG, "ffn_convert_checkpoint: the descriptor's role names and templates differ");
    const int num_layers = (int)jl->i;
    if (num_layers < 0 || (long long)jf->a.size() < num_layers)
        return fail(FFN_ERR_CONFIG, "ffn_convert_checkpoint: the descriptor names %d layers but %zu feed-forward kinds", num_layers, jf->a.size());
    for (size_t r = 0; r < jn->a.size(); ++r)
        if (jn->a[r].kind != Json::Str || jt->a[r].kind != Json::Str)
            return fail(FFN_ERR_CONFIG, "ffn_convert_checkpoint: a role name or template is not a string");

    struct Instance { int layer, role_index; std::string role, tensor; };
    std::vector<Instance> instances;
    for (int layer = 0; layer < num_layers; ++layer) {
        if (jf->a[(size_t)layer].kind != Json::Str || jf->a[(size_t)layer].s != "dense") continue;
        if (limit_layers >= 0 && layer >= limit_layers) continue;
        for (size_t r = 0; r < jn->a.size(); ++r) {
            bool wanted = false;
            for (int q = 0; q < num_roles; ++q) wanted = wanted || jn->a[r].s == roles[q];
            if (wanted) instances.push_back({layer, (int)r, jn->a[r].s, tensor_name(jt->a[r].s, layer)});
        }
    }

    /* ---- the checkpoint, hashed before anything is written */
    std::vector<std::string> shards;
    std::map<std::string, TensorInfo> index;
    int st = index_checkpoint(model_dir, shards, index);
    if (st) return st;
    std::vector<std::pair<long long, std::string>> before(shards.size());
    for (size_t k = 0; k < shards.size(); ++k)
        if (!hash_file(std::string(model_dir) + "/" + shards[k], &before[k].first, &before[k].second))
            return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: cannot hash %s", shards[k].c_str());

    const std::string root(out_dir), art_dir = root + "/artifacts";
    if ((mkdir(root.c_str(), 0777) != 0 && errno != EEXIST) || (mkdir(art_dir.c_str(), 0777) != 0 && errno != EEXIST))
        return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: cannot create %s: %s", art_dir.c_str(), strerror(errno));

    /* ---- every admitted tensor */
    DeviceBuffers dev;
    ErrorStats err;
    JOut entries = JOut::arr(), pairs = JOut::arr(), cells = JOut::arr();
    struct Written { int layer; std::string role; int role_index; long long n, k; std::vector<uint8_t> packed, scales; };
    std::vector<std::unique_ptr<Written>> gate_up; /* members kept until their layer's pair is written */
    std::vector<float> source;
    /* ---- the gate||up pair of a layer, as soon as both members exist (their bytes are dropped right after):
     * byte concatenation, gate rows first */
    auto emit_pair = [&](int layer) -> int {
        const Written *gate = nullptr, *up = nullptr;
        for (const auto &w : gate_up) {
            if (w->layer != layer) continue;
            if (w->role == "mlpGate") gate = w.get(); else up = w.get();
        }
        if (!gate || !up) return FFN_OK;
        if (gate->k != up->k) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: layer %d's gate and up differ in K", layer);
        std::vector<uint8_t> packed(gate->packed), scales(gate->scales);
        packed.insert(packed.end(), up->packed.begin(), up->packed.end());
        scales.insert(scales.end(), up->scales.begin(), up->scales.end());
        const std::string stem = "mlpGateUp_layer" + std::to_string(layer);
        if (!write_whole_file(art_dir + "/" + stem + ".packed", packed.data(), packed.size()) ||
            !write_whole_file(art_dir + "/" + stem + ".scales", scales.data(), scales.size()))
            return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: cannot write the artifacts of %s", stem.c_str());
        JOut p = JOut::obj();
        p["name"] = JOut::str("mlpGateUp");
        p["layer"] = JOut::integer(layer);
        JOut members = JOut::arr();
        for (const Written *m : {gate, up}) {
            JOut mj = JOut::obj();
            mj["role"] = JOut::str(m->role);
            mj["role_index"] = JOut::integer(m->role_index);
            members.a.push_back(mj);
        }
        p["members"] = members;
        p["rule"] = JOut::str("row concatenation: gate rows then up rows, which is the [2I, H] weight layout F1's packed "
                              "gate/up GEMM takes and the row-interleaved [T, 2I] output its activation expects");
        JOut shape = JOut::arr();
        shape.a.push_back(JOut::integer(gate->n + up->n)); shape.a.push_back(JOut::integer(gate->k));
        p["logical_shape"] = shape;
        p["packed"] = artifact_json("artifacts/" + stem + ".packed", "u8", packed, false);
        p["scales"] = artifact_json("artifacts/" + stem + ".scales", "bf16", scales, true);
        p["group"] = JOut::integer(FFN_INT4_GROUP);
        pairs.a.push_back(p);
        gate_up.erase(std::remove_if(gate_up.begin(), gate_up.end(), [&](const std::unique_ptr<Written> &w) { return w->layer == layer; }),
                      gate_up.end());
        return FFN_OK;
    };

    for (const Instance &inst : instances) {
        const auto found = index.find(inst.tensor);
        if (found == index.end()) return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: %s is not in the checkpoint", inst.tensor.c_str());
        st = read_tensor_f32(inst.tensor, found->second, source);
        if (st) return st;
        const long long n = found->second.shape[0], k = found->second.shape[1];
        std::unique_ptr<Written> w(new Written{inst.layer, inst.role, inst.role_index, n, k, {}, {}});
        st = quantize_tensor(dev, source, n, k, w->packed, w->scales, err);
        if (st) return st;
        const std::string stem = inst.role + "_layer" + std::to_string(inst.layer);
        if (!write_whole_file(art_dir + "/" + stem + ".packed", w->packed.data(), w->packed.size()) ||
            !write_whole_file(art_dir + "/" + stem + ".scales", w->scales.data(), w->scales.size()))
            return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: cannot write the artifacts of %s", stem.c_str());
        JOut e = JOut::obj();
        e["role"] = JOut::str(inst.role);
        e["role_index"] = JOut::integer(inst.role_index);
        e["layer"] = JOut::integer(inst.layer);
        e["checkpoint_tensor"] = JOut::str(inst.tensor);
        JOut shape = JOut::arr();
        shape.a.push_back(JOut::integer(n)); shape.a.push_back(JOut::integer(k));
        e["logical_shape"] = shape;
        e["local_shape"] = shape;
        e["packed"] = artifact_json("artifacts/" + stem + ".packed", "u8", w->packed, false);
        e["scales"] = artifact_json("artifacts/" + stem + ".scales", "bf16", w->scales, true);
        e["group_axis"] = JOut::str("k");
        e["group"] = JOut::integer(FFN_INT4_GROUP);
        entries.a.push_back(e);
        if (inst.role == "mlpGate" || inst.role == "mlpUp") {
            gate_up.push_back(std::move(w));
            if ((st = emit_pair(inst.layer))) return st;
        }
    }

    /* ---- the precision map: every role of every layer, quantized or retained */
    for (int layer = 0; layer < num_layers; ++layer)
        for (size_t r = 0; r < jn->a.size(); ++r) {
            bool admitted = false;
            for (const Instance &inst : instances) admitted = admitted || (inst.layer == layer && inst.role == jn->a[r].s);
            JOut c = JOut::obj();
            c["role"] = JOut::str(jn->a[r].s);
            c["layer"] = JOut::integer(layer);
            c["precision"] = JOut::str(admitted ? "int4" : "bf16");
            c["checkpoint_tensor"] = JOut::str(tensor_name(jt->a[r].s, layer));
            cells.a.push_back(c);
        }

    /* ---- the source must not have changed while it was being read */
    for (size_t k = 0; k < shards.size(); ++k) {
        long long bytes = 0;
        std::string hex;
        if (!hash_file(std::string(model_dir) + "/" + shards[k], &bytes, &hex) || bytes != before[k].first || hex != before[k].second)
            return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: the source checkpoint changed during conversion");
    }

    JOut doc = JOut::obj();
    doc["manifest_version"] = JOut::integer(1);
    JOut format = JOut::obj();
    format["name"] = JOut::str("int4_symmetric_group_bf16_scale");
    format["abi_version"] = JOut::integer(1);
    format["group"] = JOut::integer(FFN_INT4_GROUP);
    format["qmin"] = JOut::integer(-7);
    format["qmax"] = JOut::integer(7);
    format["invalid_code"] = JOut::integer(-8);
    format["zero_point"] = JOut::integer(0);
    format["packed_dtype"] = JOut::str("u8");
    format["scale_dtype"] = JOut::str("bf16");
    format["packing"] = JOut::str("two_twos_complement_nibbles_per_byte_lower_k_index_in_low_nibble");
    format["arithmetic"] = JOut::str(kFormatArithmetic); /* the definition followed; the reference's --verify compares it */
    doc["format"] = format;
    JOut converter = JOut::obj();
    converter["name"] = JOut::str("libffn_int4 ffn_convert_checkpoint");
    converter["version"] = JOut::integer(1);
    doc["converter"] = converter;
    JOut src = JOut::obj(), files = JOut::arr();
    src["model_dir"] = JOut::str(absolute_path(model_dir));
    for (size_t k = 0; k < shards.size(); ++k) {
        JOut f = JOut::obj();
        f["name"] = JOut::str(shards[k]);
        f["bytes"] = JOut::integer(before[k].first);
        f["sha256"] = JOut::str(before[k].second);
        files.a.push_back(f);
    }
    src["files"] = files;
    doc["source"] = src;
    JOut dj = JOut::obj();
    dj["path"] = JOut::str(absolute_path(descriptor_path));
    dj["sha256"] = JOut::str(sha_hex_of(desc_bytes.data(), desc_bytes.size()));
    doc["descriptor"] = dj;
    JOut qe = JOut::obj();
    qe["max_abs"] = JOut::real(err.max_abs);
    qe["rms"] = JOut::real(err.count ? sqrt(err.sum_sq / (double)err.count) : 0.0);
    qe["elements"] = JOut::integer(err.count);
    qe["note"] = JOut::str("measured against the source BF16 checkpoint's FP32 values, per element");
    doc["quantization_error"] = qe;
    doc["precision_map"] = cells;
    doc["entries"] = entries;
    doc["pairs"] = pairs;
    std::string text;
    json_write(doc, 0, text);
    text.push_back('\n');
    if (!write_whole_file(root + "/weights.manifest.json", text.data(), text.size()))
        return fail(FFN_ERR_WEIGHTS, "ffn_convert_checkpoint: cannot write %s/weights.manifest.json", out_dir);
    return FFN_OK;
}

/* ------------------------------------------------------------------------------------------- */
/* Verification: re-derive what the manifest claims (scripts/quantize_weights.py:328-461, `verify`) */
/* ------------------------------------------------------------------------------------------- */
namespace ffn {

static std::string key_text(long long layer, const std::string &role) { /* Python's repr of (layer, role) */
    return "(" + std::to_string(layer) + ", '" + role + "')";
}
static bool file_exists(const std::string &path) {
    struct stat st;
    return stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}
static long long file_size(const std::string &path) {
    struct stat st;
    return stat(path.c_str(), &st) == 0 ? (long long)st.st_size : -1;
}
static std::string jstr(const Json *j, const char *key) {
    const Json *v = j ? j->get(key) : nullptr;
    return v && v->kind == Json::Str ? v->s : std::string();
}
static long long jint(const Json *j, const char *key, long long missing = -1) {
    const Json *v = j ? j->get(key) : nullptr;
    return v && v->kind == Json::Int ? v->i : missing;
}
static std::string dirname_of(const std::string &path) {
    const size_t slash = path.find_last_of('/');
    return slash == std::string::npos ? "." : path.substr(0, slash);
}

}  // namespace ffn

extern "C" int ffn_verify_sidecar(const char *manifest_path, int rederive_samples, char *report, size_t report_bytes) {
    clear_error();
    if (!manifest_path || (report_bytes && !report)) return fail(FFN_ERR_CONFIG, "ffn_verify_sidecar: null argument");
    std::vector<uint8_t> raw;
    if (!read_whole_file(manifest_path, raw)) return fail(FFN_ERR_WEIGHTS, "ffn_verify_sidecar: cannot read %s", manifest_path);
    const std::string text(raw.begin(), raw.end());
    JsonReader reader(text.c_str());
    Json doc;
    if (!reader.value(doc) || doc.kind != Json::Obj) return fail(FFN_ERR_WEIGHTS, "ffn_verify_sidecar: %s is not a JSON object", manifest_path);
    std::vector<std::string> problems;
    auto require = [&](bool ok, const std::string &message) { if (!ok) problems.push_back(message); };

    require(jint(&doc, "manifest_version") == 1, "unknown manifest version " + std::to_string(jint(&doc, "manifest_version")));
    const Json *fmt = doc.get("format");
    const std::pair<const char *, long long> ints[] = {{"abi_version", 1}, {"group", FFN_INT4_GROUP}, {"qmin", -7}, {"qmax", 7},
                                                       {"invalid_code", -8}, {"zero_point", 0}};
    for (const auto &kv : ints)
        require(jint(fmt, kv.first, -99) == kv.second, std::string("the format's ") + kv.first + " is " +
                std::to_string(jint(fmt, kv.first, -99)) + ", expected " + std::to_string(kv.second));
    const std::pair<const char *, const char *> strs[] = {
        {"name", "int4_symmetric_group_bf16_scale"}, {"packed_dtype", "u8"}, {"scale_dtype", "bf16"},
        {"packing", "two_twos_complement_nibbles_per_byte_lower_k_index_in_low_nibble"}, {"arithmetic", kFormatArithmetic}};
    for (const auto &kv : strs)
        require(jstr(fmt, kv.first) == kv.second, std::string("the format's ") + kv.first + " is " + jstr(fmt, kv.first) +
                ", expected " + kv.second);

    const std::string out_dir = dirname_of(absolute_path(manifest_path));
    const Json *source = doc.get("source");
    const std::string source_dir = jstr(source, "model_dir");
    const Json *files = source ? source->get("files") : nullptr;
    if (files && files->kind == Json::Arr)
        for (const Json &rec : files->a) {
            const std::string name = jstr(&rec, "name"), path = source_dir + "/" + name;
            require(file_exists(path), "the source file " + name + " is gone");
            if (file_exists(path)) {
                long long bytes = 0;
                std::string hex;
                require(hash_file(path, &bytes, &hex) && hex == jstr(&rec, "sha256"),
                        "the source file " + name + " no longer matches its checksum");
            }
        }

    /* ---- entries: shapes the format admits, artifacts present, sized and hashed as recorded */
    const Json *entries = doc.get("entries");
    if (!entries || entries->kind != Json::Arr) return fail(FFN_ERR_WEIGHTS, "ffn_verify_sidecar: the manifest has no entries array");
    std::map<std::pair<long long, std::string>, const Json *> by_key;
    for (const Json &e : entries->a) {
        const long long layer = jint(&e, "layer");
        const std::string role = jstr(&e, "role"), key = key_text(layer, role);
        require(!by_key.count({layer, role}), key + " appears twice");
        by_key[{layer, role}] = &e;
        const Json *shape = e.get("logical_shape");
        long long n = 0, k = 0;
        if (shape && shape->kind == Json::Arr && shape->a.size() == 2) { n = shape->a[0].i; k = shape->a[1].i; }
        require(n > 0 && k > 0 && n % 8 == 0 && k % FFN_INT4_GROUP == 0,
                key + " has a shape the format does not admit: " + std::to_string(n) + "x" + std::to_string(k));
        const Json *pa = e.get("packed"), *sa = e.get("scales");
        const std::string packed = out_dir + "/" + jstr(pa, "file"), scales = out_dir + "/" + jstr(sa, "file");
        require(file_exists(packed), key + " has no payload at " + jstr(pa, "file"));
        require(file_exists(scales), key + " has no scales at " + jstr(sa, "file"));
        long long bytes = 0;
        std::string hex;
        if (file_exists(packed)) {
            require(file_size(packed) == n * k / 2, key + " packs to " + std::to_string(file_size(packed)) + " bytes, expected " +
                    std::to_string(n * k / 2));
            require(hash_file(packed, &bytes, &hex) && hex == jstr(pa, "sha256"), key + " payload does not match its checksum");
        }
        if (file_exists(scales)) {
            const long long expected = 2 * n * (k / FFN_INT4_GROUP);
            require(file_size(scales) == expected, key + " scales are " + std::to_string(file_size(scales)) + " bytes, expected " +
                    std::to_string(expected));
            require(hash_file(scales, &bytes, &hex) && hex == jstr(sa, "sha256"), key + " scales do not match their checksum");
        }
    }

    /* ---- the precision map covers every role of every layer once and agrees with the entries */
    const Json *dj = doc.get("descriptor");
    const std::string desc_path = jstr(dj, "path");
    std::vector<uint8_t> desc_raw;
    Json desc;
    size_t covered_cells = 0;
    if (!read_whole_file(desc_path, desc_raw)) {
        problems.push_back("the descriptor " + desc_path + " cannot be read");
    } else {
        require(sha_hex_of(desc_raw.data(), desc_raw.size()) == jstr(dj, "sha256"), "the descriptor no longer matches its checksum");
        const std::string desc_text(desc_raw.begin(), desc_raw.end());
        JsonReader dreader(desc_text.c_str());
        if (!dreader.value(desc) || desc.kind != Json::Obj) problems.push_back("the descriptor is not a JSON object");
    }
    std::map<std::pair<long long, std::string>, bool> covered;
    const Json *pmap = doc.get("precision_map");
    if (pmap && pmap->kind == Json::Arr)
        for (const Json &rec : pmap->a) {
            const long long layer = jint(&rec, "layer");
            const std::string role = jstr(&rec, "role"), key = key_text(layer, role);
            require(!covered.count({layer, role}), "the precision map lists " + key + " twice");
            covered[{layer, role}] = true;
            require((jstr(&rec, "precision") == "int4") == (by_key.count({layer, role}) != 0),
                    "the precision map and the entries disagree about " + key);
        }
    covered_cells = covered.size();
    const Json *names = desc.get("role_names");
    if (names && names->kind == Json::Arr)
        for (long long layer = 0; layer < jint(&desc, "num_layers", 0); ++layer)
            for (const Json &name : names->a)
                require(covered.count({layer, name.s}) != 0, "the precision map does not cover layer " + std::to_string(layer) + "'s " + name.s);

    /* ---- each pair is exactly its members' bytes, in the order the rule names */
    const Json *pairs = doc.get("pairs");
    size_t pair_count = 0;
    if (pairs && pairs->kind == Json::Arr)
        for (const Json &pair : pairs->a) {
            ++pair_count;
            const long long layer = jint(&pair, "layer");
            const Json *members = pair.get("members");
            std::vector<const Json *> found;
            bool missing_member = !members || members->kind != Json::Arr;
            if (!missing_member)
                for (const Json &m : members->a) {
                    const auto it = by_key.find({layer, jstr(&m, "role")});
                    if (it == by_key.end()) missing_member = true; else found.push_back(it->second);
                }
            if (missing_member) { problems.push_back("pair at layer " + std::to_string(layer) + " names a member that has no entry"); continue; }
            std::vector<uint8_t> want_packed, want_scales, got_packed, got_scales, part;
            bool all_there = read_whole_file(out_dir + "/" + jstr(pair.get("packed"), "file"), got_packed) &&
                             read_whole_file(out_dir + "/" + jstr(pair.get("scales"), "file"), got_scales);
            long long rows = 0, k = 0;
            for (const Json *m : found) {
                all_there = all_there && read_whole_file(out_dir + "/" + jstr(m->get("packed"), "file"), part);
                want_packed.insert(want_packed.end(), part.begin(), part.end());
                all_there = all_there && read_whole_file(out_dir + "/" + jstr(m->get("scales"), "file"), part);
                want_scales.insert(want_scales.end(), part.begin(), part.end());
                const Json *shape = m->get("logical_shape");
                if (shape && shape->kind == Json::Arr && shape->a.size() == 2) { rows += shape->a[0].i; if (!k) k = shape->a[1].i; }
            }
            if (!all_there) { problems.push_back("pair at layer " + std::to_string(layer) + " is missing an artifact"); continue; }
            require(got_packed == want_packed, "pair at layer " + std::to_string(layer) + " is not its members' packed rows in order");
            require(got_scales == want_scales, "pair at layer " + std::to_string(layer) + " is not its members' scale rows in order");
            const Json *shape = pair.get("logical_shape");
            const bool shape_ok = shape && shape->kind == Json::Arr && shape->a.size() == 2 && shape->a[0].i == rows && shape->a[1].i == k;
            require(shape_ok, "pair at layer " + std::to_string(layer) + " claims another shape than [" + std::to_string(rows) + ", " +
                    std::to_string(k) + "]");
        }

    /* ---- a sample of entries must re-derive from the source checkpoint, on the GPU */
    if (rederive_samples > 0 && !entries->a.empty()) {
        std::vector<std::string> shards;
        std::map<std::string, TensorInfo> index;
        int st = index_checkpoint(source_dir.c_str(), shards, index);
        if (st) return st;
        DeviceBuffers dev;
        ErrorStats unused;
        std::vector<float> src;
        std::vector<uint8_t> packed, scales, on_disk;
        for (size_t e = 0; e < entries->a.size() && e < (size_t)rederive_samples; ++e) {
            const Json &entry = entries->a[e];
            const std::string packed_path = out_dir + "/" + jstr(entry.get("packed"), "file");
            const std::string scales_path = out_dir + "/" + jstr(entry.get("scales"), "file");
            if (!file_exists(packed_path) || !file_exists(scales_path)) continue; /* already reported above */
            const std::string tensor = jstr(&entry, "checkpoint_tensor");
            const auto it = index.find(tensor);
            if (it == index.end()) { problems.push_back(tensor + " is not in the source checkpoint"); continue; }
            st = read_tensor_f32(tensor, it->second, src);
            if (st) return st;
            st = quantize_tensor(dev, src, it->second.shape[0], it->second.shape[1], packed, scales, unused);
            if (st) return st;
            const std::string label = jstr(&entry, "role") + "_" + std::to_string(jint(&entry, "layer"));
            require(read_whole_file(packed_path, on_disk) && on_disk == packed, label + " does not re-derive from the source");
            require(read_whole_file(scales_path, on_disk) && on_disk == scales, label + " scales do not re-derive from the source");
        }
    }

    std::string out;
    if (problems.empty()) {
        out = "verify: " + std::to_string(entries->a.size()) + " entries, " + std::to_string(pair_count) +
              " pair(s) match their members' rows, the precision map covers " + std::to_string(covered_cells) +
              " (role, layer) cells, the source is unchanged" +
              (rederive_samples > 0 ? " and the sampled artifacts re-derive from it" : "") + "\n";
    } else {
        for (const std::string &p : problems) out += "verify: " + p + "\n";
    }
    if (report_bytes) {
        const size_t n = out.size() < report_bytes - 1 ? out.size() : report_bytes - 1;
        memcpy(report, out.data(), n);
        report[n] = '\0';
    }
    return (int)problems.size();
}

/* The encoder by itself, for the test that compares it with Python's json.dumps(indent=2, sort_keys=True):
 * parses `json_in` and writes it back; integers, reals, strings, arrays and objects only. */
static bool to_jout(const Json &in, JOut &out) {
    switch (in.kind) {
        case Json::Int: out = JOut::integer(in.i); return true;
        case Json::Real: out = JOut::real(in.d); return true;
        case Json::Str: out = JOut::str(in.s); return true;
        case Json::Arr:
            out = JOut::arr();
            for (const Json &e : in.a) { JOut c; if (!to_jout(e, c)) return false; out.a.push_back(c); }
            return true;
        case Json::Obj:
            out = JOut::obj();
            for (const auto &kv : in.o) { JOut c; if (!to_jout(kv.second, c)) return false; out.o[kv.first] = c; }
            return true;
        default: return false;
    }
}

extern "C" int ffn_json_reencode(const char *json_in, char *out, size_t out_bytes) {
    clear_error();
    if (!json_in || !out) return fail(FFN_ERR_CONFIG, "ffn_json_reencode: null argument");
    JsonReader reader(json_in);
    Json doc;
    JOut tree;
    if (!reader.value(doc) || !to_jout(doc, tree)) return fail(FFN_ERR_CONFIG, "ffn_json_reencode: not a document of numbers, strings, arrays and objects");
    std::string text;
    json_write(tree, 0, text);
    if (text.size() + 1 > out_bytes) return fail(FFN_ERR_CONFIG, "ffn_json_reencode: the text needs %zu bytes", text.size() + 1);
    memcpy(out, text.c_str(), text.size() + 1);
    return FFN_OK;
}
