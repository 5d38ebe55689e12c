/*
 * sidecar.cu - host side of the INT4 artifact path: SHA-256, the strict reader of
 * `weights.manifest.json`, artifact reads tied to their recorded digests, the tensor-parallel shard
 * view and the per-rank slicing + upload of a layer's operands.
 *
 * Replaces, for this path: csrc/sha256.c, csrc/quant_manifest.c (quant_manifest_parse, _find_entry,
 * _find_pair, quant_artifact_read; csrc/include/quant_manifest.h:68-147), model_desc_shard_view
 * (csrc/model_desc.c:561-631, OUT_DIM / IN_DIM rules) and the slicing half of
 * engine_load_quantized_ffn (csrc/engine.cu:2207-2428).  Unlike the reference's loader, which
 * re-reads and re-hashes every artifact once per rank and uploads with blocking copies, a layer's
 * artifacts are read and hashed once per process and the slices go up through pinned staging.
 *
 * The manifest functions return the reference's QuantManifestStatus values (0 OK, 1 ARG, 2 SYNTAX,
 * 3 FORMAT, 4 SHAPE, 5 IO, 6 HASH) so the reference's refusal tests read the same against this
 * reader; the message is in ffn_int4_last_error().
 */
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"
#include "host_util.h"
#include "kernels.h"

namespace ffn {

enum { QM_OK = 0, QM_ARG = 1, QM_SYNTAX = 2, QM_FORMAT = 3, QM_SHAPE = 4, QM_IO = 5, QM_HASH = 6 };

}  // namespace ffn

/* ------------------------------------------------------------------------------------------- */
/* The manifest                                                                                  */
/* ------------------------------------------------------------------------------------------- */
namespace ffn {

struct Artifact {
    std::string file, dtype, sha256;
    long long bytes = -1, count = -1;
};
struct Entry {
    std::string role;
    int role_index = -1, layer = -1;
    long long n = 0, k = 0, group = 0;
    Artifact packed, scales;
};
struct Pair {
    std::string name, member_role[2];
    int member_role_index[2] = {-1, -1};
    int layer = -1;
    long long n = 0, k = 0, group = 0;
    Artifact packed, scales;
};
struct Manifest {
    int manifest_version = 0, format_abi_version = 0, qmin = 0, qmax = 0, zero_point = 0, invalid_code = 0;
    long long group = 0;
    std::string packed_dtype, scale_dtype, converter_name, source_model_dir;
    int converter_version = 0;
    std::vector<Entry> entries;
    std::vector<Pair> pairs;
    int int4_cells = 0, bf16_cells = 0;
};

constexpr int kMaxEntries = 256, kMaxPairs = 128; /* csrc/include/quant_manifest.h:47-51 */

static int qfail(int status, const char *fmt, ...) {
    char buf[480];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    fail(status, "%s", buf);
    return status;
}

/* ---- the reader walks the parsed document in document order and applies each check where the
 * reference's streaming reader applies it (csrc/quant_manifest.c:277-1063), so that a document with
 * one fault gets the reference's status: wrong type or missing field = SYNTAX, a string that would
 * not fit the reference's fixed buffers = ARG, disagreement with the frozen format = FORMAT,
 * disagreement between extents = SHAPE. ---- */
constexpr size_t kNameMax = 64, kPathMax = 512, kShaMax = 65; /* csrc/include/quant_manifest.h:47-51 */

static int need_str(const Json &j, size_t buffer, std::string *out, const char *what) {
    if (j.kind != Json::Str) return qfail(QM_SYNTAX, "quant manifest: %s is not a string", what);
    if (j.s.size() + 1 > buffer) return qfail(QM_ARG, "quant manifest: %s does not fit %zu bytes", what, buffer);
    *out = j.s;
    return QM_OK;
}
static int need_int(const Json &j, long long *out, const char *what) {
    if (j.kind == Json::Int) { *out = j.i; return QM_OK; }
    if (j.kind == Json::Real && j.d >= -9.0e18 && j.d <= 9.0e18 && (double)(long long)j.d == j.d) { *out = (long long)j.d; return QM_OK; }
    return qfail(QM_SYNTAX, "quant manifest: %s is not an integer", what);
}
static int need_key(const std::string &key) {
    if (key.size() + 1 > kNameMax) return qfail(QM_ARG, "quant manifest: a key does not fit %zu bytes", kNameMax);
    return QM_OK;
}
/* a value the schema does not use: anything well-formed, within the reference's scratch sizes and depth */
static int skipped(const Json &j, int depth) {
    if (depth > 32) return qfail(QM_SYNTAX, "quant manifest: nesting is too deep");
    if (j.kind == Json::Str && j.s.size() + 1 > kPathMax) return qfail(QM_ARG, "quant manifest: a string does not fit %zu bytes", kPathMax);
    if (j.kind == Json::Arr)
        for (const Json &e : j.a) { const int st = skipped(e, depth + 1); if (st) return st; }
    if (j.kind == Json::Obj)
        for (const auto &kv : j.o) {
            if (kv.first.size() + 1 > kPathMax) return qfail(QM_ARG, "quant manifest: a key does not fit %zu bytes", kPathMax);
            const int st = skipped(kv.second, depth + 1);
            if (st) return st;
        }
    return QM_OK;
}

static bool is_sha256_hex(const std::string &s) {
    if (s.size() != 64) return false;
    for (char c : s)
        if (!((c >= '0' && c <= '9') || (c >= 'a' && c <= 'f'))) return false;
    return true;
}

/* One artifact object as written; `has_count` artifacts (scales) must carry a count, payloads must not. */
static int read_artifact(const Json &j, Artifact *a, bool has_count) {
    if (j.kind != Json::Obj) return qfail(QM_SYNTAX, "quant manifest: an artifact is not an object");
    if (j.o.empty()) return qfail(QM_SYNTAX, "quant manifest: an artifact object is empty");
    bool seen_bytes = false, seen_count = false, seen_dtype = false, seen_file = false, seen_sha = false;
    a->count = -1;
    for (const auto &kv : j.o) {
        int st = need_key(kv.first);
        if (st) return st;
        bool *seen = kv.first == "bytes" ? &seen_bytes : kv.first == "count" ? &seen_count : kv.first == "dtype" ? &seen_dtype
                   : kv.first == "file" ? &seen_file : kv.first == "sha256" ? &seen_sha : nullptr;
        if (!seen) { if ((st = skipped(kv.second, 0))) return st; continue; }
        if (*seen) return qfail(QM_SYNTAX, "quant manifest: \"%s\" appears twice in an artifact", kv.first.c_str());
        *seen = true;
        if (seen == &seen_bytes) st = need_int(kv.second, &a->bytes, "an artifact's bytes");
        else if (seen == &seen_count) st = need_int(kv.second, &a->count, "an artifact's count");
        else if (seen == &seen_dtype) st = need_str(kv.second, kNameMax, &a->dtype, "an artifact's dtype");
        else if (seen == &seen_file) st = need_str(kv.second, kPathMax, &a->file, "an artifact's file");
        else st = need_str(kv.second, kShaMax, &a->sha256, "an artifact's sha256");
        if (st) return st;
    }
    if (!seen_bytes || !seen_dtype || !seen_file || !seen_sha) return qfail(QM_SYNTAX, "quant manifest: an artifact lacks one of bytes/dtype/file/sha256");
    if (has_count && !seen_count) return qfail(QM_SYNTAX, "quant manifest: a scale artifact has no count");
    if (!has_count && seen_count) return qfail(QM_SYNTAX, "quant manifest: a packed payload carries a count");
    return QM_OK;
}

/* ... and against the frozen format (require_artifact, csrc/quant_manifest.c:341-364, in its order) */
static int check_artifact(const Artifact &a, const char *want_dtype, const char *where, bool is_scales) {
    const char *kind = is_scales ? "scales" : "packed";
    if (!is_sha256_hex(a.sha256)) return qfail(QM_FORMAT, "quant manifest: %s's %s digest is not 64 lower-case hex digits", where, kind);
    if (a.bytes <= 0) return qfail(QM_FORMAT, "quant manifest: %s's %s artifact has a nonpositive byte count", where, kind);
    if (a.file.empty()) return qfail(QM_FORMAT, "quant manifest: %s's %s artifact names no file", where, kind);
    if (a.dtype != want_dtype) return qfail(QM_FORMAT, "quant manifest: %s's %s artifact is %s, the format stores %s", where, kind, a.dtype.c_str(), want_dtype);
    if (is_scales != (a.count >= 0)) return qfail(QM_FORMAT, "quant manifest: %s's %s artifact %s a scale count", where, kind, is_scales ? "is missing" : "carries");
    return QM_OK;
}

/* The format's extent rules (linear_layout_init, csrc/linear_weight.cpp:57-86). */
static int layout_of(long long n, long long k, long long group, long long *packed_bytes, long long *scale_count, const char *where) {
    if (n <= 0 || k <= 0) return qfail(QM_SHAPE, "quant manifest: %s has a nonpositive shape", where);
    if (group != FFN_INT4_GROUP) return qfail(QM_SHAPE, "quant manifest: %s groups %lld, this format's group is %d", where, group, FFN_INT4_GROUP);
    if (k % group) return qfail(QM_SHAPE, "quant manifest: %s: K=%lld is not a whole number of %lld-wide groups", where, k, group);
    if (n % 8) return qfail(QM_SHAPE, "quant manifest: %s: N=%lld is not a whole number of the 8-row tile", where, n);
    *packed_bytes = n * k / 2;
    *scale_count = n * (k / group);
    return QM_OK;
}

static int read_shape(const Json &j, long long *n, long long *k) {
    if (j.kind != Json::Arr || j.a.size() != 2) return qfail(QM_SYNTAX, "quant manifest: a shape is not a list of two integers");
    int st = need_int(j.a[0], n, "a shape's rows");
    if (!st) st = need_int(j.a[1], k, "a shape's columns");
    return st;
}

static int find_entry(const Manifest &m, int layer, const char *role) {
    for (size_t i = 0; i < m.entries.size(); ++i)
        if (m.entries[i].layer == layer && m.entries[i].role == role) return (int)i;
    return -1;
}
static int find_pair(const Manifest &m, const char *name, int layer) {
    for (size_t i = 0; i < m.pairs.size(); ++i)
        if (m.pairs[i].layer == layer && m.pairs[i].name == name) return (int)i;
    return -1;
}

static int read_format(const Json &j, Manifest *m) {
    if (j.kind != Json::Obj || j.o.empty()) return qfail(QM_SYNTAX, "quant manifest: the format block is not a filled object");
    bool seen[9] = {};
    static const char *const kInts[] = {"abi_version", "group", "qmin", "qmax", "zero_point", "invalid_code"};
    long long iv[6] = {};
    std::string name;
    for (const auto &kv : j.o) {
        int st = need_key(kv.first);
        if (st) return st;
        int which = -1;
        for (int i = 0; i < 6; ++i) if (kv.first == kInts[i]) which = i;
        if (which >= 0) { seen[which] = true; st = need_int(kv.second, &iv[which], kInts[which]); }
        else if (kv.first == "name") { seen[6] = true; st = need_str(kv.second, kNameMax, &name, "the format's name"); }
        else if (kv.first == "packed_dtype") { seen[7] = true; st = need_str(kv.second, kNameMax, &m->packed_dtype, "packed_dtype"); }
        else if (kv.first == "scale_dtype") { seen[8] = true; st = need_str(kv.second, kNameMax, &m->scale_dtype, "scale_dtype"); }
        else st = skipped(kv.second, 0);
        if (st) return st;
    }
    for (bool b : seen) if (!b) return qfail(QM_SYNTAX, "quant manifest: the format block is incomplete");
    if (iv[0] != 1) return qfail(QM_FORMAT, "quant manifest: format abi_version %lld, this reader speaks 1", iv[0]);
    if (iv[1] != FFN_INT4_GROUP || iv[2] != -7 || iv[3] != 7 || iv[4] != 0 || iv[5] != -8)
        return qfail(QM_FORMAT, "quant manifest: the format block (group %lld, codes [%lld, %lld], zero point %lld, reserved %lld) "
                     "is not the frozen format", iv[1], iv[2], iv[3], iv[4], iv[5]);
    if (m->packed_dtype != "u8" || m->scale_dtype != "bf16")
        return qfail(QM_FORMAT, "quant manifest: the format stores %s codes and %s scales, not u8 and bf16",
                     m->packed_dtype.c_str(), m->scale_dtype.c_str());
    m->format_abi_version = 1; m->group = iv[1]; m->qmin = -7; m->qmax = 7; m->zero_point = 0; m->invalid_code = -8;
    return QM_OK;
}

static int read_entries(const Json &arr, Manifest *m) {
    if (arr.kind != Json::Arr) return qfail(QM_SYNTAX, "quant manifest: entries is not a list");
    if (arr.a.empty()) return qfail(QM_FORMAT, "quant manifest: entries is empty");
    for (const Json &e : arr.a) {
        if (m->entries.size() >= (size_t)kMaxEntries) return qfail(QM_FORMAT, "quant manifest: more than %d entries", kMaxEntries);
        if (e.kind != Json::Obj || e.o.empty()) return qfail(QM_SYNTAX, "quant manifest: an entry is not a filled object");
        Entry en;
        static const char *const kNames[8] = {"role", "role_index", "layer", "logical_shape", "packed", "scales", "group", "group_axis"};
        bool seen[8] = {};
        for (const auto &kv : e.o) {
            int st = need_key(kv.first);
            if (st) return st;
            int which = -1;
            for (int i = 0; i < 8; ++i) if (kv.first == kNames[i]) which = i;
            if (which < 0) { if ((st = skipped(kv.second, 0))) return st; continue; }
            if (seen[which]) return qfail(QM_SYNTAX, "quant manifest: \"%s\" appears twice in an entry", kNames[which]);
            seen[which] = true;
            long long v = 0;
            std::string axis;
            switch (which) {
                case 0: st = need_str(kv.second, kNameMax, &en.role, "an entry's role"); break;
                case 1: st = need_int(kv.second, &v, "an entry's role_index"); en.role_index = (int)v; break;
                case 2: st = need_int(kv.second, &v, "an entry's layer"); en.layer = (int)v; break;
                case 3: st = read_shape(kv.second, &en.n, &en.k); break;
                case 4: st = read_artifact(kv.second, &en.packed, false); break;
                case 5: st = read_artifact(kv.second, &en.scales, true); break;
                case 6: st = need_int(kv.second, &en.group, "an entry's group"); break;
                default:
                    st = need_str(kv.second, kNameMax, &axis, "an entry's group_axis");
                    if (!st && axis != "k") st = qfail(QM_FORMAT, "quant manifest: an entry groups along %s, the format groups along k", axis.c_str());
            }
            if (st) return st;
        }
        if (!seen[0] || !seen[2] || !seen[3] || !seen[4] || !seen[5] || !seen[6])
            return qfail(QM_SYNTAX, "quant manifest: an entry lacks one of role/layer/logical_shape/packed/scales/group");
        if (en.role.empty()) return qfail(QM_FORMAT, "quant manifest: an entry has no role");
        if (en.layer < 0) return qfail(QM_FORMAT, "quant manifest: %s has a negative layer", en.role.c_str());
        char where[128];
        snprintf(where, sizeof(where), "%s layer %d", en.role.c_str(), en.layer);
        long long pb = 0, sc = 0;
        int st = layout_of(en.n, en.k, en.group, &pb, &sc, where);
        if (!st) st = check_artifact(en.packed, "u8", where, false);
        if (!st) st = check_artifact(en.scales, "bf16", where, true);
        if (st) return st;
        if (en.packed.bytes != pb)
            return qfail(QM_SHAPE, "quant manifest: %s records %lld packed bytes, [%lld, %lld] at group %lld is %lld", where,
                         en.packed.bytes, en.n, en.k, en.group, pb);
        if (en.scales.count != sc)
            return qfail(QM_SHAPE, "quant manifest: %s records %lld scales, [%lld, %lld] at group %lld is %lld", where,
                         en.scales.count, en.n, en.k, en.group, sc);
        if (en.scales.bytes != en.scales.count * 2)
            return qfail(QM_SHAPE, "quant manifest: %s records %lld scale bytes for %lld bf16 scales", where, en.scales.bytes, en.scales.count);
        m->entries.push_back(en);
    }
    return QM_OK;
}

static int read_pairs(const Json &arr, Manifest *m) {
    if (arr.kind != Json::Arr) return qfail(QM_SYNTAX, "quant manifest: pairs is not a list");
    for (const Json &pj : arr.a) {
        if (m->pairs.size() >= (size_t)kMaxPairs) return qfail(QM_FORMAT, "quant manifest: more than %d pairs", kMaxPairs);
        if (pj.kind != Json::Obj || pj.o.empty()) return qfail(QM_SYNTAX, "quant manifest: a pair is not a filled object");
        Pair pr;
        static const char *const kNames[7] = {"name", "layer", "logical_shape", "packed", "scales", "group", "members"};
        bool seen[7] = {};
        for (const auto &kv : pj.o) {
            int st = need_key(kv.first);
            if (st) return st;
            int which = -1;
            for (int i = 0; i < 7; ++i) if (kv.first == kNames[i]) which = i;
            if (which < 0) { if ((st = skipped(kv.second, 0))) return st; continue; }
            if (seen[which]) return qfail(QM_SYNTAX, "quant manifest: \"%s\" appears twice in a pair", kNames[which]);
            seen[which] = true;
            long long v = 0;
            switch (which) {
                case 0: st = need_str(kv.second, kNameMax, &pr.name, "a pair's name"); break;
                case 1: st = need_int(kv.second, &v, "a pair's layer"); pr.layer = (int)v; break;
                case 2: st = read_shape(kv.second, &pr.n, &pr.k); break;
                case 3: st = read_artifact(kv.second, &pr.packed, false); break;
                case 4: st = read_artifact(kv.second, &pr.scales, true); break;
                case 5: st = need_int(kv.second, &pr.group, "a pair's group"); break;
                default: {
                    const Json &ms = kv.second;
                    if (ms.kind != Json::Arr || ms.a.size() != 2) { st = qfail(QM_SYNTAX, "quant manifest: a pair's members are not a list of two"); break; }
                    for (int i = 0; i < 2 && !st; ++i) {
                        const Json &mj = ms.a[i];
                        if (mj.kind != Json::Obj || mj.o.empty()) { st = qfail(QM_SYNTAX, "quant manifest: a pair member is not a filled object"); break; }
                        bool seen_role = false, seen_index = false;
                        for (const auto &mk : mj.o) {
                            if ((st = need_key(mk.first))) break;
                            if (mk.first == "role") {
                                if (seen_role) { st = qfail(QM_SYNTAX, "quant manifest: a pair member names its role twice"); break; }
                                seen_role = true;
                                st = need_str(mk.second, kNameMax, &pr.member_role[i], "a pair member's role");
                            } else if (mk.first == "role_index") {
                                if (seen_index) { st = qfail(QM_SYNTAX, "quant manifest: a pair member gives its role_index twice"); break; }
                                seen_index = true;
                                long long ri = 0;
                                st = need_int(mk.second, &ri, "a pair member's role_index");
                                pr.member_role_index[i] = (int)ri;
                            } else {
                                st = skipped(mk.second, 0);
                            }
                            if (st) break;
                        }
                        if (!st && !seen_role) st = qfail(QM_SYNTAX, "quant manifest: a pair member has no role");
                    }
                }
            }
            if (st) return st;
        }
        for (bool b : seen) if (!b) return qfail(QM_SYNTAX, "quant manifest: a pair lacks one of name/layer/members/logical_shape/packed/scales/group");
        if (pr.member_role[0].empty() || pr.member_role[1].empty()) return qfail(QM_SYNTAX, "quant manifest: a pair has fewer than two named members");
        char where[160];
        snprintf(where, sizeof(where), "pair %s layer %d", pr.name.c_str(), pr.layer);
        int st = check_artifact(pr.packed, "u8", where, false);
        if (!st) st = check_artifact(pr.scales, "bf16", where, true);
        if (st) return st;
        if (pr.n <= 0 || pr.k <= 0) return qfail(QM_SHAPE, "quant manifest: %s has a nonpositive shape", where);
        long long rows = 0, pbytes = 0, scales = 0, k = -1;
        for (int i = 0; i < 2; ++i) {
            const int idx = find_entry(*m, pr.layer, pr.member_role[i].c_str());
            if (idx < 0)
                return qfail(QM_SHAPE, "quant manifest: %s names member %s, which is not an entry of layer %d", where,
                             pr.member_role[i].c_str(), pr.layer);
            const Entry &en = m->entries[idx];
            if (pr.member_role_index[i] >= 0 && pr.member_role_index[i] != en.role_index)
                return qfail(QM_SHAPE, "quant manifest: %s records member %s as role_index %d, the entry is %d", where,
                             en.role.c_str(), pr.member_role_index[i], en.role_index);
            if (k < 0) k = en.k;
            else if (en.k != k) return qfail(QM_SHAPE, "quant manifest: %s concatenates members of different K (%lld and %lld)", where, k, en.k);
            rows += en.n; pbytes += en.packed.bytes; scales += en.scales.count;
        }
        if (pr.k != k || pr.n != rows)
            return qfail(QM_SHAPE, "quant manifest: %s is [%lld, %lld], its members are [%lld, %lld]", where, pr.n, pr.k, rows, k);
        if (pr.packed.bytes != pbytes) return qfail(QM_SHAPE, "quant manifest: %s records %lld packed bytes, its members hold %lld", where, pr.packed.bytes, pbytes);
        if (pr.scales.count != scales || pr.scales.bytes != scales * 2)
            return qfail(QM_SHAPE, "quant manifest: %s records %lld scales, its members hold %lld", where, pr.scales.count, scales);
        if (pr.group != FFN_INT4_GROUP) return qfail(QM_FORMAT, "quant manifest: %s groups %lld, the format groups %d", where, pr.group, FFN_INT4_GROUP);
        m->pairs.push_back(pr);
    }
    return QM_OK;
}

/* the precision map and the entries have to describe the same cells */
static int read_precision_map(const Json &arr, Manifest *m) {
    if (arr.kind != Json::Arr) return qfail(QM_SYNTAX, "quant manifest: precision_map is not a list");
    if (arr.a.empty()) return qfail(QM_FORMAT, "quant manifest: the precision map is empty");
    std::vector<char> seen(m->entries.size(), 0);
    for (const Json &c : arr.a) {
        if (c.kind != Json::Obj || c.o.empty()) return qfail(QM_SYNTAX, "quant manifest: a precision cell is not a filled object");
        std::string role, prec;
        long long layer = -1;
        bool seen_role = false, seen_layer = false, seen_prec = false;
        for (const auto &kv : c.o) {
            int st = need_key(kv.first);
            if (st) return st;
            if (kv.first == "role") { seen_role = true; st = need_str(kv.second, kNameMax, &role, "a precision cell's role"); }
            else if (kv.first == "layer") { seen_layer = true; st = need_int(kv.second, &layer, "a precision cell's layer"); }
            else if (kv.first == "precision") { seen_prec = true; st = need_str(kv.second, kNameMax, &prec, "a precision cell's precision"); }
            else st = skipped(kv.second, 0);
            if (st) return st;
        }
        if (!seen_role || !seen_layer || !seen_prec) return qfail(QM_SYNTAX, "quant manifest: a precision cell lacks role, layer or precision");
        if (prec == "int4") {
            const int idx = find_entry(*m, (int)layer, role.c_str());
            if (idx < 0) return qfail(QM_SHAPE, "quant manifest: %s layer %lld is marked int4 but has no entry", role.c_str(), layer);
            if (seen[idx]) return qfail(QM_SHAPE, "quant manifest: %s layer %lld has two int4 precision cells", role.c_str(), layer);
            seen[idx] = 1;
            ++m->int4_cells;
        } else if (prec == "bf16") {
            ++m->bf16_cells;
        } else {
            return qfail(QM_FORMAT, "quant manifest: unknown precision %s", prec.c_str());
        }
    }
    for (size_t i = 0; i < seen.size(); ++i)
        if (!seen[i])
            return qfail(QM_SHAPE, "quant manifest: %s layer %d has an entry but no int4 precision cell", m->entries[i].role.c_str(), m->entries[i].layer);
    return QM_OK;
}

static int parse_manifest(const char *text, Manifest *m) {
    if (!text || !m) return qfail(QM_ARG, "quant manifest: null argument");
    JsonReader reader(text);
    reader.manifest_dialect = true;
    Json root;
    reader.ws();
    if (reader.p >= reader.end || *reader.p != '{') return qfail(QM_SYNTAX, "quant manifest: the document is not an object");
    if (!reader.value(root)) return qfail(QM_SYNTAX, "%s", reader.error.c_str());
    reader.ws();
    if (reader.p != reader.end) return qfail(QM_SYNTAX, "quant manifest: bytes follow the document");
    if (root.o.empty()) return qfail(QM_SYNTAX, "quant manifest: the document is empty");
    bool seen_version = false, seen_format = false, seen_converter = false, seen_source = false, seen_entries = false,
         seen_precision = false, seen_pairs = false;
    long long version = 0;
    for (const auto &kv : root.o) {
        int st = need_key(kv.first);
        if (st) return st;
        bool *seen = kv.first == "manifest_version" ? &seen_version : kv.first == "format" ? &seen_format
                   : kv.first == "converter" ? &seen_converter : kv.first == "source" ? &seen_source
                   : kv.first == "entries" ? &seen_entries : kv.first == "precision_map" ? &seen_precision
                   : kv.first == "pairs" ? &seen_pairs : nullptr;
        if (!seen) { if ((st = skipped(kv.second, 0))) return st; continue; }
        if (*seen) return qfail(QM_SYNTAX, "quant manifest: \"%s\" appears twice", kv.first.c_str());
        *seen = true;
        const Json &v = kv.second;
        if (seen == &seen_version) {
            st = need_int(v, &version, "manifest_version");
        } else if (seen == &seen_format) {
            st = read_format(v, m);
        } else if (seen == &seen_converter || seen == &seen_source) {
            const bool conv = seen == &seen_converter;
            if (v.kind != Json::Obj || v.o.empty()) return qfail(QM_SYNTAX, "quant manifest: %s is not a filled object", conv ? "converter" : "source");
            for (const auto &ck : v.o) {
                if ((st = need_key(ck.first))) return st;
                long long cv = 0;
                if (conv && ck.first == "name") st = need_str(ck.second, kPathMax, &m->converter_name, "the converter's name");
                else if (conv && ck.first == "version") { st = need_int(ck.second, &cv, "the converter's version"); m->converter_version = (int)cv; }
                else if (!conv && ck.first == "model_dir") st = need_str(ck.second, kPathMax, &m->source_model_dir, "the source's model_dir");
                else st = skipped(ck.second, 0);
                if (st) return st;
            }
        } else if (seen == &seen_entries) {
            st = read_entries(v, m);
        } else if (seen == &seen_precision) {
            if (!seen_entries) return qfail(QM_SYNTAX, "quant manifest: precision_map precedes entries, so it cannot be checked against them");
            st = read_precision_map(v, m);
        } else {
            if (!seen_entries) return qfail(QM_SYNTAX, "quant manifest: pairs precede entries, so a pair cannot be checked against its members");
            st = read_pairs(v, m);
        }
        if (st) return st;
    }
    if (!seen_version || !seen_format || !seen_converter || !seen_source || !seen_entries || !seen_precision)
        return qfail(QM_SYNTAX, "quant manifest: one of manifest_version/format/converter/source/entries/precision_map is missing");
    if (version != 1) return qfail(QM_FORMAT, "quant manifest: manifest_version %lld, this reader speaks 1", version);
    m->manifest_version = 1;
    if (m->converter_name.empty() || m->converter_version <= 0) return qfail(QM_FORMAT, "quant manifest: the converter is unnamed or unversioned");
    if (m->source_model_dir.empty()) return qfail(QM_FORMAT, "quant manifest: no source model directory");
    if (m->entries.empty()) return qfail(QM_FORMAT, "quant manifest: no entries");
    /* one refusal of this reader's own, after everything the reference checks: an artifact path may not leave the sidecar */
    auto outside = [](const Artifact &a) { return a.file[0] == '/' || a.file.find("..") != std::string::npos; };
    for (const Entry &e : m->entries)
        if (outside(e.packed) || outside(e.scales)) return qfail(QM_FORMAT, "quant manifest: %s layer %d names an artifact outside the sidecar directory", e.role.c_str(), e.layer);
    for (const Pair &pr : m->pairs)
        if (outside(pr.packed) || outside(pr.scales)) return qfail(QM_FORMAT, "quant manifest: pair %s layer %d names an artifact outside the sidecar directory", pr.name.c_str(), pr.layer);
    return QM_OK;
}

/* Read one artifact, checking dtype, size and SHA-256 in that order (quant_artifact_read,
 * csrc/quant_manifest.c:1085-1139). */
static int read_artifact_file(const std::string &root, const Artifact &a, const char *want_dtype, std::vector<uint8_t> *out) {
    if (want_dtype && a.dtype != want_dtype) /* a caller that passes no expectation gets no dtype check, as in the reference */
        return qfail(QM_FORMAT, "quant artifact %s is recorded as %s, %s was expected", a.file.c_str(), a.dtype.c_str(), want_dtype);
    const std::string path = root + "/" + a.file;
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return qfail(QM_IO, "quant artifact %s cannot be opened", path.c_str());
    fseek(f, 0, SEEK_END);
    const long long size = ftell(f);
    fseek(f, 0, SEEK_SET);
    if (size != a.bytes) {
        fclose(f);
        return qfail(QM_IO, "quant artifact %s is %lld bytes, the manifest records %lld", path.c_str(), size, a.bytes);
    }
    out->resize((size_t)size);
    const size_t got = size ? fread(out->data(), 1, (size_t)size, f) : 0;
    fclose(f);
    if ((long long)got != size) return qfail(QM_IO, "quant artifact %s could not be read in full", path.c_str());
    Sha256 sha;
    sha.update(out->data(), out->size());
    char hex[65];
    sha.finish(hex);
    if (a.sha256 != hex) {
        out->clear();
        return qfail(QM_HASH, "quant artifact %s hashes to %s, the manifest records %s", path.c_str(), hex, a.sha256.c_str());
    }
    return QM_OK;
}

}  // namespace ffn

/* ------------------------------------------------------------------------------------------- */
/* Shard views and the per-rank load                                                             */
/* ------------------------------------------------------------------------------------------- */
namespace ffn {

enum { SHARD_NONE = 0, SHARD_OUT_DIM = 1, SHARD_IN_DIM = 2 };

/* model_desc_shard_view's OUT_DIM / IN_DIM rules (csrc/model_desc.c:609-626). */
static int shard_view(int rule, long long rows, long long cols, int tp, int rank, long long v[4]) {
    v[0] = 0; v[1] = rows; v[2] = 0; v[3] = cols;
    if (tp <= 1) return FFN_OK;
    if (rank < 0 || rank >= tp) return fail(FFN_ERR_CONFIG, "shard view rank %d is outside [0, %d)", rank, tp);
    if (rule == SHARD_OUT_DIM) {
        if (rows % tp) return fail(FFN_ERR_CONFIG, "tp_size %d does not divide %lld rows", tp, rows);
        v[1] = rows / tp; v[0] = v[1] * rank;
    } else if (rule == SHARD_IN_DIM) {
        if (cols % tp) return fail(FFN_ERR_CONFIG, "tp_size %d does not divide %lld columns", tp, cols);
        v[3] = cols / tp; v[2] = v[3] * rank;
    } else if (rule != SHARD_NONE) {
        return fail(FFN_ERR_CONFIG, "unknown shard rule %d", rule);
    }
    return FFN_OK;
}

struct LoadedLayer {
    uint8_t *gate_up = nullptr, *down = nullptr;
    uint16_t *gate_up_scales = nullptr, *down_scales = nullptr;
};
struct QuantizedFfn {
    int device = 0, layers = 0, hidden = 0, inter_local = 0;
    std::vector<LoadedLayer> layer;
    std::vector<void *> owned;
    ~QuantizedFfn() {
        int restore = 0;
        (void)cudaGetDevice(&restore);
        (void)cudaSetDevice(device);
        for (const LoadedLayer &l : layer) { /* the k-major copies registered for these addresses go first */
            FfnMlpWeights w = {};
            w.down_i4 = l.down;
            if (l.down) (void)ffn_decode_layer_release(&w);
        }
        for (void *p : owned) cudaFree(p);
        (void)cudaSetDevice(restore);
    }
};

/* `rows` rows of `row_bytes` starting at (first_row, col_byte) of a row-major source whose rows are
 * `src_row_bytes` wide.  Payload and scales use the same walk with their own widths, so the scales
 * copied are the global ones the slice selects (slice_rows, csrc/engine.cu:2198-2205). */
static void slice_into(uint8_t *dst, const uint8_t *src, long long src_row_bytes, long long first_row, long long rows,
                       long long col_byte, long long row_bytes) {
    for (long long i = 0; i < rows; ++i)
        memcpy(dst + i * row_bytes, src + (first_row + i) * src_row_bytes + col_byte, (size_t)row_bytes);
}

struct Staging { /* pinned, double-buffered by layer parity */
    uint8_t *buf[2] = {nullptr, nullptr};
    size_t bytes = 0;
    cudaEvent_t done[2] = {nullptr, nullptr};
    ~Staging() {
        for (int i = 0; i < 2; ++i) {
            if (buf[i]) cudaFreeHost(buf[i]);
            if (done[i]) cudaEventDestroy(done[i]);
        }
    }
};

static int load_ranks(const char *dir, int num_layers, int hidden, int inter, int tp, const int *ranks, const int *devices,
                      int count, QuantizedFfn **out) {
    if (!dir || !out || !ranks || !devices || count < 1) return fail(FFN_ERR_CONFIG, "ffn_load_quantized_ffn: null argument");
    if (num_layers < 1) return fail(FFN_ERR_CONFIG, "ffn_load_quantized_ffn: this descriptor has no dense FFN layer to quantize");
    const std::string root(dir);
    std::string text;
    {
        FILE *f = fopen((root + "/weights.manifest.json").c_str(), "rb");
        if (!f) return fail(FFN_ERR_WEIGHTS, "ffn_load_quantized_ffn: cannot open %s/weights.manifest.json", dir);
        char chunk[8192];
        size_t got;
        while ((got = fread(chunk, 1, sizeof(chunk), f)) > 0) text.append(chunk, got);
        fclose(f);
    }
    Manifest m;
    if (parse_manifest(text.c_str(), &m) != QM_OK) {
        const std::string why = ffn_int4_last_error();
        return fail(FFN_ERR_WEIGHTS, "ffn_load_quantized_ffn: %s", why.c_str());
    }
    /* every dense layer or none (csrc/engine.cu:2245-2262) */
    int prepared = 0;
    for (int l = 0; l < num_layers; ++l)
        if (find_pair(m, "mlpGateUp", l) >= 0 && find_entry(m, l, "mlpDown") >= 0) ++prepared;
    if (prepared != num_layers)
        return fail(FFN_ERR_WEIGHTS, "ffn_load_quantized_ffn: the sidecar covers %d of %d dense layers", prepared, num_layers);

    std::vector<std::unique_ptr<QuantizedFfn>> result;
    for (int i = 0; i < count; ++i) {
        std::unique_ptr<QuantizedFfn> q(new QuantizedFfn());
        q->device = devices[i]; q->layers = num_layers; q->hidden = hidden; q->inter_local = inter / (tp > 0 ? tp : 1);
        q->layer.resize(num_layers);
        result.push_back(std::move(q));
    }
    std::vector<Staging> staging(count);
    std::vector<cudaStream_t> streams(count, nullptr);
    int restore = 0;
    (void)cudaGetDevice(&restore);
    int status = FFN_OK;
    auto upload = [&](int i, int parity, size_t *offset, const std::vector<uint8_t> &host, void **dev_out) -> int {
        QuantizedFfn &q = *result[i];
        void *d = nullptr;
        if (cudaMalloc(&d, host.size() ? host.size() : 16) != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(FFN_ERR_ALLOC, "ffn_load_quantized_ffn: cannot allocate %zu bytes on device %d", host.size(), q.device);
        }
        q.owned.push_back(d);
        memcpy(staging[i].buf[parity] + *offset, host.data(), host.size());
        FFN_CUDA_TRY(cudaMemcpyAsync(d, staging[i].buf[parity] + *offset, host.size(), cudaMemcpyHostToDevice, streams[i]),
                     "ffn_load_quantized_ffn: upload");
        *offset += (host.size() + 255) & ~(size_t)255;
        *dev_out = d;
        return FFN_OK;
    };

    for (int l = 0; l < num_layers && status == FFN_OK; ++l) {
        const Pair &pair = m.pairs[find_pair(m, "mlpGateUp", l)];
        const Entry &down = m.entries[find_entry(m, l, "mlpDown")];
        if (pair.n != 2ll * inter || pair.k != hidden) {
            status = fail(FFN_ERR_WEIGHTS, "ffn_load_quantized_ffn: layer %d's mlpGateUp pair is [%lld, %lld], the checkpoint's gate+up is [%lld, %d]",
                          l, pair.n, pair.k, 2ll * inter, hidden);
            break;
        }
        if (down.n != hidden || down.k != inter) {
            status = fail(FFN_ERR_WEIGHTS, "ffn_load_quantized_ffn: layer %d's mlpDown is [%lld, %lld], the checkpoint's is [%d, %d]", l,
                          down.n, down.k, hidden, inter);
            break;
        }
        if (pair.group != down.group) {
            status = fail(FFN_ERR_WEIGHTS, "ffn_load_quantized_ffn: layer %d's gate/up and down disagree on the group width", l);
            break;
        }
        /* read and hash each artifact ONCE, whatever the number of ranks */
        std::vector<uint8_t> pair_p, pair_s, down_p, down_s;
        if (read_artifact_file(root, pair.packed, "u8", &pair_p) || read_artifact_file(root, pair.scales, "bf16", &pair_s) ||
            read_artifact_file(root, down.packed, "u8", &down_p) || read_artifact_file(root, down.scales, "bf16", &down_s)) {
            const std::string why = ffn_int4_last_error();
            status = fail(FFN_ERR_WEIGHTS, "ffn_load_quantized_ffn: %s", why.c_str());
            break;
        }
        const long long half_rows = pair.n / 2;
        for (int i = 0; i < count && status == FFN_OK; ++i) {
            const int r = ranks[i];
            long long gv[4], dv[4];
            if ((status = shard_view(SHARD_OUT_DIM, half_rows, pair.k, tp, r, gv)) != FFN_OK) break;
            if ((status = shard_view(SHARD_IN_DIM, down.n, down.k, tp, r, dv)) != FFN_OK) break;
            if (gv[2] % pair.group || dv[2] % down.group || dv[3] % down.group) {
                status = fail(FFN_ERR_WEIGHTS, "ffn_load_quantized_ffn: layer %d's rank %d splits K at a non-group boundary, which cannot "
                              "retain the global scales", l, r);
                break;
            }
            const long long row_b = gv[3] / 2, srow_b = gv[3] / pair.group * 2;
            std::vector<uint8_t> gu_p((size_t)(2 * gv[1] * row_b)), gu_s((size_t)(2 * gv[1] * srow_b));
            slice_into(gu_p.data(), pair_p.data(), pair.k / 2, gv[0], gv[1], gv[2] / 2, row_b);
            slice_into(gu_p.data() + gv[1] * row_b, pair_p.data(), pair.k / 2, half_rows + gv[0], gv[1], gv[2] / 2, row_b);
            slice_into(gu_s.data(), pair_s.data(), pair.k / pair.group * 2, gv[0], gv[1], gv[2] / pair.group * 2, srow_b);
            slice_into(gu_s.data() + gv[1] * srow_b, pair_s.data(), pair.k / pair.group * 2, half_rows + gv[0], gv[1],
                       gv[2] / pair.group * 2, srow_b);
            const long long drow_b = dv[3] / 2, dsrow_b = dv[3] / down.group * 2;
            std::vector<uint8_t> d_p((size_t)(down.n * drow_b)), d_s((size_t)(down.n * dsrow_b));
            slice_into(d_p.data(), down_p.data(), down.k / 2, 0, down.n, dv[2] / 2, drow_b);
            slice_into(d_s.data(), down_s.data(), down.k / down.group * 2, 0, down.n, dv[2] / down.group * 2, dsrow_b);

            if (cudaSetDevice(devices[i]) != cudaSuccess) { status = fail(FFN_ERR_CUDA, "ffn_quantized_ffn_prepare_decode: cannot select device %d", devices[i]); break; }
            Staging &st = staging[i];
            const size_t need = gu_p.size() + gu_s.size() + d_p.size() + d_s.size() + 4 * 256;
            if (!st.buf[0]) {
                st.bytes = need;
                if (cudaMallocHost(&st.buf[0], need) != cudaSuccess || cudaMallocHost(&st.buf[1], need) != cudaSuccess ||
                    cudaEventCreateWithFlags(&st.done[0], cudaEventDisableTiming) != cudaSuccess ||
                    cudaEventCreateWithFlags(&st.done[1], cudaEventDisableTiming) != cudaSuccess ||
                    cudaStreamCreateWithFlags(&streams[i], cudaStreamNonBlocking) != cudaSuccess) {
                    status = fail(FFN_ERR_ALLOC, "ffn_load_quantized_ffn: cannot set up pinned staging");
                    break;
                }
            }
            const int parity = l & 1;
            if (l >= 2 && cudaEventSynchronize(st.done[parity]) != cudaSuccess) { status = fail(FFN_ERR_CUDA, "ffn_load_quantized_ffn: staging wait"); break; }
            size_t off = 0;
            LoadedLayer &ll = result[i]->layer[l];
            if ((status = upload(i, parity, &off, gu_p, (void **)&ll.gate_up)) || (status = upload(i, parity, &off, gu_s, (void **)&ll.gate_up_scales)) ||
                (status = upload(i, parity, &off, d_p, (void **)&ll.down)) || (status = upload(i, parity, &off, d_s, (void **)&ll.down_scales)))
                break;
            (void)cudaEventRecord(st.done[parity], streams[i]);
        }
    }
    for (int i = 0; i < count; ++i)
        if (streams[i]) {
            (void)cudaSetDevice(devices[i]);
            if (cudaStreamSynchronize(streams[i]) != cudaSuccess && status == FFN_OK) status = fail(FFN_ERR_CUDA, "ffn_load_quantized_ffn: upload failed");
            cudaStreamDestroy(streams[i]);
        }
    (void)cudaSetDevice(restore);
    if (status != FFN_OK) return status; /* unique_ptrs free what was uploaded: all or nothing */
    for (int i = 0; i < count; ++i) out[i] = result[i].release();
    return FFN_OK;
}

}  // namespace ffn

using namespace ffn;

extern "C" {

struct FfnQuantManifest { Manifest m; };

int ffn_sha256_hex(const void *data, size_t len, char *out65) {
    if ((!data && len) || !out65) return FFN_ERR_CONFIG;
    Sha256 sha;
    sha.update((const uint8_t *)data, len);
    sha.finish(out65);
    return FFN_OK;
}

int ffn_quant_manifest_parse(const char *json, FfnQuantManifest **out) {
    clear_error();
    if (!json || !out) return qfail(QM_ARG, "quant manifest: null argument");
    std::unique_ptr<FfnQuantManifest> h(new FfnQuantManifest());
    const int st = parse_manifest(json, &h->m);
    if (st != QM_OK) return st;
    *out = h.release();
    return QM_OK;
}

void ffn_quant_manifest_free(FfnQuantManifest *m) { delete m; }

int ffn_quant_manifest_counts(const FfnQuantManifest *m, int *entries, int *pairs, int *int4_cells, int *bf16_cells) {
    if (!m) return QM_ARG;
    if (entries) *entries = (int)m->m.entries.size();
    if (pairs) *pairs = (int)m->m.pairs.size();
    if (int4_cells) *int4_cells = m->m.int4_cells;
    if (bf16_cells) *bf16_cells = m->m.bf16_cells;
    return QM_OK;
}

int ffn_quant_manifest_find_entry(const FfnQuantManifest *m, int layer, const char *role) {
    return (m && role) ? find_entry(m->m, layer, role) : -1;
}

int ffn_quant_manifest_find_pair(const FfnQuantManifest *m, const char *name, int layer) {
    return (m && name) ? find_pair(m->m, name, layer) : -1;
}

int ffn_quant_manifest_entry_shape(const FfnQuantManifest *m, int index, long long *n, long long *k, long long *group, int *role_index) {
    if (!m || index < 0 || index >= (int)m->m.entries.size()) return QM_ARG;
    const Entry &e = m->m.entries[index];
    if (n) *n = e.n;
    if (k) *k = e.k;
    if (group) *group = e.group;
    if (role_index) *role_index = e.role_index;
    return QM_OK;
}

int ffn_quant_manifest_pair_shape(const FfnQuantManifest *m, int index, long long *n, long long *k, long long *group) {
    if (!m || index < 0 || index >= (int)m->m.pairs.size()) return QM_ARG;
    const Pair &p = m->m.pairs[index];
    if (n) *n = p.n;
    if (k) *k = p.k;
    if (group) *group = p.group;
    return QM_OK;
}

int ffn_quant_artifact_read(const char *root, const char *file, const char *dtype, long long bytes, const char *sha256,
                            const char *want_dtype, uint8_t **out, size_t *out_len) {
    clear_error();
    if (!root || !file || !dtype || !sha256 || !out || !out_len) return qfail(QM_ARG, "quant artifact: null argument");
    *out = nullptr;
    *out_len = 0;
    Artifact a;
    a.file = file; a.dtype = dtype; a.bytes = bytes; a.sha256 = sha256;
    std::vector<uint8_t> data;
    const int st = read_artifact_file(root, a, want_dtype, &data);
    if (st != QM_OK) return st;
    uint8_t *buf = (uint8_t *)malloc(data.size() ? data.size() : 1);
    if (!buf) return qfail(QM_IO, "quant artifact: out of memory");
    memcpy(buf, data.data(), data.size());
    *out = buf;
    *out_len = data.size();
    return QM_OK;
}

void ffn_host_free(void *p) { free(p); }

int ffn_shard_view(int rule, long long rows, long long cols, int tp, int rank, long long *view4) {
    clear_error();
    if (!view4) return fail(FFN_ERR_CONFIG, "ffn_shard_view: null argument");
    return shard_view(rule, rows, cols, tp, rank, view4);
}

/* Registers the k-major copy of every loaded layer's down projection (see ffn_decode_layer_prepare).
 * All or nothing. */
static int prepare_loaded(QuantizedFfn *q) {
    int restore = 0;
    (void)cudaGetDevice(&restore);
    int st = FFN_OK;
    if (cudaSetDevice(q->device) != cudaSuccess) st = fail(FFN_ERR_CUDA, "ffn_quantized_ffn_prepare_decode: cannot select device %d", q->device);
    FfnModelDims dims = {};
    dims.hidden_size = q->hidden;
    dims.intermediate_size = q->inter_local;
    for (int l = 0; l < q->layers && st == FFN_OK; ++l) {
        FfnMlpWeights w = {};
        w.down_i4 = q->layer[l].down;
        w.down_i4_scales = q->layer[l].down_scales;
        w.i4_group = FFN_INT4_GROUP;
        st = ffn_decode_layer_prepare(&w, &dims, nullptr);
    }
    if (st == FFN_OK && cudaDeviceSynchronize() != cudaSuccess) st = fail(FFN_ERR_CUDA, "ffn_quantized_ffn_prepare_decode: building the k-major copies failed");
    (void)cudaSetDevice(restore);
    return st;
}

int ffn_load_quantized_ffn(const char *manifest_dir, int num_layers, int hidden, int intermediate, int tp, int rank,
                           FfnQuantizedFfn **out) {
    clear_error();
    if (!out) return fail(FFN_ERR_CONFIG, "ffn_load_quantized_ffn: null argument");
    int dev = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "ffn_load_quantized_ffn: no CUDA device");
    QuantizedFfn *q = nullptr;
    int st = load_ranks(manifest_dir, num_layers, hidden, intermediate, tp < 1 ? 1 : tp, &rank, &dev, 1, &q);
    if (st == FFN_OK) *out = (FfnQuantizedFfn *)q;
    return st;
}

int ffn_quantized_ffn_prepare_decode(FfnQuantizedFfn *handle) {
    clear_error();
    if (!handle) return fail(FFN_ERR_CONFIG, "ffn_quantized_ffn_prepare_decode: null handle");
    return prepare_loaded((QuantizedFfn *)handle);
}

int ffn_load_quantized_ffn_ranks(const char *manifest_dir, int num_layers, int hidden, int intermediate, int tp,
                                 const int *devices, FfnQuantizedFfn **out) {
    clear_error();
    if (!out || !devices || tp < 1 || tp > 16) return fail(FFN_ERR_CONFIG, "ffn_load_quantized_ffn_ranks: bad arguments");
    int ranks[16];
    QuantizedFfn *q[16] = {};
    for (int i = 0; i < tp; ++i) ranks[i] = i;
    int st = load_ranks(manifest_dir, num_layers, hidden, intermediate, tp, ranks, devices, tp, q);
    if (st != FFN_OK) {
        for (int i = 0; i < tp; ++i) delete q[i];
        return st;
    }
    for (int i = 0; i < tp; ++i) out[i] = (FfnQuantizedFfn *)q[i];
    return st;
}

int ffn_quantized_ffn_layer(const FfnQuantizedFfn *handle, int layer, FfnMlpWeights *w) {
    clear_error();
    const QuantizedFfn *q = (const QuantizedFfn *)handle;
    if (!q || !w) return fail(FFN_ERR_CONFIG, "ffn_quantized_ffn_layer: null argument");
    if (layer < 0 || layer >= q->layers) return fail(FFN_ERR_CONFIG, "ffn_quantized_ffn_layer: layer %d is outside [0, %d)", layer, q->layers);
    const LoadedLayer &l = q->layer[layer];
    w->gate_up_i4 = l.gate_up;
    w->gate_up_i4_scales = l.gate_up_scales;
    w->down_i4 = l.down;
    w->down_i4_scales = l.down_scales;
    w->i4_group = FFN_INT4_GROUP;
    return FFN_OK;
}

int ffn_quantized_ffn_free(FfnQuantizedFfn *handle) {
    delete (QuantizedFfn *)handle;
    return FFN_OK;
}

}  // extern "C"
