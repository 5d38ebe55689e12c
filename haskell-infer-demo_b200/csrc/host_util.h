/*
 * host_util.h - host-side pieces shared by the artifact reader and the converter: SHA-256
 * (FIPS 180-4; the reference's csrc/sha256.c) and a small strict JSON reader (objects refuse
 * duplicate keys; nothing may follow the document).  Header-only, internal to the library.
 */
#pragma once
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <utility>
#include <vector>

namespace ffn {

/* ------------------------------------------------------------------------------------------- */
/* SHA-256 (FIPS 180-4)                                                                          */
/* ------------------------------------------------------------------------------------------- */
static const uint32_t kSha256K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

struct Sha256 {
    uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    uint8_t block[64];
    size_t fill = 0;
    uint64_t total = 0;

    static uint32_t rotr(uint32_t v, int n) { return (v >> n) | (v << (32 - n)); }

    void compress(const uint8_t *p) {
        uint32_t w[64];
        for (int i = 0; i < 16; ++i)
            w[i] = ((uint32_t)p[4 * i] << 24) | ((uint32_t)p[4 * i + 1] << 16) | ((uint32_t)p[4 * i + 2] << 8) | p[4 * i + 3];
        for (int i = 16; i < 64; ++i) {
            const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], k = h[7];
        for (int i = 0; i < 64; ++i) {
            const uint32_t t1 = k + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + kSha256K[i] + w[i];
            const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
            k = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += k;
    }
    void update(const uint8_t *p, size_t n) {
        total += n;
        if (fill) {
            const size_t take = n < 64 - fill ? n : 64 - fill;
            memcpy(block + fill, p, take);
            fill += take; p += take; n -= take;
            if (fill == 64) { compress(block); fill = 0; }
        }
        for (; n >= 64; p += 64, n -= 64) compress(p);
        if (n) { memcpy(block, p, n); fill = n; }
    }
    void finish(char hex[65]) {
        const uint64_t bits = total * 8;
        const uint8_t one = 0x80, zero = 0;
        update(&one, 1);
        while (fill != 56) update(&zero, 1);
        uint8_t len[8];
        for (int i = 0; i < 8; ++i) len[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(len, 8);
        static const char *digits = "0123456789abcdef";
        for (int i = 0; i < 8; ++i)
            for (int j = 0; j < 4; ++j) {
                const uint8_t byte = (uint8_t)(h[i] >> (24 - 8 * j));
                hex[8 * i + 2 * j] = digits[byte >> 4];
                hex[8 * i + 2 * j + 1] = digits[byte & 15];
            }
        hex[64] = '\0';
    }
};

/* ------------------------------------------------------------------------------------------- */
/* A small strict JSON reader (objects refuse duplicate keys; nothing may follow the document).  */
/* `manifest_dialect` switches to what the reference's manifest reader accepts at this level      */
/* (csrc/quant_manifest.c:71-175): duplicate keys are kept for the caller to judge, raw control   */
/* bytes pass, a number may start with '+', and a \u escape above 0x7F is refused (ASCII schema). */
/* ------------------------------------------------------------------------------------------- */
struct Json {
    enum Kind { Null, Bool, Int, Real, Str, Arr, Obj } kind = Null;
    long long i = 0;
    double d = 0;
    bool b = false;
    std::string s;
    std::vector<Json> a;
    std::vector<std::pair<std::string, Json>> o;
    const Json *get(const char *key) const {
        for (const auto &kv : o)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
};

struct JsonReader {
    const char *p, *end;
    std::string error;
    int depth = 0;
    bool manifest_dialect = false;
    explicit JsonReader(const char *text) : p(text), end(text + strlen(text)) {}
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail_at(const char *what) { if (error.empty()) error = std::string("quant manifest: ") + what; return false; }
    bool string(std::string &out) {
        if (p >= end || *p != '"') return fail_at("a string was expected");
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            unsigned char c = (unsigned char)*p++;
            if (c < 0x20 && !manifest_dialect) return fail_at("a control character inside a string");
            if (c == '\\') {
                if (p >= end) return fail_at("the document ends inside a string");
                const char e = *p++;
                switch (e) {
                case '"': out += '"'; break; case '\\': out += '\\'; break; case '/': out += '/'; break;
                case 'b': out += '\b'; break; case 'f': out += '\f'; break; case 'n': out += '\n'; break;
                case 'r': out += '\r'; break; case 't': out += '\t'; break;
                case 'u': {
                    if (end - p < 4) return fail_at("a truncated \\u escape");
                    unsigned v = 0;
                    for (int k = 0; k < 4; ++k) {
                        const char h = *p++;
                        v <<= 4;
                        if (h >= '0' && h <= '9') v |= (unsigned)(h - '0');
                        else if (h >= 'a' && h <= 'f') v |= (unsigned)(h - 'a' + 10);
                        else if (h >= 'A' && h <= 'F') v |= (unsigned)(h - 'A' + 10);
                        else return fail_at("a malformed \\u escape");
                    }
                    if (manifest_dialect && v > 0x7F) return fail_at("a string outside ASCII (the schema is ASCII-only)");
                    if (v < 0x80) out += (char)v;
                    else if (v < 0x800) { out += (char)(0xC0 | (v >> 6)); out += (char)(0x80 | (v & 0x3F)); }
                    else { out += (char)(0xE0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 0x3F)); out += (char)(0x80 | (v & 0x3F)); }
                    break;
                }
                default: return fail_at("an unknown escape");
                }
            } else {
                out += (char)c;
            }
        }
        if (p >= end) return fail_at("the document ends inside a string");
        ++p;
        return true;
    }
    bool value(Json &out) {
        if (++depth > 32) return fail_at("nesting too deep");
        ws();
        if (p >= end) return fail_at("the document is truncated");
        bool ok = true;
        if (*p == '{') {
            out.kind = Json::Obj;
            ++p; ws();
            if (p < end && *p == '}') { ++p; }
            else {
                for (;;) {
                    ws();
                    std::string key;
                    if (!string(key)) { ok = false; break; }
                    if (!manifest_dialect && out.get(key.c_str())) { ok = fail_at(("the key \"" + key + "\" appears twice").c_str()); break; }
                    ws();
                    if (p >= end || *p != ':') { ok = fail_at("':' was expected"); break; }
                    ++p;
                    out.o.emplace_back(key, Json());
                    if (!value(out.o.back().second)) { ok = false; break; }
                    ws();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == '}') { ++p; break; }
                    ok = fail_at("',' or '}' was expected (the document is truncated or malformed)");
                    break;
                }
            }
        } else if (*p == '[') {
            out.kind = Json::Arr;
            ++p; ws();
            if (p < end && *p == ']') { ++p; }
            else {
                for (;;) {
                    out.a.emplace_back();
                    if (!value(out.a.back())) { ok = false; break; }
                    ws();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == ']') { ++p; break; }
                    ok = fail_at("',' or ']' was expected (the document is truncated or malformed)");
                    break;
                }
            }
        } else if (*p == '"') {
            out.kind = Json::Str;
            ok = string(out.s);
        } else if (!strncmp(p, "true", 4)) { out.kind = Json::Bool; out.b = true; p += 4; }
        else if (!strncmp(p, "false", 5)) { out.kind = Json::Bool; out.b = false; p += 5; }
        else if (!strncmp(p, "null", 4)) { out.kind = Json::Null; p += 4; }
        else {
            const char *start = p;
            if (p < end && (*p == '-' || (manifest_dialect && *p == '+'))) ++p;
            bool digits = false, real = false;
            while (p < end && *p >= '0' && *p <= '9') { ++p; digits = true; }
            if (p < end && *p == '.') { real = true; ++p; while (p < end && *p >= '0' && *p <= '9') { ++p; digits = true; } }
            if (p < end && (*p == 'e' || *p == 'E')) {
                real = true; ++p;
                if (p < end && (*p == '+' || *p == '-')) ++p;
                while (p < end && *p >= '0' && *p <= '9') ++p;
            }
            if (!digits) ok = fail_at("a value was expected");
            else {
                const std::string text(start, p);
                if (real) { out.kind = Json::Real; out.d = strtod(text.c_str(), nullptr); }
                else {
                    if (text.size() > 18) ok = fail_at("an integer is out of range");
                    out.kind = Json::Int; out.i = strtoll(text.c_str(), nullptr, 10); out.d = (double)out.i;
                }
            }
        }
        --depth;
        return ok;
    }
};

}  // namespace ffn
