// Prepared-weights loader and the TP -> EP re-partition of the routed experts.
//
// Upstream keeps a prepared model as a JSON manifest next to one binary payload `data.bin` (src/prepared.rs:15-377,
// docs/ARTIFACTS.md "Prepared target"): format 1 = file size, chunk size and one SHA-256 per chunk, a storage table
// (offset, nbytes, device), a serialized object tree whose leaves are tensors (storage index, dtype, shape, stride,
// element offset), and a preparation key.  The loader checks the geometry, verifies every chunk it reads, uploads
// the selected storages and resolves tensor paths such as `weights.layers[3].moe.experts.gt` to device pointers
// (Loaded::pointer, src/prepared.rs:366-377) -- the nine pointers of glmflash_weights.
//
// Upstream's shards are tensor parallel: every rank holds a 512-wide slice of every expert's intermediate
// (src/experts.rs:146-156).  glmflash_expert_bank_from_tp puts the four slices of an expert window back together,
// so that an expert-parallel rank owns whole experts.
//
// Everything up to glmflash_prepared_verify runs without a GPU.
#include <stdio.h>
#include <sys/stat.h>

#include <map>
#include <memory>
#include <new>
#include <string>
#include <utility>
#include <vector>

#include "common.cuh"

namespace {

// ---- SHA-256 (FIPS 180-4) ---------------------------------------------------------------------------------
struct Sha256 {
    uint32_t h[8];
    uint64_t bits = 0;
    unsigned char buf[64];
    size_t fill = 0;
    Sha256() {
        static const uint32_t init[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
        memcpy(h, init, sizeof(h));
    }
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const unsigned char *p) {
        static const uint32_t K[64] = {
            0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u, 0xd807aa98u, 0x12835b01u, 0x243185beu,
            0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u, 0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau,
            0x5cb0a9dcu, 0x76f988dau, 0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u, 0x27b70a85u,
            0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u, 0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u,
            0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u, 0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu,
            0x682e6ff3u, 0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
        uint32_t w[64];
        for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
        for (int i = 16; i < 64; ++i) {
            const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; ++i) {
            const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + K[i] + w[i];
            const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const unsigned char *p, size_t n) {
        bits += (uint64_t)n * 8;
        while (n) {
            if (fill == 0 && n >= 64) { block(p); p += 64; n -= 64; continue; }
            const size_t take = std::min(n, (size_t)64 - fill);
            memcpy(buf + fill, p, take);
            fill += take; p += take; n -= take;
            if (fill == 64) { block(buf); fill = 0; }
        }
    }
    std::string hex() {
        const uint64_t total = bits;
        unsigned char pad[72] = {0x80};
        const size_t padlen = (fill < 56 ? 56 : 120) - fill;
        unsigned char len[8];
        for (int i = 0; i < 8; ++i) len[i] = (unsigned char)(total >> (56 - 8 * i));
        update(pad, padlen);
        update(len, 8);
        char out[65];
        for (int i = 0; i < 8; ++i) snprintf(out + 8 * i, 9, "%08x", h[i]);
        return std::string(out, 64);
    }
};

// ---- a small JSON reader (objects keep their member order) -------------------------------------------------
struct JNode {
    enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
    bool b = false, is_int = false;
    double num = 0;
    int64_t inum = 0;
    std::string str;
    std::vector<JNode> arr;
    std::vector<std::pair<std::string, JNode>> obj;
    const JNode *get(const char *k) const {
        if (kind != OBJ) return nullptr;
        for (auto &kv : obj)
            if (kv.first == k) return &kv.second;
        return nullptr;
    }
};
struct JParser {
    const char *p, *end;
    std::string err;
    int depth = 0;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail(const char *m) { if (err.empty()) err = m; return false; }
    bool str(std::string &out) {
        if (p >= end || *p != '"') return fail("expected string");
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("bad escape");
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (end - p < 5) return fail("bad \\u escape");
                        unsigned v = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char c = p[i];
                            v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 0);
                        }
                        p += 4;
                        if (v < 0x80) out += (char)v;
                        else if (v < 0x800) { out += (char)(0xC0 | (v >> 6)); out += (char)(0x80 | (v & 0x3F)); }
                        else { out += (char)(0xE0 | (v >> 12)); out += (char)(0x80 | ((v >> 6) & 0x3F)); out += (char)(0x80 | (v & 0x3F)); }
                        break;
                    }
                    default: out += *p;
                }
                ++p;
            } else out += *p++;
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool value(JNode &n) {
        if (++depth > 200) return fail("nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end");
        bool ok = true;
        if (*p == '{') {
            n.kind = JNode::OBJ;
            ++p; ws();
            if (p < end && *p == '}') ++p;
            else
                for (;;) {
                    ws();
                    std::string k;
                    if (!str(k)) { ok = false; break; }
                    ws();
                    if (p >= end || *p != ':') { ok = fail("expected ':'"); break; }
                    ++p;
                    n.obj.emplace_back(std::move(k), JNode());
                    if (!value(n.obj.back().second)) { ok = false; break; }
                    ws();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == '}') { ++p; break; }
                    ok = fail("expected ',' or '}'");
                    break;
                }
        } else if (*p == '[') {
            n.kind = JNode::ARR;
            ++p; ws();
            if (p < end && *p == ']') ++p;
            else
                for (;;) {
                    n.arr.emplace_back();
                    if (!value(n.arr.back())) { ok = false; break; }
                    ws();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == ']') { ++p; break; }
                    ok = fail("expected ',' or ']'");
                    break;
                }
        } else if (*p == '"') {
            n.kind = JNode::STR;
            ok = str(n.str);
        } else if (end - p >= 4 && !strncmp(p, "true", 4)) { n.kind = JNode::BOOL; n.b = true; p += 4; }
        else if (end - p >= 5 && !strncmp(p, "false", 5)) { n.kind = JNode::BOOL; p += 5; }
        else if (end - p >= 4 && !strncmp(p, "null", 4)) { n.kind = JNode::NUL; p += 4; }
        else {
            const char *s = p;
            bool integral = true;
            if (p < end && *p == '-') ++p;
            while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) {
                if (*p == '.' || *p == 'e' || *p == 'E') integral = false;
                ++p;
            }
            if (p == s) ok = fail("unexpected character");
            else {
                const std::string t(s, p);
                n.kind = JNode::NUM;
                n.num = strtod(t.c_str(), nullptr);
                n.is_int = integral;
                if (integral) n.inum = strtoll(t.c_str(), nullptr, 10);
            }
        }
        --depth;
        return ok;
    }
};
bool as_u64(const JNode *n, uint64_t &v) {
    if (!n || n->kind != JNode::NUM || !n->is_int || n->inum < 0) return false;
    v = (uint64_t)n->inum;
    return true;
}
std::string json_key_text(const JNode &n) {          // how a dict key prints inside a tensor path (strings keep their quotes)
    switch (n.kind) {
        case JNode::STR: return "\"" + n.str + "\"";
        case JNode::NUM: return n.is_int ? std::to_string(n.inum) : std::to_string(n.num);
        case JNode::BOOL: return n.b ? "true" : "false";
        default: return "null";
    }
}

struct Storage {
    uint64_t offset = 0, nbytes = 0;
    bool cuda = false;
    void *dev = nullptr;                           // uploaded copy (cuda storages), or nullptr
    std::vector<unsigned char> host;               // loaded copy (cpu storages)
    bool loaded = false;
};
struct Tensor {
    size_t storage = 0;
    std::string dtype;
    std::vector<uint64_t> shape, stride;
    uint64_t off = 0;
    bool cuda = false;
};
int element_bytes(const std::string &d) {            // src/prepared.rs:42-50
    if (d == "bool" || d == "uint8" || d == "int8" || d == "float8_e4m3fn" || d == "float8_e5m2") return 1;
    if (d == "bfloat16" || d == "float16" || d == "int16" || d == "uint16") return 2;
    if (d == "float32" || d == "int32" || d == "uint32") return 4;
    if (d == "float64" || d == "int64" || d == "uint64") return 8;
    return 0;
}
bool mul_ok(uint64_t a, uint64_t b, uint64_t &r) { return !__builtin_mul_overflow(a, b, &r); }
bool add_ok(uint64_t a, uint64_t b, uint64_t &r) { return !__builtin_add_overflow(a, b, &r); }
// Bytes from the start of the storage to the end of the last element (src/prepared.rs:51-69); false on overflow.
bool tensor_extent(const Tensor &t, uint64_t &out) {
    const int eb = element_bytes(t.dtype);
    if (!eb || t.shape.size() != t.stride.size()) return false;
    for (uint64_t n : t.shape)
        if (n == 0) return mul_ok(t.off, (uint64_t)eb, out);
    uint64_t last = t.off;
    for (size_t i = 0; i < t.shape.size(); ++i) {
        uint64_t span;
        if (!mul_ok(t.shape[i] - 1, t.stride[i], span) || !add_ok(last, span, last)) return false;
    }
    return add_ok(last, 1, last) && mul_ok(last, (uint64_t)eb, out);
}

}  // namespace

struct glmflash_prepared {
    std::string manifest_path, data_path;
    uint64_t file_size = 0, chunk = 0;
    std::vector<std::string> chunk_sha256;
    std::vector<Storage> storages;
    std::map<std::string, Tensor> tensors;
    std::vector<std::string> names;                // tensor paths, sorted
    JNode key;
};

namespace {
int walk(const JNode &node, const std::string &path, std::map<std::string, Tensor> &out) {          // src/prepared.rs:101-137
    GF_REQUIRE(node.kind == JNode::OBJ, "prepared node is not an object: " + path);
    if (node.get("T")) {
        Tensor t;
        uint64_t v;
        GF_REQUIRE(as_u64(node.get("T"), v), "tensor storage index: " + path);
        t.storage = (size_t)v;
        const JNode *d = node.get("dtype"), *sh = node.get("shape"), *st = node.get("stride"), *dev = node.get("dev");
        GF_REQUIRE(d && d->kind == JNode::STR && sh && sh->kind == JNode::ARR && st && st->kind == JNode::ARR && dev && dev->kind == JNode::STR &&
                       as_u64(node.get("off"), t.off), "tensor record is incomplete: " + path);
        t.dtype = d->str;
        t.cuda = dev->str == "cuda";
        for (auto &x : sh->arr) { GF_REQUIRE(as_u64(&x, v), "tensor shape: " + path); t.shape.push_back(v); }
        for (auto &x : st->arr) { GF_REQUIRE(as_u64(&x, v), "tensor stride: " + path); t.stride.push_back(v); }
        out[path] = t;
    } else if (const JNode *f = node.get("f")) {
        const JNode *o = node.get("O");
        GF_REQUIRE(o && o->kind == JNode::STR, "untyped object: " + path);
        GF_REQUIRE(f->kind == JNode::OBJ, "object fields: " + path);
        for (auto &kv : f->obj)
            if (walk(kv.second, path + "." + kv.first, out)) return -1;
    } else if (node.get("L") || node.get("U")) {
        const JNode *a = node.get("L") ? node.get("L") : node.get("U");
        GF_REQUIRE(a->kind == JNode::ARR, "sequence: " + path);
        for (size_t i = 0; i < a->arr.size(); ++i)
            if (walk(a->arr[i], path + "[" + std::to_string(i) + "]", out)) return -1;
    } else if (const JNode *dct = node.get("D")) {
        GF_REQUIRE(dct->kind == JNode::ARR, "dict: " + path);
        for (auto &pair : dct->arr) {
            GF_REQUIRE(pair.kind == JNode::ARR && pair.arr.size() == 2, "dict pair: " + path);
            if (walk(pair.arr[1], path + "[" + json_key_text(pair.arr[0]) + "]", out)) return -1;
        }
    } else if (node.get("N")) {
        return gf::fail("NumPy storage is unsupported: " + path);
    } else {
        GF_REQUIRE(node.obj.size() == 1 && (node.get("P") || node.get("dev")), "unknown prepared node " + path);
    }
    return 0;
}
}  // namespace

extern "C" int glmflash_prepared_open(const char *manifest_path, glmflash_prepared **out) {
    GF_REQUIRE(manifest_path && out, "null argument");
    *out = nullptr;
    FILE *f = fopen(manifest_path, "rb");
    GF_REQUIRE(f != nullptr, std::string("cannot open manifest ") + manifest_path);
    std::string text;
    char buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    fclose(f);
    JParser jp{text.data(), text.data() + text.size()};
    JNode root;
    GF_REQUIRE(jp.value(root) && root.kind == JNode::OBJ, "manifest is not valid JSON: " + jp.err);
    std::unique_ptr<glmflash_prepared> p(new (std::nothrow) glmflash_prepared());
    GF_REQUIRE(p != nullptr, "out of host memory");
    p->manifest_path = manifest_path;
    uint64_t format = 0;
    GF_REQUIRE(as_u64(root.get("format"), format) && format == 1, "unsupported prepared format");
    GF_REQUIRE(as_u64(root.get("file_size"), p->file_size) && as_u64(root.get("chunk"), p->chunk), "manifest lacks file_size / chunk");
    GF_REQUIRE(p->chunk > 0 && p->chunk <= 128ull * 1024 * 1024, "invalid chunk size");
    const JNode *hashes = root.get("chunk_sha256"), *stor = root.get("storages"), *tree = root.get("tree"), *key = root.get("key");
    GF_REQUIRE(hashes && hashes->kind == JNode::ARR && stor && stor->kind == JNode::ARR && tree && key, "manifest lacks chunk_sha256 / storages / tree / key");
    for (auto &h : hashes->arr) {
        GF_REQUIRE(h.kind == JNode::STR && h.str.size() == 64, "chunk hash is not a SHA-256 hex string");
        p->chunk_sha256.push_back(h.str);
    }
    GF_REQUIRE(p->chunk_sha256.size() == (p->file_size + p->chunk - 1) / p->chunk, "chunk hash count");
    const std::string mp(manifest_path);
    const size_t slash = mp.find_last_of('/');
    p->data_path = (slash == std::string::npos ? std::string() : mp.substr(0, slash + 1)) + "data.bin";
    struct stat sb;
    GF_REQUIRE(stat(p->data_path.c_str(), &sb) == 0, "data.bin is missing next to the manifest");
    GF_REQUIRE((uint64_t)sb.st_size == p->file_size, "data file size mismatch");
    uint64_t prev = 0;
    for (auto &s : stor->arr) {
        Storage st;
        const JNode *dev = s.get("dev");
        GF_REQUIRE(as_u64(s.get("offset"), st.offset) && as_u64(s.get("nbytes"), st.nbytes) && dev && dev->kind == JNode::STR, "storage record is incomplete");
        GF_REQUIRE(st.nbytes > 0 && st.offset >= prev, "empty/overlapping/out-of-order storage");
        GF_REQUIRE(add_ok(st.offset, st.nbytes, prev), "storage overflow");
        GF_REQUIRE(prev <= p->file_size, "storage outside data file");
        GF_REQUIRE(dev->str == "cuda" || dev->str == "cpu", "unknown storage device");
        st.cuda = dev->str == "cuda";
        p->storages.push_back(std::move(st));
    }
    if (walk(*tree, "weights", p->tensors)) return -1;
    GF_REQUIRE(!p->tensors.empty(), "no tensors");
    for (auto &kv : p->tensors) {
        GF_REQUIRE(kv.second.storage < p->storages.size(), "missing storage: " + kv.first);
        const Storage &s = p->storages[kv.second.storage];
        uint64_t ext;
        GF_REQUIRE(tensor_extent(kv.second, ext), "tensor " + kv.first + ": unsupported dtype, rank mismatch or overflow");
        GF_REQUIRE(ext <= s.nbytes, "tensor " + kv.first + " escapes storage");
        GF_REQUIRE(kv.second.cuda == s.cuda, "tensor " + kv.first + " changes device");
        p->names.push_back(kv.first);
    }
    p->key = *key;
    *out = p.release();
    return 0;
}

extern "C" void glmflash_prepared_close(glmflash_prepared *p) {
    if (!p) return;
    for (auto &s : p->storages)
        if (s.dev) cudaFree(s.dev);
    delete p;
}

extern "C" int glmflash_prepared_key_int(const glmflash_prepared *p, const char *name, int64_t *value) {
    GF_REQUIRE(p && name && value, "null argument");
    const JNode *n = p->key.get(name);
    GF_REQUIRE(n && n->kind == JNode::NUM && n->is_int, std::string("the preparation key has no integer ") + name);
    *value = n->inum;
    return 0;
}

extern "C" int glmflash_prepared_tensor_count(const glmflash_prepared *p) { return p ? (int)p->names.size() : 0; }
extern "C" const char *glmflash_prepared_tensor_name(const glmflash_prepared *p, int i) {
    return p && i >= 0 && i < (int)p->names.size() ? p->names[i].c_str() : nullptr;
}

extern "C" int glmflash_prepared_tensor(const glmflash_prepared *p, const char *name, glmflash_tensor_info *info) {
    GF_REQUIRE(p && name && info, "null argument");
    auto it = p->tensors.find(name);
    GF_REQUIRE(it != p->tensors.end(), std::string("missing tensor ") + name);
    const Tensor &t = it->second;
    GF_REQUIRE(t.shape.size() <= 8, std::string("tensor rank above 8: ") + name);
    memset(info, 0, sizeof(*info));
    snprintf(info->dtype, sizeof(info->dtype), "%s", t.dtype.c_str());
    info->rank = (int32_t)t.shape.size();
    uint64_t dense = 1;
    bool contiguous = true;
    for (int i = info->rank - 1; i >= 0; --i) {
        info->shape[i] = (int64_t)t.shape[i];
        info->stride[i] = (int64_t)t.stride[i];
        contiguous = contiguous && t.stride[i] == dense;
        dense *= t.shape[i];
    }
    const int eb = element_bytes(t.dtype);
    uint64_t ext = 0;
    tensor_extent(t, ext);
    info->nbytes = (int64_t)(ext - t.off * eb);
    info->contiguous = contiguous;
    info->on_device = t.cuda;
    const Storage &s = p->storages[t.storage];
    if (s.loaded) info->ptr = t.cuda ? (void *)((unsigned char *)s.dev + t.off * eb) : (void *)(const_cast<unsigned char *>(s.host.data()) + t.off * eb);
    return 0;
}

namespace {
// Reads the payload chunk by chunk, checks every chunk a selected storage touches against its SHA-256 and hands the
// overlap of (chunk, storage) to `sink` (src/prepared.rs:289-341).  selected == nullptr: every chunk is checked.
template <typename Sink>
int stream_chunks(glmflash_prepared *p, const std::vector<char> *selected, unsigned char *staging, Sink sink) {
    FILE *f = fopen(p->data_path.c_str(), "rb");
    GF_REQUIRE(f != nullptr, "cannot open " + p->data_path);
    uint64_t offset = 0;
    size_t first = 0;
    int rc = 0;
    for (size_t i = 0; i < p->chunk_sha256.size() && !rc; ++i) {
        const uint64_t len = std::min(p->file_size - offset, p->chunk);
        bool needed = selected == nullptr;
        if (selected)
            for (size_t j = 0; j < p->storages.size(); ++j)
                needed = needed || ((*selected)[j] && p->storages[j].offset < offset + len && p->storages[j].offset + p->storages[j].nbytes > offset);
        if (!needed) { offset += len; continue; }
        if (fseeko(f, (off_t)offset, SEEK_SET) != 0 || fread(staging, 1, len, f) != len) { rc = gf::fail("short read from " + p->data_path); break; }
        Sha256 sha;
        sha.update(staging, len);
        if (sha.hex() != p->chunk_sha256[i]) { rc = gf::fail("weight hash mismatch in chunk " + std::to_string(i)); break; }
        while (first < p->storages.size() && p->storages[first].offset + p->storages[first].nbytes <= offset) ++first;
        for (size_t j = first; j < p->storages.size() && !rc; ++j) {
            const Storage &s = p->storages[j];
            if (s.offset >= offset + len) break;
            if (selected && !(*selected)[j]) continue;
            const uint64_t lo = std::max(s.offset, offset), hi = std::min(s.offset + s.nbytes, offset + len);
            rc = sink(j, lo - s.offset, staging + (lo - offset), hi - lo);
        }
        offset += len;
    }
    fclose(f);
    return rc;
}
}  // namespace

extern "C" int glmflash_prepared_verify(glmflash_prepared *p) {
    GF_REQUIRE(p != nullptr, "null argument");
    std::vector<unsigned char> staging(p->chunk);
    return stream_chunks(p, nullptr, staging.data(), [](size_t, uint64_t, const unsigned char *, uint64_t) { return 0; });
}

extern "C" int glmflash_prepared_load(glmflash_prepared *p, const char *const *prefixes, int n_prefixes) {
    GF_REQUIRE(p != nullptr && (n_prefixes == 0 || prefixes != nullptr), "null argument");
    std::vector<char> selected(p->storages.size(), n_prefixes == 0);
    for (auto &kv : p->tensors)
        for (int k = 0; k < n_prefixes; ++k)
            if (kv.first.compare(0, strlen(prefixes[k]), prefixes[k]) == 0) selected[kv.second.storage] = 1;
    for (size_t j = 0; j < p->storages.size(); ++j) {
        Storage &s = p->storages[j];
        if (!selected[j] || s.loaded) { selected[j] = selected[j] && !s.loaded; continue; }
        if (s.cuda) GF_CUDA(cudaMalloc(&s.dev, s.nbytes));
        else s.host.resize(s.nbytes);
    }
    unsigned char *staging = nullptr;
    GF_CUDA(cudaMallocHost((void **)&staging, p->chunk));
    const int rc = stream_chunks(p, &selected, staging, [&](size_t j, uint64_t dst, const unsigned char *src, uint64_t n) {
        Storage &s = p->storages[j];
        if (s.cuda) GF_CUDA(cudaMemcpy((unsigned char *)s.dev + dst, src, n, cudaMemcpyHostToDevice));
        else memcpy(s.host.data() + dst, src, n);
        return 0;
    });
    cudaFreeHost(staging);
    if (rc) return -1;
    for (size_t j = 0; j < p->storages.size(); ++j)
        if (selected[j]) p->storages[j].loaded = true;
    return 0;
}

// ---- TP shards -> whole experts of an expert-parallel window ------------------------------------------------
struct glmflash_expert_bank {
    int hidden = 0, inter = 0, e_lo = 0, e_hi = 0;
    void *t[9] = {};                               // gt ut dt suh_g suh_u suh_d svh_g svh_u svh_d, local experts only
};

extern "C" void glmflash_expert_bank_free(glmflash_expert_bank *b) {
    if (!b) return;
    for (void *q : b->t) cudaFree(q);
    delete b;
}

extern "C" int glmflash_expert_bank_from_tp(glmflash_prepared *const *shards, int n_shards, const char *stem, int e_lo, int e_hi, void *stream,
                                            glmflash_expert_bank **out) {
    GF_REQUIRE(shards && stem && out && n_shards >= 1 && n_shards <= 16, "null argument or shard count outside 1..16");
    *out = nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    static const char *names[9] = {"gt", "ut", "dt", "suh_g", "suh_u", "suh_d", "svh_g", "svh_u", "svh_d"};
    glmflash_tensor_info info[16][9];
    for (int r = 0; r < n_shards; ++r)
        for (int k = 0; k < 9; ++k) {
            const std::string path = std::string(stem) + "." + names[k];
            if (glmflash_prepared_tensor(shards[r], path.c_str(), &info[r][k])) return -1;
            const glmflash_tensor_info &t = info[r][k];
            GF_REQUIRE(t.ptr && t.on_device && t.contiguous, "shard tensor is not loaded on the device or not contiguous: " + path);
            GF_REQUIRE(!strcmp(t.dtype, k < 3 ? "int32" : "float16") && t.rank == (k < 3 ? 4 : 2), "unexpected dtype / rank: " + path);
            for (int d = 0; d < t.rank; ++d) GF_REQUIRE(t.shape[d] == info[0][k].shape[d], "the shards disagree on the shape of " + path);
        }
    // shapes of a shard (src/experts.rs:146-156): gt, ut [E][H/16][Ir/16][32]; dt [E][Ir/16][H/16][32]; suh_g/u, svh_d [E][H]; suh_d, svh_g/u [E][Ir]
    const int64_t E = info[0][0].shape[0], KT = info[0][0].shape[1], NTr = info[0][0].shape[2];
    const int64_t H = KT * 16, Ir = NTr * 16, I = Ir * n_shards;
    GF_REQUIRE(info[0][0].shape[3] == 32 && info[0][2].shape[0] == E && info[0][2].shape[1] == NTr && info[0][2].shape[2] == KT && info[0][2].shape[3] == 32,
               "trellis tensors do not have the TP slice layout [E][H/16][I/16][32] / [E][I/16][H/16][32]");
    GF_REQUIRE(info[0][3].shape[1] == H && info[0][4].shape[1] == H && info[0][8].shape[1] == H && info[0][5].shape[1] == Ir && info[0][6].shape[1] == Ir &&
                   info[0][7].shape[1] == Ir, "scale vectors do not match the trellis shapes");
    GF_REQUIRE(e_lo >= 0 && e_lo < e_hi && e_hi <= E, "expert window outside the bank");
    GF_REQUIRE(H % 256 == 0 && I % 256 == 0, "hidden and the re-assembled intermediate must be multiples of 256");
    std::unique_ptr<glmflash_expert_bank, void (*)(glmflash_expert_bank *)> b(new (std::nothrow) glmflash_expert_bank(), glmflash_expert_bank_free);
    GF_REQUIRE(b != nullptr, "out of host memory");
    b->hidden = (int)H; b->inter = (int)I; b->e_lo = e_lo; b->e_hi = e_hi;
    const int64_t n = e_hi - e_lo, NT = I / 16;
    const size_t bytes[9] = {(size_t)(n * KT * NT * 128), (size_t)(n * KT * NT * 128), (size_t)(n * NT * KT * 128), (size_t)(n * H * 2), (size_t)(n * H * 2),
                             (size_t)(n * I * 2), (size_t)(n * I * 2), (size_t)(n * I * 2), (size_t)(n * H * 2)};
    for (int k = 0; k < 9; ++k) GF_CUDA(cudaMalloc(&b->t[k], bytes[k]));
    for (int r = 0; r < n_shards; ++r) {
        for (int k = 0; k < 2; ++k)                  // gate / up: the shard holds columns [r*Ir, (r+1)*Ir) of every k-tile row
            GF_CUDA(cudaMemcpy2DAsync((unsigned char *)b->t[k] + (size_t)r * NTr * 128, (size_t)NT * 128,
                                      (const unsigned char *)info[r][k].ptr + (size_t)e_lo * KT * NTr * 128, (size_t)NTr * 128, (size_t)NTr * 128,
                                      (size_t)(n * KT), cudaMemcpyDeviceToDevice, s));
        // down: the shard holds k-tile rows [r*Ir/16, (r+1)*Ir/16) of every expert
        GF_CUDA(cudaMemcpy2DAsync((unsigned char *)b->t[2] + (size_t)r * NTr * KT * 128, (size_t)NT * KT * 128,
                                  (const unsigned char *)info[r][2].ptr + (size_t)e_lo * NTr * KT * 128, (size_t)NTr * KT * 128, (size_t)NTr * KT * 128,
                                  (size_t)n, cudaMemcpyDeviceToDevice, s));
        for (int k = 5; k < 8; ++k)                  // suh_d, svh_g, svh_u: sliced along the intermediate
            GF_CUDA(cudaMemcpy2DAsync((unsigned char *)b->t[k] + (size_t)r * Ir * 2, (size_t)I * 2, (const unsigned char *)info[r][k].ptr + (size_t)e_lo * Ir * 2,
                                      (size_t)Ir * 2, (size_t)Ir * 2, (size_t)n, cudaMemcpyDeviceToDevice, s));
    }
    for (int k : {3, 4, 8})                          // suh_g, suh_u, svh_d: every shard holds the whole vector
        GF_CUDA(cudaMemcpyAsync(b->t[k], (const unsigned char *)info[0][k].ptr + (size_t)e_lo * H * 2, (size_t)n * H * 2, cudaMemcpyDeviceToDevice, s));
    *out = b.release();
    return 0;
}

extern "C" int glmflash_expert_bank_weights(const glmflash_expert_bank *b, glmflash_weights *w, int32_t *hidden, int32_t *inter) {
    GF_REQUIRE(b && w, "null argument");
    // The kernels index the bank by the global expert id: the pointers are moved back by e_lo experts, so that ids of the
    // window [e_lo, e_hi) land in the allocation (ids outside the window are never dereferenced: the owners skip them).
    const size_t H = b->hidden, I = b->inter, lo = b->e_lo;
    w->gt = (const uint32_t *)b->t[0] - lo * (H / 16) * (I / 16) * 32;
    w->ut = (const uint32_t *)b->t[1] - lo * (H / 16) * (I / 16) * 32;
    w->dt = (const uint32_t *)b->t[2] - lo * (H / 16) * (I / 16) * 32;
    w->suh_g = (const uint16_t *)b->t[3] - lo * H;
    w->suh_u = (const uint16_t *)b->t[4] - lo * H;
    w->suh_d = (const uint16_t *)b->t[5] - lo * I;
    w->svh_g = (const uint16_t *)b->t[6] - lo * I;
    w->svh_u = (const uint16_t *)b->t[7] - lo * I;
    w->svh_d = (const uint16_t *)b->t[8] - lo * H;
    if (hidden) *hidden = b->hidden;
    if (inter) *inter = b->inter;
    return 0;
}
