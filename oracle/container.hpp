// CPU oracle (TEST INFRASTRUCTURE, not a product path): reader for the compact
// container (\x89PTWC) and the single-tensor frame (\x89PTWS) of ptwm-core, and
// the per-tensor decode driver.  Citations are file:line under
// crates/ptwm-core/src.  Only the production split / passthrough chains are
// understood; everything else raises "unsupported".
#pragma once
#include <array>
#include <atomic>
#include <functional>
#include <map>
#include <mutex>
#include <set>
#include <thread>

#include "codecs.hpp"

namespace oracle {

// Dynamic-schedule parallel loop over [0, n) on `threads` std::threads (the
// stand-in for the reference's rayon par_iter).
inline void parallel_for(size_t n, int threads, const std::function<void(size_t)>& fn) {
    if (threads <= 1 || n <= 1) { for (size_t i = 0; i < n; ++i) fn(i); return; }
    std::atomic<size_t> next{0};
    auto body = [&]() { for (;;) { size_t i = next.fetch_add(1); if (i >= n) return; fn(i); } };
    std::vector<std::thread> pool;
    size_t nt = std::min<size_t>(size_t(threads), n);
    for (size_t t = 1; t < nt; ++t) pool.emplace_back(body);
    body();
    for (auto& t : pool) t.join();
}

// varint.rs:57-73 (canonical LEB128) and varint.rs:76+ (Cursor)
struct Cursor {
    const uint8_t* buf; size_t len; size_t pos = 0; const char* what;
    Cursor(const uint8_t* b, size_t n, const char* w) : buf(b), len(n), what(w) {}
    [[noreturn]] void fail(const std::string& m) const { throw Error(std::string(what) + ": " + m + " at byte " + std::to_string(pos)); }
    size_t remaining() const { return len - pos; }
    uint8_t u8() { if (pos >= len) fail("truncated"); return buf[pos++]; }
    const uint8_t* take(size_t n) { if (n > remaining()) fail("truncated"); const uint8_t* p = buf + pos; pos += n; return p; }
    uint32_t u32le() { return get_u32le(take(4)); }
    uint64_t u64le() { return get_u64le(take(8)); }
    uint64_t varint() {
        uint64_t v = 0;
        for (int i = 0; i < 10; ++i) {
            if (pos + size_t(i) >= len) fail("truncated varint");
            uint8_t b = buf[pos + size_t(i)];
            if (i == 9 && b > 1) fail("varint overflows u64");
            v |= uint64_t(b & 0x7F) << (7 * i);
            if ((b & 0x80) == 0) {
                if (i > 0 && b == 0) fail("non-minimal varint");
                pos += size_t(i) + 1;
                return v;
            }
        }
        fail("varint overflows u64");
    }
    uint64_t varint_max(uint64_t max, const char* field) { uint64_t v = varint(); if (v > max) fail(std::string(field) + " too large"); return v; }
    size_t len_varint() { uint64_t v = varint(); if (v > remaining()) fail("length exceeds the buffer"); return size_t(v); }
    std::pair<const uint8_t*, size_t> len_bytes() { size_t n = len_varint(); return {take(n), n}; }
    void finish(const char* after) { if (pos != len) fail(std::string("trailing bytes after ") + after); }
};

inline void write_varint(Bytes& out, uint64_t v) {  // varint.rs:17-23
    while (v >= 0x80) { out.push_back(uint8_t(v) | 0x80); v >>= 7; }
    out.push_back(uint8_t(v));
}

// transforms/op.rs:11-36
enum OpId : uint16_t { OP_SOURCE = 0x0000, OP_REORDER16 = 0x0010, OP_REORDER32 = 0x0011, OP_REORDER_E4M3 = 0x0012, OP_REORDER_E5M2 = 0x0013,
                      OP_BYTESPLIT = 0x0020, OP_NIBBLESPLIT = 0x0021, OP_PASSTHROUGH = 0x0030, OP_INTDELTA = 0x0052, OP_MANTISSA_ZERO_STRIP = 0x0064 };

struct ChainNode { uint16_t op; Bytes params; };
struct ChainEdge { uint8_t src, src_out, dst, dst_in; };
struct ChainTerminal { uint8_t node, out, role; };
struct Chain { std::vector<ChainNode> nodes; std::vector<ChainEdge> edges; std::vector<ChainTerminal> terms; };

// chain/wire_compact.rs:258-372.  `bound` = params of a bound Source (null:
// keep it empty, the registry form).  op_ref values go through `resolve`.
template <class Resolve>
inline Chain read_chain_cw2(Cursor& r, const Bytes* bound, bool deferred, Resolve resolve) {
    Chain c;
    size_t n_nodes = size_t(r.varint_max(255, "chain node count"));
    if (n_nodes == 0) r.fail("chain has no nodes");
    size_t n_edges = size_t(r.varint_max(255, "chain edge count"));
    size_t n_terms = size_t(r.varint_max(255, "chain terminal count"));
    if (r.remaining() < 2 * n_nodes + 2 * n_terms) r.fail("chain truncated");
    for (size_t i = 0; i < n_nodes; ++i) {
        uint16_t op = resolve(r.varint());
        size_t plen = size_t(r.varint_max(255, "chain node params length"));
        ChainNode node{op, {}};
        if (op == OP_SOURCE && plen == 0) {
            if (!deferred) {
                if (!bound) r.fail("chain has a bound Source but the tensor has no bindable shape and dtype");
                node.params = *bound;
            }
        } else {
            const uint8_t* p = r.take(plen);
            node.params.assign(p, p + plen);
            if (op == OP_SOURCE && !deferred && bound && node.params == *bound) r.fail("chain Source params equal the bound Source (non-canonical)");
        }
        c.nodes.push_back(std::move(node));
    }
    if (n_edges > 0) {
        size_t n_spine = size_t(r.varint_max(n_edges, "chain spine edge count"));
        for (size_t i = 0; i < n_spine; ++i) c.edges.push_back({uint8_t(i), 0, uint8_t(i + 1), 0});
        for (size_t i = n_spine; i < n_edges; ++i) {
            uint8_t idx[4];
            for (auto& v : idx) v = uint8_t(r.varint_max(255, "chain edge index"));
            uint8_t etag = r.u8();
            if (etag != 0) r.fail("unsupported: chain edge with role override or vendor bytes");
            if (i == n_spine && idx[0] == i && idx[1] == 0 && idx[2] == i + 1 && idx[3] == 0) r.fail("chain spine edge stored explicitly (non-canonical)");
            c.edges.push_back({idx[0], idx[1], idx[2], idx[3]});
        }
    }
    for (size_t i = 0; i < n_terms; ++i) {
        uint8_t b = r.u8();
        uint8_t node, out;
        if (b == 0xFF) { node = r.u8(); out = r.u8(); if (node <= 14 && out <= 15) r.fail("chain terminal ref escaped needlessly"); }
        else if ((b >> 4) == 15) r.fail("chain terminal ref byte is reserved");
        else { node = b >> 4; out = b & 0x0F; }
        uint8_t role = r.u8();
        if (role == 0xFF) r.fail("unsupported: escaped terminal role");
        c.terms.push_back({node, out, role});
    }
    return c;
}

// transforms/source.rs:31-63,69-85 — chain dtype storage bytes and the
// public→chain dtype map.
inline uint64_t chain_dtype_bytes(uint16_t cd) {
    switch (cd) {
        case 0x0002: case 0x000F: case 0x0007: case 0x0008: return 2;
        case 0x0003: case 0x0009: case 0x000A: return 4;
        case 0x0004: case 0x000B: case 0x000C: return 8;
        default: return 1;  // bytes, fp8, packed fp4 (one byte per element)
    }
}
inline int chain_dtype_for_public(uint16_t code) {
    switch (code) {
        case 1: case 2: return 0x0003; case 4: case 5: return 0x0002; case 6: return 0x000F; case 13: return 0x0006;
        case 15: return 0x000A; case 17: return 0x0005; case 18: case 19: return 0x0007; case 20: case 21: return 0x0009;
        case 22: case 23: return 0x000B; case 29: return 0x0010; case 30: return 0x0011; case 31: return 0x001F;
        default: return -1;
    }
}
// dtype.rs:60-66,140-170 — element size of a public dtype code, 0 if unknown.
inline uint32_t public_dtype_size(uint16_t code) {
    switch (code) {
        case 13: case 17: case 24: case 29: case 30: case 31: return 1;
        case 4: case 5: case 6: case 18: case 19: return 2;
        case 1: case 2: case 15: case 20: case 21: return 4;
        case 22: case 23: return 8;
        default: return 0;
    }
}
// transforms/source.rs:96-106
inline bool bound_source_params(const std::vector<uint64_t>& shape, uint16_t dtype_code, Bytes& out) {
    int cd = chain_dtype_for_public(dtype_code);
    if (cd < 0 || shape.size() > 255) return false;
    out.clear();
    out.push_back(uint8_t(shape.size()));
    for (uint64_t d : shape) { if (d > 0xFFFFFFFFull) return false; uint8_t b[4]; put_u32le(b, uint32_t(d)); out.insert(out.end(), b, b + 4); }
    out.push_back(uint8_t(cd)); out.push_back(uint8_t(cd >> 8));
    return true;
}

// A per-plane op between the split and the terminal (python/ptwm/preprocessing/_chains.py:360-389,486-534).
enum PostOp : uint8_t { POST_NONE = 0, POST_INTDELTA = 1, POST_MZS = 2 };
struct ChainInfo {
    MergeKind kind; uint64_t source_len; uint64_t plane_len; uint64_t row_len; /* Source last dim, 0 = scalar */
    uint8_t post[4] = {0, 0, 0, 0};    // PostOp of terminal plane i
    uint8_t post_k[4] = {0, 0, 0, 0};  // MantissaZeroStrip: bits stripped
};

// transforms/int_delta.rs:36-44 at byte width (the split planes are byte planes): out[i] = in[i] - in[i-1], wrapping.
inline void int_delta_forward_u8(Bytes& b) { uint8_t prev = 0; for (auto& v : b) { uint8_t cur = v; v = uint8_t(cur - prev); prev = cur; } }
inline void int_delta_inverse_u8(Bytes& b) { uint8_t acc = 0; for (auto& v : b) { acc = uint8_t(acc + v); v = acc; } }
// transforms/mantissa_zero.rs:38-44: forward shifts every byte right by k (all low k bits must be zero), inverse shifts left.
inline void mzs_forward(Bytes& b, unsigned k) {
    for (auto v : b) if (v & ((1u << k) - 1)) throw Error("MantissaZeroStrip.forward: plane has a byte with non-zero low bits");
    for (auto& v : b) v = uint8_t(v >> k);
}
inline void mzs_inverse(Bytes& b, unsigned k) { for (auto& v : b) v = uint8_t(v << k); }
inline void post_forward(const ChainInfo& info, size_t plane, Bytes& b) {
    if (info.post[plane] == POST_INTDELTA) int_delta_forward_u8(b); else if (info.post[plane] == POST_MZS) mzs_forward(b, info.post_k[plane]);
}
inline void post_inverse(const ChainInfo& info, size_t plane, Bytes& b) {
    if (info.post[plane] == POST_INTDELTA) int_delta_inverse_u8(b); else if (info.post[plane] == POST_MZS) mzs_inverse(b, info.post_k[plane]);
}

// Source params (transforms/source.rs:120-178) + the descriptor walk of
// chain/runtime.rs:359-439 restricted to the production chains
// (python/ptwm/preprocessing/_chains.py:320-357,610-727) and their variants
// with IntDelta or MantissaZeroStrip on single planes of a byte split
// (_chains.py:360-389,486-560).
inline ChainInfo analyse_chain(const Chain& c) {
    if (c.nodes.empty() || c.nodes[0].op != OP_SOURCE) throw Error("chain: node[0] must be Source");
    const Bytes& sp = c.nodes[0].params;
    if (sp.size() < 3 || sp.size() != size_t(3 + 4 * sp[0])) throw Error("chain: malformed Source params");
    uint64_t n_elem = 1, last = 0;
    for (size_t d = 0; d < sp[0]; ++d) {
        uint64_t dim = get_u32le(&sp[1 + 4 * d]);
        if (dim != 0 && n_elem > UINT64_MAX / dim) throw Error("chain: Source element count overflows");
        n_elem *= dim; last = dim;
    }
    uint16_t cd = uint16_t(sp[sp.size() - 2] | (sp[sp.size() - 1] << 8));
    ChainInfo info{PASS, n_elem * chain_dtype_bytes(cd), 0, sp[0] ? last : 0};
    if (c.edges.size() + 1 != c.nodes.size()) throw Error("unsupported: chain is not a tree over its nodes");
    const size_t nn = c.nodes.size();
    // nodes after a byte split: each takes one output of the split (node 2) and feeds one terminal
    const bool split16 = nn >= 3 && c.nodes[1].op == OP_REORDER16 && c.nodes[2].op == OP_BYTESPLIT && c.nodes[2].params == Bytes{2};
    const bool split32 = nn >= 3 && c.nodes[1].op == OP_REORDER32 && c.nodes[2].op == OP_BYTESPLIT && c.nodes[2].params == Bytes{4};
    const size_t spine = (split16 || split32) ? 2 : c.edges.size();
    for (size_t i = 0; i < spine; ++i) {
        const ChainEdge& e = c.edges[i];
        if (e.src != i || e.src_out != 0 || e.dst != i + 1 || e.dst_in != 0) throw Error("unsupported: chain is not a linear spine");
    }
    auto terms_are = [&](size_t node, size_t n) {
        if (c.terms.size() != n) return false;
        for (size_t i = 0; i < n; ++i) if (c.terms[i].node != node || c.terms[i].out != i) return false;
        return true;
    };
    if (split16 || split32) {
        const size_t np = split16 ? 2 : 4;
        if (info.source_len % np) throw Error(split16 ? "chain: 16-bit split of an odd length" : "chain: 32-bit split of a length not divisible by 4");
        info.kind = split16 ? M16 : M32; info.plane_len = info.source_len / np;
        int node_of_plane[4] = {-1, -1, -1, -1};
        for (size_t i = 2; i < c.edges.size(); ++i) {
            const ChainEdge& e = c.edges[i];
            if (e.src != 2 || e.src_out >= np || e.dst < 3 || e.dst >= nn || e.dst_in != 0 || node_of_plane[e.src_out] >= 0)
                throw Error("unsupported: chain outside the production split/passthrough set");
            for (size_t j = 2; j < i; ++j) if (c.edges[j].dst == e.dst) throw Error("unsupported: chain outside the production split/passthrough set");
            const ChainNode& nd = c.nodes[e.dst];
            if (nd.op == OP_INTDELTA && nd.params.empty()) info.post[e.src_out] = POST_INTDELTA;
            else if (nd.op == OP_MANTISSA_ZERO_STRIP && nd.params.size() == 1 && nd.params[0] >= 1 && nd.params[0] <= 7) { info.post[e.src_out] = POST_MZS; info.post_k[e.src_out] = nd.params[0]; }
            else throw Error("unsupported: chain outside the production split/passthrough set");
            node_of_plane[e.src_out] = e.dst;
        }
        if (c.terms.size() != np) throw Error("unsupported: chain outside the production split/passthrough set");
        for (size_t i = 0; i < np; ++i) {
            const bool direct = node_of_plane[i] < 0 && c.terms[i].node == 2 && c.terms[i].out == i;
            const bool via = node_of_plane[i] >= 0 && c.terms[i].node == node_of_plane[i] && c.terms[i].out == 0;
            if (!direct && !via) throw Error("unsupported: chain outside the production split/passthrough set");
        }
        return info;
    }
    if (nn == 1 && terms_are(0, 1)) { info.kind = PASS; info.plane_len = info.source_len; }
    else if (nn == 2 && c.nodes[1].op == OP_PASSTHROUGH && terms_are(1, 1)) { info.kind = PASS; info.plane_len = info.source_len; }
    else if (nn == 3 && c.nodes[1].op == OP_REORDER_E4M3 && c.nodes[2].op == OP_NIBBLESPLIT && terms_are(2, 2)) { info.kind = FP8_E4M3; info.plane_len = info.source_len; }
    else if (nn == 3 && c.nodes[1].op == OP_REORDER_E5M2 && c.nodes[2].op == OP_NIBBLESPLIT && terms_are(2, 2)) { info.kind = FP8_E5M2; info.plane_len = info.source_len; }
    else throw Error("unsupported: chain outside the production split/passthrough set");
    return info;
}

// Compact Extension Table (extension/compact_table.rs:50-261): built-ins only.
struct TableEntry { int kind; /* 1 op, 2 codec, 3 named */ uint16_t id; std::string name; };
inline std::vector<TableEntry> read_compact_table(const uint8_t* b, size_t n) {
    Cursor r(b, n, "compact extension table");
    uint64_t count = r.varint_max(1 << 16, "entry count");
    if (count > n / 2) r.fail("entry count exceeds the table bytes");
    std::vector<TableEntry> out;
    std::set<std::pair<int, std::string>> seen;
    for (uint64_t i = 0; i < count; ++i) {
        uint8_t tag = r.u8();
        TableEntry e{tag, 0, {}};
        if (tag == 1 || tag == 2) e.id = uint16_t(r.varint_max(0xFFFF, "wire id"));
        else if (tag == 3) { uint64_t l = r.varint_max(255, "built-in name length"); if (l == 0) r.fail("empty built-in name"); const uint8_t* p = r.take(size_t(l)); e.name.assign(reinterpret_cast<const char*>(p), size_t(l)); }
        else if (tag == 0x7F) r.fail("unsupported: third-party extension entry");
        else r.fail("unknown entry tag");
        if (!seen.insert({tag, e.name + "#" + std::to_string(e.id)}).second) r.fail("duplicate entry");
        out.push_back(e);
    }
    r.finish("the last entry");
    return out;
}

struct PreludeEntry { uint16_t id, codec; uint8_t version, mask; uint64_t hash; Bytes state; };
inline std::vector<PreludeEntry> parse_prelude(const uint8_t* b, size_t n) {  // prelude.rs:66-160
    if (n < 4) throw Error("prelude too short");
    size_t count = get_u32le(b);
    if (count > (n - 4) / 22) throw Error("prelude count exceeds buffer capacity");
    size_t pos = 4;
    std::vector<PreludeEntry> out;
    for (size_t i = 0; i < count; ++i) {
        if (pos + 18 > n) throw Error("prelude entry truncated");
        PreludeEntry e;
        e.id = uint16_t(b[pos] | (b[pos + 1] << 8)); e.codec = uint16_t(b[pos + 2] | (b[pos + 3] << 8));
        e.version = b[pos + 4]; e.mask = b[pos + 5];
        e.hash = get_u64le(b + pos + 8);
        size_t name_len = size_t(b[pos + 16]) | size_t(b[pos + 17]) << 8;
        pos += 18;
        size_t pad = (4 - name_len % 4) % 4;
        if (pos + name_len + pad + 4 > n) throw Error("prelude entry name truncated");
        pos += name_len + pad;
        size_t sl = get_u32le(b + pos); pos += 4;
        if (pos + sl > n) throw Error("prelude entry state_bytes truncated");
        e.state.assign(b + pos, b + pos + sl); pos += sl;
        out.push_back(std::move(e));
    }
    if (pos != n) throw Error("prelude has trailing bytes");
    return out;
}

struct ChunkEntry { uint32_t offset, decoded; };
struct PlaneRec {
    uint8_t pflags, role; uint16_t codec_ref, codec_id; int state_source; uint8_t state_version = 0; uint16_t state_info = 0;
    uint64_t row_len = 0; bool has_crc = false; uint32_t crc = 0; bool chunked = false; std::vector<ChunkEntry> chunks;
    const uint8_t* inline_state = nullptr; size_t inline_len = 0; const uint8_t* payload = nullptr; size_t payload_len = 0;
};
struct TensorRec {
    std::string name; uint8_t tflags; int chain_id = -1; uint16_t dtype_code; uint8_t input_format; uint64_t orig_size;
    bool has_shape = false; std::vector<uint64_t> shape; std::string dtype_name; bool has_hash = false; uint64_t hash = 0;
    Chain chain; ChainInfo info; std::vector<PlaneRec> planes; size_t rec_off = 0, rec_len = 0;
    std::string unsupported;  // non-empty: the record uses a feature outside the hot path; decode refuses it
};

inline const char* canonical_dtype_name(uint16_t code) {  // dtype.rs:140-165
    switch (code) {
        case 1: return "float32"; case 2: return "float"; case 4: return "float16"; case 5: return "half"; case 6: return "bfloat16";
        case 13: return "uint8"; case 15: return "uint32"; case 17: return "int8"; case 18: return "int16"; case 19: return "short";
        case 20: return "int32"; case 21: return "int"; case 22: return "int64"; case 23: return "long"; case 24: return "bool";
        case 29: return "float8_e4m3fn"; case 30: return "float8_e5m2"; case 31: return "float4_e2m1fn_x2"; default: return nullptr;
    }
}

struct Container {
    const uint8_t* buf; size_t len;
    std::vector<TableEntry> table; std::vector<PreludeEntry> prelude; std::vector<Chain> registry; std::vector<TensorRec> tensors;
};

static const uint8_t MAGIC_PTWC[9] = {0x89, 'P', 'T', 'W', 'C', '\r', '\n', 0x1a, '\n'};
static const uint8_t EOF_SENTINEL[8] = {0x89, 'T', 'W', 'M', 'E', 'O', 'F', 0x1a};
static const uint8_t MAGIC_PTWS[5] = {0x89, 'P', 'T', 'W', 'S'};

// tensor_record_compact.rs:659-811
inline PlaneRec read_plane(Cursor& r, const std::vector<TableEntry>& table) {
    PlaneRec p;
    p.pflags = r.u8();
    if (p.pflags & ~0x3F) r.fail("unknown pflags bits");
    p.state_source = (p.pflags & 0x0C) >> 2;
    p.role = r.u8();
    static const uint8_t roles[] = {1, 2, 3, 4, 5, 6, 0x10, 0x11, 0x12, 0x13};
    if (std::find(std::begin(roles), std::end(roles), p.role) == std::end(roles)) r.fail("unknown plane role");
    p.codec_ref = uint16_t(r.varint_max(0xFFFF, "codec_ref"));
    if (p.codec_ref >= table.size()) r.fail("codec_ref is outside the Extension Table");
    if (table[p.codec_ref].kind != 2) r.fail("codec_ref names an entry that is not a plane codec");
    p.codec_id = table[p.codec_ref].id;
    if (p.pflags & 0x20) {
        p.state_version = r.u8();
        p.state_info = uint16_t(r.varint_max(0xFFFF, "state_info"));
        if (p.state_version == 0 && p.state_info == 0) r.fail("PF_STATE_EXTRA with zero state_version and state_info");
    }
    if (p.state_source == 1) p.inline_len = r.len_varint();
    p.payload_len = r.len_varint();
    if (p.pflags & 0x10) { p.row_len = r.varint_max(0xFFFFFFFFull, "row_len"); if (p.row_len == 0) r.fail("row_len 0"); }
    if (p.pflags & 0x01) { p.has_crc = true; p.crc = r.u32le(); }
    if (p.pflags & 0x02) {
        p.chunked = true;
        uint64_t n = r.varint_max(p.payload_len, "chunk count");
        if (n > r.remaining() / 2) r.fail("chunk count exceeds the record");
        for (uint64_t i = 0; i < n; ++i) {
            uint32_t off = uint32_t(r.varint_max(0xFFFFFFFFull, "chunk offset"));
            uint32_t sz = uint32_t(r.varint_max(0xFFFFFFFFull, "chunk decoded size"));
            p.chunks.push_back({off, sz});
        }
    }
    if (p.state_source == 3) r.fail("unsupported: external plane state");
    p.inline_state = r.take(p.inline_len);
    p.payload = r.take(p.payload_len);
    return p;
}

// tensor_record_compact.rs:497-657 (dependencies and inline chains with
// third-party ops are outside the hot path: rejected as unsupported).
inline TensorRec parse_record(const uint8_t* b, size_t n, const Container& c) {
    Cursor r(b, n, "compact tensor record");
    TensorRec t;
    t.tflags = r.u8();
    if (t.tflags & ~0x3F) r.fail("unknown tflags bits");
    bool inline_chain = t.tflags & 0x02;
    if ((t.tflags & 0x10) && !(t.tflags & 0x08)) r.fail("TF_DTYPE_NAME without TF_SHAPE");
    if ((t.tflags & 0x20) && (t.tflags & 0x08)) r.fail("TF_RAW_META with TF_SHAPE");
    if (!inline_chain) {
        uint64_t id = r.varint();
        if (id >= c.registry.size()) r.fail("chain id is not in the registry");
        t.chain_id = int(id);
    }
    t.dtype_code = uint16_t(r.varint_max(0xFFFF, "dtype_code"));
    t.input_format = r.u8();
    t.orig_size = r.varint();
    Bytes binding; bool have_binding = false;
    if (t.tflags & 0x08) {
        size_t ndim = size_t(r.varint_max(64, "ndim"));
        if (ndim > r.remaining()) r.fail("truncated shape");
        for (size_t i = 0; i < ndim; ++i) t.shape.push_back(r.varint());
        t.has_shape = true;
        const char* canon = canonical_dtype_name(t.dtype_code);
        if (t.tflags & 0x10) {
            auto [p, l] = r.len_bytes();
            t.dtype_name.assign(reinterpret_cast<const char*>(p), l);
            if (canon && t.dtype_name == canon) r.fail("stored dtype name equals the canonical name (non-canonical)");
        } else {
            if (!canon) r.fail("shape without a dtype name for a dtype_code that has no canonical name");
            t.dtype_name = canon;
        }
        have_binding = bound_source_params(t.shape, t.dtype_code, binding);
    } else if (t.tflags & 0x20) {
        r.len_bytes();  // raw CBOR metadata: carried, not interpreted
    }
    if (t.tflags & 0x01) { t.has_hash = true; t.hash = r.u64le(); }
    if (inline_chain) {
        auto [et, etl] = r.len_bytes();
        std::vector<TableEntry> ops = read_compact_table(et, etl);
        auto [cb, cl] = r.len_bytes();
        Cursor cr(cb, cl, "compact chain");
        t.chain = read_chain_cw2(cr, have_binding ? &binding : nullptr, false, [&](uint64_t ref) -> uint16_t {
            if (ref >= ops.size() || ops[size_t(ref)].kind != 1) cr.fail("inline chain op_ref outside its table");
            return ops[size_t(ref)].id;
        });
        cr.finish("chain");
    } else {
        t.chain = c.registry[size_t(t.chain_id)];
        // container.rs:1826-1841 — a bound Source takes the record's shape.
        if (t.chain.nodes[0].op == OP_SOURCE && t.chain.nodes[0].params.empty()) {
            if (!have_binding) r.fail("registry chain has a bound Source, but the record has no shape that binds it");
            t.chain.nodes[0].params = binding;
        }
    }
    if (t.tflags & 0x04) r.fail("unsupported: tensor dependencies");
    uint64_t n_planes = r.varint_max(255, "plane count");
    if (n_planes > r.remaining() / 4) r.fail("plane count exceeds the record");
    for (uint64_t i = 0; i < n_planes; ++i) t.planes.push_back(read_plane(r, c.table));
    r.finish("the last plane");
    t.info = analyse_chain(t.chain);
    return t;
}

// ptwc.rs:105-297 + container.rs:1525-1626
inline Container open_container(const uint8_t* buf, size_t len) {
    Container c{buf, len, {}, {}, {}, {}};
    if (len < 9 + 2 + 16 || std::memcmp(buf, MAGIC_PTWC, 9) != 0) throw Error("compact container: bad magic or file too short");
    if (std::memcmp(buf + len - 8, EOF_SENTINEL, 8) != 0) throw Error("compact container: missing EOF sentinel");
    size_t footer = len - 16;
    Cursor r(buf, footer, "compact container header");
    r.take(9);
    uint16_t hflags = uint16_t(r.u8()); hflags |= uint16_t(r.u8()) << 8;
    if (hflags != 0) r.fail("unknown hflags bits");
    uint64_t et_len = r.varint(), prelude_len = r.varint(), registry_len = r.varint();
    size_t hash_pos = r.pos;
    uint64_t stored = r.u64le();
    size_t hdr_end = r.pos;
    auto section = [&](size_t start, uint64_t l, const char* w) { if (l > footer - start) throw Error(std::string("compact container: ") + w + " section exceeds the file"); return start + size_t(l); };
    size_t et_end = section(hdr_end, et_len, "extension table");
    size_t pre_end = section(et_end, prelude_len, "prelude");
    size_t reg_end = section(pre_end, registry_len, "registry");
    uint64_t index_len = get_u64le(buf + footer);
    if (index_len > footer) throw Error("compact container: index_len exceeds the file");
    size_t index_start = footer - size_t(index_len);
    if (reg_end > index_start) throw Error("compact container: index overlaps the registry");
    Bytes meta(buf, buf + hash_pos);
    meta.insert(meta.end(), buf + hdr_end, buf + reg_end);
    if (xxh64(meta.data(), meta.size(), 0) != stored) throw Error("compact container: meta_xxh64 mismatch");
    c.table = read_compact_table(buf + hdr_end, et_end - hdr_end);
    c.prelude = parse_prelude(buf + et_end, pre_end - et_end);
    {
        Cursor rr(buf + pre_end, reg_end - pre_end, "compact chain registry");
        size_t count = size_t(rr.varint_max(0x8000, "chain count"));
        if (count > (reg_end - pre_end) / 6) rr.fail("chain count exceeds the registry bytes");
        for (size_t i = 0; i < count; ++i) {
            auto [cb, cl] = rr.len_bytes();
            Cursor cr(cb, cl, "compact chain");
            c.registry.push_back(read_chain_cw2(cr, nullptr, true, [&](uint64_t ref) -> uint16_t {
                if (ref >= c.table.size() || c.table[size_t(ref)].kind != 1) cr.fail("op_ref is not a built-in transform");
                return c.table[size_t(ref)].id;
            }));
            cr.finish("chain");
        }
        rr.finish("the last chain");
    }
    Cursor ir(buf + index_start, footer - index_start, "compact container index");
    uint64_t count = ir.varint();
    if (count > (footer - index_start) / 3) ir.fail("entry count exceeds the index bytes");
    size_t off = reg_end;
    std::set<std::string> names;
    for (uint64_t i = 0; i < count; ++i) {
        size_t nl = size_t(ir.varint_max(65535, "name length"));
        if (nl == 0) ir.fail("empty tensor name");
        const uint8_t* np = ir.take(nl);
        std::string name(reinterpret_cast<const char*>(np), nl);
        if (!names.insert(name).second) ir.fail("duplicate tensor name");
        uint64_t rl = ir.varint();
        if (rl < 3) ir.fail("record too short");
        if (rl > index_start - off) ir.fail("record runs past the body");
        TensorRec t;
        try { t = parse_record(buf + off, size_t(rl), c); }
        catch (const Error& e) {
            if (std::string(e.what()).find("unsupported") == std::string::npos) throw;
            t = TensorRec{}; t.unsupported = e.what(); t.info = ChainInfo{PASS, 0, 0, 0};
        }
        t.name = name; t.rec_off = off; t.rec_len = size_t(rl);
        c.tensors.push_back(std::move(t));
        off += size_t(rl);
    }
    ir.finish("the last index entry");
    if (off != index_start) throw Error("compact container: records do not cover the body");
    return c;
}

// container.rs:1795-2196 (strict = compact layout).  `threads` > 1 decodes
// the chunks of a plane in parallel like the reference's par_iter
// (container.rs:1995-2045); tensors are parallelised by the caller.
inline Bytes decode_record(const Container& c, const TensorRec& t, bool verify = true, int threads = 1) {
    if (!t.unsupported.empty()) throw Error(t.unsupported);
    const ChainInfo& info = t.info;
    if (info.source_len != t.orig_size) throw Error("decode_tensor: chain Source size differs from orig_size");
    if (int(t.planes.size()) != merge_planes(info.kind)) throw Error("decode_tensor: plane count differs from the chain's terminals");
    const uint64_t plane_bound = t.orig_size * 16 + 4096;  // chain/runtime.rs:317-319
    std::vector<Bytes> planes(t.planes.size());
    for (size_t pi = 0; pi < t.planes.size(); ++pi) {
        const PlaneRec& p = t.planes[pi];
        CodecId cid = CodecId(p.codec_id);
        Bytes& out = planes[pi];
        if (p.chunked) {
            uint64_t total = 0;
            for (auto& e : p.chunks) total += e.decoded;
            if (total > plane_bound || total != info.plane_len) throw Error("chunk table does not decode to the plane's length");
            out.resize(size_t(total));
            std::vector<size_t> dst_off(p.chunks.size());
            size_t acc = 0;
            for (size_t i = 0; i < p.chunks.size(); ++i) { dst_off[i] = acc; acc += p.chunks[i].decoded; }
            std::string err;
            std::mutex err_mu;
            parallel_for(p.chunks.size(), threads, [&](size_t i) {
                try {
                    size_t start = p.chunks[size_t(i)].offset;
                    size_t end = size_t(i) + 1 < p.chunks.size() ? p.chunks[size_t(i) + 1].offset : p.payload_len;
                    if (start > end || end > p.payload_len) throw Error("chunk table offset out of bounds");
                    const uint8_t* frame = p.payload + start; size_t fl = end - start;
                    if (fl < 5) throw Error("chunk frame truncated");
                    uint8_t sv = frame[0];
                    size_t sl = get_u32le(frame + 1);
                    if (fl - 5 < sl) throw Error("chunk frame state_len exceeds frame");
                    size_t want = p.chunks[size_t(i)].decoded;
                    Bytes d = plane_decode(cid, sv, frame + 5, sl, frame + 5 + sl, fl - 5 - sl, p.row_len, want, want);
                    if (d.size() != want) throw Error("chunk decoded_size mismatch");
                    std::memcpy(out.data() + dst_off[size_t(i)], d.data(), want);
                } catch (const std::exception& e) {
                    std::lock_guard<std::mutex> g(err_mu);
                    err = e.what();
                }
            });
            if (!err.empty()) throw Error(err);
        } else {
            const uint8_t* state = nullptr; size_t sl = 0; uint8_t sv = 0;
            if (p.state_source == 1) { state = p.inline_state; sl = p.inline_len; sv = p.state_version; }
            else if (p.state_source == 2) {
                const PreludeEntry* pe = nullptr;
                for (auto& e : c.prelude) if (e.id == p.state_info) { pe = &e; break; }
                if (!pe) throw Error("shared state not in prelude");
                if (p.state_version != pe->version) throw Error("shared state version mismatch");
                if (p.role >= 1 && p.role <= 8 && !(pe->mask & (1u << (p.role - 1)))) throw Error("shared state applies_to_mask does not cover the plane role");
                if (xxh64(pe->state.data(), pe->state.size(), 0) != pe->hash) throw Error("shared state xxhash64 mismatch");
                state = pe->state.data(); sl = pe->state.size(); sv = pe->version;
            }
            out = plane_decode(cid, sv, state, sl, p.payload, p.payload_len, p.row_len, size_t(info.plane_len), size_t(info.plane_len));
            if (out.size() != info.plane_len) throw Error("decoded plane length differs from its descriptor");
        }
        if (verify && p.has_crc && crc32(out.data(), out.size()) != p.crc) throw Error("plane CRC mismatch");  // of the terminal's bytes
        post_inverse(info, pi, out);
    }
    Bytes raw = merge_inverse(info.kind, planes);
    if (raw.size() != t.orig_size) throw Error("decode_tensor: chain decoded a different length than orig_size");
    if (verify && t.has_hash && xxh64(raw.data(), raw.size(), 0) != t.hash) throw Error("tensor payload hash mismatch");
    return raw;
}

// compact.rs:321-551 — single-tensor frame.
struct CompactTensor { uint16_t dtype_code; uint8_t input_format; bool has_shape; std::vector<uint64_t> shape; std::string dtype_name; Bytes raw; };
inline CompactTensor decode_compact(const uint8_t* buf, size_t len) {
    Cursor r(buf, len, "compact frame");
    if (len < 5 || std::memcmp(buf, MAGIC_PTWS, 5) != 0) r.fail("bad magic");
    r.take(5);
    uint8_t flags = r.u8();
    if (flags & 0x80) r.fail("unknown flag bits");
    if ((flags & 0x02) && (flags & 0x01)) r.fail("plane CRC flag with payload hash");
    CompactTensor t;
    t.dtype_code = uint16_t(r.varint_max(0xFFFF, "dtype_code"));
    t.input_format = r.u8();
    bool have_stored = flags & 0x40; uint64_t stored = 0;
    if (have_stored) stored = r.varint();
    t.has_shape = flags & 0x04;
    const char* canon = canonical_dtype_name(t.dtype_code);
    if (t.has_shape) {
        uint64_t ndim = r.varint_max(64, "ndim");
        for (uint64_t i = 0; i < ndim; ++i) t.shape.push_back(r.varint());
        if (canon) t.dtype_name = canon;
    }
    if (flags & 0x08) {
        if (!t.has_shape) r.fail("dtype name without shape");
        auto [p, l] = r.len_bytes();
        std::string nm(reinterpret_cast<const char*>(p), l);
        if (canon && nm == canon) r.fail("stored dtype name equals the canonical name");
        t.dtype_name = nm;
    } else if (t.has_shape && !canon) r.fail("shape without a dtype name for unknown dtype_code");
    bool have_derived = false; uint64_t derived = 0;
    if (t.has_shape && public_dtype_size(t.dtype_code)) {
        derived = public_dtype_size(t.dtype_code); have_derived = true;
        for (uint64_t d : t.shape) { if (d != 0 && derived > UINT64_MAX / d) { have_derived = false; break; } derived *= d; }
    }
    uint64_t orig;
    if (have_stored && have_derived && stored == derived) r.fail("stored orig_size equals the size the shape gives");
    if (have_stored) orig = stored; else if (have_derived) orig = derived; else r.fail("no orig_size and no shape that gives it");
    if (flags & 0x10) r.take(32);
    bool has_hash = flags & 0x01; uint64_t hash = 0;
    if (has_hash) hash = r.u64le();
    if (flags & 0x20) {
        if (flags & 0x02) r.fail("stored frame with plane CRC flag");
        if (r.remaining() != orig) r.fail("stored body length differs from orig_size");
        const uint8_t* p = r.take(size_t(orig));
        t.raw.assign(p, p + orig);
    } else {
        Bytes binding; bool hb = t.has_shape && bound_source_params(t.shape, t.dtype_code, binding);
        Chain ch = read_chain_cw2(r, hb ? &binding : nullptr, false, [&](uint64_t ref) -> uint16_t { if (ref > 0xFFFF) r.fail("op id exceeds u16"); return uint16_t(ref); });
        ChainInfo info = analyse_chain(ch);
        if (info.source_len != orig) r.fail("chain Source size differs from the header");
        std::vector<Bytes> planes;
        for (int pi = 0; pi < merge_planes(info.kind); ++pi) {
            uint64_t head = r.varint();
            if ((head >> 2) > 0xFFFF) r.fail("codec id exceeds u16");
            CodecId cid = CodecId(head >> 2);
            uint8_t sv = 0; const uint8_t* st = nullptr; size_t sl = 0;
            switch (head & 3) {
                case 0: case 2: break;
                case 1: { sv = r.u8(); auto [p, l] = r.len_bytes(); st = p; sl = l; if (sv == 0 && sl == 0) r.fail("empty version-0 inline state must use state code 2"); break; }
                default: r.fail("unknown state code");
            }
            size_t pl = r.len_varint();
            bool has_crc = flags & 0x02; uint32_t crc = 0;
            if (has_crc) crc = r.u32le();
            const uint8_t* payload = r.take(pl);
            // The frame stores no layout: it follows the chain's Source (compact.rs:500-503).
            uint64_t row_len = info.kind == PASS ? info.row_len : 0;
            Bytes d = plane_decode(cid, sv, st, sl, payload, pl, row_len, size_t(info.plane_len), size_t(info.plane_len));
            if (d.size() != info.plane_len) r.fail("plane decoded to a different length than the chain says");
            if (has_crc && crc32(d.data(), d.size()) != crc) r.fail("plane CRC mismatch");
            post_inverse(info, size_t(pi), d);
            planes.push_back(std::move(d));
        }
        t.raw = merge_inverse(info.kind, planes);
        if (t.raw.size() != orig) r.fail("decoded length differs from the header");
    }
    r.finish("body");
    if (has_hash && xxh64(t.raw.data(), t.raw.size(), 0) != hash) r.fail("payload hash mismatch");
    return t;
}

}  // namespace oracle
