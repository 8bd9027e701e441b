// Host-side reader for the containers of ptwm-core: the compact container
// (\x89PTWC: ptwc.rs, tensor_record_compact.rs, extension/compact_table.rs,
// chain/wire_compact.rs, prelude.rs) and the single-tensor frame (\x89PTWS:
// compact.rs).  It never copies payload bytes: every plane and chunk is
// described by absolute offsets into the file, which later become Refs into
// the device copy of the same bytes.  Paths in comments are relative to
// crates/ptwm-core/src of the reference.
#pragma once
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_set>
#include <vector>

#include "blake3.hpp"
#include "plan.h"

namespace ptwm {

struct FormatError : std::runtime_error {
    bool unsupported;
    FormatError(const std::string& m, bool unsup = false) : std::runtime_error(m), unsupported(unsup) {}
};

inline uint32_t le32(const uint8_t* p) { return uint32_t(p[0]) | uint32_t(p[1]) << 8 | uint32_t(p[2]) << 16 | uint32_t(p[3]) << 24; }
inline uint64_t le64(const uint8_t* p) { return uint64_t(le32(p)) | uint64_t(le32(p + 4)) << 32; }

// XXH64 with seed 0 (xxhash-rust 0.8.18; used for meta_xxh64 and shared state: ptwc.rs:144-149, container.rs:2089).
inline uint64_t xxh64_host(const uint8_t* p, size_t len) {
    const uint64_t P1 = 11400714785074694791ull, P2 = 14029467366897019727ull, P3 = 1609587929392839161ull, P4 = 9650029242287828579ull,
                   P5 = 2870177450012600261ull;
    auto rotl = [](uint64_t x, int r) { return (x << r) | (x >> (64 - r)); };
    auto round = [&](uint64_t acc, uint64_t in) { return rotl(acc + in * P2, 31) * P1; };
    const uint8_t* end = p + len;
    uint64_t h;
    if (len >= 32) {
        uint64_t v[4] = {P1 + P2, P2, 0, 0 - P1};
        for (; p + 32 <= end; p += 32) for (int i = 0; i < 4; ++i) v[i] = round(v[i], le64(p + 8 * i));
        h = rotl(v[0], 1) + rotl(v[1], 7) + rotl(v[2], 12) + rotl(v[3], 18);
        for (int i = 0; i < 4; ++i) h = (h ^ round(0, v[i])) * P1 + P4;
    } else h = P5;
    h += len;
    for (; p + 8 <= end; p += 8) h = rotl(h ^ round(0, le64(p)), 27) * P1 + P4;
    if (p + 4 <= end) { h = rotl(h ^ (uint64_t(le32(p)) * P1), 23) * P2 + P3; p += 4; }
    for (; p < end; ++p) h = rotl(h ^ (uint64_t(*p) * P5), 11) * P1;
    h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
    return h;
}

// Bounds-checked view over one section; varints are canonical LEB128 (varint.rs:57-73).
class Span {
  public:
    Span(const uint8_t* base, size_t begin, size_t end, const char* what) : base_(base), pos_(begin), end_(end), what_(what) {}
    size_t pos() const { return pos_; }
    size_t left() const { return end_ - pos_; }
    [[noreturn]] void bad(const std::string& m, bool unsup = false) const { throw FormatError(std::string(what_) + ": " + m + " (byte " + std::to_string(pos_) + ")", unsup); }
    uint8_t byte() { need(1); return base_[pos_++]; }
    size_t skip(size_t n) { need(n); size_t at = pos_; pos_ += n; return at; }
    uint32_t u32() { return le32(base_ + skip(4)); }
    uint64_t u64() { return le64(base_ + skip(8)); }
    uint64_t var() {
        uint64_t v = 0;
        for (int i = 0; i < 10; ++i) {
            if (pos_ + size_t(i) >= end_) bad("truncated varint");
            uint8_t b = base_[pos_ + size_t(i)];
            if (i == 9 && b > 1) bad("varint overflows u64");
            v |= uint64_t(b & 0x7F) << (7 * i);
            if (!(b & 0x80)) { if (i > 0 && b == 0) bad("non-minimal varint"); pos_ += size_t(i) + 1; return v; }
        }
        bad("varint overflows u64");
    }
    uint64_t var_max(uint64_t max, const char* field) { uint64_t v = var(); if (v > max) bad(std::string(field) + " out of range"); return v; }
    size_t var_len() { uint64_t v = var(); if (v > left()) bad("length exceeds the section"); return size_t(v); }
    void done(const char* after) const { if (pos_ != end_) bad(std::string("trailing bytes after ") + after); }
    const uint8_t* at(size_t off) const { return base_ + off; }

  private:
    void need(size_t n) const { if (n > end_ - pos_) bad("truncated"); }
    const uint8_t* base_;
    size_t pos_, end_;
    const char* what_;
};

struct ChunkDesc {
    uint64_t frame_off;   // absolute offset of the chunk frame (or of the plane payload when unchunked)
    uint64_t body_off;    // codec payload after the frame header and state
    uint64_t body_len;
    uint64_t state_off, state_len;
    uint8_t state_version;
    uint32_t decoded;
    uint64_t plane_off;   // first plane byte of this chunk
    // filled by classify_chunk:
    bool raw;             // bytes stored verbatim at data_off
    uint64_t data_off, data_len;  // raw bytes, or the codec blob after TAG and length prefix
    uint8_t max_sym;      // rANS coded chunks: alphabet bound from the first blob byte (sizes the decoder's tables)
    uint16_t distinct;    // rANS coded chunks: symbols with a non-zero frequency (picks the decoder variant); 256 when unknown
};

struct PlaneDesc {
    uint16_t codec = 0;
    uint8_t role = 0;
    uint8_t state_source = 0;
    uint8_t post = 0, post_k = 0;  // op between the split and this terminal (detail::POST_*), bits stripped by MantissaZeroStrip
    uint64_t row_len = 0;
    bool has_crc = false;
    uint32_t crc = 0;
    bool chunked = false;
    uint64_t payload_off = 0, payload_len = 0;
    uint64_t decoded_len = 0;
    std::vector<ChunkDesc> chunks;  // one pseudo chunk when the plane is not chunked
};

struct TensorDesc {
    std::string name;
    uint16_t dtype_code = 0;
    std::string dtype_name;
    bool has_shape = false;
    std::vector<uint64_t> shape;
    uint64_t orig_size = 0;
    bool has_hash = false;
    uint64_t hash = 0;
    uint8_t kind = K_PASS;
    bool stored = false;      // \x89PTWS stored frame: raw bytes at stored_off
    uint64_t stored_off = 0;
    std::vector<PlaneDesc> planes;
    std::string unsupported;  // non-empty: outside the hot path (reason)
    uint64_t record_len = 0;  // compact layout: bytes of the tensor record (known from the index even when the record was not read)
};

struct SharedState { uint16_t id, codec; uint8_t version, mask; uint64_t hash; uint64_t off, len; bool checked = false; };

struct ParsedFile {
    std::vector<TensorDesc> tensors;
    std::vector<SharedState> shared;
    bool single_frame = false;
    bool legacy = false;      // read from the legacy \x89PTWM layout
};

namespace detail {

struct Node { uint16_t op; uint64_t params_off; uint32_t params_len; bool bound; };
// A plane may pass through one more op between the split and its terminal (python/ptwm/preprocessing/_chains.py:360-389,
// 486-560): IntDelta (transforms/int_delta.rs, byte width on split planes) or MantissaZeroStrip(k) (transforms/mantissa_zero.rs).
struct ChainShape { uint8_t kind; uint64_t source_len, plane_len, row_len; uint8_t post[4] = {0, 0, 0, 0}; uint8_t post_k[4] = {0, 0, 0, 0}; };

// transforms/op.rs:11-36
enum : uint16_t { OP_SOURCE = 0, OP_R16 = 0x10, OP_R32 = 0x11, OP_RE4M3 = 0x12, OP_RE5M2 = 0x13, OP_BYTESPLIT = 0x20, OP_NIBSPLIT = 0x21, OP_PASS = 0x30,
                  OP_INTDELTA = 0x52, OP_MZS = 0x64 };

struct RawChain {
    std::vector<Node> nodes;
    std::vector<std::pair<uint8_t, uint8_t>> terms;  // (node, output)
    struct Edge { uint8_t src, src_out, dst, dst_in; };
    std::vector<Edge> edges;  // spine edges written out like the others
};

// chain/wire_compact.rs:258-372.  resolve(op_ref) -> op wire id.
template <class F>
RawChain read_cw2(Span& r, F resolve) {
    RawChain c;
    size_t nn = size_t(r.var_max(255, "chain node count"));
    if (!nn) r.bad("chain has no nodes");
    size_t ne = size_t(r.var_max(255, "chain edge count"));
    size_t nt = size_t(r.var_max(255, "chain terminal count"));
    if (r.left() < 2 * nn + 2 * nt) r.bad("chain truncated");
    for (size_t i = 0; i < nn; ++i) {
        uint16_t op = resolve(r.var());
        uint32_t pl = uint32_t(r.var_max(255, "chain node params length"));
        Node n{op, 0, pl, op == OP_SOURCE && pl == 0};
        n.params_off = r.skip(pl);
        c.nodes.push_back(n);
    }
    if (ne) {
        size_t spine = size_t(r.var_max(ne, "chain spine edge count"));
        for (size_t i = 0; i < spine; ++i) c.edges.push_back({uint8_t(i), 0, uint8_t(i + 1), 0});
        for (size_t i = spine; i < ne; ++i) {
            uint8_t idx[4];
            for (auto& v : idx) v = uint8_t(r.var_max(255, "chain edge index"));
            uint8_t etag = r.byte();
            if (etag & ~3u) r.bad("chain edge tag has unknown bits");
            if (etag) r.bad("chain edge with a role override or vendor bytes", true);
            if (i == spine && idx[0] == i && idx[1] == 0 && idx[2] == i + 1 && idx[3] == 0) r.bad("chain spine edge stored explicitly (non-canonical)");
            c.edges.push_back({idx[0], idx[1], idx[2], idx[3]});
        }
    }
    for (size_t i = 0; i < nt; ++i) {
        uint8_t b = r.byte(), node, out;
        if (b == 0xFF) { node = r.byte(); out = r.byte(); if (node <= 14 && out <= 15) r.bad("chain terminal ref escaped needlessly (non-canonical)"); }
        else if ((b >> 4) == 15) r.bad("chain terminal ref byte is reserved");
        else { node = b >> 4; out = b & 15; }
        uint8_t role = r.byte();
        if (role == 0xFF) r.bad("escaped terminal role", true);
        if (role > 0x1C && role < 0x40 && role != 0x18 && role != 0x19 && role != 0x1A && role != 0x1B) r.bad("unknown compact role byte");
        c.terms.push_back({node, out});
    }
    return c;
}

// transforms/source.rs:18-63: bytes per element of a chain-internal dtype.
inline uint64_t chain_dtype_bytes(uint16_t cd) {
    switch (cd) {
        case 0x0002: case 0x000F: case 0x0007: case 0x0008: return 2;
        case 0x0003: case 0x0009: case 0x000A: return 4;
        case 0x0004: case 0x000B: case 0x000C: return 8;
        default: return 1;
    }
}
inline int chain_dtype_for_public(uint16_t code) {  // transforms/source.rs:69-85
    switch (code) {
        case 1: case 2: return 0x0003; case 4: case 5: return 0x0002; case 6: return 0x000F; case 13: return 0x0006; case 15: return 0x000A;
        case 17: return 0x0005; case 18: case 19: return 0x0007; case 20: case 21: return 0x0009; case 22: case 23: return 0x000B;
        case 29: return 0x0010; case 30: return 0x0011; case 31: return 0x001F; default: return -1;
    }
}
inline uint32_t public_dtype_bytes(uint16_t code) {  // dtype.rs element_size
    switch (code) {
        case 13: case 17: case 24: case 29: case 30: case 31: return 1;
        case 4: case 5: case 6: case 18: case 19: return 2;
        case 1: case 2: case 15: case 20: case 21: return 4;
        case 22: case 23: return 8;
        default: return 0;
    }
}
inline const char* canonical_dtype_name(uint16_t code) {  // dtype.rs canonical_name
    switch (code) {
        case 1: return "float32"; case 2: return "float"; case 4: return "float16"; case 5: return "half"; case 6: return "bfloat16"; case 13: return "uint8";
        case 15: return "uint32"; case 17: return "int8"; case 18: return "int16"; case 19: return "short"; case 20: return "int32"; case 21: return "int";
        case 22: return "int64"; case 23: return "long"; case 24: return "bool"; case 29: return "float8_e4m3fn"; case 30: return "float8_e5m2";
        case 31: return "float4_e2m1fn_x2"; default: return nullptr;
    }
}

// The Source descriptor (transforms/source.rs:120-178) and the terminal plane
// lengths of the production chains (chain/runtime.rs:359-439 restricted to
// python/ptwm/preprocessing/_chains.py:320-357,610-727).
inline ChainShape chain_shape(const RawChain& c, const uint8_t* base, const std::vector<uint64_t>* rec_shape, uint16_t rec_dtype) {
    const Node& s = c.nodes[0];
    if (s.op != OP_SOURCE) throw FormatError("chain: node[0] must be Source");
    uint64_t n = 1, last = 0; size_t ndim; uint16_t cd;
    if (s.bound) {
        int m = rec_shape ? chain_dtype_for_public(rec_dtype) : -1;
        if (m < 0 || rec_shape->size() > 255) throw FormatError("chain has a bound Source but the tensor has no bindable shape and dtype");
        ndim = rec_shape->size(); cd = uint16_t(m);
        for (uint64_t d : *rec_shape) {
            if (d > 0xFFFFFFFFull) throw FormatError("chain has a bound Source but a dimension exceeds u32");
            if (d && n > UINT64_MAX / d) throw FormatError("Source element count overflows");
            n *= d; last = d;
        }
    } else {
        const uint8_t* p = base + s.params_off;
        if (s.params_len < 3 || s.params_len != 3u + 4u * p[0]) throw FormatError("chain: malformed Source params");
        ndim = p[0];
        for (size_t d = 0; d < ndim; ++d) { uint64_t dim = le32(p + 1 + 4 * d); if (dim && n > UINT64_MAX / dim) throw FormatError("Source element count overflows"); n *= dim; last = dim; }
        cd = uint16_t(p[s.params_len - 2] | (p[s.params_len - 1] << 8));
    }
    ChainShape sh{K_PASS, n * chain_dtype_bytes(cd), 0, ndim ? last : 0};
    const size_t nn = c.nodes.size();
    if (c.edges.size() + 1 != nn) throw FormatError("chain is not a tree over its nodes", true);
    auto param1 = [&](const Node& nd, uint8_t v) { return nd.params_len == 1 && base[nd.params_off] == v; };
    const bool split16 = nn >= 3 && c.nodes[1].op == OP_R16 && c.nodes[2].op == OP_BYTESPLIT && param1(c.nodes[2], 2);
    const bool split32 = nn >= 3 && c.nodes[1].op == OP_R32 && c.nodes[2].op == OP_BYTESPLIT && param1(c.nodes[2], 4);
    // the leading nodes form a spine; after a byte split further nodes each hang off one output of the split
    const size_t spine = (split16 || split32) ? 2 : c.edges.size();
    for (size_t i = 0; i < spine; ++i) {
        const RawChain::Edge& e = c.edges[i];
        if (e.src != i || e.src_out != 0 || e.dst != i + 1 || e.dst_in != 0) throw FormatError("chain is not a linear spine", true);
    }
    auto terms = [&](size_t node, size_t cnt) {
        if (c.terms.size() != cnt) return false;
        for (size_t i = 0; i < cnt; ++i) if (c.terms[i].first != node || c.terms[i].second != i) return false;
        return true;
    };
    const char* outside = "chain outside the production split/passthrough set";
    if (split16 || split32) {
        const size_t np = split16 ? 2 : 4;
        if (sh.source_len % np) throw FormatError(split16 ? "16-bit split of an odd length" : "32-bit split of a length not divisible by 4");
        sh.kind = split16 ? K_M16 : K_M32; sh.plane_len = sh.source_len / np;
        int via[4] = {-1, -1, -1, -1};  // node between output p of the split and its terminal
        for (size_t i = 2; i < c.edges.size(); ++i) {
            const RawChain::Edge& e = c.edges[i];
            if (e.src != 2 || e.src_out >= np || e.dst < 3 || e.dst >= nn || e.dst_in != 0 || via[e.src_out] >= 0) throw FormatError(outside, true);
            for (size_t j = 2; j < i; ++j) if (c.edges[j].dst == e.dst) throw FormatError(outside, true);
            const Node& nd = c.nodes[e.dst];
            if (nd.op == OP_INTDELTA && nd.params_len == 0) sh.post[e.src_out] = POST_INTDELTA;
            else if (nd.op == OP_MZS && nd.params_len == 1 && base[nd.params_off] >= 1 && base[nd.params_off] <= 7) { sh.post[e.src_out] = POST_MZS; sh.post_k[e.src_out] = base[nd.params_off]; }
            else throw FormatError(outside, true);
            via[e.src_out] = e.dst;
        }
        if (c.terms.size() != np) throw FormatError(outside, true);
        for (size_t i = 0; i < np; ++i) {
            const bool direct = via[i] < 0 && c.terms[i].first == 2 && c.terms[i].second == i;
            const bool through = via[i] >= 0 && c.terms[i].first == via[i] && c.terms[i].second == 0;
            if (!direct && !through) throw FormatError(outside, true);
        }
    }
    else if ((nn == 1 && terms(0, 1)) || (nn == 2 && c.nodes[1].op == OP_PASS && terms(1, 1))) { sh.kind = K_PASS; sh.plane_len = sh.source_len; }
    else if (nn == 3 && c.nodes[1].op == OP_RE4M3 && c.nodes[2].op == OP_NIBSPLIT && terms(2, 2)) { sh.kind = K_E4M3; sh.plane_len = sh.source_len; }
    else if (nn == 3 && c.nodes[1].op == OP_RE5M2 && c.nodes[2].op == OP_NIBSPLIT && terms(2, 2)) { sh.kind = K_E5M2; sh.plane_len = sh.source_len; }
    else throw FormatError(outside, true);
    return sh;
}

struct TableEntry { uint8_t tag; uint16_t id; };

inline std::vector<TableEntry> read_table(const uint8_t* base, size_t begin, size_t end) {  // extension/compact_table.rs:176-261
    Span r(base, begin, end, "compact extension table");
    uint64_t count = r.var_max(1u << 16, "entry count");
    if (count > (end - begin) / 2) r.bad("entry count exceeds the table bytes");
    std::vector<TableEntry> out;
    std::unordered_set<uint32_t> seen;
    for (uint64_t i = 0; i < count; ++i) {
        uint8_t tag = r.byte();
        TableEntry e{tag, 0};
        if (tag == 1 || tag == 2) {
            e.id = uint16_t(r.var_max(0xFFFF, "wire id"));
            if (!seen.insert(uint32_t(tag) << 16 | e.id).second) r.bad("duplicate entry");
        } else if (tag == 3) { uint64_t l = r.var_max(255, "built-in name length"); if (!l) r.bad("empty built-in name"); r.skip(size_t(l)); }
        else if (tag == 0x7F) r.skip(r.var_len());  // third-party entry: kept as a non-codec, non-op slot
        else r.bad("unknown entry tag");
        out.push_back(e);
    }
    r.done("the last entry");
    return out;
}

// Frame header, tag byte and length prefix of one chunk (compressor.rs:316-321;
// codecs/{huffman,rans,tans}.rs decode; codecs/length_prefix.rs:29-33).
inline void classify_chunk(const uint8_t* base, uint16_t codec, ChunkDesc& ch) {
    ch.raw = false; ch.data_off = ch.body_off; ch.data_len = ch.body_len; ch.max_sym = 255; ch.distinct = 256;
    if (codec == C_IDENTITY) {
        ch.raw = true;
        if (ch.body_len != ch.decoded) throw FormatError("identity plane length differs from its decoded length");
        return;
    }
    if (codec == C_O1SAC) return;
    if (codec != C_HUFFMAN && codec != C_RANS && codec != C_TANS) throw FormatError("plane codec outside the hot path (wire id " + std::to_string(codec) + ")", true);
    if (ch.body_len == 0) throw FormatError("empty payload");
    uint8_t tag = base[ch.body_off];
    if (tag == 0) {
        ch.raw = true; ch.data_off = ch.body_off + 1; ch.data_len = ch.body_len - 1;
        if (ch.data_len != ch.decoded) throw FormatError("raw-tagged plane length differs from its decoded length");
        return;
    }
    if (tag != 1) throw FormatError("bad codec tag");
    if (ch.body_len < 5) throw FormatError("payload too short for length prefix");
    uint64_t orig = le32(base + ch.body_off + 1), enc = ch.body_len - 5;
    bool ok = codec == C_HUFFMAN ? orig <= enc * 32 + 4096 : (orig <= (1ull << 30) || orig <= enc * 64);
    if (!ok) throw FormatError("implausible orig_len for the encoded bytes");
    if (orig != ch.decoded) throw FormatError("decoded length differs from the length the chunk declares");
    ch.data_off = ch.body_off + 5; ch.data_len = enc;
    ch.max_sym = (codec == C_RANS && enc) ? base[ch.data_off] : 255;
    if (codec == C_RANS && enc >= 1 + 2 * (uint64_t(ch.max_sym) + 1)) {
        // frequency table: u16 per symbol after the alphabet bound (rans/decompress.rs:36-47)
        const uint8_t* f = base + ch.data_off + 1;
        uint32_t d = 0;
        for (uint32_t k = 0; k <= ch.max_sym; ++k) d += (f[2 * k] | f[2 * k + 1]) != 0;
        ch.distinct = uint16_t(d);
    }
}

}  // namespace detail

// Order1ScaleAC pre-checks that need the state bytes (order1_scale_ac.rs:174-220,449-471).
inline void check_o1sac(const uint8_t* state, uint64_t state_len, uint8_t version, uint64_t payload_len, uint64_t decoded, uint64_t row_len);

class FileReader {
  public:
    FileReader(const uint8_t* buf, size_t len) : b_(buf), n_(len) {}
    // Only the records of shard `rank` of `world` are read (compact layout; the other layouts are read whole).
    void set_shard(uint32_t rank, uint32_t world) { shard_rank_ = rank; shard_world_ = world; }
    ParsedFile parse() {
        static const uint8_t PTWC[9] = {0x89, 'P', 'T', 'W', 'C', '\r', '\n', 0x1a, '\n'};
        static const uint8_t PTWS[5] = {0x89, 'P', 'T', 'W', 'S'};
        if (n_ >= 5 && !std::memcmp(b_, PTWS, 5)) return parse_frame();
        if (n_ >= 9 && !std::memcmp(b_, PTWC, 9)) return parse_container();
        static const uint8_t PTWM[9] = {0x89, 'P', 'T', 'W', 'M', '\r', '\n', 0x1a, '\n'};
        static const uint8_t PTWX[9] = {0x89, 'P', 'T', 'W', 'X', '\r', '\n', 0x1a, '\n'};
        if (n_ >= 9 && (!std::memcmp(b_, PTWM, 9) || !std::memcmp(b_, PTWX, 9))) return parse_legacy();
        throw FormatError("not a .ptwm container or frame");
    }

  private:
    const uint8_t* b_;
    size_t n_;
    std::vector<detail::TableEntry> table_;
    std::vector<detail::RawChain> registry_;
    ParsedFile out_;
    std::mutex shared_mu_;
    uint32_t shard_rank_ = 0, shard_world_ = 0;

    void make_chunks(PlaneDesc& p, bool chunked, const std::vector<std::pair<uint32_t, uint32_t>>& entries, uint64_t inline_off, uint64_t inline_len,
                     uint8_t state_version, uint16_t state_info) {
        if (chunked) {
            uint64_t total = 0;
            for (size_t i = 0; i < entries.size(); ++i) {
                uint64_t start = entries[i].first, end = i + 1 < entries.size() ? entries[i + 1].first : p.payload_len;
                if (start > end || end > p.payload_len) throw FormatError("chunk table offset out of bounds");
                if (end - start < 5) throw FormatError("chunk frame truncated");
                const uint8_t* f = b_ + p.payload_off + start;
                uint64_t sl = le32(f + 1);
                if (end - start - 5 < sl) throw FormatError("chunk frame state_len exceeds frame");
                ChunkDesc ch{};
                ch.frame_off = p.payload_off + start; ch.state_version = f[0]; ch.state_off = ch.frame_off + 5; ch.state_len = sl;
                ch.body_off = ch.state_off + sl; ch.body_len = end - start - 5 - sl; ch.decoded = entries[i].second; ch.plane_off = total;
                total += ch.decoded;
                detail::classify_chunk(b_, p.codec, ch);
                p.chunks.push_back(ch);
            }
            if (total != p.decoded_len) throw FormatError("chunk table does not decode to the plane's length");  // container.rs:1982-1994
        } else {
            ChunkDesc ch{};
            ch.frame_off = p.payload_off; ch.body_off = p.payload_off; ch.body_len = p.payload_len; ch.decoded = uint32_t(p.decoded_len); ch.plane_off = 0;
            if (p.decoded_len > 0xFFFFFFFFull) throw FormatError("unchunked plane longer than u32", true);
            if (p.state_source == 1) { ch.state_off = inline_off; ch.state_len = inline_len; ch.state_version = state_version; }
            else if (p.state_source == 2) {  // container.rs:2058-2102
                SharedState* e = nullptr;
                for (auto& s : out_.shared) if (s.id == state_info) { e = &s; break; }
                if (!e) throw FormatError("shared state not in prelude");
                if (state_version != e->version) throw FormatError("plane state_version does not match the prelude entry");
                if (p.role >= 1 && p.role <= 8 && !(e->mask & (1u << (p.role - 1)))) throw FormatError("shared state applies_to_mask does not cover the plane role");
                {
                    std::lock_guard<std::mutex> g(shared_mu_);  // records are read by several threads
                    if (!e->checked) { if (xxh64_host(b_ + e->off, e->len) != e->hash) throw FormatError("shared state xxhash64 mismatch"); e->checked = true; }
                }
                ch.state_off = e->off; ch.state_len = e->len; ch.state_version = e->version;
            } else if (p.state_source == 3) throw FormatError("External state not supported");
            detail::classify_chunk(b_, p.codec, ch);
            p.chunks.push_back(ch);
        }
        if (p.codec == C_O1SAC)
            for (auto& ch : p.chunks) check_o1sac(b_ + ch.state_off, ch.state_len, ch.state_version, ch.body_len, ch.decoded, p.row_len);
    }

    // tensor_record_compact.rs:659-811
    PlaneDesc read_plane(Span& r, uint64_t plane_len) {
        PlaneDesc p;
        uint8_t pf = r.byte();
        if (pf & ~0x3Fu) r.bad("unknown pflags bits");
        p.state_source = (pf >> 2) & 3;
        p.role = r.byte();
        if (!((p.role >= 1 && p.role <= 6) || (p.role >= 0x10 && p.role <= 0x13))) r.bad("unknown plane role");
        uint64_t ref = r.var_max(0xFFFF, "codec_ref");
        if (ref >= table_.size()) r.bad("codec_ref is outside the Extension Table");
        if (table_[size_t(ref)].tag == 1 || table_[size_t(ref)].tag == 3) r.bad("codec_ref names an entry that is not a plane codec");
        bool third_party = table_[size_t(ref)].tag == 0x7F;
        p.codec = table_[size_t(ref)].id;
        uint8_t sv = 0; uint16_t info = 0;
        if (pf & 0x20) { sv = r.byte(); info = uint16_t(r.var_max(0xFFFF, "state_info")); if (!sv && !info) r.bad("PF_STATE_EXTRA with zero state_version and state_info"); }
        size_t inline_len = p.state_source == 1 ? r.var_len() : 0;
        p.payload_len = r.var_len();
        if (pf & 0x10) { p.row_len = r.var_max(0xFFFFFFFFull, "row_len"); if (!p.row_len) r.bad("row_len 0"); }
        if (pf & 0x01) { p.has_crc = true; p.crc = r.u32(); }
        std::vector<std::pair<uint32_t, uint32_t>> entries;
        if (pf & 0x02) {
            p.chunked = true;
            uint64_t cnt = r.var_max(p.payload_len, "chunk count");
            if (cnt > r.left() / 2) r.bad("chunk count exceeds the record");
            entries.reserve(size_t(cnt));
            for (uint64_t i = 0; i < cnt; ++i) {
                uint32_t off = uint32_t(r.var_max(0xFFFFFFFFull, "chunk offset"));
                uint32_t sz = uint32_t(r.var_max(0xFFFFFFFFull, "chunk decoded size"));
                entries.push_back({off, sz});
            }
        }
        if (p.state_source == 3) {
            r.byte(); uint8_t fl = r.byte();
            if (fl & ~1u) r.bad("unknown external state flag bits");
            r.skip(size_t(r.var_max(0xFFFF, "external state ref length"))); r.byte();
            if (fl & 1) r.skip(32);
        }
        uint64_t inline_off = r.skip(inline_len);
        p.payload_off = r.skip(size_t(p.payload_len));
        p.decoded_len = plane_len;
        if (third_party) throw FormatError("third-party plane codec", true);
        make_chunks(p, p.chunked, entries, inline_off, inline_len, sv, info);
        return p;
    }

    TensorDesc read_record(size_t begin, size_t end) {
        Span r(b_, begin, end, "compact tensor record");
        TensorDesc t;
        uint8_t tf = r.byte();
        if (tf & ~0x3Fu) r.bad("unknown tflags bits");
        if ((tf & 0x10) && !(tf & 0x08)) r.bad("TF_DTYPE_NAME without TF_SHAPE");
        if ((tf & 0x20) && (tf & 0x08)) r.bad("TF_RAW_META with TF_SHAPE");
        bool inline_chain = tf & 0x02;
        uint64_t chain_id = 0;
        if (!inline_chain) { chain_id = r.var(); if (chain_id >= registry_.size()) r.bad("chain id is not in the registry"); }
        t.dtype_code = uint16_t(r.var_max(0xFFFF, "dtype_code"));
        r.byte();  // input_format
        t.orig_size = r.var();
        if (tf & 0x08) {
            size_t nd = size_t(r.var_max(64, "ndim"));
            if (nd > r.left()) r.bad("truncated shape");
            for (size_t i = 0; i < nd; ++i) t.shape.push_back(r.var());
            t.has_shape = true;
            const char* canon = detail::canonical_dtype_name(t.dtype_code);
            if (tf & 0x10) {
                size_t l = r.var_len();
                t.dtype_name.assign(reinterpret_cast<const char*>(b_ + r.skip(l)), l);
                if (canon && t.dtype_name == canon) r.bad("stored dtype name equals the canonical name (non-canonical)");
            } else { if (!canon) r.bad("shape without a dtype name for a dtype_code that has no canonical name"); t.dtype_name = canon; }
        } else if (tf & 0x20) r.skip(r.var_len());
        if (tf & 0x01) { t.has_hash = true; t.hash = r.u64(); }
        detail::RawChain local;
        const detail::RawChain* chain;
        if (inline_chain) {
            size_t etl = r.var_len(); size_t et = r.skip(etl);
            auto ops = detail::read_table(b_, et, et + etl);
            size_t cl = r.var_len(); size_t cb = r.skip(cl);
            Span cr(b_, cb, cb + cl, "compact chain");
            local = detail::read_cw2(cr, [&](uint64_t ref) -> uint16_t { if (ref >= ops.size() || ops[size_t(ref)].tag != 1) cr.bad("inline chain op_ref outside its table"); return ops[size_t(ref)].id; });
            cr.done("chain");
            chain = &local;
        } else chain = &registry_[size_t(chain_id)];
        if (tf & 0x04) r.bad("tensor dependencies (delta against another tensor)", true);
        detail::ChainShape sh = detail::chain_shape(*chain, b_, t.has_shape ? &t.shape : nullptr, t.dtype_code);
        if (sh.source_len != t.orig_size) r.bad("chain Source declares a different size than orig_size");  // container.rs:1856-1861
        t.kind = sh.kind;
        uint64_t np = r.var_max(255, "plane count");
        if (np > r.left() / 4) r.bad("plane count exceeds the record");
        if (np != uint64_t(kind_planes(sh.kind))) r.bad("plane count differs from the chain's terminals");
        for (uint64_t i = 0; i < np; ++i) { t.planes.push_back(read_plane(r, sh.plane_len)); t.planes.back().post = sh.post[i]; t.planes.back().post_k = sh.post_k[i]; }
        r.done("the last plane");
        return t;
    }

    ParsedFile parse_container() {  // ptwc.rs:105-297
        static const uint8_t EOFS[8] = {0x89, 'T', 'W', 'M', 'E', 'O', 'F', 0x1a};
        if (n_ < 9 + 2 + 16) throw FormatError("compact container: file too short");
        if (std::memcmp(b_ + n_ - 8, EOFS, 8)) throw FormatError("compact container: missing EOF sentinel");
        size_t footer = n_ - 16;
        Span h(b_, 9, footer, "compact container header");
        uint16_t hflags = uint16_t(h.byte()); hflags |= uint16_t(h.byte()) << 8;
        if (hflags) h.bad("unknown hflags bits");
        uint64_t l_et = h.var(), l_pre = h.var(), l_reg = h.var();
        size_t hash_pos = h.pos();
        uint64_t stored = h.u64();
        size_t p0 = h.pos();
        auto sect = [&](size_t start, uint64_t l, const char* w) { if (l > footer - start) throw FormatError(std::string("compact container: ") + w + " section exceeds the file"); return start + size_t(l); };
        size_t p1 = sect(p0, l_et, "extension table"), p2 = sect(p1, l_pre, "prelude"), p3 = sect(p2, l_reg, "registry");
        uint64_t index_len = le64(b_ + footer);
        if (index_len > footer) throw FormatError("compact container: index_len exceeds the file");
        size_t index_start = footer - size_t(index_len);
        if (p3 > index_start) throw FormatError("compact container: index overlaps the registry");
        {
            std::vector<uint8_t> meta(b_, b_ + hash_pos);
            meta.insert(meta.end(), b_ + p0, b_ + p3);
            if (xxh64_host(meta.data(), meta.size()) != stored) throw FormatError("compact container: meta_xxh64 mismatch");
        }
        table_ = detail::read_table(b_, p0, p1);
        parse_prelude(p1, p2);
        {
            Span r(b_, p2, p3, "compact chain registry");
            size_t count = size_t(r.var_max(0x8000, "chain count"));
            if (count > (p3 - p2) / 6) r.bad("chain count exceeds the registry bytes");
            for (size_t i = 0; i < count; ++i) {
                size_t cl = r.var_len(); size_t cb = r.skip(cl);
                Span cr(b_, cb, cb + cl, "compact chain");
                registry_.push_back(detail::read_cw2(cr, [&](uint64_t ref) -> uint16_t { if (ref >= table_.size() || table_[size_t(ref)].tag != 1) cr.bad("op_ref is not a built-in transform"); return table_[size_t(ref)].id; }));
                cr.done("chain");
            }
            r.done("the last chain");
        }
        Span ir(b_, index_start, footer, "compact container index");
        uint64_t count = ir.var();
        if (count > (footer - index_start) / 3) ir.bad("entry count exceeds the index bytes");
        size_t off = p3;
        std::unordered_set<std::string> names;
        struct Rec { std::string name; size_t off, len; };
        std::vector<Rec> recs;
        for (uint64_t i = 0; i < count; ++i) {
            size_t nl = size_t(ir.var_max(65535, "name length"));
            if (!nl) ir.bad("empty tensor name");
            std::string name(reinterpret_cast<const char*>(b_ + ir.skip(nl)), nl);
            if (!names.insert(name).second) ir.bad("duplicate tensor name");
            uint64_t rl = ir.var();
            if (rl < 3) ir.bad("record too short");
            if (rl > index_start - off) ir.bad("record runs past the body");
            recs.push_back(Rec{std::move(name), off, size_t(rl)});
            off += size_t(rl);
        }
        // Reading a record touches every chunk header of its planes, scattered over the whole file: for a large
        // container that is a hundred thousand cache misses, so the records are read by several threads.  The
        // first failing record (in index order) is the one reported, as if they had been read in turn.
        out_.tensors.resize(recs.size());
        std::vector<std::string> failed(recs.size());
        std::vector<uint8_t> has_failed(recs.size(), 0);
        // A rank of a multi-GPU load reads only the records of its own shard: a contiguous run chosen by record
        // bytes, the same cut on every rank (rank r ends at the first record where the running size reaches
        // (r + 1) / world of the total, a record counting where its middle falls).
        size_t shard_lo = 0, shard_hi = recs.size();
        if (shard_world_ > 1) {
            double total = 0;
            for (auto& r : recs) total += double(r.len);
            std::vector<size_t> bounds{0};
            double run = 0;
            size_t i = 0;
            for (uint32_t r = 1; r < shard_world_; ++r) {
                const double target = total * r / shard_world_;
                while (i < recs.size() && run + double(recs[i].len) / 2 <= target) { run += double(recs[i].len); ++i; }
                bounds.push_back(i);
            }
            bounds.push_back(recs.size());
            shard_lo = bounds[shard_rank_]; shard_hi = bounds[shard_rank_ + 1];
        }
        auto read_one = [&](size_t i) {
            TensorDesc t;
            if (i < shard_lo || i >= shard_hi) {
                t.unsupported = "record not read: it belongs to another rank's shard";
                t.name = recs[i].name; t.record_len = recs[i].len;
                out_.tensors[i] = std::move(t);
                return;
            }
            try { t = read_record(recs[i].off, recs[i].off + recs[i].len); }
            catch (const FormatError& e) {
                if (!e.unsupported) { failed[i] = e.what(); has_failed[i] = 1; return; }
                t = TensorDesc{}; t.unsupported = e.what();
            }
            // anything else (an allocation a hostile length asked for) must not leave a worker thread: record it like a parse failure
            catch (const std::exception& e) { failed[i] = std::string("record could not be read: ") + e.what(); has_failed[i] = 1; return; }
            catch (...) { failed[i] = "record could not be read"; has_failed[i] = 1; return; }
            t.name = recs[i].name; t.record_len = recs[i].len;
            out_.tensors[i] = std::move(t);
        };
        size_t workers = std::thread::hardware_concurrency();
        workers = std::min<size_t>(std::min<size_t>(workers ? workers : 1, 16), recs.size() / 4);
        if (n_ < (size_t(64) << 20) || workers < 2) {
            for (size_t i = 0; i < recs.size(); ++i) { read_one(i); if (has_failed[i]) break; }
        } else {
            std::atomic<size_t> next{0};
            std::vector<std::thread> pool;
            for (size_t w = 0; w < workers; ++w)
                pool.emplace_back([&] { for (size_t i = next.fetch_add(1); i < recs.size(); i = next.fetch_add(1)) read_one(i); });
            for (auto& th : pool) th.join();
        }
        for (size_t i = 0; i < recs.size(); ++i) if (has_failed[i]) throw FormatError(failed[i]);
        ir.done("the last index entry");
        if (off != index_start) throw FormatError("compact container: records do not cover the body");
        return std::move(out_);
    }

    size_t parse_prelude(size_t begin, size_t end) {  // prelude.rs:66-160; returns where the entries end
        if (end - begin < 4) throw FormatError("prelude too short");
        size_t count = le32(b_ + begin);
        if (count > (end - begin - 4) / 22) throw FormatError("prelude count exceeds buffer capacity");
        size_t pos = begin + 4;
        for (size_t i = 0; i < count; ++i) {
            if (pos + 18 > end) throw FormatError("prelude entry truncated");
            SharedState s{};
            s.id = uint16_t(b_[pos] | (b_[pos + 1] << 8)); s.codec = uint16_t(b_[pos + 2] | (b_[pos + 3] << 8)); s.version = b_[pos + 4]; s.mask = b_[pos + 5];
            s.hash = le64(b_ + pos + 8);
            size_t nl = size_t(b_[pos + 16]) | size_t(b_[pos + 17]) << 8;
            pos += 18;
            size_t pad = (4 - nl % 4) % 4;
            if (pos + nl + pad + 4 > end) throw FormatError("prelude entry name truncated");
            pos += nl + pad;
            s.len = le32(b_ + pos); pos += 4;
            if (pos + s.len > end) throw FormatError("prelude entry state_bytes truncated");
            s.off = pos; pos += size_t(s.len);
            out_.shared.push_back(s);
        }
        return pos;
    }

    // ---- legacy container (\x89PTWM / \x89PTWX) --------------------------------------------------
    // header.rs:112-200, extension/table.rs:95-110, prelude.rs:66-160, chain/wire.rs:146-300,
    // tensor_record.rs:276-440, plane_record.rs:118-260, index.rs:29-70 of the reference.  Built-in entries are
    // recognised by their label (io.ptwm.builtin.<name>@<version>): the blake3 hash of the Extension Table and the
    // re-derivation of built-in ids are not checked here.
    struct LegacyEntry { uint8_t tag; uint16_t id; };  // tag 1 op, 2 codec, 0x7F anything else
    // One Extension Table starting at `pos`; returns the position after it.
    size_t read_legacy_table(size_t pos, size_t end, std::vector<LegacyEntry>& out) {
        Span r(b_, pos, end, "legacy extension table");
        uint32_t count = r.u32();
        if (count > 65536) r.bad("entry count too large");
        static const struct { const char* name; uint8_t tag; uint16_t id; } known[] = {
            {"identity", 2, C_IDENTITY}, {"huffman", 2, C_HUFFMAN}, {"rans", 2, C_RANS}, {"zstd", 2, C_ZSTD}, {"tans", 2, C_TANS}, {"order1_scale_ac", 2, C_O1SAC},
            {"source", 1, detail::OP_SOURCE}, {"bit_reorder_ieee16", 1, detail::OP_R16}, {"bit_reorder_ieee32", 1, detail::OP_R32},
            {"bit_reorder_fp8_e4m3", 1, detail::OP_RE4M3}, {"bit_reorder_fp8_e5m2", 1, detail::OP_RE5M2}, {"byte_split", 1, detail::OP_BYTESPLIT},
            {"nibble_split", 1, detail::OP_NIBSPLIT}, {"byte_passthrough", 1, detail::OP_PASS}, {"int_delta", 1, detail::OP_INTDELTA},
            {"mantissa_zero_strip", 1, detail::OP_MZS}};
        for (uint32_t i = 0; i < count; ++i) {
            const uint8_t* canonical = b_ + r.skip(32);             // canonical id
            size_t ll = size_t(r.byte()); ll |= size_t(r.byte()) << 8;
            std::string label(reinterpret_cast<const char*>(b_ + r.skip(ll)), ll);
            uint16_t kind = uint16_t(r.byte()); kind |= uint16_t(r.byte()) << 8;
            r.skip(2 + 1 + 1);                                       // abi_version, lifecycle, flavor_hints
            uint32_t cap = r.u32();
            if (cap > (1u << 20)) r.bad("capabilities too long");
            r.skip(cap);
            r.byte();                                                // attestation kind
            size_t al = size_t(r.byte()); al |= size_t(r.byte()) << 8;
            r.skip(al);
            size_t hl = size_t(r.byte()); hl |= size_t(r.byte()) << 8;
            r.skip(hl);
            r.skip(16);                                              // embedded wasm offset and length
            LegacyEntry e{0x7F, 0xFFFF};
            static const std::string prefix = "io.ptwm.builtin.";
            size_t at = label.find('@', std::min(prefix.size(), label.size()));
            if (label.compare(0, prefix.size(), prefix) == 0 && at != std::string::npos && at > prefix.size()) {
                // A built-in of any release is io.ptwm.builtin.<name>@<version> whose id is
                // blake3(author key || 0 || name || 0 || version) under the built-in author key
                // (extension/builtins.rs:283-333, extension/id.rs:21-31); anything else with such a label is
                // somebody else's entry, i.e. an extension that is not installed.
                const std::string name = label.substr(prefix.size(), at - prefix.size()), version = label.substr(at + 1);
                bool genuine = !version.empty() && version.size() <= 64 && version.find('@') == std::string::npos;
                if (genuine) {
                    std::vector<uint8_t> msg(32, 0xBB);
                    msg.push_back(0); msg.insert(msg.end(), name.begin(), name.end());
                    msg.push_back(0); msg.insert(msg.end(), version.begin(), version.end());
                    uint8_t id[32];
                    blake3_hash(msg.data(), msg.size(), id);
                    genuine = std::memcmp(id, canonical, 32) == 0;
                }
                if (genuine) {
                    // kind: 1 Transform, 2 PlaneCodec in the reference's numbering is not relied on; the name decides
                    bool hit = false;
                    for (auto& k : known) if (name == k.name) { e = LegacyEntry{k.tag, k.id}; hit = true; }
                    if (!hit) e = LegacyEntry{uint8_t(0x7E), 0xFFFF};  // a built-in outside the hot path
                }
            }
            (void)kind;
            out.push_back(e);
        }
        return r.pos();
    }
    static size_t legacy_role_len(Span& r) {  // types/role.rs:250-345
        uint8_t t = r.byte();
        switch (t) {
            case 0x00: case 0x04: case 0x07: r.byte(); return 2;
            case 0x01: { uint8_t f = r.byte(); if (f == 1) r.byte(); else if (f != 0) r.bad("unknown value format"); return 0; }
            case 0x02: case 0x05: r.skip(2); return 3;
            case 0x03: case 0x08: case 0x09: return 1;
            case 0x06: { uint8_t f = r.byte(); if (f == 1) r.skip(2); else if (f != 0) r.bad("unknown residual format"); return 0; }
            case 0xFF: { r.skip(2); size_t l = size_t(r.byte()); l |= size_t(r.byte()) << 8; r.skip(l); return 0; }
            default: r.bad("unknown role tag");
        }
    }
    // One chain in the legacy wire starting at `pos`; returns the position after it.
    size_t read_legacy_chain(size_t pos, size_t end, const std::vector<LegacyEntry>& table, detail::RawChain& c) {
        Span h(b_, pos, end, "legacy chain");
        size_t nn = h.byte(), ne = h.byte(), nt = h.byte();
        size_t nl = size_t(h.byte()); nl |= size_t(h.byte()) << 8;
        size_t el = size_t(h.byte()); el |= size_t(h.byte()) << 8;
        size_t tl = size_t(h.byte()); tl |= size_t(h.byte()) << 8;
        size_t n0 = h.skip(nl), e0 = h.skip(el), t0 = h.skip(tl);
        if (!nn) h.bad("chain has no nodes");
        Span nr(b_, n0, n0 + nl, "legacy chain nodes");
        for (size_t i = 0; i < nn; ++i) {
            size_t idx = size_t(nr.byte()); idx |= size_t(nr.byte()) << 8;
            if (idx >= table.size()) nr.bad("node op is outside the Extension Table");
            if (table[idx].tag == 0x7E || table[idx].tag == 0x7F) throw FormatError("chain uses a transform outside the production split/passthrough set", true);
            if (table[idx].tag != 1) nr.bad("node op names an entry that is not a transform");
            uint32_t pl = nr.byte();
            detail::Node n{table[idx].id, 0, pl, table[idx].id == detail::OP_SOURCE && pl == 0};
            n.params_off = nr.skip(pl);
            c.nodes.push_back(n);
        }
        Span er(b_, e0, e0 + el, "legacy chain edges");
        for (size_t i = 0; i < ne; ++i) {
            uint8_t src = er.byte(), so = er.byte(), dst = er.byte(), di = er.byte(), has_role = er.byte();
            if (has_role > 1) er.bad("edge role_present byte has an unknown value");
            if (has_role) legacy_role_len(er);
            size_t vl = size_t(er.byte()); vl |= size_t(er.byte()) << 8;
            er.skip(vl);
            if (vl) throw FormatError("chain edge with vendor bytes", true);  // a role override only relabels the plane: nothing to do at decode
            c.edges.push_back({src, so, dst, di});
        }
        Span tr(b_, t0, t0 + tl, "legacy chain terminals");
        for (size_t i = 0; i < nt; ++i) {
            uint8_t node = tr.byte(), out = tr.byte();
            legacy_role_len(tr);
            c.terms.push_back({node, out});
        }
        return h.pos();
    }
    // {"shape": [...], "dtype": "..."} (metadata.rs:54-190)
    void read_shape_metadata(size_t begin, size_t end, TensorDesc& t) {
        Span r(b_, begin, end, "shape metadata");
        auto head = [&](uint8_t major) -> uint64_t {
            uint8_t f = r.byte();
            if ((f & 0xE0) != major) r.bad("unexpected CBOR major type");
            uint8_t a = f & 0x1F;
            if (a < 24) return a;
            size_t n = a == 24 ? 1 : a == 25 ? 2 : a == 26 ? 4 : a == 27 ? 8 : 0;
            if (!n) r.bad("unsupported CBOR argument");
            uint64_t v = 0;
            for (size_t i = 0; i < n; ++i) v = (v << 8) | r.byte();
            return v;
        };
        auto text = [&]() { uint64_t l = head(0x60); if (l > r.left()) r.bad("text string truncated"); return std::string(reinterpret_cast<const char*>(b_ + r.skip(size_t(l))), size_t(l)); };
        if (head(0xA0) != 2) r.bad("expected a map of two pairs");
        bool got_shape = false, got_dtype = false;
        for (int k = 0; k < 2; ++k) {
            std::string key = text();
            if (key == "shape") {
                uint64_t n = head(0x80);
                if (n > r.left()) r.bad("shape array truncated");
                for (uint64_t i = 0; i < n; ++i) t.shape.push_back(head(0x00));
                got_shape = true;
            } else if (key == "dtype") { t.dtype_name = text(); got_dtype = true; }
            else r.bad("unknown key");
        }
        if (!got_shape || !got_dtype) r.bad("missing shape or dtype");
        t.has_shape = true;
    }
    PlaneDesc read_legacy_plane(Span& r, uint64_t plane_len, const std::vector<LegacyEntry>& table) {
        PlaneDesc p;
        p.role = r.byte();
        uint8_t pf = r.byte();
        r.skip(2);  // codec_id: duplicates the table entry, the reader dispatches on codec_table_idx (plane_record.rs:140-148)
        size_t idx = size_t(r.byte()); idx |= size_t(r.byte()) << 8;
        if (idx >= table.size()) r.bad("codec_table_idx is outside the Extension Table");
        if (table[idx].tag == 1) r.bad("codec_table_idx names a transform");
        bool outside = table[idx].tag != 2;
        p.codec = table[idx].id;
        p.state_source = r.byte();
        if (p.state_source > 3) r.bad("unknown state_source");
        uint8_t sv = r.byte();
        uint16_t info = uint16_t(r.byte()); info |= uint16_t(r.byte()) << 8;
        size_t inline_len = r.u32();
        p.payload_len = r.u64();
        if (pf & 0x02) { p.has_crc = true; p.crc = r.u32(); }
        std::vector<std::pair<uint32_t, uint32_t>> entries;
        if (pf & 0x01) {
            p.chunked = true;
            uint32_t cnt = r.u32();
            if (cnt > r.left() / 8) r.bad("chunk_count exceeds remaining bytes");
            for (uint32_t i = 0; i < cnt; ++i) { uint32_t off = r.u32(), sz = r.u32(); entries.push_back({off, sz}); }
        }
        if (p.state_source == 3) {
            r.byte(); uint8_t fl = r.byte();
            size_t rl = size_t(r.byte()); rl |= size_t(r.byte()) << 8;
            r.skip(rl); r.byte();
            if (fl & 1) r.skip(32);
        }
        uint8_t layout = r.byte();
        if (layout == 1) { p.row_len = r.u32(); if (!p.row_len) r.bad("row_len 0"); }
        else if (layout != 0) r.bad("unknown plane layout");
        if (p.state_source != 1 && inline_len) r.bad("inline state bytes without an inline state source");
        uint64_t inline_off = r.skip(inline_len);
        if (p.payload_len > r.left()) r.bad("plane payload exceeds the record");
        p.payload_off = r.skip(size_t(p.payload_len));
        p.decoded_len = plane_len;
        if (outside) throw FormatError("plane codec outside the hot path", true);
        make_chunks(p, p.chunked, entries, inline_off, inline_len, sv, info);
        return p;
    }
    TensorDesc read_legacy_record(size_t begin, size_t end, const std::vector<LegacyEntry>& table, const std::vector<std::pair<uint16_t, detail::RawChain>>& registry) {
        Span r(b_, begin, end, "legacy tensor record");
        TensorDesc t;
        uint16_t chain_ref = uint16_t(r.byte()); chain_ref |= uint16_t(r.byte()) << 8;
        t.dtype_code = uint16_t(r.byte()); t.dtype_code |= uint16_t(r.byte()) << 8;
        r.byte();  // input_format
        size_t np = r.byte();
        uint8_t flags = r.byte();
        r.byte();  // reserved
        t.orig_size = r.u64();
        size_t nl = size_t(r.byte()); nl |= size_t(r.byte()) << 8;
        t.name.assign(reinterpret_cast<const char*>(b_ + r.skip(nl)), nl);
        r.skip((4 - nl % 4) % 4);
        if (flags & 0x04) { t.has_hash = true; t.hash = r.u64(); }
        detail::RawChain local;
        const detail::RawChain* chain = nullptr;
        std::vector<LegacyEntry> inline_table;
        const std::vector<LegacyEntry>* plane_table = &table;
        std::string chain_problem;
        try {
            if (chain_ref & 0x8000) {
                size_t after = read_legacy_table(r.pos(), end, inline_table);
                r.skip(after - r.pos());
                after = read_legacy_chain(r.pos(), end, inline_table, local);
                r.skip(after - r.pos());
                chain = &local;
            } else {
                for (auto& e : registry) if (e.first == chain_ref) chain = &e.second;
                if (!chain) r.bad("chain id is not in the registry");
            }
        } catch (const FormatError& e) { if (!e.unsupported) throw; chain_problem = e.what(); }
        if (!chain_problem.empty()) throw FormatError(chain_problem, true);
        if (flags & 0x01) r.bad("tensor dependencies (delta against another tensor)", true);
        if (flags & 0x02) { uint32_t ml = r.u32(); size_t mo = r.skip(ml); read_shape_metadata(mo, mo + ml, t); }
        detail::ChainShape sh = detail::chain_shape(*chain, b_, t.has_shape ? &t.shape : nullptr, t.dtype_code);
        if (sh.source_len != t.orig_size) r.bad("chain Source declares a different size than orig_size");
        t.kind = sh.kind;
        if (np != size_t(kind_planes(sh.kind))) r.bad("plane count differs from the chain's terminals");
        for (size_t i = 0; i < np; ++i) { t.planes.push_back(read_legacy_plane(r, sh.plane_len, *plane_table)); t.planes.back().post = sh.post[i]; t.planes.back().post_k = sh.post_k[i]; }
        return t;
    }
    ParsedFile parse_legacy() {
        static const uint8_t EOFS[8] = {0x89, 'T', 'W', 'M', 'E', 'O', 'F', 0x1a};
        if (n_ < 91 + 8) throw FormatError("legacy container: file too short");
        if (std::memcmp(b_ + n_ - 8, EOFS, 8)) throw FormatError("legacy container: missing EOF sentinel");
        const size_t body_end = n_ - 8;
        uint16_t flags = uint16_t(b_[9] | (b_[10] << 8));
        if (bool(flags & 1) != (b_[4] == 'X')) throw FormatError("legacy container: PTWX flag does not match the magic");
        uint64_t et_off = le64(b_ + 11), et_len = le64(b_ + 19), idx_off = le64(b_ + 59), idx_len = le64(b_ + 67), pre_off = le64(b_ + 75), pre_len = le64(b_ + 83);
        auto inside = [&](uint64_t off, uint64_t len, const char* what) {
            if (off < 91 || off > body_end || len > body_end - off) throw FormatError(std::string("legacy container: ") + what + " section exceeds the file");
        };
        inside(et_off, et_len, "extension table"); inside(idx_off, idx_len, "tensor index"); inside(pre_off, pre_len, "shared prelude");
        std::vector<LegacyEntry> table;
        if (et_len) {  // container.rs:1283-1304: the header commits to the table bytes
            uint8_t h[32];
            blake3_hash(b_ + et_off, size_t(et_len), h);
            if (std::memcmp(h, b_ + 27, 32)) throw FormatError("legacy container: extension table hash mismatch");
            read_legacy_table(size_t(et_off), size_t(et_off + et_len), table);
        }
        std::vector<std::pair<uint16_t, detail::RawChain>> registry;
        {
            const size_t end = size_t(pre_off + pre_len);
            size_t pos = parse_prelude(size_t(pre_off), end);
            Span r(b_, pos, end, "legacy chain registry");
            size_t count = size_t(r.byte()); count |= size_t(r.byte()) << 8;
            if (count > 0x8000) r.bad("too many chains");
            for (size_t i = 0; i < count; ++i) {
                uint16_t id = uint16_t(r.byte()); id |= uint16_t(r.byte()) << 8;
                detail::RawChain c;
                size_t after;
                try { after = read_legacy_chain(r.pos(), end, table, c); registry.push_back({id, std::move(c)}); }
                catch (const FormatError& e) {
                    if (!e.unsupported) throw;
                    // a chain outside the hot path: skip its bytes, tensors that use it are reported as unsupported
                    Span h(b_, r.pos(), end, "legacy chain");
                    h.skip(3);
                    size_t a = size_t(h.byte()); a |= size_t(h.byte()) << 8;
                    size_t b = size_t(h.byte()); b |= size_t(h.byte()) << 8;
                    size_t d = size_t(h.byte()); d |= size_t(h.byte()) << 8;
                    h.skip(a); h.skip(b); h.skip(d);
                    after = h.pos();
                    unsupported_chains_.push_back(id);
                }
                r.skip(after - r.pos());
            }
        }
        if (idx_len < 8) throw FormatError("legacy container: index section too short");
        uint64_t count = le64(b_ + idx_off);
        if (count > (idx_len - 8) / 24) throw FormatError("legacy container: index count exceeds the section");
        struct Rec { uint64_t off, len; };
        std::vector<Rec> recs;
        for (uint64_t i = 0; i < count; ++i) {
            const uint8_t* e = b_ + idx_off + 8 + 24 * i;
            uint64_t off = le64(e + 8), len = le64(e + 16);
            if (off < 91 || off > body_end || len > body_end - off) throw FormatError("legacy container: index entry points outside the file");
            recs.push_back(Rec{off, len});
        }
        std::sort(recs.begin(), recs.end(), [](const Rec& a, const Rec& b) { return a.off < b.off; });  // record (write) order
        for (const Rec& rec : recs) {
            TensorDesc t;
            try {
                // a record whose chain was skipped above is unsupported, not malformed
                uint16_t chain_ref = uint16_t(b_[rec.off] | (b_[rec.off + 1] << 8));
                bool skipped = false;
                if (rec.len >= 2 && !(chain_ref & 0x8000)) for (uint16_t id : unsupported_chains_) skipped |= id == chain_ref;
                if (skipped) throw FormatError("chain outside the production split/passthrough set", true);
                t = read_legacy_record(size_t(rec.off), size_t(rec.off + rec.len), table, registry);
            } catch (const FormatError& e) {
                if (!e.unsupported) throw;
                std::string name = legacy_record_name(size_t(rec.off), size_t(rec.off + rec.len));
                t = TensorDesc{}; t.unsupported = e.what(); t.name = name;
            }
            out_.tensors.push_back(std::move(t));
        }
        out_.legacy = true;
        return std::move(out_);
    }
    std::string legacy_record_name(size_t begin, size_t end) {
        Span r(b_, begin, end, "legacy tensor record");
        r.skip(16);
        size_t nl = size_t(r.byte()); nl |= size_t(r.byte()) << 8;
        return std::string(reinterpret_cast<const char*>(b_ + r.skip(nl)), nl);
    }
    std::vector<uint16_t> unsupported_chains_;

    ParsedFile parse_frame() {  // compact.rs:321-551
        out_.single_frame = true;
        Span r(b_, 5, n_, "compact frame");
        TensorDesc t;
        t.name = "_";
        uint8_t flags = r.byte();
        if (flags & 0x80) r.bad("unknown flag bits");
        if ((flags & 0x02) && (flags & 0x01)) r.bad("plane CRC flag with payload hash");
        t.dtype_code = uint16_t(r.var_max(0xFFFF, "dtype_code"));
        r.byte();
        bool has_stored = flags & 0x40; uint64_t stored = has_stored ? r.var() : 0;
        const char* canon = detail::canonical_dtype_name(t.dtype_code);
        if (flags & 0x04) {
            uint64_t nd = r.var_max(64, "ndim");
            for (uint64_t i = 0; i < nd; ++i) t.shape.push_back(r.var());
            t.has_shape = true;
            if (canon) t.dtype_name = canon;
        }
        if (flags & 0x08) {
            if (!t.has_shape) r.bad("dtype name without shape");
            size_t l = r.var_len();
            std::string nm(reinterpret_cast<const char*>(b_ + r.skip(l)), l);
            if (canon && nm == canon) r.bad("stored dtype name equals the canonical name");
            t.dtype_name = nm;
        } else if (t.has_shape && !canon) r.bad("shape without a dtype name for unknown dtype_code");
        bool has_derived = false; uint64_t derived = 0;
        if (t.has_shape && detail::public_dtype_bytes(t.dtype_code)) {
            derived = detail::public_dtype_bytes(t.dtype_code); has_derived = true;
            for (uint64_t d : t.shape) { if (d && derived > UINT64_MAX / d) { has_derived = false; break; } derived *= d; }
        }
        if (has_stored && has_derived && stored == derived) r.bad("stored orig_size equals the size the shape gives");
        if (has_stored) t.orig_size = stored; else if (has_derived) t.orig_size = derived; else r.bad("no orig_size and no shape that gives it");
        if (flags & 0x10) r.bad("delta reference", true);
        if (flags & 0x01) { t.has_hash = true; t.hash = r.u64(); }
        if (flags & 0x20) {
            if (flags & 0x02) r.bad("stored frame with plane CRC flag");
            if (r.left() != t.orig_size) r.bad("stored body length differs from orig_size");
            t.stored = true; t.stored_off = r.skip(size_t(t.orig_size)); t.kind = K_PASS;
        } else {
            try {
                detail::RawChain c = detail::read_cw2(r, [&](uint64_t ref) -> uint16_t { if (ref > 0xFFFF) r.bad("op id exceeds u16"); return uint16_t(ref); });
                detail::ChainShape sh = detail::chain_shape(c, b_, t.has_shape ? &t.shape : nullptr, t.dtype_code);
                if (sh.source_len != t.orig_size) r.bad("chain Source declares a different size than the header");
                t.kind = sh.kind;
                for (int pi = 0; pi < kind_planes(sh.kind); ++pi) {
                    PlaneDesc p;
                    uint64_t head = r.var();
                    if ((head >> 2) > 0xFFFF) r.bad("codec id exceeds u16");
                    p.codec = uint16_t(head >> 2);
                    uint8_t sv = 0; uint64_t so = 0, sl = 0;
                    switch (head & 3) {
                        case 0: case 2: break;
                        case 1: { sv = r.byte(); sl = r.var_len(); so = r.skip(size_t(sl)); if (!sv && !sl) r.bad("empty version-0 inline state must use state code 2"); p.state_source = 1; break; }
                        default: r.bad("unknown state code");
                    }
                    p.payload_len = r.var_len();
                    if (flags & 0x02) { p.has_crc = true; p.crc = r.u32(); }
                    p.payload_off = r.skip(size_t(p.payload_len));
                    p.decoded_len = sh.plane_len;
                    p.post = sh.post[pi]; p.post_k = sh.post_k[pi];
                    p.row_len = sh.kind == K_PASS ? sh.row_len : 0;  // the frame stores no layout: it follows the chain (compact.rs:500-503)
                    make_chunks(p, false, {}, so, sl, sv, 0);
                    t.planes.push_back(std::move(p));
                }
            } catch (const FormatError& e) {
                if (!e.unsupported) throw;
                t.unsupported = e.what(); t.planes.clear();
                out_.tensors.push_back(std::move(t));
                return std::move(out_);
            }
        }
        r.done("body");
        out_.tensors.push_back(std::move(t));
        return std::move(out_);
    }
};

inline void check_o1sac(const uint8_t* st, uint64_t state_len, uint8_t version, uint64_t payload_len, uint64_t decoded, uint64_t row_len) {
    if (version != 1) throw FormatError("Order1ScaleAC: unknown state_format_version");
    if (state_len < 32 + 512) throw FormatError("Order1ScaleAC: state shorter than header");
    uint64_t pop = 0;
    for (int i = 0; i < 32; ++i) pop += uint64_t(__builtin_popcount(st[i]));
    if (state_len != 32 + 512 + pop * 512) throw FormatError("Order1ScaleAC: state length mismatch");
    uint32_t p_max = 0;
    for (uint64_t t = 0; t < 1 + pop; ++t) {
        uint32_t sum = 0;
        for (int i = 0; i < 256; ++i) {
            uint32_t v = uint32_t(st[32 + t * 512 + 2 * i]) | uint32_t(st[32 + t * 512 + 2 * i + 1]) << 8;
            if (!v) throw FormatError("Order1ScaleAC: zero PMF entry");
            sum += v; p_max = v > p_max ? v : p_max;
        }
        if (sum != 4096) throw FormatError("Order1ScaleAC: PMF sum mismatch");
    }
    uint64_t rl = row_len ? row_len : (decoded ? decoded : 1);
    if (decoded % rl) throw FormatError("Order1ScaleAC: row_len does not divide decoded length");
    if (p_max && p_max < 4096) {
        double bps = __builtin_log2(4096.0 / double(p_max));
        double budget = 8.0 * double(payload_len > 5 ? payload_len - 5 : 0);
        double n = __builtin_floor(budget / bps) + 1.0;
        if (double(decoded) > n) throw FormatError("Order1ScaleAC: declared length exceeds what the payload can encode");
    }
}

}  // namespace ptwm
