// CPU oracle (TEST INFRASTRUCTURE, not a product path): range coder,
// Order1ScaleAC, the tagged plane-codec wrappers, the fused split/merge
// transforms and the integrity hashes of ptwm-core.  Citations are
// file:line under crates/ptwm-core/src.
#pragma once
#include <array>
#include <cmath>

#include "entropy.hpp"

namespace oracle {

// ---------------------------------------------------------------------------
// Integrity: CRC-32/IEEE (crc32fast 1.5.0, zlib compatible) and XXH64
// (xxhash-rust 0.8.18) — published algorithms; call sites container.rs:2153-2159,
// 2184-2194.
// ---------------------------------------------------------------------------
inline uint32_t crc32(const uint8_t* p, size_t n, uint32_t crc = 0) {
    static uint32_t table[256];
    static bool init = false;
    if (!init) {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
            table[i] = c;
        }
        init = true;
    }
    crc = ~crc;
    for (size_t i = 0; i < n; ++i) crc = table[(crc ^ p[i]) & 0xFF] ^ (crc >> 8);
    return ~crc;
}

inline uint64_t rotl64(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }

inline uint64_t xxh64(const uint8_t* p, size_t len, uint64_t seed = 0) {
    const uint64_t P1 = 11400714785074694791ULL, P2 = 14029467366897019727ULL, P3 = 1609587929392839161ULL,
                   P4 = 9650029242287828579ULL, P5 = 2870177450012600261ULL;
    const uint8_t* end = p + len;
    uint64_t h;
    auto round = [&](uint64_t acc, uint64_t in) { acc += in * P2; acc = rotl64(acc, 31); return acc * P1; };
    auto merge = [&](uint64_t hh, uint64_t v) { v = round(0, v); hh ^= v; return hh * P1 + P4; };
    if (len >= 32) {
        uint64_t v1 = seed + P1 + P2, v2 = seed + P2, v3 = seed, v4 = seed - P1;
        const uint8_t* limit = end - 32;
        do {
            v1 = round(v1, get_u64le(p)); v2 = round(v2, get_u64le(p + 8));
            v3 = round(v3, get_u64le(p + 16)); v4 = round(v4, get_u64le(p + 24));
            p += 32;
        } while (p <= limit);
        h = rotl64(v1, 1) + rotl64(v2, 7) + rotl64(v3, 12) + rotl64(v4, 18);
        h = merge(h, v1); h = merge(h, v2); h = merge(h, v3); h = merge(h, v4);
    } else {
        h = seed + P5;
    }
    h += uint64_t(len);
    while (p + 8 <= end) { h ^= round(0, get_u64le(p)); h = rotl64(h, 27) * P1 + P4; p += 8; }
    if (p + 4 <= end) { h ^= uint64_t(get_u32le(p)) * P1; h = rotl64(h, 23) * P2 + P3; p += 4; }
    while (p < end) { h ^= uint64_t(*p) * P5; h = rotl64(h, 11) * P1; ++p; }
    h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
    return h;
}

// ---------------------------------------------------------------------------
// Range coder (range_coder.rs:16-198)
// ---------------------------------------------------------------------------
struct RangeEncoder {
    uint64_t low = 0, range = 0xFFFFFFFFull;
    uint8_t cache = 0;
    uint32_t cache_size = 0;
    Bytes out;
    void shift_low() {  // range_coder.rs:92-113
        uint8_t carry = uint8_t(low >> 32);
        uint8_t top = uint8_t((low >> 24) & 0xFF);
        if (top == 0xFF && carry == 0) {
            cache_size++;
        } else {
            out.push_back(uint8_t(cache + carry));
            uint8_t fill = carry ? 0x00 : 0xFF;
            for (uint32_t i = 0; i < cache_size; ++i) out.push_back(fill);
            cache_size = 0;
            cache = top;
        }
        low = (low & 0x00FFFFFFull) << 8;
    }
    void encode(uint32_t cumulative, uint32_t prob, uint32_t total) {  // :52-67
        uint64_t rpt = range / total;
        low += uint64_t(cumulative) * rpt;
        range = uint64_t(prob) * rpt;
        while (range < (1ull << 24)) { shift_low(); range <<= 8; }
    }
    Bytes finish() {  // :73-85
        for (int i = 0; i < 5; ++i) shift_low();
        out.push_back(cache);
        for (uint32_t i = 0; i < cache_size; ++i) out.push_back(0xFF);
        return out;
    }
};

struct RangeDecoder {  // range_coder.rs:122-198
    uint64_t low = 0, range = 0xFFFFFFFFull, code = 0;
    const uint8_t* src; size_t len, pos = 0;
    RangeDecoder(const uint8_t* s, size_t n) : src(s), len(n) {
        while (pos < 5) { uint8_t b = pos < len ? src[pos] : 0; code = (code << 8) | b; pos++; }
    }
    uint32_t target(uint32_t total) const {
        uint64_t rpt = range / total;
        uint64_t offset = ((code & 0xFFFFFFFFull) - low) & 0xFFFFFFFFull;
        return uint32_t(std::min<uint64_t>(offset / rpt, total - 1));
    }
    void advance(uint32_t cumulative, uint32_t prob, uint32_t total) {
        uint64_t rpt = range / total;
        low += uint64_t(cumulative) * rpt;
        range = uint64_t(prob) * rpt;
        low &= 0xFFFFFFFFull;
        while (range < (1ull << 24)) {
            uint8_t b = pos < len ? src[pos] : 0;
            pos++;
            code = ((code & 0xFFFFFFFFFFull) << 8) | b;
            low = (low & 0x00FFFFFFull) << 8;
            range <<= 8;
        }
    }
};

// ---------------------------------------------------------------------------
// PMF quantiser (quantize.rs:13-45): Laplace +1, round-half-away, last
// argmax shaved, first argmin grown.
// ---------------------------------------------------------------------------
inline void quantize_pmf(const uint32_t* raw, size_t n, uint32_t total, uint16_t* out) {
    if (n == 0) return;
    double sum = 0;
    for (size_t i = 0; i < n; ++i) sum += double(raw[i] + 1);
    uint32_t current = 0;
    for (size_t i = 0; i < n; ++i) {
        double v = std::round((double(raw[i] + 1) / sum) * double(total));
        if (v < 1.0) v = 1.0;
        out[i] = uint16_t(v);
        current += out[i];
    }
    while (current > total) {
        size_t am = 0;
        for (size_t i = 0; i < n; ++i) if (out[i] >= out[am]) am = i;  // Iterator::max_by_key keeps the last maximum
        if (out[am] > 1) { out[am]--; current--; } else break;
    }
    while (current < total) {
        size_t am = 0;
        for (size_t i = 0; i < n; ++i) if (out[i] < out[am]) am = i;  // min_by_key keeps the first minimum
        out[am]++; current++;
    }
}

// ---------------------------------------------------------------------------
// Order1ScaleAC (codecs/order1_scale_ac.rs)
// ---------------------------------------------------------------------------
namespace o1sac {

constexpr uint32_t TOTAL = 4096;  // quantize.rs:8
constexpr uint8_t STATE_FORMAT_VERSION = 1;

struct State {
    uint8_t bitmap[32] = {0};
    uint16_t marginal[256] = {0};
    std::vector<std::array<uint16_t, 256>> rows;
    uint32_t marginal_cum[257] = {0};
    std::vector<std::array<uint32_t, 257>> rows_cum;
    void materialize() {  // :117-141
        uint32_t acc = 0;
        for (int i = 0; i < 256; ++i) { marginal_cum[i] = acc; acc += marginal[i]; }
        marginal_cum[256] = acc;
        rows_cum.resize(rows.size());
        for (size_t r = 0; r < rows.size(); ++r) {
            acc = 0;
            for (int i = 0; i < 256; ++i) { rows_cum[r][i] = acc; acc += rows[r][i]; }
            rows_cum[r][256] = acc;
        }
    }
    bool has(uint8_t prev) const { return bitmap[prev >> 3] & (1 << (prev & 7)); }  // :85-90
    size_t rank(uint8_t prev) const {  // :95-103
        size_t r = 0;
        for (int b = 0; b < (prev >> 3); ++b) r += size_t(__builtin_popcount(bitmap[b]));
        r += size_t(__builtin_popcount(bitmap[prev >> 3] & ((1u << (prev & 7)) - 1)));
        return r;
    }
    const uint32_t* cum_for(int prev) const {  // :145-151
        if (prev < 0) return marginal_cum;
        return has(uint8_t(prev)) ? rows_cum[rank(uint8_t(prev))].data() : marginal_cum;
    }
};

inline void validate_pmf(const uint16_t* pmf) {  // quantize.rs:53-71
    uint32_t sum = 0;
    for (int i = 0; i < 256; ++i) { if (pmf[i] == 0) throw Error("o1sac: zero PMF entry"); sum += pmf[i]; }
    if (sum != TOTAL) throw Error("o1sac: PMF sum mismatch");
}

inline Bytes serialize_state(const State& s) {  // :158-171
    Bytes out(s.bitmap, s.bitmap + 32);
    for (int i = 0; i < 256; ++i) { out.push_back(uint8_t(s.marginal[i])); out.push_back(uint8_t(s.marginal[i] >> 8)); }
    for (auto& r : s.rows) for (int i = 0; i < 256; ++i) { out.push_back(uint8_t(r[i])); out.push_back(uint8_t(r[i] >> 8)); }
    return out;
}

inline State deserialize_state(const uint8_t* b, size_t n) {  // :174-220
    if (n < 32 + 512) throw Error("o1sac: state shorter than header");
    State s;
    std::memcpy(s.bitmap, b, 32);
    size_t pop = 0;
    for (int i = 0; i < 32; ++i) pop += size_t(__builtin_popcount(s.bitmap[i]));
    if (n != 32 + 512 + pop * 512) throw Error("o1sac: state length mismatch");
    size_t off = 32;
    for (int i = 0; i < 256; ++i, off += 2) s.marginal[i] = uint16_t(b[off] | (b[off + 1] << 8));
    validate_pmf(s.marginal);
    s.rows.resize(pop);
    for (size_t r = 0; r < pop; ++r) {
        for (int i = 0; i < 256; ++i, off += 2) s.rows[r][i] = uint16_t(b[off] | (b[off + 1] << 8));
        validate_pmf(s.rows[r].data());
    }
    s.materialize();
    return s;
}

// :963-1025 — per-row lag-1 counts then quantise; only contexts with a count
// get a row.
inline State fit(const uint8_t* plane, size_t n, size_t row_len) {
    std::vector<std::array<uint32_t, 256>> joint(256);
    for (auto& r : joint) r.fill(0);
    uint32_t marg[256] = {0};
    for (size_t base = 0; base < n; base += row_len) {
        size_t end = std::min(n, base + row_len);
        marg[plane[base]]++;
        for (size_t i = base + 1; i < end; ++i) joint[plane[i - 1]][plane[i]]++;
    }
    State s;
    quantize_pmf(marg, 256, TOTAL, s.marginal);
    for (int prev = 0; prev < 256; ++prev) {
        uint64_t rs = 0;
        for (int i = 0; i < 256; ++i) rs += joint[prev][i];
        if (rs == 0) continue;
        s.bitmap[prev >> 3] |= uint8_t(1u << (prev & 7));
        std::array<uint16_t, 256> row;
        quantize_pmf(joint[prev].data(), 256, TOTAL, row.data());
        s.rows.push_back(row);
    }
    s.materialize();
    return s;
}

// row_len 0 = Flat layout (row = whole plane) (:411-432)
inline size_t resolve_row_len(size_t plane_len, size_t row_len) {
    size_t r = row_len ? row_len : std::max<size_t>(plane_len, 1);
    if (plane_len % r != 0) throw Error("o1sac: row_len does not divide plane length");
    return r;
}

// :620-663 — inline state when no shared state is given.
inline void encode(const uint8_t* plane, size_t n, size_t row_len_layout, const uint8_t* shared, size_t shared_len,
                   Bytes& state_bytes, Bytes& payload) {
    size_t row_len = resolve_row_len(n, row_len_layout);
    State s;
    if (shared) { s = deserialize_state(shared, shared_len); state_bytes.clear(); }
    else {
        s = fit(plane, n, row_len);
        validate_pmf(s.marginal);
        for (auto& r : s.rows) validate_pmf(r.data());
        state_bytes = serialize_state(s);
    }
    RangeEncoder enc;
    for (size_t base = 0; base < n; base += row_len) {
        int prev = -1;
        for (size_t i = base; i < std::min(n, base + row_len); ++i) {
            const uint32_t* cs = s.cum_for(prev);
            uint32_t c = cs[plane[i]], p = cs[plane[i] + 1] - c;
            enc.encode(c, p, TOTAL);
            prev = plane[i];
        }
    }
    payload = enc.finish();
}

inline size_t max_decodable_len(const State& s, size_t payload_len) {  // :449-471
    uint32_t p_max = 0;
    for (auto& r : s.rows) for (int i = 0; i < 256; ++i) p_max = std::max<uint32_t>(p_max, r[i]);
    for (int i = 0; i < 256; ++i) p_max = std::max<uint32_t>(p_max, s.marginal[i]);
    if (p_max == 0 || p_max >= TOTAL) return SIZE_MAX;
    double bps = std::log2(double(TOTAL) / double(p_max));
    double budget = 8.0 * double(payload_len > 5 ? payload_len - 5 : 0);
    double n = std::floor(budget / bps) + 1.0;
    if (n >= double(SIZE_MAX)) return SIZE_MAX;
    return size_t(n);
}

inline size_t binary_search_cumsum(const uint32_t* cs, uint32_t target) {  // :474-486
    size_t lo = 0, hi = 256;
    while (lo + 1 < hi) { size_t mid = (lo + hi) / 2; if (cs[mid] <= target) lo = mid; else hi = mid; }
    return lo;
}

inline Bytes decode(uint8_t state_version, const uint8_t* state, size_t state_len, const uint8_t* payload, size_t payload_len,
                    size_t row_len_layout, size_t decoded_len) {  // :665-706
    if (state_version != STATE_FORMAT_VERSION) throw Error("o1sac: unknown state_format_version");
    State s = deserialize_state(state, state_len);
    size_t row_len = row_len_layout ? row_len_layout : std::max<size_t>(decoded_len, 1);
    if (decoded_len % row_len != 0) throw Error("o1sac: row_len does not divide decoded length");
    if (decoded_len > max_decodable_len(s, payload_len)) throw Error("o1sac: declared length exceeds what the payload can encode");
    RangeDecoder dec(payload, payload_len);
    Bytes out(decoded_len);
    size_t row_pos = 0; int prev = -1;
    for (size_t i = 0; i < decoded_len; ++i) {
        if (row_pos == 0) prev = -1;
        const uint32_t* cs = s.cum_for(prev);
        uint32_t t = dec.target(TOTAL);
        size_t sym = binary_search_cumsum(cs, t);
        dec.advance(cs[sym], cs[sym + 1] - cs[sym], TOTAL);
        out[i] = uint8_t(sym);
        prev = int(sym);
        row_pos = (row_pos + 1) % row_len;
    }
    return out;
}

}  // namespace o1sac

// ---------------------------------------------------------------------------
// Plane codecs (codec.rs:5-23 wire ids; codecs/{identity,huffman,rans,tans}.rs)
// ---------------------------------------------------------------------------
enum CodecId : uint16_t { IDENTITY = 0, HUFFMAN = 1, RANS = 3, ZSTD = 4, TANS = 7, O1SAC = 0x11 };

// Zstd planes are outside the hot path.  The reference's golden fixtures hold
// some (codecs/zstd.rs:65-106: a plain Zstd frame), so a test may install the
// system libzstd's ZSTD_decompress here to read them; nothing else uses it.
using ZstdDecompressFn = size_t (*)(void* dst, size_t cap, const void* src, size_t len);
using ZstdIsErrorFn = unsigned (*)(size_t code);
inline ZstdDecompressFn& zstd_decompress_hook() { static ZstdDecompressFn f = nullptr; return f; }
inline ZstdIsErrorFn& zstd_is_error_hook() { static ZstdIsErrorFn f = nullptr; return f; }

struct Encoded { Bytes state; uint8_t state_version = 0; Bytes payload; };

// codecs/length_prefix.rs:15-33
inline bool length_accepted(size_t decoded_len, size_t body_len) {
    const size_t RATIO_FREE = size_t(1) << 30, MAX_RATIO = 64;
    if (decoded_len > 0xFFFFFFFFull) return false;
    return decoded_len <= RATIO_FREE || decoded_len <= body_len * MAX_RATIO;
}

inline Bytes tagged(uint8_t tag, const uint8_t* plane, size_t n, const Bytes* blob) {
    Bytes p;
    p.push_back(tag);
    if (tag == 0) p.insert(p.end(), plane, plane + n);
    else {
        uint8_t l[4]; put_u32le(l, uint32_t(n));
        p.insert(p.end(), l, l + 4);
        p.insert(p.end(), blob->begin(), blob->end());
    }
    return p;
}

// row_len: 0 = Flat.  shared: optional shared state bytes (O1SAC only).
inline Encoded plane_encode(CodecId id, const uint8_t* plane, size_t n, size_t row_len = 0,
                            const uint8_t* shared = nullptr, size_t shared_len = 0) {
    Encoded e;
    switch (id) {
        case IDENTITY: e.payload.assign(plane, plane + n); return e;  // identity.rs:27-38
        case HUFFMAN: {  // huffman.rs:37-88
            if (n == 0) { e.payload = {0}; return e; }
            Bytes blob = huffman::compress(plane, n);
            bool ok = !blob.empty() && n <= 0xFFFFFFFFull;
            e.payload = tagged(ok ? 1 : 0, plane, n, &blob);
            return e;
        }
        case RANS: {  // rans.rs:38-95
            if (n == 0) { e.payload = {0}; return e; }
            Bytes blob = rans::compress(plane, n);
            bool ok = !blob.empty() && length_accepted(n, blob.size());
            e.payload = tagged(ok ? 1 : 0, plane, n, &blob);
            return e;
        }
        case TANS: {  // tans.rs:39-90
            if (n == 0) { e.payload = {0}; return e; }
            Bytes blob = tans::compress(plane, n, n);
            bool ok = !blob.empty() && length_accepted(n, blob.size());
            e.payload = tagged(ok ? 1 : 0, plane, n, &blob);
            return e;
        }
        case O1SAC: {
            o1sac::encode(plane, n, row_len, shared, shared_len, e.state, e.payload);
            e.state_version = o1sac::STATE_FORMAT_VERSION;
            return e;
        }
        default: throw Error("unsupported: codec outside the hot path");
    }
}

// PlaneCodec::decode_bounded (codec.rs:182-202 default; rans.rs:148-170 and
// tans.rs:139-163 check the length prefix first).
inline Bytes plane_decode(CodecId id, uint8_t state_version, const uint8_t* state, size_t state_len, const uint8_t* payload,
                          size_t payload_len, size_t row_len, size_t decoded_len, size_t max_len) {
    Bytes out;
    auto tagged_decode = [&](const char* name, auto&& accept, auto&& inner) {
        if (payload_len == 0) throw Error(std::string(name) + ": empty payload");
        uint8_t tag = payload[0];
        const uint8_t* rest = payload + 1; size_t rl = payload_len - 1;
        if (tag == 0) { out.assign(rest, rest + rl); return; }
        if (tag != 1) throw Error(std::string(name) + ": bad tag");
        if (rl < 4) throw Error(std::string(name) + ": payload too short for length prefix");
        size_t orig = get_u32le(rest);
        if (!accept(orig, rl - 4)) throw Error(std::string(name) + ": implausible orig_len");
        out.resize(orig);
        inner(out.data(), orig, rest + 4, rl - 4);
    };
    switch (id) {
        case IDENTITY: out.assign(payload, payload + payload_len); break;
        case HUFFMAN:
            tagged_decode("huffman", [](size_t o, size_t e) { return o <= e * 32 + 4096; },
                          [](uint8_t* d, size_t n, const uint8_t* s, size_t l) { huffman::decompress(d, n, s, l); });
            break;
        case RANS:
        case TANS: {
            if (payload_len >= 5 && payload[0] == 1 && get_u32le(payload + 1) > max_len) throw Error("payload declares more than the bound");
            if (id == RANS)
                tagged_decode("rans", length_accepted,
                              [](uint8_t* d, size_t n, const uint8_t* s, size_t l) { if (n) rans::decompress(d, n, s, l); });
            else
                tagged_decode("tans", length_accepted,
                              [](uint8_t* d, size_t n, const uint8_t* s, size_t l) { tans::decompress(d, n, s, l); });
            break;
        }
        case O1SAC: out = o1sac::decode(state_version, state, state_len, payload, payload_len, row_len, decoded_len); break;
        case ZSTD: {
            if (!zstd_decompress_hook()) throw Error("unsupported: zstd plane (out of scope; test hook not installed)");
            if (payload_len == 0) break;  // codec_tagged.rs:207-210
            out.resize(max_len ? max_len : 1);
            size_t got = zstd_decompress_hook()(out.data(), max_len, payload, payload_len);
            if (zstd_is_error_hook()(got)) throw Error("zstd: decode failed or output exceeds the bound");
            out.resize(got);
            break;
        }
        default: throw Error("unsupported: codec outside the hot path");
    }
    if (out.size() > max_len) throw Error("plane decodes past its bound");
    return out;
}

// ---------------------------------------------------------------------------
// Fused split/merge (transforms/fusion.rs; split/dtype{8,16,32}.rs)
// ---------------------------------------------------------------------------
enum MergeKind : int { PASS = 0, M16 = 1, M32 = 2, FP8_E4M3 = 3, FP8_E5M2 = 4 };

inline int merge_planes(MergeKind k) { return k == PASS ? 1 : k == M32 ? 4 : 2; }

// forward: raw -> planes (fusion.rs:35-122, 207-262, 329-371, 431-473)
inline std::vector<Bytes> split_forward(MergeKind k, const uint8_t* src, size_t n) {
    std::vector<Bytes> p(size_t(merge_planes(k)));
    switch (k) {
        case PASS: p[0].assign(src, src + n); break;
        case M16: {
            if (n % 2) throw Error("split16: odd length");
            p[0].resize(n / 2); p[1].resize(n / 2);
            for (size_t i = 0; i < n / 2; ++i) {
                uint16_t v = uint16_t(src[2 * i] | (src[2 * i + 1] << 8));
                uint16_t r = uint16_t(((v << 1) & 0xFF00) | ((v >> 8) & 0x0080) | (v & 0x007F));  // dtype16.rs:11-16
                p[0][i] = uint8_t(r); p[1][i] = uint8_t(r >> 8);
            }
            break;
        }
        case M32: {
            if (n % 4) throw Error("split32: length not divisible by 4");
            for (auto& b : p) b.resize(n / 4);
            for (size_t i = 0; i < n / 4; ++i) {
                uint32_t v = get_u32le(src + 4 * i);
                uint32_t r = ((v << 1) & 0xFF000000u) | ((v >> 8) & 0x00800000u) | (v & 0x007FFFFFu);  // fusion.rs:226-231
                for (int j = 0; j < 4; ++j) p[size_t(j)][i] = uint8_t(r >> (8 * j));
            }
            break;
        }
        case FP8_E4M3:
        case FP8_E5M2: {
            p[0].resize(n); p[1].resize(n);
            for (size_t i = 0; i < n; ++i) {
                uint8_t v = src[i];
                uint8_t r = k == FP8_E4M3 ? uint8_t(((v & 0x78) << 1) | ((v & 0x80) >> 4) | (v & 0x07))   // dtype8.rs:30-35
                                          : uint8_t(((v & 0x7C) << 1) | ((v & 0x80) >> 5) | (v & 0x03));  // dtype8.rs:48-53
                p[0][i] = r >> 4; p[1][i] = r & 0x0F;
            }
            break;
        }
    }
    return p;
}

// inverse: planes -> raw (fusion.rs:124-193, 264-315, 373-417, 475-519)
inline Bytes merge_inverse(MergeKind k, const std::vector<Bytes>& p) {
    if (int(p.size()) != merge_planes(k)) throw Error("merge: wrong plane count");
    for (auto& b : p) if (b.size() != p[0].size()) throw Error("merge: plane lengths differ");
    size_t m = p[0].size();
    Bytes out;
    switch (k) {
        case PASS: out = p[0]; break;
        case M16:
            out.resize(2 * m);
            for (size_t i = 0; i < m; ++i) {
                uint16_t r = uint16_t(p[0][i] | (p[1][i] << 8));
                uint16_t v = uint16_t(((r << 8) & 0x8000) | ((r >> 1) & 0x7F80) | (r & 0x007F));  // dtype16.rs:20-25
                out[2 * i] = uint8_t(v); out[2 * i + 1] = uint8_t(v >> 8);
            }
            break;
        case M32:
            out.resize(4 * m);
            for (size_t i = 0; i < m; ++i) {
                uint32_t r = uint32_t(p[0][i]) | uint32_t(p[1][i]) << 8 | uint32_t(p[2][i]) << 16 | uint32_t(p[3][i]) << 24;
                uint32_t v = ((r << 8) & 0x80000000u) | ((r >> 1) & 0x7F800000u) | (r & 0x007FFFFFu);  // fusion.rs:287-292
                put_u32le(&out[4 * i], v);
            }
            break;
        case FP8_E4M3:
        case FP8_E5M2:
            out.resize(m);
            for (size_t i = 0; i < m; ++i) {
                uint8_t r = uint8_t(((p[0][i] & 0x0F) << 4) | (p[1][i] & 0x0F));
                out[i] = k == FP8_E4M3 ? uint8_t(((r & 0xF0) >> 1) | ((r & 0x08) << 4) | (r & 0x07))   // dtype8.rs:39-44
                                       : uint8_t(((r & 0xF8) >> 1) | ((r & 0x04) << 5) | (r & 0x03));  // dtype8.rs:57-62
            }
            break;
    }
    return out;
}

}  // namespace oracle
