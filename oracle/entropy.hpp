// CPU oracle (TEST INFRASTRUCTURE, not a product path): restatement of the
// byte-alphabet entropy coders of ptwm-core.  Each function cites the
// reference file:line (paths relative to crates/ptwm-core/src) it follows.
// Only tests, the smoke check and the bench's CPU-baseline leg may use it.
//
// Pinned against the reference's own vectors (tests/golden/reference): Huffman,
// tANS, Identity and the three merges through the legacy_trimmed table,
// Order1ScaleAC (shared prelude state, rows) and a chunked tANS plane through
// the legacy_v1_1_0 / legacy_v1_0_0 tables, the compact reader and writer
// through ptwc_bound_source (byte-identical rewrite), 21 self-verifying
// compact frames, XXH64 / CRC-32 against independent implementations.
// rANS coded payloads: parity unpinned by a stored vector (the reference keeps
// none); encoder and decoder are restated from entropy/rans/*.rs and checked by
// round trips over the reference's unit-test inputs.
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <queue>
#include <stdexcept>
#include <string>
#include <vector>

namespace oracle {

using Bytes = std::vector<uint8_t>;

struct Error : std::runtime_error {
    explicit Error(const std::string& m) : std::runtime_error(m) {}
};

// entropy/stream_frame.rs:27-41 — four contiguous segments, the first len%4
// one byte longer.
inline void split_four(size_t len, size_t start[4], size_t end[4]) {
    size_t base = len / 4, rem = len % 4, s = 0;
    for (int i = 0; i < 4; ++i) {
        size_t seg = base + (size_t(i) < rem ? 1 : 0);
        start[i] = s;
        end[i] = s + seg;
        s = end[i];
    }
}
constexpr size_t JUMP_TABLE_BYTES = 16;  // stream_frame.rs:11

inline void put_u32le(uint8_t* p, uint32_t v) {
    p[0] = uint8_t(v); p[1] = uint8_t(v >> 8); p[2] = uint8_t(v >> 16); p[3] = uint8_t(v >> 24);
}
inline uint32_t get_u32le(const uint8_t* p) {
    return uint32_t(p[0]) | uint32_t(p[1]) << 8 | uint32_t(p[2]) << 16 | uint32_t(p[3]) << 24;
}
inline uint64_t get_u64le(const uint8_t* p) {
    return uint64_t(get_u32le(p)) | uint64_t(get_u32le(p + 4)) << 32;
}

// ---------------------------------------------------------------------------
// Canonical Huffman (entropy/huffman/)
// ---------------------------------------------------------------------------
namespace huffman {

constexpr int MAX_TABLE_LOG = 11;  // tree.rs:5

struct Tree {
    uint8_t lengths[256] = {0};
    int max_bits = 1;
    std::vector<uint16_t> table;  // len<<8 | sym, 1<<max_bits entries
    uint16_t rev_codes[256] = {0};
};

inline uint16_t reverse_bits(uint16_t code, int nbits) {  // tree.rs:244-251
    uint16_t out = 0;
    for (int i = 0; i < nbits; ++i) { out = uint16_t((out << 1) | (code & 1)); code >>= 1; }
    return out;
}

// tree.rs:103-177 — canonical codes from lengths, reversed into LSB-first
// order, decode table with (max_bits<<8) fallback entries.
inline bool from_lengths(const uint8_t lengths[256], Tree& t) {
    int max_bits = 0;
    for (int i = 0; i < 256; ++i) max_bits = std::max<int>(max_bits, lengths[i]);
    max_bits = std::max(max_bits, 1);
    if (max_bits > MAX_TABLE_LOG) return false;
    uint32_t counts[MAX_TABLE_LOG + 1] = {0};
    uint32_t total = 0;
    for (int i = 0; i < 256; ++i) if (lengths[i] > 0) { counts[lengths[i]]++; total++; }
    if (total == 0) return false;
    uint32_t next_code[MAX_TABLE_LOG + 1] = {0};
    uint32_t code = 0;
    for (int bits = 1; bits <= max_bits; ++bits) {
        code = (code + counts[bits - 1]) << 1;
        if (code > (1u << bits)) return false;
        next_code[bits] = code;
    }
    uint32_t codes[256] = {0};
    for (int sym = 0; sym < 256; ++sym) {
        int len = lengths[sym];
        if (len == 0) continue;
        uint32_t c = next_code[len];
        if (c >= (1u << len)) return false;
        codes[sym] = c;
        next_code[len] = c + 1;
    }
    const uint16_t fallback = uint16_t(max_bits << 8);
    t.table.assign(size_t(1) << max_bits, fallback);
    std::memcpy(t.lengths, lengths, 256);
    t.max_bits = max_bits;
    for (int sym = 0; sym < 256; ++sym) {
        int len = lengths[sym];
        t.rev_codes[sym] = 0;
        if (len == 0) continue;
        uint16_t rev = reverse_bits(uint16_t(codes[sym]), len);
        t.rev_codes[sym] = rev;
        size_t spread = size_t(1) << (max_bits - len);
        uint16_t entry = uint16_t((len << 8) | sym);
        for (size_t i = 0; i < spread; ++i) {
            size_t idx = size_t(rev) | (i << len);
            if (t.table[idx] != fallback && t.table[idx] != entry) return false;
            t.table[idx] = entry;
        }
    }
    return true;
}

// tree.rs:212-242 — clamp to max_len, then lengthen the shortest active
// code (first such symbol) until the Kraft sum fits.
inline void enforce_max_code_length(uint8_t lengths[256], int max_len) {
    bool clamped = false;
    for (int i = 0; i < 256; ++i) if (lengths[i] > max_len) { lengths[i] = uint8_t(max_len); clamped = true; }
    if (!clamped) return;
    const uint32_t capacity = 1u << max_len;
    auto kraft = [&]() { uint32_t s = 0; for (int i = 0; i < 256; ++i) if (lengths[i]) s += 1u << (max_len - lengths[i]); return s; };
    while (kraft() > capacity) {
        int victim = -1;
        for (int s = 0; s < 256; ++s)
            if (lengths[s] > 0 && lengths[s] < max_len && (victim < 0 || lengths[s] < lengths[victim])) victim = s;
        if (victim < 0) break;
        lengths[victim]++;
    }
}

// tree.rs:19-85 — heap Huffman; ties ordered by (freq, node id), leaves take
// ids in symbol order, internal nodes the next ids.
inline bool from_frequencies(const uint32_t freqs[256], Tree& t) {
    std::vector<int> symbols;
    for (int i = 0; i < 256; ++i) if (freqs[i] > 0) symbols.push_back(i);
    if (symbols.empty()) return false;
    uint8_t lengths[256] = {0};
    if (symbols.size() == 1) { lengths[symbols[0]] = 1; return from_lengths(lengths, t); }
    size_t n = symbols.size();
    std::vector<uint64_t> nf(2 * n, 0);
    std::vector<int> left(2 * n, -1), right(2 * n, -1);
    using Item = std::pair<uint64_t, size_t>;
    std::priority_queue<Item, std::vector<Item>, std::greater<Item>> heap;
    for (size_t id = 0; id < n; ++id) { nf[id] = freqs[symbols[id]]; heap.push({nf[id], id}); }
    size_t next_id = n;
    while (heap.size() > 1) {
        Item a = heap.top(); heap.pop();
        Item b = heap.top(); heap.pop();
        size_t id = next_id++;
        nf[id] = a.first + b.first;
        left[id] = int(a.second);
        right[id] = int(b.second);
        heap.push({nf[id], id});
    }
    size_t root = heap.top().second;
    std::vector<std::pair<size_t, int>> stack{{root, 0}};
    while (!stack.empty()) {
        auto [id, depth] = stack.back(); stack.pop_back();
        if (id < n) lengths[symbols[id]] = uint8_t(std::min(depth, 255));
        else {
            int nd = std::min(depth + 1, 255);
            if (left[id] >= 0) stack.push_back({size_t(left[id]), nd});
            if (right[id] >= 0) stack.push_back({size_t(right[id]), nd});
        }
    }
    enforce_max_code_length(lengths, MAX_TABLE_LOG);
    return from_lengths(lengths, t);
}

// weights.rs:8-32
inline void encode_weights(const uint8_t* w, size_t n, Bytes& out) {
    if (n <= 127) out.push_back(uint8_t(0x80 | n));
    else { out.push_back(0x80); out.push_back(uint8_t(n)); }
    for (size_t i = 0; i < n; i += 2) {
        uint8_t lo = w[i] & 0x0F, hi = (i + 1 < n ? w[i + 1] : 0) & 0x0F;
        out.push_back(uint8_t(lo | (hi << 4)));
    }
}

// weights.rs:34-85 — returns bytes consumed; weights has n_symbols entries.
inline size_t decode_weights(const uint8_t* src, size_t len, std::vector<uint8_t>& weights) {
    if (len == 0) throw Error("huffman: missing weight header");
    uint8_t header = src[0];
    if ((header & 0x80) == 0) throw Error("huffman: invalid weight header byte");
    size_t n, hb;
    if (header == 0x80) {
        if (len < 2) throw Error("huffman: truncated extended weight header");
        size_t c = src[1];
        n = c == 0 ? 256 : c;
        if (n < 128) throw Error("huffman: invalid extended weight count");
        hb = 2;
    } else {
        n = header & 0x7F;
        hb = 1;
    }
    size_t needed = hb + (n + 1) / 2;
    if (len < needed) throw Error("huffman: weight payload truncated");
    weights.resize(n);
    for (size_t i = 0; i < n; ++i) {
        uint8_t b = src[hb + i / 2];
        weights[i] = (i % 2 == 0) ? (b & 0x0F) : ((b >> 4) & 0x0F);
    }
    return needed;
}

// bitstream.rs:3-51 — LSB-first bit packing written backward: the stream is
// the byte-reversed LSB-first sequence, ceil(bits/8) bytes.
inline void encode_stream(const uint8_t* src, size_t n, const Tree& t, Bytes& out) {
    Bytes fwd;
    fwd.reserve(n * 2 + 8);
    uint64_t acc = 0; int cnt = 0;
    for (size_t i = 0; i < n; ++i) {
        int len = t.lengths[src[i]];
        if (len == 0) throw Error("huffman: missing code for symbol");
        acc |= uint64_t(t.rev_codes[src[i]]) << cnt;
        cnt += len;
        while (cnt >= 8) { fwd.push_back(uint8_t(acc)); acc >>= 8; cnt -= 8; }
    }
    if (cnt > 0) fwd.push_back(uint8_t(acc));
    out.assign(fwd.rbegin(), fwd.rend());
}

// compress.rs:9-103 — returns the blob, or empty when the outcome is not
// Encoded (Incompressible / NotBeneficial / DstTooSmall): caller stores raw.
inline Bytes compress(const uint8_t* src, size_t n) {
    if (n == 0) return {};
    uint32_t freqs[256] = {0};
    for (size_t i = 0; i < n; ++i) freqs[src[i]]++;
    Tree t;
    if (!from_frequencies(freqs, t)) return {};
    size_t nw = 0;
    for (int i = 255; i >= 0; --i) if (t.lengths[i] > 0) { nw = size_t(i) + 1; break; }
    Bytes out;
    encode_weights(t.lengths, nw, out);
    size_t jump_pos = out.size();
    out.resize(out.size() + JUMP_TABLE_BYTES, 0);
    const size_t dst_cap = n * 2 + 4096;  // codec_tagged.rs:148-150 output bound
    if (out.size() >= dst_cap) return {};
    size_t st[4], en[4];
    split_four(n, st, en);
    uint32_t lens[4];
    for (int i = 0; i < 4; ++i) {
        Bytes s;
        encode_stream(src + st[i], en[i] - st[i], t, s);
        if (out.size() + s.size() > dst_cap) return {};
        lens[i] = uint32_t(s.size());
        out.insert(out.end(), s.begin(), s.end());
    }
    if (out.size() >= n) return {};  // NotBeneficial (compress.rs:72-75)
    for (int i = 0; i < 4; ++i) put_u32le(&out[jump_pos + 4 * i], lens[i]);
    return out;
}

// bitstream.rs:54-187 + decompress.rs:8-211.  The reference interleaves a
// fast loop and a checked tail; for every stream they accept the result
// equals this sequential form: peek max_bits (zero padded past the stream
// start), look up, require nbits <= remaining bits, consume.  Afterwards
// every stream must have no unread byte and only zero leftover bits
// (decompress.rs:140-144, bitstream.rs:184-186).
inline void decode_stream(const uint8_t* s, size_t slen, const Tree& t, uint8_t* out, size_t n) {
    uint64_t cont = 0; int cnt = 0;
    long idx = long(slen) - 1;
    const uint32_t mask = (1u << t.max_bits) - 1;
    for (size_t i = 0; i < n; ++i) {
        while (cnt <= 56 && idx >= 0) { cont |= uint64_t(s[idx]) << cnt; cnt += 8; --idx; }
        if (cnt == 0) throw Error("huffman: unexpected end of bitstream");
        uint16_t e = t.table[cont & mask];
        int nb = e >> 8;
        if (nb > cnt) throw Error("huffman: bitstream ended mid-symbol");
        cont >>= nb; cnt -= nb;
        out[i] = uint8_t(e & 0xFF);
    }
    while (cnt <= 56 && idx >= 0) { cont |= uint64_t(s[idx]) << cnt; cnt += 8; --idx; }
    if (idx >= 0 || cont != 0) throw Error("huffman: bitstream not fully consumed");
}

inline void decompress(uint8_t* dst, size_t n, const uint8_t* src, size_t len) {
    std::vector<uint8_t> w;
    size_t pos = decode_weights(src, len, w);
    uint8_t lengths[256] = {0};
    for (size_t i = 0; i < w.size(); ++i) {
        if (w[i] > MAX_TABLE_LOG) throw Error("huffman: invalid weight");
        lengths[i] = w[i];
    }
    Tree t;
    if (!from_lengths(lengths, t)) throw Error("huffman: invalid weight table");
    if (len - pos < JUMP_TABLE_BYTES) throw Error("huffman: truncated jump table");
    uint64_t lens[4], total = 0;
    for (int i = 0; i < 4; ++i) { lens[i] = get_u32le(src + pos + 4 * i); total += lens[i]; }
    pos += JUMP_TABLE_BYTES;
    if (total != len - pos) throw Error("huffman: jump table sum does not match payload tail");
    size_t st[4], en[4];
    split_four(n, st, en);
    size_t off = pos;
    for (int i = 0; i < 4; ++i) {
        decode_stream(src + off, size_t(lens[i]), t, dst + st[i], en[i] - st[i]);
        off += size_t(lens[i]);
    }
}

}  // namespace huffman

// ---------------------------------------------------------------------------
// rANS (entropy/rans/)
// ---------------------------------------------------------------------------
namespace rans {

constexpr uint32_t PROB_BITS = 11, PROB_SCALE = 1u << PROB_BITS, PROB_MASK = PROB_SCALE - 1;
constexpr uint32_t RANS_L = 1u << 23;

// compress.rs:72-122 — floor scaling with min 1, the excess/deficit goes to
// the first most-frequent symbol.  Returns false for "Incompressible".
inline bool normalize_freqs(const uint32_t raw[256], uint16_t freqs[256], uint16_t cum[256]) {
    uint64_t total = 0;
    for (int i = 0; i < 256; ++i) total += raw[i];
    if (total == 0) return false;
    std::memset(freqs, 0, 512);
    std::memset(cum, 0, 512);
    uint32_t assigned = 0;
    int max_sym = 0, max_freq_sym = 0;
    for (int i = 0; i < 256; ++i) {
        if (raw[i] > 0) {
            uint64_t f = uint64_t(raw[i]) * PROB_SCALE / total;
            if (f < 1) f = 1;
            freqs[i] = uint16_t(f);
            assigned += uint32_t(f);
            max_sym = i;
            if (raw[i] > raw[max_freq_sym]) max_freq_sym = i;
        }
    }
    if (assigned > PROB_SCALE) {
        uint32_t excess = assigned - PROB_SCALE;
        if (freqs[max_freq_sym] > excess) freqs[max_freq_sym] = uint16_t(freqs[max_freq_sym] - excess);
        else return false;
    } else if (assigned < PROB_SCALE) {
        freqs[max_freq_sym] = uint16_t(freqs[max_freq_sym] + (PROB_SCALE - assigned));
    }
    uint32_t running = 0;
    for (int i = 0; i <= max_sym; ++i) { cum[i] = uint16_t(running); running += freqs[i]; }
    return true;
}

// compress.rs:140-185 — encode backward from x = L; emit low bytes while
// x >= ((L>>11)<<8)*freq; stream = final state LE then the bytes reversed.
// The reference's reciprocal multiply equals the div/mod form used here
// (compress.rs:166-176 asserts the identity).
inline void encode_stream(const uint8_t* src, size_t n, const uint16_t freqs[256], const uint16_t cum[256], Bytes& out) {
    Bytes rev;
    rev.reserve(n + 8);
    uint32_t x = RANS_L;
    for (size_t k = n; k-- > 0;) {
        uint32_t f = freqs[src[k]], c = cum[src[k]];
        uint32_t max_state = ((RANS_L >> PROB_BITS) << 8) * f;
        while (x >= max_state) { rev.push_back(uint8_t(x)); x >>= 8; }
        x = (x / f) * PROB_SCALE + (x % f) + c;
    }
    out.resize(4);
    put_u32le(out.data(), x);
    out.insert(out.end(), rev.rbegin(), rev.rend());
}

// compress.rs:187-259
inline Bytes compress(const uint8_t* src, size_t n) {
    if (n == 0) return {};
    uint32_t raw[256] = {0};
    for (size_t i = 0; i < n; ++i) raw[src[i]]++;
    uint16_t freqs[256], cum[256];
    if (!normalize_freqs(raw, freqs, cum)) return {};
    int max_sym = 0;
    for (int i = 255; i >= 0; --i) if (freqs[i] > 0) { max_sym = i; break; }
    Bytes out;
    out.push_back(uint8_t(max_sym));
    for (int i = 0; i <= max_sym; ++i) { out.push_back(uint8_t(freqs[i])); out.push_back(uint8_t(freqs[i] >> 8)); }
    size_t jump_pos = out.size();
    out.resize(out.size() + JUMP_TABLE_BYTES, 0);
    const size_t dst_cap = n * 2 + 4096;  // codec_tagged.rs:168-172
    if (out.size() >= dst_cap) return {};
    size_t st[4], en[4];
    split_four(n, st, en);
    uint32_t lens[4];
    for (int i = 0; i < 4; ++i) {
        Bytes s;
        encode_stream(src + st[i], en[i] - st[i], freqs, cum, s);
        if (out.size() + s.size() > dst_cap) return {};
        lens[i] = uint32_t(s.size());
        out.insert(out.end(), s.begin(), s.end());
    }
    if (out.size() >= n) return {};
    for (int i = 0; i < 4; ++i) put_u32le(&out[jump_pos + 4 * i], lens[i]);
    return out;
}

// decompress.rs:24-164.  The final state is not checked (decompress.rs:80-111).
inline void decompress(uint8_t* dst, size_t n, const uint8_t* src, size_t len) {
    if (len == 0) throw Error("rans: empty input");
    size_t max_sym = src[0];
    size_t needed = 1 + 2 * (max_sym + 1);
    if (len < needed) throw Error("rans: truncated frequency table");
    uint16_t freqs[256] = {0};
    uint32_t total = 0;
    for (size_t i = 0; i <= max_sym; ++i) { freqs[i] = uint16_t(src[1 + 2 * i] | (src[2 + 2 * i] << 8)); total += freqs[i]; }
    if (total != PROB_SCALE) throw Error("rans: frequency table does not sum to 2048");
    size_t pos = needed;
    if (len - pos < JUMP_TABLE_BYTES) throw Error("rans: truncated jump table");
    uint64_t lens[4], tot = 0;
    for (int i = 0; i < 4; ++i) { lens[i] = get_u32le(src + pos + 4 * i); tot += lens[i]; }
    pos += JUMP_TABLE_BYTES;
    if (tot != len - pos) throw Error("rans: jump table sum does not match payload tail");
    struct Entry { uint8_t sym; uint16_t freq, start; };
    std::vector<Entry> table(PROB_SCALE);
    uint32_t p = 0;
    for (int s = 0; s < 256; ++s) {
        for (uint32_t j = 0; j < freqs[s]; ++j) table[p + j] = Entry{uint8_t(s), freqs[s], uint16_t(p)};
        p += freqs[s];
    }
    size_t st[4], en[4];
    split_four(n, st, en);
    size_t off = pos;
    for (int i = 0; i < 4; ++i) {
        const uint8_t* s = src + off;
        size_t slen = size_t(lens[i]);
        off += slen;
        if (st[i] == en[i]) continue;
        if (slen < 4) throw Error("rans: stream too short for initial state");
        uint32_t x = get_u32le(s);
        size_t sp = 4;
        for (size_t k = st[i]; k < en[i]; ++k) {
            uint32_t idx = x & PROB_MASK;
            const Entry& e = table[idx];
            dst[k] = e.sym;
            x = uint32_t(e.freq) * (x >> PROB_BITS) + idx - e.start;
            while (x < RANS_L) {
                if (sp >= slen) throw Error("rans: unexpected end of stream during renormalization");
                x = (x << 8) | s[sp++];
            }
        }
    }
}

}  // namespace rans

// ---------------------------------------------------------------------------
// tANS (entropy/tans/mod.rs)
// ---------------------------------------------------------------------------
namespace tans {

constexpr uint32_t TABLE_LOG = 11;
constexpr uint32_t L = 1u << TABLE_LOG;

inline uint32_t highbit(uint32_t x) { return 31 - uint32_t(__builtin_clz(x)); }

// mod.rs:153-194
inline void normalize(const uint32_t counts[256], uint64_t total, uint32_t norm[256]) {
    std::memset(norm, 0, 1024);
    uint32_t sum = 0, max_count = 0; int max_sym = 0;
    for (int s = 0; s < 256; ++s) {
        uint32_t c = counts[s];
        if (c == 0) continue;
        uint32_t v = uint32_t(uint64_t(c) * L / total);
        if (v == 0) v = 1;
        norm[s] = v; sum += v;
        if (c > max_count) { max_count = c; max_sym = s; }
    }
    while (sum > L) {
        int bi = -1; uint32_t bv = 1;
        for (int s = 0; s < 256; ++s) if (norm[s] > bv) { bv = norm[s]; bi = s; }
        norm[bi]--; sum--;
    }
    while (sum < L) { norm[max_sym]++; sum++; }
}

// mod.rs:199-211
inline void spread(const uint32_t norm[256], uint8_t table[L]) {
    const uint32_t step = (L >> 1) + (L >> 3) + 3, mask = L - 1;
    uint32_t pos = 0;
    for (int s = 0; s < 256; ++s)
        for (uint32_t k = 0; k < norm[s]; ++k) { table[pos] = uint8_t(s); pos = (pos + step) & mask; }
}

// mod.rs:268-339 — returns the blob or empty for "store raw".
inline Bytes compress(const uint8_t* src, size_t n, size_t dst_cap) {
    if (n == 0) return {};
    uint32_t counts[256] = {0};
    for (size_t i = 0; i < n; ++i) counts[src[i]]++;
    size_t nsym = 0;
    for (int s = 0; s < 256; ++s) nsym += counts[s] != 0;
    if (nsym < 2) return {};
    uint32_t norm[256];
    normalize(counts, n, norm);
    std::vector<uint8_t> sym(L);
    spread(norm, sym.data());
    // build_encode (mod.rs:225-266)
    uint32_t cumul[256], fill[256], running = 0;
    for (int s = 0; s < 256; ++s) { cumul[s] = running; running += norm[s]; }
    std::memcpy(fill, cumul, sizeof fill);
    std::vector<uint16_t> state_table(L);
    for (uint32_t u = 0; u < L; ++u) { int s = sym[u]; state_table[fill[s]++] = uint16_t(L + u); }
    uint32_t dnb[256] = {0}; int32_t dfs[256] = {0};
    int32_t tot = 0;
    for (int s = 0; s < 256; ++s) {
        uint32_t c = norm[s];
        if (c == 0) continue;
        if (c == 1) { dnb[s] = (TABLE_LOG << 16) - L; dfs[s] = tot - 1; tot += 1; }
        else {
            uint32_t max_bits = TABLE_LOG - highbit(c - 1);
            uint32_t min_state_plus = c << max_bits;
            dnb[s] = (max_bits << 16) - min_state_plus;
            dfs[s] = tot - int32_t(c);
            tot += int32_t(c);
        }
    }
    Bytes bits; bits.reserve(n);
    uint64_t acc = 0; uint32_t nb_acc = 0; uint64_t total_bits = 0;
    auto add_bits = [&](uint64_t value, uint32_t nb) {
        if (nb == 0) return;
        acc |= (value & ((uint64_t(1) << nb) - 1)) << nb_acc;
        nb_acc += nb; total_bits += nb;
        while (nb_acc >= 8) { bits.push_back(uint8_t(acc)); acc >>= 8; nb_acc -= 8; }
    };
    uint32_t value = L;
    for (size_t k = n; k-- > 0;) {
        int b = src[k];
        uint32_t nb = (value + dnb[b]) >> 16;
        add_bits(value, nb);
        int32_t idx = int32_t(value >> nb) + dfs[b];
        value = state_table[size_t(idx)];
    }
    add_bits(value, TABLE_LOG);
    if (nb_acc > 0) bits.push_back(uint8_t(acc));
    size_t header_len = 1 + 2 + nsym * 3 + 8;
    size_t blob_len = header_len + bits.size();
    if (blob_len >= n || blob_len > dst_cap) return {};
    Bytes out;
    out.reserve(blob_len);
    out.push_back(uint8_t(TABLE_LOG));
    out.push_back(uint8_t(nsym)); out.push_back(uint8_t(nsym >> 8));
    for (int s = 0; s < 256; ++s) {
        if (norm[s] == 0) continue;
        out.push_back(uint8_t(s)); out.push_back(uint8_t(norm[s])); out.push_back(uint8_t(norm[s] >> 8));
    }
    for (int i = 0; i < 8; ++i) out.push_back(uint8_t(total_bits >> (8 * i)));
    out.insert(out.end(), bits.begin(), bits.end());
    return out;
}

// mod.rs:372-451
inline void decompress(uint8_t* dst, size_t n, const uint8_t* src, size_t len) {
    if (n == 0) return;
    if (len < 3) throw Error("tans: blob too short for header");
    if (src[0] != TABLE_LOG) throw Error("tans: unsupported table_log");
    size_t nsym = size_t(src[1]) | size_t(src[2]) << 8;
    if (nsym < 2 || nsym > 256) throw Error("tans: bad symbol count");
    size_t pos = 3, pairs_end = pos + nsym * 3;
    if (pairs_end + 8 > len) throw Error("tans: truncated frequency table");
    uint32_t norm[256] = {0}, sum = 0;
    for (size_t i = 0; i < nsym; ++i) {
        int s = src[pos];
        uint32_t f = uint32_t(src[pos + 1]) | uint32_t(src[pos + 2]) << 8;
        if (norm[s] != 0) throw Error("tans: duplicate symbol in frequency table");
        if (f == 0) throw Error("tans: zero frequency in table");
        norm[s] = f; sum += f; pos += 3;
    }
    if (sum != L) throw Error("tans: frequencies do not sum to table size");
    uint64_t total_bits = get_u64le(src + pos);
    pos += 8;
    const uint8_t* bs = src + pos;
    size_t bslen = len - pos;
    if (total_bits > uint64_t(bslen) * 8) throw Error("tans: bitstream shorter than declared bit length");
    std::vector<uint8_t> sym(L);
    spread(norm, sym.data());
    struct DE { uint8_t symbol, nb; uint16_t baseline; };
    std::vector<DE> dt(L);
    uint32_t next[256];
    std::memcpy(next, norm, sizeof next);
    for (uint32_t u = 0; u < L; ++u) {
        int s = sym[u];
        uint32_t x = next[s]++;
        uint32_t nb = TABLE_LOG - highbit(x);
        dt[u] = DE{uint8_t(s), uint8_t(nb), uint16_t((x << nb) - L)};
    }
    uint64_t bpos = total_bits;
    auto read = [&](uint32_t nb) -> uint32_t {
        if (nb == 0) return 0;
        if (bpos < nb) throw Error("tans: bitstream underrun");
        uint64_t start = bpos - nb;
        size_t bi = size_t(start >> 3);
        uint32_t bo = uint32_t(start & 7);
        uint32_t window = bs[bi];
        if (bi + 1 < bslen) window |= uint32_t(bs[bi + 1]) << 8;
        if (bi + 2 < bslen) window |= uint32_t(bs[bi + 2]) << 16;
        bpos = start;
        return (window >> bo) & ((1u << nb) - 1);
    };
    uint32_t state = read(TABLE_LOG);
    if (state >= L) throw Error("tans: initial state out of range");
    for (size_t i = 0; i < n; ++i) {
        const DE& e = dt[state];
        dst[i] = e.symbol;
        state = uint32_t(e.baseline) + read(e.nb);
        if (state >= L) throw Error("tans: state out of range");
    }
    if (bpos != 0) throw Error("tans: trailing bits after decode");
    if (state != 0) throw Error("tans: decode did not return to start state");
}

}  // namespace tans

}  // namespace oracle
