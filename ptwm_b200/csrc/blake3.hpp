// BLAKE3 (unkeyed hash, 32-byte output), written from the published
// specification: the legacy container layout commits to its Extension Table
// with it (crates/ptwm-core/src/extension/table.rs:136-141, checked at
// container.rs:1299-1301) and built-in entries carry ids derived with it
// (crates/ptwm-core/src/extension/id.rs:21-31).  Host code for inputs of a few
// kilobytes: one thread, no SIMD.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace ptwm {
namespace blake3_detail {

constexpr uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au, 0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
constexpr uint8_t PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
enum : uint32_t { CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8 };
constexpr size_t BLOCK = 64, CHUNK = 1024;

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
inline void g(uint32_t* s, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
    s[a] = s[a] + s[b] + mx; s[d] = rotr(s[d] ^ s[a], 16);
    s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 12);
    s[a] = s[a] + s[b] + my; s[d] = rotr(s[d] ^ s[a], 8);
    s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 7);
}
// The compression function; `out` receives the new chaining value (the first eight words of the output).
inline void compress(const uint32_t cv[8], const uint32_t block[16], uint64_t counter, uint32_t block_len, uint32_t flags, uint32_t out[8]) {
    uint32_t s[16], m[16];
    for (int i = 0; i < 8; ++i) s[i] = cv[i];
    for (int i = 0; i < 4; ++i) s[8 + i] = IV[i];
    s[12] = uint32_t(counter); s[13] = uint32_t(counter >> 32); s[14] = block_len; s[15] = flags;
    for (int i = 0; i < 16; ++i) m[i] = block[i];
    for (int round = 0; round < 7; ++round) {
        g(s, 0, 4, 8, 12, m[0], m[1]);   g(s, 1, 5, 9, 13, m[2], m[3]);
        g(s, 2, 6, 10, 14, m[4], m[5]);  g(s, 3, 7, 11, 15, m[6], m[7]);
        g(s, 0, 5, 10, 15, m[8], m[9]);  g(s, 1, 6, 11, 12, m[10], m[11]);
        g(s, 2, 7, 8, 13, m[12], m[13]); g(s, 3, 4, 9, 14, m[14], m[15]);
        uint32_t p[16];
        for (int i = 0; i < 16; ++i) p[i] = m[PERM[i]];
        for (int i = 0; i < 16; ++i) m[i] = p[i];
    }
    for (int i = 0; i < 8; ++i) out[i] = s[i] ^ s[i + 8];
}
inline void load_block(const uint8_t* p, size_t n, uint32_t w[16]) {
    uint8_t b[BLOCK] = {0};
    std::memcpy(b, p, n);
    for (int i = 0; i < 16; ++i) w[i] = uint32_t(b[4 * i]) | uint32_t(b[4 * i + 1]) << 8 | uint32_t(b[4 * i + 2]) << 16 | uint32_t(b[4 * i + 3]) << 24;
}
// Chaining value of one chunk (at most 1024 bytes; an empty input is one empty block).
inline void chunk_cv(const uint8_t* p, size_t n, uint64_t chunk_index, bool root, uint32_t out[8]) {
    uint32_t cv[8];
    for (int i = 0; i < 8; ++i) cv[i] = IV[i];
    const size_t blocks = n ? (n + BLOCK - 1) / BLOCK : 1;
    for (size_t b = 0; b < blocks; ++b) {
        const size_t len = b + 1 < blocks ? BLOCK : n - b * BLOCK;
        uint32_t w[16];
        load_block(p + b * BLOCK, len, w);
        uint32_t flags = (b == 0 ? CHUNK_START : 0) | (b + 1 == blocks ? CHUNK_END | (root ? ROOT : 0) : 0);
        compress(cv, w, chunk_index, uint32_t(len), flags, cv);
    }
    for (int i = 0; i < 8; ++i) out[i] = cv[i];
}
// Chaining value of the subtree over p[0, n): the left child takes the largest power-of-two number of chunks that leaves
// at least one byte for the right child.
inline void subtree_cv(const uint8_t* p, size_t n, uint64_t first_chunk, bool root, uint32_t out[8]) {
    if (n <= CHUNK) { chunk_cv(p, n, first_chunk, root, out); return; }
    size_t left = CHUNK;
    while (left * 2 < n) left *= 2;
    uint32_t w[16];
    subtree_cv(p, left, first_chunk, false, w);
    subtree_cv(p + left, n - left, first_chunk + left / CHUNK, false, w + 8);
    compress(IV, w, 0, uint32_t(BLOCK), PARENT | (root ? ROOT : 0), out);
}

}  // namespace blake3_detail

inline void blake3_hash(const uint8_t* p, size_t n, uint8_t out[32]) {
    uint32_t cv[8];
    blake3_detail::subtree_cv(p, n, 0, true, cv);
    for (int i = 0; i < 8; ++i) for (int k = 0; k < 4; ++k) out[4 * i + k] = uint8_t(cv[i] >> (8 * k));
}

}  // namespace ptwm
