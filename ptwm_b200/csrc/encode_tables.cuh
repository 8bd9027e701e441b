// Code/table construction of the encoders, usable from host and device code.
// They must make the same choices as the reference's encoders so that the
// bytes written equal what ptwm-core would write for the same plane:
//   rANS     entropy/rans/compress.rs:72-122 (normalize_freqs)
//   Huffman  entropy/huffman/tree.rs:19-85 (from_frequencies), :212-242
//            (enforce_max_code_length), :119-141 (canonical codes)
//   tANS     entropy/tans/mod.rs:153-194 (normalize)
//   O1SAC    quantize.rs:13-45 (quantize_pmf)
#pragma once
#include <math.h>
#include <stdint.h>

namespace ptwm {

// Normalised rANS frequencies (sum 2048, every present symbol >= 1; the
// rounding excess or deficit goes to the first most frequent symbol).
// Returns max_sym, or -1 when the plane must be stored raw.
__host__ __device__ inline int rans_normalize(const uint32_t* raw, uint64_t total, uint16_t* freqs) {
    if (total == 0) return -1;
    uint32_t assigned = 0;
    int max_sym = 0, max_freq_sym = 0;
    for (int i = 0; i < 256; ++i) {
        freqs[i] = 0;
        if (raw[i] > 0) {
            uint64_t f = uint64_t(raw[i]) * 2048u / total;
            if (f < 1) f = 1;
            freqs[i] = uint16_t(f);
            assigned += uint32_t(f);
            max_sym = i;
            if (raw[i] > raw[max_freq_sym]) max_freq_sym = i;
        }
    }
    if (assigned > 2048) {
        uint32_t excess = assigned - 2048;
        if (freqs[max_freq_sym] > excess) freqs[max_freq_sym] = uint16_t(freqs[max_freq_sym] - excess);
        else return -1;
    } else if (assigned < 2048) {
        freqs[max_freq_sym] = uint16_t(freqs[max_freq_sym] + (2048 - assigned));
    }
    return max_sym;
}

// Normalised tANS frequencies (sum 2048): floor(c * 2048 / total) with a floor
// of one; an excess is taken one at a time from the first largest entry above
// one, a deficit goes to the first most frequent symbol.  Returns the number
// of present symbols.
__host__ __device__ inline int tans_normalize(const uint32_t* counts, uint64_t total, uint16_t* norm) {
    uint32_t sum = 0, max_count = 0;
    int max_sym = 0, nsym = 0;
    for (int s = 0; s < 256; ++s) {
        norm[s] = 0;
        const uint32_t c = counts[s];
        if (c == 0) continue;
        uint32_t v = uint32_t(uint64_t(c) * 2048u / total);
        if (v == 0) v = 1;
        norm[s] = uint16_t(v); sum += v; ++nsym;
        if (c > max_count) { max_count = c; max_sym = s; }
    }
    while (sum > 2048) {
        int bi = -1; uint32_t bv = 1;
        for (int s = 0; s < 256; ++s) if (norm[s] > bv) { bv = norm[s]; bi = s; }
        if (bi < 0) break;
        norm[bi]--; sum--;
    }
    if (sum < 2048) norm[max_sym] = uint16_t(norm[max_sym] + (2048 - sum));
    return nsym;
}

// Probability row of the Order1ScaleAC state from raw counts: Laplace +1,
// scaled to `total` and rounded half away from zero in double precision, at
// least one each; then the last largest entry is shaved, or the first smallest
// grown, until the row sums to `total`.
__host__ __device__ inline void quantize_pmf256(const uint32_t* raw, uint32_t total, uint16_t* out) {
    double sum = 0;
    for (int i = 0; i < 256; ++i) sum += double(raw[i] + 1);
    uint32_t current = 0;
    for (int i = 0; i < 256; ++i) {
        double v = round((double(raw[i] + 1) / sum) * double(total));
        if (v < 1.0) v = 1.0;
        out[i] = uint16_t(v);
        current += out[i];
    }
    while (current > total) {
        int am = 0;
        for (int i = 0; i < 256; ++i) if (out[i] >= out[am]) am = i;
        if (out[am] > 1) { out[am]--; current--; } else break;
    }
    while (current < total) {
        int am = 0;
        for (int i = 0; i < 256; ++i) if (out[i] < out[am]) am = i;
        out[am]++; current++;
    }
}

// Huffman code lengths for a histogram: repeated merge of the two smallest
// nodes under the (frequency, node id) order, leaves numbered in symbol order
// and internal nodes after them; depth clamp to 11 with the reference's Kraft
// repair.  Returns the number of weights to store (last used symbol + 1), or
// 0 when there is no symbol.  Work arrays are caller provided so device code
// can keep them in local memory: nf[512], parent[512] (uint16), alive[512].
template <class Count>
__host__ __device__ inline int huffman_lengths(const Count* raw, uint8_t* lengths, Count* nf, uint16_t* parent, uint8_t* alive, uint8_t* sym_of) {
    int n = 0;
    for (int i = 0; i < 256; ++i) { lengths[i] = 0; if (raw[i] > 0) { nf[n] = raw[i]; sym_of[n] = uint8_t(i); alive[n] = 1; ++n; } }
    if (n == 0) return 0;
    int last = sym_of[n - 1];
    if (n == 1) { lengths[sym_of[0]] = 1; return last + 1; }
    int next = n;
    for (int merges = 0; merges < n - 1; ++merges) {
        int a = -1, b = -1;  // a = smallest, b = second smallest under (freq, id)
        for (int i = 0; i < next; ++i) {
            if (!alive[i]) continue;
            if (a < 0 || nf[i] < nf[a]) { b = a; a = i; }
            else if (b < 0 || nf[i] < nf[b]) b = i;
        }
        alive[a] = 0; alive[b] = 0;
        nf[next] = nf[a] + nf[b];
        parent[a] = uint16_t(next); parent[b] = uint16_t(next);
        alive[next] = 1;
        ++next;
    }
    // depth of a leaf = number of ancestors; parents always have larger ids
    // reuse nf[] of internal nodes as their depth, walking from the root down
    const int root = next - 1;
    nf[root] = 0;
    for (int i = root - 1; i >= n; --i) nf[i] = nf[parent[i]] + 1;
    bool clamped = false;
    for (int i = 0; i < n; ++i) {
        uint32_t d = uint32_t(nf[parent[i]]) + 1;
        if (d > 11) { d = 11; clamped = true; }
        lengths[sym_of[i]] = uint8_t(d);
    }
    if (clamped) {
        for (;;) {
            uint32_t kraft = 0;
            for (int s = 0; s < 256; ++s) if (lengths[s]) kraft += 1u << (11 - lengths[s]);
            if (kraft <= 2048) break;
            int victim = -1;
            for (int s = 0; s < 256; ++s) if (lengths[s] > 0 && lengths[s] < 11 && (victim < 0 || lengths[s] < lengths[victim])) victim = s;
            if (victim < 0) break;
            lengths[victim]++;
        }
    }
    return last + 1;
}

// Canonical codes, bit-reversed for the LSB-first stream (tree.rs:119-170).
__host__ __device__ inline void huffman_codes(const uint8_t* lengths, uint16_t* rev_codes) {
    uint32_t counts[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}, next_code[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < 256; ++s) if (lengths[s]) counts[lengths[s]]++;
    uint32_t code = 0;
    for (int bits = 1; bits < 12; ++bits) { code = (code + counts[bits - 1]) << 1; next_code[bits] = code; }
    for (int s = 0; s < 256; ++s) {
        int len = lengths[s];
        rev_codes[s] = 0;
        if (!len) continue;
        uint32_t c = next_code[len]++;
        uint32_t r = 0;
        for (int k = 0; k < len; ++k) { r = (r << 1) | (c & 1); c >>= 1; }
        rev_codes[s] = uint16_t(r);
    }
}

}  // namespace ptwm
