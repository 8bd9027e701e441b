// Device code of the encode path: forward bit reorder + plane split, per-chunk
// histograms, per-chunk table build, per-stream rANS / Huffman encoding and
// the gather that lays chunk frames out in the container.
//
// Byte-exact targets under crates/ptwm-core/src of the reference:
//   split      transforms/fusion.rs:35-122,207-262,329-371,431-473
//   rANS       entropy/rans/compress.rs:35-259
//   Huffman    entropy/huffman/{compress.rs:9-103, bitstream.rs:3-51, weights.rs:8-32}
//   framing    compressor.rs:316-381, codecs/{huffman,rans}.rs encode
#pragma once
#include "encode_tables.cuh"
#include "kernels.cuh"

namespace ptwm {

struct SplitItem {
    const uint8_t* src;  // raw tensor bytes (device)
    uint64_t plane_off[4];  // where each plane starts in the planes buffer
    uint64_t n;          // elements (= bytes per plane)
    uint32_t kind;
    uint32_t first_tile;
};
constexpr uint32_t SPLIT_TILE = 8192;

struct EncChunk {
    uint64_t plane_off;  // this chunk's bytes in the planes buffer
    uint64_t slot_off;   // four stream slots of slot_cap bytes each in the slot buffer
    uint32_t n;
    uint32_t slot_cap;
    uint32_t plane;      // global plane index
    uint32_t pad;
};
struct EncResult {       // per chunk, read back by the host
    uint32_t stream_len[4];
    uint32_t hdr_n;      // rANS: max_sym; Huffman: number of weights
    uint32_t coded;      // 0: no table could be built, store raw
};
struct GatherItem {
    uint64_t dst;        // absolute offset of the chunk frame in the container
    uint32_t chunk;
    uint32_t mode;       // 0 identity (bare bytes), 1 raw-tagged, 2 rANS, 3 Huffman; + GATHER_BARE: the payload alone, no chunk frame header
};
constexpr uint32_t GATHER_BARE = 0x100;

// layout of the 1 KiB table area per chunk
//   rANS:    freqs u16[256] | cum u16[256]
//   Huffman: lengths u8[256] | unused[256] | rev codes u16[256]
constexpr uint32_t ENC_TABLE_BYTES = 1024;

__global__ void __launch_bounds__(256) split_kernel(const SplitItem* __restrict__ items, uint32_t n_items, uint8_t* __restrict__ planes) {
    uint32_t tile = blockIdx.x;
    uint32_t lo = 0, hi = n_items;
    while (lo + 1 < hi) { uint32_t mid = (lo + hi) >> 1; if (items[mid].first_tile <= tile) lo = mid; else hi = mid; }
    const SplitItem it = items[lo];
    uint64_t base = uint64_t(tile - it.first_tile) * SPLIT_TILE;
    uint32_t n = it.n - base < SPLIT_TILE ? uint32_t(it.n - base) : SPLIT_TILE;
    const int eb = kind_elem_bytes(int(it.kind));
    const uint8_t* src = it.src + base * uint64_t(eb);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        switch (it.kind) {
            case K_PASS: planes[it.plane_off[0] + base + i] = src[i]; break;
            case K_M16: {
                uint32_t v = uint32_t(src[2 * i]) | uint32_t(src[2 * i + 1]) << 8;
                uint32_t r = ((v << 1) & 0xFF00u) | ((v >> 8) & 0x0080u) | (v & 0x007Fu);
                planes[it.plane_off[0] + base + i] = uint8_t(r);
                planes[it.plane_off[1] + base + i] = uint8_t(r >> 8);
                break;
            }
            case K_M32: {
                uint32_t v = ld_u32_unaligned(src + 4 * i);
                uint32_t r = ((v << 1) & 0xFF000000u) | ((v >> 8) & 0x00800000u) | (v & 0x007FFFFFu);
#pragma unroll
                for (int p = 0; p < 4; ++p) planes[it.plane_off[p] + base + i] = uint8_t(r >> (8 * p));
                break;
            }
            default: {
                uint32_t v = src[i];
                uint32_t r = it.kind == K_E4M3 ? (((v & 0x78) << 1) | ((v & 0x80) >> 4) | (v & 0x07)) : (((v & 0x7C) << 1) | ((v & 0x80) >> 5) | (v & 0x03));
                planes[it.plane_off[0] + base + i] = uint8_t(r >> 4);
                planes[it.plane_off[1] + base + i] = uint8_t(r & 0x0F);
                break;
            }
        }
    }
}

// One CTA of 128 threads per chunk: shared-memory histogram, then the chunk's
// counts go to global memory and are added to the plane's totals.
__global__ void __launch_bounds__(128) hist_kernel(const EncChunk* __restrict__ chunks, const uint8_t* __restrict__ planes, uint32_t* __restrict__ hist,
                                                   unsigned long long* __restrict__ plane_hist) {
    __shared__ uint32_t h[256];
    const EncChunk c = chunks[blockIdx.x];
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) h[i] = 0;
    __syncthreads();
    const uint8_t* p = planes + c.plane_off;
    for (uint32_t i = threadIdx.x; i < c.n; i += blockDim.x) atomicAdd(&h[p[i]], 1u);
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) {
        hist[uint64_t(blockIdx.x) * 256 + i] = h[i];
        if (h[i]) atomicAdd(&plane_hist[uint64_t(c.plane) * 256 + i], (unsigned long long)h[i]);
    }
}

// One thread per chunk builds the chunk's table for the codec its plane uses.
__global__ void __launch_bounds__(64) table_kernel(const EncChunk* __restrict__ chunks, uint32_t n_chunks, const uint8_t* __restrict__ plane_codec,
                                                   const uint32_t* __restrict__ hist, uint8_t* __restrict__ tables, EncResult* __restrict__ results) {
    uint32_t ci = blockIdx.x * blockDim.x + threadIdx.x;
    if (ci >= n_chunks) return;
    const EncChunk c = chunks[ci];
    const uint32_t* raw = hist + uint64_t(ci) * 256;
    uint8_t* tab = tables + uint64_t(ci) * ENC_TABLE_BYTES;
    EncResult r{{0, 0, 0, 0}, 0, 0};
    int codec = plane_codec[c.plane];
    if (codec == C_RANS && c.n) {
        uint16_t* freqs = reinterpret_cast<uint16_t*>(tab);
        uint16_t* cum = freqs + 256;
        int ms = rans_normalize(raw, c.n, freqs);
        if (ms >= 0) {
            uint32_t run = 0;
            for (int i = 0; i < 256; ++i) { cum[i] = uint16_t(run); run += freqs[i]; }
            r.hdr_n = uint32_t(ms); r.coded = 1;
        }
    } else if (codec == C_HUFFMAN && c.n) {
        uint32_t nf[512]; uint16_t parent[512]; uint8_t alive[512]; uint8_t sym_of[256];
        uint8_t* lengths = tab;
        int nw = huffman_lengths<uint32_t>(raw, lengths, nf, parent, alive, sym_of);
        if (nw > 0) {
            huffman_codes(lengths, reinterpret_cast<uint16_t*>(tab + 512));
            r.hdr_n = uint32_t(nw); r.coded = 1;
        }
    }
    results[ci] = r;
}

// One thread per stream.  Bytes are produced last-to-first for both codecs, so
// each stream is written downward from the end of its slot and ends up in
// decode order; stream_len tells the gather where it starts.
__global__ void __launch_bounds__(128) encode_kernel(const EncChunk* __restrict__ chunks, uint32_t n_chunks, const uint8_t* __restrict__ plane_codec,
                                                     const uint8_t* __restrict__ planes, const uint8_t* __restrict__ tables, uint8_t* __restrict__ slots,
                                                     EncResult* __restrict__ results) {
    uint32_t gi = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t ci = gi >> 2, s = gi & 3;
    if (ci >= n_chunks) return;
    const EncChunk c = chunks[ci];
    if (!results[ci].coded) return;
    int codec = plane_codec[c.plane];
    uint32_t start, len;
    split_four_dev(c.n, s, start, len);
    const uint8_t* src = planes + c.plane_off + start;
    uint8_t* slot_end = slots + c.slot_off + uint64_t(s + 1) * c.slot_cap;
    uint8_t* w = slot_end;
    // Bytes go out downward.  Single byte stores to global memory are what this kernel used to wait for, so
    // once the write position is 8-byte aligned eight bytes are collected (the first produced ends up highest,
    // as in memory) and stored as one word.
    uint64_t acc = 0;
    uint32_t have = 0;
    auto put = [&](uint32_t b) {
        if (have == 0 && (reinterpret_cast<uintptr_t>(w) & 7)) { *--w = uint8_t(b); return; }
        acc = (acc << 8) | (b & 0xFFu);
        if (++have == 8) { w -= 8; *reinterpret_cast<uint64_t*>(w) = acc; have = 0; acc = 0; }
    };
    auto flush = [&]() { while (have) { --have; *--w = uint8_t(acc >> (8 * have)); } };
    const uint8_t* tab = tables + uint64_t(ci) * ENC_TABLE_BYTES;
    if (codec == C_RANS) {
        const uint16_t* freqs = reinterpret_cast<const uint16_t*>(tab);
        const uint16_t* cum = freqs + 256;
        uint32_t x = 1u << 23;
        for (uint32_t k = len; k-- > 0;) {
            uint32_t sym = src[k];
            uint32_t f = freqs[sym], cs = cum[sym];
            uint32_t max_state = ((1u << 12) << 8) * f;  // ((L >> 11) << 8) * freq
            while (x >= max_state) { put(x); x >>= 8; }
            x = (x / f) * 2048u + (x % f) + cs;
        }
        put(x >> 24); put(x >> 16); put(x >> 8); put(x);  // the final state, little-endian, below the renormalisation bytes
    } else {
        const uint8_t* lengths = tab;
        const uint16_t* rev = reinterpret_cast<const uint16_t*>(tab + 512);
        uint64_t bits = 0; uint32_t cnt = 0;
        for (uint32_t k = 0; k < len; ++k) {
            uint32_t sym = src[k];
            bits |= uint64_t(rev[sym]) << cnt;
            cnt += lengths[sym];
            while (cnt >= 8) { put(uint32_t(bits)); bits >>= 8; cnt -= 8; }
        }
        if (cnt) put(uint32_t(bits));
    }
    flush();
    results[ci].stream_len[s] = uint32_t(slot_end - w);
}

// One CTA per chunk frame: [state_version 0][state_len 0 u32] then the codec
// payload, written at its final place in the container.
__global__ void __launch_bounds__(128) gather_kernel(const GatherItem* __restrict__ items, const EncChunk* __restrict__ chunks, const EncResult* __restrict__ results,
                                                     const uint8_t* __restrict__ planes, const uint8_t* __restrict__ tables, const uint8_t* __restrict__ slots,
                                                     uint8_t* __restrict__ out) {
    const GatherItem g = items[blockIdx.x];
    const EncChunk c = chunks[g.chunk];
    const EncResult r = results[g.chunk];
    uint8_t* d = out + g.dst;
    const uint32_t t = threadIdx.x;
    const uint32_t mode = g.mode & 0xFFu;
    if (!(g.mode & GATHER_BARE)) {
        if (t < 5) d[t] = 0;
        d += 5;
    }
    if (mode <= 1) {
        if (mode == 1) { if (t == 0) d[0] = 0; d += 1; }
        const uint8_t* p = planes + c.plane_off;
        for (uint32_t i = t; i < c.n; i += blockDim.x) d[i] = p[i];
        return;
    }
    if (t == 0) { d[0] = 1; d[1] = uint8_t(c.n); d[2] = uint8_t(c.n >> 8); d[3] = uint8_t(c.n >> 16); d[4] = uint8_t(c.n >> 24); }
    d += 5;
    const uint8_t* tab = tables + uint64_t(g.chunk) * ENC_TABLE_BYTES;
    uint32_t hdr;
    if (mode == 2) {
        const uint16_t* freqs = reinterpret_cast<const uint16_t*>(tab);
        hdr = 1 + 2 * (r.hdr_n + 1);
        if (t == 0) d[0] = uint8_t(r.hdr_n);
        for (uint32_t i = t; i <= r.hdr_n; i += blockDim.x) { d[1 + 2 * i] = uint8_t(freqs[i]); d[2 + 2 * i] = uint8_t(freqs[i] >> 8); }
    } else {
        const uint32_t nw = r.hdr_n;
        uint32_t hb = nw <= 127 ? 1 : 2;
        hdr = hb + (nw + 1) / 2;
        if (t == 0) { if (nw <= 127) d[0] = uint8_t(0x80 | nw); else { d[0] = 0x80; d[1] = uint8_t(nw); } }
        for (uint32_t i = t; i < (nw + 1) / 2; i += blockDim.x) {
            uint32_t lo = tab[2 * i] & 0x0F, hi = (2 * i + 1 < nw ? tab[2 * i + 1] : 0) & 0x0F;
            d[hb + i] = uint8_t(lo | (hi << 4));
        }
    }
    d += hdr;
    if (t < 16) d[t] = uint8_t(r.stream_len[t >> 2] >> (8 * (t & 3)));
    d += 16;
    for (uint32_t s = 0; s < 4; ++s) {
        const uint8_t* sp = slots + c.slot_off + uint64_t(s + 1) * c.slot_cap - r.stream_len[s];
        for (uint32_t i = t; i < r.stream_len[s]; i += blockDim.x) d[i] = sp[i];
        d += r.stream_len[s];
    }
}

// Scatter host-built byte pieces (record headers, index, footer) into the container.
__global__ void __launch_bounds__(128) scatter_kernel(const uint8_t* __restrict__ staged, const uint64_t* __restrict__ triples, uint8_t* __restrict__ out) {
    uint64_t dst = triples[3 * blockIdx.x], src = triples[3 * blockIdx.x + 1], len = triples[3 * blockIdx.x + 2];
    for (uint64_t i = threadIdx.x; i < len; i += blockDim.x) out[dst + i] = staged[src + i];
}

}  // namespace ptwm
