// Device code of the encode path: forward bit reorder + plane split, per-chunk
// histograms, per-chunk table build, per-stream rANS / Huffman encoding and
// the gather that lays chunk frames out in the container.
//
// Byte-exact targets under crates/ptwm-core/src of the reference:
//   split      transforms/fusion.rs:35-122,207-262,329-371,431-473
//   rANS       entropy/rans/compress.rs:35-259
//   Huffman    entropy/huffman/{compress.rs:9-103, bitstream.rs:3-51, weights.rs:8-32}
//   tANS       entropy/tans/mod.rs:199-339
//   O1SAC      codecs/order1_scale_ac.rs:620-663,963-1025, quantize.rs:13-45, range_coder.rs:16-113
//   framing    compressor.rs:316-381, codecs/{huffman,rans,tans}.rs encode
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
    uint64_t slot_off;   // four stream slots of slot_cap bytes each in the slot buffer (tANS / O1SAC: one stream over all four)
    uint64_t table_off;  // this chunk's area in the table buffer (size by codec, see below)
    uint32_t n;
    uint32_t slot_cap;
    uint32_t plane;      // global plane index
    uint32_t row_len;    // O1SAC: symbols per row (context resets at row starts); 0 = one row spanning the chunk
};
struct EncResult {       // per chunk, read back by the host
    uint32_t stream_len[4];  // tANS: [0] bytes of bits, [1..2] total bits (lo, hi); O1SAC: [0] payload bytes, [1] state bytes
    uint32_t hdr_n;      // rANS: max_sym; Huffman: number of weights; tANS: present symbols; O1SAC: context rows
    uint32_t coded;      // 0: no table could be built, store raw
};
struct GatherItem {
    uint64_t dst;        // absolute offset of the chunk frame in the container
    uint32_t chunk;
    uint32_t mode;       // 0 identity (bare bytes), 1 raw-tagged, 2 rANS, 3 Huffman, 4 tANS, 5 Order1ScaleAC (state inside the frame);
                         // + GATHER_BARE: the payload alone, no chunk frame header (and no state)
};
constexpr uint32_t GATHER_BARE = 0x100;
constexpr uint32_t GATHER_NOFRAME = 0x200;  // an unchunked plane: inline state (if the codec has one) and payload, no frame header

// layout of the table area of a chunk
//   rANS:    freqs u16[256] | per symbol {reciprocal u32, bias u32, 2048 - freq u32, reciprocal shift u32}   (4.5 KiB)
//   Huffman: lengths u8[256] | unused[256] | rev codes u16[256]                            (1 KiB)
//   tANS:    norm u16[256] | delta_nb u32[256] | delta_find_state i32[256] | next-state u16[2048] | spread symbols u8[2048]
//   O1SAC:   joint counts u32[256][256] | row-start counts u32[256] | present u8[256] | rank u16[256] |
//            pmf u16[257][256] (row 0 marginal, row 1 + c for context c) | cum u16[257][256]
constexpr uint32_t ENC_TABLE_BYTES = 1024;
constexpr uint32_t ENC_RANS_TABLE_BYTES = 512 + 4096;
constexpr uint32_t ENC_TANS_TABLE_BYTES = 512 + 1024 + 1024 + 4096 + 2048;
constexpr uint32_t O1E_JOINT = 0, O1E_MARG = 262144, O1E_PRESENT = O1E_MARG + 1024, O1E_RANK = O1E_PRESENT + 256, O1E_PMF = O1E_RANK + 512,
                   O1E_CUM = O1E_PMF + 257 * 512, ENC_O1SAC_TABLE_BYTES = O1E_CUM + 257 * 512;
constexpr uint32_t O1SAC_TOTAL = 4096;
__host__ __device__ inline uint32_t enc_table_bytes(int codec) {
    return codec == C_RANS ? ENC_RANS_TABLE_BYTES : codec == C_TANS ? ENC_TANS_TABLE_BYTES : codec == C_O1SAC ? ENC_O1SAC_TABLE_BYTES : ENC_TABLE_BYTES;
}

// The bytes of [p, p + n) handed to `f` one at a time, last to first (BACKWARD) or first to last, read from memory
// in aligned 16-byte blocks wherever a whole block lies inside the range.  An encoding thread walks its own stream:
// with single-byte loads every byte costs a 32-byte sector fetch of its own once the lines have left the L1.
template <bool BACKWARD, class F>
__device__ __forceinline__ void for_each_byte(const uint8_t* p, uint32_t n, F&& f) {
    const uintptr_t lo = reinterpret_cast<uintptr_t>(p), hi = lo + n;
    const uintptr_t first_block = (lo + 15) & ~uintptr_t(15), last_block = hi & ~uintptr_t(15);  // whole blocks: [first_block, last_block)
    if (first_block >= last_block) {
        if (BACKWARD) for (uint32_t k = n; k-- > 0;) f(uint32_t(p[k]));
        else for (uint32_t k = 0; k < n; ++k) f(uint32_t(p[k]));
        return;
    }
    if (BACKWARD) {
        for (uintptr_t a = hi; a-- > last_block;) f(uint32_t(*reinterpret_cast<const uint8_t*>(a)));
        for (uintptr_t b = last_block; b > first_block;) {
            b -= 16;
            const uint4 v = *reinterpret_cast<const uint4*>(b);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 15; k >= 0; --k) f((w[k >> 2] >> (8 * (k & 3))) & 0xFFu);
        }
        for (uintptr_t a = first_block; a-- > lo;) f(uint32_t(*reinterpret_cast<const uint8_t*>(a)));
    } else {
        for (uintptr_t a = lo; a < first_block; ++a) f(uint32_t(*reinterpret_cast<const uint8_t*>(a)));
        for (uintptr_t b = first_block; b < last_block; b += 16) {
            const uint4 v = *reinterpret_cast<const uint4*>(b);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 16; ++k) f((w[k >> 2] >> (8 * (k & 3))) & 0xFFu);
        }
        for (uintptr_t a = last_block; a < hi; ++a) f(uint32_t(*reinterpret_cast<const uint8_t*>(a)));
    }
}

__global__ void __launch_bounds__(256) split_kernel(const SplitItem* __restrict__ items, uint32_t n_items, uint8_t* __restrict__ planes) {
    uint32_t tile = blockIdx.x;
    uint32_t lo = 0, hi = n_items;
    while (lo + 1 < hi) { uint32_t mid = (lo + hi) >> 1; if (items[mid].first_tile <= tile) lo = mid; else hi = mid; }
    const SplitItem it = items[lo];
    uint64_t base = uint64_t(tile - it.first_tile) * SPLIT_TILE;
    uint32_t n = it.n - base < SPLIT_TILE ? uint32_t(it.n - base) : SPLIT_TILE;
    const int eb = kind_elem_bytes(int(it.kind));
    const uint8_t* src = it.src + base * uint64_t(eb);
    // Sixteen elements per thread and step where the source is 16-byte aligned: 128-bit loads, one 128-bit store per
    // plane.  (Plane offsets and tile bases are multiples of 16 by construction.)  The rest goes element by element.
    uint32_t done = 0;
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0 && it.kind != K_PASS) {
        const uint32_t groups = n / 16;
        for (uint32_t g = threadIdx.x; g < groups; g += blockDim.x) {
            const uint64_t at = base + uint64_t(g) * 16;
            if (it.kind == K_M16) {
                const uint4 a = reinterpret_cast<const uint4*>(src)[2 * g], b = reinterpret_cast<const uint4*>(src)[2 * g + 1];
                const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {  // two words = four elements -> one word per plane
                    const uint32_t r0 = ((w[2 * k] << 1) & 0xFF00FF00u) | ((w[2 * k] >> 8) & 0x00800080u) | (w[2 * k] & 0x007F007Fu);
                    const uint32_t r1 = ((w[2 * k + 1] << 1) & 0xFF00FF00u) | ((w[2 * k + 1] >> 8) & 0x00800080u) | (w[2 * k + 1] & 0x007F007Fu);
                    lo[k] = __byte_perm(r0, r1, 0x6420);
                    hi[k] = __byte_perm(r0, r1, 0x7531);
                }
                *reinterpret_cast<uint4*>(planes + it.plane_off[0] + at) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4*>(planes + it.plane_off[1] + at) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            } else if (it.kind == K_M32) {
                uint32_t pl[4][4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {  // four elements -> one word per plane
                    const uint4 v = reinterpret_cast<const uint4*>(src)[4 * g + q];
                    const uint32_t e[4] = {v.x, v.y, v.z, v.w};
                    uint32_t r[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) r[k] = ((e[k] << 1) & 0xFF000000u) | ((e[k] >> 8) & 0x00800000u) | (e[k] & 0x007FFFFFu);
                    const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[2], r[3], 0x5140);  // bytes 0,1 of the pairs
                    const uint32_t t2 = __byte_perm(r[0], r[1], 0x7362), t3 = __byte_perm(r[2], r[3], 0x7362);  // bytes 2,3
                    pl[0][q] = __byte_perm(t0, t1, 0x5410); pl[1][q] = __byte_perm(t0, t1, 0x7632);
                    pl[2][q] = __byte_perm(t2, t3, 0x5410); pl[3][q] = __byte_perm(t2, t3, 0x7632);
                }
#pragma unroll
                for (int p = 0; p < 4; ++p) *reinterpret_cast<uint4*>(planes + it.plane_off[p] + at) = make_uint4(pl[p][0], pl[p][1], pl[p][2], pl[p][3]);
            } else {
                const uint4 v = reinterpret_cast<const uint4*>(src)[g];
                const uint32_t e[4] = {v.x, v.y, v.z, v.w};
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t r = it.kind == K_E4M3 ? (((e[k] & 0x78787878u) << 1) | ((e[k] & 0x80808080u) >> 4) | (e[k] & 0x07070707u))
                                                        : (((e[k] & 0x7C7C7C7Cu) << 1) | ((e[k] & 0x80808080u) >> 5) | (e[k] & 0x03030303u));
                    hi[k] = (r >> 4) & 0x0F0F0F0Fu; lo[k] = r & 0x0F0F0F0Fu;
                }
                *reinterpret_cast<uint4*>(planes + it.plane_off[0] + at) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(planes + it.plane_off[1] + at) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
        done = groups * 16;
    } else if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const uint32_t groups = n / 16;
        for (uint32_t g = threadIdx.x; g < groups; g += blockDim.x)
            *reinterpret_cast<uint4*>(planes + it.plane_off[0] + base + uint64_t(g) * 16) = reinterpret_cast<const uint4*>(src)[g];
        done = groups * 16;
    }
    for (uint32_t i = done + threadIdx.x; i < n; i += blockDim.x) {
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
    // Eight copies of the histogram, laid out [symbol][copy]: the lanes of a warp spread over the copies (an exponent plane
    // sends most of them to the same three or four symbols) and the copies of a symbol sit in different banks.  The plane
    // is read 16 bytes at a time.
    __shared__ uint32_t h[256 * 8];
    const EncChunk c = chunks[blockIdx.x];
    for (uint32_t i = threadIdx.x; i < 256 * 8; i += blockDim.x) h[i] = 0;
    __syncthreads();
    const uint8_t* p = planes + c.plane_off;
    uint32_t* mine = h + (threadIdx.x & 7);
    const uintptr_t lo = reinterpret_cast<uintptr_t>(p), hi = lo + c.n;
    const uintptr_t first_block = (lo + 15) & ~uintptr_t(15), last_block = hi & ~uintptr_t(15);
    if (first_block >= last_block) {
        for (uint32_t i = threadIdx.x; i < c.n; i += blockDim.x) atomicAdd(&mine[uint32_t(p[i]) * 8], 1u);
    } else {
        const uint32_t head = uint32_t(first_block - lo), tail = uint32_t(hi - last_block);
        if (threadIdx.x < head) atomicAdd(&mine[uint32_t(p[threadIdx.x]) * 8], 1u);
        if (threadIdx.x < tail) atomicAdd(&mine[uint32_t(*reinterpret_cast<const uint8_t*>(last_block + threadIdx.x)) * 8], 1u);
        const uint32_t blocks = uint32_t((last_block - first_block) >> 4);
        for (uint32_t b = threadIdx.x; b < blocks; b += blockDim.x) {
            const uint4 v = *reinterpret_cast<const uint4*>(first_block + 16 * uintptr_t(b));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 16; ++k) atomicAdd(&mine[((w[k >> 2] >> (8 * (k & 3))) & 0xFFu) * 8], 1u);
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) {
        uint32_t total = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) total += h[i * 8 + k];
        hist[uint64_t(blockIdx.x) * 256 + i] = total;
        if (total) atomicAdd(&plane_hist[uint64_t(c.plane) * 256 + i], (unsigned long long)total);
    }
}

// One thread per chunk builds the chunk's table for the codec its plane uses.
__global__ void __launch_bounds__(64) table_kernel(const EncChunk* __restrict__ chunks, uint32_t n_chunks, const uint8_t* __restrict__ plane_codec,
                                                   const uint32_t* __restrict__ hist, uint8_t* __restrict__ tables, EncResult* __restrict__ results) {
    uint32_t ci = blockIdx.x * blockDim.x + threadIdx.x;
    if (ci >= n_chunks) return;
    const EncChunk c = chunks[ci];
    const uint32_t* raw = hist + uint64_t(ci) * 256;
    uint8_t* tab = tables + c.table_off;
    EncResult r{{0, 0, 0, 0}, 0, 0};
    int codec = plane_codec[c.plane];
    if (codec == C_O1SAC) return;  // fitted by its own kernels
    if (codec == C_RANS && c.n) {
        uint16_t* freqs = reinterpret_cast<uint16_t*>(tab);
        uint4* sym = reinterpret_cast<uint4*>(tab + 512);
        int ms = rans_normalize(raw, c.n, freqs);
        if (ms >= 0) {
            // x' = x + bias + floor(x / f) * (2048 - f) with the quotient from a rounded-up reciprocal: exact for every
            // state below 2^31, i.e. identical to (x / f) * 2048 + x % f + start (entropy/rans/compress.rs:140-185)
            uint32_t run = 0;
            for (int i = 0; i < 256; ++i) {
                const uint32_t f = freqs[i];
                uint4 e = make_uint4(0, 0, 0, 0);
                if (f == 1) e = make_uint4(0xFFFFFFFFu, run + 2047u, 2047u, 0u);
                else if (f > 1) {
                    uint32_t shift = 0;
                    while (f > (1u << shift)) ++shift;
                    e = make_uint4(uint32_t(((1ull << (shift + 31)) + f - 1) / f), run, 2048u - f, shift - 1);
                }
                sym[i] = e;
                run += f;
            }
            r.hdr_n = uint32_t(ms); r.coded = 1;
            // A chunk that cannot come out smaller than it is gets no encoding pass: the coder's output is at least the
            // information content of the chunk under its table, less the four initial states, so when that alone (with a
            // margin for the float logarithm) reaches the chunk's size the result would be discarded anyway
            // (compress.rs: NotBeneficial).  Sign / mantissa planes are the usual case.
            float bits = 0.f;
            for (int i = 0; i <= ms; ++i) if (raw[i]) bits += float(raw[i]) * (11.f - log2f(float(freqs[i])));
            const float lower = bits * (1.f - 1e-4f) / 8.f - 16.f + float(1 + 2 * (ms + 1) + 16);
            if (lower >= float(c.n) + 64.f) r.coded = 0;
        }
    } else if (codec == C_HUFFMAN && c.n) {
        uint32_t nf[512]; uint16_t parent[512]; uint8_t alive[512]; uint8_t sym_of[256];
        uint8_t* lengths = tab;
        int nw = huffman_lengths<uint32_t>(raw, lengths, nf, parent, alive, sym_of);
        if (nw > 0) {
            huffman_codes(lengths, reinterpret_cast<uint16_t*>(tab + 512));
            r.hdr_n = uint32_t(nw); r.coded = 1;
            // the four streams together hold at least ceil(total bits / 8) bytes: no encoding pass for a chunk that cannot shrink
            uint64_t total_bits = 0;
            for (int i = 0; i < nw; ++i) total_bits += uint64_t(raw[i]) * lengths[i];
            if ((total_bits + 7) / 8 + (nw <= 127 ? 1 : 2) + (uint32_t(nw) + 1) / 2 + 16 >= c.n) r.coded = 0;
        }
    } else if (codec == C_TANS && c.n) {  // entropy/tans/mod.rs:199-266
        uint16_t* norm = reinterpret_cast<uint16_t*>(tab);
        uint32_t* dnb = reinterpret_cast<uint32_t*>(tab + 512);
        int32_t* dfs = reinterpret_cast<int32_t*>(tab + 1536);
        uint16_t* next_state = reinterpret_cast<uint16_t*>(tab + 2560);
        uint8_t* spread = tab + 6656;
        const int nsym = tans_normalize(raw, c.n, norm);
        if (nsym >= 2) {
            uint32_t pos = 0;
            for (int s = 0; s < 256; ++s)
                for (uint32_t k = 0; k < norm[s]; ++k) { spread[pos] = uint8_t(s); pos = (pos + 1283u) & 2047u; }
            uint16_t fill[256];
            uint32_t running = 0;
            int32_t tot = 0;
            for (int s = 0; s < 256; ++s) {
                fill[s] = uint16_t(running); running += norm[s];
                const uint32_t cnt = norm[s];
                dnb[s] = 0; dfs[s] = 0;
                if (cnt == 1) { dnb[s] = (11u << 16) - 2048u; dfs[s] = tot - 1; tot += 1; }
                else if (cnt > 1) {
                    const uint32_t max_bits = 11u - (31u - uint32_t(__clz(cnt - 1)));
                    dnb[s] = (max_bits << 16) - (cnt << max_bits);
                    dfs[s] = tot - int32_t(cnt); tot += int32_t(cnt);
                }
            }
            for (uint32_t u = 0; u < 2048; ++u) { const int s = spread[u]; next_state[fill[s]++] = uint16_t(2048u + u); }
            r.hdr_n = uint32_t(nsym); r.coded = 1;
        }
    }
    results[ci] = r;
}

// tANS (entropy/tans/mod.rs:268-318): one stream per chunk, so one lane per chunk; the symbols are walked last to first and the
// bits go upward from the start of the chunk's slot area.  A symbol is two table look-ups that depend on the running
// state, so the tables of the 32 chunks of a block sit in shared memory, laid out [entry][lane] like the decoder's:
// next state (u16 x 2048), and per symbol the bit-count term (u32) and the state offset (i16).  With the tables in global
// memory every symbol waited for the L2 twice.
constexpr int TENC_CHUNKS = 32;
constexpr int TENC_NEXT_BYTES = 2048 * 32 * 2, TENC_DNB_BYTES = 256 * 32 * 4, TENC_DFS_BYTES = 256 * 32 * 2;
constexpr int TENC_SMEM = TENC_NEXT_BYTES + TENC_DNB_BYTES + TENC_DFS_BYTES;
__global__ void __launch_bounds__(32, 1) tans_encode_kernel(const EncChunk* __restrict__ chunks, const uint32_t* __restrict__ list, uint32_t n_list,
                                                            const uint8_t* __restrict__ planes, const uint8_t* __restrict__ tables, uint8_t* __restrict__ slots,
                                                            EncResult* __restrict__ results) {
    extern __shared__ __align__(16) uint8_t tenc_smem[];
    const uint32_t lane = threadIdx.x, li = blockIdx.x * TENC_CHUNKS + lane;
    if (li >= n_list) return;
    const uint32_t ci = list[li];
    const EncChunk c = chunks[ci];
    if (!results[ci].coded || !c.n) return;  // lanes do not depend on one another
    uint16_t* next_state = reinterpret_cast<uint16_t*>(tenc_smem) + lane;                                 // entry e at next_state[e * 32]
    uint32_t* dnb = reinterpret_cast<uint32_t*>(tenc_smem + TENC_NEXT_BYTES) + lane;                       // symbol s at dnb[s * 32]
    int16_t* dfs = reinterpret_cast<int16_t*>(tenc_smem + TENC_NEXT_BYTES + TENC_DNB_BYTES) + lane;       // symbol s at dfs[s * 32]
    {
        const uint8_t* tab = tables + c.table_off;  // table areas start on 16-byte boundaries
        const uint4* g_dnb = reinterpret_cast<const uint4*>(tab + 512);
        const uint4* g_dfs = reinterpret_cast<const uint4*>(tab + 1536);
        const uint4* g_next = reinterpret_cast<const uint4*>(tab + 2560);
        for (uint32_t k = 0; k < 64; ++k) {
            const uint4 a = g_dnb[k], b = g_dfs[k];
            dnb[(4 * k + 0) * 32] = a.x; dnb[(4 * k + 1) * 32] = a.y; dnb[(4 * k + 2) * 32] = a.z; dnb[(4 * k + 3) * 32] = a.w;
            dfs[(4 * k + 0) * 32] = int16_t(int32_t(b.x)); dfs[(4 * k + 1) * 32] = int16_t(int32_t(b.y));
            dfs[(4 * k + 2) * 32] = int16_t(int32_t(b.z)); dfs[(4 * k + 3) * 32] = int16_t(int32_t(b.w));
        }
        for (uint32_t k = 0; k < 256; ++k) {
            const uint4 v = g_next[k];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) next_state[(8 * k + j) * 32] = uint16_t(w[j >> 1] >> (16 * (j & 1)));
        }
    }
    uint32_t* w32 = reinterpret_cast<uint32_t*>(slots + c.slot_off);  // slot areas start on 16-byte boundaries
    uint64_t acc = 0, total_bits = 0;
    uint32_t nb_acc = 0, words = 0, value = 2048;
    auto add_bits = [&](uint32_t v, uint32_t nb) {
        acc |= uint64_t(v & ((1u << nb) - 1u)) << nb_acc;
        nb_acc += nb; total_bits += nb;
        if (nb_acc >= 32) { w32[words++] = uint32_t(acc); acc >>= 32; nb_acc -= 32; }
    };
    auto step = [&](uint32_t b) {
        const uint32_t nb = (value + dnb[b * 32]) >> 16;
        add_bits(value, nb);
        value = next_state[uint32_t(int32_t(value >> nb) + int32_t(dfs[b * 32])) * 32];
    };
    // the plane's bytes last to first: single bytes down to a 16-byte boundary, then aligned blocks, each requested while the
    // one before it is coded, then the bytes below the first boundary
    const uintptr_t lo = reinterpret_cast<uintptr_t>(planes + c.plane_off), hi = lo + c.n;
    const uintptr_t first_block = (lo + 15) & ~uintptr_t(15), last_block = hi & ~uintptr_t(15);
    if (first_block >= last_block) {
        for (uintptr_t a = hi; a-- > lo;) step(*reinterpret_cast<const uint8_t*>(a));
    } else {
        for (uintptr_t a = hi; a-- > last_block;) step(*reinterpret_cast<const uint8_t*>(a));
        uintptr_t b = last_block - 16;
        uint4 ahead = *reinterpret_cast<const uint4*>(b);
        for (;;) {
            const uint4 v = ahead;
            const bool more = b > first_block;
            if (more) ahead = *reinterpret_cast<const uint4*>(b - 16);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 15; k >= 0; --k) step((w[k >> 2] >> (8 * (k & 3))) & 0xFFu);
            if (!more) break;
            b -= 16;
        }
        for (uintptr_t a = first_block; a-- > lo;) step(*reinterpret_cast<const uint8_t*>(a));
    }
    add_bits(value, 11);
    uint8_t* tail = reinterpret_cast<uint8_t*>(w32 + words);
    uint32_t bytes = words * 4;
    while (nb_acc > 0) { *tail++ = uint8_t(acc); acc >>= 8; nb_acc = nb_acc > 8 ? nb_acc - 8 : 0; ++bytes; }
    results[ci].stream_len[0] = bytes;
    results[ci].stream_len[1] = uint32_t(total_bits);
    results[ci].stream_len[2] = uint32_t(total_bits >> 32);
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
    int codec = plane_codec[c.plane];
    if (codec == C_O1SAC || codec == C_TANS || !results[ci].coded) return;  // those two have kernels of their own
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
    const uint8_t* tab = tables + c.table_off;
    if (codec == C_RANS) {
        const uint4* syms = reinterpret_cast<const uint4*>(tab + 512);
        uint32_t x = 1u << 23;
        for_each_byte<true>(src, len, [&](uint32_t sym) {
            const uint4 e = __ldg(syms + sym);
            const uint32_t max_state = (2048u - e.z) << 20;  // ((L >> 11) << 8) * freq
            while (x >= max_state) { put(x); x >>= 8; }
            x = x + e.y + (__umulhi(x, e.x) >> e.w) * e.z;
        });
        put(x >> 24); put(x >> 16); put(x >> 8); put(x);  // the final state, little-endian, below the renormalisation bytes
    } else {
        const uint8_t* lengths = tab;
        const uint16_t* rev = reinterpret_cast<const uint16_t*>(tab + 512);
        uint64_t bits = 0; uint32_t cnt = 0;
        for_each_byte<false>(src, len, [&](uint32_t sym) {
            bits |= uint64_t(rev[sym]) << cnt;
            cnt += lengths[sym];
            while (cnt >= 8) { put(uint32_t(bits)); bits >>= 8; cnt -= 8; }
        });
        if (cnt) put(uint32_t(bits));
    }
    flush();
    results[ci].stream_len[s] = uint32_t(slot_end - w);
}

// n bytes from s to d by the threads of a block: d is brought to a 16-byte boundary, then every thread moves 16 bytes at
// a time, the source words taken aligned and shifted into place (a word that holds a needed byte is read whole; device
// allocations are padded beyond that).
__device__ __forceinline__ void block_copy(uint8_t* d, const uint8_t* s, uint32_t n, uint32_t t, uint32_t nt) {
    uint32_t head = uint32_t((16 - (reinterpret_cast<uintptr_t>(d) & 15)) & 15);
    if (head > n) head = n;
    for (uint32_t i = t; i < head; i += nt) d[i] = s[i];
    d += head; s += head; n -= head;
    const uint32_t blocks = n >> 4;
    const uint32_t sh = uint32_t(reinterpret_cast<uintptr_t>(s) & 3) * 8;
    const uint32_t* sw = reinterpret_cast<const uint32_t*>(reinterpret_cast<uintptr_t>(s) & ~uintptr_t(3));
    for (uint32_t b = t; b < blocks; b += nt) {
        const uint32_t* q = sw + 4 * size_t(b);
        const uint32_t w0 = q[0], w1 = q[1], w2 = q[2], w3 = q[3];
        uint4 v = make_uint4(w0, w1, w2, w3);
        if (sh) {
            const uint32_t w4 = q[4];
            v = make_uint4(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh), __funnelshift_r(w2, w3, sh), __funnelshift_r(w3, w4, sh));
        }
        *reinterpret_cast<uint4*>(d + 16 * size_t(b)) = v;
    }
    for (uint32_t i = blocks * 16 + t; i < n; i += nt) d[i] = s[i];
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
    const bool framed = !(g.mode & (GATHER_BARE | GATHER_NOFRAME));
    if (framed) {
        if (t < 5 && mode != 5) d[t] = 0;
        d += 5;
    }
    if (mode <= 1) {
        if (mode == 1) { if (t == 0) d[0] = 0; d += 1; }
        const uint8_t* p = planes + c.plane_off;
        block_copy(d, p, c.n, t, blockDim.x);
        return;
    }
    const uint8_t* tab = tables + c.table_off;
    if (mode == 5) {  // Order1ScaleAC: inline state [bitmap 32][marginal 512][rows 512 each, contexts in increasing order], then the coder's bytes
        const uint8_t* present = tab + O1E_PRESENT;
        const uint16_t* rank = reinterpret_cast<const uint16_t*>(tab + O1E_RANK);
        const uint16_t* pmf = reinterpret_cast<const uint16_t*>(tab + O1E_PMF);
        if (!(g.mode & GATHER_BARE)) {
            const uint32_t state_len = r.stream_len[1];
            if (framed && t == 0) {  // frame header: state_version 1, state length
                uint8_t* fh = d - 5;
                fh[0] = 1; fh[1] = uint8_t(state_len); fh[2] = uint8_t(state_len >> 8); fh[3] = uint8_t(state_len >> 16); fh[4] = uint8_t(state_len >> 24);
            }
            if (t < 32) { uint32_t bits = 0; for (int k = 0; k < 8; ++k) bits |= uint32_t(present[8 * t + k] != 0) << k; d[t] = uint8_t(bits); }
            for (uint32_t i = t; i < 256; i += blockDim.x) { d[32 + 2 * i] = uint8_t(pmf[i]); d[33 + 2 * i] = uint8_t(pmf[i] >> 8); }
            for (uint32_t ctx = 0; ctx < 256; ++ctx) {
                if (!present[ctx]) continue;
                uint8_t* row = d + 32 + 512 + 512 * uint32_t(rank[ctx]);
                const uint16_t* pr = pmf + 256 * (1 + ctx);
                for (uint32_t i = t; i < 256; i += blockDim.x) { row[2 * i] = uint8_t(pr[i]); row[2 * i + 1] = uint8_t(pr[i] >> 8); }
            }
            d += state_len;
        }
        const uint8_t* sp = slots + c.slot_off;
        block_copy(d, sp, r.stream_len[0], t, blockDim.x);
        return;
    }
    if (t == 0) { d[0] = 1; d[1] = uint8_t(c.n); d[2] = uint8_t(c.n >> 8); d[3] = uint8_t(c.n >> 16); d[4] = uint8_t(c.n >> 24); }
    d += 5;
    if (mode == 4) {  // tANS blob: [11][nsym u16][(symbol, freq u16) per present symbol][total bits u64][bits]
        const uint16_t* norm = reinterpret_cast<const uint16_t*>(tab);
        if (t == 0) {
            d[0] = 11; d[1] = uint8_t(r.hdr_n); d[2] = uint8_t(r.hdr_n >> 8);
            uint8_t* q = d + 3;
            for (int sy = 0; sy < 256; ++sy) if (norm[sy]) { q[0] = uint8_t(sy); q[1] = uint8_t(norm[sy]); q[2] = uint8_t(norm[sy] >> 8); q += 3; }
            for (int k = 0; k < 4; ++k) { q[k] = uint8_t(r.stream_len[1] >> (8 * k)); q[4 + k] = uint8_t(r.stream_len[2] >> (8 * k)); }
        }
        d += 3 + 3 * r.hdr_n + 8;
        const uint8_t* sp = slots + c.slot_off;
        block_copy(d, sp, r.stream_len[0], t, blockDim.x);
        return;
    }
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
        block_copy(d, sp, r.stream_len[s], t, blockDim.x);
        d += r.stream_len[s];
    }
}

// ---- ops between a byte split and a terminal (transforms/int_delta.rs:36-44, transforms/mantissa_zero.rs) ------
// IntDelta forward, byte width: every byte minus the one before it, modulo 256, over the whole plane (out of place).
__global__ void __launch_bounds__(256) delta_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n) {
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x)
        dst[i] = uint8_t(src[i] - (i ? src[i - 1] : 0));
}
// OR of all bytes of a plane: MantissaZeroStrip(k) applies when the low k bits of that are clear.
__global__ void __launch_bounds__(256) or_bytes_kernel(const uint8_t* __restrict__ src, uint64_t n, uint32_t* __restrict__ out) {
    uint32_t v = 0;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x) v |= src[i];
    v = __reduce_or_sync(0xFFFFFFFFu, v);
    if ((threadIdx.x & 31) == 0 && v) atomicOr(out, v);
}
__global__ void __launch_bounds__(256) shift_right_kernel(uint8_t* __restrict__ p, uint64_t n, uint32_t k) {
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x) p[i] = uint8_t(p[i] >> k);
}
// The chunk histograms of a plane whose bytes were just shifted right by k (all with k clear low bits): count v moves to v >> k.
__global__ void __launch_bounds__(256) relabel_hist_kernel(uint32_t* __restrict__ hist, uint32_t first_chunk, uint32_t k) {
    uint32_t* h = hist + uint64_t(first_chunk + blockIdx.x) * 256;
    const uint32_t v = threadIdx.x, c = h[v];
    __syncthreads();
    h[v] = 0;
    __syncthreads();
    if (c) h[v >> k] = c;
}

// ---- Order1ScaleAC encode (codecs/order1_scale_ac.rs:620-663, 963-1025) -------------------------------------
// Lag-1 counts of one chunk: the first symbol of a row counts toward the marginal, every other symbol toward the row
// of the symbol before it.  One CTA per listed chunk; the count areas were cleared beforehand.
__global__ void __launch_bounds__(256) o1sac_count_kernel(const EncChunk* __restrict__ chunks, const uint32_t* __restrict__ list, const uint8_t* __restrict__ planes,
                                                          uint8_t* __restrict__ tables) {
    const EncChunk c = chunks[list[blockIdx.x]];
    uint32_t* joint = reinterpret_cast<uint32_t*>(tables + c.table_off + O1E_JOINT);
    uint32_t* marg = reinterpret_cast<uint32_t*>(tables + c.table_off + O1E_MARG);
    const uint8_t* p = planes + c.plane_off;
    const uint32_t row_len = c.row_len ? c.row_len : (c.n ? c.n : 1);
    for (uint32_t i = threadIdx.x; i < c.n; i += blockDim.x) {
        if (i % row_len == 0) atomicAdd(&marg[p[i]], 1u);
        else atomicAdd(&joint[uint32_t(p[i - 1]) * 256 + p[i]], 1u);
    }
}
// Probability rows from the counts (a context gets a row when it was seen at all), their cumulative sums for the coder,
// and the rank of every present context (its place among the rows of the serialized state).  One CTA of 288 threads per chunk:
// thread c < 256 owns context c, thread 256 the marginal.
__global__ void __launch_bounds__(288) o1sac_fit_kernel(const EncChunk* __restrict__ chunks, const uint32_t* __restrict__ list, uint8_t* __restrict__ tables,
                                                        EncResult* __restrict__ results) {
    const uint32_t ci = list[blockIdx.x];
    uint8_t* tab = tables + chunks[ci].table_off;
    const uint32_t* joint = reinterpret_cast<const uint32_t*>(tab + O1E_JOINT);
    const uint32_t* marg = reinterpret_cast<const uint32_t*>(tab + O1E_MARG);
    uint8_t* present = tab + O1E_PRESENT;
    uint16_t* rank = reinterpret_cast<uint16_t*>(tab + O1E_RANK);
    uint16_t* pmf = reinterpret_cast<uint16_t*>(tab + O1E_PMF);
    uint16_t* cum = reinterpret_cast<uint16_t*>(tab + O1E_CUM);
    const uint32_t t = threadIdx.x;
    __shared__ uint32_t seen[256];
    if (t <= 256) {
        const uint32_t* raw = t < 256 ? joint + 256 * t : marg;
        const uint32_t row = t < 256 ? 1 + t : 0;
        bool use = true;
        if (t < 256) {
            uint64_t total = 0;
            for (int i = 0; i < 256; ++i) total += raw[i];
            use = total != 0;
            present[t] = use;
            seen[t] = use;
        }
        if (use) {
            uint16_t* out = pmf + 256 * row;
            quantize_pmf256(raw, O1SAC_TOTAL, out);
            uint32_t acc = 0;
            for (int i = 0; i < 256; ++i) { cum[256 * row + i] = uint16_t(acc); acc += out[i]; }
        }
    }
    __syncthreads();
    if (t == 0) {
        uint32_t k = 0;
        for (int ctx = 0; ctx < 256; ++ctx) { rank[ctx] = uint16_t(k); k += seen[ctx]; }
        results[ci].hdr_n = k;
        results[ci].stream_len[1] = 32 + 512 + 512 * k;
        results[ci].coded = 1;
    }
}
// The range coder over one chunk (range_coder.rs:16-113): 64-bit low, 32-bit range, carry held back in a cache byte and
// a run of 0xFF bytes; total 4096 makes range / total a shift.  One thread per listed chunk, bytes upward from the
// start of the chunk's slot area.
__global__ void __launch_bounds__(64) o1sac_encode_kernel(const EncChunk* __restrict__ chunks, const uint32_t* __restrict__ list, uint32_t n_list,
                                                          const uint8_t* __restrict__ planes, const uint8_t* __restrict__ tables, uint8_t* __restrict__ slots,
                                                          EncResult* __restrict__ results) {
    const uint32_t li = blockIdx.x * blockDim.x + threadIdx.x;
    if (li >= n_list) return;
    const uint32_t ci = list[li];
    const EncChunk c = chunks[ci];
    const uint8_t* tab = tables + c.table_off;
    const uint8_t* present = tab + O1E_PRESENT;
    const uint16_t* pmf = reinterpret_cast<const uint16_t*>(tab + O1E_PMF);
    const uint16_t* cum = reinterpret_cast<const uint16_t*>(tab + O1E_CUM);
    const uint8_t* p = planes + c.plane_off;
    uint8_t* out = slots + c.slot_off;
    uint32_t written = 0;
    uint64_t low = 0, range = 0xFFFFFFFFull;
    uint32_t cache = 0, cache_size = 0;
    auto shift_low = [&]() {
        const uint32_t carry = uint32_t(low >> 32) & 0xFFu, top = uint32_t(low >> 24) & 0xFFu;
        if (top == 0xFF && carry == 0) ++cache_size;
        else {
            out[written++] = uint8_t(cache + carry);
            const uint8_t fill = carry ? 0x00 : 0xFF;
            for (uint32_t i = 0; i < cache_size; ++i) out[written++] = fill;
            cache_size = 0;
            cache = top;
        }
        low = (low & 0x00FFFFFFull) << 8;
    };
    const uint32_t row_len = c.row_len ? c.row_len : (c.n ? c.n : 1);
    uint32_t in_row = 0, row = 0;
    for (uint32_t i = 0; i < c.n; ++i) {
        const uint32_t sym = p[i];
        const uint32_t cu = cum[256 * row + sym], pr = pmf[256 * row + sym];
        const uint64_t rpt = range >> 12;
        low += uint64_t(cu) * rpt;
        range = uint64_t(pr) * rpt;
        while (range < (1ull << 24)) { shift_low(); range <<= 8; }
        if (++in_row == row_len) { in_row = 0; row = 0; }
        else row = present[sym] ? 1 + sym : 0;
    }
    for (int i = 0; i < 5; ++i) shift_low();
    out[written++] = uint8_t(cache);
    for (uint32_t i = 0; i < cache_size; ++i) out[written++] = 0xFF;
    results[ci].stream_len[0] = written;
}

// Scatter host-built byte pieces (record headers, index, footer) into the container.
__global__ void __launch_bounds__(128) scatter_kernel(const uint8_t* __restrict__ staged, const uint64_t* __restrict__ triples, uint8_t* __restrict__ out) {
    uint64_t dst = triples[3 * blockIdx.x], src = triples[3 * blockIdx.x + 1], len = triples[3 * blockIdx.x + 2];
    for (uint64_t i = threadIdx.x; i < len; i += blockDim.x) out[dst + i] = staged[src + i];
}

}  // namespace ptwm
