// Device code of the PTWM decode path for sm_100a: chunk-parallel rANS /
// canonical-Huffman / tANS / Order1ScaleAC decoders with the plane merge and
// inverse bit reorder fused into their epilogue, the stand-alone merge kernel
// and the integrity kernels (CRC-32 of the re-split planes, XXH64).
//
// Bit-exact targets, all under crates/ptwm-core/src of the reference:
//   rANS        entropy/rans/decompress.rs:24-164
//   Huffman     entropy/huffman/{weights.rs:34-85, tree.rs:103-177, bitstream.rs:54-187, decompress.rs:8-211}
//   tANS        entropy/tans/mod.rs:199-211,346-451
//   O1SAC       range_coder.rs:122-198, codecs/order1_scale_ac.rs:85-151,474-486,665-706
//   merges      transforms/fusion.rs:124-193,264-315,373-417,475-519
//
// All of this is integer / byte work bounded by instruction issue, shared
// memory capacity and HBM; nothing here is GEMM-shaped, so no tensor cores.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "plan.h"

namespace ptwm {

__device__ __forceinline__ const uint8_t* rd(const Bases& b, Ref r) {
    uint64_t off = r & ((1ull << 62) - 1);
    uint32_t sp = uint32_t(r >> 62);
    return sp == SP_BLOB ? b.blob + off : sp == SP_SCRATCH ? b.scratch + off : b.out + off;
}
__device__ __forceinline__ uint8_t* wr(const Bases& b, Ref r) {
    uint64_t off = r & ((1ull << 62) - 1);
    return (uint32_t(r >> 62) == SP_SCRATCH ? b.scratch : b.out) + off;
}

__device__ __forceinline__ uint32_t ld_u32_unaligned(const uint8_t* p) {
    return uint32_t(p[0]) | uint32_t(p[1]) << 8 | uint32_t(p[2]) << 16 | uint32_t(p[3]) << 24;
}

// Eight bytes from any address.  The two aligned words both overlap the
// requested range, so nothing outside the 8-byte-aligned span of the source
// is touched.
__device__ __forceinline__ uint64_t ld8_unaligned(const uint8_t* p) {
    uintptr_t a = reinterpret_cast<uintptr_t>(p);
    uint32_t sh = uint32_t(a & 7) * 8;
    const uint64_t* q = reinterpret_cast<const uint64_t*>(a & ~uintptr_t(7));
    uint64_t lo = __ldg(q);
    if (sh == 0) return lo;
    uint64_t hi = __ldg(q + 1);
    return (lo >> sh) | (hi << (64 - sh));
}
__device__ __forceinline__ uint64_t ld_bytes(const uint8_t* p, uint32_t count) {
    uint64_t v = 0;
    for (uint32_t i = 0; i < count; ++i) v |= uint64_t(p[i]) << (8 * i);
    return v;
}

// ---- element composition ---------------------------------------------------
__device__ __forceinline__ uint32_t revert16x2(uint32_t r) {  // split/dtype16.rs:20-25
    return ((r << 8) & 0x80008000u) | ((r >> 1) & 0x7F807F80u) | (r & 0x007F007Fu);
}
__device__ __forceinline__ uint32_t revert32(uint32_t r) {  // transforms/fusion.rs:287-292
    return ((r << 8) & 0x80000000u) | ((r >> 1) & 0x7F800000u) | (r & 0x007FFFFFu);
}
__device__ __forceinline__ uint64_t revert_fp8x8(uint64_t h, uint64_t l, bool e4m3) {  // split/dtype8.rs:39-44,57-62
    uint64_t r = ((h & 0x0F0F0F0F0F0F0F0Full) << 4) | (l & 0x0F0F0F0F0F0F0F0Full);
    return e4m3 ? ((r & 0xF0F0F0F0F0F0F0F0ull) >> 1) | ((r & 0x0808080808080808ull) << 4) | (r & 0x0707070707070707ull)
                : ((r & 0xF8F8F8F8F8F8F8F8ull) >> 1) | ((r & 0x0404040404040404ull) << 5) | (r & 0x0303030303030303ull);
}

// Store `count` (<= 8) elements starting at element `pos` of a tensor whose
// planes' bytes for those elements are b[0..np).  Full groups on aligned
// addresses go out as 128-bit (or 64-bit) stores.
__device__ __forceinline__ void compose_store(int kind, uint8_t* dst, uint64_t pos, uint32_t count, const uint64_t b[4]) {
    switch (kind) {
        case K_PASS: {
            uint8_t* p = dst + pos;
            if (count == 8 && (reinterpret_cast<uintptr_t>(p) & 7) == 0) *reinterpret_cast<uint64_t*>(p) = b[0];
            else for (uint32_t i = 0; i < count; ++i) p[i] = uint8_t(b[0] >> (8 * i));
            break;
        }
        case K_E4M3:
        case K_E5M2: {
            uint64_t v = revert_fp8x8(b[0], b[1], kind == K_E4M3);
            uint8_t* p = dst + pos;
            if (count == 8 && (reinterpret_cast<uintptr_t>(p) & 7) == 0) *reinterpret_cast<uint64_t*>(p) = v;
            else for (uint32_t i = 0; i < count; ++i) p[i] = uint8_t(v >> (8 * i));
            break;
        }
        case K_M16: {
            uint32_t l0 = uint32_t(b[0]), l1 = uint32_t(b[0] >> 32), h0 = uint32_t(b[1]), h1 = uint32_t(b[1] >> 32);
            uint4 v;
            v.x = revert16x2(__byte_perm(l0, h0, 0x5140));
            v.y = revert16x2(__byte_perm(l0, h0, 0x7362));
            v.z = revert16x2(__byte_perm(l1, h1, 0x5140));
            v.w = revert16x2(__byte_perm(l1, h1, 0x7362));
            uint8_t* p = dst + pos * 2;
            if (count == 8 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) *reinterpret_cast<uint4*>(p) = v;
            else {
                uint32_t w[4] = {v.x, v.y, v.z, v.w};
                for (uint32_t i = 0; i < count; ++i) {
                    uint32_t e = (w[i >> 1] >> (16 * (i & 1))) & 0xFFFF;
                    p[2 * i] = uint8_t(e); p[2 * i + 1] = uint8_t(e >> 8);
                }
            }
            break;
        }
        case K_M32: {
            uint32_t w[8];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t p0 = uint32_t(b[0] >> (32 * half)), p1 = uint32_t(b[1] >> (32 * half)), p2 = uint32_t(b[2] >> (32 * half)),
                         p3 = uint32_t(b[3] >> (32 * half));
                uint32_t t0 = __byte_perm(p0, p1, 0x5140), t1 = __byte_perm(p2, p3, 0x5140);
                uint32_t t2 = __byte_perm(p0, p1, 0x7362), t3 = __byte_perm(p2, p3, 0x7362);
                w[4 * half + 0] = revert32(__byte_perm(t0, t1, 0x5410));
                w[4 * half + 1] = revert32(__byte_perm(t0, t1, 0x7632));
                w[4 * half + 2] = revert32(__byte_perm(t2, t3, 0x5410));
                w[4 * half + 3] = revert32(__byte_perm(t2, t3, 0x7632));
            }
            uint8_t* p = dst + pos * 4;
            if (count == 8 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
                reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
                for (uint32_t i = 0; i < count; ++i) {
                    p[4 * i] = uint8_t(w[i]); p[4 * i + 1] = uint8_t(w[i] >> 8); p[4 * i + 2] = uint8_t(w[i] >> 16); p[4 * i + 3] = uint8_t(w[i] >> 24);
                }
            }
            break;
        }
    }
}

// Epilogue of a decoding lane: where its symbols go.
struct Epilogue {
    uint8_t* dst;
    const uint8_t* partner[3];
    int kind, slot, fused;
};
__device__ __forceinline__ Epilogue make_epilogue(const Bases& bases, const DecodeItem& it) {
    Epilogue e;
    e.dst = wr(bases, it.dst);
    e.kind = it.kind; e.slot = it.slot; e.fused = it.fused;
    int np = it.fused ? kind_planes(it.kind) : 1;
    for (int j = 0; j < 3; ++j) e.partner[j] = (j < np - 1) ? rd(bases, it.partner[j]) : nullptr;
    return e;
}
// Bytes of the other planes for `count` elements at `pos` (fused lanes only).
// Issued before the group's symbols are decoded so the loads overlap the decode.
__device__ __forceinline__ void gather_partners(const Epilogue& e, uint64_t pos, uint32_t count, uint64_t b[4]) {
    b[0] = b[1] = b[2] = b[3] = 0;
    if (!e.fused) return;
    int np = kind_planes(e.kind);
    int j = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        if (p >= np) break;
        if (p == e.slot) continue;
        const uint8_t* q = e.partner[j++] + pos;
        b[p] = count == 8 ? ld8_unaligned(q) : ld_bytes(q, count);
    }
}
// `pos` is the symbol index inside the chunk, `syms` holds `count` symbols,
// b[] the partner bytes from gather_partners.
__device__ __forceinline__ void emit_with(const Epilogue& e, uint64_t pos, uint32_t count, uint64_t syms, uint64_t b[4]) {
    if (!e.fused) { b[0] = syms; compose_store(K_PASS, e.dst, pos, count, b); return; }
#pragma unroll
    for (int p = 0; p < 4; ++p) if (p == e.slot) b[p] = syms;
    compose_store(e.kind, e.dst, pos, count, b);
}
__device__ __forceinline__ void emit(const Epilogue& e, uint64_t pos, uint32_t count, uint64_t syms) {
    uint64_t b[4];
    gather_partners(e, pos, count, b);
    emit_with(e, pos, count, syms, b);
}
// The other planes' bytes of a fused lane, read as a stream of aligned 8-byte
// words one group ahead of their use: a group of eight elements needs the
// words w0 and w1, the word after them is requested while the group's symbols
// are still being decoded, so its DRAM latency hides behind the decode.
struct PartnerStream {
    const uint64_t* q[3];    // word that holds the first byte of the current group
    const uint64_t* lim[3];  // first word that must not be read
    uint64_t w0[3], w1[3], w2[3];
    uint32_t sh[3];
    int n;                   // partners (planes - 1), 0 for a plain lane
    __device__ __forceinline__ void start(const Epilogue& e, uint64_t pos, uint32_t chunk_n) {
        n = e.fused ? kind_planes(e.kind) - 1 : 0;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            if (j >= n) break;
            uintptr_t a = reinterpret_cast<uintptr_t>(e.partner[j]) + pos;
            q[j] = reinterpret_cast<const uint64_t*>(a & ~uintptr_t(7));
            sh[j] = uint32_t(a & 7) * 8;
            lim[j] = reinterpret_cast<const uint64_t*>((reinterpret_cast<uintptr_t>(e.partner[j]) + chunk_n + 7) & ~uintptr_t(7));
            w0[j] = q[j] < lim[j] ? __ldg(q[j]) : 0;
            w1[j] = q[j] + 1 < lim[j] ? __ldg(q[j] + 1) : 0;
        }
    }
    __device__ __forceinline__ void prefetch() {
#pragma unroll
        for (int j = 0; j < 3; ++j) { if (j >= n) break; w2[j] = q[j] + 2 < lim[j] ? __ldg(q[j] + 2) : 0; }
    }
    // plane bytes of the current group into b[] (slot = the plane the lane itself decodes), then step to the next group
    __device__ __forceinline__ void take(int slot, uint64_t b[4]) {
        int p = 0;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            if (j >= n) break;
            if (p == slot) ++p;
            b[p++] = sh[j] ? (w0[j] >> sh[j]) | (w1[j] << (64 - sh[j])) : w0[j];
            w0[j] = w1[j]; w1[j] = w2[j]; q[j] += 1;
        }
    }
};

// Length of the first group so that later groups start on an 8-element
// boundary of the destination.
__device__ __forceinline__ uint32_t first_group(const Epilogue& e, uint64_t pos, uint32_t remaining) {
    uintptr_t a = reinterpret_cast<uintptr_t>(e.dst) / uint32_t(e.fused ? kind_elem_bytes(e.kind) : 1) + pos;
    uint32_t g = 8 - uint32_t(a & 7);
    return g < remaining ? g : remaining;
}

__device__ __forceinline__ void split_four_dev(uint32_t n, uint32_t s, uint32_t& start, uint32_t& len) {  // entropy/stream_frame.rs:27-41
    uint32_t base = n >> 2, rem = n & 3;
    len = base + (s < rem ? 1u : 0u);
    start = s * base + (s < rem ? s : rem);
}

// ---- per-lane byte window over a stream ------------------------------------
// A lane reads its stream one byte (rANS, forward) or one aligned word
// (Huffman, backward) at a time.  Global memory is fetched in aligned 16-byte
// blocks one step ahead of use and parked in a 64-byte ring per lane in shared
// memory, laid out [ring word][lane] so that any mix of positions across the
// warp is bank-conflict free.
struct Ring {
    uint32_t* base;  // &ring[0][lane]
    __device__ __forceinline__ uint32_t& word(uintptr_t addr) { return base[((addr >> 2) & 15) * 32]; }
    __device__ __forceinline__ uint8_t byte(uintptr_t addr) { return reinterpret_cast<uint8_t*>(&word(addr))[addr & 3]; }
    __device__ __forceinline__ void put(uintptr_t addr16, uint4 v) {
        word(addr16) = v.x; word(addr16 + 4) = v.y; word(addr16 + 8) = v.z; word(addr16 + 12) = v.w;
    }
};
// Aligned 16-byte block, zero outside [lo16, hi16) (the 16-byte hull of the blob).
__device__ __forceinline__ uint4 fetch16(uintptr_t a, uintptr_t lo16, uintptr_t hi16) {
    if (a < lo16 || a >= hi16) return make_uint4(0, 0, 0, 0);
    return __ldg(reinterpret_cast<const uint4*>(a));
}

// ---- rANS ------------------------------------------------------------------
constexpr uint32_t RANS_L = 1u << 23;
constexpr int RANS_WARP_CHUNKS = 8;
constexpr int RING_SMEM = 16 * 32 * 4;
// Shared memory per chunk: a rank table for slot pairs (which present symbol
// covers slot 2k+1: 1024 bytes) and one word per present symbol
// (symbol | freq << 8 | start << 20), `l_entries` words (alphabet bound + 2).
// A slot pair can straddle at most one symbol boundary, so the even slot is
// covered by that symbol or the one before it; both words are read and the
// right one is kept.  This is 1.6 KiB per chunk for a bf16 exponent plane
// instead of the 3 KiB of a full slot table, which is what bounds the number
// of streams an SM holds.
__host__ __device__ inline uint32_t rans_l_entries(uint32_t max_sym) { return (max_sym + 3 + 3) & ~3u; }
__host__ __device__ inline uint32_t rans_smem_bytes(uint32_t l_entries) { return RANS_WARP_CHUNKS * (1024 + 4 * l_entries) + RING_SMEM; }

__global__ void __launch_bounds__(32) rans_decode_kernel(const DecodeItem* __restrict__ items, uint32_t n_items, Bases bases, uint32_t* __restrict__ status,
                                                         uint32_t l_entries) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t lane = threadIdx.x, c = lane >> 2, s = lane & 3;
    uint8_t* ranktab = smem;                                                             // [8][1024]
    uint32_t* symlist = reinterpret_cast<uint32_t*>(smem + RANS_WARP_CHUNKS * 1024);     // [8][l_entries], entry 0 is a pad
    Ring ring{reinterpret_cast<uint32_t*>(smem + RANS_WARP_CHUNKS * (1024 + 4 * l_entries)) + lane};

    const uint32_t item_idx = blockIdx.x * RANS_WARP_CHUNKS + c;
    const bool valid = item_idx < n_items;
    DecodeItem it;
    if (valid) it = items[item_idx];
    const uint8_t* src = valid ? rd(bases, it.src) : nullptr;
    uint32_t err = ST_OK;

    // header: [max_sym][freq u16 x (max_sym+1)][4 x u32 stream lengths]
    uint32_t max_sym = 0, hdr = 0, my_off = 0, my_len = 0;
    if (valid) {
        if (it.src_len < 1) err = ST_BAD_HEADER;
        else {
            max_sym = src[0];
            hdr = 1 + 2 * (max_sym + 1);
            if (it.src_len < hdr + 16 || max_sym + 3 > l_entries) err = ST_BAD_HEADER;
            else {
                uint64_t total = 0;
                uint32_t off = hdr + 16;
                for (uint32_t k = 0; k < 4; ++k) {
                    uint32_t l = ld_u32_unaligned(src + hdr + 4 * k);
                    if (k == s) { my_off = off + uint32_t(total); my_len = l; }
                    total += l;
                }
                if (total != uint64_t(it.src_len - hdr - 16)) err = ST_BAD_HEADER;
            }
        }
    }

    // tables: the whole warp builds one chunk's tables at a time
    for (uint32_t c2 = 0; c2 < RANS_WARP_CHUNKS; ++c2) {
        const uint32_t leader = c2 * 4;
        uintptr_t psrc = __shfl_sync(0xFFFFFFFFu, reinterpret_cast<uintptr_t>(src), leader);
        uint32_t pms = __shfl_sync(0xFFFFFFFFu, max_sym, leader);
        uint32_t perr = __shfl_sync(0xFFFFFFFFu, err, leader);
        uint32_t pvalid = __shfl_sync(0xFFFFFFFFu, uint32_t(valid), leader);
        if (!pvalid || perr) continue;
        const uint8_t* ps = reinterpret_cast<const uint8_t*>(psrc);
        uint32_t f[8], sum = 0, present = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t sym = lane * 8 + k;
            f[k] = sym <= pms ? uint32_t(ps[1 + 2 * sym]) | uint32_t(ps[2 + 2 * sym]) << 8 : 0u;
            sum += f[k];
            present += f[k] != 0;
        }
        uint32_t incl = sum, rincl = present;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, d), r = __shfl_up_sync(0xFFFFFFFFu, rincl, d);
            if (lane >= d) { incl += t; rincl += r; }
        }
        uint32_t total = __shfl_sync(0xFFFFFFFFu, incl, 31);
        bool bad = total != 2048;  // decompress.rs:49-55
        if (bad) { if (c == c2) err = ST_BAD_HEADER; continue; }
        uint32_t start = incl - sum, rank = rincl - present;
        uint8_t* tab = ranktab + c2 * 1024;
        uint32_t* lst = symlist + c2 * l_entries;
        if (lane == 0) lst[0] = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t sym = lane * 8 + k, fr = f[k];
            if (!fr) continue;
            lst[rank + 1] = sym | (fr << 8) | (start << 20);
            uint32_t a = start >> 1, e = (start + fr) >> 1;  // pairs whose odd slot lies in [start, start + fr)
            while (a < e && (a & 3)) tab[a++] = uint8_t(rank);
            uint32_t rep = rank * 0x01010101u;
            while (a + 4 <= e) { *reinterpret_cast<uint32_t*>(tab + a) = rep; a += 4; }
            while (a < e) tab[a++] = uint8_t(rank);
            start += fr; ++rank;
        }
    }
    __syncwarp();

    uint32_t seg_start = 0, seg_len = 0;
    if (valid) split_four_dev(it.n, s, seg_start, seg_len);
    if (valid && !err && seg_len > 0) {
        if (my_len < 4) err = ST_STREAM_UNDERRUN;  // decompress.rs:82-86
        else {
            const uint8_t* tab = ranktab + c * 1024;
            const uint32_t* lst = symlist + c * l_entries;
            Epilogue ep = make_epilogue(bases, it);
            const uint8_t* st = src + my_off;
            uint32_t x = ld_u32_unaligned(st);
            // ring cursor as a 32-bit offset from the 16-byte aligned block that holds the first renorm byte
            const uintptr_t g0 = (reinterpret_cast<uintptr_t>(st) + 4) & ~uintptr_t(15);
            uint32_t rq = uint32_t(reinterpret_cast<uintptr_t>(st) + 4 - g0);
            const uint32_t end_q = uint32_t(reinterpret_cast<uintptr_t>(st) + my_len - g0);
            const uintptr_t lo16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_first) & ~uintptr_t(15);
            const uintptr_t hi16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_end + 15) & ~uintptr_t(15);
            const uint8_t* rb = reinterpret_cast<const uint8_t*>(ring.base);
#define RING_BYTE(q) rb[(((q) & 60u) << 5) | ((q) & 3u)]
            uint32_t fq = 0;
            ring.put(fq, fetch16(g0 + fq, lo16, hi16)); fq += 16;
            ring.put(fq, fetch16(g0 + fq, lo16, hi16)); fq += 16;
            ring.put(fq, fetch16(g0 + fq, lo16, hi16)); fq += 16;
            uint4 pending = fetch16(g0 + fq, lo16, hi16);

            uint64_t pos = seg_start;
            uint32_t remaining = seg_len;
            uint32_t g = first_group(ep, pos, remaining);
            PartnerStream ps;
            bool streaming = false;
            while (remaining) {
                if (fq - rq < 32) { ring.put(fq, pending); fq += 16; pending = fetch16(g0 + fq, lo16, hi16); }
                uint64_t pb[4] = {0, 0, 0, 0};
                if (streaming) ps.prefetch();
                uint32_t s_lo = 0, s_hi = 0;
                if (g == 8) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint32_t nb = RING_BYTE(rq);  // next renorm byte, read before it is known to be needed
                        uint32_t idx = x & 2047u;
                        uint32_t r = tab[idx >> 1];
                        uint32_t ea = lst[r + 1], eb = lst[r];
                        uint32_t e = idx < (ea >> 20) ? eb : ea;
                        uint32_t sym = e & 0xFFu;
                        x = ((e >> 8) & 0xFFFu) * (x >> 11) + idx - (e >> 20);
                        if (j < 4) s_lo |= sym << (8 * j); else s_hi |= sym << (8 * (j - 4));
                        bool need = x < RANS_L;
                        x = need ? (x << 8) | nb : x;
                        rq += need ? 1u : 0u;
                        if (x < RANS_L) {
                            x = (x << 8) | RING_BYTE(rq); ++rq;
                            if (x < RANS_L) { x = (x << 8) | RING_BYTE(rq); ++rq; }
                        }
                    }
                } else {
                    for (uint32_t j = 0; j < g; ++j) {
                        uint32_t idx = x & 2047u;
                        uint32_t r = tab[idx >> 1];
                        uint32_t ea = lst[r + 1], eb = lst[r];
                        uint32_t e = idx < (ea >> 20) ? eb : ea;
                        uint32_t sym = e & 0xFFu;
                        x = ((e >> 8) & 0xFFFu) * (x >> 11) + idx - (e >> 20);
                        if (j < 4) s_lo |= sym << (8 * j); else s_hi |= sym << (8 * (j - 4));
                        for (int r = 0; r < 3 && x < RANS_L; ++r) { x = (x << 8) | RING_BYTE(rq); ++rq; }
                    }
                }
                if (streaming) ps.take(ep.slot, pb);
                else gather_partners(ep, pos, g, pb);  // the first group may be short and start anywhere
                emit_with(ep, pos, g, uint64_t(s_lo) | uint64_t(s_hi) << 32, pb);
                pos += g; remaining -= g;
                g = remaining < 8 ? remaining : 8;
                if (!streaming && remaining) { ps.start(ep, pos, it.n); streaming = true; }
            }
#undef RING_BYTE
            if (rq > end_q) err = ST_STREAM_UNDERRUN;  // decompress.rs:99-104
        }
    }
    if (err) atomicMax(&status[it.id], err);
}

// ---- canonical Huffman -----------------------------------------------------
constexpr int HUF_WARP_CHUNKS = 8;
constexpr int HUF_SMEM_PER_CHUNK = 2048 * 2;  // 2^11 entries of len<<8 | sym
constexpr int HUF_SMEM = HUF_WARP_CHUNKS * HUF_SMEM_PER_CHUNK + RING_SMEM;

__global__ void __launch_bounds__(32) huffman_decode_kernel(const DecodeItem* __restrict__ items, uint32_t n_items, Bases bases, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t lane = threadIdx.x, c = lane >> 2, s = lane & 3;
    uint16_t* table = reinterpret_cast<uint16_t*>(smem) + c * 2048;
    Ring ring{reinterpret_cast<uint32_t*>(smem + HUF_WARP_CHUNKS * HUF_SMEM_PER_CHUNK) + lane};

    const uint32_t item_idx = blockIdx.x * HUF_WARP_CHUNKS + c;
    const bool valid = item_idx < n_items;
    DecodeItem it;
    if (valid) it = items[item_idx];
    const uint8_t* src = valid ? rd(bases, it.src) : nullptr;
    uint32_t err = ST_OK;
    uint32_t max_bits = 1, my_off = 0, my_len = 0;

    // weights header + canonical table: lane s == 0 of each chunk builds it
    // (weights.rs:34-85, tree.rs:103-177); the other three lanes help fill.
    uint32_t nsym = 0, hb = 0, hdr = 0;
    if (valid) {
        if (it.src_len < 1 || (src[0] & 0x80) == 0) err = ST_BAD_HEADER;
        else if (src[0] == 0x80) {
            if (it.src_len < 2) err = ST_BAD_HEADER;
            else { nsym = src[1] == 0 ? 256u : src[1]; hb = 2; if (nsym < 128) err = ST_BAD_HEADER; }
        } else { nsym = src[0] & 0x7F; hb = 1; }
        if (!err) {
            hdr = hb + (nsym + 1) / 2;
            if (it.src_len < hdr + 16) err = ST_BAD_HEADER;
        }
        if (!err) {
            uint64_t total = 0;
            uint32_t off = hdr + 16;
            for (uint32_t k = 0; k < 4; ++k) {
                uint32_t l = ld_u32_unaligned(src + hdr + 4 * k);
                if (k == s) { my_off = off + uint32_t(total); my_len = l; }
                total += l;
            }
            if (total != uint64_t(it.src_len - hdr - 16)) err = ST_BAD_HEADER;
        }
    }
    auto weight = [&](uint32_t i) -> uint32_t { uint8_t b = src[hb + (i >> 1)]; return (i & 1) ? (b >> 4) : (b & 0x0F); };
    uint32_t next_code[12];
    if (valid && !err) {
        uint32_t counts[12];
#pragma unroll
        for (int k = 0; k < 12; ++k) counts[k] = 0;
        uint32_t mb = 0, tot = 0;
        for (uint32_t i = 0; i < nsym; ++i) {
            uint32_t w = weight(i);
            if (w > 11) { err = ST_BAD_HEADER; break; }
            if (w) {
                tot++;
                mb = w > mb ? w : mb;
#pragma unroll
                for (int k = 1; k < 12; ++k) counts[k] += (w == uint32_t(k));
            }
        }
        if (tot == 0) err = ST_BAD_HEADER;
        max_bits = mb < 1 ? 1 : mb;
        uint32_t code = 0;
#pragma unroll
        for (int bits = 1; bits < 12; ++bits) {
            next_code[bits] = 0;
            if (uint32_t(bits) <= max_bits) {
                code = (code + counts[bits - 1]) << 1;
                if (code > (1u << bits)) err = ST_BAD_HEADER;
                next_code[bits] = code;
            }
        }
    }
    // fill with the fallback entry, then place the codes (only lane s == 0
    // walks the symbols: canonical code assignment is sequential per length)
    if (valid && !err) {
        uint32_t size = 1u << max_bits;
        uint16_t fb = uint16_t(max_bits << 8);
        for (uint32_t i = s; i < size; i += 4) table[i] = fb;
    }
    __syncwarp();
    if (valid && !err && s == 0) {
        uint16_t fb = uint16_t(max_bits << 8);
        for (uint32_t sym = 0; sym < nsym; ++sym) {
            uint32_t len = weight(sym);
            if (!len) continue;
            uint32_t cde = 0;
#pragma unroll
            for (int k = 1; k < 12; ++k) if (len == uint32_t(k)) { cde = next_code[k]; next_code[k] = cde + 1; }
            if (cde >= (1u << len)) { err = ST_BAD_HEADER; break; }
            uint32_t rev = __brev(cde) >> (32 - len);
            uint16_t entry = uint16_t((len << 8) | sym);
            for (uint32_t idx = rev; idx < (1u << max_bits); idx += (1u << len)) {
                if (table[idx] != fb && table[idx] != entry) err = ST_BAD_HEADER;
                table[idx] = entry;
            }
        }
    }
    { uint32_t be = __shfl_sync(0xFFFFFFFFu, err, c * 4); err = be > err ? be : err; }  // table errors of the builder lane reach its chunk
    __syncwarp();

    uint32_t seg_start = 0, seg_len = 0;
    if (valid) split_four_dev(it.n, s, seg_start, seg_len);
    if (valid && !err) {
        Epilogue ep = make_epilogue(bases, it);
        const uintptr_t start = reinterpret_cast<uintptr_t>(src + my_off);
        uintptr_t rp = start + my_len;  // one past the next byte to read (moves down)
        const uintptr_t lo16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_first) & ~uintptr_t(15);
        const uintptr_t hi16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_end + 15) & ~uintptr_t(15);
        // ring holds [fetched, ...): blocks are fetched downward
        uintptr_t fetched = (rp + 15) & ~uintptr_t(15);
        for (int k = 0; k < 3; ++k) { fetched -= 16; ring.put(fetched, fetch16(fetched, lo16, hi16)); }
        uint4 pending = fetch16(fetched - 16, lo16, hi16);

        uint64_t cont = 0;
        uint32_t cnt = 0;
        // byte steps until the read position is word aligned
        while ((rp & 3) && rp > start) { --rp; cont |= uint64_t(ring.byte(rp)) << cnt; cnt += 8; }
        const uint32_t mask = (1u << max_bits) - 1;
        uint64_t pos = seg_start;
        uint32_t remaining = seg_len;
        uint32_t g = remaining ? first_group(ep, pos, remaining) : 0;
        PartnerStream ps;
        bool streaming = false;
        auto refill = [&]() {
            // one aligned word (or the last partial one) when at most 32 bits are left
            if (cnt <= 32 && rp > start) {
                uint32_t w = __byte_perm(ring.word(rp - 4), 0, 0x0123);  // byte rp-1 becomes the lowest
                uint32_t take = rp - start >= 4 ? 4u : uint32_t(rp - start);
                if (take < 4) w &= (1u << (8 * take)) - 1;
                cont |= uint64_t(w) << cnt;
                cnt += 8 * take;
                rp -= take;
            }
        };
        while (remaining) {
            if (rp - fetched < 32 && fetched > start) { fetched -= 16; ring.put(fetched, pending); pending = fetch16(fetched - 16, lo16, hi16); }
            uint64_t pb[4] = {0, 0, 0, 0};
            if (streaming) ps.prefetch();
            uint64_t syms = 0;
            if (g == 8) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if ((j & 1) == 0) refill();  // two symbols need at most 22 bits, a refill leaves more than 32
                    uint32_t e = table[uint32_t(cont) & mask];
                    uint32_t nb = e >> 8;
                    if (nb > cnt) { err = ST_STREAM_UNDERRUN; nb = cnt; }  // decompress.rs:176-196
                    cont >>= nb; cnt -= nb;
                    syms |= uint64_t(e & 0xFF) << (8 * j);
                }
            } else {
                for (uint32_t j = 0; j < g; ++j) {
                    refill();
                    uint32_t e = table[uint32_t(cont) & mask];
                    uint32_t nb = e >> 8;
                    if (nb > cnt) { err = ST_STREAM_UNDERRUN; nb = cnt; }
                    cont >>= nb; cnt -= nb;
                    syms |= uint64_t(e & 0xFF) << (8 * j);
                }
            }
            if (streaming) ps.take(ep.slot, pb);
            else gather_partners(ep, pos, g, pb);
            emit_with(ep, pos, g, syms, pb);
            pos += g; remaining -= g;
            g = remaining < 8 ? remaining : 8;
            if (!streaming && remaining) { ps.start(ep, pos, it.n); streaming = true; }
        }
        // every stream must end with no unread byte and only zero bits left
        // (decompress.rs:140-144, bitstream.rs:184-186)
        while (rp > start && !err) {
            if (rp - fetched < 32 && fetched > start) { fetched -= 16; ring.put(fetched, pending); pending = fetch16(fetched - 16, lo16, hi16); }
            --rp;
            if (ring.byte(rp)) err = ST_NOT_CONSUMED;
        }
        if (!err && cont != 0) err = ST_NOT_CONSUMED;
    }
    if (err) atomicMax(&status[it.id], err);
}

// ---- tANS ------------------------------------------------------------------
// One stream per chunk: lane 4k decodes chunk k of the warp, all lanes help
// build the 2048-entry table (symbol | nb<<8 | baseline<<16).
constexpr int TANS_WARP_CHUNKS = 8;
constexpr int TANS_SMEM_PER_CHUNK = 2048 * 4 + 2048;  // decode table + spread symbols
constexpr int TANS_SMEM = TANS_WARP_CHUNKS * TANS_SMEM_PER_CHUNK;

__global__ void __launch_bounds__(32) tans_decode_kernel(const DecodeItem* __restrict__ items, uint32_t n_items, Bases bases, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t lane = threadIdx.x;
    uint32_t* dt_all = reinterpret_cast<uint32_t*>(smem);
    uint8_t* spread_all = smem + TANS_WARP_CHUNKS * 2048 * 4;
    for (uint32_t c = 0; c < TANS_WARP_CHUNKS; ++c) {
        const uint32_t item_idx = blockIdx.x * TANS_WARP_CHUNKS + c;
        if (item_idx >= n_items) break;
        const DecodeItem it = items[item_idx];
        const uint8_t* src = rd(bases, it.src);
        uint32_t* dt = dt_all + c * 2048;
        uint8_t* sp = spread_all + c * 2048;
        uint32_t err = ST_OK;
        // header (mod.rs:388-425): every lane parses it redundantly
        uint32_t nsym = 0;
        if (it.src_len < 3 || src[0] != 11) err = ST_BAD_HEADER;
        else {
            nsym = uint32_t(src[1]) | uint32_t(src[2]) << 8;
            if (nsym < 2 || nsym > 256 || 3 + nsym * 3 + 8 > it.src_len) err = ST_BAD_HEADER;
        }
        if (err) { if (lane == 0) atomicMax(&status[it.id], err); continue; }
        // lane 0 builds the tables: the spread walks a running position and
        // the decode entries count earlier slots of the same symbol, so both
        // are sequential (mod.rs:199-211,346-369).
        if (lane == 0) {
            uint32_t norm[256];
            for (uint32_t i = 0; i < 256; ++i) norm[i] = 0;
            uint32_t sum = 0;
            for (uint32_t i = 0; i < nsym; ++i) {
                uint32_t sy = src[3 + 3 * i], fr = uint32_t(src[4 + 3 * i]) | uint32_t(src[5 + 3 * i]) << 8;
                if (fr == 0 || norm[sy] != 0) { err = ST_BAD_HEADER; break; }  // mod.rs:404-411
                norm[sy] = fr;
                sum += fr;
            }
            if (!err && sum != 2048) err = ST_BAD_HEADER;
            if (!err) {
                uint32_t pos = 0;
                for (uint32_t sy = 0; sy < 256; ++sy)
                    for (uint32_t k = 0; k < norm[sy]; ++k) { sp[pos] = uint8_t(sy); pos = (pos + 1283u) & 2047u; }
                for (uint32_t u = 0; u < 2048; ++u) {
                    uint32_t sy = sp[u];
                    uint32_t x = norm[sy]++;
                    uint32_t nb = 11 - (31 - __clz(x));
                    uint32_t baseline = (x << nb) - 2048;
                    dt[u] = sy | (nb << 8) | (baseline << 16);
                }
            }
        }
        err = __shfl_sync(0xFFFFFFFFu, err, 0);
        if (err) { if (lane == 0) atomicMax(&status[it.id], err); continue; }
        __syncwarp();
        if (lane == 0) {
            Epilogue ep = make_epilogue(bases, it);
            const uint8_t* hp = src + 3 + nsym * 3;
            uint64_t total_bits = uint64_t(ld_u32_unaligned(hp)) | uint64_t(ld_u32_unaligned(hp + 4)) << 32;
            const uint8_t* bs = hp + 8;
            uint64_t bslen = it.src_len - (3 + nsym * 3 + 8);
            if (total_bits > bslen * 8) err = ST_BAD_HEADER;
            else {
                // LIFO reader (mod.rs:118-147): bits [bpos-cnt, bpos) sit right-aligned in `cont`
                uint64_t nbytes = (total_bits + 7) >> 3;  // bytes that hold declared bits
                uint64_t bi = nbytes;                      // next byte to load is bs[bi-1]
                uint64_t cont = 0; uint32_t cnt = 0;
                uint32_t top = uint32_t(total_bits & 7);
                if (top) { --bi; cont = bs[bi] & ((1u << top) - 1); cnt = top; }
                auto read = [&](uint32_t nb) -> uint32_t {
                    if (nb == 0) return 0;
                    while (cnt < nb && bi > 0) { --bi; cont = (cont << 8) | bs[bi]; cnt += 8; }
                    if (cnt < nb) { err = ST_STREAM_UNDERRUN; return 0; }
                    uint32_t v = uint32_t(cont >> (cnt - nb)) & ((1u << nb) - 1);
                    cnt -= nb;
                    cont &= (cnt ? ((1ull << cnt) - 1) : 0ull);
                    return v;
                };
                uint32_t state = read(11);
                uint64_t pos = 0;
                uint32_t remaining = it.n;
                uint32_t g = first_group(ep, pos, remaining);
                while (remaining && !err) {
                    uint64_t syms = 0;
                    for (uint32_t j = 0; j < g; ++j) {
                        uint32_t e = dt[state & 2047u];
                        syms |= uint64_t(e & 0xFF) << (8 * j);
                        state = (e >> 16) + read((e >> 8) & 0xFF);
                        if (state >= 2048) { err = ST_STREAM_UNDERRUN; state = 0; }
                    }
                    emit(ep, pos, g, syms);
                    pos += g; remaining -= g;
                    g = remaining < 8 ? remaining : 8;
                }
                if (!err && (cnt != 0 || bi != 0 || state != 0)) err = ST_NOT_CONSUMED;  // mod.rs:442-449
            }
            if (err) atomicMax(&status[it.id], err);
        }
        __syncwarp();
    }
}

// ---- Order1ScaleAC ---------------------------------------------------------
// One range-coder stream per chunk.  The warp first turns the chunk's PMFs
// into cumulative tables in the scratch arena (u16, 257 per context), then
// lane 0 decodes.
__global__ void __launch_bounds__(32) o1sac_decode_kernel(const DecodeItem* __restrict__ items, uint32_t n_items, Bases bases, uint32_t* __restrict__ status) {
    const uint32_t lane = threadIdx.x;
    const uint32_t item_idx = blockIdx.x;
    if (item_idx >= n_items) return;
    const DecodeItem it = items[item_idx];
    const uint8_t* st = rd(bases, it.state);
    uint32_t err = ST_OK;
    __shared__ uint8_t bitmap[32];
    __shared__ uint8_t rank_of[256];
    if (it.state_version != 1 || it.state_len < 32 + 512) err = ST_BAD_STATE;
    uint32_t pop = 0;
    if (!err) {
        bitmap[lane] = st[lane];
        __syncwarp();
        for (int i = 0; i < 32; ++i) pop += __popc(uint32_t(bitmap[i]));
        if (it.state_len != 32 + 512 + pop * 512) err = ST_BAD_STATE;
    }
    if (err) { if (lane == 0) atomicMax(&status[it.id], err); return; }
    // rank of every context (order1_scale_ac.rs:95-103)
    for (uint32_t p = lane; p < 256; p += 32) {
        uint32_t r = 0;
        for (uint32_t b = 0; b < (p >> 3); ++b) r += __popc(uint32_t(bitmap[b]));
        r += __popc(uint32_t(bitmap[p >> 3]) & ((1u << (p & 7)) - 1));
        rank_of[p] = uint8_t(r);  // ranks 0..255 fit: a present context has rank <= 255
    }
    // cumulative tables: table t (0 = marginal, 1+r = row r) = 257 u16 at work + t*514
    uint16_t* cum = reinterpret_cast<uint16_t*>(wr(bases, it.work));
    for (uint32_t t = lane; t < 1 + pop; t += 32) {
        const uint8_t* pm = st + 32 + t * 512;
        uint16_t* ct = cum + t * 257;
        uint32_t acc = 0; bool zero = false;
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t v = uint32_t(pm[2 * i]) | uint32_t(pm[2 * i + 1]) << 8;
            zero |= v == 0;
            ct[i] = uint16_t(acc);
            acc += v;
        }
        ct[256] = uint16_t(acc);
        if (zero || acc != 4096) err = ST_BAD_STATE;  // quantize.rs:53-71
    }
    err = __reduce_max_sync(0xFFFFFFFFu, err);
    __syncwarp();
    __threadfence_block();
    if (err) { if (lane == 0) atomicMax(&status[it.id], err); return; }
    if (lane != 0) return;

    Epilogue ep = make_epilogue(bases, it);
    const uint8_t* src = rd(bases, it.src);
    const uint32_t slen = it.src_len;
    // range_coder.rs:137-155
    uint64_t code = 0; uint32_t rpos = 0;
    for (; rpos < 5; ++rpos) code = (code << 8) | (rpos < slen ? src[rpos] : 0);
    uint32_t low = 0;
    uint64_t range = 0xFFFFFFFFull;
    const uint32_t row_len = it.row_len ? it.row_len : (it.n ? it.n : 1);
    uint32_t row_pos = 0; int prev = -1;
    uint64_t pos = 0;
    uint32_t remaining = it.n;
    uint32_t g = remaining ? first_group(ep, pos, remaining) : 0;
    while (remaining) {
        uint64_t syms = 0;
        for (uint32_t j = 0; j < g; ++j) {
            if (row_pos == 0) prev = -1;
            const uint16_t* ct = cum;
            if (prev >= 0 && ((bitmap[prev >> 3] >> (prev & 7)) & 1)) ct = cum + (1 + rank_of[prev]) * 257;
            uint32_t rpt = uint32_t(range >> 12);  // range / 4096
            uint32_t offset = uint32_t(code) - low;
            uint32_t target = offset / rpt;
            if (target > 4095) target = 4095;
            uint32_t lo = 0, hi = 256;  // order1_scale_ac.rs:474-486
            while (lo + 1 < hi) { uint32_t mid = (lo + hi) >> 1; if (ct[mid] <= target) lo = mid; else hi = mid; }
            uint32_t cumv = ct[lo], prob = uint32_t(ct[lo + 1]) - cumv;
            low = low + cumv * rpt;  // & 0xFFFFFFFF by width
            range = uint64_t(prob) * rpt;
            while (range < (1ull << 24)) {
                uint32_t b = rpos < slen ? src[rpos] : 0;
                ++rpos;
                code = ((code & 0xFFFFFFFFFFull) << 8) | b;
                low = (low & 0x00FFFFFFu) << 8;
                range <<= 8;
            }
            syms |= uint64_t(lo) << (8 * j);
            prev = int(lo);
            row_pos = row_pos + 1 == row_len ? 0 : row_pos + 1;
        }
        emit(ep, pos, g, syms);
        pos += g; remaining -= g;
        g = remaining < 8 ? remaining : 8;
    }
}

// ---- stand-alone merge / copy ---------------------------------------------
constexpr uint32_t MERGE_TILE = 8192;  // elements per CTA
__global__ void __launch_bounds__(256) merge_kernel(const MergeItem* __restrict__ items, const uint32_t* __restrict__ tile_first, uint32_t n_items, Bases bases) {
    // tile_first[i] = first tile index of item i (n_items + 1 entries); find the item by binary search
    uint32_t tile = blockIdx.x;
    uint32_t lo = 0, hi = n_items;
    while (lo + 1 < hi) { uint32_t mid = (lo + hi) >> 1; if (tile_first[mid] <= tile) lo = mid; else hi = mid; }
    const MergeItem it = items[lo];
    uint64_t base = uint64_t(tile - tile_first[lo]) * MERGE_TILE;
    uint32_t n = it.n - base < MERGE_TILE ? uint32_t(it.n - base) : MERGE_TILE;
    int np = kind_planes(int(it.kind));
    const uint8_t* src[4];
    for (int p = 0; p < 4; ++p) src[p] = p < np ? rd(bases, it.src[p]) + base : nullptr;
    uint8_t* dst = wr(bases, it.dst) + base * uint64_t(kind_elem_bytes(int(it.kind)));
    // groups are aligned to the destination: a short head, full groups, a tail
    uintptr_t a = reinterpret_cast<uintptr_t>(dst) / uint32_t(kind_elem_bytes(int(it.kind)));
    uint32_t head = uint32_t((8 - (a & 7)) & 7);
    if (head > n) head = n;
    uint32_t full = (n - head) >> 3;
    for (uint32_t gidx = threadIdx.x; gidx < full + 2; gidx += blockDim.x) {
        uint32_t pos, count;
        if (gidx == 0) { pos = 0; count = head; }
        else if (gidx <= full) { pos = head + (gidx - 1) * 8; count = 8; }
        else { pos = head + full * 8; count = n - pos; }
        if (count == 0) continue;
        uint64_t b[4] = {0, 0, 0, 0};
        for (int p = 0; p < np; ++p) b[p] = count == 8 ? ld8_unaligned(src[p] + pos) : ld_bytes(src[p] + pos, count);
        compose_store(int(it.kind), dst, pos, count, b);
    }
}

// ---- integrity -------------------------------------------------------------
// CRC-32/IEEE in the reflected form (poly 0xEDB88320).  Each thread takes the
// remainder of one run of plane bytes from state 0, multiplies it by
// x^(8*bytes_after) mod P and XORs it into the plane's accumulator; the host
// adds the init/final terms, which depend only on the plane length.
__host__ __device__ __forceinline__ uint32_t gf2_mulmod(uint32_t a, uint32_t b) {
    uint32_t p = 0;
    for (uint32_t m = 1u << 31; m; m >>= 1) {
        if (a & m) p ^= b;
        b = (b & 1) ? (b >> 1) ^ 0xEDB88320u : b >> 1;
    }
    return p;
}
struct CrcTables { uint32_t byte_table[256]; uint32_t x2n[64]; };  // x2n[k] = x^(2^k) mod P

__host__ __device__ __forceinline__ uint32_t x_pow_8n(const uint32_t* x2n, uint64_t nbytes) {
    uint32_t p = 1u << 31;  // x^0
    uint32_t k = 3;         // x^(8n) = x^(n * 2^3)
    while (nbytes) { if (nbytes & 1) p = gf2_mulmod(x2n[k & 63], p); nbytes >>= 1; ++k; }
    return p;
}

__global__ void __launch_bounds__(128) crc_planes_kernel(const VerifyTensor* __restrict__ tensors, uint32_t n_tensors, uint64_t n_runs, Bases bases,
                                                         const CrcTables* __restrict__ tabs, uint32_t* __restrict__ acc) {
    __shared__ uint32_t T[256];
    __shared__ uint32_t X[64];
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) T[i] = tabs->byte_table[i];
    if (threadIdx.x < 64) X[threadIdx.x] = tabs->x2n[threadIdx.x];
    __syncthreads();
    uint64_t run = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (run >= n_runs) return;
    uint32_t lo = 0, hi = n_tensors;
    while (lo + 1 < hi) { uint32_t mid = (lo + hi) >> 1; if (tensors[mid].first_run <= run) lo = mid; else hi = mid; }
    const VerifyTensor t = tensors[lo];
    uint64_t first = (run - t.first_run) * VERIFY_RUN;
    uint32_t n = t.n_elems - first < VERIFY_RUN ? uint32_t(t.n_elems - first) : VERIFY_RUN;
    const uint8_t* out = rd(bases, t.out);
    uint32_t c[4] = {0, 0, 0, 0};
    switch (t.kind) {
        case K_PASS:
            for (uint32_t i = 0; i < n; ++i) c[0] = T[(c[0] ^ out[first + i]) & 0xFF] ^ (c[0] >> 8);
            break;
        case K_M16:
            for (uint32_t i = 0; i < n; ++i) {
                uint32_t v = uint32_t(out[2 * (first + i)]) | uint32_t(out[2 * (first + i) + 1]) << 8;
                uint32_t r = ((v << 1) & 0xFF00u) | ((v >> 8) & 0x0080u) | (v & 0x007Fu);
                c[0] = T[(c[0] ^ r) & 0xFF] ^ (c[0] >> 8);
                c[1] = T[(c[1] ^ (r >> 8)) & 0xFF] ^ (c[1] >> 8);
            }
            break;
        case K_M32:
            for (uint32_t i = 0; i < n; ++i) {
                uint32_t v = ld_u32_unaligned(out + 4 * (first + i));
                uint32_t r = ((v << 1) & 0xFF000000u) | ((v >> 8) & 0x00800000u) | (v & 0x007FFFFFu);
#pragma unroll
                for (int p = 0; p < 4; ++p) c[p] = T[(c[p] ^ (r >> (8 * p))) & 0xFF] ^ (c[p] >> 8);
            }
            break;
        default:
            for (uint32_t i = 0; i < n; ++i) {
                uint32_t v = out[first + i];
                uint32_t r = t.kind == K_E4M3 ? (((v & 0x78) << 1) | ((v & 0x80) >> 4) | (v & 0x07)) : (((v & 0x7C) << 1) | ((v & 0x80) >> 5) | (v & 0x03));
                c[0] = T[(c[0] ^ (r >> 4)) & 0xFF] ^ (c[0] >> 8);
                c[1] = T[(c[1] ^ (r & 0x0F)) & 0xFF] ^ (c[1] >> 8);
            }
            break;
    }
    uint32_t shift = x_pow_8n(X, t.n_elems - first - n);
    int np = kind_planes(int(t.kind));
    for (int p = 0; p < np; ++p) atomicXor(&acc[t.acc_base + p], gf2_mulmod(shift, c[p]));
}

// XXH64 (seed 0) of each tensor: the four accumulators of the stripe loop are
// independent, so four lanes share a tensor; the rest is sequential by design
// of the hash.
__device__ __forceinline__ uint64_t rotl64(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
__device__ __forceinline__ uint64_t ld_u64_unaligned(const uint8_t* p) { return uint64_t(ld_u32_unaligned(p)) | uint64_t(ld_u32_unaligned(p + 4)) << 32; }

__global__ void __launch_bounds__(32) xxh64_kernel(const HashItem* __restrict__ items, uint32_t n_items, Bases bases, uint64_t* __restrict__ out) {
    const uint64_t P1 = 11400714785074694791ull, P2 = 14029467366897019727ull, P3 = 1609587929392839161ull, P4 = 9650029242287828579ull,
                   P5 = 2870177450012600261ull;
    uint32_t lane = threadIdx.x, sub = lane & 3;
    uint32_t idx = blockIdx.x * 8 + (lane >> 2);
    bool valid = idx < n_items;
    HashItem it = valid ? items[idx] : HashItem{0, 0};
    const uint8_t* p = valid ? rd(bases, it.data) : nullptr;
    uint64_t len = it.len;
    uint64_t v = sub == 0 ? P1 + P2 : sub == 1 ? P2 : sub == 2 ? 0 : 0 - P1;
    uint64_t stripes = len / 32;
    const bool aligned = (reinterpret_cast<uintptr_t>(p) & 7) == 0;
    for (uint64_t s = 0; s < stripes; ++s) {
        const uint8_t* q = p + s * 32 + sub * 8;
        uint64_t in = aligned ? *reinterpret_cast<const uint64_t*>(q) : ld_u64_unaligned(q);
        v += in * P2; v = rotl64(v, 31); v *= P1;
    }
    uint64_t v1 = __shfl_sync(0xFFFFFFFFu, v, (lane & ~3u) + 0), v2 = __shfl_sync(0xFFFFFFFFu, v, (lane & ~3u) + 1),
             v3 = __shfl_sync(0xFFFFFFFFu, v, (lane & ~3u) + 2), v4 = __shfl_sync(0xFFFFFFFFu, v, (lane & ~3u) + 3);
    if (!valid || sub != 0) return;
    auto round = [&](uint64_t acc, uint64_t in) { acc += in * P2; acc = rotl64(acc, 31); return acc * P1; };
    auto merge = [&](uint64_t h, uint64_t x) { x = round(0, x); h ^= x; return h * P1 + P4; };
    uint64_t h;
    if (len >= 32) {
        h = rotl64(v1, 1) + rotl64(v2, 7) + rotl64(v3, 12) + rotl64(v4, 18);
        h = merge(h, v1); h = merge(h, v2); h = merge(h, v3); h = merge(h, v4);
    } else h = P5;
    h += len;
    const uint8_t* q = p + stripes * 32;
    const uint8_t* end = p + len;
    while (q + 8 <= end) { h ^= round(0, ld_u64_unaligned(q)); h = rotl64(h, 27) * P1 + P4; q += 8; }
    if (q + 4 <= end) { h ^= uint64_t(ld_u32_unaligned(q)) * P1; h = rotl64(h, 23) * P2 + P3; q += 4; }
    while (q < end) { h ^= uint64_t(*q) * P5; h = rotl64(h, 11) * P1; ++q; }
    h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
    out[idx] = h;
}

}  // namespace ptwm
