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

__device__ __forceinline__ void stg256(void* p, uint4 a, uint4 b);

// ---- element composition ---------------------------------------------------
__device__ __forceinline__ uint32_t revert16x2(uint32_t r) {  // split/dtype16.rs:20-25
    return ((r << 8) & 0x80008000u) | ((r >> 1) & 0x7F807F80u) | (r & 0x007F007Fu);
}
// Four 16-bit elements from four bytes of the low plane ([S M7]) and four of
// the high plane (E8): the bit reorder done on the packed planes, then the
// interleave.  Same result as revert16x2 on the interleaved words.
__device__ __forceinline__ void compose16x4(uint32_t lo, uint32_t hi, uint32_t& v0, uint32_t& v1) {
    uint32_t oh = (lo & 0x80808080u) | ((hi >> 1) & 0x7F7F7F7Fu);
    uint32_t ol = ((hi << 7) & 0x80808080u) | (lo & 0x7F7F7F7Fu);
    v0 = __byte_perm(ol, oh, 0x5140);
    v1 = __byte_perm(ol, oh, 0x7362);
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
            compose16x4(l0, h0, v.x, v.y);
            compose16x4(l1, h1, v.z, v.w);
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
            if (count == 8 && (reinterpret_cast<uintptr_t>(p) & 31) == 0) {
                stg256(p, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));  // one sector per lane and instruction
            } else if (count == 8 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
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

// 256-bit global accesses (sm_100): a lane that walks its own stream touches
// one 32-byte sector per instruction instead of half of one, which halves the
// load/store-pipe cost of these scattered accesses.
struct Block32 { uint32_t w[8]; };
__device__ __forceinline__ Block32 ldg256(const void* p) {
    Block32 b;
    asm("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(b.w[0]), "=r"(b.w[1]), "=r"(b.w[2]), "=r"(b.w[3]), "=r"(b.w[4]), "=r"(b.w[5]), "=r"(b.w[6]), "=r"(b.w[7])
        : "l"(p));
    return b;
}
__device__ __forceinline__ void stg256(void* p, uint4 a, uint4 b) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}
// Aligned 32-byte block at `a`; bytes outside [lo, hi) read as zero and are not touched.
__device__ __forceinline__ Block32 load_block_guarded(uintptr_t a, uintptr_t lo, uintptr_t hi) {
    if (a >= lo && a + 32 <= hi) return ldg256(reinterpret_cast<const void*>(a));
    Block32 b;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            uintptr_t q = a + 4 * k + i;
            if (q >= lo && q < hi) v |= uint32_t(__ldg(reinterpret_cast<const uint8_t*>(q))) << (8 * i);
        }
        b.w[k] = v;
    }
    return b;
}
// The 32 bytes that start `off` (0..31) bytes into the 64 bytes (cur, nxt), as eight words.
__device__ __forceinline__ void extract32(const Block32& cur, const Block32& nxt, uint32_t off, uint32_t out[8]) {
    uint32_t a[16], b[12], c[10], d[9];
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = cur.w[i]; a[8 + i] = nxt.w[i]; }
    const bool j4 = off & 16, j2 = off & 8, j1 = off & 4;
#pragma unroll
    for (int i = 0; i < 12; ++i) b[i] = j4 ? a[i + 4] : a[i];
#pragma unroll
    for (int i = 0; i < 10; ++i) c[i] = j2 ? b[i + 2] : b[i];
#pragma unroll
    for (int i = 0; i < 9; ++i) d[i] = j1 ? c[i + 1] : c[i];
    const uint32_t sel = 0x3210u + 0x1111u * (off & 3u);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __byte_perm(d[i], d[i + 1], sel);
}

// ---- fast output loops of a decoding lane -----------------------------------
// `dec8(s_lo, s_hi)` decodes the lane's next eight symbols (symbol j in byte
// j & 3 of s_lo for j < 4, of s_hi above); the loops below place them.
//
// Fused lane, 16-bit elements, one partner plane.  Rounds of 32 elements: the
// partner bytes come as aligned 32-byte blocks two rounds ahead of their use
// (cur, nxt, and one in flight), the composed elements leave as two 32-byte
// stores.  Blocks that are not wholly inside the partner's chunk are never read
// whole, so nothing outside the caller's buffers is touched.  What does not
// fill a round is left to the caller.
template <class Dec8>
__device__ __forceinline__ void fused16_rounds(const Epilogue& ep, uint32_t chunk_n, uint32_t& pos, uint32_t& remaining, Dec8&& dec8) {
    if (remaining >= 8 && ((reinterpret_cast<uintptr_t>(ep.dst) + size_t(pos) * 2) & 31) != 0) {
        uint32_t s_lo, s_hi;  // one more group of eight brings the destination to a 32-byte boundary
        dec8(s_lo, s_hi);
        emit(ep, pos, 8, uint64_t(s_lo) | uint64_t(s_hi) << 32);
        pos += 8; remaining -= 8;
    }
    const uintptr_t p_lo = reinterpret_cast<uintptr_t>(ep.partner[0]), p_hi = p_lo + chunk_n;
    const uintptr_t pa = p_lo + pos;
    uintptr_t q = pa & ~uintptr_t(31);
    uint8_t* out = ep.dst + size_t(pos) * 2;
    // round r reads the block at q + 32 (r + 2): it must end inside the chunk
    uint32_t rounds = 0;
    if ((reinterpret_cast<uintptr_t>(out) & 31) == 0 && q + 96 <= p_hi) {
        rounds = uint32_t((p_hi - q - 96) >> 5) + 1;
        if (rounds > (remaining >> 5)) rounds = remaining >> 5;
    }
    if (!rounds) return;
    const uint32_t off = uint32_t(pa & 31);
    const bool low_plane = ep.slot == 0;  // the lane decodes the low bytes, the partner holds the high bytes
    Block32 cur = load_block_guarded(q, p_lo, p_hi), nxt = ldg256(reinterpret_cast<const void*>(q + 32));
    for (uint32_t r = 0; r < rounds; ++r) {
        const Block32 ahead = ldg256(reinterpret_cast<const void*>(q + 64));
        uint32_t pw[8];
        uint4 v[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint32_t s_lo, s_hi;
            dec8(s_lo, s_hi);
            if (g == 0) extract32(cur, nxt, off, pw);
            if (low_plane) { compose16x4(s_lo, pw[2 * g], v[g].x, v[g].y); compose16x4(s_hi, pw[2 * g + 1], v[g].z, v[g].w); }
            else { compose16x4(pw[2 * g], s_lo, v[g].x, v[g].y); compose16x4(pw[2 * g + 1], s_hi, v[g].z, v[g].w); }
        }
        stg256(out, v[0], v[1]);
        stg256(out + 32, v[2], v[3]);
        out += 64; q += 32;
        cur = nxt; nxt = ahead;
    }
    pos += rounds * 32; remaining -= rounds * 32;
}
// Fused lane, fp8 elements: the two nibble planes (one nibble per byte) of 32 elements become one 32-byte store.
__device__ __forceinline__ uint32_t compose_fp8x4(uint32_t hi, uint32_t lo, bool e4m3) {  // split/dtype8.rs:39-44,57-62 on four elements
    uint32_t r = ((hi & 0x0F0F0F0Fu) << 4) | (lo & 0x0F0F0F0Fu);
    return e4m3 ? ((r & 0xF0F0F0F0u) >> 1) | ((r & 0x08080808u) << 4) | (r & 0x07070707u)
                : ((r & 0xF8F8F8F8u) >> 1) | ((r & 0x04040404u) << 5) | (r & 0x03030303u);
}
template <class Dec8>
__device__ __forceinline__ void fused8_rounds(const Epilogue& ep, uint32_t chunk_n, uint32_t& pos, uint32_t& remaining, Dec8&& dec8) {
    while (remaining >= 8 && ((reinterpret_cast<uintptr_t>(ep.dst) + pos) & 31) != 0) {
        uint32_t s_lo, s_hi;  // groups of eight up to a 32-byte boundary of the destination
        dec8(s_lo, s_hi);
        emit(ep, pos, 8, uint64_t(s_lo) | uint64_t(s_hi) << 32);
        pos += 8; remaining -= 8;
    }
    const uintptr_t p_lo = reinterpret_cast<uintptr_t>(ep.partner[0]), p_hi = p_lo + chunk_n;
    const uintptr_t pa = p_lo + pos;
    uintptr_t q = pa & ~uintptr_t(31);
    uint8_t* out = ep.dst + pos;
    uint32_t rounds = 0;
    if ((reinterpret_cast<uintptr_t>(out) & 31) == 0 && q + 96 <= p_hi) {
        rounds = uint32_t((p_hi - q - 96) >> 5) + 1;
        if (rounds > (remaining >> 5)) rounds = remaining >> 5;
    }
    if (!rounds) return;
    const uint32_t off = uint32_t(pa & 31);
    const bool high_plane = ep.slot == 0, e4m3 = ep.kind == K_E4M3;  // plane 0 holds the high nibbles
    Block32 cur = load_block_guarded(q, p_lo, p_hi), nxt = ldg256(reinterpret_cast<const void*>(q + 32));
    for (uint32_t r = 0; r < rounds; ++r) {
        const Block32 ahead = ldg256(reinterpret_cast<const void*>(q + 64));
        uint32_t pw[8], v[8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint32_t s_lo, s_hi;
            dec8(s_lo, s_hi);
            if (g == 0) extract32(cur, nxt, off, pw);
            v[2 * g] = high_plane ? compose_fp8x4(s_lo, pw[2 * g], e4m3) : compose_fp8x4(pw[2 * g], s_lo, e4m3);
            v[2 * g + 1] = high_plane ? compose_fp8x4(s_hi, pw[2 * g + 1], e4m3) : compose_fp8x4(pw[2 * g + 1], s_hi, e4m3);
        }
        stg256(out, make_uint4(v[0], v[1], v[2], v[3]), make_uint4(v[4], v[5], v[6], v[7]));
        out += 32; q += 32;
        cur = nxt; nxt = ahead;
    }
    pos += rounds * 32; remaining -= rounds * 32;
}
// Fused lane, 32-bit elements, the lane decoding plane 3 (the exponent byte, the usual case: the three mantissa
// planes are stored raw or were decoded before).  Rounds of 16 elements: each of the three partner planes arrives as
// aligned 16-byte blocks one round ahead, the composed elements leave as two 32-byte stores.
__device__ __forceinline__ uint4 load_block16_guarded(uintptr_t a, uintptr_t lo, uintptr_t hi) {
    if (a >= lo && a + 16 <= hi) return __ldg(reinterpret_cast<const uint4*>(a));
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) {
            uintptr_t q = a + 4 * k + i;
            if (q >= lo && q < hi) v |= uint32_t(__ldg(reinterpret_cast<const uint8_t*>(q))) << (8 * i);
        }
        w[k] = v;
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
// The 16 bytes that start `off` (0..15) bytes into the 32 bytes (cur, nxt), as four words.
__device__ __forceinline__ void extract16(const uint4& cur, const uint4& nxt, uint32_t off, uint32_t out[4]) {
    const uint32_t a[8] = {cur.x, cur.y, cur.z, cur.w, nxt.x, nxt.y, nxt.z, nxt.w};
    uint32_t b[6], c[5];
    const bool j2 = off & 8, j1 = off & 4;
#pragma unroll
    for (int i = 0; i < 6; ++i) b[i] = j2 ? a[i + 2] : a[i];
#pragma unroll
    for (int i = 0; i < 5; ++i) c[i] = j1 ? b[i + 1] : b[i];
    const uint32_t sel = 0x3210u + 0x1111u * (off & 3u);
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = __byte_perm(c[i], c[i + 1], sel);
}
template <class Dec8>
__device__ __forceinline__ void fused32_rounds(const Epilogue& ep, uint32_t chunk_n, uint32_t& pos, uint32_t& remaining, Dec8&& dec8) {
    uint8_t* out = ep.dst + size_t(pos) * 4;
    uintptr_t q[3], lo[3], hi[3];
    uint32_t off[3], rounds = remaining >> 4;
    if (reinterpret_cast<uintptr_t>(out) & 31) rounds = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        lo[j] = reinterpret_cast<uintptr_t>(ep.partner[j]); hi[j] = lo[j] + chunk_n;
        const uintptr_t pa = lo[j] + pos;
        q[j] = pa & ~uintptr_t(15); off[j] = uint32_t(pa & 15);
        // round r reads the block at q + 16 (r + 2): it must end inside the chunk
        const uint32_t fit = q[j] + 48 <= hi[j] ? uint32_t((hi[j] - q[j] - 48) >> 4) + 1 : 0;
        rounds = fit < rounds ? fit : rounds;
    }
    if (!rounds) return;
    uint4 cur[3], nxt[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) { cur[j] = load_block16_guarded(q[j], lo[j], hi[j]); nxt[j] = __ldg(reinterpret_cast<const uint4*>(q[j] + 16)); }
    for (uint32_t r = 0; r < rounds; ++r) {
        uint4 ahead[3];
#pragma unroll
        for (int j = 0; j < 3; ++j) ahead[j] = __ldg(reinterpret_cast<const uint4*>(q[j] + 32));
        uint32_t sy[4], pw[3][4], w[16];
        dec8(sy[0], sy[1]);
        dec8(sy[2], sy[3]);
#pragma unroll
        for (int j = 0; j < 3; ++j) extract16(cur[j], nxt[j], off[j], pw[j]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // four elements: bytes 0..2 from the partner planes, byte 3 from this lane (transforms/fusion.rs:287-292)
            const uint32_t t0 = __byte_perm(pw[0][k], pw[1][k], 0x5140), t1 = __byte_perm(pw[2][k], sy[k], 0x5140);
            const uint32_t t2 = __byte_perm(pw[0][k], pw[1][k], 0x7362), t3 = __byte_perm(pw[2][k], sy[k], 0x7362);
            w[4 * k + 0] = revert32(__byte_perm(t0, t1, 0x5410));
            w[4 * k + 1] = revert32(__byte_perm(t0, t1, 0x7632));
            w[4 * k + 2] = revert32(__byte_perm(t2, t3, 0x5410));
            w[4 * k + 3] = revert32(__byte_perm(t2, t3, 0x7632));
        }
        stg256(out, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
        stg256(out + 32, make_uint4(w[8], w[9], w[10], w[11]), make_uint4(w[12], w[13], w[14], w[15]));
        out += 64;
#pragma unroll
        for (int j = 0; j < 3; ++j) { cur[j] = nxt[j]; nxt[j] = ahead[j]; q[j] += 16; }
    }
    pos += rounds * 16; remaining -= rounds * 16;
}
// Plain lane: eight symbols are eight bytes of the plane; 32 bytes per store.
template <class Dec8>
__device__ __forceinline__ void plain_rounds(const Epilogue& ep, uint32_t& pos, uint32_t& remaining, Dec8&& dec8) {
    uint8_t* out = ep.dst + pos;
    if (reinterpret_cast<uintptr_t>(out) & 7) return;
    while (remaining >= 8 && (reinterpret_cast<uintptr_t>(out) & 31) != 0) {
        uint32_t s_lo, s_hi;
        dec8(s_lo, s_hi);
        *reinterpret_cast<uint2*>(out) = make_uint2(s_lo, s_hi);
        out += 8; pos += 8; remaining -= 8;
    }
    const uint32_t rounds = remaining >> 5;
    for (uint32_t r = 0; r < rounds; ++r) {
        uint4 a, b;
        dec8(a.x, a.y); dec8(a.z, a.w); dec8(b.x, b.y); dec8(b.z, b.w);
        stg256(out, a, b);
        out += 32;
    }
    pos += rounds * 32; remaining -= rounds * 32;
}
// Other fused kinds: partner words streamed one group ahead, 128-bit stores.
template <class Dec8>
__device__ __forceinline__ void fused_groups(const Epilogue& ep, uint32_t chunk_n, uint32_t& pos, uint32_t& remaining, Dec8&& dec8) {
    if (remaining < 8) return;
    PartnerStream ps;
    ps.start(ep, pos, chunk_n);
    while (remaining >= 8) {
        uint32_t s_lo, s_hi;
        uint64_t pb[4] = {0, 0, 0, 0};
        ps.prefetch();
        dec8(s_lo, s_hi);
        ps.take(ep.slot, pb);
        emit_with(ep, pos, 8, uint64_t(s_lo) | uint64_t(s_hi) << 32, pb);
        pos += 8; remaining -= 8;
    }
}
template <class Dec8>
__device__ __forceinline__ void fast_groups(const Epilogue& ep, uint32_t chunk_n, uint32_t& pos, uint32_t& remaining, Dec8&& dec8) {
    if (!ep.fused) plain_rounds(ep, pos, remaining, dec8);
    else if (ep.kind == K_M16) fused16_rounds(ep, chunk_n, pos, remaining, dec8);
    else if (ep.kind == K_E4M3 || ep.kind == K_E5M2) fused8_rounds(ep, chunk_n, pos, remaining, dec8);
    else {
        if (ep.kind == K_M32 && ep.slot == 3) fused32_rounds(ep, chunk_n, pos, remaining, dec8);
        fused_groups(ep, chunk_n, pos, remaining, dec8);  // the other plane orders, and what the rounds left
    }
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
// How many distinct symbols a chunk may hold for the kernel that keeps a copy
// of the symbol list per lane (two pad entries come on top).
constexpr uint32_t RANS_NARROW_SYMBOLS = 38;
// From this many distinct symbols on a chunk counts as nearly incompressible (packed fp4 values, mantissa-like bytes).
constexpr uint32_t RANS_DENSE_SYMBOLS = 96;
// Shared memory per chunk:
//  * a rank table over the 2048 slots: 128 words of (16-bit boundary bitmap,
//    boundaries before the word << 16).  Bit i of a bitmap is set when slot
//    16 w + i is the first slot of a symbol, so the symbol covering a slot is
//    number count + popc(bits up to the slot) among the present symbols: 512
//    bytes instead of a byte per slot, and shared memory per chunk is what
//    bounds the number of streams an SM keeps in flight;
//  * one word per present symbol (symbol | freq << 8 | start << 20), entry 0 a
//    pad so that the count above indexes it directly.  Two layouts:
//    shared by the four lanes of a chunk, `l_entries` words per chunk (alphabet
//    bound + 2), any alphabet; or one copy per lane (PER_LANE), entry k of lane
//    l in word k * 32 + l, a bank of its own, so the read is conflict free.
//    `l_entries` is then the number of rows and bounds the distinct symbols of
//    a chunk; the host sends only chunks that fit.
constexpr int RANS_RANK_BYTES = 512;
__host__ __device__ inline uint32_t rans_l_entries(uint32_t max_sym) { return (max_sym + 3 + 3) & ~3u; }
__host__ __device__ inline uint32_t rans_smem_bytes(uint32_t l_entries, bool per_lane = false) {
    return RANS_WARP_CHUNKS * RANS_RANK_BYTES + (per_lane ? 128 * l_entries : RANS_WARP_CHUNKS * 4 * l_entries) + RING_SMEM;
}

// Ring addressing: byte q of a lane's ring lives in word (q >> 2) & 15 of the
// [word][lane] array, `rw` points at the lane's column.
__device__ __forceinline__ uint32_t ring_byte(const uint32_t* rw, uint32_t q) {
    return reinterpret_cast<const uint8_t*>(rw)[((q & 60u) << 5) | (q & 3u)];
}
// The eight ring bytes from q on, big-endian: byte q is the top byte of `wh`.
__device__ __forceinline__ void ring_window_be(const uint32_t* rw, uint32_t q, uint32_t& wh, uint32_t& wl) {
    const uint8_t* rb = reinterpret_cast<const uint8_t*>(rw);
    const uint32_t t = q << 5;  // word k of the ring sits at byte (k & 15) * 128 of the lane's column
    uint32_t w0 = *reinterpret_cast<const uint32_t*>(rb + (t & 0x780u));
    uint32_t w1 = *reinterpret_cast<const uint32_t*>(rb + ((t + 0x80u) & 0x780u));
    uint32_t w2 = *reinterpret_cast<const uint32_t*>(rb + ((t + 0x100u) & 0x780u));
    uint32_t sel = 0x0123u + 0x1111u * (q & 3u);
    wh = __byte_perm(w0, w1, sel);
    wl = __byte_perm(w1, w2, sel);
}
// One symbol (decompress.rs:118-139): slot -> number of the covering symbol ->
// (symbol | freq << 8 | start << 20), state update.  `e` is returned whole; its
// low byte is the symbol.  LS = distance in words between list entries.
template <int LS>
__device__ __forceinline__ uint32_t rans_lookup(const uint32_t* tab, const uint32_t* lst, uint32_t& x) {
    uint32_t idx = x & 2047u;
    uint32_t w = tab[idx >> 4];
    uint32_t k = (w >> 16) + __popc(w << ((~idx & 15u) | 16u));  // boundaries at or below the slot: the count above the bitmap, the bitmap's bits up to the slot
    uint32_t e = lst[k * LS];
    x = ((e >> 8) & 0xFFFu) * (x >> 11) + (idx - (e >> 20));
    return e;
}
// Up to eight symbols, renormalising a byte at a time straight from the ring.
template <int LS>
__device__ __forceinline__ void rans_short_group(const uint32_t* tab, const uint32_t* lst, const uint32_t* rw, uint32_t& x, uint32_t& rq, uint32_t g,
                                                 uint32_t& s_lo, uint32_t& s_hi) {
    s_lo = 0; s_hi = 0;
    for (uint32_t j = 0; j < g; ++j) {
        uint32_t sym = rans_lookup<LS>(tab, lst, x) & 0xFFu;
        if (j < 4) s_lo |= sym << (8 * j); else s_hi |= sym << (8 * (j - 4));
        for (int k = 0; k < 3 && x < RANS_L; ++k) { x = (x << 8) | ring_byte(rw, rq); ++rq; }
    }
}
// The same for the group decoder's second try, out of line and by value (state, read position, symbols 0-3, symbols 4-7 come
// back in registers): one copy of the loop instead of one in every instance of the group decoder, which the instruction
// cache repays (14.28 -> 14.20 ms per pass of the benchmark container).
template <int LS>
__device__ __noinline__ uint4 rans_short_group8(const uint32_t* tab, const uint32_t* lst, const uint32_t* rw, uint32_t x, uint32_t rq) {
    uint32_t s_lo, s_hi;
    rans_short_group<LS>(tab, lst, rw, x, rq, 8, s_lo, s_hi);
    return make_uint4(x, rq, s_lo, s_hi);
}
// Exactly eight symbols, without a branch per symbol.  The next eight stream
// bytes sit big-endian in two registers behind the state; renormalising by
// 0..3 bytes (the count follows from the leading zeros of the state) is a
// funnel shift of state and window.  Eight bytes cover a group unless its
// symbols average more than one byte each; the total is checked once per group
// and a group that needed more is decoded again byte-wise.  On a plane of
// nearly incompressible bytes (many symbols, close to a byte each) that would
// happen in every other group, so a lane whose chunk has many distinct symbols
// (`dense`, only where DENSE_OK) reloads the window after four symbols.
// The byte count is ((leading zeros - 1) & 24) / 8, which holds for every state
// below 2^31.  An update never takes a state from below 2^31 to above it
// (freq <= 2^11, x >> 11 < 2^20), so only a stream whose stored initial state
// has the top bit set can get there: such a lane passes `slow` and takes the
// byte-wise path for every group.
template <int LS, bool DENSE_OK>
__device__ __forceinline__ void rans_group8(const uint32_t* tab, const uint32_t* lst, const uint32_t* rw, uint32_t& x, uint32_t& rq, uint32_t& s_lo,
                                            uint32_t& s_hi, bool dense, bool slow) {
    uint32_t wh, wl, used = 0, over = 0;
    const uint32_t x0 = x, rq0 = rq;
    ring_window_be(rw, rq, wh, wl);
    s_lo = 0; s_hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (DENSE_OK && j == 4 && dense) {
            over = used;  // the first half must have fit its window too
            rq += used >> 3; used = 0;
            ring_window_be(rw, rq, wh, wl);
        }
        uint32_t e = rans_lookup<LS>(tab, lst, x);
        const uint32_t ins = (0x3210u & ~(0xFu << (4 * (j & 3)))) | (4u << (4 * (j & 3)));  // low byte of e into byte j & 3
        if (j < 4) s_lo = __byte_perm(s_lo, e, ins); else s_hi = __byte_perm(s_hi, e, ins);
        // bytes until x >= 2^23, at most three: 0 for clz <= 8, 1 for 9..16, 2 for 17..24, 3 above
        uint32_t sh = (uint32_t(__clz(x)) - 1u) & 0x18u;
        x = __funnelshift_l(wh, x, sh);
        wh = __funnelshift_l(wl, wh, sh);
        wl <<= sh;
        used += sh;
    }
    if (used > 64 || over > 64 || slow) {
        const uint4 again = rans_short_group8<LS>(tab, lst, rw, x0, rq0);
        x = again.x; rq = again.y; s_lo = again.z; s_hi = again.w;
    } else {
        rq += used >> 3;
    }
}

// 20 blocks per SM lets the compiler use 96 registers (21 blocks), which the 32-bit rounds need to stay out of local
// memory; shared memory allows 22, and more blocks than that gave nothing (the load/store pipe, the integer pipe and the
// issue slots are each about 55-60 % busy there).
template <bool PER_LANE>
__global__ void __launch_bounds__(32, 20) rans_decode_kernel_t(const DecodeItem* __restrict__ items, uint32_t n_items, Bases bases, uint32_t* __restrict__ status,
                                                           uint32_t l_entries) {
    constexpr int LS = PER_LANE ? 32 : 1;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t lane = threadIdx.x, c = lane >> 2, s = lane & 3;
    uint32_t* ranktab = reinterpret_cast<uint32_t*>(smem);                                       // [8][128]
    uint32_t* symlist = reinterpret_cast<uint32_t*>(smem + RANS_WARP_CHUNKS * RANS_RANK_BYTES);  // entry 0 of every list is a pad
    const uint32_t list_bytes = PER_LANE ? 128 * l_entries : RANS_WARP_CHUNKS * 4 * l_entries;
    Ring ring{reinterpret_cast<uint32_t*>(smem + RANS_WARP_CHUNKS * RANS_RANK_BYTES + list_bytes) + lane};

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
            if (it.src_len < hdr + 16) err = ST_BAD_HEADER;
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
    bool dense = false;  // this lane's chunk is close to incompressible (see rans_group8)
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
        uint32_t total = __shfl_sync(0xFFFFFFFFu, incl, 31), distinct = __shfl_sync(0xFFFFFFFFu, rincl, 31);
        bool bad = total != 2048;  // decompress.rs:49-55
        if (!PER_LANE && c == c2) dense = distinct >= RANS_DENSE_SYMBOLS;
        if (distinct + 2 > l_entries) bad = true;  // the host sizes the list from the planned bytes; a blob that differs from them may not fit
        if (bad) { if (c == c2) err = ST_BAD_HEADER; continue; }
        uint32_t start = incl - sum, rank = rincl - present;
        uint32_t* tab = ranktab + c2 * 128;
        uint32_t* lst = PER_LANE ? symlist + c2 * 4 : symlist + c2 * l_entries;
        if (lane == 0) {
            if (PER_LANE) *reinterpret_cast<uint4*>(lst) = make_uint4(0, 0, 0, 0); else lst[0] = 0;
        }
        *reinterpret_cast<uint4*>(tab + 4 * lane) = make_uint4(0, 0, 0, 0);
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t sym = lane * 8 + k, fr = f[k];
            if (!fr) continue;
            uint32_t entry = sym | (fr << 8) | (start << 20);
            if (PER_LANE) *reinterpret_cast<uint4*>(lst + (rank + 1) * 32) = make_uint4(entry, entry, entry, entry);  // the four lanes of the chunk
            else lst[rank + 1] = entry;
            atomicOr(&tab[start >> 4], 1u << (start & 15));
            start += fr; ++rank;
        }
        __syncwarp();
        // boundaries before each word: lane l owns words 4l .. 4l+3
        uint4 bm = *reinterpret_cast<uint4*>(tab + 4 * lane);
        uint32_t p0 = __popc(bm.x), p1 = __popc(bm.y), p2 = __popc(bm.z), p3 = __popc(bm.w), scan = p0 + p1 + p2 + p3;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t t = __shfl_up_sync(0xFFFFFFFFu, scan, d);
            if (lane >= d) scan += t;
        }
        uint32_t before = scan - (p0 + p1 + p2 + p3);
        bm.x |= before << 16; before += p0;
        bm.y |= before << 16; before += p1;
        bm.z |= before << 16; before += p2;
        bm.w |= before << 16;
        *reinterpret_cast<uint4*>(tab + 4 * lane) = bm;
    }
    __syncwarp();

    uint32_t seg_start = 0, seg_len = 0;
    if (valid) split_four_dev(it.n, s, seg_start, seg_len);
    if (valid && !err && seg_len > 0) {
        if (my_len < 4) err = ST_STREAM_UNDERRUN;  // decompress.rs:82-86
        else {
            const uint32_t* tab = ranktab + c * 128;
            const uint32_t* lst = PER_LANE ? symlist + lane : symlist + c * l_entries;
            const uint32_t* rw = ring.base;
            Epilogue ep = make_epilogue(bases, it);
            const uint8_t* st = src + my_off;
            uint32_t x = ld_u32_unaligned(st);
            const bool slow = x >> 31;  // see rans_group8
            // ring cursor as a 32-bit offset from the 16-byte aligned block that holds the first renorm byte
            const uintptr_t g0 = (reinterpret_cast<uintptr_t>(st) + 4) & ~uintptr_t(15);
            uint32_t rq = uint32_t(reinterpret_cast<uintptr_t>(st) + 4 - g0);
            const uint32_t end_q = uint32_t(reinterpret_cast<uintptr_t>(st) + my_len - g0);
            const uintptr_t lo16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_first) & ~uintptr_t(15);
            const uintptr_t hi16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_end + 15) & ~uintptr_t(15);
            uint32_t fq = 0;
            ring.put(fq, fetch16(g0 + fq, lo16, hi16)); fq += 16;
            ring.put(fq, fetch16(g0 + fq, lo16, hi16)); fq += 16;
            ring.put(fq, fetch16(g0 + fq, lo16, hi16)); fq += 16;
            uint4 pending = fetch16(g0 + fq, lo16, hi16);
            // A group consumes at most 24 bytes; 32 valid bytes at its start always suffice.
            // The lanes of a warp drain their rings at similar rates: when any active lane runs low,
            // every lane with room for a block takes one, so the refill code runs once per several groups.
            auto top_up = [&]() {
                if (__any_sync(__activemask(), fq - rq < 32)) {
                    if (fq - rq <= 48) { ring.put(fq, pending); fq += 16; pending = fetch16(g0 + fq, lo16, hi16); }
                }
            };

            uint32_t pos = seg_start, remaining = seg_len;
            // head: a short group up to the next 8-element boundary of the destination
            {
                uint32_t g = first_group(ep, pos, remaining);
                if (g < 8 || remaining < 16) {
                    uint32_t s_lo, s_hi;
                    top_up();
                    rans_short_group<LS>(tab, lst, rw, x, rq, g, s_lo, s_hi);
                    emit(ep, pos, g, uint64_t(s_lo) | uint64_t(s_hi) << 32);
                    pos += g; remaining -= g;
                }
            }
            fast_groups(ep, it.n, pos, remaining, [&](uint32_t& s_lo, uint32_t& s_hi) {
                top_up();
                rans_group8<LS, !PER_LANE>(tab, lst, rw, x, rq, s_lo, s_hi, dense, slow);
            });
            // tail: whatever the fast loops left
            while (remaining) {
                uint32_t g = remaining < 8 ? remaining : 8, s_lo, s_hi;
                top_up();
                rans_short_group<LS>(tab, lst, rw, x, rq, g, s_lo, s_hi);
                emit(ep, pos, g, uint64_t(s_lo) | uint64_t(s_hi) << 32);
                pos += g; remaining -= g;
            }
            if (rq > end_q) err = ST_STREAM_UNDERRUN;  // decompress.rs:99-104
        }
    }
    if (err) atomicMax(&status[it.id], err);
}

// ---- canonical Huffman -----------------------------------------------------
// Shared memory per chunk:
//  * a one-symbol table over the next HUF_LUT_BITS stream bits, (length << 8) |
//    symbol, 0 when the code is longer than the window: 1 KiB instead of the
//    4 KiB of a table over all eleven bits, and shared memory per chunk is what
//    bounds the streams an SM keeps in flight;
//  * the canonical description (first code, count and list offset per length,
//    the symbols in canonical order): codes longer than the window (the rarest
//    symbols) and windows that no code covers are decoded from it.
constexpr int HUF_WARP_CHUNKS = 8;
constexpr int HUF_LUT_BITS = 9;
constexpr int HUF_LUT_BYTES = 2 << HUF_LUT_BITS;
constexpr int HUF_CANON_BYTES = 256 + 3 * 16 * 2;  // symbols in canonical order; u16 first[16], count[16], offs[16]
constexpr int HUF_SMEM = HUF_WARP_CHUNKS * (HUF_LUT_BYTES + HUF_CANON_BYTES) + RING_SMEM;

struct HuffCanon {
    const uint8_t* syms;
    const uint16_t* first;  // first[0] = max_bits
    const uint16_t* count;  // count[0] = 1 when the tables are usable
    const uint16_t* offs;
};
// One symbol from the low `max_bits` bits of `window` (stream order, first bit lowest): (length << 8) | symbol.
// A window that no code covers reads as symbol 0 of full length, like an unassigned slot of the reference's table
// (huffman/tree.rs:128-177).  Kept out of line: the decode loops meet a code longer than the table's window once in a
// few hundred symbols, and eight inlined copies of this loop per group of eight symbols, in every instance of the
// group decoder, made the kernel wait for its own instructions.  Four scalar arguments travel in registers; the
// canonical description (symbols, then first code / count / list offset per length) is addressed from its base.
__device__ __noinline__ uint32_t huff_canon_decode(const uint8_t* canon, uint32_t max_bits, uint32_t window, uint32_t shortest) {
    const uint16_t* first = reinterpret_cast<const uint16_t*>(canon + 256);
    const uint16_t* count = reinterpret_cast<const uint16_t*>(canon + 256 + 32);
    const uint16_t* offs = reinterpret_cast<const uint16_t*>(canon + 256 + 64);
    const uint32_t v = __brev(window) >> (32 - max_bits);  // code bits, first bit highest
    for (uint32_t len = shortest; len <= max_bits; ++len) {
        uint32_t d = (v >> (max_bits - len)) - first[len];
        if (d < count[len]) return (len << 8) | canon[offs[len] + d];
    }
    return max_bits << 8;
}

__global__ void __launch_bounds__(32) huffman_decode_kernel(const DecodeItem* __restrict__ items, uint32_t n_items, Bases bases, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t lane = threadIdx.x, c = lane >> 2, s = lane & 3;
    uint16_t* lut_all = reinterpret_cast<uint16_t*>(smem);                                  // [8][512]
    uint8_t* canon_all = smem + HUF_WARP_CHUNKS * HUF_LUT_BYTES;                            // [8][HUF_CANON_BYTES]
    Ring ring{reinterpret_cast<uint32_t*>(smem + HUF_WARP_CHUNKS * (HUF_LUT_BYTES + HUF_CANON_BYTES)) + lane};
    auto canon_of = [&](uint32_t chunk) {
        uint8_t* base = canon_all + chunk * HUF_CANON_BYTES;
        return HuffCanon{base, reinterpret_cast<uint16_t*>(base + 256), reinterpret_cast<uint16_t*>(base + 256 + 32), reinterpret_cast<uint16_t*>(base + 256 + 64)};
    };

    const uint32_t item_idx = blockIdx.x * HUF_WARP_CHUNKS + c;
    const bool valid = item_idx < n_items;
    DecodeItem it;
    if (valid) it = items[item_idx];
    const uint8_t* src = valid ? rd(bases, it.src) : nullptr;
    uint32_t err = ST_OK;
    uint32_t max_bits = 1, my_off = 0, my_len = 0;

    // weights header (weights.rs:34-85)
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

    // canonical description: lane s == 0 of each chunk (tree.rs:103-177); code assignment is sequential per length
    if (s == 0) {
        HuffCanon hc = canon_of(c);
        uint16_t* first = const_cast<uint16_t*>(hc.first);
        uint16_t* count = const_cast<uint16_t*>(hc.count);
        uint16_t* offs = const_cast<uint16_t*>(hc.offs);
        uint8_t* syms = const_cast<uint8_t*>(hc.syms);
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
            uint32_t code = 0, before = 0;
#pragma unroll
            for (int bits = 1; bits < 12; ++bits) {
                next_code[bits] = 0;
                if (uint32_t(bits) <= max_bits) {
                    code = (code + counts[bits - 1]) << 1;
                    if (code > (1u << bits)) err = ST_BAD_HEADER;
                    next_code[bits] = code;
                }
                first[bits] = uint16_t(code); count[bits] = uint16_t(counts[bits]); offs[bits] = uint16_t(before);
                before += counts[bits];
            }
        }
        if (valid && !err) {
            uint32_t placed[12];
#pragma unroll
            for (int k = 0; k < 12; ++k) placed[k] = 0;
            for (uint32_t sym = 0; sym < nsym; ++sym) {
                uint32_t len = weight(sym);
                if (!len) continue;
                uint32_t cde = 0, at = 0;
#pragma unroll
                for (int k = 1; k < 12; ++k) if (len == uint32_t(k)) { cde = next_code[k]; next_code[k] = cde + 1; at = offs[k] + placed[k]; placed[k]++; }
                if (cde >= (1u << len)) { err = ST_BAD_HEADER; break; }
                syms[at] = uint8_t(sym);
            }
        }
        first[0] = uint16_t(max_bits);
        count[0] = uint16_t(valid && !err);
    }
    { uint32_t be = __shfl_sync(0xFFFFFFFFu, err, c * 4); err = be > err ? be : err; }  // table errors of the builder lane reach its chunk
    max_bits = __shfl_sync(0xFFFFFFFFu, max_bits, c * 4);
    __syncwarp();

    // table: the four lanes of a chunk fill it, one symbol of the canonical list at a time
    {
        const HuffCanon hc = canon_of(c);
        const bool build = valid && !err;
        uint16_t* lut = lut_all + c * (1 << HUF_LUT_BITS);
        if (build) {
            const uint16_t fill = max_bits <= HUF_LUT_BITS ? uint16_t(max_bits << 8) : uint16_t(0);  // a slot no code covers; with longer codes the canonical decoder decides
            for (uint32_t i = s; i < (1u << HUF_LUT_BITS); i += 4) lut[i] = fill;
        }
        __syncwarp();
        if (build) {
            const uint32_t total = uint32_t(hc.offs[11]) + hc.count[11];
            for (uint32_t k = s; k < total; k += 4) {
                uint32_t len = 1;
                while (len < 11 && k >= uint32_t(hc.offs[len]) + hc.count[len]) ++len;
                if (len > HUF_LUT_BITS) continue;
                const uint32_t code = hc.first[len] + (k - hc.offs[len]);
                const uint32_t rev = __brev(code) >> (32 - len);
                const uint16_t entry = uint16_t((len << 8) | hc.syms[k]);
                for (uint32_t idx = rev; idx < (1u << HUF_LUT_BITS); idx += (1u << len)) lut[idx] = entry;
            }
        }
        __syncwarp();
    }

    uint32_t seg_start = 0, seg_len = 0;
    if (valid) split_four_dev(it.n, s, seg_start, seg_len);
    if (valid && !err) {
        const uint16_t* lut = lut_all + c * (1 << HUF_LUT_BITS);
        const HuffCanon hc = canon_of(c);
        Epilogue ep = make_epilogue(bases, it);
        // Stream positions are 32-bit offsets from `org`, a 16-byte aligned address two blocks below the stream's
        // first byte (the look-ahead fetch reaches one block below the stream), so that the compares and steps of
        // the loop are single instructions.
        const uintptr_t org = (reinterpret_cast<uintptr_t>(src + my_off) & ~uintptr_t(15)) - 32;
        const uint32_t start = uint32_t(reinterpret_cast<uintptr_t>(src + my_off) - org);
        uint32_t rp = start + my_len;  // one past the next byte to read (moves down)
        const uintptr_t lo16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_first) & ~uintptr_t(15);
        const uintptr_t hi16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_end + 15) & ~uintptr_t(15);
        // ring holds [fetched, ...): blocks are fetched downward
        uint32_t fetched = (rp + 15) & ~15u;
        for (int k = 0; k < 3; ++k) { fetched -= 16; ring.put(fetched, fetch16(org + fetched, lo16, hi16)); }
        uint4 pending = fetch16(org + fetched - 16, lo16, hi16);

        // bit container: 64 bits kept as two words so that every shift is one funnel shift (a code has at most 11 bits)
        uint32_t c_lo = 0, c_hi = 0;
        int32_t cnt = 0;  // bits in the container
        auto push = [&](uint32_t w) {  // w's bits go above the cnt (<= 32) bits held
            c_lo |= __funnelshift_lc(0u, w, uint32_t(cnt));
            c_hi |= __funnelshift_lc(w, 0u, uint32_t(cnt));
        };
        auto drop = [&](uint32_t nb) { c_lo = __funnelshift_r(c_lo, c_hi, nb); c_hi >>= nb; };
        // byte steps until the read position is word aligned
        while ((rp & 3) && rp > start) { --rp; push(ring.byte(rp)); cnt += 8; }
        const uint32_t mask = (1u << max_bits) - 1;
        uint32_t pos = seg_start, remaining = seg_len;
        // The lanes of a warp drain at similar rates: when any active lane runs low, every lane with room refills,
        // so the refill code runs once per several groups instead of (for some lane) in every one.
        auto ring_top_up = [&]() {
            if (__any_sync(__activemask(), rp - fetched < 32 && fetched > start)) {
                if (rp - fetched <= 48 && fetched > start) { fetched -= 16; ring.put(fetched, pending); pending = fetch16(org + fetched - 16, lo16, hi16); }
            }
        };
        // one aligned word (or the last partial one) into the bit container when it holds at most 32 bits
        auto take_word = [&]() {
            if (cnt <= 32 && rp > start) {
                uint32_t w = __byte_perm(ring.word(rp - 4), 0, 0x0123);  // byte rp-1 becomes the lowest
                uint32_t take = rp - start >= 4 ? 4u : uint32_t(rp - start);
                if (take < 4) w &= (1u << (8 * take)) - 1;
                push(w);
                cnt += 8 * int32_t(take);
                rp -= take;
            }
        };
        // (length << 8) | symbol of the next code, without consuming it
        auto peek = [&]() -> uint32_t {
            uint32_t e = lut[c_lo & ((1u << HUF_LUT_BITS) - 1)];
            if (e == 0) e = huff_canon_decode(hc.syms, max_bits, c_lo & mask, HUF_LUT_BITS + 1);  // the rarest symbols, or a window no code covers
            return e;
        };
        // one symbol with the reference's checks (decompress.rs:176-196)
        auto one_symbol = [&]() -> uint32_t {
            take_word();
            uint32_t e = peek();
            int32_t nb = int32_t(e >> 8);
            if (nb > cnt) { err = ST_STREAM_UNDERRUN; nb = cnt; }
            drop(uint32_t(nb)); cnt -= nb;
            return e;
        };
        // Eight symbols in two halves.  After a refill the container holds more than 32 bits (unless the stream is
        // at its end); four symbols take 44 bits at most and around ten on an exponent plane, so the halves run
        // without a check per symbol: the lowest bit count seen is tested once, and a group that ran out of bits is
        // decoded again one symbol at a time.
        auto dec8 = [&](uint32_t& s_lo, uint32_t& s_hi) {
            ring_top_up();
            const uint32_t lo0 = c_lo, hi0 = c_hi;
            const int32_t cnt0 = cnt;
            const uint32_t rp0 = rp;
            // With eight or more stream bytes left both refills of the group are whole aligned words: one conditional
            // word each, no partial-word handling.  Otherwise the group starts with a negative `lowest` and goes down
            // the checked path.
            int32_t lowest = rp - start >= 8 ? 0 : -1;
            s_lo = 0; s_hi = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if ((j & 3) == 0 && cnt <= 32) {
                    push(__byte_perm(ring.word(rp - 4), 0, 0x0123));  // byte rp-1 becomes the lowest
                    cnt += 32; rp -= 4;
                }
                uint32_t e = peek();
                const uint32_t nb = e >> 8;
                drop(nb); cnt -= int32_t(nb);
                if ((j & 3) == 3) lowest |= cnt;  // the count only falls between two refills
                const uint32_t ins = (0x3210u & ~(0xFu << (4 * (j & 3)))) | (4u << (4 * (j & 3)));  // low byte of e into byte j & 3
                if (j < 4) s_lo = __byte_perm(s_lo, e, ins); else s_hi = __byte_perm(s_hi, e, ins);
            }
            if (lowest < 0) {
                c_lo = lo0; c_hi = hi0; cnt = cnt0; rp = rp0;
                s_lo = 0; s_hi = 0;
                for (uint32_t j = 0; j < 8; ++j) {
                    uint32_t sym = one_symbol() & 0xFFu;
                    if (j < 4) s_lo |= sym << (8 * j); else s_hi |= sym << (8 * (j - 4));
                }
            }
        };
        auto short_group = [&](uint32_t g) {
            uint64_t syms = 0;
            ring_top_up();
            for (uint32_t j = 0; j < g; ++j) syms |= uint64_t(one_symbol() & 0xFFu) << (8 * j);
            emit(ep, pos, g, syms);
            pos += g; remaining -= g;
        };
        if (remaining) {
            uint32_t g = first_group(ep, pos, remaining);
            if (g < 8 || remaining < 16) short_group(g);
        }
        fast_groups(ep, it.n, pos, remaining, dec8);
        while (remaining) short_group(remaining < 8 ? remaining : 8);
        // every stream must end with no unread byte and only zero bits left
        // (decompress.rs:140-144, bitstream.rs:184-186)
        while (rp > start && !err) {
            if (rp - fetched < 32 && fetched > start) { fetched -= 16; ring.put(fetched, pending); pending = fetch16(org + fetched - 16, lo16, hi16); }
            --rp;
            if (ring.byte(rp)) err = ST_NOT_CONSUMED;
        }
        if (!err && (c_lo | c_hi) != 0) err = ST_NOT_CONSUMED;
    }
    if (err) atomicMax(&status[it.id], err);
}

// ---- tANS ------------------------------------------------------------------
// One stream per chunk, so one lane per chunk, and an entry per state: the
// spread symbols (u8 per state) and (baseline << 5 | bit count) (u16 per
// state), 6 KiB per chunk, so an SM holds 32 chunks whatever the kernel does.
// Both tables are laid out [state][lane]: the address of an entry is one
// multiply-add from the state and a lane only touches its own columns.
//
// With 32 streams an SM's throughput is 32 / (time of one symbol), and a lone
// warp pays for every instruction it issues, so the work is split over two
// warps that run on different schedulers.  Warp 0 walks the state chain and
// nothing else: per symbol one table load, three funnel shifts, the count and
// the next state, and one store of the state it left into an exchange buffer.
// Warp 1 turns those states into symbols (the second table), merges them with
// the other planes' bytes, writes the output and keeps the decoder's window of
// stream bytes filled.  They meet once per round of 32 symbols per lane, over
// two exchange buffers in shared memory, on named barriers.  Groups that do
// not fill a round, plane orders without a placing routine below, and the
// checked path near a stream's end run on warp 0 alone.
constexpr int TANS_CTA_CHUNKS = 32;
constexpr int TANS_THREADS = 64;
constexpr int TANS_SYM_BYTES = 2048 * 32;       // [state][lane] of u8
constexpr int TANS_NB_BYTES = 2048 * 2 * 32;    // [state][lane] of u16
constexpr int TANS_RING_WORDS = 64;             // 256 bytes of stream per lane
constexpr int TANS_RING_BYTES = TANS_RING_WORDS * 32 * 4;
constexpr int TANS_XCH_BYTES = 2 * 32 * 32 * 2; // [buffer][symbol of the round][lane] of u16
constexpr int TANS_PUB_BYTES = 2 * 32 * 4;      // [buffer][lane]: read position at the end of the round
constexpr int TANS_HAND_BYTES = 8 * 32 * 4;     // [word][lane]: rounds, position, lowest stream offset fetched, -, first stream offset, window origin (low, high)
constexpr int TANS_NORM_BYTES = 256 * 32 * 2;   // [symbol][lane] of u16: normalised counts while the tables are built (in local memory every state would
                                                // cost an L2 round trip); afterwards the staging area of the other planes' bytes
constexpr int TANS_SMEM = TANS_SYM_BYTES + TANS_NB_BYTES + TANS_RING_BYTES + TANS_XCH_BYTES + TANS_PUB_BYTES + TANS_HAND_BYTES + TANS_NORM_BYTES;

struct TansRing {
    uint32_t* base;  // &ring[0][lane]
    __device__ __forceinline__ uint32_t& word(uint32_t off) { return base[((off >> 2) & (TANS_RING_WORDS - 1)) * 32]; }
    __device__ __forceinline__ uint8_t byte(uint32_t off) { return reinterpret_cast<uint8_t*>(&word(off))[off & 3]; }
    __device__ __forceinline__ void put(uint32_t off16, uint4 v) {
        word(off16) = v.x; word(off16 + 4) = v.y; word(off16 + 8) = v.z; word(off16 + 12) = v.w;
    }
};
// How a lane's symbols are placed by the second warp.
enum : uint32_t { TP_NONE = 0, TP_PLAIN = 1, TP_M16 = 2, TP_FP8 = 3, TP_M32 = 4 };
__device__ __forceinline__ uint32_t tans_place_mode(const Epilogue& ep) {
    if (!ep.fused) return TP_PLAIN;
    if (ep.kind == K_M16) return TP_M16;
    if (ep.kind == K_E4M3 || ep.kind == K_E5M2) return TP_FP8;
    if (ep.kind == K_M32 && ep.slot == 3) return TP_M32;
    return TP_NONE;
}
__device__ __forceinline__ uint32_t tans_elem_bytes(uint32_t mode) { return mode == TP_M16 ? 2u : mode == TP_M32 ? 4u : 1u; }
__device__ __forceinline__ uint32_t tans_partners(uint32_t mode) { return mode == TP_PLAIN ? 0u : mode == TP_M32 ? 3u : 1u; }
// Rounds of 32 elements that can be placed from `pos` on: the output must sit on a 32-byte boundary and round r reads
// the aligned 32-byte block r + 2 of every partner plane, which must end inside the partner's chunk.
__device__ __forceinline__ uint32_t tans_rounds(const Epilogue& ep, uint32_t mode, uint32_t chunk_n, uint32_t pos, uint32_t remaining) {
    if (mode == TP_NONE) return 0;
    if ((reinterpret_cast<uintptr_t>(ep.dst) + size_t(pos) * tans_elem_bytes(mode)) & 31) return 0;
    uint32_t rounds = remaining >> 5;
    const uint32_t np = tans_partners(mode);
#pragma unroll
    for (uint32_t p = 0; p < 3; ++p) {
        if (p >= np) break;
        const uintptr_t lo = reinterpret_cast<uintptr_t>(ep.partner[p]), hi = lo + chunk_n;
        const uintptr_t q = (lo + pos) & ~uintptr_t(31);
        const uint32_t fit = q + 96 <= hi ? uint32_t((hi - q - 96) >> 5) + 1 : 0;
        rounds = fit < rounds ? fit : rounds;
    }
    return rounds;
}
// The two warps of a block meet on named barriers of 64 threads: the warp that filled (or emptied) an exchange
// buffer arrives, the other one waits.  Every arrival below has exactly one matching wait (both warps run the same
// number of rounds, taken from the same shared-memory words), and a barrier orders the shared-memory accesses of
// the threads that take part without waiting for their global loads in flight, which a memory fence would do.
__device__ __forceinline__ void tans_bar_arrive(uint32_t id) {
    __syncwarp();
    asm volatile("bar.arrive %0, 64;" ::"r"(id) : "memory");
}
__device__ __forceinline__ void tans_bar_wait(uint32_t id) {
    __syncwarp();
    asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}
constexpr uint32_t TANS_BAR_FULL = 1, TANS_BAR_EMPTY = 3;  // + buffer index; barrier 0 is __syncthreads

__global__ void __launch_bounds__(TANS_THREADS, 1) tans_decode_kernel(const DecodeItem* __restrict__ items, uint32_t n_items, Bases bases, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t lane = threadIdx.x & 31;
    const bool placer = threadIdx.x >= 32;  // warp 1
    const uint32_t item_idx = blockIdx.x * TANS_CTA_CHUNKS + lane;
    const bool live = item_idx < n_items;
    const DecodeItem it = items[live ? item_idx : 0];
    const uint8_t* src = rd(bases, it.src);
    uint8_t* sym_tab = smem + lane;
    uint8_t* nb_tab = smem + TANS_SYM_BYTES + lane * 2;
    uint8_t* area = smem + TANS_SYM_BYTES + TANS_NB_BYTES;
    TansRing ring{reinterpret_cast<uint32_t*>(area) + lane};
    uint16_t* xch = reinterpret_cast<uint16_t*>(area + TANS_RING_BYTES) + lane;                       // element (b, j) at xch[(b * 32 + j) * 32]
    uint32_t* pub = reinterpret_cast<uint32_t*>(area + TANS_RING_BYTES + TANS_XCH_BYTES) + lane;      // buffer b at pub[b * 32]
    uint32_t* hand = reinterpret_cast<uint32_t*>(area + TANS_RING_BYTES + TANS_XCH_BYTES + TANS_PUB_BYTES) + lane;  // word k at hand[k * 32]
    uint16_t* norm_tab = reinterpret_cast<uint16_t*>(area + TANS_RING_BYTES + TANS_XCH_BYTES + TANS_PUB_BYTES + TANS_HAND_BYTES) + lane;
    auto norm = [&](uint32_t sy) -> uint16_t& { return norm_tab[sy << 5]; };
    auto sym_at = [&](uint32_t u) -> uint8_t& { return sym_tab[u << 5]; };
    auto nb_at = [&](uint32_t u) -> uint16_t& { return *reinterpret_cast<uint16_t*>(nb_tab + (u << 6)); };
    const Epilogue ep = make_epilogue(bases, it);
    const uint32_t mode = tans_place_mode(ep);
    const uintptr_t lo16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_first) & ~uintptr_t(15);
    const uintptr_t hi16 = (reinterpret_cast<uintptr_t>(bases.blob) + bases.blob_end + 15) & ~uintptr_t(15);

    // ---- the placing warp -------------------------------------------------------
    if (placer) {
        __syncthreads();  // tables built, leading groups placed, the hand-over words written
        const uint32_t my_rounds = hand[0];
        const uint32_t max_rounds = __reduce_max_sync(0xFFFFFFFFu, my_rounds);
        uint32_t pos = hand[32], fetched = hand[2 * 32];
        const uint32_t start = hand[4 * 32];
        const uintptr_t org = uintptr_t(hand[5 * 32]) | uintptr_t(hand[6 * 32]) << 32;
        const uint32_t np = tans_partners(mode);
        uintptr_t q[3] = {0, 0, 0};
        uint32_t off[3] = {0, 0, 0};
        // Nothing this warp asks of global memory is waited for in the round that asked: both the other planes' bytes
        // and the stream bytes travel by asynchronous copies (cp.async) straight into shared memory, one group of
        // copies per round, and a round waits for the group issued two rounds earlier.  Partner planes: round r
        // merges the aligned 32-byte blocks r and r + 1 of each plane and requests block r + 3; block k waits in
        // slot k & 3 of a staging area (the space the normalised counts used while the tables were built), laid
        // out [slot][plane][half][lane] in 16-byte units.  Stream bytes go into the decoder's window directly.
        const uint32_t stage = uint32_t(__cvta_generic_to_shared(area + TANS_RING_BYTES + TANS_XCH_BYTES + TANS_PUB_BYTES + TANS_HAND_BYTES)) + lane * 16;
        auto stage_at = [&](uint32_t slot, uint32_t p, uint32_t half) -> uint32_t { return stage + (((slot & 3) * 3 + p) * 2 + half) * 512; };
        auto stage_block = [&](uint32_t slot, uint32_t p) -> Block32 {
            Block32 v;
            asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "r"(stage_at(slot, p, 0)) : "memory");
            asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7]) : "r"(stage_at(slot, p, 1)) : "memory");
            return v;
        };
        const uint32_t ring_sh = uint32_t(__cvta_generic_to_shared(ring.base));
        Block32 cur[3];
        uint8_t* out = ep.dst + size_t(pos) * tans_elem_bytes(mode);
        if (my_rounds) {
#pragma unroll
            for (uint32_t p = 0; p < 3; ++p) {
                if (p >= np) break;
                const uintptr_t lo = reinterpret_cast<uintptr_t>(ep.partner[p]);
                q[p] = (lo + pos) & ~uintptr_t(31); off[p] = uint32_t((lo + pos) & 31);
                cur[p] = load_block_guarded(q[p], lo, lo + it.n);  // block 0 may start below the chunk
                // blocks 1 and 2: inside the chunk for every lane with a round (tans_rounds)
#pragma unroll
                for (uint32_t k = 1; k < 3; ++k)
#pragma unroll
                    for (uint32_t h = 0; h < 2; ++h)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(stage_at(k, p, h)), "l"(q[p] + 32 * k + 16 * h) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");  // so that the first round waits for the group above like every later one
        for (uint32_t r = 0; r < max_rounds; ++r) {
            tans_bar_wait(TANS_BAR_FULL + (r & 1));
            const uint32_t b = r & 1;
            if (r < my_rounds) {
                // Stream bytes: these blocks are visible to the decoder before its round r + 4, by when it is at most
                // 176 bytes below the position it published, so the window is brought down to 241 - 256 bytes below that.
                const int32_t floor_off = int32_t(pub[b * 32]) - 256;
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    if (int32_t(fetched) - 16 >= floor_off && fetched > start) {
                        fetched -= 16;
                        const uintptr_t a = org + fetched;
                        const uint32_t n = (a >= lo16 && a < hi16) ? 4u : 0u;  // outside the blob's hull: zeros, nothing read
#pragma unroll
                        for (uint32_t i = 0; i < 4; ++i)
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(ring_sh + ((((fetched >> 2) + i) & (TANS_RING_WORDS - 1)) * 32) * 4), "l"(a + 4 * i), "r"(n) : "memory");
                    }
                }
                if (r + 3 <= my_rounds) {
#pragma unroll
                    for (uint32_t p = 0; p < 3; ++p) {
                        if (p >= np) break;
#pragma unroll
                        for (uint32_t h = 0; h < 2; ++h)
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(stage_at(r + 3, p, h)), "l"(q[p] + 96 + 16 * h) : "memory");
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 2;" ::: "memory");  // the groups of rounds r - 2 and earlier have landed
            if (r < my_rounds) {
                uint32_t w[8];
                const uint16_t* xs = xch + b * 32 * 32;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const uint32_t sy = sym_at(xs[j * 32]);
                    if ((j & 3) == 0) w[j >> 2] = sy; else w[j >> 2] |= sy << (8 * (j & 3));
                }
                uint32_t pw[3][8];
#pragma unroll
                for (uint32_t p = 0; p < 3; ++p) {
                    if (p >= np) break;
                    const Block32 nxt = stage_block(r + 1, p);
                    extract32(cur[p], nxt, off[p], pw[p]);
                    cur[p] = nxt;
                    q[p] += 32;
                }
                if (mode == TP_PLAIN) {
                    stg256(out, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
                    out += 32;
                } else if (mode == TP_M16) {
                    uint4 v[4];
                    const bool low_plane = ep.slot == 0;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        if (low_plane) { compose16x4(w[2 * g], pw[0][2 * g], v[g].x, v[g].y); compose16x4(w[2 * g + 1], pw[0][2 * g + 1], v[g].z, v[g].w); }
                        else { compose16x4(pw[0][2 * g], w[2 * g], v[g].x, v[g].y); compose16x4(pw[0][2 * g + 1], w[2 * g + 1], v[g].z, v[g].w); }
                    }
                    stg256(out, v[0], v[1]);
                    stg256(out + 32, v[2], v[3]);
                    out += 64;
                } else if (mode == TP_FP8) {
                    const bool high_plane = ep.slot == 0, e4m3 = ep.kind == K_E4M3;
                    uint32_t v[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[k] = high_plane ? compose_fp8x4(w[k], pw[0][k], e4m3) : compose_fp8x4(pw[0][k], w[k], e4m3);
                    stg256(out, make_uint4(v[0], v[1], v[2], v[3]), make_uint4(v[4], v[5], v[6], v[7]));
                    out += 32;
                } else {  // TP_M32: bytes 0..2 from the partner planes, byte 3 from this lane (transforms/fusion.rs:287-292)
#pragma unroll
                    for (int k = 0; k < 8; k += 2) {
                        uint32_t v[8];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t t0 = __byte_perm(pw[0][k + h], pw[1][k + h], 0x5140), t1 = __byte_perm(pw[2][k + h], w[k + h], 0x5140);
                            const uint32_t t2 = __byte_perm(pw[0][k + h], pw[1][k + h], 0x7362), t3 = __byte_perm(pw[2][k + h], w[k + h], 0x7362);
                            v[4 * h + 0] = revert32(__byte_perm(t0, t1, 0x5410));
                            v[4 * h + 1] = revert32(__byte_perm(t0, t1, 0x7632));
                            v[4 * h + 2] = revert32(__byte_perm(t2, t3, 0x5410));
                            v[4 * h + 3] = revert32(__byte_perm(t2, t3, 0x7632));
                        }
                        stg256(out, make_uint4(v[0], v[1], v[2], v[3]), make_uint4(v[4], v[5], v[6], v[7]));
                        out += 32;
                    }
                }
            }
            if (r + 2 < max_rounds) tans_bar_arrive(TANS_BAR_EMPTY + b);  // the decoder waits for it before round r + 2
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // the stream bytes asked for in the last two rounds
        hand[2 * 32] = fetched;
        __syncthreads();  // the rounds are over: the decoding warp takes the window back
        return;
    }

    // ---- the decoding warp ------------------------------------------------------
    uint32_t err = ST_OK;
    // header (mod.rs:388-425)
    uint32_t nsym = 0;
    if (!live) err = ST_BAD_HEADER;  // never reported: the lane has no item
    else if (it.src_len < 3 || src[0] != 11) err = ST_BAD_HEADER;
    else {
        nsym = uint32_t(src[1]) | uint32_t(src[2]) << 8;
        if (nsym < 2 || nsym > 256 || 3 + nsym * 3 + 8 > it.src_len) err = ST_BAD_HEADER;
    }
    // tables: the spread walks a running position and the decode entries count earlier states of the same
    // symbol, so both are sequential (mod.rs:199-211,346-369); every lane builds its own chunk's
    if (!err) {
        for (uint32_t i = 0; i < 256; ++i) norm(i) = 0;
        uint32_t sum = 0;
        bool bad = false;
        for (uint32_t i = 0; i < nsym; ++i) {  // no early exit: the loads of later entries need not wait for the checks of earlier ones
            const uint32_t sy = src[3 + 3 * i], fr = uint32_t(src[4 + 3 * i]) | uint32_t(src[5 + 3 * i]) << 8;
            bad |= fr == 0 || norm(sy) != 0;  // mod.rs:404-411
            bad |= fr > 2048;                 // the sum cannot come out right; keeps the 16-bit counters exact
            if (!bad) norm(sy) = uint16_t(fr);
            sum += fr;
        }
        if (bad || sum != 2048) err = ST_BAD_HEADER;
        if (!err) {
            uint32_t pos = 0;
            for (uint32_t sy = 0; sy < 256; ++sy) {
                const uint32_t f = norm(sy);
                for (uint32_t k = 0; k < f; ++k) { sym_at(pos) = uint8_t(sy); pos = (pos + 1283u) & 2047u; }
            }
            // the symbols of eight states are read ahead of the counter updates, which depend on one another through memory
            for (uint32_t u0 = 0; u0 < 2048; u0 += 8) {
                uint32_t sy[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) sy[i] = sym_at(u0 + i);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t x = norm(sy[i]);
                    norm(sy[i]) = uint16_t(x + 1);
                    const uint32_t nb = 11 - (31 - __clz(x));
                    nb_at(u0 + i) = uint16_t((((x << nb) - 2048) << 5) | nb);  // baseline above the bit count: a shift by the entry takes its low five bits
                }
            }
        }
    }
    uint64_t total_bits = 0, bslen = 0;
    const uint8_t* bs = src;
    if (!err) {
        const uint8_t* hp = src + 3 + nsym * 3;
        total_bits = uint64_t(ld_u32_unaligned(hp)) | uint64_t(ld_u32_unaligned(hp + 4)) << 32;
        bs = hp + 8;
        bslen = it.src_len - (3 + nsym * 3 + 8);
        if (total_bits > bslen * 8) err = ST_BAD_HEADER;
    }
    // LIFO reader (mod.rs:118-147): the stream is read from its last byte down, every byte from its high bit
    // down.  The `cnt` unread bits sit at the top of the 64-bit container c_hi:c_lo, the next to be used highest, so taking n bits is
    // one funnel shift; a word read little-endian from below the read position has its bytes in that order.
    // (the container is two words, so that every shift on the way of a symbol is one funnel shift)
    uint32_t c_hi = 0, c_lo = 0;
    int32_t cnt = 0;
    // Stream bytes pass through a 256-byte ring per lane in shared memory, filled downward in aligned 16-byte
    // blocks.  Positions are 32-bit offsets from `org`, a 16-byte aligned address two blocks below the stream.
    // While this warp decodes alone it requests blocks one step ahead (`pending`); a lane's loads must not be
    // waited for by the other lanes of the warp (the scoreboard is per warp), so blocks are taken by all lanes
    // with room at once, when any lane runs low, every few groups.
    const uintptr_t org = (reinterpret_cast<uintptr_t>(bs) & ~uintptr_t(15)) - 32;
    const uint32_t start = uint32_t(reinterpret_cast<uintptr_t>(bs) - org);
    uint32_t rp = start, fetched = start, state = 0;
    uint4 pending = make_uint4(0, 0, 0, 0);
    uint32_t pos = 0, remaining = err ? 0 : it.n;
    auto ring_top_up = [&]() {
        if (__any_sync(__activemask(), rp - fetched < 32 && fetched > start)) {
            if (rp - fetched <= 240 && fetched > start) { fetched -= 16; ring.put(fetched, pending); pending = fetch16(org + fetched - 16, lo16, hi16); }
        }
    };
    auto refill = [&]() {  // up to more than 32 bits, by bytes until the position is word aligned, then by words
        while (uint32_t(cnt) <= 32u && rp > start) {  // (a negative count only occurs in a group that is about to be decoded again)
            if (rp - start >= 4 && (rp & 3) == 0) {
                const uint32_t word = ring.word(rp - 4);
                const uint32_t s = uint32_t(32 - cnt);  // 0..32: the word goes below the cnt bits held
                c_hi |= __funnelshift_lc(word, 0u, s);
                c_lo |= __funnelshift_lc(0u, word, s);
                cnt += 32; rp -= 4;
            } else {
                --rp;
                const uint64_t t = uint64_t(ring.byte(rp)) << (56 - cnt);
                c_hi |= uint32_t(t >> 32); c_lo |= uint32_t(t);
                cnt += 8;
            }
        }
    };
    auto take = [&](uint32_t e) -> uint32_t {  // the bit count (<= 11) is the low five bits of e, which is all a funnel shift looks at
        const uint32_t v = __funnelshift_l(c_hi, 0u, e);  // the top bits; 0 for a count of 0
        c_hi = __funnelshift_l(c_lo, c_hi, e);
        c_lo = __funnelshift_l(0u, c_lo, e);
        cnt -= int32_t(e & 31u);
        return v;
    };
    // one symbol with the reference's checks
    auto one_symbol = [&]() -> uint32_t {
        refill();
        const uint32_t sy = sym_at(state), e = nb_at(state), nb = e & 31u;
        if (int32_t(nb) > cnt) { err = ST_STREAM_UNDERRUN; return sy; }
        state = (e >> 5) + take(e);
        if (state >= 2048) { err = ST_STREAM_UNDERRUN; state = 0; }
        return sy;
    };
    // a refill by one aligned word, taken when 32 bits or fewer are held
    auto refill_word = [&]() {
        if (cnt <= 32) {
            const uint32_t word = ring.word(rp - 4);
            const uint32_t s = uint32_t(32 - cnt);
            c_hi |= __funnelshift_lc(word, 0u, s);
            c_lo |= __funnelshift_lc(0u, word, s);
            cnt += 32; rp -= 4;
        }
    };
    // Eight symbols in two halves of four: after a refill the container holds more than 32 bits (unless the
    // stream is at its end) and four symbols take at most 44, around ten on an exponent plane, so the
    // halves run unchecked; a group that ran out of bits is decoded again one symbol at a time.
    auto dec8 = [&](uint32_t& s_lo, uint32_t& s_hi) {
        const uint32_t hi0 = c_hi, lo0 = c_lo;
        const int32_t cnt0 = cnt;
        ring_top_up();
        const uint32_t rp0 = rp, state0 = state;
        int32_t lowest = 0;
        s_lo = 0; s_hi = 0;
        // Away from the stream's first bytes the read position is word aligned and stays so: a refill is then
        // one word, taken or not, with no loop and no byte steps.  `lowest` starts negative otherwise, which
        // sends the group down the checked path.
        const bool words = (rp & 3) == 0 && rp - start >= 8;
        if (!words) lowest = -1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if ((j & 3) == 0) refill_word();
            const uint32_t sy = sym_at(state), e = nb_at(state);
            state = (e >> 5) + take(e);  // below 2048 whatever the stream holds: the baseline has its low bits clear and the stream adds fewer than 2^count
            if ((j & 3) == 3) lowest |= cnt;  // the count only falls between two refills
            const uint32_t ins = (0x3210u & ~(0xFu << (4 * (j & 3)))) | (4u << (4 * (j & 3)));
            if (j < 4) s_lo = __byte_perm(s_lo, sy, ins); else s_hi = __byte_perm(s_hi, sy, ins);
        }
        if (lowest < 0) {
            c_hi = hi0; c_lo = lo0; cnt = cnt0; rp = rp0; state = state0;
            s_lo = 0; s_hi = 0;
            for (uint32_t j = 0; j < 8 && !err; ++j) {
                uint32_t sy = one_symbol();
                if (j < 4) s_lo |= sy << (8 * j); else s_hi |= sy << (8 * (j - 4));
            }
        }
    };
    auto short_group = [&](uint32_t g) {
        uint64_t syms = 0;
        ring_top_up();
        for (uint32_t j = 0; j < g && !err; ++j) syms |= uint64_t(one_symbol()) << (8 * j);
        emit(ep, pos, g, syms);
        pos += g; remaining -= g;
    };
    uint32_t rounds = 0;
    if (!err) {
        uint32_t bi = uint32_t((total_bits + 7) >> 3);  // bytes that hold declared bits; the next to load is bs[bi-1]
        const uint32_t top = uint32_t(total_bits & 7);
        if (top) { --bi; c_hi = (bs[bi] & ((1u << top) - 1)) << (32 - top); cnt = int32_t(top); }
        rp = start + bi;  // one past the next byte to read (moves down)
        fetched = (rp + 15) & ~15u;
        for (int k = 0; k < 15; ++k) { if (fetched <= start) break; fetched -= 16; ring.put(fetched, fetch16(org + fetched, lo16, hi16)); }
        pending = fetch16(org + fetched - 16, lo16, hi16);
        refill();
        if (cnt < 11) err = ST_STREAM_UNDERRUN; else state = take(11);
        // leading groups, until the elements that follow start on a 32-byte boundary of the output
        if (!err && remaining) {
            uint32_t g = first_group(ep, pos, remaining);
            if (g < 8 || remaining < 16) short_group(g);
        }
        const uint32_t eb = tans_elem_bytes(mode);
        while (!err && mode != TP_NONE && remaining >= 40 && ((reinterpret_cast<uintptr_t>(ep.dst) + size_t(pos) * eb) & 31) != 0) short_group(8);
        if (!err) rounds = tans_rounds(ep, mode, it.n, pos, remaining);
        if (rounds) {
            // hand the window over full: what the second warp adds becomes visible from the fifth round on
            while (int32_t(fetched) - 16 >= int32_t(rp) - 256 && fetched > start) { fetched -= 16; ring.put(fetched, pending); pending = fetch16(org + fetched - 16, lo16, hi16); }
        }
    }
    hand[0] = rounds; hand[32] = pos; hand[2 * 32] = fetched; hand[4 * 32] = start;
    hand[5 * 32] = uint32_t(org); hand[6 * 32] = uint32_t(uint64_t(org) >> 32);
    __syncthreads();
    {
        const uint32_t max_rounds = __reduce_max_sync(0xFFFFFFFFu, rounds);
        for (uint32_t r = 0; r < max_rounds; ++r) {
            if (r >= 2) tans_bar_wait(TANS_BAR_EMPTY + (r & 1));  // the buffer of round r - 2 has been placed
            if (r < rounds) {
                uint16_t* xs = xch + (r & 1) * 32 * 32;
                const uint32_t hi0 = c_hi, lo0 = c_lo, rp0 = rp, state0 = state;
                const int32_t cnt0 = cnt;
                // eight word refills at most: the read position must be word aligned and 32 bytes above the stream's first
                int32_t lowest = ((rp & 3) == 0 && rp - start >= 32) ? 0 : -1;
                if (lowest == 0) {
                    // The word a refill would take is loaded four symbols before the count says whether it is
                    // taken, so that no shared-memory load sits between a symbol's bits and the next state.
                    uint32_t ahead_word = ring.word(rp - 4);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if ((j & 3) == 0) {
                            const bool need = cnt <= 32;
                            const uint32_t sft = uint32_t(32 - cnt);  // clamped to 32 by the shifts; unused when the word is not taken
                            const uint32_t in_hi = __funnelshift_lc(ahead_word, 0u, sft), in_lo = __funnelshift_lc(0u, ahead_word, sft);
                            c_hi |= need ? in_hi : 0u; c_lo |= need ? in_lo : 0u;
                            cnt += need ? 32 : 0; rp -= need ? 4u : 0u;
                            ahead_word = ring.word(rp - 4);
                        }
                        const uint32_t e = nb_at(state);
                        xs[j * 32] = uint16_t(state);
                        state = (e >> 5) + take(e);
                        if ((j & 3) == 3) lowest |= cnt;
                    }
                }
                if (lowest < 0) {  // near the stream's end, or out of bits: again with the reference's checks
                    c_hi = hi0; c_lo = lo0; cnt = cnt0; rp = rp0; state = state0;
                    for (uint32_t j = 0; j < 32; ++j) {
                        xs[j * 32] = uint16_t(state);
                        if (!err) one_symbol();
                    }
                }
                pub[(r & 1) * 32] = rp;
            }
            tans_bar_arrive(TANS_BAR_FULL + (r & 1));
        }
    }
    __syncthreads();
    if (rounds) {
        pos += rounds * 32; remaining -= rounds * 32;
        fetched = hand[2 * 32];
        pending = fetch16(org + fetched - 16, lo16, hi16);
    }
    if (!err) fast_groups(ep, it.n, pos, remaining, dec8);
    while (remaining && !err) short_group(remaining < 8 ? remaining : 8);
    if (!err && (cnt != 0 || rp != start || state != 0)) err = ST_NOT_CONSUMED;  // mod.rs:442-449
    if (err && live) atomicMax(&status[it.id], err);
}

// ---- Order1ScaleAC ---------------------------------------------------------
// One range-coder stream per chunk, one warp per chunk.  The warp first turns
// the chunk's PMFs into cumulative tables (u16, 256 per context: the count
// below each symbol), then decodes the stream together: every lane carries the
// same coder state.  The tables live in shared memory when the launch was
// given room for the chunk's contexts (`smem_tables`, the largest table count
// of the launch), else in the scratch arena.
constexpr uint32_t O1_MAX_SMEM_TABLES = 192;  // 96 KiB; launches with more contexts per chunk keep their tables in global memory
template <bool SMEM, bool LEAN>
__global__ void __launch_bounds__(32) o1sac_decode_kernel_t(const DecodeItem* __restrict__ items, uint32_t n_items, Bases bases, uint32_t* __restrict__ status,
                                                            uint32_t smem_tables) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t lane = threadIdx.x;
    const uint32_t item_idx = blockIdx.x;
    if (item_idx >= n_items) return;
    const DecodeItem it = items[item_idx];
    const uint8_t* st = rd(bases, it.state);
    uint32_t err = ST_OK;
    __shared__ uint8_t bitmap[32];
    __shared__ uint16_t table_of[256];  // which cumulative table a previous byte selects: 0 = marginal, 1 + rank of the context otherwise
    if (it.state_version != 1 || it.state_len < 32 + 512) err = ST_BAD_STATE;
    uint32_t pop = 0;
    if (!err) {
        bitmap[lane] = st[lane];
        __syncwarp();
        for (int i = 0; i < 32; ++i) pop += __popc(uint32_t(bitmap[i]));
        if (it.state_len != 32 + 512 + pop * 512) err = ST_BAD_STATE;
        if (SMEM && 1 + pop > smem_tables) err = ST_BAD_STATE;  // the host sized the launch from the same lengths
    }
    if (err) { if (lane == 0) atomicMax(&status[it.id], err); return; }
    // rank of every context (order1_scale_ac.rs:95-103)
    for (uint32_t p = lane; p < 256; p += 32) {
        uint32_t r = 0;
        for (uint32_t b = 0; b < (p >> 3); ++b) r += __popc(uint32_t(bitmap[b]));
        r += __popc(uint32_t(bitmap[p >> 3]) & ((1u << (p & 7)) - 1));
        table_of[p] = ((bitmap[p >> 3] >> (p & 7)) & 1) ? uint16_t(1 + r) : uint16_t(0);
    }
    // cumulative tables: table t (0 = marginal, 1+r = row r) = 256 u16 at cum + t*256; the total is 4096 by the check below
    uint16_t* cum = SMEM ? reinterpret_cast<uint16_t*>(smem) : reinterpret_cast<uint16_t*>(wr(bases, it.work));
    for (uint32_t t = lane; t < 1 + pop; t += 32) {
        const uint8_t* pm = st + 32 + t * 512;
        uint16_t* ct = cum + t * 256;
        uint32_t acc = 0; bool zero = false;
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t v = uint32_t(pm[2 * i]) | uint32_t(pm[2 * i + 1]) << 8;
            zero |= v == 0;
            ct[i] = uint16_t(acc);
            acc += v;
        }
        if (zero || acc != 4096) err = ST_BAD_STATE;  // quantize.rs:53-71
    }
    err = __reduce_max_sync(0xFFFFFFFFu, err);
    __syncwarp();
    __threadfence_block();
    if (err) { if (lane == 0) atomicMax(&status[it.id], err); return; }

    // The stream is serial, so the warp shares it: one 16-byte load per lane brings the whole table of the context,
    // every lane counts those of its eight counts that are at or below the target (order1_scale_ac.rs:474-486: the
    // symbol is the largest index whose count is <= target) and a warp reduction gives the symbol.  Lane 0 places
    // the symbols.  Two ways to the symbol's count and probability, by the size of the launch: with fewer chunks
    // than the GPU holds warps a chunk's own chain is what counts, with more the instructions issued are.
    Epilogue ep = make_epilogue(bases, it);
    const uint8_t* src = rd(bases, it.src);
    const uint32_t slen = it.src_len;
    // range_coder.rs:137-155: five bytes start the code register, of which the last four count
    uint32_t code = 0, rpos = 0;
    for (; rpos < 5; ++rpos) code = (code << 8) | (rpos < slen ? src[rpos] : 0);
    uint32_t low = 0, range = 0xFFFFFFFFu;
    const uint32_t row_len = it.row_len ? it.row_len : (it.n ? it.n : 1);
    uint32_t row_pos = 0; int prev = -1;
    uint64_t pos = 0;
    uint32_t remaining = it.n;
    uint32_t g = remaining ? first_group(ep, pos, remaining) : 0;
    // the next stream bytes, four at a time (zero past the end)
    auto next_bytes = [&](uint32_t at) -> uint32_t {
        uint32_t v = 0;
        for (uint32_t k = 0; k < 4; ++k) if (at + k < slen) v |= uint32_t(src[at + k]) << (8 * k);
        return v;
    };
    uint32_t ahead = next_bytes(rpos), ahead_left = 4;
    auto one_symbol = [&]() -> uint32_t {
        if (row_pos == 0) prev = -1;
        const uint16_t* ct = cum + (prev >= 0 ? uint32_t(table_of[prev]) * 256u : 0u);
        const uint4 q = *reinterpret_cast<const uint4*>(ct + lane * 8);  // the lane's eight counts, ascending
        const uint32_t rpt = range >> 12;  // range / 4096
        const uint32_t offset = code - low;
        // target = min(offset / rpt, 4095) and "count <= target" is "count * rpt <= offset": no division
        // (counts are below 4096, rpt < 2^20, so the products fit 32 bits)
        const uint32_t c[8] = {q.x & 0xFFFFu, q.x >> 16, q.y & 0xFFFFu, q.y >> 16, q.z & 0xFFFFu, q.z >> 16, q.w & 0xFFFFu, q.w >> 16};
        uint32_t lo, cumv, nextv;
        if (LEAN) {
            // few instructions: count, one reduction, then the symbol's count and the next one read back from the table
            uint32_t fit = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) fit += c[i] * rpt <= offset ? 1u : 0u;
            lo = __reduce_add_sync(0xFFFFFFFFu, fit) - 1;  // >= 0: entry 0 is 0
            cumv = ct[lo];
            nextv = lo < 255u ? uint32_t(ct[lo + 1]) : 4096u;
        } else {
            // short chain: the symbol's count is the largest that qualifies, the next count the smallest that does not
            // (4096 when all do); three reductions side by side and no second look at the table
            uint32_t fit = 0, below = 0, above = 4096;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const bool ok = c[i] * rpt <= offset;
                fit += ok;
                below = ok ? max(below, c[i]) : below;
                above = ok ? above : min(above, c[i]);
            }
            lo = __reduce_add_sync(0xFFFFFFFFu, fit) - 1;
            cumv = __reduce_max_sync(0xFFFFFFFFu, below);
            nextv = __reduce_min_sync(0xFFFFFFFFu, above);
        }
        low += cumv * rpt;
        range = (nextv - cumv) * rpt;
        while (range < (1u << 24)) {
            if (ahead_left == 0) { ahead = next_bytes(rpos); ahead_left = 4; }
            const uint32_t b = ahead & 0xFFu;
            ahead >>= 8; --ahead_left;
            ++rpos;
            code = (code << 8) | b;
            low <<= 8;
            range <<= 8;
        }
        prev = int(lo);
        row_pos = row_pos + 1 == row_len ? 0 : row_pos + 1;
        return lo;
    };
    while (remaining) {
        uint32_t s_lo = 0, s_hi = 0;
        if (g == 8) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t sy = one_symbol();
                if (j < 4) s_lo |= sy << (8 * j); else s_hi |= sy << (8 * (j - 4));
            }
        } else {
            for (uint32_t j = 0; j < g; ++j) {
                const uint32_t sy = one_symbol();
                if (j < 4) s_lo |= sy << (8 * j); else s_hi |= sy << (8 * (j - 4));
            }
        }
        if (lane == 0) emit(ep, pos, g, uint64_t(s_lo) | uint64_t(s_hi) << 32);
        pos += g; remaining -= g;
        g = remaining < 8 ? remaining : 8;
    }
}

// Tables of a chunk whose state has `state_len` bytes (0 when the state is too short to hold any).
inline uint32_t o1sac_tables(uint64_t state_len) { return state_len >= 32 + 512 ? uint32_t((state_len - 32 - 512) / 512) + 1 : 0; }
// `tables` = the largest table count among the items.  A launch that fills the GPU several times over runs the variant
// with fewer instructions and its tables in shared memory (when they fit); a smaller one the variant with the shorter chain.
constexpr uint32_t O1_LEAN_FROM_ITEMS = 1024;  // about seven warps per SM: 2016 chunks measured 8.7 ms this way against 10.4 ms the other, 168 chunks 6.9 against 6.3
inline void o1sac_launch(const DecodeItem* items, uint32_t n, const Bases& bases, uint32_t* status, uint32_t tables, cudaStream_t st) {
    if (n >= O1_LEAN_FROM_ITEMS && tables && tables <= O1_MAX_SMEM_TABLES) o1sac_decode_kernel_t<true, true><<<n, 32, tables * 512, st>>>(items, n, bases, status, tables);
    else o1sac_decode_kernel_t<false, false><<<n, 32, 0, st>>>(items, n, bases, status, 0);
}
inline cudaError_t o1sac_allow_shared_tables() {
    return cudaFuncSetAttribute(o1sac_decode_kernel_t<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(O1_MAX_SMEM_TABLES * 512));
}

// ---- stand-alone merge / copy ---------------------------------------------
constexpr uint32_t MERGE_TILE = 32768;  // elements per CTA: one chunk of the default size, so the search for the item is paid once per chunk
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
    // Sixteen elements per thread where the destination allows it: 16 bytes of every plane (two aligned 16-byte loads,
    // shifted into place; a block that is not wholly inside the plane is read bytewise) and 16 x element size bytes out,
    // on a boundary of that size.  The elements before the first such boundary and after the last go in groups of eight.
    const uint32_t eb = uint32_t(kind_elem_bytes(int(it.kind)));
    const uintptr_t a = reinterpret_cast<uintptr_t>(dst) / eb;
    uint32_t head = uint32_t((16 - (a & 15)) & 15);
    if (head > n) head = n;
    const uint32_t full = (n - head) >> 4, tail_at = head + full * 16;
    auto slow = [&](uint32_t begin, uint32_t end) {  // fewer than 16 elements: at most two groups
        const uint32_t pos = begin + 8 * threadIdx.x;
        if (pos >= end) return;
        const uint32_t count = end - pos < 8 ? end - pos : 8;
        uint64_t b[4] = {0, 0, 0, 0};
        for (int p = 0; p < np; ++p) b[p] = ld_bytes(src[p] + pos, count);
        compose_store(int(it.kind), dst, pos, count, b);
    };
    slow(0, head);
    slow(tail_at, n);
    uintptr_t p_lo[4] = {0, 0, 0, 0}, p_hi[4] = {0, 0, 0, 0};
    for (int p = 0; p < np; ++p) { p_lo[p] = reinterpret_cast<uintptr_t>(rd(bases, it.src[p])); p_hi[p] = p_lo[p] + it.n; }
    for (uint32_t g = threadIdx.x; g < full; g += blockDim.x) {
        const uint32_t pos = head + g * 16;
        uint32_t pw[4][4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            if (p >= np) break;
            const uintptr_t at = reinterpret_cast<uintptr_t>(src[p]) + pos, q = at & ~uintptr_t(15);
            const uint4 cur = load_block16_guarded(q, p_lo[p], p_hi[p]);
            const uint32_t off = uint32_t(at & 15);
            if (off) { const uint4 nxt = load_block16_guarded(q + 16, p_lo[p], p_hi[p]); extract16(cur, nxt, off, pw[p]); }
            else { pw[p][0] = cur.x; pw[p][1] = cur.y; pw[p][2] = cur.z; pw[p][3] = cur.w; }
        }
        uint8_t* out = dst + size_t(pos) * eb;
        switch (int(it.kind)) {
            case K_PASS: *reinterpret_cast<uint4*>(out) = make_uint4(pw[0][0], pw[0][1], pw[0][2], pw[0][3]); break;
            case K_E4M3:
            case K_E5M2: {
                const bool e4m3 = it.kind == K_E4M3;
                *reinterpret_cast<uint4*>(out) = make_uint4(compose_fp8x4(pw[0][0], pw[1][0], e4m3), compose_fp8x4(pw[0][1], pw[1][1], e4m3),
                                                            compose_fp8x4(pw[0][2], pw[1][2], e4m3), compose_fp8x4(pw[0][3], pw[1][3], e4m3));
                break;
            }
            case K_M16: {
                uint4 v[2];
                compose16x4(pw[0][0], pw[1][0], v[0].x, v[0].y); compose16x4(pw[0][1], pw[1][1], v[0].z, v[0].w);
                compose16x4(pw[0][2], pw[1][2], v[1].x, v[1].y); compose16x4(pw[0][3], pw[1][3], v[1].z, v[1].w);
                stg256(out, v[0], v[1]);
                break;
            }
            default: {  // K_M32 (transforms/fusion.rs:287-292)
#pragma unroll
                for (int k = 0; k < 4; k += 2) {
                    uint32_t w[8];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t t0 = __byte_perm(pw[0][k + h], pw[1][k + h], 0x5140), t1 = __byte_perm(pw[2][k + h], pw[3][k + h], 0x5140);
                        const uint32_t t2 = __byte_perm(pw[0][k + h], pw[1][k + h], 0x7362), t3 = __byte_perm(pw[2][k + h], pw[3][k + h], 0x7362);
                        w[4 * h + 0] = revert32(__byte_perm(t0, t1, 0x5410));
                        w[4 * h + 1] = revert32(__byte_perm(t0, t1, 0x7632));
                        w[4 * h + 2] = revert32(__byte_perm(t2, t3, 0x5410));
                        w[4 * h + 3] = revert32(__byte_perm(t2, t3, 0x7632));
                    }
                    stg256(out + 16 * k, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
                }
                break;
            }
        }
    }
}

// ---- per-plane ops between the split and a terminal, undone in scratch -------
// A CTA of 256 threads owns one tile of POST_TILE bytes; thread t owns the 64
// bytes from 64 t on.  Tiles of all items are numbered through `tile_first`
// like the merge tiles.  IntDelta (transforms/int_delta.rs:36-44, byte width)
// takes three launches: the byte sum of every tile, an exclusive scan of the
// sums per plane, then the running sum inside every tile started from the
// tile's carry.  All arithmetic is modulo 256 per byte (__vadd4).
struct PostTile { PostItem it; uint64_t base; uint32_t n; uint32_t local; };
__device__ __forceinline__ PostTile post_tile_of(const PostItem* items, const uint32_t* tile_first, uint32_t n_items) {
    uint32_t tile = blockIdx.x, lo = 0, hi = n_items;
    while (lo + 1 < hi) { uint32_t mid = (lo + hi) >> 1; if (tile_first[mid] <= tile) lo = mid; else hi = mid; }
    PostTile t;
    t.it = items[lo];
    t.local = tile - tile_first[lo];
    t.base = uint64_t(t.local) * POST_TILE;
    t.n = t.it.n - t.base < POST_TILE ? uint32_t(t.it.n - t.base) : POST_TILE;
    return t;
}
// The thread's 64 bytes as sixteen words, zero beyond the plane's end.  The plane starts on a 256-byte boundary of the scratch arena.
__device__ __forceinline__ void post_load64(const uint8_t* tile, uint32_t n, uint32_t w[16]) {
    const uint32_t at = threadIdx.x * 64;
    if (at + 64 <= n) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { uint4 v = *reinterpret_cast<const uint4*>(tile + at + 16 * q); w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w; }
    } else {
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            uint32_t v = 0;
            for (int i = 0; i < 4; ++i) if (at + 4 * k + i < n) v |= uint32_t(tile[at + 4 * k + i]) << (8 * i);
            w[k] = v;
        }
    }
}
__device__ __forceinline__ void post_store64(uint8_t* tile, uint32_t n, const uint32_t w[16]) {
    const uint32_t at = threadIdx.x * 64;
    if (at + 64 <= n) {
#pragma unroll
        for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(tile + at + 16 * q) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    } else {
        for (int k = 0; k < 16; ++k) for (int i = 0; i < 4; ++i) if (at + 4 * k + i < n) tile[at + 4 * k + i] = uint8_t(w[k] >> (8 * i));
    }
}
// Sum over the block of one byte-sized value per thread; with `exclusive`, every thread gets the sum of the threads before it.
__device__ __forceinline__ uint32_t post_block_sum(uint32_t v, uint32_t* exclusive) {
    __shared__ uint32_t warp_total[8];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { uint32_t t = __shfl_up_sync(0xFFFFFFFFu, incl, d); if (lane >= d) incl += t; }
    __syncthreads();  // the array may still be read from an earlier call
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    uint32_t before = 0, total = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) { if (k < int(warp)) before += warp_total[k]; total += warp_total[k]; }
    if (exclusive) *exclusive = (before + incl - v) & 0xFFu;
    return total & 0xFFu;
}
__global__ void __launch_bounds__(256) post_tile_sums_kernel(const PostItem* __restrict__ items, const uint32_t* __restrict__ tile_first, uint32_t n_items, Bases bases) {
    const PostTile t = post_tile_of(items, tile_first, n_items);
    if (t.it.op != POST_INTDELTA) return;
    uint32_t w[16], acc = 0;
    post_load64(wr(bases, t.it.plane) + t.base, t.n, w);
#pragma unroll
    for (int k = 0; k < 16; ++k) acc = __vadd4(acc, w[k]);
    acc = (acc + (acc >> 8) + (acc >> 16) + (acc >> 24)) & 0xFFu;
    const uint32_t total = post_block_sum(acc, nullptr);
    if (threadIdx.x == 0) reinterpret_cast<uint32_t*>(wr(bases, t.it.sums))[t.local] = total;
}
// One CTA per plane: the tile sums become the sum of all tiles before each.
__global__ void __launch_bounds__(256) post_scan_sums_kernel(const PostItem* __restrict__ items, uint32_t n_items, Bases bases) {
    const PostItem it = items[blockIdx.x];
    if (it.op != POST_INTDELTA) return;
    uint32_t* sums = reinterpret_cast<uint32_t*>(wr(bases, it.sums));
    const uint64_t tiles = (it.n + POST_TILE - 1) / POST_TILE;
    uint32_t carry = 0;
    for (uint64_t first = 0; first < tiles; first += 256) {
        const uint64_t i = first + threadIdx.x;
        const uint32_t v = i < tiles ? sums[i] : 0u;
        uint32_t excl;
        const uint32_t total = post_block_sum(v, &excl);
        if (i < tiles) sums[i] = (carry + excl) & 0xFFu;
        carry = (carry + total) & 0xFFu;
    }
}
__global__ void __launch_bounds__(256) post_apply_kernel(const PostItem* __restrict__ items, const uint32_t* __restrict__ tile_first, uint32_t n_items, Bases bases) {
    const PostTile t = post_tile_of(items, tile_first, n_items);
    uint8_t* tile = wr(bases, t.it.plane) + t.base;
    uint32_t w[16];
    post_load64(tile, t.n, w);
    if (t.it.op == POST_MZS) {  // transforms/mantissa_zero.rs: inverse shifts every byte left by k
        const uint32_t keep = 0x01010101u * (0xFFu >> t.it.k);
#pragma unroll
        for (int k = 0; k < 16; ++k) w[k] = (w[k] & keep) << t.it.k;
    } else if (t.it.op == POST_INTDELTA) {
        uint32_t run = 0;  // sum of the thread's earlier words, in every byte
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            uint32_t v = w[k];
            v = __vadd4(v, v << 8);
            v = __vadd4(v, v << 16);  // running sum inside the word
            v = __vadd4(v, run);
            run = (v >> 24) * 0x01010101u;
            w[k] = v;
        }
        uint32_t excl;
        post_block_sum(run & 0xFFu, &excl);
        const uint32_t carry = ((reinterpret_cast<const uint32_t*>(rd(bases, t.it.sums))[t.local] + excl) & 0xFFu) * 0x01010101u;
#pragma unroll
        for (int k = 0; k < 16; ++k) w[k] = __vadd4(w[k], carry);
    }
    post_store64(tile, t.n, w);
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

// Plane bytes of one element (byte p = plane p) as their terminals hold them: the forward direction of the per-plane
// ops, from this element's and the previous element's plane bytes.
__device__ __forceinline__ uint32_t terminal_bytes(uint32_t cur, uint32_t prev, uint32_t post, uint32_t post_k, int planes) {
    uint32_t r = 0;
    for (int p = 0; p < planes; ++p) {
        const uint32_t op = (post >> (8 * p)) & 0xFFu, k = (post_k >> (8 * p)) & 0xFFu;
        uint32_t b = (cur >> (8 * p)) & 0xFFu;
        if (op == POST_INTDELTA) b = (b - ((prev >> (8 * p)) & 0xFFu)) & 0xFFu;
        else if (op == POST_MZS) b >>= k;
        r |= b << (8 * p);
    }
    return r;
}

// The byte table is kept 32 times over in shared memory, entry i of lane l at word 32 i + l: a lookup never leaves
// the lane's own bank, whatever the 32 indices of a warp are (one shared copy took 2.15 passes per lookup).  Tensor
// bytes are read 16 at a time; a thread walks its own run, so every wider load saves that many single-sector requests.
__global__ void __launch_bounds__(128) crc_planes_kernel(const VerifyTensor* __restrict__ tensors, uint32_t n_tensors, uint64_t n_runs, Bases bases,
                                                         const CrcTables* __restrict__ tabs, uint32_t* __restrict__ acc) {
    __shared__ uint32_t T32[256 * 32];
    __shared__ uint32_t X[64];
    for (uint32_t i = threadIdx.x; i < 256 * 32; i += blockDim.x) T32[i] = tabs->byte_table[i >> 5];
    if (threadIdx.x < 64) X[threadIdx.x] = tabs->x2n[threadIdx.x];
    __syncthreads();
    uint64_t run = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (run >= n_runs) return;
    const uint32_t* T = T32 + (threadIdx.x & 31);
    auto step = [&](uint32_t crc, uint32_t byte) { return T[((crc ^ byte) & 0xFFu) << 5] ^ (crc >> 8); };
    uint32_t lo = 0, hi = n_tensors;
    while (lo + 1 < hi) { uint32_t mid = (lo + hi) >> 1; if (tensors[mid].first_run <= run) lo = mid; else hi = mid; }
    const VerifyTensor t = tensors[lo];
    uint64_t first = (run - t.first_run) * VERIFY_RUN;
    uint32_t n = t.n_elems - first < VERIFY_RUN ? uint32_t(t.n_elems - first) : VERIFY_RUN;
    const uint8_t* out = rd(bases, t.out);
    uint32_t c[4] = {0, 0, 0, 0};
    const bool wide = !t.post && (reinterpret_cast<uintptr_t>(out + first * uint64_t(kind_elem_bytes(int(t.kind)))) & 15) == 0;
    switch (t.kind) {
        case K_PASS: {
            uint32_t i = 0;
            if (wide) {
                const uint4* q = reinterpret_cast<const uint4*>(out + first);
                uint4 ahead = i + 16 <= n ? __ldg(q) : make_uint4(0, 0, 0, 0);  // the next block is on its way while this one is folded in
                for (; i + 16 <= n; i += 16) {
                    const uint4 v = ahead;
                    ++q;
                    if (i + 2 * 16 <= n) ahead = __ldg(q);
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int k = 0; k < 16; ++k) c[0] = step(c[0], w[k >> 2] >> (8 * (k & 3)));
                }
            }
            for (; i < n; ++i) c[0] = step(c[0], out[first + i]);
            break;
        }
        case K_M16: {
            auto planes_of = [&](uint64_t e) {
                uint32_t v = uint32_t(out[2 * e]) | uint32_t(out[2 * e + 1]) << 8;
                return ((v << 1) & 0xFF00u) | ((v >> 8) & 0x0080u) | (v & 0x007Fu);
            };
            uint32_t i = 0;
            if (wide) {
                const uint4* q = reinterpret_cast<const uint4*>(out + first * 2);
                uint4 ahead = i + 8 <= n ? __ldg(q) : make_uint4(0, 0, 0, 0);  // the next block is on its way while this one is folded in
                for (; i + 8 <= n; i += 8) {
                    const uint4 v = ahead;
                    ++q;
                    if (i + 2 * 8 <= n) ahead = __ldg(q);
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {  // two elements per word: the forward reorder of split/dtype16.rs:11-18 on both halves
                        const uint32_t r = ((w[k] << 1) & 0xFF00FF00u) | ((w[k] >> 8) & 0x00800080u) | (w[k] & 0x007F007Fu);
                        c[0] = step(c[0], r); c[1] = step(c[1], r >> 8);
                        c[0] = step(c[0], r >> 16); c[1] = step(c[1], r >> 24);
                    }
                }
            }
            uint32_t prev = (t.post && first) ? planes_of(first - 1) : 0u;
            for (; i < n; ++i) {
                uint32_t r = planes_of(first + i);
                if (t.post) { uint32_t cur = r; r = terminal_bytes(r, prev, t.post, t.post_k, 2); prev = cur; }
                c[0] = step(c[0], r);
                c[1] = step(c[1], r >> 8);
            }
            break;
        }
        case K_M32: {
            auto reorder = [](uint32_t v) { return ((v << 1) & 0xFF000000u) | ((v >> 8) & 0x00800000u) | (v & 0x007FFFFFu); };
            auto planes_of = [&](uint64_t e) { return reorder(ld_u32_unaligned(out + 4 * e)); };
            uint32_t i = 0;
            if (wide) {
                const uint4* q = reinterpret_cast<const uint4*>(out + first * 4);
                uint4 ahead = i + 4 <= n ? __ldg(q) : make_uint4(0, 0, 0, 0);  // the next block is on its way while this one is folded in
                for (; i + 4 <= n; i += 4) {
                    const uint4 v = ahead;
                    ++q;
                    if (i + 2 * 4 <= n) ahead = __ldg(q);
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t r = reorder(w[k]);
#pragma unroll
                        for (int p = 0; p < 4; ++p) c[p] = step(c[p], r >> (8 * p));
                    }
                }
            }
            uint32_t prev = (t.post && first) ? planes_of(first - 1) : 0u;
            for (; i < n; ++i) {
                uint32_t r = planes_of(first + i);
                if (t.post) { uint32_t cur = r; r = terminal_bytes(r, prev, t.post, t.post_k, 4); prev = cur; }
#pragma unroll
                for (int p = 0; p < 4; ++p) c[p] = step(c[p], r >> (8 * p));
            }
            break;
        }
        default: {
            auto nibbles = [&](uint32_t v) { return t.kind == K_E4M3 ? (((v & 0x78) << 1) | ((v & 0x80) >> 4) | (v & 0x07)) : (((v & 0x7C) << 1) | ((v & 0x80) >> 5) | (v & 0x03)); };
            uint32_t i = 0;
            if (wide) {
                const uint4* q = reinterpret_cast<const uint4*>(out + first);
                uint4 ahead = i + 16 <= n ? __ldg(q) : make_uint4(0, 0, 0, 0);  // the next block is on its way while this one is folded in
                for (; i + 16 <= n; i += 16) {
                    const uint4 v = ahead;
                    ++q;
                    if (i + 2 * 16 <= n) ahead = __ldg(q);
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        const uint32_t r = nibbles((w[k >> 2] >> (8 * (k & 3))) & 0xFFu);
                        c[0] = step(c[0], r >> 4); c[1] = step(c[1], r & 0x0F);
                    }
                }
            }
            for (; i < n; ++i) {
                const uint32_t r = nibbles(out[first + i]);
                c[0] = step(c[0], r >> 4);
                c[1] = step(c[1], r & 0x0F);
            }
            break;
        }
    }
    uint32_t shift = x_pow_8n(X, t.n_elems - first - n);
    int np = kind_planes(int(t.kind));
    for (int p = 0; p < np; ++p) atomicXor(&acc[t.acc_base + p], gf2_mulmod(shift, c[p]));
}

// XXH64 (seed 0) of each tensor, one warp per tensor.  The hash is sequential by design: four accumulators, each
// fed one 8-byte word of every 32-byte stripe through add, rotate and a 64-bit multiply, so four lanes carry the
// state and a tensor cannot go faster than that dependent chain allows (add, rotate, one 64-bit multiply per 32
// bytes).  What the rest of the warp does is keep the chain short and fed: all 32 lanes fetch the next 4 KiB of the
// tensor with 128-bit loads and multiply the current block's words by the second prime, while lanes 0-3 work through
// the 128 stripes of the current block out of shared memory, so neither DRAM latency nor that multiply shows.  Tensors hash
// concurrently, one per block, and the host lists the largest first: the longest tensor is the critical path.
__device__ __forceinline__ uint64_t rotl64(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
__device__ __forceinline__ uint64_t ld_u64_unaligned(const uint8_t* p) { return uint64_t(ld_u32_unaligned(p)) | uint64_t(ld_u32_unaligned(p + 4)) << 32; }
constexpr uint32_t XXH_BLOCK = 4096;

__global__ void __launch_bounds__(32) xxh64_kernel(const HashItem* __restrict__ items, uint32_t n_items, Bases bases, uint64_t* __restrict__ out) {
    const uint64_t P1 = 11400714785074694791ull, P2 = 14029467366897019727ull, P3 = 1609587929392839161ull, P4 = 9650029242287828579ull,
                   P5 = 2870177450012600261ull;
    __shared__ __align__(16) uint8_t stage[XXH_BLOCK];
    const uint32_t lane = threadIdx.x, idx = blockIdx.x;
    if (idx >= n_items) return;
    const HashItem it = items[idx];
    const uint8_t* p = rd(bases, it.data);
    const uint64_t len = it.len, stripes = len / 32;
    uint64_t v = lane == 0 ? P1 + P2 : lane == 1 ? P2 : lane == 2 ? 0 : 0 - P1;
    uint64_t done = 0;  // stripes consumed
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        const uint64_t blocks = len / XXH_BLOCK;
        uint4 nxt[8];
        if (blocks) {
#pragma unroll
            for (int k = 0; k < 8; ++k) nxt[k] = __ldg(reinterpret_cast<const uint4*>(p) + k * 32 + lane);
        }
        for (uint64_t b = 0; b < blocks; ++b) {
            __syncwarp();  // the previous block has been read
#pragma unroll
            for (int k = 0; k < 8; ++k) reinterpret_cast<uint4*>(stage)[k * 32 + lane] = nxt[k];
            if (b + 1 < blocks) {
                const uint4* q = reinterpret_cast<const uint4*>(p + (b + 1) * XXH_BLOCK);
#pragma unroll
                for (int k = 0; k < 8; ++k) nxt[k] = __ldg(q + k * 32 + lane);
            }
            __syncwarp();
            {   // the products word * P2 do not depend on the accumulators: all lanes take them off the serial chain
                uint64_t* w = reinterpret_cast<uint64_t*>(stage);
#pragma unroll
                for (int k = 0; k < int(XXH_BLOCK / 8 / 32); ++k) w[k * 32 + lane] *= P2;
            }
            __syncwarp();
            if (lane < 4) {
                const uint64_t* w = reinterpret_cast<const uint64_t*>(stage) + lane;
#pragma unroll 16
                for (int st = 0; st < int(XXH_BLOCK / 32); ++st) { v += w[4 * st]; v = rotl64(v, 31); v *= P1; }
            }
        }
        done = blocks * (XXH_BLOCK / 32);
    }
    if (lane < 4) {  // what is left of the stripes (all of them for a source that is not 16-byte aligned)
        const bool aligned = (reinterpret_cast<uintptr_t>(p) & 7) == 0;
        for (uint64_t st = done; st < stripes; ++st) {
            const uint8_t* q = p + st * 32 + lane * 8;
            const uint64_t in = aligned ? *reinterpret_cast<const uint64_t*>(q) : ld_u64_unaligned(q);
            v += in * P2; v = rotl64(v, 31); v *= P1;
        }
    }
    const uint64_t v1 = __shfl_sync(0xFFFFFFFFu, v, 0), v2 = __shfl_sync(0xFFFFFFFFu, v, 1), v3 = __shfl_sync(0xFFFFFFFFu, v, 2), v4 = __shfl_sync(0xFFFFFFFFu, v, 3);
    if (lane != 0) return;
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

// Copies 16-byte words; the host side uses it to bring a plan's work lists from pinned host memory to the device
// without queueing behind the copy engine's transfers.
__global__ void __launch_bounds__(256) stage_in_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += size_t(gridDim.x) * blockDim.x) dst[i] = src[i];
}

}  // namespace ptwm
