// Work descriptors shared by the host planner and the CUDA kernels.
//
// The host parses a container once (format.hpp) and flattens it into arrays of
// fixed-size items; a decode pass is then a handful of kernel launches over
// those arrays.  Every byte location is a Ref: an offset into one of three
// device regions (the compressed blob, the scratch arena, the output arena),
// so a plan is independent of where the caller puts those regions.
#pragma once
#include <stdint.h>

namespace ptwm {

enum Space : uint32_t { SP_BLOB = 0, SP_SCRATCH = 1, SP_OUT = 2 };

// Top two bits name the region, the rest is the byte offset inside it.
typedef uint64_t Ref;
constexpr Ref REF_NONE = ~0ull;
inline __host__ __device__ Ref make_ref(Space s, uint64_t off) { return (uint64_t(s) << 62) | off; }

// Wire ids of the plane codecs on the hot path (codec.rs:5-23 of ptwm-core).
enum Codec : uint16_t { C_IDENTITY = 0, C_HUFFMAN = 1, C_RANS = 3, C_ZSTD = 4, C_TANS = 7, C_O1SAC = 0x11 };

// How the planes of one tensor recombine (transforms/fusion.rs of ptwm-core).
enum Kind : uint8_t { K_PASS = 0, K_M16 = 1, K_M32 = 2, K_E4M3 = 3, K_E5M2 = 4 };
inline __host__ __device__ int kind_planes(int k) { return k == K_PASS ? 1 : k == K_M32 ? 4 : 2; }
inline __host__ __device__ int kind_elem_bytes(int k) { return k == K_M16 ? 2 : k == K_M32 ? 4 : 1; }

// One coded chunk of one plane.  Huffman / rANS chunks hold four streams and
// are decoded by four lanes; tANS / Order1ScaleAC chunks hold one.
struct DecodeItem {
    Ref src;            // codec blob: Huffman weights / rANS table / tANS header / range-coder bytes
    uint32_t src_len;
    uint32_t n;         // decoded symbols
    Ref dst;            // plain: where the plane bytes go.  fused: output bytes of this chunk's first element
    Ref partner[3];     // fused: the other planes' bytes for this chunk, in plane order without `slot`
    Ref state;          // Order1ScaleAC: serialized state (bitmap, marginal, rows)
    Ref work;           // Order1ScaleAC: scratch for the cumulative tables, (1+rows)*514 bytes, 2-byte aligned
    uint32_t state_len;
    uint32_t row_len;   // Order1ScaleAC rows; 0 = one row spanning the chunk
    uint32_t id;        // index into the status array
    uint8_t kind;       // fused: Kind of the tensor
    uint8_t slot;       // fused: which plane this chunk supplies
    uint8_t fused;      // 0 = plain store, 1 = merge with partners and store elements
    uint8_t state_version;
};

// Planes that are all available as bytes (stored raw in the blob or decoded
// to scratch): recombine n elements.  K_PASS is a plain copy.
struct MergeItem {
    Ref src[4];
    Ref dst;
    uint32_t n;     // elements (= bytes per plane)
    uint32_t kind;
};

// Plane CRC check over a decoded tensor: the kernel re-splits the output
// bytes into planes (the forward transform) in runs of VERIFY_RUN elements,
// takes the CRC-32 remainder of each run, shifts it by the plane bytes that
// follow and XORs it into accumulator acc_base + plane.
struct VerifyTensor {
    Ref out;
    uint64_t n_elems;    // = bytes per plane
    uint64_t first_run;  // index of this tensor's first run among all runs of the launch
    uint32_t kind;
    uint32_t acc_base;
    uint32_t post;       // byte p: op between the split and terminal p (POST_*); the CRC covers the terminal's bytes
    uint32_t post_k;     // byte p: bits stripped by MantissaZeroStrip
};

// A plane in scratch that passed through one more op on the way from the split
// to its terminal: undo it in place before the planes are recombined.
// IntDelta (byte width): running sum modulo 256 over the whole plane, done in
// tiles of POST_TILE bytes with one word per tile at `sums`.
// MantissaZeroStrip(k): every byte shifted left by k.
enum : uint32_t { POST_NONE = 0, POST_INTDELTA = 1, POST_MZS = 2 };
struct PostItem {
    Ref plane;
    uint64_t n;
    uint32_t op;
    uint32_t k;
    Ref sums;
};
constexpr uint32_t POST_TILE = 16384;
constexpr uint32_t VERIFY_RUN = 2048;

struct HashItem {
    Ref data;
    uint64_t len;
};

// blob addresses file offset 0 of the container; only offsets
// [blob_first, blob_end) are resident on the device.
struct Bases {
    const uint8_t* blob;
    uint64_t blob_first, blob_end;
    uint8_t* scratch;
    uint8_t* out;
};

// Status codes written per item (0 = ok).
enum Status : uint32_t {
    ST_OK = 0,
    ST_BAD_HEADER = 1,      // weights / frequency table / jump table malformed
    ST_STREAM_UNDERRUN = 2, // a stream ended before its symbols did
    ST_NOT_CONSUMED = 3,    // Huffman: unread bytes or non-zero leftover bits; tANS: trailing bits / wrong final state
    ST_BAD_STATE = 4,       // Order1ScaleAC state invalid
};

}  // namespace ptwm
