// Host side of the encode path: chain choice per tensor, per-plane codec
// selection, the device pipeline (split, histogram, tables, streams, gather)
// and the compact-container writer (ptwc.rs:76-93,160-226,
// tensor_record_compact.rs:203-493, chain/wire_compact.rs:140-245,
// extension/compact_table.rs:123-158 of the reference).
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "encode.cuh"
#include "shared_fit.cuh"
#include "format.hpp"
#include "host_common.hpp"

using namespace ptwm;

namespace {

void put_varint(std::vector<uint8_t>& out, uint64_t v) {  // varint.rs:17-23
    while (v >= 0x80) { out.push_back(uint8_t(v) | 0x80); v >>= 7; }
    out.push_back(uint8_t(v));
}
void put_u32(std::vector<uint8_t>& out, uint32_t v) { for (int i = 0; i < 4; ++i) out.push_back(uint8_t(v >> (8 * i))); }
void put_u64(std::vector<uint8_t>& out, uint64_t v) { for (int i = 0; i < 8; ++i) out.push_back(uint8_t(v >> (8 * i))); }

struct ChainDef {
    uint8_t kind;
    std::vector<std::pair<uint16_t, std::vector<uint8_t>>> nodes;  // (op wire id, params)
    std::vector<uint8_t> roles;                                    // compact terminal role bytes
    int post_plane = -1;  // >= 0: the last node is an op between output `post_plane` of the split (node 2) and that plane's terminal
    bool operator==(const ChainDef& o) const { return nodes == o.nodes && roles == o.roles && post_plane == o.post_plane; }
};

std::vector<uint8_t> source_params(const uint64_t* shape, int ndim, uint16_t chain_dtype) {
    std::vector<uint8_t> p;
    p.push_back(uint8_t(ndim));
    for (int d = 0; d < ndim; ++d) put_u32(p, uint32_t(shape[d]));
    p.push_back(uint8_t(chain_dtype)); p.push_back(uint8_t(chain_dtype >> 8));
    return p;
}

// Production chains (python/ptwm/preprocessing/_chains.py:320-357,610-727) and
// their compact role bytes (chain/wire_compact.rs:434-459).
bool chain_for(const ptwm_b200_encode_tensor& t, ChainDef& c, std::string& why) {
    using namespace detail;
    auto src = [&](uint16_t cd) { return std::make_pair(uint16_t(OP_SOURCE), source_params(t.shape, t.ndim, cd)); };
    auto op = [](uint16_t id, std::vector<uint8_t> p = {}) { return std::make_pair(id, p); };
    const uint16_t dt = t.dtype_code;
    if (t.usage == 1) {
        if (dt == 29) c = {K_PASS, {src(0x0010), op(OP_PASS)}, {0x01}};
        else if (dt == 13) c = {K_PASS, {src(0x0006), op(OP_PASS)}, {0x00}};
        else { why = "scale usage needs float8_e4m3fn or uint8"; return false; }
    } else if (t.usage == 2) c = {K_PASS, {src(0x0003), op(OP_PASS)}, {0x08 + 3}};
    else if (t.usage == 3 || dt == 31) c = {K_PASS, {src(0x001F), op(OP_PASS)}, {0x18}};
    else if (dt == 6 || dt == 4) c = {K_M16, {src(0x000F), op(OP_R16), op(OP_BYTESPLIT, {2})}, {0x40 + 8 * 1 + 0, 0x19}};  // fp16 rides the bf16 chain (_chains.py:326)
    else if (dt == 1) c = {K_M32, {src(0x0003), op(OP_R32), op(OP_BYTESPLIT, {4})}, {0x40 + 8 * 3 + 0, 0x40 + 8 * 3 + 1, 0x40 + 8 * 3 + 2, 0x19}};
    else if (dt == 29) c = {K_E4M3, {src(0x0010), op(OP_RE4M3), op(OP_NIBSPLIT)}, {0x10, 0x11}};
    else if (dt == 30) c = {K_E5M2, {src(0x0011), op(OP_RE5M2), op(OP_NIBSPLIT)}, {0x10, 0x11}};
    else if (dt == 13 || dt == 17) c = {K_PASS, {src(uint16_t(chain_dtype_for_public(dt))), op(OP_PASS)}, {0xC0 + 8 - 1}};
    else { why = "no production chain for dtype code " + std::to_string(dt); return false; }
    return true;
}

uint8_t plane_role_byte(uint8_t role) {  // compressor.rs:124-147
    if (role >= 0x40 && role < 0x80) return 5;
    switch (role) {
        case 0x00: case 0x01: case 0x0B: return 2;
        case 0x10: case 0x19: return 3;
        case 0x11: return 4;
        default: return 1;
    }
}

struct PlanePlan {
    uint64_t len = 0, buf_off = 0;   // bytes, offset in the planes buffer
    uint32_t first_chunk = 0, n_chunks = 0;
    int codec = C_IDENTITY;
    uint32_t crc = 0;
    uint8_t role = 0;        // compact terminal role byte of the chain
    uint32_t row_len = 0;    // rows layout of the plane (last dimension of a passthrough tensor), 0 = flat
    // layout
    std::vector<uint64_t> frame_size;  // per chunk (or one entry for an empty plane)
    uint64_t payload_len = 0, state_len = 0;  // state_len: inline state of an unchunked Order1ScaleAC plane
    int shared = -1;         // Order1ScaleAC against this shared state of the prelude instead of a state of its own
};
struct TensorPlan {
    ChainDef chain;
    uint32_t chain_id = 0;
    std::vector<PlanePlan> planes;
    uint64_t hash = 0;
    // candidate chains: the exponent plane after IntDelta lives in a plane of its own until the choice is made
    bool has_delta = false;
    PlanePlan delta;          // plane index = delta_index
    uint32_t delta_index = 0, first_plane = 0;
    uint32_t try_mzs = 0;     // word index of the OR of mantissa plane 0's bytes, + 1 (0 = not looked at)
    int post_op = 0, post_k = 0;  // what was chosen (or given): 1 IntDelta on the last plane, 2 MantissaZeroStrip(post_k) on plane 0
};

// Size of the whole plane under each codec of the menu, the way the reference's
// trial encode compares them (select.rs:27-64: smallest state + payload, the
// first on ties, over dispatch.rs:13-49's order: Order1ScaleAC where it accepts
// the plane, Huffman, rANS, tANS, Identity).  The sizes come from the plane's
// histograms instead of three or four full serial encodes of the plane:
// Huffman is exact up to the per-stream byte rounding, rANS and tANS use the
// information content under their normalised tables, Order1ScaleAC the
// information content under the rows it would fit (`o1sac_bytes` < 0: the
// codec does not accept this plane).
int select_codec(const unsigned long long* hist, uint64_t n, uint32_t menu, double o1sac_bytes, double* best_size = nullptr) {
    double best = 0; int best_codec = -1;
    struct Report { double& b; double* out; ~Report() { if (out) *out = b; } } report{best, best_size};
    auto offer = [&](int codec, double size) { if (best_codec < 0 || size < best) { best = size; best_codec = codec; } };
    uint32_t raw32[256];
    for (int i = 0; i < 256; ++i) raw32[i] = uint32_t(hist[i]);
    if ((menu & PTWM_B200_MENU_O1SAC) && o1sac_bytes >= 0) offer(C_O1SAC, o1sac_bytes);
    if ((menu & PTWM_B200_MENU_HUFFMAN)) {
        double size = 1;
        if (n) {
            uint8_t lengths[256], alive[512], sym_of[256]; uint16_t parent[512]; uint64_t nf[512], raw[256];
            for (int i = 0; i < 256; ++i) raw[i] = hist[i];
            int nw = huffman_lengths<uint64_t>(raw, lengths, nf, parent, alive, sym_of);
            double bits = 0;
            for (int i = 0; i < 256; ++i) bits += double(hist[i]) * lengths[i];
            double blob = (nw <= 127 ? 1 : 2) + (nw + 1) / 2 + 16 + std::ceil(bits / 8) + 2;
            size = blob >= double(n) ? 1.0 + double(n) : 5.0 + blob;
        }
        offer(C_HUFFMAN, size);
    }
    if ((menu & PTWM_B200_MENU_RANS)) {
        double size = 1;
        if (n) {
            uint16_t freqs[256];
            int ms = rans_normalize(raw32, n, freqs);
            if (ms < 0) size = 1.0 + double(n);
            else {
                double bits = 0;
                for (int i = 0; i < 256; ++i) if (hist[i]) bits += double(hist[i]) * std::log2(2048.0 / freqs[i]);
                double blob = 1 + 2 * (ms + 1) + 16 + 16 + std::ceil(bits / 8) + 2;
                size = blob >= double(n) ? 1.0 + double(n) : 5.0 + blob;
            }
        }
        offer(C_RANS, size);
    }
    if ((menu & PTWM_B200_MENU_TANS)) {
        double size = 1;
        if (n) {
            uint16_t norm[256];
            int nsym = n <= 0xFFFFFFFFull ? tans_normalize(raw32, n, norm) : 0;
            if (nsym < 2) size = 1.0 + double(n);
            else {
                double bits = 11;
                for (int i = 0; i < 256; ++i) if (hist[i]) bits += double(hist[i]) * std::log2(2048.0 / norm[i]);
                double blob = 3 + 3 * nsym + 8 + std::ceil(bits / 8);
                size = blob >= double(n) ? 1.0 + double(n) : 5.0 + blob;
            }
        }
        offer(C_TANS, size);
    }
    if ((menu & PTWM_B200_MENU_IDENTITY)) offer(C_IDENTITY, double(n));
    return best_codec;
}

// Order1ScaleAC accepts byte planes with a row layout whose role is a block or global scale in E4M3, E5M2 or E8M0
// (order1_scale_ac.rs:493-514); role bytes as in chain/wire_compact.rs:434-459.
bool o1sac_accepts(uint8_t role, uint32_t row_len) { return row_len && (role <= 0x02 || (role >= 0x08 && role <= 0x0A)); }

// state + payload bytes Order1ScaleAC would need for a plane with these lag-1 counts (the tables of one chunk area, on the host)
double o1sac_estimate(const uint32_t* joint, const uint32_t* marg) {
    double bits = 0;
    uint32_t rows = 0;
    uint16_t pmf[256];
    quantize_pmf256(marg, O1SAC_TOTAL, pmf);
    for (int i = 0; i < 256; ++i) if (marg[i]) bits += double(marg[i]) * std::log2(double(O1SAC_TOTAL) / pmf[i]);
    for (int ctx = 0; ctx < 256; ++ctx) {
        const uint32_t* raw = joint + 256 * ctx;
        uint64_t total = 0;
        for (int i = 0; i < 256; ++i) total += raw[i];
        if (!total) continue;
        ++rows;
        quantize_pmf256(raw, O1SAC_TOTAL, pmf);
        for (int i = 0; i < 256; ++i) if (raw[i]) bits += double(raw[i]) * std::log2(double(O1SAC_TOTAL) / pmf[i]);
    }
    return 32.0 + 512.0 + 512.0 * rows + std::ceil(bits / 8) + 6;
}

struct Piece { uint64_t dst; std::vector<uint8_t> bytes; };

}  // namespace

struct ptwm_b200_encoded {
    uint8_t* d_out = nullptr;
    uint64_t size = 0;
    int device = 0;
    std::vector<std::vector<int>> plane_codecs;
    ~ptwm_b200_encoded() { if (d_out) { DeviceGuard g{device}; cudaFree(d_out); } }
};

namespace {

struct DeviceBuf {
    void* p = nullptr;
    ~DeviceBuf() { if (p) cudaFree(p); }
    template <class T> T* as() { return static_cast<T*>(p); }
    cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 1); }
};

template <class T>
cudaError_t upload_vec(DeviceBuf& b, const std::vector<T>& v, cudaStream_t st) {
    cudaError_t e = b.alloc(v.size() * sizeof(T));
    if (e != cudaSuccess || v.empty()) return e;
    return cudaMemcpyAsync(b.p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice, st);
}

int64_t encode_impl(const ptwm_b200_encode_tensor* tensors, size_t n_tensors, const ptwm_b200_encode_options& opt, int device, cudaStream_t st,
                    CrcTables* d_tabs, ptwm_b200_encoded& enc) {
    const bool chunked = opt.chunk_size != PTWM_B200_CHUNK_NONE;
    const uint64_t chunk_size = !chunked ? (1ull << 32) : opt.chunk_size ? opt.chunk_size : 65536u;
    const uint32_t menu = opt.menu ? opt.menu : 31u;
    if (opt.forced_codec >= 0 && opt.forced_codec != C_IDENTITY && opt.forced_codec != C_HUFFMAN && opt.forced_codec != C_RANS && opt.forced_codec != C_TANS &&
        opt.forced_codec != C_O1SAC)
        return fail(PTWM_RC_UNSUPPORTED, "device encode offers identity, huffman, rans, tans and order1_scale_ac");

    // PTWM_B200_PROFILE=1 prints the wall time of every phase to stderr (the reference's PTWM_PROFILE, compressor.rs:1004-1016)
    const bool profile = std::getenv("PTWM_B200_PROFILE") != nullptr;
    auto prof_t = std::chrono::steady_clock::now();
    auto prof = [&](const char* label) {
        if (!profile) return;
        cudaStreamSynchronize(st);
        auto now = std::chrono::steady_clock::now();
        std::fprintf(stderr, "[ptwm_b200-profile] %s: %.2f ms\n", label, std::chrono::duration<double, std::milli>(now - prof_t).count());
        prof_t = now;
    };
    // ---- chains, registry, planes, chunks -----------------------------------
    std::vector<TensorPlan> plan(n_tensors);
    std::vector<ChainDef> registry;
    std::vector<SplitItem> splits;
    std::vector<EncChunk> chunks;
    std::vector<HashItem> hash_items;
    uint64_t planes_bytes = 0, slots_bytes = 0;
    uint32_t n_planes = 0, tile = 0, n_or_words = 0;
    for (size_t i = 0; i < n_tensors; ++i) {
        const ptwm_b200_encode_tensor& t = tensors[i];
        std::string why;
        if (!t.name || !*t.name || std::strlen(t.name) > 65535) return fail(PTWM_RC_INVALID_INPUT, "tensor name must be 1..65535 bytes");
        if (t.ndim > 8) return fail(PTWM_RC_UNSUPPORTED, "more than 8 dimensions");
        if (!chain_for(t, plan[i].chain, why)) return fail(PTWM_RC_UNSUPPORTED, std::string(t.name) + ": " + why);
        uint64_t elems = 1;
        for (int d = 0; d < t.ndim; ++d) { if (t.shape[d] > 0xFFFFFFFFull) return fail(PTWM_RC_UNSUPPORTED, "dimension exceeds u32"); elems *= t.shape[d]; }
        if (elems * detail::public_dtype_bytes(t.dtype_code) != t.nbytes) return fail(PTWM_RC_INVALID_INPUT, std::string(t.name) + ": nbytes does not match shape x dtype");
        if (t.nbytes && !t.dev_ptr) return fail(PTWM_RC_INVALID_INPUT, "null device pointer");
        const int kind = plan[i].chain.kind, np = kind_planes(kind);
        if (t.post_op) {
            if (kind != K_M16 && kind != K_M32) return fail(PTWM_RC_INVALID_INPUT, std::string(t.name) + ": per-plane ops go on the planes of a byte split");
            if (t.post_op == 1 && t.post_plane != np - 1) return fail(PTWM_RC_UNSUPPORTED, std::string(t.name) + ": IntDelta goes on the exponent plane");
            if (t.post_op == 2 && (t.post_plane != 0 || t.post_k < 1 || t.post_k > 7)) return fail(PTWM_RC_UNSUPPORTED, std::string(t.name) + ": MantissaZeroStrip(1..7) goes on mantissa plane 0");
            if (t.post_op > 2) return fail(PTWM_RC_UNSUPPORTED, std::string(t.name) + ": unknown per-plane op");
        }
        plan[i].first_plane = n_planes;
        const uint64_t plane_len = t.nbytes / uint64_t(kind_elem_bytes(kind));
        if (plane_len > 0xFFFFFFFFull) return fail(PTWM_RC_UNSUPPORTED, "plane longer than 4 GiB");
        SplitItem sp{reinterpret_cast<const uint8_t*>(uintptr_t(t.dev_ptr)), {0, 0, 0, 0}, plane_len, uint32_t(kind), tile};
        plan[i].planes.resize(size_t(np));
        for (int p = 0; p < np; ++p) {
            PlanePlan& pp = plan[i].planes[size_t(p)];
            pp.len = plane_len; pp.buf_off = planes_bytes; pp.first_chunk = uint32_t(chunks.size());
            pp.role = plan[i].chain.roles[size_t(p)];
            // a passthrough plane keeps the tensor's rows (its last dimension); split planes are flat (transforms/byte_split.rs:76)
            pp.row_len = kind == K_PASS && t.ndim >= 1 && t.shape[t.ndim - 1] && plane_len ? uint32_t(t.shape[t.ndim - 1]) : 0u;
            sp.plane_off[p] = planes_bytes;
            planes_bytes += align_up(plane_len, 16);
            for (uint64_t off = 0; off < plane_len; off += chunk_size) {
                uint32_t n = uint32_t(std::min<uint64_t>(chunk_size, plane_len - off));
                uint32_t cap = uint32_t(align_up(uint64_t((n + 3) / 4) * 3 / 2 + 16, 16));  // <= 12 bits per symbol plus the rANS state
                // chunks are coded flat (compressor.rs:352-355); a whole plane keeps its rows
                chunks.push_back(EncChunk{pp.buf_off + off, 0, 0, n, cap, n_planes, chunked ? 0u : pp.row_len});
            }
            pp.n_chunks = uint32_t(chunks.size()) - pp.first_chunk;
            ++n_planes;
        }
        if (plane_len) { splits.push_back(sp); tile += uint32_t((plane_len + SPLIT_TILE - 1) / SPLIT_TILE); }
        if (opt.emit_payload_hash) hash_items.push_back(HashItem{make_ref(SP_BLOB, t.dev_ptr), t.nbytes});
        const bool split_kind = (kind == K_M16 || kind == K_M32) && plane_len;
        plan[i].post_op = t.post_op; plan[i].post_k = t.post_k;
        plan[i].has_delta = split_kind && (t.post_op == 1 || (!t.post_op && (opt.candidates & PTWM_B200_TRY_INTDELTA)));
        if (split_kind && (t.post_op == 2 || (!t.post_op && (opt.candidates & PTWM_B200_TRY_MZS)))) plan[i].try_mzs = ++n_or_words;
    }
    // the IntDelta candidates' exponent planes: planes of their own behind the others
    for (size_t i = 0; i < n_tensors; ++i) {
        TensorPlan& tp = plan[i];
        if (!tp.has_delta) continue;
        const PlanePlan& ex = tp.planes.back();
        PlanePlan& pp = tp.delta;
        pp.len = ex.len; pp.buf_off = planes_bytes; pp.first_chunk = uint32_t(chunks.size()); pp.role = ex.role; pp.row_len = 0;
        planes_bytes += align_up(pp.len, 16);
        for (uint32_t k = 0; k < ex.n_chunks; ++k) { EncChunk c = chunks[ex.first_chunk + k]; c.plane_off = pp.buf_off + (c.plane_off - ex.buf_off); c.plane = n_planes; chunks.push_back(c); }
        pp.n_chunks = ex.n_chunks;
        tp.delta_index = n_planes++;
    }
    const uint32_t n_chunks = uint32_t(chunks.size());

    prof("plan (host)");
    // ---- device pipeline: split, histograms ---------------------------------
    DeviceBuf d_planes, d_splits, d_chunks, d_hist, d_plane_hist, d_codec, d_tables, d_results, d_slots;
    CUDA_TRY(d_planes.alloc(planes_bytes));
    CUDA_TRY(upload_vec(d_splits, splits, st));
    CUDA_TRY(upload_vec(d_chunks, chunks, st));
    CUDA_TRY(d_hist.alloc(uint64_t(n_chunks) * 1024));
    CUDA_TRY(d_plane_hist.alloc(uint64_t(n_planes) * 256 * 8));
    CUDA_TRY(cudaMemsetAsync(d_plane_hist.p, 0, uint64_t(n_planes) * 256 * 8 + (n_planes ? 0 : 1), st));
    if (tile) { split_kernel<<<tile, 256, 0, st>>>(d_splits.as<SplitItem>(), uint32_t(splits.size()), d_planes.as<uint8_t>()); CUDA_TRY(cudaGetLastError()); }
    DeviceBuf d_or;
    std::vector<uint32_t> or_words(n_or_words);
    if (n_or_words) { CUDA_TRY(d_or.alloc(uint64_t(n_or_words) * 4)); CUDA_TRY(cudaMemsetAsync(d_or.p, 0, uint64_t(n_or_words) * 4, st)); }
    for (auto& tp : plan) {
        auto blocks = [](uint64_t n) { return unsigned(std::min<uint64_t>((n + 4095) / 4096, 2368)); };
        if (tp.has_delta) { delta_kernel<<<blocks(tp.delta.len), 256, 0, st>>>(d_planes.as<uint8_t>() + tp.planes.back().buf_off, d_planes.as<uint8_t>() + tp.delta.buf_off, tp.delta.len); CUDA_TRY(cudaGetLastError()); }
        if (tp.try_mzs) { or_bytes_kernel<<<blocks(tp.planes[0].len), 256, 0, st>>>(d_planes.as<uint8_t>() + tp.planes[0].buf_off, tp.planes[0].len, d_or.as<uint32_t>() + tp.try_mzs - 1); CUDA_TRY(cudaGetLastError()); }
    }
    if (n_or_words) CUDA_TRY(cudaMemcpyAsync(or_words.data(), d_or.p, uint64_t(n_or_words) * 4, cudaMemcpyDeviceToHost, st));
    if (n_chunks) { hist_kernel<<<n_chunks, 128, 0, st>>>(d_chunks.as<EncChunk>(), d_planes.as<uint8_t>(), d_hist.as<uint32_t>(), d_plane_hist.as<unsigned long long>()); CUDA_TRY(cudaGetLastError()); }
    std::vector<unsigned long long> plane_hist(size_t(n_planes) * 256);
    if (n_planes) CUDA_TRY(cudaMemcpyAsync(plane_hist.data(), d_plane_hist.p, plane_hist.size() * 8, cudaMemcpyDeviceToHost, st));

    // plane CRCs and payload hashes run on the same stream meanwhile
    DeviceBuf d_verify, d_acc, d_hitems, d_hout;
    std::vector<VerifyTensor> verify;
    uint64_t n_runs = 0;
    if (opt.emit_plane_crc) {
        auto add = [&](const PlanePlan& pp, uint32_t acc) {
            if (pp.len) { verify.push_back(VerifyTensor{make_ref(SP_OUT, pp.buf_off), pp.len, n_runs, K_PASS, acc}); n_runs += (pp.len + VERIFY_RUN - 1) / VERIFY_RUN; }
        };
        for (auto& tp : plan) {  // accumulator = global plane index; a plane CRC covers the terminal's bytes, so the delta planes get theirs too
            for (size_t p = 0; p < tp.planes.size(); ++p) add(tp.planes[p], tp.first_plane + uint32_t(p));
            if (tp.has_delta) add(tp.delta, tp.delta_index);
        }
        CUDA_TRY(upload_vec(d_verify, verify, st));
        CUDA_TRY(d_acc.alloc(uint64_t(n_planes) * 4));
        CUDA_TRY(cudaMemsetAsync(d_acc.p, 0, uint64_t(n_planes) * 4 + (n_planes ? 0 : 1), st));
        if (n_runs) {
            Bases b{nullptr, 0, 0, nullptr, d_planes.as<uint8_t>()};
            crc_planes_kernel<<<uint32_t((n_runs + 127) / 128), 128, 0, st>>>(d_verify.as<VerifyTensor>(), uint32_t(verify.size()), n_runs, b, d_tabs, d_acc.as<uint32_t>());
            CUDA_TRY(cudaGetLastError());
        }
    }
    std::vector<uint64_t> hashes(hash_items.size());
    if (!hash_items.empty()) {
        CUDA_TRY(upload_vec(d_hitems, hash_items, st));
        CUDA_TRY(d_hout.alloc(hash_items.size() * 8));
        Bases b{nullptr, 0, 0, nullptr, nullptr};
        xxh64_kernel<<<uint32_t(hash_items.size()), 32, 0, st>>>(d_hitems.as<HashItem>(), uint32_t(hash_items.size()), b, d_hout.as<uint64_t>());
        CUDA_TRY(cudaGetLastError());
        CUDA_TRY(cudaMemcpyAsync(hashes.data(), d_hout.p, hashes.size() * 8, cudaMemcpyDeviceToHost, st));
    }
    std::vector<uint32_t> accs(n_planes);
    if (opt.emit_plane_crc && n_planes) CUDA_TRY(cudaMemcpyAsync(accs.data(), d_acc.p, accs.size() * 4, cudaMemcpyDeviceToHost, st));

    // Lag-1 counts of every plane Order1ScaleAC accepts, with the plane's rows, for the size comparison below.
    std::vector<double> o1sac_size(n_planes, -1.0);
    std::vector<uint32_t> counts, which;      // the counts stay for the shared-state passes
    std::vector<int> counts_of(n_planes, -1); // plane -> its place in `which`
    if (opt.forced_codec < 0 && (menu & PTWM_B200_MENU_O1SAC)) {
        std::vector<EncChunk> whole;
        std::vector<uint32_t> list;
        uint32_t pi = 0;
        for (auto& tp : plan) for (auto& pp : tp.planes) {
            if (pp.len && o1sac_accepts(pp.role, pp.row_len) && pp.len % pp.row_len == 0) {
                list.push_back(uint32_t(whole.size()));
                whole.push_back(EncChunk{pp.buf_off, 0, uint64_t(whole.size()) * (O1E_PRESENT), uint32_t(pp.len), 0, pi, pp.row_len});
                which.push_back(pi);
            }
            ++pi;
        }
        if (!whole.empty()) {
            DeviceBuf d_whole, d_list, d_counts;
            CUDA_TRY(upload_vec(d_whole, whole, st));
            CUDA_TRY(upload_vec(d_list, list, st));
            CUDA_TRY(d_counts.alloc(whole.size() * size_t(O1E_PRESENT)));
            CUDA_TRY(cudaMemsetAsync(d_counts.p, 0, whole.size() * size_t(O1E_PRESENT), st));
            o1sac_count_kernel<<<uint32_t(whole.size()), 256, 0, st>>>(d_whole.as<EncChunk>(), d_list.as<uint32_t>(), d_planes.as<uint8_t>(), d_counts.as<uint8_t>());
            CUDA_TRY(cudaGetLastError());
            counts.resize(whole.size() * size_t(O1E_PRESENT / 4));
            CUDA_TRY(cudaMemcpyAsync(counts.data(), d_counts.p, counts.size() * 4, cudaMemcpyDeviceToHost, st));
            CUDA_TRY(cudaStreamSynchronize(st));
            for (size_t k = 0; k < whole.size(); ++k) {
                const uint32_t* base = counts.data() + k * size_t(O1E_PRESENT / 4);
                o1sac_size[which[k]] = o1sac_estimate(base + O1E_JOINT / 4, base + O1E_MARG / 4);
                counts_of[which[k]] = int(k);
            }
        }
    }
    CUDA_TRY(cudaStreamSynchronize(st));

    prof("split, histograms, CRC / hash, counts");
    // ---- shared states (compressor.rs:834-881): only whole planes can use one (a chunked plane carries its states inline,
    //      compressor.rs:324-381), and only when the codec is chosen, not forced
    FitResult shared;
    std::vector<std::vector<uint8_t>> shared_bytes;
    if (!chunked && opt.forced_codec < 0 && (opt.candidates & PTWM_B200_TRY_SHARED_STATE) && !which.empty()) {
        std::vector<FitCounts> fc;
        for (size_t k = 0; k < which.size(); ++k) {
            const uint32_t* base = counts.data() + k * size_t(O1E_PRESENT / 4);
            fc.push_back(FitCounts{base + O1E_JOINT / 4, base + O1E_MARG / 4});
        }
        cudaError_t fit_err = cudaSuccess;
        shared = fit_shared_order1(fc, [&](const std::vector<FitState>& own, const std::vector<uint32_t>& pairs) {
            std::vector<double> d(pairs.size() / 2, 0.0);
            std::vector<uint16_t> dense(own.size() * size_t(257 * 256));
            for (size_t k = 0; k < own.size(); ++k) fit_dense_rows(own[k], dense.data() + k * size_t(257 * 256));
            DeviceBuf d_dense, d_pairs, d_dist;
            if ((fit_err = upload_vec(d_dense, dense, st)) != cudaSuccess || (fit_err = upload_vec(d_pairs, pairs, st)) != cudaSuccess ||
                (fit_err = d_dist.alloc(d.size() * sizeof(double))) != cudaSuccess) return d;
            fit_pair_distance_kernel<<<uint32_t(d.size()), 256, 0, st>>>(d_dense.as<uint16_t>(), d_pairs.as<uint32_t>(), d_dist.as<double>());
            if ((fit_err = cudaGetLastError()) != cudaSuccess) return d;
            if ((fit_err = cudaMemcpyAsync(d.data(), d_dist.p, d.size() * sizeof(double), cudaMemcpyDeviceToHost, st)) != cudaSuccess) return d;
            fit_err = cudaStreamSynchronize(st);
            return d;
        });
        CUDA_TRY(fit_err);
        for (auto& stt : shared.states) shared_bytes.push_back(stt.serialize());
    }

    prof("shared-state fit");
    // ---- codec per plane ------------------------------------------------------
    std::vector<uint8_t> plane_codec(n_planes);
    std::vector<uint32_t> tans_chunks;  // chunks of tANS planes, for the kernel that codes them
    std::vector<uint32_t> o1sac_chunks, o1shared_chunks, o1shared_state;  // chunks that fit their own state / that code against shared state o1shared_state[k]
    uint64_t tables_bytes = 0;
    std::vector<std::pair<uint32_t, uint32_t>> recrc;  // (tensor, accumulator) of planes shifted by MantissaZeroStrip: their CRC is taken again below
    {
        const CrcTables& T = crc_tables();
        const uint32_t sel_menu = opt.forced_codec >= 0 ? (opt.forced_codec == C_IDENTITY ? PTWM_B200_MENU_IDENTITY : opt.forced_codec == C_HUFFMAN ? PTWM_B200_MENU_HUFFMAN :
                                                           opt.forced_codec == C_RANS ? PTWM_B200_MENU_RANS : opt.forced_codec == C_TANS ? PTWM_B200_MENU_TANS : 0u) : menu;
        auto pick = [&](uint32_t plane_index, const unsigned long long* hist, uint64_t len, double* size) {
            if (opt.forced_codec == C_O1SAC) { if (size) *size = double(len); return int(C_O1SAC); }
            int c = select_codec(hist, len, sel_menu, opt.forced_codec >= 0 ? -1.0 : o1sac_size[plane_index], size);
            return opt.forced_codec >= 0 ? opt.forced_codec : c;
        };
        for (size_t i = 0; i < n_tensors; ++i) {
            TensorPlan& tp = plan[i];
            enc.plane_codecs.emplace_back();
            const size_t np = tp.planes.size();
            std::vector<double> size(np, 0.0);
            for (size_t p = 0; p < np; ++p) {
                tp.planes[p].codec = pick(tp.first_plane + uint32_t(p), &plane_hist[size_t(tp.first_plane + p) * 256], tp.planes[p].len, &size[p]);
                if (tp.planes[p].codec < 0) return fail(PTWM_RC_INVALID_INPUT, "empty codec menu");
                // the same plane against every shared state, in prelude order: such a payload carries no state, and the first
                // strictly smaller candidate wins (compressor.rs:883-939, select.rs:27-64)
                const int ck = counts_of[tp.first_plane + p];
                if (ck >= 0 && !shared.states.empty()) {
                    const uint32_t* base = counts.data() + size_t(ck) * size_t(O1E_PRESENT / 4);
                    const FitCounts fc{base + O1E_JOINT / 4, base + O1E_MARG / 4};
                    for (size_t sj = 0; sj < shared.states.size(); ++sj) {
                        const double est = std::ceil(fit_cross_entropy_bits(fc, shared.states[sj]) / 8) + 6;
                        if (est < size[p]) { size[p] = est; tp.planes[p].codec = C_O1SAC; tp.planes[p].shared = int(sj); }
                    }
                }
            }
            // ---- chain: the plain split, or the candidate with the smallest total, the first in the reference's candidate order on ties
            //      (split, IntDelta, MantissaZeroStrip 1..4: python/ptwm/preprocessing/_chains.py:1151-1185; compressor.rs:504-665)
            double delta_size = 0; int delta_codec = -1;
            if (tp.has_delta) delta_codec = pick(tp.delta_index, &plane_hist[size_t(tp.delta_index) * 256], tp.delta.len, &delta_size);
            const uint32_t orv = tp.try_mzs ? or_words[tp.try_mzs - 1] : 0xFFu;
            auto strip_fits = [&](int k) { return tp.planes[0].len && (orv & ((1u << k) - 1)) == 0; };
            auto stripped = [&](int k, double* sz) {  // plane 0 after the shift: the same counts under other labels
                unsigned long long h[256] = {0};
                const unsigned long long* src = &plane_hist[size_t(tp.first_plane) * 256];
                for (int v = 0; v < 256; ++v) if (src[v]) h[v >> k] += src[v];
                return pick(tp.first_plane, h, tp.planes[0].len, sz);
            };
            if (tp.post_op == 2 && !strip_fits(tp.post_k))
                return fail(PTWM_RC_INVALID_INPUT, std::string(tensors[i].name) + ": MantissaZeroStrip(" + std::to_string(tp.post_k) + "): the plane has a byte with non-zero low bits");
            if (!tp.post_op && (tp.has_delta || tp.try_mzs)) {
                double base = 0;
                for (double v : size) base += v;
                double best = base;
                if (tp.has_delta && base - size[np - 1] + delta_size < best) { best = base - size[np - 1] + delta_size; tp.post_op = 1; }
                if (tp.try_mzs) for (int k = 1; k <= 4 && strip_fits(k); ++k) {
                    double sz; stripped(k, &sz);
                    if (base - size[0] + sz < best) { best = base - size[0] + sz; tp.post_op = 2; tp.post_k = k; }
                }
            }
            if (tp.post_op == 1) {  // the exponent plane is the delta plane from here on
                if (delta_codec < 0) return fail(PTWM_RC_INTERNAL, "IntDelta chosen without its plane");
                tp.delta.codec = delta_codec;
                tp.planes[np - 1] = tp.delta;
                tp.chain.nodes.push_back({uint16_t(detail::OP_INTDELTA), {}});
                tp.chain.post_plane = int(np) - 1;
            } else if (tp.post_op == 2) {
                tp.planes[0].codec = stripped(tp.post_k, nullptr);
                const uint64_t n = tp.planes[0].len;
                shift_right_kernel<<<unsigned(std::min<uint64_t>((n + 4095) / 4096, 2368)), 256, 0, st>>>(d_planes.as<uint8_t>() + tp.planes[0].buf_off, n, uint32_t(tp.post_k));
                CUDA_TRY(cudaGetLastError());
                relabel_hist_kernel<<<tp.planes[0].n_chunks, 256, 0, st>>>(d_hist.as<uint32_t>(), tp.planes[0].first_chunk, uint32_t(tp.post_k));
                CUDA_TRY(cudaGetLastError());
                tp.chain.nodes.push_back({uint16_t(detail::OP_MZS), {uint8_t(tp.post_k)}});
                tp.chain.post_plane = 0;
                if (opt.emit_plane_crc) recrc.push_back({uint32_t(i), tp.first_plane});
            }
            // the chain is final: register it (a Source whose params equal the record's own shape/dtype is written bound: compressor.rs:708-715)
            {
                const ptwm_b200_encode_tensor& t = tensors[i];
                ChainDef reg = tp.chain;
                int cd = detail::chain_dtype_for_public(t.dtype_code);
                if (cd >= 0 && reg.nodes[0].second == source_params(t.shape, t.ndim, uint16_t(cd))) reg.nodes[0].second.clear();
                auto found = std::find(registry.begin(), registry.end(), reg);
                if (found == registry.end()) { registry.push_back(reg); found = registry.end() - 1; }
                tp.chain_id = uint32_t(found - registry.begin());
                if (registry.size() > 0x8000) return fail(PTWM_RC_UNSUPPORTED, "more than 32768 distinct chains");
            }
            for (size_t p = 0; p < np; ++p) {
                PlanePlan& pp = tp.planes[p];
                const uint32_t pi = (tp.post_op == 1 && p == np - 1) ? tp.delta_index : tp.first_plane + uint32_t(p);
                if (pp.codec == C_O1SAC && !chunked && pp.row_len && pp.len % pp.row_len) return fail(PTWM_RC_INVALID_INPUT, "order1_scale_ac: the row length does not divide the plane");
                plane_codec[pi] = uint8_t(pp.codec);
                enc.plane_codecs.back().push_back(pp.codec);
                if (opt.emit_plane_crc) pp.crc = pp.len ? ~(accs[pi] ^ gf2_mulmod(x_pow_8n(T.x2n, pp.len), 0xFFFFFFFFu)) : 0u;
                if (pp.codec != C_IDENTITY)  // stream slots and table areas only for planes that get coded
                    for (uint32_t k = 0; k < pp.n_chunks; ++k) {
                        EncChunk& ch = chunks[pp.first_chunk + k];
                        ch.slot_off = slots_bytes; slots_bytes += uint64_t(ch.slot_cap) * 4;
                        ch.table_off = tables_bytes; tables_bytes += enc_table_bytes(pp.codec);
                        if (pp.codec == C_O1SAC) (pp.shared >= 0 ? o1shared_chunks : o1sac_chunks).push_back(pp.first_chunk + k);
                        if (pp.codec == C_TANS) tans_chunks.push_back(pp.first_chunk + k);
                        if (pp.codec == C_O1SAC && pp.shared >= 0) o1shared_state.push_back(uint32_t(pp.shared));
                    }
            }
            if (opt.emit_payload_hash) tp.hash = hashes[i];
        }
        // planes that are not written (the exponent plane or its delta twin, whichever lost) get no encoding pass: plane_codec stays Identity
        if (!recrc.empty()) {  // CRC of the shifted planes
            std::vector<VerifyTensor> again;
            uint64_t runs = 0;
            for (auto& rc : recrc) {
                const PlanePlan& pp = plan[rc.first].planes[0];
                again.push_back(VerifyTensor{make_ref(SP_OUT, pp.buf_off), pp.len, runs, K_PASS, rc.second});
                runs += (pp.len + VERIFY_RUN - 1) / VERIFY_RUN;
                CUDA_TRY(cudaMemsetAsync(d_acc.as<uint32_t>() + rc.second, 0, 4, st));
            }
            DeviceBuf d_again;
            CUDA_TRY(upload_vec(d_again, again, st));
            Bases b{nullptr, 0, 0, nullptr, d_planes.as<uint8_t>()};
            crc_planes_kernel<<<uint32_t((runs + 127) / 128), 128, 0, st>>>(d_again.as<VerifyTensor>(), uint32_t(again.size()), runs, b, d_tabs, d_acc.as<uint32_t>());
            CUDA_TRY(cudaGetLastError());
            CUDA_TRY(cudaMemcpyAsync(accs.data(), d_acc.p, accs.size() * 4, cudaMemcpyDeviceToHost, st));
            CUDA_TRY(cudaStreamSynchronize(st));
            for (auto& rc : recrc) {
                PlanePlan& pp = plan[rc.first].planes[0];
                pp.crc = ~(accs[rc.second] ^ gf2_mulmod(x_pow_8n(T.x2n, pp.len), 0xFFFFFFFFu));
            }
        }
    }

    prof("codec and chain choice (host)");
    // ---- tables and streams ---------------------------------------------------
    CUDA_TRY(upload_vec(d_codec, plane_codec, st));
    if (n_chunks) CUDA_TRY(cudaMemcpyAsync(d_chunks.p, chunks.data(), chunks.size() * sizeof(EncChunk), cudaMemcpyHostToDevice, st));
    CUDA_TRY(d_tables.alloc(tables_bytes));
    CUDA_TRY(d_results.alloc(uint64_t(n_chunks) * sizeof(EncResult)));
    CUDA_TRY(cudaMemsetAsync(d_results.p, 0, uint64_t(n_chunks) * sizeof(EncResult) + (n_chunks ? 0 : 1), st));
    CUDA_TRY(d_slots.alloc(slots_bytes));
    std::vector<EncResult> results(n_chunks);
    prof("  work memory for tables and streams");
    DeviceBuf d_o1list, d_tanslist;
    if (!o1sac_chunks.empty()) {  // Order1ScaleAC: counts, rows, then the range coder, one chunk per block / thread
        CUDA_TRY(upload_vec(d_o1list, o1sac_chunks, st));
        for (uint32_t ci : o1sac_chunks) CUDA_TRY(cudaMemsetAsync(d_tables.as<uint8_t>() + chunks[ci].table_off, 0, O1E_PRESENT, st));
        const uint32_t n_o1 = uint32_t(o1sac_chunks.size());
        o1sac_count_kernel<<<n_o1, 256, 0, st>>>(d_chunks.as<EncChunk>(), d_o1list.as<uint32_t>(), d_planes.as<uint8_t>(), d_tables.as<uint8_t>());
        CUDA_TRY(cudaGetLastError());
        o1sac_fit_kernel<<<n_o1, 288, 0, st>>>(d_chunks.as<EncChunk>(), d_o1list.as<uint32_t>(), d_tables.as<uint8_t>(), d_results.as<EncResult>());
        CUDA_TRY(cudaGetLastError());
        o1sac_encode_kernel<<<(n_o1 + 63) / 64, 64, 0, st>>>(d_chunks.as<EncChunk>(), d_o1list.as<uint32_t>(), n_o1, d_planes.as<uint8_t>(), d_tables.as<uint8_t>(),
                                                             d_slots.as<uint8_t>(), d_results.as<EncResult>());
        CUDA_TRY(cudaGetLastError());
    }
    DeviceBuf d_o1shared;
    if (!o1shared_chunks.empty()) {  // the coder's tables of a shared state, laid out like the ones o1sac_fit_kernel leaves, one copy per plane
        std::vector<std::vector<uint8_t>> images;
        for (auto& stt : shared.states) {
            images.emplace_back(size_t(ENC_O1SAC_TABLE_BYTES - O1E_PRESENT), uint8_t(0));
            uint8_t* img = images.back().data();
            uint8_t* present = img;
            uint16_t* rank = reinterpret_cast<uint16_t*>(img + (O1E_RANK - O1E_PRESENT));
            uint16_t* pmf = reinterpret_cast<uint16_t*>(img + (O1E_PMF - O1E_PRESENT));
            uint16_t* cum = reinterpret_cast<uint16_t*>(img + (O1E_CUM - O1E_PRESENT));
            auto put_row = [&](uint32_t row, const uint16_t* src) {
                uint32_t acc = 0;
                for (int i = 0; i < 256; ++i) { pmf[256 * row + i] = src[i]; cum[256 * row + i] = uint16_t(acc); acc += src[i]; }
            };
            put_row(0, stt.marginal);
            uint32_t k = 0;
            for (uint32_t ctx = 0; ctx < 256; ++ctx) {
                const bool has = (stt.bitmap[ctx >> 3] >> (ctx & 7)) & 1;
                present[ctx] = has; rank[ctx] = uint16_t(k);
                if (has) put_row(1 + ctx, stt.rows[k++].data());
            }
        }
        for (size_t k = 0; k < o1shared_chunks.size(); ++k)
            CUDA_TRY(cudaMemcpyAsync(d_tables.as<uint8_t>() + chunks[o1shared_chunks[k]].table_off + O1E_PRESENT, images[o1shared_state[k]].data(),
                                     images[o1shared_state[k]].size(), cudaMemcpyHostToDevice, st));
        CUDA_TRY(upload_vec(d_o1shared, o1shared_chunks, st));
        const uint32_t n_sh = uint32_t(o1shared_chunks.size());
        o1sac_encode_kernel<<<(n_sh + 63) / 64, 64, 0, st>>>(d_chunks.as<EncChunk>(), d_o1shared.as<uint32_t>(), n_sh, d_planes.as<uint8_t>(), d_tables.as<uint8_t>(),
                                                             d_slots.as<uint8_t>(), d_results.as<EncResult>());
        CUDA_TRY(cudaGetLastError());
        CUDA_TRY(cudaStreamSynchronize(st));  // the images are host memory of this scope
    }
    prof("  order1_scale_ac chunks");
    if (n_chunks) {
        table_kernel<<<(n_chunks + 63) / 64, 64, 0, st>>>(d_chunks.as<EncChunk>(), n_chunks, d_codec.as<uint8_t>(), d_hist.as<uint32_t>(), d_tables.as<uint8_t>(), d_results.as<EncResult>());
        CUDA_TRY(cudaGetLastError());
        prof("  table_kernel");
        encode_kernel<<<(n_chunks * 4 + 127) / 128, 128, 0, st>>>(d_chunks.as<EncChunk>(), n_chunks, d_codec.as<uint8_t>(), d_planes.as<uint8_t>(), d_tables.as<uint8_t>(), d_slots.as<uint8_t>(), d_results.as<EncResult>());
        CUDA_TRY(cudaGetLastError());
        if (!tans_chunks.empty()) {
            CUDA_TRY(upload_vec(d_tanslist, tans_chunks, st));
            const uint32_t n_t = uint32_t(tans_chunks.size());
            CUDA_TRY(cudaFuncSetAttribute(tans_encode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TENC_SMEM));  // per device; cheap to repeat
            tans_encode_kernel<<<(n_t + TENC_CHUNKS - 1) / TENC_CHUNKS, 32, TENC_SMEM, st>>>(d_chunks.as<EncChunk>(), d_tanslist.as<uint32_t>(), n_t, d_planes.as<uint8_t>(),
                                                                                         d_tables.as<uint8_t>(), d_slots.as<uint8_t>(), d_results.as<EncResult>());
            CUDA_TRY(cudaGetLastError());
        }
        prof("  encode_kernel");
        CUDA_TRY(cudaMemcpyAsync(results.data(), d_results.p, results.size() * sizeof(EncResult), cudaMemcpyDeviceToHost, st));
    }
    CUDA_TRY(cudaStreamSynchronize(st));

    prof("tables and streams");
    // ---- layout: chunk frames, plane payloads, records ------------------------
    std::vector<uint32_t> chunk_mode(n_chunks);
    const uint64_t frame_hdr = chunked ? 5 : 0;  // [state_version][state_len u32] in front of every chunk; an unchunked plane has none
    for (auto& tp : plan) for (auto& pp : tp.planes) {
        if (pp.len == 0) {  // an empty plane is one empty chunk (compressor.rs:333-345), or an empty payload / the raw tag alone when unchunked
            // Order1ScaleAC fitted to no symbols: no rows, the smoothed marginal (16 everywhere), and the coder's six flush bytes
            const uint64_t body = pp.codec == C_IDENTITY ? 0 : pp.codec == C_O1SAC ? 6 : 1;
            if (pp.codec == C_O1SAC) pp.state_len = 32 + 512;
            pp.frame_size.push_back(frame_hdr + pp.state_len + body);
            pp.payload_len = pp.frame_size[0];
            continue;
        }
        for (uint32_t k = 0; k < pp.n_chunks; ++k) {
            uint32_t ci = pp.first_chunk + k;
            const EncResult& r = results[ci];
            uint64_t n = chunks[ci].n, size;
            if (pp.codec == C_IDENTITY) { chunk_mode[ci] = 0; size = frame_hdr + n; }
            else if (pp.codec == C_O1SAC) {
                chunk_mode[ci] = pp.shared >= 0 ? (5 | GATHER_BARE) : 5;
                const uint64_t own_state = pp.shared >= 0 ? 0 : r.stream_len[1];
                size = frame_hdr + own_state + r.stream_len[0];  // a plane's own state sits in front of the coder's bytes
                if (!chunked) pp.state_len = own_state;
            } else {
                uint64_t blob;
                if (pp.codec == C_TANS) blob = 3 + 3 * uint64_t(r.hdr_n) + 8 + r.stream_len[0];
                else {
                    uint64_t hdr = pp.codec == C_RANS ? 1 + 2 * (uint64_t(r.hdr_n) + 1) : (r.hdr_n <= 127 ? 1 : 2) + (uint64_t(r.hdr_n) + 1) / 2;
                    blob = hdr + 16 + uint64_t(r.stream_len[0]) + r.stream_len[1] + r.stream_len[2] + r.stream_len[3];
                }
                // stored raw when coding does not shrink the chunk (compress.rs NotBeneficial) or the length rule refuses it (length_prefix.rs:29-33)
                bool coded = r.coded && blob < n && (pp.codec == C_HUFFMAN || n <= (1ull << 30) || n <= blob * 64);
                chunk_mode[ci] = coded ? (pp.codec == C_RANS ? 2 : pp.codec == C_HUFFMAN ? 3 : 4) : 1;
                size = coded ? frame_hdr + 1 + 4 + blob : frame_hdr + 1 + n;
            }
            if (!chunked) chunk_mode[ci] |= GATHER_NOFRAME;
            pp.frame_size.push_back(size);
            pp.payload_len += size;
        }
        if (pp.payload_len > 0xFFFFFFFFull) return fail(PTWM_RC_UNSUPPORTED, "plane payload exceeds the u32 offset range (compressor.rs:370-372)");
    }

    // Extension Table: chain ops in registry order, then the used codecs in built-in order (container.rs:167-223)
    std::vector<std::pair<uint8_t, uint16_t>> table;
    for (auto& c : registry) for (auto& nd : c.nodes) if (std::find(table.begin(), table.end(), std::make_pair(uint8_t(1), nd.first)) == table.end()) table.push_back({1, nd.first});
    for (int codec : {int(C_IDENTITY), int(C_HUFFMAN), int(C_RANS), int(C_TANS), int(C_O1SAC)}) {
        bool used = false;
        for (auto& tp : plan) for (auto& pp : tp.planes) used |= pp.codec == codec;
        if (used) table.push_back({2, uint16_t(codec)});
    }
    auto table_index = [&](uint8_t tag, uint16_t id) { return uint64_t(std::find(table.begin(), table.end(), std::make_pair(tag, id)) - table.begin()); };
    std::vector<uint8_t> et, prelude, reg;
    {   // prelude.rs:23-57: the shared states some plane uses, under the ids the fit gave them (compressor.rs:945-949)
        std::vector<char> used(shared.states.size(), 0);
        for (auto& tp : plan) for (auto& pp : tp.planes) if (pp.shared >= 0) used[size_t(pp.shared)] = 1;
        uint32_t n_used = 0;
        for (char u : used) n_used += u;
        put_u32(prelude, n_used);
        for (size_t k = 0; k < used.size(); ++k) {
            if (!used[k]) continue;
            const std::vector<uint8_t>& sb = shared_bytes[k];
            const std::string& name = shared.names[k];
            prelude.push_back(uint8_t(k)); prelude.push_back(uint8_t(k >> 8));
            prelude.push_back(uint8_t(C_O1SAC)); prelude.push_back(uint8_t(C_O1SAC >> 8));
            prelude.push_back(1);       // state_format_version of Order1ScaleAC
            prelude.push_back(0x02);    // applies_to_mask: scale planes (fit/order1.rs:333,369)
            prelude.push_back(0); prelude.push_back(0);
            put_u64(prelude, xxh64_host(sb.data(), sb.size()));
            prelude.push_back(uint8_t(name.size())); prelude.push_back(uint8_t(name.size() >> 8));
            prelude.insert(prelude.end(), name.begin(), name.end());
            for (size_t z = (4 - name.size() % 4) % 4; z; --z) prelude.push_back(0);
            put_u32(prelude, uint32_t(sb.size()));
            prelude.insert(prelude.end(), sb.begin(), sb.end());
        }
    }
    put_varint(et, table.size());
    for (auto& e : table) { et.push_back(e.first); put_varint(et, e.second); }
    put_varint(reg, registry.size());
    for (auto& c : registry) {  // CW2, every edge a spine edge (chain/wire_compact.rs:140-245)
        std::vector<uint8_t> cb;
        // nodes, edges, terminals; the leading edges (i, 0) -> (i + 1, 0) are the spine and only counted, an op between the split
        // (node 2) and a terminal hangs off output `post_plane` by an explicit edge and takes that terminal over
        const size_t last = c.nodes.size() - 1, split = c.post_plane >= 0 ? last - 1 : last;
        put_varint(cb, c.nodes.size()); put_varint(cb, last); put_varint(cb, c.roles.size());
        for (auto& nd : c.nodes) { put_varint(cb, table_index(1, nd.first)); put_varint(cb, nd.second.size()); cb.insert(cb.end(), nd.second.begin(), nd.second.end()); }
        const bool on_spine = c.post_plane == 0;  // (split, 0) -> (last, 0) has the form of a spine edge and must be counted as one
        if (last > 0) put_varint(cb, on_spine ? last : split);
        if (c.post_plane > 0) { put_varint(cb, split); put_varint(cb, uint64_t(c.post_plane)); put_varint(cb, last); put_varint(cb, 0); cb.push_back(0); }
        for (size_t i = 0; i < c.roles.size(); ++i) {
            if (int(i) == c.post_plane) cb.push_back(uint8_t(last << 4)); else cb.push_back(uint8_t((split << 4) | i));
            cb.push_back(c.roles[i]);
        }
        put_varint(reg, cb.size());
        reg.insert(reg.end(), cb.begin(), cb.end());
    }
    std::vector<uint8_t> head = {0x89, 'P', 'T', 'W', 'C', '\r', '\n', 0x1a, '\n', 0, 0};
    put_varint(head, et.size()); put_varint(head, prelude.size()); put_varint(head, reg.size());
    {
        std::vector<uint8_t> meta = head;
        meta.insert(meta.end(), et.begin(), et.end()); meta.insert(meta.end(), prelude.begin(), prelude.end()); meta.insert(meta.end(), reg.begin(), reg.end());
        put_u64(head, xxh64_host(meta.data(), meta.size()));
    }
    head.insert(head.end(), et.begin(), et.end()); head.insert(head.end(), prelude.begin(), prelude.end()); head.insert(head.end(), reg.begin(), reg.end());

    std::vector<uint8_t> staged = head;
    std::vector<uint64_t> triples = {0, 0, head.size()};
    std::vector<GatherItem> gathers;
    std::vector<uint8_t> index;
    put_varint(index, n_tensors);
    uint64_t pos = head.size();
    for (size_t i = 0; i < n_tensors; ++i) {
        const ptwm_b200_encode_tensor& t = tensors[i];
        const uint64_t rec_start = pos;
        auto flush = [&](std::vector<uint8_t>& bytes) {
            triples.push_back(pos); triples.push_back(staged.size()); triples.push_back(bytes.size());
            staged.insert(staged.end(), bytes.begin(), bytes.end());
            pos += bytes.size();
            bytes.clear();
        };
        std::vector<uint8_t> b;
        b.push_back(uint8_t(0x08 | (opt.emit_payload_hash ? 0x01 : 0)));
        put_varint(b, plan[i].chain_id); put_varint(b, t.dtype_code); b.push_back(2 /* Format.TORCH */); put_varint(b, t.nbytes);
        put_varint(b, t.ndim);
        for (int d = 0; d < t.ndim; ++d) put_varint(b, t.shape[d]);
        if (opt.emit_payload_hash) put_u64(b, plan[i].hash);
        put_varint(b, plan[i].planes.size());
        for (size_t p = 0; p < plan[i].planes.size(); ++p) {
            PlanePlan& pp = plan[i].planes[p];
            if (!chunked) {
                // one payload per plane with the state in front of it (tensor_record_compact.rs:203-493): every codec but Identity
                // is written with an inline state (empty unless Order1ScaleAC), the plane's row layout is recorded
                // (a plane coded against a shared state names it instead: state source Shared, the state's version and id)
                const bool use_shared = pp.shared >= 0, inline_state = pp.codec != C_IDENTITY && !use_shared, extra = pp.codec == C_O1SAC;
                b.push_back(uint8_t((inline_state ? 0x04 : 0) | (use_shared ? 0x08 : 0) | (opt.emit_plane_crc ? 0x01 : 0) | (pp.row_len ? 0x10 : 0) | (extra ? 0x20 : 0)));
                b.push_back(plane_role_byte(plan[i].chain.roles[p]));
                put_varint(b, table_index(2, uint16_t(pp.codec)));
                if (extra) { b.push_back(1); put_varint(b, use_shared ? uint64_t(pp.shared) : 0); }
                if (inline_state) put_varint(b, pp.state_len);
                put_varint(b, pp.payload_len - pp.state_len);
                if (pp.row_len) put_varint(b, pp.row_len);
                if (opt.emit_plane_crc) put_u32(b, pp.crc);
                if (pp.len == 0) {
                    if (pp.codec == C_O1SAC) {  // state of an empty plane: no rows, the marginal of no counts (16 everywhere); payload: the coder's flush
                        for (int z = 0; z < 32; ++z) b.push_back(0);
                        for (int z = 0; z < 256; ++z) { b.push_back(16); b.push_back(0); }
                        for (int z = 0; z < 6; ++z) b.push_back(0);
                    } else if (pp.codec != C_IDENTITY) b.push_back(0);
                    flush(b);
                    continue;
                }
                flush(b);
                gathers.push_back(GatherItem{pos, pp.first_chunk, chunk_mode[pp.first_chunk]});
                pos += pp.frame_size[0];
                continue;
            }
            b.push_back(uint8_t(0x02 | (opt.emit_plane_crc ? 0x01 : 0)));
            b.push_back(plane_role_byte(plan[i].chain.roles[p]));
            put_varint(b, table_index(2, uint16_t(pp.codec)));
            put_varint(b, pp.payload_len);
            if (opt.emit_plane_crc) put_u32(b, pp.crc);
            put_varint(b, pp.frame_size.size());
            uint64_t off = 0;
            for (size_t k = 0; k < pp.frame_size.size(); ++k) {
                put_varint(b, off);
                put_varint(b, pp.len ? chunks[pp.first_chunk + k].n : 0);
                off += pp.frame_size[k];
            }
            if (pp.len == 0) {  // the one empty frame is host data
                if (pp.codec == C_O1SAC) {
                    b.push_back(1); put_u32(b, 32 + 512);
                    for (int z = 0; z < 32; ++z) b.push_back(0);
                    for (int z = 0; z < 256; ++z) { b.push_back(16); b.push_back(0); }
                    for (int z = 0; z < 6; ++z) b.push_back(0);
                } else {
                    for (int z = 0; z < 5; ++z) b.push_back(0);
                    if (pp.codec != C_IDENTITY) b.push_back(0);
                }
                flush(b);
                continue;
            }
            flush(b);
            for (size_t k = 0; k < pp.frame_size.size(); ++k) {
                gathers.push_back(GatherItem{pos, pp.first_chunk + uint32_t(k), chunk_mode[pp.first_chunk + k]});
                pos += pp.frame_size[k];
            }
        }
        if (!b.empty()) flush(b);
        size_t nl = std::strlen(t.name);
        put_varint(index, nl); index.insert(index.end(), t.name, t.name + nl); put_varint(index, pos - rec_start);
    }
    {
        std::vector<uint8_t> tail = index;
        put_u64(tail, index.size());
        const uint8_t eofs[8] = {0x89, 'T', 'W', 'M', 'E', 'O', 'F', 0x1a};
        tail.insert(tail.end(), eofs, eofs + 8);
        triples.push_back(pos); triples.push_back(staged.size()); triples.push_back(tail.size());
        staged.insert(staged.end(), tail.begin(), tail.end());
        pos += tail.size();
    }

    prof("layout and records (host)");
    // ---- write the container ----------------------------------------------------
    enc.size = pos; enc.device = device;
    CUDA_TRY(cudaMalloc(&enc.d_out, pos));
    DeviceBuf d_staged, d_triples, d_gathers;
    CUDA_TRY(upload_vec(d_staged, staged, st));
    CUDA_TRY(upload_vec(d_triples, triples, st));
    CUDA_TRY(upload_vec(d_gathers, gathers, st));
    scatter_kernel<<<uint32_t(triples.size() / 3), 128, 0, st>>>(d_staged.as<uint8_t>(), d_triples.as<uint64_t>(), enc.d_out);
    CUDA_TRY(cudaGetLastError());
    if (!gathers.empty()) {
        gather_kernel<<<uint32_t(gathers.size()), 128, 0, st>>>(d_gathers.as<GatherItem>(), d_chunks.as<EncChunk>(), d_results.as<EncResult>(), d_planes.as<uint8_t>(),
                                                                d_tables.as<uint8_t>(), d_slots.as<uint8_t>(), enc.d_out);
        CUDA_TRY(cudaGetLastError());
    }
    CUDA_TRY(cudaStreamSynchronize(st));
    prof("scatter and gather");
    return 0;
}

}  // namespace

// One plane into one payload, device to device: the body of ptwm_plane_codec_v1_encode_cuda.
// Identity copies; Huffman and rANS run the container encoder's kernels on a single chunk that spans the
// plane and keep the reference's rules for falling back to the raw-tagged form (codecs/huffman.rs:37-88,
// codecs/rans.rs:38-95).  `needed` receives the payload size, also when `out_cap` is too small (-2).
int64_t ptwm::encode_plane_cuda(int codec, const uint8_t* state, size_t state_len, uint8_t state_version, uint64_t in_dev, size_t n, uint64_t out_dev, size_t out_cap,
                                uint64_t* needed, cudaStream_t st) {
    // the required size goes to *needed only when the output buffer cannot hold it
    auto need = [&](uint64_t v) { if (needed && v > out_cap) *needed = v; return v; };
    uint8_t* out = reinterpret_cast<uint8_t*>(uintptr_t(out_dev));
    const uint8_t* in = reinterpret_cast<const uint8_t*>(uintptr_t(in_dev));
    if (codec == C_IDENTITY) {
        if (need(n) > out_cap) return fail(PTWM_RC_BUFFER_TOO_SMALL, "output buffer too small");
        if (n) CUDA_TRY(cudaMemcpyAsync(out, in, n, cudaMemcpyDeviceToDevice, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        return int64_t(n);
    }
    if (n > 0xFFFFFFFFull && codec == C_O1SAC) return fail(PTWM_RC_UNSUPPORTED, "plane too long for the device encoder");
    DeviceBuf d_chunk, d_codec, d_hist, d_phist, d_tables, d_results, d_slots, d_gather, d_list, d_tlist;
    const uint64_t slot_cap = ((n / 4 + 1) * 12 + 7) / 8 + 64;  // a symbol takes at most 12 bits in any of the codecs
    EncChunk chunk{0, 0, 0, uint32_t(n), uint32_t(slot_cap), 0, 0};
    const uint8_t codec_byte = uint8_t(codec);
    if (codec == C_O1SAC) {
        // The flat ABI has no way to return a fitted state, so the rows come from the caller (the shared-state form of
        // order1_scale_ac.rs:620-633): [bitmap 32][marginal 512][rows 512 each], one row spanning the plane.
        if (!state_len) return fail(PTWM_RC_UNSUPPORTED, "order1_scale_ac through the plane-codec ABI needs the state to encode with (state_ptr, state_len)");
        try { check_o1sac(state, state_len, state_version, 5, 0, 0); } catch (const FormatError& e) { return fail(PTWM_RC_INVALID_INPUT, e.what()); }
        if (slot_cap > 0x3FFFFFFFull) return fail(PTWM_RC_UNSUPPORTED, "plane too long for the device encoder");
        std::vector<uint8_t> tab(ENC_O1SAC_TABLE_BYTES, 0);
        uint16_t* pmf = reinterpret_cast<uint16_t*>(tab.data() + O1E_PMF);
        uint16_t* cum = reinterpret_cast<uint16_t*>(tab.data() + O1E_CUM);
        auto load_row = [&](uint32_t row, const uint8_t* src) {
            uint32_t acc = 0;
            for (int i = 0; i < 256; ++i) { pmf[256 * row + i] = uint16_t(src[2 * i] | (src[2 * i + 1] << 8)); cum[256 * row + i] = uint16_t(acc); acc += pmf[256 * row + i]; }
        };
        load_row(0, state + 32);
        uint32_t k = 0;
        for (uint32_t ctx = 0; ctx < 256; ++ctx)
            if (state[ctx >> 3] & (1u << (ctx & 7))) { tab[O1E_PRESENT + ctx] = 1; load_row(1 + ctx, state + 32 + 512 + 512 * size_t(k)); ++k; }
        const uint32_t zero = 0;
        CUDA_TRY(d_chunk.alloc(sizeof(EncChunk)));
        CUDA_TRY(d_tables.alloc(tab.size()));
        CUDA_TRY(d_results.alloc(sizeof(EncResult)));
        CUDA_TRY(d_slots.alloc(4 * slot_cap));
        CUDA_TRY(d_list.alloc(4));
        CUDA_TRY(cudaMemcpyAsync(d_chunk.p, &chunk, sizeof(chunk), cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(d_tables.p, tab.data(), tab.size(), cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(d_list.p, &zero, 4, cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemsetAsync(d_results.p, 0, sizeof(EncResult), st));
        o1sac_encode_kernel<<<1, 64, 0, st>>>(d_chunk.as<EncChunk>(), d_list.as<uint32_t>(), 1, in, d_tables.as<uint8_t>(), d_slots.as<uint8_t>(), d_results.as<EncResult>());
        CUDA_TRY(cudaGetLastError());
        EncResult r;
        CUDA_TRY(cudaMemcpyAsync(&r, d_results.p, sizeof(r), cudaMemcpyDeviceToHost, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        if (need(r.stream_len[0]) > out_cap) return fail(PTWM_RC_BUFFER_TOO_SMALL, "output buffer too small");
        CUDA_TRY(cudaMemcpyAsync(out, d_slots.p, r.stream_len[0], cudaMemcpyDeviceToDevice, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        return int64_t(r.stream_len[0]);
    }
    if (codec != C_HUFFMAN && codec != C_RANS && codec != C_TANS) return fail(PTWM_RC_UNSUPPORTED, "device encode covers identity, huffman, rans, tans and order1_scale_ac");
    if (n == 0) {  // an empty plane is the raw tag alone
        if (need(1) > out_cap) return fail(PTWM_RC_BUFFER_TOO_SMALL, "output buffer too small");
        CUDA_TRY(cudaMemsetAsync(out, 0, 1, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        return 1;
    }
    uint32_t mode = 1;
    uint64_t size = 1 + uint64_t(n);
    CUDA_TRY(d_chunk.alloc(sizeof(EncChunk)));
    CUDA_TRY(d_results.alloc(sizeof(EncResult)));
    CUDA_TRY(d_tables.alloc(enc_table_bytes(codec)));
    if (n <= 0xFFFFFFFFull) {  // the length prefix is a u32; longer planes stay raw
        if (slot_cap > 0x3FFFFFFFull) return fail(PTWM_RC_UNSUPPORTED, "plane too long for the device encoder");
        CUDA_TRY(d_codec.alloc(1));
        CUDA_TRY(d_hist.alloc(256 * sizeof(uint32_t)));
        CUDA_TRY(d_phist.alloc(256 * sizeof(unsigned long long)));
        CUDA_TRY(d_slots.alloc(4 * slot_cap));
        CUDA_TRY(cudaMemcpyAsync(d_chunk.p, &chunk, sizeof(chunk), cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(d_codec.p, &codec_byte, 1, cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemsetAsync(d_phist.p, 0, 256 * sizeof(unsigned long long), st));
        hist_kernel<<<1, 128, 0, st>>>(d_chunk.as<EncChunk>(), in, d_hist.as<uint32_t>(), d_phist.as<unsigned long long>());
        table_kernel<<<1, 64, 0, st>>>(d_chunk.as<EncChunk>(), 1, d_codec.as<uint8_t>(), d_hist.as<uint32_t>(), d_tables.as<uint8_t>(), d_results.as<EncResult>());
        encode_kernel<<<1, 128, 0, st>>>(d_chunk.as<EncChunk>(), 1, d_codec.as<uint8_t>(), in, d_tables.as<uint8_t>(), d_slots.as<uint8_t>(), d_results.as<EncResult>());
        if (codec == C_TANS) {
            CUDA_TRY(d_tlist.alloc(4));
            CUDA_TRY(cudaMemsetAsync(d_tlist.p, 0, 4, st));  // the list of chunks to code: chunk 0
            CUDA_TRY(cudaFuncSetAttribute(tans_encode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TENC_SMEM));
            tans_encode_kernel<<<1, 32, TENC_SMEM, st>>>(d_chunk.as<EncChunk>(), d_tlist.as<uint32_t>(), 1, in, d_tables.as<uint8_t>(), d_slots.as<uint8_t>(), d_results.as<EncResult>());
        }
        CUDA_TRY(cudaGetLastError());
        EncResult r;
        CUDA_TRY(cudaMemcpyAsync(&r, d_results.p, sizeof(r), cudaMemcpyDeviceToHost, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        uint64_t blob;
        if (codec == C_TANS) blob = 3 + 3 * uint64_t(r.hdr_n) + 8 + r.stream_len[0];
        else {
            const uint64_t hdr = codec == C_RANS ? 1 + 2 * (uint64_t(r.hdr_n) + 1) : (r.hdr_n <= 127 ? 1 : 2) + (uint64_t(r.hdr_n) + 1) / 2;
            blob = hdr + 16 + uint64_t(r.stream_len[0]) + r.stream_len[1] + r.stream_len[2] + r.stream_len[3];
        }
        const bool coded = r.coded && blob < n && (codec == C_HUFFMAN || n <= (1ull << 30) || n <= blob * 64);
        if (coded) { mode = codec == C_RANS ? 2 : codec == C_HUFFMAN ? 3 : 4; size = 1 + 4 + blob; }
    } else {
        CUDA_TRY(d_slots.alloc(16));
    }
    if (need(size) > out_cap) return fail(PTWM_RC_BUFFER_TOO_SMALL, "output buffer too small");
    if (mode == 1 && n > 0xFFFFFFFFull) {  // raw: tag byte, then the plane
        CUDA_TRY(cudaMemsetAsync(out, 0, 1, st));
        CUDA_TRY(cudaMemcpyAsync(out + 1, in, n, cudaMemcpyDeviceToDevice, st));
    } else {
        const GatherItem g{0, 0, mode | GATHER_BARE};
        CUDA_TRY(d_gather.alloc(sizeof(g)));
        CUDA_TRY(cudaMemcpyAsync(d_gather.p, &g, sizeof(g), cudaMemcpyHostToDevice, st));
        gather_kernel<<<1, 128, 0, st>>>(d_gather.as<GatherItem>(), d_chunk.as<EncChunk>(), d_results.as<EncResult>(), in, d_tables.as<uint8_t>(), d_slots.as<uint8_t>(), out);
        CUDA_TRY(cudaGetLastError());
    }
    CUDA_TRY(cudaStreamSynchronize(st));
    return int64_t(size);
}

extern "C" {

int64_t ptwm_b200_encode_model(const ptwm_b200_encode_tensor* tensors, size_t n, const ptwm_b200_encode_options* options, uint32_t device_ordinal, uint64_t stream,
                               ptwm_b200_encoded** out) {
    if ((!tensors && n) || !out) return fail(PTWM_RC_INVALID_INPUT, "null argument");
    ptwm_b200_encode_options opt{0, 0, -1, 0, 0, 0, {0}};
    if (options) opt = *options;
    DeviceGuard guard{int(device_ordinal)};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(guard.err));
    DeviceState* ds;
    int64_t rc = device_state(int(device_ordinal), &ds);
    if (rc < 0) return rc;
    cudaStream_t st = stream ? reinterpret_cast<cudaStream_t>(uintptr_t(stream)) : ds->stream;
    try {
        std::unique_ptr<ptwm_b200_encoded> e(new ptwm_b200_encoded);
        rc = encode_impl(tensors, n, opt, int(device_ordinal), st, ds->d_tabs, *e);
        if (rc < 0) return rc;
        *out = e.release();
        return 0;
    } catch (const std::exception& ex) { return fail(PTWM_RC_INTERNAL, ex.what()); }
}
int64_t ptwm_b200_fit_shared_states_host(const uint8_t* const* planes, const uint64_t* lens, const uint32_t* row_lens, size_t n, uint8_t* out, size_t cap,
                                         uint32_t state_lens[8]) {
    if ((n && (!planes || !lens || !row_lens)) || !state_lens || (cap && !out)) return fail(PTWM_RC_INVALID_INPUT, "null argument");
    try {
        // counts per plane (order1_scale_ac.rs:974-995): the first symbol of a row to the marginal, every other one after its predecessor
        std::vector<std::vector<uint32_t>> joint(n, std::vector<uint32_t>(65536, 0)), marg(n, std::vector<uint32_t>(256, 0));
        std::vector<FitCounts> fc;
        for (size_t k = 0; k < n; ++k) {
            if (!row_lens[k]) return fail(PTWM_RC_INVALID_INPUT, "row length 0");
            const uint8_t* p = planes[k];
            for (uint64_t i = 0; i < lens[k]; ++i) {
                if (i % row_lens[k] == 0) marg[k][p[i]]++;
                else joint[k][size_t(p[i - 1]) * 256 + p[i]]++;
            }
            fc.push_back(FitCounts{joint[k].data(), marg[k].data()});
        }
        FitResult r = fit_shared_order1(fc, [](const std::vector<FitState>& own, const std::vector<uint32_t>& pairs) {
            std::vector<double> d(pairs.size() / 2);
            for (size_t k = 0; k < d.size(); ++k) {  // what fit_pair_distance_kernel computes, in the same order
                const FitState& P = own[pairs[2 * k]];
                const FitState& Q = own[pairs[2 * k + 1]];
                double total = 0;
                for (int prev = 0; prev < 256; ++prev) {
                    const uint16_t* p = P.row_or_marginal(prev);
                    const uint16_t* q = Q.row_or_marginal(prev);
                    double kl_pq = 0, kl_qp = 0;
                    for (int i = 0; i < 256; ++i) {
                        const double pp = double(p[i]) / 4096.0, qq = double(q[i]) / 4096.0;
                        if (pp > 0.0 && qq > 0.0) { kl_pq += pp * std::log(pp / qq); kl_qp += qq * std::log(qq / pp); }
                    }
                    const double ln2 = 0.693147180559945309417232121458;
                    total += 0.5 * (double(P.marginal[prev]) / 4096.0 + double(Q.marginal[prev]) / 4096.0) * (kl_pq / ln2 + kl_qp / ln2);
                }
                d[k] = total;
            }
            return d;
        });
        size_t pos = 0;
        for (size_t k = 0; k < r.states.size(); ++k) {
            const std::vector<uint8_t> b = r.states[k].serialize();
            if (pos + b.size() > cap) return fail(PTWM_RC_BUFFER_TOO_SMALL, "shared states do not fit the buffer");
            std::memcpy(out + pos, b.data(), b.size());
            state_lens[k] = uint32_t(b.size());
            pos += b.size();
        }
        return int64_t(r.states.size());
    } catch (const std::exception& ex) { return fail(PTWM_RC_INTERNAL, ex.what()); }
}
uint64_t ptwm_b200_encoded_size(const ptwm_b200_encoded* e) { return e ? e->size : 0; }
uint64_t ptwm_b200_encoded_device_ptr(const ptwm_b200_encoded* e) { return e ? uint64_t(reinterpret_cast<uintptr_t>(e->d_out)) : 0; }
int64_t ptwm_b200_encoded_copy(const ptwm_b200_encoded* e, uint8_t* host_dst, size_t cap) {
    if (!e || !host_dst) return fail(PTWM_RC_INVALID_INPUT, "null argument");
    if (cap < e->size) return fail(PTWM_RC_BUFFER_TOO_SMALL, "host buffer smaller than the container");
    DeviceGuard guard{e->device};
    CUDA_TRY(cudaMemcpy(host_dst, e->d_out, e->size, cudaMemcpyDeviceToHost));
    return int64_t(e->size);
}
int64_t ptwm_b200_encoded_copy_to_device(const ptwm_b200_encoded* e, uint64_t dst_dev_ptr, uint64_t cap, uint64_t stream) {
    if (!e || !dst_dev_ptr) return fail(PTWM_RC_INVALID_INPUT, "null argument");
    if (cap < e->size) return fail(PTWM_RC_BUFFER_TOO_SMALL, "device buffer smaller than the container");
    DeviceGuard guard{e->device};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(uintptr_t(stream));
    CUDA_TRY(cudaMemcpyAsync(reinterpret_cast<void*>(uintptr_t(dst_dev_ptr)), e->d_out, e->size, cudaMemcpyDeviceToDevice, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    return int64_t(e->size);
}
int32_t ptwm_b200_encoded_plane_codec(const ptwm_b200_encoded* e, size_t tensor, size_t plane) {
    if (!e || tensor >= e->plane_codecs.size() || plane >= e->plane_codecs[tensor].size()) return -1;
    return e->plane_codecs[tensor][plane];
}
void ptwm_b200_encoded_free(ptwm_b200_encoded* e) { delete e; }

}  // extern "C"
