// Host side of libptwm_b200.so: the planner that flattens a parsed container
// into kernel work lists, the runner that launches them, and the C ABI
// declared in include/ptwm_b200.h.
#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "format.hpp"
#include "host_common.hpp"

using namespace ptwm;

namespace ptwm {

std::string& last_error_ref() { thread_local std::string e; return e; }

namespace {
std::mutex g_dev_mu;
std::map<int, DeviceState> g_dev;

CrcTables host_crc_tables() {
    CrcTables t;
    for (uint32_t i = 0; i < 256; ++i) {
        uint32_t c = i;
        for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
        t.byte_table[i] = c;
    }
    uint32_t p = 1u << 30;  // x^1
    for (int k = 0; k < 64; ++k) { t.x2n[k] = p; p = gf2_mulmod(p, p); }
    return t;
}
}  // namespace

const CrcTables& crc_tables() { static CrcTables t = host_crc_tables(); return t; }

int64_t device_state(int dev, DeviceState** out) {
    std::lock_guard<std::mutex> g(g_dev_mu);
    DeviceState& s = g_dev[dev];
    if (!s.stream) CUDA_TRY(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
    if (!s.d_tabs) {
        CUDA_TRY(cudaMalloc(&s.d_tabs, sizeof(CrcTables)));
        CUDA_TRY(cudaMemcpy(s.d_tabs, &crc_tables(), sizeof(CrcTables), cudaMemcpyHostToDevice));
    }
    if (!s.attrs) {
        CUDA_TRY(cudaFuncSetAttribute(rans_decode_kernel_t<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rans_smem_bytes(rans_l_entries(255)))));
        CUDA_TRY(cudaFuncSetAttribute(rans_decode_kernel_t<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rans_smem_bytes(RANS_NARROW_SYMBOLS + 2, true))));
        CUDA_TRY(cudaFuncSetAttribute(rans_decode_kernel_t<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        CUDA_TRY(cudaFuncSetAttribute(huffman_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, HUF_SMEM));
        CUDA_TRY(cudaFuncSetAttribute(tans_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TANS_SMEM));
        CUDA_TRY(o1sac_allow_shared_tables());
        // the decoders are limited by how many chunk tables fit in an SM: ask for the largest shared-memory carve-out
        CUDA_TRY(cudaFuncSetAttribute(rans_decode_kernel_t<false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        CUDA_TRY(cudaFuncSetAttribute(huffman_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        CUDA_TRY(cudaFuncSetAttribute(tans_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        s.attrs = true;
    }
    *out = &s;
    return 0;
}

}  // namespace ptwm

struct ptwm_b200_container {
    ParsedFile file;
    uint64_t blob_len = 0;
    std::vector<uint64_t> compressed, first_byte, end_byte;
    std::vector<uint8_t> has_crc;
};

namespace {

struct CrcExpect { uint32_t acc; uint32_t crc; uint64_t plane_len; uint32_t tensor; };
struct HashExpect { uint64_t hash; uint32_t tensor; };

struct DevicePlan {
    DecodeItem* items = nullptr;       // all decode lists back to back
    MergeItem* merges = nullptr;
    uint32_t* tiles = nullptr;
    PostItem* posts = nullptr;
    uint32_t* post_tiles = nullptr;
    VerifyTensor* verify = nullptr;
    HashItem* hashes = nullptr;
    uint32_t* status = nullptr;        // [0] = summary, [1 + id] per item
    uint32_t* acc = nullptr;
    uint64_t* hash_out = nullptr;
    cudaEvent_t ev[24] = {nullptr};   // begin/end per launch slot, created on first timed run
    bool timed[12] = {false};
    uint8_t* arena = nullptr;          // everything above lives in this one block
    bool external = false;             // the block belongs to the caller (ptwm_b200_plan_prepare_in)
    void release() {
        for (auto& e : ev) if (e) cudaEventDestroy(e);
        if (!external) cudaFree(arena);
        *this = DevicePlan{};
    }
};

}  // namespace

struct ptwm_b200_plan {
    const ptwm_b200_container* c = nullptr;
    std::vector<uint32_t> tensors;
    std::vector<uint64_t> out_off;
    uint64_t out_bytes = 0, scratch_bytes = 0, blob_lo = 0, blob_hi = 0, bytes_read = 0, bytes_written = 0;
    // decode lists: [phase][codec class] with class 0 rANS, 1 Huffman, 2 tANS, 3 O1SAC
    std::vector<DecodeItem> dec[2][4];
    // merge lists: [0] copies into scratch, [1] final recombination
    std::vector<MergeItem> merges[2];
    std::vector<uint32_t> tiles[2];
    // planes in scratch with an IntDelta or MantissaZeroStrip to undo between the two phases, and the first tile of each
    std::vector<PostItem> posts;
    std::vector<uint32_t> post_tiles;
    std::vector<VerifyTensor> verify;
    uint64_t n_runs = 0;
    std::vector<CrcExpect> crc_expect;
    uint32_t n_acc = 0;
    std::vector<HashItem> hashes;
    std::vector<HashExpect> hash_expect;
    std::vector<uint32_t> item_tensor;  // item id -> tensor index (for error messages)
    uint32_t launches = 0;
    // per launch slot: 0-3 phase-0 decoders (rANS, Huffman, tANS, O1SAC), 4 scratch copies, 5-8 phase-1 decoders, 9 final merge, 10 CRC, 11 XXH64
    // rANS chunks per phase: the first `rans_narrow` items hold few distinct symbols and go to the kernel with a symbol
    // list per lane (`rans_rows` rows); the rest go to the general kernel, whose shared list is sized by the most distinct symbols among them.
    uint32_t rans_wide_distinct[2] = {0, 0}, rans_narrow[2] = {0, 0}, rans_rows[2] = {0, 0};
    uint32_t o1_tables[2] = {0, 0};  // most cumulative tables among the Order1ScaleAC chunks of a phase
    uint64_t slot_bytes[12] = {0};
    uint32_t slot_items[12] = {0};
    std::mutex mu;
    std::map<int, DevicePlan> dev;
    ~ptwm_b200_plan() {
        for (auto& kv : dev) { DeviceGuard g(kv.first); kv.second.release(); }
    }
};

namespace {

int codec_class(uint16_t codec) { return codec == C_RANS ? 0 : codec == C_HUFFMAN ? 1 : codec == C_TANS ? 2 : 3; }

// Turn one tensor into work items.  See DecodeItem / MergeItem in plan.h.
void plan_tensor(ptwm_b200_plan& pl, uint32_t ti, const TensorDesc& t, uint64_t out_off) {
    const int np = int(t.planes.size());
    const int eb = kind_elem_bytes(t.kind);
    auto new_id = [&]() { pl.item_tensor.push_back(ti); return uint32_t(pl.item_tensor.size() - 1); };
    auto span = [&](uint64_t off, uint64_t len) { if (!len) return; pl.blob_lo = std::min(pl.blob_lo, off); pl.blob_hi = std::max(pl.blob_hi, off + len); pl.bytes_read += len; };
    pl.bytes_written += t.orig_size;
    if (t.stored) {
        span(t.stored_off, t.orig_size);
        if (t.orig_size) pl.merges[1].push_back(MergeItem{{make_ref(SP_BLOB, t.stored_off), REF_NONE, REF_NONE, REF_NONE}, make_ref(SP_OUT, out_off), uint32_t(t.orig_size), K_PASS});
        return;
    }
    // scratch plane buffers are handed out lazily
    std::vector<uint64_t> plane_scratch(size_t(np), UINT64_MAX);
    auto scratch_of = [&](int p) {
        if (plane_scratch[size_t(p)] == UINT64_MAX) { plane_scratch[size_t(p)] = pl.scratch_bytes; pl.scratch_bytes += align_up(t.planes[size_t(p)].decoded_len, 256); }
        return plane_scratch[size_t(p)];
    };
    auto decode_item = [&](const PlaneDesc& p, const ChunkDesc& ch) {
        DecodeItem it{};
        it.src = make_ref(SP_BLOB, ch.data_off); it.src_len = uint32_t(ch.data_len); it.n = ch.decoded; it.id = new_id();
        it.partner[0] = it.partner[1] = it.partner[2] = REF_NONE; it.state = REF_NONE; it.work = REF_NONE;
        span(ch.data_off, ch.data_len);
        it.row_len = uint32_t(ch.max_sym) | uint32_t(ch.distinct) << 16;  // rANS: alphabet bound and distinct symbols, for the planner only (the kernels read row_len for Order1ScaleAC)
        if (p.codec == C_O1SAC) {
            it.state = make_ref(SP_BLOB, ch.state_off); it.state_len = uint32_t(ch.state_len); it.state_version = ch.state_version;
            it.row_len = uint32_t(p.row_len);
            span(ch.state_off, ch.state_len);
            uint64_t tables = (ch.state_len - 32) / 512;
            pl.scratch_bytes = align_up(pl.scratch_bytes, 16);
            it.work = make_ref(SP_SCRATCH, pl.scratch_bytes);
            pl.scratch_bytes += align_up(tables * 514, 16);
        }
        return it;
    };
    bool aligned = true;
    for (int p = 1; p < np && aligned; ++p) {
        if (t.planes[size_t(p)].chunks.size() != t.planes[0].chunks.size()) aligned = false;
        else for (size_t k = 0; k < t.planes[0].chunks.size(); ++k) if (t.planes[size_t(p)].chunks[k].decoded != t.planes[0].chunks[k].decoded) { aligned = false; break; }
    }
    bool has_post = false;
    for (const PlaneDesc& pd : t.planes) has_post |= pd.post != POST_NONE;
    if (aligned && !has_post) {
        for (size_t k = 0; k < t.planes[0].chunks.size(); ++k) {
            const uint32_t n = t.planes[0].chunks[k].decoded;
            if (!n) continue;
            const uint64_t plane_off = t.planes[0].chunks[k].plane_off;
            const Ref out_ref = make_ref(SP_OUT, out_off + plane_off * uint64_t(eb));
            int fused_plane = -1;
            for (int p = 0; p < np; ++p) {
                const ChunkDesc& ch = t.planes[size_t(p)].chunks[k];
                uint16_t codec = t.planes[size_t(p)].codec;
                if (!ch.raw && (codec == C_RANS || codec == C_HUFFMAN || codec == C_TANS)) fused_plane = p;
            }
            if (np == 1) {
                const ChunkDesc& ch = t.planes[0].chunks[k];
                if (ch.raw) { span(ch.data_off, ch.data_len); pl.merges[1].push_back(MergeItem{{make_ref(SP_BLOB, ch.data_off), REF_NONE, REF_NONE, REF_NONE}, out_ref, n, K_PASS}); }
                else { DecodeItem it = decode_item(t.planes[0], ch); it.dst = out_ref; pl.dec[1][codec_class(t.planes[0].codec)].push_back(it); }
                continue;
            }
            Ref srcs[4] = {REF_NONE, REF_NONE, REF_NONE, REF_NONE};
            for (int p = 0; p < np; ++p) {
                const PlaneDesc& pd = t.planes[size_t(p)];
                const ChunkDesc& ch = pd.chunks[k];
                if (ch.raw) { srcs[p] = make_ref(SP_BLOB, ch.data_off); span(ch.data_off, ch.data_len); }
                else if (p != fused_plane) {
                    DecodeItem it = decode_item(pd, ch);
                    it.dst = make_ref(SP_SCRATCH, scratch_of(p) + ch.plane_off);
                    srcs[p] = it.dst;
                    pl.dec[0][codec_class(pd.codec)].push_back(it);
                }
            }
            if (fused_plane >= 0) {
                const PlaneDesc& pd = t.planes[size_t(fused_plane)];
                DecodeItem it = decode_item(pd, pd.chunks[k]);
                it.dst = out_ref; it.fused = 1; it.kind = t.kind; it.slot = uint8_t(fused_plane);
                int j = 0;
                for (int p = 0; p < np; ++p) if (p != fused_plane) it.partner[j++] = srcs[p];
                pl.dec[1][codec_class(pd.codec)].push_back(it);
            } else {
                pl.merges[1].push_back(MergeItem{{srcs[0], srcs[1], srcs[2], srcs[3]}, out_ref, n, uint32_t(t.kind)});
            }
        }
    } else {
        // planes chunked differently, or a plane with an op to undo first: materialise every plane in scratch, then recombine once
        Ref srcs[4] = {REF_NONE, REF_NONE, REF_NONE, REF_NONE};
        for (int p = 0; p < np; ++p) {
            const PlaneDesc& pd = t.planes[size_t(p)];
            uint64_t base = scratch_of(p);
            srcs[p] = make_ref(SP_SCRATCH, base);
            for (const ChunkDesc& ch : pd.chunks) {
                if (!ch.decoded) continue;
                Ref dst = make_ref(SP_SCRATCH, base + ch.plane_off);
                if (ch.raw) { span(ch.data_off, ch.data_len); pl.merges[0].push_back(MergeItem{{make_ref(SP_BLOB, ch.data_off), REF_NONE, REF_NONE, REF_NONE}, dst, ch.decoded, K_PASS}); }
                else { DecodeItem it = decode_item(pd, ch); it.dst = dst; pl.dec[0][codec_class(pd.codec)].push_back(it); }
            }
            if (pd.post != POST_NONE && pd.decoded_len) {
                PostItem po{srcs[p], pd.decoded_len, pd.post, pd.post_k, REF_NONE};
                if (pd.post == POST_INTDELTA) {
                    pl.scratch_bytes = align_up(pl.scratch_bytes, 16);
                    po.sums = make_ref(SP_SCRATCH, pl.scratch_bytes);
                    pl.scratch_bytes += align_up(4 * ((pd.decoded_len + POST_TILE - 1) / POST_TILE), 16);
                }
                pl.posts.push_back(po);
            }
        }
        uint64_t n = t.planes[0].decoded_len;
        for (uint64_t done = 0; done < n; done += 0x80000000ull) {
            uint32_t part = uint32_t(std::min<uint64_t>(n - done, 0x80000000ull));
            MergeItem m{{REF_NONE, REF_NONE, REF_NONE, REF_NONE}, make_ref(SP_OUT, out_off + done * uint64_t(eb)), part, uint32_t(t.kind)};
            for (int p = 0; p < np; ++p) m.src[p] = srcs[p] + done;
            pl.merges[1].push_back(m);
        }
    }
}

void finish_lists(ptwm_b200_plan& pl) {
    for (int ph = 0; ph < 2; ++ph) {
        for (int cc = 0; cc < 4; ++cc) {
            auto& v = pl.dec[ph][cc];
            auto narrow = [cc](const DecodeItem& a) { return cc == 0 && (a.row_len >> 16) <= RANS_NARROW_SYMBOLS; };
            std::stable_sort(v.begin(), v.end(), [&](const DecodeItem& a, const DecodeItem& b) {
                bool na = narrow(a), nb = narrow(b);
                return na != nb ? na : a.n > b.n;
            });
            if (!v.empty()) pl.launches++;
            int slot = ph * 5 + cc;
            pl.slot_items[slot] = uint32_t(v.size());
            if (cc == 0) {
                uint32_t most = 0;
                for (auto& it : v) {
                    if (narrow(it)) { pl.rans_narrow[ph]++; most = std::max(most, it.row_len >> 16); }
                    else pl.rans_wide_distinct[ph] = std::max(pl.rans_wide_distinct[ph], it.row_len >> 16);  // most distinct symbols among the rest
                }
                pl.rans_rows[ph] = most + 2;
                if (pl.rans_narrow[ph] && pl.rans_narrow[ph] < v.size()) pl.launches++;
            }
            if (cc == 3) for (auto& it : v) pl.o1_tables[ph] = std::max(pl.o1_tables[ph], o1sac_tables(it.state_len));
            for (auto& it : v) {
                uint64_t np = it.fused ? uint64_t(kind_planes(it.kind)) : 1, eb = it.fused ? uint64_t(kind_elem_bytes(it.kind)) : 1;
                pl.slot_bytes[slot] += uint64_t(it.src_len) + it.state_len + uint64_t(it.n) * (np - 1) + uint64_t(it.n) * eb;
            }
        }
        auto& m = pl.merges[ph];
        pl.slot_items[ph * 5 + 4] = uint32_t(m.size());
        for (auto& it : m) pl.slot_bytes[ph * 5 + 4] += uint64_t(it.n) * uint64_t(kind_planes(int(it.kind))) + uint64_t(it.n) * uint64_t(kind_elem_bytes(int(it.kind)));
        pl.tiles[ph].clear();
        uint32_t tile = 0;
        for (auto& it : m) { pl.tiles[ph].push_back(tile); tile += (it.n + MERGE_TILE - 1) / MERGE_TILE; }
        pl.tiles[ph].push_back(tile);
        if (!m.empty()) pl.launches++;
    }
    pl.post_tiles.clear();
    uint32_t tile = 0;
    bool delta = false;
    for (auto& po : pl.posts) { pl.post_tiles.push_back(tile); tile += uint32_t((po.n + POST_TILE - 1) / POST_TILE); delta |= po.op == POST_INTDELTA; }
    pl.post_tiles.push_back(tile);
    if (!pl.posts.empty()) pl.launches += delta ? 3 : 1;
}

// A plan's work lists reach the device through a kernel that reads them out of pinned host memory, not through a
// host-to-device copy: a caller that streams a container to the GPU has tens of large copies queued on the copy
// engine, and a small copy issued now would only run after all of them (the plan of the first piece would be ready
// when the last byte of the container has arrived).  The kernel runs on the library's stream beside those copies.
std::mutex g_stage_mu;  // one staging buffer per device, used under this lock
template <class T>
int64_t upload(T* dst, const std::vector<T>& v, DeviceState& ds) {
    if (v.empty()) return 0;
    const size_t bytes = v.size() * sizeof(T), padded = (bytes + 15) & ~size_t(15);
    std::lock_guard<std::mutex> g(g_stage_mu);
    if (ds.stage_cap < padded) {  // grows only on the first large plan of a process: pinning synchronises with the device
        if (ds.stage) CUDA_TRY(cudaFreeHost(ds.stage));
        ds.stage = nullptr; ds.stage_cap = 0;
        const size_t cap = std::max<size_t>(padded + padded / 2, size_t(32) << 20);
        CUDA_TRY(cudaMallocHost(&ds.stage, cap));
        ds.stage_cap = cap;
    }
    std::memcpy(ds.stage, v.data(), bytes);
    const size_t n16 = padded / 16;
    stage_in_kernel<<<unsigned(std::min<size_t>((n16 + 255) / 256, 1184)), 256, 0, ds.stream>>>(static_cast<const uint4*>(ds.stage), reinterpret_cast<uint4*>(dst), n16);
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaStreamSynchronize(ds.stream));  // the staging buffer is free again, and the list is in place before any launch that uses it
    return 0;
}

// Device bytes a plan needs for its work lists and status arrays, each part on a 256-byte boundary.
struct PlanLayout { uint64_t off[10]; uint64_t total; };
PlanLayout plan_layout(const ptwm_b200_plan& pl) {
    size_t n_items = 0, n_merges = 0, n_tiles = 0;
    for (int ph = 0; ph < 2; ++ph) { for (int cc = 0; cc < 4; ++cc) n_items += pl.dec[ph][cc].size(); n_merges += pl.merges[ph].size(); n_tiles += pl.tiles[ph].size(); }
    const uint64_t sizes[10] = {n_items * sizeof(DecodeItem), n_merges * sizeof(MergeItem), n_tiles * 4, pl.posts.size() * sizeof(PostItem), pl.post_tiles.size() * 4,
                                pl.verify.size() * sizeof(VerifyTensor), pl.hashes.size() * sizeof(HashItem), (pl.item_tensor.size() + 1) * 4, (uint64_t(pl.n_acc) + 1) * 4,
                                (pl.hashes.size() + 1) * 8};
    PlanLayout L{};
    uint64_t at = 0;
    for (int k = 0; k < 10; ++k) { L.off[k] = at; at += align_up(sizes[k], 256); }
    L.total = at ? at : 256;
    return L;
}

// Caller holds the plan mutex and a DeviceGuard.  `mem` / `cap`: device memory of the caller to build the plan in, or null.
int64_t device_plan(ptwm_b200_plan& pl, int dev, DeviceState& ds, DevicePlan** out, uint8_t* mem = nullptr, uint64_t cap = 0) {
    auto found = pl.dev.find(dev);
    if (found != pl.dev.end()) { *out = &found->second; return 0; }
    DevicePlan d;
    const PlanLayout L = plan_layout(pl);
    if (mem) {
        if (cap < L.total || (reinterpret_cast<uintptr_t>(mem) & 255)) return fail(PTWM_RC_BUFFER_TOO_SMALL, "plan memory smaller than ptwm_b200_plan_device_bytes or not 256-byte aligned");
        d.arena = mem; d.external = true;
    } else {
        CUDA_TRY(cudaMalloc(&d.arena, L.total));
    }
    d.items = reinterpret_cast<DecodeItem*>(d.arena + L.off[0]); d.merges = reinterpret_cast<MergeItem*>(d.arena + L.off[1]);
    d.tiles = reinterpret_cast<uint32_t*>(d.arena + L.off[2]); d.posts = reinterpret_cast<PostItem*>(d.arena + L.off[3]);
    d.post_tiles = reinterpret_cast<uint32_t*>(d.arena + L.off[4]); d.verify = reinterpret_cast<VerifyTensor*>(d.arena + L.off[5]);
    d.hashes = reinterpret_cast<HashItem*>(d.arena + L.off[6]); d.status = reinterpret_cast<uint32_t*>(d.arena + L.off[7]);
    d.acc = reinterpret_cast<uint32_t*>(d.arena + L.off[8]); d.hash_out = reinterpret_cast<uint64_t*>(d.arena + L.off[9]);
    std::vector<DecodeItem> all;
    for (int ph = 0; ph < 2; ++ph) for (int cc = 0; cc < 4; ++cc) all.insert(all.end(), pl.dec[ph][cc].begin(), pl.dec[ph][cc].end());
    std::vector<MergeItem> allm;
    std::vector<uint32_t> allt;
    for (int ph = 0; ph < 2; ++ph) { allm.insert(allm.end(), pl.merges[ph].begin(), pl.merges[ph].end()); allt.insert(allt.end(), pl.tiles[ph].begin(), pl.tiles[ph].end()); }
    int64_t rc;
    if ((rc = upload(d.items, all, ds)) < 0 || (rc = upload(d.merges, allm, ds)) < 0 || (rc = upload(d.tiles, allt, ds)) < 0 || (rc = upload(d.posts, pl.posts, ds)) < 0 ||
        (rc = upload(d.post_tiles, pl.post_tiles, ds)) < 0 || (rc = upload(d.verify, pl.verify, ds)) < 0 ||
        (rc = upload(d.hashes, pl.hashes, ds)) < 0) { d.release(); return rc; }
    pl.dev[dev] = d;
    *out = &pl.dev[dev];
    return 0;
}

int64_t enqueue(ptwm_b200_plan& pl, DevicePlan& d, const Bases& bases, uint32_t flags, CrcTables* d_tabs, cudaStream_t st) {
    CUDA_TRY(cudaMemsetAsync(d.status, 0, (pl.item_tensor.size() + 1) * sizeof(uint32_t), st));
    uint32_t* status = d.status + 1;
    size_t item_base = 0, merge_base = 0, tile_base = 0;
    const bool timing = flags & PTWM_B200_TIME_KERNELS;
    for (bool& t : d.timed) t = false;
    if (timing) for (auto& e : d.ev) if (!e) CUDA_TRY(cudaEventCreate(&e));
    auto mark = [&](int slot, int end) -> cudaError_t { if (!timing) return cudaSuccess; d.timed[slot] = true; return cudaEventRecord(d.ev[2 * slot + end], st); };
    auto launch_decodes = [&](int ph) -> int64_t {
        for (int cc = 0; cc < 4; ++cc) {
            uint32_t n = uint32_t(pl.dec[ph][cc].size());
            const DecodeItem* it = d.items + item_base;
            item_base += n;
            if (!n) continue;
            CUDA_TRY(mark(ph * 5 + cc, 0));
            switch (cc) {
                case 0: {
                    const uint32_t nn = pl.rans_narrow[ph], nw = n - nn;
                    if (nn) {
                        const uint32_t rows = pl.rans_rows[ph];
                        rans_decode_kernel_t<true><<<(nn + RANS_WARP_CHUNKS - 1) / RANS_WARP_CHUNKS, 32, rans_smem_bytes(rows, true), st>>>(it, nn, bases, status, rows);
                        CUDA_TRY(cudaGetLastError());
                    }
                    if (nw) {
                        const uint32_t le = (pl.rans_wide_distinct[ph] + 2 + 3) & ~3u;
                        rans_decode_kernel_t<false><<<(nw + RANS_WARP_CHUNKS - 1) / RANS_WARP_CHUNKS, 32, rans_smem_bytes(le), st>>>(it + nn, nw, bases, status, le);
                    }
                    break;
                }
                case 1: huffman_decode_kernel<<<(n + HUF_WARP_CHUNKS - 1) / HUF_WARP_CHUNKS, 32, HUF_SMEM, st>>>(it, n, bases, status); break;
                case 2: tans_decode_kernel<<<(n + TANS_CTA_CHUNKS - 1) / TANS_CTA_CHUNKS, TANS_THREADS, TANS_SMEM, st>>>(it, n, bases, status); break;
                default: o1sac_launch(it, n, bases, status, pl.o1_tables[ph], st); break;
            }
            CUDA_TRY(cudaGetLastError());
            CUDA_TRY(mark(ph * 5 + cc, 1));
        }
        return 0;
    };
    auto launch_merges = [&](int ph) -> int64_t {
        uint32_t n = uint32_t(pl.merges[ph].size());
        const MergeItem* m = d.merges + merge_base;
        const uint32_t* tf = d.tiles + tile_base;
        merge_base += n; tile_base += pl.tiles[ph].size();
        if (!n) return 0;
        uint32_t tiles = pl.tiles[ph].back();
        if (tiles) {
            CUDA_TRY(mark(ph * 5 + 4, 0));
            merge_kernel<<<tiles, 256, 0, st>>>(m, tf, n, bases);
            CUDA_TRY(cudaGetLastError());
            CUDA_TRY(mark(ph * 5 + 4, 1));
        }
        return 0;
    };
    // planes in scratch are complete after the first phase: undo IntDelta / MantissaZeroStrip in place before anything reads them
    auto launch_posts = [&]() -> int64_t {
        if (pl.posts.empty()) return 0;
        const uint32_t n = uint32_t(pl.posts.size()), tiles = pl.post_tiles.back();
        bool delta = false;
        for (auto& po : pl.posts) delta |= po.op == POST_INTDELTA;
        if (delta) {
            post_tile_sums_kernel<<<tiles, 256, 0, st>>>(d.posts, d.post_tiles, n, bases);
            CUDA_TRY(cudaGetLastError());
            post_scan_sums_kernel<<<n, 256, 0, st>>>(d.posts, n, bases);
            CUDA_TRY(cudaGetLastError());
        }
        post_apply_kernel<<<tiles, 256, 0, st>>>(d.posts, d.post_tiles, n, bases);
        CUDA_TRY(cudaGetLastError());
        return 0;
    };
    int64_t rc;
    if ((rc = launch_decodes(0)) < 0 || (rc = launch_merges(0)) < 0 || (rc = launch_posts()) < 0 || (rc = launch_decodes(1)) < 0 || (rc = launch_merges(1)) < 0) return rc;
    if ((flags & PTWM_B200_VERIFY_CRC) && !pl.verify.empty()) {
        CUDA_TRY(cudaMemsetAsync(d.acc, 0, (pl.n_acc + 1) * sizeof(uint32_t), st));
        uint64_t blocks = (pl.n_runs + 127) / 128;
        CUDA_TRY(mark(10, 0));
        crc_planes_kernel<<<uint32_t(blocks), 128, 0, st>>>(d.verify, uint32_t(pl.verify.size()), pl.n_runs, bases, d_tabs, d.acc);
        CUDA_TRY(cudaGetLastError());
        CUDA_TRY(mark(10, 1));
    }
    if ((flags & PTWM_B200_VERIFY_HASH) && !pl.hashes.empty()) {
        uint32_t n = uint32_t(pl.hashes.size());
        CUDA_TRY(mark(11, 0));
        xxh64_kernel<<<n, 32, 0, st>>>(d.hashes, n, bases, d.hash_out);
        CUDA_TRY(cudaGetLastError());
        CUDA_TRY(mark(11, 1));
    }
    return 0;
}

const char* status_text(uint32_t s) {
    switch (s) {
        case ST_BAD_HEADER: return "malformed codec header (weights, frequency table or jump table)";
        case ST_STREAM_UNDERRUN: return "stream ended before its symbols did";
        case ST_NOT_CONSUMED: return "bitstream not fully consumed";
        case ST_BAD_STATE: return "invalid Order1ScaleAC state";
        default: return "unknown decode failure";
    }
}

int64_t evaluate(ptwm_b200_plan& pl, DevicePlan& d, uint32_t flags, cudaStream_t st) {
    CUDA_TRY(cudaStreamSynchronize(st));
    // decode status: items write their own slot; scan on the host
    std::vector<uint32_t> status(pl.item_tensor.size() + 1);
    CUDA_TRY(cudaMemcpy(status.data(), d.status, status.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    for (size_t i = 1; i < status.size(); ++i)
        if (status[i]) return fail(PTWM_RC_CORRUPT, "tensor '" + pl.c->file.tensors[pl.item_tensor[i - 1]].name + "': " + status_text(status[i]));
    if ((flags & PTWM_B200_VERIFY_CRC) && !pl.crc_expect.empty()) {
        std::vector<uint32_t> acc(pl.n_acc);
        CUDA_TRY(cudaMemcpy(acc.data(), d.acc, acc.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost));
        const CrcTables& T = crc_tables();
        for (const CrcExpect& e : pl.crc_expect) {
            // crc = ~(remainder ^ 0xFFFFFFFF * x^(8 len))
            uint32_t got = ~(acc[e.acc] ^ gf2_mulmod(x_pow_8n(T.x2n, e.plane_len), 0xFFFFFFFFu));
            if (got != e.crc) return fail(PTWM_RC_CORRUPT, "tensor '" + pl.c->file.tensors[e.tensor].name + "': plane CRC mismatch");
        }
    }
    if ((flags & PTWM_B200_VERIFY_HASH) && !pl.hash_expect.empty()) {
        std::vector<uint64_t> h(pl.hash_expect.size());
        CUDA_TRY(cudaMemcpy(h.data(), d.hash_out, h.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < h.size(); ++i)
            if (h[i] != pl.hash_expect[i].hash) return fail(PTWM_RC_CORRUPT, "tensor '" + pl.c->file.tensors[pl.hash_expect[i].tensor].name + "': tensor payload hash mismatch");
    }
    return 0;
}

// Built-in codec canonical ids: blake3([0xBB;32] || 0 || name || 0 || "1.1.0")
// (extension/id.rs:21-31, extension/mod.rs:36, Cargo.toml:6 of the reference).
struct BuiltinId { uint8_t id[32]; uint16_t codec; const char* name; };
const BuiltinId kBuiltins[] = {
    {{0xfc,0x2d,0xea,0x12,0x65,0xe3,0x39,0x4c,0x57,0xc2,0xdf,0x3b,0x86,0x8b,0x73,0x2c,0xca,0xa1,0xee,0x87,0x6b,0xd4,0xb1,0xce,0x27,0xd3,0x8f,0x84,0x2c,0x61,0x12,0xb5}, C_IDENTITY, "identity"},
    {{0x61,0x41,0x55,0xb5,0xa8,0xc9,0xef,0xb6,0x89,0x21,0x9b,0xcc,0xa3,0xcb,0xf7,0x85,0x5e,0x29,0xd3,0x02,0x32,0x08,0xce,0x61,0xcc,0xa7,0xa3,0x68,0x49,0x24,0x8e,0x33}, C_HUFFMAN, "huffman"},
    {{0x39,0xc8,0x75,0xef,0x97,0x93,0xa9,0xc5,0xeb,0xe1,0x99,0x11,0x6d,0xeb,0xac,0x4c,0x9d,0x53,0x88,0xb8,0xb7,0xcf,0x2f,0xe6,0xb5,0x75,0x84,0x5f,0x0c,0xa1,0x62,0x4e}, C_RANS, "rans"},
    {{0xe4,0x86,0x85,0x45,0xe7,0xb2,0x22,0x82,0x69,0x59,0x72,0x44,0x14,0x94,0xe7,0x05,0x69,0xab,0x27,0x59,0x5d,0x19,0x34,0x91,0x14,0xe8,0x52,0x12,0x5d,0x96,0xda,0xa4}, C_TANS, "tans"},
    {{0x0b,0x84,0x26,0xe0,0xa6,0x70,0xd1,0x14,0xf2,0x4e,0xe4,0x61,0x48,0x37,0xc9,0x57,0x8f,0xf3,0x03,0x4f,0x11,0xe4,0xe9,0xe9,0xc0,0xf5,0xd9,0x2a,0x49,0x88,0x77,0x70}, C_O1SAC, "order1_scale_ac"},
};

// One plane payload, device to device: the body of the reference-facing symbols.
int64_t decode_plane_cuda(uint8_t sfv, const uint8_t* state, size_t state_len, const uint8_t* codec_id, size_t codec_id_len, uint64_t in_dev, size_t in_len,
                          uint64_t out_dev, size_t out_cap, uint32_t device) {
    if (!codec_id || codec_id_len != 32) return fail(PTWM_RC_INVALID_INPUT, "codec_id must be a 32-byte canonical id");
    int codec = -1;
    for (const BuiltinId& b : kBuiltins) if (!std::memcmp(b.id, codec_id, 32)) codec = b.codec;
    if (codec < 0) return fail(PTWM_RC_UNSUPPORTED, "codec id is not one of identity, huffman, rans, tans, order1_scale_ac");
    if ((in_len && !in_dev) || (out_cap && !out_dev)) return fail(PTWM_RC_INVALID_INPUT, "null device pointer");
    if (in_len > 0xFFFFFFFFull) return fail(PTWM_RC_UNSUPPORTED, "payload longer than 4 GiB");
    DeviceGuard guard{int(device)};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(guard.err));
    DeviceState* ds;
    int64_t rc = device_state(int(device), &ds);
    if (rc < 0) return rc;
    cudaStream_t st = ds->stream;
    // The tag and length prefix decide what runs: read them back, in stream order.  The producer of the
    // payload was ordered against this stream (the caller hands the stream handle to the tensor's DLPack
    // export, native.rs:105-112 of the reference); a copy on the legacy default stream would not wait for it,
    // because this stream is non-blocking.
    uint8_t head[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (in_len) {
        CUDA_TRY(cudaMemcpyAsync(head, reinterpret_cast<const void*>(in_dev), std::min<size_t>(in_len, 8), cudaMemcpyDeviceToHost, st));
        CUDA_TRY(cudaStreamSynchronize(st));
    }
    ChunkDesc ch{};
    ch.body_off = 0; ch.body_len = in_len;
    uint64_t decoded;
    try {
        if (codec == C_IDENTITY) decoded = in_len;
        else if (codec == C_O1SAC) decoded = out_cap;
        else {
            if (!in_len) throw FormatError("empty payload");
            if (head[0] == 0) decoded = in_len - 1;
            else if (head[0] == 1 && in_len >= 5) decoded = le32(head + 1);
            else throw FormatError("bad codec tag or payload too short for length prefix");
        }
        if (decoded > out_cap) return fail(PTWM_RC_BUFFER_TOO_SMALL, "output buffer smaller than the decoded plane");
        ch.decoded = uint32_t(decoded);
        detail::classify_chunk(head, uint16_t(codec), ch);  // only reads head[0..6)
        if (codec == C_O1SAC) check_o1sac(state, state_len, sfv, in_len, decoded, 0);
    } catch (const FormatError& e) { return fail(PTWM_RC_INVALID_INPUT, e.what()); }
    if (!decoded) return 0;
    Bases bases{reinterpret_cast<const uint8_t*>(in_dev), 0, in_len, nullptr, reinterpret_cast<uint8_t*>(out_dev)};
    if (ch.raw) {
        CUDA_TRY(cudaMemcpyAsync(reinterpret_cast<void*>(out_dev), reinterpret_cast<const void*>(in_dev + ch.data_off), decoded, cudaMemcpyDeviceToDevice, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        return int64_t(decoded);
    }
    DecodeItem it{};
    it.src = make_ref(SP_BLOB, ch.data_off); it.src_len = uint32_t(ch.data_len); it.n = uint32_t(decoded); it.dst = make_ref(SP_OUT, 0);
    it.partner[0] = it.partner[1] = it.partner[2] = REF_NONE; it.state = REF_NONE; it.work = REF_NONE; it.id = 0;
    // device scratch for the item, the status word and (O1SAC) the state and its tables
    size_t tables = codec == C_O1SAC ? (state_len - 32) / 512 : 0;
    size_t work_off = 256, state_off = work_off + align_up(tables * 514, 256), total = state_off + align_up(state_len, 256);
    uint8_t* scratch = nullptr;
    CUDA_TRY(cudaMalloc(&scratch, total));
    struct Free { uint8_t* p; ~Free() { cudaFree(p); } } freer{scratch};
    bases.scratch = scratch;
    if (codec == C_O1SAC) {
        it.state = make_ref(SP_SCRATCH, state_off); it.state_len = uint32_t(state_len); it.state_version = sfv; it.row_len = 0;
        it.work = make_ref(SP_SCRATCH, work_off);
        CUDA_TRY(cudaMemcpyAsync(scratch + state_off, state, state_len, cudaMemcpyHostToDevice, st));
    }
    CUDA_TRY(cudaMemsetAsync(scratch, 0, 256, st));
    CUDA_TRY(cudaMemcpyAsync(scratch + 64, &it, sizeof it, cudaMemcpyHostToDevice, st));
    const DecodeItem* d_it = reinterpret_cast<const DecodeItem*>(scratch + 64);
    uint32_t* d_status = reinterpret_cast<uint32_t*>(scratch);
    switch (codec) {
        case C_RANS: rans_decode_kernel_t<false><<<1, 32, rans_smem_bytes(rans_l_entries(255)), st>>>(d_it, 1, bases, d_status, rans_l_entries(255)); break;
        case C_HUFFMAN: huffman_decode_kernel<<<1, 32, HUF_SMEM, st>>>(d_it, 1, bases, d_status); break;
        case C_TANS: tans_decode_kernel<<<1, TANS_THREADS, TANS_SMEM, st>>>(d_it, 1, bases, d_status); break;
        default: o1sac_launch(d_it, 1, bases, d_status, o1sac_tables(state_len), st); break;
    }
    CUDA_TRY(cudaGetLastError());
    uint32_t status = 0;
    CUDA_TRY(cudaMemcpyAsync(&status, d_status, 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    if (status) return fail(PTWM_RC_CORRUPT, status_text(status));  // the payload itself is damaged: same code as plan_finish
    return int64_t(decoded);
}

uint64_t stream_handle(uint32_t device) {
    DeviceGuard guard{int(device)};
    if (guard.err != cudaSuccess) return 0;
    DeviceState* ds;
    if (device_state(int(device), &ds) < 0) return 0;
    return uint64_t(reinterpret_cast<uintptr_t>(ds->stream));
}

}  // namespace

extern "C" {

const char* ptwm_b200_last_error(void) { return last_error_ref().c_str(); }
void ptwm_b200_blake3(const uint8_t* data, size_t len, uint8_t out[32]) { blake3_hash(data, len, out); }
uint64_t ptwm_b200_xxh64(const uint8_t* data, size_t len) { return xxh64_host(data, len); }

uint64_t ptwm_hardware_backend_v1_cuda_stream_handle(uint32_t device_ordinal) { return stream_handle(device_ordinal); }
uint64_t ptwm_plane_codec_v1_cuda_stream_handle(uint32_t device_ordinal) { return stream_handle(device_ordinal); }

int64_t ptwm_hardware_backend_v1_dispatch_decode_cuda(uint8_t sfv, const uint8_t* state_ptr, size_t state_len, const uint8_t* codec_id_ptr, size_t codec_id_len,
                                                      uint64_t in_dev_ptr, size_t in_len, uint64_t out_dev_ptr, size_t out_len, uint32_t device_ordinal) {
    return decode_plane_cuda(sfv, state_ptr, state_len, codec_id_ptr, codec_id_len, in_dev_ptr, in_len, out_dev_ptr, out_len, device_ordinal);
}
int64_t ptwm_plane_codec_v1_decode_cuda(uint8_t sfv, const uint8_t* state_ptr, size_t state_len, const uint8_t* codec_id_ptr, size_t codec_id_len,
                                        uint64_t in_dev_ptr, size_t in_len, uint64_t out_dev_ptr, size_t out_cap, uint32_t device_ordinal) {
    return decode_plane_cuda(sfv, state_ptr, state_len, codec_id_ptr, codec_id_len, in_dev_ptr, in_len, out_dev_ptr, out_cap, device_ordinal);
}
int64_t ptwm_plane_codec_v1_encode_cuda(uint8_t sfv, const uint8_t* state_ptr, size_t state_len, const uint8_t* codec_id, size_t codec_id_len, uint64_t in_dev, size_t in_len,
                                        uint64_t out_dev, size_t out_cap, uint64_t* needed_out, uint32_t device_ordinal) {
    // *needed_out is written only together with PTWM_RC_BUFFER_TOO_SMALL and left untouched otherwise (native.rs:176-184)
    if (!codec_id || codec_id_len != 32) return fail(PTWM_RC_INVALID_INPUT, "codec_id must be a 32-byte canonical id");
    int codec = -1;
    for (const BuiltinId& b : kBuiltins) if (!std::memcmp(b.id, codec_id, 32)) codec = b.codec;
    if (codec < 0) return fail(PTWM_RC_UNSUPPORTED, "codec id is not one of identity, huffman, rans, tans, order1_scale_ac");
    if ((in_len && !in_dev) || (out_cap && !out_dev)) return fail(PTWM_RC_INVALID_INPUT, "null device pointer");
    DeviceGuard guard{int(device_ordinal)};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(guard.err));
    DeviceState* ds;
    int64_t rc = device_state(int(device_ordinal), &ds);
    if (rc < 0) return rc;
    return encode_plane_cuda(codec, state_len ? state_ptr : nullptr, state_len, sfv, in_dev, in_len, out_dev, out_cap, needed_out, ds->stream);
}
// Host buffers, rANS (the codec this bundle registers as its plane codec): the payload is built on GPU 0.
int64_t ptwm_plane_codec_v1_encode(const uint8_t* in, size_t in_len, uint8_t* out, size_t out_len) {
    if ((in_len && !in) || (out_len && !out)) return fail(PTWM_RC_INVALID_INPUT, "null buffer");
    DeviceGuard guard{0};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_MISSING_CAPABILITY, "no CUDA device");
    DeviceState* ds;
    int64_t rc = device_state(0, &ds);
    if (rc < 0) return rc;
    const size_t cap = in_len + 16;
    uint8_t *d_in = nullptr, *d_out = nullptr;
    CUDA_TRY(cudaMalloc(&d_in, in_len ? in_len : 1));
    struct Free { uint8_t* p; ~Free() { cudaFree(p); } } f1{d_in};
    CUDA_TRY(cudaMalloc(&d_out, cap));
    Free f2{d_out};
    CUDA_TRY(cudaMemcpy(d_in, in, in_len, cudaMemcpyHostToDevice));
    uint64_t needed = 0;
    int64_t n = encode_plane_cuda(C_RANS, nullptr, 0, 0, uint64_t(reinterpret_cast<uintptr_t>(d_in)), in_len, uint64_t(reinterpret_cast<uintptr_t>(d_out)), cap, &needed, ds->stream);
    if (n < 0) return n;
    if (size_t(n) > out_len) return fail(PTWM_RC_BUFFER_TOO_SMALL, "output buffer too small");
    CUDA_TRY(cudaMemcpy(out, d_out, size_t(n), cudaMemcpyDeviceToHost));
    return n;
}

int64_t ptwm_plane_codec_v1_decode_stateful(uint8_t sv, const uint8_t* state, size_t state_len, const uint8_t* in, size_t in_len, uint8_t* out, size_t out_cap) {
    if ((in_len && !in) || (out_cap && !out)) return fail(PTWM_RC_INVALID_INPUT, "null buffer");
    DeviceGuard guard{0};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_MISSING_CAPABILITY, "no CUDA device");
    uint8_t *d_in = nullptr, *d_out = nullptr;
    CUDA_TRY(cudaMalloc(&d_in, in_len ? in_len : 1));
    struct Free { uint8_t* p; ~Free() { cudaFree(p); } } f1{d_in};
    CUDA_TRY(cudaMalloc(&d_out, out_cap ? out_cap : 1));
    Free f2{d_out};
    CUDA_TRY(cudaMemcpy(d_in, in, in_len, cudaMemcpyHostToDevice));
    int64_t n = decode_plane_cuda(sv, state, state_len, kBuiltins[2].id, 32, uint64_t(reinterpret_cast<uintptr_t>(d_in)), in_len,
                                  uint64_t(reinterpret_cast<uintptr_t>(d_out)), out_cap, 0);
    if (n < 0) return n;
    CUDA_TRY(cudaMemcpy(out, d_out, size_t(n), cudaMemcpyDeviceToHost));
    return n;
}
int64_t ptwm_plane_codec_v1_decode(const uint8_t* in, size_t in_len, uint8_t* out, size_t out_len) {
    return ptwm_plane_codec_v1_decode_stateful(0, nullptr, 0, in, in_len, out, out_len);
}

int64_t ptwm_b200_open(const uint8_t* blob, size_t blob_len, ptwm_b200_container** out) { return ptwm_b200_open_shard(blob, blob_len, 0, 1, out); }

int64_t ptwm_b200_open_shard(const uint8_t* blob, size_t blob_len, uint32_t rank, uint32_t world, ptwm_b200_container** out) {
    if (!blob || !out) return fail(PTWM_RC_INVALID_INPUT, "null argument");
    if (!world || rank >= world) return fail(PTWM_RC_INVALID_INPUT, "rank must be below world");
    try {
        std::unique_ptr<ptwm_b200_container> c(new ptwm_b200_container);
        FileReader reader(blob, blob_len);
        reader.set_shard(rank, world);
        c->file = reader.parse();
        c->blob_len = blob_len;
        for (const TensorDesc& t : c->file.tensors) {
            uint64_t comp = 0, lo = UINT64_MAX, hi = 0; uint8_t crc = 0;
            if (t.stored) { comp = t.orig_size; lo = t.stored_off; hi = t.stored_off + t.orig_size; }
            for (const PlaneDesc& p : t.planes) {
                comp += p.payload_len; crc |= p.has_crc;
                lo = std::min(lo, p.payload_off); hi = std::max(hi, p.payload_off + p.payload_len);
                for (const ChunkDesc& ch : p.chunks) if (ch.state_len) { lo = std::min(lo, ch.state_off); hi = std::max(hi, ch.state_off + ch.state_len); }
            }
            if (lo == UINT64_MAX) lo = hi = 0;
            if (!comp && t.record_len && !t.unsupported.empty()) comp = t.record_len;  // a record that was not read: its size from the index
            c->compressed.push_back(comp); c->first_byte.push_back(lo); c->end_byte.push_back(hi); c->has_crc.push_back(crc);
        }
        *out = c.release();
        return 0;
    } catch (const FormatError& e) { return fail(e.unsupported ? PTWM_RC_UNSUPPORTED : PTWM_RC_INVALID_INPUT, e.what()); }
    catch (const std::exception& e) { return fail(PTWM_RC_INTERNAL, e.what()); }
}
void ptwm_b200_close(ptwm_b200_container* c) { delete c; }
size_t ptwm_b200_tensor_count(const ptwm_b200_container* c) { return c ? c->file.tensors.size() : 0; }

int64_t ptwm_b200_tensor_info_get(const ptwm_b200_container* c, size_t index, ptwm_b200_tensor_info* info) {
    if (!c || !info || index >= c->file.tensors.size()) return fail(PTWM_RC_INVALID_INPUT, "tensor index out of range");
    const TensorDesc& t = c->file.tensors[index];
    std::memset(info, 0, sizeof *info);
    info->name = t.name.c_str(); info->dtype_name = t.dtype_name.c_str(); info->dtype_code = t.dtype_code;
    info->has_shape = t.has_shape && t.shape.size() <= 8; info->ndim = uint8_t(std::min<size_t>(t.shape.size(), 8));
    for (size_t d = 0; d < info->ndim; ++d) info->shape[d] = t.shape[d];
    info->has_hash = t.has_hash; info->has_crc = c->has_crc[index]; info->supported = t.unsupported.empty(); info->kind = t.kind;
    info->orig_size = t.orig_size; info->compressed = c->compressed[index]; info->first_byte = c->first_byte[index]; info->end_byte = c->end_byte[index];
    info->unsupported_reason = t.unsupported.c_str();
    return 0;
}

int64_t ptwm_b200_plan_create(const ptwm_b200_container* c, const uint32_t* indices, size_t n, ptwm_b200_plan** out) {
    if (!c || !out) return fail(PTWM_RC_INVALID_INPUT, "null argument");
    try {
        std::unique_ptr<ptwm_b200_plan> pl(new ptwm_b200_plan);
        pl->c = c;
        if (!indices) { n = c->file.tensors.size(); for (size_t i = 0; i < n; ++i) pl->tensors.push_back(uint32_t(i)); }
        else pl->tensors.assign(indices, indices + n);
        pl->blob_lo = UINT64_MAX;
        for (uint32_t ti : pl->tensors) {
            if (ti >= c->file.tensors.size()) return fail(PTWM_RC_INVALID_INPUT, "tensor index out of range");
            const TensorDesc& t = c->file.tensors[ti];
            if (!t.unsupported.empty()) return fail(PTWM_RC_UNSUPPORTED, "tensor '" + t.name + "': " + t.unsupported);
            uint64_t off = pl->out_bytes;
            pl->out_off.push_back(off);
            pl->out_bytes += align_up(t.orig_size, 256);
            plan_tensor(*pl, ti, t, off);
            bool any_crc = false;
            for (const PlaneDesc& p : t.planes) any_crc |= p.has_crc;
            if (any_crc && t.planes[0].decoded_len) {
                VerifyTensor v{make_ref(SP_OUT, off), t.planes[0].decoded_len, pl->n_runs, t.kind, pl->n_acc, 0, 0};
                for (size_t p = 0; p < t.planes.size() && p < 4; ++p) { v.post |= uint32_t(t.planes[p].post) << (8 * p); v.post_k |= uint32_t(t.planes[p].post_k) << (8 * p); }
                pl->n_runs += (v.n_elems + VERIFY_RUN - 1) / VERIFY_RUN;
                pl->slot_bytes[10] += t.orig_size; pl->slot_items[10]++;  // the check reads the decoded tensor once
                for (size_t p = 0; p < t.planes.size(); ++p) if (t.planes[p].has_crc) pl->crc_expect.push_back({pl->n_acc + uint32_t(p), t.planes[p].crc, t.planes[p].decoded_len, ti});
                pl->n_acc += uint32_t(t.planes.size());
                pl->verify.push_back(v);
            } else if (any_crc) {
                for (const PlaneDesc& p : t.planes) if (p.has_crc && p.crc != 0) return fail(PTWM_RC_CORRUPT, "tensor '" + t.name + "': plane CRC mismatch");
            }
            if (t.has_hash) {
                pl->hashes.push_back(HashItem{make_ref(SP_OUT, off), t.orig_size}); pl->hash_expect.push_back({t.hash, ti});
                pl->slot_bytes[11] += t.orig_size; pl->slot_items[11]++;
            }
        }
        if (pl->blob_lo == UINT64_MAX) pl->blob_lo = pl->blob_hi = 0;
        pl->scratch_bytes = align_up(pl->scratch_bytes, 256);
        {   // the payload hash of a tensor is one serial chain: the longest tensors start first, the longest one is the critical path
            std::vector<size_t> order(pl->hashes.size());
            for (size_t k = 0; k < order.size(); ++k) order[k] = k;
            std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return pl->hashes[a].len > pl->hashes[b].len; });
            std::vector<HashItem> hs; std::vector<HashExpect> he;
            for (size_t k : order) { hs.push_back(pl->hashes[k]); he.push_back(pl->hash_expect[k]); }
            pl->hashes.swap(hs); pl->hash_expect.swap(he);
        }
        finish_lists(*pl);
        *out = pl.release();
        return 0;
    } catch (const std::exception& e) { return fail(PTWM_RC_INTERNAL, e.what()); }
}
void ptwm_b200_plan_destroy(ptwm_b200_plan* p) { delete p; }
uint64_t ptwm_b200_plan_out_bytes(const ptwm_b200_plan* p) { return p->out_bytes; }
uint64_t ptwm_b200_plan_scratch_bytes(const ptwm_b200_plan* p) { return p->scratch_bytes; }
uint64_t ptwm_b200_plan_out_offset(const ptwm_b200_plan* p, size_t k) { return k < p->out_off.size() ? p->out_off[k] : UINT64_MAX; }
void ptwm_b200_plan_blob_span(const ptwm_b200_plan* p, uint64_t* lo, uint64_t* hi) { if (lo) *lo = p->blob_lo; if (hi) *hi = p->blob_hi; }
void ptwm_b200_plan_stats(const ptwm_b200_plan* p, uint64_t* r, uint64_t* w, uint32_t* launches) { if (r) *r = p->bytes_read; if (w) *w = p->bytes_written; if (launches) *launches = p->launches; }

int64_t ptwm_b200_plan_run(ptwm_b200_plan* p, uint64_t blob_dev_ptr, uint64_t blob_first, uint64_t blob_len, uint64_t out_dev_ptr, uint64_t out_cap,
                           uint64_t scratch_dev_ptr, uint64_t scratch_cap, uint32_t flags, uint32_t device_ordinal, uint64_t stream) {
    if (!p) return fail(PTWM_RC_INVALID_INPUT, "null plan");
    if (out_cap < p->out_bytes) return fail(PTWM_RC_BUFFER_TOO_SMALL, "output arena smaller than ptwm_b200_plan_out_bytes");
    if (scratch_cap < p->scratch_bytes) return fail(PTWM_RC_BUFFER_TOO_SMALL, "scratch arena smaller than ptwm_b200_plan_scratch_bytes");
    if (p->blob_hi > p->blob_lo && (blob_first > p->blob_lo || blob_first + blob_len < p->blob_hi)) return fail(PTWM_RC_INVALID_INPUT, "resident blob span does not cover ptwm_b200_plan_blob_span");
    if ((p->out_bytes && !out_dev_ptr) || (p->scratch_bytes && !scratch_dev_ptr) || (p->blob_hi > p->blob_lo && !blob_dev_ptr)) return fail(PTWM_RC_INVALID_INPUT, "null device pointer");
    DeviceGuard guard{int(device_ordinal)};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(guard.err));
    DeviceState* ds;
    int64_t rc = device_state(int(device_ordinal), &ds);
    if (rc < 0) return rc;
    cudaStream_t st = stream ? reinterpret_cast<cudaStream_t>(uintptr_t(stream)) : ds->stream;
    std::lock_guard<std::mutex> lock(p->mu);
    DevicePlan* d;
    if ((rc = device_plan(*p, int(device_ordinal), *ds, &d)) < 0) return rc;
    // Refs hold file offsets; the kernels clamp their 16-byte fetches to the resident span
    Bases launch{reinterpret_cast<const uint8_t*>(uintptr_t(blob_dev_ptr)), blob_first, blob_first + blob_len, reinterpret_cast<uint8_t*>(uintptr_t(scratch_dev_ptr)),
                 reinterpret_cast<uint8_t*>(uintptr_t(out_dev_ptr))};
    if ((rc = enqueue(*p, *d, launch, flags, ds->d_tabs, st)) < 0) return rc;
    if (flags & PTWM_B200_NO_SYNC) return 0;
    return evaluate(*p, *d, flags, st);
}

int64_t ptwm_b200_plan_prepare(ptwm_b200_plan* p, uint32_t device_ordinal) {
    if (!p) return fail(PTWM_RC_INVALID_INPUT, "null plan");
    DeviceGuard guard{int(device_ordinal)};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(guard.err));
    DeviceState* ds;
    int64_t rc = device_state(int(device_ordinal), &ds);
    if (rc < 0) return rc;
    std::lock_guard<std::mutex> lock(p->mu);
    DevicePlan* d;
    return device_plan(*p, int(device_ordinal), *ds, &d);
}

uint64_t ptwm_b200_plan_device_bytes(const ptwm_b200_plan* p) { return p ? plan_layout(*p).total : 0; }
int64_t ptwm_b200_plan_prepare_in(ptwm_b200_plan* p, uint32_t device_ordinal, uint64_t dev_ptr, uint64_t cap) {
    if (!p || !dev_ptr) return fail(PTWM_RC_INVALID_INPUT, "null plan or memory");
    DeviceGuard guard{int(device_ordinal)};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(guard.err));
    DeviceState* ds;
    int64_t rc = device_state(int(device_ordinal), &ds);
    if (rc < 0) return rc;
    std::lock_guard<std::mutex> lock(p->mu);
    if (p->dev.count(int(device_ordinal))) return fail(PTWM_RC_INVALID_INPUT, "the plan is already prepared on this device");
    DevicePlan* d;
    return device_plan(*p, int(device_ordinal), *ds, &d, reinterpret_cast<uint8_t*>(uintptr_t(dev_ptr)), cap);
}

int64_t ptwm_b200_plan_finish(ptwm_b200_plan* p, uint32_t flags, uint32_t device_ordinal, uint64_t stream) {
    if (!p) return fail(PTWM_RC_INVALID_INPUT, "null plan");
    DeviceGuard guard{int(device_ordinal)};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(guard.err));
    DeviceState* ds;
    int64_t rc = device_state(int(device_ordinal), &ds);
    if (rc < 0) return rc;
    cudaStream_t st = stream ? reinterpret_cast<cudaStream_t>(uintptr_t(stream)) : ds->stream;
    std::lock_guard<std::mutex> lock(p->mu);
    auto it = p->dev.find(int(device_ordinal));
    if (it == p->dev.end()) return fail(PTWM_RC_INVALID_INPUT, "plan has not run on this device");
    return evaluate(*p, it->second, flags, st);
}

int64_t ptwm_b200_plan_timings(ptwm_b200_plan* p, uint32_t device_ordinal, float* ms, uint64_t* bytes, uint32_t* items) {
    if (!p) return fail(PTWM_RC_INVALID_INPUT, "null plan");
    DeviceGuard guard{int(device_ordinal)};
    std::lock_guard<std::mutex> lock(p->mu);
    auto it = p->dev.find(int(device_ordinal));
    if (it == p->dev.end()) return fail(PTWM_RC_INVALID_INPUT, "plan has not run on this device");
    for (int s = 0; s < 12; ++s) {
        float t = -1.0f;
        if (it->second.timed[s]) CUDA_TRY(cudaEventElapsedTime(&t, it->second.ev[2 * s], it->second.ev[2 * s + 1]));
        if (ms) ms[s] = t;
        if (bytes) bytes[s] = p->slot_bytes[s];
        if (items) items[s] = p->slot_items[s];
    }
    return 12;
}

uint32_t ptwm_b200_crc32_by_runs(const uint8_t* data, size_t len, size_t run) {
    const CrcTables& T = crc_tables();
    if (!run) run = VERIFY_RUN;
    uint32_t acc = 0;
    for (size_t first = 0; first < len; first += run) {
        size_t n = std::min(run, len - first);
        uint32_t c = 0;
        for (size_t i = 0; i < n; ++i) c = T.byte_table[(c ^ data[first + i]) & 0xFF] ^ (c >> 8);
        acc ^= gf2_mulmod(x_pow_8n(T.x2n, len - first - n), c);
    }
    return ~(acc ^ gf2_mulmod(x_pow_8n(T.x2n, len), 0xFFFFFFFFu));
}

}  // extern "C"
