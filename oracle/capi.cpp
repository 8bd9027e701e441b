// CPU oracle (TEST INFRASTRUCTURE, not a product path): C entry points over
// the restatement in entropy.hpp / codecs.hpp / container.hpp, loaded with
// ctypes by oracle/__init__.py.  Buffers returned through `uint8_t**` are
// malloc'ed and released with oracle_free.
#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <sstream>

#include "container.hpp"

using namespace oracle;

static thread_local std::string g_err;

static int fail(const std::exception& e) { g_err = e.what(); return -1; }
static uint8_t* dup(const Bytes& b) {
    uint8_t* p = static_cast<uint8_t*>(std::malloc(b.size() ? b.size() : 1));
    if (b.size()) std::memcpy(p, b.data(), b.size());
    return p;
}

extern "C" {

const char* oracle_last_error() { return g_err.c_str(); }
void oracle_free(void* p) { std::free(p); }

uint32_t oracle_crc32(const uint8_t* p, size_t n) { return crc32(p, n); }
uint64_t oracle_xxh64(const uint8_t* p, size_t n, uint64_t seed) { return xxh64(p, n, seed); }

int oracle_plane_encode(int codec, const uint8_t* plane, size_t n, size_t row_len, const uint8_t* shared, size_t shared_len,
                        uint8_t** state, size_t* state_len, uint8_t* state_version, uint8_t** payload, size_t* payload_len) {
    try {
        Encoded e = plane_encode(CodecId(codec), plane, n, row_len, shared, shared_len);
        *state = dup(e.state); *state_len = e.state.size(); *state_version = e.state_version;
        *payload = dup(e.payload); *payload_len = e.payload.size();
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

int oracle_plane_decode(int codec, uint8_t state_version, const uint8_t* state, size_t state_len, const uint8_t* payload, size_t payload_len,
                        size_t row_len, size_t decoded_len, size_t max_len, uint8_t** out, size_t* out_len) {
    try {
        Bytes d = plane_decode(CodecId(codec), state_version, state, state_len, payload, payload_len, row_len, decoded_len, max_len);
        *out = dup(d); *out_len = d.size();
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

// Raw codec blobs without the tag/length wrapper (entropy/{huffman,rans,tans}).
int oracle_raw_compress(int codec, const uint8_t* src, size_t n, uint8_t** out, size_t* out_len) {
    try {
        Bytes b = codec == HUFFMAN ? huffman::compress(src, n) : codec == RANS ? rans::compress(src, n) : tans::compress(src, n, n);
        *out = dup(b); *out_len = b.size();
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}
int oracle_raw_decompress(int codec, const uint8_t* src, size_t len, uint8_t* dst, size_t n) {
    try {
        if (codec == HUFFMAN) huffman::decompress(dst, n, src, len);
        else if (codec == RANS) rans::decompress(dst, n, src, len);
        else tans::decompress(dst, n, src, len);
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

// planes_out receives the planes back to back (merge_planes(kind) × plane_len).
int oracle_split_forward(int kind, const uint8_t* src, size_t n, uint8_t** planes_out, size_t* plane_len) {
    try {
        auto p = split_forward(MergeKind(kind), src, n);
        Bytes all;
        for (auto& b : p) all.insert(all.end(), b.begin(), b.end());
        *planes_out = dup(all); *plane_len = p[0].size();
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}
int oracle_merge_inverse(int kind, const uint8_t* planes, size_t plane_len, uint8_t** out, size_t* out_len) {
    try {
        std::vector<Bytes> p;
        p.resize(size_t(merge_planes(MergeKind(kind))));
        for (size_t i = 0; i < p.size(); ++i) p[i].assign(planes + i * plane_len, planes + (i + 1) * plane_len);
        Bytes r = merge_inverse(MergeKind(kind), p);
        *out = dup(r); *out_len = r.size();
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

int oracle_quantize_pmf(const uint32_t* raw, size_t n, uint32_t total, uint16_t* out) { quantize_pmf(raw, n, total, out); return 0; }

// ---- containers -----------------------------------------------------------
void* oracle_container_open(const uint8_t* buf, size_t len) {
    try { return new Container(open_container(buf, len)); } catch (const std::exception& e) { fail(e); return nullptr; }
}
void oracle_container_close(void* h) { delete static_cast<Container*>(h); }
size_t oracle_container_count(void* h) { return static_cast<Container*>(h)->tensors.size(); }

// One JSON object per container: names, dtypes, shapes, sizes and per-plane
// codec / chunk facts, for the Python wrapper.
int oracle_container_describe(void* h, uint8_t** out, size_t* out_len) {
    try {
        Container& c = *static_cast<Container*>(h);
        std::ostringstream o;
        o << "{\"tensors\":[";
        for (size_t i = 0; i < c.tensors.size(); ++i) {
            const TensorRec& t = c.tensors[i];
            if (i) o << ",";
            o << "{\"name\":\"";
            for (char ch : t.name) { if (ch == '"' || ch == '\\') o << '\\'; o << ch; }
            o << "\",\"dtype_code\":" << t.dtype_code << ",\"dtype_name\":\"" << t.dtype_name << "\",\"orig_size\":" << t.orig_size
              << ",\"has_shape\":" << (t.has_shape ? "true" : "false") << ",\"shape\":[";
            for (size_t d = 0; d < t.shape.size(); ++d) o << (d ? "," : "") << t.shape[d];
            o << "],\"has_hash\":" << (t.has_hash ? "true" : "false") << ",\"hash\":" << t.hash << ",\"kind\":" << int(t.info.kind)
              << ",\"unsupported\":" << (t.unsupported.empty() ? "false" : "true") << ",\"rec_off\":" << t.rec_off << ",\"rec_len\":" << t.rec_len << ",\"planes\":[";
            for (size_t p = 0; p < t.planes.size(); ++p) {
                const PlaneRec& pr = t.planes[p];
                o << (p ? "," : "") << "{\"codec\":" << pr.codec_id << ",\"role\":" << int(pr.role) << ",\"payload_len\":" << pr.payload_len
                  << ",\"payload_off\":" << size_t(pr.payload - c.buf) << ",\"state_source\":" << pr.state_source << ",\"row_len\":" << pr.row_len
                  << ",\"has_crc\":" << (pr.has_crc ? "true" : "false") << ",\"crc\":" << pr.crc << ",\"n_chunks\":" << (pr.chunked ? long(pr.chunks.size()) : -1L) << "}";
            }
            o << "]}";
        }
        o << "]}";
        std::string s = o.str();
        Bytes b(s.begin(), s.end());
        *out = dup(b); *out_len = b.size();
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

int oracle_container_decode_tensor(void* h, size_t index, int verify, uint8_t* out, size_t cap) {
    try {
        Container& c = *static_cast<Container*>(h);
        if (index >= c.tensors.size()) throw Error("tensor index out of range");
        Bytes raw = decode_record(c, c.tensors[index], verify != 0);
        if (raw.size() > cap) throw Error("output buffer too small");
        std::memcpy(out, raw.data(), raw.size());
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

// Decode tensors [first, first+count) with `threads` OpenMP threads (tensors
// in parallel, chunks of a plane in parallel inside: container.rs:1772-1779,
// 1995-2045).  `out` may be null (decode and discard, for timing).  Returns
// the decoded byte total through *decoded and wall seconds through *seconds.
int oracle_container_decode_range(void* h, size_t first, size_t count, int threads, int verify, uint8_t* out, const uint64_t* out_offsets,
                                  uint64_t* decoded, double* seconds) {
    try {
        Container& c = *static_cast<Container*>(h);
        if (first + count > c.tensors.size()) throw Error("tensor range out of bounds");
        if (threads <= 0) threads = int(std::thread::hardware_concurrency());
        int outer = int(std::min<size_t>(size_t(threads), count ? count : 1));
        int inner = std::max(1, threads / outer);
        std::string err;
        std::mutex mu;
        std::atomic<uint64_t> total{0};
        auto t0 = std::chrono::steady_clock::now();
        parallel_for(count, outer, [&](size_t i) {
            try {
                Bytes raw = decode_record(c, c.tensors[first + i], verify != 0, inner);
                if (out) std::memcpy(out + out_offsets[i], raw.data(), raw.size());
                total += raw.size();
            } catch (const std::exception& e) {
                std::lock_guard<std::mutex> g(mu);
                err = e.what();
            }
        });
        auto t1 = std::chrono::steady_clock::now();
        if (!err.empty()) throw Error(err);
        *decoded = total;
        *seconds = std::chrono::duration<double>(t1 - t0).count();
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

// \x89PTWS frame → raw bytes plus a small JSON description.
int oracle_decode_compact(const uint8_t* buf, size_t len, uint8_t** raw, size_t* raw_len, uint8_t** desc, size_t* desc_len) {
    try {
        CompactTensor t = decode_compact(buf, len);
        std::ostringstream o;
        o << "{\"dtype_code\":" << t.dtype_code << ",\"dtype_name\":\"" << t.dtype_name << "\",\"has_shape\":" << (t.has_shape ? "true" : "false") << ",\"shape\":[";
        for (size_t d = 0; d < t.shape.size(); ++d) o << (d ? "," : "") << t.shape[d];
        o << "]}";
        std::string s = o.str();
        *raw = dup(t.raw); *raw_len = t.raw.size();
        Bytes b(s.begin(), s.end());
        *desc = dup(b); *desc_len = b.size();
        return 0;
    } catch (const std::exception& e) { return fail(e); }
}

// Test-only: let Zstd planes of the reference's golden fixtures decode through
// the system libzstd (ZSTD_decompress / ZSTD_isError).  Returns 0 on success.
int oracle_install_zstd(const char* path) {
    void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) { g_err = "cannot load libzstd"; return -1; }
    auto d = reinterpret_cast<ZstdDecompressFn>(dlsym(h, "ZSTD_decompress"));
    auto e = reinterpret_cast<ZstdIsErrorFn>(dlsym(h, "ZSTD_isError"));
    if (!d || !e) { g_err = "libzstd lacks ZSTD_decompress"; return -1; }
    zstd_decompress_hook() = d;
    zstd_is_error_hook() = e;
    return 0;
}

int oracle_num_procs() { return int(std::thread::hardware_concurrency()); }

}  // extern "C"
