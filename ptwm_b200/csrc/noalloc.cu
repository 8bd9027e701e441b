// One extra entry point for callers that are not allowed to allocate device
// memory.  It decodes a single plane payload like
// ptwm_hardware_backend_v1_dispatch_decode_cuda, but everything the kernel
// needs besides the caller's input and output (the work item, the status
// word, and for Order1ScaleAC the state bytes and their cumulative tables)
// lives in one fixed array in device memory that is part of this library's
// image.  Every GPU that loads the library carries that array until the
// process exits.
#include "host_common.hpp"

using namespace ptwm;

// Scratch of the no-allocation entry point.  64 KiB: 256 bytes for the status
// word and the work item, the rest for an Order1ScaleAC state plus its tables
// (up to 62 context rows).  The name below is only a host-side handle for the
// symbol; the device address comes from cudaGetSymbolAddress.
#define PTWM_B200_NOALLOC_SCRATCH_BYTES 65536
static __device__ __align__(256) uint8_t g_noalloc_scratch[PTWM_B200_NOALLOC_SCRATCH_BYTES];

namespace {

std::mutex g_noalloc_mu;
std::map<int, uint8_t*> g_noalloc_ptr;  // device ordinal -> device address of g_noalloc_scratch on that device

// Once per device, with that device current.
int64_t noalloc_scratch_for(int device, uint8_t** out) {
    std::lock_guard<std::mutex> g(g_noalloc_mu);
    auto it = g_noalloc_ptr.find(device);
    if (it == g_noalloc_ptr.end()) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaGetSymbolAddress(g_noalloc_scratch): ") + cudaGetErrorString(e));
        // the decoders need more dynamic shared memory than the default limit; an attribute, not an allocation
        CUDA_TRY(cudaFuncSetAttribute(rans_decode_kernel_t<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rans_smem_bytes(rans_l_entries(255)))));
        CUDA_TRY(cudaFuncSetAttribute(huffman_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, HUF_SMEM));
        CUDA_TRY(cudaFuncSetAttribute(tans_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TANS_SMEM));
        CUDA_TRY(o1sac_allow_shared_tables());
        it = g_noalloc_ptr.emplace(device, static_cast<uint8_t*>(p)).first;
    }
    *out = it->second;
    return 0;
}

}  // namespace

extern "C" int64_t ptwm_b200_decode_plane_noalloc(uint8_t state_format_version, const uint8_t* state_ptr, size_t state_len, const uint8_t* codec_id_ptr,
                                                  size_t codec_id_len, uint64_t in_dev_ptr, size_t in_len, uint64_t out_dev_ptr, size_t out_cap,
                                                  uint32_t device_ordinal, uint64_t stream) {
    if (!codec_id_ptr || codec_id_len != 32) return fail(PTWM_RC_INVALID_INPUT, "codec_id must be a 32-byte canonical id");
    int codec = -1;
    for (const BuiltinId& b : kBuiltins) if (!std::memcmp(b.id, codec_id_ptr, 32)) codec = b.codec;
    if (codec < 0) return fail(PTWM_RC_UNSUPPORTED, "codec id is not one of identity, huffman, rans, tans, order1_scale_ac");
    if ((in_len && !in_dev_ptr) || (out_cap && !out_dev_ptr)) return fail(PTWM_RC_INVALID_INPUT, "null device pointer");
    if (in_len > 0xFFFFFFFFull) return fail(PTWM_RC_UNSUPPORTED, "payload longer than 4 GiB");
    if (!stream) return fail(PTWM_RC_INVALID_INPUT, "pass the stream to run on (1 = the legacy default stream): this entry point creates none");
    DeviceGuard guard{int(device_ordinal)};
    if (guard.err != cudaSuccess) return fail(PTWM_RC_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(guard.err));
    uint8_t* scratch = nullptr;
    int64_t rc = noalloc_scratch_for(int(device_ordinal), &scratch);
    if (rc < 0) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(uintptr_t(stream));

    uint8_t head[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (in_len) {  // tag and length prefix, read in the order of the caller's stream: whatever produced the payload there has finished
        CUDA_TRY(cudaMemcpyAsync(head, reinterpret_cast<const void*>(uintptr_t(in_dev_ptr)), std::min<size_t>(in_len, 8), cudaMemcpyDeviceToHost, st));
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
        detail::classify_chunk(head, uint16_t(codec), ch);
        if (codec == C_O1SAC) check_o1sac(state_ptr, state_len, state_format_version, in_len, decoded, 0);
    } catch (const FormatError& e) { return fail(PTWM_RC_INVALID_INPUT, e.what()); }
    if (!decoded) return 0;
    if (ch.raw) {
        CUDA_TRY(cudaMemcpyAsync(reinterpret_cast<void*>(uintptr_t(out_dev_ptr)), reinterpret_cast<const void*>(uintptr_t(in_dev_ptr + ch.data_off)), decoded,
                                 cudaMemcpyDeviceToDevice, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        return int64_t(decoded);
    }
    // layout of the fixed scratch: [0,4) status, [64, 64+sizeof item) work item, then (Order1ScaleAC) tables and state
    const size_t tables = codec == C_O1SAC ? (state_len - 32) / 512 : 0;
    const size_t work_off = 256, state_off = work_off + align_up(tables * 514, 256), total = state_off + align_up(codec == C_O1SAC ? state_len : 0, 256);
    if (total > PTWM_B200_NOALLOC_SCRATCH_BYTES)
        return fail(PTWM_RC_BUFFER_TOO_SMALL, "Order1ScaleAC state with " + std::to_string(tables - 1) + " context rows needs " + std::to_string(total) +
                                                  " bytes of scratch; the built-in scratch of ptwm_b200_decode_plane_noalloc holds " +
                                                  std::to_string(PTWM_B200_NOALLOC_SCRATCH_BYTES) + " (use ptwm_hardware_backend_v1_dispatch_decode_cuda)");
    DecodeItem it{};
    it.src = make_ref(SP_BLOB, ch.data_off); it.src_len = uint32_t(ch.data_len); it.n = uint32_t(decoded); it.dst = make_ref(SP_OUT, 0);
    it.partner[0] = it.partner[1] = it.partner[2] = REF_NONE; it.state = REF_NONE; it.work = REF_NONE; it.id = 0;
    Bases bases{reinterpret_cast<const uint8_t*>(uintptr_t(in_dev_ptr)), 0, in_len, scratch, reinterpret_cast<uint8_t*>(uintptr_t(out_dev_ptr))};
    if (codec == C_O1SAC) {
        it.state = make_ref(SP_SCRATCH, state_off); it.state_len = uint32_t(state_len); it.state_version = state_format_version; it.row_len = 0;
        it.work = make_ref(SP_SCRATCH, work_off);
        CUDA_TRY(cudaMemcpyAsync(scratch + state_off, state_ptr, state_len, cudaMemcpyHostToDevice, st));
    }
    // the array keeps what the previous call left: the status word must start at zero
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
    if (status) return fail(PTWM_RC_CORRUPT, status_text(status));
    return int64_t(decoded);
}
