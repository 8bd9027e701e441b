// Helpers shared by the translation units of libptwm_b200.so: error string,
// CUDA error macro, device guard and the per-device persistent state.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/ptwm_b200.h"
#include "kernels.cuh"

namespace ptwm {

// Last error of the calling thread (returned by ptwm_b200_last_error).
std::string& last_error_ref();
inline int64_t fail(int64_t rc, const std::string& m) { last_error_ref() = m; return rc; }

#define CUDA_TRY(expr)                                                                                        \
    do {                                                                                                      \
        cudaError_t e_ = (expr);                                                                              \
        if (e_ != cudaSuccess) return ::ptwm::fail(PTWM_RC_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e_)); \
    } while (0)

// Makes `dev` current for the scope and restores the previous device.
struct DeviceGuard {
    int prev = -1;
    cudaError_t err;
    explicit DeviceGuard(int dev) { err = cudaGetDevice(&prev); if (err == cudaSuccess && prev != dev) err = cudaSetDevice(dev); }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

struct DeviceState {
    cudaStream_t stream = nullptr;   // the library's process-persistent stream for the device
    CrcTables* d_tabs = nullptr;     // CRC byte table and x^(2^k) powers
    bool attrs = false;
    void* stage = nullptr;           // pinned host buffer the plan work lists pass through on their way to the device
    size_t stage_cap = 0;
};

// Caller holds a DeviceGuard for `dev`.
int64_t device_state(int dev, DeviceState** out);
const CrcTables& crc_tables();

inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// One plane into one payload on the device (encoder.cu); body of ptwm_plane_codec_v1_encode_cuda.
int64_t encode_plane_cuda(int codec, const uint8_t* state, size_t state_len, uint8_t state_version, uint64_t in_dev, size_t n, uint64_t out_dev, size_t out_cap,
                          uint64_t* needed, cudaStream_t st);

}  // namespace ptwm
