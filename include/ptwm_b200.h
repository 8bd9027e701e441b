/* C ABI of libptwm_b200.so — B200 (sm_100a) decode/encode of ptwm containers.
 *
 * Two groups of entry points:
 *
 *  1. The native-extension symbols the reference's loader binds
 *     (crates/ptwm-core/src/flavor/native.rs of khwstolle/ptwm).  Exporting
 *     them makes this library a drop-in `hardware_backend` and `plane_codec`
 *     contribution: one plane payload per call, synchronous.
 *
 *  2. The batched container API (ptwm_b200_*): parse a whole container once on
 *     the host, then decode any subset of its tensors with a few kernel
 *     launches.  This is what the reference's ContainerReader::decode_model /
 *     decode_tensor (crates/ptwm-core/src/container.rs:1766-2196) do on the
 *     CPU, and what ptwm_b200.Decompressor calls.
 *
 * Conventions shared by both groups (native.rs:105-129,634-657): plain
 * pointers and sizes only; device pointers travel as uint64_t; the caller owns
 * every buffer; return values >= 0 mean success (bytes written where that
 * makes sense), negative values are error codes.
 */
#ifndef PTWM_B200_H
#define PTWM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Return codes (native.rs:634-657). */
#define PTWM_RC_INVALID_INPUT      (-1)
#define PTWM_RC_BUFFER_TOO_SMALL   (-2)
#define PTWM_RC_MISSING_CAPABILITY (-3)
#define PTWM_RC_MISSING_NATIVE_DEP (-4)
#define PTWM_RC_UNSUPPORTED        (-5)
#define PTWM_RC_INTERNAL           (-6)
#define PTWM_RC_CUDA               (-7)   /* CUDA runtime error; decoded as InternalError by the reference */
#define PTWM_RC_CORRUPT            (-8)   /* payload failed to decode or an integrity check failed */

/* ---- 1. reference native-extension ABI ---------------------------------- */

/* kind = "hardware_backend".  Replaces HardwareBackendCudaStreamHandleFn
 * (native.rs:112): the library's process-persistent stream for the device,
 * as an integer; 0 = failure. */
uint64_t ptwm_hardware_backend_v1_cuda_stream_handle(uint32_t device_ordinal);

/* Replaces HardwareBackendCudaDispatchDecodeFn (native.rs:130-141).  Decodes
 * one plane payload exactly as stored in a plane record or chunk frame
 * (TAG|len|blob for huffman / rans / tans, bare bytes for identity and
 * order1_scale_ac) from device memory into device memory and returns the
 * decoded byte count.  codec_id is the 32-byte canonical id of a built-in
 * codec (extension/id.rs:21-31).  state_ptr is host memory and is not read
 * when state_len == 0.  Returns after the kernel has completed. */
int64_t ptwm_hardware_backend_v1_dispatch_decode_cuda(uint8_t state_format_version, const uint8_t* state_ptr, size_t state_len,
                                                      const uint8_t* codec_id_ptr, size_t codec_id_len, uint64_t in_dev_ptr, size_t in_len,
                                                      uint64_t out_dev_ptr, size_t out_len, uint32_t device_ordinal);

/* kind = "plane_codec".  Replace PlaneCodecCudaStreamHandleFn / PlaneCodecCudaDecodeFn /
 * PlaneCodecCudaEncodeFn (native.rs:150,163-174,185-197).  encode_cuda turns one plane in
 * device memory into its payload (identity: the bytes; huffman / rans: TAG|len|blob with the
 * reference's raw fallback, byte for byte what codecs/huffman.rs:37-88 and codecs/rans.rs:38-95
 * produce; tans: codecs/tans.rs:39-90).  order1_scale_ac encodes with the state the caller passes
 * (the flat ABI has no way to hand a fitted state back) and answers PTWM_RC_UNSUPPORTED without
 * one.  *needed_out receives the payload size when out_cap is too small
 * (PTWM_RC_BUFFER_TOO_SMALL) and is left untouched otherwise (native.rs:176-184). */
uint64_t ptwm_plane_codec_v1_cuda_stream_handle(uint32_t device_ordinal);
int64_t ptwm_plane_codec_v1_decode_cuda(uint8_t state_format_version, const uint8_t* state_ptr, size_t state_len, const uint8_t* codec_id_ptr,
                                        size_t codec_id_len, uint64_t in_dev_ptr, size_t in_len, uint64_t out_dev_ptr, size_t out_cap,
                                        uint32_t device_ordinal);
int64_t ptwm_plane_codec_v1_encode_cuda(uint8_t state_format_version, const uint8_t* state_ptr, size_t state_len, const uint8_t* codec_id_ptr,
                                        size_t codec_id_len, uint64_t in_dev_ptr, size_t in_len, uint64_t out_dev_ptr, size_t out_cap,
                                        uint64_t* needed_out, uint32_t device_ordinal);

/* Host-buffer pair every plane_codec library must export (PlaneCodecFn /
 * PlaneCodecStatefulFn, native.rs:62-83).  They stage through device 0 and
 * run the same kernels; the flat ABI carries no codec id, so they speak the
 * rANS plane payload (TAG|len|blob), the codec the reference's own decode
 * benchmark forces (benchmarks/decode_throughput.py:41-42). */
int64_t ptwm_plane_codec_v1_encode(const uint8_t* in, size_t in_len, uint8_t* out, size_t out_len);
int64_t ptwm_plane_codec_v1_decode(const uint8_t* in, size_t in_len, uint8_t* out, size_t out_len);
int64_t ptwm_plane_codec_v1_decode_stateful(uint8_t state_version, const uint8_t* state, size_t state_len, const uint8_t* in, size_t in_len,
                                            uint8_t* out, size_t out_cap);

/* ---- 2. batched container API ------------------------------------------- */

typedef struct ptwm_b200_container ptwm_b200_container;
typedef struct ptwm_b200_plan ptwm_b200_plan;

/* Message of the last failure on the calling thread. */
const char* ptwm_b200_last_error(void);

/* BLAKE3 (unkeyed, 32 bytes) of a host buffer: the hash the legacy layout's
 * header holds of its Extension Table (extension/table.rs:136-141) and the
 * derivation of built-in ids (extension/id.rs:21-31).  Host code. */
void ptwm_b200_blake3(const uint8_t* data, size_t len, uint8_t out[32]);
/* XXH64, seed 0, of a host buffer: the hash behind meta_xxh64 (ptwc.rs:144-149), shared-state
 * entries (container.rs:2089) and the `ptwm_bytes_xxhash64` key of a ptwm-shell file
 * (python/ptwm/integrations/_safetensors.py:141-146).  Host code. */
uint64_t ptwm_b200_xxh64(const uint8_t* data, size_t len);

/* Parse a \x89PTWC container or a \x89PTWS frame held in host memory
 * (ContainerReader::open, container.rs:1395-1626; compact.rs:321-405).  The
 * bytes are only read during this call.  A frame opens as a container with one
 * tensor named "_". */
int64_t ptwm_b200_open(const uint8_t* blob, size_t blob_len, ptwm_b200_container** out);
/* ptwm_b200_open for one rank of a multi-GPU load: header, tables and index are
 * read whole, tensor records only for shard `rank` of `world`, a contiguous run
 * of records cut by record bytes (the same cut on every rank; the shards
 * partition the container).  The other tensors are listed with supported = 0
 * and their record size as `compressed`.  Compact layout only; the legacy
 * layout and single frames are read whole. */
int64_t ptwm_b200_open_shard(const uint8_t* blob, size_t blob_len, uint32_t rank, uint32_t world, ptwm_b200_container** out);
void ptwm_b200_close(ptwm_b200_container* c);

typedef struct ptwm_b200_tensor_info {
    const char* name;        /* owned by the container */
    const char* dtype_name;  /* "" when the record stores none */
    uint16_t dtype_code;     /* public dtype code (dtype.rs:25-50) */
    uint8_t ndim;            /* valid when has_shape */
    uint8_t has_shape;
    uint8_t has_hash;        /* record carries an XXH64 payload hash */
    uint8_t has_crc;         /* at least one plane carries a CRC-32 */
    uint8_t supported;       /* 0: uses a chain or codec outside the hot path */
    uint8_t kind;            /* 0 passthrough, 1 16-bit split, 2 32-bit split, 3 fp8 e4m3, 4 fp8 e5m2 */
    uint64_t shape[8];
    uint64_t orig_size;      /* decoded bytes */
    uint64_t compressed;     /* plane payload bytes in the file */
    uint64_t first_byte;     /* file span [first_byte, end_byte) holding the tensor's payload bytes */
    uint64_t end_byte;
    const char* unsupported_reason;
} ptwm_b200_tensor_info;

size_t ptwm_b200_tensor_count(const ptwm_b200_container* c);
int64_t ptwm_b200_tensor_info_get(const ptwm_b200_container* c, size_t index, ptwm_b200_tensor_info* info);

/* Build the launch plan for a subset of tensors (all when indices == NULL).
 * Outputs go into one arena at 256-byte aligned offsets in the order given. */
int64_t ptwm_b200_plan_create(const ptwm_b200_container* c, const uint32_t* indices, size_t n, ptwm_b200_plan** out);
void ptwm_b200_plan_destroy(ptwm_b200_plan* p);
uint64_t ptwm_b200_plan_out_bytes(const ptwm_b200_plan* p);
uint64_t ptwm_b200_plan_scratch_bytes(const ptwm_b200_plan* p);
uint64_t ptwm_b200_plan_out_offset(const ptwm_b200_plan* p, size_t k);   /* arena offset of the k-th planned tensor */
/* File bytes [lo, hi) the plan reads; a caller may keep only that span on the
 * device and pass blob_dev_ptr = span_dev_ptr - lo with blob_first = lo. */
void ptwm_b200_plan_blob_span(const ptwm_b200_plan* p, uint64_t* lo, uint64_t* hi);
/* Algorithmic traffic of one run: compressed payload bytes read, decoded bytes written, kernels launched. */
void ptwm_b200_plan_stats(const ptwm_b200_plan* p, uint64_t* bytes_read, uint64_t* bytes_written, uint32_t* launches);

#define PTWM_B200_VERIFY_CRC  1u   /* check the plane CRC-32s the records carry */
#define PTWM_B200_VERIFY_HASH 2u   /* check the XXH64 payload hashes the records carry */
#define PTWM_B200_NO_SYNC     4u   /* enqueue only; call ptwm_b200_plan_finish later */
#define PTWM_B200_TIME_KERNELS 8u  /* record CUDA events around every launch (read with ptwm_b200_plan_timings) */

/* Decode the planned tensors.  blob_dev_ptr addresses file offset 0 of the
 * container on the device (see ptwm_b200_plan_blob_span), of which bytes
 * [blob_first, blob_first + blob_len) are resident.  stream: a cudaStream_t as
 * integer, 0 = the library's stream for the device (pass cudaStreamLegacy, 1,
 * for the legacy default stream).  Without
 * PTWM_B200_NO_SYNC the call returns after completion with all checks done
 * (ContainerReader::decode_model semantics, container.rs:1766-1780).
 * A plan keeps one set of status words per device: at most one run of a plan
 * may be in flight on a device (finish it before the next run); different
 * plans, or one plan on different devices, run side by side. */
int64_t ptwm_b200_plan_run(ptwm_b200_plan* p, uint64_t blob_dev_ptr, uint64_t blob_first, uint64_t blob_len, uint64_t out_dev_ptr, uint64_t out_cap,
                           uint64_t scratch_dev_ptr, uint64_t scratch_cap, uint32_t flags, uint32_t device_ordinal, uint64_t stream);
/* Copy the plan's work lists to the device now instead of in the first
 * ptwm_b200_plan_run.  The copies are synchronous: a pipeline that enqueues large
 * transfers prepares its plans first, so that no run waits behind them. */
int64_t ptwm_b200_plan_prepare(ptwm_b200_plan* p, uint32_t device_ordinal);
/* The same with the plan's device memory (work lists, status words) supplied by the caller:
 * ptwm_b200_plan_device_bytes bytes at a 256-byte aligned address, which must outlive the plan's
 * runs on that device.  Neither call allocates device memory then (cudaMalloc may wait for queued
 * transfers; a loader that prepares plans beside a streaming copy takes the memory from its own pool).
 * The lists reach the device through a kernel reading pinned host memory, not through the copy
 * engine, so preparing a plan does not wait behind transfers that are already queued. */
uint64_t ptwm_b200_plan_device_bytes(const ptwm_b200_plan* p);
int64_t ptwm_b200_plan_prepare_in(ptwm_b200_plan* p, uint32_t device_ordinal, uint64_t dev_ptr, uint64_t cap);
/* Wait for an enqueued run and evaluate decode status and integrity checks. */
int64_t ptwm_b200_plan_finish(ptwm_b200_plan* p, uint32_t flags, uint32_t device_ordinal, uint64_t stream);


/* ---- 3. encode ------------------------------------------------------------ */

/* One tensor to encode; the bytes are read from device memory. */
typedef struct ptwm_b200_encode_tensor {
    const char* name;
    uint64_t dev_ptr;
    uint64_t nbytes;
    uint64_t shape[8];
    uint16_t dtype_code;     /* public dtype code (dtype.rs:25-50) */
    uint8_t ndim;
    uint8_t usage;           /* 0 standard, 1 block scale (E4M3 / E8M0), 2 fp32 global scale, 3 packed fp4 values:
                                which production chain the tensor gets (python/ptwm/preprocessing/_chains.py:320-357,610-727) */
    uint8_t post_op;         /* one more op between the byte split and one of its terminals (16- and 32-bit float tensors):
                                0 none (or chosen per PTWM_B200_TRY_*), 1 IntDelta, 2 MantissaZeroStrip(post_k)
                                (_chains.py:360-389,486-560) */
    uint8_t post_plane;      /* the plane the op goes on: the exponent plane for IntDelta, mantissa plane 0 for MantissaZeroStrip */
    uint8_t post_k;          /* MantissaZeroStrip: bits stripped, 1..7 */
    uint8_t reserved_;
} ptwm_b200_encode_tensor;

#define PTWM_B200_MENU_IDENTITY 1u
#define PTWM_B200_MENU_HUFFMAN  2u
#define PTWM_B200_MENU_RANS     4u
#define PTWM_B200_MENU_TANS     8u
#define PTWM_B200_MENU_O1SAC    16u   /* offered only to scale planes with a row layout (order1_scale_ac.rs:493-514) */
#define PTWM_B200_CHUNK_NONE    0xFFFFFFFFu   /* chunk_size: write unchunked planes, the reference's default (compressor.rs:112-113) */

typedef struct ptwm_b200_encode_options {
    uint32_t chunk_size;     /* plane bytes per chunk (CompressorOptions.chunk_size, compressor.rs:112-113); 0 = 65536; PTWM_B200_CHUNK_NONE = unchunked */
    uint32_t menu;           /* PTWM_B200_MENU_* bits the per-plane selection may use; 0 = all five */
    int32_t forced_codec;    /* codec wire id to force on every plane (CompressorOptions.forced_codec), -1 = select */
    uint8_t emit_plane_crc;  /* CompressorOptions.emit_plane_crc */
    uint8_t emit_payload_hash; /* CompressorOptions.emit_payload_hash */
    uint8_t candidates;      /* PTWM_B200_TRY_* bits: candidate chains tried beside the plain split for every 16- / 32-bit float tensor
                                without an explicit post_op; the chain with the smallest total wins, the first in the reference's
                                order on ties (pass1_select_chain, compressor.rs:504-665; candidates of _chains.py:1151-1185) */
    uint8_t reserved[1];
} ptwm_b200_encode_options;
#define PTWM_B200_TRY_INTDELTA 1u   /* split + IntDelta on the exponent plane */
#define PTWM_B200_TRY_MZS      2u   /* split + MantissaZeroStrip(k), k = 1..4, on mantissa plane 0 */
#define PTWM_B200_TRY_SHARED_STATE 4u /* whole planes only (chunk_size = PTWM_B200_CHUNK_NONE), codec chosen from the menu: fit shared Order1ScaleAC states over all
                                         scale planes (clusters chosen by description length), write them to the prelude, and let every scale plane code
                                         against one of them when that is smaller (compressor.rs:834-939, fit/order1.rs) */

typedef struct ptwm_b200_encoded ptwm_b200_encoded;

/* compress_model (compressor.rs:972-1200) for the production split / passthrough
 * chains, compact \x89PTWC layout: split + reorder, histograms, table build and
 * stream encoding (identity, huffman, rans, tans, order1_scale_ac) run on the
 * device; the host lays out records, index and footer.  A plane's codec is the
 * one with the smallest state + payload over the menu, first in dispatch order
 * on ties (select.rs:27-64, dispatch.rs:13-49), judged on the whole plane from
 * its histograms; the plane is then written in chunks of chunk_size bytes, or
 * whole (one record payload with an inline state) for PTWM_B200_CHUNK_NONE.
 * The container is left in device memory. */
int64_t ptwm_b200_encode_model(const ptwm_b200_encode_tensor* tensors, size_t n, const ptwm_b200_encode_options* options, uint32_t device_ordinal,
                               uint64_t stream, ptwm_b200_encoded** out);
uint64_t ptwm_b200_encoded_size(const ptwm_b200_encoded* e);
uint64_t ptwm_b200_encoded_device_ptr(const ptwm_b200_encoded* e);
/* Copy the container bytes to host memory. */
int64_t ptwm_b200_encoded_copy(const ptwm_b200_encoded* e, uint8_t* host_dst, size_t cap);
/* Copy the container bytes into another device buffer (same device). */
int64_t ptwm_b200_encoded_copy_to_device(const ptwm_b200_encoded* e, uint64_t dst_dev_ptr, uint64_t cap, uint64_t stream);
/* Codec wire id chosen for plane `plane` of tensor `tensor`, or -1. */
int32_t ptwm_b200_encoded_plane_codec(const ptwm_b200_encoded* e, size_t tensor, size_t plane);
void ptwm_b200_encoded_free(ptwm_b200_encoded* e);

/* ---- 4. decode without allocating ----------------------------------------- */

/* No counterpart in the reference.  Same work and same arguments as
 * ptwm_hardware_backend_v1_dispatch_decode_cuda (one plane payload, device to
 * device, returns the decoded byte count), for callers that may not allocate
 * device memory: a loader that runs after the serving engine has handed all of
 * HBM to its own pool, or inside a sandbox that accounts for every allocation,
 * cannot afford the cudaMalloc the regular entry point does for its per-call
 * scratch.  Here that scratch is a fixed 64 KiB array inside the library's
 * device image (every GPU that loads the library holds it until the process
 * exits), and the call makes no cudaMalloc / cudaFree and creates no stream:
 * `stream` must be given (1 = the legacy default stream).
 *
 * - Limit: identity / huffman / rans / tans payloads of any size fit; an
 *   Order1ScaleAC state fits up to 62 context rows, a larger one is refused with
 *   PTWM_RC_BUFFER_TOO_SMALL and a message naming the limit.
 * - The first call on a device looks the array's address up
 *   (cudaGetSymbolAddress) and raises the kernels' shared-memory limit; make that
 *   first call before any stream capture begins.  Every call waits on `stream`
 *   twice: once to read the payload's tag and length prefix back, once for the
 *   kernel, so it returns with the plane decoded, like the regular entry point.
 * - A payload that fails to decode answers PTWM_RC_CORRUPT.
 * - All calls share the one array.  Its status word is cleared at the start of
 *   each call; two calls that overlap on the same GPU (different streams or
 *   threads) race on it and must be serialised by the caller. */
int64_t ptwm_b200_decode_plane_noalloc(uint8_t state_format_version, const uint8_t* state_ptr, size_t state_len, const uint8_t* codec_id_ptr,
                                       size_t codec_id_len, uint64_t in_dev_ptr, size_t in_len, uint64_t out_dev_ptr, size_t out_cap,
                                       uint32_t device_ordinal, uint64_t stream);

/* Per-launch figures of the last finished run made with PTWM_B200_TIME_KERNELS.
 * Twelve slots: 0-3 first-pass decoders (rANS, Huffman, tANS, Order1ScaleAC),
 * 4 copies to scratch, 5-8 second-pass decoders (fused with the merge where a
 * tensor has several planes), 9 stand-alone merge, 10 plane CRC, 11 XXH64.
 * ms[s] < 0: the slot did not launch.  bytes[s]: algorithmic bytes (compressed
 * and partner bytes read + bytes written) of the slot; items[s]: work items. */
int64_t ptwm_b200_plan_timings(ptwm_b200_plan* p, uint32_t device_ordinal, float* ms, uint64_t* bytes, uint32_t* items);

/* CRC-32 computed the way the verification kernel does it (per-run remainders,
 * GF(2) shifts, XOR fold), on the host, for testing that arithmetic without a GPU. */
uint32_t ptwm_b200_crc32_by_runs(const uint8_t* data, size_t len, size_t run);

/* The shared-state fit of the encoder (PTWM_B200_TRY_SHARED_STATE) on planes in host memory, with the pairwise
 * distances of the GPU kernel computed by the same arithmetic in a host loop: for testing the counting, the states,
 * the clustering and the choice of the cluster count without a GPU (fit/order1.rs).  planes[k] has lens[k] bytes in
 * rows of row_lens[k].  Returns the number of shared states (0..8); their serialized bytes are written back to back to
 * `out` and their lengths to state_lens[0..]; -2 when `cap` is too small. */
int64_t ptwm_b200_fit_shared_states_host(const uint8_t* const* planes, const uint64_t* lens, const uint32_t* row_lens, size_t n, uint8_t* out, size_t cap,
                                         uint32_t state_lens[8]);

#ifdef __cplusplus
}
#endif
#endif /* PTWM_B200_H */
