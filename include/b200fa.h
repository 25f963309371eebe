/*
 * b200fa — C ABI of the B200 (sm_100a) flash-attention library.
 *
 * This is the native boundary behind aten::_scaled_dot_product_flash_attention and
 * aten::_scaled_dot_product_flash_attention_backward on the `mojo` PyTorch device.  It takes
 * the place of the reference's CPython bridge functions, which receive raw device addresses,
 * sizes and a scale as positional integers/floats:
 *   forward : torch_mojo_backend/eager_flash_attention/fa4_ops.mojo:61-102 (dense),
 *             :428-449 (strided q/k/v), :666-744 (BHSD)
 *   backward: torch_mojo_backend/eager_flash_attention/fa4_ops.mojo:158-226
 *   call sites: torch_mojo_backend/eager_kernels/aten_fast.py:7216-7281 and :7325-7399
 *
 * Conventions
 *   - Every pointer is a DEVICE address (except `status_word`, also a device address, and the
 *     descriptor structs themselves, which are host memory).
 *   - Tensors are described in logical (B, H, S, D) order with strides in ELEMENTS, so dense
 *     BHSD tensors, BTHD-stored transposed views and fused-QKV gapped views all go through
 *     the same entry point without a copy.  The D stride must be 1.
 *   - The library never allocates or frees device memory and never synchronises; work is
 *     enqueued on `stream` (a cudaStream_t; NULL = the legacy default stream).
 *   - All arguments are validated before anything is launched.  Functions return 0 on
 *     success or a negative B200FA_ERR_* code; no C++ exception crosses this boundary.
 *   - `status_word` (optional, may be NULL) points to a zero-initialised uint32 in device
 *     memory.  A kernel whose internal wait exceeded its budget writes a non-zero code there
 *     and finishes early instead of hanging; the caller reads it after synchronising.
 */
#ifndef B200FA_H_
#define B200FA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200FA_VERSION 2

/* element types */
#define B200FA_F32 0
#define B200FA_BF16 1
#define B200FA_F16 2

/* error codes */
#define B200FA_OK 0
#define B200FA_ERR_BAD_DTYPE (-1)
#define B200FA_ERR_BAD_SHAPE (-2)
#define B200FA_ERR_BAD_STRIDE (-3)
#define B200FA_ERR_MISALIGNED (-4)
#define B200FA_ERR_WORKSPACE (-5)
#define B200FA_ERR_UNSUPPORTED (-6)
#define B200FA_ERR_CUDA (-7)
#define B200FA_ERR_NULL (-8)
#define B200FA_ERR_TIMEOUT (-9)

/* causal argument of every entry point: query row i sees key column j iff
 *   B200FA_CAUSAL_NONE          always
 *   B200FA_CAUSAL_TOP_LEFT      j <= i                 (torch's is_causal on the CPU / math SDPA paths)
 *   B200FA_CAUSAL_BOTTOM_RIGHT  j <= i + (Sk - Sq)     (the reference kernels' convention,
 *                               torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:266-273)
 * The two coincide when Sq == Sk.  A query row that sees no key at all (possible when
 * Sq > Sk under the bottom-right rule) gets out = 0, lse = -inf and zero gradients. */
#define B200FA_CAUSAL_NONE 0
#define B200FA_CAUSAL_TOP_LEFT 1
#define B200FA_CAUSAL_BOTTOM_RIGHT 2

/* A 4-D tensor view in logical (batch, head, sequence, head_dim) order; strides in elements. */
typedef struct b200fa_tensor4 {
  void* ptr;
  int64_t shape[4];
  int64_t stride[4];
} b200fa_tensor4;

/*
 * Forward: out = softmax(scale * q k^T [+ causal mask]) v,  lse = logsumexp of the scaled,
 * masked scores (natural log), fp32, contiguous (B, Hq, Sq).
 *   q, out : (B, Hq, Sq, D);  k, v : (B, Hkv, Sk, D) with Hq % Hkv == 0 (query head h reads
 *   key/value head h / (Hq / Hkv));  D in {64, 128};  any Sq, Sk, masked or not (the reference's
 *   gate needs Sq == Sk, aten_fast.py:7029-7030); `causal` is one of B200FA_CAUSAL_*.
 *   dtype  : B200FA_BF16 / B200FA_F16 run the tcgen05 tensor-core kernel,
 *            B200FA_F32 runs an exact-fp32 SIMT kernel.
 * Replaces flash_attention_fwd_<dtype>_d<D>_causal{,_strided_qkv,_bhsd}
 * (torch_mojo_backend/eager_flash_attention/fa4_ops.mojo:61-102, 428-449, 666-744).
 */
int b200fa_fwd(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
               const b200fa_tensor4* out, float* lse, int dtype, int causal, float scale,
               void* stream, int device, uint32_t* status_word);

/*
 * Scratch bytes b200fa_bwd needs for a problem of this size: two fp32 per-row statistic
 * arrays, (B, Hq, ceil(S/128)*128) each.  The reference allocates the same two arrays plus an
 * fp32 dQ accumulator (torch_mojo_backend/eager_kernels/aten_fast.py:7314-7324); this library
 * keeps the dQ accumulator in tensor memory instead.
 */
size_t b200fa_bwd_workspace_bytes(int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seqlen,
                                  int64_t head_dim, int dtype);

/*
 * Backward: given dout and the forward's out/lse, writes dq (B,Hq,Sq,D) and dk, dv (B,Hkv,Sk,D);
 * `seqlen` of b200fa_bwd_workspace_bytes is Sq.
 * `workspace` is caller-owned device scratch of at least b200fa_bwd_workspace_bytes(...)
 * bytes, 256-byte aligned; its contents on entry are irrelevant (the library clears what it
 * needs on `stream`).
 * Everything is ordered on `stream`: work enqueued before the call is seen, work enqueued
 * after it sees dq, dk and dv.  For causal 16-bit problems one of the kernels runs on a side
 * stream of a small per-device pool the library keeps (picked by the value of `stream`), forked
 * from and joined back into `stream` with events (this also works inside stream capture); a
 * side stream and its two events are created at the first call that picks them, so make that
 * call outside capture.
 * Replaces flash_attention_bwd_<dtype>_d<D>_causal{,_strided_qkv}
 * (torch_mojo_backend/eager_flash_attention/fa4_ops.mojo:158-226).
 */
int b200fa_bwd(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
               const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
               const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv,
               void* workspace, size_t workspace_bytes, int dtype, int causal, float scale,
               void* stream, int device, uint32_t* status_word);

/*
 * Forward and backward with dropout on the attention probabilities.  Element (b, h, i, j) is
 * kept when its byte of a Philox4x32-10 stream keyed by (philox_seed, philox_offset) is
 * >= b200fa_dropout_threshold(dropout_p) = round(256 p) (at most 255): the drop probability is
 * quantised to threshold/256 and kept probabilities are scaled by 256/(256 - threshold).  The
 * logsumexp is that of the undropped scores.  Counter layout: key = seed; counter =
 * (j / 16, i, low and high word of philox_offset + b*Hq + h); byte 4*w + r of the call (word w,
 * byte r from the low end) belongs to column 16*(j/16) + 4*w + r.  One forward consumes B*Hq
 * consecutive offsets; the backward must be given the same (dropout_p, seed, offset).
 * `exact_fp32` != 0 runs the exact-fp32 SIMT kernels (cross-checks).  dropout_p == 0 is
 * b200fa_fwd / b200fa_bwd.  The reference reserves the (seed, offset) pair on the host
 * (torch_mojo_backend/mojo_device/torch_mojo_device_module.py:84-99) and returns placeholder
 * slots for it (torch_mojo_backend/eager_kernels/aten_fast.py:7726-7734); no reference kernel
 * consumes it.
 */
int b200fa_fwd_dropout(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                       const b200fa_tensor4* out, float* lse, int dtype, int causal, float scale,
                       float dropout_p, uint64_t philox_seed, uint64_t philox_offset, int exact_fp32,
                       void* stream, int device, uint32_t* status_word);
int b200fa_bwd_dropout(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                       const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
                       const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv,
                       void* workspace, size_t workspace_bytes, int dtype, int causal, float scale,
                       float dropout_p, uint64_t philox_seed, uint64_t philox_offset, int exact_fp32,
                       void* stream, int device, uint32_t* status_word);
uint32_t b200fa_dropout_threshold(float dropout_p);
/* Host-side evaluation of the same stream: the 16 bytes of key columns [16*col_block,
 * 16*col_block + 16) of query row `row` of head `batch_head` = b*Hq + h (tests; no device work). */
void b200fa_dropout_bytes_host(uint64_t philox_seed, uint64_t philox_offset, int64_t batch_head, int64_t row,
                               int64_t col_block, uint8_t* out16);

/*
 * Forward for short query blocks against a long key/value sequence (decode): the key sequence
 * is split over many thread blocks, each streams its share of K and V once for every query
 * head of the GQA group and every query row, and the last block of a KV head to finish merges
 * the partial softmax results (one kernel launch, preceded by a memset of the workspace's
 * counters on the same stream).  Needs (Hq / Hkv) * Sq <= B200FA_SPLITKV_MAX_ROWS; any dtype; same out / lse
 * contract as b200fa_fwd.  `workspace`: b200fa_fwd_splitkv_workspace_bytes(...) bytes of
 * caller-owned device scratch, 256-byte aligned (fp32 partial outputs and (max, sum) pairs per
 * split, one counter per KV head); calls that overlap on the GPU need workspaces of their own.  Takes the place of the reference's single-kernel decode path
 * (torch_mojo_backend/eager_kernels/aten_fast.py:9171-9203: q_len == 1, kv_len <= 4096).
 */
#define B200FA_SPLITKV_MAX_ROWS 16
size_t b200fa_fwd_splitkv_workspace_bytes(int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seqlen_q,
                                          int64_t seqlen_k, int64_t head_dim);
int b200fa_fwd_splitkv(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                       const b200fa_tensor4* out, float* lse, void* workspace, size_t workspace_bytes,
                       int dtype, int causal, float scale, void* stream, int device,
                       uint32_t* status_word);

/*
 * b200fa_bwd for callers that cannot allocate device memory.  (No counterpart in the
 * reference, whose Python host allocates the scratch tensors itself.)
 *
 * Who needs it: a host that only passes through device pointers owned by some other runtime
 * and has no CUDA allocator to ask for scratch; a backward that runs on a thread where the
 * framework's allocator must not be re-entered; a serving loop that bans allocation once it
 * is warm.  Instead of a workspace argument, the scratch (the per-row statistics of the
 * backward) lives in a fixed array compiled into the library, B200FA_NO_ALLOC_SCRATCH_BYTES
 * (8 MiB) per GPU, held by every GPU that loads the library until the process exits.
 *
 *   - Problems whose b200fa_bwd_workspace_bytes(...) exceeds that size are refused with
 *     B200FA_ERR_WORKSPACE (b200fa_last_error_detail() says how much was needed); nothing is
 *     launched.  8 MiB covers B*Hq*ceil(S/128)*128 up to 1,048,576 rows (GPT-2-small
 *     attention, B=8 H=12 S=1024, needs 0.8 MB; B=4 Hq=32 S=4096 needs 4 MB).
 *   - The call makes no cudaMalloc / cudaFree and calls no allocating routine.  The first
 *     call on each device looks up the array's device address (cudaGetSymbolAddress with that
 *     device current) and caches it; make that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the previous call
 *     left there.  Nothing in it has to start at zero: the preprocess kernel overwrites every
 *     element the other kernels read, on `stream`, before they run.  Because the array is shared, two calls whose
 *     kernels can overlap on the GPU (different streams, or different host threads without
 *     ordering between them) race on it: serialise them on one stream or with events.
 *   - Inputs, outputs, return codes and numerics are those of b200fa_bwd.
 */
#define B200FA_NO_ALLOC_SCRATCH_BYTES (8u << 20)
int b200fa_bwd_no_alloc(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                        const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
                        const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv,
                        int dtype, int causal, float scale, void* stream, int device,
                        uint32_t* status_word);

/* B200FA_NO_ALLOC_SCRATCH_BYTES as the loaded library was built with. */
size_t b200fa_no_alloc_scratch_bytes(void);

/*
 * Same contracts as b200fa_fwd / b200fa_bwd, but always run the exact-fp32 SIMT kernels
 * whatever the storage type (16-bit inputs are widened to fp32 on load).  They exist so the
 * tensor-core kernels can be cross-checked on the device at sizes where a CPU comparison
 * would take minutes; they have no counterpart in the reference.
 */
int b200fa_fwd_simt(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                    const b200fa_tensor4* out, float* lse, int dtype, int causal, float scale,
                    void* stream, int device, uint32_t* status_word);
int b200fa_bwd_simt(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                    const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
                    const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv,
                    void* workspace, size_t workspace_bytes, int dtype, int causal, float scale,
                    void* stream, int device, uint32_t* status_word);

/*
 * b200fa_bwd restricted to a subset of its three kernels, for timing one kernel alone with
 * CUDA events: `parts` is a bit mask, 1 = preprocess, 2 = the dK/dV tensor-core kernel,
 * 4 = the dQ tensor-core kernel (7 == b200fa_bwd).  16-bit dtypes only.  Results are only meaningful when
 * the parts are run in order; it has no counterpart in the reference.
 */
int b200fa_bwd_parts(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                     const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
                     const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv,
                     void* workspace, size_t workspace_bytes, int dtype, int causal, float scale,
                     void* stream, int device, uint32_t* status_word, int parts);

/*
 * Bounded waits.  Every wait inside the tensor-core kernels gives up after a budget of SM
 * cycles (default about 2 s; environment variable B200FA_WAIT_BUDGET, or this setter; 0 restores
 * the default), writes 0x5741xxxx (xxxx = where it gave up) to the status word and lets the
 * kernel finish; later thread blocks that see a non-zero status word leave at once.
 * b200fa_status_to_error maps a status word read back from the device to B200FA_OK or
 * B200FA_ERR_TIMEOUT.  b200fa_selftest_wait_timeout launches a one-warp kernel whose only job
 * is to wait `budget_cycles` on a barrier nobody arrives at, so the give-up path can be tested
 * without disturbing an attention kernel.  No counterpart in the reference.
 */
void b200fa_set_wait_budget(long long cycles);
long long b200fa_wait_budget(void);
int b200fa_status_to_error(uint32_t status_value);
int b200fa_selftest_wait_timeout(uint32_t* status_word, long long budget_cycles, void* stream, int device);

/*
 * Shape of the tensor-core forward kernel: 2 = one thread block per SM with two 128-row query
 * tiles, 1 = two thread blocks per SM with one query tile each, 0 = chosen per problem (one tile
 * at head dimension 64, two at 128; the default; environment variable B200FA_FWD_TILES).  Both
 * shapes compute the same values; the setter exists for tests and measurements.  No counterpart
 * in the reference.
 */
void b200fa_set_fwd_tiles(int tiles);
int b200fa_fwd_tiles(void);

/* Human-readable text for a B200FA_ERR_* code (static storage). */
const char* b200fa_strerror(int code);

/* Name and text of the CUDA error behind the calling thread's most recent B200FA_ERR_CUDA
 * (thread-local static storage; empty if none). */
const char* b200fa_last_error_detail(void);

/* B200FA_VERSION the library was built from. */
int b200fa_version(void);

/* Number of kernels the library has launched in this process (test/bench accounting; the
 * reference counts bridge calls the same way, torch_mojo_backend/testing.py:32-136). */
uint64_t b200fa_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B200FA_H_ */
