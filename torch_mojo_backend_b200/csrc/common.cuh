// Shared declarations between the host entry points (api.cu) and the kernel translation
// units.  Everything here is internal to the library; the public surface is include/b200fa.h.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200fa {

// A validated (B, H, S, D) view: base pointer plus element strides (D stride is 1).
struct View4 {
  void* ptr;
  int64_t sb, sh, ss;
};

// Dropout: element (b, h, i, j) of the attention matrix is kept when its byte of a
// Philox4x32-10 stream keyed by `seed` is >= `threshold` (see philox.cuh); kept probabilities
// are multiplied by `inv_keep` = 1 / (1 - p).  threshold == 0 means no dropout.
struct DropoutParams {
  uint64_t seed;
  uint64_t offset;
  uint32_t threshold;  // 0..255: bytes below it are dropped
  float inv_keep;
};

struct FwdParams {
  View4 q, k, v, out;
  float* lse;        // (B, Hq, Sq) fp32 contiguous
  int B, Hq, Hkv, Sq, Sk, D;
  int causal;        // 0: no mask; otherwise query row i sees key column j iff j <= i + causal_off
  int causal_off;    // 0 (top-left aligned diagonal) or Sk - Sq (bottom-right aligned)
  float scale;       // softmax scale
  float scale_log2;  // scale * log2(e)
  uint32_t* status;  // optional device status word
  int tiles_per_cta;      // forward kernel shape: 0 = chosen by the launcher, 1 or 2 = forced
  long long wait_budget;  // SM cycles any single internal wait may take before the kernel gives up
  DropoutParams drop;
};

struct BwdParams {
  View4 q, k, v, out, dout, dq, dk, dv;
  const float* lse;  // (B, Hq, S) fp32 contiguous (natural log)
  float* dpsum;      // workspace: (B, Hq, Spad) rowsum(dO * O)   (the tensor-core route stores both
  float* lse_log2;   // workspace: (B, Hq, Spad) lse * log2(e)     statistics negated, the SIMT route as is)
  int B, Hq, Hkv, S, Sk, Spad, D;   // S: query rows (Spad: padded to 128); Sk: key rows
  int causal;
  int causal_off;
  float scale;
  float scale_log2;
  uint32_t* status;
  long long wait_budget;
  int parts;  // bit 0 preprocess, bit 1 dK/dV kernel, bit 2 dQ kernel (7 = the whole backward);
              // bit 3: keep every kernel on the caller's stream (no side stream, nothing created)
  DropoutParams drop;
};

// Split-KV forward for short query blocks (decode): partial (max, sum, O) per key split.
struct SplitKvParams {
  View4 q, k, v, out;
  float* lse;
  float* part_o;    // workspace: (B, Hq, Sq, nsplit, D) fp32
  float* part_ml;   // workspace: (B, Hq, Sq, nsplit, 2) fp32: running max (log2 domain), row sum
  unsigned* counters;   // workspace: (B, Hkv) splits finished so far, zeroed before the launch
  int B, Hq, Hkv, Sq, Sk, D;
  int causal, causal_off;
  int nsplit, split_len;   // keys per split (a multiple of 64)
  float scale, scale_log2;
};

// dtype tags shared with the C header
constexpr int kF32 = 0, kBF16 = 1, kF16 = 2;

// Launchers implemented in the kernel translation units.  Each returns a cudaError_t and
// adds the number of kernels it enqueued to *launches.
cudaError_t launch_fwd_sm100(const FwdParams& p, int dtype, cudaStream_t stream, int* launches);
cudaError_t launch_fwd_simt(const FwdParams& p, int dtype, cudaStream_t stream, int* launches);
cudaError_t launch_fwd_splitkv(const SplitKvParams& p, int dtype, cudaStream_t stream, int* launches);
cudaError_t launch_bwd_sm100(const BwdParams& p, int dtype, cudaStream_t stream, int* launches);
cudaError_t launch_bwd_simt(const BwdParams& p, int dtype, cudaStream_t stream, int* launches);
// A one-warp kernel whose only job is to wait, with `budget` SM cycles, on a barrier nobody
// arrives at: exercises the bounded-wait give-up path without touching the attention kernels.
cudaError_t launch_wait_timeout_selftest(uint32_t* status, long long budget, cudaStream_t stream, int* launches);

// Encodes a 4-D tiled tensor map over a (B,H,S,D) view of 16-bit elements with a
// {64 x box_rows x 1 x 1} box and 128-byte swizzle.  Returns false if the driver entry
// point is unavailable or the encode fails.
bool encode_map_16bit(CUtensorMap* map, const View4& t, int B, int H, int S, int D, int box_rows, bool bf16);

}  // namespace b200fa
