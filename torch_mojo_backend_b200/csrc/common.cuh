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

struct FwdParams {
  View4 q, k, v, out;
  float* lse;        // (B, Hq, Sq) fp32 contiguous
  int B, Hq, Hkv, Sq, Sk, D;
  int causal;
  float scale;       // softmax scale
  float scale_log2;  // scale * log2(e)
  uint32_t* status;  // optional device status word
};

struct BwdParams {
  View4 q, k, v, out, dout, dq, dk, dv;
  const float* lse;  // (B, Hq, S) fp32 contiguous (natural log)
  float* dpsum;      // workspace: (B, Hq, Spad) rowsum(dO * O)
  float* lse_log2;   // workspace: (B, Hq, Spad) lse * log2(e)
  int B, Hq, Hkv, S, Sk, Spad, D;   // S: query rows (Spad: padded to 128); Sk: key rows (== S when causal)
  int causal;
  float scale;
  float scale_log2;
  uint32_t* status;
  int parts;  // bit 0 preprocess, bit 1 dK/dV kernel, bit 2 dQ kernel (7 = the whole backward);
              // bit 3: keep every kernel on the caller's stream (no side stream, nothing created)
};

// dtype tags shared with the C header
constexpr int kF32 = 0, kBF16 = 1, kF16 = 2;

// Launchers implemented in the kernel translation units.  Each returns a cudaError_t and
// adds the number of kernels it enqueued to *launches.
cudaError_t launch_fwd_sm100(const FwdParams& p, int dtype, cudaStream_t stream, int* launches);
cudaError_t launch_fwd_simt(const FwdParams& p, int dtype, cudaStream_t stream, int* launches);
cudaError_t launch_bwd_sm100(const BwdParams& p, int dtype, cudaStream_t stream, int* launches);
cudaError_t launch_bwd_simt(const BwdParams& p, int dtype, cudaStream_t stream, int* launches);

// Encodes a 4-D tiled tensor map over a (B,H,S,D) view of 16-bit elements with a
// {64 x box_rows x 1 x 1} box and 128-byte swizzle.  Returns false if the driver entry
// point is unavailable or the encode fails.
bool encode_map_16bit(CUtensorMap* map, const View4& t, int B, int H, int S, int D, int box_rows, bool bf16);

}  // namespace b200fa
