// Split-KV forward for short query blocks (decode: one or a few new tokens against a long
// key/value cache).  The prefill kernel gives such a problem one 256-row CTA per (batch, head)
// with a handful of useful rows in it; here the key sequence is split over many CTAs so that
// the whole GPU streams K and V, which are read from HBM once per KV head (all query heads of
// a GQA group and all query rows share the pass), and a second kernel merges the partial
// softmax results.  The reference serves this case with a separate single-kernel decode path
// (torch_mojo_backend/eager_kernels/aten_fast.py:9171-9203: q_len == 1, kv_len <= 4096, no
// split); the arithmetic is the forward's (fa4_fwd_kernel.mojo:650-861): exp2-domain online
// softmax with c = scale*log2(e), fp32 accumulation, LSE = max*ln2 + ln(sum).
//
// Kernel 1, one CTA per (key split, kv head, batch): rows r = (query head of the group, query
// row), at most 16 of them.  Per 64-key tile: stage K and V as fp32 in shared memory; scores
// S[r][key] by threads (r, key); one warp per row does the online-softmax update; thread
// (r, d) accumulates O[r][d].  Writes (max, sum, O) per split.
// Kernel 2, one warp per output row: merges the splits, writes out and lse.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200fa {
namespace {

constexpr int kKeys = 64;       // keys per tile
constexpr int kMaxRows = 16;    // query rows (group * Sq) one CTA carries
constexpr int kThreadsDecode = 256;

template <typename T>
__device__ __forceinline__ float ld_f32(const T* p);
template <>
__device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float ld_f32<__half>(const __half* p) { return __half2float(*p); }

template <typename T>
__device__ __forceinline__ T st_f32(float x);
template <>
__device__ __forceinline__ float st_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 st_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half st_f32<__half>(float x) { return __float2half_rn(x); }

template <int kD>
constexpr int decode_smem_bytes() {
  // K tile [64][D+1], V tile [64][D], Q rows [16][D], scores [16][64], per-row max / sum / correction [3][16]
  return (kKeys * (kD + 1) + kKeys * kD + kMaxRows * kD + kMaxRows * kKeys + 3 * kMaxRows) * 4;
}

template <typename T, int kD>
__global__ void __launch_bounds__(kThreadsDecode) splitkv_partial_kernel(const SplitKvParams p) {
  extern __shared__ float sm[];
  float* sK = sm;                          // [64][kD+1]
  float* sV = sK + kKeys * (kD + 1);       // [64][kD]
  float* sQ = sV + kKeys * kD;             // [rows][kD]
  float* sS = sQ + kMaxRows * kD;          // [rows][64]: scores, then probabilities
  float* sM = sS + kMaxRows * kKeys;       // [rows] running max (log2 domain)
  float* sL = sM + kMaxRows;               // [rows] running sum
  float* sC = sL + kMaxRows;               // [rows] correction factor of this tile
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int rows = group * p.Sq;           // <= kMaxRows
  const int k_begin = split * p.split_len;
  const int k_end = min(p.Sk, k_begin + p.split_len);
  const float c = p.scale_log2;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // row r <-> query head hk*group + r / Sq, query row r % Sq
  for (int idx = tid; idx < rows * kD; idx += kThreadsDecode) {
    const int r = idx / kD, d = idx - r * kD;
    const int h = hk * group + r / p.Sq, qi = r % p.Sq;
    const T* q = reinterpret_cast<const T*>(p.q.ptr) + (int64_t)b * p.q.sb + (int64_t)h * p.q.sh + (int64_t)qi * p.q.ss;
    sQ[idx] = ld_f32<T>(q + d);
  }
  if (tid < kMaxRows) {
    sM[tid] = -INFINITY;
    sL[tid] = 0.f;
  }
  // thread (r, d-slot) owns O[r][d] for d = d-slot, d-slot + stride ...: rows * kD accumulators over 256 threads
  constexpr int kAccPerThread = kMaxRows * kD / kThreadsDecode;   // 4 (D=64) or 8 (D=128)
  float acc[kAccPerThread];
#pragma unroll
  for (int i = 0; i < kAccPerThread; ++i) acc[i] = 0.f;

  for (int n0 = k_begin; n0 < k_end; n0 += kKeys) {
    __syncthreads();   // the previous tile's K, V and probabilities are no longer read
    // 16 bytes per load: rows are 16-byte aligned with a unit head_dim stride
    constexpr int kVec = 16 / static_cast<int>(sizeof(T));
    for (int idx = tid; idx < kKeys * (kD / kVec); idx += kThreadsDecode) {
      const int r = idx / (kD / kVec), d = (idx - r * (kD / kVec)) * kVec;
      const int key = n0 + r;
      float kf[kVec], vf[kVec];
      if (key < k_end) {
        const T* kp = reinterpret_cast<const T*>(p.k.ptr) + (int64_t)b * p.k.sb + (int64_t)hk * p.k.sh + (int64_t)key * p.k.ss + d;
        const T* vp = reinterpret_cast<const T*>(p.v.ptr) + (int64_t)b * p.v.sb + (int64_t)hk * p.v.sh + (int64_t)key * p.v.ss + d;
        const uint4 kw = *reinterpret_cast<const uint4*>(kp);
        const uint4 vw = *reinterpret_cast<const uint4*>(vp);
        const T* ke = reinterpret_cast<const T*>(&kw);
        const T* ve = reinterpret_cast<const T*>(&vw);
#pragma unroll
        for (int e = 0; e < kVec; ++e) {
          kf[e] = ld_f32<T>(ke + e);
          vf[e] = ld_f32<T>(ve + e);
        }
      } else {
#pragma unroll
        for (int e = 0; e < kVec; ++e) kf[e] = vf[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < kVec; ++e) {
        sK[r * (kD + 1) + d + e] = kf[e];
        sV[r * kD + d + e] = vf[e];
      }
    }
    __syncthreads();
    // scores, scaled into the log2 domain; masked entries are -inf
    for (int idx = tid; idx < rows * kKeys; idx += kThreadsDecode) {
      const int r = idx / kKeys, kk = idx - r * kKeys;
      const int key = n0 + kk;
      const int qi = r % p.Sq;
      float s = 0.f;
#pragma unroll 8
      for (int d = 0; d < kD; ++d) s = fmaf(sQ[r * kD + d], sK[kk * (kD + 1) + d], s);
      const bool masked = key >= k_end || (p.causal && key > qi + p.causal_off);
      sS[idx] = masked ? -INFINITY : s * c;
    }
    __syncthreads();
    // online softmax: one warp per row (two keys per lane)
    for (int r = warp; r < rows; r += kThreadsDecode / 32) {
      const float s0 = sS[r * kKeys + lane], s1 = sS[r * kKeys + 32 + lane];
      float mx = fmaxf(s0, s1);
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_old = sM[r];
      float m_new = fmaxf(m_old, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;   // a fully masked row so far: keep everything at zero
      const float p0 = exp2f(s0 - m_use), p1 = exp2f(s1 - m_use);
      float sum = p0 + p1;
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float corr = exp2f(m_old - m_use);   // 0 on the first tile that has a visible key
      sS[r * kKeys + lane] = p0;
      sS[r * kKeys + 32 + lane] = p1;
      if (lane == 0) {
        sM[r] = m_new;
        sL[r] = sL[r] * corr + sum;
        sC[r] = corr;
      }
    }
    __syncthreads();
    // O[r][d] = O[r][d] * corr + sum_key P[r][key] V[key][d]
#pragma unroll
    for (int i = 0; i < kAccPerThread; ++i) {
      const int idx = tid + i * kThreadsDecode;
      const int r = idx / kD, d = idx - r * kD;
      if (r < rows) {
        float a = acc[i] * sC[r];
#pragma unroll 8
        for (int kk = 0; kk < kKeys; ++kk) a = fmaf(sS[r * kKeys + kk], sV[kk * kD + d], a);
        acc[i] = a;
      }
    }
  }
  __syncthreads();
  // partial results of this split: (B, Hq, Sq, nsplit, D) and (B, Hq, Sq, nsplit, 2)
#pragma unroll
  for (int i = 0; i < kAccPerThread; ++i) {
    const int idx = tid + i * kThreadsDecode;
    const int r = idx / kD, d = idx - r * kD;
    if (r < rows) {
      const int h = hk * group + r / p.Sq, qi = r % p.Sq;
      const int64_t row = (((int64_t)b * p.Hq + h) * p.Sq + qi) * p.nsplit + split;
      p.part_o[row * kD + d] = acc[i];
    }
  }
  if (tid < rows) {
    const int h = hk * group + tid / p.Sq, qi = tid % p.Sq;
    const int64_t row = (((int64_t)b * p.Hq + h) * p.Sq + qi) * p.nsplit + split;
    p.part_ml[row * 2] = sM[tid];
    p.part_ml[row * 2 + 1] = sL[tid];
  }
}

// one warp per (b, h, query row): merge the splits
template <typename T, int kD>
__global__ void __launch_bounds__(256) splitkv_combine_kernel(const SplitKvParams p) {
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = (int64_t)p.B * p.Hq * p.Sq;
  if (row >= total) return;
  const float* ml = p.part_ml + row * p.nsplit * 2;
  float m = -INFINITY;
  for (int s = 0; s < p.nsplit; ++s) m = fmaxf(m, ml[s * 2]);
  const float m_use = (m == -INFINITY) ? 0.f : m;
  float l = 0.f;
  constexpr int kPerLane = kD / 32;
  float o[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) o[i] = 0.f;
  for (int s = 0; s < p.nsplit; ++s) {
    const float ms = ml[s * 2];
    if (ms == -INFINITY) continue;   // this split saw no visible key
    const float w = exp2f(ms - m_use);
    l += ml[s * 2 + 1] * w;
    const float* po = p.part_o + (row * p.nsplit + s) * kD;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) o[i] = fmaf(po[lane + 32 * i], w, o[i]);
  }
  const int qi = (int)(row % p.Sq);
  const int h = (int)((row / p.Sq) % p.Hq);
  const int b = (int)(row / ((int64_t)p.Sq * p.Hq));
  T* out = reinterpret_cast<T*>(p.out.ptr) + (int64_t)b * p.out.sb + (int64_t)h * p.out.sh + (int64_t)qi * p.out.ss;
  const float inv = l > 0.f ? 1.f / l : 0.f;   // a row that saw no key at all: 0 with lse -inf
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) out[lane + 32 * i] = st_f32<T>(o[i] * inv);
  if (lane == 0) p.lse[row] = l > 0.f ? m * 0.6931471805599453f + logf(l) : -INFINITY;
}

template <typename T, int kD>
cudaError_t launch_t(const SplitKvParams& p, cudaStream_t stream) {
  constexpr int smem = decode_smem_bytes<kD>();
  auto k1 = splitkv_partial_kernel<T, kD>;
  cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  k1<<<dim3(p.nsplit, p.Hkv, p.B), kThreadsDecode, smem, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
  splitkv_combine_kernel<T, kD><<<(unsigned)((rows * 32 + 255) / 256), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd_splitkv(const SplitKvParams& p, int dtype, cudaStream_t stream, int* launches) {
  cudaError_t e = cudaErrorInvalidValue;
  if (dtype == kF32) e = (p.D == 64) ? launch_t<float, 64>(p, stream) : launch_t<float, 128>(p, stream);
  else if (dtype == kBF16)
    e = (p.D == 64) ? launch_t<__nv_bfloat16, 64>(p, stream) : launch_t<__nv_bfloat16, 128>(p, stream);
  else if (dtype == kF16) e = (p.D == 64) ? launch_t<__half, 64>(p, stream) : launch_t<__half, 128>(p, stream);
  if (e == cudaSuccess && launches) *launches += 2;
  return e;
}

}  // namespace b200fa
