// Exact-fp32 SIMT attention kernels (forward and backward).
//
// These serve fp32 tensors, where tensor-core input rounding (TF32 or 16-bit) would not meet
// a 1e-3 tolerance on out / logsumexp.  All products and sums are fp32 FMAs; the softmax
// uses exp2f on scale*log2(e)-scaled scores, the same formulation as the tensor-core path
// (reference math: torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:650-861 and
// fa4_bwd_kernel.mojo:1-44, 810-980).  They are templated on the storage type so the same
// code can also read 16-bit tensors, which the tests use as an on-device cross-check of the
// tcgen05 kernels at sizes where a CPU oracle would take minutes.
//
// Tiling: a 256-thread block owns 64 query rows (forward, dQ) or 64 key rows (dK/dV) and
// walks the other sequence in 64-row tiles staged in shared memory as fp32.  Thread
// (ty, tx) of the 16x16 layout owns rows ty+16i and columns tx+16k, which keeps every
// shared-memory access either a broadcast or bank-conflict free.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "philox.cuh"

namespace b200fa {
namespace {

constexpr int kT = 64;  // tile edge
constexpr float kLog2e = 1.4426950408889634f;

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

template <typename T>
__device__ __forceinline__ const T* row_ptr(const View4& t, int b, int h, int s) {
  return reinterpret_cast<const T*>(t.ptr) + (int64_t)b * t.sb + (int64_t)h * t.sh + (int64_t)s * t.ss;
}
template <typename T>
__device__ __forceinline__ T* row_ptr_mut(const View4& t, int b, int h, int s) {
  return reinterpret_cast<T*>(t.ptr) + (int64_t)b * t.sb + (int64_t)h * t.sh + (int64_t)s * t.ss;
}

// Stage up to kT rows x kD columns into shared memory as fp32 (row stride `ld`); rows past
// `S` are zero.
template <typename T, int kD>
__device__ __forceinline__ void stage_tile(float* dst, int ld, const View4& t, int b, int h, int s0, int S) {
  for (int idx = threadIdx.x; idx < kT * kD; idx += blockDim.x) {
    const int r = idx / kD, c = idx - r * kD;
    const int s = s0 + r;
    dst[r * ld + c] = (s < S) ? to_f32<T>(row_ptr<T>(t, b, h, s)[c]) : 0.f;
  }
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int kD>
constexpr int simt_smem_bytes() {
  // four [kT][kD+1] operand tiles, one [kT][kT+1] score tile, two [kT] row-statistic vectors
  return (4 * kT * (kD + 1) + kT * (kT + 1) + 2 * kT) * 4;
}

// ------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------
template <typename T, int kD>
__global__ void __launch_bounds__(256) fwd_simt_kernel(const FwdParams p) {
  extern __shared__ float sm[];
  float* sQ = sm;                       // [kT][kD+1]
  float* sK = sQ + kT * (kD + 1);       // [kT][kD+1]
  float* sV = sK + kT * (kD + 1);       // [kT][kD]
  float* sP = sV + kT * kD;             // [kT][kT+1]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.x * kT;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const float c = p.scale_log2;

  stage_tile<T, kD>(sQ, kD + 1, p.q, b, h, m0, p.Sq);
  float o[4][kD / 16];
  float mrow[4], lrow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    mrow[i] = -INFINITY;
    lrow[i] = 0.f;
#pragma unroll
    for (int k = 0; k < kD / 16; ++k) o[i][k] = 0.f;
  }
  const bool drop = p.drop.threshold != 0;
  // query row i sees key column j iff j <= i + causal_off
  const int n_end = p.causal ? max(0, min(p.Sk, m0 + kT + p.causal_off)) : p.Sk;
  for (int n0 = 0; n0 < n_end; n0 += kT) {
    __syncthreads();
    stage_tile<T, kD>(sK, kD + 1, p.k, b, hk, n0, p.Sk);
    stage_tile<T, kD>(sV, kD, p.v, b, hk, n0, p.Sk);
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int k = 0; k < 4; ++k) s[i][k] = 0.f;
    for (int d = 0; d < kD; ++d) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sQ[(ty + 16 * i) * (kD + 1) + d];
#pragma unroll
      for (int k = 0; k < 4; ++k) bb[k] = sK[(tx + 16 * k) * (kD + 1) + d];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) s[i][k] = fmaf(a[i], bb[k], s[i][k]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qr = m0 + ty + 16 * i;
      float mx = -INFINITY;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int col = n0 + tx + 16 * k;
        const bool masked = (col >= p.Sk) || (p.causal && col > qr + p.causal_off);
        s[i][k] = masked ? -INFINITY : s[i][k];
        mx = fmaxf(mx, s[i][k]);
      }
      mx = half_warp_max(mx);
      float m_new = fmaxf(mrow[i], mx);
      if (m_new == -INFINITY) m_new = 0.f;
      const float corr = exp2f((mrow[i] - m_new) * c);
      float rs = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float pv = exp2f((s[i][k] - m_new) * c);
        rs += pv;   // the row sum keeps every probability; only what multiplies V is dropped
        const bool kept = !drop || dropout_keep(p.drop, b * p.Hq + h, qr, n0 + tx + 16 * k);
        sP[(ty + 16 * i) * (kT + 1) + tx + 16 * k] = kept ? pv : 0.f;
      }
      rs = half_warp_sum(rs);
      lrow[i] = lrow[i] * corr + rs;
      mrow[i] = m_new;
#pragma unroll
      for (int k = 0; k < kD / 16; ++k) o[i][k] *= corr;
    }
    __syncthreads();
    for (int n = 0; n < kT; ++n) {
      float pv[4], vv[kD / 16];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = sP[(ty + 16 * i) * (kT + 1) + n];
#pragma unroll
      for (int k = 0; k < kD / 16; ++k) vv[k] = sV[n * kD + tx + 16 * k];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) o[i][k] = fmaf(pv[i], vv[k], o[i][k]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qr = m0 + ty + 16 * i;
    if (qr < p.Sq) {
      // a row that saw no key at all (possible under a bottom-right aligned mask) is 0 with lse -inf
      const float inv = lrow[i] > 0.f ? (drop ? p.drop.inv_keep : 1.f) / lrow[i] : 0.f;
      T* orow = row_ptr_mut<T>(p.out, b, h, qr);
#pragma unroll
      for (int k = 0; k < kD / 16; ++k) orow[tx + 16 * k] = from_f32<T>(o[i][k] * inv);
      if (tx == 0)
        p.lse[((int64_t)b * p.Hq + h) * p.Sq + qr] = lrow[i] > 0.f ? mrow[i] * p.scale + logf(lrow[i]) : -INFINITY;
    }
  }
}

// ------------------------------------------------------------------------------------------
// backward, part 1: dK and dV.  One block per (64-row KV tile, kv head, batch); loops over
// the query heads of the group and over query tiles at or below the diagonal.
//   P = exp2(S*c - lse*log2e),  dV += P^T dO,  dS = P * (dP - dpsum),  dK += scale * dS^T Q
// ------------------------------------------------------------------------------------------
template <typename T, int kD>
__global__ void __launch_bounds__(256) bwd_dkdv_simt_kernel(const BwdParams p) {
  extern __shared__ float sm[];
  float* sK = sm;                        // [kT][kD+1]
  float* sV = sK + kT * (kD + 1);        // [kT][kD+1]
  float* sQ = sV + kT * (kD + 1);        // [kT][kD+1]  (row = query)
  float* sdO = sQ + kT * (kD + 1);       // [kT][kD+1]  (row = query)
  float* sP = sdO + kT * (kD + 1);       // [kT][kT+1]  (row = query, col = key): P, then dS
  float* sLse = sP + kT * (kT + 1);      // [kT]
  float* sDps = sLse + kT;               // [kT]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int n0 = blockIdx.x * kT;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const float c = p.scale_log2;
  const bool drop = p.drop.threshold != 0;

  stage_tile<T, kD>(sK, kD + 1, p.k, b, hk, n0, p.Sk);
  stage_tile<T, kD>(sV, kD + 1, p.v, b, hk, n0, p.Sk);
  // thread owns key rows ty+16i and d columns tx+16k of dK/dV
  float dk[4][kD / 16], dv[4][kD / 16];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int k = 0; k < kD / 16; ++k) dk[i][k] = dv[i][k] = 0.f;

  for (int g = 0; g < group; ++g) {
    const int h = hk * group + g;
    const int m_begin = p.causal ? (max(0, n0 - p.causal_off) / kT) * kT : 0;
    for (int m0 = m_begin; m0 < p.S; m0 += kT) {
      __syncthreads();
      stage_tile<T, kD>(sQ, kD + 1, p.q, b, h, m0, p.S);
      stage_tile<T, kD>(sdO, kD + 1, p.dout, b, h, m0, p.S);
      if (threadIdx.x < kT) {
        const int qr = m0 + threadIdx.x;
        float l2 = INFINITY;   // rows past the end, and rows that saw no key (lse = -inf): P = 0
        if (qr < p.S) {
          const float l = p.lse[((int64_t)b * p.Hq + h) * p.S + qr];
          if (l != -INFINITY) l2 = l * kLog2e;
        }
        sLse[threadIdx.x] = l2;
        sDps[threadIdx.x] = (qr < p.S) ? p.dpsum[((int64_t)b * p.Hq + h) * p.Spad + qr] : 0.f;
      }
      __syncthreads();
      // S[q][k] and dP[q][k] for q = ty+16i, k = tx+16j
      float s[4][4], dp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
      for (int d = 0; d < kD; ++d) {
        float qa[4], da[4], kb[4], vb[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          qa[i] = sQ[(ty + 16 * i) * (kD + 1) + d];
          da[i] = sdO[(ty + 16 * i) * (kD + 1) + d];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          kb[j] = sK[(tx + 16 * j) * (kD + 1) + d];
          vb[j] = sV[(tx + 16 * j) * (kD + 1) + d];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            s[i][j] = fmaf(qa[i], kb[j], s[i][j]);
            dp[i][j] = fmaf(da[i], vb[j], dp[i][j]);
          }
      }
      // P and dS; P goes to sP now, dS is kept in registers until dV has consumed P
      float ds[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int ql = ty + 16 * i;
        const int qr = m0 + ql;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kc = n0 + tx + 16 * j;
          const bool masked = (kc >= p.Sk) || (qr >= p.S) || (p.causal && kc > qr + p.causal_off);
          const float pv = masked ? 0.f : exp2f(s[i][j] * c - sLse[ql]);
          // dropout multiplier of this entry: 0 or 1 / (1 - p)
          const float dm = !drop ? 1.f : (dropout_keep(p.drop, b * p.Hq + h, qr, kc) ? p.drop.inv_keep : 0.f);
          ds[i][j] = pv * (dp[i][j] * dm - sDps[ql]);
          sP[ql * (kT + 1) + tx + 16 * j] = pv * dm;
        }
      }
      __syncthreads();
      // dV[k][d] += sum_q P[q][k] dO[q][d]
      for (int q = 0; q < kT; ++q) {
        float pa[4], dob[kD / 16];
#pragma unroll
        for (int i = 0; i < 4; ++i) pa[i] = sP[q * (kT + 1) + ty + 16 * i];
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) dob[k] = sdO[q * (kD + 1) + tx + 16 * k];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int k = 0; k < kD / 16; ++k) dv[i][k] = fmaf(pa[i], dob[k], dv[i][k]);
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sP[(ty + 16 * i) * (kT + 1) + tx + 16 * j] = ds[i][j];
      __syncthreads();
      // dK[k][d] += sum_q dS[q][k] Q[q][d]
      for (int q = 0; q < kT; ++q) {
        float pa[4], qb[kD / 16];
#pragma unroll
        for (int i = 0; i < 4; ++i) pa[i] = sP[q * (kT + 1) + ty + 16 * i];
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) qb[k] = sQ[q * (kD + 1) + tx + 16 * k];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int k = 0; k < kD / 16; ++k) dk[i][k] = fmaf(pa[i], qb[k], dk[i][k]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int kr = n0 + ty + 16 * i;
    if (kr < p.Sk) {
      T* dkrow = row_ptr_mut<T>(p.dk, b, hk, kr);
      T* dvrow = row_ptr_mut<T>(p.dv, b, hk, kr);
#pragma unroll
      for (int k = 0; k < kD / 16; ++k) {
        dkrow[tx + 16 * k] = from_f32<T>(dk[i][k] * p.scale);
        dvrow[tx + 16 * k] = from_f32<T>(dv[i][k]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// backward, part 2: dQ.  One block per (64-row query tile, q head, batch); loops over KV
// tiles up to the diagonal.  dQ = scale * dS K.  Deterministic: no atomics.
// ------------------------------------------------------------------------------------------
template <typename T, int kD>
__global__ void __launch_bounds__(256) bwd_dq_simt_kernel(const BwdParams p) {
  extern __shared__ float sm[];
  float* sQ = sm;                        // [kT][kD+1]  (row = query)
  float* sdO = sQ + kT * (kD + 1);       // [kT][kD+1]  (row = query)
  float* sK = sdO + kT * (kD + 1);       // [kT][kD+1]  (row = key)
  float* sV = sK + kT * (kD + 1);        // [kT][kD+1]  (row = key)
  float* sP = sV + kT * (kD + 1);        // [kT][kT+1]  (row = query, col = key): dS
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.x * kT;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const float c = p.scale_log2;

  stage_tile<T, kD>(sQ, kD + 1, p.q, b, h, m0, p.S);
  stage_tile<T, kD>(sdO, kD + 1, p.dout, b, h, m0, p.S);
  float lse2[4], dps[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qr = m0 + ty + 16 * i;
    lse2[i] = INFINITY;
    if (qr < p.S) {
      const float l = p.lse[((int64_t)b * p.Hq + h) * p.S + qr];
      if (l != -INFINITY) lse2[i] = l * kLog2e;
    }
    dps[i] = (qr < p.S) ? p.dpsum[((int64_t)b * p.Hq + h) * p.Spad + qr] : 0.f;
  }
  float dq[4][kD / 16];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int k = 0; k < kD / 16; ++k) dq[i][k] = 0.f;

  const bool drop = p.drop.threshold != 0;
  const int n_end = p.causal ? max(0, min(p.Sk, m0 + kT + p.causal_off)) : p.Sk;
  for (int n0 = 0; n0 < n_end; n0 += kT) {
    __syncthreads();
    stage_tile<T, kD>(sK, kD + 1, p.k, b, hk, n0, p.Sk);
    stage_tile<T, kD>(sV, kD + 1, p.v, b, hk, n0, p.Sk);
    __syncthreads();
    float s[4][4], dp[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
    for (int d = 0; d < kD; ++d) {
      float qa[4], da[4], kb[4], vb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        qa[i] = sQ[(ty + 16 * i) * (kD + 1) + d];
        da[i] = sdO[(ty + 16 * i) * (kD + 1) + d];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kb[j] = sK[(tx + 16 * j) * (kD + 1) + d];
        vb[j] = sV[(tx + 16 * j) * (kD + 1) + d];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s[i][j] = fmaf(qa[i], kb[j], s[i][j]);
          dp[i][j] = fmaf(da[i], vb[j], dp[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ql = ty + 16 * i;
      const int qr = m0 + ql;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kc = n0 + tx + 16 * j;
        const bool masked = (kc >= p.Sk) || (qr >= p.S) || (p.causal && kc > qr + p.causal_off);
        const float pv = masked ? 0.f : exp2f(s[i][j] * c - lse2[i]);
        const float dm = !drop ? 1.f : (dropout_keep(p.drop, b * p.Hq + h, qr, kc) ? p.drop.inv_keep : 0.f);
        sP[ql * (kT + 1) + tx + 16 * j] = pv * (dp[i][j] * dm - dps[i]);
      }
    }
    __syncthreads();
    // dQ[q][d] += sum_k dS[q][k] K[k][d]
    for (int n = 0; n < kT; ++n) {
      float pa[4], kb[kD / 16];
#pragma unroll
      for (int i = 0; i < 4; ++i) pa[i] = sP[(ty + 16 * i) * (kT + 1) + n];
#pragma unroll
      for (int k = 0; k < kD / 16; ++k) kb[k] = sK[n * (kD + 1) + tx + 16 * k];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) dq[i][k] = fmaf(pa[i], kb[k], dq[i][k]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qr = m0 + ty + 16 * i;
    if (qr < p.S) {
      T* row = row_ptr_mut<T>(p.dq, b, h, qr);
#pragma unroll
      for (int k = 0; k < kD / 16; ++k) row[tx + 16 * k] = from_f32<T>(dq[i][k] * p.scale);
    }
  }
}

// dpsum[b,h,s] = sum_d dO * O (fp32), one warp per row.
template <typename T>
__global__ void dpsum_simt_kernel(const BwdParams p) {
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)p.B * p.Hq * p.S;
  if (warp >= rows) return;
  const int s = (int)(warp % p.S);
  const int h = (int)((warp / p.S) % p.Hq);
  const int b = (int)(warp / ((int64_t)p.S * p.Hq));
  const T* o = row_ptr<T>(p.out, b, h, s);
  const T* d = row_ptr<T>(p.dout, b, h, s);
  float acc = 0.f;
  for (int i = lane; i < p.D; i += 32) acc = fmaf(to_f32<T>(o[i]), to_f32<T>(d[i]), acc);
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) p.dpsum[((int64_t)b * p.Hq + h) * p.Spad + s] = acc;
}

template <typename T, int kD>
cudaError_t launch_fwd_t(const FwdParams& p, cudaStream_t stream) {
  constexpr int smem = simt_smem_bytes<kD>();
  auto kern = fwd_simt_kernel<T, kD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  dim3 grid((p.Sq + kT - 1) / kT, p.Hq, p.B);
  kern<<<grid, 256, smem, stream>>>(p);
  return cudaGetLastError();
}

template <typename T, int kD>
cudaError_t launch_bwd_t(const BwdParams& p, cudaStream_t stream) {
  constexpr int smem = simt_smem_bytes<kD>();
  const int64_t rows = (int64_t)p.B * p.Hq * p.S;
  dpsum_simt_kernel<T><<<(unsigned)((rows * 32 + 255) / 256), 256, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  auto k1 = bwd_dkdv_simt_kernel<T, kD>;
  auto k2 = bwd_dq_simt_kernel<T, kD>;
  e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  const int tiles = (p.S + kT - 1) / kT;
  const int kv_tiles = (p.Sk + kT - 1) / kT;
  k1<<<dim3(kv_tiles, p.Hkv, p.B), 256, smem, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  k2<<<dim3(tiles, p.Hq, p.B), 256, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd_simt(const FwdParams& p, int dtype, cudaStream_t stream, int* launches) {
  cudaError_t e = cudaErrorInvalidValue;
  if (dtype == kF32) e = (p.D == 64) ? launch_fwd_t<float, 64>(p, stream) : launch_fwd_t<float, 128>(p, stream);
  else if (dtype == kBF16)
    e = (p.D == 64) ? launch_fwd_t<__nv_bfloat16, 64>(p, stream) : launch_fwd_t<__nv_bfloat16, 128>(p, stream);
  else if (dtype == kF16)
    e = (p.D == 64) ? launch_fwd_t<__half, 64>(p, stream) : launch_fwd_t<__half, 128>(p, stream);
  if (e == cudaSuccess && launches) *launches += 1;
  return e;
}

cudaError_t launch_bwd_simt(const BwdParams& p, int dtype, cudaStream_t stream, int* launches) {
  cudaError_t e = cudaErrorInvalidValue;
  if (dtype == kF32) e = (p.D == 64) ? launch_bwd_t<float, 64>(p, stream) : launch_bwd_t<float, 128>(p, stream);
  else if (dtype == kBF16)
    e = (p.D == 64) ? launch_bwd_t<__nv_bfloat16, 64>(p, stream) : launch_bwd_t<__nv_bfloat16, 128>(p, stream);
  else if (dtype == kF16)
    e = (p.D == 64) ? launch_bwd_t<__half, 64>(p, stream) : launch_bwd_t<__half, 128>(p, stream);
  if (e == cudaSuccess && launches) *launches += 3;
  return e;
}

}  // namespace b200fa
