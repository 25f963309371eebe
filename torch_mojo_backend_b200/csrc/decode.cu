// Split-KV forward for short query blocks (decode: one or a few new tokens against a long
// key/value cache).  The prefill kernel gives such a problem one 256-row CTA per (batch, head)
// with a handful of useful rows in it; here the key sequence is split over many CTAs so that
// the whole GPU streams K and V, which are read from HBM once per KV head (all query heads of
// a GQA group and all query rows share the pass), and the last CTA of a KV head to finish merges
// the partial softmax results, in the same launch.  The reference serves this case with a separate single-kernel decode path
// (torch_mojo_backend/eager_kernels/aten_fast.py:9171-9203: q_len == 1, kv_len <= 4096, no
// split); the arithmetic is the forward's (fa4_fwd_kernel.mojo:650-861): exp2-domain online
// softmax with c = scale*log2(e), fp32 accumulation, LSE = max*ln2 + ln(sum).
//
// One CTA per (key split, kv head, batch).  Rows r = (query head of the group, query
// row), at most 16 of them.  K and V rows go from global memory straight to registers, coalesced,
// with no shared-memory staging and no block-wide barrier in the loop; the warps' (max, sum, O) are
// merged through shared memory at the end.  HBM-bound by design: 2*Sk*D*sizeof(T) bytes per KV head,
// read once.  Two forms:
//   * 16-bit inputs: splitkv_partial_mma_kernel, four warps, 16 keys a step on the warp-level
//     tensor-core path (described at the kernel);
//   * fp32 inputs: splitkv_partial_kernel, eight warps, at most 8 rows per warp (more: the warps form
//     two groups).  A lane owns D/32 head-dim elements: it holds those of every query row in registers
//     and reads the same elements of each K and V row.  Keys go in blocks of eight, dealt round-robin
//     to the warps: partial dot products per lane, a reduce-scatter over the lanes that leaves lane L
//     with the score of key L mod 8, the online-softmax update on those, probabilities broadcast back
//     by shuffles for O += P V.  About 90 instructions per key and warp at 4 rows: the schedulers, not
//     HBM, bound it (measured with 16-bit inputs before the tensor-core form existed: 0.55 of the copy
//     rate, issue slots 59 % busy).
// The merge (finish_split): one warp per output row combines the splits, writes out and lse.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200fa {
namespace {

constexpr int kKeyBlock = 8;        // keys per step of a warp
constexpr int kWarpsDecode = 8;
constexpr int kThreadsDecode = kWarpsDecode * 32;

template <typename T>
__device__ __forceinline__ T st_f32(float x);
template <>
__device__ __forceinline__ float st_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 st_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half st_f32<__half>(float x) { return __float2half_rn(x); }

// kN consecutive elements (2 or 4) starting at p, as floats, with one vector load
template <typename T, int kN>
__device__ __forceinline__ void load_vec(const T* p, float* out);
template <>
__device__ __forceinline__ void load_vec<float, 4>(const float* p, float* out) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <>
__device__ __forceinline__ void load_vec<float, 2>(const float* p, float* out) {
  const float2 v = *reinterpret_cast<const float2*>(p);
  out[0] = v.x; out[1] = v.y;
}
// The last CTA of a (batch, kv head) to finish merges that head's splits: every CTA publishes its
// partial results (fence), then bumps the head's counter; the one that sees nsplit - 1 owns the
// merge.  No CTA waits for another.
template <typename T, int kD>
__device__ __forceinline__ void finish_split(const SplitKvParams& p, int b, int hk, int rows, int tid, int nthreads) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(p.counters + (int64_t)b * p.Hkv + hk, 1u);
    s_last = prev == static_cast<unsigned>(p.nsplit - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // All rows at once: nthreads / (rows padded to a power of two) threads per row, each with a
  // contiguous slice of the head dimension, so that few loads depend on one another (the merge runs
  // while other CTAs still saturate HBM, and a load takes a while).  The partials were written by
  // other SMs: read them from L2.
  int rows_pad = 1;
  while (rows_pad < rows) rows_pad <<= 1;
  const int tpr = nthreads / rows_pad;           // threads per row: 8 .. 256
  const int rr = tid / tpr, part = tid % tpr;
  if (rr >= rows) return;
  const int group = p.Hq / p.Hkv;
  const int h = hk * group + rr / p.Sq, qi = rr % p.Sq;
  const int64_t row = ((int64_t)b * p.Hq + h) * p.Sq + qi;
  const float2* ml = reinterpret_cast<const float2*>(p.part_ml) + row * p.nsplit;
  float m = -INFINITY;
#pragma unroll 8
  for (int sp = 0; sp < p.nsplit; ++sp) m = fmaxf(m, __ldcg(ml + sp).x);
  const float m_use = (m == -INFINITY) ? 0.f : m;
  T* out = reinterpret_cast<T*>(p.out.ptr) + (int64_t)b * p.out.sb + (int64_t)h * p.out.sh + (int64_t)qi * p.out.ss;
  float l = 0.f;
  if (tpr * 4 <= kD) {
    // 4, 8 or 16 elements per thread, in float4 pieces dealt round-robin to the row's threads
    constexpr int kMaxVec = kD / 4 / 8;            // pieces per thread at 8 threads per row
    const int nvec = kD / 4 / tpr;                 // 1 .. kMaxVec
    float4 o[kMaxVec];
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4* po = reinterpret_cast<const float4*>(p.part_o + row * p.nsplit * kD) + part;
#pragma unroll 4
    for (int sp = 0; sp < p.nsplit; ++sp) {
      const float2 v = __ldcg(ml + sp);
      const float w = exp2f(v.x - m_use);          // 0 for a split that saw no visible key
      l = fmaf(v.y, w, l);
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        if (i < nvec) {
          const float4 x = __ldcg(po + sp * (kD / 4) + i * tpr);
          o[i].x = fmaf(x.x, w, o[i].x); o[i].y = fmaf(x.y, w, o[i].y);
          o[i].z = fmaf(x.z, w, o[i].z); o[i].w = fmaf(x.w, w, o[i].w);
        }
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;     // a row that saw no key at all: 0 with lse -inf
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      if (i < nvec) {
        T* dst = out + (part + i * tpr) * 4;
        dst[0] = st_f32<T>(o[i].x * inv); dst[1] = st_f32<T>(o[i].y * inv);
        dst[2] = st_f32<T>(o[i].z * inv); dst[3] = st_f32<T>(o[i].w * inv);
      }
    }
  } else {
    // more threads than float4 pieces: one or two elements per thread (or none)
    const int per = tpr >= kD ? 1 : kD / tpr;      // 1 or 2
    const int d0 = part * per;
    if (d0 >= kD) return;
    float o0 = 0.f, o1 = 0.f;
    const float* po = p.part_o + row * p.nsplit * kD + d0;
#pragma unroll 4
    for (int sp = 0; sp < p.nsplit; ++sp) {
      const float2 v = __ldcg(ml + sp);
      const float w = exp2f(v.x - m_use);
      l = fmaf(v.y, w, l);
      o0 = fmaf(__ldcg(po + (int64_t)sp * kD), w, o0);
      if (per == 2) o1 = fmaf(__ldcg(po + (int64_t)sp * kD + 1), w, o1);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    out[d0] = st_f32<T>(o0 * inv);
    if (per == 2) out[d0 + 1] = st_f32<T>(o1 * inv);
  }
  if (part == 0) p.lse[row] = l > 0.f ? m * 0.6931471805599453f + logf(l) : -INFINITY;
}

// kR: query rows a warp carries (the rows of the problem padded up to 1, 2, 4 or 8)
template <typename T, int kD, int kR>
__global__ void __launch_bounds__(kThreadsDecode, kR <= 4 ? 2 : 1) splitkv_partial_kernel(const SplitKvParams p) {
  constexpr int kDP = kD / 32;   // head-dim elements per lane
  __shared__ float sMerge[kWarpsDecode][kR][kD + 2];   // per warp and row: O, then max and sum
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int rows = group * p.Sq;                       // <= 16
  const int ngroups = (rows + kR - 1) / kR;            // 1 or 2 groups of warps, kR rows each
  const int wpg = kWarpsDecode / ngroups;              // warps that share a group's rows and split its keys
  const int k_begin = split * p.split_len;
  const int k_end = min(p.Sk, k_begin + p.split_len);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp / wpg, wi = warp - rg * wpg;
  const int r0 = rg * kR;
  const int d0 = lane * kDP;
  constexpr unsigned kFull = 0xffffffffu;

  // this lane's elements of the group's query rows, already multiplied by scale*log2(e)
  float q[kR][kDP];
  int q_limit[kR];   // last key a row sees (causal), or the last key of the split
#pragma unroll
  for (int r = 0; r < kR; ++r) {
    const int rr = r0 + r;
    q_limit[r] = -1;   // a padding row sees nothing
#pragma unroll
    for (int e = 0; e < kDP; ++e) q[r][e] = 0.f;
    if (rr < rows) {
      const int h = hk * group + rr / p.Sq, qi = rr % p.Sq;
      const T* qp = reinterpret_cast<const T*>(p.q.ptr) + (int64_t)b * p.q.sb + (int64_t)h * p.q.sh + (int64_t)qi * p.q.ss + d0;
      load_vec<T, kDP>(qp, q[r]);
#pragma unroll
      for (int e = 0; e < kDP; ++e) q[r][e] *= p.scale_log2;
      q_limit[r] = p.causal ? min(k_end - 1, qi + p.causal_off) : k_end - 1;
    }
  }
  float m[kR], l[kR], o[kR][kDP];
#pragma unroll
  for (int r = 0; r < kR; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int e = 0; e < kDP; ++e) o[r][e] = 0.f;
  }
  const T* kbase = reinterpret_cast<const T*>(p.k.ptr) + (int64_t)b * p.k.sb + (int64_t)hk * p.k.sh + d0;
  const T* vbase = reinterpret_cast<const T*>(p.v.ptr) + (int64_t)b * p.v.sb + (int64_t)hk * p.v.sh + d0;

  // K and V elements of eight keys: sixteen independent loads, no branch among them (a key past the
  // end of the split re-reads the split's last key, and its score is masked in `step`)
  auto load_block = [&](int key0, float (&kf)[kKeyBlock][kDP], float (&vf)[kKeyBlock][kDP]) {
#pragma unroll
    for (int kk = 0; kk < kKeyBlock; ++kk) {
      const int key = min(key0 + kk, k_end - 1);
      load_vec<T, kDP>(kbase + (int64_t)key * p.k.ss, kf[kk]);
      load_vec<T, kDP>(vbase + (int64_t)key * p.v.ss, vf[kk]);
    }
  };
  auto step = [&](int key0, const float (&kf)[kKeyBlock][kDP], const float (&vf)[kKeyBlock][kDP]) {
    const int my_key = key0 + (lane & 7);   // the key whose score this lane ends up with
#pragma unroll
    for (int r = 0; r < kR; ++r) {
      // partial dot products over this lane's head-dim elements, eight keys
      float part[kKeyBlock];
#pragma unroll
      for (int kk = 0; kk < kKeyBlock; ++kk) {
        float2 a2 = __fmul2_rn(make_float2(q[r][0], q[r][1]), make_float2(kf[kk][0], kf[kk][1]));
        if constexpr (kDP == 4) a2 = __ffma2_rn(make_float2(q[r][2], q[r][3]), make_float2(kf[kk][2], kf[kk][3]), a2);
        part[kk] = a2.x + a2.y;
      }
      // reduce-scatter over lane bits 2, 1, 0: lane L keeps key L & 7; then the four groups of eight lanes are summed
      float h4[4], h2[2];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const bool up = lane & 4;
        const float keep = up ? part[kk + 4] : part[kk], send = up ? part[kk] : part[kk + 4];
        h4[kk] = keep + __shfl_xor_sync(kFull, send, 4);
      }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const bool up = lane & 2;
        const float keep = up ? h4[kk + 2] : h4[kk], send = up ? h4[kk] : h4[kk + 2];
        h2[kk] = keep + __shfl_xor_sync(kFull, send, 2);
      }
      float sc;
      {
        const bool up = lane & 1;
        const float keep = up ? h2[1] : h2[0], send = up ? h2[0] : h2[1];
        sc = keep + __shfl_xor_sync(kFull, send, 1);
      }
      sc += __shfl_xor_sync(kFull, sc, 8);
      sc += __shfl_xor_sync(kFull, sc, 16);
      if (my_key > q_limit[r]) sc = -INFINITY;   // masked, past the end, or a padding row
      // online softmax over the eight keys (log2 domain)
      float bm = sc;
      bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, 1));
      bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, 2));
      bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, 4));
      const float m_new = fmaxf(m[r], bm);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;   // nothing visible so far: everything stays zero
      const float pr = exp2f(sc - m_use);
      const float corr = exp2f(m[r] - m_use);                   // 0 on the first block with a visible key
      m[r] = m_new;
      l[r] = l[r] * corr + (lane < 8 ? pr : 0.f);               // every key once (the four lane groups hold copies)
#pragma unroll
      for (int e = 0; e < kDP; ++e) o[r][e] *= corr;
#pragma unroll
      for (int kk = 0; kk < kKeyBlock; ++kk) {
        const float pk = __shfl_sync(kFull, pr, kk);
        const float2 pk2 = make_float2(pk, pk);
#pragma unroll
        for (int e = 0; e < kDP; e += 2) {
          const float2 t = __ffma2_rn(pk2, make_float2(vf[kk][e], vf[kk][e + 1]), make_float2(o[r][e], o[r][e + 1]));
          o[r][e] = t.x;
          o[r][e + 1] = t.y;
        }
      }
    }
  };
  const int stride = wpg * kKeyBlock;
  for (int key0 = k_begin + wi * kKeyBlock; key0 < k_end; key0 += stride) {
    float kf[kKeyBlock][kDP], vf[kKeyBlock][kDP];
    load_block(key0, kf, vf);
    step(key0, kf, vf);
  }
  // this warp's results to shared memory
#pragma unroll
  for (int r = 0; r < kR; ++r) {
    float ls = l[r];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) ls += __shfl_xor_sync(kFull, ls, off);
#pragma unroll
    for (int e = 0; e < kDP; ++e) sMerge[warp][r][d0 + e] = o[r][e];
    if (lane == 0) {
      sMerge[warp][r][kD] = m[r];
      sMerge[warp][r][kD + 1] = ls;
    }
  }
  __syncthreads();
  // merge the warps of a group; partial results of this split go to (B, Hq, Sq, nsplit, D) and (B, Hq, Sq, nsplit, 2)
  for (int idx = tid; idx < ngroups * kR * kD; idx += kThreadsDecode) {
    const int g = idx / (kR * kD), r = (idx / kD) % kR, d = idx % kD;
    const int rr = g * kR + r;
    if (rr >= rows) continue;
    float mm = -INFINITY;
    for (int w = 0; w < wpg; ++w) mm = fmaxf(mm, sMerge[g * wpg + w][r][kD]);
    const float m_use = (mm == -INFINITY) ? 0.f : mm;
    float acc = 0.f, ls = 0.f;
    for (int w = 0; w < wpg; ++w) {
      const float wgt = exp2f(sMerge[g * wpg + w][r][kD] - m_use);
      acc = fmaf(sMerge[g * wpg + w][r][d], wgt, acc);
      ls = fmaf(sMerge[g * wpg + w][r][kD + 1], wgt, ls);
    }
    const int h = hk * group + rr / p.Sq, qi = rr % p.Sq;
    const int64_t row = (((int64_t)b * p.Hq + h) * p.Sq + qi) * p.nsplit + split;
    p.part_o[row * kD + d] = acc;
    if (d == 0) {
      p.part_ml[row * 2] = mm;
      p.part_ml[row * 2 + 1] = ls;
    }
  }
  finish_split<T, kD>(p, b, hk, rows, tid, kThreadsDecode);
}

// ---- 16-bit inputs: the same pass on the warp-level tensor-core path ------------------------------
// For bf16/fp16 the scalar kernel above spends some 90 instructions per key and warp on conversions,
// dot products and shuffles, and the schedulers, not HBM, bound it.  Here a warp takes 16 keys a step
// and computes S^T = K Q^T and O^T += V^T P^T with mma.sync m16n8k16 (fp32 accumulation): keys (then
// head-dim elements) are the M dimension, the query rows the N dimension (8 a tile, kNT tiles), so no
// tensor-core row is padding.  Operands go from global memory to the fragment registers directly:
//   * the contraction index of S^T is the head dimension, and any permutation of it may be used as
//     long as K and Q use the same one.  Thread (g = lane/4, t = lane%4) reads 16 bytes at offset
//     (4i + t) * 16 of key rows g and g+8 (i = 0 .. D/32-1; the four t of a row read 64 contiguous
//     bytes per instruction) and the same bytes of query row g; the two halves of such a 16-byte piece
//     are the two 8-byte fragments of one k16 step.
//   * O^T's M index is a head-dim element.  Thread (g, t) reads 16 bytes at offset 128h + 16g of V
//     rows 2t, 2t+1, 2t+8, 2t+9 (the eight g of a row read 128 contiguous bytes); register q of such
//     a piece holds elements d and d+1 of its key, and a byte permute of the registers of two
//     neighbouring keys makes the (key, key+1) pairs the A fragment wants, for M slot g (element d)
//     and slot g+8 (element d+1) of tile (h, q).
//   * P^T (keys x rows) comes out of the softmax as an accumulator fragment (key g, rows 2t, 2t+1);
//     movmatrix transposes the packed 8x8 tiles into the B fragment (keys 2t, 2t+1; row g).
// A thread owns query rows 2t and 2t+1 of each tile: their running max is reduced over the eight g
// lanes by three shuffles, their sums stay per-thread until the end.  Loads of the next step's K are
// issued as soon as the current K fragments are consumed, V's likewise, so a warp has 16 KB (D=128)
// in flight most of the time.
constexpr int kMmaKeys = 16;
constexpr int kMmaWarps = 4;

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                        uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t reg_of(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// kNT: tiles of eight query rows (1 or 2)
template <typename T, int kD, int kNT>
__global__ void __launch_bounds__(kMmaWarps * 32, kNT == 1 ? 3 : 2) splitkv_partial_mma_kernel(const SplitKvParams p) {
  constexpr int kKL = kD / 32;   // 16-byte pieces of a K (and Q) row per thread
  constexpr int kVL = kD / 64;   // 16-byte pieces of a V row per thread
  constexpr int kRows = 8 * kNT;
  constexpr unsigned kFull = 0xffffffffu;
  __shared__ float sMerge[kMmaWarps][kRows][kD + 2];   // per warp and row: O, then max and sum
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int rows = group * p.Sq;   // <= 8 * kNT
  const int k_begin = split * p.split_len;
  const int k_end = min(p.Sk, k_begin + p.split_len);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;

  // Q^T fragments: query row 8n + g, the bytes this thread also reads of a K row
  uint4 qf[kNT][kKL];
#pragma unroll
  for (int n = 0; n < kNT; ++n) {
    const int rr = 8 * n + g;
#pragma unroll
    for (int i = 0; i < kKL; ++i) qf[n][i] = make_uint4(0, 0, 0, 0);
    if (rr < rows) {
      const int h = hk * group + rr / p.Sq, qi = rr % p.Sq;
      const T* qp = reinterpret_cast<const T*>(p.q.ptr) + (int64_t)b * p.q.sb + (int64_t)h * p.q.sh + (int64_t)qi * p.q.ss;
#pragma unroll
      for (int i = 0; i < kKL; ++i) qf[n][i] = *reinterpret_cast<const uint4*>(qp + (4 * i + t) * 8);
    }
  }
  // rows 2t and 2t+1 of each tile are this thread's in the softmax: the last key each of them sees
  int q_limit[kNT][2];
#pragma unroll
  for (int n = 0; n < kNT; ++n)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int rr = 8 * n + 2 * t + e;
      const int qi = rr % p.Sq;
      q_limit[n][e] = rr >= rows ? -1 : (p.causal ? min(k_end - 1, qi + p.causal_off) : k_end - 1);
    }
  float m[kNT][2], l[kNT][2];
  float o[kNT][kVL * 4][4];   // O^T tiles (h, q): [0] (d, row 2t) [1] (d, row 2t+1) [2] (d+1, row 2t) [3] (d+1, row 2t+1)
#pragma unroll
  for (int n = 0; n < kNT; ++n) {
    m[n][0] = m[n][1] = -INFINITY;
    l[n][0] = l[n][1] = 0.f;
#pragma unroll
    for (int j = 0; j < kVL * 4; ++j) o[n][j][0] = o[n][j][1] = o[n][j][2] = o[n][j][3] = 0.f;
  }
  const T* kbase = reinterpret_cast<const T*>(p.k.ptr) + (int64_t)b * p.k.sb + (int64_t)hk * p.k.sh + t * 8;
  const T* vbase = reinterpret_cast<const T*>(p.v.ptr) + (int64_t)b * p.v.sb + (int64_t)hk * p.v.sh + g * 8;
  const int last = k_end - 1;
  uint4 kf[2][kKL];   // key rows g, g+8
  uint4 vf[4][kVL];   // key rows 2t, 2t+1, 2t+8, 2t+9
  // a key past the end of the split re-reads the split's last key; its score is masked
  auto load_k = [&](int key0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const T* row = kbase + (int64_t)min(key0 + g + 8 * r, last) * p.k.ss;
#pragma unroll
      for (int i = 0; i < kKL; ++i) kf[r][i] = __ldg(reinterpret_cast<const uint4*>(row + i * 32));
    }
  };
  auto load_v = [&](int key0) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const T* row = vbase + (int64_t)min(key0 + 2 * t + (r & 1) + 8 * (r >> 1), last) * p.v.ss;
#pragma unroll
      for (int h = 0; h < kVL; ++h) vf[r][h] = __ldg(reinterpret_cast<const uint4*>(row + h * 64));
    }
  };
  const int stride = kMmaWarps * kMmaKeys;
  int key0 = k_begin + warp * kMmaKeys;
  if (key0 < k_end) {
    load_k(key0);
    load_v(key0);
  }
  for (; key0 < k_end; key0 += stride) {
    // S^T (16 keys x rows): [0] (key g, row 2t) [1] (key g, row 2t+1) [2] (key g+8, row 2t) [3] (key g+8, row 2t+1)
    float s[kNT][4];
#pragma unroll
    for (int n = 0; n < kNT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int i = 0; i < kKL; ++i)
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int n = 0; n < kNT; ++n)
          mma16816<T>(s[n], reg_of(kf[0][i], 2 * half), reg_of(kf[1][i], 2 * half), reg_of(kf[0][i], 2 * half + 1),
                      reg_of(kf[1][i], 2 * half + 1), reg_of(qf[n][i], 2 * half), reg_of(qf[n][i], 2 * half + 1));
    load_k(key0 + stride);
    uint32_t pb[kNT][2];
#pragma unroll
    for (int n = 0; n < kNT; ++n) {
      float corr[2];
      float pr[4];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float s_lo = s[n][e] * p.scale_log2, s_hi = s[n][2 + e] * p.scale_log2;
        if (key0 + g > q_limit[n][e]) s_lo = -INFINITY;   // masked, past the end, or a padding row
        if (key0 + g + 8 > q_limit[n][e]) s_hi = -INFINITY;
        float bm = fmaxf(s_lo, s_hi);
        bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, 4));
        bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, 8));
        bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, 16));
        const float m_new = fmaxf(m[n][e], bm);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;   // nothing visible so far: everything stays zero
        corr[e] = exp2f(m[n][e] - m_use);                         // 0 on the first step with a visible key
        pr[e] = exp2f(s_lo - m_use);
        pr[2 + e] = exp2f(s_hi - m_use);
        m[n][e] = m_new;
        l[n][e] = l[n][e] * corr[e] + pr[e] + pr[2 + e];          // this thread's two keys; summed over g at the end
      }
#pragma unroll
      for (int j = 0; j < kVL * 4; ++j) {
        o[n][j][0] *= corr[0];
        o[n][j][1] *= corr[1];
        o[n][j][2] *= corr[0];
        o[n][j][3] *= corr[1];
      }
      pb[n][0] = movmatrix_trans(pack2<T>(pr[0], pr[1]));   // keys 2t, 2t+1 of row g
      pb[n][1] = movmatrix_trans(pack2<T>(pr[2], pr[3]));   // keys 2t+8, 2t+9 of row g
    }
#pragma unroll
    for (int h = 0; h < kVL; ++h)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t a0 = __byte_perm(reg_of(vf[0][h], q), reg_of(vf[1][h], q), 0x5410);   // element d of keys 2t, 2t+1
        const uint32_t a1 = __byte_perm(reg_of(vf[0][h], q), reg_of(vf[1][h], q), 0x7632);   // element d+1
        const uint32_t a2 = __byte_perm(reg_of(vf[2][h], q), reg_of(vf[3][h], q), 0x5410);   // keys 2t+8, 2t+9
        const uint32_t a3 = __byte_perm(reg_of(vf[2][h], q), reg_of(vf[3][h], q), 0x7632);
#pragma unroll
        for (int n = 0; n < kNT; ++n) mma16816<T>(o[n][h * 4 + q], a0, a1, a2, a3, pb[n][0], pb[n][1]);
      }
    load_v(key0 + stride);
  }
  // this warp's results to shared memory: element d = 64h + 8g + 2q (and d+1) of rows 2t, 2t+1
#pragma unroll
  for (int n = 0; n < kNT; ++n) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float ls = l[n][e];
      ls += __shfl_xor_sync(kFull, ls, 4);
      ls += __shfl_xor_sync(kFull, ls, 8);
      ls += __shfl_xor_sync(kFull, ls, 16);
      const int r = 8 * n + 2 * t + e;
#pragma unroll
      for (int j = 0; j < kVL * 4; ++j) {
        const int d = 64 * (j >> 2) + 8 * g + 2 * (j & 3);
        sMerge[warp][r][d] = o[n][j][e];
        sMerge[warp][r][d + 1] = o[n][j][2 + e];
      }
      if (g == 0) {
        sMerge[warp][r][kD] = m[n][e];
        sMerge[warp][r][kD + 1] = ls;
      }
    }
  }
  __syncthreads();
  // merge the warps; partial results of this split go to (B, Hq, Sq, nsplit, D) and (B, Hq, Sq, nsplit, 2)
  for (int idx = tid; idx < rows * kD; idx += kMmaWarps * 32) {
    const int r = idx / kD, d = idx % kD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) mm = fmaxf(mm, sMerge[w][r][kD]);
    const float m_use = (mm == -INFINITY) ? 0.f : mm;
    float acc = 0.f, ls = 0.f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float wgt = exp2f(sMerge[w][r][kD] - m_use);
      acc = fmaf(sMerge[w][r][d], wgt, acc);
      ls = fmaf(sMerge[w][r][kD + 1], wgt, ls);
    }
    const int h = hk * group + r / p.Sq, qi = r % p.Sq;
    const int64_t row = (((int64_t)b * p.Hq + h) * p.Sq + qi) * p.nsplit + split;
    p.part_o[row * kD + d] = acc;
    if (d == 0) {
      p.part_ml[row * 2] = mm;
      p.part_ml[row * 2 + 1] = ls;
    }
  }
  finish_split<T, kD>(p, b, hk, rows, tid, kMmaWarps * 32);
}

template <typename T, int kD, int kR>
cudaError_t launch_rows(const SplitKvParams& p, cudaStream_t stream) {
  splitkv_partial_kernel<T, kD, kR><<<dim3(p.nsplit, p.Hkv, p.B), kThreadsDecode, 0, stream>>>(p);
  return cudaGetLastError();
}

template <typename T, int kD, int kNT>
cudaError_t launch_mma(const SplitKvParams& p, cudaStream_t stream) {
  splitkv_partial_mma_kernel<T, kD, kNT><<<dim3(p.nsplit, p.Hkv, p.B), kMmaWarps * 32, 0, stream>>>(p);
  return cudaGetLastError();
}

template <typename T, int kD>
cudaError_t launch_t(const SplitKvParams& p, cudaStream_t stream) {
  const int rows = (p.Hq / p.Hkv) * p.Sq;
  if constexpr (sizeof(T) == 2) {
    // 16-bit inputs: the tensor-core kernel, one or two tiles of eight query rows
    return rows <= 8 ? launch_mma<T, kD, 1>(p, stream) : launch_mma<T, kD, 2>(p, stream);
  } else {
    // fp32: rows a warp carries, padded to a power of two, at most 8 (9-16 rows: two groups of warps)
    if (rows <= 1) return launch_rows<T, kD, 1>(p, stream);
    if (rows <= 2) return launch_rows<T, kD, 2>(p, stream);
    if (rows <= 4) return launch_rows<T, kD, 4>(p, stream);
    return launch_rows<T, kD, 8>(p, stream);
  }
}

}  // namespace

cudaError_t launch_fwd_splitkv(const SplitKvParams& p, int dtype, cudaStream_t stream, int* launches) {
  // the per-head counters of finished splits start at zero (a memset node, not a kernel)
  cudaError_t e = cudaMemsetAsync(p.counters, 0, sizeof(unsigned) * p.B * p.Hkv, stream);
  if (e != cudaSuccess) return e;
  e = cudaErrorInvalidValue;
  if (dtype == kF32) e = (p.D == 64) ? launch_t<float, 64>(p, stream) : launch_t<float, 128>(p, stream);
  else if (dtype == kBF16)
    e = (p.D == 64) ? launch_t<__nv_bfloat16, 64>(p, stream) : launch_t<__nv_bfloat16, 128>(p, stream);
  else if (dtype == kF16) e = (p.D == 64) ? launch_t<__half, 64>(p, stream) : launch_t<__half, 128>(p, stream);
  if (e == cudaSuccess && launches) *launches += 1;
  return e;
}

}  // namespace b200fa
