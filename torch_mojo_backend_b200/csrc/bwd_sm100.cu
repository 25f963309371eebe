// Backward flash attention for sm_100a: preprocess, a dK/dV/dQ tcgen05 pipeline, and the
// fp32 -> 16-bit dQ conversion.
//
// Math (same as the reference's three backward kernels,
// torch_mojo_backend/eager_flash_attention/fa4_bwd_kernel.mojo:1-44, 810-980, 1443-1444,
// 1634-1662, 1855), with c = scale*log2(e):
//   dpsum = rowsum(dO * O)                      (preprocess; also lse2 = lse*log2(e))
//   S^T   = K Q^T          dP^T = V dO^T        (tensor core, transposed so that ...)
//   P^T   = exp2(S^T*c - lse2)                  (... P^T / dS^T land in TMEM as A operands)
//   dV   += P^T dO         dS^T = P^T * (dP^T - dpsum)
//   dK   += dS^T Q         dQ  += dS K          (dQ accumulated in fp32 global memory)
//   dK *= scale (epilogue), dQ *= scale (convert kernel)
//
// One CTA owns one 128-row K/V tile of one (batch, kv head) and walks every query tile at
// or below the causal diagonal, for every query head of the GQA group, so dK and dV
// accumulate in tensor memory without atomics.
//
//   warps 0-3   compute, query columns 0-63 of each S^T / dP^T tile  (thread <-> key row)
//   warps 4-7   compute, query columns 64-127
//   warps 8-11  dQ drain: TMEM -> red.global.add.f32 into the fp32 accumulator
//   warp  12    MMA issuer          warp 13   TMA producer        warps 14-15 idle
//
// TMEM columns: [0,128) S^T, overwritten in place by 16-bit P^T; [128,256) dP^T, overwritten
// by 16-bit dS^T and then by the dQ accumulator; dV and dK after that.
#include "common.cuh"
#include "ptx.cuh"

#ifdef B200FA_TRACE
#define TRACE(role, ev)                                                                          \
  do {                                                                                           \
    if (p.status != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 &&          \
        (threadIdx.x & 31) == 0 && trace_n < 2000) {                                             \
      reinterpret_cast<unsigned long long*>(p.status + 16)[(role) * 2048 + trace_n++] =          \
          (static_cast<unsigned long long>(clock64()) << 8) | (ev);                              \
    }                                                                                            \
  } while (0)
#else
#define TRACE(role, ev) do {} while (0)
#endif

namespace b200fa {
namespace {

constexpr int kTile = 128;
constexpr int kThreads = 512;
constexpr int kSubTileBytes = 128 * 128;

template <int kD>
struct BwdCfg {
  static constexpr int kTileBytes = kTile * kD * 2;
  static constexpr int kSub = kD / 64;
  static constexpr int kStages = 2;
  static constexpr int kTmemS = 0, kTmemDP = 128, kTmemDV = 256, kTmemDK = 256 + kD;
  // D=128 has no spare columns, so dQ re-uses the dP columns; D=64 gives it its own
  static constexpr int kTmemDQ = (kD == 128) ? kTmemDP : (256 + 2 * kD);
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTileBytes;
  static constexpr int kOffQ = 2 * kTileBytes;
  static constexpr int kOffDO = kOffQ + kStages * kTileBytes;
  static constexpr int kOffDS = kOffDO + kStages * kTileBytes;
  static constexpr int kOffStat = kOffDS + 128 * 128 * 2;         // [stage][lse2|dpsum][128] fp32
  static constexpr int kOffBars = kOffStat + kStages * 2 * 128 * 4;
  static constexpr int kNumBars = 1 + 3 * kStages + 7;
  static constexpr int kSmemBytes = kOffBars + kNumBars * 8 + 16;
};

template <int kD, bool kBf16, bool kCausal>
__global__ void __launch_bounds__(kThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
           const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
           const BwdParams p) {
  using Cfg = BwdCfg<kD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem + Cfg::kOffK;
  uint8_t* sV = smem + Cfg::kOffV;
  uint8_t* sQ = smem + Cfg::kOffQ;
  uint8_t* sDO = smem + Cfg::kOffDO;
  uint8_t* sDS = smem + Cfg::kOffDS;
  float* sStat = reinterpret_cast<float*>(smem + Cfg::kOffStat);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* kv_full = bars;                       // [1]
  uint64_t* q_full = kv_full + 1;                 // [kStages]  Q tile + lse2
  uint64_t* do_full = q_full + Cfg::kStages;      // [kStages]  dO tile + dpsum
  uint64_t* qdo_empty = do_full + Cfg::kStages;   // [kStages]
  uint64_t* s_full = qdo_empty + Cfg::kStages;    // S^T ready
  uint64_t* dp_full = s_full + 1;                 // dP^T ready
  uint64_t* p_full = dp_full + 1;                 // P^T written (8 warp arrivals)
  uint64_t* ds_full = p_full + 1;                 // dS^T written (8 warp arrivals)
  uint64_t* dq_full = ds_full + 1;                // dQ tile ready
  uint64_t* dq_empty = dq_full + 1;               // dQ tile drained (4 warp arrivals)
  uint64_t* dkdv_full = dq_empty + 1;             // everything accumulated
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dkdv_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef B200FA_TRACE
  int trace_n = 0;
#endif
  const int n_tile = blockIdx.x;
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int n0 = n_tile * kTile;
  const int m_tiles = (p.S + kTile - 1) / kTile;
  const int m_start = kCausal ? n_tile : 0;
  const int per_head = m_tiles - m_start;
  const int steps = group * per_head;

  // The swizzled tiles assume a 1024-byte aligned shared-memory window.
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, 0x414c0000u);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&do_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    // one elected arrival per warp: 8 compute warps, 4 drain warps
    mbar_init(p_full, 8);
    mbar_init(ds_full, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 4);
    mbar_init(dkdv_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 12) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 13 && lane == 0) {
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
    tma_prefetch_desc(&mapDO);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

#define B200FA_WAIT(bar, parity, site) \
  if (!mbar_wait((bar), (parity), abort_flag, p.status, (site))) goto teardown

  if (warp < 8) {
    // =========================== compute warps ===========================
    reg_alloc<168>();
    const int wg = warp >> 2;                       // which 64-column half of the query tile
    const int j = (warp & 3) * 32 + lane;           // key row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_off + Cfg::kTmemS + wg * 64;
    const uint32_t tDP = tmem_base + lane_off + Cfg::kTmemDP + wg * 64;
    const float c = p.scale_log2;
    uint8_t* ds_row = sDS + wg * kSubTileBytes + j * 128;
    for (int i = 0; i < steps; ++i) {
      const int stage = i % Cfg::kStages;
      const int m_tile = m_start + i % per_head;
      const float* lse2 = sStat + stage * 256 + wg * 64;
      const float* dps = lse2 + 128;
      // ---- P^T = exp2(S^T * c - lse2)
      B200FA_WAIT(s_full, i & 1, 0x500);
      // lse2 rode in with the Q tile; observing its barrier directly makes the bulk copy visible here
      B200FA_WAIT(&q_full[stage], (i / Cfg::kStages) & 1, 0x501);
      tc_fence_after();
      if ((warp & 3) == 0) TRACE(wg, 1);
      float pf[64];
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t s[32];
        tmem_ld32(tS + ch * 32, s);
        tmem_wait_ld();
        const float* sf = reinterpret_cast<const float*>(s);
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float v = ex2_approx(fmaf(sf[e], c, -lse2[ch * 32 + e]));
          if (kCausal && m_tile == n_tile) {
            // on the diagonal tile, query column q sees key row j only if j <= q
            if (j > wg * 64 + ch * 32 + e) v = 0.f;
          }
          pf[ch * 32 + e] = v;
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = pack2<kBf16>(pf[ch * 32 + 2 * e], pf[ch * 32 + 2 * e + 1]);
        tmem_st16(tS + ch * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(p_full);
      if ((warp & 3) == 0) TRACE(wg, 2);
      // ---- dS^T = P^T * (dP^T - dpsum)
      B200FA_WAIT(dp_full, i & 1, 0x510);
      B200FA_WAIT(&do_full[stage], (i / Cfg::kStages) & 1, 0x511);
      tc_fence_after();
      if ((warp & 3) == 0) TRACE(wg, 3);
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t d[32];
        tmem_ld32(tDP + ch * 32, d);
        tmem_wait_ld();
        const float* df = reinterpret_cast<const float*>(d);
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float a0 = pf[ch * 32 + 2 * e] * (df[2 * e] - dps[ch * 32 + 2 * e]);
          const float a1 = pf[ch * 32 + 2 * e + 1] * (df[2 * e + 1] - dps[ch * 32 + 2 * e + 1]);
          pk[e] = pack2<kBf16>(a0, a1);
        }
        tmem_st16(tDP + ch * 16, pk);
        // the same values, as the 128-byte-swizzled [key row][query column] tile the dQ MMA reads
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const int chunk = ch * 4 + v;
          *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (j & 7)) << 4)) =
              make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive_warp(ds_full);
      if ((warp & 3) == 0) TRACE(wg, 4);
    }
    // ---- epilogue: dV and dK (this warpgroup's half of the head dimension)
    B200FA_WAIT(dkdv_full, 0, 0x520);
    tc_fence_after();
    {
      const int krow = n0 + j;
      const bool valid = krow < p.S;
      constexpr int kHalf = kD / 2;
      uint16_t* dv_row = reinterpret_cast<uint16_t*>(p.dv.ptr) +
                         (static_cast<int64_t>(b) * p.dv.sb + static_cast<int64_t>(hk) * p.dv.sh +
                          static_cast<int64_t>(krow) * p.dv.ss) + wg * kHalf;
      uint16_t* dk_row = reinterpret_cast<uint16_t*>(p.dk.ptr) +
                         (static_cast<int64_t>(b) * p.dk.sb + static_cast<int64_t>(hk) * p.dk.sh +
                          static_cast<int64_t>(krow) * p.dk.ss) + wg * kHalf;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t tacc = tmem_base + lane_off + (which == 0 ? Cfg::kTmemDV : Cfg::kTmemDK) + wg * kHalf;
        uint16_t* dst = which == 0 ? dv_row : dk_row;
        const float mul = which == 0 ? 1.f : p.scale;
#pragma unroll
        for (int ch = 0; ch < kHalf / 32; ++ch) {
          uint32_t a[32];
          tmem_ld32(tacc + ch * 32, a);
          tmem_wait_ld();
          if (valid) {
            const float* af = reinterpret_cast<const float*>(a);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack2<kBf16>(af[v * 8 + 0] * mul, af[v * 8 + 1] * mul);
              w.y = pack2<kBf16>(af[v * 8 + 2] * mul, af[v * 8 + 3] * mul);
              w.z = pack2<kBf16>(af[v * 8 + 4] * mul, af[v * 8 + 5] * mul);
              w.w = pack2<kBf16>(af[v * 8 + 6] * mul, af[v * 8 + 7] * mul);
              *reinterpret_cast<uint4*>(dst + ch * 32 + v * 8) = w;
            }
          }
        }
      }
    }
  } else if (warp < 12) {
    // =========================== dQ drain warps ===========================
    reg_dealloc<88>();
    const int row = (warp & 3) * 32 + lane;  // query row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tDQ = tmem_base + lane_off + Cfg::kTmemDQ;
    for (int i = 0; i < steps; ++i) {
      const int g = i / per_head;
      const int m_tile = m_start + i % per_head;
      const int h = hk * group + g;
      float* acc = p.dq_accum +
                   ((static_cast<int64_t>(b) * p.Hq + h) * p.Spad + m_tile * kTile + row) * kD;
      B200FA_WAIT(dq_full, i & 1, 0x600);
      tc_fence_after();
      if (warp == 8) TRACE(2, 10);
#pragma unroll
      for (int ch = 0; ch < kD / 32; ++ch) {
        uint32_t a[32];
        tmem_ld32(tDQ + ch * 32, a);
        tmem_wait_ld();
        if (ch == kD / 32 - 1) {
          // every column is in registers: the accumulator columns may be overwritten
          tc_fence_before();
          mbar_arrive_warp(dq_empty);
          if (warp == 8) TRACE(2, 11);
        }
        const float* af = reinterpret_cast<const float*>(a);
#pragma unroll
        for (int v = 0; v < 8; ++v)
          red_add_v4(acc + ch * 32 + v * 4, af[4 * v], af[4 * v + 1], af[4 * v + 2], af[4 * v + 3]);
      }
    }
  } else {
    reg_dealloc<88>();
    if (warp == 12) {
      // =========================== MMA issuer ===========================
      if (lane == 0) {
        constexpr uint32_t idesc_st = umma_idesc(kBf16, false, false, 128, 128);  // S^T, dP^T
        constexpr uint32_t idesc_acc = umma_idesc(kBf16, false, true, 128, kD);   // dV, dK (A from TMEM)
        constexpr uint32_t idesc_dq = umma_idesc(kBf16, true, true, 128, kD);     // dQ (A, B MN-major)
        const uint32_t tS = tmem_base + Cfg::kTmemS, tDP = tmem_base + Cfg::kTmemDP,
                       tDV = tmem_base + Cfg::kTmemDV, tDK = tmem_base + Cfg::kTmemDK,
                       tDQ = tmem_base + Cfg::kTmemDQ;
        // Descriptors: fixed high word + start-address low word; K-major form (LBO unused) for
        // the S^T / dP^T operands, MN-major form (LBO = next 64-column sub-tile) for the rest.
        const UmmaDesc kK = umma_desc_split(smem_u32(sK), 16, 1024), kV = umma_desc_split(smem_u32(sV), 16, 1024),
                       kQ = umma_desc_split(smem_u32(sQ), 16, 1024), kDO = umma_desc_split(smem_u32(sDO), 16, 1024);
        const UmmaDesc mK = umma_desc_split(smem_u32(sK), kSubTileBytes, 1024),
                       mQ = umma_desc_split(smem_u32(sQ), kSubTileBytes, 1024),
                       mDO = umma_desc_split(smem_u32(sDO), kSubTileBytes, 1024),
                       mDS = umma_desc_split(smem_u32(sDS), kSubTileBytes, 1024);
        // D[128 x 128] = A[128 x kD] * B[128 x kD]^T, both K-major
        auto issue_kmajor = [&](uint32_t d_tmem, const UmmaDesc& a, const UmmaDesc& b, uint32_t b_stage_lo) {
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) {
            const uint32_t off = umma_off((kk >> 2) * kSubTileBytes + (kk & 3) * 32);
            if (kk == 0) umma_ss_fast<false>(d_tmem, a.lo + off, a.hi, b.lo + b_stage_lo + off, b.hi, idesc_st);
            else         umma_ss_fast<true>(d_tmem, a.lo + off, a.hi, b.lo + b_stage_lo + off, b.hi, idesc_st);
          }
        };
        // D[128 x kD] (+)= A^T-in-TMEM[128 x 128] * B[128 x kD] (B rows are the contraction index)
        auto issue_ts = [&](uint32_t d_tmem, uint32_t a_tmem, const UmmaDesc& b, uint32_t b_stage_lo, bool acc) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t a_col = (kk < 4) ? kk * 8 : 64 + (kk - 4) * 8;
            const uint32_t b_lo = b.lo + b_stage_lo + umma_off(kk * 2048);
            if (kk == 0 && !acc) umma_ts_fast<false>(d_tmem, a_tmem + a_col, b_lo, b.hi, idesc_acc);
            else                 umma_ts_fast<true>(d_tmem, a_tmem + a_col, b_lo, b.hi, idesc_acc);
          }
        };
        B200FA_WAIT(kv_full, 0, 0x700);
        B200FA_WAIT(&q_full[0], 0, 0x701);
        tc_fence_after();
        issue_kmajor(tS, kK, kQ, 0);
        umma_commit(s_full);
        B200FA_WAIT(&do_full[0], 0, 0x702);
        tc_fence_after();
        issue_kmajor(tDP, kV, kDO, 0);
        umma_commit(dp_full);
        for (int i = 0; i < steps; ++i) {
          const int stage = i % Cfg::kStages;
          const uint32_t stage_lo = stage * umma_off(Cfg::kTileBytes);
          const bool has_next = (i + 1 < steps);
          const int nstage = (i + 1) % Cfg::kStages;
          const uint32_t nstage_lo = nstage * umma_off(Cfg::kTileBytes);
          const uint32_t nphase = static_cast<uint32_t>(((i + 1) / Cfg::kStages) & 1);
          // dV += P^T dO
          TRACE(3, 20);
          B200FA_WAIT(p_full, i & 1, 0x710);
          tc_fence_after();
          TRACE(3, 21);
          issue_ts(tDV, tS, mDO, stage_lo, i > 0);
          // S^T of the next step can start as soon as P^T has been consumed (in issue order)
          if (has_next) {
            B200FA_WAIT(&q_full[nstage], nphase, 0x711);
            tc_fence_after();
            issue_kmajor(tS, kK, kQ, nstage_lo);
            umma_commit(s_full);
          }
          // dK += dS^T Q ; dQ = dS K
          TRACE(3, 22);
          B200FA_WAIT(ds_full, i & 1, 0x712);
          tc_fence_after();
          TRACE(3, 23);
          issue_ts(tDK, tDP, mQ, stage_lo, i > 0);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = umma_off(kk * 2048);
            if (kk == 0) umma_ss_fast<false>(tDQ, mDS.lo + off, mDS.hi, mK.lo + off, mK.hi, idesc_dq);
            else         umma_ss_fast<true>(tDQ, mDS.lo + off, mDS.hi, mK.lo + off, mK.hi, idesc_dq);
          }
          umma_commit(dq_full);
          umma_commit(&qdo_empty[stage]);
          TRACE(3, 24);
          if (has_next) {
            B200FA_WAIT(&do_full[nstage], nphase, 0x713);
            B200FA_WAIT(dq_empty, i & 1, 0x714);
            tc_fence_after();
            TRACE(3, 25);
            issue_kmajor(tDP, kV, kDO, nstage_lo);
            umma_commit(dp_full);
          }
        }
        umma_commit(dkdv_full);
      }
    } else if (warp == 13) {
      // =========================== TMA producer ===========================
      if (lane == 0) {
        auto load_tile = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int srow, int head) {
#pragma unroll
          for (int cs = 0; cs < Cfg::kSub; ++cs) tma_load_4d(dst + cs * kSubTileBytes, map, bar, cs * 64, srow, head, b);
        };
        mbar_arrive_expect_tx(kv_full, 2 * Cfg::kTileBytes);
        load_tile(&mapK, sK, kv_full, n0, hk);
        load_tile(&mapV, sV, kv_full, n0, hk);
        for (int i = 0; i < steps; ++i) {
          const int stage = i % Cfg::kStages;
          const int g = i / per_head;
          const int m_tile = m_start + i % per_head;
          const int h = hk * group + g;
          if (i >= Cfg::kStages) {
            B200FA_WAIT(&qdo_empty[stage], ((i / Cfg::kStages) - 1) & 1, 0x800);
          }
          const int64_t stat_off = (static_cast<int64_t>(b) * p.Hq + h) * p.Spad + m_tile * kTile;
          float* st = sStat + stage * 256;
          mbar_arrive_expect_tx(&q_full[stage], Cfg::kTileBytes + 512);
          load_tile(&mapQ, sQ + stage * Cfg::kTileBytes, &q_full[stage], m_tile * kTile, h);
          bulk_load_1d(st, p.lse_log2 + stat_off, 512, &q_full[stage]);
          mbar_arrive_expect_tx(&do_full[stage], Cfg::kTileBytes + 512);
          load_tile(&mapDO, sDO + stage * Cfg::kTileBytes, &do_full[stage], m_tile * kTile, h);
          bulk_load_1d(st + 128, p.dpsum + stat_off, 512, &do_full[stage]);
        }
      }
    }
  }

teardown:
#undef B200FA_WAIT
  tc_fence_before();
  __syncthreads();
  if (warp == 12) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------
// preprocess: dpsum = rowsum(dO * O), lse2 = lse * log2(e), zero the fp32 dQ accumulator.
// Rows in [S, Spad) get lse2 = +inf and dpsum = 0 so their probabilities vanish.
// One row per group of D/8 lanes; every lane moves 16 bytes of O and of dO.
// ------------------------------------------------------------------------------------------
template <int kD, bool kBf16>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const BwdParams p) {
  constexpr int kLanesPerRow = kD / 8;
  constexpr int kRowsPerWarp = 32 / kLanesPerRow;
  const int lane = threadIdx.x & 31;
  const int sub = lane / kLanesPerRow;
  const int li = lane % kLanesPerRow;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t row_global = warp_global * kRowsPerWarp + sub;
  const int64_t total_rows = static_cast<int64_t>(p.B) * p.Hq * p.Spad;
  if (row_global >= total_rows) return;
  const int s = static_cast<int>(row_global % p.Spad);
  const int64_t bh = row_global / p.Spad;
  const int h = static_cast<int>(bh % p.Hq);
  const int b = static_cast<int>(bh / p.Hq);
  float acc = 0.f;
  if (s < p.S) {
    const uint16_t* o = reinterpret_cast<const uint16_t*>(p.out.ptr) +
                        (static_cast<int64_t>(b) * p.out.sb + static_cast<int64_t>(h) * p.out.sh +
                         static_cast<int64_t>(s) * p.out.ss) + li * 8;
    const uint16_t* d = reinterpret_cast<const uint16_t*>(p.dout.ptr) +
                        (static_cast<int64_t>(b) * p.dout.sb + static_cast<int64_t>(h) * p.dout.sh +
                         static_cast<int64_t>(s) * p.dout.ss) + li * 8;
    const uint4 ov = *reinterpret_cast<const uint4*>(o);
    const uint4 dv = *reinterpret_cast<const uint4*>(d);
    const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
    const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float o0, o1, d0, d1;
      if constexpr (kBf16) {
        o0 = __uint_as_float(ow[i] << 16); o1 = __uint_as_float(ow[i] & 0xffff0000u);
        d0 = __uint_as_float(dw[i] << 16); d1 = __uint_as_float(dw[i] & 0xffff0000u);
      } else {
        asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi;}"
            : "=f"(o0), "=f"(o1) : "r"(ow[i]));
        asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.f32.f16 %0, lo; cvt.f32.f16 %1, hi;}"
            : "=f"(d0), "=f"(d1) : "r"(dw[i]));
      }
      acc = fmaf(o0, d0, acc);
      acc = fmaf(o1, d1, acc);
    }
  }
#pragma unroll
  for (int off = kLanesPerRow / 2; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (li == 0) {
    p.dpsum[row_global] = (s < p.S) ? acc : 0.f;
    p.lse_log2[row_global] =
        (s < p.S) ? p.lse[(static_cast<int64_t>(b) * p.Hq + h) * p.S + s] * 1.4426950408889634f : INFINITY;
  }
  float4* z = reinterpret_cast<float4*>(p.dq_accum + row_global * kD + li * 8);
  z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
  z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// convert: dQ = (fp32 accumulator * scale) rounded to the 16-bit type; 8 elements per thread.
template <int kD, bool kBf16>
__global__ void __launch_bounds__(256) bwd_convert_kernel(const BwdParams p) {
  constexpr int kVecPerRow = kD / 8;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(p.B) * p.Hq * p.S * kVecPerRow;
  if (idx >= total) return;
  const int vec = static_cast<int>(idx % kVecPerRow);
  const int64_t row = idx / kVecPerRow;
  const int s = static_cast<int>(row % p.S);
  const int64_t bh = row / p.S;
  const int h = static_cast<int>(bh % p.Hq);
  const int b = static_cast<int>(bh / p.Hq);
  const float4* src = reinterpret_cast<const float4*>(p.dq_accum + (bh * p.Spad + s) * kD + vec * 8);
  const float4 a = src[0], c = src[1];
  uint4 w;
  w.x = pack2<kBf16>(a.x * p.scale, a.y * p.scale);
  w.y = pack2<kBf16>(a.z * p.scale, a.w * p.scale);
  w.z = pack2<kBf16>(c.x * p.scale, c.y * p.scale);
  w.w = pack2<kBf16>(c.z * p.scale, c.w * p.scale);
  uint16_t* dst = reinterpret_cast<uint16_t*>(p.dq.ptr) +
                  (static_cast<int64_t>(b) * p.dq.sb + static_cast<int64_t>(h) * p.dq.sh +
                   static_cast<int64_t>(s) * p.dq.ss) + vec * 8;
  *reinterpret_cast<uint4*>(dst) = w;
}

template <int kD, bool kBf16, bool kCausal>
cudaError_t launch_one(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                       const BwdParams& p, cudaStream_t stream) {
  using Cfg = BwdCfg<kD>;
  constexpr int kRowsPerWarp = 32 / (kD / 8);
  const int64_t total_rows = static_cast<int64_t>(p.B) * p.Hq * p.Spad;
  const int64_t pre_warps = (total_rows + kRowsPerWarp - 1) / kRowsPerWarp;
  cudaError_t e = cudaSuccess;
  if (p.parts & 1) {
    bwd_preprocess_kernel<kD, kBf16><<<static_cast<unsigned>((pre_warps + 7) / 8), 256, 0, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }

  auto kern = bwd_kernel<kD, kBf16, kCausal>;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  if (p.parts & 2) {
    dim3 grid((p.S + kTile - 1) / kTile, p.Hkv, p.B);
    kern<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(mq, mk, mv, mdo, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  if (p.parts & 4) {
    const int64_t total_vec = static_cast<int64_t>(p.B) * p.Hq * p.S * (kD / 8);
    bwd_convert_kernel<kD, kBf16><<<static_cast<unsigned>((total_vec + 255) / 256), 256, 0, stream>>>(p);
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace

cudaError_t launch_bwd_sm100(const BwdParams& p, int dtype, cudaStream_t stream, int* launches) {
  const bool bf16 = (dtype == kBF16);
  CUtensorMap mq, mk, mv, mdo;
  if (!encode_map_16bit(&mq, p.q, p.B, p.Hq, p.S, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mk, p.k, p.B, p.Hkv, p.S, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mv, p.v, p.B, p.Hkv, p.S, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mdo, p.dout, p.B, p.Hq, p.S, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  cudaError_t e;
#define B200FA_DISPATCH(D_, BF_, C_) e = launch_one<D_, BF_, C_>(mq, mk, mv, mdo, p, stream)
  if (p.D == 128) {
    if (bf16) { if (p.causal) B200FA_DISPATCH(128, true, true); else B200FA_DISPATCH(128, true, false); }
    else      { if (p.causal) B200FA_DISPATCH(128, false, true); else B200FA_DISPATCH(128, false, false); }
  } else {
    if (bf16) { if (p.causal) B200FA_DISPATCH(64, true, true); else B200FA_DISPATCH(64, true, false); }
    else      { if (p.causal) B200FA_DISPATCH(64, false, true); else B200FA_DISPATCH(64, false, false); }
  }
#undef B200FA_DISPATCH
  if (e == cudaSuccess && launches) *launches += (p.parts & 1) + ((p.parts >> 1) & 1) + ((p.parts >> 2) & 1);
  return e;
}

}  // namespace b200fa
