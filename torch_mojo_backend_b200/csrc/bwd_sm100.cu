// Backward flash attention for sm_100a: a preprocess pass and two tcgen05 kernels, one that
// owns dK/dV and one that owns dQ.
//
// Math (same as the reference's backward kernels,
// torch_mojo_backend/eager_flash_attention/fa4_bwd_kernel.mojo:1-44, 810-980, 1443-1444,
// 1634-1662, 1855), with c = scale*log2(e):
//   dpsum = rowsum(dO * O),  lse2 = lse*log2(e)              (preprocess; stored negated, so that
//                                                             both enter packed two-wide adds and FMAs)
//   P  = exp2(S*c - lse2),   dS = P * (dP - dpsum)
//   dV = P^T dO,   dK = scale * dS^T Q,   dQ = scale * dS K
//
// The reference accumulates dQ from every K/V tile into an fp32 buffer with bulk reduce-adds
// and converts it afterwards.  On B200 that accumulation is the bottleneck: fp32 reductions
// into L2 sustain 1.9-3.3 TB/s depending on the access pattern, and a 4k-token Llama-style
// backward needs 4.4 GB of them.  Here nothing is accumulated in global memory: the
// dK/dV kernel gives each CTA one 128-row K/V tile (S^T = K Q^T, dP^T = V dO^T, so P^T and
// dS^T land in tensor memory as the A operands of dV += P^T dO and dK += dS^T Q), and the dQ
// kernel gives each CTA one 128-row query tile (S = Q K^T, dP = dO V^T, dS in tensor memory
// as the A operand of dQ += dS K).  S and dP are computed twice (7 tile GEMMs per tile pair
// instead of 5), every accumulator lives in TMEM, and the results are deterministic.
//
// Both kernels: warps 0-3 and 4-7 are two compute warpgroups that split the 128 score
// columns of a tile in halves (thread <-> TMEM lane), warps 8 and 9 each issue one of the two
// independent MMA chains (the dK/dV kernel uses warp 10 for a third), the next warp drives TMA.
#include <mutex>

#include "common.cuh"
#include "philox.cuh"
#include "ptx.cuh"

namespace b200fa {
namespace {

constexpr int kTile = 128;
constexpr int kThreads = 384;        // dQ kernel: 8 compute warps + 4
constexpr int kDkdvThreads = 640;    // dK/dV kernel: 16 compute warps + 4
constexpr int kSubTileBytes = 128 * 128;

template <int kD>
struct BwdCfg {
  static constexpr int kTileBytes = kTile * kD * 2;
  static constexpr int kSub = kD / 64;
  static constexpr int kStages = 2;
  // resident pair of tiles, then kStages pairs of streamed tiles, then per-stage row statistics
  static constexpr int kOffResident = 0;
  static constexpr int kOffStream = 2 * kTileBytes;
  static constexpr int kOffP = kOffStream + kStages * 2 * kTileBytes;     // dK/dV kernel: 128 x 128 16-bit P^T tile
  static constexpr int kOffStat = kOffP + 128 * 128 * 2;                  // [stage][lse2|dpsum][128] fp32
  static constexpr int kOffBars = kOffStat + kStages * 2 * 128 * 4;
  static constexpr int kNumBars = 20;
  // the dQ kernel keeps 2 resident + 3 K + 2 V tiles and no per-stage statistics
  static constexpr int kOffDqBars = 7 * kTileBytes;
  static constexpr int kSmemBytes =
      (kOffBars > kOffDqBars ? kOffBars : kOffDqBars) + kNumBars * 8 + 16;
};

#define B200FA_WAIT(bar, parity, site) \
  if (!mbar_wait((bar), (parity), abort_flag, p.status, (site), p.wait_budget)) goto teardown

// two exponentials on the special function unit
__device__ __forceinline__ float2 exp2_mufu2(float2 x) { return make_float2(ex2_approx(x.x), ex2_approx(x.y)); }

// ------------------------------------------------------------------------------------------
// dK / dV kernel.  One CTA = one 128-row K/V tile of one (batch, kv head); it walks every
// query tile at or below the causal diagonal for every query head of the GQA group.
// TMEM columns: [0,128) S^T; [128,256) dP^T, overwritten by 16-bit dS^T (the A operand of the
// dK MMA); then the dV and dK accumulators.  16-bit P^T goes through shared memory instead, so
// S^T of the next step can be issued while the exponentials of this step are still running.
// ------------------------------------------------------------------------------------------
template <int kD, bool kBf16, bool kCausal, bool kDropout>
__global__ void __launch_bounds__(kDkdvThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                const __grid_constant__ CUtensorMap mapDK, const __grid_constant__ CUtensorMap mapDV,
                const BwdParams p, const int sched_group) {
  using Cfg = BwdCfg<kD>;
  // TMEM: two 128-column work buffers (step i uses buffer i & 1 for S^T, then dP^T, then dS^T),
  // then the dV and dK accumulators.
  constexpr int kTmemWork = 0, kTmemDV = 256, kTmemDK = 256 + kD;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem + Cfg::kOffResident;
  uint8_t* sV = sK + Cfg::kTileBytes;
  uint8_t* sQ = smem + Cfg::kOffStream;                          // stage s: sQ + s * 2 * tile, dO right behind
  uint8_t* sP = smem + Cfg::kOffP;                               // 16-bit P^T, [key row][query column], swizzled
  float* sStat = reinterpret_cast<float*>(smem + Cfg::kOffStat);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* kv_full = bars;                        // [1]
  uint64_t* q_full = kv_full + 1;                  // [kStages]  Q tile + lse2
  uint64_t* do_full = q_full + Cfg::kStages;       // [kStages]  dO tile + dpsum
  uint64_t* qdo_empty = do_full + Cfg::kStages;    // [kStages]
  uint64_t* s_full = qdo_empty + Cfg::kStages;     // [2]  S^T ready in work buffer b
  uint64_t* buf_free = s_full + 2;                 // [2]  dK MMA has consumed dS^T from work buffer b
  uint64_t* dp_full = buf_free + 2;                // dP^T ready
  uint64_t* p_full = dp_full + 1;                  // P^T written  (8 warp arrivals)
  uint64_t* ds_full = p_full + 1;                  // dS^T written (8 warp arrivals)
  uint64_t* acc_full = ds_full + 1;                // dK, dV complete
  uint64_t* s_free = acc_full + 1;                 // S^T read into registers (8 warp arrivals)
  uint64_t* p_empty = s_free + 1;                  // dV MMA has consumed the P^T tile
  uint64_t* staged = p_empty + 1;                  // dV and dK tiles staged in shared memory (16 warp arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Block order: (batch, kv head) pairs are walked `sched_group` at a time, few enough that the
  // Q / dO rows they stream stay in L2, and inside such a group the K/V tiles with the most
  // causal work (the earliest) come first, so the last wave of CTAs is made of short ones.
  const int m_tiles = (p.S + kTile - 1) / kTile;      // query tiles
  const int n_tiles = (p.Sk + kTile - 1) / kTile;     // K/V tiles (== m_tiles when causal)
  int n_tile, hk, b;
  {
    const int pairs = p.B * p.Hkv;
    const int per_group = sched_group * n_tiles;
    const int g = static_cast<int>(blockIdx.x) / per_group;
    const int gsize = min(sched_group, pairs - g * sched_group);
    const int within = static_cast<int>(blockIdx.x) - g * per_group;
    n_tile = within / gsize;
    const int pair = g * sched_group + within % gsize;
    b = pair / p.Hkv;
    hk = pair - b * p.Hkv;
  }
  const int group = p.Hq / p.Hkv;
  const int n0 = n_tile * kTile;
  // query row i sees key column j iff j <= i + causal_off: the first query tile with a row that
  // sees a key of this tile (none: the tile's dK and dV are zero)
  const int m_start = kCausal ? min(m_tiles, max(0, n0 - p.causal_off) / kTile) : 0;
  const int per_head = m_tiles - m_start;
  const int steps = group * per_head;

  // A launch whose status word already reports a failed wait is not worth running; the swizzled
  // tiles assume a 1024-byte aligned shared-memory window.
  if (status_is_set(p.status)) return;
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, 0x414c0000u);
    return;
  }
  // Lane 0 of the producer warp sets up the barriers and at once issues the loads the first MMAs
  // wait for, so that their latency overlaps the TMEM allocation and the block-wide synchronisation.
  auto load_tile = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int srow, int head) {
#pragma unroll
    for (int cs = 0; cs < Cfg::kSub; ++cs) tma_load_4d(dst + cs * kSubTileBytes, map, bar, cs * 64, srow, head, b);
  };
  // Q (with lse2) and dO (with dpsum) of step i into ring stage i % kStages
  auto load_step = [&](int i) {
    const int stage = i % Cfg::kStages;
    const int h = hk * group + i / per_head;
    const int m_tile = m_start + i % per_head;
    const int64_t stat_off = (static_cast<int64_t>(b) * p.Hq + h) * p.Spad + m_tile * kTile;
    float* st = sStat + stage * 256;
    uint8_t* q_dst = sQ + stage * 2 * Cfg::kTileBytes;
    mbar_arrive_expect_tx(&q_full[stage], Cfg::kTileBytes + 512);
    load_tile(&mapQ, q_dst, &q_full[stage], m_tile * kTile, h);
    bulk_load_1d(st, p.lse_log2 + stat_off, 512, &q_full[stage]);
    mbar_arrive_expect_tx(&do_full[stage], Cfg::kTileBytes + 512);
    load_tile(&mapDO, q_dst + Cfg::kTileBytes, &do_full[stage], m_tile * kTile, h);
    bulk_load_1d(st + 128, p.dpsum + stat_off, 512, &do_full[stage]);
  };
  if (warp == 19 && lane == 0) {
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapDO);
    tma_prefetch_desc(&mapV);
    mbar_init(kv_full, 1);
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&do_full[i], 1);
      mbar_init(&qdo_empty[i], 2);   // both MMA-issuing lanes release a stage
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&buf_free[i], 1);
    }
    mbar_init(dp_full, 1);
    mbar_init(p_full, 16);   // one elected arrival per compute warp
    mbar_init(ds_full, 16);
    mbar_init(acc_full, 2);        // both MMA-issuing lanes
    mbar_init(s_free, 16);
    mbar_init(p_empty, 1);
    mbar_init(staged, 16);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    mbar_arrive_expect_tx(kv_full, 2 * Cfg::kTileBytes);
    load_tile(&mapK, sK, kv_full, n0, hk);
    if (steps > 0) load_step(0);
    load_tile(&mapV, sV, kv_full, n0, hk);
  }
  if (warp == 16) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 16) {
    // =========================== compute warps ===========================
    const int wg = warp >> 2;                       // which 32-column (query) quarter of the tile
    const int j = (warp & 3) * 32 + lane;           // key row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tWork = tmem_base + lane_off + kTmemWork + wg * 32;
    const float c = p.scale_log2;
    // this thread's 64 bytes (32 query columns) of its row of the 128-byte-swizzled P^T tile
    uint8_t* p_row = sP + (wg >> 1) * kSubTileBytes + j * 128;
    const int chunk0 = (wg & 1) * 4;
    for (int i = 0; i < steps; ++i) {
      const int stage = i % Cfg::kStages;
      const uint32_t ring_phase = static_cast<uint32_t>((i / Cfg::kStages) & 1);
      const int m_tile = m_start + i % per_head;
      const float4* lse2 = reinterpret_cast<const float4*>(sStat + stage * 256 + wg * 32);
      const float4* dps = lse2 + 32;
      // ---- P^T = exp2(S^T * c - lse2).  S^T is pulled into registers in one go and released
      // at once, so the S^T MMA of the next step can run while the exponentials do;
      // P^T goes to shared memory (the A operand of dV += P^T dO) instead of back over S^T.
      // S^T, dP^T and dS^T of this step live one after the other in work buffer i & 1
      const uint32_t tS = tWork + (i & 1) * 128, tDP = tS;
      B200FA_WAIT(&s_full[i & 1], (i >> 1) & 1, 0x500);
      // lse2 rode in with the Q tile; observing its barrier directly makes the bulk copy visible here
      B200FA_WAIT(&q_full[stage], ring_phase, 0x501);
      tc_fence_after();
      float pf[32];
      {
        tmem_ld32(tS, reinterpret_cast<uint32_t*>(pf));
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive_warp(s_free);
      }
      const float2 c2 = make_float2(c, c);
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        const float4 l4 = lse2[e4];   // minus lse2
        float2 x0 = __ffma2_rn(make_float2(pf[e4 * 4 + 0], pf[e4 * 4 + 1]), c2, make_float2(l4.x, l4.y));
        float2 x1 = __ffma2_rn(make_float2(pf[e4 * 4 + 2], pf[e4 * 4 + 3]), c2, make_float2(l4.z, l4.w));
        x0 = exp2_mufu2(x0);
        x1 = exp2_mufu2(x1);
        pf[e4 * 4 + 0] = x0.x; pf[e4 * 4 + 1] = x0.y; pf[e4 * 4 + 2] = x1.x; pf[e4 * 4 + 3] = x1.y;
      }
      if (kCausal && n0 + kTile - 1 > m_tile * kTile + p.causal_off) {
        // a tile the diagonal crosses: query column q sees key row j only if j <= q + causal_off
        const int first_q = n0 + j - p.causal_off - (m_tile * kTile + wg * 32);  // first column (of these 32) that sees key j
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (e < first_q) pf[e] = 0.f;
        }
      }
      // dropout: bit e of `keep` <-> query column e of these 32.  Lane L draws the bits of query
      // row L against this warp's 32 key rows (two Philox calls), and 32 ballots transpose them.
      uint32_t keep = 0xffffffffu;
      if constexpr (kDropout) {
        const int h_now = hk * group + i / per_head;
        const int q_glob = m_tile * kTile + wg * 32 + lane;
        const int blk = (n0 + (warp & 3) * 32) >> 4;
        const uint32_t mine = dropout_bits16(p.drop, b * p.Hq + h_now, q_glob, blk) |
                              (dropout_bits16(p.drop, b * p.Hq + h_now, q_glob, blk + 1) << 16);
        keep = 0;
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const uint32_t word = __ballot_sync(0xffffffffu, (mine >> jj) & 1u);
          if (lane == jj) keep = word;
        }
      }
      // the previous step's dV MMA must have finished reading the P^T tile
      if (i > 0) { B200FA_WAIT(p_empty, (i - 1) & 1, 0x502); }
#pragma unroll
      for (int chunk = 0; chunk < 4; ++chunk) {
        float pd[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          pd[e] = pf[chunk * 8 + e];
          if constexpr (kDropout) pd[e] = ((keep >> (chunk * 8 + e)) & 1u) ? pd[e] * p.drop.inv_keep : 0.f;
        }
        uint4 w;
        w.x = pack2<kBf16>(pd[0], pd[1]);
        w.y = pack2<kBf16>(pd[2], pd[3]);
        w.z = pack2<kBf16>(pd[4], pd[5]);
        w.w = pack2<kBf16>(pd[6], pd[7]);
        *reinterpret_cast<uint4*>(p_row + (((chunk0 + chunk) ^ (j & 7)) << 4)) = w;
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(p_full);
      // ---- dS^T = P^T * (dP^T - dpsum)
      B200FA_WAIT(dp_full, i & 1, 0x510);
      B200FA_WAIT(&do_full[stage], ring_phase, 0x511);
      tc_fence_after();
      {
        uint32_t d[32];
        tmem_ld32(tDP, d);
        tmem_wait_ld();
        const float* df = reinterpret_cast<const float*>(d);
        uint32_t pk[16];
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 d4 = dps[e4];
          float g0 = df[e4 * 4 + 0], g1 = df[e4 * 4 + 1], g2 = df[e4 * 4 + 2], g3 = df[e4 * 4 + 3];
          if constexpr (kDropout) {
            // the gradient reaches a probability only through the entries that were kept
            const uint32_t kb = keep >> (e4 * 4);
            g0 = (kb & 1u) ? g0 * p.drop.inv_keep : 0.f;
            g1 = (kb & 2u) ? g1 * p.drop.inv_keep : 0.f;
            g2 = (kb & 4u) ? g2 * p.drop.inv_keep : 0.f;
            g3 = (kb & 8u) ? g3 * p.drop.inv_keep : 0.f;
          }
          // d4 holds minus dpsum
          const float2 s0 = __fmul2_rn(make_float2(pf[e4 * 4 + 0], pf[e4 * 4 + 1]), __fadd2_rn(make_float2(g0, g1), make_float2(d4.x, d4.y)));
          const float2 s1 = __fmul2_rn(make_float2(pf[e4 * 4 + 2], pf[e4 * 4 + 3]), __fadd2_rn(make_float2(g2, g3), make_float2(d4.z, d4.w)));
          pk[e4 * 2] = pack2<kBf16>(s0.x, s0.y);
          pk[e4 * 2 + 1] = pack2<kBf16>(s1.x, s1.y);
        }
        tmem_st16(tDP, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(ds_full);
    }
    // ---- epilogue: dV and dK (this warpgroup's quarter of the head dimension)
    B200FA_WAIT(acc_full, 0, 0x520);
    tc_fence_after();
    {
      // The 16-bit dV and dK tiles are staged in the Q / dO ring (every MMA that read it has
      // completed) in the swizzled box layout and leave through TMA stores: whole 128-byte
      // lines, key rows past the end of the sequence clipped by the tensor map.
      constexpr int kQuarter = kD / 4;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        uint8_t* stage = sQ + which * Cfg::kTileBytes;
        const uint32_t tacc = tmem_base + lane_off + (which == 0 ? kTmemDV : kTmemDK) + wg * kQuarter;
        const float mul = which == 0 ? 1.f : p.scale;
        uint32_t a[kQuarter];
        if (steps > 0) {
          if constexpr (kQuarter == 32) tmem_ld32(tacc, a); else tmem_ld16(tacc, a);
          tmem_wait_ld();
        } else {
          // no query row sees this K/V tile: nothing was accumulated, the gradients are zero
#pragma unroll
          for (int e = 0; e < kQuarter; ++e) a[e] = 0u;
        }
        const float* af = reinterpret_cast<const float*>(a);
#pragma unroll
        for (int v = 0; v < kQuarter / 8; ++v) {
          uint4 w;
          w.x = pack2<kBf16>(af[v * 8 + 0] * mul, af[v * 8 + 1] * mul);
          w.y = pack2<kBf16>(af[v * 8 + 2] * mul, af[v * 8 + 3] * mul);
          w.z = pack2<kBf16>(af[v * 8 + 4] * mul, af[v * 8 + 5] * mul);
          w.w = pack2<kBf16>(af[v * 8 + 6] * mul, af[v * 8 + 7] * mul);
          const int chunk = wg * (kQuarter / 8) + v;   // 16-byte chunk of the row
          *reinterpret_cast<uint4*>(stage + (chunk >> 3) * kSubTileBytes + j * 128 + (((chunk & 7) ^ (j & 7)) << 4)) = w;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(staged);
      if (threadIdx.x == 0) {
        B200FA_WAIT(staged, 0, 0x521);
#pragma unroll
        for (int cs = 0; cs < Cfg::kSub; ++cs) {
          tma_store_4d(&mapDV, sQ + cs * kSubTileBytes, cs * 64, n0, hk, b);
          tma_store_4d(&mapDK, sQ + Cfg::kTileBytes + cs * kSubTileBytes, cs * 64, n0, hk, b);
        }
        tma_store_commit();
        tma_store_wait_read();
      }
    }
  } else if (warp >= 16 && warp <= 18) {
    // =========================== MMA issuers ===========================
    // A tcgen05.mma only issues once the tensor pipe has room, so an issuing lane is stalled
    // for about as long as its MMAs run, and it handles its waits strictly in program order.
    // The three dependency chains of a step therefore get a lane each, so none of them waits
    // behind another chain's operands:
    //   warp 16: S^T of the next step      (needs the next Q tile and S^T of this step in registers)
    //   warp 17: dK, then dP^T of the next step   (needs dS^T, the next dO tile)
    //   warp 18: dV                        (needs P^T in shared memory); frees the Q/dO stage
    if (lane == 0) {
      constexpr uint32_t idesc_st = umma_idesc(kBf16, false, false, 128, 128);  // S^T, dP^T
      constexpr uint32_t idesc_acc = umma_idesc(kBf16, false, true, 128, kD);   // dV (A in smem), dK (A in TMEM)
      const uint32_t tWork = tmem_base + kTmemWork, tDV = tmem_base + kTmemDV, tDK = tmem_base + kTmemDK;
      // Descriptors: fixed high word + start-address low word.  K-major form for the S^T / dP^T
      // operands and the P^T tile, MN-major form (LBO = next 64-column sub-tile) when Q / dO
      // are the B operand of an accumulating MMA.
      const UmmaDesc kK = umma_desc_split(smem_u32(sK), 16, 1024), kV = umma_desc_split(smem_u32(sV), 16, 1024),
                     kQ = umma_desc_split(smem_u32(sQ), 16, 1024),
                     kDO = umma_desc_split(smem_u32(sQ) + Cfg::kTileBytes, 16, 1024),
                     kP = umma_desc_split(smem_u32(sP), 16, 1024);
      const UmmaDesc mQ = umma_desc_split(smem_u32(sQ), kSubTileBytes, 1024),
                     mDO = umma_desc_split(smem_u32(sQ) + Cfg::kTileBytes, kSubTileBytes, 1024);
      // D[128 x 128] = A[128 x kD] * B[128 x kD]^T, both K-major
      auto issue_kmajor = [&](uint32_t d_tmem, const UmmaDesc& a, const UmmaDesc& bd, uint32_t b_stage_lo) {
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = umma_off((kk >> 2) * kSubTileBytes + (kk & 3) * 32);
          if (kk == 0) umma_ss_fast<false>(d_tmem, a.lo + off, a.hi, bd.lo + b_stage_lo + off, bd.hi, idesc_st);
          else         umma_ss_fast<true>(d_tmem, a.lo + off, a.hi, bd.lo + b_stage_lo + off, bd.hi, idesc_st);
        }
      };
      constexpr uint32_t kStageLo = umma_off(2 * Cfg::kTileBytes);
      if (warp == 16) {
        B200FA_WAIT(kv_full, 0, 0x700);
        for (int i = 0; i < steps; ++i) {
          const int stage = i % Cfg::kStages;
          B200FA_WAIT(&q_full[stage], static_cast<uint32_t>((i / Cfg::kStages) & 1), 0x711);
          // the dK MMA of step i - 2 must have consumed dS^T from this work buffer
          if (i >= 2) { B200FA_WAIT(&buf_free[i & 1], ((i >> 1) - 1) & 1, 0x714); }
          tc_fence_after();
          issue_kmajor(tWork + (i & 1) * 128, kK, kQ, stage * kStageLo);
          umma_commit(&s_full[i & 1]);
        }
      } else if (warp == 17) {
        B200FA_WAIT(kv_full, 0, 0x720);
        if (steps > 0) {
          B200FA_WAIT(&do_full[0], 0, 0x702);
          B200FA_WAIT(s_free, 0, 0x703);     // dP^T goes where S^T was once it sits in registers
          tc_fence_after();
          issue_kmajor(tWork, kV, kDO, 0);
          umma_commit(dp_full);
        }
        for (int i = 0; i < steps; ++i) {
          const int stage = i % Cfg::kStages;
          const uint32_t stage_lo = stage * kStageLo;
          // dK += dS^T Q   (A = 16-bit dS^T in the work buffer)
          const uint32_t tDP = tWork + (i & 1) * 128;
          B200FA_WAIT(&q_full[stage], static_cast<uint32_t>((i / Cfg::kStages) & 1), 0x716);
          B200FA_WAIT(ds_full, i & 1, 0x712);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t a_col = (kk >> 1) * 32 + (kk & 1) * 8;
            const uint32_t b_lo = mQ.lo + stage_lo + umma_off(kk * 2048);
            if (kk == 0 && i == 0) umma_ts_fast<false>(tDK, tDP + a_col, b_lo, mQ.hi, idesc_acc);
            else                   umma_ts_fast<true>(tDK, tDP + a_col, b_lo, mQ.hi, idesc_acc);
          }
          umma_commit(&qdo_empty[stage]);   // this lane is done with Q_i (dK) and dO_i (dP^T)
          umma_commit(&buf_free[i & 1]);
          if (i + 1 < steps) {
            // dP^T of the next step replaces S^T of the next step in the other work buffer
            const int nstage = (i + 1) % Cfg::kStages;
            B200FA_WAIT(&do_full[nstage], static_cast<uint32_t>(((i + 1) / Cfg::kStages) & 1), 0x713);
            B200FA_WAIT(s_free, (i + 1) & 1, 0x717);
            tc_fence_after();
            issue_kmajor(tWork + ((i + 1) & 1) * 128, kV, kDO, nstage * kStageLo);
            umma_commit(dp_full);
          }
        }
        umma_commit(acc_full);
      } else {
        for (int i = 0; i < steps; ++i) {
          const int stage = i % Cfg::kStages;
          const uint32_t stage_lo = stage * kStageLo;
          // dV += P^T dO   (A = P^T tile in shared memory, K-major over the query index)
          B200FA_WAIT(&do_full[stage], static_cast<uint32_t>((i / Cfg::kStages) & 1), 0x715);
          B200FA_WAIT(p_full, i & 1, 0x710);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t a_off = umma_off((kk >> 2) * kSubTileBytes + (kk & 3) * 32);
            const uint32_t b_lo = mDO.lo + stage_lo + umma_off(kk * 2048);
            if (kk == 0 && i == 0) umma_ss_fast<false>(tDV, kP.lo + a_off, kP.hi, b_lo, mDO.hi, idesc_acc);
            else                   umma_ss_fast<true>(tDV, kP.lo + a_off, kP.hi, b_lo, mDO.hi, idesc_acc);
          }
          umma_commit(p_empty);
          umma_commit(&qdo_empty[stage]);   // this lane is done with dO_i; S^T of Q_i completed long ago
        }
        umma_commit(acc_full);
      }
    }
  } else if (warp == 19) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      // step 0 went out before the block-wide synchronisation
      for (int i = 1; i < steps; ++i) {
        if (i >= Cfg::kStages) {
          B200FA_WAIT(&qdo_empty[i % Cfg::kStages], ((i / Cfg::kStages) - 1) & 1, 0x800);
        }
        load_step(i);
      }
    }
  }

teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 16) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------
// dQ kernel.  One CTA = one 128-row query tile of one (batch, query head); it walks the K/V
// tiles up to the causal diagonal.  Thread <-> query row, so lse2 and dpsum are per-thread
// scalars.  TMEM columns: S double-buffered at [0,128) and [128,256) (16-bit dS overwrites
// the buffer it was computed from), dP at [256,384), the dQ accumulator after that.
// ------------------------------------------------------------------------------------------
template <int kD, bool kBf16, bool kCausal, bool kDropout>
__global__ void __launch_bounds__(kThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
              const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
              const __grid_constant__ CUtensorMap mapDQ, const BwdParams p) {
  using Cfg = BwdCfg<kD>;
  constexpr int kTmemS = 0, kTmemDP = 256, kTmemDQ = 384;
  extern __shared__ __align__(1024) uint8_t smem[];
  // K_j is needed twice, a whole step apart (S_j, then dQ += dS_j K_j); V_j only once (dP_j).
  // Separate rings - three K slots, two V slots - keep a full step of TMA prefetch ahead of
  // the tensor pipe within the shared-memory budget.
  uint8_t* sQ = smem + Cfg::kOffResident;
  uint8_t* sDO = sQ + Cfg::kTileBytes;
  uint8_t* sK = smem + Cfg::kOffStream;                       // [3] tiles
  uint8_t* sV = sK + 3 * Cfg::kTileBytes;                     // [2] tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffDqBars);
  uint64_t* q_full = bars;                         // [1]  Q tile
  uint64_t* do_full = q_full + 1;                  // [1]  dO tile
  uint64_t* k_full = do_full + 1;                  // [3]
  uint64_t* k_empty = k_full + 3;                  // [3]
  uint64_t* v_full = k_empty + 3;                  // [2]
  uint64_t* v_empty = v_full + 2;                  // [2]
  uint64_t* s_full = v_empty + 2;                  // [2]  S buffer ready
  uint64_t* dp_full = s_full + 2;                  // dP ready
  uint64_t* ds_full = dp_full + 1;                 // dS written, dP consumed (8 warp arrivals)
  uint64_t* acc_full = ds_full + 1;                // dQ complete
  uint64_t* staged = acc_full + 1;                 // dQ tile staged in shared memory (8 warp arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.S + kTile - 1) / kTile;
  const int m_tile = m_tiles - 1 - static_cast<int>(blockIdx.x);  // heaviest (latest) causal tiles first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int m0 = m_tile * kTile;
  // query row i sees key column j iff j <= i + causal_off: K/V tiles up to the one the tile's
  // last real row still sees (none: dQ of the tile is zero)
  const int nkv_total = (p.Sk + kTile - 1) / kTile;
  int n_tiles = nkv_total;
  if (kCausal) {
    const int last = min(m0 + kTile - 1, p.S - 1) + p.causal_off;
    n_tiles = last < 0 ? 0 : min(nkv_total, last / kTile + 1);
  }

  if (status_is_set(p.status)) return;
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, 0x414c0001u);
    return;
  }
  // Lane 0 of the producer warp sets up the barriers and at once issues the loads the first MMAs
  // wait for (Q and K_0 for S_0 first), so that their latency overlaps the TMEM allocation and the
  // block-wide synchronisation.
  auto load_tile = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int srow, int head) {
    mbar_arrive_expect_tx(bar, Cfg::kTileBytes);
#pragma unroll
    for (int cs = 0; cs < Cfg::kSub; ++cs) tma_load_4d(dst + cs * kSubTileBytes, map, bar, cs * 64, srow, head, b);
  };
  if (warp == 10 && lane == 0) {
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapDO);
    tma_prefetch_desc(&mapV);
    mbar_init(q_full, 1);
    mbar_init(do_full, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 8);
    mbar_init(acc_full, 1);
    mbar_init(staged, 8);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    if (n_tiles > 0) {
      load_tile(&mapQ, sQ, q_full, m0, h);
      load_tile(&mapK, sK, &k_full[0], 0, hk);
      load_tile(&mapDO, sDO, do_full, m0, h);
      load_tile(&mapV, sV, &v_full[0], 0, hk);
    }
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    // =========================== compute warps ===========================
    const int wg = warp >> 2;                      // which 64-column (key) half of the tile
    const int r = (warp & 3) * 32 + lane;          // query row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tDP = tmem_base + lane_off + kTmemDP + wg * 64;
    const float c = p.scale_log2;
    const int64_t stat = (static_cast<int64_t>(b) * p.Hq + h) * p.Spad + m0 + r;  // padded rows exist
    const float nlse2 = p.lse_log2[stat];   // minus lse2
    const float ndps = p.dpsum[stat];       // minus dpsum
    const float2 c2 = make_float2(c, c), nl2 = make_float2(nlse2, nlse2), nd2 = make_float2(ndps, ndps);
    for (int j = 0; j < n_tiles; ++j) {
      const int buf = j & 1;
      const uint32_t tS = tmem_base + lane_off + kTmemS + buf * 128 + wg * 64;
      B200FA_WAIT(&s_full[buf], (j >> 1) & 1, 0x900);
      tc_fence_after();
      float pf[64];
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t s[32];
        tmem_ld32(tS + ch * 32, s);
        tmem_wait_ld();
        const float* sf = reinterpret_cast<const float*>(s);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float2 x = __ffma2_rn(make_float2(sf[2 * e], sf[2 * e + 1]), c2, nl2);
          x = exp2_mufu2(x);
          pf[ch * 32 + 2 * e] = x.x;
          pf[ch * 32 + 2 * e + 1] = x.y;
        }
        // Columns to blank: beyond the causal diagonal, and beyond the last key.  K rows past Sk are
        // zero-filled, so their dS would be multiplied by zero, but with a very negative lse their
        // probability exp2(0 - lse2) overflows the 16-bit dS to inf, and inf * 0 is NaN.
        const bool diagonal = kCausal && j * kTile + kTile - 1 > m0 + p.causal_off;
        const bool past_end = (j + 1) * kTile > p.Sk;
        if (diagonal || past_end) {
          const int col0 = j * kTile + wg * 64 + ch * 32;
          int last_e = 31;   // last visible of these 32
          if (diagonal) last_e = m0 + r + p.causal_off - col0;   // query row r sees a key column only if column <= r + causal_off
          if (past_end) last_e = min(last_e, p.Sk - 1 - col0);
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            if (e > last_e) pf[ch * 32 + e] = 0.f;
          }
        }
      }
      uint32_t keep[2] = {0xffffffffu, 0xffffffffu};   // dropout: bit e of keep[ch] <-> key column ch*32 + e of this half
      if constexpr (kDropout) {
        const int blk = (j * kTile + wg * 64) >> 4;
        const int bh = b * p.Hq + h;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          keep[ch] = dropout_bits16(p.drop, bh, m0 + r, blk + 2 * ch) |
                     (dropout_bits16(p.drop, bh, m0 + r, blk + 2 * ch + 1) << 16);
        }
      }
      B200FA_WAIT(dp_full, j & 1, 0x910);
      tc_fence_after();
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t d[32];
        tmem_ld32(tDP + ch * 32, d);
        tmem_wait_ld();
        const float* df = reinterpret_cast<const float*>(d);
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float g0 = df[2 * e], g1 = df[2 * e + 1];
          if constexpr (kDropout) {
            const uint32_t kb = keep[ch] >> (2 * e);
            g0 = (kb & 1u) ? g0 * p.drop.inv_keep : 0.f;
            g1 = (kb & 2u) ? g1 * p.drop.inv_keep : 0.f;
          }
          const float2 a = __fmul2_rn(make_float2(pf[ch * 32 + 2 * e], pf[ch * 32 + 2 * e + 1]), __fadd2_rn(make_float2(g0, g1), nd2));
          pk[e] = pack2<kBf16>(a.x, a.y);
        }
        tmem_st16(tS + ch * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(ds_full);
    }
    // ---- epilogue: dQ (this warpgroup's half of the head dimension)
    B200FA_WAIT(acc_full, 0, 0x920);
    tc_fence_after();
    {
      // The scaled 16-bit dQ tile is staged in the Q buffer (every MMA that read it has
      // completed) in the swizzled box layout and leaves through TMA stores: whole 128-byte
      // lines, rows past the end of the sequence clipped by the tensor map, and nothing for
      // the CTA to wait on but the read of shared memory.
      constexpr int kHalf = kD / 2;
      const uint32_t tacc = tmem_base + lane_off + kTmemDQ + wg * kHalf;
#pragma unroll
      for (int ch = 0; ch < kHalf / 32; ++ch) {
        uint32_t a[32];
        if (n_tiles > 0) {
          tmem_ld32(tacc + ch * 32, a);
          tmem_wait_ld();
        } else {
          // no key is visible from this query tile: nothing was accumulated, dQ is zero
#pragma unroll
          for (int e = 0; e < 32; ++e) a[e] = 0u;
        }
        const float* af = reinterpret_cast<const float*>(a);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 w;
          w.x = pack2<kBf16>(af[v * 8 + 0] * p.scale, af[v * 8 + 1] * p.scale);
          w.y = pack2<kBf16>(af[v * 8 + 2] * p.scale, af[v * 8 + 3] * p.scale);
          w.z = pack2<kBf16>(af[v * 8 + 4] * p.scale, af[v * 8 + 5] * p.scale);
          w.w = pack2<kBf16>(af[v * 8 + 6] * p.scale, af[v * 8 + 7] * p.scale);
          const int chunk = (wg * kHalf + ch * 32) / 8 + v;   // 16-byte chunk of the row
          *reinterpret_cast<uint4*>(sQ + (chunk >> 3) * kSubTileBytes + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)) = w;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(staged);
      if (threadIdx.x == 0) {
        B200FA_WAIT(staged, 0, 0x921);
#pragma unroll
        for (int cs = 0; cs < Cfg::kSub; ++cs) tma_store_4d(&mapDQ, sQ + cs * kSubTileBytes, cs * 64, m0, h, b);
        tma_store_commit();
        tma_store_wait_read();
      }
    }
  } else if (warp == 8 || warp == 9) {
    // =========================== MMA issuers ===========================
    // Warp 8: dQ += dS_j K_j, then S of tile j+2 into the buffer dS_j just left.
    // Warp 9: dP of tile j+1.  Separate lanes so that neither chain stalls behind the other's
    // operands (an issuing lane is blocked while the tensor pipe is full).
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(kBf16, false, false, 128, 128);   // S, dP
      constexpr uint32_t idesc_dq = umma_idesc(kBf16, false, true, 128, kD);    // dQ (A from TMEM, K MN-major)
      const uint32_t tDP = tmem_base + kTmemDP, tDQ = tmem_base + kTmemDQ;
      const UmmaDesc kQ = umma_desc_split(smem_u32(sQ), 16, 1024), kDO = umma_desc_split(smem_u32(sDO), 16, 1024),
                     kK = umma_desc_split(smem_u32(sK), 16, 1024), kV = umma_desc_split(smem_u32(sV), 16, 1024);
      const UmmaDesc mK = umma_desc_split(smem_u32(sK), kSubTileBytes, 1024);
      auto issue_kmajor = [&](uint32_t d_tmem, const UmmaDesc& a, const UmmaDesc& bd, uint32_t b_slot_lo) {
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = umma_off((kk >> 2) * kSubTileBytes + (kk & 3) * 32);
          if (kk == 0) umma_ss_fast<false>(d_tmem, a.lo + off, a.hi, bd.lo + b_slot_lo + off, bd.hi, idesc_s);
          else         umma_ss_fast<true>(d_tmem, a.lo + off, a.hi, bd.lo + b_slot_lo + off, bd.hi, idesc_s);
        }
      };
      constexpr uint32_t kTileLo = umma_off(Cfg::kTileBytes);
      if (warp == 8) {
        // prologue: S_0, S_1
        if (n_tiles > 0) {
          B200FA_WAIT(q_full, 0, 0xa00);
          B200FA_WAIT(&k_full[0], 0, 0xa01);
          tc_fence_after();
          issue_kmajor(tmem_base + kTmemS, kQ, kK, 0);
          umma_commit(&s_full[0]);
        }
        if (n_tiles > 1) {
          B200FA_WAIT(&k_full[1], 0, 0xa02);
          tc_fence_after();
          issue_kmajor(tmem_base + kTmemS + 128, kQ, kK, kTileLo);
          umma_commit(&s_full[1]);
        }
        int kslot = 0;  // ring slot of K_j
        for (int j = 0; j < n_tiles; ++j) {
          const int buf = j & 1;
          const uint32_t tSj = tmem_base + kTmemS + buf * 128;
          const int k2slot = (kslot == 0) ? 2 : kslot - 1;   // slot of K_{j+2} = (j + 2) % 3
          // compute has written dS_j over S_j
          B200FA_WAIT(ds_full, j & 1, 0xa10);
          tc_fence_after();
          // dQ += dS_j K_j   (A = 16-bit dS in the S_j columns, B = K_j rows as the contraction index)
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t a_col = (kk < 4) ? kk * 8 : 64 + (kk - 4) * 8;
            const uint32_t b_lo = mK.lo + kslot * kTileLo + umma_off(kk * 2048);
            if (kk == 0 && j == 0) umma_ts_fast<false>(tDQ, tSj + a_col, b_lo, mK.hi, idesc_dq);
            else                   umma_ts_fast<true>(tDQ, tSj + a_col, b_lo, mK.hi, idesc_dq);
          }
          umma_commit(&k_empty[kslot]);
          if (j + 2 < n_tiles) {
            // S of tile j+2 re-uses this S buffer
            B200FA_WAIT(&k_full[k2slot], static_cast<uint32_t>(((j + 2) / 3) & 1), 0xa11);
            tc_fence_after();
            issue_kmajor(tSj, kQ, kK, k2slot * kTileLo);
            umma_commit(&s_full[buf]);
          }
          if (++kslot == 3) kslot = 0;
        }
        umma_commit(acc_full);
      } else if (n_tiles > 0) {
        // dP_0, then dP_{j+1} whenever the compute warps have consumed dP_j
        B200FA_WAIT(do_full, 0, 0xa20);
        B200FA_WAIT(&v_full[0], 0, 0xa03);
        tc_fence_after();
        issue_kmajor(tDP, kDO, kV, 0);
        umma_commit(dp_full);
        umma_commit(&v_empty[0]);
        for (int j = 0; j + 1 < n_tiles; ++j) {
          const int vslot = (j + 1) & 1;
          B200FA_WAIT(&v_full[vslot], ((j + 1) >> 1) & 1, 0xa12);
          B200FA_WAIT(ds_full, j & 1, 0xa13);
          tc_fence_after();
          issue_kmajor(tDP, kDO, kV, vslot * kTileLo);
          umma_commit(dp_full);
          umma_commit(&v_empty[vslot]);
        }
      }
    }
  } else if (warp == 10) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      // K_0 and V_0 went out before the block-wide synchronisation
      int kslot = 1;
      for (int j = 1; j < n_tiles; ++j) {
        if (j >= 3) { B200FA_WAIT(&k_empty[kslot], static_cast<uint32_t>((j / 3 - 1) & 1), 0xb00); }
        load_tile(&mapK, sK + kslot * Cfg::kTileBytes, &k_full[kslot], j * kTile, hk);
        const int vslot = j & 1;
        if (j >= 2) { B200FA_WAIT(&v_empty[vslot], ((j >> 1) - 1) & 1, 0xb01); }
        load_tile(&mapV, sV + vslot * Cfg::kTileBytes, &v_full[vslot], j * kTile, hk);
        if (++kslot == 3) kslot = 0;
      }
    }
  }

teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}
#undef B200FA_WAIT

// ------------------------------------------------------------------------------------------
// preprocess: dpsum = rowsum(dO * O), lse2 = lse * log2(e), per (b, h, row), padded to a
// multiple of 128 rows, both stored negated.  Rows in [S, Spad) get -lse2 = -inf and dpsum = 0 so their
// probabilities vanish.  One row per group of D/8 lanes; every lane moves 16 bytes of O and dO.
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
    p.dpsum[row_global] = (s < p.S) ? -acc : 0.f;
    // a row that saw no key (lse = -inf) gets -lse2 = -inf like the padding rows: its probabilities vanish
    float l2 = -INFINITY;
    if (s < p.S) {
      const float l = p.lse[(static_cast<int64_t>(b) * p.Hq + h) * p.S + s];
      if (l != -INFINITY) l2 = l * -1.4426950408889634f;
    }
    p.lse_log2[row_global] = l2;
  }
}

// The dK/dV kernel and the dQ kernel only depend on the preprocess kernel, not on each other.
// Run back to back on one stream, the second cannot start until the last, partly idle wave of
// the first has drained; forked onto a side stream its CTAs fill those SMs as they free up.
// Every device owns a small pool of side streams, each with a fork/join event pair, created on
// first use and kept until the process exits; the caller's stream handle picks the pool entry,
// so backward passes issued on different streams do not queue behind one another.  The mutex
// covers one call's record / wait / launch / record / wait sequence on an entry.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool tried = false;
  std::mutex mutex;
};
constexpr int kSidePool = 4;
SideStream* side_stream_for(int dev, cudaStream_t caller) {
  static SideStream pool[64][kSidePool];
  if (dev < 0 || dev >= 64) return nullptr;
  const uintptr_t h = reinterpret_cast<uintptr_t>(caller);
  SideStream& s = pool[dev][(h >> 4 ^ h >> 12) % kSidePool];
  std::lock_guard<std::mutex> lock(s.mutex);
  if (!s.tried) {
    s.tried = true;
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      s.stream = nullptr;
    }
  }
  return s.stream ? &s : nullptr;
}

// cudaFuncSetAttribute for one kernel, once per device, safe against concurrent first calls.
// `once` and `result` belong to the kernel (the caller keeps them as statics of the function
// template that names it: kernels of the same signature must not share them).
template <typename Kernel>
cudaError_t allow_dynamic_smem(Kernel kern, int bytes, std::once_flag (&once)[64], cudaError_t (&result)[64]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  std::call_once(once[dev], [&] {
    result[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  });
  return result[dev];
}

template <int kD, bool kBf16, bool kCausal, bool kDropout>
cudaError_t launch_one(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                       const CUtensorMap& mdq, const CUtensorMap& mdk, const CUtensorMap& mdv, const BwdParams& p,
                       cudaStream_t stream) {
  using Cfg = BwdCfg<kD>;
  cudaError_t e = cudaSuccess;
  auto k1 = bwd_dkdv_kernel<kD, kBf16, kCausal, kDropout>;
  auto k2 = bwd_dq_kernel<kD, kBf16, kCausal, kDropout>;
  static std::once_flag once1[64], once2[64];
  static cudaError_t result1[64], result2[64];
  if ((e = allow_dynamic_smem(k1, Cfg::kSmemBytes, once1, result1)) != cudaSuccess) return e;
  if ((e = allow_dynamic_smem(k2, Cfg::kSmemBytes, once2, result2)) != cudaSuccess) return e;
  if (p.parts & 1) {
    constexpr int kRowsPerWarp = 32 / (kD / 8);
    const int64_t total_rows = static_cast<int64_t>(p.B) * p.Hq * p.Spad;
    const int64_t pre_warps = (total_rows + kRowsPerWarp - 1) / kRowsPerWarp;
    bwd_preprocess_kernel<kD, kBf16><<<static_cast<unsigned>((pre_warps + 7) / 8), 256, 0, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  const int tiles = (p.S + kTile - 1) / kTile;        // query tiles: the dQ kernel's grid
  const int kv_tiles = (p.Sk + kTile - 1) / kTile;    // K/V tiles: the dK/dV kernel's grid
  // fork: the dQ kernel goes to the side stream, behind everything enqueued so far.  Only
  // causal problems: their CTAs differ in length, which is what leaves a long partly idle tail;
  // with equal CTAs the tail is short and interleaving the two kernels only costs L2 hits.
  SideStream* side = (kCausal && (p.parts & 6) == 6 && !(p.parts & 8)) ? side_stream_for(dev, stream) : nullptr;
  std::unique_lock<std::mutex> side_lock;
  if (side) {
    side_lock = std::unique_lock<std::mutex>(side->mutex);
    e = cudaEventRecord(side->fork, stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(side->stream, side->fork, 0);
    if (e != cudaSuccess) return e;   // nothing has been enqueued on the side stream yet
  }
  if (p.parts & 2) {
    // (batch, kv head) pairs whose streamed Q / dO rows (both, all query heads of the pair)
    // add up to about 48 MiB share a scheduling group
    const int64_t pair_bytes = static_cast<int64_t>(p.Hq / p.Hkv) * p.S * p.D * 2 * 2;
    int64_t sched_group = (48ll << 20) / (pair_bytes > 0 ? pair_bytes : 1);
    const int64_t pairs = static_cast<int64_t>(p.B) * p.Hkv;
    if (sched_group < 1) sched_group = 1;
    if (sched_group > pairs) sched_group = pairs;
    k1<<<static_cast<unsigned>(kv_tiles * pairs), kDkdvThreads, Cfg::kSmemBytes, stream>>>(
        mq, mk, mv, mdo, mdk, mdv, p, static_cast<int>(sched_group));
    e = cudaGetLastError();
  }
  if (e == cudaSuccess && (p.parts & 4)) {
    k2<<<dim3(tiles, p.Hq, p.B), kThreads, Cfg::kSmemBytes, side ? side->stream : stream>>>(mq, mk, mv, mdo, mdq, p);
    e = cudaGetLastError();
  }
  if (side) {
    // join, whatever happened in between: once the side stream has been made to wait on the
    // caller's stream it must flow back into it (a stream capture would otherwise stay forked)
    cudaError_t e2 = cudaEventRecord(side->join, side->stream);
    if (e2 == cudaSuccess) e2 = cudaStreamWaitEvent(stream, side->join, 0);
    if (e == cudaSuccess) e = e2;
  }
  return e;
}

template <int kD, bool kBf16>
cudaError_t launch_mask(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mdo,
                        const CUtensorMap& mdq, const CUtensorMap& mdk, const CUtensorMap& mdv, const BwdParams& p,
                        cudaStream_t stream) {
  const bool drop = p.drop.threshold != 0;
  if (p.causal) {
    return drop ? launch_one<kD, kBf16, true, true>(mq, mk, mv, mdo, mdq, mdk, mdv, p, stream)
                : launch_one<kD, kBf16, true, false>(mq, mk, mv, mdo, mdq, mdk, mdv, p, stream);
  }
  return drop ? launch_one<kD, kBf16, false, true>(mq, mk, mv, mdo, mdq, mdk, mdv, p, stream)
              : launch_one<kD, kBf16, false, false>(mq, mk, mv, mdo, mdq, mdk, mdv, p, stream);
}

}  // namespace

cudaError_t launch_bwd_sm100(const BwdParams& p, int dtype, cudaStream_t stream, int* launches) {
  const bool bf16 = (dtype == kBF16);
  CUtensorMap mq, mk, mv, mdo, mdq, mdk, mdv;
  if (!encode_map_16bit(&mq, p.q, p.B, p.Hq, p.S, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mk, p.k, p.B, p.Hkv, p.Sk, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mv, p.v, p.B, p.Hkv, p.Sk, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mdo, p.dout, p.B, p.Hq, p.S, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mdq, p.dq, p.B, p.Hq, p.S, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mdk, p.dk, p.B, p.Hkv, p.Sk, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mdv, p.dv, p.B, p.Hkv, p.Sk, p.D, kTile, bf16)) return cudaErrorInvalidValue;
  cudaError_t e;
  if (p.D == 128) {
    e = bf16 ? launch_mask<128, true>(mq, mk, mv, mdo, mdq, mdk, mdv, p, stream)
             : launch_mask<128, false>(mq, mk, mv, mdo, mdq, mdk, mdv, p, stream);
  } else {
    e = bf16 ? launch_mask<64, true>(mq, mk, mv, mdo, mdq, mdk, mdv, p, stream)
             : launch_mask<64, false>(mq, mk, mv, mdo, mdq, mdk, mdv, p, stream);
  }
  if (e == cudaSuccess && launches) *launches += (p.parts & 1) + ((p.parts >> 1) & 1) + ((p.parts >> 2) & 1);
  return e;
}

}  // namespace b200fa
