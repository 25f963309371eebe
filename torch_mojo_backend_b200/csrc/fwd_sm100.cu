// Forward flash attention for sm_100a: TMA-staged Q/K/V tiles in 128-byte-swizzled shared
// memory feed tcgen05 MMAs whose S and O accumulators live in tensor memory.
//
// Computes what the reference's fwd_fa4_kernel computes
// (torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:530-543, 650-861, 1014-1022,
// 1138-1160): S = Q K^T, causal mask, online softmax in the exp2 domain with
// c = scale*log2(e), P rounded to the 16-bit input type before P V, O / rowsum and
// LSE = rowmax*scale + ln(rowsum).  The structure is new: one CTA owns TWO 128-row query
// tiles of one (batch, head) and ping-pongs them through the tensor core, and a CTA that has
// finished its work item can take over the work item of a thread block that has not started
// yet (cluster launch control), so that barriers, tensor memory and the K/V ring are set up
// once per SM and the output of one item drains while the next item's first MMAs run.
//
//   warps 0-3   softmax of query tile 0   (thread i <-> TMEM lane i <-> query row i)
//   warps 4-7   softmax of query tile 1
//   warps 8-11  correction: rescale O in TMEM when a row max moved; epilogue: O / l staged in
//               shared memory and written with TMA stores, LSE
//   warps 12-13 MMA issuers, one per query tile (one elected lane each issues tcgen05.mma / commit)
//   warp  14    TMA producer (Q, then a ring of K/V tiles); also asks for the next work item
//   warp  15    idle (it only donates registers)
//
// TMEM columns: S0 | S1 | O0 | O1.  P (16-bit, two per column) overwrites the first half of
// its own S columns and is consumed as the TMEM A-operand of the P V MMA.
#include <mutex>

#include "common.cuh"
#include "philox.cuh"
#include "ptx.cuh"

namespace b200fa {
namespace {

constexpr int kBM = 128;        // query rows per tile
constexpr int kBN = 128;        // key rows per tile
constexpr int kThreads = 512;
constexpr int kSubTileBytes = 128 * 128;  // one 128-row x 64-column (128 B) swizzled box

// Lazy rescaling threshold (log2 domain): O and l are only rescaled when the running row
// maximum grows by more than this, so P can be as large as 2^8 against a stale maximum.
constexpr float kRescaleLog2 = 8.f;

// Of every 8 column pairs, this many take their exponentials on the FMA pipe (range reduction
// + cubic) instead of the special-function unit, which delivers 16 exponentials per clock per
// SM: exactly what the two query tiles of a CTA need while their MMAs run.
#ifndef B200FA_EMU_OF8
#define B200FA_EMU_OF8 0
#endif
constexpr int kEmuOf8 = B200FA_EMU_OF8;

// 2^x for x <= ~127 on the FMA pipe, two values at a time: x = n + f with n = floor(x),
// 2^f by a cubic fitted on [0,1) (max relative error 8.7e-5, far below 16-bit rounding of
// P), and n added straight into the exponent field.
#ifdef B200FA_X_NOFMAX3
#define fmax3(a, b, c) fmaxf(fmaxf((a), (b)), (c))
#endif
__device__ __forceinline__ float2 exp2_emulated2(float2 x) {
  const float kMagic = 12582912.f;  // 1.5 * 2^23: x + kMagic (rounded down) holds floor(x) in its low mantissa bits
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 xi = __fadd2_rd(x, make_float2(kMagic, kMagic));
  const float2 fl = __fadd2_rn(xi, make_float2(-kMagic, -kMagic));
  const float2 f = __fadd2_rn(x, make_float2(-fl.x, -fl.y));
  float2 r = __ffma2_rn(make_float2(0.07705805f, 0.07705805f), f, make_float2(0.22764558f, 0.22764558f));
  r = __ffma2_rn(r, f, make_float2(0.69512289f, 0.69512289f));
  r = __ffma2_rn(r, f, make_float2(1.f, 1.f));
  r.x = __int_as_float(__float_as_int(r.x) + (__float_as_int(xi.x) << 23));
  r.y = __int_as_float(__float_as_int(r.y) + (__float_as_int(xi.y) << 23));
  return r;
}

template <int kD>
struct FwdCfg {
  static constexpr int kTileBytes = kBM * kD * 2;
  static constexpr int kSub = kD / 64;                  // 64-column boxes per tile
  static constexpr int kStages = (kD == 128) ? 4 : 8;   // K/V ring slots
  static constexpr int kTmemS0 = 0, kTmemS1 = 128, kTmemO0 = 256, kTmemO1 = 256 + kD;
  static constexpr int kNumBars = 2 + 2 + 2 * kStages + 2 + 4 + 2 + 2 + 2 + 2 + 2 + 2;
  // Q tiles | K/V ring | output staging tile | messages | barriers | next-item answers
  static constexpr int kOffKV = 2 * kTileBytes;
  static constexpr int kOffStage = kOffKV + kStages * kTileBytes;
  static constexpr int kOffMsg = kOffStage + kTileBytes;
  static constexpr int kOffBars = kOffMsg + 4 * 128 * 4;
  static constexpr int kOffClc = kOffBars + kNumBars * 8;
  static constexpr int kSmemBytes = kOffClc + 2 * 16 + 16;
};

// How a CTA finds the work item after the one its block index names.
constexpr int kSchedOnePerCta = 0;   // it does not: one item per thread block
constexpr int kSchedSteal = 1;       // it cancels a thread block that has not started and takes its index
constexpr int kSchedStride = 2;      // grid of one CTA per SM, items taken with a stride of the grid size

struct FwdSched {
  int npairs;      // 256-row query pairs per (b, h)
  int group;       // heads scheduled together so their K/V stay L2-resident
  int nkv_total;   // ceil(Sk / 128)
  int total_items; // npairs * B * Hq
  int mode;        // kSched*
};

struct Item {
  int b, h, hk, row0;
  int n_t[2];   // KV tiles each query tile visits
  int n_max;
};

template <int kD, bool kBf16, bool kCausal, bool kDropout>
__global__ void __launch_bounds__(kThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
           const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO, const FwdParams p,
           const FwdSched sched) {
  using Cfg = FwdCfg<kD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;                                   // 2 tiles
  uint8_t* sKV = smem + Cfg::kOffKV;                    // ring
  uint8_t* sStage = smem + Cfg::kOffStage;              // 16-bit output tile on its way to global memory
  float* sMsg = reinterpret_cast<float*>(smem + Cfg::kOffMsg);  // [2][128]
  float* sMax = sMsg + 256;                             // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBars);
  uint64_t* q_full = bars;                      // [2]
  uint64_t* q_empty = q_full + 2;               // [2] the last Q K^T of an item has read the Q tile
  uint64_t* kv_full = q_empty + 2;              // [kStages]
  uint64_t* kv_empty = kv_full + Cfg::kStages;  // [kStages]
  uint64_t* s_full = kv_empty + Cfg::kStages;   // [2]
  uint64_t* p_full = s_full + 2;                // [2 tiles][2 halves of the KV columns]
  uint64_t* o_full = p_full + 4;                // [2]
  uint64_t* sc_full = o_full + 2;               // [2]
  uint64_t* sc_empty = sc_full + 2;             // [2]
  uint64_t* turn = sc_empty + 2;                // [2] MMA issuers' turn-taking
  uint64_t* clc_full = turn + 2;                // [2] the answer to "which item next" has arrived
  uint64_t* clc_empty = clc_full + 2;           // [2] every role has read that answer
  uint4* clc_resp = reinterpret_cast<uint4*>(smem + Cfg::kOffClc);   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(clc_resp + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // A launch whose status word already reports a failed wait is not worth running; the swizzled
  // tiles assume a 1024-byte aligned shared-memory window.
  if (status_is_set(p.status)) return;
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, kStatusOk, 0x414c0002u);
    return;
  }

  // ---- work item w -> (pair, head, batch): head groups keep K/V in L2, and inside a group
  // the heaviest (latest) causal pairs come first.
  const int total_bh = p.B * p.Hq;
  auto decode = [&](int w, Item& it) {
    const int per_group = sched.group * sched.npairs;
    const int g = w / per_group;
    const int gsize = min(sched.group, total_bh - g * sched.group);
    const int within = w - g * per_group;
    const int pair = sched.npairs - 1 - within / gsize;
    const int bh = g * sched.group + within % gsize;
    it.b = bh / p.Hq;
    it.h = bh - it.b * p.Hq;
    it.hk = it.h / (p.Hq / p.Hkv);
    it.row0 = pair * 2 * kBM;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int r0 = it.row0 + t * kBM;
      int n;
      if (r0 >= p.Sq) {
        n = 0;
      } else if (kCausal) {
        // the tile's last real row sees key columns 0 .. row + causal_off; a tile none of whose
        // rows sees a key still runs one fully masked step so that it writes zeros and -inf
        const int last = min(r0 + kBM - 1, p.Sq - 1) + p.causal_off;
        n = last < 0 ? 1 : min(sched.nkv_total, last / kBN + 1);
      } else {
        n = sched.nkv_total;
      }
      it.n_t[t] = n;
    }
    it.n_max = max(it.n_t[0], it.n_t[1]);
  };

  // Every role walks the same sequence of items.  `k` counts the items this CTA has finished;
  // the answer to request k (which item comes after item k) sits in answer slot k & 1.
  // Returns the next item index, or -1 when there is none (or the CTA is aborting).
  constexpr int kRoleWarp = 0, kRoleLane = 1, kRoleRequester = 2;
  auto next_item = [&](int w, int k, int role) -> int {
    if (sched.mode == kSchedOnePerCta) return -1;
    if (sched.mode == kSchedStride) {
      const int n = w + static_cast<int>(gridDim.x);
      return n < sched.total_items ? n : -1;
    }
    const int slot = k & 1;
    if (!mbar_wait(&clc_full[slot], (k >> 1) & 1, abort_flag, p.status, 0x600, p.wait_budget)) return -1;
    const uint4 r = clc_resp[slot];
    uint32_t canceled, x;
    asm volatile(
        "{\n\t.reg .b128 resp;\n\t.reg .pred pc;\n\t"
        "mov.b128 resp, {%2, %3};\n\t"
        "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 pc, resp;\n\t"
        "selp.u32 %0, 1, 0, pc;\n\t"
        "mov.u32 %1, 0;\n\t"
        "@pc clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %1, resp;\n\t}"
        : "=r"(canceled), "=r"(x)
        : "l"(static_cast<uint64_t>(r.x) | (static_cast<uint64_t>(r.y) << 32)),
          "l"(static_cast<uint64_t>(r.z) | (static_cast<uint64_t>(r.w) << 32)));
    if (role != kRoleRequester) {
      // this reader's use of the answer is ordered before the slot's next (asynchronous) overwrite
      fence_proxy_async_smem();
      if (role == kRoleWarp) mbar_arrive_warp(&clc_empty[slot]);
      else mbar_arrive(&clc_empty[slot]);
    }
    return canceled ? static_cast<int>(x) : -1;
  };

  Item it;
  int w = blockIdx.x;
  decode(w, it);

  auto load_tile = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int srow, int head, int b) {
    mbar_arrive_expect_tx(bar, Cfg::kTileBytes);
#pragma unroll
    for (int cs = 0; cs < Cfg::kSub; ++cs) {
      tma_load_4d(dst + cs * kSubTileBytes, map, bar, cs * 64, srow, head, b);
    }
  };
  // Asks the hardware to cancel a thread block of this grid that has not started and to hand
  // over its block index: the answer (16 bytes) lands in clc_resp[slot] and completes
  // clc_full[slot].  Only ever called after the previous request succeeded.
  auto request_next = [&](int k) -> bool {
    if (sched.mode != kSchedSteal) return true;
    const int slot = k & 1;
    if (k >= 2) {
      if (!mbar_wait(&clc_empty[slot], ((k >> 1) - 1) & 1, abort_flag, p.status, 0x601, p.wait_budget)) return false;
    }
    fence_proxy_async_smem();
    mbar_arrive_expect_tx(&clc_full[slot], 16);
    asm volatile(
        "clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
        ::"r"(smem_u32(&clc_resp[slot])), "r"(smem_u32(&clc_full[slot]))
        : "memory");
    return true;
  };

  // Lane 0 of the producer warp sets up the barriers and at once issues the loads that need
  // no free slot and are needed first (Q, K_0, V_0 of the first item), so that their latency
  // overlaps the TMEM allocation and the block-wide synchronisation below.
  constexpr int kEarlyLoads = 2;
  if (warp == 14 && lane == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&q_empty[t], 1);
      mbar_init(&s_full[t], 1);
      // fed by four warps each, one elected arrival per warp
      mbar_init(&p_full[t * 2], 8);      // 4 softmax warps (P half 0) + 4 correction warps (O ready)
      mbar_init(&p_full[t * 2 + 1], 4);
      mbar_init(&o_full[t], 1);
      mbar_init(&sc_full[t], 4);
      mbar_init(&sc_empty[t], 4);
      mbar_init(&turn[t], 1);
      mbar_init(&clc_full[t], 1);
      mbar_init(&clc_empty[t], 14);      // 8 softmax + 4 correction warps + 2 MMA-issuing lanes
    }
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 2);  // released by both query tiles' MMA issuers
    }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    // Q tile 0 rides ahead of K_0, Q tile 1 right behind it, then V_0 (tile 0 always has rows)
    load_tile(&mapQ, sQ, &q_full[0], it.row0, it.h, it.b);
    load_tile(&mapK, sKV, &kv_full[0], 0, it.hk, it.b);
    if (it.n_t[1] > 0) load_tile(&mapQ, sQ + Cfg::kTileBytes, &q_full[1], it.row0 + kBM, it.h, it.b);
    load_tile(&mapV, sKV + Cfg::kTileBytes, &kv_full[1], 0, it.hk, it.b);
  }
  if (warp == 12) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

#define B200FA_WAIT(bar, parity, site) \
  if (!mbar_wait((bar), (parity), abort_flag, p.status, (site), p.wait_budget)) goto teardown

  if (warp < 8) {
    // =========================== softmax warps ===========================
    reg_alloc<168>();
    const int t = warp >> 2;
    const int row = threadIdx.x & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_off + (t == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
    const float c = p.scale_log2;
    uint32_t n_s = 0;     // S tiles consumed so far (phase of s_full / p_full)
    uint32_t n_msg = 0;   // messages sent to the correction warps so far (phase of sc_full / sc_empty)
    for (int k = 0;; ++k) {
      const int nblk = it.n_t[t];
      const int q_row = it.row0 + t * kBM + row;  // global query row
      // m: the row maximum the exponentials are taken against.  It is only raised when the
      // true maximum has grown by more than 2^kRescaleLog2 (lazy rescaling), so most KV
      // tiles need no correction of O; l is the row sum relative to that same m.
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < nblk; ++j) {
        B200FA_WAIT(&s_full[t], n_s & 1, 0x100 + t);
        tc_fence_after();
        uint32_t s[128];
        tmem_ld32(tS + 0, s + 0);
        tmem_ld32(tS + 32, s + 32);
        tmem_ld32(tS + 64, s + 64);
        tmem_ld32(tS + 96, s + 96);
        tmem_wait_ld();
        float* sf = reinterpret_cast<float*>(s);
        const int col0 = j * kBN;
        // mask: causal diagonal tile and/or columns beyond Sk
        const bool need_mask =
            (kCausal && (col0 + kBN - 1 > it.row0 + t * kBM + p.causal_off)) || (col0 + kBN > p.Sk);
        if (need_mask) {
          const int limit = kCausal ? min(q_row + p.causal_off, p.Sk - 1) : (p.Sk - 1);  // last visible column
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            if (col0 + i > limit) sf[i] = -INFINITY;
          }
        }
        // row max: four independent chains of three-input maxima
        float mx0 = fmax3(sf[0], sf[1], sf[2]), mx1 = fmax3(sf[3], sf[4], sf[5]);
        float mx2 = fmax3(sf[6], sf[7], sf[8]), mx3 = fmax3(sf[9], sf[10], sf[11]);
#pragma unroll
        for (int i = 12; i < 124; i += 8) {
          mx0 = fmax3(mx0, sf[i], sf[i + 1]);
          mx1 = fmax3(mx1, sf[i + 2], sf[i + 3]);
          mx2 = fmax3(mx2, sf[i + 4], sf[i + 5]);
          mx3 = fmax3(mx3, sf[i + 6], sf[i + 7]);
        }
        mx0 = fmax3(mx0, sf[124], sf[125]);
        mx1 = fmax3(mx1, sf[126], sf[127]);
        float m_new = fmax3(fmaxf(mx0, mx1), fmaxf(mx2, mx3), m);
        // rows past the end of the sequence (or fully masked) must not produce NaN
        if (m_new == -INFINITY) m_new = 0.f;
        float sc = 1.f;
        if ((m_new - m) * c > kRescaleLog2) {  // always true on the first tile (m = -inf)
          sc = ex2_approx((m - m_new) * c);
          m = m_new;
        }
        if (n_msg > 0) {
          B200FA_WAIT(&sc_empty[t], (n_msg - 1) & 1, 0x110 + t);
        }
        sMsg[t * 128 + row] = sc;
        mbar_arrive_warp(&sc_full[t]);
        ++n_msg;
        const float mc = m * c;
        const float2 c2 = make_float2(c, c);
        const float2 nmc2 = make_float2(-mc, -mc);
        float2 rsa = make_float2(0.f, 0.f), rsb = make_float2(0.f, 0.f);
        uint32_t pk[64];
        uint32_t keep_bits[4] = {0, 0, 0, 0};   // dropout: one bit per column of this row of the tile
        if constexpr (kDropout) {
          dropout_row_bits(p.drop, it.b * p.Hq + it.h, q_row, col0, keep_bits);
        }
        // P leaves in four 32-column quarters.  The wait for a quarter's store to land is put off
        // until the next quarter's exponentials have been issued, and the MMA lane is told about
        // a half (two quarters) at a time: P V starts on the first half while the second is
        // still being exponentiated.
#ifdef B200FA_X_HALVES
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int i = half * 32; i < half * 32 + 32; ++i) {
            const float2 x = __ffma2_rn(make_float2(sf[2 * i], sf[2 * i + 1]), c2, nmc2);
            float2 pv;
            if ((i & 7) < kEmuOf8) {
              pv = exp2_emulated2(x);
            } else {
              pv = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            }
            if (i & 1) rsb = __fadd2_rn(rsb, pv); else rsa = __fadd2_rn(rsa, pv);
            pk[i] = pack2<kBf16>(pv.x, pv.y);
          }
          tmem_st32(tS + half * 32, pk + half * 32);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive_warp(&p_full[t * 2 + half]);
        }
#else
#pragma unroll
        for (int qt = 0; qt < 4; ++qt) {
#pragma unroll
          for (int i = qt * 16; i < qt * 16 + 16; ++i) {
            const float2 x = __ffma2_rn(make_float2(sf[2 * i], sf[2 * i + 1]), c2, nmc2);
            float2 pv;
            if ((i & 7) < kEmuOf8) {
              pv = exp2_emulated2(x);
            } else {
              pv = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            }
            if (i & 1) rsb = __fadd2_rn(rsb, pv); else rsa = __fadd2_rn(rsa, pv);
            if constexpr (kDropout) {
              // the row sum keeps every probability; only what feeds P V is dropped
              const uint32_t bits = keep_bits[i >> 4] >> ((2 * i) & 31);
              if (!(bits & 1u)) pv.x = 0.f;
              if (!(bits & 2u)) pv.y = 0.f;
            }
            pk[i] = pack2<kBf16>(pv.x, pv.y);
          }
          if (qt == 2) {
            // quarters 0 and 1 were stored a quarter's worth of exponentials ago
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&p_full[t * 2]);
          }
          tmem_st16(tS + qt * 16, pk + qt * 16);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&p_full[t * 2 + 1]);
#endif
        l = l * sc + ((rsa.x + rsa.y) + (rsb.x + rsb.y));
        ++n_s;
      }
      if (nblk > 0) {
        B200FA_WAIT(&sc_empty[t], (n_msg - 1) & 1, 0x120 + t);
        sMsg[t * 128 + row] = l;
        sMax[t * 128 + row] = m;
        mbar_arrive_warp(&sc_full[t]);
        ++n_msg;
      }
      w = next_item(w, k, kRoleWarp);
      if (w < 0) break;
      decode(w, it);
    }
  } else if (warp < 12) {
    // =========================== correction warps ===========================
    reg_dealloc<96>();
    const int row = threadIdx.x & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t n_msg[2] = {0, 0};   // messages read so far, per tile
    uint32_t n_s[2] = {0, 0};     // s_full completions of earlier items, per tile
    uint32_t n_o[2] = {0, 0};     // o_full completions consumed so far, per tile
    bool store_pending = false;   // (warp 8, lane 0) a TMA store may still be reading the staging tile
    auto epilogue = [&](int t) -> bool {
      const int nblk = it.n_t[t];
      if (nblk == 0) return true;
      if (!mbar_wait(&sc_full[t], n_msg[t] & 1, abort_flag, p.status, 0x200 + t, p.wait_budget)) return false;
      const float l = sMsg[t * 128 + row];
      const float m = sMax[t * 128 + row];
      mbar_arrive_warp(&sc_empty[t]);
      ++n_msg[t];
      if (!mbar_wait(&o_full[t], n_o[t] & 1, abort_flag, p.status, 0x210 + t, p.wait_budget)) return false;
      ++n_o[t];
      tc_fence_after();
      // a row that saw no key at all (possible under a bottom-right aligned mask) is 0 with lse -inf
      float inv_l = l > 0.f ? 1.f / l : 0.f;
      if constexpr (kDropout) inv_l *= p.drop.inv_keep;
      const int q_row = it.row0 + t * kBM + row;
      const uint32_t tO = tmem_base + lane_off + (t == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
      // The 16-bit output tile is staged in shared memory in the swizzled box layout and leaves
      // through TMA stores: whole 128-byte lines, nothing for the CTA to wait on but the read of
      // shared memory, and rows past the end of the sequence are clipped by the tensor map.
      // The staging tile is free once the previous store has read it.
      if (warp == 8 && lane == 0 && store_pending) tma_store_wait_read();
      named_bar_sync(1, 128);
#pragma unroll
      for (int cidx = 0; cidx < kD / 32; ++cidx) {
        uint32_t o[32];
        tmem_ld32(tO + cidx * 32, o);
        tmem_wait_ld();
        const float* of = reinterpret_cast<const float*>(o);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 wv;
          wv.x = pack2<kBf16>(of[v * 8 + 0] * inv_l, of[v * 8 + 1] * inv_l);
          wv.y = pack2<kBf16>(of[v * 8 + 2] * inv_l, of[v * 8 + 3] * inv_l);
          wv.z = pack2<kBf16>(of[v * 8 + 4] * inv_l, of[v * 8 + 5] * inv_l);
          wv.w = pack2<kBf16>(of[v * 8 + 6] * inv_l, of[v * 8 + 7] * inv_l);
          const int chunk = cidx * 4 + v;   // 16-byte chunk of the row
          *reinterpret_cast<uint4*>(sStage + (chunk >> 3) * kSubTileBytes + row * 128 +
                                    (((chunk & 7) ^ (row & 7)) << 4)) = wv;
        }
      }
      // O has been read out of tensor memory: the next item's first P V may overwrite it once
      // this warp has arrived on that item's p_full (program order in this warp)
      tc_fence_before();
      fence_proxy_async_smem();
      named_bar_sync(1, 128);
      if (warp == 8 && lane == 0) {
#pragma unroll
        for (int cs = 0; cs < Cfg::kSub; ++cs) {
          tma_store_4d(&mapO, sStage + cs * kSubTileBytes, cs * 64, it.row0 + t * kBM, it.h, it.b);
        }
        tma_store_commit();
        store_pending = true;
      }
      if (q_row < p.Sq) {
        p.lse[(static_cast<int64_t>(it.b) * p.Hq + it.h) * p.Sq + q_row] =
            l > 0.f ? m * p.scale + logf(l) : -INFINITY;
      }
      return true;
    };
    for (int k = 0;; ++k) {
      for (int j = 0; j < it.n_max; ++j) {
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < it.n_t[t]) {
            B200FA_WAIT(&sc_full[t], n_msg[t] & 1, 0x220 + t);
            const float sc = sMsg[t * 128 + row];
            mbar_arrive_warp(&sc_empty[t]);
            ++n_msg[t];
            if (j > 0) {
              // Q K^T of tile j was issued after P V of tile j-1, so its commit covers both
              B200FA_WAIT(&s_full[t], (n_s[t] + j) & 1, 0x230 + t);
              tc_fence_after();
              if (__any_sync(0xffffffffu, sc != 1.f)) {
                const uint32_t tO = tmem_base + lane_off + (t == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
#pragma unroll
                for (int cidx = 0; cidx < kD / 32; ++cidx) {
                  uint32_t o[32];
                  tmem_ld32(tO + cidx * 32, o);
                  tmem_wait_ld();
                  float* of = reinterpret_cast<float*>(o);
#pragma unroll
                  for (int i = 0; i < 32; ++i) of[i] *= sc;
                  tmem_st32(tO + cidx * 32, o);
                }
                tmem_wait_st();
              }
            }
            tc_fence_before();
            mbar_arrive_warp(&p_full[t * 2]);
          }
        }
        // a tile that just saw its last KV block can be finished while the other still runs
        if (it.n_t[0] != it.n_t[1] && j == it.n_t[0] - 1) {
          if (!epilogue(0)) goto teardown;
        }
      }
      if (it.n_t[0] == it.n_t[1]) {
        if (!epilogue(0)) goto teardown;
      }
      if (!epilogue(1)) goto teardown;
      n_s[0] += it.n_t[0];
      n_s[1] += it.n_t[1];
      w = next_item(w, k, kRoleWarp);
      if (w < 0) break;
      decode(w, it);
    }
    // the staged output tile must have been read before shared memory is given back
    if (warp == 8 && lane == 0 && store_pending) tma_store_wait_read();
  } else {
    // (all four warps of a warpgroup have to name the same register count)
    reg_dealloc<80>();
    if (warp == 12 || warp == 13) {
      // =========================== MMA issuers (one per query tile) ===========================
      // A tcgen05.mma only issues once the tensor pipe has room, so the issuing lane is stalled
      // for about as long as its MMAs run, and every wait or commit it executes in between is
      // time the pipe could drain.  Giving each query tile its own issuing lane lets one
      // lane's waits overlap the other lane's MMAs.
      const int t = warp - 12;
      if (lane == 0) {
        constexpr uint32_t idesc_qk = umma_idesc(kBf16, false, false, 128, 128);
        constexpr uint32_t idesc_pv = umma_idesc(kBf16, false, true, 128, kD);
        const uint32_t tS = tmem_base + (t == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
        const uint32_t tO = tmem_base + (t == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
        // descriptors are a fixed high word plus a start-address word; stepping along the
        // contraction dimension or to another ring slot only adds to the low word
        const UmmaDesc dQ = umma_desc_split(smem_u32(sQ) + t * Cfg::kTileBytes, 16, 1024);  // K-major Q tile
        const UmmaDesc dK = umma_desc_split(smem_u32(sKV), 16, 1024);             // ring slot as K-major K
        const UmmaDesc dV = umma_desc_split(smem_u32(sKV), kSubTileBytes, 1024);  // ring slot as MN-major V
        auto issue_qk = [&](uint32_t slot_lo) {
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) {
            const uint32_t off = umma_off((kk >> 2) * kSubTileBytes + (kk & 3) * 32);
            if (kk == 0) umma_ss_fast<false>(tS, dQ.lo + off, dQ.hi, dK.lo + slot_lo + off, dK.hi, idesc_qk);
            else         umma_ss_fast<true>(tS, dQ.lo + off, dQ.hi, dK.lo + slot_lo + off, dK.hi, idesc_qk);
          }
        };
        // half 0: KV rows 0-63 of the tile, half 1: rows 64-127 (P arrives in two halves)
        auto issue_pv = [&](uint32_t slot_lo, bool first, int half) {
#pragma unroll
          for (int kq = 0; kq < 4; ++kq) {
            const int kk = half * 4 + kq;
            const uint32_t b_lo = dV.lo + slot_lo + umma_off(kk * 2048);
            if (kk == 0 && first) umma_ts_fast<false>(tO, tS + kk * 8, b_lo, dV.hi, idesc_pv);
            else                  umma_ts_fast<true>(tO, tS + kk * 8, b_lo, dV.hi, idesc_pv);
          }
        };
        // The two issuing lanes take turns: a lane issues one block of MMAs (P V of the
        // current KV tile, then Q K^T of the next) only while it holds the turn, and hands it
        // over before it commits.  That keeps the two query tiles in anti-phase - one tile's
        // MMAs run while the other tile is in softmax - instead of drifting into lockstep.
        // turn[t] completes once per block of the OTHER lane; lane 0 opens.  Both lanes take
        // n_max + 1 turns per item, so the count simply runs on from item to item.
        uint32_t turn_k = 0;
        auto take_turn = [&]() -> bool {
          bool ok = true;
          if (t == 1) ok = mbar_wait(&turn[1], turn_k & 1, abort_flag, p.status, 0x370, p.wait_budget);
          else if (turn_k > 0) ok = mbar_wait(&turn[0], (turn_k - 1) & 1, abort_flag, p.status, 0x371, p.wait_budget);
          ++turn_k;
          return ok;
        };
        // The K/V ring runs on from item to item: `slot`/`phase` name the ring entry of K_0 at
        // the start of an item (entries of an item: K_0 V_0 K_1 V_1 ...).
        int slot = 0;
        uint32_t phase = 0;
        auto advance = [&]() { if (++slot == Cfg::kStages) { slot = 0; phase ^= 1; } };
        uint32_t n_q = 0;   // items in which this query tile took part (phase of q_full)
        uint32_t n_p = 0;   // P tiles consumed so far (phase of p_full)
        for (int k = 0;; ++k) {
          const int nblk = it.n_t[t];
          const int n_max = it.n_max;
          if (nblk > 0) {
            // block 0: S_t = Q_t K_0^T
            B200FA_WAIT(&q_full[t], n_q & 1, 0x301 + t);
            ++n_q;
            B200FA_WAIT(&kv_full[slot], phase, 0x300);
            if (!take_turn()) goto teardown;
            tc_fence_after();
            issue_qk(slot * umma_off(Cfg::kTileBytes));
            mbar_arrive(&turn[1 - t]);
            umma_commit(&s_full[t]);
            umma_commit(&kv_empty[slot]);
            if (nblk == 1) umma_commit(&q_empty[t]);
            advance();   // now at V_0
            for (int j = 0; j < nblk; ++j) {
              const int vslot = slot;
              const uint32_t vphase = phase;
              advance();   // now at K_{j+1}
              const bool has_next = (j + 1 < nblk);
              // everything that can be waited for without holding the turn
              B200FA_WAIT(&kv_full[vslot], vphase, 0x310);
              if (has_next) { B200FA_WAIT(&kv_full[slot], phase, 0x340); }
              B200FA_WAIT(&p_full[t * 2], n_p & 1, 0x320 + t);  // P half 0 written and O ready
              if (!take_turn()) goto teardown;
              tc_fence_after();
              issue_pv(vslot * umma_off(Cfg::kTileBytes), j == 0, 0);
              B200FA_WAIT(&p_full[t * 2 + 1], n_p & 1, 0x324 + t);
              ++n_p;
              tc_fence_after();
              issue_pv(vslot * umma_off(Cfg::kTileBytes), false, 1);
              if (has_next) issue_qk(slot * umma_off(Cfg::kTileBytes));
              mbar_arrive(&turn[1 - t]);
              if (has_next) {
                // also tells the correction warps that P V of tile j has completed
                umma_commit(&s_full[t]);
                umma_commit(&kv_empty[slot]);
                if (j + 2 == nblk) umma_commit(&q_empty[t]);   // that was the item's last Q K^T
              } else {
                umma_commit(&o_full[t]);
              }
              umma_commit(&kv_empty[vslot]);
              if (has_next) advance();   // now at V_{j+1}
            }
            // `slot` now names K_nblk.  KV tiles only the other query tile visits still need this
            // tile's release, and the other lane still needs its turns
            for (int j = nblk; j < n_max; ++j) {
              B200FA_WAIT(&kv_full[slot], phase, 0x350);
              mbar_arrive(&kv_empty[slot]);
              advance();
              B200FA_WAIT(&kv_full[slot], phase, 0x351);
              mbar_arrive(&kv_empty[slot]);
              advance();
              if (!take_turn()) goto teardown;
              mbar_arrive(&turn[1 - t]);
            }
          } else {
            // this query tile lies wholly past the end of the sequence: release each K/V slot
            // as it fills and pass every turn straight back
            for (int blk = 0; blk <= n_max; ++blk) {
              // block blk of the other tile consumes K_0 (blk = 0) or V_{blk-1} and, if there is one, K_blk
              const int n_release = (blk == 0 || blk == n_max) ? 1 : 2;
              for (int r = 0; r < n_release; ++r) {
                B200FA_WAIT(&kv_full[slot], phase, 0x360);
                mbar_arrive(&kv_empty[slot]);
                advance();
              }
              if (!take_turn()) goto teardown;
              mbar_arrive(&turn[1 - t]);
            }
          }
          w = next_item(w, k, kRoleLane);
          if (w < 0) break;
          decode(w, it);
        }
      }
    } else if (warp == 14) {
      // =========================== TMA producer ===========================
      if (lane == 0) {
        // ring entries produced so far, over all items; Q tiles loaded so far, per query tile
        // (the first kEarlyLoads entries and the first Q tiles went out before the synchronisation)
        uint32_t seq = kEarlyLoads;
        uint32_t n_q[2] = {1u, it.n_t[1] > 0 ? 1u : 0u};
        for (int k = 0;; ++k) {
          // ask for the item after this one while this one is being loaded
          if (!request_next(k)) goto teardown;
          const int n_loads = 2 * it.n_max;
          for (int e = (k == 0 ? kEarlyLoads : 0); e < n_loads; ++e, ++seq) {
            const int slot = seq % Cfg::kStages;
            if (seq >= static_cast<uint32_t>(Cfg::kStages)) {
              B200FA_WAIT(&kv_empty[slot], ((seq / Cfg::kStages) - 1) & 1, 0x400);
            }
            uint8_t* dst = sKV + slot * Cfg::kTileBytes;
            if (e == 0) {
              // Q tile 0 rides ahead of K_0, Q tile 1 right behind it; a Q buffer is free once
              // the previous item's last Q K^T on it has completed
              if (n_q[0] > 0) { B200FA_WAIT(&q_empty[0], (n_q[0] - 1) & 1, 0x410); }
              load_tile(&mapQ, sQ, &q_full[0], it.row0, it.h, it.b);
              ++n_q[0];
              load_tile(&mapK, dst, &kv_full[slot], 0, it.hk, it.b);
              if (it.n_t[1] > 0) {
                if (n_q[1] > 0) { B200FA_WAIT(&q_empty[1], (n_q[1] - 1) & 1, 0x411); }
                load_tile(&mapQ, sQ + Cfg::kTileBytes, &q_full[1], it.row0 + kBM, it.h, it.b);
                ++n_q[1];
              }
            } else {
              load_tile((e & 1) ? &mapV : &mapK, dst, &kv_full[slot], (e >> 1) * kBN, it.hk, it.b);
            }
          }
          w = next_item(w, k, kRoleRequester);
          if (w < 0) break;
          decode(w, it);
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
cudaError_t launch_one(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                       const FwdParams& p, const FwdSched& sched, cudaStream_t stream) {
  using Cfg = FwdCfg<kD>;
  auto kern = fwd_kernel<kD, kBf16, kCausal, kDropout>;
  static std::once_flag once[64];
  static cudaError_t result[64];
  cudaError_t e = allow_dynamic_smem(kern, Cfg::kSmemBytes, once, result);
  if (e != cudaSuccess) return e;
  int grid = sched.total_items;
  if (sched.mode == kSchedStride) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms > 0 && sms < grid) grid = sms;
  }
  kern<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(mq, mk, mv, mo, p, sched);
  return cudaGetLastError();
}

template <int kD, bool kBf16>
cudaError_t launch_mask(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                        const FwdParams& p, const FwdSched& sched, cudaStream_t stream) {
  const bool drop = p.drop.threshold != 0;
  if (p.causal) {
    return drop ? launch_one<kD, kBf16, true, true>(mq, mk, mv, mo, p, sched, stream)
                : launch_one<kD, kBf16, true, false>(mq, mk, mv, mo, p, sched, stream);
  }
  return drop ? launch_one<kD, kBf16, false, true>(mq, mk, mv, mo, p, sched, stream)
              : launch_one<kD, kBf16, false, false>(mq, mk, mv, mo, p, sched, stream);
}

}  // namespace

cudaError_t launch_fwd_sm100(const FwdParams& p, int dtype, cudaStream_t stream, int* launches) {
  const bool bf16 = (dtype == kBF16);
  CUtensorMap mq, mk, mv, mo;
  if (!encode_map_16bit(&mq, p.q, p.B, p.Hq, p.Sq, p.D, kBM, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mk, p.k, p.B, p.Hkv, p.Sk, p.D, kBN, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mv, p.v, p.B, p.Hkv, p.Sk, p.D, kBN, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mo, p.out, p.B, p.Hq, p.Sq, p.D, kBM, bf16)) return cudaErrorInvalidValue;
  FwdSched sched;
  sched.npairs = (p.Sq + 2 * kBM - 1) / (2 * kBM);
  sched.nkv_total = (p.Sk + kBN - 1) / kBN;
  // keep roughly 32 MiB of K/V hot in L2: that many heads are walked together
  const int64_t kv_bytes_per_head = static_cast<int64_t>(p.Sk) * p.D * 2 * 2;
  int64_t group = (32ll << 20) / (kv_bytes_per_head > 0 ? kv_bytes_per_head : 1);
  const int64_t total_bh = static_cast<int64_t>(p.B) * p.Hq;
  if (group < 1) group = 1;
  if (group > total_bh) group = total_bh;
  sched.group = static_cast<int>(group);
  sched.total_items = static_cast<int>(sched.npairs * total_bh);
  static const int mode = env_int("B200FA_FWD_SCHED", kSchedSteal);
  sched.mode = (mode >= kSchedOnePerCta && mode <= kSchedStride) ? mode : kSchedSteal;
  cudaError_t e;
  if (p.D == 128) {
    e = bf16 ? launch_mask<128, true>(mq, mk, mv, mo, p, sched, stream)
             : launch_mask<128, false>(mq, mk, mv, mo, p, sched, stream);
  } else {
    e = bf16 ? launch_mask<64, true>(mq, mk, mv, mo, p, sched, stream)
             : launch_mask<64, false>(mq, mk, mv, mo, p, sched, stream);
  }
  if (e == cudaSuccess && launches) *launches += 1;
  return e;
}

}  // namespace b200fa
