// Forward flash attention for sm_100a: TMA-staged Q/K/V tiles in 128-byte-swizzled shared
// memory feed tcgen05 MMAs whose S and O accumulators live in tensor memory.
//
// Computes what the reference's fwd_fa4_kernel computes
// (torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:530-543, 650-861, 1014-1022,
// 1138-1160): S = Q K^T, causal mask, online softmax in the exp2 domain with
// c = scale*log2(e), P rounded to the 16-bit input type before P V, O / rowsum and
// LSE = rowmax*scale + ln(rowsum).  The structure is new: one CTA owns TWO 128-row query
// tiles of one (batch, head) and ping-pongs them through the tensor core (kTiles = 2, below);
// at head dimension 64 two CTAs with ONE query tile each share an SM instead (kTiles = 1: warps
// 0-3 softmax, 4-7 epilogue, 8 MMA, 10 TMA).
//
//   warps 0-3   softmax of query tile 0   (thread i <-> TMEM lane i <-> query row i)
//   warps 4-7   softmax of query tile 1
//   warps 8-11  epilogue: O / l staged in shared memory and written with TMA stores, LSE (the
//               softmax warps rescale O themselves on the rare tile where a row max moved, so no
//               KV step hands anything to these warps)
//   warps 12-13 MMA issuers, one per query tile (one elected lane each issues tcgen05.mma / commit)
//               per half-block: P V of one half of the key columns, then the next block's Q K^T for
//               that half, into the S columns the P V just freed
//   warp  14    TMA producer (Q once, then a ring of K/V tiles)
//   warp  15    idle (it only donates registers)
//
// TMEM columns: S0 | S1 | O0 | O1.  The 128 key columns of a block are handled as two halves of
// 64 with their own S columns: P of a half (16-bit, two per column) overwrites the first 32 of
// that half's S columns and is consumed as the TMEM A-operand of the P V MMA, and the softmax of
// one half runs while the tensor pipe works on the other.
#include <mutex>

#include "common.cuh"
#include "philox.cuh"
#include "ptx.cuh"

namespace b200fa {
namespace {

constexpr int kBM = 128;        // query rows per tile
constexpr int kBN = 128;        // key rows per tile
constexpr int kSubTileBytes = 128 * 128;  // one 128-row x 64-column (128 B) swizzled box

// Lazy rescaling threshold (log2 domain): O and l are only rescaled when the running row
// maximum grows by more than this, so P can be as large as 2^12 against a stale maximum (well
// inside fp16; what such a stale maximum costs is the weight of terms 2^-12 and less of the
// largest, far below a 16-bit rounding step).  A rescale stalls the warp on the tile's P V
// and rewrites its rows of O, so it should stay an event of the first blocks of a row.
constexpr float kRescaleLog2 = 12.f;
// kTiles = 2: one CTA per SM owns two query tiles (512 threads, the whole of TMEM and shared memory).
// kTiles = 1: a CTA owns one query tile with half of everything (384 threads, 256 TMEM columns, half
// the K/V ring), so that two CTAs share an SM and each one's set-up, first loads and epilogue run
// under the other's KV loop: for problems made of many short CTAs, where that fixed cost dominates.
template <int kD, int kTiles>
struct FwdCfg {
  static constexpr int kTileBytes = kBM * kD * 2;
  static constexpr int kSub = kD / 64;                  // 64-column boxes per tile
  static constexpr int kStages = ((kD == 128) ? 4 : 8) / (kTiles == 2 ? 1 : 2);   // K/V ring slots
  static constexpr int kThreads = kTiles == 2 ? 512 : 384;
  // warp roles: 4 softmax warps per tile, 4 epilogue warps, one MMA-issuing warp per tile, one TMA warp
  static constexpr int kEpiWarp0 = 4 * kTiles, kMmaWarp0 = kEpiWarp0 + 4, kTmaWarp = kMmaWarp0 + 2;
  // registers per thread after the set-up (the launch gives every warp 65536 / threads per SM)
  static constexpr int kRegSoftmax = kTiles == 2 ? 176 : 144, kRegEpi = kTiles == 2 ? 88 : 56, kRegRest = kTiles == 2 ? 72 : 40;
  static constexpr int kTmemCols = kTiles == 2 ? 512 : 256;
  static constexpr int kTmemS0 = 0, kTmemS1 = 128, kTmemO0 = 128 * kTiles, kTmemO1 = 128 * kTiles + kD;
  static constexpr int kNumBars = 2 + 2 * kStages + 24;
  static constexpr int kSmemBytes = 1024 /*align slack*/ + kTiles * kTileBytes + kStages * kTileBytes +
                                    4 * 128 * 4 /*msg+max*/ + kNumBars * 8 + 64;
};

struct FwdSched {
  int npairs;      // query units (256-row pairs, or 128-row tiles of the one-tile kernel) per (b, h)
  int group;       // heads scheduled together so their K/V stay L2-resident
  int nkv_total;   // ceil(Sk / 128)
  bool one_tile;   // the one-tile-per-CTA kernel (two CTAs per SM)
};

template <int kD, bool kBf16, bool kCausal, bool kDropout, int kTiles>
__global__ void __launch_bounds__(FwdCfg<kD, kTiles>::kThreads, kTiles == 2 ? 1 : 2)
fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
           const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO, const FwdParams p,
           const FwdSched sched) {
  using Cfg = FwdCfg<kD, kTiles>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // 2 tiles
  uint8_t* sKV = sQ + kTiles * Cfg::kTileBytes;         // ring
  float* sMsg = reinterpret_cast<float*>(sKV + Cfg::kStages * Cfg::kTileBytes);  // [2][128]
  float* sMax = sMsg + 256;                             // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sMax + 256);
  uint64_t* q_full = bars;                      // [2]
  uint64_t* kv_full = q_full + 2;               // [kStages]
  uint64_t* kv_empty = kv_full + Cfg::kStages;  // [kStages]
  uint64_t* s_full = kv_empty + Cfg::kStages;   // [2 tiles][2 halves of the KV columns]
  uint64_t* p_full = s_full + 4;                // [2 tiles][2 halves of the KV columns]
  uint64_t* pv_done = p_full + 4;               // [2] one completion per P V half-block of the tile
  uint64_t* o_full = pv_done + 2;               // [2]
  uint64_t* o_ready = o_full + 2;               // [2]
  uint64_t* sc_full = o_ready + 2;              // [2] final row statistics (l, m) of a tile are in shared memory
  uint64_t* xturn = sc_full + 2;                // [2 tiles][4 warps] the two tiles' exponential phases take turns
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xturn + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // a launch whose status word already reports a failed wait is not worth running
  if (status_is_set(p.status)) return;

  // ---- which (pair, head, batch) this CTA owns: head groups keep K/V in L2, and inside a
  // group the heaviest (latest) causal pairs are scheduled first.
  const int total_bh = p.B * p.Hq;
  int pair, bh;
  {
    const int per_group = sched.group * sched.npairs;
    const int g = blockIdx.x / per_group;
    const int gsize = min(sched.group, total_bh - g * sched.group);
    const int within = blockIdx.x - g * per_group;
    pair = sched.npairs - 1 - within / gsize;
    bh = g * sched.group + within % gsize;
  }
  const int b = bh / p.Hq;
  const int h = bh - b * p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int row0 = pair * kTiles * kBM;  // first query row of tile 0

  // KV tiles each query tile visits
  int n_t[2] = {0, 0};
#pragma unroll
  for (int t = 0; t < kTiles; ++t) {
    const int r0 = row0 + t * kBM;
    if (r0 >= p.Sq) {
      n_t[t] = 0;
    } else if (kCausal) {
      // query row i sees key columns 0 .. i + causal_off: tiles up to the one the tile's last real
      // row still sees; a tile none of whose rows sees a key still runs one fully masked step so
      // that it writes zeros and -inf
      const int last = min(r0 + kBM - 1, p.Sq - 1) + p.causal_off;
      n_t[t] = last < 0 ? 1 : min(sched.nkv_total, last / kBN + 1);
    } else {
      n_t[t] = sched.nkv_total;
    }
  }
  const int n_max = max(n_t[0], n_t[1]);

  // Lane 0 of the producer warp sets up the barriers and at once issues the loads that need
  // no free slot and are needed first (Q, K_0, V_0), so that their latency overlaps the TMEM
  // allocation and the block-wide synchronisation below.
  auto load_tile = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int srow, int head) {
    mbar_arrive_expect_tx(bar, Cfg::kTileBytes);
#pragma unroll
    for (int cs = 0; cs < Cfg::kSub; ++cs) {
      tma_load_4d(dst + cs * kSubTileBytes, map, bar, cs * 64, srow, head, b);
    }
  };
  // K/V ring entry `seq`: K_j for even seq, V_j for odd, j = seq / 2; Q rides along with K_0
  auto produce = [&](int seq) {
    const int slot = seq % Cfg::kStages;
    const int j = seq >> 1;
    if (seq == 0) {
      // Q tile 0 rides ahead of K_0, Q tile 1 right behind it
      if (n_t[0] > 0) load_tile(&mapQ, sQ, &q_full[0], row0, h);
      load_tile(&mapK, sKV + slot * Cfg::kTileBytes, &kv_full[slot], 0, hk);
      if (kTiles == 2 && n_t[1] > 0) load_tile(&mapQ, sQ + Cfg::kTileBytes, &q_full[1], row0 + kBM, h);
    } else {
      load_tile((seq & 1) ? &mapV : &mapK, sKV + slot * Cfg::kTileBytes, &kv_full[slot], j * kBN, hk);
    }
  };
  const int n_loads = 2 * n_max;
  constexpr int kEarlyLoads = 2;   // Q, K_0 and V_0: what the first MMAs wait for; more would only delay the sync
  if (warp == Cfg::kTmaWarp && lane == 0) {
    mbar_init(&q_full[0], 1);
    mbar_init(&q_full[1], 1);
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], kTiles);  // released by every query tile's MMA issuer
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t * 2], 1);
      mbar_init(&s_full[t * 2 + 1], 1);
      mbar_init(&pv_done[t], 1);
      // fed by four warps each, one elected arrival per warp
      mbar_init(&p_full[t * 2], 4);      // the 4 softmax warps of the tile (P half 0 written, O rescaled if it had to be)
      mbar_init(&p_full[t * 2 + 1], 4);
      mbar_init(&o_full[t], 1);
      mbar_init(&o_ready[t], 4);         // the four correction warps have staged the output tile
      mbar_init(&sc_full[t], 4);
      for (int w = 0; w < 4; ++w) mbar_init(&xturn[t * 4 + w], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    for (int seq = 0; seq < min(n_loads, kEarlyLoads); ++seq) produce(seq);
  }
  if (warp == Cfg::kMmaWarp0) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

#define B200FA_WAIT(bar, parity, site) \
  if (!mbar_wait((bar), (parity), abort_flag, p.status, (site), p.wait_budget)) goto teardown

  if (warp < 4 * kTiles) {
    // =========================== softmax warps ===========================
    reg_alloc<Cfg::kRegSoftmax>();
    const int t = warp >> 2;
    const int row = threadIdx.x & 127;
    const int nblk = n_t[t];
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_off + (t == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
    const float c = p.scale_log2;
    const int q_row = row0 + t * kBM + row;  // global query row
    // m: the row maximum the exponentials are taken against.  It is only raised when the
    // true maximum has grown by more than 2^kRescaleLog2 (lazy rescaling), so most KV
    // tiles need no correction of O; l is the row sum relative to that same m.
    float m = -INFINITY, l = 0.f;
    const uint32_t tO = tmem_base + lane_off + (t == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
    const float2 c2 = make_float2(c, c);
    for (int j = 0; j < nblk; ++j) {
      uint32_t keep_bits[4] = {0, 0, 0, 0};   // dropout: one bit per column of this row of the KV block
      if constexpr (kDropout) {
        dropout_row_bits(p.drop, b * p.Hq + h, q_row, j * kBN, keep_bits);
      }
      // The 128 key columns of a block are scored, exponentiated and fed to P V in two halves of
      // 64, each with its own S columns: while this warp works on one half, the tensor pipe runs
      // P V of the other half and then the next block's Q K^T into the columns that P V just freed.
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t tSh = tS + half * 64;
        B200FA_WAIT(&s_full[t * 2 + half], j & 1, 0x100 + t * 2 + half);
        tc_fence_after();
        uint32_t s[64];
        float* sf = reinterpret_cast<float*>(s);
        const int col0 = j * kBN + half * 64;
        // mask: causal diagonal and/or columns beyond Sk
        const bool need_mask = (kCausal && (col0 + 63 > row0 + t * kBM + p.causal_off)) || (col0 + 64 > p.Sk);
        auto load_scores = [&]() {
          tmem_ld32(tSh + 0, s + 0);
          tmem_ld32(tSh + 32, s + 32);
          tmem_wait_ld();
          if (need_mask) {
            const int limit = kCausal ? min(q_row + p.causal_off, p.Sk - 1) : (p.Sk - 1);  // last visible column
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              if (col0 + i > limit) sf[i] = -INFINITY;
            }
          }
        };
        load_scores();
        // row max, eight independent chains
        float mx[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx[i] = sf[i];
#pragma unroll
        for (int i = 8; i < 64; i += 8) {
#pragma unroll
          for (int u = 0; u < 8; ++u) mx[u] = fmaxf(mx[u], sf[i + u]);
        }
        float m_new = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
        m_new = fmaxf(m_new, m);
        // rows past the end of the sequence (or fully masked) must not produce NaN
        if (m_new == -INFINITY) m_new = 0.f;
        // Lazy rescaling: nothing moves until some row's true maximum has grown by more than
        // 2^kRescaleLog2 over the maximum its exponentials are taken against.  When one does (the
        // first blocks of a row; rarely later), the warp rewrites its 32 rows of O anyway, so every
        // row of the warp moves to its own true maximum: the next event is then a full threshold
        // away for all of them, instead of each row tripping the warp at its own time.  It is this
        // warp that rescales its rows of O in tensor memory, once the P V of the previous half-block
        // has completed (P V of this half cannot start before this warp announces P).  The common
        // step has no hand-over to another warp at all.
        const bool any_moved = __any_sync(0xffffffffu, (m_new - m) * c > kRescaleLog2);   // always on the first half-block (m = -inf)
        float sc = 1.f;
        if (any_moved && m_new > m) {
          sc = ex2_approx((m - m_new) * c);
          m = m_new;
        }
        const int hb = 2 * j + half;   // half-block index
        if (hb > 0 && any_moved) {
          B200FA_WAIT(&pv_done[t], (hb - 1) & 1, 0x108 + t);
          tc_fence_after();
#pragma unroll
          for (int cidx = 0; cidx < kD / 32; ++cidx) {
            uint32_t* o = s + (cidx & 1) * 32;   // the score registers are free here: S is read again below
            tmem_ld32(tO + cidx * 32, o);
            tmem_wait_ld();
            float* of = reinterpret_cast<float*>(o);
#pragma unroll
            for (int i = 0; i < 32; ++i) of[i] *= sc;
            tmem_st32(tO + cidx * 32, o);
          }
          tmem_wait_st();
          load_scores();
        }
        // The special function unit of a scheduler is shared by one warp of each query tile.  The two
        // take turns at the exponentials, so that one tile's loads, maxima and stores run under the
        // other tile's exponentials instead of both tiles halving the unit's rate at the same time and
        // leaving it idle together.  (Only the overlap depends on the turns, no result does.)
        if constexpr (kTiles == 2) {
          if (t == 0) {
            if (hb > 0 && hb - 1 < 2 * n_t[1]) { B200FA_WAIT(&xturn[warp & 3], (hb - 1) & 1, 0x110); }
          } else {
            if (hb < 2 * n_t[0]) { B200FA_WAIT(&xturn[4 + (warp & 3)], hb & 1, 0x111); }
          }
        }
        const float mc = m * c;
        const float2 nmc2 = make_float2(-mc, -mc);
        float2 rsa = make_float2(0.f, 0.f), rsb = make_float2(0.f, 0.f);
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float2 x = __ffma2_rn(make_float2(sf[2 * i], sf[2 * i + 1]), c2, nmc2);
          float2 pv = make_float2(ex2_approx(x.x), ex2_approx(x.y));
          if (i & 1) rsb = __fadd2_rn(rsb, pv); else rsa = __fadd2_rn(rsa, pv);
          if constexpr (kDropout) {
            // the row sum keeps every probability; only what feeds P V is dropped
            const uint32_t bits = keep_bits[half * 2 + (i >> 4)] >> ((2 * i) & 31);
            if (!(bits & 1u)) pv.x = 0.f;
            if (!(bits & 2u)) pv.y = 0.f;
          }
          pk[i] = pack2<kBf16>(pv.x, pv.y);
        }
        if constexpr (kTiles == 2) mbar_arrive_warp(&xturn[(1 - t) * 4 + (warp & 3)]);
        // P (16-bit, two per column) goes over the first 32 of this half's own S columns
        tmem_st32(tSh, pk);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive_warp(&p_full[t * 2 + half]);
        l = l * sc + ((rsa.x + rsa.y) + (rsb.x + rsb.y));
      }
    }
    if (nblk > 0) {
      // the row statistics go to the epilogue warps
      sMsg[t * 128 + row] = l;
      sMax[t * 128 + row] = m;
      mbar_arrive_warp(&sc_full[t]);
    }
  } else if (warp < Cfg::kEpiWarp0 + 4) {
    // =========================== epilogue warps ===========================
    reg_dealloc<Cfg::kRegEpi>();
    const int row = threadIdx.x & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int es_shift = 1;  // 16-bit elements
    (void)es_shift;
    auto epilogue = [&](int t) -> bool {
      const int nblk = n_t[t];
      if (nblk == 0) return true;
      if (!mbar_wait(&sc_full[t], 0, abort_flag, p.status, 0x200 + t, p.wait_budget)) return false;
      const float l = sMsg[t * 128 + row];
      const float m = sMax[t * 128 + row];
      if (!mbar_wait(&o_full[t], 0, abort_flag, p.status, 0x210 + t, p.wait_budget)) return false;
      tc_fence_after();
      // a row that saw no key at all (possible under a bottom-right aligned mask) is 0 with lse -inf
      float inv_l = l > 0.f ? 1.f / l : 0.f;
      if constexpr (kDropout) inv_l *= p.drop.inv_keep;
      const int q_row = row0 + t * kBM + row;
      const uint32_t tO = tmem_base + lane_off + (t == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
      // The 16-bit output tile is staged in this query tile's own Q buffer (every MMA that
      // read it has completed), in the swizzled box layout, and leaves through TMA stores:
      // whole 128-byte lines, nothing for the CTA to wait on but the read of shared memory,
      // and rows past the end of the sequence are clipped by the tensor map.
      uint8_t* stage = sQ + t * Cfg::kTileBytes;
#pragma unroll
      for (int cidx = 0; cidx < kD / 32; ++cidx) {
        uint32_t o[32];
        tmem_ld32(tO + cidx * 32, o);
        tmem_wait_ld();
        const float* of = reinterpret_cast<const float*>(o);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 w;
          w.x = pack2<kBf16>(of[v * 8 + 0] * inv_l, of[v * 8 + 1] * inv_l);
          w.y = pack2<kBf16>(of[v * 8 + 2] * inv_l, of[v * 8 + 3] * inv_l);
          w.z = pack2<kBf16>(of[v * 8 + 4] * inv_l, of[v * 8 + 5] * inv_l);
          w.w = pack2<kBf16>(of[v * 8 + 6] * inv_l, of[v * 8 + 7] * inv_l);
          const int chunk = cidx * 4 + v;   // 16-byte chunk of the row
          *reinterpret_cast<uint4*>(stage + (chunk >> 3) * kSubTileBytes + row * 128 +
                                    (((chunk & 7) ^ (row & 7)) << 4)) = w;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(&o_ready[t]);
      if (q_row < p.Sq) {
        p.lse[(static_cast<int64_t>(b) * p.Hq + h) * p.Sq + q_row] = l > 0.f ? m * p.scale + logf(l) : -INFINITY;
      }
      if (warp == Cfg::kEpiWarp0 && lane == 0) {
        if (!mbar_wait(&o_ready[t], 0, abort_flag, p.status, 0x218 + t, p.wait_budget)) return false;
#pragma unroll
        for (int cs = 0; cs < Cfg::kSub; ++cs) {
          tma_store_4d(&mapO, stage + cs * kSubTileBytes, cs * 64, row0 + t * kBM, h, b);
        }
        tma_store_commit();
      }
      return true;
    };
    // (a tile that sees its last KV block a step before the other is written out while the other still runs)
    if (!epilogue(0)) goto teardown;
    if constexpr (kTiles == 2) {
      if (!epilogue(1)) goto teardown;
    }
  } else {
    reg_dealloc<Cfg::kRegRest>();
    if (warp >= Cfg::kMmaWarp0 && warp < Cfg::kMmaWarp0 + kTiles) {
      // =========================== MMA issuers (one per query tile) ===========================
      // A tcgen05.mma only issues once the tensor pipe has room, so the issuing lane is stalled
      // for about as long as its MMAs run, and every wait or commit it executes in between is
      // time the pipe could drain.  Giving each query tile its own issuing lane lets one
      // lane's waits overlap the other lane's MMAs.
      const int t = warp - Cfg::kMmaWarp0;
      const int nblk = n_t[t];
      if (lane == 0 && nblk > 0) {
        constexpr uint32_t idesc_qk = umma_idesc(kBf16, false, false, 128, 64);   // one half of the key columns
        constexpr uint32_t idesc_pv = umma_idesc(kBf16, false, true, 128, kD);
        const uint32_t tS = tmem_base + (t == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
        const uint32_t tO = tmem_base + (t == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
        // descriptors are a fixed high word plus a start-address word; stepping along the
        // contraction dimension or to another ring slot only adds to the low word
        const UmmaDesc dQ = umma_desc_split(smem_u32(sQ) + t * Cfg::kTileBytes, 16, 1024);  // K-major Q tile
        const UmmaDesc dK = umma_desc_split(smem_u32(sKV), 16, 1024);             // ring slot as K-major K
        const UmmaDesc dV = umma_desc_split(smem_u32(sKV), kSubTileBytes, 1024);  // ring slot as MN-major V
        // S columns [64 half, 64 half + 64) = Q_t (key rows 64 half .. 64 half + 63 of the K tile)^T
        auto issue_qk = [&](uint32_t slot_lo, int half) {
          const uint32_t krows = umma_off(half * 64 * 128);
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) {
            const uint32_t off = umma_off((kk >> 2) * kSubTileBytes + (kk & 3) * 32);
            if (kk == 0) umma_ss_fast<false>(tS + half * 64, dQ.lo + off, dQ.hi, dK.lo + slot_lo + krows + off, dK.hi, idesc_qk);
            else         umma_ss_fast<true>(tS + half * 64, dQ.lo + off, dQ.hi, dK.lo + slot_lo + krows + off, dK.hi, idesc_qk);
          }
        };
        // half 0: KV rows 0-63 of the tile, half 1: rows 64-127; P of a half sits in the first 32 of the half's S columns
        auto issue_pv = [&](uint32_t slot_lo, bool first, int half) {
#pragma unroll
          for (int kq = 0; kq < 4; ++kq) {
            const int kk = half * 4 + kq;
            const uint32_t b_lo = dV.lo + slot_lo + umma_off(kk * 2048);
            if (kk == 0 && first) umma_ts_fast<false>(tO, tS + half * 64 + kq * 8, b_lo, dV.hi, idesc_pv);
            else                  umma_ts_fast<true>(tO, tS + half * 64 + kq * 8, b_lo, dV.hi, idesc_pv);
          }
        };
        // The two lanes issue independently: the softmax of a half only waits for its own half's
        // S, so neither tile's chain runs through the other lane's MMAs.
        // block 0: S_t = Q_t K_0^T, both halves
        B200FA_WAIT(&q_full[t], 0, 0x301 + t);
        B200FA_WAIT(&kv_full[0], 0, 0x300);
        tc_fence_after();
        issue_qk(0, 0);
        umma_commit(&s_full[t * 2]);
        issue_qk(0, 1);
        umma_commit(&s_full[t * 2 + 1]);
        umma_commit(&kv_empty[0]);
        int slot = 1;         // ring slot of V_j; K_{j+1} follows in the next slot
        uint32_t phase = 0;   // parity of the ring pass V_j's slot is in
        for (int j = 0; j < nblk; ++j) {
          const int vslot = slot;
          const uint32_t vphase = phase;
          if (++slot == Cfg::kStages) { slot = 0; phase ^= 1; }
          const bool has_next = (j + 1 < nblk);
          B200FA_WAIT(&kv_full[vslot], vphase, 0x310);
          if (has_next) { B200FA_WAIT(&kv_full[slot], phase, 0x340); }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            // one half-block: P V of this half, then the next block's Q K^T into the S columns it frees
            B200FA_WAIT(&p_full[t * 2 + half], j & 1, 0x320 + t * 2 + half);
            tc_fence_after();
            issue_pv(vslot * umma_off(Cfg::kTileBytes), j == 0 && half == 0, half);
            umma_commit(&pv_done[t]);
            if (has_next) {
              issue_qk(slot * umma_off(Cfg::kTileBytes), half);
              umma_commit(&s_full[t * 2 + half]);
            }
          }
          if (has_next) {
            umma_commit(&kv_empty[slot]);
          } else {
            umma_commit(&o_full[t]);
          }
          umma_commit(&kv_empty[vslot]);
          if (++slot == Cfg::kStages) { slot = 0; phase ^= 1; }
        }
        // KV tiles only the other query tile visits still need this tile's release
        for (int j = nblk; j < n_max; ++j) {
          // K_j sits in the slot before V_j; slot/phase currently point at V_j
          const int kslot = (slot == 0) ? Cfg::kStages - 1 : slot - 1;
          const uint32_t kphase = (slot == 0) ? (phase ^ 1) : phase;
          B200FA_WAIT(&kv_full[kslot], kphase, 0x350);
          mbar_arrive(&kv_empty[kslot]);
          B200FA_WAIT(&kv_full[slot], phase, 0x351);
          mbar_arrive(&kv_empty[slot]);
          if (++slot == Cfg::kStages) { slot = 0; phase ^= 1; }
          if (++slot == Cfg::kStages) { slot = 0; phase ^= 1; }
        }
      } else if (lane == 0 && n_max > 0) {
        // this query tile lies wholly past the end of the sequence: release each K/V slot as it fills
        int slot = 0;
        uint32_t phase = 0;
        for (int k = 0; k <= n_max; ++k) {
          // block k of the other tile consumes K_0 (k = 0) or V_{k-1} and, if there is one, K_k
          const int n_release = (k == 0 || k == n_max) ? 1 : 2;
          for (int r = 0; r < n_release; ++r) {
            B200FA_WAIT(&kv_full[slot], phase, 0x360);
            mbar_arrive(&kv_empty[slot]);
            if (++slot == Cfg::kStages) { slot = 0; phase ^= 1; }
          }
        }
      }
    } else if (warp == Cfg::kTmaWarp) {
      // =========================== TMA producer ===========================
      if (lane == 0) {
        // the first kEarlyLoads entries went out before the block-wide synchronisation
        for (int seq = kEarlyLoads; seq < n_loads; ++seq) {
          if (seq >= Cfg::kStages) {
            B200FA_WAIT(&kv_empty[seq % Cfg::kStages], ((seq / Cfg::kStages) - 1) & 1, 0x400);
          }
          produce(seq);
        }
      }
    }
  }

teardown:
#undef B200FA_WAIT
  // the staged output tiles must have been read before shared memory is given back
  if (warp == Cfg::kEpiWarp0 && lane == 0) tma_store_wait_read();
  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::kMmaWarp0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int kD, bool kBf16, bool kCausal, bool kDropout, int kTiles>
cudaError_t launch_tiles(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                       const FwdParams& p, const FwdSched& sched, cudaStream_t stream) {
  using Cfg = FwdCfg<kD, kTiles>;
  auto kern = fwd_kernel<kD, kBf16, kCausal, kDropout, kTiles>;
  // cudaFuncSetAttribute once per device for THIS kernel (the flags are statics of this function
  // template: kernels of the same signature must not share them), safe against concurrent first calls
  static std::once_flag once[64];
  static cudaError_t result[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  } else {
    std::call_once(once[dev], [&] {
      result[dev] = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    });
    e = result[dev];
  }
  if (e != cudaSuccess) return e;
  const int grid = sched.npairs * p.B * p.Hq;
  kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(mq, mk, mv, mo, p, sched);
  return cudaGetLastError();
}

template <int kD, bool kBf16, bool kCausal, bool kDropout>
cudaError_t launch_one(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                       const FwdParams& p, FwdSched sched, cudaStream_t stream) {
  if (sched.one_tile) {
    sched.npairs = (p.Sq + kBM - 1) / kBM;
    return launch_tiles<kD, kBf16, kCausal, kDropout, 1>(mq, mk, mv, mo, p, sched, stream);
  }
  return launch_tiles<kD, kBf16, kCausal, kDropout, 2>(mq, mk, mv, mo, p, sched, stream);
}

// Which kernel shape.  Two CTAs per SM with one query tile each hide a CTA's set-up, first loads
// and epilogue under the other CTA's KV loop, but have half the K/V ring each and load every K/V
// tile once per query tile instead of once per pair.  Measured on B200: at D = 64 (16 KB tiles, the
// ring still four deep) it is 11-13 % faster on problems of many short CTAs (B32 H12 S1024: 0.145
// -> 0.129 ms) and equal on long ones; at D = 128 the ring of two stalls every P V on its V load
// (C3 0.49 -> 0.65 ms).  `forced` (0 = this rule, 1, 2) is for tests and measurements.
bool choose_one_tile(const FwdParams& p, int forced) {
  if (forced == 1) return true;
  if (forced == 2) return false;
  return p.D == 64;
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
  sched.one_tile = choose_one_tile(p, p.tiles_per_cta);
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
