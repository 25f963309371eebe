// Forward flash attention for sm_100a: TMA-staged Q/K/V tiles in 128-byte-swizzled shared
// memory feed tcgen05 MMAs whose S and O accumulators live in tensor memory.
//
// Computes what the reference's fwd_fa4_kernel computes
// (torch_mojo_backend/eager_flash_attention/fa4_fwd_kernel.mojo:530-543, 650-861, 1014-1022,
// 1138-1160): S = Q K^T, causal mask, online softmax in the exp2 domain with
// c = scale*log2(e), P rounded to the 16-bit input type before P V, O / rowsum and
// LSE = rowmax*scale + ln(rowsum).  The structure is new: one CTA owns TWO 128-row query
// tiles of one (batch, head) and ping-pongs them through the tensor core.
//
//   warps 0-3   softmax of query tile 0   (thread i <-> TMEM lane i <-> query row i)
//   warps 4-7   softmax of query tile 1
//   warps 8-11  correction: rescale O in TMEM when a row max moved, final O/l + LSE epilogue
//   warp  12    MMA issuer (one elected lane issues every tcgen05.mma / commit)
//   warp  13    TMA producer (Q once, then a ring of K/V tiles)
//   warps 14-15 idle (they only donate registers)
//
// TMEM columns: S0 | S1 | O0 | O1.  P (16-bit, two per column) overwrites the first half of
// its own S columns and is consumed as the TMEM A-operand of the P V MMA.
#include "common.cuh"
#include "ptx.cuh"

namespace b200fa {
namespace {

constexpr int kBM = 128;        // query rows per tile
constexpr int kBN = 128;        // key rows per tile
constexpr int kThreads = 512;
constexpr int kSubTileBytes = 128 * 128;  // one 128-row x 64-column (128 B) swizzled box

template <int kD>
struct FwdCfg {
  static constexpr int kTileBytes = kBM * kD * 2;
  static constexpr int kSub = kD / 64;                  // 64-column boxes per tile
  static constexpr int kStages = (kD == 128) ? 4 : 8;   // K/V ring slots
  static constexpr int kTmemS0 = 0, kTmemS1 = 128, kTmemO0 = 256, kTmemO1 = 256 + kD;
  static constexpr int kNumBars = 2 + 2 * kStages + 12;
  static constexpr int kSmemBytes = 1024 /*align slack*/ + 2 * kTileBytes + kStages * kTileBytes +
                                    4 * 128 * 4 /*msg+max*/ + kNumBars * 8 + 64;
};

struct FwdSched {
  int npairs;      // 256-row query pairs per (b, h)
  int group;       // heads scheduled together so their K/V stay L2-resident
  int nkv_total;   // ceil(Sk / 128)
};

template <int kD, bool kBf16, bool kCausal>
__global__ void __launch_bounds__(kThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
           const __grid_constant__ CUtensorMap mapV, const FwdParams p, const FwdSched sched) {
  using Cfg = FwdCfg<kD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // 2 tiles
  uint8_t* sKV = sQ + 2 * Cfg::kTileBytes;              // ring
  float* sMsg = reinterpret_cast<float*>(sKV + Cfg::kStages * Cfg::kTileBytes);  // [2][128]
  float* sMax = sMsg + 256;                             // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sMax + 256);
  uint64_t* q_full = bars;                      // [2]
  uint64_t* kv_full = q_full + 2;               // [kStages]
  uint64_t* kv_empty = kv_full + Cfg::kStages;  // [kStages]
  uint64_t* s_full = kv_empty + Cfg::kStages;   // [2]
  uint64_t* p_full = s_full + 2;                // [2]
  uint64_t* o_full = p_full + 2;                // [2]
  uint64_t* o_ready = o_full + 2;               // [2]
  uint64_t* sc_full = o_ready + 2;              // [2]
  uint64_t* sc_empty = sc_full + 2;             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

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
  const int row0 = pair * 2 * kBM;  // first query row of tile 0

  // KV tiles each query tile visits
  int n_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = row0 + t * kBM;
    if (r0 >= p.Sq) {
      n_t[t] = 0;
    } else if (kCausal) {
      n_t[t] = min(sched.nkv_total, r0 / kBN + 1);
    } else {
      n_t[t] = sched.nkv_total;
    }
  }
  const int n_max = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    mbar_init(&q_full[0], 1);
    mbar_init(&q_full[1], 1);
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&o_full[t], 1);
      mbar_init(&o_ready[t], 128);
      mbar_init(&sc_full[t], 128);
      mbar_init(&sc_empty[t], 128);
    }
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
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

#define B200FA_WAIT(bar, parity, site) \
  if (!mbar_wait((bar), (parity), abort_flag, p.status, (site))) goto teardown

  if (warp < 8) {
    // =========================== softmax warps ===========================
    reg_alloc<184>();
    const int t = warp >> 2;
    const int row = threadIdx.x & 127;
    const int nblk = n_t[t];
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_off + (t == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
    const float c = p.scale_log2;
    const int q_row = row0 + t * kBM + row;  // global query row
    float m = -INFINITY, l = 0.f;
    for (int j = 0; j < nblk; ++j) {
      B200FA_WAIT(&s_full[t], j & 1, 0x100 + t);
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
      const bool need_mask = (kCausal && (col0 + kBN - 1 > row0 + t * kBM)) || (col0 + kBN > p.Sk);
      if (need_mask) {
        const int limit = kCausal ? min(q_row, p.Sk - 1) : (p.Sk - 1);  // last visible column
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if (col0 + i > limit) sf[i] = -INFINITY;
        }
      }
      float mx = sf[0];
#pragma unroll
      for (int i = 1; i < 128; ++i) mx = fmaxf(mx, sf[i]);
      float m_new = fmaxf(m, mx);
      // rows past the end of the sequence (or fully masked) must not produce NaN
      if (m_new == -INFINITY) m_new = 0.f;
      const float sc = ex2_approx((m - m_new) * c);
      if (j > 0) {
        B200FA_WAIT(&sc_empty[t], (j - 1) & 1, 0x110 + t);
      }
      sMsg[t * 128 + row] = sc;
      mbar_arrive(&sc_full[t]);
      m = m_new;
      const float mc = m * c;
      float rs = 0.f;
      uint32_t pk[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float p0 = ex2_approx(fmaf(sf[2 * i], c, -mc));
        const float p1 = ex2_approx(fmaf(sf[2 * i + 1], c, -mc));
        rs += p0 + p1;
        pk[i] = pack2<kBf16>(p0, p1);
      }
      tmem_st32(tS + 0, pk + 0);
      tmem_st32(tS + 32, pk + 32);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[t]);
      l = l * sc + rs;
    }
    if (nblk > 0) {
      B200FA_WAIT(&sc_empty[t], (nblk - 1) & 1, 0x120 + t);
      sMsg[t * 128 + row] = l;
      sMax[t * 128 + row] = m;
      mbar_arrive(&sc_full[t]);
    }
  } else if (warp < 12) {
    // =========================== correction warps ===========================
    reg_dealloc<88>();
    const int row = threadIdx.x & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int es_shift = 1;  // 16-bit elements
    (void)es_shift;
    auto epilogue = [&](int t) -> bool {
      const int nblk = n_t[t];
      if (nblk == 0) return true;
      if (!mbar_wait(&sc_full[t], nblk & 1, abort_flag, p.status, 0x200 + t)) return false;
      const float l = sMsg[t * 128 + row];
      const float m = sMax[t * 128 + row];
      if (!mbar_wait(&o_full[t], (nblk - 1) & 1, abort_flag, p.status, 0x210 + t)) return false;
      tc_fence_after();
      const float inv_l = 1.f / l;
      const int q_row = row0 + t * kBM + row;
      const uint32_t tO = tmem_base + lane_off + (t == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
      const bool valid = q_row < p.Sq;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.out.ptr) +
                       (static_cast<int64_t>(b) * p.out.sb + static_cast<int64_t>(h) * p.out.sh +
                        static_cast<int64_t>(q_row) * p.out.ss);
#pragma unroll
      for (int cidx = 0; cidx < kD / 32; ++cidx) {
        uint32_t o[32];
        tmem_ld32(tO + cidx * 32, o);
        tmem_wait_ld();
        if (valid) {
          const float* of = reinterpret_cast<const float*>(o);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 w;
            w.x = pack2<kBf16>(of[v * 8 + 0] * inv_l, of[v * 8 + 1] * inv_l);
            w.y = pack2<kBf16>(of[v * 8 + 2] * inv_l, of[v * 8 + 3] * inv_l);
            w.z = pack2<kBf16>(of[v * 8 + 4] * inv_l, of[v * 8 + 5] * inv_l);
            w.w = pack2<kBf16>(of[v * 8 + 6] * inv_l, of[v * 8 + 7] * inv_l);
            *reinterpret_cast<uint4*>(orow + cidx * 32 + v * 8) = w;
          }
        }
      }
      if (valid) {
        p.lse[(static_cast<int64_t>(b) * p.Hq + h) * p.Sq + q_row] = m * p.scale + logf(l);
      }
      return true;
    };
    for (int j = 0; j < n_max; ++j) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (j < n_t[t]) {
          B200FA_WAIT(&sc_full[t], j & 1, 0x220 + t);
          const float sc = sMsg[t * 128 + row];
          mbar_arrive(&sc_empty[t]);
          if (j > 0) {
            B200FA_WAIT(&o_full[t], (j - 1) & 1, 0x230 + t);
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
            tc_fence_before();
          }
          mbar_arrive(&o_ready[t]);
        }
      }
      // a tile that just saw its last KV block can be finished while the other still runs
      if (n_t[0] != n_t[1] && j == n_t[0] - 1) {
        if (!epilogue(0)) goto teardown;
      }
    }
    if (n_t[0] == n_t[1] || n_t[0] == 0) {
      if (!epilogue(0)) goto teardown;
    }
    if (!epilogue(1)) goto teardown;
  } else {
    reg_dealloc<56>();
    if (warp == 12) {
      // =========================== MMA issuer ===========================
      if (lane == 0) {
        constexpr uint32_t idesc_qk = umma_idesc(kBf16, false, false, 128, 128);
        constexpr uint32_t idesc_pv = umma_idesc(kBf16, false, true, 128, kD);
        const uint32_t sQ_addr = smem_u32(sQ);
        const uint32_t sKV_addr = smem_u32(sKV);
        const uint32_t tS[2] = {tmem_base + Cfg::kTmemS0, tmem_base + Cfg::kTmemS1};
        const uint32_t tO[2] = {tmem_base + Cfg::kTmemO0, tmem_base + Cfg::kTmemO1};
        auto issue_qk = [&](int t, uint32_t k_addr) {
          const uint32_t q_addr = sQ_addr + t * Cfg::kTileBytes;
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kSubTileBytes + (kk & 3) * 32;
            umma_ss(tS[t], umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024),
                    idesc_qk, kk > 0);
          }
        };
        auto issue_pv = [&](int t, uint32_t v_addr, bool acc) {
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk) {
            umma_ts(tO[t], tS[t] + kk * 8, umma_smem_desc(v_addr + kk * 2048, kSubTileBytes, 1024), idesc_pv,
                    (acc || kk > 0) ? 1u : 0u);
          }
        };
        auto slot_addr = [&](int seq) { return sKV_addr + (seq % Cfg::kStages) * Cfg::kTileBytes; };
        auto slot_phase = [&](int seq) { return static_cast<uint32_t>((seq / Cfg::kStages) & 1); };
        if (n_max > 0) {
          // prologue: S_t = Q_t K_0^T
          B200FA_WAIT(&kv_full[0], 0, 0x300);
          for (int t = 0; t < 2; ++t) {
            if (n_t[t] > 0) {
              B200FA_WAIT(&q_full[t], 0, 0x301 + t);
              tc_fence_after();
              issue_qk(t, slot_addr(0));
              umma_commit(&s_full[t]);
            }
          }
          umma_commit(&kv_empty[0]);
          for (int j = 0; j < n_max; ++j) {
            const int vseq = 2 * j + 1, kseq = 2 * j + 2;
            B200FA_WAIT(&kv_full[vseq % Cfg::kStages], slot_phase(vseq), 0x310);
            const bool has_next = (j + 1 < n_max);
            bool k_ready = false;
            for (int t = 0; t < 2; ++t) {
              if (j < n_t[t]) {
                B200FA_WAIT(&p_full[t], j & 1, 0x320 + t);
                B200FA_WAIT(&o_ready[t], j & 1, 0x330 + t);
                tc_fence_after();
                issue_pv(t, slot_addr(vseq), j > 0);
                umma_commit(&o_full[t]);
                if (j + 1 < n_t[t]) {
                  if (!k_ready) {
                    B200FA_WAIT(&kv_full[kseq % Cfg::kStages], slot_phase(kseq), 0x340);
                    tc_fence_after();
                    k_ready = true;
                  }
                  issue_qk(t, slot_addr(kseq));
                  umma_commit(&s_full[t]);
                }
              }
            }
            umma_commit(&kv_empty[vseq % Cfg::kStages]);
            if (has_next) umma_commit(&kv_empty[kseq % Cfg::kStages]);
          }
        }
      }
    } else if (warp == 13) {
      // =========================== TMA producer ===========================
      if (lane == 0 && n_max > 0) {
        int seq = 0;
        auto load_tile = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int srow, int head) {
          mbar_arrive_expect_tx(bar, Cfg::kTileBytes);
#pragma unroll
          for (int cs = 0; cs < Cfg::kSub; ++cs) {
            tma_load_4d(dst + cs * kSubTileBytes, map, bar, cs * 64, srow, head, b);
          }
        };
        for (int j = 0; j < n_max; ++j) {
          for (int which = 0; which < 2; ++which) {  // 0 = K_j, 1 = V_j
            const int slot = seq % Cfg::kStages;
            if (seq >= Cfg::kStages) {
              B200FA_WAIT(&kv_empty[slot], ((seq / Cfg::kStages) - 1) & 1, 0x400);
            }
            if (j == 0 && which == 0) {
              // Q tile 0 rides ahead of K_0, Q tile 1 right behind it
              if (n_t[0] > 0) load_tile(&mapQ, sQ, &q_full[0], row0, h);
              load_tile(&mapK, sKV + slot * Cfg::kTileBytes, &kv_full[slot], j * kBN, hk);
              if (n_t[1] > 0) load_tile(&mapQ, sQ + Cfg::kTileBytes, &q_full[1], row0 + kBM, h);
            } else {
              load_tile(which == 0 ? &mapK : &mapV, sKV + slot * Cfg::kTileBytes, &kv_full[slot], j * kBN, hk);
            }
            ++seq;
          }
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

template <int kD, bool kBf16, bool kCausal>
cudaError_t launch_one(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FwdParams& p,
                       const FwdSched& sched, cudaStream_t stream) {
  using Cfg = FwdCfg<kD>;
  auto kern = fwd_kernel<kD, kBf16, kCausal>;
  static bool attr_set[16] = {};  // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const int grid = sched.npairs * p.B * p.Hq;
  kern<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(mq, mk, mv, p, sched);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd_sm100(const FwdParams& p, int dtype, cudaStream_t stream, int* launches) {
  const bool bf16 = (dtype == kBF16);
  CUtensorMap mq, mk, mv;
  if (!encode_map_16bit(&mq, p.q, p.B, p.Hq, p.Sq, p.D, kBM, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mk, p.k, p.B, p.Hkv, p.Sk, p.D, kBN, bf16)) return cudaErrorInvalidValue;
  if (!encode_map_16bit(&mv, p.v, p.B, p.Hkv, p.Sk, p.D, kBN, bf16)) return cudaErrorInvalidValue;
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
  cudaError_t e;
#define B200FA_DISPATCH(D_, BF_, C_) e = launch_one<D_, BF_, C_>(mq, mk, mv, p, sched, stream)
  if (p.D == 128) {
    if (bf16) { if (p.causal) B200FA_DISPATCH(128, true, true); else B200FA_DISPATCH(128, true, false); }
    else      { if (p.causal) B200FA_DISPATCH(128, false, true); else B200FA_DISPATCH(128, false, false); }
  } else {
    if (bf16) { if (p.causal) B200FA_DISPATCH(64, true, true); else B200FA_DISPATCH(64, true, false); }
    else      { if (p.causal) B200FA_DISPATCH(64, false, true); else B200FA_DISPATCH(64, false, false); }
  }
#undef B200FA_DISPATCH
  if (e == cudaSuccess && launches) *launches += 1;
  return e;
}

}  // namespace b200fa
