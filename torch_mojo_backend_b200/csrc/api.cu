// Host side of the C ABI declared in include/b200fa.h: argument validation (always before
// any launch, like the reference's bridge does in
// torch_mojo_backend/eager_flash_attention/fa4_ops.mojo:309-396, 625-663, 857-892),
// TMA descriptor encoding, kernel selection and launch accounting.
#include <algorithm>
#include <atomic>
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/b200fa.h"
#include "common.cuh"
#include "philox.cuh"
#include "ptx.cuh"

namespace b200fa {
namespace {

std::atomic<uint64_t> g_launches{0};

// Cycle budget of every bounded wait inside the kernels: B200FA_WAIT_BUDGET (SM cycles) if set,
// else about two seconds; b200fa_set_wait_budget overrides both.
std::atomic<long long> g_wait_budget{0};
long long wait_budget() {
  long long b = g_wait_budget.load();
  if (b <= 0) {
    const char* env = std::getenv("B200FA_WAIT_BUDGET");
    const long long from_env = env ? std::atoll(env) : 0;
    b = from_env > 0 ? from_env : kWaitBudgetCycles;
    g_wait_budget.store(b);
  }
  return b;
}

// Query tiles per forward CTA: 0 = the launcher's rule, 1 or 2 = forced (B200FA_FWD_TILES, b200fa_set_fwd_tiles).
std::atomic<int> g_fwd_tiles{-1};
int fwd_tiles() {
  int t = g_fwd_tiles.load();
  if (t < 0) {
    const char* env = std::getenv("B200FA_FWD_TILES");
    t = env ? std::atoi(env) : 0;
    if (t < 0 || t > 2) t = 0;
    g_fwd_tiles.store(t);
  }
  return t;
}

// Text of the most recent CUDA failure seen by this thread (for b200fa_last_error_detail).
thread_local char g_detail[256] = "";

void note_cuda_error(const char* where, cudaError_t e) {
  snprintf(g_detail, sizeof(g_detail), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(sym);
    }
  });
  return fn;
}

int elem_size(int dtype) { return dtype == kF32 ? 4 : 2; }

// Checks one (B,H,S,D) view; fills `out`.  A tensor the library writes (`is_output`) must not
// alias itself: dimensions sorted by stride, each stride has to clear the extent below it.
int check_view(const b200fa_tensor4* t, int64_t B, int64_t H, int64_t S, int64_t D, int dtype, View4* out,
               bool is_output = false) {
  if (!t || !t->ptr) return B200FA_ERR_NULL;
  if (t->shape[0] != B || t->shape[1] != H || t->shape[2] != S || t->shape[3] != D) return B200FA_ERR_BAD_SHAPE;
  if (t->stride[3] != 1) return B200FA_ERR_BAD_STRIDE;
  const int es = elem_size(dtype);
  for (int i = 0; i < 3; ++i) {
    if (t->stride[i] < 0) return B200FA_ERR_BAD_STRIDE;
    // a broadcast (stride 0 over more than one index) cannot be expressed in a tensor map, and
    // the element-wise kernels would disagree with the tiled ones about it
    if (t->stride[i] == 0 && t->shape[i] > 1) return B200FA_ERR_BAD_STRIDE;
    // rows are moved 16 bytes at a time (TMA boxes, vector stores)
    if ((t->stride[i] * es) % 16 != 0) return B200FA_ERR_BAD_STRIDE;
    // tensor-map strides are 40-bit byte counts
    if (t->stride[i] * es >= (int64_t(1) << 40)) return B200FA_ERR_BAD_STRIDE;
  }
  if (S > 1 && t->stride[2] < D) return B200FA_ERR_BAD_STRIDE;
  if (is_output) {
    struct Dim { int64_t stride, size; } dims[3] = {{t->stride[0], B}, {t->stride[1], H}, {t->stride[2], S}};
    std::sort(dims, dims + 3, [](const Dim& a, const Dim& b) { return a.stride < b.stride; });
    int64_t extent = D;   // elements covered by the dimensions below
    for (const Dim& d : dims) {
      if (d.size <= 1) continue;
      if (d.stride < extent) return B200FA_ERR_BAD_STRIDE;
      extent = d.stride * (d.size - 1) + extent;
    }
  }
  if (reinterpret_cast<uintptr_t>(t->ptr) % 16 != 0) return B200FA_ERR_MISALIGNED;
  out->ptr = t->ptr;
  out->sb = t->stride[0];
  out->sh = t->stride[1];
  out->ss = t->stride[2];
  return B200FA_OK;
}

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    // Always set the device, even when it is already the current ordinal: a thread that has
    // made no runtime call yet (the autograd engine's worker) has no context bound, and the
    // driver-API tensor-map encode needs one.
    if (cudaSetDevice(device) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    int cur = -1;
    if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
  }
};

int check_device_is_sm100(int device) {
  static int cached[64];
  static std::once_flag once;
  std::call_once(once, [] { std::memset(cached, 0, sizeof(cached)); });
  if (device < 0 || device >= 64) return B200FA_ERR_CUDA;
  if (cached[device] == 0) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess)
      return B200FA_ERR_CUDA;
    cached[device] = (major == 10) ? 1 : -1;
  }
  return cached[device] == 1 ? B200FA_OK : B200FA_ERR_UNSUPPORTED;
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace

bool encode_map_16bit(CUtensorMap* map, const View4& t, int B, int H, int S, int D, int box_rows, bool bf16) {
  EncodeFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  // a size-1 dimension may come with stride 0, which is not encodable: any 16-byte multiple works there
  // (check_view has refused stride 0 on every larger dimension)
  auto stride_bytes = [&](int64_t s_elems, int64_t fallback) {
    const int64_t s = (s_elems > 0 ? s_elems : fallback) * 2;
    return static_cast<cuuint64_t>(s);
  };
  const int64_t row = t.ss > 0 ? t.ss : D;
  cuuint64_t strides[3] = {stride_bytes(t.ss, D), stride_bytes(t.sh, row * S),
                           stride_bytes(t.sb, row * S * (H > 0 ? H : 1))};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, t.ptr, dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

namespace {

// one warp waits, for `budget` SM cycles, on a barrier that nobody ever arrives at
__global__ void wait_timeout_selftest_kernel(uint32_t* status, long long budget) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  (void)mbar_wait(&bar, 0, &abort_flag, status, 0xfffeu, budget);
}

}  // namespace

cudaError_t launch_wait_timeout_selftest(uint32_t* status, long long budget, cudaStream_t stream, int* launches) {
  wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(status, budget);
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && launches) *launches += 1;
  return e;
}

}  // namespace b200fa

using namespace b200fa;

namespace {

struct Options {
  bool force_simt = false;
  int parts = 7;
  float dropout_p = 0.f;
  uint64_t seed = 0, offset = 0;
};

// causal argument -> (flag, diagonal offset); false if it is not one of the three modes
bool causal_mode(int causal, int64_t Sq, int64_t Sk, int* flag, int* off) {
  if (causal == B200FA_CAUSAL_NONE) { *flag = 0; *off = 0; return true; }
  if (causal == B200FA_CAUSAL_TOP_LEFT) { *flag = 1; *off = 0; return true; }
  if (causal == B200FA_CAUSAL_BOTTOM_RIGHT) { *flag = 1; *off = static_cast<int>(Sk - Sq); return true; }
  return false;
}

bool dropout_params(float p, uint64_t seed, uint64_t offset, DropoutParams* d) {
  if (!(p >= 0.f) || !(p < 1.f)) return false;
  const uint32_t thr = b200fa_dropout_threshold(p);
  d->seed = seed;
  d->offset = offset;
  d->threshold = thr;
  d->inv_keep = 256.f / static_cast<float>(256u - thr);
  return true;
}

int fwd_impl(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v, const b200fa_tensor4* out,
             float* lse, int dtype, int causal, float scale, void* stream, int device, uint32_t* status_word,
             const Options& opt) {
  if (!q || !k || !v || !out || !lse) return B200FA_ERR_NULL;
  if (dtype != kF32 && dtype != kBF16 && dtype != kF16) return B200FA_ERR_BAD_DTYPE;
  const int64_t B = q->shape[0], Hq = q->shape[1], Sq = q->shape[2], D = q->shape[3];
  const int64_t Hkv = k->shape[1], Sk = k->shape[2];
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Sk <= 0) return B200FA_ERR_BAD_SHAPE;
  if (B > 65535 || Hq > 65535 || Sq > (1 << 24) || Sk > (1 << 24)) return B200FA_ERR_BAD_SHAPE;
  if (D != 64 && D != 128) return B200FA_ERR_UNSUPPORTED;
  if (Hq % Hkv != 0) return B200FA_ERR_BAD_SHAPE;
  // one thread block per 256 query rows of a (batch, head): the grid index is a 32-bit int
  if (B * Hq * ((Sq + 255) / 256) > INT_MAX || B * Hq * ((Sq + 63) / 64) > INT_MAX) return B200FA_ERR_BAD_SHAPE;
  FwdParams p;
  std::memset(&p, 0, sizeof(p));
  if (!causal_mode(causal, Sq, Sk, &p.causal, &p.causal_off)) return B200FA_ERR_UNSUPPORTED;
  if (!(scale > 0.f) || !std::isfinite(scale)) return B200FA_ERR_UNSUPPORTED;
  if (!dropout_params(opt.dropout_p, opt.seed, opt.offset, &p.drop)) return B200FA_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(lse) % 4 != 0) return B200FA_ERR_MISALIGNED;
  int rc;
  if ((rc = check_view(q, B, Hq, Sq, D, dtype, &p.q)) != B200FA_OK) return rc;
  if ((rc = check_view(k, B, Hkv, Sk, D, dtype, &p.k)) != B200FA_OK) return rc;
  if ((rc = check_view(v, B, Hkv, Sk, D, dtype, &p.v)) != B200FA_OK) return rc;
  if ((rc = check_view(out, B, Hq, Sq, D, dtype, &p.out, true)) != B200FA_OK) return rc;
  p.lse = lse;
  p.B = static_cast<int>(B); p.Hq = static_cast<int>(Hq); p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(Sq); p.Sk = static_cast<int>(Sk); p.D = static_cast<int>(D);
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word;
  p.tiles_per_cta = fwd_tiles();
  p.wait_budget = wait_budget();

  DeviceGuard guard(device);
  if (!guard.ok) {
    note_cuda_error("cudaSetDevice", cudaGetLastError());
    return B200FA_ERR_CUDA;
  }
  if ((rc = check_device_is_sm100(device)) != B200FA_OK) return rc;
  int launches = 0;
  // A stale error left on this thread by an earlier, unrelated runtime call must not be
  // mistaken for a launch failure.
  (void)cudaGetLastError();
  cudaError_t e = (dtype == kF32 || opt.force_simt)
                      ? launch_fwd_simt(p, dtype, static_cast<cudaStream_t>(stream), &launches)
                      : launch_fwd_sm100(p, dtype, static_cast<cudaStream_t>(stream), &launches);
  g_launches += launches;
  if (e != cudaSuccess) note_cuda_error("b200fa_fwd", e);
  return e == cudaSuccess ? B200FA_OK : B200FA_ERR_CUDA;
}

int bwd_impl(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v, const b200fa_tensor4* out,
             const b200fa_tensor4* dout, const float* lse, const b200fa_tensor4* dq, const b200fa_tensor4* dk,
             const b200fa_tensor4* dv, void* workspace, size_t workspace_bytes, int dtype, int causal, float scale,
             void* stream, int device, uint32_t* status_word, const Options& opt) {
  if (!q || !k || !v || !out || !dout || !lse || !dq || !dk || !dv) return B200FA_ERR_NULL;
  if (dtype != kF32 && dtype != kBF16 && dtype != kF16) return B200FA_ERR_BAD_DTYPE;
  const int64_t B = q->shape[0], Hq = q->shape[1], S = q->shape[2], D = q->shape[3];
  const int64_t Hkv = k->shape[1], Sk = k->shape[2];
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || Sk <= 0) return B200FA_ERR_BAD_SHAPE;
  if (B > 65535 || Hq > 65535 || S > (1 << 24) || Sk > (1 << 24)) return B200FA_ERR_BAD_SHAPE;
  if (D != 64 && D != 128) return B200FA_ERR_UNSUPPORTED;
  if (Hq % Hkv != 0) return B200FA_ERR_BAD_SHAPE;
  // one thread block per 64 or 128 key rows of a (batch, kv head): the grid index is a 32-bit int
  if (B * Hkv * ((Sk + 63) / 64) > INT_MAX || B * Hq * ((S + 127) / 128 * 128) > INT_MAX) return B200FA_ERR_BAD_SHAPE;
  BwdParams p;
  std::memset(&p, 0, sizeof(p));
  if (!causal_mode(causal, S, Sk, &p.causal, &p.causal_off)) return B200FA_ERR_UNSUPPORTED;
  if (!(scale > 0.f) || !std::isfinite(scale)) return B200FA_ERR_UNSUPPORTED;
  if (!dropout_params(opt.dropout_p, opt.seed, opt.offset, &p.drop)) return B200FA_ERR_UNSUPPORTED;
  int rc;
  if ((rc = check_view(q, B, Hq, S, D, dtype, &p.q)) != B200FA_OK) return rc;
  if ((rc = check_view(k, B, Hkv, Sk, D, dtype, &p.k)) != B200FA_OK) return rc;
  if ((rc = check_view(v, B, Hkv, Sk, D, dtype, &p.v)) != B200FA_OK) return rc;
  if ((rc = check_view(out, B, Hq, S, D, dtype, &p.out)) != B200FA_OK) return rc;
  if ((rc = check_view(dout, B, Hq, S, D, dtype, &p.dout)) != B200FA_OK) return rc;
  if ((rc = check_view(dq, B, Hq, S, D, dtype, &p.dq, true)) != B200FA_OK) return rc;
  if ((rc = check_view(dk, B, Hkv, Sk, D, dtype, &p.dk, true)) != B200FA_OK) return rc;
  if ((rc = check_view(dv, B, Hkv, Sk, D, dtype, &p.dv, true)) != B200FA_OK) return rc;
  const size_t need = b200fa_bwd_workspace_bytes(B, Hq, Hkv, S, D, dtype);
  if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return B200FA_ERR_WORKSPACE;
  const size_t spad = static_cast<size_t>((S + 127) / 128 * 128);
  const size_t rows = static_cast<size_t>(B) * Hq * spad;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.dpsum = reinterpret_cast<float*>(ws);
  p.lse_log2 = reinterpret_cast<float*>(ws + align256(rows * 4));
  p.lse = lse;
  p.B = static_cast<int>(B); p.Hq = static_cast<int>(Hq); p.Hkv = static_cast<int>(Hkv);
  p.S = static_cast<int>(S); p.Sk = static_cast<int>(Sk); p.Spad = static_cast<int>(spad); p.D = static_cast<int>(D);
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word;
  p.wait_budget = wait_budget();
  p.parts = opt.parts;

  DeviceGuard guard(device);
  if (!guard.ok) {
    note_cuda_error("cudaSetDevice", cudaGetLastError());
    return B200FA_ERR_CUDA;
  }
  if ((rc = check_device_is_sm100(device)) != B200FA_OK) return rc;
  int launches = 0;
  (void)cudaGetLastError();
  cudaError_t e = (dtype == kF32 || opt.force_simt)
                      ? launch_bwd_simt(p, dtype, static_cast<cudaStream_t>(stream), &launches)
                      : launch_bwd_sm100(p, dtype, static_cast<cudaStream_t>(stream), &launches);
  g_launches += launches;
  if (e != cudaSuccess) note_cuda_error("b200fa_bwd", e);
  return e == cudaSuccess ? B200FA_OK : B200FA_ERR_CUDA;
}

// Key splits of the split-KV forward.  The partial kernel keeps three 4-warp CTAs per SM (444 at
// a time on 148 SMs) when a KV head has up to eight query rows, two with more, and a grid runs
// for about (its waves) x (keys in a split + a fixed cost per CTA worth some 192 keys: prologue,
// merge of the warps, the partial written and combined).  Among the split counts up to 64 with
// at least 256 keys a split, take the cheapest by that model; the first found wins a tie, which
// is the one with fewer splits.
int splitkv_splits(int64_t B, int64_t Hkv, int64_t rows, int64_t Sk, int* split_len) {
  const int64_t slots = (rows <= 8 ? 3 : 2) * 148;
  int64_t max_n = (Sk + 255) / 256;
  if (max_n > 64) max_n = 64;
  if (max_n < 1) max_n = 1;
  int64_t best_n = 1, best_len = (Sk + 63) / 64 * 64, best_cost = -1;
  for (int64_t cand = 1; cand <= max_n; ++cand) {
    const int64_t len = ((Sk + cand - 1) / cand + 63) / 64 * 64;
    const int64_t n = (Sk + len - 1) / len;
    const int64_t waves = (B * Hkv * n + slots - 1) / slots;
    const int64_t cost = waves * (len + 192);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_n = n;
      best_len = len;
    }
  }
  *split_len = static_cast<int>(best_len);
  return static_cast<int>(best_n);
}

}  // namespace

extern "C" {

int b200fa_version(void) { return B200FA_VERSION; }

uint64_t b200fa_launch_count(void) { return g_launches.load(); }

const char* b200fa_last_error_detail(void) { return g_detail; }

void b200fa_set_wait_budget(long long cycles) { g_wait_budget.store(cycles > 0 ? cycles : 0); }

long long b200fa_wait_budget(void) { return wait_budget(); }

void b200fa_set_fwd_tiles(int tiles) { g_fwd_tiles.store(tiles == 1 || tiles == 2 ? tiles : 0); }

int b200fa_fwd_tiles(void) { return fwd_tiles(); }

uint32_t b200fa_dropout_threshold(float p) {
  if (!(p > 0.f)) return 0;
  const float t = std::floor(p * 256.f + 0.5f);
  return t > 255.f ? 255u : static_cast<uint32_t>(t);
}

const char* b200fa_strerror(int code) {
  switch (code) {
    case B200FA_OK: return "ok";
    case B200FA_ERR_BAD_DTYPE: return "unsupported element type (expected fp32, bf16 or fp16)";
    case B200FA_ERR_BAD_SHAPE: return "tensor shapes are inconsistent or out of range";
    case B200FA_ERR_BAD_STRIDE: return "tensor strides are unsupported (head_dim stride must be 1, others non-zero multiples of 16 bytes, outputs must not overlap themselves)";
    case B200FA_ERR_MISALIGNED: return "a tensor base address is not 16-byte aligned";
    case B200FA_ERR_WORKSPACE: return "workspace is missing, misaligned or too small";
    case B200FA_ERR_UNSUPPORTED: return "configuration is not supported (head_dim must be 64 or 128, causal in {0, 1, 2}, scale > 0, 0 <= dropout_p < 1, sm_100 device)";
    case B200FA_ERR_CUDA: return "a CUDA runtime or driver call failed";
    case B200FA_ERR_NULL: return "a required pointer is null";
    case B200FA_ERR_TIMEOUT: return "a kernel gave up waiting on an internal barrier";
    default: return "unknown b200fa error";
  }
}

int b200fa_fwd(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
               const b200fa_tensor4* out, float* lse, int dtype, int causal, float scale, void* stream,
               int device, uint32_t* status_word) {
  return fwd_impl(q, k, v, out, lse, dtype, causal, scale, stream, device, status_word, Options{});
}

int b200fa_fwd_simt(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                    const b200fa_tensor4* out, float* lse, int dtype, int causal, float scale, void* stream,
                    int device, uint32_t* status_word) {
  Options opt;
  opt.force_simt = true;
  return fwd_impl(q, k, v, out, lse, dtype, causal, scale, stream, device, status_word, opt);
}

int b200fa_fwd_dropout(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                       const b200fa_tensor4* out, float* lse, int dtype, int causal, float scale, float dropout_p,
                       uint64_t philox_seed, uint64_t philox_offset, int exact_fp32, void* stream, int device,
                       uint32_t* status_word) {
  Options opt;
  opt.force_simt = exact_fp32 != 0;
  opt.dropout_p = dropout_p;
  opt.seed = philox_seed;
  opt.offset = philox_offset;
  return fwd_impl(q, k, v, out, lse, dtype, causal, scale, stream, device, status_word, opt);
}

size_t b200fa_bwd_workspace_bytes(int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seqlen,
                                  int64_t head_dim, int dtype) {
  (void)heads_kv;
  (void)dtype;
  if (batch <= 0 || heads_q <= 0 || seqlen <= 0 || head_dim <= 0) return 0;
  const size_t spad = static_cast<size_t>((seqlen + 127) / 128 * 128);
  const size_t rows = static_cast<size_t>(batch) * heads_q * spad;
  // two fp32 row-statistic arrays (rowsum(dO*O) and lse*log2e), padded to whole 128-row tiles
  return 2 * align256(rows * 4);
}

int b200fa_bwd(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
               const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
               const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv, void* workspace,
               size_t workspace_bytes, int dtype, int causal, float scale, void* stream, int device,
               uint32_t* status_word) {
  return bwd_impl(q, k, v, out, dout, lse, dq, dk, dv, workspace, workspace_bytes, dtype, causal, scale, stream,
                  device, status_word, Options{});
}

int b200fa_bwd_dropout(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                       const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
                       const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv, void* workspace,
                       size_t workspace_bytes, int dtype, int causal, float scale, float dropout_p,
                       uint64_t philox_seed, uint64_t philox_offset, int exact_fp32, void* stream, int device,
                       uint32_t* status_word) {
  Options opt;
  opt.force_simt = exact_fp32 != 0;
  opt.dropout_p = dropout_p;
  opt.seed = philox_seed;
  opt.offset = philox_offset;
  return bwd_impl(q, k, v, out, dout, lse, dq, dk, dv, workspace, workspace_bytes, dtype, causal, scale, stream,
                  device, status_word, opt);
}

int b200fa_bwd_parts(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                     const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
                     const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv, void* workspace,
                     size_t workspace_bytes, int dtype, int causal, float scale, void* stream, int device,
                     uint32_t* status_word, int parts) {
  if (dtype == kF32 || parts < 1 || parts > 7) return B200FA_ERR_UNSUPPORTED;
  Options opt;
  opt.parts = parts;
  return bwd_impl(q, k, v, out, dout, lse, dq, dk, dv, workspace, workspace_bytes, dtype, causal, scale, stream,
                  device, status_word, opt);
}

int b200fa_bwd_simt(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                    const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
                    const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv, void* workspace,
                    size_t workspace_bytes, int dtype, int causal, float scale, void* stream, int device,
                    uint32_t* status_word) {
  Options opt;
  opt.force_simt = true;
  return bwd_impl(q, k, v, out, dout, lse, dq, dk, dv, workspace, workspace_bytes, dtype, causal, scale, stream,
                  device, status_word, opt);
}

size_t b200fa_fwd_splitkv_workspace_bytes(int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seqlen_q,
                                          int64_t seqlen_k, int64_t head_dim) {
  if (batch <= 0 || heads_q <= 0 || heads_kv <= 0 || seqlen_q <= 0 || seqlen_k <= 0 || head_dim <= 0) return 0;
  int split_len = 0;
  const int n = splitkv_splits(batch, heads_kv, heads_q / heads_kv * seqlen_q, seqlen_k, &split_len);
  const size_t rows = static_cast<size_t>(batch) * heads_q * seqlen_q * n;
  return align256(rows * head_dim * 4) + align256(rows * 2 * 4) + align256(static_cast<size_t>(batch) * heads_kv * 4);
}

int b200fa_fwd_splitkv(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                       const b200fa_tensor4* out, float* lse, void* workspace, size_t workspace_bytes, int dtype,
                       int causal, float scale, void* stream, int device, uint32_t* status_word) {
  (void)status_word;   // these kernels wait on nothing but __syncthreads
  if (!q || !k || !v || !out || !lse) return B200FA_ERR_NULL;
  if (dtype != kF32 && dtype != kBF16 && dtype != kF16) return B200FA_ERR_BAD_DTYPE;
  const int64_t B = q->shape[0], Hq = q->shape[1], Sq = q->shape[2], D = q->shape[3];
  const int64_t Hkv = k->shape[1], Sk = k->shape[2];
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Sk <= 0) return B200FA_ERR_BAD_SHAPE;
  if (B > 65535 || Hq > 65535 || Hkv > 65535 || Sk > (1 << 24)) return B200FA_ERR_BAD_SHAPE;
  if (D != 64 && D != 128) return B200FA_ERR_UNSUPPORTED;
  if (Hq % Hkv != 0) return B200FA_ERR_BAD_SHAPE;
  // all query rows of a GQA group ride in one CTA
  if ((Hq / Hkv) * Sq > B200FA_SPLITKV_MAX_ROWS) return B200FA_ERR_UNSUPPORTED;
  SplitKvParams p;
  std::memset(&p, 0, sizeof(p));
  if (!causal_mode(causal, Sq, Sk, &p.causal, &p.causal_off)) return B200FA_ERR_UNSUPPORTED;
  if (!(scale > 0.f) || !std::isfinite(scale)) return B200FA_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(lse) % 4 != 0) return B200FA_ERR_MISALIGNED;
  int rc;
  if ((rc = check_view(q, B, Hq, Sq, D, dtype, &p.q)) != B200FA_OK) return rc;
  if ((rc = check_view(k, B, Hkv, Sk, D, dtype, &p.k)) != B200FA_OK) return rc;
  if ((rc = check_view(v, B, Hkv, Sk, D, dtype, &p.v)) != B200FA_OK) return rc;
  if ((rc = check_view(out, B, Hq, Sq, D, dtype, &p.out, true)) != B200FA_OK) return rc;
  const size_t need = b200fa_fwd_splitkv_workspace_bytes(B, Hq, Hkv, Sq, Sk, D);
  if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return B200FA_ERR_WORKSPACE;
  p.nsplit = splitkv_splits(B, Hkv, Hq / Hkv * Sq, Sk, &p.split_len);
  const size_t rows = static_cast<size_t>(B) * Hq * Sq * p.nsplit;
  p.part_o = reinterpret_cast<float*>(workspace);
  p.part_ml = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + align256(rows * D * 4));
  p.counters = reinterpret_cast<unsigned*>(static_cast<uint8_t*>(workspace) + align256(rows * D * 4) + align256(rows * 2 * 4));
  p.lse = lse;
  p.B = static_cast<int>(B); p.Hq = static_cast<int>(Hq); p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(Sq); p.Sk = static_cast<int>(Sk); p.D = static_cast<int>(D);
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  DeviceGuard guard(device);
  if (!guard.ok) {
    note_cuda_error("cudaSetDevice", cudaGetLastError());
    return B200FA_ERR_CUDA;
  }
  int launches = 0;
  (void)cudaGetLastError();
  const cudaError_t e = launch_fwd_splitkv(p, dtype, static_cast<cudaStream_t>(stream), &launches);
  g_launches += launches;
  if (e != cudaSuccess) note_cuda_error("b200fa_fwd_splitkv", e);
  return e == cudaSuccess ? B200FA_OK : B200FA_ERR_CUDA;
}

int b200fa_selftest_wait_timeout(uint32_t* status_word, long long budget_cycles, void* stream, int device) {
  if (!status_word) return B200FA_ERR_NULL;
  if (budget_cycles <= 0 || budget_cycles > kWaitBudgetCycles) return B200FA_ERR_UNSUPPORTED;
  DeviceGuard guard(device);
  if (!guard.ok) {
    note_cuda_error("cudaSetDevice", cudaGetLastError());
    return B200FA_ERR_CUDA;
  }
  int launches = 0;
  (void)cudaGetLastError();
  const cudaError_t e = launch_wait_timeout_selftest(status_word, budget_cycles, static_cast<cudaStream_t>(stream), &launches);
  g_launches += launches;
  if (e != cudaSuccess) note_cuda_error("b200fa_selftest_wait_timeout", e);
  return e == cudaSuccess ? B200FA_OK : B200FA_ERR_CUDA;
}

void b200fa_dropout_bytes_host(uint64_t philox_seed, uint64_t philox_offset, int64_t batch_head, int64_t row,
                               int64_t col_block, uint8_t* out16) {
  DropoutParams d;
  d.seed = philox_seed;
  d.offset = philox_offset;
  d.threshold = 0;
  d.inv_keep = 1.f;
  uint32_t r[4];
  dropout_bytes16(d, static_cast<int>(batch_head), static_cast<int>(row), static_cast<int>(col_block), r);
  for (int w = 0; w < 4; ++w)
    for (int q = 0; q < 4; ++q) out16[4 * w + q] = static_cast<uint8_t>(r[w] >> (8 * q));
}

int b200fa_status_to_error(uint32_t status_value) {
  if (status_value == 0) return B200FA_OK;
  return (status_value & 0xffff0000u) == kStatusWaitTimeout ? B200FA_ERR_TIMEOUT : B200FA_ERR_CUDA;
}

// ------------------------------------------------------------------------------------------
// Backward without any caller-provided scratch: b200fa_bwd_no_alloc.
//
// Some hosts of this library own no CUDA allocator of their own and must not call one while
// the backward runs: a runtime that hands over raw device pointers from its own pool (the
// reference's MAX DeviceContext is one), an autograd engine thread whose allocator is locked
// or already at its limit, or a serving loop that forbids allocation after warm-up.  For
// them the two scratch arrays of the backward live in this fixed device array instead of
// a workspace argument.  Every GPU that loads the library holds these bytes until the
// process exits.
// ------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[B200FA_NO_ALLOC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address:
// the address each device gave the array is looked up once per device, with that device
// current, and cached here.
static void* g_static_scratch_addr[64] = {};
static std::mutex g_static_scratch_mutex;

static int static_scratch_for(int device, void** out) {
  if (device < 0 || device >= 64) return B200FA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_addr[device]) {
    DeviceGuard guard(device);
    if (!guard.ok) {
      note_cuda_error("cudaSetDevice", cudaGetLastError());
      return B200FA_ERR_CUDA;
    }
    void* addr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&addr, g_static_scratch);
    if (e != cudaSuccess || !addr) {
      note_cuda_error("cudaGetSymbolAddress(g_static_scratch)", e);
      return B200FA_ERR_CUDA;
    }
    g_static_scratch_addr[device] = addr;
  }
  *out = g_static_scratch_addr[device];
  return B200FA_OK;
}

size_t b200fa_no_alloc_scratch_bytes(void) { return B200FA_NO_ALLOC_SCRATCH_BYTES; }

int b200fa_bwd_no_alloc(const b200fa_tensor4* q, const b200fa_tensor4* k, const b200fa_tensor4* v,
                        const b200fa_tensor4* out, const b200fa_tensor4* dout, const float* lse,
                        const b200fa_tensor4* dq, const b200fa_tensor4* dk, const b200fa_tensor4* dv, int dtype,
                        int causal, float scale, void* stream, int device, uint32_t* status_word) {
  if (!q || !k) return B200FA_ERR_NULL;
  const size_t need = b200fa_bwd_workspace_bytes(q->shape[0], q->shape[1], k->shape[1], q->shape[2], q->shape[3], dtype);
  if (need > B200FA_NO_ALLOC_SCRATCH_BYTES) {
    snprintf(g_detail, sizeof(g_detail),
             "b200fa_bwd_no_alloc: this problem needs %zu bytes of scratch but the built-in scratch holds %zu; "
             "use b200fa_bwd with a caller-provided workspace",
             need, static_cast<size_t>(B200FA_NO_ALLOC_SCRATCH_BYTES));
    return B200FA_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  const int rc = static_scratch_for(device, &scratch);
  if (rc != B200FA_OK) return rc;
  // parts 7 | 8: the whole backward, every kernel on the caller's stream, so that this entry
  // point creates no stream or event either
  Options opt;
  opt.parts = 7 | 8;
  return bwd_impl(q, k, v, out, dout, lse, dq, dk, dv, scratch, B200FA_NO_ALLOC_SCRATCH_BYTES, dtype, causal, scale,
                  stream, device, status_word, opt);
}

}  // extern "C"
