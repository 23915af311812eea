// Host side of the C ABI declared in include/sage_b200.h: argument checks, TMA tensor maps,
// kernel selection and launches.  No torch types, no allocation, no synchronisation.
#include "../../include/sage_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "attn_kernel.cuh"
#include "merge_kernels.cuh"
#include "prep_kernels.cuh"

// K-mean scratch of sage_quant_qk_int8_smooth_static: part of the library image, never allocated.
// In host code this name is only a handle for cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) unsigned char g_static_kmean[SAGE_STATIC_KMEAN_MAX_ELEMS * 2];

namespace {

thread_local char g_err[512] = "";
std::atomic<long long> g_wait_limit_cycles{sage::kWaitLimitCycles};
std::atomic<int> g_test_drop_v_load{0};
std::atomic<int*> g_status_host[64];      // per device: mapped pinned host word for failure codes (sage_set_status_mirror)

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define SAGE_REQUIRE(cond, ...) \
  do {                          \
    if (!(cond)) return fail(SAGE_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define SAGE_CUDA(expr)                                                                        \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    if (e_ != cudaSuccess) return fail(SAGE_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool strides_ok(const sage_strided_t* t) {
  return t->stride_b % 8 == 0 && t->stride_h % 8 == 0 && t->stride_s % 8 == 0;
}
sage::StridedView view_of(const sage_strided_t* t) {
  sage::StridedView v;
  v.ptr = t->ptr;
  v.stride_b = t->stride_b;
  v.stride_h = t->stride_h;
  v.stride_s = t->stride_s;
  return v;
}

// cuTensorMapEncodeTiled is taken from the driver at run time, so the library links against the
// CUDA runtime only.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

int encode_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims,
               const cuuint64_t* strides_bytes, const cuuint32_t* box, CUtensorMapSwizzle swz, const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(SAGE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint32_t ones[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims, strides_bytes, box, ones,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SAGE_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  return SAGE_OK;
}

// Tiled map of a 16-bit [B,H,S,D] tensor in the caller's layout: dimensions (D, S, H, B) with the
// caller's element strides, boxes of `box_rows` rows x 64 columns, 128-byte swizzle.  A dimension of
// extent 1 may carry any stride in the caller's tensor; it gets the span of the others so that the
// map stays well formed.
int encode_strided_16bit(CUtensorMap* map, CUtensorMapDataType dt, const void* base, int D, long long S, long long H,
                         long long B, long long stride_s, long long stride_h, long long stride_b, int box_rows,
                         const char* what) {
  cuuint64_t ss = (cuuint64_t)stride_s * 2, sh = (cuuint64_t)stride_h * 2, sb = (cuuint64_t)stride_b * 2;
  cuuint64_t span = (cuuint64_t)D * 2;
  if (S > 1 && ss * S > span) span = ss * S;
  if (H > 1 && sh * H > span) span = sh * H;
  if (B > 1 && sb * B > span) span = sb * B;
  span = (span + 15) & ~(cuuint64_t)15;
  if (S == 1) ss = span;
  if (H == 1) sh = span;
  if (B == 1) sb = span;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {ss, sh, sb};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  return encode_map(map, dt, 4, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, what);
}

template <typename T, int D>
int launch_prep(const sage::PrepParams& p, int v_blocks, cudaStream_t stream) {
  const int grid = p.q_blocks + p.k_blocks + v_blocks;
  if (grid == 0) return SAGE_OK;
  sage::sage_prep_kernel<T, D><<<grid, sage::kPrepThreads, 0, stream>>>(p);
  SAGE_CUDA(cudaGetLastError());
  return SAGE_OK;
}

int dispatch_prep(int dtype, int D, const sage::PrepParams& p, int v_blocks, cudaStream_t stream) {
  if (dtype == SAGE_DTYPE_F16) {
    return D == 64 ? launch_prep<__half, 64>(p, v_blocks, stream) : launch_prep<__half, 128>(p, v_blocks, stream);
  }
  return D == 64 ? launch_prep<__nv_bfloat16, 64>(p, v_blocks, stream)
                 : launch_prep<__nv_bfloat16, 128>(p, v_blocks, stream);
}

int v_block_count(long long B, long long H, long long S, int D) {
  const long long n_vec = B * H * S * (D / 8);
  return static_cast<int>((n_vec + sage::kPrepThreads * 4 - 1) / (sage::kPrepThreads * 4));
}

// The fields of AttnParams that do not depend on the kind of Q / K.
void fill_attn_params(sage::AttnParams* pp, void* o, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                      int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv, float* lse, int* status) {
  sage::AttnParams& p = *pp;
  memset(&p, 0, sizeof(p));
  p.o = o; p.o_stride_b = o_stride_b; p.o_stride_h = o_stride_h; p.o_stride_s = o_stride_s;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv;
  p.q_groups = (Sq + sage::kQGroupRows - 1) / sage::kQGroupRows;
  p.k_groups = (Skv + sage::kKGroupRows - 1) / sage::kKGroupRows;
  p.n_q_tiles = (Sq + sage::kBlockM - 1) / sage::kBlockM;
  // 8 heads at a time (each needs Skv * D * 3 bytes of K and V in L2), whole GQA groups only
  const int rep = Hq / Hkv;
  p.head_group = rep * ((8 + rep - 1) / rep);
  p.out_bf16 = (out_dtype == SAGE_DTYPE_BF16);
  p.lse = lse;
  p.status = status;
  {
    int dev = 0;
    p.status_host = (status != nullptr && cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64)
                        ? g_status_host[dev].load(std::memory_order_relaxed) : nullptr;
  }
  // Every barrier wait in the kernel gives up after this many SM clocks (about one second) and
  // reports through `status`.  The failure-detection test shortens the bound and makes one wait run
  // out on purpose through sage_test_set_wait_limit_us / sage_test_drop_v_load; the dropped load is
  // only honoured together with a shortened bound.
  const long long limit = g_wait_limit_cycles.load(std::memory_order_relaxed);
  p.wait_limit_cycles = limit;
  p.test_drop_v_load = (g_test_drop_v_load.load(std::memory_order_relaxed) != 0 && limit < sage::kWaitLimitCycles) ? 1 : 0;
}

int sm_count(int* out) {
  static std::atomic<int> cached[64];
  int dev = 0;
  SAGE_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64) {
    const int have = cached[dev].load(std::memory_order_relaxed);
    if (have > 0) {
      *out = have;
      return SAGE_OK;
    }
  }
  int sms = 0;
  SAGE_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (dev >= 0 && dev < 64) cached[dev].store(sms, std::memory_order_relaxed);
  *out = sms;
  return SAGE_OK;
}

// Choice between the plain and the persistent launch: -1 = by the cost model, 0 = never persistent,
// 1 = always.  SAGE_STREAMK in the environment (read once, at the first use) gives the initial
// value; sage_set_streamk changes it afterwards.
std::atomic<int> g_streamk_mode{-2};      // -2: environment not looked at yet
int streamk_override() {
  static std::once_flag once;
  std::call_once(once, [] {
    int value = -1;
    const char* e = getenv("SAGE_STREAMK");
    if (e != nullptr && (e[0] == '0' || e[0] == '1')) value = e[0] - '0';
    int expected = -2;
    g_streamk_mode.compare_exchange_strong(expected, value);
  });
  return g_streamk_mode.load(std::memory_order_relaxed);
}

// Persistent ("stream-K") scheduling.  The plain launch gives every CTA one whole item (a 128-row
// query tile with all of its KV tiles); with two CTAs per SM that fills the GPU in waves of
// 2 * SMs items, and a problem of 320 items (B=1, H=10, S=4096) takes two waves where 1.08 would do.
// The persistent launch cuts the T = sum of KV-tile steps into 2 * SMs equal spans instead; a span
// that covers part of an item leaves a partial result in the workspace and a merge kernel combines
// them.  It costs about three KV-tile steps per CTA (a second pipeline fill and drain, the merge), so
// it is used when the estimate says it saves at least 8 %.
struct StreamKPlan {
  bool use = false;
  int grid = 0;
  int nkv_full = 0;
  int tiles_per_head = 0;
  long long total_tiles = 0;
  size_t workspace_bytes = 0;
};

int plan_streamk(StreamKPlan* plan, int B, int Hq, int Sq, int Skv, int D, int is_causal) {
  *plan = StreamKPlan();
  if (Sq <= 0 || Skv <= 0) return SAGE_OK;
  const int forced = streamk_override();
  if (forced == 0) return SAGE_OK;
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc) return rc;
  const long long slots = 2LL * sms;
  const long long nq = (Sq + sage::kBlockM - 1) / sage::kBlockM;
  const long long nkv = (Skv + sage::kBlockN - 1) / sage::kBlockN;
  long long per_head;
  if (!is_causal) per_head = nq * nkv;
  else if (nq <= nkv) per_head = nq * (nq + 1) / 2;
  else per_head = nkv * (nkv + 1) / 2 + (nq - nkv) * nkv;
  const long long items = nq * B * Hq;
  const long long total = per_head * B * Hq;
  if (per_head > 0x7fffffffLL || items > 0x7fffffffLL) return SAGE_OK;
  const long long grid = total < slots ? total : slots;
  // Makespans in KV-tile steps of a CTA that shares its SM with another one.  Plain launch: full
  // waves of `slots` items, then a tail wave that runs about 1.4x faster per CTA if it leaves every
  // CTA alone on its SM; under a causal mask the heavy-first order packs items almost evenly.  About
  // 3 steps of fixed cost per wave (set-up, pipeline fill and drain, epilogue).  Persistent launch:
  // 1.04 T / G steps, the same fixed cost once, two more pipeline restarts at item boundaries, and the
  // merge (about 5 us plus its traffic at 4 TB/s; one step is about 1.95 us).
  double plain;
  if (is_causal) {
    plain = std::max<double>(static_cast<double>(std::min(nq, nkv)), 1.03 * total / slots) + 3.0;
  } else {
    const long long full = items / slots, tail = items % slots;
    plain = static_cast<double>(full) * (nkv + 3.0);
    if (tail > 0) plain += (tail <= sms ? 0.72 : 1.0) * nkv + 3.0;
  }
  const double merge_mb = (static_cast<double>(grid) * 2 * sage::kBlockM * D * 4 +
                           static_cast<double>(std::min<long long>(items, 2 * grid)) * sage::kBlockM * D * 2) / 1e6;
  const double merge_steps = (5.0 + merge_mb / 4.0) / 1.95;
  // (1.04: the persistent CTAs of an SM run in lock-step, without the de-phasing yield of the plain launch)
  const double persistent = 1.04 * static_cast<double>(total) / grid + 5.0 + merge_steps;
  bool use = persistent < 0.95 * plain;
  if (forced == 1) use = true;
  if (!use) return SAGE_OK;
  plan->use = true;
  plan->grid = static_cast<int>(grid);
  plan->nkv_full = static_cast<int>(nkv);
  plan->tiles_per_head = static_cast<int>(per_head);
  plan->total_tiles = total;
  plan->workspace_bytes = static_cast<size_t>(grid) * 2 * sage::kBlockM * (D + 1) * sizeof(float);
  return SAGE_OK;
}

// (Setting the attribute twice from two host threads that race on the first call is harmless.)
template <typename Kernel>
int configure_smem(Kernel kern, int smem_bytes, std::atomic<bool>* configured) {
  int dev = 0;
  SAGE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    SAGE_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  return SAGE_OK;
}

template <int D, bool CAUSAL, bool DUMP, bool QKF = false, int KST = 0>
int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                const sage::AttnParams& p, cudaStream_t stream) {
  auto kern = sage::sage_attn_kernel<D, CAUSAL, DUMP, QKF, KST>;
  constexpr int kSmem = sage::AttnSmem<D, QKF ? 2 : 1, KST>::kTotal;
  static std::atomic<bool> configured[64];
  int rc = configure_smem(kern, kSmem, configured);
  if (rc) return rc;
  const long long grid = static_cast<long long>(p.n_q_tiles) * p.B * p.Hq;
  if (grid > 0x7fffffffLL) return fail(SAGE_ERR_INVALID, "too many query tiles for one launch (%lld)", grid);
  kern<<<static_cast<unsigned>(grid), sage::kAttnThreads, kSmem, stream>>>(tq, tk, tv, to, p);
  SAGE_CUDA(cudaGetLastError());
  return SAGE_OK;
}

// The persistent launch and its merge.  `workspace` holds the partial results:
// [grid][2][128][D] fp32 outputs, then [grid][2][128] fp32 log-sum-exps.
template <int D, bool CAUSAL, bool QKF>
int launch_attn_streamk(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& to,
                        sage::AttnParams p, const StreamKPlan& plan, void* workspace, cudaStream_t stream) {
  auto kern = sage::sage_attn_kernel<D, CAUSAL, false, QKF, 0, true>;
  constexpr int kSmem = sage::AttnSmem<D, QKF ? 2 : 1, 0>::kTotal;
  static std::atomic<bool> configured[64];
  int rc = configure_smem(kern, kSmem, configured);
  if (rc) return rc;
  p.sk_total_tiles = plan.total_tiles;
  p.sk_tiles_per_head = plan.tiles_per_head;
  p.sk_nkv_full = plan.nkv_full;
  p.part_o = static_cast<float*>(workspace);
  p.part_lse = p.part_o + static_cast<size_t>(plan.grid) * 2 * sage::kBlockM * D;
  kern<<<static_cast<unsigned>(plan.grid), sage::kAttnThreads, kSmem, stream>>>(tq, tk, tv, to, p);
  SAGE_CUDA(cudaGetLastError());
  sage::MergeParams m;
  m.part_o = p.part_o; m.part_lse = p.part_lse;
  m.o = p.o; m.o_stride_b = p.o_stride_b; m.o_stride_h = p.o_stride_h; m.o_stride_s = p.o_stride_s;
  m.lse = p.lse;
  m.Hq = p.Hq; m.Sq = p.Sq; m.n_q_tiles = p.n_q_tiles;
  m.nkv_full = plan.nkv_full; m.tiles_per_head = plan.tiles_per_head; m.total_tiles = plan.total_tiles;
  m.attn_grid = plan.grid;
  m.causal = CAUSAL ? 1 : 0; m.out_bf16 = p.out_bf16;
  const long long items = static_cast<long long>(p.n_q_tiles) * p.B * p.Hq;
  sage::sage_attn_merge_kernel<D><<<static_cast<unsigned>(items * sage::kMergeSplit), 256, 0, stream>>>(m);
  SAGE_CUDA(cudaGetLastError());
  return SAGE_OK;
}

// Device address of g_static_kmean on the current device, looked up once per device.
int static_kmean_address(void** out) {
  static void* addr[64] = {};
  static std::mutex mu;
  int dev = 0;
  SAGE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SAGE_ERR_INVALID, "device index %d is out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    SAGE_CUDA(cudaGetSymbolAddress(&p, g_static_kmean));
    addr[dev] = p;
  }
  *out = addr[dev];
  return SAGE_OK;
}

}  // namespace

extern "C" {

int sage_abi_version(void) { return SAGE_ABI_VERSION; }
const char* sage_last_error(void) { return g_err; }

int sage_set_status_mirror(int* host_word) {
  int dev = 0;
  SAGE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SAGE_ERR_INVALID, "device index %d is out of range", dev);
  g_status_host[dev].store(host_word, std::memory_order_relaxed);
  return SAGE_OK;
}
int sage_test_set_wait_limit_us(long long us) {
  g_wait_limit_cycles.store(us > 0 ? us * 2000 : sage::kWaitLimitCycles, std::memory_order_relaxed);   // ~2 GHz
  return SAGE_OK;
}
int sage_set_streamk(int mode) {
  if (mode < -1 || mode > 1) return fail(SAGE_ERR_INVALID, "sage_set_streamk: mode must be -1 (auto), 0 (off) or 1 (on)");
  streamk_override();                     // settle the environment's value first, so that it cannot overwrite this one
  g_streamk_mode.store(mode, std::memory_order_relaxed);
  return SAGE_OK;
}
int sage_test_drop_v_load(int on) {
  g_test_drop_v_load.store(on ? 1 : 0, std::memory_order_relaxed);
  return SAGE_OK;
}

int sage_mean_seq(const sage_strided_t* k, int dtype, int B, int H, int S, int D, void* mean_out, void* stream) {
  SAGE_REQUIRE(k && k->ptr && mean_out, "sage_mean_seq: null pointer");
  SAGE_REQUIRE(dtype == SAGE_DTYPE_F16 || dtype == SAGE_DTYPE_BF16, "sage_mean_seq: dtype must be f16 or bf16");
  SAGE_REQUIRE(D == 64 || D == 128, "sage_mean_seq: head_dim must be 64 or 128, got %d", D);
  SAGE_REQUIRE(B > 0 && H > 0 && S > 0, "sage_mean_seq: empty tensor (B=%d H=%d S=%d)", B, H, S);
  SAGE_REQUIRE(H <= 65535 && B <= 65535, "sage_mean_seq: B and H must be <= 65535");
  SAGE_REQUIRE(aligned16(k->ptr) && strides_ok(k), "sage_mean_seq: k needs a 16-byte aligned base and strides % 8 == 0");
  sage::MeanParams p;
  p.k = view_of(k);
  p.mean_out = mean_out;
  p.B = B; p.H = H; p.S = S; p.D = D;
  dim3 grid(sage::kMeanCluster, H, B);                  // one cluster of 8 CTAs per (b, h)
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SAGE_DTYPE_F16) {
    if (D == 128) sage::sage_kmean_kernel<__half, 128><<<grid, 256, 0, st>>>(p);
    else sage::sage_kmean_kernel<__half, 64><<<grid, 256, 0, st>>>(p);
  } else {
    if (D == 128) sage::sage_kmean_kernel<__nv_bfloat16, 128><<<grid, 256, 0, st>>>(p);
    else sage::sage_kmean_kernel<__nv_bfloat16, 64><<<grid, 256, 0, st>>>(p);
  }
  SAGE_CUDA(cudaGetLastError());
  return SAGE_OK;
}

int sage_quant_qk_int8(const sage_strided_t* q, const sage_strided_t* k, const void* k_mean,
                       const sage_strided_t* v, void* v16, int dtype, int B, int Hq, int Hkv, int Sq, int Skv,
                       int D, float sm_scale, int8_t* q_i8, float* q_scale, int8_t* k_i8, float* k_scale,
                       void* stream) {
  // One side may be empty (Sq == 0 or Skv == 0): its pointers are not looked at.  That is how a
  // caller quantises K once and Q per call.
  SAGE_REQUIRE(Sq <= 0 || (q && q->ptr && q_i8 && q_scale), "sage_quant_qk_int8: null q pointer");
  SAGE_REQUIRE(Skv <= 0 || (k && k->ptr && k_i8 && k_scale), "sage_quant_qk_int8: null k pointer");
  SAGE_REQUIRE(dtype == SAGE_DTYPE_F16 || dtype == SAGE_DTYPE_BF16, "sage_quant_qk_int8: dtype must be f16 or bf16");
  SAGE_REQUIRE(D == 64 || D == 128, "sage_quant_qk_int8: head_dim must be 64 or 128, got %d", D);
  SAGE_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Sq >= 0 && Skv >= 0, "sage_quant_qk_int8: bad sizes");
  SAGE_REQUIRE(Sq == 0 || (aligned16(q->ptr) && strides_ok(q) && aligned16(q_i8)),
               "sage_quant_qk_int8: q needs a 16-byte aligned base and strides % 8 == 0, q_i8 a 16-byte aligned base");
  SAGE_REQUIRE(Skv == 0 || (aligned16(k->ptr) && strides_ok(k) && aligned16(k_i8)),
               "sage_quant_qk_int8: k needs a 16-byte aligned base and strides % 8 == 0, k_i8 a 16-byte aligned base");
  SAGE_REQUIRE(k_mean == nullptr || aligned16(k_mean), "sage_quant_qk_int8: k_mean must be 16-byte aligned");
  const bool do_v = (v != nullptr && v16 != nullptr);
  if (do_v) {
    SAGE_REQUIRE(v->ptr && aligned16(v->ptr) && strides_ok(v) && aligned16(v16),
                 "sage_quant_qk_int8: v / v16 need 16-byte aligned bases and strides % 8 == 0");
  }
  sage::PrepParams p;
  memset(&p, 0, sizeof(p));
  if (Sq > 0) p.q = view_of(q);
  if (Skv > 0) p.k = view_of(k);
  if (do_v) p.v = view_of(v);
  p.q_i8 = q_i8; p.k_i8 = k_i8; p.q_scale = q_scale; p.k_scale = k_scale;
  p.k_mean = k_mean;
  p.v16 = do_v ? static_cast<__half*>(v16) : nullptr;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv;
  p.q_groups = (Sq + sage::kQGroupRows - 1) / sage::kQGroupRows;
  p.k_groups = (Skv + sage::kKGroupRows - 1) / sage::kKGroupRows;
  // csrc/attn_gfx11.cu:34,1995: float(sm_scale) * 1.4426950408889634f, one fp32 multiply
  volatile float s = sm_scale;
  volatile float l2e = 1.4426950408889634f;
  p.sm_scale_log2e = s * l2e;
  const long long qg = static_cast<long long>(B) * Hq * p.q_groups;
  const long long kg = static_cast<long long>(B) * Hkv * p.k_groups;
  p.q_blocks = static_cast<int>((qg + sage::kQGroupsPerBlock - 1) / sage::kQGroupsPerBlock);
  p.k_blocks = static_cast<int>((kg + sage::kKGroupsPerBlock - 1) / sage::kKGroupsPerBlock);
  const int v_blocks = do_v ? v_block_count(B, Hkv, Skv, D) : 0;
  return dispatch_prep(dtype, D, p, v_blocks, static_cast<cudaStream_t>(stream));
}

int sage_prep_smooth_preferred(int B, int Hkv) {
  // The one-launch form keeps one cluster of 8 CTAs busy per (batch, kv-head) for the length of a
  // dependent chain (sum, exchange, quantise: about 30 us at S = 8192): it wins while all heads are
  // resident at once with room to spare for the Q and V blocks, i.e. up to a quarter of the CTA slots.
  int sms = 0;
  if (B <= 0 || Hkv <= 0 || sm_count(&sms) != SAGE_OK) return 0;
  return static_cast<long long>(B) * Hkv <= sms / sage::kMeanCluster ? 1 : 0;
}

int sage_prep_smooth_qkv(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v, void* v16, int dtype,
                         int B, int Hq, int Hkv, int Sq, int Skv, int D, float sm_scale, int8_t* q_i8, float* q_scale,
                         int8_t* k_i8, float* k_scale, void* k_mean_out, void* stream) {
  SAGE_REQUIRE(Sq <= 0 || (q && q->ptr && q_i8 && q_scale), "sage_prep_smooth_qkv: null q pointer");
  SAGE_REQUIRE(k && k->ptr && k_i8 && k_scale && k_mean_out, "sage_prep_smooth_qkv: null k pointer");
  SAGE_REQUIRE(dtype == SAGE_DTYPE_F16 || dtype == SAGE_DTYPE_BF16, "sage_prep_smooth_qkv: dtype must be f16 or bf16");
  SAGE_REQUIRE(D == 64 || D == 128, "sage_prep_smooth_qkv: head_dim must be 64 or 128, got %d", D);
  SAGE_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Sq >= 0 && Skv >= 1, "sage_prep_smooth_qkv: bad sizes (Skv must be >= 1)");
  SAGE_REQUIRE(Sq <= 0 || (aligned16(q->ptr) && strides_ok(q) && aligned16(q_i8)),
               "sage_prep_smooth_qkv: q needs a 16-byte aligned base and strides % 8 == 0, q_i8 a 16-byte aligned base");
  SAGE_REQUIRE(aligned16(k->ptr) && strides_ok(k) && aligned16(k_i8) && aligned16(k_mean_out),
               "sage_prep_smooth_qkv: k needs a 16-byte aligned base and strides % 8 == 0, k_i8 / k_mean 16-byte aligned bases");
  const bool do_v = (v != nullptr && v16 != nullptr);
  if (do_v) {
    SAGE_REQUIRE(v->ptr && aligned16(v->ptr) && strides_ok(v) && aligned16(v16),
                 "sage_prep_smooth_qkv: v / v16 need 16-byte aligned bases and strides % 8 == 0");
  }
  sage::PrepParams p;
  memset(&p, 0, sizeof(p));
  if (Sq > 0) p.q = view_of(q);
  p.k = view_of(k);
  if (do_v) p.v = view_of(v);
  p.q_i8 = q_i8; p.k_i8 = k_i8; p.q_scale = q_scale; p.k_scale = k_scale;
  p.v16 = do_v ? static_cast<__half*>(v16) : nullptr;
  p.k_mean_out = k_mean_out;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Skv = Skv;
  p.q_groups = (Sq + sage::kQGroupRows - 1) / sage::kQGroupRows;
  p.k_groups = (Skv + sage::kKGroupRows - 1) / sage::kKGroupRows;
  volatile float s = sm_scale;                          // csrc/attn_gfx11.cu:34,1995: one fp32 multiply
  volatile float l2e = 1.4426950408889634f;
  p.sm_scale_log2e = s * l2e;
  // K clusters: at most two K CTAs per SM at a time, every cluster the same number of heads (+-1)
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc) return rc;
  const int n_heads = B * Hkv;
  const int max_clusters = std::max(1, 2 * sms / sage::kMeanCluster);
  const int rounds = (n_heads + max_clusters - 1) / max_clusters;
  p.k_clusters = (n_heads + rounds - 1) / rounds;
  constexpr int kQGroupsPerBlock = sage::kFusedThreads / 64;
  const long long qg = static_cast<long long>(B) * Hq * p.q_groups;
  p.q_blocks = static_cast<int>((qg + kQGroupsPerBlock - 1) / kQGroupsPerBlock);
  p.k_blocks = p.k_clusters * sage::kMeanCluster;
  long long v_blocks = 0;
  if (do_v) {
    const long long n_vec = static_cast<long long>(B) * Hkv * Skv * (D / 8);
    v_blocks = (n_vec + sage::kFusedThreads * 4 - 1) / (sage::kFusedThreads * 4);
  }
  long long grid = p.k_blocks + p.q_blocks + v_blocks;
  grid = (grid + sage::kMeanCluster - 1) / sage::kMeanCluster * sage::kMeanCluster;     // whole clusters
  SAGE_REQUIRE(grid <= 0x7fffffffLL, "sage_prep_smooth_qkv: too many blocks for one launch (%lld)", grid);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned g = static_cast<unsigned>(grid);
  if (dtype == SAGE_DTYPE_F16) {
    if (D == 128) sage::sage_prep_smooth_kernel<__half, 128><<<g, sage::kFusedThreads, 0, st>>>(p);
    else sage::sage_prep_smooth_kernel<__half, 64><<<g, sage::kFusedThreads, 0, st>>>(p);
  } else {
    if (D == 128) sage::sage_prep_smooth_kernel<__nv_bfloat16, 128><<<g, sage::kFusedThreads, 0, st>>>(p);
    else sage::sage_prep_smooth_kernel<__nv_bfloat16, 64><<<g, sage::kFusedThreads, 0, st>>>(p);
  }
  SAGE_CUDA(cudaGetLastError());
  return SAGE_OK;
}

int sage_quant_qk_int8_smooth_static(const sage_strided_t* q, const sage_strided_t* k, int dtype, int B, int Hq,
                                     int Hkv, int Sq, int Skv, int D, float sm_scale, int8_t* q_i8, float* q_scale,
                                     int8_t* k_i8, float* k_scale, void* stream) {
  SAGE_REQUIRE(B > 0 && Hkv > 0 && D > 0 && Skv >= 1, "sage_quant_qk_int8_smooth_static: bad sizes (Skv must be >= 1)");
  const long long elems = static_cast<long long>(B) * Hkv * D;
  SAGE_REQUIRE(elems <= SAGE_STATIC_KMEAN_MAX_ELEMS,
               "sage_quant_qk_int8_smooth_static: B*Hkv*D = %lld exceeds the built-in K-mean buffer of %d elements; "
               "use sage_mean_seq + sage_quant_qk_int8 with a caller-allocated mean",
               elems, SAGE_STATIC_KMEAN_MAX_ELEMS);
  void* mean = nullptr;
  int rc = static_kmean_address(&mean);
  if (rc) return rc;
  rc = sage_mean_seq(k, dtype, B, Hkv, Skv, D, mean, stream);
  if (rc) return rc;
  return sage_quant_qk_int8(q, k, mean, nullptr, nullptr, dtype, B, Hq, Hkv, Sq, Skv, D, sm_scale, q_i8, q_scale,
                            k_i8, k_scale, stream);
}

int sage_v_to_f16(const sage_strided_t* v, int dtype, int B, int H, int S, int D, void* v16, void* stream) {
  SAGE_REQUIRE(v && v->ptr && v16, "sage_v_to_f16: null pointer");
  SAGE_REQUIRE(dtype == SAGE_DTYPE_F16 || dtype == SAGE_DTYPE_BF16, "sage_v_to_f16: dtype must be f16 or bf16");
  SAGE_REQUIRE(D == 64 || D == 128, "sage_v_to_f16: head_dim must be 64 or 128, got %d", D);
  SAGE_REQUIRE(B > 0 && H > 0 && S >= 0, "sage_v_to_f16: bad sizes");
  SAGE_REQUIRE(aligned16(v->ptr) && strides_ok(v) && aligned16(v16),
               "sage_v_to_f16: v / v16 need 16-byte aligned bases and strides % 8 == 0");
  sage::PrepParams p;
  memset(&p, 0, sizeof(p));
  p.v = view_of(v);
  p.v16 = static_cast<__half*>(v16);
  p.B = B; p.Hq = H; p.Hkv = H; p.Sq = 0; p.Skv = S;
  return dispatch_prep(dtype, D, p, v_block_count(B, H, S, D), static_cast<cudaStream_t>(stream));
}

int sage_qk_int8_sv_f16_attn(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o,
                             int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, const float* q_scale,
                             const float* k_scale, int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv, int D,
                             int is_causal, int32_t* s_dump, int* status, void* stream) {
  return sage_qk_int8_sv_f16_attn_lse(q_i8, k_i8, v16, o, o_stride_b, o_stride_h, o_stride_s, q_scale, k_scale,
                                      out_dtype, B, Hq, Hkv, Sq, Skv, D, is_causal, nullptr, s_dump, status, stream);
}

int sage_qk_int8_sv_f16_attn_lse(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o,
                                 int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, const float* q_scale,
                                 const float* k_scale, int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv,
                                 int D, int is_causal, float* lse, int32_t* s_dump, int* status, void* stream) {
  return sage_qk_int8_sv_f16_attn_ws(q_i8, k_i8, v16, o, o_stride_b, o_stride_h, o_stride_s, q_scale, k_scale,
                                     out_dtype, B, Hq, Hkv, Sq, Skv, D, is_causal, lse, s_dump, status, nullptr, 0,
                                     stream);
}

int64_t sage_attn_workspace_bytes(int B, int Hq, int Sq, int Skv, int D, int is_causal) {
  StreamKPlan plan;
  if (B <= 0 || Hq <= 0 || (D != 64 && D != 128)) return 0;
  if (plan_streamk(&plan, B, Hq, Sq, Skv, D, is_causal) != SAGE_OK) return 0;
  return plan.use ? static_cast<int64_t>(plan.workspace_bytes) : 0;
}

namespace {
int attn_int8_impl(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o, int64_t o_stride_b,
                   int64_t o_stride_h, int64_t o_stride_s, const float* q_scale, const float* k_scale, int out_dtype,
                   int B, int Hq, int Hkv, int Sq, int Skv, int D, int is_causal, float* lse, int32_t* s_dump,
                   int* status, void* workspace, int64_t workspace_bytes, int n_peers, void* const* peer_o, void* stream);
}  // namespace

int sage_qk_int8_sv_f16_attn_ws(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o,
                                int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, const float* q_scale,
                                const float* k_scale, int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv,
                                int D, int is_causal, float* lse, int32_t* s_dump, int* status, void* workspace,
                                int64_t workspace_bytes, void* stream) {
  return attn_int8_impl(q_i8, k_i8, v16, o, o_stride_b, o_stride_h, o_stride_s, q_scale, k_scale, out_dtype, B, Hq, Hkv,
                        Sq, Skv, D, is_causal, lse, s_dump, status, workspace, workspace_bytes, 0, nullptr, stream);
}

int sage_qk_int8_sv_f16_attn_scatter(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o,
                                     int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, const float* q_scale,
                                     const float* k_scale, int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv,
                                     int D, int is_causal, float* lse, int* status, int n_peers, void* const* peer_o,
                                     void* stream) {
  static_assert(sage::kMaxPeers == SAGE_MAX_PEERS, "the header and the kernel agree on the number of peers");
  {
    SAGE_REQUIRE(n_peers >= 0 && n_peers <= sage::kMaxPeers, "sage_qk_int8_sv_f16_attn_scatter: n_peers must be 0..%d, got %d",
                 sage::kMaxPeers, n_peers);
    SAGE_REQUIRE(n_peers == 0 || peer_o != nullptr, "sage_qk_int8_sv_f16_attn_scatter: null peer list");
    for (int i = 0; i < n_peers; ++i) {
      SAGE_REQUIRE(peer_o[i] != nullptr && aligned16(peer_o[i]) && peer_o[i] != o,
                   "sage_qk_int8_sv_f16_attn_scatter: peer buffer %d must be a 16-byte aligned address other than o", i);
    }
  }
  return attn_int8_impl(q_i8, k_i8, v16, o, o_stride_b, o_stride_h, o_stride_s, q_scale, k_scale, out_dtype, B, Hq, Hkv,
                        Sq, Skv, D, is_causal, lse, nullptr, status, nullptr, 0, n_peers, peer_o, stream);
}

// Mapping of another process's device buffer (one process per GPU on one node): the owner exports
// the CUDA IPC handle of the allocation that holds `ptr` and the offset of `ptr` inside it, the
// others open it.  Peer access from the current device is enabled by the open.
int sage_peer_export(const void* ptr, unsigned char handle[64], int64_t* offset) {
  SAGE_REQUIRE(ptr != nullptr && handle != nullptr && offset != nullptr, "sage_peer_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  // (taken from the driver at run time, like the tensor-map encoder: the library links the runtime only)
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range_fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      range_fn = reinterpret_cast<RangeFn>(sym);
    }
  });
  if (range_fn == nullptr) return fail(SAGE_ERR_CUDA, "cuMemGetAddressRange is not available from the driver");
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult cr = range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  SAGE_REQUIRE(cr == CUDA_SUCCESS, "sage_peer_export: not a device allocation (driver error %d)", static_cast<int>(cr));
  cudaIpcMemHandle_t h;
  SAGE_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle, &h, 64);
  *offset = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return SAGE_OK;
}

int sage_peer_open(const unsigned char handle[64], int64_t offset, void** mapped) {
  SAGE_REQUIRE(handle != nullptr && mapped != nullptr && offset >= 0, "sage_peer_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* base = nullptr;
  SAGE_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *mapped = static_cast<unsigned char*>(base) + offset;
  return SAGE_OK;
}

int sage_peer_close(void* mapped, int64_t offset) {
  SAGE_REQUIRE(mapped != nullptr && offset >= 0, "sage_peer_close: bad argument");
  SAGE_CUDA(cudaIpcCloseMemHandle(static_cast<unsigned char*>(mapped) - offset));
  return SAGE_OK;
}

namespace {
int attn_int8_impl(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o, int64_t o_stride_b,
                   int64_t o_stride_h, int64_t o_stride_s, const float* q_scale, const float* k_scale, int out_dtype,
                   int B, int Hq, int Hkv, int Sq, int Skv, int D, int is_causal, float* lse, int32_t* s_dump,
                   int* status, void* workspace, int64_t workspace_bytes, int n_peers, void* const* peer_o, void* stream) {
  SAGE_REQUIRE(q_i8 && v16 && o && q_scale, "sage_qk_int8_sv_f16_attn: null pointer");
  SAGE_REQUIRE(Skv == 0 || (k_i8 && v16->ptr && k_scale), "sage_qk_int8_sv_f16_attn: null pointer");
  SAGE_REQUIRE(out_dtype == SAGE_DTYPE_F16 || out_dtype == SAGE_DTYPE_BF16,
               "sage_qk_int8_sv_f16_attn: out_dtype must be f16 or bf16");
  SAGE_REQUIRE(D == 64 || D == 128, "sage_qk_int8_sv_f16_attn: head_dim must be 64 or 128, got %d", D);
  SAGE_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Sq >= 0 && Skv >= 0, "sage_qk_int8_sv_f16_attn: bad sizes");
  SAGE_REQUIRE(Hq % Hkv == 0, "sage_qk_int8_sv_f16_attn: Hq (%d) must be a multiple of Hkv (%d)", Hq, Hkv);
  SAGE_REQUIRE(aligned16(q_i8) && aligned16(k_i8), "sage_qk_int8_sv_f16_attn: int8 inputs must be 16-byte aligned");
  SAGE_REQUIRE(aligned16(v16->ptr) && strides_ok(v16),
               "sage_qk_int8_sv_f16_attn: v needs a 16-byte aligned base and strides % 8 == 0");
  SAGE_REQUIRE(aligned16(o) && o_stride_b % 8 == 0 && o_stride_h % 8 == 0 && o_stride_s % 8 == 0,
               "sage_qk_int8_sv_f16_attn: o needs a 16-byte aligned base and strides % 8 == 0");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (Sq == 0) return SAGE_OK;

  sage::AttnParams p;
  fill_attn_params(&p, o, o_stride_b, o_stride_h, o_stride_s, out_dtype, B, Hq, Hkv, Sq, Skv, lse, status);
  p.q_scale = q_scale; p.k_scale = k_scale;
  p.s_dump = s_dump;
  p.n_peers = n_peers;                                  // (the persistent launch does not scatter: plain launch)
  for (int i = 0; i < n_peers; ++i) p.peer_o[i] = peer_o[i];
  if (n_peers > 0 && is_causal) {
    // Order of the causal items.  Output tiles exist only when items end; heaviest-first (the best
    // balance) ends none of them in the first third of the launch, so the links idle and the stores
    // then outlast the computation.  When the transfer is somewhat the longer of the two, start with
    // the lightest items instead: tiles flow from the first microseconds on (8 GPUs, B=2 H=32
    // S=8192: 0.253 instead of 0.287 ms per step).  When it is longer by far the links are the
    // bound in either order and heaviest-first measured slightly better.  Estimates with the
    // measured constants of this kernel (7 us per item + 1.9 us per KV tile at head_dim 128, two
    // CTAs per SM) and 660 GB/s of peer stores per GPU.
    int sms = 0;
    if (sm_count(&sms) == SAGE_OK && sms > 0) {
      const double items = static_cast<double>(B) * Hq * p.n_q_tiles;
      const double nkv = (Skv + sage::kBlockN - 1) / sage::kBlockN;
      double tiles_per_head = 0.0;
      for (int qt = 0; qt < p.n_q_tiles; ++qt) tiles_per_head += std::min<double>(qt + 1, nkv);
      const double per_tile_us = (D == 128) ? 1.9 : 1.3;
      const double heaviest = 7.0 + per_tile_us * std::min<double>(p.n_q_tiles, nkv);
      const double compute_us =
          std::max(heaviest, (static_cast<double>(B) * Hq * tiles_per_head * per_tile_us + items * 7.0) / (2.0 * sms));
      const double transfer_us = items * sage::kBlockM * D * 2.0 * n_peers / 660e3;
      p.light_first = (transfer_us > 1.15 * compute_us && transfer_us < 2.0 * compute_us) ? 1 : 0;
    }
  }

  // With no keys every row has l == 0 and the output is 0 (csrc/attn_gfx11.cu:771).  The kernel
  // handles that without touching K or V, but a tensor map cannot have a zero extent: describe one
  // dummy row instead (it is never loaded).
  const int skv_map = Skv > 0 ? Skv : 1;
  const void* k_base = Skv > 0 ? static_cast<const void*>(k_i8) : static_cast<const void*>(q_i8);
  const void* v_base = Skv > 0 ? v16->ptr : static_cast<const void*>(q_i8);

  CUtensorMap tq, tk, tv, to;
  const CUtensorMapSwizzle swz_qk = (D == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)Sq, (cuuint64_t)B * Hq};
    cuuint64_t strides[2] = {(cuuint64_t)D, (cuuint64_t)Sq * D};
    cuuint32_t box[3] = {(cuuint32_t)D, (cuuint32_t)sage::kBlockM, 1};
    int rc = encode_map(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, q_i8, dims, strides, box, swz_qk, "q_i8");
    if (rc) return rc;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)skv_map, (cuuint64_t)B * Hkv};
    cuuint64_t strides[2] = {(cuuint64_t)D, (cuuint64_t)skv_map * D};
    cuuint32_t box[3] = {(cuuint32_t)D, (cuuint32_t)sage::kBlockN, 1};
    int rc = encode_map(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, k_base, dims, strides, box, swz_qk, "k_i8");
    if (rc) return rc;
  }
  {
    int rc = encode_strided_16bit(&tv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, v_base, D, skv_map, Hkv, B, v16->stride_s,
                                  v16->stride_h, v16->stride_b, sage::kBlockN, "v16");
    if (rc) return rc;
    // O in the caller's layout; the kernel stores boxes of 32 rows x 64 columns.
    rc = encode_strided_16bit(&to, p.out_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, o,
                              D, Sq, Hq, B, o_stride_s, o_stride_h, o_stride_b, 32, "o");
    if (rc) return rc;
  }
  const bool dump = (s_dump != nullptr);
  if (workspace != nullptr && !dump && n_peers == 0) {
    StreamKPlan plan;
    int rc = plan_streamk(&plan, B, Hq, Sq, Skv, D, is_causal);
    if (rc) return rc;
    if (plan.use && static_cast<size_t>(workspace_bytes) >= plan.workspace_bytes) {
      SAGE_REQUIRE(aligned16(workspace), "sage_qk_int8_sv_f16_attn_ws: workspace must be 16-byte aligned");
      if (D == 128) {
        return is_causal ? launch_attn_streamk<128, true, false>(tq, tk, tv, to, p, plan, workspace, st)
                         : launch_attn_streamk<128, false, false>(tq, tk, tv, to, p, plan, workspace, st);
      }
      return is_causal ? launch_attn_streamk<64, true, false>(tq, tk, tv, to, p, plan, workspace, st)
                       : launch_attn_streamk<64, false, false>(tq, tk, tv, to, p, plan, workspace, st);
    }
  }
#define SAGE_LAUNCH(DD, CC)                                                     \
  (dump ? launch_attn<DD, CC, true>(tq, tk, tv, to, p, st) : launch_attn<DD, CC, false>(tq, tk, tv, to, p, st))
  if (D == 128) return is_causal ? SAGE_LAUNCH(128, true) : SAGE_LAUNCH(128, false);
  return is_causal ? SAGE_LAUNCH(64, true) : SAGE_LAUNCH(64, false);
#undef SAGE_LAUNCH
}
}  // namespace

int sage_fold_attn_partial(const sage_strided_t* o_acc, float* lse_acc, int64_t lse_stride_b, int64_t lse_stride_h,
                           const sage_strided_t* o_part, int part_dtype, const float* lse_part, int B, int H, int S, int D,
                           int first, void* stream) {
  SAGE_REQUIRE(o_acc && o_acc->ptr && lse_acc && o_part && o_part->ptr && lse_part, "sage_fold_attn_partial: null pointer");
  SAGE_REQUIRE(part_dtype == SAGE_DTYPE_F16 || part_dtype == SAGE_DTYPE_BF16, "sage_fold_attn_partial: the partial must be f16 or bf16");
  SAGE_REQUIRE(D == 64 || D == 128, "sage_fold_attn_partial: head_dim must be 64 or 128, got %d", D);
  SAGE_REQUIRE(B >= 0 && H >= 0 && S >= 0, "sage_fold_attn_partial: bad sizes");
  SAGE_REQUIRE((reinterpret_cast<uintptr_t>(o_acc->ptr) & 31u) == 0 && o_acc->stride_b % 8 == 0 && o_acc->stride_h % 8 == 0 &&
                   o_acc->stride_s % 8 == 0,
               "sage_fold_attn_partial: the fp32 accumulator needs a 32-byte aligned base and strides % 8 == 0");
  SAGE_REQUIRE(aligned16(o_part->ptr) && strides_ok(o_part),
               "sage_fold_attn_partial: the partial needs a 16-byte aligned base and strides % 8 == 0");
  const long long n_vec = static_cast<long long>(B) * H * S * (D / 8);
  if (n_vec == 0) return SAGE_OK;
  sage::FoldParams p;
  p.o_acc = const_cast<float*>(static_cast<const float*>(o_acc->ptr));
  p.acc_stride_b = o_acc->stride_b; p.acc_stride_h = o_acc->stride_h; p.acc_stride_s = o_acc->stride_s;
  p.lse_acc = lse_acc; p.lse_acc_stride_b = lse_stride_b; p.lse_acc_stride_h = lse_stride_h;
  p.o_part = o_part->ptr;
  p.part_stride_b = o_part->stride_b; p.part_stride_h = o_part->stride_h; p.part_stride_s = o_part->stride_s;
  p.lse_part = lse_part;
  p.B = B; p.H = H; p.S = S; p.D = D;
  p.part_bf16 = (part_dtype == SAGE_DTYPE_BF16);
  p.first = first ? 1 : 0;
  const long long blocks = (n_vec + sage::kFoldThreads - 1) / sage::kFoldThreads;
  SAGE_REQUIRE(blocks <= 0x7fffffffLL, "sage_fold_attn_partial: too many blocks for one launch (%lld)", blocks);
  sage::sage_fold_partial_kernel<<<static_cast<unsigned>(blocks), sage::kFoldThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  SAGE_CUDA(cudaGetLastError());
  return SAGE_OK;
}

int sage_direct_attn(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v16, void* o,
                     int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int dtype, int B, int Hq, int Hkv,
                     int Sq, int Skv, int D, int is_causal, float sm_scale, float* lse, int* status, void* stream) {
  return sage_direct_attn_ws(q, k, v16, o, o_stride_b, o_stride_h, o_stride_s, dtype, B, Hq, Hkv, Sq, Skv, D, is_causal,
                             sm_scale, lse, status, nullptr, 0, stream);
}

namespace {
int check_peers(const char* who, int n_peers, void* const* peer_o, const void* o) {
  SAGE_REQUIRE(n_peers >= 0 && n_peers <= sage::kMaxPeers, "%s: n_peers must be 0..%d, got %d", who, sage::kMaxPeers, n_peers);
  SAGE_REQUIRE(n_peers == 0 || peer_o != nullptr, "%s: null peer list", who);
  for (int i = 0; i < n_peers; ++i) {
    SAGE_REQUIRE(peer_o[i] != nullptr && aligned16(peer_o[i]) && peer_o[i] != o,
                 "%s: peer buffer %d must be a 16-byte aligned address other than o", who, i);
  }
  return SAGE_OK;
}
int direct_attn_impl(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v16, void* o,
                     int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int dtype, int B, int Hq, int Hkv,
                     int Sq, int Skv, int D, int is_causal, float sm_scale, float* lse, int* status, void* workspace,
                     int64_t workspace_bytes, int n_peers, void* const* peer_o, void* stream);
}  // namespace

int sage_direct_attn_ws(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v16, void* o,
                        int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int dtype, int B, int Hq, int Hkv,
                        int Sq, int Skv, int D, int is_causal, float sm_scale, float* lse, int* status,
                        void* workspace, int64_t workspace_bytes, void* stream) {
  return direct_attn_impl(q, k, v16, o, o_stride_b, o_stride_h, o_stride_s, dtype, B, Hq, Hkv, Sq, Skv, D, is_causal,
                          sm_scale, lse, status, workspace, workspace_bytes, 0, nullptr, stream);
}

int sage_direct_attn_scatter(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v16, void* o,
                             int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int dtype, int B, int Hq,
                             int Hkv, int Sq, int Skv, int D, int is_causal, float sm_scale, float* lse, int* status,
                             int n_peers, void* const* peer_o, void* stream) {
  const int rc = check_peers("sage_direct_attn_scatter", n_peers, peer_o, o);
  if (rc) return rc;
  return direct_attn_impl(q, k, v16, o, o_stride_b, o_stride_h, o_stride_s, dtype, B, Hq, Hkv, Sq, Skv, D, is_causal,
                          sm_scale, lse, status, nullptr, 0, n_peers, peer_o, stream);
}

namespace {
int direct_attn_impl(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v16, void* o,
                     int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int dtype, int B, int Hq, int Hkv,
                     int Sq, int Skv, int D, int is_causal, float sm_scale, float* lse, int* status, void* workspace,
                     int64_t workspace_bytes, int n_peers, void* const* peer_o, void* stream) {
  SAGE_REQUIRE(q && q->ptr && v16 && o, "sage_direct_attn: null pointer");
  SAGE_REQUIRE(Skv == 0 || (k && k->ptr && v16->ptr), "sage_direct_attn: null pointer");
  SAGE_REQUIRE(dtype == SAGE_DTYPE_F16 || dtype == SAGE_DTYPE_BF16, "sage_direct_attn: dtype must be f16 or bf16");
  SAGE_REQUIRE(D == 64 || D == 128, "sage_direct_attn: head_dim must be 64 or 128, got %d", D);
  SAGE_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Sq >= 0 && Skv >= 0, "sage_direct_attn: bad sizes");
  SAGE_REQUIRE(Hq % Hkv == 0, "sage_direct_attn: Hq (%d) must be a multiple of Hkv (%d)", Hq, Hkv);
  SAGE_REQUIRE(aligned16(q->ptr) && strides_ok(q), "sage_direct_attn: q needs a 16-byte aligned base and strides % 8 == 0");
  SAGE_REQUIRE(Skv == 0 || (aligned16(k->ptr) && strides_ok(k) && aligned16(v16->ptr) && strides_ok(v16)),
               "sage_direct_attn: k / v need 16-byte aligned bases and strides % 8 == 0");
  SAGE_REQUIRE(aligned16(o) && o_stride_b % 8 == 0 && o_stride_h % 8 == 0 && o_stride_s % 8 == 0,
               "sage_direct_attn: o needs a 16-byte aligned base and strides % 8 == 0");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (Sq == 0) return SAGE_OK;

  sage::AttnParams p;
  fill_attn_params(&p, o, o_stride_b, o_stride_h, o_stride_s, dtype, B, Hq, Hkv, Sq, Skv, lse, status);
  p.qk_bf16 = (dtype == SAGE_DTYPE_BF16);
  p.score_scale = sm_scale * 1.4426950408889634f;       // csrc/attn_gfx11.cu:34, as for the quantised path
  p.n_peers = n_peers;                                  // (short sequences: the order of the items is left alone)
  for (int i = 0; i < n_peers; ++i) p.peer_o[i] = peer_o[i];

  // No keys: nothing is loaded (see sage_qk_int8_sv_f16_attn_lse); the maps describe one dummy row.
  const int skv_map = Skv > 0 ? Skv : 1;
  const void* k_base = Skv > 0 ? k->ptr : q->ptr;
  const void* v_base = Skv > 0 ? v16->ptr : q->ptr;
  const sage_strided_t kk = Skv > 0 ? *k : sage_strided_t{q->ptr, 0, 0, (int64_t)D};
  const sage_strided_t vv = Skv > 0 ? *v16 : sage_strided_t{q->ptr, 0, 0, (int64_t)D};
  const CUtensorMapDataType qk_dt = p.qk_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;

  CUtensorMap tq, tk, tv, to;
  int rc = encode_strided_16bit(&tq, qk_dt, q->ptr, D, Sq, Hq, B, q->stride_s, q->stride_h, q->stride_b, sage::kBlockM, "q");
  if (rc) return rc;
  rc = encode_strided_16bit(&tk, qk_dt, k_base, D, skv_map, Hkv, B, kk.stride_s, kk.stride_h, kk.stride_b, sage::kBlockN, "k");
  if (rc) return rc;
  rc = encode_strided_16bit(&tv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, v_base, D, skv_map, Hkv, B, vv.stride_s, vv.stride_h,
                            vv.stride_b, sage::kBlockN, "v16");
  if (rc) return rc;
  rc = encode_strided_16bit(&to, qk_dt, o, D, Sq, Hq, B, o_stride_s, o_stride_h, o_stride_b, 32, "o");
  if (rc) return rc;
  if (workspace != nullptr && n_peers == 0) {
    StreamKPlan plan;
    rc = plan_streamk(&plan, B, Hq, Sq, Skv, D, is_causal);
    if (rc) return rc;
    if (plan.use && static_cast<size_t>(workspace_bytes) >= plan.workspace_bytes) {
      SAGE_REQUIRE(aligned16(workspace), "sage_direct_attn_ws: workspace must be 16-byte aligned");
      if (D == 128) {
        return is_causal ? launch_attn_streamk<128, true, true>(tq, tk, tv, to, p, plan, workspace, st)
                         : launch_attn_streamk<128, false, true>(tq, tk, tv, to, p, plan, workspace, st);
      }
      return is_causal ? launch_attn_streamk<64, true, true>(tq, tk, tv, to, p, plan, workspace, st)
                       : launch_attn_streamk<64, false, true>(tq, tk, tv, to, p, plan, workspace, st);
    }
  }
  if (D == 128) {
    // A grid that cannot put two CTAs on every SM anyway takes the deeper K/V rings (one CTA per SM).
    int sms = 0;
    rc = sm_count(&sms);
    if (rc) return rc;
    const long long ctas = static_cast<long long>(p.n_q_tiles) * B * Hq;
    if (ctas <= sms) {
      return is_causal ? launch_attn<128, true, false, true, 2>(tq, tk, tv, to, p, st)
                       : launch_attn<128, false, false, true, 2>(tq, tk, tv, to, p, st);
    }
    return is_causal ? launch_attn<128, true, false, true>(tq, tk, tv, to, p, st)
                     : launch_attn<128, false, false, true>(tq, tk, tv, to, p, st);
  }
  return is_causal ? launch_attn<64, true, false, true>(tq, tk, tv, to, p, st)
                   : launch_attn<64, false, false, true>(tq, tk, tv, to, p, st);
}
}  // namespace

}  // extern "C"
