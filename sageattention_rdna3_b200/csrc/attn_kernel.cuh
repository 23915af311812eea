// Fused attention for sm_100a: replaces attn_kernel_impl_t / attn_kernel_impl_32_t, the un-quantised
// direct_attn_kernel_impl_t and the WMMA helpers of the reference (csrc/attn_gfx11.cu:409-1243,
// :1468-1846, csrc/mma_gfx11.h).
//
// A CTA works on 128-row query tiles of one (batch, query head) and streams the KV sequence in
// 128-row tiles:
//   warp 4   : TMA producer   - Q, then K (int8, or fp16 / bf16 in the un-quantised variant) and
//                               V (fp16) tiles into a shared-memory ring
//   warp 5   : MMA issuer     - S = Q.K^T  (tcgen05.mma kind::i8, int32 accumulator in TMEM; kind::f16
//                               with an fp32 accumulator in the un-quantised variant),
//                               O += P.V   (tcgen05.mma kind::f16, P read from TMEM, fp32 accumulator)
//   warps 0-3: softmax        - thread t owns query row t: tcgen05.ld of S, dequantise with
//                               q_scale[row/32]*k_scale[col/16] (or scale by sm_scale*log2e), causal /
//                               length mask, base-2 online softmax in fp32, P rounded to fp16 and
//                               written back into TMEM over S, lazy rescale of O, final
//                               normalisation and store (optionally the log-sum-exp).
// Two CTAs fit on one SM (112 KB of shared memory and 256 TMEM columns each), so the tensor pipe of
// one overlaps the softmax of the other.
// Launch shapes: one CTA per query tile (plain), or 2 * SMs persistent CTAs that each work through an
// equal span of KV-tile steps and leave partial results for sage_attn_merge_kernel (STREAMK).
//
// TMEM columns: [0,128) S as int32 / fp32, reused in place as P (fp16 pairs in columns [0,64));
//               [128,128+D) O as fp32.
// Numerics follow csrc/attn_gfx11.cu:487-502,608-689,769-786: exact int32 scores, fp32 softmax in
// base 2 with the row sum taken before P is rounded, P in fp16, V in fp16, fp32 accumulation, one
// rounding of acc/l to the output type.  The running maximum is only moved when it grows by more
// than 2^14 ("lazy rescale"); acc and l use the same maximum, so acc/l is unchanged by that.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cfloat>
#include <cstdint>
#include <type_traits>

#include "ptx_sm100.cuh"

namespace sage {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kAttnThreads = 192;
constexpr int kTmemCols = 256;
constexpr int kColS = 0;
constexpr int kColP = 0;
constexpr int kColO = 128;
constexpr float kMaskValue = -FLT_MAX * 0.5f;       // csrc/attn_gfx11.cu:499,628-631
// Lazy rescale: the running maximum moves only when it grew by more than 2^14.  P = exp2(s - m) then
// stays below 2^14 = 16384, a quarter of the largest fp16, and the accumulators are fp32.  (2^8
// measured the same on N(0,1) inputs and 16 % slower on 4x sharper scores.)
#ifndef SAGE_LAZY_LOG2
#define SAGE_LAZY_LOG2 14
#endif
constexpr float kLazyRescaleLog2 = static_cast<float>(SAGE_LAZY_LOG2);
constexpr float kOptimisticSumMax = static_cast<float>(1 << SAGE_LAZY_LOG2);   // 64 values: each is below it
constexpr float kRefusedBarLog2 = static_cast<float>(SAGE_LAZY_LOG2) - 6.5f;   // sum > 2^T -> max > 2^(T-6)

// Device status codes written to AttnParams::status (0 = ok).
enum AttnStatus : int {
  kStatusOk = 0,
  kStatusSmemMisaligned = 1,
  kStatusWaitTimeout = 2,       // + 16 * (id of the barrier the wait gave up on)
};

constexpr int kMaxPeers = 15;
struct AttnParams {
  const float* q_scale;         // [B,Hq,q_groups]
  const float* k_scale;         // [B,Hkv,k_groups]
  void* o;                      // caller layout; fp16 or bf16
  long long o_stride_b, o_stride_h, o_stride_s;   // elements
  int B, Hq, Hkv, Sq, Skv;
  int q_groups, k_groups;
  int n_q_tiles;
  int head_group;               // (batch, head) pairs scheduled together (a multiple of Hq/Hkv)
  int out_bf16;
  int qk_bf16;                  // un-quantised variant only: Q and K are bf16 (else fp16)
  float score_scale;            // un-quantised variant only: sm_scale * log2(e)
  int32_t* s_dump;              // optional [B,Hq,Sq,Skv] int32 copy of Q.K^T (debug / parity)
  float* lse;                   // optional [B,Hq,Sq]: natural-log sum of exp of the scaled scores
  int* status;                  // optional device word, stays 0 on success
  int* status_host;             // optional word in mapped pinned host memory that receives the same code
  long long wait_limit_cycles;  // bound of every barrier wait, in SM clocks
  int test_drop_v_load;         // test hook: the producer never loads V of the first KV tile
  // Persistent ("stream-K") variant only: the (query tile, KV tile) steps of the whole problem are
  // laid out in one line, item after item, and cut into gridDim.x equal spans.
  long long sk_total_tiles;     // KV-tile steps of the whole problem
  int sk_tiles_per_head;        // ... of one (batch, query head)
  int sk_nkv_full;              // ceil(Skv / 128)
  float* part_o;                // [gridDim.x][2][128][D] fp32: acc / l of a span that covers part of an item
  float* part_lse;              // [gridDim.x][2][128] fp32: m + log2 l of the same (base 2)
  // Output scatter (plain launch only): every finished tile is also written, with ordinary 16-byte
  // stores, to `n_peers` more buffers that have the layout and strides of `o` - the same slice of the
  // gathered output in the memory of the other GPUs of the node.
  int n_peers;
  void* peer_o[kMaxPeers];
  // Causal, plain launch: 0 = the heaviest (last) query tiles of a head group start first (best
  // balance), 1 = the lightest first, so that finished tiles - and with them the peer stores - start
  // flowing early in the launch; the launcher picks 1 when the transfer outlasts the computation.
  int light_first;
};

// QKB = bytes per element of Q and K in shared memory: 1 (int8) or 2 (fp16 / bf16, the
// un-quantised variant).
// KST = depth of the K and V rings, 0 for the default.  16-bit Q/K with head_dim 128 has two
// shapes: one K and one V tile (32 KB each) next to Q (32 KB) keep two CTAs on an SM - the
// half-tile order of the tensor pipe still leaves each refill about one softmax half-step of lead
// time - and two tiles each (160 KB, one CTA per SM) for grids that do not fill the SMs twice.
template <int D, int QKB = 1, int KST = 0>
struct AttnSmem {
  static constexpr int kStages = KST > 0 ? KST : (QKB == 2) ? (D == 128 ? 1 : 2) : (D == 128 ? 2 : 4);
  static constexpr int kQBytes = kBlockM * D * QKB;
  static constexpr int kKBytes = kBlockN * D * QKB;
  static constexpr int kVBytes = kBlockN * D * 2;        // fp16
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + kQBytes;
  static constexpr int kOffV = kOffK + kStages * kKBytes;
  static constexpr int kOffBar = kOffV + kStages * kVBytes;
  // barriers: q_full, o_final, s_full[2], p_full[2], pv_done[2], q_empty, o_free, epi_done (the
  // last three only cycle in the persistent variant), then per stage k_full[], v_full[], k_empty[],
  // v_empty[]
  static constexpr int kNumBars = 11 + 4 * kStages;
  static constexpr int kOffMisc = kOffBar + 8 * kNumBars;   // tmem base (u32), abort flag, fail code
  static constexpr int kTotal = kOffMisc + 16;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));   // first source -> upper half
  return r;
}
__device__ __forceinline__ uint32_t pack_bf162(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
constexpr int kHalfN = kBlockN / 2;      // the softmax works on 64-column halves of a KV tile

// Two CTAs share an SM, and warp w of one shares a scheduler - and its exponential unit - with warp
// w of the other.  Left alone, the two settle into a fixed relative phase, often one in which their
// exponential passes coincide and both run at half speed.  Every second CTA to start on an SM
// therefore yields (nanosleep 0) once per half-step: its period becomes a little longer, the relative
// phase drifts through all values, and the pair sees the average overlap instead of the worst
// (2-2.5 % on long sequences).  The counter is only ever read for its parity; it is never reset.
#ifndef SAGE_DEPHASE
#define SAGE_DEPHASE 1
#endif
static __device__ unsigned g_sm_arrivals[1024];

// What one pass of the pipeline works on: KV tiles [kv_lo, kv_lo + n_kv) of one 128-row query tile
// of one (batch, query head).  slot < 0: the pass covers every KV tile of the item and writes the
// output; slot 0 / 1: it covers a part, and acc / l and m + log2 l go to that slot of the CTA's
// partial buffers, to be merged by sage_attn_merge_kernel.
struct Segment {
  int bh, b, hq, hkv, q_base, kv_lo, n_kv, slot;
};

// STREAMK = false: one CTA = one whole item.  (batch, head) pairs are taken `head_group` at a time;
// within a group the heaviest (last) query tiles go first and neighbouring CTAs are neighbouring
// heads.  The CTAs resident at any moment then read the K/V of a few heads only (they stay in L2),
// and the query heads of one KV head (GQA) run together.
// STREAMK = true: the KV-tile steps of all items, in (batch, head, query tile) order, form one line
// of sk_total_tiles steps; CTA c owns steps [c*T/G, (c+1)*T/G) and walks through the items they
// belong to: the tail of one item, whole items, the head of another.  All CTAs get the same amount
// of work whatever the number of items is.
template <bool CAUSAL, bool STREAMK>
struct SegIter {
  const AttnParams& p;
  long long t, t_end;
  bool first;
  __device__ __forceinline__ explicit SegIter(const AttnParams& pp) : p(pp), first(true) {
    if constexpr (STREAMK) {
      t = (p.sk_total_tiles * blockIdx.x) / gridDim.x;
      t_end = (p.sk_total_tiles * (blockIdx.x + 1)) / gridDim.x;
    } else {
      t = 0;
      t_end = 1;
    }
  }
  __device__ __forceinline__ void fill(Segment& s, int bh, int qt) const {
    s.bh = bh;
    s.b = bh / p.Hq;
    s.hq = bh % p.Hq;
    s.hkv = s.hq / (p.Hq / p.Hkv);                                     // csrc/attn_gfx11.cu:464
    s.q_base = qt * kBlockM;
  }
  // Tiles of query tile qt: csrc/attn_gfx11.cu:502 (kBlockM == kBlockN)
  __device__ __forceinline__ int item_tiles(int qt) const {
    return CAUSAL ? min(qt + 1, p.sk_nkv_full) : p.sk_nkv_full;
  }
  __device__ __forceinline__ bool next(Segment& s) {
    if constexpr (!STREAMK) {
      if (!first) return false;
      first = false;
      const int n_bh = p.B * p.Hq;
      const int per_group = p.n_q_tiles * p.head_group;
      const int group = blockIdx.x / per_group;
      const int g_first = group * p.head_group;
      const int g_size = min(p.head_group, n_bh - g_first);
      const int within = blockIdx.x - group * per_group;
      const int qt = p.light_first ? within / g_size : p.n_q_tiles - 1 - within / g_size;
      fill(s, g_first + within % g_size, qt);
      const int kv_limit = CAUSAL ? min(s.q_base + kBlockM, p.Skv) : p.Skv;   // csrc/attn_gfx11.cu:502
      s.kv_lo = 0;
      s.n_kv = (kv_limit + kBlockN - 1) / kBlockN;
      s.slot = -1;
      return true;
    } else {
      if (t >= t_end) return false;
      const int bh = static_cast<int>(t / p.sk_tiles_per_head);
      const int r = static_cast<int>(t - static_cast<long long>(bh) * p.sk_tiles_per_head);
      int qt, off;
      if (!CAUSAL) {
        qt = r / p.sk_nkv_full;
        off = r - qt * p.sk_nkv_full;
      } else {
        // tiles before query tile qt: qt(qt+1)/2 while qt <= NKV, then NKV more per query tile
        const int nkv = p.sk_nkv_full;
        const int tri = nkv * (nkv + 1) / 2;
        if (r < tri) {
          qt = static_cast<int>((sqrtf(8.0f * static_cast<float>(r) + 1.0f) - 1.0f) * 0.5f);
          while (qt * (qt + 1) / 2 > r) --qt;
          while ((qt + 1) * (qt + 2) / 2 <= r) ++qt;
          off = r - qt * (qt + 1) / 2;
        } else {
          qt = nkv + (r - tri) / nkv;
          off = (r - tri) - (qt - nkv) * nkv;
        }
      }
      fill(s, bh, qt);
      const int tiles = item_tiles(qt);
      const long long left = t_end - t;
      s.kv_lo = off;
      s.n_kv = static_cast<int>(min(static_cast<long long>(tiles - off), left));
      s.slot = (off == 0 && s.n_kv == tiles) ? -1 : (first ? 0 : 1);
      first = false;
      t += s.n_kv;
      return true;
    }
  }
};

// QKF = false: Q and K are the int8 tensors of the quantised path (scores = int32 products times
// q_scale*k_scale).  QKF = true: Q and K are the caller's fp16 / bf16 tensors, the scores are fp32
// products times sm_scale*log2(e) - the reference's un-quantised kernels for short sequences
// (direct_attn_kernel_impl_t, csrc/attn_gfx11.cu:1468-1846) on the same pipeline.
// STREAMK = true: persistent CTAs, each working through an equal span of KV-tile steps (SegIter);
// TMEM, barriers and the K/V ring are set up once per CTA, barrier phases keep counting across
// segments (kt = KV tiles so far, it = segments so far), and the loads and first Q.K^T of the next
// segment overlap the epilogue of the previous one.
template <int D, bool CAUSAL, bool DUMP, bool QKF = false, int KST = 0, bool STREAMK = false>
__global__ void __launch_bounds__(kAttnThreads, 2)
sage_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                 const AttnParams p) {
  using L = AttnSmem<D, QKF ? 2 : 1, KST>;
  constexpr int kStages = L::kStages;
  static_assert(!(QKF && DUMP), "the int32 score dump belongs to the quantised variant");
  extern __shared__ __align__(1024) uint8_t smem[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if ((smem_u32(smem) & 1023u) != 0u) {        // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kStatusSmemMisaligned);
    return;
  }

  uint8_t* s_q = smem + L::kOffQ;
  uint8_t* s_k = smem + L::kOffK;
  uint8_t* s_v = smem + L::kOffV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars + 0;
  uint64_t* o_final = bars + 1;
  uint64_t* s_full = bars + 2;      // [2] one per half: S_h holds Q.K_h^T
  uint64_t* p_full = bars + 4;      // [2] P_h written (and O rescaled) by all 128 softmax threads
  uint64_t* pv_done = bars + 6;     // [2] O += P_h.V_h has completed
  uint64_t* q_empty = bars + 8;     // every Q.K^T of the segment is complete: Q may be overwritten
  uint64_t* o_free = bars + 9;      // all 128 softmax threads hold the segment's O in registers
  uint64_t* epi_done = bars + 10;   // the 4 softmax warps are done with the output staging area (V stage 0)
  uint64_t* k_full = bars + 11;
  uint64_t* v_full = bars + 11 + kStages;
  uint64_t* k_empty = bars + 11 + 2 * kStages;
  uint64_t* v_empty = bars + 11 + 3 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 4);
  int* fail_code = reinterpret_cast<int*>(smem + L::kOffMisc + 8);

  if (threadIdx.x == 0) {
    // A status word that is already set means an earlier CTA of this launch (or an earlier launch
    // the caller has not looked at yet) gave up: this CTA leaves through the abort path at once, so a
    // failing launch costs about one wait bound and not one per wave of CTAs.
    *abort_flag = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    *fail_code = 0;
  }
  // TMA loads of the producer thread.  int8 Q / K are contiguous [B*H, S, D] (3-D maps); 16-bit Q / K
  // come in the caller's layout, one [128 rows][64 columns] box per 64 columns of head_dim.
  auto load_q = [&](const Segment& g) {
    if constexpr (QKF) {
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_4d(s_q + c * (kBlockM * 128), &tm_q, q_full, c * 64, g.q_base, g.hq, g.b);
    } else {
      tma_load_3d(s_q, &tm_q, q_full, 0, g.q_base, g.bh);
    }
  };
  auto load_k = [&](const Segment& g, int tile, int stage) {
    if constexpr (QKF) {
#pragma unroll
      for (int c = 0; c < D / 64; ++c)
        tma_load_4d(s_k + stage * L::kKBytes + c * (kBlockN * 128), &tm_k, k_full + stage, c * 64, tile * kBlockN, g.hkv,
                    g.b);
    } else {
      tma_load_3d(s_k + stage * L::kKBytes, &tm_k, k_full + stage, 0, tile * kBlockN, g.b * p.Hkv + g.hkv);
    }
  };
  if (warp == 4 && lane == 0) {
    // The producer thread sets the barriers up itself and starts the first loads (Q and K tile 0,
    // which wait for nothing) at once, so their latency overlaps the TMEM allocation and the
    // CTA-wide barrier below.
    mbar_init(q_full, 1);
    mbar_init(o_final, 1);
    mbar_init(q_empty, 1);
    mbar_init(o_free, 128);
    mbar_init(epi_done, 4);
    for (int h = 0; h < 2; ++h) {
      mbar_init(s_full + h, 1);
      mbar_init(p_full + h, 128);
      mbar_init(pv_done + h, 1);
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(v_full + s, 1);
      mbar_init(k_empty + s, 1);
      mbar_init(v_empty + s, 1);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o);
    SegIter<CAUSAL, STREAMK> first_iter(p);
    Segment g0;
    if (first_iter.next(g0) && g0.n_kv > 0) {
      mbar_arrive_expect_tx(q_full, L::kQBytes);
      load_q(g0);
      mbar_arrive_expect_tx(k_full, L::kKBytes);
      load_k(g0, g0.kv_lo, 0);
    }
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool dead_on_arrival = *abort_flag != 0;

// A failed wait records which barrier it was and leaves the role's loop.
#ifndef SAGE_HINT_TMA
#define SAGE_HINT_TMA true
#endif
#ifndef SAGE_HINT_MMA
#define SAGE_HINT_MMA true
#endif
#ifndef SAGE_HINT_SOFTMAX
#define SAGE_HINT_SOFTMAX true
#endif
#define SAGE_WAIT_ROLE_OR(hinted, bar_ptr, parity, bar_id, action)   \
  if (!mbar_wait<hinted>((bar_ptr), (parity), abort_flag, p.wait_limit_cycles)) { \
    atomicCAS(fail_code, 0, kStatusWaitTimeout + 16 * (bar_id));    \
    action;                                                         \
  }
#define SAGE_WAIT_OR(bar_ptr, parity, bar_id, action) SAGE_WAIT_ROLE_OR(kHintRole, bar_ptr, parity, bar_id, action)

  if (dead_on_arrival) {
    // nothing to do: the first loads of the producer land during the teardown wait
  } else if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    constexpr bool kHintRole = SAGE_HINT_TMA;
    // Per segment: Q, K(first tile), then for every tile K(j+1) before V(j): K is needed first.  Q and
    // K of the CTA's first segment are already on their way.
    if (lane == 0) {
      SegIter<CAUSAL, STREAMK> iter(p);
      Segment g;
      int kt = 0, it = 0;                 // KV tiles / segments so far (constant 0 unless STREAMK)
      bool ok = true;
#pragma unroll 1
      while (ok && iter.next(g)) {
        if (g.n_kv > 0) {
          if (STREAMK && it > 0) {
            SAGE_WAIT_OR(q_empty, (it - 1) & 1, 13, { ok = false; break; });
            mbar_arrive_expect_tx(q_full, L::kQBytes);
            load_q(g);
            const int s0 = kt % kStages;
            SAGE_WAIT_OR(k_empty + s0, ((kt / kStages) & 1) ^ 1u, 1, { ok = false; break; });
            mbar_arrive_expect_tx(k_full + s0, L::kKBytes);
            load_k(g, g.kv_lo, s0);
          }
          // V stage 0 doubles as the output staging area of the previous segment's epilogue: wait for
          // `epi_done` before the first refill of stage 0.  The wait is made in every segment (at its
          // end if no tile of the segment lands in stage 0): a parity wait can only tell the current
          // phase from the one before, so no phase of the barrier may go unobserved.
          bool epi_waited = !(STREAMK && it > 0);
#pragma unroll 1
          for (int j = 0; j < g.n_kv; ++j) {
            if (j + 1 < g.n_kv) {
              const int t1 = kt + j + 1;
              const int s1 = t1 % kStages;
              SAGE_WAIT_OR(k_empty + s1, ((t1 / kStages) & 1) ^ 1u, 1, { ok = false; break; });
              mbar_arrive_expect_tx(k_full + s1, L::kKBytes);
              load_k(g, g.kv_lo + j + 1, s1);
            }
            const int t = kt + j;
            const int sv = t % kStages;
            SAGE_WAIT_OR(v_empty + sv, ((t / kStages) & 1) ^ 1u, 2, { ok = false; break; });
            if (sv == 0 && !epi_waited) {
              SAGE_WAIT_OR(epi_done, (it - 1) & 1, 15, { ok = false; break; });
              epi_waited = true;
            }
            if (p.test_drop_v_load && t == 0) continue;   // failure-detection test: v_full never completes
            mbar_arrive_expect_tx(v_full + sv, L::kVBytes);
#pragma unroll
            for (int h = 0; h < D / 64; ++h) {
              tma_load_4d(s_v + sv * L::kVBytes + h * (kBlockN * 128), &tm_v, v_full + sv, h * 64,
                          (g.kv_lo + j) * kBlockN, g.hkv, g.b);
            }
          }
          if (ok && !epi_waited) SAGE_WAIT_OR(epi_done, (it - 1) & 1, 15, { ok = false; break; });
          if (STREAMK) {
            kt += g.n_kv;
            ++it;
          }
        }
        if (!STREAMK) break;
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr bool kHintRole = SAGE_HINT_MMA;
    // Program order of the tensor pipe: QK(0,0) QK(0,1) | PV(0,0) QK(1,0) PV(0,1) QK(1,1) | ...
    // so the scores of the next half are ready while the softmax warps work on the current one.
    if (lane == 0) {
      constexpr uint32_t kIdescQK = umma_idesc(2, 1, 1, 0, 0, kBlockM, kHalfN);   // s32 = s8 x s8
      constexpr uint32_t kIdescPV = umma_idesc(1, 0, 0, 0, 1, kBlockM, D);        // f32 = f16 x f16, V MN-major
      constexpr uint32_t kSwzQK = (D == 128) ? kSwizzle128B : kSwizzle64B;
      constexpr uint32_t kSboQK = 8 * D;               // 8 rows of D bytes
      constexpr uint32_t kHalfKBytes = kHalfN * D;     // 64 K rows
      const uint64_t desc_q = umma_smem_desc(smem_u32(s_q), 16, kSboQK, kSwzQK);
      const uint32_t t_o = tmem_base + kColO;
      bool ok = true;
      // un-quantised variant: f32 = f16 x f16 or bf16 x bf16, both operands K-major
      const uint32_t idesc_qk16 = umma_idesc(1, p.qk_bf16 ? 1u : 0u, p.qk_bf16 ? 1u : 0u, 0, 0, kBlockM, kHalfN);

      auto issue_qk = [&](int stage, int h) {
        if constexpr (QKF) {
          // Q and K tiles are D/64 slabs of [128 rows][64 elements = 128 bytes], 128-byte swizzle
          // (8 rows = 1024 bytes); an instruction takes 16 elements = 32 bytes of head_dim, half h of
          // K starts 64 rows = 8192 bytes into each slab.
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t slab = (k / 4) * (kBlockM * 128);
            const uint64_t dq = umma_smem_desc(smem_u32(s_q + slab), 16, 1024, kSwizzle128B) + 2 * (k % 4);
            const uint64_t dk =
                umma_smem_desc(smem_u32(s_k + stage * L::kKBytes + slab + h * (kHalfN * 128)), 16, 1024, kSwizzle128B) +
                2 * (k % 4);
            mma_f16_ss(tmem_base + kColS + h * kHalfN, dq, dk, idesc_qk16, k > 0 ? 1u : 0u);
          }
        } else {
          const uint64_t desc_k =
              umma_smem_desc(smem_u32(s_k + stage * L::kKBytes + h * kHalfKBytes), 16, kSboQK, kSwzQK);
#pragma unroll
          for (int k = 0; k < D / 32; ++k) {           // 32 int8 of head_dim per instruction
            mma_i8_ss(tmem_base + kColS + h * kHalfN, desc_q + 2 * k, desc_k + 2 * k, kIdescQK, k > 0 ? 1u : 0u);
          }
        }
        tc_commit(s_full + h);
      };

      SegIter<CAUSAL, STREAMK> iter(p);
      Segment g;
      int kt = 0, it = 0;                 // KV tiles / segments so far (constant 0 unless STREAMK)
#pragma unroll 1
      while (ok && iter.next(g)) {
        const int n_kv = g.n_kv;
        if (n_kv > 0) {
          SAGE_WAIT_OR(q_full, it & 1, 3, { ok = false; break; });
          {
            const int s0 = kt % kStages;
            SAGE_WAIT_OR(k_full + s0, (kt / kStages) & 1, 4, { ok = false; break; });
            tc_fence_after();
            issue_qk(s0, 0);
            issue_qk(s0, 1);
            tc_commit(k_empty + s0);                     // K(first) is consumed once QK(first,1) is done
            if (STREAMK && n_kv == 1) tc_commit(q_empty);  // ... and so is Q when this was the only tile
          }
#pragma unroll 1
          for (int j = 0; ok && j < n_kv; ++j) {
            const int t = kt + j;
            const int s = t % kStages;
            const uint32_t ph = (t / kStages) & 1;
            const int s1 = (t + 1) % kStages;
            const uint32_t ph1 = ((t + 1) / kStages) & 1;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              SAGE_WAIT_OR(p_full + h, t & 1, 5, { ok = false; break; });
              if (h == 0) SAGE_WAIT_OR(v_full + s, ph, 6, { ok = false; break; });
              // the first P.V of a segment overwrites O: the previous segment's O must have been read
              if (STREAMK && h == 0 && j == 0 && it > 0) SAGE_WAIT_OR(o_free, (it - 1) & 1, 14, { ok = false; break; });
              tc_fence_after();
              // V tile: [128 kv rows][64 fp16] blocks of 16 KB, one per 64 columns of head_dim;
              // half h starts 64 rows = 8192 bytes in, each instruction takes 16 rows = 2048 bytes.
              const uint64_t desc_v = umma_smem_desc(smem_u32(s_v + s * L::kVBytes + h * (kHalfN * 128)), kBlockN * 128,
                                                     1024, kSwizzle128B);
#pragma unroll
              for (int k = 0; k < kHalfN / 16; ++k) {
                mma_f16_ts(t_o, tmem_base + kColP + h * kHalfN + 8 * k, desc_v + 128 * k, kIdescPV,
                           (j > 0 || h > 0 || k > 0) ? 1u : 0u);
              }
              tc_commit(pv_done + h);
              if (h == 1) tc_commit(v_empty + s);
              if (j + 1 < n_kv) {
                if (h == 0) SAGE_WAIT_OR(k_full + s1, ph1, 7, { ok = false; break; });
                tc_fence_after();
                issue_qk(s1, h);
                if (h == 1) {
                  tc_commit(k_empty + s1);               // K(j+1) is consumed once QK(j+1,1) is done
                  if (STREAMK && j + 2 == n_kv) tc_commit(q_empty);   // that was the segment's last Q.K^T
                }
              }
            }
          }
          tc_commit(o_final);
          if (STREAMK) {
            kt += n_kv;
            ++it;
          }
        }
        if (!STREAMK) break;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    constexpr bool kHintRole = SAGE_HINT_SOFTMAX;
    bool yields = false;
    // (not in the persistent variant: its CTAs are given equal spans and must run at equal speed)
    if (SAGE_DEPHASE && !STREAMK) {
      volatile unsigned* arrival = reinterpret_cast<volatile unsigned*>(smem + L::kOffMisc + 12);
      if (threadIdx.x == 0) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        *arrival = atomicAdd(&g_sm_arrivals[smid & 1023u], 1u);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");      // the four softmax warps only
      yields = (*arrival & 1u) != 0u;
    }
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t t_o = tmem_base + lane_base + kColO;
    bool ok = true;
    int kt = 0, it = 0;                   // KV tiles / segments so far (constant 0 unless STREAMK)
    SegIter<CAUSAL, STREAMK> iter(p);
    Segment sg;
#pragma unroll 1
    while (ok && iter.next(sg)) {
    const int bh = sg.bh, b = sg.b, hq = sg.hq, hkv = sg.hkv, q_base = sg.q_base, n_kv = sg.n_kv;
    const int row = q_base + threadIdx.x;
    const int q_grp = (q_base + warp * 32) / 32;
    float qs = 0.0f;
    const float* ks_base = nullptr;
    if constexpr (!QKF) {
      qs = (q_grp < p.q_groups) ? __ldg(p.q_scale + static_cast<long long>(bh) * p.q_groups + q_grp) : 0.0f;
      ks_base = p.k_scale + static_cast<long long>(b * p.Hkv + hkv) * p.k_groups;
    }

    float m_used = kMaskValue;
    float l = 0.0f;
    int distrust = 0;                     // > 1: the optimistic attempt is skipped (see below)

    // k_scale of the next half is fetched one half ahead, off the critical path
    float ks_next[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int kg = sg.kv_lo * (kBlockN / 16) + g;
      ks_next[g] = (!QKF && kg < p.k_groups) ? __ldg(ks_base + kg) : 0.0f;
    }

    const int n_half = 2 * n_kv;
#pragma unroll 1
    for (int hh = 0; hh < n_half; ++hh) {
      const int t = kt + (hh >> 1);                     // KV tiles since the CTA started: barrier phases
      const int h = hh & 1;
      const int kv_base = (2 * sg.kv_lo + hh) * kHalfN;
      const uint32_t t_s = tmem_base + lane_base + kColS + h * kHalfN;

      float cg[4];                                      // q_scale * k_scale per 16 columns (:621)
#pragma unroll
      for (int g = 0; g < 4; ++g) cg[g] = QKF ? p.score_scale : __fmul_rn(qs, ks_next[g]);

      SAGE_WAIT_OR(s_full + h, t & 1, 8, { ok = false; break; });
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(t_s, sr[0]);
      tmem_ld32(t_s + 32, sr[1]);
      if constexpr (!QKF) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int kg = (kv_base + kHalfN) / 16 + g;
          ks_next[g] = (kg < p.k_groups) ? __ldg(ks_base + kg) : 0.0f;
        }
      }
      tc_wait_ld();

      if (DUMP && p.s_dump != nullptr && row < p.Sq) {
        int32_t* dst = p.s_dump + (static_cast<long long>(bh) * p.Sq + row) * p.Skv + kv_base;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kv_base + 32 * c + i < p.Skv) dst[32 * c + i] = static_cast<int32_t>(sr[c][i]);
      }

      const bool masked = (CAUSAL && kv_base + kHalfN - 1 > q_base) || (kv_base + kHalfN > p.Skv);
      // columns below this bound are visible to this row (causal: col <= row; length: col < Skv)
      const int col_end = masked ? min(p.Skv, CAUSAL ? row + 1 : p.Skv) - kv_base : kHalfN;

      // p = exp2(s - m), row sum before rounding (:676-689), P -> fp16 pairs.  Returns the sum of
      // the 64 values of this half.
      // raw accumulator word -> fp32: an int32 product sum (exact), or the fp32 dot product itself
      auto score_of = [](uint32_t w) -> float {
        if constexpr (QKF) return __uint_as_float(w);
        else return __int2float_rn(static_cast<int>(w));
      };
      uint32_t pk[32];
      f32x2_t cg2[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) cg2[g] = pack2(cg[g], cg[g]);
      auto exp_pass = [&](auto masked_tag, float m_now) -> float {
        constexpr bool kMasked = decltype(masked_tag)::value;
        const f32x2_t neg_m = pack2(-m_now, -m_now);
        f32x2_t acc = pack2(0.0f, 0.0f);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int e = 32 * c + 2 * i;
            const f32x2_t sf = pack2(score_of(sr[c][2 * i]), score_of(sr[c][2 * i + 1]));
            const float2 x = unpack2(ffma2(sf, cg2[e >> 4], neg_m));
            float2 pp = make_float2(fast_exp2(x.x), fast_exp2(x.y));
            if constexpr (kMasked) {
              if (e >= col_end) pp.x = 0.0f;
              if (e + 1 >= col_end) pp.y = 0.0f;
            }
            acc = fadd2(acc, pack2(pp.x, pp.y));
            pk[16 * c + i] = pack_half2(pp.x, pp.y);
          }
        }
        const float2 a = unpack2(acc);
        return a.x + a.y;
      };

      // Common case (not the first half, no mask): exponentiate against the running maximum
      // straight away.  If the 64 values add up to no more than 2^14, none of them exceeded 2^14:
      // the lazy-rescale rule would not have moved the maximum, P fits fp16 comfortably, and the
      // step is done without a pass over the scores for the maximum.  Otherwise (or if the sum is
      // not a number) fall through to the exact path and redo the step.
      if (yields) __nanosleep(0);                       // see SAGE_DEPHASE
      bool done = false;
      float m_half = kMaskValue;
      const bool first_or_masked = (hh == 0) || masked;
      // The attempt is skipped while the data keeps refusing it: a refused attempt or a step that
      // had to move the maximum raises `distrust`, a step that did not lowers it.  Data whose maxima
      // keep jumping (heavy tails) would pay for two exp passes on most steps otherwise.
      const bool attempt = !first_or_masked && distrust < 2;
      if (attempt) {
        const float sum = exp_pass(std::false_type{}, m_used);
        if (!__any_sync(0xffffffffu, !(sum <= kOptimisticSumMax))) {
          l += sum;
          done = true;
        }
      }
      if (attempt) distrust = done ? max(distrust - 1, 0) : min(distrust + 2, 4);
      if (!done && !masked && !QKF) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {                   // scales are >= 0: max commutes with the scaling
          int mx = static_cast<int>(sr[g >> 1][(g & 1) * 16]);
#pragma unroll
          for (int i = 1; i < 16; ++i) mx = max(mx, static_cast<int>(sr[g >> 1][(g & 1) * 16 + i]));
          m_half = fmaxf(m_half, __int2float_rn(mx) * cg[g]);
        }
      } else if (!done) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float sv = score_of(sr[c][i]) * cg[(32 * c + i) >> 4];   // (:1679) for the fp32 scores
            if (32 * c + i < col_end) m_half = fmaxf(m_half, sv);
          }
      }

      if (!done) {
        // lazy rescale: move the running maximum only when it grew by more than 2^14
        if (hh == 0) {
          m_used = m_half;
        } else {
          // After a refused attempt the bar is lower: a row whose 64 values added up to more
          // than 2^14 has a maximum above 2^8, and it must move or it would be refused again.
          const bool need = m_half > m_used + (attempt ? kRefusedBarLog2 : kLazyRescaleLog2);
          const bool moved = __any_sync(0xffffffffu, need);
          if (!attempt) distrust = moved ? min(distrust + 1, 4) : distrust - 1;
          if (moved) {
            // O must be at rest: the P.V of the previous half has to be complete
            const int hp = h ^ 1;
            const int tp = h ? t : t - 1;
            SAGE_WAIT_OR(pv_done + hp, tp & 1, 9, { ok = false; break; });
            tc_fence_after();
            const float alpha = need ? fast_exp2(m_used - m_half) : 1.0f;   // (:667)
            if (need) m_used = m_half;
            l *= alpha;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t orr[32];
              tmem_ld32(t_o + 32 * c, orr);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
              tmem_st32(t_o + 32 * c, orr);
            }
          }
        }
        // Two copies of the loop: only tiles on the diagonal or at the ragged end pay for masking.
        if (masked) l += exp_pass(std::true_type{}, m_used);
        else l += exp_pass(std::false_type{}, m_used);
      }
      tmem_st32(tmem_base + lane_base + kColP + h * kHalfN, pk);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(p_full + h);
    }

    // ---- epilogue: o = acc * (1/l), one rounding to the output type (:769-786)
    if (!ok) break;
    if (n_kv > 0) {
      SAGE_WAIT_OR(o_final, it & 1, 10, { ok = false; break; });
      tc_fence_after();
    }
    {
      // A pass over the whole item writes the output: each warp stages its 32 rows in shared memory
      // (V stage 0: idle by now, and the producer does not refill it before `epi_done`), one
      // [32 rows][64 columns] box of 128-byte rows per 64 columns of head_dim, written with the
      // 128-byte swizzle so that the 32 row owners do not collide on banks, and one lane hands the
      // boxes to the TMA, which clips rows past Sq and follows the caller's strides.
      // A pass over part of an item (persistent variant) writes acc / l and m + log2 l in fp32 to the
      // CTA's partial buffers instead.
      const float inv_l = (l > 0.0f) ? (1.0f / l) : 0.0f;
      const bool whole = !STREAMK || sg.slot < 0;
      if (whole) {
        if (p.lse != nullptr && row < p.Sq) {
          // scores are in base 2 (log2(e) is folded into the Q scale): ln sum exp = (m + log2 l) ln 2;
          // a row without keys gets -inf
          p.lse[static_cast<long long>(bh) * p.Sq + row] =
              (l > 0.0f) ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
      } else {
        p.part_lse[(static_cast<long long>(blockIdx.x) * 2 + sg.slot) * kBlockM + threadIdx.x] =
            (l > 0.0f) ? (m_used + log2f(l)) : -INFINITY;
      }
      uint8_t* stage = s_v + warp * ((D / 64) * 4096);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        if (n_kv > 0) {
          tmem_ld32(t_o + 32 * c, orr);
          tc_wait_ld();
          if (STREAMK && c == D / 32 - 1) {             // O is in registers: the next segment may overwrite it
            tc_fence_before();
            mbar_arrive(o_free);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = 0u;
        }
        if (!whole) {
          float4* dst = reinterpret_cast<float4*>(
              p.part_o + ((static_cast<long long>(blockIdx.x) * 2 + sg.slot) * kBlockM + threadIdx.x) * D + 32 * c);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dst[i] = make_float4(__uint_as_float(orr[4 * i]) * inv_l, __uint_as_float(orr[4 * i + 1]) * inv_l,
                                 __uint_as_float(orr[4 * i + 2]) * inv_l, __uint_as_float(orr[4 * i + 3]) * inv_l);
          }
          continue;
        }
        uint32_t out[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = __uint_as_float(orr[2 * i]) * inv_l;
          const float bb = __uint_as_float(orr[2 * i + 1]) * inv_l;
          out[i] = p.out_bf16 ? pack_bf162(a, bb) : pack_half2(a, bb);
        }
        uint8_t* box = stage + (c >> 1) * 4096 + lane * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int chunk = ((c & 1) * 4 + i) ^ (lane & 7);
          *reinterpret_cast<uint4*>(box + chunk * 16) =
              make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
        }
      }
      if (whole) fence_proxy_async_smem();
      __syncwarp();
      const bool store_local = whole && q_base + warp * 32 < p.Sq;
      if (lane == 0 && store_local) {
#pragma unroll
        for (int bx = 0; bx < D / 64; ++bx)
          tma_store_4d(&tm_o, stage + bx * 4096, bx * 64, q_base + warp * 32, hq, b);
        tma_store_commit();
      }
      if (!STREAMK && p.n_peers > 0) {
        // The staged rows go to the peers as well, while the TMA reads them for the local copy: 8 lanes cover the 128 bytes of one row of a box
        // (undoing the swizzle), so a warp instruction writes four rows of 128 contiguous bytes.
        const int sub = lane >> 3, piece = lane & 7;
#pragma unroll
        for (int bx = 0; bx < D / 64; ++bx) {
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const int r = rr * 4 + sub;
            const int row_g = q_base + warp * 32 + r;
            const uint4 val = *reinterpret_cast<const uint4*>(stage + bx * 4096 + r * 128 + ((piece ^ (r & 7)) * 16));
            if (row_g < p.Sq) {
              const long long off = b * p.o_stride_b + hq * p.o_stride_h + static_cast<long long>(row_g) * p.o_stride_s +
                                    bx * 64 + piece * 8;                     // in 16-bit elements
              for (int pe = 0; pe < p.n_peers; ++pe)
                *reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.peer_o[pe]) + off) = val;
            }
          }
        }
      }
      if (lane == 0) {
        if (store_local) tma_store_wait_read();
        if (STREAMK && n_kv > 0) mbar_arrive(epi_done);   // the staging area may be refilled with V
      }
      __syncwarp();
    }
    if (STREAMK && n_kv > 0) {
      kt += n_kv;
      ++it;
    }
    if (!STREAMK) break;
    }  // segments
  }
#undef SAGE_WAIT_OR
#undef SAGE_WAIT_ROLE_OR

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up.  Let copies and MMAs that are still in flight land before the shared memory
    // and TMEM of this CTA are handed back, then report.
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) {
      const int code = *fail_code ? *fail_code : kStatusWaitTimeout;
      if (p.status) atomicCAS(p.status, 0, code);
      if (p.status_host) {              // the host can see the failure without synchronising
        *reinterpret_cast<volatile int*>(p.status_host) = code;
        __threadfence_system();
      }
    }
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Merge of the partial results of the persistent variant.  One CTA per item (query tile of one
// (batch, head)); items that one attention CTA covered completely were written by it and are
// skipped.  For the others, part k (k = 0 .. n-1) holds o_k = acc_k / l_k and e_k = m_k + log2 l_k
// over its share of the keys, and
//     o = sum_k 2^(e_k - E) o_k / sum_k 2^(e_k - E),   E = max_k e_k,   lse = (E + log2 sum) ln 2.
// Which CTA holds which part follows from the same arithmetic as SegIter: CTA c owns the steps
// [c*T/G, (c+1)*T/G); a part that starts at the first step of its CTA is in slot 0, the other
// possible part of a CTA (its last segment) in slot 1.
struct MergeParams {
  const float* part_o;
  const float* part_lse;
  void* o;
  long long o_stride_b, o_stride_h, o_stride_s;
  float* lse;                   // optional [B,Hq,Sq]
  int Hq, Sq, n_q_tiles;
  int nkv_full, tiles_per_head;
  long long total_tiles;
  int attn_grid;                // G
  int causal, out_bf16;
};

constexpr int kMergeRows = 32;                          // rows of an item per merge CTA
constexpr int kMergeSplit = kBlockM / kMergeRows;       // merge CTAs per item

template <int D>
__global__ void __launch_bounds__(256) sage_attn_merge_kernel(const MergeParams p) {
  __shared__ float row_max[kMergeRows];
  __shared__ float row_inv[kMergeRows];
  const int item = blockIdx.x / kMergeSplit;
  const int row0 = (blockIdx.x - item * kMergeSplit) * kMergeRows;     // first row of this CTA within the item
  const int bh = item / p.n_q_tiles;
  const int qt = item - bh * p.n_q_tiles;
  if (qt * kBlockM + row0 >= p.Sq) return;
  const int nkv = p.nkv_full;
  const int tiles = p.causal ? min(qt + 1, nkv) : nkv;
  long long before;                                      // steps of this head before query tile qt
  if (!p.causal) before = static_cast<long long>(qt) * nkv;
  else if (qt <= nkv) before = static_cast<long long>(qt) * (qt + 1) / 2;
  else before = static_cast<long long>(nkv) * (nkv + 1) / 2 + static_cast<long long>(qt - nkv) * nkv;
  const long long start = static_cast<long long>(bh) * p.tiles_per_head + before;
  const long long end = start + tiles;
  const long long G = p.attn_grid, T = p.total_tiles;
  const int c_first = static_cast<int>(((start + 1) * G - 1) / T);     // CTA that owns step `start`
  const int c_last = static_cast<int>((end * G - 1) / T);              // ... step `end - 1`
  if (c_first == c_last) return;
  const int n_parts = c_last - c_first + 1;
  const int first_slot = ((T * c_first) / G == start) ? 0 : 1;
  // rows of part k start at this offset (in rows) of the partial buffers
  auto part_row0 = [&](int k) -> long long {
    return (static_cast<long long>(c_first + k) * 2 + (k == 0 ? first_slot : 0)) * kBlockM + row0;
  };

  const int tid = threadIdx.x;
  if (tid < kMergeRows) {
    float e_max = -INFINITY;
    for (int k = 0; k < n_parts; ++k) e_max = fmaxf(e_max, p.part_lse[part_row0(k) + tid]);
    float sum = 0.0f;
    for (int k = 0; k < n_parts; ++k) {
      const float e = p.part_lse[part_row0(k) + tid];
      sum += (e == -INFINITY) ? 0.0f : exp2f(e - e_max);
    }
    row_max[tid] = e_max;
    row_inv[tid] = (sum > 0.0f) ? 1.0f / sum : 0.0f;
    const int row = qt * kBlockM + row0 + tid;
    if (p.lse != nullptr && row < p.Sq) {
      p.lse[static_cast<long long>(bh) * p.Sq + row] =
          (sum > 0.0f) ? (e_max + log2f(sum)) * 0.6931471805599453f : -INFINITY;
    }
  }
  __syncthreads();
  const int b = bh / p.Hq, h = bh - b * p.Hq;
  constexpr int kVecPerRow = D / 4;
  constexpr int kPerThread = kMergeRows * kVecPerRow / 256;   // 4 (D = 128) or 2 (D = 64) float4 per thread
  float4 acc[kPerThread];
#pragma unroll
  for (int u = 0; u < kPerThread; ++u) acc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int k = 0; k < n_parts; ++k) {
    const long long pr = part_row0(k);
    float4 x[kPerThread];
    float w[kPerThread];
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
      const int idx = tid + u * 256;
      const int r = idx / kVecPerRow, c4 = idx - r * kVecPerRow;
      const float e = p.part_lse[pr + r];
      w[u] = (e == -INFINITY) ? 0.0f : exp2f(e - row_max[r]);
      x[u] = *reinterpret_cast<const float4*>(p.part_o + (pr + r) * D + 4 * c4);
    }
#pragma unroll
    for (int u = 0; u < kPerThread; ++u) {
      if (w[u] == 0.0f) continue;                         // a part without visible keys may hold anything
      acc[u].x += w[u] * x[u].x; acc[u].y += w[u] * x[u].y; acc[u].z += w[u] * x[u].z; acc[u].w += w[u] * x[u].w;
    }
  }
#pragma unroll
  for (int u = 0; u < kPerThread; ++u) {
    const int idx = tid + u * 256;
    const int r = idx / kVecPerRow, c4 = idx - r * kVecPerRow;
    const int row = qt * kBlockM + row0 + r;
    if (row >= p.Sq) continue;
    const float inv = row_inv[r];
    const long long off = b * p.o_stride_b + h * p.o_stride_h + static_cast<long long>(row) * p.o_stride_s + 4 * c4;
    uint2 out;
    if (p.out_bf16) {
      out.x = pack_bf162(acc[u].x * inv, acc[u].y * inv);
      out.y = pack_bf162(acc[u].z * inv, acc[u].w * inv);
    } else {
      out.x = pack_half2(acc[u].x * inv, acc[u].y * inv);
      out.y = pack_half2(acc[u].z * inv, acc[u].w * inv);
    }
    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.o) + off) = out;
  }
}

}  // namespace sage
