// Preparation kernels of the INT8 attention path (HBM-bound byte work):
//   * sage_kmean_kernel : per-(b,h,d) mean of K over the sequence (only for smooth_k);
//   * sage_prep_kernel  : per-block INT8 quantisation of Q (32-row groups, sm_scale*log2e folded
//                         in) and of K (16-row groups, optional mean subtraction) with fp32 scales,
//                         plus, in the same launch, the bf16 -> fp16 copy of V that P.V consumes.
// They replace mean_hnd_kernel, quant_qk_int8_hnd_kernel and the dtype half of v_transpose_kernel
// of the reference (csrc/attn_gfx11.cu:94-145, :147-321, :326-407).
//
// Bit-exactness.  The quantisation arithmetic is written with __fmul_rn/__fadd_rn/__fdiv_rn so
// that nvcc cannot contract a multiply and an add into an FMA; the results are the ones separate
// IEEE fp32 operations give.  The group maximum is taken on the un-scaled magnitudes and scaled
// once: fp32 rounding is monotone, so max_i fl(|x_i|*s) == fl(max_i|x_i| * s).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <type_traits>

#include "ptx_sm100.cuh"

namespace sage {

struct StridedView {        // one of q / k / v in the caller's layout, strides in elements
  const void* ptr;
  long long stride_b, stride_h, stride_s;
};

struct PrepParams {
  StridedView q, k, v;
  int8_t* q_i8;             // [B,Hq,Sq,D]
  int8_t* k_i8;             // [B,Hkv,Skv,D]
  float* q_scale;           // [B,Hq,ceil(Sq/32)]
  float* k_scale;           // [B,Hkv,ceil(Skv/16)]
  const void* k_mean;       // [B,Hkv,D] in the input dtype, or nullptr
  __half* v16;              // [B,Hkv,Skv,D] fp16 copy of V, or nullptr (no conversion)
  int B, Hq, Hkv, Sq, Skv;
  int q_groups, k_groups;   // ceil(Sq/32), ceil(Skv/16)
  float sm_scale_log2e;
  int q_blocks, k_blocks;   // CTAs spent on Q groups, on K groups; the rest convert V
  // sage_prep_smooth_kernel only: the mean it computes goes to k_mean_out ([B,Hkv,D], input dtype);
  // k_clusters clusters of 8 CTAs share the (batch, kv-head) pairs between them
  void* k_mean_out;
  int k_clusters;
};

constexpr int kPrepThreads = 256;
constexpr int kPrepWarps = kPrepThreads / 32;
constexpr int kQGroupRows = 32;   // csrc/attn_gfx11.cu:46
constexpr int kKGroupRows = 16;   // csrc/attn_gfx11.cu:47

template <typename T> __device__ __forceinline__ float elem_to_float(T v);
template <> __device__ __forceinline__ float elem_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float elem_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

// csrc/attn_gfx11.cu:85-92: add +-0.5 (sign of the value), convert toward zero, clamp to
// [-128, 127].  Returned as int32 without the clamp; pack_s8x4 saturates.  copysign differs from
// the reference's (x >= 0 ? .5 : -.5) only for -0.0 and NaN, which both give 0 either way.
__device__ __forceinline__ int quantise_one(float y) {
  return __float2int_rz(__fadd_rn(y, copysignf(0.5f, y)));
}
// Four int32 -> four saturated int8 in one word, a in the lowest byte.
__device__ __forceinline__ uint32_t pack_s8x4(int a, int b, int c, int d) {
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
  return out;
}

// One warp handles 16 consecutive rows (all D columns) of one (b,h): a K group, or half of a Q
// group (the two warps of a Q group exchange their maxima through shared memory).  A row is D/8
// lanes x 16 bytes, so a warp reads 32*8/D rows per 512-byte load and keeps 16*D*2/32 bytes in
// registers between the max pass and the quantisation pass.
constexpr int kRowsPerWarp = 16;
constexpr int kQGroupsPerBlock = kPrepWarps / 2;
constexpr int kKGroupsPerBlock = kPrepWarps;

// Two 16-bit elements of one 32-bit word as fp32 (exact).
template <typename T> __device__ __forceinline__ float2 word_to_float2(uint32_t w);
template <> __device__ __forceinline__ float2 word_to_float2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
template <> __device__ __forceinline__ float2 word_to_float2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
// |x| of a 16-bit float from its magnitude bits (the bit pattern orders like the value).
template <typename T> __device__ __forceinline__ float magnitude_to_float(uint32_t m16);
template <> __device__ __forceinline__ float magnitude_to_float<__nv_bfloat16>(uint32_t m16) {
  return __uint_as_float(m16 << 16);
}
template <> __device__ __forceinline__ float magnitude_to_float<__half>(uint32_t m16) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(m16)));
}

// 16-byte read-only loads with an L2 eviction priority: `evict_last` keeps lines that will be read
// again soon ahead of streaming traffic, `evict_first` gives them up.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint4 ldg_l2_hint(const uint4* ptr, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr), "l"(policy));
  return v;
}

template <typename T, int D, bool HAS_MEAN>
struct RowSlab {
  static constexpr int kLanesPerRow = D / 8;
  static constexpr int kRowsPerPass = 32 / kLanesPerRow;
  static constexpr int kPasses = kRowsPerWarp / kRowsPerPass;
  uint4 raw[kPasses];
  f32x2_t neg_mean2[4];     // -mean of my 8 columns, as pairs: x - mean == x + (-mean) exactly
  int sub, col;

  // `mean_bh` (global memory, read through the read-only path) or `mean_vec` (the 8 means of this
  // lane's columns, already in registers) - at most one of them
  // `l2_policy` != 0: the rows are read with that L2 eviction policy.
  __device__ __forceinline__ void load(const T* __restrict__ in_bh, long long stride_s, int row0, int S,
                                       const T* __restrict__ mean_bh, int lane, const uint4* mean_vec = nullptr,
                                       uint64_t l2_policy = 0) {
    sub = lane / kLanesPerRow;
    col = (lane % kLanesPerRow) * 8;
    const T* src = in_bh + static_cast<long long>(row0 + sub) * stride_s + col;
    const long long step = static_cast<long long>(kRowsPerPass) * stride_s;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      raw[p] = make_uint4(0u, 0u, 0u, 0u);
      if (row0 + p * kRowsPerPass + sub < S) {
        raw[p] = l2_policy ? ldg_l2_hint(reinterpret_cast<const uint4*>(src), l2_policy)
                           : __ldg(reinterpret_cast<const uint4*>(src));
      }
      src += step;
    }
    if (HAS_MEAN) {
      const uint4 mraw = mean_vec ? *mean_vec : __ldg(reinterpret_cast<const uint4*>(mean_bh + col));
      const uint32_t* mw = reinterpret_cast<const uint32_t*>(&mraw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 m = word_to_float2<T>(mw[i]);
        neg_mean2[i] = pack2(-m.x, -m.y);
      }
    }
  }

  // pass 1 (csrc/attn_gfx11.cu:189-237): abs-max of (x - mean) over the warp's rows.  Without a
  // mean the maximum is taken on the 15 magnitude bits, two elements per instruction; rows past
  // the end were loaded as zeros and cannot win.
  __device__ __forceinline__ float abs_max(int row0, int S) const {
    float vmax = 0.0f;
    if (!HAS_MEAN) {
      uint32_t m2 = 0u;
#pragma unroll
      for (int p = 0; p < kPasses; ++p) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw[p]);
#pragma unroll
        for (int i = 0; i < 4; ++i) m2 = __vmaxu2(m2, w[i] & 0x7FFF7FFFu);
      }
      vmax = magnitude_to_float<T>(max(m2 & 0xFFFFu, m2 >> 16));
    } else {
#pragma unroll
      for (int p = 0; p < kPasses; ++p) {
        if (row0 + p * kRowsPerPass + sub < S) {
          const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw[p]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 x = word_to_float2<T>(w[i]);
            const float2 v = unpack2(fadd2(pack2(x.x, x.y), neg_mean2[i]));
            vmax = fmaxf(vmax, fmaxf(fabsf(v.x), fabsf(v.y)));
          }
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
    return vmax;
  }

  // pass 2 (csrc/attn_gfx11.cu:250-318): quantise from the registers, 8 bytes per lane and row.
  // mul and add stay separate IEEE operations (packed two at a time), never an FMA.
  __device__ __forceinline__ void quantise(int row0, int S, float iscale, int8_t* __restrict__ out_bh) const {
    const f32x2_t iscale2 = pack2(iscale, iscale);
    int8_t* dst = out_bh + static_cast<long long>(row0 + sub) * D + col;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      if (row0 + p * kRowsPerPass + sub < S) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw[p]);
        int qv[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 x = word_to_float2<T>(w[i]);
          f32x2_t v2 = pack2(x.x, x.y);
          if (HAS_MEAN) v2 = fadd2(v2, neg_mean2[i]);
          const f32x2_t y2 = fmul2(v2, iscale2);
          const float2 y = unpack2(y2);
          const float2 z = unpack2(fadd2(y2, pack2(copysignf(0.5f, y.x), copysignf(0.5f, y.y))));
          qv[2 * i] = __float2int_rz(z.x);
          qv[2 * i + 1] = __float2int_rz(z.y);
        }
        *reinterpret_cast<uint2*>(dst) =
            make_uint2(pack_s8x4(qv[0], qv[1], qv[2], qv[3]), pack_s8x4(qv[4], qv[5], qv[6], qv[7]));
      }
      dst += kRowsPerPass * D;
    }
  }
};

// The three kinds of block, for a block of THREADS threads.
// Q: a group of 32 rows per warp pair.
template <typename T, int D, int THREADS>
__device__ __forceinline__ void prep_q_block(const PrepParams& p, int blk, float* warp_max) {
  constexpr int kGroupsPerBlock = THREADS / 64;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long g = static_cast<long long>(blk) * kGroupsPerBlock + (warp >> 1);
  const long long total = static_cast<long long>(p.B) * p.Hq * p.q_groups;
  const bool valid = g < total;
  const int grp = valid ? static_cast<int>(g % p.q_groups) : 0;
  const int bh = valid ? static_cast<int>(g / p.q_groups) : 0;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int row0 = grp * kQGroupRows + (warp & 1) * kRowsPerWarp;
  const int S = valid ? p.Sq : 0;
  const T* in_bh = reinterpret_cast<const T*>(p.q.ptr) + b * p.q.stride_b + h * p.q.stride_h;
  RowSlab<T, D, false> slab;
  slab.load(in_bh, p.q.stride_s, row0, S, nullptr, lane);
  const float mine = slab.abs_max(row0, S);
  if (lane == 0) warp_max[warp] = mine;
  __syncthreads();
  const float vmax = fmaxf(warp_max[warp], warp_max[warp ^ 1]);
  const float s_mul = p.sm_scale_log2e;
  const float amax = fmaxf(1e-7f, __fmul_rn(vmax, fabsf(s_mul)));      // :192,224
  if (valid && lane == 0 && (warp & 1) == 0) p.q_scale[g] = __fdiv_rn(amax, 127.0f);   // :244-245
  const float iscale = __fmul_rn(__fdiv_rn(127.0f, amax), s_mul);      // :252,296
  slab.quantise(row0, S, iscale, p.q_i8 + static_cast<long long>(bh) * p.Sq * D);
}

// K: one group of 16 rows of (batch*head) `bh`, by one warp.  The mean comes from global memory
// (`p.k_mean`) or, if `mean_vec` is given, from registers.
template <typename T, int D>
__device__ __forceinline__ void prep_k_group(const PrepParams& p, int bh, int grp, int lane, const uint4* mean_vec,
                                             uint64_t l2_policy = 0) {
  const int b = bh / p.Hkv, h = bh % p.Hkv;
  const int row0 = grp * kKGroupRows;
  const T* in_bh = reinterpret_cast<const T*>(p.k.ptr) + b * p.k.stride_b + h * p.k.stride_h;
  const T* mean_bh =
      (p.k_mean && !mean_vec) ? reinterpret_cast<const T*>(p.k_mean) + static_cast<long long>(bh) * D : nullptr;
  float* scale_out = p.k_scale + static_cast<long long>(bh) * p.k_groups + grp;
  int8_t* out_bh = p.k_i8 + static_cast<long long>(bh) * p.Skv * D;
  auto run = [&](auto slab) {
    slab.load(in_bh, p.k.stride_s, row0, p.Skv, mean_bh, lane, mean_vec, l2_policy);
    const float amax = fmaxf(1e-7f, slab.abs_max(row0, p.Skv));        // s = 1 for K
    if (lane == 0) *scale_out = __fdiv_rn(amax, 127.0f);
    slab.quantise(row0, p.Skv, __fdiv_rn(127.0f, amax), out_bh);
  };
  if (mean_bh != nullptr || mean_vec != nullptr) run(RowSlab<T, D, true>{});
  else run(RowSlab<T, D, false>{});
}

// V: 16-bit copy to fp16 [B,Hkv,Skv,D] (csrc/attn_gfx11.cu:377-381: __float2half_rn).
// Each thread converts four 16-byte vectors, THREADS * 16 bytes apart in the output, so a warp moves
// 512 B per load; the four loads are issued before the first store.  (batch*head, position) of the
// first vector comes from one division, the others follow by stepping THREADS / (D/8) rows.
template <typename T, int D, int THREADS>
__device__ __forceinline__ void prep_v_block(const PrepParams& p, int blk) {
  if (p.v16 == nullptr) return;
  constexpr int kVecPerRow = D / 8;
  constexpr int kRowStep = THREADS / kVecPerRow;
  const long long n_vec = static_cast<long long>(p.B) * p.Hkv * p.Skv * kVecPerRow;
  const long long base = static_cast<long long>(blk) * (THREADS * 4) + threadIdx.x;
  const int c = static_cast<int>(base % kVecPerRow) * 8;
  const long long row0 = base / kVecPerRow;
  int bh = static_cast<int>(row0 / p.Skv);
  int s = static_cast<int>(row0 - static_cast<long long>(bh) * p.Skv);
  uint4 raw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    raw[i] = make_uint4(0u, 0u, 0u, 0u);
    if (base + static_cast<long long>(i) * THREADS < n_vec) {
      const int b = bh / p.Hkv, h = bh - b * p.Hkv;
      const T* src = reinterpret_cast<const T*>(p.v.ptr) + b * p.v.stride_b + h * p.v.stride_h +
                     static_cast<long long>(s) * p.v.stride_s + c;
      raw[i] = __ldg(reinterpret_cast<const uint4*>(src));
    }
    s += kRowStep;
    while (s >= p.Skv) {
      s -= p.Skv;
      ++bh;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long vec = base + static_cast<long long>(i) * THREADS;
    if (vec < n_vec) {
      const T* xv = reinterpret_cast<const T*>(&raw[i]);
      uint4 out;
      uint32_t* o32 = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 h2 = __floats2half2_rn(elem_to_float<T>(xv[2 * j]), elem_to_float<T>(xv[2 * j + 1]));
        o32[j] = *reinterpret_cast<const uint32_t*>(&h2);
      }
      *reinterpret_cast<uint4*>(p.v16 + vec * 8) = out;
    }
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kPrepThreads, 4) sage_prep_kernel(const PrepParams p) {
  __shared__ float warp_max[kPrepWarps];
  int blk = blockIdx.x;
  if (blk < p.q_blocks) {
    prep_q_block<T, D, kPrepThreads>(p, blk, warp_max);
    return;
  }
  blk -= p.q_blocks;
  if (blk < p.k_blocks) {                                   // ---- K: a group of 16 rows per warp
    const long long g = static_cast<long long>(blk) * kKGroupsPerBlock + (threadIdx.x >> 5);
    const long long total = static_cast<long long>(p.B) * p.Hkv * p.k_groups;
    if (g >= total) return;
    prep_k_group<T, D>(p, static_cast<int>(g / p.k_groups), static_cast<int>(g % p.k_groups), threadIdx.x & 31, nullptr);
    return;
  }
  blk -= p.k_blocks;
  prep_v_block<T, D, kPrepThreads>(p, blk);
}

// ---------------------------------------------------------------------------------------------
// K mean over the sequence, in the reference's summation order (csrc/attn_gfx11.cu:94-145):
// 256 partial sums (partial t adds rows t, t+256, ... in fp32), then the 256 partials are added
// serially from 0 to 255, then one fp32 division by float(S) and one rounding to the input type.
//
// One cluster of 8 CTAs = one (b, h).  CTA r of the cluster owns the partials [32r, 32r+32): it
// reads, for every block of 256 rows, the 32 consecutive rows that feed them (whole rows, 16 bytes
// per thread, so a warp reads 512 contiguous bytes of a dense K), and keeps their running sums in
// registers.  The partials are then exchanged through distributed shared memory: CTA o of the
// cluster receives all 256 partials of the D/8 columns [o*D/8, (o+1)*D/8) and D/8 of its threads
// add them in order.  Eight CTAs per (b, h) put 8x more loads in flight than one CTA per column
// slab did, with every DRAM line read once by one warp.
struct MeanParams {
  StridedView k;
  void* mean_out;   // [B,H,D] in the input dtype
  int B, H, S, D;
};

constexpr int kMeanCluster = 8;                  // CTAs per (b, h)
constexpr int kMeanPartials = 256;               // csrc/attn_gfx11.cu:94-145: one partial per thread of its block
constexpr int kMeanPartialsPerCta = kMeanPartials / kMeanCluster;

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t map_to_cta(const void* smem_ptr, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_ptr))), "r"(cta_rank));
  return remote;
}
__device__ __forceinline__ void st_cluster_f32x4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <typename T, int D>
__global__ void __cluster_dims__(kMeanCluster, 1, 1) __launch_bounds__(256) sage_kmean_kernel(const MeanParams p) {
  constexpr int kLanesPerRow = D / 8;                       // 16-byte pieces of a row
  constexpr int kRowsPerPass = 256 / kLanesPerRow;          // rows the CTA reads at once
  constexpr int kSets = kMeanPartialsPerCta / kRowsPerPass; // partials per thread
  constexpr int kOwnCols = D / kMeanCluster;                // columns this CTA sums in the end
  static_assert(kSets >= 1 && kOwnCols % 8 == 0, "tile shape");
  __shared__ __align__(16) float part[kMeanPartials][kOwnCols];

  const int tid = threadIdx.x;
  const uint32_t rank = blockIdx.x;                         // cluster = the 8 CTAs of one blockIdx.(y,z)
  const int h = blockIdx.y, b = blockIdx.z;
  const int rr = tid / kLanesPerRow, c = tid % kLanesPerRow;
  const T* base = reinterpret_cast<const T*>(p.k.ptr) + b * p.k.stride_b + h * p.k.stride_h + c * 8;

  cluster_arrive();     // matched by the wait before the first remote store: every CTA has started

  float acc[kSets][8];
#pragma unroll
  for (int j = 0; j < kSets; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.0f;

  const int p0 = static_cast<int>(rank) * kMeanPartialsPerCta + rr;        // first partial of this thread
  constexpr int kUnroll = 4;
  for (int s0 = 0; s0 < p.S; s0 += kMeanPartials * kUnroll) {
    uint4 r[kUnroll][kSets];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int j = 0; j < kSets; ++j) {
        const int srow = s0 + u * kMeanPartials + p0 + j * kRowsPerPass;
        r[u][j] = make_uint4(0u, 0u, 0u, 0u);
        if (srow < p.S) r[u][j] = __ldg(reinterpret_cast<const uint4*>(base + static_cast<long long>(srow) * p.k.stride_s));
      }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int j = 0; j < kSets; ++j) {
        const int srow = s0 + u * kMeanPartials + p0 + j * kRowsPerPass;
        if (srow < p.S) {                                   // a missing row adds nothing (not +0.0)
          const T* x = reinterpret_cast<const T*>(&r[u][j]);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[j][e] = __fadd_rn(acc[j][e], elem_to_float<T>(x[e]));
        }
      }
  }

  // hand the partials to the CTAs that own their columns
  cluster_wait();
  const uint32_t owner = static_cast<uint32_t>((c * 8) / kOwnCols);
  const int col_in_owner = (c * 8) % kOwnCols;
#pragma unroll
  for (int j = 0; j < kSets; ++j) {
    const int pidx = p0 + j * kRowsPerPass;
    const uint32_t dst = map_to_cta(&part[pidx][col_in_owner], owner);
    st_cluster_f32x4(dst, acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
    st_cluster_f32x4(dst + 16, acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
  }
  cluster_arrive();
  cluster_wait();       // all 256 partials of this CTA's columns have landed; nobody writes here again

  if (tid < kOwnCols) {
    float sum = 0.0f;
#pragma unroll 16
    for (int i = 0; i < kMeanPartials; ++i) sum = __fadd_rn(sum, part[i][tid]);
    const float value = __fdiv_rn(sum, static_cast<float>(p.S));
    T* out = reinterpret_cast<T*>(p.mean_out) + (static_cast<long long>(b) * p.H + h) * D + rank * kOwnCols + tid;
    if constexpr (std::is_same<T, __half>::value) {
      *out = __float2half_rn(value);
    } else {
      *out = __float2bfloat16_rn(value);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// smooth_k in one launch: K mean, quantisation of K against it, quantisation of Q and the fp16 copy of
// V.  K is read from DRAM once: the cluster that has just summed a (batch, kv-head) quantises the same
// rows again while they are still in L2 (2 MiB per head at S = 8192, D = 128), instead of a second
// kernel reading all of K again after all of it has been through the cache.
//
// Blocks of 512 threads in clusters of 8.  The first 8 * k_clusters CTAs work on K: cluster c takes the
// heads c, c + k_clusters, ... one after the other.  Per head:
//   1. mean, exactly as sage_kmean_kernel: CTA r owns the partials [32r, 32r+32) of the reference's
//      order and reads the rows that feed them; partials go to the CTA that owns their columns
//      (distributed shared memory), which adds them serially, divides, rounds once;
//   2. every CTA sends the D/8 means it owns to all eight CTAs (and to global memory: the caller gets
//      the mean as well);
//   3. each warp quantises 16-row groups of the rows its CTA read in step 1.
// The other CTAs quantise Q and convert V as in sage_prep_kernel; they run next to the K clusters, so
// the launch as a whole moves |Q| + |K| + |V| in and the int8 / fp16 copies out.
constexpr int kFusedThreads = 512;

__device__ __forceinline__ void st_cluster_u16(uint32_t addr, unsigned short v) {
  asm volatile("st.shared::cluster.u16 [%0], %1;" :: "r"(addr), "h"(v) : "memory");
}

template <typename T, int D>
__global__ void __cluster_dims__(kMeanCluster, 1, 1) __launch_bounds__(kFusedThreads, 2)
sage_prep_smooth_kernel(const PrepParams p) {
  constexpr int kLanesPerRow = D / 8;
  constexpr int kActive = kMeanPartialsPerCta * kLanesPerRow;     // threads that read rows in step 1
  constexpr int kOwnCols = D / kMeanCluster;
  static_assert(kActive <= kFusedThreads && kOwnCols % 8 == 0, "tile shape");
  __shared__ __align__(16) float part[kMeanPartials][kOwnCols];
  __shared__ __align__(16) T mean_s[D];
  __shared__ float warp_max[kFusedThreads / 32];

  const int tid = threadIdx.x;
  const int n_k_ctas = p.k_clusters * kMeanCluster;
  if (static_cast<int>(blockIdx.x) >= n_k_ctas) {
    int blk = blockIdx.x - n_k_ctas;
    if (blk < p.q_blocks) {
      prep_q_block<T, D, kFusedThreads>(p, blk, warp_max);
      return;
    }
    prep_v_block<T, D, kFusedThreads>(p, blk - p.q_blocks);        // blocks past the end do nothing
    return;
  }

  const uint32_t rank = blockIdx.x % kMeanCluster;
  const int cluster_id = blockIdx.x / kMeanCluster;
  const int n_heads = p.B * p.Hkv;
  const int warp = tid >> 5, lane = tid & 31;
  const int rr = tid / kLanesPerRow, c = tid % kLanesPerRow;
  const int p0 = static_cast<int>(rank) * kMeanPartialsPerCta + rr;          // the partial this thread sums
  const int n_blocks256 = (p.Skv + kMeanPartials - 1) / kMeanPartials;
  // K is read twice by the same CTA, a few microseconds apart, while Q and V stream through the same
  // L2: the first read asks the L2 to keep the lines, the second gives them up.
  const uint64_t keep = l2_policy_evict_last(), release = l2_policy_evict_first();

#pragma unroll 1
  for (int bh = cluster_id; bh < n_heads; bh += p.k_clusters) {
    const int b = bh / p.Hkv, h = bh % p.Hkv;
    const T* base = reinterpret_cast<const T*>(p.k.ptr) + b * p.k.stride_b + h * p.k.stride_h + c * 8;
    cluster_arrive();       // every CTA of the cluster is here: `part` and `mean_s` of the last head are free

    // ---- step 1: partial sums (csrc/attn_gfx11.cu:121-127), eight blocks of 256 rows in flight
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
    if (tid < kActive) {
      constexpr int kUnroll = 8;
      for (int s0 = 0; s0 < p.Skv; s0 += kMeanPartials * kUnroll) {
        uint4 r[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int srow = s0 + u * kMeanPartials + p0;
          r[u] = make_uint4(0u, 0u, 0u, 0u);
          if (srow < p.Skv) {
            r[u] = ldg_l2_hint(reinterpret_cast<const uint4*>(base + static_cast<long long>(srow) * p.k.stride_s), keep);
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int srow = s0 + u * kMeanPartials + p0;
          if (srow < p.Skv) {                               // a missing row adds nothing (not +0.0)
            const T* x = reinterpret_cast<const T*>(&r[u]);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = __fadd_rn(acc[e], elem_to_float<T>(x[e]));
          }
        }
      }
    }
    cluster_wait();
    if (tid < kActive) {
      const uint32_t owner = static_cast<uint32_t>((c * 8) / kOwnCols);
      const uint32_t dst = map_to_cta(&part[p0][(c * 8) % kOwnCols], owner);
      st_cluster_f32x4(dst, acc[0], acc[1], acc[2], acc[3]);
      st_cluster_f32x4(dst + 16, acc[4], acc[5], acc[6], acc[7]);
    }
    cluster_arrive();
    cluster_wait();         // all 256 partials of this CTA's columns have landed

    // ---- step 2: serial sum of the partials (:131-136), one division, one rounding; to everybody
    if (tid < kOwnCols) {
      float sum = 0.0f;
#pragma unroll 16
      for (int i = 0; i < kMeanPartials; ++i) sum = __fadd_rn(sum, part[i][tid]);
      const float value = __fdiv_rn(sum, static_cast<float>(p.Skv));
      T m;
      if constexpr (std::is_same<T, __half>::value) m = __float2half_rn(value);
      else m = __float2bfloat16_rn(value);
      const int col = static_cast<int>(rank) * kOwnCols + tid;
      reinterpret_cast<T*>(p.k_mean_out)[static_cast<long long>(bh) * D + col] = m;
      const unsigned short bits = *reinterpret_cast<const unsigned short*>(&m);
#pragma unroll
      for (uint32_t dst_rank = 0; dst_rank < kMeanCluster; ++dst_rank) st_cluster_u16(map_to_cta(&mean_s[col], dst_rank), bits);
    }
    cluster_arrive();
    cluster_wait();         // the D means are in every CTA's mean_s

    // ---- step 3: quantise the rows this CTA read (two 16-row groups per block of 256 rows)
    const uint4 mean_vec = *reinterpret_cast<const uint4*>(&mean_s[(lane % kLanesPerRow) * 8]);
    for (int u = warp; u < 2 * n_blocks256; u += kFusedThreads / 32) {
      const int row0 = (u >> 1) * kMeanPartials + static_cast<int>(rank) * kMeanPartialsPerCta + (u & 1) * kKGroupRows;
      if (row0 < p.Skv) prep_k_group<T, D>(p, bh, row0 / kKGroupRows, lane, &mean_vec, release);
    }
  }
}

}  // namespace sage
