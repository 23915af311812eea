// Folding of partial attention results over disjoint sets of keys (the ring of the sequence-parallel
// path): HBM-bound element-wise work, one launch per fold.
//
//   lse' = log(exp(lse) + exp(lse_j)),   o' = o * exp(lse - lse') + o_j * exp(lse_j - lse')
//
// with lse the natural-log sum of exponentials per query row as the attention kernels return it.
// The reference has no counterpart: its `return_lse` is a placeholder (sageattention/core.py:203-211).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace sage {

struct FoldParams {
  float* o_acc;             // [B,H,S,D] fp32 accumulator, element strides below
  long long acc_stride_b, acc_stride_h, acc_stride_s;
  float* lse_acc;           // fp32 [B,H,S], element strides below (a row slice of a larger tensor is allowed)
  long long lse_acc_stride_b, lse_acc_stride_h;
  const void* o_part;       // partial result, fp16 / bf16, element strides below
  long long part_stride_b, part_stride_h, part_stride_s;
  const float* lse_part;    // fp32 [B,H,S] contiguous
  int B, H, S, D;
  int part_bf16;
  int first;                // 1: the accumulators hold nothing yet and are overwritten
};

constexpr int kFoldThreads = 256;

// One thread = 8 consecutive columns of one row; a warp covers 32 * 8 columns = 2 (D = 128) or 4
// (D = 64) rows: 16-byte loads of the partial, 32-byte loads and stores of the accumulator.
__global__ void __launch_bounds__(kFoldThreads) sage_fold_partial_kernel(const FoldParams p) {
  const int vec_per_row = p.D / 8;
  const long long n_vec = static_cast<long long>(p.B) * p.H * p.S * vec_per_row;
  const long long idx = static_cast<long long>(blockIdx.x) * kFoldThreads + threadIdx.x;
  if (idx >= n_vec) return;
  const int c = static_cast<int>(idx % vec_per_row) * 8;
  const long long row = idx / vec_per_row;
  const int s = static_cast<int>(row % p.S);
  const long long bh = row / p.S;
  const int h = static_cast<int>(bh % p.H), b = static_cast<int>(bh / p.H);

  float* lse_slot = p.lse_acc + b * p.lse_acc_stride_b + h * p.lse_acc_stride_h + s;
  const float lse_j = p.lse_part[row];
  const float lse_old = p.first ? -INFINITY : *lse_slot;
  // a row that has seen no key on either side keeps -inf and zeros
  const float top = fmaxf(lse_old, lse_j);
  float w_old = 0.0f, w_new = 0.0f, lse_new = -INFINITY;
  if (top > -INFINITY) {
    const float e_old = expf(lse_old - top), e_new = expf(lse_j - top);
    const float sum = e_old + e_new;
    lse_new = top + logf(sum);
    w_old = e_old / sum;
    w_new = e_new / sum;
  }

  const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.o_part) + b * p.part_stride_b +
                                                    h * p.part_stride_h + static_cast<long long>(s) * p.part_stride_s + c);
  float x[8];
  const uint32_t* w32 = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (p.part_bf16) {
      x[2 * i] = __uint_as_float(w32[i] << 16);
      x[2 * i + 1] = __uint_as_float(w32[i] & 0xFFFF0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w32[i]));
      x[2 * i] = f.x;
      x[2 * i + 1] = f.y;
    }
  }
  float4* acc = reinterpret_cast<float4*>(p.o_acc + b * p.acc_stride_b + h * p.acc_stride_h +
                                          static_cast<long long>(s) * p.acc_stride_s + c);
  float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
  if (!p.first) {
    a0 = acc[0];
    a1 = acc[1];
  }
  a0 = make_float4(a0.x * w_old + x[0] * w_new, a0.y * w_old + x[1] * w_new, a0.z * w_old + x[2] * w_new,
                   a0.w * w_old + x[3] * w_new);
  a1 = make_float4(a1.x * w_old + x[4] * w_new, a1.y * w_old + x[5] * w_new, a1.z * w_old + x[6] * w_new,
                   a1.w * w_old + x[7] * w_new);
  acc[0] = a0;
  acc[1] = a1;
  // every thread of a row computes the same lse_new; the one that owns column 0 stores it, after all
  // of the row's threads have read the old value (they sit in the same warp: 8 or 16 lanes per row)
  __syncwarp();
  if (c == 0) *lse_slot = lse_new;
}

}  // namespace sage
