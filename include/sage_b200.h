/* C ABI of the B200 (sm_100a) INT8 SageAttention path.
 *
 * This is the drop-in boundary under the `torch.ops.sageattention.*` operators of
 * LuXuxue/sageattention-rdna3: each entry point below replaces one launcher declared in the
 * reference's csrc/attn_gfx11.h and takes plain device pointers, sizes and element strides.
 * All pointers are device pointers on the CURRENT CUDA device unless stated otherwise; all work is
 * enqueued on `stream` (a cudaStream_t passed as void*) and nothing synchronises.
 *
 * Tensors in the caller's layout are described by `sage_strided_t`: a base pointer and the
 * element strides of the batch, head and sequence dimensions; head_dim is contiguous.  For the
 * reference's layouts, with x of shape [B,H,S,D] ("HND") pass (x.stride(0), x.stride(1),
 * x.stride(2)); with [B,S,H,D] ("NHD") pass (x.stride(0), x.stride(2), x.stride(1)).
 * Base pointers must be 16-byte aligned and strides multiples of 8 elements (16-byte vector
 * access, as the reference's kernels assume).
 *
 * Return value: 0 on success, a SAGE_ERR_* code otherwise; sage_last_error() describes the last
 * failure of the calling thread.
 */
#ifndef SAGE_B200_H_
#define SAGE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAGE_ABI_VERSION 7

#define SAGE_DTYPE_F16 0
#define SAGE_DTYPE_BF16 1

#define SAGE_OK 0
#define SAGE_ERR_INVALID 1   /* bad argument (shape, alignment, dtype, null pointer) */
#define SAGE_ERR_CUDA 2      /* a CUDA runtime / driver call failed                  */
#define SAGE_ERR_DEVICE 3    /* the device status word reported a kernel-side error  */

typedef struct sage_strided {
  const void* ptr;
  int64_t stride_b, stride_h, stride_s; /* in elements */
} sage_strided_t;

int sage_abi_version(void);
const char* sage_last_error(void);

/* The `status` word of the attention entry points (optional, a device int32 the caller zeroes):
 * the kernels write a non-zero code there when they had to give up (1 = shared memory misaligned,
 * 2 + 16*k = the bounded wait on barrier k ran out) and return instead of hanging; CTAs that start
 * while the word is already non-zero return at once, so a failed launch costs about one wait bound
 * and later launches do nothing until the caller has read and cleared the word.  With status ==
 * NULL such a failure goes unreported and the output is left partly unwritten.  The reference has
 * no counterpart (its launchers check nothing after the launch, csrc/attn_gfx11.cu:2069-2273).
 *
 * sage_set_status_mirror: a word in MAPPED PINNED HOST memory (cudaHostAlloc; the pointer must be
 * usable on the current device) that a failing attention kernel of the current device also writes
 * its code to, next to the `status` word of the call.  A host that never synchronises can poll it
 * between calls.  NULL switches the mirror off.  Kernels launched without a `status` word do not
 * write it.  No counterpart in the reference.
 *
 * Test hooks, for the failure-detection tests only (process-wide, not for production use; no
 * counterpart in the reference).  sage_test_set_wait_limit_us shortens the bound of every barrier
 * wait in the attention kernels (us <= 0 restores the default of about one second);
 * sage_test_drop_v_load(1) makes the TMA producer skip the V load of the first KV tile, so that a
 * wait runs out for real - it is honoured only while a shortened bound is set. */
int sage_set_status_mirror(int* host_word);
int sage_test_set_wait_limit_us(long long us);
int sage_test_drop_v_load(int on);

/* Launch schedule of the attention entry points that take a workspace: -1 = the library's cost
 * model decides between one CTA per query tile and persistent CTAs (default), 0 = never
 * persistent, 1 = always.  Process-wide; the environment variable SAGE_STREAMK=0|1, read once at
 * the first launch, sets the initial value.  Takes the place of the reference's per-launch
 * environment overrides of its tile choice (csrc/attn_gfx11.cu:2101-2114). */
int sage_set_streamk(int mode);

/* Mean of K over the sequence, per (batch, head, channel), in the input dtype.
 * Replaces mean_seq_gfx11 (csrc/attn_gfx11.h:48; csrc/attn_gfx11.cu:1937-1972, kernel :94-145):
 * same fp32 summation order (256 strided partial sums, added serially), one fp32 division, one
 * rounding.  mean_out: [B,H,D] contiguous, dtype as the input.  D must be 64 or 128. */
int sage_mean_seq(const sage_strided_t* k, int dtype, int B, int H, int S, int D, void* mean_out, void* stream);

/* Per-block INT8 quantisation of Q and K.
 * Replaces quant_qk_int8_gfx11 (csrc/attn_gfx11.h:41-46; csrc/attn_gfx11.cu:1974-2067, kernel
 * :147-321).  Q: groups of 32 rows, sm_scale*log2(e) folded in; K: groups of 16 rows, k_mean
 * ([B,Hkv,D], input dtype; may be NULL) subtracted in fp32 first.
 * Outputs: q_i8 [B,Hq,Sq,D], k_i8 [B,Hkv,Skv,D] (int8, contiguous), q_scale [B,Hq,ceil(Sq/32)],
 * k_scale [B,Hkv,ceil(Skv/16)] (fp32).
 * Sq == 0 or Skv == 0 quantises one side only (the pointers of the empty side are not looked
 * at): K once, Q per call, for keys that are reused.
 * If `v` and `v16` are both non-NULL the same launch also writes v16 = fp16(v), [B,Hkv,Skv,D]
 * contiguous: the dtype half of v_transpose_gfx11 (csrc/attn_gfx11.h:51; csrc/attn_gfx11.cu:377-381). */
int sage_quant_qk_int8(const sage_strided_t* q, const sage_strided_t* k, const void* k_mean,
                       const sage_strided_t* v, void* v16, int dtype, int B, int Hq, int Hkv, int Sq, int Skv,
                       int D, float sm_scale, int8_t* q_i8, float* q_scale, int8_t* k_i8, float* k_scale,
                       void* stream);

/* v16 = fp16(v), [B,H,S,D] contiguous.  The dtype half of v_transpose_gfx11
 * (csrc/attn_gfx11.h:51); the transpose itself is an RDNA3 layout detail with no counterpart here. */
int sage_v_to_f16(const sage_strided_t* v, int dtype, int B, int H, int S, int D, void* v16, void* stream);

/* Fused INT8 attention: O = softmax2(dequant(Q_i8 K_i8^T)) V.
 * Replaces qk_int8_sv_bf16_attn_gfx11_t (csrc/attn_gfx11.h:10-19; csrc/attn_gfx11.cu:2069-2273,
 * kernels :409-1243).  q_i8/k_i8/scales as produced by sage_quant_qk_int8; v16 is fp16 in any
 * strided layout; `o` has strides (o_stride_b, o_stride_h, o_stride_s) in elements and dtype
 * `out_dtype` (SAGE_DTYPE_*).  Hq must be a multiple of Hkv (GQA: hkv = hq / (Hq/Hkv)).
 * is_causal masks col > row (top-left aligned).
 * s_dump (optional, may be NULL): [B,Hq,Sq,Skv] int32, receives the raw Q_i8.K_i8^T products of
 * every KV tile the kernel visits (debug / parity aid, slow).
 * status (optional, may be NULL): one device int that the caller zeroes; it stays 0 unless the
 * kernel gave up on an internal wait or found its shared memory misaligned. */
int sage_qk_int8_sv_f16_attn(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o,
                             int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, const float* q_scale,
                             const float* k_scale, int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv, int D,
                             int is_causal, int32_t* s_dump, int* status, void* stream);

/* The same launch with the log-sum-exp of every query row written next to O.
 * The reference accepts return_lse but returns zeros (sageattention/core.py:203-211, "LSE not
 * computed by this kernel"); this entry point computes it, for callers that merge partial
 * attention results (ring / context parallelism).
 * lse (may be NULL: then this is sage_qk_int8_sv_f16_attn): [B,Hq,Sq] fp32, contiguous;
 * lse[b,h,i] = ln sum_j exp(sm_scale * q_i . k_j) over the visible keys of row i, computed from
 * the quantised scores (for K quantised with a mean subtracted it refers to the centred keys: add
 * sm_scale * q_i . mean to obtain the value for the original keys); -inf for a row with no
 * visible key. */
int sage_qk_int8_sv_f16_attn_lse(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o,
                                 int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, const float* q_scale,
                                 const float* k_scale, int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv,
                                 int D, int is_causal, float* lse, int32_t* s_dump, int* status, void* stream);

/* Persistent scheduling for problems that do not fill the GPU evenly.
 * No counterpart in the reference.  sage_qk_int8_sv_f16_attn gives every thread block one whole
 * 128-row query tile; a B200 runs 296 of them at a time, so 320 tiles (B=1, H=10, S=4096) take two
 * rounds.  Given a workspace, the _ws entry points cut the work into 296 equal spans of KV-tile
 * steps instead, keep partial results (fp32) in the workspace and merge them with a second small
 * kernel; they fall back to the plain launch when that would not pay, when the workspace is NULL
 * or too small, or when s_dump is set.  Results agree with the plain launch to fp32 rounding of
 * the merge (same int8 products, same softmax).
 * sage_attn_workspace_bytes: bytes the _ws calls want for this problem on the current device, 0 if
 * they would use the plain launch anyway.  The workspace needs no initialisation and may be
 * reused by the next call on the same stream. */
int64_t sage_attn_workspace_bytes(int B, int Hq, int Sq, int Skv, int D, int is_causal);
int sage_qk_int8_sv_f16_attn_ws(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o,
                                int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, const float* q_scale,
                                const float* k_scale, int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv,
                                int D, int is_causal, float* lse, int32_t* s_dump, int* status, void* workspace,
                                int64_t workspace_bytes, void* stream);

/* Attention whose output is also scattered to the other GPUs of the node, for the all-gather that
 * follows when (batch, kv-head) units are sharded over GPUs.
 * No counterpart in the reference (single GPU).  As sage_qk_int8_sv_f16_attn_lse, and every finished
 * 32-row piece of the output is written, with ordinary 16-byte stores from the epilogue, to n_peers
 * (0..SAGE_MAX_PEERS) further buffers peer_o[i] as well: device addresses, normally in the memory of
 * other GPUs (sage_peer_open), each with the layout and strides of `o` - the caller passes the
 * address of THIS rank's slice inside every peer's copy of the gathered output.  The transfer thus
 * runs under the computation, tile by tile.  The stores are complete when the launch is (stream
 * order); the peers learn of that through whatever cross-rank synchronisation the caller uses after
 * it (an all-reduce of one element is enough).  Always the plain launch; no s_dump. */
#define SAGE_MAX_PEERS 15
int sage_qk_int8_sv_f16_attn_scatter(const int8_t* q_i8, const int8_t* k_i8, const sage_strided_t* v16, void* o,
                                     int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, const float* q_scale,
                                     const float* k_scale, int out_dtype, int B, int Hq, int Hkv, int Sq, int Skv,
                                     int D, int is_causal, float* lse, int* status, int n_peers, void* const* peer_o,
                                     void* stream);

/* The same for the un-quantised kernel (sage_direct_attn). */
int sage_direct_attn_scatter(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v16, void* o,
                             int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int dtype, int B, int Hq,
                             int Hkv, int Sq, int Skv, int D, int is_causal, float sm_scale, float* lse, int* status,
                             int n_peers, void* const* peer_o, void* stream);

/* Mapping of a device buffer that another process of the node owns (one process per GPU).
 * No counterpart in the reference.  sage_peer_export, in the owner: the 64-byte CUDA IPC handle of the
 * allocation that contains `ptr` (memory from cudaMalloc, which is what PyTorch's default allocator
 * hands out) and the offset of `ptr` in it.  sage_peer_open, in another process with its own GPU
 * current: maps the allocation and returns the address that corresponds to `ptr`; peer access from
 * the current device is enabled by the call.  sage_peer_close undoes one open. */
int sage_peer_export(const void* ptr, unsigned char handle[64], int64_t* offset);
int sage_peer_open(const unsigned char handle[64], int64_t offset, void** mapped);
int sage_peer_close(void* mapped, int64_t offset);

/* Un-quantised attention for short sequences: O = softmax2(sm_scale*log2(e) * Q K^T) V with Q and K
 * in fp16 or bf16 as the caller holds them.
 * Replaces fp16_attn_gfx11_t / bf16_attn_gfx11_t (csrc/attn_gfx11.h:21-39; csrc/attn_gfx11.cu:2275-2472,
 * kernel direct_attn_kernel_impl_t :1468-1846), the branch the reference's sageattn takes when the
 * quantisation launches would cost more than INT8 saves (sageattention/core.py:113-163).  Same
 * arithmetic as there: fp32 accumulation of the 16-bit products, scores scaled by
 * sm_scale*1.4426950408889634 in fp32, causal / length mask, base-2 online softmax, P in fp16,
 * V in fp16, fp32 accumulation, one rounding of acc/l.
 * q, k: strided views, dtype `dtype` (SAGE_DTYPE_*); v16: fp16 in any strided layout (for bf16
 * inputs run sage_v_to_f16 first, as the reference converts inside v_transpose); o: dtype `dtype`.
 * lse, status: as for sage_qk_int8_sv_f16_attn_lse (both may be NULL). */
int sage_direct_attn(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v16, void* o,
                     int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int dtype, int B, int Hq, int Hkv,
                     int Sq, int Skv, int D, int is_causal, float sm_scale, float* lse, int* status, void* stream);

/* sage_direct_attn with a workspace for persistent scheduling (see sage_attn_workspace_bytes). */
int sage_direct_attn_ws(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v16, void* o,
                        int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int dtype, int B, int Hq, int Hkv,
                        int Sq, int Skv, int D, int is_causal, float sm_scale, float* lse, int* status,
                        void* workspace, int64_t workspace_bytes, void* stream);

/* smooth_k preparation in ONE launch: the K mean, K quantised against it, Q quantised, and (if `v` and
 * `v16` are non-NULL) the fp16 copy of V.  Replaces the sequence mean_seq_gfx11 -> quant_qk_int8_gfx11
 * (-> v_transpose_gfx11) that sageattention/core.py:186-193 issues for smooth_k=True
 * (csrc/attn_gfx11.h:41-48; kernels csrc/attn_gfx11.cu:94-145, :147-321): same arithmetic and summation
 * order, bit-identical outputs, but K is read from DRAM once - the cluster of CTAs that has summed a
 * (batch, kv-head) quantises it while it is still in L2.  k_mean_out: [B,Hkv,D], input dtype.
 * Skv must be >= 1; other arguments as for sage_quant_qk_int8. */
int sage_prep_smooth_qkv(const sage_strided_t* q, const sage_strided_t* k, const sage_strided_t* v, void* v16, int dtype,
                         int B, int Hq, int Hkv, int Sq, int Skv, int D, float sm_scale, int8_t* q_i8, float* q_scale,
                         int8_t* k_i8, float* k_scale, void* k_mean_out, void* stream);
/* 1 if sage_prep_smooth_qkv is the faster way to prepare B * Hkv (batch, kv-head) pairs on the current
 * device, 0 if sage_mean_seq followed by sage_quant_qk_int8 is (many heads: measured on B200, the
 * one-launch form wins up to about SMs / 8 pairs).  Same results either way.  No counterpart in the
 * reference (its launch sequence is fixed, sageattention/core.py:186-193). */
int sage_prep_smooth_preferred(int B, int Hkv);

/* Smooth-K quantisation for callers that must not allocate device memory.
 * No counterpart in the reference (its launchers allocate through torch).
 *
 * Who this is for: hosts in which a device allocation at call time is off limits - an inference
 * engine that sized all of its memory when it started and treats a later cudaMalloc as a bug, a
 * plugin whose host owns the only allocator and does not lend it out, a latency-critical loop that
 * cannot take the driver lock and implicit device-wide synchronisation of cudaMalloc / cudaFree.
 * sage_quant_qk_int8 with smooth_k needs one intermediate, the per-channel mean of K
 * ([B,Hkv,D] in the input dtype); the other entry points leave it to the caller to allocate.  This
 * one keeps it in a fixed buffer that is part of the library image, so the caller passes only the
 * inputs (q, k) and the outputs (q_i8, q_scale, k_i8, k_scale), exactly as for
 * sage_quant_qk_int8; the results are bit-identical to sage_mean_seq + sage_quant_qk_int8.
 *
 * Limit: B * Hkv * D <= SAGE_STATIC_KMEAN_MAX_ELEMS (65536 elements = 128 KB; every GPU on which
 * the library is used holds that buffer until the process exits).  Larger problems are refused with
 * SAGE_ERR_INVALID and a message; Skv must be >= 1.
 * The function calls no cudaMalloc / cudaFree and no allocating library routine.  The first call
 * on each device looks up the buffer's device address (cudaGetSymbolAddress); make that first call
 * outside of any stream capture.
 * The buffer is shared by all calls and keeps the last call's contents.  Nothing in it has to start
 * at zero: the mean kernel overwrites every element the quantisation reads.  Two calls that may
 * overlap on the GPU (different streams, or different host threads without ordering) race on it:
 * order them with events or use the allocating entry points. */
#define SAGE_STATIC_KMEAN_MAX_ELEMS 65536
int sage_quant_qk_int8_smooth_static(const sage_strided_t* q, const sage_strided_t* k, int dtype, int B, int Hq,
                                     int Hkv, int Sq, int Skv, int D, float sm_scale, int8_t* q_i8, float* q_scale,
                                     int8_t* k_i8, float* k_scale, void* stream);

/* Fold one partial attention result into running accumulators - the merge step of attention over a
 * sequence that is split across GPUs (each partial covers a disjoint set of keys):
 *   lse' = log(exp(lse) + exp(lse_j)),  o' = o * exp(lse - lse') + o_j * exp(lse_j - lse').
 * o_acc: fp32 [B,H,S,D] described by element strides (32-byte aligned base); lse_acc: fp32 rows of
 * length S at lse_acc + b * lse_stride_b + h * lse_stride_h; o_part: the partial output (f16 / bf16)
 * as the attention entry points write it; lse_part: fp32 [B,H,S] contiguous, as they return it.
 * first != 0: the accumulators are overwritten instead of read.  No counterpart in the reference,
 * whose `return_lse` is a placeholder (sageattention/core.py:203-211). */
int sage_fold_attn_partial(const sage_strided_t* o_acc, float* lse_acc, int64_t lse_stride_b, int64_t lse_stride_h,
                           const sage_strided_t* o_part, int part_dtype, const float* lse_part, int B, int H, int S, int D,
                           int first, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SAGE_B200_H_ */
