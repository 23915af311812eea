// torch.ops.sageattention.* for B200: a thin wrapper that turns tensors into the pointers, sizes
// and strides of the C ABI (include/sage_b200.h).  It takes the place of the reference's
// csrc/pybind_gfx11.cpp (op schemas :18-38, CUDA registrations :40-47) and of the host launchers
// declared in csrc/attn_gfx11.h.  `tensor_layout`: 0 = NHD [B,S,H,D], 1 = HND [B,H,S,D]
// (csrc/attn_gfx11.cu:32-33).
#include <Python.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include <cuda_runtime.h>

#include <vector>

#include "../../include/sage_b200.h"

namespace {

constexpr int64_t kNHD = 0;
constexpr int64_t kHND = 1;

struct Dims {
  int64_t B, H, S, D;
};

Dims dims_of(const at::Tensor& t, int64_t layout) {
  TORCH_CHECK(t.dim() == 4, "expected a 4-D tensor, got ", t.dim(), "-D");
  TORCH_CHECK(layout == kNHD || layout == kHND, "tensor_layout must be 0 (NHD) or 1 (HND)");
  if (layout == kHND) return {t.size(0), t.size(1), t.size(2), t.size(3)};
  return {t.size(0), t.size(2), t.size(1), t.size(3)};
}

sage_strided_t strided_of(const at::Tensor& t, int64_t layout) {
  sage_strided_t s;
  s.ptr = t.data_ptr();
  s.stride_b = t.stride(0);
  s.stride_h = (layout == kHND) ? t.stride(1) : t.stride(2);
  s.stride_s = (layout == kHND) ? t.stride(2) : t.stride(1);
  return s;
}

int dtype_code(const at::Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kHalf || t.scalar_type() == at::kBFloat16,
              "expected an fp16 or bf16 tensor, got ", t.scalar_type());
  return t.scalar_type() == at::kHalf ? SAGE_DTYPE_F16 : SAGE_DTYPE_BF16;
}

void check_16b(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.stride(-1) == 1, name, ": last dim must be contiguous");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0 && t.stride(0) % 8 == 0 && t.stride(1) % 8 == 0 &&
                  t.stride(2) % 8 == 0,
              name, " needs a 16-byte aligned base and strides that are multiples of 8 elements; got strides ",
              t.strides(), ". Use a contiguous tensor.");
}

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == SAGE_OK, what, " failed: ", sage_last_error());
}

void* current_stream(const at::Tensor& t) {
  return static_cast<void*>(at::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

// mean_seq(Tensor input, int tensor_layout) -> Tensor        (csrc/pybind_gfx11.cpp:36)
at::Tensor mean_seq(const at::Tensor& input, int64_t layout) {
  check_16b(input, "input");
  const Dims d = dims_of(input, layout);
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor out = at::empty({d.B, d.H, d.D}, input.options());
  const sage_strided_t k = strided_of(input, layout);
  check_rc(sage_mean_seq(&k, dtype_code(input), (int)d.B, (int)d.H, (int)d.S, (int)d.D, out.data_ptr(),
                         current_stream(input)),
           "mean_seq");
  return out;
}

// Shared body of quant_qk_int8 and prep_qkv.
std::vector<at::Tensor> quant_impl(const at::Tensor& q, const at::Tensor& k, const at::Tensor& k_mean,
                                   const at::Tensor* v, int64_t layout, double sm_scale) {
  check_16b(q, "query");
  check_16b(k, "key");
  TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.device() == k.device(), "query/key dtype or device mismatch");
  const Dims dq = dims_of(q, layout), dk = dims_of(k, layout);
  TORCH_CHECK(dq.B == dk.B && dq.D == dk.D, "query/key batch or head_dim mismatch");
  TORCH_CHECK(dq.D == 64 || dq.D == 128, "head_dim must be 64 or 128, got ", dq.D);
  c10::cuda::CUDAGuard guard(q.device());
  const auto i8 = q.options().dtype(at::kChar);
  const auto f32 = q.options().dtype(at::kFloat);
  at::Tensor q_i8 = at::empty({dq.B, dq.H, dq.S, dq.D}, i8);
  at::Tensor k_i8 = at::empty({dk.B, dk.H, dk.S, dk.D}, i8);
  at::Tensor q_scale = at::empty({dq.B, dq.H, (dq.S + 31) / 32}, f32);
  at::Tensor k_scale = at::empty({dk.B, dk.H, (dk.S + 15) / 16}, f32);
  const void* mean_ptr = nullptr;
  if (k_mean.numel() > 0) {
    TORCH_CHECK(k_mean.is_contiguous() && k_mean.numel() == dk.B * dk.H * dk.D && k_mean.scalar_type() == k.scalar_type(),
                "key_mean must be a contiguous [B,Hkv,D] tensor of the input dtype");
    mean_ptr = k_mean.data_ptr();
  }
  const sage_strided_t qs = strided_of(q, layout), ks = strided_of(k, layout);
  sage_strided_t vs;
  at::Tensor v16;
  const bool convert_v = (v != nullptr);
  if (convert_v) {
    check_16b(*v, "value");
    const Dims dv = dims_of(*v, layout);
    TORCH_CHECK(dv.B == dk.B && dv.H == dk.H && dv.S == dk.S && dv.D == dk.D, "key/value shape mismatch");
    TORCH_CHECK(v->scalar_type() == k.scalar_type(), "key/value dtype mismatch");
    v16 = at::empty({dk.B, dk.H, dk.S, dk.D}, q.options().dtype(at::kHalf));
    vs = strided_of(*v, layout);
  }
  if (dq.S > 0 || dk.S > 0) {
    check_rc(sage_quant_qk_int8(&qs, &ks, mean_ptr, convert_v ? &vs : nullptr, convert_v ? v16.data_ptr() : nullptr,
                                dtype_code(q), (int)dq.B, (int)dq.H, (int)dk.H, (int)dq.S, (int)dk.S, (int)dq.D,
                                static_cast<float>(sm_scale), q_i8.data_ptr<int8_t>(), q_scale.data_ptr<float>(),
                                k_i8.data_ptr<int8_t>(), k_scale.data_ptr<float>(), current_stream(q)),
             "quant_qk_int8");
  }
  std::vector<at::Tensor> out{q_i8, q_scale, k_i8, k_scale};
  if (convert_v) out.push_back(v16);
  return out;
}

// quant_qk_int8(Tensor query, Tensor key, Tensor key_mean, int tensor_layout, float sm_scale) -> Tensor[]
// (csrc/pybind_gfx11.cpp:32-35).  Returns [q_int8, q_scale, k_int8, k_scale].
std::vector<at::Tensor> quant_qk_int8(const at::Tensor& q, const at::Tensor& k, const at::Tensor& k_mean,
                                      int64_t layout, double sm_scale) {
  return quant_impl(q, k, k_mean, nullptr, layout, sm_scale);
}

// prep_qkv: quant_qk_int8 plus the fp16 copy of V in the same launch.
// Returns [q_int8, q_scale, k_int8, k_scale, v_fp16 ([B,Hkv,Skv,D] contiguous)].
std::vector<at::Tensor> prep_qkv(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                 const at::Tensor& k_mean, int64_t layout, double sm_scale) {
  return quant_impl(q, k, k_mean, &v, layout, sm_scale);
}

// prep_smooth_qkv(Tensor query, Tensor key, Tensor? value, int tensor_layout, float sm_scale) -> Tensor[]
// smooth_k in one launch: what mean_seq followed by quant_qk_int8 / prep_qkv computes (the sequence of
// sageattention/core.py:186-193), with K read from DRAM once.  Returns [q_int8, q_scale, k_int8,
// k_scale, key_mean] and, if `value` is given, its fp16 copy [B,Hkv,Skv,D] as a sixth tensor.
std::vector<at::Tensor> prep_smooth_qkv(const at::Tensor& q, const at::Tensor& k, const c10::optional<at::Tensor>& v,
                                        int64_t layout, double sm_scale) {
  check_16b(q, "query");
  check_16b(k, "key");
  TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.device() == k.device(), "query/key dtype or device mismatch");
  const Dims dq = dims_of(q, layout), dk = dims_of(k, layout);
  TORCH_CHECK(dq.B == dk.B && dq.D == dk.D, "query/key batch or head_dim mismatch");
  TORCH_CHECK(dq.D == 64 || dq.D == 128, "head_dim must be 64 or 128, got ", dq.D);
  TORCH_CHECK(dk.S >= 1 && dk.B >= 1 && dk.H >= 1 && dq.H >= 1, "prep_smooth_qkv needs at least one key");
  c10::cuda::CUDAGuard guard(q.device());
  const auto i8 = q.options().dtype(at::kChar);
  const auto f32 = q.options().dtype(at::kFloat);
  at::Tensor q_i8 = at::empty({dq.B, dq.H, dq.S, dq.D}, i8);
  at::Tensor k_i8 = at::empty({dk.B, dk.H, dk.S, dk.D}, i8);
  at::Tensor q_scale = at::empty({dq.B, dq.H, (dq.S + 31) / 32}, f32);
  at::Tensor k_scale = at::empty({dk.B, dk.H, (dk.S + 15) / 16}, f32);
  at::Tensor k_mean = at::empty({dk.B, dk.H, dk.D}, k.options());
  const sage_strided_t qs = strided_of(q, layout), ks = strided_of(k, layout);
  sage_strided_t vs;
  at::Tensor v16;
  const bool convert_v = v.has_value();
  if (convert_v) {
    check_16b(*v, "value");
    const Dims dv = dims_of(*v, layout);
    TORCH_CHECK(dv.B == dk.B && dv.H == dk.H && dv.S == dk.S && dv.D == dk.D, "key/value shape mismatch");
    TORCH_CHECK(v->scalar_type() == k.scalar_type(), "key/value dtype mismatch");
    v16 = at::empty({dk.B, dk.H, dk.S, dk.D}, q.options().dtype(at::kHalf));
    vs = strided_of(*v, layout);
  }
  check_rc(sage_prep_smooth_qkv(&qs, &ks, convert_v ? &vs : nullptr, convert_v ? v16.data_ptr() : nullptr, dtype_code(q),
                                (int)dq.B, (int)dq.H, (int)dk.H, (int)dq.S, (int)dk.S, (int)dq.D,
                                static_cast<float>(sm_scale), q_i8.data_ptr<int8_t>(), q_scale.data_ptr<float>(),
                                k_i8.data_ptr<int8_t>(), k_scale.data_ptr<float>(), k_mean.data_ptr(), current_stream(q)),
           "prep_smooth_qkv");
  std::vector<at::Tensor> out{q_i8, q_scale, k_i8, k_scale, k_mean};
  if (convert_v) out.push_back(v16);
  return out;
}

// v_to_f16(Tensor value, int tensor_layout) -> Tensor: the dtype half of the reference's
// v_transpose (csrc/pybind_gfx11.cpp:37); output is [B,H,S,D] contiguous fp16.
at::Tensor v_to_f16(const at::Tensor& v, int64_t layout) {
  check_16b(v, "value");
  const Dims d = dims_of(v, layout);
  c10::cuda::CUDAGuard guard(v.device());
  at::Tensor out = at::empty({d.B, d.H, d.S, d.D}, v.options().dtype(at::kHalf));
  if (out.numel() == 0) return out;
  const sage_strided_t vs = strided_of(v, layout);
  check_rc(sage_v_to_f16(&vs, dtype_code(v), (int)d.B, (int)d.H, (int)d.S, (int)d.D, out.data_ptr(), current_stream(v)),
           "v_to_f16");
  return out;
}

// qk_int8_sv_f16_attn(Tensor query, Tensor key, Tensor value, Tensor(a!) output, Tensor q_scale,
//                     Tensor k_scale, int tensor_layout, int is_causal, float sm_scale, *,
//                     int value_layout=-1, Tensor? s_dump, Tensor? status, Tensor? lse,
//                     int[]? peer_ptrs) -> Tensor
// Counterpart of qk_int8_sv_bf16_attn_t (csrc/pybind_gfx11.cpp:19-23), call-compatible with its nine
// positional arguments: query/key are the int8 [B,H,S,D] tensors from quant_qk_int8; `value` is fp16
// in `value_layout` (keyword; -1 = the same as `tensor_layout`); `output` is fp16/bf16 in
// `tensor_layout`.  sm_scale is already folded into q_scale and is accepted for signature parity.
// `lse` (optional, fp32 [B,Hq,Sq]) receives the natural-log sum of exponentials of every row.
// `peer_ptrs` (optional): device addresses of further copies of `output` (same layout and strides,
// normally in other GPUs' memory) that the kernel writes as well (sage_qk_int8_sv_f16_attn_scatter).
at::Tensor qk_int8_sv_f16_attn(const at::Tensor& q_i8, const at::Tensor& k_i8, const at::Tensor& v, at::Tensor& o,
                               const at::Tensor& q_scale, const at::Tensor& k_scale, int64_t layout,
                               int64_t is_causal, double /*sm_scale*/, int64_t value_layout,
                               const c10::optional<at::Tensor>& s_dump, const c10::optional<at::Tensor>& status,
                               const c10::optional<at::Tensor>& lse, at::OptionalIntArrayRef peer_ptrs) {
  TORCH_CHECK(q_i8.is_cuda() && q_i8.scalar_type() == at::kChar && q_i8.is_contiguous() && q_i8.dim() == 4,
              "query must be a contiguous int8 CUDA tensor [B,Hq,Sq,D]");
  TORCH_CHECK(k_i8.scalar_type() == at::kChar && k_i8.is_contiguous() && k_i8.dim() == 4,
              "key must be a contiguous int8 tensor [B,Hkv,Skv,D]");
  TORCH_CHECK(v.scalar_type() == at::kHalf, "value must be fp16 (convert bf16 with v_to_f16 / prep_qkv)");
  check_16b(v, "value");
  check_16b(o, "output");
  if (value_layout < 0) value_layout = layout;
  const int64_t B = q_i8.size(0), Hq = q_i8.size(1), Sq = q_i8.size(2), D = q_i8.size(3);
  const int64_t Hkv = k_i8.size(1), Skv = k_i8.size(2);
  const Dims dv = dims_of(v, value_layout), d_o = dims_of(o, layout);
  TORCH_CHECK(k_i8.size(0) == B && k_i8.size(3) == D, "query/key batch or head_dim mismatch");
  TORCH_CHECK(dv.B == B && dv.H == Hkv && dv.S == Skv && dv.D == D, "value shape does not match key");
  TORCH_CHECK(d_o.B == B && d_o.H == Hq && d_o.S == Sq && d_o.D == D, "output shape does not match query");
  TORCH_CHECK(D == 64 || D == 128, "head_dim must be 64 or 128, got ", D);
  TORCH_CHECK(Hq % Hkv == 0, "num_qo_heads must be a multiple of num_kv_heads");
  TORCH_CHECK(q_scale.scalar_type() == at::kFloat && q_scale.is_contiguous() && q_scale.numel() == B * Hq * ((Sq + 31) / 32),
              "q_scale must be a contiguous fp32 [B,Hq,ceil(Sq/32)] tensor");
  TORCH_CHECK(k_scale.scalar_type() == at::kFloat && k_scale.is_contiguous() && k_scale.numel() == B * Hkv * ((Skv + 15) / 16),
              "k_scale must be a contiguous fp32 [B,Hkv,ceil(Skv/16)] tensor");
  int32_t* dump_ptr = nullptr;
  if (s_dump.has_value()) {
    TORCH_CHECK(s_dump->scalar_type() == at::kInt && s_dump->is_contiguous() && s_dump->numel() == B * Hq * Sq * Skv,
                "s_dump must be a contiguous int32 [B,Hq,Sq,Skv] tensor");
    dump_ptr = s_dump->data_ptr<int32_t>();
  }
  int* status_ptr = nullptr;
  if (status.has_value()) {
    TORCH_CHECK(status->scalar_type() == at::kInt && status->numel() >= 1 && status->is_cuda(), "status must be an int32 CUDA tensor");
    status_ptr = status->data_ptr<int>();
  }
  float* lse_ptr = nullptr;
  if (lse.has_value()) {
    TORCH_CHECK(lse->scalar_type() == at::kFloat && lse->is_contiguous() && lse->numel() == B * Hq * Sq && lse->is_cuda(),
                "lse must be a contiguous fp32 CUDA tensor [B,Hq,Sq]");
    lse_ptr = lse->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(q_i8.device());
  const sage_strided_t vs = strided_of(v, value_layout);
  const sage_strided_t os = strided_of(o, layout);
  if (peer_ptrs.has_value() && !peer_ptrs->empty()) {
    TORCH_CHECK(!dump_ptr, "peer_ptrs and s_dump cannot be combined");
    std::vector<void*> peers;
    for (int64_t a : *peer_ptrs) peers.push_back(reinterpret_cast<void*>(static_cast<uintptr_t>(a)));
    check_rc(sage_qk_int8_sv_f16_attn_scatter(q_i8.data_ptr<int8_t>(), k_i8.data_ptr<int8_t>(), &vs, o.data_ptr(),
                                              os.stride_b, os.stride_h, os.stride_s, q_scale.data_ptr<float>(),
                                              k_scale.data_ptr<float>(), dtype_code(o), (int)B, (int)Hq, (int)Hkv,
                                              (int)Sq, (int)Skv, (int)D, (int)is_causal, lse_ptr, status_ptr,
                                              (int)peers.size(), peers.data(), current_stream(q_i8)),
             "qk_int8_sv_f16_attn");
    return o;
  }
  // Problems that would fill the GPU unevenly run on persistent CTAs and need scratch for partial results.
  at::Tensor workspace;
  const int64_t ws_bytes = dump_ptr ? 0 : sage_attn_workspace_bytes((int)B, (int)Hq, (int)Sq, (int)Skv, (int)D, (int)is_causal);
  if (ws_bytes > 0) workspace = at::empty({ws_bytes}, q_i8.options().dtype(at::kByte));
  check_rc(sage_qk_int8_sv_f16_attn_ws(q_i8.data_ptr<int8_t>(), k_i8.data_ptr<int8_t>(), &vs, o.data_ptr(), os.stride_b,
                                       os.stride_h, os.stride_s, q_scale.data_ptr<float>(),
                                       k_scale.data_ptr<float>(), dtype_code(o), (int)B, (int)Hq, (int)Hkv, (int)Sq,
                                       (int)Skv, (int)D, (int)is_causal, lse_ptr, dump_ptr, status_ptr,
                                       ws_bytes > 0 ? workspace.data_ptr() : nullptr, ws_bytes, current_stream(q_i8)),
           "qk_int8_sv_f16_attn");
  return o;
}

// fp16_attn / bf16_attn(Tensor query, Tensor key, Tensor value, Tensor(a!) output, int tensor_layout,
//                       int value_layout, int is_causal, float sm_scale, int bm_sel, Tensor? status,
//                       Tensor? lse) -> Tensor
// Counterparts of fp16_attn_t / bf16_attn_t (csrc/pybind_gfx11.cpp:24-31): the un-quantised kernel
// for short sequences.  query/key are fp16 (fp16_attn) or bf16 (bf16_attn) in `tensor_layout`;
// `value` is fp16 [..,S,D] in `value_layout` (the reference passes the transposed fp16 V_T);
// `bm_sel` picked a tile height on RDNA3 and is accepted and ignored.
at::Tensor direct_attn(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& o, int64_t layout,
                       int64_t value_layout, int64_t is_causal, double sm_scale, int64_t /*bm_sel*/,
                       const c10::optional<at::Tensor>& status, const c10::optional<at::Tensor>& lse,
                       at::ScalarType want, const char* name, at::OptionalIntArrayRef peer_ptrs = c10::nullopt) {
  TORCH_CHECK(q.scalar_type() == want && k.scalar_type() == want && o.scalar_type() == want, name,
              ": query, key and output must be ", want);
  TORCH_CHECK(v.scalar_type() == at::kHalf, name, ": value must be fp16 (convert bf16 with v_to_f16)");
  check_16b(q, "query");
  check_16b(k, "key");
  check_16b(v, "value");
  check_16b(o, "output");
  const Dims dq = dims_of(q, layout), dk = dims_of(k, layout), dv = dims_of(v, value_layout), d_o = dims_of(o, layout);
  TORCH_CHECK(dk.B == dq.B && dk.D == dq.D, "query/key batch or head_dim mismatch");
  TORCH_CHECK(dv.B == dk.B && dv.H == dk.H && dv.S == dk.S && dv.D == dk.D, "value shape does not match key");
  TORCH_CHECK(d_o.B == dq.B && d_o.H == dq.H && d_o.S == dq.S && d_o.D == dq.D, "output shape does not match query");
  TORCH_CHECK(dq.D == 64 || dq.D == 128, "head_dim must be 64 or 128, got ", dq.D);
  TORCH_CHECK(dk.H > 0 && dq.H % dk.H == 0, "num_qo_heads must be a multiple of num_kv_heads");
  int* status_ptr = nullptr;
  if (status.has_value()) {
    TORCH_CHECK(status->scalar_type() == at::kInt && status->numel() >= 1 && status->is_cuda(), "status must be an int32 CUDA tensor");
    status_ptr = status->data_ptr<int>();
  }
  float* lse_ptr = nullptr;
  if (lse.has_value()) {
    TORCH_CHECK(lse->scalar_type() == at::kFloat && lse->is_contiguous() && lse->numel() == dq.B * dq.H * dq.S && lse->is_cuda(),
                "lse must be a contiguous fp32 CUDA tensor [B,Hq,Sq]");
    lse_ptr = lse->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(q.device());
  const sage_strided_t qs = strided_of(q, layout), ks = strided_of(k, layout), vs = strided_of(v, value_layout);
  const sage_strided_t os = strided_of(o, layout);
  if (peer_ptrs.has_value() && !peer_ptrs->empty()) {
    std::vector<void*> peers;
    for (int64_t a : *peer_ptrs) peers.push_back(reinterpret_cast<void*>(static_cast<uintptr_t>(a)));
    check_rc(sage_direct_attn_scatter(&qs, &ks, &vs, o.data_ptr(), os.stride_b, os.stride_h, os.stride_s, dtype_code(q),
                                      (int)dq.B, (int)dq.H, (int)dk.H, (int)dq.S, (int)dk.S, (int)dq.D, (int)is_causal,
                                      (float)sm_scale, lse_ptr, status_ptr, (int)peers.size(), peers.data(),
                                      current_stream(q)),
             name);
    return o;
  }
  at::Tensor workspace;
  const int64_t ws_bytes = sage_attn_workspace_bytes((int)dq.B, (int)dq.H, (int)dq.S, (int)dk.S, (int)dq.D, (int)is_causal);
  if (ws_bytes > 0) workspace = at::empty({ws_bytes}, q.options().dtype(at::kByte));
  check_rc(sage_direct_attn_ws(&qs, &ks, &vs, o.data_ptr(), os.stride_b, os.stride_h, os.stride_s, dtype_code(q),
                               (int)dq.B, (int)dq.H, (int)dk.H, (int)dq.S, (int)dk.S, (int)dq.D, (int)is_causal,
                               (float)sm_scale, lse_ptr, status_ptr, ws_bytes > 0 ? workspace.data_ptr() : nullptr,
                               ws_bytes, current_stream(q)),
           name);
  return o;
}
at::Tensor fp16_attn(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& o, int64_t layout,
                     int64_t value_layout, int64_t is_causal, double sm_scale, int64_t bm_sel,
                     const c10::optional<at::Tensor>& status, const c10::optional<at::Tensor>& lse) {
  return direct_attn(q, k, v, o, layout, value_layout, is_causal, sm_scale, bm_sel, status, lse, at::kHalf, "fp16_attn");
}
at::Tensor bf16_attn(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& o, int64_t layout,
                     int64_t value_layout, int64_t is_causal, double sm_scale, int64_t bm_sel,
                     const c10::optional<at::Tensor>& status, const c10::optional<at::Tensor>& lse) {
  return direct_attn(q, k, v, o, layout, value_layout, is_causal, sm_scale, bm_sel, status, lse, at::kBFloat16,
                     "bf16_attn");
}

// sageattn_fwd(Tensor query, Tensor key, Tensor value, int tensor_layout, int is_causal, float sm_scale,
//              int smooth_k, int use_direct, Tensor status, Tensor? lse, Tensor? out, int[]? peer_ptrs) -> Tensor[]
// The whole of the reference's sageattn body after its assertions (sageattention/core.py:96-201) in
// one operator call: allocate the output, then either the un-quantised branch (:141-163: fp16 V,
// fp16_attn / bf16_attn) or the INT8 branch (:165-198: [mean,] quantise, attention).  Returns
// [output] or, with smooth_k on the INT8 branch, [output, key_mean] (the caller needs the mean to
// refer a log-sum-exp to the original keys).  One Python -> C++ crossing instead of two to four.
std::vector<at::Tensor> sageattn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, int64_t layout,
                                     int64_t is_causal, double sm_scale, int64_t smooth_k, int64_t use_direct,
                                     const at::Tensor& status, const c10::optional<at::Tensor>& lse,
                                     const c10::optional<at::Tensor>& out, at::OptionalIntArrayRef peer_ptrs) {
  at::Tensor o;
  if (out.has_value()) {
    TORCH_CHECK(out->sizes() == q.sizes() && out->scalar_type() == q.scalar_type() && out->device() == q.device(),
                "out must have the shape, dtype and device of query");
    o = *out;
  } else {
    o = at::empty_like(q);
  }

  const bool bf16 = q.scalar_type() == at::kBFloat16;
  const c10::optional<at::Tensor> st(status), none;
  if (use_direct) {
    if (bf16) {
      direct_attn(q, k, v_to_f16(v, layout), o, layout, kHND, is_causal, sm_scale, 0, st, lse, at::kBFloat16, "bf16_attn",
                  peer_ptrs);
    } else {
      direct_attn(q, k, v, o, layout, layout, is_causal, sm_scale, 0, st, lse, at::kHalf, "fp16_attn", peer_ptrs);
    }
    return {o};
  }
  const Dims dk_all = dims_of(k, layout);
  c10::cuda::CUDAGuard guard(q.device());
  if (smooth_k && sage_prep_smooth_preferred((int)dk_all.B, (int)dk_all.H)) {
    // few heads: one launch for the mean and the quantisation against it
    std::vector<at::Tensor> parts =
        prep_smooth_qkv(q, k, bf16 ? c10::optional<at::Tensor>(v) : c10::optional<at::Tensor>(), layout, sm_scale);
    qk_int8_sv_f16_attn(parts[0], parts[2], bf16 ? parts[5] : v, o, parts[1], parts[3], layout, is_causal, sm_scale,
                        bf16 ? kHND : layout, none, st, lse, peer_ptrs);
    return {o, parts[4]};
  }
  at::Tensor k_mean = smooth_k ? mean_seq(k, layout) : at::empty({0}, q.options());
  std::vector<at::Tensor> parts = quant_impl(q, k, k_mean, bf16 ? &v : nullptr, layout, sm_scale);
  qk_int8_sv_f16_attn(parts[0], parts[2], bf16 ? parts[4] : v, o, parts[1], parts[3], layout, is_causal, sm_scale,
                      bf16 ? kHND : layout, none, st, lse, peer_ptrs);
  if (smooth_k) return {o, k_mean};
  return {o};
}

// fold_partial(Tensor(a!) o_acc, Tensor(b!) lse_acc, Tensor o_part, Tensor lse_part, int tensor_layout, int first) -> ()
// One launch that folds a partial result (o_part fp16 / bf16 in `tensor_layout`, lse_part fp32 [B,H,S])
// into fp32 accumulators (o_acc in `tensor_layout`, lse_acc [B,H,S]; both may be row slices of larger
// tensors).  The merge step of attention over a sequence split across GPUs.
void fold_partial(at::Tensor& o_acc, at::Tensor& lse_acc, const at::Tensor& o_part, const at::Tensor& lse_part,
                  int64_t layout, int64_t first) {
  TORCH_CHECK(o_acc.is_cuda() && o_acc.scalar_type() == at::kFloat && o_acc.dim() == 4 && o_acc.stride(-1) == 1,
              "o_acc must be a 4-D fp32 CUDA tensor with a contiguous last dim");
  check_16b(o_part, "o_part");
  const Dims d = dims_of(o_part, layout), da = dims_of(o_acc, layout);
  TORCH_CHECK(da.B == d.B && da.H == d.H && da.S == d.S && da.D == d.D, "o_acc and o_part differ in shape");
  TORCH_CHECK(lse_part.scalar_type() == at::kFloat && lse_part.is_contiguous() && lse_part.numel() == d.B * d.H * d.S,
              "lse_part must be a contiguous fp32 [B,H,S] tensor");
  TORCH_CHECK(lse_acc.scalar_type() == at::kFloat && lse_acc.dim() == 3 && lse_acc.size(0) == d.B && lse_acc.size(1) == d.H &&
                  lse_acc.size(2) == d.S && lse_acc.stride(2) == 1,
              "lse_acc must be an fp32 [B,H,S] tensor with a contiguous last dim");
  c10::cuda::CUDAGuard guard(o_part.device());
  const sage_strided_t acc = strided_of(o_acc, layout), part = strided_of(o_part, layout);
  check_rc(sage_fold_attn_partial(&acc, lse_acc.data_ptr<float>(), lse_acc.stride(0), lse_acc.stride(1), &part,
                                  dtype_code(o_part), lse_part.data_ptr<float>(), (int)d.B, (int)d.H, (int)d.S, (int)d.D,
                                  (int)first, current_stream(o_part)),
           "fold_partial");
}

}  // namespace

TORCH_LIBRARY(sageattention, m) {
  m.def("fold_partial(Tensor(a!) o_acc, Tensor(b!) lse_acc, Tensor o_part, Tensor lse_part, int tensor_layout, int first) -> ()");
  m.def("sageattn_fwd(Tensor query, Tensor key, Tensor value, int tensor_layout, int is_causal, float sm_scale, "
        "int smooth_k, int use_direct, Tensor status, Tensor? lse=None, Tensor? out=None, int[]? peer_ptrs=None) -> Tensor[]");
  m.def("fp16_attn(Tensor query, Tensor key, Tensor value, Tensor(a!) output, int tensor_layout, int value_layout, "
        "int is_causal, float sm_scale, int bm_sel=0, Tensor? status=None, Tensor? lse=None) -> Tensor");
  m.def("bf16_attn(Tensor query, Tensor key, Tensor value, Tensor(a!) output, int tensor_layout, int value_layout, "
        "int is_causal, float sm_scale, int bm_sel=0, Tensor? status=None, Tensor? lse=None) -> Tensor");
  m.def("qk_int8_sv_f16_attn(Tensor query, Tensor key, Tensor value, Tensor(a!) output, Tensor q_scale, "
        "Tensor k_scale, int tensor_layout, int is_causal, float sm_scale, *, int value_layout=-1, "
        "Tensor? s_dump=None, Tensor? status=None, Tensor? lse=None, int[]? peer_ptrs=None) -> Tensor");
  m.def("quant_qk_int8(Tensor query, Tensor key, Tensor key_mean, int tensor_layout, float sm_scale) -> Tensor[]");
  m.def("prep_qkv(Tensor query, Tensor key, Tensor value, Tensor key_mean, int tensor_layout, float sm_scale) "
        "-> Tensor[]");
  m.def("prep_smooth_qkv(Tensor query, Tensor key, Tensor? value, int tensor_layout, float sm_scale) -> Tensor[]");
  m.def("mean_seq(Tensor input, int tensor_layout) -> Tensor");
  m.def("v_to_f16(Tensor value, int tensor_layout) -> Tensor");
}

TORCH_LIBRARY_IMPL(sageattention, CUDA, m) {
  m.impl("sageattn_fwd", &sageattn_fwd);
  m.impl("qk_int8_sv_f16_attn", &qk_int8_sv_f16_attn);
  m.impl("fp16_attn", &fp16_attn);
  m.impl("bf16_attn", &bf16_attn);
  m.impl("quant_qk_int8", &quant_qk_int8);
  m.impl("prep_qkv", &prep_qkv);
  m.impl("fold_partial", &fold_partial);
  m.impl("prep_smooth_qkv", &prep_smooth_qkv);
  m.impl("mean_seq", &mean_seq);
  m.impl("v_to_f16", &v_to_f16);
}

// An otherwise empty CPython module, so that `import sageattention_rdna3_b200._C` loads the
// library and runs the registrations above (the reference does the same, csrc/pybind_gfx11.cpp:6-16).
static struct PyModuleDef sage_module_def = {PyModuleDef_HEAD_INIT, "_C", nullptr, -1, nullptr};
PyMODINIT_FUNC PyInit__C(void) { return PyModule_Create(&sage_module_def); }
