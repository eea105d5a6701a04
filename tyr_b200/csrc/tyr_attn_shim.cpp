// Lean-facing shim over the C ABI of include/tyr_b200_attn.h.
//
// This file is meant to be dropped into Tyr's cc/src/ next to tyr.cpp and linked
// into libTyrC (cc/Makefile picks up cc/src/*.cpp).  It lifts raw device pointers,
// sizes and strides out of Tyr's tensor handles (Lean external objects owning a
// c10::TensorImpl*, cc/src/tyr.cpp:111-159) and calls the library; no ATen
// operator runs between pointer extraction and launch, only the allocation of the
// result tensor for the pure (surface A) entry points.
//
// It compiles only where <lean/lean.h> and the LibTorch headers exist (same
// __has_include idiom as cc/src/tyr.cpp:72-81); elsewhere it is an empty
// translation unit.  The image this library is developed in has no Lean toolchain.
#if defined(__has_include)
#if __has_include(<lean/lean.h>) && __has_include(<torch/torch.h>)
#define TYR_B200_SHIM_ENABLED 1
#endif
#endif

#ifdef TYR_B200_SHIM_ENABLED
#include <lean/lean.h>
#include <torch/torch.h>
#if __has_include(<c10/cuda/CUDAStream.h>)
#include <c10/cuda/CUDAStream.h>
#define TYR_B200_HAS_CUDA_STREAM 1
#endif

#include <cstring>

#include "tyr_b200_attn.h"

// provided by cc/src/tyr.cpp
torch::Tensor borrowTensor(b_lean_obj_arg o);
lean_object* giveTensor(torch::Tensor t);

namespace {

lean_object* io_error(const char* msg) {
  return lean_io_result_mk_error(lean_mk_io_user_error(lean_mk_string(msg)));
}

bool eligible(const torch::Tensor& t) {
  return t.defined() && t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 4 &&
         t.stride(3) == 1;
}

void fill_strides(int64_t* s, const torch::Tensor& t) {
  s[0] = t.stride(0);
  s[1] = t.stride(1);
  s[2] = t.stride(2);
}

// Fills `a` from [B,H,S,D] tensors.  `o` must already exist.
void fill_args(TyrAttnPrefillArgs& a, const torch::Tensor& q, const torch::Tensor& k,
               const torch::Tensor& v, const torch::Tensor& o, float* lse, bool is_causal) {
  std::memset(&a, 0, sizeof(a));
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.o = o.data_ptr();
  a.lse = lse;
  a.batch = (int32_t)q.size(0);
  a.n_head = (int32_t)q.size(1);
  a.q_seq = (int32_t)q.size(2);
  a.head_dim = (int32_t)q.size(3);
  a.n_kv_head = (int32_t)k.size(1);
  a.kv_seq = (int32_t)k.size(2);
  fill_strides(a.q_stride, q);
  fill_strides(a.k_stride, k);
  fill_strides(a.v_stride, v);
  fill_strides(a.o_stride, o);
  a.dtype = TYR_ATTN_BF16;
  a.is_causal = is_causal ? 1 : 0;
}

void* current_stream(const torch::Tensor& t) {
#ifdef TYR_B200_HAS_CUDA_STREAM
  return c10::cuda::getCurrentCUDAStream(t.get_device()).stream();
#else
  (void)t;
  return nullptr;
#endif
}

// Differentiable form of the call: LibTorch autograd (`autograd.backward`, Tyr/Torch.lean:742 ->
// cc/src/tyr.cpp:2111-2122) reaches tyr_b200_attn_backward through this node instead of
// differentiating ATen's SDPA.  Forward keeps O and the per-row LSE; backward is three launches
// on the current stream.  `key_bytes` is an undefined tensor or uint8 [batch, kv_seq].
struct TyrB200SdpaFn : public torch::autograd::Function<TyrB200SdpaFn> {
  static torch::Tensor forward(torch::autograd::AutogradContext* ctx, torch::Tensor q, torch::Tensor k,
                               torch::Tensor v, bool is_causal, int64_t window_size, torch::Tensor key_bytes) {
    torch::Tensor o = torch::empty(q.sizes(), q.options());
    torch::Tensor lse = torch::empty({q.size(0), q.size(1), q.size(2)}, q.options().dtype(torch::kFloat));
    TyrAttnPrefillArgs a;
    fill_args(a, q, k, v, o, lse.data_ptr<float>(), is_causal);
    a.window_size = (int32_t)window_size;
    if (key_bytes.defined()) {
      a.key_mask = key_bytes.data_ptr<uint8_t>();
      a.key_mask_stride = key_bytes.stride(0);
    }
    const int rc = tyr_b200_attn_prefill(&a, current_stream(q));
    if (rc != 0) throw std::runtime_error(tyr_b200_attn_strerror(rc));
    ctx->save_for_backward({q, k, v, o, lse, key_bytes});
    ctx->saved_data["is_causal"] = is_causal;
    ctx->saved_data["window_size"] = window_size;
    return o;
  }

  static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                               torch::autograd::tensor_list grad_outputs) {
    auto saved = ctx->get_saved_variables();
    const torch::Tensor &q = saved[0], &k = saved[1], &v = saved[2], &o = saved[3], &lse = saved[4],
                        &key_bytes = saved[5];
    torch::Tensor d_o = grad_outputs[0].to(q.scalar_type()).contiguous();
    torch::Tensor d_q = torch::empty(q.sizes(), q.options()), d_k = torch::empty(k.sizes(), k.options()),
                  d_v = torch::empty(v.sizes(), v.options());
    const uint64_t ws_bytes = tyr_b200_attn_backward_workspace_bytes((int32_t)q.size(0), (int32_t)q.size(1),
                                                                     (int32_t)q.size(2));
    torch::Tensor ws = torch::empty({(int64_t)(ws_bytes / 4)}, q.options().dtype(torch::kFloat));
    TyrAttnBackwardArgs a;
    std::memset(&a, 0, sizeof(a));
    a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr();
    a.d_o = d_o.data_ptr(); a.lse = lse.data_ptr<float>();
    a.d_q = d_q.data_ptr(); a.d_k = d_k.data_ptr(); a.d_v = d_v.data_ptr();
    a.workspace = ws.data_ptr();
    a.workspace_bytes = ws_bytes;
    a.batch = (int32_t)q.size(0); a.n_head = (int32_t)q.size(1); a.n_kv_head = (int32_t)k.size(1);
    a.q_seq = (int32_t)q.size(2); a.kv_seq = (int32_t)k.size(2); a.head_dim = (int32_t)q.size(3);
    fill_strides(a.q_stride, q); fill_strides(a.k_stride, k); fill_strides(a.v_stride, v);
    fill_strides(a.o_stride, o); fill_strides(a.do_stride, d_o); fill_strides(a.dq_stride, d_q);
    fill_strides(a.dk_stride, d_k); fill_strides(a.dv_stride, d_v);
    a.dtype = TYR_ATTN_BF16;
    a.is_causal = ctx->saved_data["is_causal"].toBool() ? 1 : 0;
    a.window_size = (int32_t)ctx->saved_data["window_size"].toInt();
    if (key_bytes.defined()) {
      a.key_mask = key_bytes.data_ptr<uint8_t>();
      a.key_mask_stride = key_bytes.stride(0);
    }
    const int rc = tyr_b200_attn_backward(&a, current_stream(q));
    if (rc != 0) throw std::runtime_error(tyr_b200_attn_strerror(rc));
    return {d_q, d_k, d_v, torch::Tensor(), torch::Tensor(), torch::Tensor()};
  }
};

}  // namespace

// Surface A helper: try the B200 kernel; false means "not eligible, keep the LibTorch
// call".  The pure Lean externs cannot fail, so every rejection falls through.
//   usage inside lean_torch_sdpa_gqa (cc/src/tyr.cpp:3913-3949), before the
//   repeat_interleave:   torch::Tensor out; if (tyr_b200_try_sdpa(q, k, v, dropout_p,
//   is_causal, enable_gqa, &out)) return giveTensor(out);
// `window_size` > 0: the sliding window of lean_torch_sdpa_gqa_window (cc/src/tyr.cpp:3953-4018).
// `padding_mask` defined: the [batch, seq] key mask of lean_torch_sdpa_gqa_mask (4024-4095).
bool tyr_b200_try_sdpa(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                       double dropout_p, bool is_causal, bool enable_gqa, torch::Tensor* out,
                       uint64_t window_size = 0, const torch::Tensor& padding_mask = torch::Tensor()) {
  if (dropout_p != 0.0 || !eligible(q) || !eligible(k) || !eligible(v)) return false;
  if (!enable_gqa && q.size(1) != k.size(1)) return false;
  if (k.size(1) == 0 || q.size(1) % k.size(1) != 0) return false;
  if (q.size(3) != 64 && q.size(3) != 128) return false;
  if (window_size > 0x7fffffffu || (window_size > 0 && q.size(2) != k.size(2))) return false;
  torch::Tensor key_bytes;  // one byte per key, kept alive until the launch is queued
  if (padding_mask.defined()) {
    if (padding_mask.dim() != 2 || padding_mask.size(0) != k.size(0) || padding_mask.size(1) != k.size(2))
      return false;
    key_bytes = padding_mask.to(q.device()).ne(0).to(torch::kUInt8).contiguous();
  }
  for (const auto* t : {&q, &k, &v})
    for (int i = 0; i < 3; ++i)
      if (t->size(i) > 1 && (t->stride(i) <= 0 || (t->stride(i) & 7))) return false;
  if ((reinterpret_cast<uintptr_t>(q.data_ptr()) | reinterpret_cast<uintptr_t>(k.data_ptr()) |
       reinterpret_cast<uintptr_t>(v.data_ptr())) & 15u)
    return false;
  if (torch::GradMode::is_enabled() && (q.requires_grad() || k.requires_grad() || v.requires_grad())) {
    // every rejection the library could make was ruled out above, so the node's forward does not throw
    *out = TyrB200SdpaFn::apply(q, k, v, is_causal, (int64_t)window_size, key_bytes);
    return true;
  }
  torch::Tensor o = torch::empty(q.sizes(), q.options());  // allocation only
  TyrAttnPrefillArgs a;
  fill_args(a, q, k, v, o, nullptr, is_causal);
  a.window_size = (int32_t)window_size;
  if (key_bytes.defined()) {
    a.key_mask = key_bytes.data_ptr<uint8_t>();
    a.key_mask_stride = key_bytes.stride(0);
  }
  if (tyr_b200_attn_prefill(&a, current_stream(q)) != 0) return false;
  *out = o;
  return true;
}

// Surface B: launcher in the shape of the generated lean_launch_* functions
// (Tyr/GPU/Codegen/Attribute.lean:346-386): borrowed tensor handles, scalars,
// stream last, IO result.  Outputs are caller-allocated and written in place.
extern "C" lean_object* lean_launch_tyrB200AttnFwd(b_lean_obj_arg q_, b_lean_obj_arg k_,
                                                   b_lean_obj_arg v_, b_lean_obj_arg o_,
                                                   b_lean_obj_arg lse_, uint8_t is_causal,
                                                   uint64_t stream, lean_object* /*w*/) {
  try {
    auto q = borrowTensor(q_), k = borrowTensor(k_), v = borrowTensor(v_), o = borrowTensor(o_),
         lse = borrowTensor(lse_);
    for (const auto* t : {&q, &k, &v, &o}) {
      if (!t->is_cuda()) return io_error("tyrB200AttnFwd: tensors must be CUDA tensors");
      if (t->dim() != 4) return io_error("tyrB200AttnFwd: tensors must be [batch, heads, seq, head_dim]");
      if (t->scalar_type() != at::kBFloat16) return io_error("tyrB200AttnFwd: tensors must be bfloat16");
      if (t->stride(3) != 1) return io_error("tyrB200AttnFwd: head_dim must have unit stride");
    }
    if (!lse.is_cuda() || !lse.is_contiguous() || lse.scalar_type() != at::kFloat ||
        lse.numel() != q.size(0) * q.size(1) * q.size(2))
      return io_error("tyrB200AttnFwd: lse must be a contiguous float32 [batch, n_head, seq] CUDA tensor");
    TyrAttnPrefillArgs a;
    fill_args(a, q, k, v, o, lse.data_ptr<float>(), is_causal != 0);
    int rc = tyr_b200_attn_prefill(&a, reinterpret_cast<void*>(stream));
    if (rc != 0) return io_error(tyr_b200_attn_strerror(rc));
    return lean_io_result_mk_ok(lean_box(0));
  } catch (const std::exception& e) {
    return io_error(e.what());
  }
}

// The same launcher with the caller's scratch for the key-split of a half-empty last round
// (`workspace`: uint8 CUDA tensor, 256-byte aligned; one with no elements means none), and the
// size query the caller sizes that tensor with (0: this call would not split).
extern "C" lean_object* lean_launch_tyrB200AttnFwdWs(b_lean_obj_arg q_, b_lean_obj_arg k_, b_lean_obj_arg v_,
                                                     b_lean_obj_arg o_, b_lean_obj_arg lse_,
                                                     b_lean_obj_arg workspace_, uint8_t is_causal,
                                                     uint64_t stream, lean_object* /*w*/) {
  try {
    auto q = borrowTensor(q_), k = borrowTensor(k_), v = borrowTensor(v_), o = borrowTensor(o_),
         lse = borrowTensor(lse_), ws = borrowTensor(workspace_);
    for (const auto* t : {&q, &k, &v, &o}) {
      if (!t->is_cuda()) return io_error("tyrB200AttnFwdWs: tensors must be CUDA tensors");
      if (t->dim() != 4) return io_error("tyrB200AttnFwdWs: tensors must be [batch, heads, seq, head_dim]");
      if (t->scalar_type() != at::kBFloat16) return io_error("tyrB200AttnFwdWs: tensors must be bfloat16");
      if (t->stride(3) != 1) return io_error("tyrB200AttnFwdWs: head_dim must have unit stride");
    }
    if (!lse.is_cuda() || !lse.is_contiguous() || lse.scalar_type() != at::kFloat ||
        lse.numel() != q.size(0) * q.size(1) * q.size(2))
      return io_error("tyrB200AttnFwdWs: lse must be a contiguous float32 [batch, n_head, seq] CUDA tensor");
    if (ws.numel() > 0 && (!ws.is_cuda() || !ws.is_contiguous() || ws.element_size() != 1))
      return io_error("tyrB200AttnFwdWs: workspace must be a contiguous one-byte-per-element CUDA tensor");
    TyrAttnPrefillArgs a;
    fill_args(a, q, k, v, o, lse.data_ptr<float>(), is_causal != 0);
    if (ws.numel() > 0) {
      a.workspace = ws.data_ptr();
      a.workspace_bytes = static_cast<int64_t>(ws.numel());
    }
    int rc = tyr_b200_attn_prefill(&a, reinterpret_cast<void*>(stream));
    if (rc != 0) return io_error(tyr_b200_attn_strerror(rc));
    return lean_io_result_mk_ok(lean_box(0));
  } catch (const std::exception& e) {
    return io_error(e.what());
  }
}
extern "C" uint64_t lean_tyrB200AttnFwdWorkspaceBytes(b_lean_obj_arg q_, b_lean_obj_arg k_, b_lean_obj_arg v_,
                                                      uint8_t is_causal) {
  try {
    auto q = borrowTensor(q_), k = borrowTensor(k_), v = borrowTensor(v_);
    if (!q.is_cuda() || q.dim() != 4 || k.dim() != 4 || v.dim() != 4 || q.scalar_type() != at::kBFloat16) return 0;
    TyrAttnPrefillArgs a;
    fill_args(a, q, k, v, q, nullptr, is_causal != 0);  // only shapes and strides are looked at
    const int64_t n = tyr_b200_attn_prefill_workspace_bytes(&a);
    return n > 0 ? static_cast<uint64_t>(n) : 0;
  } catch (const std::exception&) {
    return 0;
  }
}

// Decode over Tyr's dense KVCache ([batch, n_kv_head, maxLen, head_dim],
// Tyr/Model/Qwen/Attention.lean:54-68) with the cache's shared `seq` counter as kv_len.
extern "C" lean_object* lean_launch_tyrB200AttnDecode(b_lean_obj_arg q_, b_lean_obj_arg kcache_,
                                                      b_lean_obj_arg vcache_, b_lean_obj_arg o_,
                                                      b_lean_obj_arg workspace_, uint64_t kv_len,
                                                      uint64_t stream, lean_object* /*w*/) {
  try {
    auto q = borrowTensor(q_), kc = borrowTensor(kcache_), vc = borrowTensor(vcache_),
         o = borrowTensor(o_), ws = borrowTensor(workspace_);
    if (!q.is_cuda() || !kc.is_cuda() || !vc.is_cuda() || !o.is_cuda() || !ws.is_cuda())
      return io_error("tyrB200AttnDecode: tensors must be CUDA tensors");
    if (q.dim() != 4 || q.size(2) != 1 || kc.dim() != 4 || vc.dim() != 4 || o.dim() != 4)
      return io_error("tyrB200AttnDecode: q/o must be [batch, n_head, 1, head_dim], caches 4-D");
    if (kv_len == 0 || (int64_t)kv_len > kc.size(2)) return io_error("tyrB200AttnDecode: bad kv_len");
    TyrAttnDecodeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.q = q.data_ptr();
    a.o = o.data_ptr();
    a.k = kc.data_ptr();
    a.v = vc.data_ptr();
    a.batch = (int32_t)q.size(0);
    a.n_head = (int32_t)q.size(1);
    a.n_kv_head = (int32_t)kc.size(1);
    a.max_kv_seq = (int32_t)kv_len;
    a.head_dim = (int32_t)q.size(3);
    a.q_stride[0] = q.stride(0); a.q_stride[1] = q.stride(1);
    a.o_stride[0] = o.stride(0); a.o_stride[1] = o.stride(1);
    fill_strides(a.k_stride, kc);
    fill_strides(a.v_stride, vc);
    a.workspace = ws.data_ptr();
    a.workspace_bytes = (size_t)ws.nbytes();
    int rc = tyr_b200_attn_decode(&a, reinterpret_cast<void*>(stream));
    if (rc != 0) return io_error(tyr_b200_attn_strerror(rc));
    return lean_io_result_mk_ok(lean_box(0));
  } catch (const std::exception& e) {
    return io_error(e.what());
  }
}

// Backward of the prefill call: dQ, dK, dV written in place into caller-allocated tensors.
// Takes the place of LibTorch autograd's derivative of SDPA (`autograd.backward`,
// Tyr/Torch.lean:742 -> cc/src/tyr.cpp:2111-2122) for callers that keep O and the LSE of
// lean_launch_tyrB200AttnFwd.  `workspace` is a float32 CUDA tensor of at least
// tyr_b200_attn_backward_workspace_bytes(batch, n_head, seq) bytes.  `window_size` is the forward's
// (0: none).  `key_mask_` is the forward's padding mask as a uint8 CUDA tensor [batch, kv_seq]
// (0 = padding key), or a tensor with no elements for "no mask": the gradient of
// lean_torch_sdpa_gqa_mask (cc/src/tyr.cpp:4024-4095).
extern "C" lean_object* lean_launch_tyrB200AttnBwd(b_lean_obj_arg q_, b_lean_obj_arg k_,
                                                   b_lean_obj_arg v_, b_lean_obj_arg o_,
                                                   b_lean_obj_arg lse_, b_lean_obj_arg d_o_,
                                                   b_lean_obj_arg d_q_, b_lean_obj_arg d_k_,
                                                   b_lean_obj_arg d_v_, b_lean_obj_arg workspace_,
                                                   b_lean_obj_arg key_mask_,
                                                   uint8_t is_causal, uint64_t window_size,
                                                   uint64_t stream, lean_object* /*w*/) {
  try {
    auto q = borrowTensor(q_), k = borrowTensor(k_), v = borrowTensor(v_), o = borrowTensor(o_),
         lse = borrowTensor(lse_), d_o = borrowTensor(d_o_), d_q = borrowTensor(d_q_),
         d_k = borrowTensor(d_k_), d_v = borrowTensor(d_v_), ws = borrowTensor(workspace_);
    for (const auto* t : {&q, &k, &v, &o, &d_o, &d_q, &d_k, &d_v}) {
      if (!t->is_cuda()) return io_error("tyrB200AttnBwd: tensors must be CUDA tensors");
      if (t->dim() != 4) return io_error("tyrB200AttnBwd: tensors must be [batch, heads, seq, head_dim]");
      if (t->scalar_type() != at::kBFloat16) return io_error("tyrB200AttnBwd: tensors must be bfloat16");
      if (t->stride(3) != 1) return io_error("tyrB200AttnBwd: head_dim must have unit stride");
    }
    if (o.sizes() != q.sizes() || d_o.sizes() != q.sizes() || d_q.sizes() != q.sizes() ||
        v.sizes() != k.sizes() || d_k.sizes() != k.sizes() || d_v.sizes() != k.sizes())
      return io_error("tyrB200AttnBwd: shape mismatch");
    if (!lse.is_cuda() || !lse.is_contiguous() || lse.scalar_type() != at::kFloat ||
        lse.numel() != q.size(0) * q.size(1) * q.size(2))
      return io_error("tyrB200AttnBwd: lse must be a contiguous float32 [batch, n_head, seq] CUDA tensor");
    if (!ws.is_cuda() || !ws.is_contiguous())
      return io_error("tyrB200AttnBwd: workspace must be a contiguous CUDA tensor");
    TyrAttnBackwardArgs a;
    std::memset(&a, 0, sizeof(a));
    a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr();
    a.d_o = d_o.data_ptr(); a.lse = lse.data_ptr<float>();
    a.d_q = d_q.data_ptr(); a.d_k = d_k.data_ptr(); a.d_v = d_v.data_ptr();
    a.workspace = ws.data_ptr();
    a.workspace_bytes = (uint64_t)ws.nbytes();
    a.batch = (int32_t)q.size(0); a.n_head = (int32_t)q.size(1); a.n_kv_head = (int32_t)k.size(1);
    a.q_seq = (int32_t)q.size(2); a.kv_seq = (int32_t)k.size(2); a.head_dim = (int32_t)q.size(3);
    fill_strides(a.q_stride, q); fill_strides(a.k_stride, k); fill_strides(a.v_stride, v);
    fill_strides(a.o_stride, o); fill_strides(a.do_stride, d_o); fill_strides(a.dq_stride, d_q);
    fill_strides(a.dk_stride, d_k); fill_strides(a.dv_stride, d_v);
    a.dtype = TYR_ATTN_BF16;
    a.is_causal = is_causal != 0;
    a.scale = 0.f;
    if (window_size > 0x7fffffffu) return io_error("tyrB200AttnBwd: window_size too large");
    a.window_size = (int32_t)window_size;  // 0: none; the forward's window otherwise
    auto km = borrowTensor(key_mask_);
    if (km.defined() && km.numel() > 0) {
      if (!km.is_cuda() || km.scalar_type() != at::kByte || km.dim() != 2 || km.stride(1) != 1 ||
          km.size(0) != k.size(0) || km.size(1) != k.size(2))
        return io_error("tyrB200AttnBwd: key_mask must be a uint8 CUDA tensor [batch, kv_seq]");
      a.key_mask = km.data_ptr<uint8_t>();
      a.key_mask_stride = km.stride(0);
    }
    int rc = tyr_b200_attn_backward(&a, reinterpret_cast<void*>(stream));
    if (rc != 0) return io_error(tyr_b200_attn_strerror(rc));
    return lean_io_result_mk_ok(lean_box(0));
  } catch (const std::exception& e) {
    return io_error(e.what());
  }
}

// Decode with one length per sequence: `kv_lens_` is an int32 CUDA tensor [batch] (the per-sequence
// form of KVCache.seq, Tyr/Model/Qwen/Attention.lean:54-58); `max_kv_len` bounds them and sizes the
// grid and the workspace.  Dense cache layout as above.
extern "C" lean_object* lean_launch_tyrB200AttnDecodeRagged(b_lean_obj_arg q_, b_lean_obj_arg kcache_,
                                                            b_lean_obj_arg vcache_, b_lean_obj_arg kv_lens_,
                                                            b_lean_obj_arg o_, b_lean_obj_arg workspace_,
                                                            uint64_t max_kv_len, uint64_t stream,
                                                            lean_object* /*w*/) {
  try {
    auto q = borrowTensor(q_), kc = borrowTensor(kcache_), vc = borrowTensor(vcache_),
         lens = borrowTensor(kv_lens_), o = borrowTensor(o_), ws = borrowTensor(workspace_);
    if (!q.is_cuda() || !kc.is_cuda() || !vc.is_cuda() || !o.is_cuda() || !ws.is_cuda() || !lens.is_cuda())
      return io_error("tyrB200AttnDecodeRagged: tensors must be CUDA tensors");
    if (q.dim() != 4 || q.size(2) != 1 || kc.dim() != 4 || vc.dim() != 4 || o.dim() != 4)
      return io_error("tyrB200AttnDecodeRagged: q/o must be [batch, n_head, 1, head_dim], caches 4-D");
    if (lens.scalar_type() != at::kInt || !lens.is_contiguous() || lens.numel() != q.size(0))
      return io_error("tyrB200AttnDecodeRagged: kv_lens must be a contiguous int32 [batch] tensor");
    if (max_kv_len == 0 || (int64_t)max_kv_len > kc.size(2))
      return io_error("tyrB200AttnDecodeRagged: bad max_kv_len");
    TyrAttnDecodeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.q = q.data_ptr();
    a.o = o.data_ptr();
    a.k = kc.data_ptr();
    a.v = vc.data_ptr();
    a.kv_lens = lens.data_ptr<int32_t>();
    a.batch = (int32_t)q.size(0);
    a.n_head = (int32_t)q.size(1);
    a.n_kv_head = (int32_t)kc.size(1);
    a.max_kv_seq = (int32_t)max_kv_len;
    a.head_dim = (int32_t)q.size(3);
    a.q_stride[0] = q.stride(0); a.q_stride[1] = q.stride(1);
    a.o_stride[0] = o.stride(0); a.o_stride[1] = o.stride(1);
    fill_strides(a.k_stride, kc);
    fill_strides(a.v_stride, vc);
    a.workspace = ws.data_ptr();
    a.workspace_bytes = (size_t)ws.nbytes();
    int rc = tyr_b200_attn_decode(&a, reinterpret_cast<void*>(stream));
    if (rc != 0) return io_error(tyr_b200_attn_strerror(rc));
    return lean_io_result_mk_ok(lean_box(0));
  } catch (const std::exception& e) {
    return io_error(e.what());
  }
}

// Fused prologue: per-head RMSNorm + rotary + [B,S,H,D] -> [B,H,S,D] + in-place cache append, the
// one-pass form of applyHeadNorm / rotary.applyRotaryEmb / transpose_for_attention /
// data.sliceScatter (Tyr/Model/Qwen/Attention.lean:73-98, 132-144, 189-193).  `norm_weight_`, `cos_`,
// `sin_` are float32 CUDA tensors, `positions_` int32 [batch]; any of them may be a tensor with no
// elements to skip that step (positions: `position0` is used for every sequence).  `out_at_row0` != 0:
// the position selects the rotary row only and the result is written at rows 0.. of out (the query of
// a decode step).
extern "C" lean_object* lean_launch_tyrB200QkPrologue(b_lean_obj_arg x_, b_lean_obj_arg out_,
                                                      b_lean_obj_arg norm_weight_, b_lean_obj_arg cos_,
                                                      b_lean_obj_arg sin_, b_lean_obj_arg positions_,
                                                      uint64_t position0, double eps, uint8_t out_at_row0,
                                                      uint64_t stream, lean_object* /*w*/) {
  try {
    auto x = borrowTensor(x_), out = borrowTensor(out_), w = borrowTensor(norm_weight_),
         cs = borrowTensor(cos_), sn = borrowTensor(sin_), pos = borrowTensor(positions_);
    if (!x.is_cuda() || !out.is_cuda() || x.dim() != 4 || out.dim() != 4 ||
        x.scalar_type() != at::kBFloat16 || out.scalar_type() != at::kBFloat16 || x.stride(3) != 1 ||
        out.stride(3) != 1)
      return io_error("tyrB200QkPrologue: x must be bf16 [batch, seq, heads, head_dim], out bf16 [batch, heads, cap, head_dim]");
    if (out.size(0) != x.size(0) || out.size(1) != x.size(2) || out.size(3) != x.size(3))
      return io_error("tyrB200QkPrologue: out does not match x");
    auto f32_or_empty = [](const torch::Tensor& t) {
      return !t.defined() || t.numel() == 0 || (t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kFloat);
    };
    if (!f32_or_empty(w) || !f32_or_empty(cs) || !f32_or_empty(sn))
      return io_error("tyrB200QkPrologue: norm_weight / cos / sin must be contiguous float32 CUDA tensors");
    const bool has_pos = pos.defined() && pos.numel() > 0;
    if (has_pos && (!pos.is_cuda() || pos.scalar_type() != at::kInt || !pos.is_contiguous() ||
                    pos.numel() != x.size(0)))
      return io_error("tyrB200QkPrologue: positions must be a contiguous int32 [batch] CUDA tensor");
    if (position0 > 0x7fffffffu) return io_error("tyrB200QkPrologue: position0 too large");
    TyrAttnPrologueArgs a;
    std::memset(&a, 0, sizeof(a));
    a.x = x.data_ptr();
    a.out = out.data_ptr();
    a.norm_weight = (w.defined() && w.numel() > 0) ? w.data_ptr<float>() : nullptr;
    const bool rot = cs.defined() && cs.numel() > 0;
    a.cos = rot ? cs.data_ptr<float>() : nullptr;
    a.sin = (sn.defined() && sn.numel() > 0) ? sn.data_ptr<float>() : nullptr;
    a.positions = has_pos ? pos.data_ptr<int32_t>() : nullptr;
    a.position0 = (int32_t)position0;
    a.batch = (int32_t)x.size(0); a.seq = (int32_t)x.size(1); a.n_head = (int32_t)x.size(2);
    a.head_dim = (int32_t)x.size(3);
    fill_strides(a.x_stride, x);
    fill_strides(a.out_stride, out);
    a.eps = (float)eps;
    a.cap = (int32_t)out.size(2);
    a.max_pos = rot ? (int32_t)cs.size(0) : 0;
    a.out_at_row0 = out_at_row0 ? 1 : 0;
    int rc = tyr_b200_attn_qk_prologue(&a, reinterpret_cast<void*>(stream));
    if (rc != 0) return io_error(tyr_b200_attn_strerror(rc));
    return lean_io_result_mk_ok(lean_box(0));
  } catch (const std::exception& e) {
    return io_error(e.what());
  }
}

// LSE merge of two partial results over disjoint key sets (ringAttnReduce,
// Tyr/GPU/Kernels/RingAttn.lean:164-180): float32 CUDA tensors, o_* [rows, head_dim], lse_* [rows].
extern "C" lean_object* lean_launch_tyrB200AttnMerge(b_lean_obj_arg o_a_, b_lean_obj_arg lse_a_,
                                                     b_lean_obj_arg o_b_, b_lean_obj_arg lse_b_,
                                                     b_lean_obj_arg o_out_, b_lean_obj_arg lse_out_,
                                                     uint64_t stream, lean_object* /*w*/) {
  try {
    auto oa = borrowTensor(o_a_), la = borrowTensor(lse_a_), ob = borrowTensor(o_b_), lb = borrowTensor(lse_b_),
         oo = borrowTensor(o_out_), lo = borrowTensor(lse_out_);
    for (const auto* t : {&oa, &la, &ob, &lb, &oo, &lo})
      if (!t->is_cuda() || !t->is_contiguous() || t->scalar_type() != at::kFloat)
        return io_error("tyrB200AttnMerge: tensors must be contiguous float32 CUDA tensors");
    if (oa.dim() < 2 || oa.sizes() != ob.sizes() || oa.sizes() != oo.sizes() || la.numel() != lb.numel() ||
        la.numel() != lo.numel() || la.numel() * oa.size(-1) != oa.numel())
      return io_error("tyrB200AttnMerge: shape mismatch");
    int rc = tyr_b200_attn_merge(oa.data_ptr<float>(), la.data_ptr<float>(), ob.data_ptr<float>(),
                                 lb.data_ptr<float>(), oo.data_ptr<float>(), lo.data_ptr<float>(),
                                 la.numel(), (int32_t)oa.size(-1), reinterpret_cast<void*>(stream));
    if (rc != 0) return io_error(tyr_b200_attn_strerror(rc));
    return lean_io_result_mk_ok(lean_box(0));
  } catch (const std::exception& e) {
    return io_error(e.what());
  }
}
#endif  // TYR_B200_SHIM_ENABLED
