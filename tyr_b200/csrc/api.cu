// C ABI of the attention library: argument checks, dispatch to the kernels,
// the host-buffer call and the per-device status word.  The checks mirror the
// pre-launch checks of Tyr's generated launchers (is_cuda / is_contiguous /
// dim <= 4 -> IO error string, Tyr/GPU/Codegen/Attribute.lean:333-336) in
// raw-pointer terms: non-null, sizes, alignment, dtype.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <initializer_list>
#include <mutex>

#include "attn_internal.h"
#include "ptx_sm100.cuh"

namespace tyr {
namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mu;       // guards g_state
std::mutex g_host_mu;  // serialises the host-buffer call and guards g_stage
DeviceState g_state[kMaxDevices];
std::atomic<uint64_t> g_launches{0};

constexpr int kHostChunks = 4;            // pieces the host-buffer call aims for (its two end pieces are halved)
constexpr int kMaxHostChunks = kHostChunks + 2;
struct HostStage {  // device staging buffers of the host-buffer call, grown on demand
  void* buf = nullptr;
  size_t bytes = 0;
  cudaStream_t stream = nullptr;      // host->device copies (one copy engine)
  cudaStream_t compute = nullptr;     // the kernels
  cudaStream_t out_stream = nullptr;  // device->host copies (the other copy engine)
  cudaEvent_t landed[kMaxHostChunks] = {};  // inputs of chunk i are on the device
  cudaEvent_t done[kMaxHostChunks] = {};    // kernel of chunk i finished
};
HostStage g_stage[kMaxDevices];

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// scale <= 0 (or NaN) selects ATen's default 1/sqrt(head_dim); the kernels take the row maximum
// of the raw scores before scaling, which is only valid for a positive scale
float resolve_scale(float scale, int d) { return scale > 0.f ? scale : 1.0f / std::sqrt((float)d); }

std::atomic<long long> g_wait_limit{0};  // 0: the compiled default

int current_device_checked(int* dev) {
  cudaError_t e = cudaGetDevice(dev);
  if (e != cudaSuccess) return (int)e;
  if (*dev < 0 || *dev >= kMaxDevices) return -TYR_ATTN_ERR_NO_DEVICE;
  return 0;
}

// A call with a zero extent, as ATen's operator treats it: an output without elements is nothing
// to do, and attention over no keys is O = 0 (softmax over an empty row times an empty V).
// 1: nothing to do; 2: no keys; 0: an ordinary call (or one the checks will refuse).
int empty_kind(const TyrAttnPrefillArgs* a) {
  if (!a || a->batch < 0 || a->n_head < 0 || a->n_kv_head < 0 || a->q_seq < 0 || a->kv_seq < 0 || a->head_dim <= 0) return 0;
  if (a->batch == 0 || a->n_head == 0 || a->q_seq == 0) return 1;
  if (a->kv_seq == 0 && a->o && (a->dtype == TYR_ATTN_BF16 || a->dtype == TYR_ATTN_F32)) return 2;
  return 0;
}

// Zeros into every row of a [batch, heads, seq, d] tensor with element strides (rows of d contiguous
// elements of `esize` bytes), and -inf into `lse` [batch, heads, seq] when given: one thread per 2 bytes.
struct ZeroRows {
  void* base;
  float* lse;
  int64_t batch, heads, seq, d, stride[3];
  int esize;
};
__global__ void zero_rows_kernel(const ZeroRows z) {
  const int64_t per_row = z.d * z.esize / 2;  // 2-byte units of a row
  const int64_t rows = z.batch * z.heads * z.seq;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * per_row) return;
  const int64_t row = i / per_row, c = i - row * per_row;
  const int64_t s = row % z.seq, h = (row / z.seq) % z.heads, b = row / (z.seq * z.heads);
  uint16_t* o = static_cast<uint16_t*>(z.base) + (b * z.stride[0] + h * z.stride[1] + s * z.stride[2]) * (z.esize / 2);
  o[c] = 0;
  if (c == 0 && z.lse) z.lse[row] = -INFINITY;
}

int launch_zero_rows(void* base, float* lse, int64_t batch, int64_t heads, int64_t seq, int64_t d, const int64_t* stride,
                     int esize, cudaStream_t st) {
  const int64_t n = batch * heads * seq * d * esize / 2;
  if (n == 0) return 0;
  if (n > 0x7fffffffLL * 256) return -TYR_ATTN_ERR_TOO_LARGE;
  const ZeroRows z{base, lse, batch, heads, seq, d, {stride[0], stride[1], stride[2]}, esize};
  zero_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(z);
  count_launch();
  return (int)cudaGetLastError();
}

// attention over no keys: O = 0 and LSE = -inf for every query row
int launch_no_keys(const TyrAttnPrefillArgs& a, cudaStream_t st) {
  return launch_zero_rows(a.o, a.lse, a.batch, a.n_head, a.q_seq, a.head_dim, a.o_stride, a.dtype == TYR_ATTN_F32 ? 4 : 2, st);
}

int check_prefill(const TyrAttnPrefillArgs* a) {
  if (!a || !a->q || !a->k || !a->v || !a->o) return -TYR_ATTN_ERR_NULL;
  if (a->batch <= 0 || a->n_head <= 0 || a->n_kv_head <= 0 || a->q_seq <= 0 || a->kv_seq <= 0 ||
      a->head_dim <= 0)
    return -TYR_ATTN_ERR_SHAPE;
  if (a->n_head % a->n_kv_head != 0) return -TYR_ATTN_ERR_SHAPE;
  if (a->dtype != TYR_ATTN_BF16 && a->dtype != TYR_ATTN_F32) return -TYR_ATTN_ERR_DTYPE;
  if (a->dtype == TYR_ATTN_F32 && !a->check_mode) return -TYR_ATTN_ERR_DTYPE;
  if (a->n_head > 65535 || a->batch > 65535) return -TYR_ATTN_ERR_TOO_LARGE;
  // the windowed call has one sequence length (cc/src/tyr.cpp:3953-3965); with more queries than
  // keys + window an item would have no key tile at all
  if (a->window_size < 0 || (a->window_size > 0 && a->q_seq != a->kv_seq)) return -TYR_ATTN_ERR_SHAPE;
  if (a->key_mask && a->batch > 1 && a->key_mask_stride < a->kv_seq) return -TYR_ATTN_ERR_SHAPE;
  if (!a->check_mode) {
    if (a->head_dim != 64 && a->head_dim != 128) return -TYR_ATTN_ERR_HEAD_DIM;
    if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o))
      return -TYR_ATTN_ERR_ALIGN;
    const int64_t* s[4] = {a->q_stride, a->k_stride, a->v_stride, a->o_stride};
    const int dims[4][3] = {{a->batch, a->n_head, a->q_seq},
                            {a->batch, a->n_kv_head, a->kv_seq},
                            {a->batch, a->n_kv_head, a->kv_seq},
                            {a->batch, a->n_head, a->q_seq}};
    for (int t = 0; t < 4; ++t)
      for (int i = 0; i < 3; ++i)
        if (dims[t][i] > 1 && (s[t][i] <= 0 || (s[t][i] & 7))) return -TYR_ATTN_ERR_ALIGN;
  } else if (a->head_dim > 256) {
    return -TYR_ATTN_ERR_HEAD_DIM;
  }
  return 0;
}

void contiguous_strides(int64_t* s, int64_t heads, int64_t seq, int64_t d) {
  s[2] = d;
  s[1] = seq * d;
  s[0] = heads * seq * d;
}

int sdpa_contiguous(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t q_seq,
                    uint64_t kv_seq, uint64_t head_dim, const void* q, const void* k, const void* v,
                    void* out, double dropout_p, uint8_t is_causal, void* stream,
                    uint64_t window_size = 0, const uint8_t* key_mask = nullptr) {
  if (dropout_p != 0.0) return -TYR_ATTN_ERR_DROPOUT;
  if (batch > 0x7fffffffu || n_head > 0x7fffffffu || n_kv_head > 0x7fffffffu ||
      q_seq > 0x7fffffffu || kv_seq > 0x7fffffffu || head_dim > 0x7fffffffu)
    return -TYR_ATTN_ERR_TOO_LARGE;
  TyrAttnPrefillArgs a;
  std::memset(&a, 0, sizeof(a));
  a.q = q; a.k = k; a.v = v; a.o = out; a.lse = nullptr;
  a.batch = (int)batch; a.n_head = (int)n_head; a.n_kv_head = (int)n_kv_head;
  a.q_seq = (int)q_seq; a.kv_seq = (int)kv_seq; a.head_dim = (int)head_dim;
  contiguous_strides(a.q_stride, a.n_head, a.q_seq, a.head_dim);
  contiguous_strides(a.k_stride, a.n_kv_head, a.kv_seq, a.head_dim);
  contiguous_strides(a.v_stride, a.n_kv_head, a.kv_seq, a.head_dim);
  contiguous_strides(a.o_stride, a.n_head, a.q_seq, a.head_dim);
  a.dtype = TYR_ATTN_BF16;
  a.is_causal = is_causal ? 1 : 0;
  a.window_size = (int32_t)std::min<uint64_t>(window_size, 0x7fffffffu);
  a.key_mask = key_mask;
  a.key_mask_stride = (int64_t)kv_seq;
  return tyr_b200_attn_prefill(&a, stream);
}

}  // namespace

DeviceState* device_state(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState& s = g_state[device];
  if (!s.ready) {
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess) return nullptr;
    if (cudaSetDevice(device) != cudaSuccess) return nullptr;
    bool ok = cudaMalloc(&s.status, sizeof(int)) == cudaSuccess &&
              cudaMemset(s.status, 0, sizeof(int)) == cudaSuccess;
    cudaSetDevice(prev);
    if (!ok) return nullptr;
    s.ready = true;
  }
  return &s;
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

long long wait_limit_cycles() {
  const long long v = g_wait_limit.load(std::memory_order_relaxed);
  return v > 0 ? v : 4000000000ll;
}

}  // namespace tyr

using namespace tyr;

extern "C" {

int tyr_b200_attn_prefill(const TyrAttnPrefillArgs* a, void* stream) {
  if (const int kind = empty_kind(a)) return kind == 1 ? 0 : launch_no_keys(*a, static_cast<cudaStream_t>(stream));
  int rc = check_prefill(a);
  if (rc) return rc;
  const float scale = resolve_scale(a->scale, a->head_dim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->check_mode) return launch_prefill_check(*a, scale, st);
  int dev = 0;
  if ((rc = current_device_checked(&dev))) return rc;
  DeviceState* ds = device_state(dev);
  if (!ds) return -TYR_ATTN_ERR_NO_DEVICE;
  return launch_prefill_sm100(*a, scale, ds->status, st);
}

int tyr_b200_sdpa_4d(uint64_t batch, uint64_t n_head, uint64_t seq, uint64_t head_dim, const void* q,
                     const void* k, const void* v, void* out, double dropout_p, uint8_t is_causal,
                     void* stream) {
  return sdpa_contiguous(batch, n_head, n_head, seq, seq, head_dim, q, k, v, out, dropout_p,
                         is_causal, stream);
}

int tyr_b200_sdpa_gqa(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t seq,
                      uint64_t head_dim, const void* q, const void* k, const void* v, void* out,
                      double dropout_p, uint8_t is_causal, uint8_t enable_gqa, void* stream) {
  if (!enable_gqa && n_head != n_kv_head) return -TYR_ATTN_ERR_SHAPE;
  return sdpa_contiguous(batch, n_head, n_kv_head, seq, seq, head_dim, q, k, v, out, dropout_p,
                         is_causal, stream);
}

int tyr_b200_sdpa_gqa_qkv(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t q_seq,
                          uint64_t kv_seq, uint64_t head_dim, const void* q, const void* k,
                          const void* v, void* out, double dropout_p, uint8_t is_causal,
                          uint8_t enable_gqa, void* stream) {
  if (!enable_gqa && n_head != n_kv_head) return -TYR_ATTN_ERR_SHAPE;
  return sdpa_contiguous(batch, n_head, n_kv_head, q_seq, kv_seq, head_dim, q, k, v, out, dropout_p,
                         is_causal, stream);
}

int tyr_b200_sdpa_gqa_window(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t seq,
                             uint64_t head_dim, const void* q, const void* k, const void* v,
                             void* out, double dropout_p, uint8_t /*is_causal*/, uint8_t enable_gqa,
                             uint64_t window_size, void* stream) {
  if (!enable_gqa && n_head != n_kv_head) return -TYR_ATTN_ERR_SHAPE;
  if (window_size == 0) return -TYR_ATTN_ERR_SHAPE;  // the reference's mask would hide every key
  return sdpa_contiguous(batch, n_head, n_kv_head, seq, seq, head_dim, q, k, v, out, dropout_p, 1,
                         stream, window_size);
}

int tyr_b200_sdpa_gqa_mask(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t seq,
                           uint64_t head_dim, const void* q, const void* k, const void* v,
                           const uint8_t* key_mask, void* out, double dropout_p, uint8_t is_causal,
                           uint8_t enable_gqa, void* stream) {
  if (!enable_gqa && n_head != n_kv_head) return -TYR_ATTN_ERR_SHAPE;
  if (!key_mask) return -TYR_ATTN_ERR_NULL;
  return sdpa_contiguous(batch, n_head, n_kv_head, seq, seq, head_dim, q, k, v, out, dropout_p,
                         is_causal, stream, 0, key_mask);
}

size_t tyr_b200_attn_decode_workspace_bytes(int32_t batch, int32_t n_head, int32_t head_dim,
                                            int32_t max_kv_seq, int32_t max_splits) {
  if (batch <= 0 || n_head <= 0 || head_dim <= 0 || max_kv_seq <= 0) return 0;
  return decode_workspace_bytes(batch, n_head, head_dim, max_kv_seq, max_splits);
}

int tyr_b200_attn_decode(const TyrAttnDecodeArgs* a, void* stream) {
  if (a && a->batch == 0 && a->n_head >= 0 && a->n_kv_head >= 0 && a->head_dim > 0) return 0;  // no sequence: nothing to do
  if (!a || !a->q || !a->o) return -TYR_ATTN_ERR_NULL;
  const bool ragged = a->k_ptrs != nullptr || a->v_ptrs != nullptr;
  if (ragged ? (!a->k_ptrs || !a->v_ptrs) : (!a->k || !a->v)) return -TYR_ATTN_ERR_NULL;
  if (a->batch <= 0 || a->n_head <= 0 || a->n_kv_head <= 0 || a->max_kv_seq <= 0)
    return -TYR_ATTN_ERR_SHAPE;
  if (a->n_head % a->n_kv_head != 0) return -TYR_ATTN_ERR_SHAPE;
  if (a->head_dim != 64 && a->head_dim != 128) return -TYR_ATTN_ERR_HEAD_DIM;
  if (a->batch > 65535) return -TYR_ATTN_ERR_TOO_LARGE;
  if ((a->k_stride[2] & 7) || (a->v_stride[2] & 7) || a->k_stride[2] <= 0 || a->v_stride[2] <= 0)
    return -TYR_ATTN_ERR_ALIGN;
  if (!ragged) {
    if (!aligned16(a->k) || !aligned16(a->v)) return -TYR_ATTN_ERR_ALIGN;
    if ((a->k_stride[0] & 7) || (a->k_stride[1] & 7) || (a->v_stride[0] & 7) || (a->v_stride[1] & 7))
      return -TYR_ATTN_ERR_ALIGN;
  }
  if ((reinterpret_cast<uintptr_t>(a->q) & 3u) || (a->q_stride[0] & 1) || (a->q_stride[1] & 1))
    return -TYR_ATTN_ERR_ALIGN;
  const float scale = resolve_scale(a->scale, a->head_dim);
  return launch_decode(*a, scale, static_cast<cudaStream_t>(stream));
}

int tyr_b200_attn_merge(const float* o_a, const float* lse_a, const float* o_b, const float* lse_b,
                        float* o_out, float* lse_out, int64_t rows, int32_t head_dim, void* stream) {
  if (!o_a || !lse_a || !o_b || !lse_b || !o_out || !lse_out) return -TYR_ATTN_ERR_NULL;
  if (rows <= 0 || head_dim <= 0) return -TYR_ATTN_ERR_SHAPE;
  return launch_merge2(o_a, lse_a, o_b, lse_b, o_out, lse_out, rows, head_dim,
                       static_cast<cudaStream_t>(stream));
}

int tyr_b200_attn_qk_prologue(const TyrAttnPrologueArgs* a, void* stream) {
  if (!a || !a->x || !a->out) return -TYR_ATTN_ERR_NULL;
  if ((a->cos == nullptr) != (a->sin == nullptr)) return -TYR_ATTN_ERR_NULL;
  if (a->pe && a->cos) return -TYR_ATTN_ERR_SHAPE;  // one rotary form per call
  if (a->batch <= 0 || a->seq <= 0 || a->n_head <= 0 || a->position0 < 0) return -TYR_ATTN_ERR_SHAPE;
  if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256) return -TYR_ATTN_ERR_HEAD_DIM;
  // every written row and every rotary row must exist: the reference guards its append with
  // `cache.seq < cache.maxLen` (Tyr/Model/Qwen/Attention.lean:189)
  if (a->cap <= 0 || ((a->cos || a->pe) && a->max_pos <= 0)) return -TYR_ATTN_ERR_SHAPE;
  if (a->out_at_row0 && a->seq > a->cap) return -TYR_ATTN_ERR_RANGE;
  if (!a->positions) {
    if (!a->out_at_row0 && (int64_t)a->position0 + a->seq > a->cap) return -TYR_ATTN_ERR_RANGE;
    if ((a->cos || a->pe) && (int64_t)a->position0 + a->seq > a->max_pos) return -TYR_ATTN_ERR_RANGE;
  }
  if (!aligned16(a->x) || !aligned16(a->out) || (a->norm_weight && !aligned16(a->norm_weight)) ||
      (a->cos && (!aligned16(a->cos) || !aligned16(a->sin))) || (a->pe && !aligned16(a->pe)))
    return -TYR_ATTN_ERR_ALIGN;
  for (int i = 0; i < 3; ++i)
    if ((a->x_stride[i] & 7) || (a->out_stride[i] & 7)) return -TYR_ATTN_ERR_ALIGN;
  if (a->pe && (a->pe_batch_stride & 3)) return -TYR_ATTN_ERR_ALIGN;
  int dev = 0, rc;
  if ((rc = current_device_checked(&dev))) return rc;
  DeviceState* ds = device_state(dev);
  if (!ds) return -TYR_ATTN_ERR_NO_DEVICE;
  return launch_qk_prologue(*a, ds->status, static_cast<cudaStream_t>(stream));
}

uint64_t tyr_b200_attn_backward_workspace_bytes(int32_t batch, int32_t n_head, int32_t q_seq) {
  if (batch <= 0 || n_head <= 0 || q_seq <= 0) return 0;
  return backward_workspace_bytes(batch, n_head, q_seq);
}

int tyr_b200_attn_backward(const TyrAttnBackwardArgs* a, void* stream) {
  // Zero extents as autograd of ATen's operator treats them: without queries (or heads, or a batch)
  // dQ has no element and dK, dV are zeros; without keys dK, dV have no element and dQ is zeros.
  if (a && a->batch >= 0 && a->n_head >= 0 && a->n_kv_head >= 0 && a->q_seq >= 0 && a->kv_seq >= 0 &&
      a->dtype == TYR_ATTN_BF16 && (a->head_dim == 64 || a->head_dim == 128) &&
      (a->batch == 0 || a->n_head == 0 || a->q_seq == 0 || a->kv_seq == 0)) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a->batch == 0) return 0;
    if (a->kv_seq == 0) {
      if (a->n_head == 0 || a->q_seq == 0) return 0;
      if (!a->d_q) return -TYR_ATTN_ERR_NULL;
      return launch_zero_rows(a->d_q, nullptr, a->batch, a->n_head, a->q_seq, a->head_dim, a->dq_stride, 2, st);
    }
    if (a->n_kv_head == 0) return 0;
    if (!a->d_k || !a->d_v) return -TYR_ATTN_ERR_NULL;
    const int rc = launch_zero_rows(a->d_k, nullptr, a->batch, a->n_kv_head, a->kv_seq, a->head_dim, a->dk_stride, 2, st);
    return rc ? rc : launch_zero_rows(a->d_v, nullptr, a->batch, a->n_kv_head, a->kv_seq, a->head_dim, a->dv_stride, 2, st);
  }
  if (!a || !a->q || !a->k || !a->v || !a->o || !a->d_o || !a->lse || !a->d_q || !a->d_k || !a->d_v)
    return -TYR_ATTN_ERR_NULL;
  if (a->batch <= 0 || a->n_head <= 0 || a->n_kv_head <= 0 || a->q_seq <= 0 || a->kv_seq <= 0)
    return -TYR_ATTN_ERR_SHAPE;
  if (a->n_head % a->n_kv_head != 0) return -TYR_ATTN_ERR_SHAPE;
  if (a->dtype != TYR_ATTN_BF16) return -TYR_ATTN_ERR_DTYPE;
  if (a->head_dim != 64 && a->head_dim != 128) return -TYR_ATTN_ERR_HEAD_DIM;
  if (a->n_head > 65535 || a->batch > 65535) return -TYR_ATTN_ERR_TOO_LARGE;
  // the windowed call has one sequence length (cc/src/tyr.cpp:3953-3965)
  if (a->window_size < 0 || (a->window_size > 0 && a->q_seq != a->kv_seq)) return -TYR_ATTN_ERR_SHAPE;
  if (a->key_mask && a->batch > 1 && a->key_mask_stride < a->kv_seq) return -TYR_ATTN_ERR_SHAPE;
  const void* ptrs[8] = {a->q, a->k, a->v, a->o, a->d_o, a->d_q, a->d_k, a->d_v};
  const int64_t* strides[8] = {a->q_stride, a->k_stride, a->v_stride, a->o_stride,
                               a->do_stride, a->dq_stride, a->dk_stride, a->dv_stride};
  for (int t = 0; t < 8; ++t) {
    if (!aligned16(ptrs[t])) return -TYR_ATTN_ERR_ALIGN;
    const bool kv = (t == 1 || t == 2 || t == 6 || t == 7);
    const int dims[3] = {a->batch, kv ? a->n_kv_head : a->n_head, kv ? a->kv_seq : a->q_seq};
    for (int i = 0; i < 3; ++i)
      if (dims[i] > 1 && (strides[t][i] <= 0 || (strides[t][i] & 7))) return -TYR_ATTN_ERR_ALIGN;
  }
  if (!a->workspace || (reinterpret_cast<uintptr_t>(a->workspace) & 15u) ||
      a->workspace_bytes < backward_workspace_bytes(a->batch, a->n_head, a->q_seq))
    return -TYR_ATTN_ERR_WORKSPACE;
  int dev = 0, rc;
  if ((rc = current_device_checked(&dev))) return rc;
  DeviceState* ds = device_state(dev);
  if (!ds) return -TYR_ATTN_ERR_NO_DEVICE;
  return launch_backward_sm100(*a, resolve_scale(a->scale, a->head_dim), ds->status,
                               static_cast<cudaStream_t>(stream));
}

int64_t tyr_b200_attn_prefill_workspace_bytes(const TyrAttnPrefillArgs* a) {
  const int rc = check_prefill(a);
  if (rc) return rc;
  if (a->dtype != TYR_ATTN_BF16 || a->check_mode) return 0;
  return tyr::prefill_split_workspace_bytes(*a);
}

int tyr_b200_attn_prefill_host(const TyrAttnPrefillArgs* a, int32_t device) {
  if (const int kind = empty_kind(a)) {
    if (kind == 2) {  // no keys: the host output rows are zeros, their LSE -inf
      const size_t row_bytes = (size_t)a->head_dim * (a->dtype == TYR_ATTN_F32 ? 4 : 2);
      for (int64_t b = 0; b < a->batch; ++b)
        for (int64_t h = 0; h < a->n_head; ++h)
          for (int64_t r = 0; r < a->q_seq; ++r) {
            const int64_t off = b * a->o_stride[0] + h * a->o_stride[1] + r * a->o_stride[2];
            std::memset(static_cast<char*>(a->o) + off * (int64_t)(row_bytes / a->head_dim), 0, row_bytes);
            if (a->lse) a->lse[(b * a->n_head + h) * a->q_seq + r] = -INFINITY;
          }
    }
    return 0;
  }
  int rc = check_prefill(a);
  if (rc && rc != -TYR_ATTN_ERR_ALIGN) return rc;  // host pointers need no 16-byte alignment
  if (device < 0 || device >= kMaxDevices) return -TYR_ATTN_ERR_NO_DEVICE;
  if (a->key_mask) return -TYR_ATTN_ERR_DTYPE;  // the host-buffer call takes no padding mask
  {
    // the pieces below are cut out of contiguous [batch, heads, seq, head_dim] storage
    const int64_t* strides[4] = {a->q_stride, a->k_stride, a->v_stride, a->o_stride};
    const int64_t heads[4] = {a->n_head, a->n_kv_head, a->n_kv_head, a->n_head};
    const int64_t seqs[4] = {a->q_seq, a->kv_seq, a->kv_seq, a->q_seq};
    for (int t = 0; t < 4; ++t) {
      int64_t want[3];
      contiguous_strides(want, heads[t], seqs[t], a->head_dim);
      const int64_t extent[3] = {a->batch, heads[t], seqs[t]};
      for (int i = 0; i < 3; ++i)
        if (extent[i] > 1 && strides[t][i] != want[i]) return -TYR_ATTN_ERR_SHAPE;
    }
  }
  const size_t es = a->dtype == TYR_ATTN_F32 ? 4 : 2;
  const size_t nq = (size_t)a->batch * a->n_head * a->q_seq * a->head_dim;
  const size_t nk = (size_t)a->batch * a->n_kv_head * a->kv_seq * a->head_dim;
  const size_t nl = (size_t)a->batch * a->n_head * a->q_seq;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  const size_t off_k = up(nq * es), off_v = off_k + up(nk * es), off_o = off_v + up(nk * es),
               off_l = off_o + up(nq * es), total = off_l + up(nl * 4);

  cudaError_t e;
  int prev = 0;
  if ((e = cudaGetDevice(&prev)) != cudaSuccess) return (int)e;
  if ((e = cudaSetDevice(device)) != cudaSuccess) return (int)e;
  std::lock_guard<std::mutex> lock(g_host_mu);  // one host-buffer call per process at a time
  HostStage& hs = g_stage[device];
  // every way out drains the three streams first: the caller's host buffers are theirs again on return
  auto fail = [&](int code) {
    for (cudaStream_t s : {hs.out_stream, hs.compute, hs.stream})
      if (s) cudaStreamSynchronize(s);
    cudaSetDevice(prev);
    return code;
  };
  if (!hs.stream && (e = cudaStreamCreateWithFlags(&hs.stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail((int)e);
  if (hs.bytes < total) {
    if (hs.buf) cudaFree(hs.buf);
    hs.buf = nullptr;
    hs.bytes = 0;
    if ((e = cudaMalloc(&hs.buf, total)) != cudaSuccess) return fail((int)e);
    hs.bytes = total;
  }
  char* base = static_cast<char*>(hs.buf);
  TyrAttnPrefillArgs d = *a;
  d.q = base; d.k = base + off_k; d.v = base + off_v; d.o = base + off_o;
  d.lse = a->lse ? reinterpret_cast<float*>(base + off_l) : nullptr;
  contiguous_strides(d.q_stride, a->n_head, a->q_seq, a->head_dim);
  contiguous_strides(d.k_stride, a->n_kv_head, a->kv_seq, a->head_dim);
  contiguous_strides(d.v_stride, a->n_kv_head, a->kv_seq, a->head_dim);
  contiguous_strides(d.o_stride, a->n_head, a->q_seq, a->head_dim);
  if (!hs.out_stream &&
      (e = cudaStreamCreateWithFlags(&hs.out_stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail((int)e);
  if (!hs.compute && (e = cudaStreamCreateWithFlags(&hs.compute, cudaStreamNonBlocking)) != cudaSuccess)
    return fail((int)e);
  // Pipeline over (batch, KV-head range) chunks on three streams: while chunk i computes and
  // chunk i-1 drains to the host on the device->host copy engine, chunk i+1 is already arriving
  // on the host->device one.  In [batch, heads, seq, dim] storage the heads of one batch element are
  // contiguous, so a chunk is one contiguous piece of each tensor.  What the pipeline cannot cover
  // is the first chunk's way in and the last chunk's kernel and way out, so those two chunks are
  // halved; against that every piece costs copy-engine and launch time (five copies, a kernel on a
  // slice of the grid), and few pieces win: Qwen3-8B-shaped (403 MB in, 272 MB out) 10.9 ms as one
  // or two pieces, 9.0 ms with 4 to 8 (+2 for the halved ends), 9.4 with 16, 10.9 with 32 or 64; the
  // smaller workloads are fastest at 4 as well.  9.0 ms is the 403 MB at the 45 GB/s the link
  // gives each direction while both are busy.
  const int g = a->n_head / a->n_kv_head;
  const int per_batch = a->batch >= kHostChunks ? 1 : std::min<int>(a->n_kv_head, kHostChunks / a->batch);
  const int batch_chunks = a->batch >= kHostChunks ? kHostChunks : a->batch;
  struct Piece { int b0, b1, h0, h1; };  // batch elements [b0, b1) x KV heads [h0, h1); heads partial only when b1 = b0 + 1
  Piece pieces[kMaxHostChunks];
  int n_pieces = 0;
  for (int bc = 0; bc < batch_chunks; ++bc) {
    const int b0 = (int)((long long)a->batch * bc / batch_chunks), b1 = (int)((long long)a->batch * (bc + 1) / batch_chunks);
    for (int hc = 0; hc < per_batch; ++hc) {
      const int h0 = (int)((long long)a->n_kv_head * hc / per_batch), h1 = (int)((long long)a->n_kv_head * (hc + 1) / per_batch);
      const bool end = (bc == 0 && hc == 0) || (bc == batch_chunks - 1 && hc == per_batch - 1);
      if (end && b1 - b0 == 1 && h1 - h0 >= 2) {
        const int hm = (h0 + h1) / 2;
        pieces[n_pieces++] = {b0, b1, h0, hm};
        pieces[n_pieces++] = {b0, b1, hm, h1};
      } else if (end && b1 - b0 >= 2) {
        const int bm = (b0 + b1) / 2;
        pieces[n_pieces++] = {b0, bm, 0, a->n_kv_head};
        pieces[n_pieces++] = {bm, b1, 0, a->n_kv_head};
      } else {
        pieces[n_pieces++] = {b0, b1, h0, h1};
      }
    }
  }
  cudaStream_t st = hs.stream, sc = hs.compute, so = hs.out_stream;
  const char *hq = static_cast<const char*>(a->q), *hk = static_cast<const char*>(a->k),
             *hv = static_cast<const char*>(a->v);
  char* ho = static_cast<char*>(a->o);
  const size_t qh1 = (size_t)a->q_seq * a->head_dim * es;   // one query head of one batch element
  const size_t kh1 = (size_t)a->kv_seq * a->head_dim * es;  // one KV head
  const size_t lh1 = (size_t)a->q_seq * 4;
  for (int c = 0; c < n_pieces; ++c) {
    const int b0 = pieces[c].b0, b1 = pieces[c].b1, h0 = pieces[c].h0, h1 = pieces[c].h1;
    const bool part = (h1 - h0) < a->n_kv_head;  // some of the KV heads of one batch element
    const size_t nbat = (size_t)(b1 - b0), nkv = (size_t)(h1 - h0);
    const size_t q_off = ((size_t)b0 * a->n_head + (size_t)h0 * g) * qh1, q_len = (part ? nkv * g : nbat * a->n_head) * qh1;
    const size_t k_off = ((size_t)b0 * a->n_kv_head + h0) * kh1, k_len = (part ? nkv : nbat * a->n_kv_head) * kh1;
    const size_t l_off = ((size_t)b0 * a->n_head + (size_t)h0 * g) * lh1, l_len = (part ? nkv * g : nbat * a->n_head) * lh1;
    if (!hs.done[c] && (e = cudaEventCreateWithFlags(&hs.done[c], cudaEventDisableTiming)) != cudaSuccess)
      return fail((int)e);
    if (!hs.landed[c] && (e = cudaEventCreateWithFlags(&hs.landed[c], cudaEventDisableTiming)) != cudaSuccess)
      return fail((int)e);
    if ((e = cudaMemcpyAsync(base + q_off, hq + q_off, q_len, cudaMemcpyHostToDevice, st)) != cudaSuccess ||
        (e = cudaMemcpyAsync(base + off_k + k_off, hk + k_off, k_len, cudaMemcpyHostToDevice, st)) != cudaSuccess ||
        (e = cudaMemcpyAsync(base + off_v + k_off, hv + k_off, k_len, cudaMemcpyHostToDevice, st)) != cudaSuccess ||
        (e = cudaEventRecord(hs.landed[c], st)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(sc, hs.landed[c], 0)) != cudaSuccess)
      return fail((int)e);
    TyrAttnPrefillArgs dc = d;
    dc.batch = (int32_t)nbat;
    if (part) {
      dc.n_kv_head = (int32_t)nkv;
      dc.n_head = (int32_t)(nkv * g);
    }
    dc.q = base + q_off;
    dc.k = base + off_k + k_off;
    dc.v = base + off_v + k_off;
    dc.o = base + off_o + q_off;
    dc.lse = d.lse ? reinterpret_cast<float*>(base + off_l + l_off) : nullptr;
    rc = tyr_b200_attn_prefill(&dc, sc);
    if (rc) return fail(rc);
    if ((e = cudaEventRecord(hs.done[c], sc)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(so, hs.done[c], 0)) != cudaSuccess ||
        (e = cudaMemcpyAsync(ho + q_off, base + off_o + q_off, q_len, cudaMemcpyDeviceToHost, so)) != cudaSuccess)
      return fail((int)e);
    if (a->lse && (e = cudaMemcpyAsync(reinterpret_cast<char*>(a->lse) + l_off, base + off_l + l_off, l_len,
                                       cudaMemcpyDeviceToHost, so)) != cudaSuccess)
      return fail((int)e);
  }
  e = cudaStreamSynchronize(so);
  if (e == cudaSuccess) e = cudaStreamSynchronize(sc);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaSetDevice(prev);
  return (int)e;
}

int tyr_b200_attn_device_status(int32_t device, int32_t clear) {
  DeviceState* ds = device_state(device);
  if (!ds) return -TYR_ATTN_ERR_NO_DEVICE;
  int prev = 0, v = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(&v, ds->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && clear) e = cudaMemset(ds->status, 0, sizeof(int));
  cudaSetDevice(prev);
  if (e != cudaSuccess) return -(1000 + (int)e);
  return v;
}

int tyr_b200_attn_device_check(int32_t device) {
  const int v = tyr_b200_attn_device_status(device, 1);
  if (v <= 0) return v;
  if (v & (kStatusWaitTimeout | kStatusAborted)) return -TYR_ATTN_ERR_DEVICE_WAIT;
  return -TYR_ATTN_ERR_RANGE;
}

void tyr_b200_attn_test_set_wait_limit(int64_t cycles) {
  g_wait_limit.store(cycles > 0 ? (long long)cycles : 0, std::memory_order_relaxed);
}

int tyr_b200_attn_test_stalled_wait(int64_t limit_cycles, void* stream) {
  if (limit_cycles <= 0 || limit_cycles > 4000000000ll) return -TYR_ATTN_ERR_SHAPE;
  int dev = 0, rc;
  if ((rc = current_device_checked(&dev))) return rc;
  DeviceState* ds = device_state(dev);
  if (!ds) return -TYR_ATTN_ERR_NO_DEVICE;
  return launch_stalled_wait((long long)limit_cycles, ds->status, static_cast<cudaStream_t>(stream));
}

const char* tyr_b200_attn_strerror(int code) {
  if (code == 0) return "ok";
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  switch (-code) {
    case TYR_ATTN_ERR_NULL: return "tyr_b200_attn: a required pointer is NULL";
    case TYR_ATTN_ERR_SHAPE: return "tyr_b200_attn: bad shape (sizes must be positive, n_head % n_kv_head == 0)";
    case TYR_ATTN_ERR_HEAD_DIM: return "tyr_b200_attn: head_dim must be 64 or 128 (<= 256 in check mode)";
    case TYR_ATTN_ERR_ALIGN: return "tyr_b200_attn: pointers need 16-byte alignment and strides multiples of 8 elements";
    case TYR_ATTN_ERR_DTYPE: return "tyr_b200_attn: dtype must be bf16 (fp32 only in check mode)";
    case TYR_ATTN_ERR_DROPOUT: return "tyr_b200_attn: dropout_p must be 0";
    case TYR_ATTN_ERR_WORKSPACE: return "tyr_b200_attn: decode workspace missing or too small";
    case TYR_ATTN_ERR_NO_DEVICE: return "tyr_b200_attn: no usable CUDA device or driver entry point";
    case TYR_ATTN_ERR_DEVICE_WAIT: return "tyr_b200_attn: a bounded in-kernel wait gave up";
    case TYR_ATTN_ERR_TOO_LARGE: return "tyr_b200_attn: size beyond the supported maximum";
    case TYR_ATTN_ERR_RANGE: return "tyr_b200_attn: a cache position or sequence length lies outside its limits";
    default: return "tyr_b200_attn: unknown error";
  }
}

int tyr_b200_attn_abi_version(void) { return TYR_ATTN_ABI_VERSION; }

uint64_t tyr_b200_attn_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
