// Check-mode attention forward: plain fp32 FMA arithmetic, no tensor cores.
// One warp per query row, keys visited 32 at a time, online softmax with
// accurate expf/logf.  Accepts bf16 or fp32 tensors and any head_dim <= 256.
// It exists to bound the tensor-core kernel's error from the device side and to
// give callers an fp32-accumulate path; it states the same arithmetic as the
// reference's fixture generator (Examples/GPU/RunFlashAttn.lean:30-48) in the
// online form of Tyr/GPU/Codegen/Macros.lean:121-163.
#include <cuda_bf16.h>

#include "attn_internal.h"

namespace tyr {
namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxD = 256;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void from_f32(float* p, float x) { *p = x; }
__device__ __forceinline__ void from_f32(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

struct CheckParams {
  const void *q, *k, *v;
  void* o;
  float* lse;
  int batch, n_head, n_kv_head, q_seq, kv_seq, d, causal, window;
  int64_t qs[3], ks[3], vs[3], os[3];
  const uint8_t* key_mask;  // [batch, kv_seq], 0 = padding key; or null
  int64_t key_mask_stride;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
check_kernel(const CheckParams p) {
  __shared__ float q_sh[kWarpsPerBlock][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_id = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  const int64_t total = (int64_t)p.batch * p.n_head * p.q_seq;
  if (row_id >= total) return;
  const int i = (int)(row_id % p.q_seq);
  const int h = (int)((row_id / p.q_seq) % p.n_head);
  const int b = (int)(row_id / ((int64_t)p.q_seq * p.n_head));
  const int hk = h / (p.n_head / p.n_kv_head);
  const int D = p.d;

  const T* q = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + i * p.qs[2];
  const T* kbase = static_cast<const T*>(p.k) + b * p.ks[0] + hk * p.ks[1];
  const T* vbase = static_cast<const T*>(p.v) + b * p.vs[0] + hk * p.vs[1];
  for (int d = lane; d < D; d += 32) q_sh[warp][d] = to_f32(q[d]);
  __syncwarp();

  const int n_keys = p.causal ? min(p.kv_seq, i + 1) : p.kv_seq;  // key j masked when j > i
  const int key_lo = p.window > 0 ? max(0, i - p.window + 1) : 0;  // and when i - j >= window
  float m = -INFINITY, l = 0.f;
  float acc[kMaxD / 32];
#pragma unroll
  for (int x = 0; x < kMaxD / 32; ++x) acc[x] = 0.f;

  for (int k0 = key_lo; k0 < n_keys; k0 += 32) {
    const int key = k0 + lane;
    float s = -INFINITY;
    const bool seen = key < n_keys && (p.key_mask == nullptr || p.key_mask[b * p.key_mask_stride + key] != 0);
    if (seen) {
      const T* kr = kbase + (int64_t)key * p.ks[2];
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(q_sh[warp][d], to_f32(kr[d]), dot);
      s = dot * p.scale;
    }
    float mx = s;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float m_new = fmaxf(m, mx);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float pr = (seen && m_new != -INFINITY) ? expf(s - m_new) : 0.f;
    float ps = pr;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l = l * alpha + ps;
    m = m_new;
    // block-local partial sums keep the long accumulation short
    float part[kMaxD / 32];
#pragma unroll
    for (int x = 0; x < kMaxD / 32; ++x) part[x] = 0.f;
    const int nk = min(32, n_keys - k0);
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pr, kk);
      const T* vr = vbase + (int64_t)(k0 + kk) * p.vs[2];
#pragma unroll
      for (int x = 0; x < kMaxD / 32; ++x) {
        const int d = lane + 32 * x;
        if (d < D) part[x] = fmaf(pk, to_f32(vr[d]), part[x]);
      }
    }
#pragma unroll
    for (int x = 0; x < kMaxD / 32; ++x) acc[x] = acc[x] * alpha + part[x];
  }

  T* o = static_cast<T*>(p.o) + b * p.os[0] + h * p.os[1] + i * p.os[2];
  const float inv = 1.0f / l;
#pragma unroll
  for (int x = 0; x < kMaxD / 32; ++x) {
    const int d = lane + 32 * x;
    if (d < D) from_f32(o + d, acc[x] * inv);
  }
  if (lane == 0 && p.lse != nullptr)
    p.lse[((int64_t)b * p.n_head + h) * p.q_seq + i] = m + logf(l);
}

}  // namespace

int launch_prefill_check(const TyrAttnPrefillArgs& a, float scale, cudaStream_t st) {
  if (a.head_dim > kMaxD) return -TYR_ATTN_ERR_HEAD_DIM;
  CheckParams p;
  p.q = a.q; p.k = a.k; p.v = a.v; p.o = a.o; p.lse = a.lse;
  p.batch = a.batch; p.n_head = a.n_head; p.n_kv_head = a.n_kv_head;
  p.q_seq = a.q_seq; p.kv_seq = a.kv_seq; p.d = a.head_dim;
  p.causal = (a.is_causal || a.window_size > 0) ? 1 : 0;
  p.window = a.window_size > 0 ? a.window_size : 0;
  p.key_mask = a.key_mask;
  p.key_mask_stride = a.key_mask_stride;
  for (int i = 0; i < 3; ++i) {
    p.qs[i] = a.q_stride[i]; p.ks[i] = a.k_stride[i]; p.vs[i] = a.v_stride[i]; p.os[i] = a.o_stride[i];
  }
  p.scale = scale;
  const int64_t rows = (int64_t)a.batch * a.n_head * a.q_seq;
  const int64_t blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7fffffffLL) return -TYR_ATTN_ERR_TOO_LARGE;
  if (a.dtype == TYR_ATTN_F32)
    check_kernel<float><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, st>>>(p);
  else
    check_kernel<__nv_bfloat16><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, st>>>(p);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace tyr
