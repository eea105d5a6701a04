// Fused prologue of the attention call: per-head RMSNorm, rotary embedding and the
// [batch, seq, head, dim] -> [batch, head, seq, dim] layout change in one pass,
// written either to a fresh Q/K/V tensor or straight into the KV cache at each
// sequence's current length (in-place append).
//
// Replaces, for one projected tensor, the chain Tyr runs before every attention call:
//   applyHeadNorm        Tyr/Model/Qwen/Attention.lean:73-98  (x * rsqrt(mean(x^2) + eps) * weight)
//   rotary.applyRotaryEmb cc/src/tyr.cpp:3824-3861             ([x1,x2] -> [x1*cos - x2*sin, x1*sin + x2*cos])
//   transpose_for_attention cc/src/tyr.cpp:2402-2414          (permute(0,2,1,3).contiguous())
//   data.sliceScatter     cc/src/tyr.cpp:2261-2277            (clone of the whole cache + copy_ of one row)
// about ten elementwise ATen kernels and one full-cache copy per token.  Arithmetic is
// fp32 with one rounding to bf16 at the end.  HBM-bound: one read and one write per element.
#include <cuda_bf16.h>

#include "attn_internal.h"

namespace tyr {
namespace {

constexpr int kWarps = 8;

struct PrologueParams {
  const __nv_bfloat16* x;
  __nv_bfloat16* out;
  const float *w, *cs, *sn;
  const int32_t* positions;
  int position0, batch, seq, n_head, d;
  int64_t xs[3], os[3];
  float eps;
};

// D/16 lanes per (batch, token, head) row: a lane owns elements [8k, 8k+8) of BOTH halves
// of the row (two 16-byte loads), so every rotary pair (i, i + D/2) lives in one lane and
// a warp covers 512/D rows per pass.
template <int D>
__global__ void __launch_bounds__(kWarps * 32)
prologue_kernel(const PrologueParams p) {
  constexpr int kHalf = D / 2;
  constexpr int kLanes = D / 16;          // lanes per row
  constexpr int kRowsPerWarp = 32 / kLanes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / kLanes, k8 = (lane % kLanes) * 8;
  const int64_t rows = (int64_t)p.batch * p.seq * p.n_head;
  const int64_t row = ((int64_t)blockIdx.x * kWarps + warp) * kRowsPerWarp + sub;
  const bool live = row < rows;
  const int64_t rr = live ? row : rows - 1;  // idle lanes redo the last row and skip the store
  const int h = (int)(rr % p.n_head);
  const int s = (int)((rr / p.n_head) % p.seq);
  const int b = (int)(rr / ((int64_t)p.n_head * p.seq));
  const int pos = (p.positions ? p.positions[b] : p.position0) + s;  // output row and rotary position

  const __nv_bfloat16* xr = p.x + b * p.xs[0] + s * p.xs[1] + h * p.xs[2];
  __nv_bfloat16* orow = p.out + b * p.os[0] + h * p.os[1] + (int64_t)pos * p.os[2];

  const uint4 ra = *reinterpret_cast<const uint4*>(xr + k8);
  const uint4 rc = *reinterpret_cast<const uint4*>(xr + kHalf + k8);
  float a[8], c[8];
  {
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
    const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&rc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 fa = __bfloat1622float2(pa[i]), fc = __bfloat1622float2(pc[i]);
      a[2 * i] = fa.x; a[2 * i + 1] = fa.y; c[2 * i] = fc.x; c[2 * i + 1] = fc.y;
    }
  }
  if (p.w != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + c[i] * c[i];
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)D + p.eps);
    const float4 w0 = *reinterpret_cast<const float4*>(p.w + k8), w1 = *reinterpret_cast<const float4*>(p.w + k8 + 4);
    const float4 w2 = *reinterpret_cast<const float4*>(p.w + kHalf + k8), w3 = *reinterpret_cast<const float4*>(p.w + kHalf + k8 + 4);
    const float wa[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    const float wc[8] = {w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] *= inv * wa[i];
      c[i] *= inv * wc[i];
    }
  }
  if (p.cs != nullptr) {
    const float* cp = p.cs + (int64_t)pos * kHalf + k8;
    const float* sp = p.sn + (int64_t)pos * kHalf + k8;
    const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
    const float co[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float si[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float y1 = a[i] * co[i] - c[i] * si[i], y2 = a[i] * si[i] + c[i] * co[i];
      a[i] = y1;
      c[i] = y2;
    }
  }
  if (live) {
    uint4 oa, oc;
    __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* qc = reinterpret_cast<__nv_bfloat162*>(&oc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      qa[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
      qc[i] = __floats2bfloat162_rn(c[2 * i], c[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(orow + k8) = oa;
    *reinterpret_cast<uint4*>(orow + kHalf + k8) = oc;
  }
}

}  // namespace

int launch_qk_prologue(const TyrAttnPrologueArgs& a, cudaStream_t st) {
  PrologueParams p;
  p.x = static_cast<const __nv_bfloat16*>(a.x);
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.w = a.norm_weight;
  p.cs = a.cos;
  p.sn = a.sin;
  p.positions = a.positions;
  p.position0 = a.position0;
  p.batch = a.batch; p.seq = a.seq; p.n_head = a.n_head; p.d = a.head_dim;
  for (int i = 0; i < 3; ++i) { p.xs[i] = a.x_stride[i]; p.os[i] = a.out_stride[i]; }
  p.eps = a.eps;
  const int64_t rows = (int64_t)a.batch * a.seq * a.n_head;
  const int rows_per_block = kWarps * (512 / a.head_dim);
  const int64_t blocks = (rows + rows_per_block - 1) / rows_per_block;
  if (blocks > 0x7fffffffLL) return -TYR_ATTN_ERR_TOO_LARGE;
  if (a.head_dim == 128) prologue_kernel<128><<<(unsigned)blocks, kWarps * 32, 0, st>>>(p);
  else if (a.head_dim == 64) prologue_kernel<64><<<(unsigned)blocks, kWarps * 32, 0, st>>>(p);
  else if (a.head_dim == 256) prologue_kernel<256><<<(unsigned)blocks, kWarps * 32, 0, st>>>(p);
  else return -TYR_ATTN_ERR_HEAD_DIM;
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace tyr
