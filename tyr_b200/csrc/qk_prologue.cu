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

// One warp per (batch, token, head) row.  Lane l owns elements {2l, 2l+1} (+64k) of each
// half of the row, so a rotary pair (i, i + d/2) lives in one lane.
template <int D>
__global__ void __launch_bounds__(kWarps * 32)
prologue_kernel(const PrologueParams p) {
  constexpr int kHalf = D / 2;
  constexpr int kPer = kHalf / 64 > 0 ? kHalf / 64 : 1;  // bf16x2 pairs per lane per half
  constexpr bool kNarrow = kHalf < 64;                   // d = 64: one element per lane per half
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarps + warp;
  const int64_t rows = (int64_t)p.batch * p.seq * p.n_head;
  if (row >= rows) return;
  const int h = (int)(row % p.n_head);
  const int s = (int)((row / p.n_head) % p.seq);
  const int b = (int)(row / ((int64_t)p.n_head * p.seq));
  const int pos = (p.positions ? p.positions[b] : p.position0) + s;  // output row and rotary position

  const __nv_bfloat16* xr = p.x + b * p.xs[0] + s * p.xs[1] + h * p.xs[2];
  __nv_bfloat16* orow = p.out + b * p.os[0] + h * p.os[1] + (int64_t)pos * p.os[2];

  float x1[2 * kPer], x2[2 * kPer];
  float ss = 0.f;
  if (kNarrow) {
    x1[0] = __bfloat162float(xr[lane]);
    x2[0] = __bfloat162float(xr[kHalf + lane]);
    ss = x1[0] * x1[0] + x2[0] * x2[0];
  } else {
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      const int i = 64 * k + 2 * lane;
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + i));
      const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + kHalf + i));
      x1[2 * k] = a.x; x1[2 * k + 1] = a.y; x2[2 * k] = c.x; x2[2 * k + 1] = c.y;
      ss += a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
    }
  }
  float inv = 1.f;
  if (p.w != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    inv = rsqrtf(ss / (float)D + p.eps);
  }
  constexpr int kN = kNarrow ? 1 : 2 * kPer;
#pragma unroll
  for (int e = 0; e < kN; ++e) {
    const int i = kNarrow ? lane : 64 * (e >> 1) + 2 * lane + (e & 1);
    float a = x1[e], c = x2[e];
    if (p.w != nullptr) {
      a *= inv * p.w[i];
      c *= inv * p.w[kHalf + i];
    }
    if (p.cs != nullptr) {
      const float co = p.cs[(int64_t)pos * kHalf + i], si = p.sn[(int64_t)pos * kHalf + i];
      const float y1 = a * co - c * si, y2 = a * si + c * co;
      a = y1;
      c = y2;
    }
    x1[e] = a;
    x2[e] = c;
  }
  if (kNarrow) {
    orow[lane] = __float2bfloat16_rn(x1[0]);
    orow[kHalf + lane] = __float2bfloat16_rn(x2[0]);
  } else {
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      const int i = 64 * k + 2 * lane;
      *reinterpret_cast<__nv_bfloat162*>(orow + i) = __floats2bfloat162_rn(x1[2 * k], x1[2 * k + 1]);
      *reinterpret_cast<__nv_bfloat162*>(orow + kHalf + i) = __floats2bfloat162_rn(x2[2 * k], x2[2 * k + 1]);
    }
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
  const int64_t blocks = (rows + kWarps - 1) / kWarps;
  if (blocks > 0x7fffffffLL) return -TYR_ATTN_ERR_TOO_LARGE;
  if (a.head_dim == 128) prologue_kernel<128><<<(unsigned)blocks, kWarps * 32, 0, st>>>(p);
  else if (a.head_dim == 64) prologue_kernel<64><<<(unsigned)blocks, kWarps * 32, 0, st>>>(p);
  else if (a.head_dim == 256) prologue_kernel<256><<<(unsigned)blocks, kWarps * 32, 0, st>>>(p);
  else return -TYR_ATTN_ERR_HEAD_DIM;
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace tyr
