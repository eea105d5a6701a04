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
//   flux.applyRope        Tyr/Model/Flux/RoPE.lean:71-96       (the interleaved-pair rotary with a 2x2 table per pair)
// about ten elementwise ATen kernels and one full-cache copy per token.  Arithmetic is
// fp32 with one rounding to bf16 at the end.  HBM-bound: one read and one write per element.
#include <cuda_bf16.h>

#include "attn_internal.h"
#include "ptx_sm100.cuh"

namespace tyr {
namespace {

constexpr int kWarps = 8;
// Heads whose loads are issued before the first is used, and CTAs per SM the register budget is
// held to.  Measured on 16 x 4096 tokens x 8 heads x 128: (4, 1) 5.36 TB/s, (8, 1) 4.31, (4, 3) 5.71,
// (2, 4) 5.38; streaming load/store hints changed nothing.
constexpr int kHeadsInFlight = 4;
constexpr int kMinCtasPerSm = 3;  // 2 for the Flux rotary form, whose 32 table values per lane would spill

struct PrologueParams {
  const __nv_bfloat16* x;
  __nv_bfloat16* out;
  const float *w, *cs, *sn, *pe;
  const int32_t* positions;
  int position0, batch, seq, n_head, d, cap, max_pos, out_at_row0;
  int64_t xs[3], os[3], pe_bs;
  float eps;
  int* status;
};

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// D/16 lanes per TOKEN: a lane owns elements [8k, 8k+8) of BOTH halves of a head's row (two
// 16-byte loads), so every rotate-half pair (i, i + D/2) and every interleaved pair (2i, 2i+1)
// lives in one lane.  The lane group walks over the heads of its token, kHeadsInFlight rows of
// loads in flight at a time, and keeps the token's rotary row and the norm weight in registers
// (they are the same for every head).  A warp covers 512/D consecutive tokens, so for one
// head its stores are 512/D consecutive rows of the [batch, head, seq, dim] output.
// kRot: 0 = no rotary, 1 = rotate-half with cos/sin tables, 2 = interleaved pairs with 2x2 tables.
template <int D, int kRot>
__global__ void __launch_bounds__(kWarps * 32, kRot == 2 ? 2 : kMinCtasPerSm)
prologue_kernel(const PrologueParams p) {
  constexpr int kHalf = D / 2;
  constexpr int kLanes = D / 16;          // lanes per token
  constexpr int kTokPerWarp = 32 / kLanes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / kLanes, k8 = (lane % kLanes) * 8;
  const int64_t tokens = (int64_t)p.batch * p.seq;
  const int64_t tok = ((int64_t)blockIdx.x * kWarps + warp) * kTokPerWarp + sub;
  const bool live = tok < tokens;
  const int64_t tt = live ? tok : tokens - 1;  // idle lane groups redo the last token and skip the stores
  const int s = (int)(tt % p.seq);
  const int b = (int)(tt / p.seq);
  const int64_t pos = (int64_t)(p.positions ? p.positions[b] : p.position0) + s;  // output row and rotary row
  // a row outside the cache or the rotary table is skipped and reported, never written
  const int64_t out_row = p.out_at_row0 ? s : pos;
  const bool in_range = pos >= 0 && out_row < p.cap && (kRot == 0 || pos < p.max_pos);
  if (live && !in_range && k8 == 0) atomicOr(p.status, kStatusOutOfRange);
  const bool store = live && in_range;
  const int64_t pos_ld = in_range ? pos : 0;

  float wa[8], wc[8];
  if (p.w != nullptr) {
    load8(p.w + k8, wa);
    load8(p.w + kHalf + k8, wc);
  }
  float ra[16], rc[16];  // rotary coefficients of this lane's elements (kRot 1: 8 cos in ra, 8 sin in rc)
  if (kRot == 1) {
    load8(p.cs + pos_ld * kHalf + k8, reinterpret_cast<float(&)[8]>(ra[0]));
    load8(p.sn + pos_ld * kHalf + k8, reinterpret_cast<float(&)[8]>(rc[0]));
  } else if (kRot == 2) {
    // elements [k8, k8+8) are pairs k8/2 .. k8/2+3: 16 floats; the second half's pairs follow D/4 later
    const float* t = p.pe + b * p.pe_bs + pos_ld * (2 * D);
    load8(t + (k8 / 2) * 4, reinterpret_cast<float(&)[8]>(ra[0]));
    load8(t + (k8 / 2) * 4 + 8, reinterpret_cast<float(&)[8]>(ra[8]));
    load8(t + ((kHalf + k8) / 2) * 4, reinterpret_cast<float(&)[8]>(rc[0]));
    load8(t + ((kHalf + k8) / 2) * 4 + 8, reinterpret_cast<float(&)[8]>(rc[8]));
  }

  const __nv_bfloat16* xt = p.x + b * p.xs[0] + s * p.xs[1];
  __nv_bfloat16* ot = p.out + b * p.os[0] + (in_range ? out_row : 0) * p.os[2];

  for (int h0 = 0; h0 < p.n_head; h0 += kHeadsInFlight) {
    uint4 raw_a[kHeadsInFlight], raw_c[kHeadsInFlight];
#pragma unroll
    for (int u = 0; u < kHeadsInFlight; ++u) {
      const int h = min(h0 + u, p.n_head - 1);
      const __nv_bfloat16* xr = xt + h * p.xs[2];
      raw_a[u] = *reinterpret_cast<const uint4*>(xr + k8);
      raw_c[u] = *reinterpret_cast<const uint4*>(xr + kHalf + k8);
    }
#pragma unroll
    for (int u = 0; u < kHeadsInFlight; ++u) {
      float a[8], c[8];
      const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&raw_a[u]);
      const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&raw_c[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fa = __bfloat1622float2(pa[i]), fc = __bfloat1622float2(pc[i]);
        a[2 * i] = fa.x; a[2 * i + 1] = fa.y; c[2 * i] = fc.x; c[2 * i + 1] = fc.y;
      }
      if (p.w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += a[i] * a[i] + c[i] * c[i];
#pragma unroll
        for (int o = kLanes / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          a[i] *= inv * wa[i];
          c[i] *= inv * wc[i];
        }
      }
      if (kRot == 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float y1 = a[i] * ra[i] - c[i] * rc[i], y2 = a[i] * rc[i] + c[i] * ra[i];
          a[i] = y1;
          c[i] = y2;
        }
      } else if (kRot == 2) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a0 = a[2 * i], a1 = a[2 * i + 1], c0 = c[2 * i], c1 = c[2 * i + 1];
          a[2 * i] = ra[4 * i] * a0 + ra[4 * i + 1] * a1;
          a[2 * i + 1] = ra[4 * i + 2] * a0 + ra[4 * i + 3] * a1;
          c[2 * i] = rc[4 * i] * c0 + rc[4 * i + 1] * c1;
          c[2 * i + 1] = rc[4 * i + 2] * c0 + rc[4 * i + 3] * c1;
        }
      }
      if (store && h0 + u < p.n_head) {
        uint4 oa, oc;
        __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
        __nv_bfloat162* qc = reinterpret_cast<__nv_bfloat162*>(&oc);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          qa[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
          qc[i] = __floats2bfloat162_rn(c[2 * i], c[2 * i + 1]);
        }
        __nv_bfloat16* orow = ot + (int64_t)(h0 + u) * p.os[1];
        *reinterpret_cast<uint4*>(orow + k8) = oa;
        *reinterpret_cast<uint4*>(orow + kHalf + k8) = oc;
      }
    }
  }
}

template <int D>
int launch_d(const PrologueParams& p, unsigned blocks, cudaStream_t st) {
  if (p.pe != nullptr) prologue_kernel<D, 2><<<blocks, kWarps * 32, 0, st>>>(p);
  else if (p.cs != nullptr) prologue_kernel<D, 1><<<blocks, kWarps * 32, 0, st>>>(p);
  else prologue_kernel<D, 0><<<blocks, kWarps * 32, 0, st>>>(p);
  return 0;
}

}  // namespace

int launch_qk_prologue(const TyrAttnPrologueArgs& a, int* status, cudaStream_t st) {
  PrologueParams p;
  p.x = static_cast<const __nv_bfloat16*>(a.x);
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.w = a.norm_weight;
  p.cs = a.cos;
  p.sn = a.sin;
  p.pe = a.pe;
  p.pe_bs = a.pe_batch_stride;
  p.positions = a.positions;
  p.position0 = a.position0;
  p.batch = a.batch; p.seq = a.seq; p.n_head = a.n_head; p.d = a.head_dim;
  p.cap = a.cap; p.max_pos = a.max_pos; p.out_at_row0 = a.out_at_row0;
  for (int i = 0; i < 3; ++i) { p.xs[i] = a.x_stride[i]; p.os[i] = a.out_stride[i]; }
  p.eps = a.eps;
  p.status = status;
  const int64_t tokens = (int64_t)a.batch * a.seq;
  const int tok_per_block = kWarps * (512 / a.head_dim);
  const int64_t blocks = (tokens + tok_per_block - 1) / tok_per_block;
  if (blocks > 0x7fffffffLL) return -TYR_ATTN_ERR_TOO_LARGE;
  if (a.head_dim == 128) launch_d<128>(p, (unsigned)blocks, st);
  else if (a.head_dim == 64) launch_d<64>(p, (unsigned)blocks, st);
  else if (a.head_dim == 256) launch_d<256>(p, (unsigned)blocks, st);
  else return -TYR_ATTN_ERR_HEAD_DIM;
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace tyr
