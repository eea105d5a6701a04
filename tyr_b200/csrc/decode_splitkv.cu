// Split-KV flash-decoding for one query token per sequence over a ragged KV
// cache, plus the LSE merge of the partial results.
//
// Replaces the q_seq = 1 call of QwenAttention.forwardStep
// (Tyr/Model/Qwen/Attention.lean:198-200 -> cc/src/tyr.cpp:4100-4133), which
// repeat_interleaves the whole cache per token.  Here every K/V byte is read
// from HBM exactly once: one CTA owns (sequence, KV head, chunk of keys) and
// serves all query heads of that KV head together.  The merge is the formula of
// ringAttnReduce (Tyr/GPU/Kernels/RingAttn.lean:164-180), kept in the log2 domain.
//
// The kernel is HBM-bound.  Keys stream global -> shared with 16-byte cp.async
// into a 3-stage ring (XOR-swizzled rows, conflict-free for ldmatrix); the tiny
// contractions (<=16 query rows) run on warp-level m16n8k16 MMAs so that issue
// slots stay free for the loads.  Each warp owns 16 of the 64 keys of a stage and
// keeps its own (max, sum, O); the four warps merge through shared memory.
#include <cuda_bf16.h>

#include <mutex>

#include "attn_internal.h"
#include "mma_sync.cuh"
#include "ptx_sm100.cuh"

namespace tyr {
namespace {

constexpr int kThreads = 128;
constexpr int kTileKeys = 64;   // keys per pipeline stage
constexpr int kStages = 3;
constexpr int kMinChunk = 256;  // keys; shorter chunks only add merge traffic
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct DecodeParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* o;
  float* lse;
  const __nv_bfloat16 *k, *v;
  const void* const* k_ptrs;
  const void* const* v_ptrs;
  const int32_t* kv_lens;
  const int64_t* kv_head_strides;
  int batch, n_head, n_kv_head, max_kv_seq, group, head_groups;
  int64_t qs[2], os[2], ks[3], vs[3];
  float scale_log2;
  int chunk_len, n_splits;
  float* ws_o;    // [batch, n_head, n_splits, D] normalised partial outputs
  float* ws_lse;  // [batch, n_head, n_splits] log2-domain partial LSE
  int* status;    // per-device status word (out-of-range lengths are reported there)
};

// A length outside [1, max_kv_seq] (the workspace and the grid are sized for max_kv_seq, so a
// longer one would index past both): report it once per sequence, give a sequence without any
// key a defined row (zeros, LSE = -inf), and return the length forced into [0, max_kv_seq].
// Kept out of line so that this rare path costs the scan loop no registers.
template <int D>
__device__ __noinline__ int bad_length(int raw, int max_kv_seq, bool first_cta_of_row, int* status,
                                       __nv_bfloat16* o_row0, int64_t o_head_stride, float* lse_row0,
                                       int head0, int heads_here) {
  const int len = min(max(raw, 0), max_kv_seq);
  if (first_cta_of_row) {
    if (threadIdx.x == 0 && head0 == 0) atomicOr(status, kStatusOutOfRange);
    if (len == 0) {
      for (int idx = threadIdx.x; idx < heads_here * D; idx += blockDim.x) {
        const int head = head0 + idx / D, d = idx % D;
        o_row0[(int64_t)head * o_head_stride + d] = __float2bfloat16_rn(0.f);
        if (d == 0 && lse_row0) lse_row0[head] = -INFINITY;
      }
    }
  }
  return len;
}

template <int D>
struct DCfg {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kChunksPerRow = D / 8;  // 16-byte chunks
  static constexpr int kTileBytes = kTileKeys * kRowBytes;
  static constexpr int kStageBytes = 2 * kTileBytes;  // K then V
  static constexpr int kSmemBytes = kStages * kStageBytes;
  // cross-warp merge reuses the ring: 4 warps x 16 rows of D floats, rows padded by 4 floats so that
  // the eight rows a warp stores at once fall on different banks, + 2 floats of (max, sum) per row
  static constexpr int kMergeStride = D + 4;
  static_assert(4 * 16 * (kMergeStride + 2) * 4 <= kSmemBytes, "merge scratch fits in the ring");
};

template <int D>
__global__ void __launch_bounds__(kThreads)
decode_kernel(const DecodeParams p) {
  using C = DCfg<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem));

  // the merge kernel behind this one may start to become resident (it waits for this grid itself)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int split = blockIdx.x;
  const int hkv = blockIdx.y / p.head_groups;
  const int hg = blockIdx.y % p.head_groups;
  const int b = blockIdx.z;
  int len = p.kv_lens ? p.kv_lens[b] : p.max_kv_seq;
  if (len <= 0 || len > p.max_kv_seq)
    len = bad_length<D>(len, p.max_kv_seq, split == 0, p.status, p.o + b * p.os[0], p.os[1],
                        p.lse ? p.lse + (int64_t)b * p.n_head : nullptr, hkv * p.group + hg * 16,
                        min(16, p.group - hg * 16));
  const int n_chunks = (len + p.chunk_len - 1) / p.chunk_len;
  if (split >= n_chunks) return;
  const int key_begin = split * p.chunk_len;
  const int key_end = min(len, key_begin + p.chunk_len);
  const int n_tiles = (key_end - key_begin + kTileKeys - 1) / kTileKeys;

  const __nv_bfloat16 *kbase, *vbase;
  if (p.k_ptrs) {
    const int64_t hs_k = p.kv_head_strides ? p.kv_head_strides[b] : (int64_t)len * p.ks[2];
    const int64_t hs_v = p.kv_head_strides ? p.kv_head_strides[b] : (int64_t)len * p.vs[2];
    kbase = static_cast<const __nv_bfloat16*>(p.k_ptrs[b]) + hkv * hs_k;
    vbase = static_cast<const __nv_bfloat16*>(p.v_ptrs[b]) + hkv * hs_v;
  } else {
    kbase = p.k + b * p.ks[0] + hkv * p.ks[1];
    vbase = p.v + b * p.vs[0] + hkv * p.vs[1];
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = lane >> 2, t4 = lane & 3;

  // ---- stage loader: 64 keys x D bf16 of K and of V, 16 bytes per cp.async
  auto load_tile = [&](int tile, int stage) {
    const uint32_t sk = sbase + stage * C::kStageBytes, sv = sk + C::kTileBytes;
    const int k0 = key_begin + tile * kTileKeys;
#pragma unroll
    for (int it = 0; it < kTileKeys * C::kChunksPerRow / kThreads; ++it) {
      const int idx = it * kThreads + tid;
      const int kr = idx / C::kChunksPerRow, c = idx % C::kChunksPerRow;
      const int key = min(k0 + kr, key_end - 1);  // rows past the end re-read the last valid key
      cp_async16(sk + sw_off<D>(kr, c), kbase + (int64_t)key * p.ks[2] + c * 8);
      cp_async16(sv + sw_off<D>(kr, c), vbase + (int64_t)key * p.vs[2] + c * 8);
    }
  };

  // ---- Q fragments (A operand, 16 rows = query heads of this KV head)
  const int head0 = hkv * p.group + hg * 16;       // first query head of this CTA
  const int heads_here = min(16, p.group - hg * 16);
  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* qb = p.q + b * p.qs[0];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {      // rows quad, quad + 8
        const int r = quad + half * 8;
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {          // d, d + 8
          uint32_t val = 0;
          if (r < heads_here)
            val = *reinterpret_cast<const uint32_t*>(qb + (int64_t)(head0 + r) * p.qs[1] + ks * 16 +
                                                     kh * 8 + t4 * 2);
          qa[ks][half + 2 * kh] = val;
        }
      }
    }
  }

#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_tiles) load_tile(s, s);
    cp_async_commit();
  }

  float m_run[2] = {-INFINITY, -INFINITY};  // rows quad, quad + 8 (log2 domain)
  float l_run[2] = {0.f, 0.f};
  float oacc[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int x = 0; x < 4; ++x) oacc[n][x] = 0.f;

  for (int tile = 0; tile < n_tiles; ++tile) {
    cp_async_wait<kStages - 2>();
    __syncthreads();
    if (tile + kStages - 1 < n_tiles) load_tile(tile + kStages - 1, (tile + kStages - 1) % kStages);
    cp_async_commit();

    const int stage = tile % kStages;
    const uint32_t sk = sbase + stage * C::kStageBytes, sv = sk + C::kTileBytes;
    const int wkey0 = warp * 16;                              // this warp's keys in the tile
    const int gkey0 = key_begin + tile * kTileKeys + wkey0;   // global index of the first
    if (gkey0 >= key_end) continue;                           // warp-uniform: nothing valid

    // S = Q K^T for 16 keys: two n-tiles of 8 keys
    float sacc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int x = 0; x < 4; ++x) sacc[n][x] = 0.f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int c = 0; c < C::kChunksPerRow; c += 4) {
        uint32_t kb[4];
        ldsm_x4(sk + sw_off<D>(wkey0 + n * 8 + (lane & 7), c + (lane >> 3)), kb);
        mma_bf16_16816(sacc[n], qa[c / 2], kb[0], kb[1]);
        mma_bf16_16816(sacc[n], qa[c / 2 + 1], kb[2], kb[3]);
      }
    }
    // scale, mask the tail, online softmax per row (rows quad and quad+8)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int key = gkey0 + n * 8 + t4 * 2 + (x & 1);
        const float sv2 = (key < key_end) ? sacc[n][x] * p.scale_log2 : -INFINITY;
        sacc[n][x] = sv2;
        mx[x >> 1] = fmaxf(mx[x >> 1], sv2);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);  // finite: key gkey0 is valid
      alpha[h] = ex2f(m_run[h] - m_new);           // 0 on the first tile
      m_run[h] = m_new;
    }
    float ps[2] = {0.f, 0.f};
    uint32_t pa[4];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const float p0 = ex2f(sacc[n][0] - m_run[0]), p1 = ex2f(sacc[n][1] - m_run[0]);
      const float p2 = ex2f(sacc[n][2] - m_run[1]), p3 = ex2f(sacc[n][3] - m_run[1]);
      ps[0] += p0 + p1;
      ps[1] += p2 + p3;
      pa[2 * n] = pack2(p0, p1);      // rows quad,   keys n*8 + t4*2..
      pa[2 * n + 1] = pack2(p2, p3);  // rows quad+8
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      ps[h] += __shfl_xor_sync(0xffffffffu, ps[h], 1);
      ps[h] += __shfl_xor_sync(0xffffffffu, ps[h], 2);
      l_run[h] = l_run[h] * alpha[h] + ps[h];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      oacc[n][0] *= alpha[0];
      oacc[n][1] *= alpha[0];
      oacc[n][2] *= alpha[1];
      oacc[n][3] *= alpha[1];
    }
    // O += P V : k = this warp's 16 keys, n-tiles of 8 output dims
#pragma unroll
    for (int c = 0; c < C::kChunksPerRow; c += 2) {
      uint32_t vb[4];
      ldsm_x4_trans(sv + sw_off<D>(wkey0 + (lane & 7) + ((lane >> 3) & 1) * 8, c + (lane >> 4)), vb);
      mma_bf16_16816(oacc[c], pa, vb[0], vb[1]);
      mma_bf16_16816(oacc[c + 1], pa, vb[2], vb[3]);
    }
  }

  // ---- merge the four warps through shared memory
  cp_async_wait<0>();
  __syncthreads();
  constexpr int kMS = C::kMergeStride;
  float* sc_o = reinterpret_cast<float*>(smem);               // [4][16][D + 4]
  float* sc_ml = sc_o + 4 * 16 * kMS;                         // [4][16][2]
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int d = n * 8 + t4 * 2;
    float* r0 = sc_o + (warp * 16 + quad) * kMS + d;
    float* r1 = sc_o + (warp * 16 + quad + 8) * kMS + d;
    r0[0] = oacc[n][0]; r0[1] = oacc[n][1];
    r1[0] = oacc[n][2]; r1[1] = oacc[n][3];
  }
  if (t4 == 0) {
    sc_ml[(warp * 16 + quad) * 2] = m_run[0];
    sc_ml[(warp * 16 + quad) * 2 + 1] = l_run[0];
    sc_ml[(warp * 16 + quad + 8) * 2] = m_run[1];
    sc_ml[(warp * 16 + quad + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  for (int idx = tid; idx < heads_here * D; idx += kThreads) {
    const int r = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sc_ml[(w * 16 + r) * 2]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sc_ml[(w * 16 + r) * 2];
      const float f = (mw == -INFINITY) ? 0.f : ex2f(mw - M);
      L += sc_ml[(w * 16 + r) * 2 + 1] * f;
      acc += sc_o[(w * 16 + r) * kMS + d] * f;
    }
    const int head = head0 + r;
    const float outv = acc / L;
    const float lse2 = M + log2f(L);
    if (n_chunks == 1) {
      p.o[b * p.os[0] + (int64_t)head * p.os[1] + d] = __float2bfloat16_rn(outv);
      if (d == 0 && p.lse) p.lse[(int64_t)b * p.n_head + head] = kLn2 * lse2;
    } else {
      const int64_t slot = ((int64_t)b * p.n_head + head) * p.n_splits + split;
      p.ws_o[slot * D + d] = outv;
      if (d == 0) p.ws_lse[slot] = lse2;
    }
  }
}

// One CTA per (query head, sequence): weights w_c = 2^(L_c - max L), O = sum w_c O_c / sum w_c.
// Launched with programmatic stream serialisation: its CTAs may become resident while the split
// kernel is still draining, and wait here until that grid has completed and its writes are visible,
// so the launch latency of this second kernel hides behind the tail of the first.
template <int D>
__global__ void __launch_bounds__(D)
decode_merge_kernel(const DecodeParams p) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int len = p.kv_lens ? min(max(p.kv_lens[b], 0), p.max_kv_seq) : p.max_kv_seq;
  const int n_chunks = (len + p.chunk_len - 1) / p.chunk_len;
  if (n_chunks <= 1) return;  // the split kernel already wrote the final row
  const int64_t slot0 = ((int64_t)b * p.n_head + head) * p.n_splits;
  float M = -INFINITY;
  for (int c = 0; c < n_chunks; ++c) M = fmaxf(M, p.ws_lse[slot0 + c]);
  float W = 0.f, acc = 0.f;
  for (int c = 0; c < n_chunks; ++c) {
    const float w = ex2f(p.ws_lse[slot0 + c] - M);
    W += w;
    acc = fmaf(w, p.ws_o[(slot0 + c) * D + d], acc);
  }
  p.o[b * p.os[0] + (int64_t)head * p.os[1] + d] = __float2bfloat16_rn(acc / W);
  if (d == 0 && p.lse) p.lse[(int64_t)b * p.n_head + head] = kLn2 * (M + log2f(W));
}

// Two-way merge, natural-log LSE (the formula of RingAttn.lean:164-180).
__global__ void merge2_kernel(const float* o_a, const float* lse_a, const float* o_b,
                              const float* lse_b, float* o_out, float* lse_out, int64_t rows, int d) {
  const int64_t r = blockIdx.x;
  if (r >= rows) return;
  const float la = lse_a[r], lb = lse_b[r];
  const float mx = fmaxf(la, lb);
  const float L = (mx == -INFINITY) ? -INFINITY : mx + log1pf(expf(fminf(la, lb) - mx));
  const float wa = (la == -INFINITY) ? 0.f : expf(la - L), wb = (lb == -INFINITY) ? 0.f : expf(lb - L);
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    o_out[r * d + i] = o_a[r * d + i] * wa + o_b[r * d + i] * wb;
  __syncthreads();
  if (threadIdx.x == 0) lse_out[r] = L;
}

template <int D>
int launch_d(const TyrAttnDecodeArgs& a, DecodeParams& p, cudaStream_t st) {
  using C = DCfg<D>;
  // per-device attribute: set on every launch so that any current device is covered
  cudaError_t attr_err = cudaFuncSetAttribute(
      decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes);
  if (attr_err != cudaSuccess) return (int)attr_err;
  dim3 grid(p.n_splits, a.n_kv_head * p.head_groups, a.batch);
  decode_kernel<D><<<grid, kThreads, C::kSmemBytes, st>>>(p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (p.n_splits > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.n_head, a.batch);
    cfg.blockDim = dim3(D);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, decode_merge_kernel<D>, p);
    count_launch();
    if (e == cudaSuccess) e = cudaGetLastError();
  }
  return (int)e;
}

}  // namespace

int decode_num_splits(int max_kv_seq, int max_splits, int* chunk_len) {
  if (max_splits <= 0 || max_splits > 64) max_splits = 64;
  int chunk = (max_kv_seq + max_splits - 1) / max_splits;
  chunk = (chunk + kTileKeys - 1) / kTileKeys * kTileKeys;
  if (chunk < kMinChunk) chunk = kMinChunk;
  if (chunk_len) *chunk_len = chunk;
  return (max_kv_seq + chunk - 1) / chunk;
}

// Chunk length of a launch.  decode_num_splits gives the most chunks the workspace is sized for;
// a launch uses longer chunks than that when it can: every CTA pays for filling its load pipeline,
// the cross-warp merge and a partial output row.
//  * A launch with at least four CTAs for every CTA slot of the device at 2048-key chunks takes
//    those (64 sequences of up to 32 K keys: 5.9 -> 6.95 TB/s against 512-key chunks).
//  * A launch of fewer than three CTAs per slot at 2048-key chunks whose lengths the host knows (one
//    shared length, or the caller's total_kv_len) takes the shortest chunks that still fit in ONE
//    wave of CTAs, all resident at once: each pays its start-up once and none waits for a slot
//    (one sequence of 32 K keys: 37.1 -> 31.3 us; 4 x 32 K: 106 -> 86 us; 8 x 8 K: 66 -> 53 us;
//    eight ragged sequences of up to 32 K, 2.8 CTAs per slot: 149 -> 134 us; 8 x 32 K, 3.5 CTAs per
//    slot, lost 4 % that way and stays with the rule below).
//  * Any other launch halves the chunks from 2048 keys down while it would have fewer than four CTAs
//    per slot (by the longest sequence's count when the lengths are only on the device: ragged
//    lengths leave about half of those with work).
int decode_launch_splits(int max_kv_seq, int max_splits, int batch, int ctas_per_seq_chunk, long long total_kv_len,
                         bool lengths_known, int* chunk_len) {
  int cap_chunk = 0;
  decode_num_splits(max_kv_seq, max_splits, &cap_chunk);
  total_kv_len = std::min<long long>(total_kv_len, (long long)batch * max_kv_seq);  // a hint, not trusted beyond the shapes
  const long long slots = 2ll * sm_count();  // two CTAs are resident per SM
  // CTAs that find work with chunks of `chunk` keys
  auto ctas = [&](int chunk) -> long long {
    if (total_kv_len > 0) return ctas_per_seq_chunk * (total_kv_len / chunk + (batch + 1) / 2);
    return (long long)ctas_per_seq_chunk * batch * ((max_kv_seq + chunk - 1) / chunk);
  };
  const int whole = (max_kv_seq + kTileKeys - 1) / kTileKeys * kTileKeys;  // one chunk per sequence
  int chunk = 2048;
  if (ctas(chunk) < 4 * slots) {
    long long one_wave = 0;  // chunk length of the one-wave cut, 0 when the launch does not take it
    if (lengths_known && ctas(chunk) < 3 * slots) {
      const long long keys = total_kv_len > 0 ? total_kv_len : (long long)batch * max_kv_seq;
      long long c = (keys * ctas_per_seq_chunk + slots - 1) / slots;
      c = (c + kTileKeys - 1) / kTileKeys * kTileKeys;
      c = std::min<long long>(std::max<long long>(c, kMinChunk), whole);
      while (c < whole && ctas((int)c) > slots) c += kTileKeys;
      // short sequences, many of them: even one CTA per (sequence, KV head) is more than a wave
      if (ctas((int)c) <= slots) one_wave = c;
    }
    if (one_wave > 0) {
      chunk = (int)one_wave;
    } else {
      while (chunk > cap_chunk && ctas(chunk) < 4 * slots) chunk /= 2;
    }
  }
  if (chunk < cap_chunk) chunk = cap_chunk;  // never more chunks than the workspace holds
  *chunk_len = chunk;
  return (max_kv_seq + chunk - 1) / chunk;
}

size_t decode_workspace_bytes(int batch, int n_head, int head_dim, int max_kv_seq, int max_splits) {
  const int n = decode_num_splits(max_kv_seq, max_splits, nullptr);
  if (n <= 1) return 0;
  return (size_t)batch * n_head * n * ((size_t)head_dim + 1) * sizeof(float);
}

int launch_decode(const TyrAttnDecodeArgs& a, float scale, cudaStream_t st) {
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(a.q);
  p.o = static_cast<__nv_bfloat16*>(a.o);
  p.lse = a.lse;
  p.k = static_cast<const __nv_bfloat16*>(a.k);
  p.v = static_cast<const __nv_bfloat16*>(a.v);
  p.k_ptrs = a.k_ptrs;
  p.v_ptrs = a.v_ptrs;
  p.kv_lens = a.kv_lens;
  p.kv_head_strides = a.kv_head_strides;
  p.batch = a.batch; p.n_head = a.n_head; p.n_kv_head = a.n_kv_head; p.max_kv_seq = a.max_kv_seq;
  p.group = a.n_head / a.n_kv_head;
  p.head_groups = (p.group + 15) / 16;
  for (int i = 0; i < 2; ++i) { p.qs[i] = a.q_stride[i]; p.os[i] = a.o_stride[i]; }
  for (int i = 0; i < 3; ++i) { p.ks[i] = a.k_stride[i]; p.vs[i] = a.v_stride[i]; }
  p.scale_log2 = scale * kLog2e;
  p.n_splits = decode_launch_splits(a.max_kv_seq, a.max_splits, a.batch, a.n_kv_head * p.head_groups,
                                    a.total_kv_len > 0 ? a.total_kv_len : 0, a.kv_lens == nullptr || a.total_kv_len > 0,
                                    &p.chunk_len);
  p.ws_o = nullptr;
  p.ws_lse = nullptr;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -TYR_ATTN_ERR_NO_DEVICE;
    DeviceState* ds = device_state(dev);
    if (!ds) return -TYR_ATTN_ERR_NO_DEVICE;
    p.status = ds->status;
  }
  if (p.n_splits > 1) {
    const size_t need = decode_workspace_bytes(a.batch, a.n_head, a.head_dim, a.max_kv_seq, a.max_splits);
    if (a.workspace == nullptr || a.workspace_bytes < need) return -TYR_ATTN_ERR_WORKSPACE;
    p.ws_o = static_cast<float*>(a.workspace);
    p.ws_lse = p.ws_o + (size_t)a.batch * a.n_head * p.n_splits * a.head_dim;
  }
  if (a.head_dim == 128) return launch_d<128>(a, p, st);
  if (a.head_dim == 64) return launch_d<64>(a, p, st);
  return -TYR_ATTN_ERR_HEAD_DIM;
}

int launch_merge2(const float* o_a, const float* lse_a, const float* o_b, const float* lse_b,
                  float* o_out, float* lse_out, int64_t rows, int head_dim, cudaStream_t st) {
  if (rows > 0x7fffffffLL) return -TYR_ATTN_ERR_TOO_LARGE;
  merge2_kernel<<<(unsigned)rows, 128, 0, st>>>(o_a, lse_a, o_b, lse_b, o_out, lse_out, rows, head_dim);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace tyr

// ---------------------------------------------------------------------------
// Decode without any allocation: the split-KV scratch lives in a fixed array
// inside the library image instead of a caller-provided workspace.
// ---------------------------------------------------------------------------
namespace tyr {
namespace {

constexpr size_t kStaticScratchBytes = TYR_ATTN_DECODE_STATIC_SCRATCH_BYTES;

// Held by every GPU that loads this library until the process exits.
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

constexpr int kMaxStaticDevices = 64;
std::mutex g_static_mu;
void* g_static_scratch_ptr[kMaxStaticDevices] = {};  // device address of the array, per device

// In host code `g_decode_static_scratch` is only a stand-in for the symbol; the
// address a kernel can use has to be asked for, once per device, with that device current.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxStaticDevices) return -TYR_ATTN_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (ptr == nullptr) return -TYR_ATTN_ERR_NO_DEVICE;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}

}  // namespace
}  // namespace tyr

extern "C" int tyr_b200_attn_decode_static(const TyrAttnDecodeArgs* args, void* stream) {
  using namespace tyr;
  if (args == nullptr) return -TYR_ATTN_ERR_NULL;
  if (args->batch <= 0 || args->n_head <= 0 || args->head_dim <= 0 || args->max_kv_seq <= 0)
    return -TYR_ATTN_ERR_SHAPE;
  const size_t need = decode_workspace_bytes(args->batch, args->n_head, args->head_dim,
                                             args->max_kv_seq, args->max_splits);
  if (need > kStaticScratchBytes) return -TYR_ATTN_ERR_TOO_LARGE;
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // Nothing in the scratch has to start at zero: the split kernel writes every
  // (row, chunk) slot the merge kernel later reads, so stale contents of an
  // earlier call are never observed.
  TyrAttnDecodeArgs a = *args;
  a.workspace = scratch;
  a.workspace_bytes = kStaticScratchBytes;
  return tyr_b200_attn_decode(&a, stream);
}
