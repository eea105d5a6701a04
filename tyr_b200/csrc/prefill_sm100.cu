// Flash-attention forward for sm_100a: TMA-staged Q/K/V tiles, tcgen05.mma with
// fp32 accumulators in tensor memory for S = Q K^T and O += P V, online softmax
// in the exp2 domain by two softmax warpgroups that each own one 128-row Q tile,
// P handed back to the tensor core through tensor memory, O written by TMA store.
//
// Replaces, for bf16 CUDA tensors, the ATen call behind Tyr's typed attention
// (cc/src/tyr.cpp:2578, 3941, 4126) and the SM90-only DSL kernels
// (Tyr/GPU/Kernels/MhaH100.lean:14-192, FlashAttn3.lean:70-287).  Softmax state
// follows Tyr/GPU/Codegen/Macros.lean:121-163: running max, running sum, rescale
// of the output accumulator, LSE = log(rowSum) + rowMax of the scaled scores.
//
// One CTA = 256 query rows (two 128-row tiles) of one (batch, query head).
//   warp 0     : TMA producer (one elected lane)
//   warp 1     : tcgen05.mma issuer (one elected lane)
//   warp 2     : tensor-memory allocation
//   warps 4-7  : softmax + epilogue of Q tile 0 (thread = one row = one TMEM lane)
//   warps 8-11 : softmax + epilogue of Q tile 1
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D);
// P_t (bf16, 64 columns) overwrites the first half of S_t once the row is in registers.
// Issue order S0(j+1) / PV1(j) / S1(j+1) / PV0(j+1) keeps the tensor pipe busy
// while each softmax warpgroup has two MMA slots of time per KV tile.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <mutex>

#include "attn_internal.h"
#include "ptx_sm100.cuh"

namespace tyr {
namespace {

constexpr int kBM = 128;        // query rows per tile (= TMEM lanes)
constexpr int kBN = 128;        // keys per KV tile
constexpr int kThreads = 384;   // 12 warps
constexpr float kRescaleThreshold = 8.0f;  // log2 units; below it the stale max is kept

struct PrefillParams {
  float* lse;
  int64_t lse_stride_b, lse_stride_h;
  int q_seq, kv_seq, group, causal;
  float scale_log2;  // scale * log2(e)
  int* status;
};

template <int D>
struct Cfg {
  static constexpr int kBoxes = D / 64;                // 128-byte boxes per row
  static constexpr uint32_t kBoxBytes = 128u * 128u;   // 128 rows x 128 B
  static constexpr uint32_t kTileBytes = kBoxes * kBoxBytes;
  static constexpr int kKStages = (D == 128) ? 2 : 4;
  static constexpr int kVStages = (D == 128) ? 2 : 4;
  static constexpr uint32_t kQOff = 0;
  static constexpr uint32_t kKOff = 2 * kTileBytes;
  static constexpr uint32_t kVOff = kKOff + kKStages * kTileBytes;
  static constexpr uint32_t kBarOff = kVOff + kVStages * kTileBytes;
  static constexpr int kNumBars = 2 + 2 * kKStages + 2 * kVStages + 2 + 2 + 2 + 2 + 2;
  static constexpr uint32_t kSmemBytes = kBarOff + kNumBars * 8 + 16 + 1024;  // + align slack
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kTmemS = 0, kTmemO = 256;
  static_assert(256 + 2 * D <= 512, "tensor memory budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// barrier indices
template <int D>
struct Bars {
  using C = Cfg<D>;
  static constexpr int q_full = 0;                        // [2]
  static constexpr int k_full = 2;                        // [KS]
  static constexpr int k_empty = k_full + C::kKStages;    // [KS]
  static constexpr int v_full = k_empty + C::kKStages;    // [VS]
  static constexpr int v_empty = v_full + C::kVStages;    // [VS]
  static constexpr int s_full = v_empty + C::kVStages;    // [2]
  static constexpr int p_full = s_full + 2;               // [2]
  static constexpr int o_full = p_full + 2;               // [2]
  static constexpr int e_full = o_full + 2;               // [2] epilogue rows staged in smem
  static constexpr int p_half = e_full + 2;               // [2] first 64 keys of P_t written
};

template <int D>
__device__ __forceinline__ void issue_qk(uint32_t s_tmem, uint32_t q_smem, uint32_t k_smem) {
  constexpr uint32_t idesc = umma_idesc_bf16(kBM, kBN, false);
#pragma unroll
  for (int kb = 0; kb < D / 64; ++kb) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint32_t off = kb * Cfg<D>::kBoxBytes + ks * 32;
      umma_ss(s_tmem, umma_smem_desc(q_smem + off, 16, 1024), umma_smem_desc(k_smem + off, 16, 1024),
              idesc, (kb | ks) != 0);
    }
  }
}

// `half` selects keys [64*half, 64*half + 64) of the tile.
template <int D>
__device__ __forceinline__ void issue_pv(uint32_t o_tmem, uint32_t p_tmem, uint32_t v_smem,
                                         bool accumulate, int half) {
  constexpr uint32_t idesc = umma_idesc_bf16(kBM, D, true);
#pragma unroll
  for (int k4 = 0; k4 < kBN / 32; ++k4) {
    const int kk = half * (kBN / 32) + k4;
    // 16 keys = two 8-row groups of the V tile; 16 bf16 of P = 8 TMEM columns
    umma_ts(o_tmem, p_tmem + kk * 8, umma_smem_desc(v_smem + kk * 2048, Cfg<D>::kBoxBytes, 1024),
            idesc, (accumulate || kk != 0) ? 1u : 0u);
  }
}

// exp2 of one 32-column chunk of a score row, packed to bf16x2, with the row sum.
// kPoly of every 8 column pairs go through the FMA-pipe polynomial, the rest
// through ex2.approx, so that neither unit alone bounds the softmax.
template <int kPoly>
__device__ __forceinline__ void exp_chunk(const uint32_t (&sr)[32], uint64_t sl2x2, uint64_t negx2,
                                          uint32_t (&pk)[16], uint64_t& sum_a, uint64_t& sum_b) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint64_t t2 = fma_f32x2(pack_u32x2(sr[2 * i], sr[2 * i + 1]), sl2x2, negx2);
    float p0, p1;
    if ((i & 7) < kPoly) {
      ex2_poly_x2(t2, p0, p1);
    } else {
      float t0, t1;
      unpack_f32x2(t2, t0, t1);
      p0 = ex2_approx(t0);
      p1 = ex2_approx(t1);
    }
    if (i & 1) sum_b = add_f32x2(sum_b, pack_f32x2(p0, p1));
    else sum_a = add_f32x2(sum_a, pack_f32x2(p0, p1));
    pk[i] = pack_bf16x2(p0, p1);
  }
}

template <int D, int kPoly>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               const PrefillParams p) {
  using C = Cfg<D>;
  using B = Bars<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 128B-swizzle atoms need 1024-byte alignment
  const uint32_t sQ = base + C::kQOff, sK = base + C::kKOff, sV = base + C::kVOff;
  const uint32_t sBar = base + C::kBarOff;
  auto bar = [&](int i) { return sBar + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mblk = gridDim.x - 1 - blockIdx.x;  // causal: longest rows first
  const int hq = blockIdx.y, b = blockIdx.z, hkv = hq / p.group;
  const int row0 = mblk * 2 * kBM;
  const int nkv_total = (p.kv_seq + kBN - 1) / kBN;
  // KV tiles each Q tile visits.  Top-left causal: tile m needs keys <= its last row.
  const int n0 = p.causal ? min(nkv_total, 2 * mblk + 1) : nkv_total;
  const int n1 = p.causal ? min(nkv_total, 2 * mblk + 2) : nkv_total;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < C::kNumBars; ++i) mbar_init(bar(i), ((i >= B::p_full && i < B::p_full + 2) || i >= B::e_full) ? 128u : 1u);  // p_full, e_full, p_half: one arrival per softmax thread
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abortp = &abort_flag;

  // Register budget: the four warps of the first warpgroup only issue copies and
  // MMAs; the softmax warpgroups hold a whole 128-column score row per thread.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        mbar_expect_tx(bar(B::q_full + t), C::kTileBytes);
#pragma unroll
        for (int kb = 0; kb < C::kBoxes; ++kb)
          tma_load_4d(sQ + t * C::kTileBytes + kb * C::kBoxBytes, &tm_q, bar(B::q_full + t), kb * 64,
                      row0 + t * kBM, hq, b);
      }
      auto load_k = [&](int j) {
        const int s = j % C::kKStages;
        if (j >= C::kKStages) ok = ok && mbar_wait(bar(B::k_empty + s), ((j / C::kKStages) - 1) & 1, abortp);
        if (!ok) return;
        mbar_expect_tx(bar(B::k_full + s), C::kTileBytes);
#pragma unroll
        for (int kb = 0; kb < C::kBoxes; ++kb)
          tma_load_4d(sK + s * C::kTileBytes + kb * C::kBoxBytes, &tm_k, bar(B::k_full + s), kb * 64,
                      j * kBN, hkv, b);
      };
      auto load_v = [&](int j) {
        const int s = j % C::kVStages;
        if (j >= C::kVStages) ok = ok && mbar_wait(bar(B::v_empty + s), ((j / C::kVStages) - 1) & 1, abortp);
        if (!ok) return;
        mbar_expect_tx(bar(B::v_full + s), C::kTileBytes);
#pragma unroll
        for (int kb = 0; kb < C::kBoxes; ++kb)
          tma_load_4d(sV + s * C::kTileBytes + kb * C::kBoxBytes, &tm_v, bar(B::v_full + s), kb * 64,
                      j * kBN, hkv, b);
      };
      load_k(0);
      for (int j = 0; j < n1 && ok; ++j) {
        if (j + 1 < n1) load_k(j + 1);
        load_v(j);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t tS0 = tmem + C::kTmemS, tS1 = tS0 + kBN;
      const uint32_t tO0 = tmem + C::kTmemO, tO1 = tO0 + D;
      bool ok = mbar_wait(bar(B::q_full + 0), 0, abortp) && mbar_wait(bar(B::q_full + 1), 0, abortp) &&
                mbar_wait(bar(B::k_full + 0), 0, abortp);
      if (ok) {
        tc_fence_after();
        issue_qk<D>(tS0, sQ, sK);
        umma_commit(bar(B::s_full + 0));
        issue_qk<D>(tS1, sQ + C::kTileBytes, sK);
        umma_commit(bar(B::s_full + 1));
        umma_commit(bar(B::k_empty + 0));
      }
      for (int j = 0; j < n1 && ok; ++j) {
        const int vs = j % C::kVStages;
        const bool next = (j + 1 < n1);
        const int ks = (j + 1) % C::kKStages;
        ok = mbar_wait(bar(B::v_full + vs), (j / C::kVStages) & 1, abortp);
        if (ok && next) ok = mbar_wait(bar(B::k_full + ks), ((j + 1) / C::kKStages) & 1, abortp);
        if (!ok) break;
        const uint32_t v_smem = sV + vs * C::kTileBytes;
        const uint32_t k_smem = sK + ks * C::kTileBytes;
        if (j < n0) {
          ok = mbar_wait(bar(B::p_half + 0), j & 1, abortp);
          if (!ok) break;
          tc_fence_after();
          issue_pv<D>(tO0, tS0, v_smem, j > 0, 0);
          ok = mbar_wait(bar(B::p_full + 0), j & 1, abortp);
          if (!ok) break;
          tc_fence_after();
          issue_pv<D>(tO0, tS0, v_smem, true, 1);
          if (j == n0 - 1) umma_commit(bar(B::o_full + 0));
        }
        if (j + 1 < n0) {
          issue_qk<D>(tS0, sQ, k_smem);
          umma_commit(bar(B::s_full + 0));
        }
        ok = mbar_wait(bar(B::p_half + 1), j & 1, abortp);
        if (!ok) break;
        tc_fence_after();
        issue_pv<D>(tO1, tS1, v_smem, j > 0, 0);
        ok = mbar_wait(bar(B::p_full + 1), j & 1, abortp);
        if (!ok) break;
        tc_fence_after();
        issue_pv<D>(tO1, tS1, v_smem, true, 1);
        umma_commit(bar(B::v_empty + vs));
        if (j == n1 - 1) umma_commit(bar(B::o_full + 1));
        if (next) {
          issue_qk<D>(tS1, sQ + C::kTileBytes, k_smem);
          umma_commit(bar(B::s_full + 1));
          umma_commit(bar(B::k_empty + ks));
        }
      }
    }
  }
  } else {
    // --------------------------------------------------- softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int t = (warp - 4) >> 2;          // Q tile of this warpgroup
    const int quarter = warp & 3;           // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;      // row within the tile = TMEM lane
    const int row = row0 + t * kBM + r;     // query index
    const int n_t = t ? n1 : n0;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_addr + C::kTmemS + t * kBN;
    const uint32_t tO = tmem + lane_addr + C::kTmemO + t * D;
    const float sl2 = p.scale_log2;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;

    for (int j = 0; j < n_t; ++j) {
      ok = mbar_wait(bar(B::s_full + t), j & 1, abortp);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[kBN / 32][32];  // the row's scores, raw fp32 bits
#pragma unroll
      for (int c = 0; c < kBN / 32; ++c) tmem_ld32(tS + c * 32, sr[c]);
      tmem_wait_ld();

      // keys this row may see in this tile: [0, limit)
      int limit = p.kv_seq - j * kBN;
      if (p.causal) limit = min(limit, row + 1 - j * kBN);
      if (limit < kBN) {
#pragma unroll
        for (int c = 0; c < kBN; ++c)
          if (c >= limit) sr[c >> 5][c & 31] = 0xff800000u;  // -inf
      }
      float mxa[4];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        mxa[c] = max3_f32(__uint_as_float(sr[c][0]), __uint_as_float(sr[c][1]), __uint_as_float(sr[c][2]));
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 3; i + 1 < 32; i += 2)
          mxa[c] = max3_f32(mxa[c], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
        mxa[c] = fmaxf(mxa[c], __uint_as_float(sr[c][31]));
      }
      const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));

      const float m_new = fmaxf(m_ref, mx);
      if (j == 0) {
        m_ref = m_new;
      } else {
        const bool grow = (m_new - m_ref) * sl2 > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          // PV_t(j-1) has completed (s_full covers it) and PV_t(j) is not issued
          // before this thread arrives on p_full, so O_t is ours to rescale.
          const float alpha = ex2_approx((m_ref - m_new) * sl2);
          l *= alpha;
          m_ref = m_new;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + c * 32, o);
          }
        }
      }
      const float neg = -m_ref * sl2;
      const uint64_t sl2x2 = pack_f32x2(sl2, sl2), negx2 = pack_f32x2(neg, neg);
      uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t pk[16];
        exp_chunk<kPoly>(sr[c], sl2x2, negx2, pk, sum_a, sum_b);
        tmem_st16(tS + c * 16, pk);
        if (c == 1) {  // keys 0..63 of P are in tensor memory: the first half of PV may start
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(bar(B::p_half + t));
        }
      }
      {
        float s0, s1;
        unpack_f32x2(add_f32x2(sum_a, sum_b), s0, s1);
        l += s0 + s1;
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(B::p_full + t));
    }

    // epilogue: O_t / l -> bf16 -> swizzled smem (the Q tile's buffer) -> TMA store
    if (ok) {
      ok = mbar_wait(bar(B::o_full + t), 0, abortp);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      const uint32_t sO = sQ + t * C::kTileBytes;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            w[i] = pack_bf16x2(__uint_as_float(o[q4 * 8 + 2 * i]) * inv_l,
                               __uint_as_float(o[q4 * 8 + 2 * i + 1]) * inv_l);
          const int chunk = c * 4 + q4;  // 16-byte chunk of the row
          const uint32_t addr = sO + (chunk >> 3) * C::kBoxBytes + r * 128 +
                                (((chunk & 7) ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                       "r"(w[2]), "r"(w[3])
                       : "memory");
        }
      }
      if (p.lse != nullptr && row < p.q_seq)
        p.lse[b * p.lse_stride_b + hq * p.lse_stride_h + row] =
            0.6931471805599453f * (m_ref * sl2 + lg2_approx(l));
      fence_proxy_async_smem();
      mbar_arrive(bar(B::e_full + t));
      if (r == 0 && row0 + t * kBM < p.q_seq && mbar_wait(bar(B::e_full + t), 0, abortp)) {
#pragma unroll
        for (int kb = 0; kb < C::kBoxes; ++kb)
          tma_store_4d(&tm_o, sO + kb * C::kBoxBytes, kb * 64, row0 + t * kBM, hq, b);
        tma_store_commit();
        tma_store_wait_read0();
      }
    }
  }

  // ------------------------------------------------------------------ exit
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    // Some wait gave up.  Give this CTA's outstanding TMA loads a bounded time
    // to land before the shared memory goes away, then report.
    if (threadIdx.x == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
      atomicOr(p.status, abort_flag);
    }
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// ------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// [batch, heads, seq, D] bf16 with element strides {sb, sh, ss}; box = 64 x 128 rows, 128B swizzle.
int make_map(CUtensorMap* m, const void* ptr, int batch, int heads, int seq, int d,
             const int64_t* stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -TYR_ATTN_ERR_NO_DEVICE;
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)seq, (cuuint64_t)heads, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)stride[2] * 2, (cuuint64_t)stride[1] * 2,
                           (cuuint64_t)stride[0] * 2};
  // a size-1 dimension may carry any stride; TMA still wants a non-zero multiple of 16 bytes
  for (int i = 0; i < 3; ++i)
    if (dims[i + 1] == 1) strides[i] = (i == 0 ? (cuuint64_t)d * 2 : strides[i - 1] * dims[i]);
  cuuint32_t box[4] = {64, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -TYR_ATTN_ERR_ALIGN;
}

template <int D, int kPoly>
int launch(const TyrAttnPrefillArgs& a, float scale, int* status, cudaStream_t st) {
  using C = Cfg<D>;
  CUtensorMap tq, tk, tv, to;
  int rc;
  if ((rc = make_map(&tq, a.q, a.batch, a.n_head, a.q_seq, D, a.q_stride))) return rc;
  if ((rc = make_map(&tk, a.k, a.batch, a.n_kv_head, a.kv_seq, D, a.k_stride))) return rc;
  if ((rc = make_map(&tv, a.v, a.batch, a.n_kv_head, a.kv_seq, D, a.v_stride))) return rc;
  if ((rc = make_map(&to, a.o, a.batch, a.n_head, a.q_seq, D, a.o_stride))) return rc;
  // per-device attribute: set on every launch so that any current device is covered
  cudaError_t attr_err = cudaFuncSetAttribute(
      prefill_kernel<D, kPoly>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes);
  if (attr_err != cudaSuccess) return (int)attr_err;
  PrefillParams p;
  p.lse = a.lse;
  p.lse_stride_h = a.q_seq;
  p.lse_stride_b = (int64_t)a.q_seq * a.n_head;
  p.q_seq = a.q_seq;
  p.kv_seq = a.kv_seq;
  p.group = a.n_head / a.n_kv_head;
  p.causal = a.is_causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid((a.q_seq + 2 * kBM - 1) / (2 * kBM), a.n_head, a.batch);
  prefill_kernel<D, kPoly><<<grid, kThreads, C::kSmemBytes, st>>>(tq, tk, tv, to, p);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace

int launch_prefill_sm100(const TyrAttnPrefillArgs& a, float scale, int* status, cudaStream_t st) {
  static const int poly = [] { const char* e = getenv("TYR_ATTN_POLY"); return e ? atoi(e) : 0; }();
  if (a.head_dim == 128) {
    switch (poly) {
      case 0: return launch<128, 0>(a, scale, status, st);
      case 1: return launch<128, 1>(a, scale, status, st);
      case 3: return launch<128, 3>(a, scale, status, st);
      case 4: return launch<128, 4>(a, scale, status, st);
      default: return launch<128, 2>(a, scale, status, st);
    }
  }
  if (a.head_dim == 64) return launch<64, 0>(a, scale, status, st);
  return -TYR_ATTN_ERR_HEAD_DIM;
}

}  // namespace tyr
