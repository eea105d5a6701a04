// Attention backward for sm_100a: dQ, dK, dV from dO, Q, K, V, O and the forward's LSE.
//
// Arithmetic (the formulation of Tyr/GPU/Kernels/MhaH100.lean:196-344; in the reference's
// models the same gradient comes from LibTorch autograd, cc/src/tyr.cpp:2111-2122):
//   delta_i = sum_d dO_i,d O_i,d            P_ij = exp(scale q_i.k_j - lse_i)   (0 under the mask)
//   dV_j += P_ij dO_i     dP_ij = dO_i.v_j   dS_ij = scale P_ij (dP_ij - delta_i)
//   dQ_i += dS_ij k_j     dK_j += dS_ij q_i
// with P and dS rounded to bf16 before the matrix products, fp32 accumulation.
//
// Three launches:
//   bwd_rowstats_kernel : -lse*log2(e) and -delta*scale per query row, padded to whole tiles
//                         (padding rows get -inf / 0, so they produce P = 0 downstream).
//   bwd_dkdv_kernel<D>  : persistent; one work unit = 128 keys of a (batch, KV head).  K and V tiles
//                         stay in shared memory; the Q and dO tiles of every query head of the group
//                         and every query block the keys are visible to stream through a 2-stage TMA
//                         ring, together with that block's row statistics.  Transposed orientation
//                         (rows = keys): S^T = K Q^T, dP^T = V dO^T by tcgen05.mma from shared memory
//                         into tensor memory, P^T and dS^T go back to tensor memory as bf16 and feed
//                         dV += P^T dO, dK += dS^T Q as the A operand, the streamed tile read MN-major
//                         as B.  dK and dV accumulate in tensor memory over the whole group: no
//                         atomics, a deterministic sum.  Tensor memory (512 columns): two score regions
//                         [0,128) and [128,256), dK [256,256+D), dV [256+D,256+2D).  The regions swap
//                         roles with every streamed pair: S^T of pair g sits in region g & 1 and, once
//                         in registers, leaves it to the bf16 overlays (P^T on its first 64 columns,
//                         dS^T on its last 64); dP^T of pair g sits in the other region, which takes
//                         S^T of pair g + 1 as soon as dP^T is in registers.  A step is therefore two
//                         halves: P^T from S^T alone, formed while the tensor pipe still works on the
//                         previous pair's dK and this pair's dP^T, then dS^T from P and dP^T.  Issue
//                         order per pair: dV(g), S^T(g+1), dK(g), dP^T(g+1).
//   bwd_dq_kernel<D>    : persistent; one work unit = 128 query rows of a (batch, query head).  Q and
//                         dO stay, K and V stream; S = Q K^T, dP = dO V^T, dQ += dS K, with dS in two
//                         buffers of its own so that the next score products run while dS is formed.
// Warps of both: 0 TMA producer, 1 MMA issuer, 2 TMEM allocation, 4-11 elementwise + epilogue, two
// warps per TMEM lane quarter (thread = row), each on one half of the score columns and of the
// output columns.  Units are sorted by decreasing work and dealt to the CTAs in mirrored rounds.
// Every wait is bounded and reports through the per-device status word, as in the forward.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>

#include "attn_internal.h"
#include "ptx_sm100.cuh"

namespace tyr {
namespace {

constexpr int kT = 128;           // tile rows and score-tile columns
constexpr int kBwdThreads = 384;  // 12 warps
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct BCfg {
  static constexpr int kBoxes = D / 64;                // 128-byte boxes per row
  static constexpr uint32_t kBoxBytes = 128u * 128u;   // 128 rows x 128 B
  static constexpr uint32_t kTileBytes = kBoxes * kBoxBytes;
  static constexpr int kStages = 2;
  static constexpr uint32_t kRes1 = 0, kRes2 = kTileBytes;
  static constexpr uint32_t kStr = 2 * kTileBytes;     // stage s: tile 1 at kStr + 2 s T, tile 2 one T further
  // per stage: the streamed query block's 128 row statistics, two fp32 vectors (mode 0 only)
  static constexpr uint32_t kStatOff = kStr + kStages * 2 * kTileBytes;
  static constexpr uint32_t kStatBytes = 2 * kT * 4;
  static constexpr uint32_t kBarOff = kStatOff + kStages * kStatBytes;
  // barriers
  static constexpr int res_full = 0;                   // resident pair landed
  static constexpr int str_full = 1;                   // [2] streamed pair landed
  static constexpr int str_empty = 3;                  // [2] accumulating products have read the pair
  static constexpr int s_full = 5;                     // S^T in tensor memory
  static constexpr int p_full = 6;                     // P^T written (one arrival per elementwise warp)
  static constexpr int acc_full = 7;                   // last accumulating product done
  static constexpr int pair = 8;                       // [4] per lane quarter: both warps hold their score columns
                                                       //     in registers (P / dS overwrite each other's columns)
  static constexpr int res_empty = 12;                 // the unit's last score products have read K and V
  static constexpr int acc_free = 13;                  // the epilogue has read dK and dV (8 warp arrivals)
  static constexpr int ds_half = 14;                   // dS^T of score columns 0..63 written (8 warp arrivals)
  static constexpr int ds_full = 15;                   // dS^T of score columns 64..127 written (8 warp arrivals)
  static constexpr int dp_full = 16;                   // dP^T in tensor memory
  static constexpr int dp_taken = 17;                  // dP^T is in registers: its columns are free (8 warp arrivals)
  static constexpr int kNumBars = 18;
  static constexpr uint32_t kSmemBytes = kBarOff + kNumBars * 8 + 16 + 1024;  // + align slack
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kTmemS = 0, kTmemDP = 128, kTmemAcc1 = 256, kTmemAcc2 = 256 + D;
  static_assert(256 + 2 * D <= 512, "tensor memory budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct BwdParams {
  __nv_bfloat16* out1;  // mode 0: dK, mode 1: dQ
  __nv_bfloat16* out2;  // mode 0: dV
  int64_t out1_stride[3], out2_stride[3];
  const float* neg_lse2;     // [batch * n_head, sq_pad]  -lse * log2(e); -inf on padding rows
  const float* neg_delta_s;  // [batch * n_head, sq_pad]  -delta * scale;  0 on padding rows
  int sq_pad;
  int batch, q_seq, kv_seq, n_head, n_kv_head, group, causal;
  int window;               // 0: none; w > 0: key j visible to query i only while i - j < w (with causal)
  const uint8_t* key_mask;  // [batch, kv_seq] bytes, 0 = padding key no query sees; or null
  int64_t key_mask_stride;
  int n_qblk, n_kblk;
  float sl2, scale;
  int* status;
  long long wait_limit;  // cycles any single barrier wait may take before the CTA gives up
};

constexpr uint32_t kBwdDescHi = umma_desc_hi(1024);

// score-shaped product: D[128 x 128] = A[128 x D] B[128 x D]^T, both K-major in shared memory
template <int D>
__device__ __forceinline__ void issue_nt(uint32_t issue, uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
  constexpr uint32_t idesc = umma_idesc_bf16(kT, kT, false);
  asm volatile("" : "+r"(a_lo), "+r"(b_lo));  // recomputed per use: keeps the issuer's registers few
#pragma unroll
  for (int kb = 0; kb < D / 64; ++kb) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint32_t off = (kb * BCfg<D>::kBoxBytes + ks * 32) >> 4;
      if (kb == 0 && ks == 0)
        umma_ss_lo_p<0>(d_tmem, a_lo, b_lo, kBwdDescHi, idesc, 0, issue);
      else
        umma_ss_lo_p<1>(d_tmem, a_lo + off, b_lo + off, kBwdDescHi, idesc, 1, issue);
    }
  }
}
// accumulating product: D[128 x D] (+)= A[128 x 128 bf16, tensor memory] B[128 x D], B MN-major.
// `part` 0 / 1: the first / second 64 of the 128 reduction steps only; -1: all of them.
template <int D>
__device__ __forceinline__ void issue_acc(uint32_t issue, uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                          bool accumulate, int part = -1) {
  constexpr uint32_t idesc = umma_idesc_bf16(kT, D, true);
  asm volatile("" : "+r"(b_lo), "+r"(a_tmem));
  const int k0 = part == 1 ? kT / 32 : 0, k1 = part == 0 ? kT / 32 : kT / 16;
#pragma unroll
  for (int kk = 0; kk < kT / 16; ++kk) {
    if (kk < k0 || kk >= k1) continue;
    // 16 rows of B = two 8-row groups of the tile; 16 bf16 of A = 8 TMEM columns
    if (kk == 0)
      umma_ts_lo_p<-1>(d_tmem, a_tmem, b_lo, kBwdDescHi, idesc, accumulate ? 1u : 0u, issue);
    else
      umma_ts_lo_p<1>(d_tmem, a_tmem + kk * 8, b_lo + ((kk * 2048) >> 4), kBwdDescHi, idesc, 1, issue);
  }
}

// Static schedule of the persistent kernels: in round k CTA c takes unit k G + c, mirrored in odd
// rounds (k G + G - 1 - c) so that the CTAs' totals even out over units sorted by decreasing work.
__device__ __forceinline__ int unit_of_round(int round, int n_units) {
  const int G = gridDim.x, c = blockIdx.x;
  const int u = round * G + ((round & 1) ? G - 1 - c : c);
  return u < n_units ? u : -1;
}
__device__ __forceinline__ int rounds_of(int n_units) { return (n_units + gridDim.x - 1) / gridDim.x; }

// One work unit of the dK/dV kernel: 128 keys of a (batch, KV head).  Units are numbered with the
// heaviest first (key block 0 is seen by every query block under a causal mask).
struct KvUnit {
  int blk, head, b;
  int lo;        // first query block with a row >= the unit's first key
  int per_head;  // query blocks streamed per query head
  int n_iter;    // per_head * group; 0 when no query sees these keys
};
__device__ __forceinline__ KvUnit kv_unit(int u, const BwdParams& p) {
  KvUnit w;
  const int lvl = u / (p.n_kv_head * p.batch);
  const int rem = u - lvl * p.n_kv_head * p.batch;
  w.head = rem % p.n_kv_head;
  w.b = rem / p.n_kv_head;
  w.blk = lvl;
  w.lo = p.causal ? min(w.blk, p.n_qblk) : 0;
  int hi = p.n_qblk;  // one past the last query block that sees a key of the unit
  if (p.window > 0) hi = min(hi, (w.blk * kT + kT - 1 + p.window - 1) / kT + 1);
  w.per_head = max(hi - w.lo, 0);
  w.n_iter = w.per_head * p.group;
  return w;
}

// dK / dV kernel, persistent: CTA c works on units c, c + gridDim.x, ...  Rows = keys.  The K and V
// tiles of the unit stay in shared memory (the next unit's are fetched as soon as the unit's last
// score products have read them), Q and dO stream.  Barrier phases run on across units: every role
// counts streamed tile pairs (`it`) and units with work (`rc`) for itself.
template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                const BwdParams p) {
  using C = BCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_slot;
  __shared__ WaitCtl wait_ctl;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 128B-swizzle atoms need 1024-byte alignment
  const uint32_t sBar = base + C::kBarOff;
  auto bar = [&](int i) { return sBar + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_units = p.n_kblk * p.n_kv_head * p.batch;

  if (threadIdx.x == 0) {
    wait_ctl.abort = 0;
    wait_ctl.limit = p.wait_limit;
    for (int i = 0; i < C::kNumBars; ++i)
      mbar_init(bar(i), (i == C::p_full || i == C::ds_half || i == C::ds_full || i == C::dp_taken || i == C::acc_free) ? 8u
                        : (i >= C::pair && i < C::pair + 4) ? 2u : 1u);
    mbar_fence_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile WaitCtl* abortp = &wait_ctl;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      int it = 0, rc = 0;
      for (int round = 0; round < rounds_of(n_units) && ok; ++round) {
        const int u = unit_of_round(round, n_units);
        if (u < 0) continue;
        const KvUnit w = kv_unit(u, p);
        if (w.n_iter == 0) continue;
        if (rc > 0) ok = mbar_wait_q(bar(C::res_empty), (rc - 1) & 1, abortp);
        if (!ok) break;
        mbar_expect_tx(bar(C::res_full), 2 * C::kTileBytes);
#pragma unroll
        for (int kb = 0; kb < C::kBoxes; ++kb) {
          tma_load_4d(base + C::kRes1 + kb * C::kBoxBytes, &tm_k, bar(C::res_full), kb * 64, w.blk * kT, w.head, w.b);
          tma_load_4d(base + C::kRes2 + kb * C::kBoxBytes, &tm_v, bar(C::res_full), kb * 64, w.blk * kT, w.head, w.b);
        }
        for (int i = 0; i < w.n_iter && ok; ++i, ++it) {
          const int s = it % C::kStages;
          if (it >= C::kStages) ok = mbar_wait_q(bar(C::str_empty + s), ((it / C::kStages) - 1) & 1, abortp);
          if (!ok) break;
          const int hq = w.head * p.group + i / w.per_head, qblk = w.lo + i % w.per_head;
          const uint32_t dst = base + C::kStr + s * 2 * C::kTileBytes;
          mbar_expect_tx(bar(C::str_full + s), 2 * C::kTileBytes + C::kStatBytes);
          {
            const int64_t at = ((int64_t)w.b * p.n_head + hq) * p.sq_pad + qblk * kT;
            const uint32_t sdst = base + C::kStatOff + s * C::kStatBytes;
            bulk_load(sdst, p.neg_lse2 + at, kT * 4, bar(C::str_full + s));
            bulk_load(sdst + kT * 4, p.neg_delta_s + at, kT * 4, bar(C::str_full + s));
          }
#pragma unroll
          for (int kb = 0; kb < C::kBoxes; ++kb) {
            tma_load_4d(dst + kb * C::kBoxBytes, &tm_q, bar(C::str_full + s), kb * 64, qblk * kT, hq, w.b);
            tma_load_4d(dst + C::kTileBytes + kb * C::kBoxBytes, &tm_do, bar(C::str_full + s), kb * 64, qblk * kT,
                        hq, w.b);
          }
        }
        ++rc;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // the whole warp runs the loop, convergent; one elected lane issues the MMAs and commits
    {
      const uint32_t issue = elect_one();
      const uint32_t tA1 = tmem + C::kTmemAcc1, tA2 = tmem + C::kTmemAcc2;
      const uint32_t res1_lo = umma_desc_lo(base + C::kRes1, 16), res2_lo = umma_desc_lo(base + C::kRes2, 16);
      // The two 128-column score regions swap roles from one streamed pair to the next: pair g has
      // S^T in region g & 1 and dP^T in the other.  Once S^T is in registers its region takes the two
      // bf16 overlays, P^T on its first 64 columns and dS^T on its last 64; the dP^T region is free as
      // soon as dP^T is in registers and takes S^T of pair g + 1, and when the accumulating products
      // of pair g have read the overlays their region takes dP^T of pair g + 1.
      auto region = [&](int g, int which) { return tmem + (((g + which) & 1) ? C::kTmemDP : C::kTmemS); };
      auto score_s = [&](int g) {   // S^T = K Q^T of pair g
        const int s = g % C::kStages;
        if (!mbar_wait_q(bar(C::str_full + s), (g / C::kStages) & 1, abortp)) return false;
        tc_fence_after();
        issue_nt<D>(issue, region(g, 0), res1_lo, umma_desc_lo(base + C::kStr + s * 2 * C::kTileBytes, 16));
        umma_commit_p(bar(C::s_full), issue);
        return true;
      };
      auto score_dp = [&](int g) {  // dP^T = V dO^T of pair g (its tiles have landed: S^T of the pair came first)
        const int s = g % C::kStages;
        issue_nt<D>(issue, region(g, 1), res2_lo, umma_desc_lo(base + C::kStr + s * 2 * C::kTileBytes + C::kTileBytes, 16));
        umma_commit_p(bar(C::dp_full), issue);
      };
      bool ok = true;
      int it = 0, rc = 0;
      for (int round = 0; round < rounds_of(n_units) && ok; ++round) {
        const int u = unit_of_round(round, n_units);
        if (u < 0) continue;
        const KvUnit w = kv_unit(u, p);
        if (w.n_iter == 0) continue;
        ok = mbar_wait_q(bar(C::res_full), rc & 1, abortp);
        if (ok) ok = score_s(it);
        if (ok) score_dp(it);
        if (ok && w.n_iter == 1) umma_commit_p(bar(C::res_empty), issue);
        for (int i = 0; i < w.n_iter && ok; ++i, ++it) {
          const int s = it % C::kStages;
          const uint32_t t1 = base + C::kStr + s * 2 * C::kTileBytes;
          const uint32_t tP = region(it, 0), tDS = tP + 64;
          const uint32_t q_mn = umma_desc_lo(t1, C::kBoxBytes), do_mn = umma_desc_lo(t1 + C::kTileBytes, C::kBoxBytes);
          // dV += P^T dO as soon as P^T is written (it is formed from S^T alone, ahead of dS^T)
          ok = mbar_wait_q(bar(C::p_full), it & 1, abortp);
          // the unit's first accumulating products overwrite dK / dV: the previous unit's
          // epilogue must have read them
          if (ok && i == 0 && rc > 0) ok = mbar_wait_q(bar(C::acc_free), (rc - 1) & 1, abortp);
          if (!ok) break;
          tc_fence_after();
          issue_acc<D>(issue, tA2, tP, do_mn, i > 0);
          // S^T of the next pair into the region dP^T has left
          if (i + 1 < w.n_iter) {
            ok = mbar_wait_q(bar(C::dp_taken), it & 1, abortp);
            if (!ok) break;
            tc_fence_after();
            ok = score_s(it + 1);
            if (!ok) break;
          }
          // dK += dS^T Q, the first 64 query columns while the second 64 are still being formed
          ok = mbar_wait_q(bar(C::ds_half), it & 1, abortp);
          if (!ok) break;
          tc_fence_after();
          issue_acc<D>(issue, tA1, tDS, q_mn, i > 0, 0);
          ok = mbar_wait_q(bar(C::ds_full), it & 1, abortp);
          if (!ok) break;
          tc_fence_after();
          issue_acc<D>(issue, tA1, tDS, q_mn, true, 1);
          umma_commit_p(bar(C::str_empty + s), issue);
          if (i + 1 < w.n_iter) {
            // dP^T of the next pair into the region whose overlays the products above have read
            score_dp(it + 1);
            // K and V are read by the score products only: after the unit's last pair of them
            // the producer may fetch the next unit's
            if (i + 2 == w.n_iter) umma_commit_p(bar(C::res_empty), issue);
          } else {
            umma_commit_p(bar(C::acc_full), issue);
          }
        }
        ++rc;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------ elementwise + epilogue
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;   // query columns [64 half, 64 half + 64), output columns likewise
    const int r = quarter * 32 + lane;  // key row of the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint64_t sl2x2 = pack_f32x2(p.sl2, p.sl2), scale2 = pack_f32x2(p.scale, p.scale);
    bool ok = true;
    int it = 0, rc = 0;
    for (int round = 0; round < rounds_of(n_units) && ok; ++round) {
      const int u = unit_of_round(round, n_units);
      if (u < 0) continue;
      const KvUnit w = kv_unit(u, p);
      const int row0 = w.blk * kT;
      for (int i = 0; i < w.n_iter; ++i, ++it) {
        // the score regions swap roles with every streamed pair (see the MMA issuer)
        const uint32_t tS = tmem + lane_addr + ((it & 1) ? C::kTmemDP : C::kTmemS);
        const uint32_t tDP = tmem + lane_addr + ((it & 1) ? C::kTmemS : C::kTmemDP);
        ok = mbar_wait_q(bar(C::s_full), it & 1, abortp);
        // the query columns' statistics landed with the streamed tiles: observe that barrier
        // directly (it completed before the products this warp was woken by were issued)
        if (ok) ok = mbar_wait_q(bar(C::str_full + it % C::kStages), (it / C::kStages) & 1, abortp);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const int col0 = (w.lo + i % w.per_head) * kT;  // first query of the score columns
        // under the causal mask a key row keeps the query columns with query >= key
        int c_first = p.causal ? row0 + r - col0 : 0;
        // sliding window: the key also drops out for queries with query - key >= window
        const int c_limit = p.window > 0 ? row0 + r - col0 + p.window : kT;
        // a padding key sees no query at all
        if (p.key_mask != nullptr && (row0 + r >= p.kv_seq || p.key_mask[w.b * p.key_mask_stride + row0 + r] == 0))
          c_first = kT;
        const bool masked = __any_sync(0xffffffffu, c_first > 0 || c_limit < kT);
        const float* nl_col = reinterpret_cast<const float*>(smem_raw + (base - raw) + C::kStatOff +
                                                             (it % C::kStages) * C::kStatBytes);
        const float* nd_col = nl_col + kT;
        // First half of the step, from S^T alone: P^T.  This warp's two 32-column chunks of S^T go to
        // registers: chunk `half` of the first 64 query columns and chunk 2 + `half` of the second
        // 64.  bf16 P^T of chunk c lands on columns [16 c, 16 c + 16) of the region, i.e. on chunks 0
        // and 1, which belong to different warps of the pair: the two meet once both hold their
        // columns in registers.  P stays in registers as fp32 for dS.
        uint32_t pr2[2][32];
#pragma unroll
        for (int step = 0; step < 2; ++step) tmem_ld32(tS + (2 * step + half) * 32, pr2[step]);
        tmem_wait_ld();
#pragma unroll
        for (int step = 0; step < 2; ++step) tmem_ld_ready(pr2[step]);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::pair + quarter));
#pragma unroll
        for (int step = 0; step < 2; ++step) {
          const int c = 2 * step + half;
          uint32_t(&sr)[32] = pr2[step];
          if (masked) {
#pragma unroll
            for (int x = 0; x < 32; ++x)
              if (c * 32 + x < c_first || c * 32 + x >= c_limit) sr[x] = 0xff800000u;  // -inf: P = 0
          }
          uint32_t pk_p[16];
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            // statistics of the two query columns (every lane reads the same addresses)
            const float2 a = *reinterpret_cast<const float2*>(nl_col + c * 32 + 2 * x);
            const uint64_t t2 = fma_f32x2(pack_u32x2(sr[2 * x], sr[2 * x + 1]), sl2x2, pack_f32x2(a.x, a.y));
            float t0, t1;
            unpack_f32x2(t2, t0, t1);
            const float p0 = ex2_approx(t0), p1 = ex2_approx(t1);
            sr[2 * x] = __float_as_uint(p0);
            sr[2 * x + 1] = __float_as_uint(p1);
            pk_p[x] = pack_bf16x2(p0, p1);
          }
          if (step == 0) {
            ok = mbar_wait_q(bar(C::pair + quarter), it & 1, abortp);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
          }
          tmem_st16(tS + c * 16, pk_p);
        }
        if (!ok) break;
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::p_full));

        // Second half, once dP^T has arrived: dS^T = P (scale dP - scale delta), written behind P^T on
        // the last 64 columns of the same region (they held the second 64 query columns of S^T, in
        // registers since the pair met).  The region dP^T leaves takes the next pair's S^T.
        ok = mbar_wait_q(bar(C::dp_full), it & 1, abortp);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t dp2[2][32];
#pragma unroll
        for (int step = 0; step < 2; ++step) tmem_ld32(tDP + (2 * step + half) * 32, dp2[step]);
        tmem_wait_ld();
#pragma unroll
        for (int step = 0; step < 2; ++step) tmem_ld_ready(dp2[step]);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::dp_taken));
#pragma unroll
        for (int step = 0; step < 2; ++step) {
          const int c = 2 * step + half;
          uint32_t(&pr)[32] = pr2[step];
          uint32_t(&dp)[32] = dp2[step];
          uint32_t pk_s[16];
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            const float2 d = *reinterpret_cast<const float2*>(nd_col + c * 32 + 2 * x);
            const uint64_t u2 = fma_f32x2(pack_u32x2(dp[2 * x], dp[2 * x + 1]), scale2, pack_f32x2(d.x, d.y));
            float d0, d1;
            unpack_f32x2(mul_f32x2(pack_u32x2(pr[2 * x], pr[2 * x + 1]), u2), d0, d1);
            pk_s[x] = pack_bf16x2(d0, d1);
          }
          tmem_st16(tS + 64 + c * 16, pk_s);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(step == 0 ? C::ds_half : C::ds_full));
        }
      }
      if (!ok) break;

      // epilogue: dK and dV -> bf16 -> global, one key row per thread, half of the columns per warp
      // of the pair; keys that no query sees get zeros without touching tensor memory
      if (w.n_iter > 0) {
        ok = mbar_wait_q(bar(C::acc_full), rc & 1, abortp);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
      const int row = row0 + r;
      const bool row_ok = row < p.kv_seq;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t tA = tmem + lane_addr + (which ? C::kTmemAcc2 : C::kTmemAcc1);
        const int64_t* st = which ? p.out2_stride : p.out1_stride;
        __nv_bfloat16* orow = (which ? p.out2 : p.out1) + w.b * st[0] + w.head * st[1] + (int64_t)row * st[2];
#pragma unroll
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t o[32];
          if (w.n_iter > 0) {
            tmem_ld32(tA + c * 32, o);
            tmem_wait_ld();
            tmem_ld_ready(o);
          } else {
#pragma unroll
            for (int x = 0; x < 32; ++x) o[x] = 0u;
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 wv;
            wv.x = pack_bf16x2(__uint_as_float(o[q4 * 8 + 0]), __uint_as_float(o[q4 * 8 + 1]));
            wv.y = pack_bf16x2(__uint_as_float(o[q4 * 8 + 2]), __uint_as_float(o[q4 * 8 + 3]));
            wv.z = pack_bf16x2(__uint_as_float(o[q4 * 8 + 4]), __uint_as_float(o[q4 * 8 + 5]));
            wv.w = pack_bf16x2(__uint_as_float(o[q4 * 8 + 6]), __uint_as_float(o[q4 * 8 + 7]));
            if (row_ok) *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = wv;
          }
        }
      }
      if (w.n_iter > 0) {
        // the accumulators are in registers / memory: the next unit may overwrite them
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::acc_free));
        ++rc;
      }
    }
  }

  // ------------------------------------------------------------------ exit
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (wait_ctl.abort != 0) {
    // Some wait gave up.  Give this CTA's outstanding TMA loads a bounded time
    // to land before the shared memory goes away, then report.
    if (threadIdx.x == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
      atomicOr(p.status, wait_ctl.abort);
    }
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// dQ kernel with the score products running ahead of the elementwise step, persistent like the
// dK/dV kernel.  One work unit = 128 query rows of a (batch, query head), the units with the most key
// blocks first: Q and dO stay in shared memory (the next unit's are fetched once the unit's last
// score products have read them), K streams
// through a 3-stage ring and V through a 2-stage ring.  dS does not overlay dP here: tensor memory
// has 128 columns to spare next to S, dP and dQ, enough for two bf16 dS buffers.  S and dP may
// therefore be overwritten as soon as the elementwise warps hold them in registers, so
// S(i+1) = Q K(i+1)^T and dP(i+1) = dO V(i+1)^T are computed while dS(i) is being formed, and
// dQ += dS(i) K(i) follows; the elementwise warps go from one tile to the next without waiting.
// (V is free once dP has read it, K only after the dQ product: hence the deeper K ring.)
template <int D>
struct DqCfg {
  static constexpr int kBoxes = D / 64;
  static constexpr uint32_t kBoxBytes = 128u * 128u;
  static constexpr uint32_t kTileBytes = kBoxes * kBoxBytes;
  static constexpr int kKStages = 3, kVStages = 2;
  static constexpr uint32_t kQ = 0, kDO = kTileBytes, kK = 2 * kTileBytes;
  static constexpr uint32_t kV = kK + kKStages * kTileBytes;
  static constexpr uint32_t kBarOff = kV + kVStages * kTileBytes;
  static constexpr int res_full = 0;
  static constexpr int k_full = 1;                       // [3]
  static constexpr int k_empty = k_full + kKStages;      // [3] the dQ product has read the K tile
  static constexpr int v_full = k_empty + kKStages;      // [2]
  static constexpr int v_empty = v_full + kVStages;      // [2] the dP product has read the V tile
  static constexpr int s_full = v_empty + kVStages;      // S and dP in tensor memory
  static constexpr int sdp_free = s_full + 1;            // S and dP are in registers (8 warp arrivals)
  static constexpr int p_full = sdp_free + 1;            // [2] dS buffer written (8 warp arrivals), alternating
  static constexpr int acc_full = p_full + 2;
  static constexpr int res_empty = acc_full + 1;         // the unit's last score products have read Q and dO
  static constexpr int acc_free = res_empty + 1;         // the epilogue has read dQ (8 warp arrivals)
  static constexpr int kNumBars = acc_free + 1;
  static constexpr uint32_t kSmemBytes = kBarOff + kNumBars * 8 + 16 + 1024;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kTmemS = 0, kTmemDP = 128, kTmemAcc = 256, kTmemDS = 384;  // dS: 2 x 64 columns
  static_assert(256 + D + 128 <= 512, "tensor memory budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct QUnit {
  int blk, head, b;
  int lo;      // first key block a row of the unit sees (> 0 only under a sliding window)
  int n_iter;  // key blocks lo .. lo + n_iter - 1
};
__device__ __forceinline__ QUnit q_unit(int u, const BwdParams& p) {
  QUnit w;
  const int lvl = u / (p.n_head * p.batch);
  const int rem = u - lvl * p.n_head * p.batch;
  w.head = rem % p.n_head;
  w.b = rem / p.n_head;
  w.blk = p.n_qblk - 1 - lvl;
  w.lo = p.window > 0 ? max(w.blk * kT - p.window + 1, 0) / kT : 0;
  w.n_iter = (p.causal ? min(p.n_kblk, w.blk + 1) : p.n_kblk) - w.lo;
  return w;
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
              const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
              const BwdParams p) {
  using C = DqCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_slot;
  __shared__ WaitCtl wait_ctl;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t sBar = base + C::kBarOff;
  auto bar = [&](int i) { return sBar + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_units = p.n_qblk * p.n_head * p.batch;

  if (threadIdx.x == 0) {
    wait_ctl.abort = 0;
    wait_ctl.limit = p.wait_limit;
    for (int i = 0; i < C::kNumBars; ++i)
      mbar_init(bar(i), (i == C::sdp_free || i == C::p_full || i == C::p_full + 1 || i == C::acc_free) ? 8u : 1u);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile WaitCtl* abortp = &wait_ctl;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      bool ok = true;
      int it = 0, rc = 0;
      for (int round = 0; round < rounds_of(n_units) && ok; ++round, ++rc) {
        const int u = unit_of_round(round, n_units);
        if (u < 0) break;  // only the last round can be short
        const QUnit w = q_unit(u, p);
        const int hkv = w.head / p.group;
        if (rc > 0) ok = mbar_wait_q(bar(C::res_empty), (rc - 1) & 1, abortp);
        if (!ok) break;
        mbar_expect_tx(bar(C::res_full), 2 * C::kTileBytes);
#pragma unroll
        for (int kb = 0; kb < C::kBoxes; ++kb) {
          tma_load_4d(base + C::kQ + kb * C::kBoxBytes, &tm_q, bar(C::res_full), kb * 64, w.blk * kT, w.head, w.b);
          tma_load_4d(base + C::kDO + kb * C::kBoxBytes, &tm_do, bar(C::res_full), kb * 64, w.blk * kT, w.head, w.b);
        }
        for (int i = 0; i < w.n_iter && ok; ++i, ++it) {
          const int ks = it % C::kKStages, vs = it % C::kVStages;
          if (it >= C::kKStages) ok = mbar_wait_q(bar(C::k_empty + ks), ((it / C::kKStages) - 1) & 1, abortp);
          if (!ok) break;
          mbar_expect_tx(bar(C::k_full + ks), C::kTileBytes);
#pragma unroll
          for (int kb = 0; kb < C::kBoxes; ++kb)
            tma_load_4d(base + C::kK + ks * C::kTileBytes + kb * C::kBoxBytes, &tm_k, bar(C::k_full + ks), kb * 64,
                        (w.lo + i) * kT, hkv, w.b);
          if (it >= C::kVStages) ok = mbar_wait_q(bar(C::v_empty + vs), ((it / C::kVStages) - 1) & 1, abortp);
          if (!ok) break;
          mbar_expect_tx(bar(C::v_full + vs), C::kTileBytes);
#pragma unroll
          for (int kb = 0; kb < C::kBoxes; ++kb)
            tma_load_4d(base + C::kV + vs * C::kTileBytes + kb * C::kBoxBytes, &tm_v, bar(C::v_full + vs), kb * 64,
                        (w.lo + i) * kT, hkv, w.b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // the whole warp runs the loop, convergent; one elected lane issues the MMAs and commits
    {
      const uint32_t issue = elect_one();
      const uint32_t tS = tmem + C::kTmemS, tDP = tmem + C::kTmemDP, tAcc = tmem + C::kTmemAcc;
      const uint32_t q_lo = umma_desc_lo(base + C::kQ, 16), do_lo = umma_desc_lo(base + C::kDO, 16);
      auto scores = [&](int g) {  // S = Q K^T, dP = dO V^T for streamed pair number g; V is free afterwards
        const int ks = g % C::kKStages, vs = g % C::kVStages;
        if (!mbar_wait_q(bar(C::k_full + ks), (g / C::kKStages) & 1, abortp)) return false;
        if (!mbar_wait_q(bar(C::v_full + vs), (g / C::kVStages) & 1, abortp)) return false;
        tc_fence_after();
        issue_nt<D>(issue, tS, q_lo, umma_desc_lo(base + C::kK + ks * C::kTileBytes, 16));
        issue_nt<D>(issue, tDP, do_lo, umma_desc_lo(base + C::kV + vs * C::kTileBytes, 16));
        umma_commit_p(bar(C::s_full), issue);
        umma_commit_p(bar(C::v_empty + vs), issue);
        return true;
      };
      bool ok = true;
      int it = 0, rc = 0;
      for (int round = 0; round < rounds_of(n_units) && ok; ++round, ++rc) {
        const int u = unit_of_round(round, n_units);
        if (u < 0) break;  // only the last round can be short
        const QUnit w = q_unit(u, p);
        ok = mbar_wait_q(bar(C::res_full), rc & 1, abortp);
        // S and dP of the previous unit's last pair must be in the elementwise warps' registers
        if (ok && it > 0) ok = mbar_wait_q(bar(C::sdp_free), (it - 1) & 1, abortp);
        if (ok) ok = scores(it);
        if (ok && w.n_iter == 1) umma_commit_p(bar(C::res_empty), issue);
        for (int i = 0; i < w.n_iter && ok; ++i, ++it) {
          if (i + 1 < w.n_iter) {
            // S(i) and dP(i) are in the elementwise warps' registers: the next pair may overwrite them
            ok = mbar_wait_q(bar(C::sdp_free), it & 1, abortp);
            if (ok) ok = scores(it + 1);
            if (!ok) break;
            if (i + 2 == w.n_iter) umma_commit_p(bar(C::res_empty), issue);  // Q and dO are read by score products only
          }
          ok = mbar_wait_q(bar(C::p_full + (it & 1)), (it >> 1) & 1, abortp);
          // the unit's first dQ product overwrites the accumulator the previous epilogue reads
          if (ok && i == 0 && rc > 0) ok = mbar_wait_q(bar(C::acc_free), (rc - 1) & 1, abortp);
          if (!ok) break;
          tc_fence_after();
          const int ks = it % C::kKStages;
          issue_acc<D>(issue, tAcc, tmem + C::kTmemDS + (it & 1) * 64,
                       umma_desc_lo(base + C::kK + ks * C::kTileBytes, C::kBoxBytes), i > 0);
          umma_commit_p(bar(C::k_empty + ks), issue);
        }
        if (ok) umma_commit_p(bar(C::acc_full), issue);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------ elementwise + epilogue
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;   // key columns [64 half, 64 half + 64)
    const int r = quarter * 32 + lane;  // query row of the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_addr + C::kTmemS, tDP = tmem + lane_addr + C::kTmemDP;
    const uint64_t sl2x2 = pack_f32x2(p.sl2, p.sl2), scale2 = pack_f32x2(p.scale, p.scale);
    bool ok = true;
    int it = 0, rc = 0;
    for (int round = 0; round < rounds_of(n_units) && ok; ++round, ++rc) {
      const int u = unit_of_round(round, n_units);
      if (u < 0) break;  // only the last round can be short
      const QUnit w = q_unit(u, p);
      const int row0 = w.blk * kT;
      const int64_t at = ((int64_t)w.b * p.n_head + w.head) * p.sq_pad + row0 + r;
      const float nl_row = p.neg_lse2[at], nd_row = p.neg_delta_s[at];
      const uint64_t nl2 = pack_f32x2(nl_row, nl_row), nd2 = pack_f32x2(nd_row, nd_row);
      for (int i = 0; i < w.n_iter; ++i, ++it) {
        ok = mbar_wait_q(bar(C::s_full), it & 1, abortp);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr2[2][32], dp2[2][32];
#pragma unroll
        for (int step = 0; step < 2; ++step) {
          tmem_ld32(tS + (2 * half + step) * 32, sr2[step]);
          tmem_ld32(tDP + (2 * half + step) * 32, dp2[step]);
        }
        tmem_wait_ld();
#pragma unroll
        for (int step = 0; step < 2; ++step) {
          tmem_ld_ready(sr2[step]);
          tmem_ld_ready(dp2[step]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::sdp_free));

        // keys this query row keeps under the causal mask: key <= query
        const int col0 = (w.lo + i) * kT;  // first key of the score columns
        const int c_limit = p.causal ? row0 + r - col0 + 1 : kT;
        // sliding window: keys with query - key >= window drop out
        const int c_first = p.window > 0 ? row0 + r - p.window + 1 - col0 : 0;
        // padding keys: lane l fetches the mask bytes of keys 2l, 2l+1 of this warp's 64 columns, two
        // ballots spread them to every row; column j of the 64 is bit (j >> 1) of ballot (j & 1)
        uint32_t vb[2] = {0xffffffffu, 0xffffffffu};
        if (p.key_mask != nullptr) {
          const uint8_t* mrow = p.key_mask + w.b * p.key_mask_stride + col0 + 64 * half;
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int kk = 2 * lane + e;
            vb[e] = __ballot_sync(0xffffffffu, (col0 + 64 * half + kk < p.kv_seq) && mrow[kk] != 0);
          }
        }
        const bool masked = __any_sync(0xffffffffu, c_limit < kT || c_first > 0) || (vb[0] & vb[1]) != 0xffffffffu;
        const uint32_t tDS = tmem + lane_addr + C::kTmemDS + (it & 1) * 64;
#pragma unroll
        for (int step = 0; step < 2; ++step) {
          const int c = 2 * half + step;
          uint32_t(&sr)[32] = sr2[step];
          uint32_t(&dp)[32] = dp2[step];
          if (masked) {
#pragma unroll
            for (int x = 0; x < 32; ++x)
              if (c * 32 + x >= c_limit || c * 32 + x < c_first || !((vb[x & 1] >> ((32 * step + x) >> 1)) & 1u))
                sr[x] = 0xff800000u;  // -inf: P = 0
          }
          uint32_t pk_s[16];
#pragma unroll
          for (int x = 0; x < 16; ++x) {
            const uint64_t t2 = fma_f32x2(pack_u32x2(sr[2 * x], sr[2 * x + 1]), sl2x2, nl2);
            float t0, t1;
            unpack_f32x2(t2, t0, t1);
            const float p0 = ex2_approx(t0), p1 = ex2_approx(t1);
            const uint64_t u2 = fma_f32x2(pack_u32x2(dp[2 * x], dp[2 * x + 1]), scale2, nd2);
            float d0, d1;
            unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1), u2), d0, d1);
            pk_s[x] = pack_bf16x2(d0, d1);
          }
          tmem_st16(tDS + c * 16, pk_s);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::p_full + (it & 1)));
      }
      if (!ok) break;

      // epilogue: dQ -> bf16 -> global, one row per thread, half of the columns per warp of the pair
      ok = mbar_wait_q(bar(C::acc_full), rc & 1, abortp);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = row0 + r;
      const bool row_ok = row < p.q_seq;
      const uint32_t tA = tmem + lane_addr + C::kTmemAcc;
      __nv_bfloat16* orow = p.out1 + w.b * p.out1_stride[0] + w.head * p.out1_stride[1] + (int64_t)row * p.out1_stride[2];
#pragma unroll
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t o[32];
        tmem_ld32(tA + c * 32, o);
        tmem_wait_ld();
        tmem_ld_ready(o);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 wv;
          wv.x = pack_bf16x2(__uint_as_float(o[q4 * 8 + 0]), __uint_as_float(o[q4 * 8 + 1]));
          wv.y = pack_bf16x2(__uint_as_float(o[q4 * 8 + 2]), __uint_as_float(o[q4 * 8 + 3]));
          wv.z = pack_bf16x2(__uint_as_float(o[q4 * 8 + 4]), __uint_as_float(o[q4 * 8 + 5]));
          wv.w = pack_bf16x2(__uint_as_float(o[q4 * 8 + 6]), __uint_as_float(o[q4 * 8 + 7]));
          if (row_ok) *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = wv;
        }
      }
      // dQ is in registers / memory: the next unit may overwrite the accumulator
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::acc_free));
    }
  }

  // ------------------------------------------------------------------ exit
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (wait_ctl.abort != 0) {
    if (threadIdx.x == 0) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) {
      }
      atomicOr(p.status, wait_ctl.abort);
    }
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// Row statistics of the backward: one group of D/8 lanes per query row, 16-byte loads.
template <int D>
__global__ void __launch_bounds__(256)
bwd_rowstats_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                    const float* __restrict__ lse, float* __restrict__ neg_lse2,
                    float* __restrict__ neg_delta_s, int n_head, int q_seq, int sq_pad, int64_t os_b,
                    int64_t os_h, int64_t os_s, int64_t ds_b, int64_t ds_h, int64_t ds_s, float scale,
                    int64_t total_rows) {
  constexpr int kLanes = D / 8;  // lanes per row
  const int64_t slot = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / kLanes;  // padded row index
  const int sub = threadIdx.x % kLanes;
  if (slot >= total_rows) return;
  const int i = (int)(slot % sq_pad);
  const int64_t bh = slot / sq_pad;
  const int h = (int)(bh % n_head);
  const int64_t b = bh / n_head;
  float acc = 0.f;
  if (i < q_seq) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + b * os_b + h * os_h + (int64_t)i * os_s + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + b * ds_b + h * ds_h + (int64_t)i * ds_s + sub * 8);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const float2 af = __bfloat1622float2(a2[x]), gf = __bfloat1622float2(g2[x]);
      acc = fmaf(af.x, gf.x, acc);
      acc = fmaf(af.y, gf.y, acc);
    }
  }
#pragma unroll
  for (int off = kLanes / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off, kLanes);
  if (sub == 0) {
    const bool real = i < q_seq;
    neg_lse2[slot] = real ? -lse[(b * n_head + h) * (int64_t)q_seq + i] * kLog2e : -INFINITY;
    neg_delta_s[slot] = real ? -acc * scale : 0.f;
  }
}

template <int D>
int launch_bwd(const TyrAttnBackwardArgs& a, float scale, int* status, cudaStream_t st) {
  using C = BCfg<D>;
  const int n_qblk = (a.q_seq + kT - 1) / kT, n_kblk = (a.kv_seq + kT - 1) / kT;
  const int sq_pad = n_qblk * kT;
  const int64_t padded_rows = (int64_t)a.batch * a.n_head * sq_pad;
  float* neg_lse2 = static_cast<float*>(a.workspace);
  float* neg_delta_s = neg_lse2 + padded_rows;

  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_tile_map(&tq, a.q, a.batch, a.n_head, a.q_seq, D, a.q_stride))) return rc;
  if ((rc = make_tile_map(&tk, a.k, a.batch, a.n_kv_head, a.kv_seq, D, a.k_stride))) return rc;
  if ((rc = make_tile_map(&tv, a.v, a.batch, a.n_kv_head, a.kv_seq, D, a.v_stride))) return rc;
  if ((rc = make_tile_map(&tdo, a.d_o, a.batch, a.n_head, a.q_seq, D, a.do_stride))) return rc;
  {
    static std::atomic<bool> attr_set[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -TYR_ATTN_ERR_NO_DEVICE;
    if (!attr_set[dev].load(std::memory_order_acquire)) {
      cudaError_t e = cudaFuncSetAttribute(bwd_dkdv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)C::kSmemBytes);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)DqCfg<D>::kSmemBytes);
      if (e != cudaSuccess) return (int)e;
      attr_set[dev].store(true, std::memory_order_release);
    }
  }
  {
    constexpr int kLanes = D / 8;
    const int64_t threads = padded_rows * kLanes;
    const int64_t blocks = (threads + 255) / 256;
    if (blocks > 0x7fffffffLL) return -TYR_ATTN_ERR_TOO_LARGE;
    bwd_rowstats_kernel<D><<<(unsigned)blocks, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(a.o), static_cast<const __nv_bfloat16*>(a.d_o), a.lse, neg_lse2,
        neg_delta_s, a.n_head, a.q_seq, sq_pad, a.o_stride[0], a.o_stride[1], a.o_stride[2], a.do_stride[0],
        a.do_stride[1], a.do_stride[2], scale, padded_rows);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }

  BwdParams p;
  p.neg_lse2 = neg_lse2;
  p.neg_delta_s = neg_delta_s;
  p.sq_pad = sq_pad;
  p.batch = a.batch;
  p.q_seq = a.q_seq;
  p.kv_seq = a.kv_seq;
  p.n_head = a.n_head;
  p.n_kv_head = a.n_kv_head;
  p.group = a.n_head / a.n_kv_head;
  p.causal = (a.is_causal || a.window_size > 0) ? 1 : 0;
  p.window = a.window_size > 0 ? a.window_size : 0;
  p.key_mask = a.key_mask;
  p.key_mask_stride = a.key_mask_stride;
  p.n_qblk = n_qblk;
  p.n_kblk = n_kblk;
  p.scale = scale;
  p.sl2 = scale * kLog2e;
  p.status = status;
  p.wait_limit = wait_limit_cycles();

  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const long long grid_kv = (long long)n_kblk * a.n_kv_head * a.batch;
  const long long grid_q = (long long)n_qblk * a.n_head * a.batch;
  if (grid_kv > 0x7fffffffLL || grid_q > 0x7fffffffLL) return -TYR_ATTN_ERR_TOO_LARGE;

  p.out1 = static_cast<__nv_bfloat16*>(a.d_k);
  p.out2 = static_cast<__nv_bfloat16*>(a.d_v);
  for (int i = 0; i < 3; ++i) {
    p.out1_stride[i] = a.dk_stride[i];
    p.out2_stride[i] = a.dv_stride[i];
  }
  bwd_dkdv_kernel<D><<<(unsigned)std::min<long long>(grid_kv, sms), kBwdThreads, C::kSmemBytes, st>>>(tk, tv, tq, tdo, p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;

  p.out1 = static_cast<__nv_bfloat16*>(a.d_q);
  p.out2 = nullptr;
  for (int i = 0; i < 3; ++i) {
    p.out1_stride[i] = a.dq_stride[i];
    p.out2_stride[i] = 0;
  }
  bwd_dq_kernel<D><<<(unsigned)std::min<long long>(grid_q, sms), kBwdThreads, DqCfg<D>::kSmemBytes, st>>>(tq, tdo, tk, tv, p);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace

size_t backward_workspace_bytes(int batch, int n_head, int q_seq) {
  const int64_t sq_pad = (int64_t)((q_seq + kT - 1) / kT) * kT;
  return (size_t)(2 * (int64_t)batch * n_head * sq_pad * (int64_t)sizeof(float));
}

int launch_backward_sm100(const TyrAttnBackwardArgs& a, float scale, int* status, cudaStream_t st) {
  if (a.head_dim == 128) return launch_bwd<128>(a, scale, status, st);
  if (a.head_dim == 64) return launch_bwd<64>(a, scale, status, st);
  return -TYR_ATTN_ERR_HEAD_DIM;
}

}  // namespace tyr
