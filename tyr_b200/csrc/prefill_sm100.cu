// Flash-attention forward for sm_100a: TMA-staged Q/K/V tiles, tcgen05.mma with
// fp32 accumulators in tensor memory for S = Q K^T and O += P V, online softmax
// in the exp2 domain by two softmax warpgroups that each own one 128-row Q tile,
// P handed back to the tensor core through tensor memory, O staged in shared memory and
// written by tiled TMA stores.
// Persistent: one CTA per SM loops over work items, longest causal rows first.
//
// Replaces, for bf16 CUDA tensors, the ATen call behind Tyr's typed attention
// (cc/src/tyr.cpp:2578, 3941, 4126) and the SM90-only DSL kernels
// (Tyr/GPU/Kernels/MhaH100.lean:14-192, FlashAttn3.lean:70-287).  Softmax state
// follows Tyr/GPU/Codegen/Macros.lean:121-163: running max, running sum, rescale
// of the output accumulator, LSE = log(rowSum) + rowMax of the scaled scores.
//
// One work item = two 128-row Q tiles: 256 query rows of one (batch, query head), or the same 128
// rows of two query heads that share a KV head.
//   warp 0     : TMA producer (one elected lane)
//   warp 1     : tcgen05.mma issuer (one elected lane)
//   warp 2     : tensor-memory allocation
//   warp 3     : TMA stores of finished O tiles out of the staging buffer (one elected lane)
//   warps 4-7  : softmax + epilogue of Q tile 0 (thread = one row = one TMEM lane)
//   warps 8-11 : softmax + epilogue of Q tile 1
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D);
// P_t (bf16, 64 columns) overwrites the first half of S_t once the row is in registers.
// Issue order S0(j+1) / PV1(j) / S1(j+1) / PV0(j+1) keeps the tensor pipe busy
// while each softmax warpgroup has two MMA slots of time per KV tile.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <utility>
#include <vector>

#include "attn_internal.h"
#include "ptx_sm100.cuh"

namespace tyr {

// SMs of the current device (the prefill kernels run one persistent CTA on each)
int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  static std::atomic<int> cache[64] = {};
  if (dev >= 0 && dev < 64 && (n = cache[dev].load(std::memory_order_relaxed)) > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev >= 0 && dev < 64) cache[dev].store(n, std::memory_order_relaxed);
  return n;
}
namespace {

constexpr int kBM = 128;        // query rows per tile (= TMEM lanes)
constexpr int kBN = 128;        // keys per KV tile
constexpr int kThreads = 384;   // 12 warps
constexpr float kRescaleThreshold = 8.0f;  // log2 units; below it the stale max is kept
constexpr int kExpPolyPairs = 2;           // of every 8 column pairs, computed on the FMA pipe (see exp_chunk)
// Register split.  setmaxnreg only moves registers inside what the CTA was given at
// launch (threads x the compiled per-thread count, 168 under __launch_bounds__(384, 1));
// asking for more would block a warp forever, so the sum is checked here.
constexpr int kLaunchRegs = 168, kCtrlRegs = 88, kSoftmaxRegs = 208;
static_assert(128 * kCtrlRegs + 256 * kSoftmaxRegs <= kThreads * kLaunchRegs, "register pool of the CTA");

// Division of a non-negative 32-bit number by a divisor fixed per launch, as a multiply-high and a
// shift: q = umulhi(n, mul) >> shr with mul = ceil(2^(31 + ceil(log2 d)) / d), exact for n < 2^31.
// Every role decodes its item index at every item boundary; the hardware has no integer divider,
// and seven emulated divisions are about a thousand cycles on the path between two items.
struct FastDiv {
  uint32_t mul, shr, d;
  __device__ __forceinline__ int div(int n) const {
    return d == 1u ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), mul) >> shr);
  }
};
inline FastDiv make_fastdiv(int d) {
  FastDiv f;
  f.d = static_cast<uint32_t>(std::max(d, 1));
  f.mul = 0;
  f.shr = 0;
  if (f.d > 1u) {
    int lg = 0;
    while ((1ull << lg) < f.d) ++lg;  // ceil(log2 d)
    const int pw = 31 + lg;
    f.mul = static_cast<uint32_t>(((1ull << pw) + f.d - 1) / f.d);
    f.shr = static_cast<uint32_t>(pw - 32);
  }
  return f;
}

struct PrefillParams {
  __nv_bfloat16* o;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  float* lse;
  int64_t lse_stride_b, lse_stride_h;
  int q_seq, kv_seq, group, causal;
  int window;  // 0: none; > 0: key j visible to query i only while i - j < window (causal)
  const uint8_t* key_mask;   // [batch, kv_seq] bytes, 0 = padding key hidden from every query; or null
  int64_t key_mask_stride;
  int n_head, batch, n_mblk;  // work items: n_mblk x heads_per_group_items x groups
  int pair_heads;             // 1: an item is one 128-row block of TWO query heads of a KV head
  int items_per_group;        // items per (batch, KV head): n_mblk * group (/ 2 when pairing heads)
  int n_kv_head, groups_per_chunk;  // (batch, KV head) groups whose K/V share L2 at one time
  int snake;  // 1: odd rounds of the static schedule are mirrored
  float scale_log2;           // scale * log2(e)
  int* status;
  long long wait_limit;  // cycles any single barrier wait may take before the CTA gives up
  // the item decode's divisors in multiply-high form (decode_item<., true>)
  int heads_per_level;        // items per row block per (batch, KV head): group, or group / 2 when pairing heads
  FastDiv by_chunk_items;     // / (groups_per_chunk * items_per_group)
  FastDiv by_level_full, by_level_last;  // / (groups in the chunk * heads_per_level), full chunks and the last one
  FastDiv by_heads_per_level, by_kv_heads;
  // Key-split of the last round (prefill_kernel<., ., true> only).  Items split_from .. split_from +
  // n_split - 1 are each done as n_parts (2 to 8) work items over one part of the KV tiles; a part
  // writes a normalised bf16 partial O [n_parts][n_split][2 tiles][128 rows][D] and its LSE to the
  // caller's workspace, and prefill_split_merge_kernel combines them.
  int split_from, n_split;
  __nv_bfloat16* o_part;
  float* lse_part;
  // Tabled schedule (prefill_kernel<., ., ., true> only): item_table[round * gridDim.x + CTA] is the
  // item the CTA works on in that round, -1 once it has none left.
  const int* item_table;
  int table_rounds;
  // (key-split, continued: kept behind the fields above so that their offsets stay what they were)
  int n_parts;
  FastDiv by_parts;
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
  // O leaves through a staged tile and TMA stores where items are long (D=128); at D=64 the items of
  // the workloads are a few tiles long and the extra hop costs more than the scattered stores do
  static constexpr bool kStageO = (D == 128);
  static constexpr uint32_t kOOff = kVOff + kVStages * kTileBytes;  // one O tile staged for its TMA store
  static constexpr uint32_t kBarOff = kOOff + kTileBytes;
  static constexpr int kNumBars = 2 + 2 + 2 * kKStages + 2 * kVStages + 2 + 2 + 2 + 2 + 1 + 2;
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
  static constexpr int q_full = 0;                        // [2] Q_t of the current item landed
  static constexpr int q_empty = 2;                       // [2] last S_t of the item has read Q_t
  static constexpr int k_full = 4;                        // [KS]
  static constexpr int k_empty = k_full + C::kKStages;    // [KS]
  static constexpr int v_full = k_empty + C::kKStages;    // [VS]
  static constexpr int v_empty = v_full + C::kVStages;    // [VS]
  static constexpr int s_full = v_empty + C::kVStages;    // [2] S_t in tensor memory
  static constexpr int p_half = s_full + 2;               // [2] keys 0..63 of P_t written
  static constexpr int p_full = p_half + 2;               // [2] keys 64..127 of P_t written
  static constexpr int o_full = p_full + 2;               // [2] last PV_t of the item done
  static constexpr int o_staged = o_full + 2;             // an O tile is in the staging buffer (4 warp arrivals)
  static constexpr int o_stage_free = o_staged + 1;       // [2] the TMA store of Q tile t's O has read the buffer
  __device__ static constexpr uint32_t count(int i) {
    return ((i >= p_half && i < p_half + 4) || i == o_staged) ? 4u : 1u;  // one arrival per softmax warp
  }
};

// One work item = 256 query rows of one (batch, query head).  Item order: the
// (batch, KV head) groups are cut into chunks whose K/V fit in L2 together; inside a
// chunk the longest causal rows come first (so the static round-robin over CTAs stays
// balanced and the light items fill the tail), and the query heads that share a KV
// head are neighbours, so CTAs running at the same time read the same K/V tiles.
struct Item {
  int mblk, b, hkv;
  int hq[2];   // query head of Q tile 0 / 1
  int row[2];  // first query row of Q tile 0 / 1
  int lo;      // first KV tile of the item (> 0 under a sliding window and for the second half of a split item)
  int n0, n1;  // KV tiles Q tile 0 / Q tile 1 visit, counted from `lo`
  int part_slot;  // -1, or (part of the keys this work item covers) * n_split + index among the split items
};
// Two ways to fill the two Q-tile slots of an item:
//  rows  : 256 consecutive rows of one query head (tile 1 sits 128 rows below tile 0);
//  heads : the same 128 rows of two query heads that share a KV head (GQA).  Both tiles
//          then visit exactly the same K/V tiles, so under a causal mask neither waits
//          for the other's extra diagonal tile, and a short query block wastes no slot.
// kFast: the divisions as multiply-high (FastDiv).  The D=64 instantiations take it: their
// workloads are short items (the char-level GPT shape has 2.6 items of 1-2 KV tiles per CTA, and
// the decode sat on the path between them: 24.4 -> 22.7 us).  With the long items of the D=128
// workloads nothing is gained at the boundary, and that form of this function measured 3 % slower
// there (1113 vs 1154 TFLOP/s, either order), so they keep the plain divisions.
template <bool kWindow, bool kFast>
__device__ __forceinline__ Item decode_item(int w, const PrefillParams& p) {
  Item it;
  const int n_groups = p.batch * p.n_kv_head;
  int hl;  // item within the row block of its group
  if (kFast) {
    const int chunk = p.by_chunk_items.div(w);
    const int within = w - chunk * static_cast<int>(p.by_chunk_items.d);
    const int g0 = chunk * p.groups_per_chunk;
    const bool full = n_groups - g0 >= p.groups_per_chunk;
    const FastDiv& by_level = full ? p.by_level_full : p.by_level_last;
    const int level = by_level.div(within);
    it.mblk = p.n_mblk - 1 - level;
    const int idx = within - level * static_cast<int>(by_level.d);
    const int gl = p.by_heads_per_level.div(idx);
    hl = idx - gl * p.heads_per_level;
    const int gi = g0 + gl;
    it.b = p.by_kv_heads.div(gi);
    it.hkv = gi - it.b * p.n_kv_head;
  } else {
    const int items_per_group = p.items_per_group;
    const int heads_per_level = p.pair_heads ? p.group / 2 : p.group;  // items per row block per group
    const int chunk = w / (p.groups_per_chunk * items_per_group);
    const int within = w - chunk * p.groups_per_chunk * items_per_group;
    const int g0 = chunk * p.groups_per_chunk;
    const int groups_here = min(p.groups_per_chunk, n_groups - g0);
    const int per_level = groups_here * heads_per_level;
    it.mblk = p.n_mblk - 1 - within / per_level;
    const int idx = within % per_level;
    const int gi = g0 + idx / heads_per_level;
    it.b = gi / p.n_kv_head;
    it.hkv = gi % p.n_kv_head;
    hl = idx % heads_per_level;
  }
  const int nkv_total = (p.kv_seq + kBN - 1) / kBN;
  int last0, last1;  // last KV tile (exclusive) under a causal mask
  if (p.pair_heads) {
    it.hq[0] = it.hkv * p.group + 2 * hl;
    it.hq[1] = it.hq[0] + 1;
    it.row[0] = it.row[1] = it.mblk * kBM;
    last0 = last1 = it.mblk + 1;
  } else {
    it.hq[0] = it.hq[1] = it.hkv * p.group + hl;
    it.row[0] = it.mblk * 2 * kBM;
    it.row[1] = it.row[0] + kBM;
    last0 = 2 * it.mblk + 1;  // top-left causal: a tile needs the keys up to its last row
    last1 = 2 * it.mblk + 2;
  }
  // Sliding window: the first row of the item sees no key before row - window + 1.  Both
  // Q tiles start at that tile; a tile that lies wholly before a row's window is masked
  // out for that row (the softmax copes with rows that have seen no key yet).
  it.lo = (kWindow && p.window > 0) ? max(0, it.row[0] - p.window + 1) / kBN : 0;
  it.n0 = (p.causal ? min(nkv_total, last0) : nkv_total) - it.lo;
  it.n1 = (p.causal ? min(nkv_total, last1) : nkv_total) - it.lo;
  return it;
}

// Static schedule: in round `it` CTA c takes item it*G + c; with `snake` odd rounds
// are mirrored (G-1-c), so that with costs falling along the item order every CTA
// gets the same mix of long and short items.  -1 when the CTA has no item in this round
// (which can only be its last round).
__device__ __forceinline__ int snake_item(int it, int total_items, int snake) {
  const int G = gridDim.x;
  const int c = ((it & 1) && snake) ? (G - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const long long w = (long long)it * G + c;
  if ((long long)it * G >= total_items) return -1;
  return w < total_items ? (int)w : -2;
}

// Tabled schedule: the launch's items dealt to the CTAs by the host, longest first to the least loaded
// CTA (the item order is already longest first inside every L2-sized chunk).  The static round-robin
// leaves the CTAs of the headline workload (items in three chunks, 27.7 rounds) up to 4.2 % above
// the mean load, this packing 0.4 %; measured 1155 -> 1173-1178 TFLOP/s on it, outputs bit-identical.
__device__ __forceinline__ int item_of_table(int it, const PrefillParams& p) {
  return it < p.table_rounds ? __ldg(p.item_table + (int64_t)it * gridDim.x + blockIdx.x) : -1;
}

// Work item w of the launch: the items before p.split_from as they are, the ones from there on as
// two to eight parts of their KV tiles each (non-causal launches only, so both Q tiles visit every tile).
template <int D, bool kWindow, bool kSplit>
__device__ __forceinline__ Item work_item(int w, const PrefillParams& p) {
  if (!kSplit || w < p.split_from) {
    Item it = decode_item<kWindow, D == 64>(w, p);
    it.part_slot = -1;
    return it;
  }
  const int s = w - p.split_from;
  const int slot = p.by_parts.div(s);
  const int part = s - slot * p.n_parts;
  Item it = decode_item<kWindow, D == 64>(p.split_from + slot, p);
  const int n = it.n1;  // KV tiles of the whole item; part k covers tiles [k n / parts, (k + 1) n / parts)
  it.part_slot = part * p.n_split + slot;
  it.lo = part * n / p.n_parts;
  it.n0 = it.n1 = (part + 1) * n / p.n_parts - it.lo;
  return it;
}

// The issuing thread shares its SM sub-partition with two softmax warps, so every
// instruction it spends per MMA delays the tensor pipe: descriptors are built once per
// tile and stage, and each MMA only adds a compile-time constant to the address field.
constexpr uint32_t kDescHi = umma_desc_hi(1024);  // 8-row groups of every operand tile are 1024 B apart

struct NoPeek {
  __device__ __forceinline__ void operator()() const {}
};

// `peek` runs before the last two MMAs of the group.  An MMA takes about as long to issue as to
// execute (about 50 cycles against 64), so what the issuing thread asks there, the state of the
// barrier it will wait on next, is answered by the time the group is issued, and the tensor pipe
// does not drain behind the latency of a wait that would have succeeded anyway.
template <int D, class Peek = NoPeek>
__device__ __forceinline__ void issue_qk(uint32_t issue, uint32_t s_tmem, uint32_t q_lo, uint32_t k_lo, Peek peek = Peek()) {
  constexpr uint32_t idesc = umma_idesc_bf16(kBM, kBN, false);
  // Opaque to the optimizer: the per-step descriptors are recomputed at each use instead of
  // being kept (and spilled) as loop invariants of the issuing thread.
  asm volatile("" : "+r"(q_lo), "+r"(k_lo));
#pragma unroll
  for (int kb = 0; kb < D / 64; ++kb) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint32_t off = (kb * Cfg<D>::kBoxBytes + ks * 32) >> 4;
      if (kb == D / 64 - 1 && ks == 2) peek();
      if (kb == 0 && ks == 0)
        umma_ss_lo_p<0>(s_tmem, q_lo, k_lo, kDescHi, idesc, 0, issue);
      else
        umma_ss_lo_p<1>(s_tmem, q_lo + off, k_lo + off, kDescHi, idesc, 1, issue);
    }
  }
}

// `half` selects keys [64*half, 64*half + 64) of the tile.
template <int D, class Peek = NoPeek>
__device__ __forceinline__ void issue_pv(uint32_t issue, uint32_t o_tmem, uint32_t p_tmem, uint32_t v_lo,
                                         bool accumulate, int half, Peek peek = Peek()) {
  constexpr uint32_t idesc = umma_idesc_bf16(kBM, D, true);
  asm volatile("" : "+r"(v_lo), "+r"(p_tmem));  // as in issue_qk
#pragma unroll
  for (int k4 = 0; k4 < kBN / 32; ++k4) {
    const int kk = half * (kBN / 32) + k4;
    if (k4 == kBN / 32 - 2) peek();
    // 16 keys = two 8-row groups of the V tile; 16 bf16 of P = 8 TMEM columns
    if (k4 == 0)
      umma_ts_lo_p<-1>(o_tmem, p_tmem + kk * 8, v_lo + ((kk * 2048) >> 4), kDescHi, idesc, accumulate ? 1u : 0u, issue);
    else
      umma_ts_lo_p<1>(o_tmem, p_tmem + kk * 8, v_lo + ((kk * 2048) >> 4), kDescHi, idesc, 1, issue);
  }
}

// exp2 of one 32-column chunk of a score row, packed to bf16x2, with the row sum in fp32.  kPoly of
// every 8 column pairs take the FMA-pipe polynomial, the rest ex2.approx.  With the MMA issuer
// running ahead of the tensor pipe the softmax warps are what bounds a KV tile, and a quarter of
// the exponentials off the special-function unit is the measured optimum (2 of 8: +6 % on the
// long-sequence workloads; 3 of 8 starts to spill and loses).
// (Measured and left out: ex2.approx.ftz.bf16x2 / ex2.approx.f16x2 take 16 cycles per warp
// instruction on the special-function unit against 8 for the f32 form, so packing two scores
// into one op gains nothing.)
template <int kPoly>
__device__ __forceinline__ void exp_chunk(const uint32_t (&sr)[32], uint64_t sl2x2, uint64_t negx2,
                                          uint32_t (&pk)[16], uint64_t& sum_a, uint64_t& sum_b) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint64_t t2 = fma_f32x2(pack_u32x2(sr[2 * i], sr[2 * i + 1]), sl2x2, negx2);
    float p0, p1;
    if ((i & 7) < kPoly) {
      ex2_poly_pair(t2, p0, p1);
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

// Persistent kernel: CTA c works on items c, c + gridDim.x, ...  Barrier phases
// run on across items (every role counts its own uses), tensor memory and the
// barriers are set up once, the next item's Q/K loads and first QK^T overlap the
// previous item's epilogue.
// kWindow compiles the sliding-window and padding-key masks in (rows may then meet tiles in
// which they see no key); the plain kernel carries none of those checks.
// kSplit compiles the key-split of the last round in (work_item); the plain kernel has no trace of it.
template <int D, bool kWindow, bool kSplit, bool kTabled>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               const PrefillParams p, const __grid_constant__ CUtensorMap tm_op) {
  using C = Cfg<D>;
  using B = Bars<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t tmem_slot;
  __shared__ WaitCtl wait_ctl;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 128B-swizzle atoms need 1024-byte alignment
  const uint32_t sQ = base + C::kQOff, sK = base + C::kKOff, sV = base + C::kVOff, sO = base + C::kOOff;
  const uint32_t sBar = base + C::kBarOff;
  auto bar = [&](int i) { return sBar + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the merge kernel behind a split launch may become resident as SMs fall free (it waits for this grid itself)
  if (kSplit) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int total_items = p.items_per_group * p.n_kv_head * p.batch + (kSplit ? p.n_split * (p.n_parts - 1) : 0);

  if (threadIdx.x == 0) {
    wait_ctl.abort = 0;
    wait_ctl.limit = p.wait_limit;
    for (int i = 0; i < C::kNumBars; ++i) mbar_init(bar(i), B::count(i));
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
  volatile WaitCtl* abortp = &wait_ctl;

  // Register budget: the four warps of the first warpgroup only issue copies and
  // MMAs; the softmax warpgroups hold a whole 128-column score row per thread.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kCtrlRegs));
    if (warp == 0) {
      // ---------------------------------------------------------- producer
      if (lane == 0) {
        bool ok = true;
        int kc = 0, vc = 0;  // K / V tiles loaded so far, over all items
        for (int it = 0; ok; ++it) {
          const int w = kTabled ? item_of_table(it, p) : snake_item(it, total_items, p.snake);
          if (w < 0) break;
          const Item im = work_item<D, kWindow, kSplit>(w, p);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (it > 0) ok = ok && mbar_wait(bar(B::q_empty + t), (it - 1) & 1, abortp);
            if (!ok) break;
            mbar_expect_tx(bar(B::q_full + t), C::kTileBytes);
#pragma unroll
            for (int kb = 0; kb < C::kBoxes; ++kb)
              tma_load_4d(sQ + t * C::kTileBytes + kb * C::kBoxBytes, &tm_q, bar(B::q_full + t), kb * 64,
                          im.row[t], im.hq[t], im.b);
          }
          auto load_k = [&](int j) {
            const int s = kc % C::kKStages;
            if (kc >= C::kKStages) ok = ok && mbar_wait(bar(B::k_empty + s), ((kc / C::kKStages) - 1) & 1, abortp);
            if (!ok) return;
            mbar_expect_tx(bar(B::k_full + s), C::kTileBytes);
#pragma unroll
            for (int kb = 0; kb < C::kBoxes; ++kb)
              tma_load_4d(sK + s * C::kTileBytes + kb * C::kBoxBytes, &tm_k, bar(B::k_full + s), kb * 64,
                          (im.lo + j) * kBN, im.hkv, im.b);
            ++kc;
          };
          auto load_v = [&](int j) {
            const int s = vc % C::kVStages;
            if (vc >= C::kVStages) ok = ok && mbar_wait(bar(B::v_empty + s), ((vc / C::kVStages) - 1) & 1, abortp);
            if (!ok) return;
            mbar_expect_tx(bar(B::v_full + s), C::kTileBytes);
#pragma unroll
            for (int kb = 0; kb < C::kBoxes; ++kb)
              tma_load_4d(sV + s * C::kTileBytes + kb * C::kBoxBytes, &tm_v, bar(B::v_full + s), kb * 64,
                          (im.lo + j) * kBN, im.hkv, im.b);
            ++vc;
          };
          if (ok) load_k(0);
          for (int j = 0; j < im.n1 && ok; ++j) {
            if (j + 1 < im.n1) load_k(j + 1);
            load_v(j);
          }
        }
      }
    } else if (warp == 1) {
      // -------------------------------------------------------- MMA issuer
      // The whole warp runs this loop, convergent; one elected lane issues the MMAs and commits.
      {
        const uint32_t issue = elect_one();
        const uint32_t tS0 = tmem + C::kTmemS, tS1 = tS0 + kBN;
        const uint32_t tO0 = tmem + C::kTmemO, tO1 = tO0 + D;
        const uint32_t q_desc0 = umma_desc_lo(sQ, 16);
        const uint32_t q_desc1 = umma_desc_lo(sQ + C::kTileBytes, 16);
        bool ok = true;
        int kc = 0, vc = 0;      // K / V tiles consumed so far
        int pc0 = 0, pc1 = 0;    // P tiles consumed so far, per Q tile
        for (int it = 0; ok; ++it) {
          const int w = kTabled ? item_of_table(it, p) : snake_item(it, total_items, p.snake);
          if (w < 0) break;
          const Item im = work_item<D, kWindow, kSplit>(w, p);
          const int n0 = im.n0, n1 = im.n1;
          ok = mbar_wait(bar(B::q_full + 0), it & 1, abortp) && mbar_wait(bar(B::q_full + 1), it & 1, abortp) &&
               mbar_wait(bar(B::k_full + kc % C::kKStages), (kc / C::kKStages) & 1, abortp);
          if (!ok) break;
          tc_fence_after();
          {
            const int s = kc % C::kKStages;
            const uint32_t k_desc = umma_desc_lo(sK + s * C::kTileBytes, 16);
            issue_qk<D>(issue, tS0, q_desc0, k_desc);
            umma_commit_p(bar(B::s_full + 0), issue);
            if (n0 == 1) umma_commit_p(bar(B::q_empty + 0), issue);
            issue_qk<D>(issue, tS1, q_desc1, k_desc);
            umma_commit_p(bar(B::s_full + 1), issue);
            if (n1 == 1) umma_commit_p(bar(B::q_empty + 1), issue);
            umma_commit_p(bar(B::k_empty + s), issue);
            ++kc;
          }
          // answers to the next waits, asked from inside the MMA group issued before each of them
          uint32_t pk = 0;  // bits: 1 V tile landed, 2 K tile landed, 4 / 8 first half / all of P_0 written, 16 / 32 of P_1
          for (int j = 0; j < n1 && ok; ++j) {
            const int vs = vc % C::kVStages;
            const bool next = (j + 1 < n1);
            const int ks = kc % C::kKStages;
            if (!(pk & 1u)) ok = mbar_wait(bar(B::v_full + vs), (vc / C::kVStages) & 1, abortp);
            if (ok && next && !(pk & 2u)) ok = mbar_wait(bar(B::k_full + ks), (kc / C::kKStages) & 1, abortp);
            if (!ok) break;
            const uint32_t v_smem = umma_desc_lo(sV + vs * C::kTileBytes, C::kBoxBytes);
            const uint32_t k_smem = umma_desc_lo(sK + ks * C::kTileBytes, 16);
            if (j < n0) {
              if (!(pk & 4u)) ok = mbar_wait(bar(B::p_half + 0), pc0 & 1, abortp);
              if (!ok) break;
              tc_fence_after();
              issue_pv<D>(issue, tO0, tS0, v_smem, j > 0, 0, [&] { pk |= mbar_test(bar(B::p_full + 0), pc0 & 1) << 3; });
              if (!(pk & 8u)) ok = mbar_wait(bar(B::p_full + 0), pc0 & 1, abortp);
              if (!ok) break;
              tc_fence_after();
              if (j + 1 < n0) {
                issue_pv<D>(issue, tO0, tS0, v_smem, true, 1);
              } else {  // no score product follows: ask about the other tile's P from here
                issue_pv<D>(issue, tO0, tS0, v_smem, true, 1, [&] { pk |= mbar_test(bar(B::p_half + 1), pc1 & 1) << 4; });
              }
              ++pc0;
              if (j == n0 - 1) umma_commit_p(bar(B::o_full + 0), issue);
            }
            if (j + 1 < n0) {
              issue_qk<D>(issue, tS0, q_desc0, k_smem, [&] { pk |= mbar_test(bar(B::p_half + 1), pc1 & 1) << 4; });
              umma_commit_p(bar(B::s_full + 0), issue);
              if (j + 1 == n0 - 1) umma_commit_p(bar(B::q_empty + 0), issue);
            }
            if (!(pk & 16u)) ok = mbar_wait(bar(B::p_half + 1), pc1 & 1, abortp);
            if (!ok) break;
            tc_fence_after();
            issue_pv<D>(issue, tO1, tS1, v_smem, j > 0, 0, [&] { pk |= mbar_test(bar(B::p_full + 1), pc1 & 1) << 5; });
            if (!(pk & 32u)) ok = mbar_wait(bar(B::p_full + 1), pc1 & 1, abortp);
            if (!ok) break;
            tc_fence_after();
            issue_pv<D>(issue, tO1, tS1, v_smem, true, 1);
            ++pc1;
            umma_commit_p(bar(B::v_empty + vs), issue);
            ++vc;
            if (j == n1 - 1) umma_commit_p(bar(B::o_full + 1), issue);
            if (next) {
              // the next step starts with three waits and no MMA between them: ask about all three
              pk = 0;  // every answer of this step has been used
              issue_qk<D>(issue, tS1, q_desc1, k_smem, [&] {
                pk = mbar_test(bar(B::v_full + vc % C::kVStages), (vc / C::kVStages) & 1);
                if (j + 2 < n1) pk |= mbar_test(bar(B::k_full + (kc + 1) % C::kKStages), ((kc + 1) / C::kKStages) & 1) << 1;
                if (j + 1 < n0) pk |= mbar_test(bar(B::p_half + 0), pc0 & 1) << 2;
              });
              umma_commit_p(bar(B::s_full + 1), issue);
              if (j + 1 == n1 - 1) umma_commit_p(bar(B::q_empty + 1), issue);
              umma_commit_p(bar(B::k_empty + ks), issue);
              ++kc;
            }
          }
        }
      }
    } else if (warp == 3) {
      // -------------------------------------------------------- O store
      // The softmax warps put a finished O tile into the staging buffer as bf16 (row-per-thread
      // stores to global memory would be 32 scattered 16-byte pieces per instruction); this warp
      // sends it out with one tiled TMA store per 64 columns and frees the buffer once the store
      // has read it.  Use number u = 2 item + tile; the uses are strictly ordered: a tile stages
      // only after the store of the use before it (the other tile's) has read the buffer.
      if (lane == 0 && C::kStageO) {
        bool ok = true;
        int u = 0;
        for (int it = 0; ok; ++it) {
          const int w = kTabled ? item_of_table(it, p) : snake_item(it, total_items, p.snake);
          if (w < 0) break;
          const Item im = work_item<D, kWindow, kSplit>(w, p);
#pragma unroll
          for (int t = 0; t < 2; ++t, ++u) {
            ok = mbar_wait(bar(B::o_staged), u & 1, abortp);
            if (!ok) break;
            if (kSplit && im.part_slot >= 0) {  // a half's partial tile: all 128 rows, to the workspace
#pragma unroll
              for (int kb = 0; kb < C::kBoxes; ++kb)
                tma_store_4d(&tm_op, sO + kb * C::kBoxBytes, kb * 64, 0, t, im.part_slot);
              tma_store_commit();
              tma_store_wait_read0();
            } else if (im.row[t] < p.q_seq) {  // rows past the tensor are clipped by the store; a tile wholly past it is skipped
#pragma unroll
              for (int kb = 0; kb < C::kBoxes; ++kb)
                tma_store_4d(&tm_o, sO + kb * C::kBoxBytes, kb * 64, im.row[t], im.hq[t], im.b);
              tma_store_commit();
              tma_store_wait_read0();
            }
            mbar_arrive(bar(B::o_stage_free + t));
          }
        }
        // every store has been waited for as far as its reads of shared memory go; its writes are
        // complete when the grid is
      }
    }
  } else {
    // ------------------------------------------------- softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int t = (warp - 4) >> 2;          // Q tile of this warpgroup
    const int quarter = warp & 3;           // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;      // row within the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_addr + C::kTmemS + t * kBN;
    const uint32_t tO = tmem + lane_addr + C::kTmemO + t * D;
    const float sl2 = p.scale_log2;
    bool ok = true;
    int sc = 0;  // score tiles of this Q-tile slot processed so far, over all items

    for (int it = 0; ok; ++it) {
      const int w = kTabled ? item_of_table(it, p) : snake_item(it, total_items, p.snake);
      if (w < 0) break;
      const Item im = work_item<D, kWindow, kSplit>(w, p);
      const int row = (t ? im.row[1] : im.row[0]) + r;  // query index
      const int hq = t ? im.hq[1] : im.hq[0];
      const int n_t = t ? im.n1 : im.n0;
      float m_ref = -INFINITY, l = 0.f;

      for (int j = 0; j < n_t; ++j, ++sc) {
        ok = mbar_wait(bar(B::s_full + t), sc & 1, abortp);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr[kBN / 32][32];  // the row's scores, raw fp32 bits
#pragma unroll
        for (int c = 0; c < kBN / 32; ++c) tmem_ld32(tS + c * 32, sr[c]);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < kBN / 32; ++c) tmem_ld_ready(sr[c]);

        // keys this row may see in this tile: [first, limit)
        const int key0 = (im.lo + j) * kBN;
        int limit = p.kv_seq - key0;
        if (p.causal) limit = min(limit, row + 1 - key0);
        const int first = (kWindow && p.window > 0) ? row - p.window + 1 - key0 : 0;
        if (limit < kBN || first > 0) {
#pragma unroll
          for (int c = 0; c < kBN; ++c)
            if (c >= limit || c < first) sr[c >> 5][c & 31] = 0xff800000u;  // -inf
        }
        if (kWindow && p.key_mask != nullptr) {
          // padding keys: lane i fetches the mask bytes of keys 4i..4i+3 of the tile, four
          // ballots spread them to every row; key c is bit (c >> 2) of ballot (c & 3)
          const uint8_t* mrow = p.key_mask + im.b * p.key_mask_stride + key0;
          uint32_t vb[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int kk = 4 * lane + e;
            const bool valid = (key0 + kk < p.kv_seq) && mrow[kk] != 0;
            vb[e] = __ballot_sync(0xffffffffu, valid);
          }
#pragma unroll
          for (int c = 0; c < kBN; ++c)
            if (!((vb[c & 3] >> (c >> 2)) & 1u)) sr[c >> 5][c & 31] = 0xff800000u;  // -inf
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
            // before this warp arrives on p_half, so O_t is ours to rescale.
            // a row that has seen no key yet (m_new still -inf, sliding window only) keeps its zeros
            const float alpha = (kWindow && m_new == -INFINITY) ? 1.0f : ex2_approx((m_ref - m_new) * sl2);
            l *= alpha;
            m_ref = m_new;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(tO + c * 32, o);
              tmem_wait_ld();
              tmem_ld_ready(o);
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + c * 32, o);
            }
          }
        }
        const float neg = (kWindow && m_ref == -INFINITY) ? 0.0f : -m_ref * sl2;  // all -inf scores give P = 0
        const uint64_t sl2x2 = pack_f32x2(sl2, sl2), negx2 = pack_f32x2(neg, neg);
        uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t pk[16];
          exp_chunk<kWindow ? 0 : kExpPolyPairs>(sr[c], sl2x2, negx2, pk, sum_a, sum_b);
          tmem_st16(tS + c * 16, pk);
          if (c == 1) {  // keys 0..63 of P are in tensor memory: the first half of PV may start
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B::p_half + t));
          }
        }
        {
          float s0, s1;
          unpack_f32x2(add_f32x2(sum_a, sum_b), s0, s1);
          l += s0 + s1;
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B::p_full + t));
      }
      if (!ok) break;

      // epilogue: O_t / l -> bf16 -> the staging buffer in the 128-byte-swizzled box layout of the
      // tensor map (each thread owns one row; a warp's 16-byte pieces of 32 rows land on distinct
      // bank groups), from where the store warp sends the tile out
      ok = mbar_wait(bar(B::o_full + t), it & 1, abortp);
      // The one staging buffer: the use before this one is the other tile's (tile 0 of this item
      // for tile 1, tile 1 of the previous item for tile 0).  Each tile has its own "store has
      // read the buffer" barrier, completed once per item, and the stores run in use order, so
      // the awaited barrier is never more than one phase away from the awaited phase.
      if (C::kStageO && ok && (t == 1 || it > 0))
        ok = mbar_wait(bar(B::o_stage_free + (1 - t)), (t == 1 ? it : it - 1) & 1, abortp);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float inv_l = 1.0f / l;
      const bool row_ok = row < p.q_seq;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
        tmem_wait_ld();
        tmem_ld_ready(o);
        const uint32_t row_base = sO + (c >> 1) * C::kBoxBytes + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t x = pack_bf16x2(__uint_as_float(o[q4 * 8 + 0]) * inv_l, __uint_as_float(o[q4 * 8 + 1]) * inv_l);
          const uint32_t y = pack_bf16x2(__uint_as_float(o[q4 * 8 + 2]) * inv_l, __uint_as_float(o[q4 * 8 + 3]) * inv_l);
          const uint32_t z = pack_bf16x2(__uint_as_float(o[q4 * 8 + 4]) * inv_l, __uint_as_float(o[q4 * 8 + 5]) * inv_l);
          const uint32_t wq = pack_bf16x2(__uint_as_float(o[q4 * 8 + 6]) * inv_l, __uint_as_float(o[q4 * 8 + 7]) * inv_l);
          if (C::kStageO) {
            const int piece = (c & 1) * 4 + q4;  // 16-byte piece of the row's 128 bytes in this box
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + ((piece ^ (r & 7)) << 4)),
                         "r"(x), "r"(y), "r"(z), "r"(wq)
                         : "memory");
          } else if (kSplit && im.part_slot >= 0) {
            *reinterpret_cast<uint4*>(p.o_part + ((int64_t)(im.part_slot * 2 + t) * kBM + r) * D +
                                      c * 32 + q4 * 8) = make_uint4(x, y, z, wq);
          } else if (row_ok) {  // straight from registers: 16-byte stores of one row per thread
            *reinterpret_cast<uint4*>(p.o + im.b * p.o_stride_b + hq * p.o_stride_h + (int64_t)row * p.o_stride_s +
                                      c * 32 + q4 * 8) = make_uint4(x, y, z, wq);
          }
        }
      }
      if (kSplit && im.part_slot >= 0)
        p.lse_part[(im.part_slot * 2 + t) * kBM + r] = 0.6931471805599453f * (m_ref * sl2 + lg2_approx(l));
      else if (p.lse != nullptr && row_ok)
        p.lse[im.b * p.lse_stride_b + hq * p.lse_stride_h + row] =
            0.6931471805599453f * (m_ref * sl2 + lg2_approx(l));
      // the tile is staged: make the generic-proxy writes visible to the TMA store, then tell the
      // store warp.  O_t is read as well: these loads are ordered before the next item's first
      // PV_t, which this warp gates through p_half.
      if (C::kStageO) fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (C::kStageO && lane == 0) mbar_arrive(bar(B::o_staged));
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
// Encoding a tensor map is pure host arithmetic on (pointer, sizes, strides); a model calls
// the operator with the same few tensors over and over, so each thread keeps the last few.
struct MapKey {
  const void* ptr;
  int batch, heads, seq, d;
  int64_t stride[3];
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && batch == o.batch && heads == o.heads && seq == o.seq && d == o.d &&
           stride[0] == o.stride[0] && stride[1] == o.stride[1] && stride[2] == o.stride[2];
  }
};
constexpr int kMapCache = 16;
struct MapCache {
  MapKey key[kMapCache];
  CUtensorMap map[kMapCache];
  int used = 0, next = 0;
};

int encode_map(CUtensorMap* m, const void* ptr, int batch, int heads, int seq, int d,
               const int64_t* stride);

int make_map(CUtensorMap* m, const void* ptr, int batch, int heads, int seq, int d,
             const int64_t* stride) {
  static thread_local MapCache cache;
  const MapKey k{ptr, batch, heads, seq, d, {stride[0], stride[1], stride[2]}};
  for (int i = 0; i < cache.used; ++i)
    if (cache.key[i] == k) {
      *m = cache.map[i];
      return 0;
    }
  const int rc = encode_map(m, ptr, batch, heads, seq, d, stride);
  if (rc) return rc;
  cache.key[cache.next] = k;
  cache.map[cache.next] = *m;
  cache.next = (cache.next + 1) % kMapCache;
  if (cache.used < kMapCache) ++cache.used;
  return 0;
}

int encode_map(CUtensorMap* m, const void* ptr, int batch, int heads, int seq, int d,
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

// Work items of a launch and the key-split of its last round.  A launch runs its items in rounds of
// one per SM; when the last round is at most half full, a non-causal launch does each of that
// round's items as two to eight work items over one part of the KV tiles each (as many parts as fit
// the SMs, at least four KV tiles per part), so the round takes a half to an eighth as long (216
// equal items on 148 SMs: 36 + 18 tile steps instead of 36 + 36).  The parts leave normalised
// partial outputs in the caller's workspace and prefill_split_merge_kernel combines them.
constexpr int kMaxSplitParts = 8;
struct SplitPlan {
  long long items;  // work items before any split
  int n_split;      // items of the last round to split (0: none)
  int n_parts;      // parts each of them is done in (2 to 8)
  long long bytes;  // workspace the split needs
};
SplitPlan split_plan(const TyrAttnPrefillArgs& a, int n_sm) {
  SplitPlan sp{0, 0, 0, 0};
  const int group = a.n_head / a.n_kv_head;
  const bool masked = a.is_causal || a.window_size > 0;
  const bool pair = group % 2 == 0 && (masked || a.q_seq <= kBM);
  const long long n_mblk = pair ? (a.q_seq + kBM - 1) / kBM : (a.q_seq + 2 * kBM - 1) / (2 * kBM);
  sp.items = n_mblk * (pair ? group / 2 : group) * a.n_kv_head * a.batch;
  // parts of fewer than 4 KV tiles would not pay for the merge launch
  const int nkv = (a.kv_seq + kBN - 1) / kBN;
  if (masked || a.key_mask != nullptr || nkv < 8 || a.check_mode) return sp;
  const long long rem = sp.items % n_sm;
  if (rem == 0 || 2 * rem > n_sm) return sp;
  // The split instantiation's steady state is about 4 % slower than the plain kernel's, which the
  // whole launch pays: past a few rounds that outweighs what the last round can give back (nine
  // rounds with 12 items in the last measured +1.2 %).
  if (sp.items / n_sm > 8) return sp;
  sp.n_split = (int)rem;
  sp.n_parts = (int)std::min<long long>(std::min<long long>(n_sm / rem, kMaxSplitParts), nkv / 4);
  sp.bytes = rem * sp.n_parts * 2 * kBM * ((long long)a.head_dim * 2 + 4);
  return sp;
}

// O = sum_i w_i O_i with w_i = exp(LSE_i - LSE), LSE = log sum_i exp LSE_i: the merge of
// Tyr/GPU/Kernels/RingAttn.lean:164-180 over the parts of a split item.  16 bytes of a row per lane.
template <int D>
__global__ void __launch_bounds__(256) prefill_split_merge_kernel(const PrefillParams p) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int kLanesPerRow = D / 8;            // 16 bytes of a row per lane
  constexpr int kRowsPerWarp = 32 / kLanesPerRow;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int id = (blockIdx.x * 8 + warp) * kRowsPerWarp + lane / kLanesPerRow;  // (slot, tile, row)
  const int col = (lane % kLanesPerRow) * 8;
  const int r = id & (kBM - 1), t = (id >> 7) & 1, slot = id >> 8;
  if (slot >= p.n_split) return;
  const Item im = decode_item<false, true>(p.split_from + slot, p);
  const int row = im.row[t] + r;
  if (row >= p.q_seq) return;
  const int hq = im.hq[t];
  const int64_t i0 = ((int64_t)slot * 2 + t) * kBM + r;
  const int64_t part_stride = (int64_t)p.n_split * 2 * kBM;  // rows between two parts of one item
  float m = -INFINITY;
  for (int k = 0; k < p.n_parts; ++k) m = fmaxf(m, p.lse_part[i0 + k * part_stride]);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, wsum = 0.f;
  for (int k = 0; k < p.n_parts; ++k) {
    const float wk = __expf(p.lse_part[i0 + k * part_stride] - m);
    wsum += wk;
    const uint4 vk = *reinterpret_cast<const uint4*>(p.o_part + (i0 + k * part_stride) * D + col);
    const __nv_bfloat162* pk = reinterpret_cast<const __nv_bfloat162*>(&vk);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(pk[i]);
      acc[2 * i] = fmaf(wk, f.x, acc[2 * i]);
      acc[2 * i + 1] = fmaf(wk, f.y, acc[2 * i + 1]);
    }
  }
  const float inv = 1.0f / wsum;
  uint4 vo;
  __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&vo);
#pragma unroll
  for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
  *reinterpret_cast<uint4*>(p.o + im.b * p.o_stride_b + hq * p.o_stride_h + (int64_t)row * p.o_stride_s + col) = vo;
  if (col == 0 && p.lse != nullptr) p.lse[im.b * p.lse_stride_b + hq * p.lse_stride_h + row] = m + __logf(wsum);
}


// Item tables of the tabled schedule, one per (device, launch geometry), built on first use and kept:
// a few KB of device memory each, at most kMaxItemTables of them (further geometries run the static
// schedule).  Building one allocates and copies synchronously, so a launch that is being captured
// into a graph does not build (it uses a table that exists, else the static schedule).
constexpr int kMaxItemTables = 16;
constexpr long long kMaxTabledItems = 1ll << 18;  // 1 MB of table, some 10 ms to build
struct ItemTable {
  int dev, grid, batch, n_kv_head, n_mblk, pair_heads, items_per_group, groups_per_chunk, causal, kv_seq;
  int* table;
  int rounds;
};
std::mutex g_item_table_mu;
ItemTable g_item_tables[kMaxItemTables];
int g_n_item_tables = 0;

bool item_table_for(PrefillParams& p, int grid, cudaStream_t st) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(g_item_table_mu);
  for (int i = 0; i < g_n_item_tables; ++i) {
    const ItemTable& t = g_item_tables[i];
    if (t.dev == dev && t.grid == grid && t.batch == p.batch && t.n_kv_head == p.n_kv_head && t.n_mblk == p.n_mblk &&
        t.pair_heads == p.pair_heads && t.items_per_group == p.items_per_group &&
        t.groups_per_chunk == p.groups_per_chunk && t.causal == p.causal && t.kv_seq == p.kv_seq) {
      p.item_table = t.table;
      p.table_rounds = t.rounds;
      return true;
    }
  }
  if (g_n_item_tables == kMaxItemTables) return false;
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return false;
  // cost of every item in KV-tile steps (+ half a step for the item boundary), as decode_item counts them
  const long long total = (long long)p.items_per_group * p.n_kv_head * p.batch;
  const int n_groups = p.batch * p.n_kv_head, nkv_total = (p.kv_seq + kBN - 1) / kBN;
  const int heads_per_level = p.heads_per_level;
  std::vector<long long> load(grid, 0);
  std::vector<std::vector<int>> mine(grid);
  // (load, CTA) min-heap: the next item goes to the CTA with the least work so far
  std::vector<std::pair<long long, int>> heap;
  heap.reserve(grid);
  for (int c = 0; c < grid; ++c) heap.emplace_back(0ll, c);
  auto later = [](const std::pair<long long, int>& x, const std::pair<long long, int>& y) { return x > y; };
  std::make_heap(heap.begin(), heap.end(), later);
  for (long long w = 0; w < total; ++w) {
    const long long per_chunk = (long long)p.groups_per_chunk * p.items_per_group;
    const int chunk = (int)(w / per_chunk);
    const int within = (int)(w - chunk * per_chunk);
    const int groups_here = std::min(p.groups_per_chunk, n_groups - chunk * p.groups_per_chunk);
    const int mblk = p.n_mblk - 1 - within / (groups_here * heads_per_level);
    const int last1 = p.pair_heads ? mblk + 1 : 2 * mblk + 2;
    const int n1 = p.causal ? std::min(nkv_total, last1) : nkv_total;
    std::pop_heap(heap.begin(), heap.end(), later);
    std::pair<long long, int>& top = heap.back();
    mine[top.second].push_back((int)w);
    top.first += 2 * n1 + 1;
    std::push_heap(heap.begin(), heap.end(), later);
  }
  size_t rounds = 0;
  for (int c = 0; c < grid; ++c) rounds = std::max(rounds, mine[c].size());
  std::vector<int> host(rounds * grid, -1);
  for (int c = 0; c < grid; ++c)
    for (size_t r = 0; r < mine[c].size(); ++r) host[r * grid + c] = mine[c][r];
  int* d = nullptr;
  if (cudaMalloc(&d, host.size() * sizeof(int)) != cudaSuccess) return false;
  if (cudaMemcpy(d, host.data(), host.size() * sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaFree(d);
    return false;
  }
  g_item_tables[g_n_item_tables++] = ItemTable{dev, grid, p.batch, p.n_kv_head, p.n_mblk, p.pair_heads, p.items_per_group,
                                              p.groups_per_chunk, p.causal, p.kv_seq, d, (int)rounds};
  p.item_table = d;
  p.table_rounds = (int)rounds;
  return true;
}

template <int D, bool kWindow>
int launch(const TyrAttnPrefillArgs& a, float scale, int* status, cudaStream_t st) {
  using C = Cfg<D>;
  CUtensorMap tq, tk, tv, to;
  int rc;
  if ((rc = make_map(&tq, a.q, a.batch, a.n_head, a.q_seq, D, a.q_stride))) return rc;
  if ((rc = make_map(&tk, a.k, a.batch, a.n_kv_head, a.kv_seq, D, a.k_stride))) return rc;
  if ((rc = make_map(&tv, a.v, a.batch, a.n_kv_head, a.kv_seq, D, a.v_stride))) return rc;
  if ((rc = make_map(&to, a.o, a.batch, a.n_head, a.q_seq, D, a.o_stride))) return rc;
  {
    // per-device attribute, set once per device and kernel instantiation
    static std::atomic<bool> attr_set[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -TYR_ATTN_ERR_NO_DEVICE;
    if (!attr_set[dev].load(std::memory_order_acquire)) {
      cudaError_t attr_err = cudaFuncSetAttribute(prefill_kernel<D, kWindow, false, false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)C::kSmemBytes);
      if (attr_err != cudaSuccess) return (int)attr_err;
      if (!kWindow) {
        attr_err = cudaFuncSetAttribute(prefill_kernel<D, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)C::kSmemBytes);
        if (attr_err != cudaSuccess) return (int)attr_err;
      }
      if (!kWindow && D == 128) {
        attr_err = cudaFuncSetAttribute(prefill_kernel<128, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)Cfg<128>::kSmemBytes);
        if (attr_err != cudaSuccess) return (int)attr_err;
      }
      attr_set[dev].store(true, std::memory_order_release);
    }
  }
  PrefillParams p;
  p.o = static_cast<__nv_bfloat16*>(a.o);
  p.o_stride_b = a.o_stride[0];
  p.o_stride_h = a.o_stride[1];
  p.o_stride_s = a.o_stride[2];
  p.n_head = a.n_head;
  p.batch = a.batch;
  {
    const int group = a.n_head / a.n_kv_head;
    // pair two heads of a KV head when that removes idle slots: causal masks, short query blocks
    p.pair_heads = (group % 2 == 0 && (a.is_causal || a.window_size > 0 || a.q_seq <= kBM)) ? 1 : 0;
    p.n_mblk = p.pair_heads ? (a.q_seq + kBM - 1) / kBM : (a.q_seq + 2 * kBM - 1) / (2 * kBM);
    p.items_per_group = p.n_mblk * (p.pair_heads ? group / 2 : group);
  }
  p.n_kv_head = a.n_kv_head;
  {
    // K and V of one (batch, KV head) group.  If all groups fit in L2 together (96 MB of
    // the 126 MB) the items form one chunk and the mirrored schedule balances the few
    // rounds each CTA runs; otherwise chunks of about 48 MB keep the CTAs that run at
    // the same time on K/V that is still in L2, and plain round-robin keeps them close.
    const long long group_bytes = std::max<long long>(2ll * a.kv_seq * D * 2, 1);
    const long long n_groups = (long long)a.batch * a.n_kv_head;
    const bool all_fit = group_bytes * n_groups <= (96ll << 20);
    const long long g = all_fit ? n_groups : std::max<long long>((48ll << 20) / group_bytes, 1);
    p.groups_per_chunk = (int)std::min<long long>(g, n_groups);
    p.snake = all_fit ? 1 : 0;
    p.heads_per_level = p.pair_heads ? (a.n_head / a.n_kv_head) / 2 : a.n_head / a.n_kv_head;
    const int groups_last = (int)(n_groups % p.groups_per_chunk);
    p.by_chunk_items = make_fastdiv(p.groups_per_chunk * p.items_per_group);
    p.by_level_full = make_fastdiv(p.groups_per_chunk * p.heads_per_level);
    p.by_level_last = make_fastdiv(std::max(groups_last, 1) * p.heads_per_level);
    p.by_heads_per_level = make_fastdiv(p.heads_per_level);
    p.by_kv_heads = make_fastdiv(a.n_kv_head);
  }
  p.lse = a.lse;
  p.lse_stride_h = a.q_seq;
  p.lse_stride_b = (int64_t)a.q_seq * a.n_head;
  p.q_seq = a.q_seq;
  p.kv_seq = a.kv_seq;
  p.group = a.n_head / a.n_kv_head;
  p.causal = (a.is_causal || a.window_size > 0) ? 1 : 0;
  p.window = a.window_size > 0 ? a.window_size : 0;
  p.key_mask = a.key_mask;
  p.key_mask_stride = a.key_mask_stride;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.wait_limit = wait_limit_cycles();
  const long long items = (long long)p.items_per_group * a.n_kv_head * a.batch;
  if (items > 0x7fffffffLL) return -TYR_ATTN_ERR_TOO_LARGE;
  p.split_from = (int)items;
  p.n_split = 0;
  p.n_parts = 1;
  p.by_parts = make_fastdiv(1);
  p.o_part = nullptr;
  p.lse_part = nullptr;
  p.item_table = nullptr;
  p.table_rounds = 0;
  if (!kWindow && a.workspace != nullptr) {
    const SplitPlan sp = split_plan(a, sm_count());
    if (sp.n_split > 0 && a.workspace_bytes >= sp.bytes && (reinterpret_cast<uintptr_t>(a.workspace) & 255) == 0) {
      p.n_split = sp.n_split;
      p.n_parts = sp.n_parts;
      p.by_parts = make_fastdiv(sp.n_parts);
      p.split_from = (int)(items - sp.n_split);
      p.o_part = static_cast<__nv_bfloat16*>(a.workspace);
      p.lse_part = reinterpret_cast<float*>(p.o_part + (size_t)sp.n_split * sp.n_parts * 2 * kBM * D);
      CUtensorMap top;
      const int64_t part_stride[3] = {2ll * kBM * D, (int64_t)kBM * D, D};
      if ((rc = make_map(&top, p.o_part, sp.n_parts * sp.n_split, 2, kBM, D, part_stride))) return rc;
      const int grid = (int)std::min<long long>(items + (long long)sp.n_split * (sp.n_parts - 1), sm_count());
      prefill_kernel<D, false, true, false><<<grid, kThreads, C::kSmemBytes, st>>>(tq, tk, tv, to, p, top);
      count_launch();
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return (int)e;
      // programmatic stream serialisation: the merge's launch latency hides behind the kernel's tail
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(sp.n_split * 256 / (8 * (32 / (D / 8))));   // 256 rows per item, 8 warps of 32 / (D / 8) rows
      cfg.blockDim = dim3(256);
      cfg.dynamicSmemBytes = 0;
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      e = cudaLaunchKernelEx(&cfg, prefill_split_merge_kernel<D>, p);
      count_launch();
      if (e == cudaSuccess) e = cudaGetLastError();
      return (int)e;
    }
  }
  const int grid = (int)std::min<long long>(items, sm_count());
  // Items of unequal length in several L2-sized chunks and many rounds: deal them to the CTAs by a
  // table (item_of_table).  Equal items gain nothing from it, and the tabled instantiation measured
  // 2.6 % slower than the plain one on them (Flux-shaped: 1128 vs 1158 TFLOP/s), so they stay static.
  // (and not for launches so large that the table itself would weigh: 4 bytes and a heap step per item)
  if (!kWindow && D == 128 && p.causal && !p.snake && items >= 4ll * grid && items <= kMaxTabledItems &&
      item_table_for(p, grid, st)) {
    prefill_kernel<128, false, false, true><<<grid, kThreads, Cfg<128>::kSmemBytes, st>>>(tq, tk, tv, to, p, to);
    count_launch();
    return (int)cudaGetLastError();
  }
  prefill_kernel<D, kWindow, false, false><<<grid, kThreads, C::kSmemBytes, st>>>(tq, tk, tv, to, p, to);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace

int make_tile_map(CUtensorMap* m, const void* ptr, int batch, int heads, int seq, int d, const int64_t* stride) {
  return make_map(m, ptr, batch, heads, seq, d, stride);
}

long long prefill_split_workspace_bytes(const TyrAttnPrefillArgs& a) {
  if (a.head_dim != 64 && a.head_dim != 128) return 0;
  return split_plan(a, sm_count()).bytes;
}

int launch_prefill_sm100(const TyrAttnPrefillArgs& a, float scale, int* status, cudaStream_t st) {
  const bool win = a.window_size > 0 || a.key_mask != nullptr;
  if (a.head_dim == 128) return win ? launch<128, true>(a, scale, status, st) : launch<128, false>(a, scale, status, st);
  if (a.head_dim == 64) return win ? launch<64, true>(a, scale, status, st) : launch<64, false>(a, scale, status, st);
  return -TYR_ATTN_ERR_HEAD_DIM;
}

}  // namespace tyr
