/*
 * tyr_b200_attn.h — C ABI of the B200 (sm_100a) attention operator.
 *
 * Drop-in boundary for Tyr's typed attention call.  Every entry point takes
 * plain pointers and sizes (no torch / ATen / Lean types), launches on the
 * stream the caller passes (a cudaStream_t cast to void*, exactly the value
 * Tyr's `torch.cuda_current_stream` hands to its generated launchers,
 * cc/src/tyr.cpp:4314-4331) and never synchronises the device unless the
 * entry point is documented as a host-buffer call.
 *
 * Return value of every `int` function: 0 = ok; negative = TYR_ATTN_ERR_*
 * (argument rejected before any launch); positive = a cudaError_t raised by
 * the launch itself.  tyr_b200_attn_strerror() turns either into text for the
 * IO error string Tyr's launchers return (Tyr/GPU/Codegen/Attribute.lean:376-385).
 *
 * All tensors are row-major with unit stride on the head dimension.
 * Strides are in ELEMENTS.  bf16 tensors must be 16-byte aligned with strides
 * that are multiples of 8 elements (TMA requirement).
 */
#ifndef TYR_B200_ATTN_H_
#define TYR_B200_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TYR_ATTN_ABI_VERSION 8

/* element types of Q/K/V/O */
#define TYR_ATTN_BF16 0
#define TYR_ATTN_F32 1 /* accepted only with check_mode = 1 */

/* argument errors (returned negated: -TYR_ATTN_ERR_x) */
#define TYR_ATTN_ERR_NULL 1        /* a required pointer is NULL */
#define TYR_ATTN_ERR_SHAPE 2       /* a size is negative (or zero where zero has no meaning) or n_head % n_kv_head != 0 */
#define TYR_ATTN_ERR_HEAD_DIM 3    /* head_dim not in {64,128} (tensor-core path) */
#define TYR_ATTN_ERR_ALIGN 4       /* pointer or stride breaks the 16-byte rule */
#define TYR_ATTN_ERR_DTYPE 5       /* dtype/check_mode combination not supported */
#define TYR_ATTN_ERR_DROPOUT 6     /* dropout_p != 0: caller keeps its LibTorch path */
#define TYR_ATTN_ERR_WORKSPACE 7   /* workspace missing or too small */
#define TYR_ATTN_ERR_NO_DEVICE 8   /* no sm_100 device / driver entry point missing */
#define TYR_ATTN_ERR_DEVICE_WAIT 9 /* a bounded in-kernel wait gave up (see tyr_b200_attn_device_status) */
#define TYR_ATTN_ERR_TOO_LARGE 10  /* size beyond a documented maximum */
#define TYR_ATTN_ERR_RANGE 11      /* a cache position / sequence length lies outside its stated limits */

/* bits of the per-device status word (tyr_b200_attn_device_status) */
#define TYR_ATTN_STATUS_WAIT_TIMEOUT 1 /* a bounded in-kernel barrier wait ran out */
#define TYR_ATTN_STATUS_ABORTED 2      /* a CTA left early because one of its roles gave up */
#define TYR_ATTN_STATUS_OUT_OF_RANGE 4 /* a device-side position or length was outside its limits;
                                          the offending rows were skipped (prologue) or clamped (decode) */

/* ------------------------------------------------------------------------
 * Prefill: O = softmax(Q K^T * scale + causal) V, per-row LSE.
 *
 * Raw-pointer form of Tyr's generated launcher ABI (caller-allocated outputs,
 * explicit stream; Tyr/GPU/Codegen/Attribute.lean:331-386 and the launch at
 * Examples/GPU/RunFlashAttn.lean:81).  Q head h reads KV head h / (n_head /
 * n_kv_head), the map `repeat_interleave` produces in cc/src/tyr.cpp:3931-3938.
 * `is_causal` masks key j for query i when j > i (top-left aligned, as ATen and
 * cc/src/tyr.cpp:3990-3991).  LSE is the natural log of the sum of exp of the
 * SCALED scores (Tyr/GPU/Codegen/Macros.lean:155-163).
 * Zero extents are treated as ATen's operator treats them: with batch, n_head
 * or q_seq zero the output has no element and the call returns 0 without a
 * launch (pointers may be NULL); with kv_seq zero every output row is 0 and
 * its LSE -inf.
 * ---------------------------------------------------------------------- */
typedef struct TyrAttnPrefillArgs {
  const void* q; /* [batch, n_head,    q_seq,  head_dim] */
  const void* k; /* [batch, n_kv_head, kv_seq, head_dim] */
  const void* v; /* [batch, n_kv_head, kv_seq, head_dim] */
  void* o;       /* [batch, n_head,    q_seq,  head_dim], same dtype as q */
  float* lse;    /* [batch, n_head, q_seq] fp32 contiguous, or NULL */
  int32_t batch, n_head, n_kv_head, q_seq, kv_seq, head_dim;
  int64_t q_stride[3]; /* elements: batch, head, seq */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int32_t dtype;      /* TYR_ATTN_BF16 | TYR_ATTN_F32 */
  int32_t is_causal;  /* 0 | 1 */
  float scale;        /* <= 0 => 1/sqrt(head_dim), ATen's default */
  int32_t check_mode; /* 1 => fp32-FMA kernel (no tensor cores), any head_dim <= 256 */
  int32_t window_size; /* 0 => none; w > 0 => key j is visible to query i only if j <= i and
                          i - j < w (implies is_causal), the mask lean_torch_sdpa_gqa_window
                          builds at cc/src/tyr.cpp:3986-3996.  Needs q_seq == kv_seq, as that
                          call has a single `seq` (cc/src/tyr.cpp:3953-3965) */
  const uint8_t* key_mask; /* NULL, or DEVICE bytes [batch, kv_seq]: 0 marks a padding key that
                              no query sees, any other value a valid key — the key/value part
                              of the padding mask of lean_torch_sdpa_gqa_mask
                              (cc/src/tyr.cpp:4063-4086).  A query that sees no key at all
                              gets NaN output, as it does from ATen. */
  int64_t key_mask_stride; /* bytes between the mask rows of two batch elements */
  void* workspace;         /* NULL, or DEVICE scratch of tyr_b200_attn_prefill_workspace_bytes(args)
                              bytes, 256-byte aligned, private to this call until it has finished on
                              its stream.  With it a non-causal launch whose last round of work items
                              fills at most half the SMs computes that round's items in two to eight
                              parts of their keys and merges them (Tyr/GPU/Kernels/RingAttn.lean:164-180).
                              Without it, or when it is too small, nothing is split. */
  int64_t workspace_bytes;
} TyrAttnPrefillArgs;

int tyr_b200_attn_prefill(const TyrAttnPrefillArgs* args, void* stream);
/* Bytes of `workspace` with which the call above would split its last round on the current
 * device; 0 when it would not split (causal, windowed or masked calls, short key sequences, a
 * last round that is more than half full, more than eight full rounds before it), negative
 * TYR_ATTN_ERR_* on bad arguments. */
int64_t tyr_b200_attn_prefill_workspace_bytes(const TyrAttnPrefillArgs* args);

/* Contiguous-layout forms whose argument lists mirror the Lean externs one to
 * one: tensor handles become device pointers, the result tensor becomes the
 * caller-allocated `out`, and the stream is explicit.  bf16 only.
 *   tyr_b200_sdpa_4d       <- lean_torch_sdpa_4d       cc/src/tyr.cpp:2563-2589
 *   tyr_b200_sdpa_gqa      <- lean_torch_sdpa_gqa      cc/src/tyr.cpp:3913-3949
 *   tyr_b200_sdpa_gqa_qkv  <- lean_torch_sdpa_gqa_qkv  cc/src/tyr.cpp:4100-4133
 * With enable_gqa = 0 the reference passes K/V through unchanged, which ATen
 * only accepts when n_head == n_kv_head; the same rule is enforced here. */
int tyr_b200_sdpa_4d(uint64_t batch, uint64_t n_head, uint64_t seq, uint64_t head_dim,
                     const void* q, const void* k, const void* v, void* out,
                     double dropout_p, uint8_t is_causal, void* stream);
int tyr_b200_sdpa_gqa(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t seq,
                      uint64_t head_dim, const void* q, const void* k, const void* v, void* out,
                      double dropout_p, uint8_t is_causal, uint8_t enable_gqa, void* stream);
int tyr_b200_sdpa_gqa_qkv(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t q_seq,
                          uint64_t kv_seq, uint64_t head_dim, const void* q, const void* k,
                          const void* v, void* out, double dropout_p, uint8_t is_causal,
                          uint8_t enable_gqa, void* stream);
/* tyr_b200_sdpa_gqa_window <- lean_torch_sdpa_gqa_window cc/src/tyr.cpp:3953-4018: causal
 * sliding window, each query sees the last `window_size` keys including its own.  The
 * reference ignores is_causal here (its mask is always causal | window); so does this call.
 * No [seq, seq] mask tensor is built: tiles before the window are skipped. */
int tyr_b200_sdpa_gqa_window(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t seq,
                             uint64_t head_dim, const void* q, const void* k, const void* v,
                             void* out, double dropout_p, uint8_t is_causal, uint8_t enable_gqa,
                             uint64_t window_size, void* stream);
/* tyr_b200_sdpa_gqa_mask <- lean_torch_sdpa_gqa_mask cc/src/tyr.cpp:4024-4095: padding mask
 * [batch, seq] over the keys (here as one byte per key, non-zero = valid), optionally combined
 * with the causal mask.  No [batch, 1, seq, seq] mask tensor is built. */
int tyr_b200_sdpa_gqa_mask(uint64_t batch, uint64_t n_head, uint64_t n_kv_head, uint64_t seq,
                           uint64_t head_dim, const void* q, const void* k, const void* v,
                           const uint8_t* key_mask, void* out, double dropout_p, uint8_t is_causal,
                           uint8_t enable_gqa, void* stream);

/* ------------------------------------------------------------------------
 * Decode: one query token per sequence over a (possibly ragged) KV cache,
 * split-KV partial attention followed by an LSE merge.  Replaces the
 * q_seq = 1, is_causal = false call in QwenAttention.forwardStep
 * (Tyr/Model/Qwen/Attention.lean:198-200 -> cc/src/tyr.cpp:4100-4133) without
 * the per-token repeat_interleave of the whole cache.
 *
 * Two cache layouts:
 *  dense : k/v point at [batch, n_kv_head, cap, head_dim] (Tyr's KVCache,
 *          Attention.lean:54-68); k_stride/v_stride = {batch, head, seq}.
 *  ragged: k_ptrs/v_ptrs are DEVICE arrays of `batch` device pointers, one
 *          per sequence, each to [n_kv_head, len_b, head_dim] with seq stride
 *          k_stride[2] and head stride kv_head_strides[b] (or, when that is
 *          NULL, len_b * k_stride[2] i.e. tightly packed).  k/v are ignored.
 * kv_lens: DEVICE int32[batch] of valid keys per sequence, or NULL for
 * max_kv_seq everywhere.  Every length must be in [1, max_kv_seq]; the kernels clamp
 * a length outside that range into it (a sequence of length <= 0 gets a zero output row and
 * LSE = -inf) and set TYR_ATTN_STATUS_OUT_OF_RANGE in the device status word.
 * Alignment: rows are read with 16-byte copies, so every cache base pointer (dense k/v and
 * each ragged k_ptrs[b] / v_ptrs[b]) must be 16-byte aligned and every stride, including each
 * kv_head_strides[b], a multiple of 8 elements.  The dense form is checked by the call; the
 * ragged arrays live on the device and are the caller's to keep aligned (the host mirror's
 * DecodePlan checks them when it builds the arrays).
 * ---------------------------------------------------------------------- */
typedef struct TyrAttnDecodeArgs {
  const void* q; /* [batch, n_head, head_dim] */
  void* o;       /* [batch, n_head, head_dim] */
  float* lse;    /* [batch, n_head] or NULL */
  const void* k;
  const void* v;
  const void* const* k_ptrs;
  const void* const* v_ptrs;
  const int32_t* kv_lens;
  const int64_t* kv_head_strides;
  int32_t batch, n_head, n_kv_head, max_kv_seq, head_dim;
  int64_t q_stride[2]; /* elements: batch, head */
  int64_t o_stride[2];
  int64_t k_stride[3]; /* elements: batch, head, seq (ragged: only [2] is read) */
  int64_t v_stride[3];
  float scale;        /* <= 0 => 1/sqrt(head_dim) */
  int32_t max_splits; /* 0 => 64; clamped to [1,64] */
  void* workspace;    /* device scratch, >= tyr_b200_attn_decode_workspace_bytes() */
  size_t workspace_bytes;
  int64_t total_kv_len; /* sum of the sequences' lengths when the host knows it, else 0.  Only steers the
                           chunk length of the launch (a small launch is cut into one wave of CTAs);
                           results do not depend on it */
} TyrAttnDecodeArgs;

size_t tyr_b200_attn_decode_workspace_bytes(int32_t batch, int32_t n_head, int32_t head_dim,
                                            int32_t max_kv_seq, int32_t max_splits);
int tyr_b200_attn_decode(const TyrAttnDecodeArgs* args, void* stream);

/* Decode for callers that must not allocate device memory.
 *
 * No counterpart in the reference; added for hosts of this library that cannot
 * call cudaMalloc at the point where they decode: a serving loop whose memory
 * pool already owns the whole device, a latency-critical token loop that cannot
 * afford the device-wide synchronisation an allocation implies, or a plugin
 * that is forbidden to touch the allocator of the process it is loaded into.
 * It is tyr_b200_attn_decode with the
 * split-KV scratch taken from a fixed array of
 * TYR_ATTN_DECODE_STATIC_SCRATCH_BYTES inside the library image instead of
 * args->workspace (args->workspace and args->workspace_bytes are ignored).
 * Every GPU that loads the library carries that array until the process exits.
 *
 *  - Sizes whose scratch need (tyr_b200_attn_decode_workspace_bytes) exceeds
 *    the array are refused with -TYR_ATTN_ERR_TOO_LARGE; lower max_splits or
 *    the batch, or use tyr_b200_attn_decode with your own workspace.
 *  - The first call on each device looks up the array's device address (with
 *    that device current).  Make that first call outside any stream capture.
 *  - The call itself runs no cudaMalloc, cudaFree or allocating library routine.
 *  - All calls on a device share the one array and it keeps the previous
 *    call's contents.  Nothing in it needs clearing (each call writes every
 *    slot it later reads), but two calls that overlap on the GPU, e.g. on two
 *    streams, race on it: order them on one stream or with events. */
#define TYR_ATTN_DECODE_STATIC_SCRATCH_BYTES (16u << 20)
int tyr_b200_attn_decode_static(const TyrAttnDecodeArgs* args, void* stream);

/* LSE merge of two partial attention results over disjoint key sets (the
 * reduction Tyr states in ringAttnReduce, Tyr/GPU/Kernels/RingAttn.lean:164-180):
 *   L = Lr + log(1 + exp(Lb - Lr));  O = Or*exp(Lr-L) + Ob*exp(Lb-L).
 * o_a/o_b/o_out: fp32 [rows, head_dim]; lse_*: fp32 [rows].  In place allowed. */
int tyr_b200_attn_merge(const float* o_a, const float* lse_a, const float* o_b, const float* lse_b,
                        float* o_out, float* lse_out, int64_t rows, int32_t head_dim, void* stream);

/* ------------------------------------------------------------------------
 * Fused prologue: per-head RMSNorm, rotary embedding, layout change and (for K/V)
 * in-place append to the KV cache, for one projected tensor in one pass.
 * Replaces the elementwise chain before every attention call of Tyr's models:
 * applyHeadNorm (Tyr/Model/Qwen/Attention.lean:73-98), rotary.applyRotaryEmb
 * (cc/src/tyr.cpp:3824-3861), transpose_for_attention (cc/src/tyr.cpp:2402-2414)
 * and, in decode, data.sliceScatter's clone of the whole cache
 * (cc/src/tyr.cpp:2261-2277; call site Tyr/Model/Qwen/Attention.lean:189-193).
 *
 *   y = x * rsqrt(mean(x^2) + eps) * norm_weight          (skipped when norm_weight == NULL)
 *   [y1, y2] -> [y1*cos - y2*sin, y1*sin + y2*cos]         (skipped when cos == NULL)
 *   out[b, h, pos_b + s, :] = bf16(y)      with pos_b = positions ? positions[b] : position0
 * cos/sin: fp32 [max_pos, head_dim/2] indexed by pos_b + s.  head_dim in {64,128,256}.
 * Second rotary form, Flux's (flux.applyRope, Tyr/Model/Flux/RoPE.lean:71-96): `pe` is fp32
 * [.., max_pos, head_dim/2, 2, 2], one 2x2 matrix per position and INTERLEAVED pair:
 *   [y_2i, y_2i+1] -> [pe[i][0][0]*y_2i + pe[i][0][1]*y_2i+1, pe[i][1][0]*y_2i + pe[i][1][1]*y_2i+1]
 * with batch element b reading pe + b * pe_batch_stride (0 when all share one table).  cos/sin and
 * pe exclude each other.
 * x, out, norm_weight, cos, sin, pe are 16-byte aligned; strides are multiples of 8 elements.
 * For Q pass position0 = rotary offset and an out tensor whose row 0 is that offset
 * (out pointer already shifted); for K/V pass the cache and the sequence lengths.
 * Limits: `cap` rows exist along the seq axis of out and `max_pos` rows in the rotary tables.
 * With positions == NULL a call that would pass either limit is refused (-TYR_ATTN_ERR_RANGE;
 * the reference guards its append with `cache.seq < cache.maxLen`,
 * Tyr/Model/Qwen/Attention.lean:189).  With device-side positions the kernel skips every row
 * whose pos_b + s falls outside a limit and sets TYR_ATTN_STATUS_OUT_OF_RANGE.
 * ---------------------------------------------------------------------- */
typedef struct TyrAttnPrologueArgs {
  const void* x;            /* [batch, seq, n_head, head_dim] bf16 */
  void* out;                /* [batch, n_head, cap, head_dim] bf16 */
  const float* norm_weight; /* [head_dim] fp32 or NULL */
  const float* cos;         /* [max_pos, head_dim/2] fp32 or NULL */
  const float* sin;
  const int32_t* positions; /* DEVICE int32[batch] or NULL */
  int32_t position0;
  int32_t batch, seq, n_head, head_dim;
  int64_t x_stride[3];      /* elements: batch, seq, head */
  int64_t out_stride[3];    /* elements: batch, head, seq */
  float eps;
  int32_t cap;              /* rows of out along seq (the cache capacity); > 0 */
  int32_t max_pos;          /* rows of cos / sin / pe; > 0 when a rotary table is given */
  const float* pe;          /* Flux-style [max_pos, head_dim/2, 2, 2] fp32 table or NULL */
  int64_t pe_batch_stride;  /* elements between the tables of two batch elements (0: shared) */
  int32_t out_at_row0;      /* != 0: pos_b + s selects the rotary row only and the result is written at
                               row s of out (a query of a decode step: rotated at the sequence's
                               position, stored as row 0 of a [batch, heads, seq, head_dim] tensor) */
} TyrAttnPrologueArgs;

int tyr_b200_attn_qk_prologue(const TyrAttnPrologueArgs* args, void* stream);

/* ------------------------------------------------------------------------
 * Backward of the prefill operator: dQ, dK, dV from dO, the forward inputs, the
 * forward output O and the per-row LSE the forward returned.
 * In the reference the gradient of the typed attention call comes from LibTorch
 * autograd (`output.backward(grad_output)`, cc/src/tyr.cpp:2111-2122) differentiating
 * the SDPA operator of cc/src/tyr.cpp:2563-2589 / 3910-3949; its own DSL statement of
 * the same arithmetic is Tyr/GPU/Kernels/MhaH100.lean:196-344 (a preparation kernel
 * d = rowsum(dO * O), then P = exp(scale*S - lse), dV = P^T dO, dP = dO V^T,
 * dS = scale * P * (dP - d), dQ = dS K, dK = dS^T Q, with P and dS rounded to bf16
 * before the matrix products).  This entry point follows that formulation:
 *
 *   delta[b,h,i] = sum_d dO[b,h,i,d] * O[b,h,i,d]
 *   P[i,j]  = exp(scale * q_i.k_j - lse[i])        (0 where the causal mask hides j)
 *   dV_j   += P[i,j] * dO_i     dP[i,j] = dO_i.v_j
 *   dS[i,j] = scale * P[i,j] * (dP[i,j] - delta[i])
 *   dQ_i   += dS[i,j] * k_j      dK_j   += dS[i,j] * q_i
 * dK and dV of a KV head sum over the n_head / n_kv_head query heads that share it.
 *
 * Tensors are bf16 [batch, heads, seq, head_dim] with the stride rules of the prefill
 * call (unit inner stride, 16-byte aligned rows); lse is fp32 contiguous
 * [batch, n_head, q_seq] as written by tyr_b200_attn_prefill.  head_dim in {64,128}.
 * `workspace` is caller-provided device memory of at least
 * tyr_b200_attn_backward_workspace_bytes() bytes (fp32 row statistics); nothing is
 * allocated by the call.  Three launches on `stream`: the row-statistics kernel, the
 * dK/dV kernel, the dQ kernel.  `window_size` and `key_mask` select the gradients of the
 * windowed (cc/src/tyr.cpp:3953-4018) and padding-masked (cc/src/tyr.cpp:4024-4095) calls.
 * ---------------------------------------------------------------------- */
typedef struct TyrAttnBackwardArgs {
  const void* q;            /* [batch, n_head,    q_seq,  head_dim] */
  const void* k;            /* [batch, n_kv_head, kv_seq, head_dim] */
  const void* v;            /* [batch, n_kv_head, kv_seq, head_dim] */
  const void* o;            /* forward output, [batch, n_head, q_seq, head_dim] */
  const void* d_o;          /* gradient of the loss w.r.t. o, same layout rules */
  const float* lse;         /* [batch, n_head, q_seq] fp32 from the forward */
  void* d_q;                /* out, [batch, n_head,    q_seq,  head_dim] */
  void* d_k;                /* out, [batch, n_kv_head, kv_seq, head_dim] */
  void* d_v;                /* out, [batch, n_kv_head, kv_seq, head_dim] */
  void* workspace;
  uint64_t workspace_bytes;
  int32_t batch, n_head, n_kv_head, q_seq, kv_seq, head_dim;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3], do_stride[3];
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];   /* elements: batch, head, seq */
  int32_t dtype;            /* TYR_ATTN_BF16 */
  int32_t is_causal;        /* key j hidden from query i when j > i, as in the forward */
  float scale;              /* <= 0: 1/sqrt(head_dim) */
  int32_t window_size;      /* as in TyrAttnPrefillArgs: 0 => none; w > 0 => causal sliding window */
  const uint8_t* key_mask;  /* as in TyrAttnPrefillArgs: NULL or DEVICE bytes [batch, kv_seq], 0 = padding key */
  int64_t key_mask_stride;
} TyrAttnBackwardArgs;

/* Zero extents as autograd of ATen's operator treats them: without queries (batch, n_head or q_seq
 * zero) dQ has no element and dK, dV are written as zeros; without keys dQ is written as zeros. */
uint64_t tyr_b200_attn_backward_workspace_bytes(int32_t batch, int32_t n_head, int32_t q_seq);
int tyr_b200_attn_backward(const TyrAttnBackwardArgs* args, void* stream);

/* ------------------------------------------------------------------------
 * Host-buffer call: same arithmetic as tyr_b200_attn_prefill, but every
 * pointer in `args` is HOST memory (pinned or pageable).  Copies Q/K/V to the
 * device, runs the kernel, copies O (and LSE) back and synchronises.  This is
 * the call a Tyr build makes when its tensors live on the CPU, which is the
 * only place the reference's CI ever runs attention
 * (.github/workflows/ci.yml:12-17).  Device staging buffers are cached per
 * device and grown on demand.  Tensors must be contiguous (strides that say
 * otherwise are refused with TYR_ATTN_ERR_SHAPE); no padding mask.
 * ---------------------------------------------------------------------- */
int tyr_b200_attn_prefill_host(const TyrAttnPrefillArgs* args, int32_t device);

/* Status word the kernels write (TYR_ATTN_STATUS_* bits; 0 = nothing to report).  Reads the
 * word with a device synchronise; `clear` != 0 resets it.  Negative: the read itself failed. */
int tyr_b200_attn_device_status(int32_t device, int32_t clear);
/* The same read turned into the library's error convention, for a launcher that wants one
 * call after its synchronise: 0, or -TYR_ATTN_ERR_DEVICE_WAIT when a bounded wait gave up,
 * or -TYR_ATTN_ERR_RANGE when only the out-of-range bit is set.  Always clears the word. */
int tyr_b200_attn_device_check(int32_t device);

/* Test hooks for the bounded-wait path; no counterpart in the reference, not for production use.
 * tyr_b200_attn_test_set_wait_limit: SM clock cycles any single in-kernel barrier wait may
 * take from now on (all later launches of this process; 0 restores the default of 4e9).
 * tyr_b200_attn_test_stalled_wait: launches a one-warp kernel whose only barrier is never
 * arrived at, so that its wait (the same routine the attention kernels use) runs out after
 * `limit_cycles`, sets TYR_ATTN_STATUS_WAIT_TIMEOUT and returns.  Nothing traps or faults. */
void tyr_b200_attn_test_set_wait_limit(int64_t cycles);
int tyr_b200_attn_test_stalled_wait(int64_t limit_cycles, void* stream);

const char* tyr_b200_attn_strerror(int code);
int tyr_b200_attn_abi_version(void);
/* number of kernel launches issued by this library since load (all threads) */
uint64_t tyr_b200_attn_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TYR_B200_ATTN_H_ */
