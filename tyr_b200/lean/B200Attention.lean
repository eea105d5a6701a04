/-
  Tyr/GPU/B200Attention.lean — Lean 4 bindings of the B200 attention operator.

  Not compiled in the image this library is developed in (no Lean toolchain);
  kept signature-identical to the launcher declarations Tyr generates
  (Tyr/GPU/Codegen/Attribute.lean:390-437) and to the typed calls in
  Tyr/Torch.lean:663-671, 1058-1082.
-/
import Tyr.Torch
import Tyr.GPU.Codegen.TileTypes

namespace Tyr.GPU.B200

open torch

/-- Launcher form: caller-allocated `out` and `lse`, explicit stream, IO error on
    rejection (shape, dtype, alignment, dropout).  C side: `lean_launch_tyrB200AttnFwd`. -/
@[extern "lean_launch_tyrB200AttnFwd"]
opaque tyrB200AttnFwd.launch
    (q k v out lse : @& Tensor) (isCausal : UInt8) (stream : Tyr.GPU.CudaStream) : IO Unit

/-- `tyrB200AttnFwd` with the caller's scratch for the key-split of a half-empty last round of work
    items (non-causal calls; `workspace`: uint8 CUDA tensor of `tyrB200AttnFwd.workspaceBytes` bytes,
    one with no elements for none).  C side: `lean_launch_tyrB200AttnFwdWs`. -/
@[extern "lean_launch_tyrB200AttnFwdWs"]
opaque tyrB200AttnFwdWs.launch
    (q k v out lse workspace : @& Tensor) (isCausal : UInt8) (stream : Tyr.GPU.CudaStream) : IO Unit

/-- Bytes of scratch with which the call above would split its last round (0: it would not). -/
@[extern "lean_tyrB200AttnFwdWorkspaceBytes"]
opaque tyrB200AttnFwd.workspaceBytes (q k v : @& Tensor) (isCausal : UInt8) : UInt64

/-- Single-token decode over the dense KV cache with the cache's `seq` counter as `kvLen`.
    C side: `lean_launch_tyrB200AttnDecode`. -/
@[extern "lean_launch_tyrB200AttnDecode"]
opaque tyrB200AttnDecode.launch
    (q kCache vCache out workspace : @& Tensor) (kvLen : UInt64) (stream : Tyr.GPU.CudaStream) : IO Unit

/-- Backward of `tyrB200AttnFwd`: `dQ dK dV` written in place from `dO`, the forward's inputs, its
    output and its LSE.  `workspace`: float32, `2 * b * hq * ceil(s/128)*128` elements.
    C side: `lean_launch_tyrB200AttnBwd`. -/
@[extern "lean_launch_tyrB200AttnBwd"]
opaque tyrB200AttnBwd.launch
    (q k v out lse dOut dQ dK dV workspace keyMask : @& Tensor) (isCausal : UInt8) (windowSize : UInt64)
    (stream : Tyr.GPU.CudaStream) : IO Unit

/-- Single-token decode with one cached length per sequence (`kvLens : int32 [batch]`, the
    per-sequence form of `KVCache.seq`).  C side: `lean_launch_tyrB200AttnDecodeRagged`. -/
@[extern "lean_launch_tyrB200AttnDecodeRagged"]
opaque tyrB200AttnDecodeRagged.launch
    (q kCache vCache kvLens out workspace : @& Tensor) (maxKvLen : UInt64)
    (stream : Tyr.GPU.CudaStream) : IO Unit

/-- Fused head norm + rotary + layout change + in-place cache append for one projected tensor
    (`x : [batch, seq, heads, headDim]` into `out : [batch, heads, cap, headDim]` at rows
    `positions[b] + s`; with `outAtRow0 = 1` the position selects the rotary row only and the rows are
    written from row 0, the query of a decode step).  Tensors with no elements skip a step.
    C side: `lean_launch_tyrB200QkPrologue`. -/
@[extern "lean_launch_tyrB200QkPrologue"]
opaque tyrB200QkPrologue.launch
    (x out normWeight cos sin positions : @& Tensor) (position0 : UInt64) (eps : Float)
    (outAtRow0 : UInt8) (stream : Tyr.GPU.CudaStream) : IO Unit

/-- LSE merge of two partial attention results over disjoint key sets (`ringAttnReduce`).
    C side: `lean_launch_tyrB200AttnMerge`. -/
@[extern "lean_launch_tyrB200AttnMerge"]
opaque tyrB200AttnMerge.launch
    (oA lseA oB lseB oOut lseOut : @& Tensor) (stream : Tyr.GPU.CudaStream) : IO Unit

/-- Typed wrapper: output and per-row LSE of causal / non-causal GQA attention. -/
def attentionFwd {b hq hkv s d : UInt64}
    (q : T #[b, hq, s, d]) (k v : T #[b, hkv, s, d]) (isCausal : Bool := true)
    : IO (T #[b, hq, s, d] × T #[b, hq, s]) := do
  let out : T #[b, hq, s, d] := torch.zeros_like q
  let lse : T #[b, hq, s] := torch.zeros #[b, hq, s] false (torch.device q)
  let lse32 := torch.toFloat' lse
  let stream ← torch.cuda_current_stream
  tyrB200AttnFwd.launch q k v out lse32 (if isCausal then 1 else 0) stream
  pure (out, lse32)

/-- Typed wrapper of the backward: gradients with the shapes of `q`, `k`, `v`. -/
def attentionBwd {b hq hkv s d : UInt64}
    (q : T #[b, hq, s, d]) (k v : T #[b, hkv, s, d]) (out : T #[b, hq, s, d]) (lse : T #[b, hq, s])
    (dOut : T #[b, hq, s, d]) (isCausal : Bool := true)
    : IO (T #[b, hq, s, d] × T #[b, hkv, s, d] × T #[b, hkv, s, d]) := do
  let dQ : T #[b, hq, s, d] := torch.zeros_like q
  let dK : T #[b, hkv, s, d] := torch.zeros_like k
  let dV : T #[b, hkv, s, d] := torch.zeros_like v
  let rows := ((s + 127) / 128) * 128
  let ws : T #[2, b, hq, rows] := torch.toFloat' (torch.zeros #[2, b, hq, rows] false (torch.device q))
  let stream ← torch.cuda_current_stream
  let noMask : T #[0] := torch.zeros #[0] false (torch.device q)
  tyrB200AttnBwd.launch q k v out lse dOut dQ dK dV ws noMask (if isCausal then 1 else 0) 0 stream
  pure (dQ, dK, dV)

end Tyr.GPU.B200
