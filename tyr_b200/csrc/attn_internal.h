// Internal launch interface shared by the .cu files of the attention library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tyr_b200_attn.h"

namespace tyr {

// Per-device state owned by api.cu.
struct DeviceState {
  int* status = nullptr;  // device word the kernels' bounded waits OR into
  bool ready = false;
};
DeviceState* device_state(int device);  // lazily created; nullptr on failure
void count_launch(int n = 1);
int sm_count();  // SMs of the current device (148 when it cannot be asked)
// Cycles a single in-kernel barrier wait may take before its CTA gives up (api.cu; the default
// unless a test shortened it).
long long wait_limit_cycles();
// ptx_sm100.cuh users only: a one-warp kernel whose only barrier is never arrived at, so that its
// bounded wait runs out after `limit_cycles` (stalled_wait.cu).
int launch_stalled_wait(long long limit_cycles, int* status, cudaStream_t st);

// prefill_sm100.cu — tcgen05/TMA kernel, bf16, head_dim in {64,128}.
int launch_prefill_sm100(const TyrAttnPrefillArgs& a, float scale, int* status, cudaStream_t st);
long long prefill_split_workspace_bytes(const TyrAttnPrefillArgs& a);  // 0: the launch would not split
// 128-byte-swizzled 64 x 128 box map over a bf16 [batch, heads, seq, d] tensor with element strides
// {batch, head, seq}; encoded maps are cached per thread (prefill_sm100.cu).
int make_tile_map(CUtensorMap* m, const void* ptr, int batch, int heads, int seq, int d, const int64_t* stride);
// backward_sm100.cu — tcgen05/TMA kernels, bf16, head_dim in {64,128}.
size_t backward_workspace_bytes(int batch, int n_head, int q_seq);
int launch_backward_sm100(const TyrAttnBackwardArgs& a, float scale, int* status, cudaStream_t st);
// check_fp32.cu — fp32-FMA kernel, bf16 or fp32 I/O, any head_dim <= 256.
int launch_prefill_check(const TyrAttnPrefillArgs& a, float scale, cudaStream_t st);
// decode_splitkv.cu
size_t decode_workspace_bytes(int batch, int n_head, int head_dim, int max_kv_seq, int max_splits);
int decode_num_splits(int max_kv_seq, int max_splits, int* chunk_len);
int launch_decode(const TyrAttnDecodeArgs& a, float scale, cudaStream_t st);
int launch_merge2(const float* o_a, const float* lse_a, const float* o_b, const float* lse_b,
                  float* o_out, float* lse_out, int64_t rows, int head_dim, cudaStream_t st);

// qk_prologue.cu
int launch_qk_prologue(const TyrAttnPrologueArgs& a, int* status, cudaStream_t st);

}  // namespace tyr
