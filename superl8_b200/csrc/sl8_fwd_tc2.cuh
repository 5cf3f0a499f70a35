// Arguments and entry of the one-block-per-SM forward kernel (fwd_tc2.cu): two 128-row query
// tiles per block, 128-key tiles, all 512 tensor-memory columns.
#pragma once
#include "sl8_common.cuh"

namespace sl8 {

struct Tc2Args {
  const void* q;            // int8 or 16-bit [B, Hq, M, D]
  const void* k;            // int8 or 16-bit [B, Hkv, N, D]
  const void* v;            // 16-bit [B, Hkv, N, D]
  void* out;                // [B, Hq, M, D], V's dtype
  const float* q_scale;     // int8 mode: [B, Hq, M] folded
  const float* k_scale;     // int8 mode: [B, Hkv, N]
  float* lse;               // nullable [B, Hq, M]
  const int32_t* seqlens_q; // nullable int32 [B]
  const int32_t* seqlens_k;
  int* status;
  const int32_t* gate_flag; // nullable: run only if (*gate_flag != 0) == (gate_want != 0)
  int gate_want;
  int B, Hq, Hkv, M, N, D;
  int causal;
  float scale_log2;         // 16-bit mode: softmax_scale * log2(e)
  int qk8;                  // 1: int8 Q/K with scales; 0: 16-bit Q/K of V's dtype
  int v_bf16;               // V / out (and 16-bit Q/K) are bf16 instead of fp16
};

// True when fwd_tc2 serves the shape (D = 128, no window, dense layout).
bool sl8_fwd_tc2_supported(int D, int window_left, bool packed);
// Launches the kernel (arguments validated by the caller).
int sl8_fwd_tc2(const Tc2Args& a, cudaStream_t stream);

}  // namespace sl8
