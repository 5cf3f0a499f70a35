// Checker only: thin extern "C" launchers around the REFERENCE's own device
// kernels, included from the reference checkout where it lies (the include path
// is given on the nvcc command line by oracle/build_ref.py; no reference source is
// copied here).  Built into oracle/_ref/libref_kernels.so and used by the GPU tests
// to compare this repository's kernels with the reference's on the same inputs.
// Launch shapes follow the reference launchers (csrc/kernel/attn_int8_fwd.cu:22-99,
// csrc/kernel/attn_decode.cu:79-97, csrc/kernel/quant_rowwise.cu:84-121).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "attn_decode.cuh"
#include "attn_int8_fwd.cuh"
#include "attn_varlen_fwd.cuh"
#include "attn_w8a8_fwd.cuh"
#include "quant_rowwise.cuh"

namespace {

template <int D, typename VT>
int fwd_static(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const void* v, void* out,
               float* lse, int causal, int M, int N, int64_t BH, int Hq, int g, int window, cudaStream_t s) {
  dim3 grid((M + fni8::BLOCK_M - 1) / fni8::BLOCK_M, (unsigned)BH);
  if (causal)
    fni8::attn_int8_fwd_kernel<D, true, VT><<<grid, fni8::THREADS, 0, s>>>(
        q, qs, k, ks, (const VT*)v, (VT*)out, lse, M, N, Hq, g, window);
  else
    fni8::attn_int8_fwd_kernel<D, false, VT><<<grid, fni8::THREADS, 0, s>>>(
        q, qs, k, ks, (const VT*)v, (VT*)out, lse, M, N, Hq, g, window);
  return (int)cudaGetLastError();
}

template <int D, typename VT>
int fwd_dyn(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const void* v, void* out,
            float* lse, int causal, int M, int N, int64_t BH, int Hq, int g, int window, cudaStream_t s) {
  dim3 grid((M + fni8::BLOCK_M - 1) / fni8::BLOCK_M, (unsigned)BH);
  const int smem = fni8::fwd_dyn_smem_bytes<D, VT>();
  if (causal) {
    cudaFuncSetAttribute(fni8::attn_int8_fwd_dyn_kernel<D, true, VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    fni8::attn_int8_fwd_dyn_kernel<D, true, VT><<<grid, fni8::THREADS, smem, s>>>(
        q, qs, k, ks, (const VT*)v, (VT*)out, lse, M, N, Hq, g, window);
  } else {
    cudaFuncSetAttribute(fni8::attn_int8_fwd_dyn_kernel<D, false, VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    fni8::attn_int8_fwd_dyn_kernel<D, false, VT><<<grid, fni8::THREADS, smem, s>>>(
        q, qs, k, ks, (const VT*)v, (VT*)out, lse, M, N, Hq, g, window);
  }
  return (int)cudaGetLastError();
}

template <typename VT>
int fwd_d(int D, const int8_t* q, const float* qs, const int8_t* k, const float* ks, const void* v, void* out,
          float* lse, int causal, int M, int N, int64_t BH, int Hq, int g, int window, cudaStream_t s) {
  switch (D) {
    case 32: return fwd_static<32, VT>(q, qs, k, ks, v, out, lse, causal, M, N, BH, Hq, g, window, s);
    case 64: return fwd_static<64, VT>(q, qs, k, ks, v, out, lse, causal, M, N, BH, Hq, g, window, s);
    case 72: return fwd_static<72, VT>(q, qs, k, ks, v, out, lse, causal, M, N, BH, Hq, g, window, s);
    case 80: return fwd_static<80, VT>(q, qs, k, ks, v, out, lse, causal, M, N, BH, Hq, g, window, s);
    case 128: return fwd_static<128, VT>(q, qs, k, ks, v, out, lse, causal, M, N, BH, Hq, g, window, s);
    case 256: return fwd_dyn<256, VT>(q, qs, k, ks, v, out, lse, causal, M, N, BH, Hq, g, window, s);
  }
  return -1;
}

template <int D>
int decode_d(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const __half* v, __half* out,
             float* o_part, float* m_part, float* l_part, int N, int n_splits, int64_t BHq, int Hq, int g,
             cudaStream_t s) {
  fni8::decode_split_kernel<D><<<dim3(n_splits, (unsigned)BHq), fni8::DEC_WARP, 0, s>>>(
      q, qs, k, ks, v, o_part, m_part, l_part, N, n_splits, Hq, g);
  fni8::decode_combine_kernel<D><<<(unsigned)BHq, fni8::DEC_WARP, 0, s>>>(o_part, m_part, l_part, out, n_splits);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" int ref_quantize_i8_rowwise(const void* x, int dtype, int M, int K, int8_t* q, float* scale, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (M == 0 || K == 0) return 0;
  if (dtype == 0)
    fni8::quantize_i8_rowwise_kernel<__half><<<M, fni8::QUANT_ROW_THREADS, 0, s>>>((const __half*)x, q, scale, M, K);
  else if (dtype == 1)
    fni8::quantize_i8_rowwise_kernel<__nv_bfloat16><<<M, fni8::QUANT_ROW_THREADS, 0, s>>>((const __nv_bfloat16*)x, q, scale, M, K);
  else
    fni8::quantize_i8_rowwise_kernel<float><<<M, fni8::QUANT_ROW_THREADS, 0, s>>>((const float*)x, q, scale, M, K);
  return (int)cudaGetLastError();
}

extern "C" int ref_attn_int8_fwd(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const void* v,
                                 int v_dtype, void* out, float* lse, int causal, int window_left, int B, int Hq,
                                 int Hkv, int M, int N, int D, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const int g = Hq / Hkv;
  if (v_dtype == 0)
    return fwd_d<__half>(D, q, qs, k, ks, v, out, lse, causal, M, N, (int64_t)B * Hq, Hq, g, window_left, s);
  return fwd_d<__nv_bfloat16>(D, q, qs, k, ks, v, out, lse, causal, M, N, (int64_t)B * Hq, Hq, g, window_left, s);
}

extern "C" int ref_attn_int8_decode(const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                                    const void* v, void* out, float* o_part, float* m_part, float* l_part, int B,
                                    int Hq, int Hkv, int N, int D, int n_splits, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const int g = Hq / Hkv;
  const int64_t BHq = (int64_t)B * Hq;
  switch (D) {
    case 32: return decode_d<32>(q, qs, k, ks, (const __half*)v, (__half*)out, o_part, m_part, l_part, N, n_splits, BHq, Hq, g, s);
    case 64: return decode_d<64>(q, qs, k, ks, (const __half*)v, (__half*)out, o_part, m_part, l_part, N, n_splits, BHq, Hq, g, s);
    case 128: return decode_d<128>(q, qs, k, ks, (const __half*)v, (__half*)out, o_part, m_part, l_part, N, n_splits, BHq, Hq, g, s);
    case 256: return decode_d<256>(q, qs, k, ks, (const __half*)v, (__half*)out, o_part, m_part, l_part, N, n_splits, BHq, Hq, g, s);
  }
  return -1;
}

// reference csrc/kernel/attn_varlen_fwd.cu:18-41 (grid and launch of the packed variable-length kernel)
template <int D>
static int varlen_d(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const __half* v, __half* out,
                    const int* cu_q, const int* cu_k, int batch, int max_seqlen_q, int h_q, int h_kv, int causal,
                    cudaStream_t s) {
  const dim3 grid((max_seqlen_q + fni8::BLOCK_M - 1) / fni8::BLOCK_M, (unsigned)batch, (unsigned)h_q);
  if (causal)
    fni8::attn_int8_varlen_fwd_kernel<D, true><<<grid, fni8::THREADS, 0, s>>>(q, qs, k, ks, v, out, cu_q, cu_k, h_q, h_kv, h_q / h_kv);
  else
    fni8::attn_int8_varlen_fwd_kernel<D, false><<<grid, fni8::THREADS, 0, s>>>(q, qs, k, ks, v, out, cu_q, cu_k, h_q, h_kv, h_q / h_kv);
  return (int)cudaGetLastError();
}

extern "C" int ref_attn_int8_varlen(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const void* v,
                                    void* out, const int* cu_q, const int* cu_k, int batch, int max_seqlen_q, int Hq,
                                    int Hkv, int D, int causal, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (D) {
    case 32: return varlen_d<32>(q, qs, k, ks, (const __half*)v, (__half*)out, cu_q, cu_k, batch, max_seqlen_q, Hq, Hkv, causal, s);
    case 64: return varlen_d<64>(q, qs, k, ks, (const __half*)v, (__half*)out, cu_q, cu_k, batch, max_seqlen_q, Hq, Hkv, causal, s);
    case 128: return varlen_d<128>(q, qs, k, ks, (const __half*)v, (__half*)out, cu_q, cu_k, batch, max_seqlen_q, Hq, Hkv, causal, s);
  }
  return -1;
}

// reference csrc/kernel/attn_decode.cu: int8-V cache variant (decode_split_i8v_kernel + the same combine)
template <int D>
static int decode_kv8_d(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const int8_t* v,
                        const float* vs, __half* out, float* o_part, float* m_part, float* l_part, int N, int n_splits,
                        int64_t BHq, int Hq, int g, cudaStream_t s) {
  fni8::decode_split_i8v_kernel<D><<<dim3(n_splits, (unsigned)BHq), fni8::DEC_WARP, 0, s>>>(
      q, qs, k, ks, v, vs, o_part, m_part, l_part, N, n_splits, Hq, g);
  fni8::decode_combine_kernel<D><<<(unsigned)BHq, fni8::DEC_WARP, 0, s>>>(o_part, m_part, l_part, out, n_splits);
  return (int)cudaGetLastError();
}

extern "C" int ref_attn_int8_decode_kv8(const int8_t* q, const float* qs, const int8_t* k, const float* ks,
                                        const int8_t* v, const float* vs, void* out, float* o_part, float* m_part,
                                        float* l_part, int B, int Hq, int Hkv, int N, int D, int n_splits, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const int g = Hq / Hkv;
  const int64_t BHq = (int64_t)B * Hq;
  switch (D) {
    case 32: return decode_kv8_d<32>(q, qs, k, ks, v, vs, (__half*)out, o_part, m_part, l_part, N, n_splits, BHq, Hq, g, s);
    case 64: return decode_kv8_d<64>(q, qs, k, ks, v, vs, (__half*)out, o_part, m_part, l_part, N, n_splits, BHq, Hq, g, s);
    case 128: return decode_kv8_d<128>(q, qs, k, ks, v, vs, (__half*)out, o_part, m_part, l_part, N, n_splits, BHq, Hq, g, s);
    case 256: return decode_kv8_d<256>(q, qs, k, ks, v, vs, (__half*)out, o_part, m_part, l_part, N, n_splits, BHq, Hq, g, s);
  }
  return -1;
}

// reference csrc/kernel/attn_w8a8_fwd.cu:16-39 (static shared memory variant: D = 32, 64, 128)
template <int D, bool PW>
static int w8a8_d(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const int8_t* v, const float* vs,
                  __half* out, int causal, int M, int N, int64_t BH, int Hq, int g, int diag, cudaStream_t s) {
  const dim3 grid((M + fni8::BLOCK_M - 1) / fni8::BLOCK_M, (unsigned)BH);
  if (causal)
    fni8::attn_w8a8_fwd_kernel<D, true, PW><<<grid, fni8::THREADS, 0, s>>>(q, qs, k, ks, v, vs, out, M, N, Hq, g, diag);
  else
    fni8::attn_w8a8_fwd_kernel<D, false, PW><<<grid, fni8::THREADS, 0, s>>>(q, qs, k, ks, v, vs, out, M, N, Hq, g, diag);
  return (int)cudaGetLastError();
}

extern "C" int ref_attn_w8a8_fwd(const int8_t* q, const float* qs, const int8_t* k, const float* ks, const int8_t* v,
                                 const float* vs, void* out, int causal, int causal_diag, int per_warp, int B, int Hq,
                                 int Hkv, int M, int N, int D, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const int g = Hq / Hkv;
  const int64_t BH = (int64_t)B * Hq;
  __half* o = (__half*)out;
  if (per_warp) {
    switch (D) {
      case 32: return w8a8_d<32, true>(q, qs, k, ks, v, vs, o, causal, M, N, BH, Hq, g, causal_diag, s);
      case 64: return w8a8_d<64, true>(q, qs, k, ks, v, vs, o, causal, M, N, BH, Hq, g, causal_diag, s);
      case 128: return w8a8_d<128, true>(q, qs, k, ks, v, vs, o, causal, M, N, BH, Hq, g, causal_diag, s);
    }
  } else {
    switch (D) {
      case 32: return w8a8_d<32, false>(q, qs, k, ks, v, vs, o, causal, M, N, BH, Hq, g, causal_diag, s);
      case 64: return w8a8_d<64, false>(q, qs, k, ks, v, vs, o, causal, M, N, BH, Hq, g, causal_diag, s);
      case 128: return w8a8_d<128, false>(q, qs, k, ks, v, vs, o, causal, M, N, BH, Hq, g, causal_diag, s);
    }
  }
  return -1;
}
