// Per-row symmetric int8 quantiser and the Q / K prologues that wrap it.
//
// Arithmetic contract (bit-exact with the reference's CUDA path,
// csrc/include/quant_rowwise.cuh:32-92): scale = amax * float(1/127) (a
// reciprocal MULTIPLY, not a division), an all-zero row gets scale 1, element
// = clamp(rint(x / scale), +-127) with an IEEE-rounded division.
//
// Mapping to the machine: the operation moves 3 bytes per element and is bound
// by HBM bandwidth, so a row is owned by a sub-group of lanes that each load 16
// bytes (8 two-byte elements) once, keep them in registers for both the amax and
// the rounding pass, and store 8 bytes of codes.  One 256-thread block covers
// 8 * (32 / lanes-per-row) rows per step and walks the rows grid-stride.
#include "sl8_common.cuh"

#include <cmath>

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace sl8 {
namespace {

constexpr int kQuantThreads = 256;
constexpr float kQMax = 127.0f;
constexpr float kQMaxInv = 1.0f / 127.0f;

// kGateOnly: the outlier statistic of the query mode alone -- rows are read, nothing is written
// but the flag (the reference runs its gate before it quantises, superl8/ops.py:118-130)
// kRotate: [subtract the mean if one is given, round] -> normalised Hadamard rotation of the row in
// fp32 -> round to the storage dtype -> [store the rotated row] -> [quantise, scale * fold]: the
// rotate=True prologue of the reference (superl8/quant/core.py:186-194, superl8/quant/rotation.py:41-51)
// in the registers of the row quantiser, no extra trip through HBM
enum QuantMode { kPlain = 0, kQueryFoldGate = 1, kKeySmooth = 2, kGateOnly = 3, kRotate = 4 };

struct QuantArgs {
  const void* x;
  int8_t* q;
  float* scale;         // plain: scale; query: folded scale; key: scale
  float* plain_scale;   // query mode only (nullable)
  const float* mean;    // key mode: [BH, K]
  void* smoothed;       // key mode (nullable): k - mean in x's dtype
  void* rotated;        // rotate mode (nullable): the rotated row in x's dtype
  int32_t* flag;        // query mode (nullable): OR-ed with 1 if any row is outlier dominated
  int64_t rows;
  int64_t rows_per_head;
  // key mode on a token-major packed tensor [tokens, heads, K]: row = token * heads + head and
  // the mean row is sequence(token) * heads + head, sequence bounds in cu_seqlens[n_seq + 1]
  const int32_t* cu_seqlens;
  int n_seq;
  int heads;
  int K;
  float fold;
  float ratio_threshold;
  float rot_norm;       // rotate mode: 1 / sqrt(K)
};

// Row of the mean table for a row of the key tensor (see QuantArgs).
__device__ __forceinline__ int64_t mean_row(const QuantArgs& a, int64_t row) {
  if (a.cu_seqlens == nullptr) return row / a.rows_per_head;
  const int token = (int)(row / a.heads), head = (int)(row % a.heads);
  int lo = 0, hi = a.n_seq;   // largest s with cu_seqlens[s] <= token
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(a.cu_seqlens + mid) <= token) lo = mid; else hi = mid;
  }
  return (int64_t)lo * a.heads + head;
}

__device__ __forceinline__ float quant_one(float x, float s) {
  float v = rintf(__fdiv_rn(x, s));
  return fminf(fmaxf(v, -kQMax), kQMax);
}

template <typename T> struct Vec8;  // 8 two-byte elements in a uint4
template <> struct Vec8<__half> {
  __device__ static void unpack(const uint4& u, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  // round to nearest even, two elements per conversion instruction
  __device__ static uint4 pack(const float (&f)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return u;
  }
};
template <> struct Vec8<__nv_bfloat16> {
  __device__ static void unpack(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 pack(const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
  }
};

// Packed fp16 evaluation of the outlier statistic (see the call site for the argument).
template <typename T> __device__ __forceinline__ bool half_gate_ok(float, float) { return false; }
template <> __device__ __forceinline__ bool half_gate_ok<__half>(float t0, float amax) {
  return t0 >= 0.0078125f && amax <= 65504.0f;   // 2^-7 <= max / thr, finite row
}
template <int NV>
__device__ __forceinline__ int half_gate_count(const uint4 (&raw)[NV], const bool (&has)[NV], float t0, float amax,
                                               float thr) {
  __half h = __float2half_rd(t0);
  if (!(__fdiv_rn(amax, __half2float(h) + 1e-10f) > thr)) h = __ushort_as_half((unsigned short)(__half_as_ushort(h) - 1));
  const __half2 hstar = __half2half2(h);
  __half2 cnt2 = __float2half2_rn(0.f);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if (!has[v]) continue;
    const __half2* x2 = reinterpret_cast<const __half2*>(&raw[v]);
#pragma unroll
    for (int i = 0; i < 4; ++i) cnt2 = __hadd2(cnt2, __hle2(__habs2(x2[i]), hstar));
  }
  return (int)(__low2float(cnt2) + __high2float(cnt2));
}

// Unnormalised Walsh-Hadamard transform (Sylvester order: y[k] = sum_j x[j] (-1)^popcount(j & k)) of a
// row of 8 * LPR * NV elements held by LPR lanes: lane sl keeps element i + 8 * (sl + LPR * v) in
// f[v][i], so the index bits are i (in the vector), sl (across lanes: one shuffle per value and
// stage) and v (across the lane's vectors).  One butterfly stage per index bit, any order.
template <int LPR, int NV>
__device__ __forceinline__ void wht_row(float (&f)[NV][8], int sl) {
  static_assert((NV & (NV - 1)) == 0 && (LPR & (LPR - 1)) == 0, "power-of-two row");
#pragma unroll
  for (int h = 1; h < 8; h <<= 1)
#pragma unroll
    for (int v = 0; v < NV; ++v)
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if ((i & h) == 0) {
          const float a = f[v][i], b = f[v][i + h];
          f[v][i] = a + b;
          f[v][i + h] = a - b;
        }
#pragma unroll
  for (int h = 1; h < NV; h <<= 1)
#pragma unroll
    for (int v = 0; v < NV; ++v)
      if ((v & h) == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float a = f[v][i], b = f[v + h][i];
          f[v][i] = a + b;
          f[v + h][i] = a - b;
        }
      }
#pragma unroll
  for (int h = 1; h < LPR; h <<= 1) {
    const bool upper = (sl & h) != 0;
#pragma unroll
    for (int v = 0; v < NV; ++v)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, f[v][i], h);
        f[v][i] = upper ? other - f[v][i] : f[v][i] + other;
      }
  }
}

// LPR lanes own one row; each lane holds NV vectors of 8 elements.  The block walks the row groups
// base0, base0 + stride, ... below row_end; returns whether one of this thread's rows tripped the gate.
// mean_local (key mode, nullable): the mean row of every row of the walk, in shared memory (the fused
// K prologue); otherwise the mean table a.mean is read through the read-only path.
template <typename T, int LPR, int NV, int MODE>
__device__ __forceinline__ int quant_rows_vec_body(const QuantArgs& a, int64_t base0, int64_t stride, int64_t row_end,
                                                   const float* mean_local) {
  constexpr int ROWS_PER_WARP = 32 / LPR;
  constexpr unsigned FULL = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR;       // which row of the warp's group
  const int sl = lane % LPR;        // lane within the row
  const int warp = threadIdx.x >> 5;
  const int kvec = a.K >> 3;
  const int rank_need = ((a.K - 1) >> 1) + 1;  // elements <= lower median, counted from the bottom
  int any_outlier = 0;

  for (int64_t base = base0; base < row_end; base += stride) {
    const int64_t row = base + (int64_t)warp * ROWS_PER_WARP + sub;
    const bool live = row < row_end;
    const T* xr = reinterpret_cast<const T*>(a.x) + row * a.K;
    float f[NV][8];
    uint4 raw[NV];
    bool has[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int vi = sl + v * LPR;
      has[v] = live && vi < kvec;
      raw[v] = make_uint4(0, 0, 0, 0);
      if (has[v]) raw[v] = __ldg(reinterpret_cast<const uint4*>(xr) + vi);
      Vec8<T>::unpack(raw[v], f[v]);
    }
    if (MODE == kKeySmooth || (MODE == kRotate && a.mean != nullptr)) {
      const int64_t bh = (live && mean_local == nullptr) ? mean_row(a, row) : 0;
      const float* mr = mean_local != nullptr ? mean_local : a.mean + bh * a.K;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        if (!has[v]) continue;
        const int c0 = (sl + v * LPR) * 8;
        float4 m0, m1;
        if (mean_local != nullptr) {   // written by this kernel: plain loads
          m0 = *reinterpret_cast<const float4*>(mr + c0);
          m1 = *reinterpret_cast<const float4*>(mr + c0 + 4);
        } else {
          m0 = __ldg(reinterpret_cast<const float4*>(mr + c0));
          m1 = __ldg(reinterpret_cast<const float4*>(mr + c0 + 4));
        }
        const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) f[v][i] -= mm[i];
        const uint4 t = Vec8<T>::pack(f[v]);   // rounded to the storage dtype, as torch.sub(out=)
        Vec8<T>::unpack(t, f[v]);
        if (a.smoothed != nullptr) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.smoothed) + row * a.K + c0) = t;
      }
    }
    if (MODE == kRotate) {
      // every lane of the warp takes part in the shuffles (rows past the end carry zeros)
      if constexpr (MODE == kRotate && (NV & (NV - 1)) == 0) wht_row<LPR, NV>(f, sl);
#pragma unroll
      for (int v = 0; v < NV; ++v) {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[v][i] *= a.rot_norm;
        const uint4 t = Vec8<T>::pack(f[v]);     // the reference casts the rotated row back to the input dtype
        Vec8<T>::unpack(t, f[v]);
        if (has[v] && a.rotated != nullptr)
          *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.rotated) + row * a.K + (sl + v * LPR) * 8) = t;
      }
      if (a.q == nullptr) continue;   // rotation alone
    }
    float amax = 0.0f;
#pragma unroll
    for (int v = 0; v < NV; ++v)
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[v][i]));
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, off));

    float s = amax * kQMaxInv;
    s = (s == 0.0f) ? 1.0f : s;

    if ((MODE == kQueryFoldGate || MODE == kGateOnly) && a.flag != nullptr) {
      // max / (median + 1e-10) > thr  <=>  at least rank_need elements e satisfy
      // max / (|e| + 1e-10) > thr, because the quotient is monotone in |e|.  Elements whose
      // y = |e| + 1e-10 is clearly below / above max / thr are decided by a comparison; only
      // the few inside a 1e-6 relative band take the exactly rounded division.
      const float t0 = __fdiv_rn(amax, a.ratio_threshold);
      int cnt = 0;
      if (half_gate_ok<T>(t0, amax)) {
        // fp16 input: every element is an fp16 number, so the condition is |e| <= h*, with h* the
        // largest fp16 value that still satisfies it.  h* is RD_fp16(max / thr) or its fp16
        // predecessor: fp16 neighbours are 2^13 fp32 ulps apart, so every fp16 value below
        // RD_fp16(t0) satisfies the condition, every one above t0 fails it, and only RD_fp16(t0)
        // itself needs the exactly rounded quotient.  (|e| + 1e-10 == |e| in fp32 for
        // |e| >= 2^-9, and smaller elements satisfy the condition either way because
        // t0 >= 2^-7.)  Two divisions per row, then three packed instructions per element pair.
        cnt = half_gate_count<NV>(raw, has, t0, amax, a.ratio_threshold);
      } else {
      const float t_lo = t0 * 0.999999f, t_hi = t0 * 1.000001f;
      bool ambiguous = false;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float y = fabsf(f[v][i]) + 1e-10f;
          cnt += (has[v] && y < t_lo) ? 1 : 0;
          ambiguous |= has[v] && (y >= t_lo) && (y <= t_hi);
        }
      }
      if (ambiguous) {  // rare: redo this lane's count with the exact quotient
        cnt = 0;
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
          for (int i = 0; i < 8; ++i)
            cnt += (has[v] && __fdiv_rn(amax, fabsf(f[v][i]) + 1e-10f) > a.ratio_threshold) ? 1 : 0;
      }
      }
#pragma unroll
      for (int off = LPR / 2; off > 0; off >>= 1) cnt += __shfl_xor_sync(FULL, cnt, off);
      if (live && cnt >= rank_need) any_outlier = 1;
    }
    if (MODE == kGateOnly) continue;

    // Codes.  Fast path: t = x * (1/s) + 1.5 * 2^23 rounds x / s to the nearest integer in one
    // fused operation (its low byte is the code).  1/s carries a 2^-24 relative error, so the
    // result can differ from rint(fl(x / s)) only when x / s lies within ~1.5e-5 of a
    // half-integer; those elements (|residual| >= 0.49996, also NaN / inf rows) are redone
    // with the IEEE division, rint and clamp of the reference.
    const float rcp = __frcp_rn(s);
    int8_t* qr = a.q + row * a.K;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (!has[v]) continue;
      uint32_t tb[8];
      bool redo = false;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float t = fmaf(f[v][i], rcp, 12582912.0f);
        const float e = fmaf(f[v][i], rcp, -(t - 12582912.0f));
        tb[i] = __float_as_uint(t);
        redo |= !(fabsf(e) < 0.49996f);
      }
      if (redo) {  // rare: some element sits next to a rounding boundary (or is NaN / inf)
#pragma unroll
        for (int i = 0; i < 8; ++i) tb[i] = (uint32_t)(int)quant_one(f[v][i], s);
      }
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t lo = __byte_perm(tb[4 * h], tb[4 * h + 1], 0x0040);
        const uint32_t hi = __byte_perm(tb[4 * h + 2], tb[4 * h + 3], 0x0040);
        w[h] = __byte_perm(lo, hi, 0x5410);
      }
      *reinterpret_cast<uint2*>(qr + (sl + v * LPR) * 8) = make_uint2(w[0], w[1]);
    }
    if (live && sl == 0) {
      if (MODE == kQueryFoldGate) {
        a.scale[row] = s * a.fold;
        if (a.plain_scale != nullptr) a.plain_scale[row] = s;
      } else if (MODE == kRotate) {
        a.scale[row] = s * a.fold;
      } else {
        a.scale[row] = s;
      }
    }
  }
  return any_outlier;
}

template <typename T, int LPR, int NV, int MODE>
__global__ void __launch_bounds__(kQuantThreads, 4) quant_rows_vec_kernel(QuantArgs a) {
  const int64_t rows_per_block = (int64_t)(kQuantThreads / 32) * (32 / LPR);
  int any_outlier = quant_rows_vec_body<T, LPR, NV, MODE>(a, (int64_t)blockIdx.x * rows_per_block,
                                                          (int64_t)gridDim.x * rows_per_block, a.rows, nullptr);
  if ((MODE == kQueryFoldGate || MODE == kGateOnly) && a.flag != nullptr) {
    any_outlier = __syncthreads_or(any_outlier);
    if (threadIdx.x == 0 && any_outlier) atomicOr(a.flag, 1);
  }
}

// One warp per row, scalar element access, two passes over the row (the second
// comes from L1/L2): every dtype, every K.
template <typename T, int MODE>
__global__ void __launch_bounds__(kQuantThreads) quant_rows_generic_kernel(QuantArgs a) {
  constexpr unsigned FULL = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int rank_need = ((a.K - 1) >> 1) + 1;
  int any_outlier = 0;
  for (int64_t row = (int64_t)blockIdx.x * (kQuantThreads / 32) + warp; row < a.rows;
       row += (int64_t)gridDim.x * (kQuantThreads / 32)) {
    const T* xr = reinterpret_cast<const T*>(a.x) + row * a.K;
    const float* mr = (MODE == kKeySmooth) ? a.mean + mean_row(a, row) * a.K : nullptr;
    auto elem = [&](int c) -> float {
      float v = to_f32<T>(xr[c]);
      if (MODE == kKeySmooth) v = to_f32<T>(from_f32<T>(v - mr[c]));
      return v;
    };
    float amax = 0.0f;
    for (int c = lane; c < a.K; c += 32) amax = fmaxf(amax, fabsf(elem(c)));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, off));
    float s = amax * kQMaxInv;
    s = (s == 0.0f) ? 1.0f : s;
    if ((MODE == kQueryFoldGate || MODE == kGateOnly) && a.flag != nullptr) {
      int cnt = 0;
      for (int c = lane; c < a.K; c += 32)
        cnt += (__fdiv_rn(amax, fabsf(elem(c)) + 1e-10f) > a.ratio_threshold) ? 1 : 0;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) cnt += __shfl_xor_sync(FULL, cnt, off);
      if (cnt >= rank_need) any_outlier = 1;
    }
    if (MODE == kGateOnly) continue;
    int8_t* qr = a.q + row * a.K;
    for (int c = lane; c < a.K; c += 32) {
      const float e = elem(c);
      qr[c] = (int8_t)quant_one(e, s);
      if (MODE == kKeySmooth && a.smoothed != nullptr)
        reinterpret_cast<T*>(a.smoothed)[row * a.K + c] = from_f32<T>(e);
    }
    if (lane == 0) {
      if (MODE == kQueryFoldGate) {
        a.scale[row] = s * a.fold;
        if (a.plain_scale != nullptr) a.plain_scale[row] = s;
      } else {
        a.scale[row] = s;
      }
    }
  }
  if ((MODE == kQueryFoldGate || MODE == kGateOnly) && a.flag != nullptr) {
    any_outlier = __syncthreads_or(any_outlier);
    if (threadIdx.x == 0 && any_outlier) atomicOr(a.flag, 1);
  }
}

int grid_for(int64_t rows, int64_t rows_per_block) {
  int64_t need = (rows + rows_per_block - 1) / rows_per_block;
  const int64_t cap = (int64_t)kNumSms * 16;  // 8 resident blocks per SM, two waves
  if (need > cap) need = cap;
  return (int)(need < 1 ? 1 : need);
}

template <typename T, int MODE, int LPR, int NV>
void launch_vec(const QuantArgs& a, cudaStream_t s) {
  const int64_t rpb = (int64_t)(kQuantThreads / 32) * (32 / LPR);
  quant_rows_vec_kernel<T, LPR, NV, MODE><<<grid_for(a.rows, rpb), kQuantThreads, 0, s>>>(a);
}

template <typename T, int MODE>
int launch_2byte(const QuantArgs& a, cudaStream_t s) {
  const int kvec = a.K / 8;
  const bool vec_ok = (a.K % 8 == 0) && aligned16(a.x) && (MODE == kGateOnly || reinterpret_cast<uintptr_t>(a.q) % 8 == 0) &&
                      (MODE != kKeySmooth || (aligned16(a.mean) && (a.smoothed == nullptr || aligned16(a.smoothed))));
  if (MODE == kRotate && !vec_ok) return SL8_ERR_MISALIGNED;   // the rotation lives in the vector kernel only
  // lanes per row x vectors per lane: four 16-byte vectors per lane amortise the per-row work
  // (reductions, scale, reciprocal, threshold) over 32 elements
  if (vec_ok && kvec <= 4) launch_vec<T, MODE, 2, 2>(a, s);
  else if (vec_ok && kvec <= 8) launch_vec<T, MODE, 2, 4>(a, s);
  else if (vec_ok && kvec <= 12) launch_vec<T, MODE, 4, 3>(a, s);
  else if (vec_ok && kvec <= 16) launch_vec<T, MODE, 4, 4>(a, s);
  else if (vec_ok && kvec <= 32) launch_vec<T, MODE, 8, 4>(a, s);
  else if (vec_ok && kvec <= 64) launch_vec<T, MODE, 16, 4>(a, s);
  else if (vec_ok && kvec <= 128) launch_vec<T, MODE, 32, 4>(a, s);
  else
    quant_rows_generic_kernel<T, MODE><<<grid_for(a.rows, kQuantThreads / 32), kQuantThreads, 0, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

template <int MODE>
int dispatch(const QuantArgs& a, int dtype, cudaStream_t s) {
  if (a.rows < 0 || a.K < 0) return SL8_ERR_BAD_SHAPE;
  if (a.rows == 0 || a.K == 0) return SL8_OK;
  if (a.x == nullptr || (MODE != kGateOnly && (a.q == nullptr || a.scale == nullptr))) return SL8_ERR_NULL;
  if (MODE == kGateOnly && a.flag == nullptr) return SL8_ERR_NULL;
  switch (dtype) {
    case SL8_F16: return launch_2byte<__half, MODE>(a, s);
    case SL8_BF16: return launch_2byte<__nv_bfloat16, MODE>(a, s);
    case SL8_F32:
      quant_rows_generic_kernel<float, MODE><<<grid_for(a.rows, kQuantThreads / 32), kQuantThreads, 0, s>>>(a);
      return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
    default: return SL8_ERR_BAD_DTYPE;
  }
}

// ---- K mean -------------------------------------------------------------------
constexpr int kMeanChunkRows = 1024;
constexpr int kMeanThreads = 512;

// grid (chunks, BH).  Thread (rl, cv) sums rows rl, rl + RL, ... of the chunk for
// the 8 columns of vector cv; the RL row-lanes are then added in index order.
// Column sums of rows [r0, r1) of one head (kb = its first row) into out[K] (global or shared memory),
// by the whole block of kMeanThreads threads, in a fixed order: thread (rl, cv) sums rows
// r0 + rl, r0 + rl + RL, ... for the 8 columns of vector cv, then the RL row-lanes are added in index
// order.  red: shared scratch [RL][K].  Ends with a block-wide sync.
template <typename T>
__device__ __forceinline__ void chunk_column_sums(const T* __restrict__ kb, int64_t r0, int64_t r1, int K, float* red,
                                                  float* out) {
  const int kvec = K >> 3;
  int cvp = 1;
  while (cvp < kvec) cvp <<= 1;   // column lanes, power of two <= 256
  const int RL = kMeanThreads / cvp;
  const int cv = threadIdx.x % cvp;
  const int rl = threadIdx.x / cvp;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cv < kvec) {
    // four rows in flight per thread; they are added in row order, so the sum does not depend on it
    constexpr int U = 4;
    int64_t r = r0 + rl;
    for (; r + (int64_t)(U - 1) * RL < r1; r += (int64_t)U * RL) {
      uint4 u[U];
#pragma unroll
      for (int x = 0; x < U; ++x) u[x] = __ldg(reinterpret_cast<const uint4*>(kb + (r + (int64_t)x * RL) * K) + cv);
#pragma unroll
      for (int x = 0; x < U; ++x) {
        float f[8];
        Vec8<T>::unpack(u[x], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    for (; r < r1; r += RL) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(kb + r * K) + cv);
      float f[8];
      Vec8<T>::unpack(u, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rl * K + cv * 8 + i] = acc[i];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < K; c += kMeanThreads) {
    float s = 0.0f;
    for (int r = 0; r < RL; ++r) s += red[r * K + c];
    out[c] = s;
  }
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kMeanThreads) k_mean_partial_kernel(
    const T* __restrict__ k, int64_t N, int K, const int32_t* __restrict__ seqlens, int heads_per_batch,
    float* __restrict__ partial, int nchunks) {
  extern __shared__ float red[];  // [RL][K]
  const int64_t bh = blockIdx.y;
  const int64_t len = seqlens ? (int64_t)seqlens[bh / heads_per_batch] : N;
  const int64_t r0 = (int64_t)blockIdx.x * kMeanChunkRows;
  const int64_t r1 = min(len < N ? len : N, r0 + kMeanChunkRows);
  chunk_column_sums<T>(k + bh * N * K, r0, r1, K, red, partial + (bh * nchunks + blockIdx.x) * K);
}

// ---- K prologue in one launch ---------------------------------------------------
// A cluster of kClusterCtas blocks owns one (batch, kv-head) slab [N, K].  Block r takes the 1024-row
// chunks r, r + 8, ...: (1) their column sums, chunk by chunk, into its own shared memory -- the same
// thread map and order as k_mean_partial_kernel; (2) after a cluster barrier every block adds ALL chunk
// sums of the slab in chunk order, reading the other blocks' through distributed shared memory, so
// every block holds the same mean, bit for bit the one the two-kernel path produces; (3) after a
// second cluster barrier (nobody reads a neighbour's shared memory any more) it walks its chunks
// again, subtracts the mean, rounds to the storage dtype and quantises the rows.  The second walk
// comes from L2 as long as the slabs of the resident clusters fit there (4 blocks per SM = 74
// clusters: up to about 1.5 MB per slab); beyond that it is a second read of HBM (measured on 128
// slabs of 2 MB: 531 MB read for 268 MB of K, L2 hit rate 16 %) and the kernel is still faster than
// the three-launch path because it is bound by latency, not by bytes: fewer resident blocks, which
// would keep the slabs in L2, measure slower (3 / 2 blocks per SM: 179 / 198 us against 155).
constexpr int kClusterCtas = 8;

template <typename T, int LPR, int NV>
__global__ void __cluster_dims__(kClusterCtas, 1, 1) __launch_bounds__(kMeanThreads)
    k_prologue_cluster_kernel(QuantArgs a, int64_t N, const int32_t* __restrict__ seqlens, int heads_per_batch,
                              float* __restrict__ mean_out, int nchunks, int chunks_per_cta) {
  extern __shared__ float sm[];
  const int K = a.K;
  float* mean_s = sm;                       // [K]
  float* part = sm + K;                     // [chunks_per_cta][K]: this block's chunk sums
  float* red = part + chunks_per_cta * K;   // [RL][K]
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int64_t bh = blockIdx.y;
  int64_t len = seqlens ? (int64_t)seqlens[bh / heads_per_batch] : N;
  len = len < 0 ? 0 : (len > N ? N : len);
  const T* kb = reinterpret_cast<const T*>(a.x) + bh * N * K;
  for (int jj = 0; jj < chunks_per_cta; ++jj) {
    const int j = rank + jj * kClusterCtas;
    if (j >= nchunks) break;
    const int64_t r0 = (int64_t)j * kMeanChunkRows;
    chunk_column_sums<T>(kb, r0, min(len, r0 + kMeanChunkRows), K, red, part + jj * K);
  }
  cluster.sync();
  const float inv = len > 0 ? __fdiv_rn(1.0f, (float)len) : 0.0f;
  for (int c = threadIdx.x; c < K; c += kMeanThreads) {
    float s = 0.0f;
    for (int j = 0; j < nchunks; ++j) {
      const float* remote = cluster.map_shared_rank(part, j % kClusterCtas);
      s += remote[(j / kClusterCtas) * K + c];
    }
    const float m = s * inv;
    mean_s[c] = m;
    if (rank == 0 && mean_out != nullptr) mean_out[bh * K + c] = m;
  }
  cluster.sync();
  // quantise this block's chunks (all N rows of the slab are quantised, also those past seqlens)
  const int64_t rows_per_block = (int64_t)(kMeanThreads / 32) * (32 / LPR);
  for (int jj = 0; jj < chunks_per_cta; ++jj) {
    const int j = rank + jj * kClusterCtas;
    if (j >= nchunks) break;
    const int64_t row0 = bh * N + (int64_t)j * kMeanChunkRows;
    const int64_t row1 = bh * N + min(N, (int64_t)(j + 1) * kMeanChunkRows);
    quant_rows_vec_body<T, LPR, NV, kKeySmooth>(a, row0, rows_per_block, row1, mean_s);
  }
}

__global__ void k_mean_finish_kernel(const float* __restrict__ partial, int nchunks, int K, int64_t N,
                                     const int32_t* __restrict__ seqlens, int heads_per_batch,
                                     float* __restrict__ mean) {
  const int64_t bh = blockIdx.x;
  int64_t len = seqlens ? (int64_t)seqlens[bh / heads_per_batch] : N;
  if (len > N) len = N;
  const float inv = len > 0 ? __fdiv_rn(1.0f, (float)len) : 0.0f;
  for (int c = threadIdx.x; c < K; c += blockDim.x) {
    float s = 0.0f;
    for (int j = 0; j < nchunks; ++j) s += partial[(bh * nchunks + j) * K + c];
    mean[bh * K + c] = s * inv;
  }
}

// ---- per-channel V quantiser (int8-V cache) -------------------------------------------
// grid (chunks, BH): per-channel max |v| over the chunk's rows, same thread map as the K mean.
template <typename T>
__global__ void __launch_bounds__(kMeanThreads) v_colamax_partial_kernel(const T* __restrict__ v, int64_t N, int K,
                                                                         float* __restrict__ partial, int nchunks) {
  extern __shared__ float red[];  // [RL][K]
  const int kvec = K >> 3;
  int cvp = 1;
  while (cvp < kvec) cvp <<= 1;
  const int RL = kMeanThreads / cvp;
  const int cv = threadIdx.x % cvp;
  const int rl = threadIdx.x / cvp;
  const int64_t bh = blockIdx.y;
  const int64_t r0 = (int64_t)blockIdx.x * kMeanChunkRows;
  const int64_t r1 = min(N, r0 + kMeanChunkRows);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cv < kvec) {
    const T* vb = v + bh * N * K;
    for (int64_t r = r0 + rl; r < r1; r += RL) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(vb + r * K) + cv);
      float f[8];
      Vec8<T>::unpack(u, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaxf(acc[i], fabsf(f[i]));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rl * K + cv * 8 + i] = acc[i];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < K; c += kMeanThreads) {
    float m = 0.0f;
    for (int r = 0; r < RL; ++r) m = fmaxf(m, red[r * K + c]);
    partial[(bh * nchunks + blockIdx.x) * K + c] = m;
  }
}

// scale[bh, c] = amax / 127 (0 -> 1), the rule of reference superl8/quant/core.py:107-108
__global__ void v_scale_finish_kernel(const float* __restrict__ partial, int nchunks, int K, float* __restrict__ scale) {
  const int64_t bh = blockIdx.x;
  for (int c = threadIdx.x; c < K; c += blockDim.x) {
    float m = 0.0f;
    for (int j = 0; j < nchunks; ++j) m = fmaxf(m, partial[(bh * nchunks + j) * K + c]);
    const float sc = __fdiv_rn(m, kQMax);
    scale[bh * K + c] = sc == 0.0f ? 1.0f : sc;
  }
}

// codes = clamp(rint(v / scale[channel]), -127, 127) (core.py:109); 8 channels per thread
template <typename T>
__global__ void __launch_bounds__(256) v_quant_perchannel_kernel(const T* __restrict__ v, const float* __restrict__ scale,
                                                                 int8_t* __restrict__ q, int64_t N, int K,
                                                                 int64_t total_vec) {
  const int kvec = K >> 3;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (int64_t)gridDim.x * blockDim.x) {
    const int cv = (int)(i % kvec);
    const int64_t row = i / kvec, bh = row / N;
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(v) + i);
    float f[8];
    Vec8<T>::unpack(u, f);
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(scale + bh * K + cv * 8));
    const float4 s1 = __ldg(reinterpret_cast<const float4*>(scale + bh * K + cv * 8 + 4));
    const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int c = (int)quant_one(f[e], sc[e]);
      w[e >> 2] |= (uint32_t)(c & 0xff) << (8 * (e & 3));
    }
    *reinterpret_cast<uint2*>(q + i * 8) = make_uint2(w[0], w[1]);
  }
}

// Packed token-major keys [tokens, heads, K]: mean over the tokens of one sequence for one head.
// grid (heads, sequences).  Same thread map and fixed summation order as the dense kernel:
// thread (rl, cv) sums tokens rl, rl + RL, ... for the 8 columns of vector cv, the RL lanes are
// added in index order, and the sum is multiplied by 1 / len.
template <typename T>
__global__ void __launch_bounds__(kMeanThreads) k_mean_packed_kernel(
    const T* __restrict__ k, int heads, int K, const int32_t* __restrict__ cu_seqlens, float* __restrict__ mean) {
  extern __shared__ float red[];  // [RL][K]
  const int kvec = K >> 3;
  int cvp = 1;
  while (cvp < kvec) cvp <<= 1;
  const int RL = kMeanThreads / cvp;
  const int cv = threadIdx.x % cvp;
  const int rl = threadIdx.x / cvp;
  const int head = blockIdx.x, seq = blockIdx.y;
  const int64_t t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (cv < kvec) {
    for (int64_t t = t0 + rl; t < t1; t += RL) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(k + (t * heads + head) * K) + cv);
      float f[8];
      Vec8<T>::unpack(u, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rl * K + cv * 8 + i] = acc[i];
  }
  __syncthreads();
  const int64_t len = t1 - t0;
  const float inv = len > 0 ? __fdiv_rn(1.0f, (float)len) : 0.0f;
  for (int c = threadIdx.x; c < K; c += kMeanThreads) {
    float s = 0.0f;
    for (int r = 0; r < RL; ++r) s += red[r * K + c];
    mean[((int64_t)seq * heads + head) * K + c] = s * inv;
  }
}

}  // namespace
}  // namespace sl8

using namespace sl8;

extern "C" int sl8_q_outlier_gate(const void* q, int dtype, int64_t rows, int64_t D, float ratio_threshold,
                                  int32_t* outlier_flag, void* stream) {
  if (D > (1 << 30)) return SL8_ERR_TOO_LARGE;
  QuantArgs a{};
  a.x = q; a.flag = outlier_flag; a.rows = rows; a.K = (int)D; a.rows_per_head = 1; a.ratio_threshold = ratio_threshold;
  return dispatch<kGateOnly>(a, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int sl8_quantize_v_perchannel(const void* v, int dtype, int64_t BH, int64_t N, int64_t D, int8_t* v_i8,
                                         float* v_scale, void* workspace, size_t workspace_bytes, void* stream) {
  if (BH < 0 || N < 0 || D < 0) return SL8_ERR_BAD_SHAPE;
  if (dtype != SL8_F16 && dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (D % 8 != 0 || D > 2048) return SL8_ERR_BAD_HEAD_DIM;
  if (BH == 0 || D == 0) return SL8_OK;
  if (v_scale == nullptr) return SL8_ERR_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N == 0) {   // no key: amax 0 -> scale 1 (core.py:108)
    v_scale_finish_kernel<<<(unsigned)BH, 128, 0, s>>>(nullptr, 0, (int)D, v_scale);
    return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
  }
  if (v == nullptr || v_i8 == nullptr) return SL8_ERR_NULL;
  if (!aligned16(v) || !aligned16(v_i8) || !aligned16(v_scale)) return SL8_ERR_MISALIGNED;
  if (BH > 65535) return SL8_ERR_TOO_LARGE;
  if (workspace == nullptr || workspace_bytes < sl8_k_mean_workspace(BH, N, D)) return SL8_ERR_WORKSPACE;
  const int nchunks = (int)((N + kMeanChunkRows - 1) / kMeanChunkRows);
  float* partial = reinterpret_cast<float*>(workspace);
  int cvp = 1;
  while (cvp < (int)(D >> 3)) cvp <<= 1;
  const size_t smem = (size_t)(kMeanThreads / cvp) * D * sizeof(float);
  dim3 grid((unsigned)nchunks, (unsigned)BH);
  const int64_t total_vec = BH * N * (D >> 3);
  const unsigned qblocks = (unsigned)std::min<int64_t>((total_vec + 255) / 256, (int64_t)kNumSms * 16);
  if (dtype == SL8_F16) {
    v_colamax_partial_kernel<__half><<<grid, kMeanThreads, smem, s>>>(reinterpret_cast<const __half*>(v), N, (int)D, partial, nchunks);
    v_scale_finish_kernel<<<(unsigned)BH, 128, 0, s>>>(partial, nchunks, (int)D, v_scale);
    v_quant_perchannel_kernel<__half><<<qblocks, 256, 0, s>>>(reinterpret_cast<const __half*>(v), v_scale, v_i8, N, (int)D, total_vec);
  } else {
    v_colamax_partial_kernel<__nv_bfloat16><<<grid, kMeanThreads, smem, s>>>(reinterpret_cast<const __nv_bfloat16*>(v), N, (int)D, partial, nchunks);
    v_scale_finish_kernel<<<(unsigned)BH, 128, 0, s>>>(partial, nchunks, (int)D, v_scale);
    v_quant_perchannel_kernel<__nv_bfloat16><<<qblocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(v), v_scale, v_i8, N, (int)D, total_vec);
  }
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

extern "C" int sl8_k_mean_packed(const void* k, int dtype, int64_t total_tokens, int32_t heads, int64_t D,
                                 const int32_t* cu_seqlens, int32_t n_seq, float* mean, void* stream) {
  if (total_tokens < 0 || heads < 0 || D < 0 || n_seq < 0) return SL8_ERR_BAD_SHAPE;
  if (dtype != SL8_F16 && dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (D % 8 != 0 || D > 2048) return SL8_ERR_BAD_HEAD_DIM;
  if (n_seq == 0 || heads == 0 || D == 0) return SL8_OK;
  if (mean == nullptr || cu_seqlens == nullptr || (total_tokens > 0 && k == nullptr)) return SL8_ERR_NULL;
  if (!aligned16(k)) return SL8_ERR_MISALIGNED;
  if (n_seq > 65535) return SL8_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int cvp = 1;
  while (cvp < (int)(D >> 3)) cvp <<= 1;
  const size_t smem = (size_t)(kMeanThreads / cvp) * D * sizeof(float);
  dim3 grid((unsigned)heads, (unsigned)n_seq);
  if (dtype == SL8_F16)
    k_mean_packed_kernel<__half><<<grid, kMeanThreads, smem, s>>>(reinterpret_cast<const __half*>(k), heads, (int)D, cu_seqlens, mean);
  else
    k_mean_packed_kernel<__nv_bfloat16><<<grid, kMeanThreads, smem, s>>>(reinterpret_cast<const __nv_bfloat16*>(k), heads, (int)D, cu_seqlens, mean);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

extern "C" int sl8_smooth_quant_k_packed(const void* k, int dtype, int64_t total_tokens, int32_t heads, int64_t D,
                                         const int32_t* cu_seqlens, int32_t n_seq, const float* mean,
                                         int8_t* k_i8, float* k_scale, void* k_smoothed, void* stream) {
  if (total_tokens < 0 || heads < 0 || D < 0 || n_seq < 0) return SL8_ERR_BAD_SHAPE;
  if (D > (1 << 30)) return SL8_ERR_TOO_LARGE;
  if (dtype == SL8_F32) return SL8_ERR_BAD_DTYPE;
  if (total_tokens * heads > 0 && (mean == nullptr || cu_seqlens == nullptr || n_seq == 0)) return SL8_ERR_NULL;
  QuantArgs a{};
  a.x = k; a.q = k_i8; a.scale = k_scale; a.mean = mean; a.smoothed = k_smoothed;
  a.rows = total_tokens * heads; a.K = (int)D; a.rows_per_head = 1;
  a.cu_seqlens = cu_seqlens; a.n_seq = n_seq; a.heads = heads;
  return dispatch<kKeySmooth>(a, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int sl8_quantize_i8_rowwise(const void* x, int x_dtype, int64_t M, int64_t K, int8_t* q,
                                       float* scale, void* stream) {
  if (K > (1 << 30)) return SL8_ERR_TOO_LARGE;
  QuantArgs a{};
  a.x = x; a.q = q; a.scale = scale; a.rows = M; a.K = (int)K; a.rows_per_head = 1;
  return dispatch<kPlain>(a, x_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int sl8_quant_q_prologue(const void* q, int dtype, int64_t rows, int64_t D, float fold,
                                    float ratio_threshold, int8_t* q_i8, float* q_scale_folded,
                                    float* plain_scale, int32_t* outlier_flag, void* stream) {
  if (D > (1 << 30)) return SL8_ERR_TOO_LARGE;
  QuantArgs a{};
  a.x = q; a.q = q_i8; a.scale = q_scale_folded; a.plain_scale = plain_scale; a.flag = outlier_flag;
  a.rows = rows; a.K = (int)D; a.rows_per_head = 1; a.fold = fold; a.ratio_threshold = ratio_threshold;
  return dispatch<kQueryFoldGate>(a, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" size_t sl8_k_mean_workspace(int64_t BH, int64_t N, int64_t D) {
  if (BH <= 0 || N <= 0 || D <= 0) return 16;
  const int64_t nchunks = (N + kMeanChunkRows - 1) / kMeanChunkRows;
  return (size_t)(BH * nchunks * D) * sizeof(float) + 16;
}

extern "C" int sl8_k_mean(const void* k, int dtype, int64_t BH, int64_t N, int64_t D,
                          const int32_t* seqlens, int32_t heads_per_batch, float* mean, void* workspace,
                          size_t workspace_bytes, void* stream) {
  if (BH < 0 || N < 0 || D < 0) return SL8_ERR_BAD_SHAPE;
  if (BH == 0 || D == 0) return SL8_OK;
  if (k == nullptr || mean == nullptr) return SL8_ERR_NULL;
  if (dtype != SL8_F16 && dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (D % 8 != 0 || D > 2048) return SL8_ERR_BAD_HEAD_DIM;
  if (!aligned16(k)) return SL8_ERR_MISALIGNED;
  if (seqlens != nullptr && heads_per_batch <= 0) return SL8_ERR_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N == 0) {
    SL8_CUDA_TRY(cudaMemsetAsync(mean, 0, (size_t)(BH * D) * sizeof(float), s));
    return SL8_OK;
  }
  if (workspace == nullptr || workspace_bytes < sl8_k_mean_workspace(BH, N, D)) return SL8_ERR_WORKSPACE;
  const int nchunks = (int)((N + kMeanChunkRows - 1) / kMeanChunkRows);
  int cvp = 1;
  while (cvp < D / 8) cvp <<= 1;
  const size_t smem = (size_t)(kMeanThreads / cvp) * D * sizeof(float);
  float* partial = reinterpret_cast<float*>(workspace);
  dim3 grid(nchunks, (unsigned)BH);
  if (BH > 65535) return SL8_ERR_TOO_LARGE;
  if (dtype == SL8_F16)
    k_mean_partial_kernel<__half><<<grid, kMeanThreads, smem, s>>>(
        reinterpret_cast<const __half*>(k), N, (int)D, seqlens, heads_per_batch, partial, nchunks);
  else
    k_mean_partial_kernel<__nv_bfloat16><<<grid, kMeanThreads, smem, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(k), N, (int)D, seqlens, heads_per_batch, partial, nchunks);
  k_mean_finish_kernel<<<(unsigned)BH, 128, 0, s>>>(partial, nchunks, (int)D, N, seqlens, heads_per_batch, mean);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

extern "C" int sl8_smooth_quant_k(const void* k, int dtype, int64_t BH, int64_t N, int64_t D,
                                  const float* mean, int8_t* k_i8, float* k_scale, void* k_smoothed,
                                  void* stream) {
  if (BH < 0 || N < 0 || D < 0) return SL8_ERR_BAD_SHAPE;
  if (D > (1 << 30)) return SL8_ERR_TOO_LARGE;
  if (BH * N > 0 && mean == nullptr) return SL8_ERR_NULL;
  if (dtype == SL8_F32) return SL8_ERR_BAD_DTYPE;
  QuantArgs a{};
  a.x = k; a.q = k_i8; a.scale = k_scale; a.mean = mean; a.smoothed = k_smoothed;
  a.rows = BH * N; a.K = (int)D; a.rows_per_head = N > 0 ? N : 1;
  return dispatch<kKeySmooth>(a, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int sl8_hadamard_quant_rows(const void* x, int dtype, int64_t rows, int64_t D, const float* mean,
                                       int64_t rows_per_head, float fold, int8_t* q, float* scale, void* rotated,
                                       void* stream) {
  if (rows < 0 || D < 0) return SL8_ERR_BAD_SHAPE;
  if (dtype != SL8_F16 && dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (D < 32 || D > 1024 || (D & (D - 1)) != 0) return SL8_ERR_UNSUPPORTED;   // Sylvester order: power of two
  if (rows == 0) return SL8_OK;
  if (x == nullptr || (q == nullptr && rotated == nullptr) || (q != nullptr && scale == nullptr)) return SL8_ERR_NULL;
  if (mean != nullptr && rows_per_head <= 0) return SL8_ERR_BAD_SHAPE;
  if (!aligned16(x) || (rotated != nullptr && !aligned16(rotated)) || reinterpret_cast<uintptr_t>(q) % 8 != 0 ||
      (mean != nullptr && !aligned16(mean)))
    return SL8_ERR_MISALIGNED;
  QuantArgs a{};
  a.x = x; a.q = q; a.scale = scale; a.mean = mean; a.rotated = rotated;
  a.rows = rows; a.K = (int)D; a.rows_per_head = mean != nullptr ? rows_per_head : 1; a.fold = fold;
  a.rot_norm = (float)(1.0 / sqrt((double)D));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // (dispatch<> insists on code and scale pointers; the rotation alone has none)
  return dtype == SL8_F16 ? launch_2byte<__half, kRotate>(a, s) : launch_2byte<__nv_bfloat16, kRotate>(a, s);
}

namespace {
template <typename T, int LPR, int NV>
int launch_k_prologue(const QuantArgs& a, int64_t BH, int64_t N, const int32_t* seqlens, int heads_per_batch, float* mean,
                      int nchunks, int chunks_per_cta, size_t smem, cudaStream_t s) {
  dim3 grid(kClusterCtas, (unsigned)BH);
  k_prologue_cluster_kernel<T, LPR, NV><<<grid, kMeanThreads, smem, s>>>(a, N, seqlens, heads_per_batch, mean, nchunks,
                                                                       chunks_per_cta);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}
}  // namespace

extern "C" int sl8_k_prologue_fused_ok(int dtype, int64_t BH, int64_t N, int64_t D) {
  if (dtype != SL8_F16 && dtype != SL8_BF16) return 0;
  if (D != 64 && D != 128 && D != 256) return 0;
  if (BH <= 0 || BH > 65535 || N <= 0) return 0;
  const int64_t nchunks = (N + kMeanChunkRows - 1) / kMeanChunkRows;
  const int64_t per = (nchunks + kClusterCtas - 1) / kClusterCtas;
  int cvp = 1;
  while (cvp < D / 8) cvp <<= 1;
  const int64_t smem = (D + per * D + (int64_t)(kMeanThreads / cvp) * D) * 4;
  return smem <= 48 * 1024 ? 1 : 0;
}

extern "C" int sl8_k_prologue(const void* k, int dtype, int64_t BH, int64_t N, int64_t D, const int32_t* seqlens,
                              int32_t heads_per_batch, float* mean, int8_t* k_i8, float* k_scale, void* k_smoothed,
                              void* stream) {
  if (BH < 0 || N < 0 || D < 0) return SL8_ERR_BAD_SHAPE;
  if (BH == 0 || D == 0 || N == 0) return SL8_OK;
  if (k == nullptr || mean == nullptr || k_i8 == nullptr || k_scale == nullptr) return SL8_ERR_NULL;
  if (seqlens != nullptr && heads_per_batch <= 0) return SL8_ERR_BAD_SHAPE;
  if (!sl8_k_prologue_fused_ok(dtype, BH, N, D)) return SL8_ERR_UNSUPPORTED;
  if (!aligned16(k) || !aligned16(mean) || reinterpret_cast<uintptr_t>(k_i8) % 8 != 0 ||
      (k_smoothed != nullptr && !aligned16(k_smoothed)))
    return SL8_ERR_MISALIGNED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  QuantArgs a{};
  a.x = k; a.q = k_i8; a.scale = k_scale; a.mean = mean; a.smoothed = k_smoothed;
  a.rows = BH * N; a.K = (int)D; a.rows_per_head = N;
  const int nchunks = (int)((N + kMeanChunkRows - 1) / kMeanChunkRows);
  const int per = (nchunks + kClusterCtas - 1) / kClusterCtas;
  int cvp = 1;
  while (cvp < D / 8) cvp <<= 1;
  const size_t smem = (size_t)(D + (int64_t)per * D + (int64_t)(kMeanThreads / cvp) * D) * 4;
  const bool h = dtype == SL8_F16;
  switch ((int)D) {   // lanes per row x vectors per lane as in launch_2byte
    case 64: return h ? launch_k_prologue<__half, 2, 4>(a, BH, N, seqlens, heads_per_batch, mean, nchunks, per, smem, s)
                      : launch_k_prologue<__nv_bfloat16, 2, 4>(a, BH, N, seqlens, heads_per_batch, mean, nchunks, per, smem, s);
    case 128: return h ? launch_k_prologue<__half, 4, 4>(a, BH, N, seqlens, heads_per_batch, mean, nchunks, per, smem, s)
                       : launch_k_prologue<__nv_bfloat16, 4, 4>(a, BH, N, seqlens, heads_per_batch, mean, nchunks, per, smem, s);
    case 256: return h ? launch_k_prologue<__half, 8, 4>(a, BH, N, seqlens, heads_per_batch, mean, nchunks, per, smem, s)
                       : launch_k_prologue<__nv_bfloat16, 8, 4>(a, BH, N, seqlens, heads_per_batch, mean, nchunks, per, smem, s);
  }
  return SL8_ERR_UNSUPPORTED;
}
