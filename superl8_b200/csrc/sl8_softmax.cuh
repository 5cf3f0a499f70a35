// The softmax sweep shared by the tensor-memory forward kernels: one pass over 64 accumulator
// columns of a thread's query row (conversion, scaling, running max, 2^x, row sum, packing of P).
#pragma once
#include "sl8_common.cuh"

namespace sl8 {

constexpr int kSweepCols = 64;   // columns per sweep = one tcgen05.ld of 2 x 32 columns per thread

constexpr float kLazyRescaleLog2 = 8.0f;


__device__ __forceinline__ float2 bits2(uint32_t a, uint32_t b) {
  return make_float2(__uint_as_float(a), __uint_as_float(b));
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }

// 2^x of a pair on the FMA pipe: n = round(x) through the magic-number add, f = x - n in
// [-0.5, 0.5], a degree-3 minimax polynomial for 2^f (relative error 7.5e-5, a third of the
// rounding step of fp16) and n added into the exponent field with one integer multiply-add.
// Arguments below -126 (masked keys carry -inf) give 2^-126, which rounds to zero in P.
__device__ __forceinline__ float2 exp2_poly_pair(float2 x) {
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 magic = make_float2(12582912.f, 12582912.f), nmagic = make_float2(-12582912.f, -12582912.f);
  const float2 r = __fadd2_rn(x, magic);            // the integer n sits in the low mantissa bits
  const float2 n = __fadd2_rn(r, nmagic);
  const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
  float2 p = __ffma2_rn(f, make_float2(0.055171288549900055f, 0.055171288549900055f),
                        make_float2(0.24261046946048737f, 0.24261046946048737f));
  p = __ffma2_rn(p, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
  p = __ffma2_rn(p, f, make_float2(0.9999281167984009f, 0.9999281167984009f));
  // (bits(r) << 23) == n << 23 modulo 2^32: the bias bits of the magic number shift out
  return make_float2(__uint_as_float(__float_as_uint(r.x) * 0x800000u + __float_as_uint(p.x)),
                     __uint_as_float(__float_as_uint(r.y) * 0x800000u + __float_as_uint(p.y)));
}

// Build option, off: of every 8 pairs of exponentials, SL8_POLY_OF_8 go through the polynomial and
// the rest through ex2 on the special-function unit (16 results per clock and SM).  Measured on a
// B = 4 slice of the S = 8192 causal workload: 0 / 1 / 2 / 3 of 8 give 4.10 / 4.32 / 4.28 / 4.57 ms in
// 16-bit mode and 4.12-4.16 / 4.30 / 4.07 / 4.26 ms in int8 mode -- the sweep is not bound by the
// special-function unit alone (replacing every ex2 by a multiply saves 4 % / 14 %), and the
// polynomial's ten instructions per pair cost issue slots the sweep does not have to spare.
#ifndef SL8_POLY_OF_8
#define SL8_POLY_OF_8 0
#endif
__host__ __device__ constexpr bool pair_uses_poly(int u) {
  return ((u % 8) * SL8_POLY_OF_8) / 8 != (((u % 8) + 1) * SL8_POLY_OF_8) / 8;
}

// One streaming pass over the kSweepCols columns of this thread's row:
//   FIRST: r holds the accumulators.  int8 mode: t = float(acc) * k_scale[n]; 16-bit mode: t = acc.
//          MASK = false leaves t in r (the exponent is then fma(t, qs, -m): scale and max
//          subtraction in one instruction per pair); MASK = true (tiles on the diagonal, the
//          window edge or the tail) leaves the finished logits t * qs, -inf where masked (xs = 1).
//          The maximum of what is left in r is tracked (the caller scales it by qs >= 0).
//          The reference multiplies (float(acc) * q_scale) * k_scale
//          (csrc/include/attn_int8_fwd.cuh:137); the two orders differ by fp32 rounding only.
//   both:  P = 2^(r * xs - m) goes to tensor memory as 16-bit pairs over the first kSweepCols / 2 columns
//          of the S buffer, and its fp32 row sum is returned.
// The sweep is software-pipelined by hand, in groups of G pairs: the ex2 of group g are issued,
// then the conversion / scaling / max of group g + 1 (work for the FMA and ALU pipes that does
// not depend on them), and only then the sums and the packing of group g.  A warp issues in
// order, so this is what lets the special-function unit run while the other pipes work.
// BIAS (16-bit mode, with MASK and FIRST): an additive bias row in natural-log units (element type
// VT, bias[n * bias_sn] for key n of this thread's query row; null for rows past the end) is added
// to the finished logits as bias * log2(e) -- the mask argument of the reference's full-precision
// forward (csrc/include/attn_fp16_fwd.cuh:176-178).  Eight contiguous, 16-byte aligned values are
// one load; anything else is read element by element.
template <bool QK8, bool MASK, bool FIRST, typename VT, bool BIAS = false>
__device__ __forceinline__ void softmax_pass(uint32_t (&r)[kSweepCols], const float* __restrict__ ksv, float qs, float xs,
                                             float neg_m, int n_block, int n_len, int causal, int qpos,
                                             int window_left, uint32_t t_p, float& mx, float& sum,
                                             const VT* __restrict__ bias = nullptr, int64_t bias_sn = 0) {
  static_assert(!BIAS || (MASK && FIRST && !QK8), "the bias joins the finished logits of the 16-bit mode");
  const float2 qs2 = make_float2(qs, qs), xs2 = make_float2(xs, xs), neg_m2 = make_float2(neg_m, neg_m);
  const float2* ks2 = reinterpret_cast<const float2*>(ksv);
  float mx0 = -INFINITY, mx1 = -INFINITY;
  float2 sum_a = make_float2(0.f, 0.f), sum_b = sum_a;
  constexpr int G = 4;                 // pairs per group
  constexpr int NG = kSweepCols / 2 / G;      // groups per row
  float2 x[2][G];
  uint32_t pk[16];
  // exponent arguments of group g -> x[g & 1]
  auto prep = [&](int g, float2 (&xo)[G]) {
    float2 p[G];
#pragma unroll
    for (int u = 0; u < G; ++u) {
      const int i = g * G + u;
      if (FIRST && QK8) p[u] = mul2(make_float2((float)(int)r[2 * i], (float)(int)r[2 * i + 1]), ks2[i]);
      else p[u] = bits2(r[2 * i], r[2 * i + 1]);
    }
    float bv[2 * G];
    if (BIAS) {
      const int gn0 = n_block + 2 * g * G;      // first key of the group (2 * G = 8 keys)
#pragma unroll
      for (int e = 0; e < 2 * G; ++e) bv[e] = 0.f;
      if (bias != nullptr) {
        const VT* bp = bias + (int64_t)gn0 * bias_sn;
        if (bias_sn == 1 && gn0 + 2 * G <= n_len && (reinterpret_cast<uintptr_t>(bp) & 15) == 0) {
          static_assert(G == 4, "one 16-byte load = the 8 keys of a group");
          const uint4 w = __ldg(reinterpret_cast<const uint4*>(bp));
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 t = unpack2<VT>(ww[e]);
            bv[2 * e] = t.x;
            bv[2 * e + 1] = t.y;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 2 * G; ++e)
            if (gn0 + e < n_len) bv[e] = to_f32<VT>(__ldg(bp + (int64_t)e * bias_sn));
        }
      }
    }
    if (FIRST && MASK) {
#pragma unroll
      for (int u = 0; u < G; ++u) {
        p[u] = mul2(p[u], qs2);
        if (BIAS) p[u] = __ffma2_rn(make_float2(bv[2 * u], bv[2 * u + 1]), make_float2(1.4426950408889634f, 1.4426950408889634f), p[u]);
        const int gn = n_block + 2 * (g * G + u);
        const bool v0 = (gn < n_len) && (!causal || gn <= qpos) && (window_left < 0 || gn > qpos - window_left);
        const bool v1 = (gn + 1 < n_len) && (!causal || gn + 1 <= qpos) && (window_left < 0 || gn + 1 > qpos - window_left);
        p[u].x = v0 ? p[u].x : -INFINITY;
        p[u].y = v1 ? p[u].y : -INFINITY;
      }
    }
    if (FIRST) {
#pragma unroll
      for (int u = 0; u < G; u += 2) {
        mx0 = max3f(mx0, p[u].x, p[u].y);
        mx1 = max3f(mx1, p[u + 1].x, p[u + 1].y);
      }
      if (QK8 || MASK) {
#pragma unroll
        for (int u = 0; u < G; ++u) {
          r[2 * (g * G + u)] = __float_as_uint(p[u].x);
          r[2 * (g * G + u) + 1] = __float_as_uint(p[u].y);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < G; ++u) xo[u] = __ffma2_rn(p[u], xs2, neg_m2);
  };
  prep(0, x[0]);
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    float2(&xc)[G] = x[g & 1];
#pragma unroll
    for (int u = 0; u < G; ++u)
      if (!pair_uses_poly(g * G + u)) xc[u] = make_float2(ex2_issue(xc[u].x), ex2_issue(xc[u].y));
#pragma unroll
    for (int u = 0; u < G; ++u)
      if (pair_uses_poly(g * G + u)) xc[u] = exp2_poly_pair(xc[u]);
    if (g + 1 < NG) prep(g + 1, x[(g + 1) & 1]);
#pragma unroll
    for (int u = 0; u < G; u += 2) {
      sum_a = add2(sum_a, xc[u]);
      sum_b = add2(sum_b, xc[u + 1]);
    }
#pragma unroll
    for (int u = 0; u < G; ++u) pk[(g * G + u) & 15] = pack2<VT>(xc[u].x, xc[u].y);
    if (((g + 1) * G) % 16 == 0) tc_st16(t_p + 16 * (((g + 1) * G) / 16 - 1), pk);
  }
  const float2 st = add2(sum_a, sum_b);
  sum = st.x + st.y;
  mx = fmaxf(mx0, mx1);
}

// ---- full-W8A8 mode: P re-quantised to the int8 grid before P.V ----------------------------
// The reference's W8A8 kernel (csrc/include/attn_w8a8_fwd.cuh:150-205) forms, per query row and
// 64-key tile (or per 32-key half of it), p_scale = max(max(P) / 127, 2e-38) and the codes
// P8 = rint(P / p_scale), multiplies the codes with the int8 V tile in int32 and adds
// p_scale * (P8 . V8) to the fp32 output.  Here the same codes are formed, and code * p_scale --
// a value of the int8 grid -- goes to tensor memory as fp16 for a kind::f16 P.V against V's int8
// codes held as fp16 (exact): the products are those of the integer MMA up to the fp16 rounding
// of code * p_scale (2^-11 relative), and no per-tile int32 -> fp32 fold of D columns per row is
// needed.  The row sum l uses the unquantised P, as the reference does.

// First walk: finished multiplicands in r (as softmax_pass FIRST leaves them) and the maximum of
// each 32-key half.
template <bool QK8, bool MASK>
__device__ __forceinline__ void w8_logits_pass(uint32_t (&r)[kSweepCols], const float* __restrict__ ksv, float qs,
                                               int n_block, int n_len, int causal, int qpos, int window_left,
                                               float (&mxh)[2]) {
  const float2 qs2 = make_float2(qs, qs);
  const float2* ks2 = reinterpret_cast<const float2*>(ksv);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int u = 0; u < kSweepCols / 4; ++u) {
      const int i = h * (kSweepCols / 4) + u;
      float2 p = QK8 ? mul2(make_float2((float)(int)r[2 * i], (float)(int)r[2 * i + 1]), ks2[i]) : bits2(r[2 * i], r[2 * i + 1]);
      if (MASK) {
        p = mul2(p, qs2);
        const int gn = n_block + 2 * i;
        const bool v0 = (gn < n_len) && (!causal || gn <= qpos) && (window_left < 0 || gn > qpos - window_left);
        const bool v1 = (gn + 1 < n_len) && (!causal || gn + 1 <= qpos) && (window_left < 0 || gn + 1 > qpos - window_left);
        p.x = v0 ? p.x : -INFINITY;
        p.y = v1 ? p.y : -INFINITY;
      }
      if (u & 1) m1 = max3f(m1, p.x, p.y);
      else m0 = max3f(m0, p.x, p.y);
      r[2 * i] = __float_as_uint(p.x);
      r[2 * i + 1] = __float_as_uint(p.y);
    }
    mxh[h] = fmaxf(m0, m1);
  }
}

// Second walk: P = 2^(r * xs - m), its fp32 row sum, and code * p_scale packed as 16-bit pairs
// into tensor memory.  mxh are the half maxima in r's units; per_half selects one scale per
// 32-key half instead of one per tile.
template <typename VT>
__device__ __forceinline__ void w8_exp_pass(const uint32_t (&r)[kSweepCols], float xs, float neg_m, const float (&mxh)[2],
                                            bool per_half, uint32_t t_p, float& sum) {
  const float2 xs2 = make_float2(xs, xs), neg_m2 = make_float2(neg_m, neg_m);
  float pm0 = ex2_issue(fmaf(mxh[0], xs, neg_m)), pm1 = ex2_issue(fmaf(mxh[1], xs, neg_m));
  if (!per_half) pm0 = pm1 = fmaxf(pm0, pm1);
  const float inv127 = 1.0f / 127.0f;
  constexpr float kRint = 12582912.f;        // 1.5 * 2^23: adding and subtracting it rounds to nearest even
  const float2 rint2 = make_float2(kRint, kRint), nrint2 = make_float2(-kRint, -kRint);
  float2 sum_a = make_float2(0.f, 0.f), sum_b = sum_a;
  constexpr int G = 4;
  uint32_t pk[16];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float ps = fmaxf((h ? pm1 : pm0) * inv127, 2e-38f);
    const float ip = __frcp_rn(ps);
    const float2 ps2 = make_float2(ps, ps), ip2 = make_float2(ip, ip);
#pragma unroll
    for (int g = 0; g < kSweepCols / 4 / G; ++g) {
      float2 e[G];
#pragma unroll
      for (int u = 0; u < G; ++u) {
        const int i = h * (kSweepCols / 4) + g * G + u;
        const float2 x = __ffma2_rn(bits2(r[2 * i], r[2 * i + 1]), xs2, neg_m2);
        e[u] = make_float2(ex2_issue(x.x), ex2_issue(x.y));
      }
#pragma unroll
      for (int u = 0; u < G; u += 2) {
        sum_a = add2(sum_a, e[u]);
        sum_b = add2(sum_b, e[u + 1]);
      }
#pragma unroll
      for (int u = 0; u < G; ++u) {
        const int i = h * (kSweepCols / 4) + g * G + u;
        const float2 code = add2(__ffma2_rn(e[u], ip2, rint2), nrint2);
        const float2 d = mul2(code, ps2);
        pk[i & 15] = pack2<VT>(d.x, d.y);
      }
    }
    tc_st16(t_p + 16 * h, pk);
  }
  const float2 st = add2(sum_a, sum_b);
  sum = st.x + st.y;
}

}  // namespace sl8
