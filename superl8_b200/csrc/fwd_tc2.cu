// Prefill forward, one block per SM: two 128-row query tiles of one (batch, query head) share
// every K / V stage, key tiles are 128 wide, and the block owns all 512 tensor-memory columns
// (S_0, S_1, O_0, O_1).  Same mathematics as fwd_tcgen05.cu (reference
// csrc/include/attn_int8_fwd.cuh:107-208 and csrc/include/attn_fp16_fwd.cuh:89-230); what differs
// is the division of labour:
//
//   warps 0-3 / 4-7   softmax of query tile 0 / 1 (thread = query row).  Per key tile: load the
//                     128 accumulators of the row, pass 1 = conversion, k_scale and row maximum,
//                     decide whether the running maximum moves (only when it grew by more than
//                     2^8: out = O / l does not depend on it) and publish the rescale factor,
//                     pass 2 = exponentials, row sum, P packed to V's dtype over the first 64
//                     columns of the tile's own S buffer -- handed to the issuer in two halves
//                     of 64 keys, so P.V starts while the second half is still being formed; at the
//                     end the warpgroup normalises its O_t by 1 / l and sends it out through TMA stores;
//   warps 8-11        correction: multiply O_t by the published factor when some row of the
//                     warp moved its maximum (rare) and tell the issuer that O_t is ready;
//   warp 12           issuer: S_t = Q_t.K_j^T (kind::i8 or kind::f16, M128 N128: full rate) and
//                     O_t += P_t.V_j (kind::f16, P from tensor memory), in the order
//                     P.V_0(j), Q.K_0(j+1), P.V_1(j), Q.K_1(j+1): while one tile's softmax works,
//                     the tensor pipe runs the other tile's products;
//   warp 13           producer: barrier set-up and the first copies before the block-wide sync, then TMA
//                     loads of K and V (two stages each) and, in int8 mode, the k_scale tiles (ring
//                     of four, three tiles ahead);
//   warps 14-15       none (they pad the last warpgroup).
// Registers move between the warpgroups after launch (setmaxnreg): the softmax warpgroups hold
// a whole 128-column row per thread.  Every mbarrier wait is bounded; on expiry the block
// raises the status word, frees tensor memory and exits.
#include "sl8_fwd_tc2.cuh"
#include "sl8_softmax.cuh"

#include <type_traits>

namespace sl8 {
namespace {

constexpr int kQT = 128;          // rows per query tile (two tiles per block)
constexpr int kKT = 128;          // keys per tile
constexpr int kThreads2 = 512;
constexpr int kCorrWarp0 = 8, kMmaWarp2 = 12, kProdWarp2 = 13;
constexpr int kKsStages = 4;
constexpr int kRegsSoftmax = 184, kRegsCorrection = 80, kRegsOther = 64;

template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

template <int D, bool QK8>
struct Cfg2 {
  static constexpr int QK_ROWB = D * (QK8 ? 1 : 2);
  static constexpr int QROW = QK_ROWB < 128 ? QK_ROWB : 128;
  static constexpr int QSUBS = QK_ROWB / QROW;
  static constexpr uint32_t QK_SW = QROW == 128 ? kUmmaSw128 : kUmmaSw64;
  static constexpr int Q_SUB_BYTES = kQT * QROW, Q_TILE_BYTES = kQT * QK_ROWB;
  static constexpr int K_SUB_BYTES = kKT * QROW, K_TILE_BYTES = kKT * QK_ROWB;
  static constexpr int QK_STEPS = QK_ROWB / 32;
  static constexpr int VSUBS = 2 * D / 128;
  static constexpr int V_SUB_BYTES = kKT * 128, V_TILE_BYTES = kKT * 2 * D;
  static constexpr int O_TILE_BYTES = kQT * 2 * D;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * Q_TILE_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * K_TILE_BYTES;
  // output staging: its own buffer when a Q tile is too small to hold an output tile
  static constexpr bool STAGE_IN_Q = Q_TILE_BYTES >= O_TILE_BYTES;
  static constexpr int OFF_STAGE = OFF_V + 2 * V_TILE_BYTES;
  static constexpr int OFF_KS = OFF_STAGE + (STAGE_IN_Q ? 0 : 2 * O_TILE_BYTES);
  static constexpr int OFF_SC = OFF_KS + (QK8 ? kKsStages * kKT * 4 : 0);   // rescale factors [2][128]
  static constexpr int OFF_BAR = OFF_SC + 2 * kQT * 4;
  static constexpr int SMEM = OFF_BAR + 512 + 1024;
  static_assert(SMEM <= 232448, "exceeds the shared memory of one block");
  static constexpr uint32_t COL_S = 0, COL_O = 256;   // S_t at 128 t, O_t at 256 + 128 t
  static_assert(D <= 128, "two output accumulators must fit 256 columns");
};

enum Bar2 {
  Q_FULL = 0,
  K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7,          // per stage
  S_FULL = 9, PA_FULL = 11, PB_FULL = 13, SC_READY = 15, PV_DONE = 17, O_DONE = 19,   // per query tile
  KS_EMPTY = 21, NUM_BARS2 = KS_EMPTY + kKsStages
};

// float(acc) for |acc| < 2^22 (an int8 dot product over D <= 256 stays below 127^2 * 256 < 2^22) without the
// conversion instruction, which shares the special-function unit with the exponentials:
// the integer acc + 0x4B400000 IS the float 1.5 * 2^23 + acc, and subtracting 1.5 * 2^23 is exact.
__device__ __forceinline__ float2 i2f_pair(uint32_t a, uint32_t b) {
  const float2 f = make_float2(__uint_as_float(a + 0x4B400000u), __uint_as_float(b + 0x4B400000u));
  return __fadd2_rn(f, make_float2(-12582912.f, -12582912.f));
}

// ---- softmax passes over one row of 128 accumulators ------------------------------------------
// pass 1: int8 mode t = float(acc) * k_scale[n] (left in r), 16-bit mode t = acc; returns max t.
template <bool QK8>
__device__ __forceinline__ float pass1_plain(uint32_t (&r)[kKT], const float* __restrict__ ksv) {
  const float2* ks2 = reinterpret_cast<const float2*>(ksv);
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < kKT / 2; i += 2) {
    float2 p0, p1;
    if (QK8) {
      p0 = mul2(i2f_pair(r[2 * i], r[2 * i + 1]), ks2[i]);
      p1 = mul2(i2f_pair(r[2 * i + 2], r[2 * i + 3]), ks2[i + 1]);
      r[2 * i] = __float_as_uint(p0.x); r[2 * i + 1] = __float_as_uint(p0.y);
      r[2 * i + 2] = __float_as_uint(p1.x); r[2 * i + 3] = __float_as_uint(p1.y);
    } else {
      p0 = bits2(r[2 * i], r[2 * i + 1]);
      p1 = bits2(r[2 * i + 2], r[2 * i + 3]);
    }
    mx0 = max3f(mx0, p0.x, p0.y);
    mx1 = max3f(mx1, p1.x, p1.y);
  }
  return fmaxf(mx0, mx1);
}
// pass 1 on a tile that needs masking (diagonal or tail): leaves the finished logits
// t * qs (int8: float(acc) * k_scale * q_scale), -inf where masked; returns their max.
template <bool QK8>
__device__ __forceinline__ float pass1_masked(uint32_t (&r)[kKT], const float* __restrict__ ksv, float qs, int n_block,
                                              int n_len, int causal, int qpos) {
  const float2* ks2 = reinterpret_cast<const float2*>(ksv);
  const float2 qs2 = make_float2(qs, qs);
  float mx0 = -INFINITY, mx1 = -INFINITY;
  const int lim = causal ? min(n_len - 1, qpos) : n_len - 1;   // last visible key of this row
#pragma unroll
  for (int i = 0; i < kKT / 2; ++i) {
    float2 p;
    if (QK8) p = mul2(i2f_pair(r[2 * i], r[2 * i + 1]), ks2[i]);
    else p = bits2(r[2 * i], r[2 * i + 1]);
    p = mul2(p, qs2);
    const int gn = n_block + 2 * i;
    p.x = (gn <= lim) ? p.x : -INFINITY;
    p.y = (gn + 1 <= lim) ? p.y : -INFINITY;
    r[2 * i] = __float_as_uint(p.x);
    r[2 * i + 1] = __float_as_uint(p.y);
    if (i & 1) mx1 = max3f(mx1, p.x, p.y);
    else mx0 = max3f(mx0, p.x, p.y);
  }
  return fmaxf(mx0, mx1);
}
// pass 2 on columns [OFF, OFF + 64): P = 2^(r * xs - m) packed to VT into 32 tensor-memory
// columns at t_p; returns the fp32 row sum of the half.
template <int OFF, typename VT>
__device__ __forceinline__ float pass2_half(const uint32_t (&r)[kKT], float xs, float neg_m, uint32_t t_p) {
  const float2 xs2 = make_float2(xs, xs), nm2 = make_float2(neg_m, neg_m);
  float2 sa = make_float2(0.f, 0.f), sb = sa;
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    uint32_t pk[16];
#pragma unroll
    for (int u = 0; u < 16; u += 2) {
      const int i = OFF / 2 + 16 * g + u;
      float2 x0 = __ffma2_rn(bits2(r[2 * i], r[2 * i + 1]), xs2, nm2);
      float2 x1 = __ffma2_rn(bits2(r[2 * i + 2], r[2 * i + 3]), xs2, nm2);
      x0 = make_float2(ex2_approx(x0.x), ex2_approx(x0.y));
      x1 = make_float2(ex2_approx(x1.x), ex2_approx(x1.y));
      sa = add2(sa, x0);
      sb = add2(sb, x1);
      pk[u] = pack2<VT>(x0.x, x0.y);
      pk[u + 1] = pack2<VT>(x1.x, x1.y);
    }
    tc_st16(t_p + 16 * g, pk);
  }
  const float2 s = add2(sa, sb);
  return s.x + s.y;
}

SL8_TRACE_DEFINE()

template <int D, typename VT, bool QK8>
__global__ void __launch_bounds__(kThreads2, 1) fwd_tc2_kernel(const __grid_constant__ CUtensorMap q_map,
                                                               const __grid_constant__ CUtensorMap k_map,
                                                               const __grid_constant__ CUtensorMap v_map,
                                                               const __grid_constant__ CUtensorMap o_map, Tc2Args a) {
  using C = Cfg2<D, QK8>;
  if (a.gate_flag != nullptr && ((__ldg(a.gate_flag) != 0) != (a.gate_want != 0))) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* ks_smem = reinterpret_cast<float*>(smem + C::OFF_KS);
  float* sc_smem = reinterpret_cast<float*>(smem + C::OFF_SC);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t bh = blockIdx.y;
  const int b = (int)(bh / a.Hq);
  const int G = a.Hq / a.Hkv;
  const int kv_bh = b * a.Hkv + (int)(bh % a.Hq) / G;
  const int m_len = a.seqlens_q ? min(max(a.seqlens_q[b], 0), a.M) : a.M;
  const int n_len = a.seqlens_k ? min(max(a.seqlens_k[b], 0), a.N) : a.N;
  const int m_block = (a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x) * (2 * kQT);   // heavy blocks first
  const int diag = a.causal ? n_len - m_len : 0;
  // key tiles of query tile t (rows m_block + 128 t ...): none when the tile lies past the sequence
  int nt[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int m0 = m_block + kQT * t;
    const int n_end = a.causal ? max(0, min(n_len, m0 + kQT + diag)) : n_len;
    nt[t] = (m0 < m_len) ? (n_end + kKT - 1) / kKT : 0;
  }
  const int n_max = max(nt[0], nt[1]);
  VT* const ob = reinterpret_cast<VT*>(a.out) + bh * (int64_t)a.M * D;

  if (n_max == 0) {   // no visible key for any row (or only padded rows): zeros
    for (int idx = threadIdx.x; idx < 2 * kQT * (D / 8); idx += kThreads2) {
      const int r = idx / (D / 8), c = (idx % (D / 8)) * 8;
      if (m_block + r < a.M) *reinterpret_cast<uint4*>(ob + (int64_t)(m_block + r) * D + c) = make_uint4(0, 0, 0, 0);
    }
    if (a.lse) for (int r = threadIdx.x; r < 2 * kQT; r += kThreads2)
        if (m_block + r < a.M) a.lse[bh * a.M + m_block + r] = -INFINITY;
    return;
  }

  if (threadIdx.x == 0) {
    TR(8188);
    TRV(8191, (long long)sl8_smid());
  }
  if (warp == kProdWarp2 && lane == 0) {
    // the producer's lane initialises the barriers and starts the first copies at once: Q, and the
    // first two K / V tiles (their stages are free), while the rest of the block is still setting up
    mbar_init(&bars[Q_FULL], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[K_FULL + i], 1);
      mbar_init(&bars[K_EMPTY + i], 1);
      mbar_init(&bars[V_FULL + i], 1);
      mbar_init(&bars[V_EMPTY + i], 1);
      mbar_init(&bars[S_FULL + i], QK8 ? 2 : 1);     // the MMA commit (+ the k_scale tile in int8 mode)
      mbar_init(&bars[PA_FULL + i], 8);              // four softmax warps (first half of P) + four correction warps (O ready)
      mbar_init(&bars[PB_FULL + i], 4);
      mbar_init(&bars[SC_READY + i], 4);
      mbar_init(&bars[PV_DONE + i], 1);
      mbar_init(&bars[O_DONE + i], 1);
    }
    // every softmax warpgroup that has key tiles releases each k_scale stage once per key tile
    for (int i = 0; i < kKsStages; ++i) mbar_init(&bars[KS_EMPTY + i], 4 * ((nt[0] > 0) + (nt[1] > 0)));
    mbar_fence_init();
    constexpr int es = QK8 ? 1 : 2;
    tma_prefetch_desc(&q_map);
    tma_prefetch_desc(&k_map);
    tma_prefetch_desc(&v_map);
    mbar_expect_tx(&bars[Q_FULL], 2 * C::Q_TILE_BYTES);
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int c = 0; c < C::QSUBS; ++c)
        tma_load_3d(smem + C::OFF_Q + t * C::Q_TILE_BYTES + c * C::Q_SUB_BYTES, &q_map, &bars[Q_FULL],
                    c * (C::QROW / es), m_block + kQT * t, (int)bh);
    for (int j = 0; j < 2 && j < n_max; ++j) {
      mbar_expect_tx(&bars[K_FULL + j], C::K_TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::QSUBS; ++c)
        tma_load_3d(smem + C::OFF_K + j * C::K_TILE_BYTES + c * C::K_SUB_BYTES, &k_map, &bars[K_FULL + j],
                    c * (C::QROW / es), j * kKT, kv_bh);
      if (j == 0) {
        mbar_expect_tx(&bars[V_FULL + j], C::V_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::VSUBS; ++c)
          tma_load_3d(smem + C::OFF_V + j * C::V_TILE_BYTES + c * C::V_SUB_BYTES, &v_map, &bars[V_FULL + j], c * 64,
                      j * kKT, kv_bh);
      }
    }
  }
  if (warp == kMmaWarp2) {
    tc_alloc(tmem_slot, 512);
    tc_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  bool ok = true;
  if (threadIdx.x == 0) TR(8189);

  if (warp >= kMmaWarp2) {
    reg_dec<kRegsOther>();
    if (warp == kProdWarp2) {
      // ======================= producer =======================
      constexpr int es = QK8 ? 1 : 2;
      auto fetch_ks = [&](int j, float (&dst)[kKT / 32]) {
#pragma unroll
        for (int i = 0; i < kKT / 32; ++i) {
          const int n = j * kKT + lane + 32 * i;
          dst[i] = (QK8 && j < n_max && n < n_len) ? __ldg(a.k_scale + (int64_t)kv_bh * a.N + n) : 0.f;
        }
      };
      float ks0[kKT / 32], ks1[kKT / 32], ks2[kKT / 32];
      fetch_ks(0, ks0);
      fetch_ks(1, ks1);
      fetch_ks(2, ks2);
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) - 1) & 1;
        if (lane == 0 && j >= 2) {   // K_0 and K_1 are already on their way
          ok = mbar_wait(&bars[K_EMPTY + st], par, a.status);
          if (ok) {
            mbar_expect_tx(&bars[K_FULL + st], C::K_TILE_BYTES);
#pragma unroll
            for (int c = 0; c < C::QSUBS; ++c)
              tma_load_3d(smem + C::OFF_K + st * C::K_TILE_BYTES + c * C::K_SUB_BYTES, &k_map, &bars[K_FULL + st],
                          c * (C::QROW / es), j * kKT, kv_bh);
          }
        }
        if (lane == 0 && ok && j >= 1) {   // V_0 is already on its way
          if (j >= 2) ok = mbar_wait(&bars[V_EMPTY + st], par, a.status);
          if (ok) {
            mbar_expect_tx(&bars[V_FULL + st], C::V_TILE_BYTES);
#pragma unroll
            for (int c = 0; c < C::VSUBS; ++c)
              tma_load_3d(smem + C::OFF_V + st * C::V_TILE_BYTES + c * C::V_SUB_BYTES, &v_map, &bars[V_FULL + st],
                          c * 64, j * kKT, kv_bh);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (QK8 && ok) {
          // k_scale tile j.  Its arrival completes S_FULL[t] together with the commit of Q_t.K_j^T, so it
          // must not land before the barrier's previous phase (tile j - 1) has completed.
          const int ss = j % kKsStages;
          if (j >= kKsStages) ok = mbar_wait(&bars[KS_EMPTY + ss], ((j / kKsStages) - 1) & 1, a.status);
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (ok && j >= 1 && j < nt[t]) ok = mbar_wait(&bars[S_FULL + t], (j - 1) & 1, a.status);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
#pragma unroll
          for (int i = 0; i < kKT / 32; ++i) {
            ks_smem[ss * kKT + lane + 32 * i] = ks0[i];
            ks0[i] = ks1[i];
            ks1[i] = ks2[i];
          }
          fetch_ks(j + 3, ks2);
          __syncwarp();
          if (lane == 0) {
            if (j < nt[0]) mbar_arrive(&bars[S_FULL + 0]);
            if (j < nt[1]) mbar_arrive(&bars[S_FULL + 1]);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    } else if (warp == kMmaWarp2) {
      // ======================= MMA issuer =======================
      constexpr uint32_t vfmt = std::is_same<VT, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc_qk = QK8 ? umma_idesc(2, 1, 1, 0, 0, kQT, kKT) : umma_idesc(1, vfmt, vfmt, 0, 0, kQT, kKT);
      const uint32_t idesc_pv = umma_idesc(1, vfmt, vfmt, 0, 1, kQT, D);
      const uint64_t dq = umma_smem_desc(smem_u32(smem + C::OFF_Q), 16, 8 * C::QROW, C::QK_SW);
      const uint64_t dk = umma_smem_desc(smem_u32(smem + C::OFF_K), 16, 8 * C::QROW, C::QK_SW);
      const uint64_t dv = umma_smem_desc(smem_u32(smem + C::OFF_V), C::V_SUB_BYTES, 1024, kUmmaSw128);
      // S_t = Q_t . K_j^T; the K stage was waited for by the caller
      auto issue_qk = [&](int t, int j) {
        if (elect_one()) {
          const int st = j & 1;
#pragma unroll
          for (int s = 0; s < C::QK_STEPS; ++s) {
            const uint32_t sub = 32 * s / C::QROW, within = 32 * s % C::QROW;
            const uint64_t da = umma_desc_advance(dq, t * C::Q_TILE_BYTES + sub * C::Q_SUB_BYTES + within);
            const uint64_t db = umma_desc_advance(dk, st * C::K_TILE_BYTES + sub * C::K_SUB_BYTES + within);
            if (QK8) tc_mma_i8_ss(tmem + C::COL_S + kKT * t, da, db, idesc_qk, s > 0 ? 1u : 0u);
            else tc_mma_f16_ss(tmem + C::COL_S + kKT * t, da, db, idesc_qk, s > 0 ? 1u : 0u);
          }
          tc_commit(&bars[S_FULL + t]);
          // the last product that reads K_j frees its stage
          const bool last_user = (t == 1) || (j >= nt[1]);
          if (last_user) tc_commit(&bars[K_EMPTY + st]);
        }
        __syncwarp();
      };
      ok = __all_sync(0xffffffffu, mbar_wait(&bars[Q_FULL], 0, a.status));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars[K_FULL + 0], 0, a.status));
      // The two query tiles work best half a period apart (one tile's softmax under the other's
      // products): tile 1's first product is held back until tile 0's first half of P has gone
      // into P.V, instead of being queued right behind Q_0.K_0^T.
      const bool skew = nt[0] > 0 && nt[1] > 0;
      if (ok) {
        tc_fence_after();
        if (nt[0] > 0) issue_qk(0, 0);
        if (nt[1] > 0 && !skew) issue_qk(1, 0);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j & 1;
        const uint32_t par = j & 1;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= nt[t] || !ok) continue;
          TR(4096 + 16 * j + 8 * t + 0);
          // first half of P_t (and O_t rescaled if it had to be)
          ok = __all_sync(0xffffffffu, mbar_wait(&bars[PA_FULL + t], par, a.status));
          if (ok && (t == 0 || j >= nt[0])) ok = __all_sync(0xffffffffu, mbar_wait(&bars[V_FULL + st], (j >> 1) & 1, a.status));
          if (!ok) break;
          TR(4096 + 16 * j + 8 * t + 1);
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < kKT / 32; ++kk)
              tc_mma_f16_ts(tmem + C::COL_O + D * t, tmem + C::COL_S + kKT * t + 8 * kk,
                            umma_desc_advance(dv, st * C::V_TILE_BYTES + kk * 2048), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          }
          __syncwarp();
          if (skew && j == 0 && t == 0) issue_qk(1, 0);
          ok = __all_sync(0xffffffffu, mbar_wait(&bars[PB_FULL + t], par, a.status));
          if (!ok) break;
          TR(4096 + 16 * j + 8 * t + 2);
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = kKT / 32; kk < kKT / 16; ++kk)
              tc_mma_f16_ts(tmem + C::COL_O + D * t, tmem + C::COL_S + kKT * t + 8 * kk,
                            umma_desc_advance(dv, st * C::V_TILE_BYTES + kk * 2048), idesc_pv, 1u);
            tc_commit(&bars[PV_DONE + t]);
            const bool last_user = (t == 1) || (j >= nt[1]);
            if (last_user) tc_commit(&bars[V_EMPTY + st]);
            if (j == nt[t] - 1) tc_commit(&bars[O_DONE + t]);
          }
          __syncwarp();
          if (j + 1 < nt[t]) {
            // K_{j+1}: waited once per key tile (by the first query tile that uses it)
            const bool first_user = (t == 0) || (j + 1 >= nt[0]);
            if (first_user) ok = __all_sync(0xffffffffu, mbar_wait(&bars[K_FULL + ((j + 1) & 1)], ((j + 1) >> 1) & 1, a.status));
            if (!ok) break;
            tc_fence_after();
            issue_qk(t, j + 1);
          }
          TR(4096 + 16 * j + 8 * t + 3);
        }
      }
    }
  } else if (warp >= kCorrWarp0) {
    reg_dec<kRegsCorrection>();
    // ======================= correction + epilogue =======================
    const int w = warp - kCorrWarp0;                     // tensor-memory lanes [32 w, 32 w + 32) of both tiles
    const uint32_t t_row = tmem + ((uint32_t)(32 * w) << 16);
    for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (j >= nt[t] || !ok) continue;
        ok = mbar_wait(&bars[SC_READY + t], j & 1, a.status);
        if (!ok) break;
        const float sc = sc_smem[t * kQT + 32 * w + lane];
        if (j > 0 && __any_sync(0xffffffffu, sc != 1.f)) {
          ok = mbar_wait(&bars[PV_DONE + t], (j - 1) & 1, a.status);   // O_t holds every product up to tile j - 1
          if (!ok) break;
          tc_fence_after();
          const float2 sc2 = make_float2(sc, sc);
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tc_ld32(t_row + C::COL_O + D * t + 32 * c, o);
            tc_wait_ld();
            tc_regs_ready(o);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 x = __fmul2_rn(bits2(o[2 * i], o[2 * i + 1]), sc2);
              o[2 * i] = __float_as_uint(x.x);
              o[2 * i + 1] = __float_as_uint(x.y);
            }
            tc_st32(t_row + C::COL_O + D * t + 32 * c, o);
          }
          tc_wait_st();
          tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[PA_FULL + t]);
      }
    }
    tc_fence_before();
  } else {
    reg_inc<kRegsSoftmax>();
    // ======================= softmax =======================
    const int t = warp >> 2, w = warp & 3;
    const int row = 32 * w + lane;
    const int m0 = m_block + kQT * t;
    const int m = m0 + row;
    const float qs = QK8 ? ((m < m_len) ? __ldg(a.q_scale + bh * a.M + m) : 0.f) : a.scale_log2;
    const int qpos = m + diag;
    const uint32_t t_s = tmem + ((uint32_t)(32 * w) << 16) + C::COL_S + kKT * t;
    const int my_nt = nt[t];
    float m_run = -INFINITY, l_run = 0.f;
    for (int j = 0; j < n_max && my_nt > 0; ++j) {
      const int ss = j % kKsStages;
      if (j >= my_nt) {   // the other query tile has one more key tile: only release its k_scale stage
        if (QK8) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[KS_EMPTY + ss]);
        }
        continue;
      }
      const int n_block = j * kKT;
      if (w == 0 && lane == 0) TR(16 * j + 8 * t + 0);
      ok = mbar_wait(&bars[S_FULL + t], j & 1, a.status);
      if (!ok) break;
      tc_fence_after();
      if (w == 0 && lane == 0) TR(16 * j + 8 * t + 1);
      uint32_t r[kKT];
#pragma unroll
      for (int c = 0; c < kKT / 32; ++c) tc_ld32(t_s + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
      tc_wait_ld();
#pragma unroll
      for (int c = 0; c < kKT / 32; ++c) tc_regs_ready(*reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
      if (w == 0 && lane == 0) TR(16 * j + 8 * t + 5);
      const float* ksv = ks_smem + ss * kKT;
      const bool need_mask = (n_block + kKT > n_len) || (a.causal && n_block + kKT - 1 > m0 + diag);
      float tmax;
      if (need_mask) tmax = pass1_masked<QK8>(r, ksv, qs, n_block, n_len, a.causal, qpos);
      else tmax = pass1_plain<QK8>(r, ksv) * qs;
      const float xs = need_mask ? 1.f : qs;
      if (QK8) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[KS_EMPTY + ss]);
      }
      if (w == 0 && lane == 0) TR(16 * j + 8 * t + 2);
      // the running maximum moves only when the row outgrew it by more than 2^8
      float sc = 1.f;
      if (m_run == -INFINITY) {
        m_run = tmax;
      } else if (tmax > m_run + kLazyRescaleLog2) {
        sc = exp2f(m_run - tmax);
        m_run = tmax;
      }
      sc_smem[t * kQT + row] = sc;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[SC_READY + t]);
      if (w == 0 && lane == 0) TR(16 * j + 8 * t + 6);
      const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
      float psum = pass2_half<0, VT>(r, xs, neg_m, t_s);
      if (w == 0 && lane == 0) TR(16 * j + 8 * t + 7);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[PA_FULL + t]);
      if (w == 0 && lane == 0) TR(16 * j + 8 * t + 3);
      psum += pass2_half<kKT / 2, VT>(r, xs, neg_m, t_s + kKT / 4);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[PB_FULL + t]);
      l_run = l_run * sc + psum;
      if (w == 0 && lane == 0) TR(16 * j + 8 * t + 4);
    }
    // ---- epilogue of this warpgroup's tile: O_t / l -> shared memory (128-byte-swizzled) -> TMA store ----
    if (my_nt > 0) {
      if (w == 0 && lane == 0) TR(8176 + 4 * t);
      if (ok) ok = mbar_wait(&bars[O_DONE + t], 0, a.status);
      if (ok) {
        tc_fence_after();
        if (w == 0 && lane == 0) TR(8177 + 4 * t);
        if (lane == 0) tma_prefetch_desc(&o_map);
        const float inv = (m < m_len && l_run > 0.f) ? 1.f / l_run : 0.f;
        uint8_t* const tile = smem + (C::STAGE_IN_Q ? C::OFF_Q + t * C::Q_TILE_BYTES : C::OFF_STAGE + t * C::O_TILE_BYTES);
        uint8_t* const stage = tile + w * (32 * 128) + lane * 128;
        const uint32_t t_o = tmem + ((uint32_t)(32 * w) << 16) + C::COL_O + D * t;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tc_ld32(t_o + 32 * c, o);
          tc_wait_ld();
          tc_regs_ready(o);
          uint8_t* const sub = stage + (c >> 1) * (kQT * 128);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 x;
            x.x = pack2<VT>(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
            x.y = pack2<VT>(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
            x.z = pack2<VT>(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
            x.w = pack2<VT>(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
            *reinterpret_cast<uint4*>(sub + ((((c & 1) * 4 + v) ^ (lane & 7)) << 4)) = x;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && m0 + 32 * w < a.M) {
#pragma unroll
          for (int sb = 0; sb < D / 64; ++sb)
            tma_store_3d(&o_map, tile + sb * (kQT * 128) + w * (32 * 128), 64 * sb, m0 + 32 * w, (int)bh);
          tma_store_commit();
          tma_store_wait_read();
        }
        __syncwarp();
        if (w == 0 && lane == 0) TR(8178 + 4 * t);
        if (a.lse != nullptr && m < a.M)
          a.lse[bh * a.M + m] = (m < m_len && l_run > 0.f) ? (m_run * 0.6931471805599453f + logf(l_run)) : -INFINITY;
      }
    } else if (m0 < a.M && m < a.M) {   // padded rows of the batch (beyond seqlens_q) or no visible key: zeros
      uint4* dst = reinterpret_cast<uint4*>(ob + (int64_t)m * D);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) dst[c] = make_uint4(0, 0, 0, 0);
      if (a.lse != nullptr) a.lse[bh * a.M + m] = -INFINITY;
    }
    tc_fence_before();
  }

  // ---- teardown: every role arrives here, on success and on a timed-out wait ----
  __syncthreads();
  if (threadIdx.x == 0) TR(8187);
  if (warp == kMmaWarp2) {
    tc_fence_after();
    tc_dealloc(tmem, 512);
  }
}

template <int D, typename VT, bool QK8>
int launch_tc2(const Tc2Args& a, cudaStream_t stream) {
  using C = Cfg2<D, QK8>;
  constexpr int es = QK8 ? 1 : 2;
  CUtensorMap q_map, k_map, v_map, o_map;
  int rc = sl8_make_tmap_3d(&q_map, a.q, es, D, a.M, (uint64_t)a.B * a.Hq, C::QROW / es, kQT, C::QROW);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&k_map, a.k, es, D, a.N, (uint64_t)a.B * a.Hkv, C::QROW / es, kKT, C::QROW);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&v_map, a.v, 2, D, a.N, (uint64_t)a.B * a.Hkv, 64, kKT, 128);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&o_map, a.out, 2, D, a.M, (uint64_t)a.B * a.Hq, 64, 32, 128);
  if (rc != SL8_OK) return rc;
  SL8_CUDA_TRY(cudaFuncSetAttribute(fwd_tc2_kernel<D, VT, QK8>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
  dim3 grid((a.M + 2 * kQT - 1) / (2 * kQT), (unsigned)((int64_t)a.B * a.Hq));
  fwd_tc2_kernel<D, VT, QK8><<<grid, kThreads2, C::SMEM, stream>>>(q_map, k_map, v_map, o_map, a);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

}  // namespace

bool sl8_fwd_tc2_supported(int D, int window_left, bool packed) { return D == 128 && window_left < 0 && !packed; }

int sl8_fwd_tc2(const Tc2Args& a, cudaStream_t stream) {
  if (a.D != 128) return SL8_ERR_UNSUPPORTED;
  if (a.qk8) return a.v_bf16 ? launch_tc2<128, __nv_bfloat16, true>(a, stream) : launch_tc2<128, __half, true>(a, stream);
  return a.v_bf16 ? launch_tc2<128, __nv_bfloat16, false>(a, stream) : launch_tc2<128, __half, false>(a, stream);
}

}  // namespace sl8

#ifdef SL8_TRACE
extern "C" int sl8_dbg_read_trace2(long long* host_out, int n) {
  return (int)cudaMemcpyFromSymbol(host_out, sl8::g_trace, sizeof(long long) * n);
}
#endif
