// Prefill forward on the Blackwell tensor-core path: TMA-staged Q/K/V tiles,
// S = Q.K^T as tcgen05.mma (kind::i8 with an int32 accumulator for the int8 path,
// kind::f16 for the full-precision sibling the accuracy gate demotes to) into tensor
// memory, fp32 online softmax on the CUDA cores, O += P.V as tcgen05.mma kind::f16
// with P read from tensor memory and V from shared memory.
//
// Mathematics are the reference's (csrc/include/attn_int8_fwd.cuh:107-208 and
// csrc/include/attn_fp16_fwd.cuh:89-230):
//   int8:   s = float(int32 q.k) * q_scale[m] * k_scale[n]     (that multiply order)
//   16-bit: s = (q.k) * softmax_scale * log2(e)
//   valid = n < N and (not causal or n <= m + N - M) and (window < 0 or n > pos - window)
//   online softmax in the exp2 domain (fp32 m, l), out = O / l (0 if l == 0),
//   lse = m * ln2 + ln l.
// Differences a caller can observe only inside the tolerance: tiles are 128 x 64
// (reference 64 x 64); the running max moves lazily (only when a row outgrows it by
// more than 2^8; out = O / l does not depend on it); P is rounded to V's dtype before
// P.V (reference fp32); the int8 logit is (float(acc) * k_scale) * q_scale (reference:
// q_scale first), so that scale and max subtraction are one fused multiply-add.
//
// Block = one 128-row query tile of one (batch, query head).  Six warps:
//   warps 0-3  softmax + correction + epilogue; warp w owns tensor-memory lanes
//              [32w, 32w+32) = query rows, one row per thread (no shuffles).  A tile is
//              one sweep over its 64 columns (softmax_pass): conversion, max, exponent
//              and 2^x of neighbouring column groups are interleaved by hand, P is formed
//              against the running max while the tile's own max is still being collected,
//              and only when the max has to move (first tile, rarely later) is O corrected
//              and P formed again;
//   warp 4     producer: TMA loads of Q, K and V (two stages each, K two tiles ahead;
//              the barriers the issuer commits behind QK_t and P.V_j also free the K
//              and V stages) -- 3-D tensor maps, 128-byte swizzle, zero fill past the
//              end of a head -- and the k_scale tiles (ring of four, three tiles ahead);
//              its arrival for a k_scale tile goes to the same barrier as the commit of
//              that tile's QK, so the softmax warps wait once per tile;
//   warp 5     allocates tensor memory; the whole warp walks the issue loop and polls the
//              barriers, one elected lane issues the MMAs and commits, in the order
//              QK_0, QK_1, then for each tile j: P.V_j, QK_{j+2}.
// Tensor memory (256 columns): S in two buffers of 64 columns (the logits of the next
// tile are ready while the softmax warps work on this one); P overwrites the first 32
// columns of its own S buffer as packed 16-bit pairs; O (fp32) at [128, 128 + D).
// Two blocks share an SM, so one block's softmax overlaps the other's MMAs.
// Every mbarrier wait is bounded (sl8_common.cuh); on expiry the block raises the
// workspace status word, frees tensor memory and exits.
//
// Template modes of the same kernel:
//   PACKED  token-major packed tensors [tokens, heads, D] with cu_seqlens (the variable-length
//           prefill, reference csrc/include/attn_varlen_fwd.cuh:25-190);
//   W8      full W8A8 (reference csrc/include/attn_w8a8_fwd.cuh:93-222): V holds int8 codes as
//           fp16, P is snapped to the reference's int8 grid per row and tile (or 32-key half)
//           before it is packed, v_scale multiplies the output channels in the epilogue;
//   BIAS    16-bit mode with the additive mask of the full-precision forward (reference
//           csrc/include/attn_fp16_fwd.cuh:176-178): every tile takes the finished-logits sweep
//           and each thread adds its own query row's bias values.
#include "sl8_common.cuh"
#include "sl8_fwd_tc2.cuh"
#include "sl8_softmax.cuh"

#include <algorithm>
#include <type_traits>

int sl8_fwd_mma_int8(const sl8_fwd_params* p, cudaStream_t s);  // fwd_mma.cu
int sl8_fwd_mma_int8_varlen(const sl8_varlen_params* p, cudaStream_t s);  // fwd_mma.cu

namespace sl8 {
namespace {

constexpr int kTM = 128;                               // query rows per block
constexpr int kTN = 64;                                // keys per tile
static_assert(kTN == kSweepCols, "one softmax sweep per key tile");
constexpr int kSoftmaxWarps = 4;                       // warp w owns tensor-memory lanes [32 w, 32 w + 32)
constexpr int kProducerWarp = kSoftmaxWarps, kMmaWarp = kSoftmaxWarps + 1;
// Build option, off: a block of two full warpgroups (two idle warps behind the producer and the
// issuer) whose second warpgroup hands registers to the softmax warpgroup after launch
// (setmaxnreg: 128 per thread at launch, then 192 / 64 -- the producer and issuer code does not
// fit in 56; the instruction has to sit INSIDE each role's branch, or ptxas allocates every role
// within the launch bound and spills kilobytes), so that the softmax threads of the int8
// instantiation can carry accumulators across tiles without spilling.  Measured on the B = 4 slice
// of the S = 8192 causal workload: int8 with the early load 4.00-4.04 -> 4.18 ms (the early load
// does not pay in int8 mode even with the registers for it), 16-bit 4.08-4.15 -> 3.96-4.08 ms
// (inside the run-to-run spread).
#ifndef SL8_WG_REGS
#define SL8_WG_REGS 0
#endif
constexpr bool kWgRegs = SL8_WG_REGS != 0;
constexpr int kTcThreads = kWgRegs ? 256 : 32 * (kSoftmaxWarps + 2);
constexpr int kRegsSoftmax = 192, kRegsOther = 64;
static_assert(!kWgRegs || 128 * kRegsSoftmax + 128 * kRegsOther <= 256 * 128, "the block's register pool");
template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
constexpr int kScaleStages = 4;                        // ring of k_scale tiles
// 16-bit mode loads the next tile's logits at the end of a tile (see EARLY in the kernel): measured
// + 4 % on the S = 8192 causal workload, burst and sustained alike (18.37 -> 17.67 ms for the full
// batch).  In int8 mode the same change LOSES (SL8_EARLY_LOAD=2 builds it: B = 4 slice 4.05 -> 4.49 ms
// with all 64 accumulators carried, 4.05 -> 4.75 ms with the first 32): that instantiation sits at the
// register limit of two blocks per SM and spills what it carries across the loop's back edge.
// SL8_EARLY_LOAD=0 builds without any of it.
#ifndef SL8_EARLY_LOAD
#define SL8_EARLY_LOAD 1
#endif
constexpr bool kEarlyLoad = SL8_EARLY_LOAD != 0;
#ifndef SL8_QK_PAIR
#define SL8_QK_PAIR 0
#endif
// Build option, off: Q.K^T issued for two key tiles at once (N = 128 into both S buffers).  An MMA
// with N = 64 re-reads its 128-row A operand from shared memory for 64 columns of work and runs
// at 58 % of the tensor pipe's rate (sl8_tensor_peak_probe_n: 1307 of 2222 TFLOP/s for kind::f16,
// 2578 of 4496 TOPS for kind::i8); with N = 128 it runs at full rate.  Measured on a B = 4 slice of
// the S = 8192 causal workload the pairing nevertheless LOSES (16-bit 4.10 -> 4.5-4.8 ms, int8
// 4.12 -> 5.04 ms): the pair can only be issued once both P tiles have been consumed, so the
// softmax warps wait for P.V + Q.K^T (about 770 cycles) every second tile, and the look-ahead of
// one finished S tile -- what keeps them busy in the default order -- is gone.
constexpr bool kQkPair = SL8_QK_PAIR != 0;

template <int D, bool QK8>
struct TcCfg {
  static constexpr int QK_ROWB = D * (QK8 ? 1 : 2);      // bytes of one Q/K row
  static constexpr int QROW = QK_ROWB < 128 ? QK_ROWB : 128;  // bytes per shared row of a Q/K sub-tile
  static constexpr int QSUBS = QK_ROWB / QROW;
  static constexpr uint32_t QK_SW = QROW == 128 ? kUmmaSw128 : kUmmaSw64;
  static constexpr int Q_SUB_BYTES = kTM * QROW;
  static constexpr int Q_TILE_BYTES = kTM * QK_ROWB;
  static constexpr int K_SUB_BYTES = kTN * QROW;
  static constexpr int K_TILE_BYTES = kTN * QK_ROWB;
  static constexpr int QK_STEPS = QK_ROWB / 32;           // MMA K steps of 32 bytes
  static constexpr int VSUBS = 2 * D / 128;               // 64-channel sub-tiles of kTN keys x 128 B
  static constexpr int V_SUB_BYTES = kTN * 128;
  static constexpr int V_TILE_BYTES = kTN * 2 * D;
  static constexpr int NKS = 2;                            // K stages = S buffers (one barrier frees both)
  static constexpr int NVS = 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_TILE_BYTES;
  static constexpr int OFF_V = OFF_K + NKS * K_TILE_BYTES;
  static constexpr int OFF_KS = OFF_V + NVS * V_TILE_BYTES;   // kScaleStages x kTN floats
  static constexpr int OFF_VS = OFF_KS + kScaleStages * kTN * 4;  // W8A8 mode: v_scale of the head, D floats
  static constexpr int OFF_BAR = OFF_VS + 1024;
  static constexpr int NEED = OFF_BAR + 512 + 1024;
  // never more than two blocks per SM: each holds TMEM_COLS columns of the 512
  static constexpr int SMEM = NEED < 78 * 1024 ? 78 * 1024 : NEED;
  static constexpr uint32_t TMEM_COLS = D <= 128 ? 256 : 512;
  static constexpr uint32_t COL_S = 0, COL_O = 128;        // S: two buffers of kTN columns
};

struct TcArgs {
  const float* q_scale;
  const float* k_scale;
  void* out;
  float* lse;
  const int32_t* seqlens_q;
  const int32_t* seqlens_k;
  // Packed token-major tensors [tokens, heads, D] (scales [tokens, heads]) when non-null:
  // sequence b owns tokens [cu_q[b], cu_q[b+1]) of q / out and [cu_k[b], cu_k[b+1]) of k / v.
  // The tensor maps are then {D, heads, tokens} instead of {D, rows, batch * heads}.
  const int32_t* cu_q;
  const int32_t* cu_k;
  int* status;
  // Device-side dispatch: when non-null the kernel runs only if (*gate_flag != 0) == (gate_want != 0).
  const int32_t* gate_flag;
  int gate_want;
  int Hq, Hkv, M, N;
  int causal, window_left;
  float scale_log2;  // 16-bit Q/K mode: softmax_scale * log2(e)
  // Full-W8A8 mode (kernel template W8): V holds int8 codes as fp16, v_scale fp32 [B, Hkv, D]
  // multiplies the output channels, P is snapped to the int8 grid per row and tile
  // (w8_per_half = 0) or per row and 32-key half (w8_per_half != 0).
  const float* v_scale;
  int w8_per_half;
  // 16-bit mode with an additive bias (kernel template BIAS): natural-log units, V's element type,
  // strides in elements, 0 on broadcast axes (reference csrc/include/attn_fp16_fwd.cuh:176-178)
  const void* mask;
  int64_t mask_sb, mask_sh, mask_sm, mask_sn;
};

enum Bar {
  // S_FULL[b] (commit behind QK_t, b = t & 1; in int8 mode a second arrival says that the tile's
  // k_scale values are in shared memory) also tells the producer that K stage b is free;
  // PV_DONE[b] (commit behind P.V_j, b = j & 1) also tells it that V stage b is free.
  Q_FULL = 0, O_DONE, PV_DONE, S_FULL = PV_DONE + 2, P_FULL = S_FULL + 2, K_FULL = P_FULL + 2,
  V_FULL = K_FULL + 2, KS_EMPTY = V_FULL + 2, NUM_BARS = KS_EMPTY + kScaleStages
};

SL8_TRACE_DEFINE()

// One of two register arrays, chosen at compile time (the other has one element and disappears).
template <bool FIRST, int NA, int NB>
__device__ __forceinline__ auto& pick_regs(uint32_t (&a)[NA], uint32_t (&b)[NB]) {
  if constexpr (FIRST) return a;
  else return b;
}

template <int D, typename VT, bool QK8, bool PACKED, bool W8 = false, bool BIAS = false>
__global__ void __launch_bounds__(kTcThreads, 2) fwd_tc_kernel(const __grid_constant__ CUtensorMap q_map,
                                                               const __grid_constant__ CUtensorMap k_map,
                                                               const __grid_constant__ CUtensorMap v_map,
                                                               const __grid_constant__ CUtensorMap o_map, TcArgs a) {
  using C = TcCfg<D, QK8>;
  // the accuracy gate decided on the device: the kernel of the other precision does the work
  if (a.gate_flag != nullptr && ((__ldg(a.gate_flag) != 0) != (a.gate_want != 0))) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* ks_smem = reinterpret_cast<float*>(smem + C::OFF_KS);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t bh = blockIdx.y;
  const int b = (int)(bh / a.Hq);
  const int G = a.Hq / a.Hkv;
  const int kv_bh = b * a.Hkv + (int)(bh % a.Hq) / G;
  constexpr bool packed = PACKED;   // token-major packed tensors (a.cu_q / a.cu_k set)
  const int hq = (int)(bh % a.Hq), hkv = hq / G;
  const int q0 = packed ? a.cu_q[b] : 0, k0 = packed ? a.cu_k[b] : 0;   // first token of the sequence
  const int m_len = packed ? a.cu_q[b + 1] - q0 : (a.seqlens_q ? min(max(a.seqlens_q[b], 0), a.M) : a.M);
  const int n_len = packed ? a.cu_k[b + 1] - k0 : (a.seqlens_k ? min(max(a.seqlens_k[b], 0), a.N) : a.N);
  // Where this block writes: base of its head's rows, elements between rows, and the rows it
  // may write (packed: never a neighbour's).
  const int o_rows = packed ? m_len : a.M;
  const int64_t o_row = packed ? (int64_t)a.Hq * D : D;
  VT* const ob = reinterpret_cast<VT*>(a.out) + (packed ? ((int64_t)q0 * a.Hq + hq) * D : bh * (int64_t)a.M * D);
  // TMA coordinates 1 and 2 of row r: dense (r, batch * heads + head), packed (head, first token + r)
#define SL8_QC1(r) (packed ? hq : (r))
#define SL8_QC2(r) (packed ? q0 + (r) : (int)bh)
#define SL8_KC1(r) (packed ? hkv : (r))
#define SL8_KC2(r) (packed ? k0 + (r) : kv_bh)
  const int m_block = (a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x) * kTM;
  const int causal_diag = a.causal ? n_len - m_len : 0;
  const int n_end = a.causal ? max(0, min(n_len, m_block + kTM + causal_diag)) : n_len;
  int n_begin = 0;
  if (a.window_left >= 0) n_begin = max(0, (m_block + causal_diag - a.window_left + 1)) / kTN * kTN;
  const int ntiles = (m_block < m_len && n_end > n_begin) ? (n_end - n_begin + kTN - 1) / kTN : 0;

  if (ntiles == 0) {  // no visible key for any row of the tile (or padded rows): zeros
    for (int idx = threadIdx.x; idx < kTM * (D / 8); idx += kTcThreads) {
      const int r = idx / (D / 8), c = (idx % (D / 8)) * 8;
      if (m_block + r < o_rows) *reinterpret_cast<uint4*>(ob + (int64_t)(m_block + r) * o_row + c) = make_uint4(0, 0, 0, 0);
    }
    if (a.lse) for (int r = threadIdx.x; r < kTM; r += kTcThreads)
        if (m_block + r < o_rows) a.lse[bh * a.M + m_block + r] = -INFINITY;
    return;
  }

  if (threadIdx.x == 0) {
    TR(8188);
    TRV(8191, (long long)sl8_smid());
    mbar_init(&bars[Q_FULL], 1);
    mbar_init(&bars[O_DONE], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[PV_DONE + i], 1);
      mbar_init(&bars[S_FULL + i], QK8 ? 2 : 1);   // int8: the MMA commit and the k_scale tile
      mbar_init(&bars[P_FULL + i], kSoftmaxWarps);
      mbar_init(&bars[V_FULL + i], 1);
      mbar_init(&bars[K_FULL + i], 1);
    }
    for (int i = 0; i < kScaleStages; ++i) {
      mbar_init(&bars[KS_EMPTY + i], kSoftmaxWarps);
    }
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tc_alloc(tmem_slot, C::TMEM_COLS);
    tc_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  bool ok = true;
  if (threadIdx.x == 0) TR(8189);

  if (kWgRegs && warp > kMmaWarp) {
    reg_dec<kRegsOther>();   // idle warps of the second warpgroup: they only lend their registers
  } else if (warp == kProducerWarp) {
    // ======================= producer =======================
    if (kWgRegs) reg_dec<kRegsOther>();
    if (lane == 0) {
      tma_prefetch_desc(&q_map);
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
      mbar_expect_tx(&bars[Q_FULL], C::Q_TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::QSUBS; ++c)
        tma_load_3d(smem + C::OFF_Q + c * C::Q_SUB_BYTES, &q_map, &bars[Q_FULL], c * (C::QROW / (QK8 ? 1 : 2)),
                    SL8_QC1(m_block), SL8_QC2(m_block));
    }
    auto load_k = [&](int t) -> bool {   // lane 0 only
      const int ks = t % C::NKS;
      if (t >= C::NKS && !mbar_wait(&bars[S_FULL + ks], ((t / C::NKS) - 1) & 1, a.status)) return false;
      mbar_expect_tx(&bars[K_FULL + ks], C::K_TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::QSUBS; ++c)
        tma_load_3d(smem + C::OFF_K + (kQkPair ? c * 2 * C::K_SUB_BYTES + ks * C::K_SUB_BYTES : ks * C::K_TILE_BYTES + c * C::K_SUB_BYTES),
                    &k_map, &bars[K_FULL + ks],
                    c * (C::QROW / (QK8 ? 1 : 2)), SL8_KC1(n_begin + t * kTN), SL8_KC2(n_begin + t * kTN));
      return true;
    };
    // K runs two tiles ahead of V: the issuer asks for K_{j+2} as soon as P.V_j is queued.
    if (lane == 0) {
      ok = load_k(0);
      if (ok && ntiles > 1) ok = load_k(1);
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    // k_scale values travel three tiles ahead in registers, so the latency of their global
    // loads never sits on the path of a tile.
    auto fetch_ks = [&](int t, float (&dst)[kTN / 32]) {
#pragma unroll
      for (int i = 0; i < kTN / 32; ++i) {
        const int n = n_begin + t * kTN + lane + 32 * i;
        dst[i] = (QK8 && t < ntiles && n < n_len) ? __ldg(packed ? a.k_scale + ((int64_t)(k0 + n) * a.Hkv + hkv) : a.k_scale + (int64_t)kv_bh * a.N + n) : 0.f;
      }
    };
    float ks0[kTN / 32], ks1[kTN / 32], ks2[kTN / 32];
    fetch_ks(0, ks0);
    fetch_ks(1, ks1);
    fetch_ks(2, ks2);
    for (int j = 0; j < ntiles && ok; ++j) {
      const int n_block = n_begin + j * kTN;
      if (QK8) {
        // k_scale tile through the generic proxy (its start is not 16-byte aligned in general)
        const int ss = j % kScaleStages;
        if (j >= kScaleStages) ok = mbar_wait(&bars[KS_EMPTY + ss], ((j / kScaleStages) - 1) & 1, a.status);
        if (!ok) break;
#pragma unroll
        for (int i = 0; i < kTN / 32; ++i) {
          ks_smem[ss * kTN + lane + 32 * i] = ks0[i];
          ks0[i] = ks1[i];
          ks1[i] = ks2[i];
        }
        fetch_ks(j + 3, ks2);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[S_FULL + (j & 1)]);
      }
      if (lane == 0) {
        const int vs = j % C::NVS;
        if (j + 2 < ntiles) ok = load_k(j + 2);
        if (ok && j >= C::NVS) ok = mbar_wait(&bars[PV_DONE + vs], ((j / C::NVS) - 1) & 1, a.status);
        if (ok) {
          mbar_expect_tx(&bars[V_FULL + vs], C::V_TILE_BYTES);
#pragma unroll
          for (int c = 0; c < C::VSUBS; ++c)
            tma_load_3d(smem + C::OFF_V + vs * C::V_TILE_BYTES + c * C::V_SUB_BYTES, &v_map, &bars[V_FULL + vs],
                        c * 64, SL8_KC1(n_block), SL8_KC2(n_block));
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
  } else if (warp == kMmaWarp) {
    // ======================= MMA issuer =======================
    if (kWgRegs) reg_dec<kRegsOther>();
    // Order of issue: QK_0, QK_1, then for every tile j: P.V_j, QK_{j+2}.  S has two buffers, so
    // the next tile's logits are already in tensor memory while the softmax warps work on
    // this one; QK_{j+2} reuses the buffer whose P the (earlier issued) P.V_j reads.
    // The whole warp walks the loop and polls the barriers (warp-uniform control flow and
    // addresses); one elected lane issues the MMAs and commits.  Descriptors are built once:
    // per MMA only the start-address field of a descriptor moves.
    constexpr uint32_t vfmt = std::is_same<VT, __nv_bfloat16>::value ? 1u : 0u;
    const uint32_t idesc_qk = QK8 ? umma_idesc(2, 1, 1, 0, 0, kTM, kTN) : umma_idesc(1, vfmt, vfmt, 0, 0, kTM, kTN);
    const uint32_t idesc_pv = umma_idesc(1, vfmt, vfmt, 0, 1, kTM, D);
    const uint64_t dq = umma_smem_desc(smem_u32(smem + C::OFF_Q), 16, 8 * C::QROW, C::QK_SW);
    const uint64_t dk = umma_smem_desc(smem_u32(smem + C::OFF_K), 16, 8 * C::QROW, C::QK_SW);
    const uint64_t dv = umma_smem_desc(smem_u32(smem + C::OFF_V), C::V_SUB_BYTES, 1024, kUmmaSw128);
    auto issue_qk = [&](int t, int buf) -> bool {   // buf = t & 1 = K stage = S buffer
      if (!__all_sync(0xffffffffu, mbar_wait(&bars[K_FULL + buf], (t >> 1) & 1, a.status))) return false;
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int s = 0; s < C::QK_STEPS; ++s) {
          const uint32_t sub = 32 * s / C::QROW, within = 32 * s % C::QROW;
          const uint64_t da = umma_desc_advance(dq, sub * C::Q_SUB_BYTES + within);
          const uint64_t db = umma_desc_advance(dk, buf * C::K_TILE_BYTES + sub * C::K_SUB_BYTES + within);
          if (QK8) tc_mma_i8_ss(tmem + C::COL_S + kTN * buf, da, db, idesc_qk, s > 0 ? 1u : 0u);
          else tc_mma_f16_ss(tmem + C::COL_S + kTN * buf, da, db, idesc_qk, s > 0 ? 1u : 0u);
        }
        tc_commit(&bars[S_FULL + buf]);
      }
      __syncwarp();
      return true;
    };
    // Pair mode: tiles t (even) and t + 1 in one N = 128 instruction per K step; the two key tiles
    // lie behind one another in shared memory (per 128-byte sub-tile: 128 rows).
    const uint32_t idesc_qk2 = QK8 ? umma_idesc(2, 1, 1, 0, 0, kTM, 2 * kTN) : umma_idesc(1, vfmt, vfmt, 0, 0, kTM, 2 * kTN);
    auto issue_qk_pair = [&](int t) -> bool {
      const bool both = t + 1 < ntiles;
      if (!__all_sync(0xffffffffu, mbar_wait(&bars[K_FULL + 0], (t >> 1) & 1, a.status))) return false;
      if (both && !__all_sync(0xffffffffu, mbar_wait(&bars[K_FULL + 1], (t >> 1) & 1, a.status))) return false;
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int s = 0; s < C::QK_STEPS; ++s) {
          const uint32_t sub = 32 * s / C::QROW, within = 32 * s % C::QROW;
          const uint64_t da = umma_desc_advance(dq, sub * C::Q_SUB_BYTES + within);
          const uint64_t db = umma_desc_advance(dk, sub * 2 * C::K_SUB_BYTES + within);
          if (QK8) tc_mma_i8_ss(tmem + C::COL_S, da, db, idesc_qk2, s > 0 ? 1u : 0u);
          else tc_mma_f16_ss(tmem + C::COL_S, da, db, idesc_qk2, s > 0 ? 1u : 0u);
        }
        tc_commit(&bars[S_FULL + 0]);
        if (both) tc_commit(&bars[S_FULL + 1]);
      }
      __syncwarp();
      return true;
    };
    static_assert(C::NKS == 2 && C::NVS == 2, "the issuer is unrolled over two stages");
    ok = __all_sync(0xffffffffu, mbar_wait(&bars[Q_FULL], 0, a.status));
    if (kQkPair) {
      if (ok) ok = issue_qk_pair(0);
    } else {
      if (ok) ok = issue_qk(0, 0);
      if (ok && ntiles > 1) ok = issue_qk(1, 1);
    }
    for (int j0 = 0; j0 < ntiles && ok; j0 += 2) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int j = j0 + u;
        if (j >= ntiles || !ok) break;
        const uint32_t par = (j0 >> 1) & 1;
        TR(4096 + 8 * j + 0);
        ok = __all_sync(0xffffffffu, mbar_wait(&bars[P_FULL + u], par, a.status));
        TR(4096 + 8 * j + 1);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars[V_FULL + u], par, a.status));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < kTN / 16; ++kk)
            tc_mma_f16_ts(tmem + C::COL_O, tmem + C::COL_S + kTN * u + 8 * kk,
                          umma_desc_advance(dv, u * C::V_TILE_BYTES + kk * 2048), idesc_pv,
                          (j > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&bars[PV_DONE + u]);
        }
        __syncwarp();
        TR(4096 + 8 * j + 2);
        if (kQkPair) {
          if (u == 1 && j + 1 < ntiles) ok = issue_qk_pair(j + 1);
        } else if (j + 2 < ntiles) ok = issue_qk(j + 2, u);
        TR(4096 + 8 * j + 3);
        if (j == ntiles - 1 && elect_one()) tc_commit(&bars[O_DONE]);
        __syncwarp();
      }
    }
  } else {
    // ======================= softmax / correction / epilogue =======================
    if (kWgRegs) reg_inc<kRegsSoftmax>();
    // Thread = query row: warp w reads and writes tensor-memory lanes [32 w, 32 w + 32).
    const int lg = warp;
    const int row = 32 * lg + lane;
    const int m = m_block + row;                // this thread's query row
    const float qs = QK8 ? ((m < m_len) ? __ldg(packed ? a.q_scale + ((int64_t)(q0 + m) * a.Hq + hq) : a.q_scale + bh * a.M + m) : 0.f) : a.scale_log2;
    const int qpos = m + causal_diag;
    const uint32_t t_row = tmem + ((uint32_t)(32 * lg) << 16);
    const uint32_t t_o = t_row + C::COL_O;
    float m_run = -INFINITY, l_run = 0.f;
    float* const vs_smem = reinterpret_cast<float*>(smem + C::OFF_VS);
    // this row of the additive bias (null for rows past the end: nothing is read for them)
    const VT* const bias_row = (BIAS && m < m_len)
                                   ? reinterpret_cast<const VT*>(a.mask) + (int64_t)b * a.mask_sb + (int64_t)hq * a.mask_sh + (int64_t)m * a.mask_sm
                                   : nullptr;
    if (W8) {   // read back in the epilogue, after many block-wide barriers' worth of mbarrier traffic
      for (int c = row; c < D; c += 32 * kSoftmaxWarps) vs_smem[c] = __ldg(a.v_scale + (int64_t)kv_bh * D + c);
      named_sync(1, 32 * kSoftmaxWarps);
    }

    // EARLY (16-bit mode): the tile's 64 accumulator registers live across the loop's back edge, so
    // that the next tile's logits can be loaded into them at the end of this tile.  The other
    // modes keep them local to an iteration (the int8 instantiation sits at the register limit
    // and spills when they are carried).
    constexpr bool EARLY = kEarlyLoad && (!QK8 || SL8_EARLY_LOAD == 2 || kWgRegs);
    constexpr int EARLY_CHUNKS = (QK8 && !kWgRegs) ? 1 : kTN / 32;   // 32-column pieces loaded early (experiment: int8 carries half)
    uint32_t r_carried[EARLY ? kTN : 1];
    bool loaded = false;   // the load of this tile's logits was issued at the end of the previous tile
    for (int j = 0; j < ntiles; ++j) {
      uint32_t r_local[EARLY ? 1 : kTN];
      uint32_t(&r)[kTN] = pick_regs<EARLY>(r_carried, r_local);
      const int n_block = n_begin + j * kTN;
      const int ss = j % kScaleStages;
      const uint32_t t_s = t_row + C::COL_S + kTN * (j & 1);
      if (warp == 0 && lane == 0) TR(8 * j + 0);
      if (!EARLY || !loaded) {
        ok = mbar_wait(&bars[S_FULL + (j & 1)], (j >> 1) & 1, a.status);
        if (!ok) break;
        tc_fence_after();
      }
      if (warp == 0 && lane == 0) TR(8 * j + 1);
      if (!EARLY || !loaded) {
#pragma unroll
        for (int c = 0; c < kTN / 32; ++c) tc_ld32(t_s + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
      } else {
#pragma unroll
        for (int c = EARLY_CHUNKS; c < kTN / 32; ++c) tc_ld32(t_s + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
      }
      tc_wait_ld();
#pragma unroll
      for (int c = 0; c < kTN / 32; ++c) tc_regs_ready(*reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
      if (warp == 0 && lane == 0) TR(8 * j + 2);
      const float* ksv = ks_smem + ss * kTN;
      const bool need_mask = BIAS || (n_block + kTN > n_len) || (a.causal && n_block + kTN - 1 > m_block + causal_diag) ||
                             (a.window_left >= 0 && n_block <= m_block + kTM - 1 + causal_diag - a.window_left);
      // Speculative single sweep: P is formed against the running max while the tile's own max is
      // still being collected.  Lazy rescale makes that the final answer whenever no row of the
      // warp outgrew its running max by more than 2^8 (P <= 256 then: harmless in fp16 / bf16 and
      // in the fp32 sum; out = O / l does not depend on which reference max was used).  Otherwise
      // (the first tile, and rarely later) the max moves, O is corrected and P is formed again.
      const float xs = need_mask ? 1.f : qs;      // masked tiles keep finished logits in r, the others t
      float mx, psum;
      float mxh[2] = {0.f, 0.f};
      if (W8) {
        // W8A8 mode: the tile's maxima come first (P's int8 grid hangs on them), no speculation
        if (need_mask) w8_logits_pass<QK8, true>(r, ksv, qs, n_block, n_len, a.causal, qpos, a.window_left, mxh);
        else w8_logits_pass<QK8, false>(r, ksv, qs, n_block, n_len, a.causal, qpos, a.window_left, mxh);
        mx = fmaxf(mxh[0], mxh[1]);
      } else {
        const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;
        if constexpr (BIAS) softmax_pass<QK8, true, true, VT, true>(r, ksv, qs, xs, neg_m, n_block, n_len, a.causal, qpos, a.window_left, t_s, mx, psum, bias_row, a.mask_sn);
        else if (need_mask) softmax_pass<QK8, true, true, VT>(r, ksv, qs, xs, neg_m, n_block, n_len, a.causal, qpos, a.window_left, t_s, mx, psum);
        else softmax_pass<QK8, false, true, VT>(r, ksv, qs, xs, neg_m, n_block, n_len, a.causal, qpos, a.window_left, t_s, mx, psum);
      }
      const float tmax = need_mask ? mx : mx * qs;
      if (warp == 0 && lane == 0) TR(8 * j + 3);
      const bool grow = (m_run == -INFINITY) ? (tmax > -INFINITY) : (tmax > m_run + kLazyRescaleLog2);
      float resc = 1.f;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_run, tmax);
        resc = exp2f(m_run - ((m_new == -INFINITY) ? 0.f : m_new));  // m_run = -inf -> 0
        m_run = m_new;
        if (j > 0) {
          // correction: O *= resc once the previous tile's P.V has landed in O
          ok = mbar_wait(&bars[PV_DONE + ((j - 1) & 1)], ((j - 1) >> 1) & 1, a.status);
          if (!ok) break;
          tc_fence_after();
          const float2 resc2 = make_float2(resc, resc);
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tc_ld32(t_o + 32 * c, o);
            tc_wait_ld();
            tc_regs_ready(o);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 t = __fmul2_rn(bits2(o[2 * i], o[2 * i + 1]), resc2);
              o[2 * i] = __float_as_uint(t.x);
              o[2 * i + 1] = __float_as_uint(t.y);
            }
            tc_st32(t_o + 32 * c, o);
          }
        }
        if (!W8) {
          tc_wait_st();   // the speculative P stores are done before P is stored again
          float unused;
          softmax_pass<QK8, false, false, VT>(r, ksv, qs, xs, (m_run == -INFINITY) ? 0.f : -m_run, n_block, n_len, a.causal,
                                              qpos, a.window_left, t_s, unused, psum);
        }
      }
      if (W8) w8_exp_pass<VT>(r, xs, (m_run == -INFINITY) ? 0.f : -m_run, mxh, a.w8_per_half != 0, t_s, psum);
      l_run = l_run * resc + psum;
      if (warp == 0 && lane == 0) TR(8 * j + 4);
      // The tile's logits are dead (P is final): when the next tile's are already in tensor memory --
      // its Q.K^T was queued a whole sweep ago -- start loading them now, so that the latency of the
      // load runs under this tile's store wait, fence and arrival instead of in front of the sweep.
      if constexpr (EARLY) {
        loaded = false;
        if (j + 1 < ntiles && __all_sync(0xffffffffu, mbar_test(&bars[S_FULL + ((j + 1) & 1)], ((j + 1) >> 1) & 1))) {
          tc_fence_after();
          const uint32_t t_n = t_row + C::COL_S + kTN * ((j + 1) & 1);
#pragma unroll
          for (int c = 0; c < EARLY_CHUNKS; ++c) tc_ld32(t_n + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&r[32 * c]));
          loaded = true;
        }
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars[P_FULL + (j & 1)]);
        if (QK8) mbar_arrive(&bars[KS_EMPTY + ss]);
      }
      if (warp == 0 && lane == 0) TR(8 * j + 5);
    }
    // ---- epilogue ----
    if (warp == 0 && lane == 0) TR(8185);
    if (ok) ok = mbar_wait(&bars[O_DONE], 0, a.status);
    if (warp == 0 && lane == 0) TR(8186);
    if (ok) {
      tc_fence_after();
      const float l_tot = l_run;
      const bool live = m < m_len;
      const float inv = (live && l_tot > 0.f) ? 1.f / l_tot : 0.f;
      if (!packed) {
        // Dense layout: the warp's 32 rows are staged in shared memory (the V stages are free, every
        // P.V has completed) in the 128-byte-swizzled layout of the output tensor map -- 16-byte
        // chunk j of row r sits at chunk j ^ (r & 7), so the 32 row writes of one instruction
        // spread over all banks -- and leave as one tile store per 64 channels; rows past M are
        // dropped by the copy engine, padded rows (seqlens_q) carry zeros as before.
        uint8_t* const stage = smem + C::OFF_V + lg * (32 * 128) + lane * 128;
        if (lane == 0) tma_prefetch_desc(&o_map);
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tc_ld32(t_o + 32 * c, o);
          tc_wait_ld();
          tc_regs_ready(o);
          uint8_t* const sub = stage + (c >> 1) * (kTM * 128);
          if (W8) {   // out = O * v_scale[channel] / l (reference csrc/include/attn_w8a8_fwd.cuh:207-222)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 vs4 = *reinterpret_cast<const float4*>(vs_smem + 32 * c + i);
              o[i] = __float_as_uint(__uint_as_float(o[i]) * vs4.x);
              o[i + 1] = __float_as_uint(__uint_as_float(o[i + 1]) * vs4.y);
              o[i + 2] = __float_as_uint(__uint_as_float(o[i + 2]) * vs4.z);
              o[i + 3] = __float_as_uint(__uint_as_float(o[i + 3]) * vs4.w);
            }
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 w;
            w.x = pack2<VT>(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
            w.y = pack2<VT>(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
            w.z = pack2<VT>(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
            w.w = pack2<VT>(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
            *reinterpret_cast<uint4*>(sub + ((((c & 1) * 4 + v) ^ (lane & 7)) << 4)) = w;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && m_block + 32 * lg < a.M) {
#pragma unroll
          for (int sb = 0; sb < D / 64; ++sb)
            tma_store_3d(&o_map, smem + C::OFF_V + sb * (kTM * 128) + lg * (32 * 128), 64 * sb, m_block + 32 * lg, (int)bh);
          tma_store_commit();
          tma_store_wait_read();
        }
      } else {
  #pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tc_ld32(t_o + 32 * c, o);
        tc_wait_ld();
        tc_regs_ready(o);
        if (m < o_rows) {
          uint4* dst = reinterpret_cast<uint4*>(ob + (int64_t)m * o_row + 32 * c);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 w;
            w.x = pack2<VT>(__uint_as_float(o[8 * v + 0]) * inv, __uint_as_float(o[8 * v + 1]) * inv);
            w.y = pack2<VT>(__uint_as_float(o[8 * v + 2]) * inv, __uint_as_float(o[8 * v + 3]) * inv);
            w.z = pack2<VT>(__uint_as_float(o[8 * v + 4]) * inv, __uint_as_float(o[8 * v + 5]) * inv);
            w.w = pack2<VT>(__uint_as_float(o[8 * v + 6]) * inv, __uint_as_float(o[8 * v + 7]) * inv);
            dst[v] = w;
          }
        }
      }
      }
      if (a.lse != nullptr && m < o_rows)
        a.lse[bh * a.M + m] = (live && l_tot > 0.f) ? (m_run * 0.6931471805599453f + logf(l_tot)) : -INFINITY;
    }
    if (warp == 0 && lane == 0) TR(8187);
    tc_fence_before();
  }

  // ---- teardown: every role arrives here, on success and on a timed-out wait ----
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tc_dealloc(tmem, C::TMEM_COLS);
  }
}

// ---- raw int32 logits through the same TMA + kind::i8 tile path ----------------
constexpr int kLN = 128;  // keys per tile of the logits kernel

template <int D>
__global__ void __launch_bounds__(128) qk_logits_kernel(const __grid_constant__ CUtensorMap q_map,
                                                        const __grid_constant__ CUtensorMap k_map, int32_t* s_out,
                                                        int M, int N, int* status) {
  using C = TcCfg<D, true>;
  constexpr int SUB = 128 * C::QROW, TILE = 128 * D;   // 128-row tiles of Q and of K
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * TILE);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_block = blockIdx.x * kTM, n_block = blockIdx.y * kLN;
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tc_alloc(tmem_slot, 128);
    tc_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  bool ok = true;
  if (threadIdx.x == 0) {
    mbar_expect_tx(&bars[0], 2 * TILE);
#pragma unroll
    for (int c = 0; c < C::QSUBS; ++c) {
      tma_load_3d(smem + c * SUB, &q_map, &bars[0], c * C::QROW, m_block, 0);
      tma_load_3d(smem + TILE + c * SUB, &k_map, &bars[0], c * C::QROW, n_block, 0);
    }
    ok = mbar_wait(&bars[0], 0, status);
    if (ok) {
      tc_fence_after();
      const uint32_t idesc = umma_idesc(2, 1, 1, 0, 0, kTM, kLN);
      const uint32_t q_u = smem_u32(smem), k_u = smem_u32(smem + TILE);
#pragma unroll
      for (int s = 0; s < D / 32; ++s) {
        const uint32_t off = (32 * s / C::QROW) * SUB + (32 * s % C::QROW);
        tc_mma_i8_ss(tmem, umma_smem_desc(q_u + off, 16, 8 * C::QROW, C::QK_SW),
                     umma_smem_desc(k_u + off, 16, 8 * C::QROW, C::QK_SW), idesc, s > 0 ? 1u : 0u);
      }
      tc_commit(&bars[1]);
    }
  }
  ok = mbar_wait(&bars[1], 0, status);
  if (ok) {
    tc_fence_after();
    const int m = m_block + 32 * warp + lane;
#pragma unroll 1
    for (int c = 0; c < kLN / 32; ++c) {
      uint32_t r[32];
      tc_ld32(tmem + ((uint32_t)(32 * warp) << 16) + 32 * c, r);
      tc_wait_ld();
      tc_regs_ready(r);
      if (m < M)
        for (int i = 0; i < 32; ++i) {
          const int n = n_block + 32 * c + i;
          if (n < N) s_out[(int64_t)m * N + n] = (int)r[i];
        }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tc_dealloc(tmem, 128);
  }
}

// Dense call: M, N = rows per head.  Packed call (a.cu_q set): M = longest query sequence (sizes
// the grid), total_q / total_k = tokens in the packed tensors.
template <int D, typename VT, bool QK8, bool W8 = false, bool BIAS = false>
int launch_tc_impl(const void* q, const void* k, const void* v, int B, int Hq, int Hkv, int M, int N, const TcArgs& a,
                   cudaStream_t stream, int64_t total_q = 0, int64_t total_k = 0) {
  using C = TcCfg<D, QK8>;
  constexpr int es = QK8 ? 1 : 2;
  CUtensorMap q_map, k_map, v_map, o_map;
  int rc;
  if (a.cu_q != nullptr) {
    rc = sl8_make_tmap_packed(&q_map, q, es, D, Hq, total_q, C::QROW / es, kTM, C::QROW);
    if (rc == SL8_OK) rc = sl8_make_tmap_packed(&k_map, k, es, D, Hkv, total_k, C::QROW / es, kTN, C::QROW);
    if (rc == SL8_OK) rc = sl8_make_tmap_packed(&v_map, v, 2, D, Hkv, total_k, 64, kTN, 128);
  } else {
    rc = sl8_make_tmap_3d(&q_map, q, es, D, M, (uint64_t)B * Hq, C::QROW / es, kTM, C::QROW);
    if (rc == SL8_OK) rc = sl8_make_tmap_3d(&k_map, k, es, D, N, (uint64_t)B * Hkv, C::QROW / es, kTN, C::QROW);
    if (rc == SL8_OK) rc = sl8_make_tmap_3d(&v_map, v, 2, D, N, (uint64_t)B * Hkv, 64, kTN, 128);
    // output tiles leave through the copy engine: 32 rows (one softmax warp) x 64 channels per store
    if (rc == SL8_OK) rc = sl8_make_tmap_3d(&o_map, a.out, 2, D, M, (uint64_t)B * Hq, 64, 32, 128);
  }
  if (rc != SL8_OK) return rc;
  if (a.cu_q != nullptr) o_map = q_map;   // packed rows are written with plain stores
  dim3 grid((M + kTM - 1) / kTM, (unsigned)((int64_t)B * Hq));
  if (a.cu_q != nullptr) {
    if (!QK8 || D == 256) return SL8_ERR_UNSUPPORTED;   // the packed op is int8-QK, D <= 128
    constexpr bool kPk = QK8 && D != 256;               // (keeps the unused instantiations out of the image)
    SL8_CUDA_TRY(cudaFuncSetAttribute(fwd_tc_kernel<D, VT, QK8, kPk>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    fwd_tc_kernel<D, VT, QK8, kPk><<<grid, kTcThreads, C::SMEM, stream>>>(q_map, k_map, v_map, o_map, a);
  } else {
    SL8_CUDA_TRY(cudaFuncSetAttribute(fwd_tc_kernel<D, VT, QK8, false, W8, BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    fwd_tc_kernel<D, VT, QK8, false, W8, BIAS><<<grid, kTcThreads, C::SMEM, stream>>>(q_map, k_map, v_map, o_map, a);
  }
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

template <typename VT, bool QK8>
int launch_tc_d(int D, const void* q, const void* k, const void* v, int B, int Hq, int Hkv, int M, int N,
                const TcArgs& a, cudaStream_t s, int64_t total_q = 0, int64_t total_k = 0) {
  switch (D) {
    case 64: return launch_tc_impl<64, VT, QK8>(q, k, v, B, Hq, Hkv, M, N, a, s, total_q, total_k);
    case 128: return launch_tc_impl<128, VT, QK8>(q, k, v, B, Hq, Hkv, M, N, a, s, total_q, total_k);
    case 256: return launch_tc_impl<256, VT, QK8>(q, k, v, B, Hq, Hkv, M, N, a, s, total_q, total_k);
  }
  return SL8_ERR_UNSUPPORTED;
}

// int8 codes -> the same integers as fp16 (exact), 16 per thread
__global__ void __launch_bounds__(256) v_codes_kernel(const int8_t* __restrict__ v, __half* __restrict__ out, int64_t n16) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(v) + i);
    const uint32_t in[4] = {w.x, w.y, w.z, w.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int b0 = (int8_t)(in[j] & 0xff), b1 = (int8_t)((in[j] >> 8) & 0xff), b2 = (int8_t)((in[j] >> 16) & 0xff),
                b3 = (int8_t)(in[j] >> 24);
      o[2 * j] = pack2<__half>((float)b0, (float)b1);
      o[2 * j + 1] = pack2<__half>((float)b2, (float)b3);
    }
    uint4* dst = reinterpret_cast<uint4*>(out) + 2 * i;
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

template <int D>
int launch_logits(const int8_t* q, const int8_t* k, int M, int N, int32_t* s_out, int* status, cudaStream_t stream) {
  using C = TcCfg<D, true>;
  CUtensorMap q_map, k_map;
  int rc = sl8_make_tmap_3d(&q_map, q, 1, D, M, 1, C::QROW, kTM, C::QROW);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&k_map, k, 1, D, N, 1, C::QROW, kLN, C::QROW);
  if (rc != SL8_OK) return rc;
  const int smem = 2 * 128 * D + 1024 + 64;
  SL8_CUDA_TRY(cudaFuncSetAttribute(qk_logits_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((M + kTM - 1) / kTM, (N + kLN - 1) / kLN);
  qk_logits_kernel<D><<<grid, 128, smem, stream>>>(q_map, k_map, s_out, M, N, status);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

bool head_dim_ok(int D) { return D == 32 || D == 64 || D == 72 || D == 80 || D == 128 || D == 256; }
bool tc_head_dim(int D) { return D == 64 || D == 128 || D == 256; }

}  // namespace
}  // namespace sl8

using namespace sl8;

extern "C" size_t sl8_attn_int8_fwd_workspace(const sl8_fwd_params*) { return 256; }

extern "C" int sl8_attn_int8_fwd(const sl8_fwd_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  if (p == nullptr) return SL8_ERR_NULL;
  if (p->B < 0 || p->Hq < 0 || p->Hkv < 0 || p->M < 0 || p->N < 0) return SL8_ERR_BAD_SHAPE;
  if (!head_dim_ok(p->D)) return SL8_ERR_BAD_HEAD_DIM;
  if (p->v_dtype != SL8_F16 && p->v_dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (p->Hq > 0 && (p->Hkv <= 0 || p->Hq % p->Hkv != 0)) return SL8_ERR_BAD_SHAPE;
  if ((int64_t)p->B * p->Hq * p->M == 0) return SL8_OK;  // empty output (reference attn_int8_fwd.cu:145)
  if (!p->q || !p->q_scale || !p->out) return SL8_ERR_NULL;
  if (p->N > 0 && (!p->k || !p->k_scale || !p->v)) return SL8_ERR_NULL;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return SL8_ERR_MISALIGNED;
  if ((int64_t)p->B * p->Hq > 65535) return SL8_ERR_TOO_LARGE;
  if (workspace == nullptr || workspace_bytes < 256) return SL8_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int backend = p->backend;
  if (backend == SL8_BACKEND_AUTO) backend = (tc_head_dim(p->D) && p->N > 0) ? SL8_BACKEND_TCGEN05 : SL8_BACKEND_MMA;
  if (p->gate_flag != nullptr && backend != SL8_BACKEND_TCGEN05 && backend != SL8_BACKEND_TCGEN05_2Q) return SL8_ERR_UNSUPPORTED;
  if (backend == SL8_BACKEND_MMA) return sl8_fwd_mma_int8(p, s);
  if (backend != SL8_BACKEND_TCGEN05 && backend != SL8_BACKEND_TCGEN05_2Q) return SL8_ERR_UNSUPPORTED;
  if (!tc_head_dim(p->D) || p->N == 0) return SL8_ERR_UNSUPPORTED;
  // a window that reaches past the first key hides nothing: the same call as no window at all
  const int window_eff = p->window_left >= p->N ? -1 : p->window_left;
  if (backend == SL8_BACKEND_TCGEN05_2Q && sl8_fwd_tc2_supported(p->D, window_eff, false)) {
    Tc2Args t{};
    t.q = p->q; t.k = p->k; t.v = p->v; t.out = p->out; t.q_scale = p->q_scale; t.k_scale = p->k_scale; t.lse = p->lse;
    t.seqlens_q = p->seqlens_q; t.seqlens_k = p->seqlens_k; t.status = reinterpret_cast<int*>(workspace);
    t.gate_flag = p->gate_flag; t.gate_want = p->gate_want;
    t.B = p->B; t.Hq = p->Hq; t.Hkv = p->Hkv; t.M = p->M; t.N = p->N; t.D = p->D; t.causal = p->causal;
    t.qk8 = 1; t.v_bf16 = p->v_dtype == SL8_BF16;
    return sl8_fwd_tc2(t, s);
  }
  TcArgs a{};
  a.q_scale = p->q_scale; a.k_scale = p->k_scale; a.out = p->out; a.lse = p->lse;
  a.seqlens_q = p->seqlens_q; a.seqlens_k = p->seqlens_k; a.status = reinterpret_cast<int*>(workspace);
  a.gate_flag = p->gate_flag; a.gate_want = p->gate_want;
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N; a.causal = p->causal; a.window_left = p->window_left;
  return p->v_dtype == SL8_F16
             ? launch_tc_d<__half, true>(p->D, p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s)
             : launch_tc_d<__nv_bfloat16, true>(p->D, p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s);
}

// ---- full W8A8 on the tensor-memory kernel -------------------------------------------------
namespace {
bool w8a8_tc_ok(const sl8_w8a8_params* p) {
  return tc_head_dim(p->D) && p->N > 0 && (!p->causal || p->causal_diag == p->N - p->M);
}
size_t w8a8_codes_bytes(const sl8_w8a8_params* p) { return (size_t)p->B * p->Hkv * p->N * p->D * sizeof(__half); }
}  // namespace

extern "C" size_t sl8_attn_w8a8_fwd_tc_workspace(const sl8_w8a8_params* p) {
  if (p == nullptr || p->B < 0 || p->Hkv < 0 || p->N < 0 || p->D < 0) return 256;
  return 256 + (w8a8_codes_bytes(p) + 255) / 256 * 256;
}

extern "C" int sl8_attn_w8a8_fwd_tc(const sl8_w8a8_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  if (p == nullptr) return SL8_ERR_NULL;
  if (p->B < 0 || p->Hq < 0 || p->Hkv < 0 || p->M < 0 || p->N < 0) return SL8_ERR_BAD_SHAPE;
  if (p->D != 32 && p->D != 64 && p->D != 128 && p->D != 256) return SL8_ERR_BAD_HEAD_DIM;
  if (p->Hq > 0 && (p->Hkv <= 0 || p->Hq % p->Hkv != 0)) return SL8_ERR_BAD_SHAPE;
  if ((int64_t)p->B * p->Hq * p->M == 0) return SL8_OK;   // empty output
  if (!w8a8_tc_ok(p)) return SL8_ERR_UNSUPPORTED;          // sl8_attn_w8a8_fwd serves these
  if (!p->q || !p->q_scale || !p->out || !p->k || !p->k_scale || !p->v || !p->v_scale) return SL8_ERR_NULL;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return SL8_ERR_MISALIGNED;
  if ((int64_t)p->B * p->Hq > 65535) return SL8_ERR_TOO_LARGE;
  if (workspace == nullptr || workspace_bytes < sl8_attn_w8a8_fwd_tc_workspace(p)) return SL8_ERR_WORKSPACE;
  if (!aligned16(workspace)) return SL8_ERR_MISALIGNED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __half* codes = reinterpret_cast<__half*>(static_cast<uint8_t*>(workspace) + 256);
  const int64_t n16 = (int64_t)p->B * p->Hkv * p->N * p->D / 16;   // D is a multiple of 64
  const int blocks = (int)std::min<int64_t>((n16 + 255) / 256, 148 * 16);
  SL8_CUDA_TRY(cudaMemsetAsync(workspace, 0, 256, s));   // status word of the bounded waits
  v_codes_kernel<<<blocks, 256, 0, s>>>(p->v, codes, n16);
  if (cudaGetLastError() != cudaSuccess) return SL8_ERR_CUDA;
  TcArgs a{};
  a.q_scale = p->q_scale; a.k_scale = p->k_scale; a.out = p->out; a.status = reinterpret_cast<int*>(workspace);
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N; a.causal = p->causal; a.window_left = -1;
  a.v_scale = p->v_scale; a.w8_per_half = p->per_warp_quant != 0;
  switch (p->D) {
    case 64: return launch_tc_impl<64, __half, true, true>(p->q, p->k, codes, p->B, p->Hq, p->Hkv, p->M, p->N, a, s);
    case 128: return launch_tc_impl<128, __half, true, true>(p->q, p->k, codes, p->B, p->Hq, p->Hkv, p->M, p->N, a, s);
    case 256: return launch_tc_impl<256, __half, true, true>(p->q, p->k, codes, p->B, p->Hq, p->Hkv, p->M, p->N, a, s);
  }
  return SL8_ERR_UNSUPPORTED;
}

extern "C" int sl8_attn_int8_varlen(const sl8_varlen_params* p, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  if (p == nullptr) return SL8_ERR_NULL;
  if (p->B < 0 || p->Hq < 0 || p->Hkv < 0 || p->total_q < 0 || p->total_k < 0 || p->max_seqlen_q < 0)
    return SL8_ERR_BAD_SHAPE;
  if (p->D != 32 && p->D != 64 && p->D != 128) return SL8_ERR_BAD_HEAD_DIM;
  if (p->v_dtype != SL8_F16 && p->v_dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (p->Hq > 0 && (p->Hkv <= 0 || p->Hq % p->Hkv != 0)) return SL8_ERR_BAD_SHAPE;
  if (p->B == 0 || p->Hq == 0 || p->total_q == 0 || p->max_seqlen_q == 0) return SL8_OK;   // nothing to write
  if (!p->q || !p->q_scale || !p->out || !p->cu_seqlens_q || !p->cu_seqlens_k) return SL8_ERR_NULL;
  if (p->total_k > 0 && (!p->k || !p->k_scale || !p->v)) return SL8_ERR_NULL;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return SL8_ERR_MISALIGNED;
  if ((int64_t)p->B * p->Hq > 65535 || p->total_q > INT32_MAX || p->total_k > INT32_MAX) return SL8_ERR_TOO_LARGE;
  if (workspace == nullptr || workspace_bytes < 256) return SL8_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int backend = p->backend;
  const bool tc_ok = (p->D == 64 || p->D == 128) && p->total_k > 0;
  if (backend == SL8_BACKEND_AUTO) backend = tc_ok ? SL8_BACKEND_TCGEN05 : SL8_BACKEND_MMA;
  if (backend == SL8_BACKEND_MMA) return sl8_fwd_mma_int8_varlen(p, s);
  if (backend != SL8_BACKEND_TCGEN05 || !tc_ok) return SL8_ERR_UNSUPPORTED;
  TcArgs a{};
  a.q_scale = p->q_scale; a.k_scale = p->k_scale; a.out = p->out;
  a.cu_q = p->cu_seqlens_q; a.cu_k = p->cu_seqlens_k; a.status = reinterpret_cast<int*>(workspace);
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->max_seqlen_q; a.N = 0; a.causal = p->causal; a.window_left = -1;
  return p->v_dtype == SL8_F16
             ? launch_tc_d<__half, true>(p->D, p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->max_seqlen_q, 0, a, s,
                                         p->total_q, p->total_k)
             : launch_tc_d<__nv_bfloat16, true>(p->D, p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->max_seqlen_q, 0, a, s,
                                                p->total_q, p->total_k);
}

// 16-bit Q/K forward on the tcgen05 path (D = 64, 128, 256, N > 0); parameters were validated
// by sl8_attn_fp16_fwd (fwd_mma.cu).
int sl8_fwd_tc_fp16(const sl8_fp16_fwd_params* p, int* status, cudaStream_t s) {
  if (!tc_head_dim(p->D) || p->N == 0) return SL8_ERR_UNSUPPORTED;
  const int window_eff = p->window_left >= p->N ? -1 : p->window_left;   // such a window hides nothing
  if (p->backend == SL8_BACKEND_TCGEN05_2Q && p->mask == nullptr && sl8_fwd_tc2_supported(p->D, window_eff, false)) {
    Tc2Args t{};
    t.q = p->q; t.k = p->k; t.v = p->v; t.out = p->out; t.lse = p->lse;
    t.seqlens_q = p->seqlens_q; t.seqlens_k = p->seqlens_k; t.status = status;
    t.gate_flag = p->gate_flag; t.gate_want = p->gate_want;
    t.B = p->B; t.Hq = p->Hq; t.Hkv = p->Hkv; t.M = p->M; t.N = p->N; t.D = p->D; t.causal = p->causal;
    t.scale_log2 = p->softmax_scale * 1.4426950408889634f;
    t.qk8 = 0; t.v_bf16 = p->dtype == SL8_BF16;
    return sl8_fwd_tc2(t, s);
  }
  TcArgs a{};
  a.out = p->out; a.lse = p->lse; a.seqlens_q = p->seqlens_q; a.seqlens_k = p->seqlens_k; a.status = status;
  a.gate_flag = p->gate_flag; a.gate_want = p->gate_want;
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N; a.causal = p->causal; a.window_left = p->window_left;
  a.scale_log2 = p->softmax_scale * 1.4426950408889634f;
  if (p->mask != nullptr) {   // the additive-bias instantiations
    a.mask = p->mask; a.mask_sb = p->mask_stride_b; a.mask_sh = p->mask_stride_h;
    a.mask_sm = p->mask_stride_m; a.mask_sn = p->mask_stride_n;
    const bool h = p->dtype == SL8_F16;
    switch (p->D) {
      case 64: return h ? launch_tc_impl<64, __half, false, false, true>(p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s)
                        : launch_tc_impl<64, __nv_bfloat16, false, false, true>(p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s);
      case 128: return h ? launch_tc_impl<128, __half, false, false, true>(p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s)
                         : launch_tc_impl<128, __nv_bfloat16, false, false, true>(p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s);
      case 256: return h ? launch_tc_impl<256, __half, false, false, true>(p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s)
                         : launch_tc_impl<256, __nv_bfloat16, false, false, true>(p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s);
    }
    return SL8_ERR_UNSUPPORTED;
  }
  return p->dtype == SL8_F16
             ? launch_tc_d<__half, false>(p->D, p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s)
             : launch_tc_d<__nv_bfloat16, false>(p->D, p->q, p->k, p->v, p->B, p->Hq, p->Hkv, p->M, p->N, a, s);
}

extern "C" int sl8_qk_logits_i32(const int8_t* q, const int8_t* k, int32_t M, int32_t N, int32_t D, int32_t* s_out,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  if (M < 0 || N < 0) return SL8_ERR_BAD_SHAPE;
  if (!tc_head_dim(D)) return SL8_ERR_BAD_HEAD_DIM;
  if (M == 0 || N == 0) return SL8_OK;
  if (!q || !k || !s_out) return SL8_ERR_NULL;
  if (!aligned16(q) || !aligned16(k)) return SL8_ERR_MISALIGNED;
  if (workspace == nullptr || workspace_bytes < 256) return SL8_ERR_WORKSPACE;
  int* status = reinterpret_cast<int*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (D) {
    case 64: return launch_logits<64>(q, k, M, N, s_out, status, s);
    case 128: return launch_logits<128>(q, k, M, N, s_out, status, s);
    case 256: return launch_logits<256>(q, k, M, N, s_out, status, s);
  }
  return SL8_ERR_BAD_HEAD_DIM;
}

#ifdef SL8_TRACE
extern "C" int sl8_dbg_read_trace(long long* host_out, int n) {
  return (int)cudaMemcpyFromSymbol(host_out, sl8::g_trace, sizeof(long long) * n);
}
#endif

// ---- tensor-pipe peak probe ---------------------------------------------------------------
// Back-to-back tcgen05.mma (M128 N256, K = 32 bytes) on shared-memory operands that never
// change: no softmax, no loads in the loop.  Measures what the tensor pipe sustains for
// kind::i8 and kind::f16 on this GPU, the denominator for "fraction of INT8 peak".
namespace sl8 {
namespace {
template <bool I8>
__global__ void __launch_bounds__(128) tensor_peak_kernel(int iters, int n_cols, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int A_BYTES = 128 * 128, B_BYTES = 256 * 128;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + A_BYTES + B_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 4; i += 128)
    reinterpret_cast<uint32_t*>(smem)[i] = I8 ? (0x01fe02ffu * (i + 1)) : 0x3c003c00u;  // small ints / fp16 ones
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  fence_proxy_async_smem();
  if (threadIdx.x < 32) {
    tc_alloc(tmem_slot, 512);
    tc_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  if (threadIdx.x == 0) {
    const uint32_t idesc = I8 ? umma_idesc(2, 1, 1, 0, 0, 128, n_cols) : umma_idesc(1, 0, 0, 0, 0, 128, n_cols);
    const uint32_t a_u = smem_u32(smem), b_u = smem_u32(smem + A_BYTES);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint64_t da = umma_smem_desc(a_u + 32 * s, 16, 1024, kUmmaSw128);
        const uint64_t db = umma_smem_desc(b_u + 32 * s, 16, 1024, kUmmaSw128);
        if (I8) tc_mma_i8_ss(tmem + 256 * (it & 1), da, db, idesc, s > 0 ? 1u : 0u);
        else tc_mma_f16_ss(tmem + 256 * (it & 1), da, db, idesc, s > 0 ? 1u : 0u);
      }
    }
    tc_commit(bar);
  }
  mbar_wait(bar, 0, status);
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tc_dealloc(tmem, 512);
  }
}
}  // namespace
}  // namespace sl8

extern "C" int sl8_tensor_peak_probe(int kind_i8, int iters, double* ops_per_launch, void* workspace,
                                     size_t workspace_bytes, void* stream) {
  return sl8_tensor_peak_probe_n(kind_i8, 256, iters, ops_per_launch, workspace, workspace_bytes, stream);
}

extern "C" int sl8_tensor_peak_probe_n(int kind_i8, int n_cols, int iters, double* ops_per_launch, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  if (iters <= 0 || iters > (1 << 20)) return SL8_ERR_BAD_SHAPE;
  if (n_cols != 64 && n_cols != 128 && n_cols != 256) return SL8_ERR_BAD_SHAPE;
  if (workspace == nullptr || workspace_bytes < 256) return SL8_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int smem = 128 * 128 + 256 * 128 + 1024 + 64;
  const int grid = kNumSms;
  // K per instruction: 32 int8 or 16 halves (both 32 bytes)
  if (ops_per_launch) *ops_per_launch = 2.0 * 128 * n_cols * (kind_i8 ? 32 : 16) * 4.0 * iters * grid;
  if (kind_i8) {
    SL8_CUDA_TRY(cudaFuncSetAttribute(tensor_peak_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    tensor_peak_kernel<true><<<grid, 128, smem, s>>>(iters, n_cols, reinterpret_cast<int*>(workspace));
  } else {
    SL8_CUDA_TRY(cudaFuncSetAttribute(tensor_peak_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    tensor_peak_kernel<false><<<grid, 128, smem, s>>>(iters, n_cols, reinterpret_cast<int*>(workspace));
  }
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}
