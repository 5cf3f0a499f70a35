// Backward on the Blackwell tensor-core path (D = 64, 128): the same two atomic-free passes as
// bwd.cu -- the mathematics of superl8/autograd.py:29-45, pass structure of
// csrc/include/attn_bwd.cuh:156-331 (dQ) and :337-535 (dK / dV) -- with every contraction a
// tcgen05.mma kind::f16 on TMA-staged tiles and the accumulators in tensor memory.
//
// One kernel template serves both passes.  A block owns 128 "rows" and streams 128-"column"
// tiles past them:
//   dK/dV pass  rows = 128 keys of one (batch, KV head); columns = 128 queries of one query head
//               of the group (all heads of the group, all query tiles that see a key of the block)
//                 S^T  = K Q^T          (both operands from shared memory)
//                 dP^T = V dO^T
//                 P^T  = 2^(S^T scale log2e - lse log2e),  dS^T = P^T (dP^T - D_m)
//                 dV  += P^T dO         (P^T from tensor memory, dO tile read MN-major)
//                 dK  += dS^T Q         (dS^T from tensor memory, Q tile read MN-major)
//   dQ pass     rows = 128 queries of one (batch, query head); columns = 128 keys
//                 S = Q K^T, dP = dO V^T, dS = P (dP - D_m),  dQ += dS K
// Tensor memory (512 columns): S at [0,128), dP at [128,256), first accumulator at [256,256+D),
// second at [384,384+D).  P (16-bit pairs) overwrites the first 64 columns of S, dS those of dP.
// (The dQ pass has one accumulator and keeps a second S buffer at [384,512).)
// Ten warps: 0-7 compute (thread = row = tensor-memory lane; warps w and w + 4 share a row group:
// w forms P from S, w + 4 forms dS from P and dP), 8 = TMA producer (the fixed row tiles once, then
// the column tiles through two rings of stages, plus -- dK/dV pass -- the per-query lse / D_m of
// a column tile, which ride on one extra K step of the S and dP MMAs as {hi, lo} 16-bit pairs),
// 9 = tensor-memory allocation and MMA issue.  Per column tile the issuer queues S and
// dP, the compute warps turn S into P and then dP into dS, the issuer queues the accumulating
// MMAs behind them (and the next tile's S and dP between them) and frees the stage.
// Rows and columns past the end of a tensor arrive as zeros (TMA fill) and carry a statistic
// that makes P = dS = 0 there; the causal mask is the forward's bottom-right one (key n visible to
// query m iff n <= m + N - M), evaluated per element only on tiles that straddle the diagonal.
// Every mbarrier wait is bounded; on expiry the status word is raised and the block exits.
#include "sl8_common.cuh"

#include <type_traits>

namespace sl8 {
namespace {

SL8_TRACE_DEFINE()
#ifndef SL8_TRACE_PASS
#define SL8_TRACE_PASS 1      // which pass a trace build stamps: 0 = dQ, 1 = dK/dV
#endif
#define BTR(slot) do { if (DKV == (SL8_TRACE_PASS != 0)) TR(slot); } while (0)

constexpr int kBT = 128;                       // rows per block, columns per tile
constexpr int kComputeWarps = 8;               // warps w and w + 4 share the rows 32 (w & 3) .. + 32: w makes P, w + 4 makes dS
constexpr int kBtProducerWarp = kComputeWarps, kBtMmaWarp = kComputeWarps + 1;
constexpr int kBtThreads = 32 * (kComputeWarps + 2);
constexpr float kLog2eB = 1.4426950408889634f;

template <int D, bool DKV>
struct BtCfg {
  static constexpr int SUBS = 2 * D / 128;               // 64-channel (128-byte) sub-tiles of a row
  static constexpr int SUB_BYTES = kBT * 128;
  static constexpr int TILE_BYTES = kBT * 2 * D;
  static constexpr int KSTEPS = 2 * D / 32;              // MMA K steps over the head dimension
  // Column tiles travel in two rings.  B1 (Q in the dK/dV pass, K in the dQ pass) is read by the
  // tile's first MMA and by its last, so its stage comes back late: the dQ pass, which has the
  // room, gives it three stages (a reload is then two tiles ahead of its use).  B2 (dO / V) is
  // released after the dV MMA (dK/dV pass) or right after dP (dQ pass).
  // Two S buffers wherever tensor memory has the room: the dQ pass (one accumulator) and the
  // dK/dV pass at D = 64 (two 64-column accumulators).  With them the next tile's S is ready while
  // this tile is processed, and the B1 ring gets its third stage (shared memory has the room too).
  static constexpr bool DBL_S = !DKV || D == 64;
  static constexpr int NB1 = DBL_S ? 3 : 2;
  static constexpr int NB2 = 2;
  static constexpr int OFF_A1 = 0;
  static constexpr int OFF_A2 = OFF_A1 + TILE_BYTES;
  static constexpr int OFF_B1 = OFF_A2 + TILE_BYTES;
  static constexpr int OFF_B2 = OFF_B1 + NB1 * TILE_BYTES;
  // dK/dV pass: the per-query statistics ride on one extra K step of the S and dP MMAs.  Operand
  // tiles of 128 rows x 16 elements (no swizzle: 8-row x 16-byte core matrices, the two K chunks
  // 2048 bytes apart, 8-row groups 128 bytes apart): a constant one whose rows are {1, 1, 0, ...},
  // and per B1 stage one holding {hi, lo, 0, ...} of -lse / scale and one of -D_m per query.
  static constexpr int EXT_BYTES = 2 * (kBT / 8) * 128;
  static constexpr int OFF_EXT_ONES = OFF_B2 + NB2 * TILE_BYTES;
  static constexpr int OFF_EXT_S = OFF_EXT_ONES + EXT_BYTES;          // NB1 stages
  static constexpr int OFF_EXT_DP = OFF_EXT_S + NB1 * EXT_BYTES;      // NB1 stages
  static constexpr int OFF_BAR = DKV ? OFF_EXT_DP + NB1 * EXT_BYTES : OFF_EXT_ONES;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static_assert(SMEM <= 232448, "shared memory per block");
  static constexpr uint32_t COL_S = 0, COL_DP = 128, COL_ACC1 = 256;
  static constexpr uint32_t COL_ACC2 = D == 64 ? 320 : 384;                             // dK/dV pass: dK
  static constexpr uint32_t COL_S1 = 384;                                               // second S buffer (DBL_S)
};

struct BtArgs {
  const float* lse;
  const float* delta;
  void* out1;          // dK/dV pass: dV; dQ pass: dQ
  void* out2;          // dK/dV pass: dK
  int* status;
  int Hq, Hkv, M, N;
  int causal;
  float scale;
};

// S_FULL: with one S buffer [0] completes a phase per tile; with two (DBL_S) tile i uses [i & 1].
// P_FULL in the dK/dV pass: [h] = P of the tile's queries [64 h, 64 h + 64), a phase per tile.
enum BtBar { FIX_FULL = 0, ACC_DONE, DP_FULL, P_READ, DS_FULL, P_FULL, S_FULL = P_FULL + 2, B1_FULL = S_FULL + 2, B1_EMPTY = B1_FULL + 3,
             B2_FULL = B1_EMPTY + 3, B2_EMPTY = B2_FULL + 2, BT_NUM_BARS = B2_EMPTY + 2 };

template <int D, typename VT, bool DKV>
__global__ void __launch_bounds__(kBtThreads, 1) bwd_tc_kernel(const __grid_constant__ CUtensorMap a1_map,
                                                              const __grid_constant__ CUtensorMap a2_map,
                                                              const __grid_constant__ CUtensorMap b1_map,
                                                              const __grid_constant__ CUtensorMap b2_map,
                                                              const __grid_constant__ CUtensorMap o1_map,
                                                              const __grid_constant__ CUtensorMap o2_map, BtArgs a) {
  using C = BtCfg<D, DKV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BT_NUM_BARS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = a.Hq / a.Hkv;
  const int diag = a.causal ? a.N - a.M : 0;
  // rows of this block, and the walk over column tiles
  // Launch order = heaviest blocks first when causal.  dK/dV pass: grid (batch * Hkv, key blocks) --
  // the early key blocks of every head, which see the most queries, start first; dQ pass: grid
  // (query blocks, batch * Hq) with the late query blocks first.
  const int fixed_bh = DKV ? blockIdx.x : blockIdx.y;    // dK/dV: batch * Hkv + kv head; dQ: batch * Hq + query head
  const int b = DKV ? fixed_bh / a.Hkv : fixed_bh / a.Hq;
  const int kvh = DKV ? fixed_bh % a.Hkv : (fixed_bh % a.Hq) / G;
  const int row_block = DKV ? blockIdx.y * kBT : (a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x) * kBT;
  int col_begin, tiles_per_head, heads;
  if (DKV) {
    // first query that sees a key of this block: n <= m + diag
    col_begin = a.causal ? max(0, row_block - diag) / kBT * kBT : 0;
    tiles_per_head = col_begin < a.M ? (a.M - col_begin + kBT - 1) / kBT : 0;
    heads = G;
  } else {
    col_begin = 0;
    const int n_end = a.causal ? max(0, min(a.N, row_block + kBT + diag)) : a.N;
    tiles_per_head = (n_end + kBT - 1) / kBT;
    heads = 1;
  }
  const int total = heads * tiles_per_head;
  // head (TMA coordinate 2) and first column of tile i
  auto tile_head = [&](int i) { return DKV ? b * a.Hq + kvh * G + i / tiles_per_head : b * a.Hkv + kvh; };
  auto tile_col = [&](int i) { return col_begin + (i % tiles_per_head) * kBT; };

  if (threadIdx.x == 0) {
    BTR(8188);
    mbar_init(&bars[FIX_FULL], 1);
    mbar_init(&bars[ACC_DONE], 1);
    mbar_init(&bars[DP_FULL], 1);
    mbar_init(&bars[P_FULL], 4);     // the P warps
    mbar_init(&bars[P_FULL + 1], 4);
    mbar_init(&bars[P_READ], 4);     // the dS warps, once P is in their registers (dK/dV pass)
    mbar_init(&bars[DS_FULL], 4);    // the dS warps
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[S_FULL + i], 1);
      mbar_init(&bars[B2_FULL + i], 1);
      mbar_init(&bars[B2_EMPTY + i], 1);
    }
    for (int i = 0; i < C::NB1; ++i) {
      mbar_init(&bars[B1_FULL + i], DKV ? 2 : 1);   // the tile bytes, and (dK/dV) the lse / D_m rows of the tile
      mbar_init(&bars[B1_EMPTY + i], 1);
    }
    mbar_fence_init();
  }
  if (warp == kBtMmaWarp) {
    tc_alloc(tmem_slot, 512);
    tc_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  bool ok = true;
  if (threadIdx.x == 0) BTR(8189);

  if (warp == kBtProducerWarp) {
    // ======================= producer =======================
    const float inv_scale = 1.f / a.scale;
    if (lane == 0) {
      tma_prefetch_desc(&a1_map);
      tma_prefetch_desc(&a2_map);
      tma_prefetch_desc(&b1_map);
      tma_prefetch_desc(&b2_map);
      mbar_expect_tx(&bars[FIX_FULL], 2 * C::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::SUBS; ++c) {
        tma_load_3d(smem + C::OFF_A1 + c * C::SUB_BYTES, &a1_map, &bars[FIX_FULL], 64 * c, row_block, fixed_bh);
        tma_load_3d(smem + C::OFF_A2 + c * C::SUB_BYTES, &a2_map, &bars[FIX_FULL], 64 * c, row_block, fixed_bh);
      }
    }
    if (DKV) {
      // the statistic tiles: zero everything once (only elements 0 and 1 of a row ever change)
      uint32_t* ext = reinterpret_cast<uint32_t*>(smem + C::OFF_EXT_ONES);
      for (int w = lane; w < (1 + 2 * C::NB1) * C::EXT_BYTES / 4; w += 32) ext[w] = 0u;
      __syncwarp();
      for (int r = lane; r < kBT; r += 32)
        *reinterpret_cast<uint32_t*>(smem + C::OFF_EXT_ONES + (r >> 3) * 128 + (r & 7) * 16) = pack2<VT>(1.f, 1.f);
      fence_proxy_async_smem();
      __syncwarp();
    }
    for (int i = 0; i < total && ok; ++i) {
      const int s1 = i % C::NB1, s2 = i % C::NB2;
      const int head = tile_head(i), col = tile_col(i);
      // B2 first: its stage comes back earlier
      if (i >= C::NB2) ok = mbar_wait(&bars[B2_EMPTY + s2], ((i / C::NB2) - 1) & 1, a.status);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(&bars[B2_FULL + s2], C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::SUBS; ++c)
          tma_load_3d(smem + C::OFF_B2 + s2 * C::TILE_BYTES + c * C::SUB_BYTES, &b2_map, &bars[B2_FULL + s2], 64 * c, col, head);
      }
      if (i >= C::NB1) ok = mbar_wait(&bars[B1_EMPTY + s1], ((i / C::NB1) - 1) & 1, a.status);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(&bars[B1_FULL + s1], C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::SUBS; ++c)
          tma_load_3d(smem + C::OFF_B1 + s1 * C::TILE_BYTES + c * C::SUB_BYTES, &b1_map, &bars[B1_FULL + s1], 64 * c, col, head);
      }
      if (DKV) {
        // per-query statistics of the tile's columns as {hi, lo} 16-bit pairs: x = -lse / scale (so
        // that (S + x) scale log2e is the exponent; a large negative number where P must be 0:
        // queries past M, rows without a visible key) and -D_m
        const float big = std::is_same<VT, __half>::value ? -60000.f : -1e30f;
#pragma unroll
        for (int r = lane; r < kBT; r += 32) {
          const int m = col + r;
          float x = big, d = 0.f;
          if (m < a.M) {
            const float v = __ldg(a.lse + (int64_t)head * a.M + m);
            x = (v > -INFINITY) ? fmaxf(-v * inv_scale, big) : big;
            d = -__ldg(a.delta + (int64_t)head * a.M + m);
          }
          const float xh = to_f32<VT>(from_f32<VT>(x)), dh = to_f32<VT>(from_f32<VT>(d));
          const uint32_t off = s1 * C::EXT_BYTES + (r >> 3) * 128 + (r & 7) * 16;
          *reinterpret_cast<uint32_t*>(smem + C::OFF_EXT_S + off) = pack2<VT>(xh, x - xh);
          *reinterpret_cast<uint32_t*>(smem + C::OFF_EXT_DP + off) = pack2<VT>(dh, d - dh);
        }
        fence_proxy_async_smem();     // the MMAs read these tiles through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B1_FULL + s1]);
      }
    }
  } else if (warp == kBtMmaWarp) {
    // ======================= MMA issuer =======================
    // The whole warp walks the loop and polls the barriers; one elected lane issues and commits.
    // Order of issue (the tensor pipe executes in this order, which is what lets a later MMA
    // overwrite the tensor-memory operand of an earlier one):
    //   one S buffer (dK/dV pass, D = 128)   S_0 dP_0 | dV_i S_{i+1} dK_i dP_{i+1} | ...   (S_{i+1} reuses the columns P_i sat in)
    //   two S buffers (dQ pass)              S_0 dP_0 S_1 | dQ_i dP_{i+1} S_{i+2} | ...
    //   two S buffers (dK/dV pass, D = 64)   S_0 dP_0 S_1 | dV_i dK_i dP_{i+1} S_{i+2} | ...
    constexpr uint32_t vfmt = std::is_same<VT, __nv_bfloat16>::value ? 1u : 0u;
    const uint32_t idesc_s = umma_idesc(1, vfmt, vfmt, 0, 0, kBT, kBT);
    const uint32_t idesc_acc = umma_idesc(1, vfmt, vfmt, 0, 1, kBT, D);
    const uint64_t da1 = umma_smem_desc(smem_u32(smem + C::OFF_A1), 16, 1024, kUmmaSw128);
    const uint64_t da2 = umma_smem_desc(smem_u32(smem + C::OFF_A2), 16, 1024, kUmmaSw128);
    // column tiles, viewed K-major (for S and dP) and MN-major (for the accumulating MMAs)
    const uint64_t db1_k = umma_smem_desc(smem_u32(smem + C::OFF_B1), 16, 1024, kUmmaSw128);
    const uint64_t db2_k = umma_smem_desc(smem_u32(smem + C::OFF_B2), 16, 1024, kUmmaSw128);
    const uint64_t db1_mn = umma_smem_desc(smem_u32(smem + C::OFF_B1), C::SUB_BYTES, 1024, kUmmaSw128);
    const uint64_t db2_mn = umma_smem_desc(smem_u32(smem + C::OFF_B2), C::SUB_BYTES, 1024, kUmmaSw128);
    // statistic tiles (dK/dV pass): K-major, no swizzle, K chunks 2048 bytes apart, 8-row groups 128
    const uint64_t de_ones = umma_smem_desc(smem_u32(smem + C::OFF_EXT_ONES), 2048, 128, 0);
    const uint64_t de_s = umma_smem_desc(smem_u32(smem + C::OFF_EXT_S), 2048, 128, 0);
    const uint64_t de_dp = umma_smem_desc(smem_u32(smem + C::OFF_EXT_DP), 2048, 128, 0);
    auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool {
      const bool r = __all_sync(0xffffffffu, mbar_wait(bar, parity, a.status));
      tc_fence_after();
      return r;
    };
    auto issue_s = [&](int i) {     // S_i = A1 B1_i^T
      if (elect_one()) {
        const int s1 = i % C::NB1;
        const uint32_t col = (C::DBL_S && (i & 1)) ? C::COL_S1 : C::COL_S;
#pragma unroll
        for (int k = 0; k < C::KSTEPS; ++k) {
          const uint32_t off = (32 * k / 128) * C::SUB_BYTES + (32 * k % 128);
          tc_mma_f16_ss(tmem + col, umma_desc_advance(da1, off), umma_desc_advance(db1_k, s1 * C::TILE_BYTES + off),
                        idesc_s, k > 0 ? 1u : 0u);
        }
        if (DKV) tc_mma_f16_ss(tmem + col, de_ones, umma_desc_advance(de_s, s1 * C::EXT_BYTES), idesc_s, 1u);   // S -= lse / scale
        tc_commit(&bars[S_FULL + (C::DBL_S ? (i & 1) : 0)]);
      }
      __syncwarp();
    };
    auto issue_dp = [&](int i) {    // dP_i = A2 B2_i^T (dQ pass: nothing else reads the B2 stage)
      if (elect_one()) {
        const int s2 = i % C::NB2;
#pragma unroll
        for (int k = 0; k < C::KSTEPS; ++k) {
          const uint32_t off = (32 * k / 128) * C::SUB_BYTES + (32 * k % 128);
          tc_mma_f16_ss(tmem + C::COL_DP, umma_desc_advance(da2, off), umma_desc_advance(db2_k, s2 * C::TILE_BYTES + off),
                        idesc_s, k > 0 ? 1u : 0u);
        }
        if (DKV) tc_mma_f16_ss(tmem + C::COL_DP, de_ones, umma_desc_advance(de_dp, (i % C::NB1) * C::EXT_BYTES), idesc_s, 1u);   // dP -= D_m
        tc_commit(&bars[DP_FULL]);
        if (!DKV) tc_commit(&bars[B2_EMPTY + s2]);
      }
      __syncwarp();
    };
    // dV += P_i^T dO_i over the tile's queries [64 h, 64 h + 64) (P over columns [32 h, 32 h + 32) of S;
    // B2 read MN-major): the first half is queued while the P warps still work on the second.  The
    // second half frees the B2 stage.
    auto issue_dv_half = [&](int i, int h) {
      if (elect_one()) {
        const int s2 = i % C::NB2;
#pragma unroll
        for (int kk = 4 * h; kk < 4 * h + 4; ++kk)
          tc_mma_f16_ts(tmem + C::COL_ACC1, tmem + ((C::DBL_S && (i & 1)) ? C::COL_S1 : C::COL_S) + 8 * kk,
                        umma_desc_advance(db2_mn, s2 * C::TILE_BYTES + kk * 2048), idesc_acc, (i > 0 || kk > 0) ? 1u : 0u);
        if (h == 1) tc_commit(&bars[B2_EMPTY + s2]);
      }
      __syncwarp();
    };
    auto issue_last = [&](int i) {  // dK += dS_i^T Q_i  /  dQ += dS_i K_i (dS over the first 64 columns of dP); frees the B1 stage
      if (elect_one()) {
        const int s1 = i % C::NB1;
#pragma unroll
        for (int kk = 0; kk < kBT / 16; ++kk)
          tc_mma_f16_ts(tmem + (DKV ? C::COL_ACC2 : C::COL_ACC1), tmem + C::COL_DP + 8 * kk,
                        umma_desc_advance(db1_mn, s1 * C::TILE_BYTES + kk * 2048), idesc_acc, (i > 0 || kk > 0) ? 1u : 0u);
        tc_commit(&bars[B1_EMPTY + s1]);
        if (i == total - 1) tc_commit(&bars[ACC_DONE]);
      }
      __syncwarp();
    };
    auto wait_b1 = [&](int i) { return wait_all(&bars[B1_FULL + i % C::NB1], (i / C::NB1) & 1); };
    auto wait_b2 = [&](int i) { return wait_all(&bars[B2_FULL + i % C::NB2], (i / C::NB2) & 1); };
    ok = wait_all(&bars[FIX_FULL], 0);
    if (ok && total > 0) {
      ok = wait_b1(0);
      if (ok) issue_s(0);
      if (ok) ok = wait_b2(0);
      if (ok) issue_dp(0);
      if (C::DBL_S && ok && total > 1) {
        ok = wait_b1(1);
        if (ok) issue_s(1);
      }
    }
    for (int i = 0; i < total && ok; ++i) {
      if (lane == 0 && i < 250) BTR(4096 + 8 * i + 0);
      if (DKV) {
        ok = wait_all(&bars[P_FULL + 0], i & 1);
        if (!ok) break;
        if (lane == 0 && i < 250) BTR(4096 + 8 * i + 1);
        issue_dv_half(i, 0);
        ok = wait_all(&bars[P_FULL + 1], i & 1);
        if (!ok) break;
        issue_dv_half(i, 1);
        if (lane == 0 && i < 250) BTR(4096 + 8 * i + 2);
        if (!C::DBL_S && i + 1 < total) {
          ok = wait_b1(i + 1);
          if (ok) ok = wait_all(&bars[P_READ], i & 1);     // the dS warps hold P_i: its columns may be overwritten
          if (!ok) break;
          if (lane == 0 && i < 250) BTR(4096 + 8 * i + 3);
          issue_s(i + 1);
        }
        if (lane == 0 && i < 250) BTR(4096 + 8 * i + 4);
      }
      ok = wait_all(&bars[DS_FULL], i & 1);
      if (!ok) break;
      if (lane == 0 && i < 250) BTR(4096 + 8 * i + 5);
      issue_last(i);
      if (i + 1 < total) {
        ok = wait_b2(i + 1);
        if (!ok) break;
        issue_dp(i + 1);
      }
      if (lane == 0 && i < 250) BTR(4096 + 8 * i + 6);
      if (C::DBL_S && i + 2 < total) {
        ok = wait_b1(i + 2);
        if (!ok) break;
        issue_s(i + 2);      // into the S buffer the compute warps have finished with (DS_FULL of tile i)
      }
      if (lane == 0 && i < 250) BTR(4096 + 8 * i + 7);
    }
  } else {
    // ======================= compute / epilogue =======================
    // Warps 0-3 ("P warps") turn S into P = 2^(S scale log2e - lse log2e): one exponential per
    // element, work for the special-function unit.  Warps 4-7 ("dS warps") read that P back from
    // tensor memory and turn dP into dS = P (dP - D_m): multiply-add work.  A scheduler hosts one
    // warp of each kind, so the two kinds of work overlap instead of queueing in one warp, and
    // the P warps move on to the next tile's S while the dS warps finish this one.  There is no
    // row reduction in the backward (lse is an input), so the two kinds never exchange more than
    // P itself.  P (16-bit pairs) overwrites columns [0, 64) of its S buffer, dS those of dP --
    // chunk c of 32 columns lands on columns [16 c, 16 c + 16), which the same thread has
    // already read.
    const int cw = warp & 3, half = warp >> 2;                // row group; 0 = P warp, 1 = dS warp
    const int row = 32 * cw + lane;
    const int grow = row_block + row;                         // key (dK/dV) or query (dQ) of this thread
    const uint32_t t_row = tmem + ((uint32_t)(32 * cw) << 16);
    const float scale_log2 = a.scale * kLog2eB;
    float my_nlse2 = -INFINITY, my_delta = 0.f;               // dQ pass: per-row statistics (-lse log2e; -inf: P = 0)
    if (!DKV && grow < a.M) {
      const float v = __ldg(a.lse + (int64_t)fixed_bh * a.M + grow);
      my_nlse2 = (v > -INFINITY) ? -v * kLog2eB : -INFINITY;
      my_delta = __ldg(a.delta + (int64_t)fixed_bh * a.M + grow);
    }
    for (int i = 0; i < total; ++i) {
      const int col = tile_col(i);
      const uint32_t t_s = t_row + ((C::DBL_S && (i & 1)) ? C::COL_S1 : C::COL_S);
      if (warp == 0 && lane == 0 && i < 250) BTR(8 * i + 0);
      if (warp == 4 && lane == 0 && i < 250) BTR(2048 + 8 * i + 0);
      if (half == 0) {
        // ======== P warp ========
        ok = C::DBL_S ? mbar_wait(&bars[S_FULL + (i & 1)], (i >> 1) & 1, a.status) : mbar_wait(&bars[S_FULL], i & 1, a.status);
        if (!ok) break;
        tc_fence_after();
        if (warp == 0 && lane == 0 && i < 250) BTR(8 * i + 1);
        // does the tile straddle the diagonal?  dK/dV: key = grow, query = col + c; dQ: query = grow, key = col + c
        // (dQ pass: also the tile that runs past the last key -- its zero-filled keys still give P > 0)
        const bool need_mask = DKV ? (a.causal && col + diag < row_block + kBT - 1)
                                   : ((a.causal && col + kBT - 1 > row_block + diag) || col + kBT > a.N);
        const int key_limit = a.causal ? min(a.N, grow + diag + 1) : a.N;   // dQ pass: keys [0, key_limit) are visible
#pragma unroll
        for (int h = 0; h < 2; ++h) {            // two chunks of 32 columns at a time
          uint32_t s[64], pp[32];
          tc_ld32(t_s + 64 * h, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
          tc_ld32(t_s + 64 * h + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
          tc_wait_ld();
          tc_regs_ready(*reinterpret_cast<uint32_t(*)[32]>(&s[0]));
          tc_regs_ready(*reinterpret_cast<uint32_t(*)[32]>(&s[32]));
          const int colw = col + 64 * h;
#pragma unroll
          for (int e = 0; e < 64; e += 2) {
            float p0, p1;
            if (DKV) {
              // (S already carries -lse / scale of its query: the extra K step of the S MMA)
              p0 = ex2_approx(__uint_as_float(s[e]) * scale_log2);
              p1 = ex2_approx(__uint_as_float(s[e + 1]) * scale_log2);
              if (need_mask) {
                p0 = (grow <= colw + e + diag) ? p0 : 0.f;
                p1 = (grow <= colw + e + 1 + diag) ? p1 : 0.f;
              }
            } else {
              p0 = ex2_approx(fmaf(__uint_as_float(s[e]), scale_log2, my_nlse2));
              p1 = ex2_approx(fmaf(__uint_as_float(s[e + 1]), scale_log2, my_nlse2));
              if (need_mask) {
                p0 = (colw + e < key_limit) ? p0 : 0.f;
                p1 = (colw + e + 1 < key_limit) ? p1 : 0.f;
              }
            }
            pp[e >> 1] = pack2<VT>(p0, p1);
          }
          tc_st16(t_s + 32 * h, *reinterpret_cast<uint32_t(*)[16]>(&pp[0]));
          tc_st16(t_s + 32 * h + 16, *reinterpret_cast<uint32_t(*)[16]>(&pp[16]));
          if (DKV || h == 1) {     // dK/dV pass: each half of P is handed over on its own
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[P_FULL + (DKV ? h : 0)]);
          }
        }
        if (warp == 0 && lane == 0 && i < 250) BTR(8 * i + 2);
      } else {
        // ======== dS warp ========
        ok = mbar_wait(&bars[P_FULL], i & 1, a.status);
        if (ok && DKV) ok = mbar_wait(&bars[P_FULL + 1], i & 1, a.status);
        if (!ok) break;
        tc_fence_after();
        if (warp == 4 && lane == 0 && i < 250) BTR(2048 + 8 * i + 1);
        uint32_t pp[64];
        tc_ld32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&pp[0]));
        tc_ld32(t_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&pp[32]));
        tc_wait_ld();
        tc_regs_ready(*reinterpret_cast<uint32_t(*)[32]>(&pp[0]));
        tc_regs_ready(*reinterpret_cast<uint32_t(*)[32]>(&pp[32]));
        if (DKV) {
          // P is in registers: the issuer may let the next tile's S overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[P_READ]);
        }
        ok = mbar_wait(&bars[DP_FULL], i & 1, a.status);
        if (!ok) break;
        tc_fence_after();
        if (warp == 4 && lane == 0 && i < 250) BTR(2048 + 8 * i + 2);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t dp[64], ds[32];
          tc_ld32(t_row + C::COL_DP + 64 * h, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
          tc_ld32(t_row + C::COL_DP + 64 * h + 32, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
          tc_wait_ld();
          tc_regs_ready(*reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
          tc_regs_ready(*reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
#pragma unroll
          for (int e = 0; e < 64; e += 2) {
            const float2 p = unpack2<VT>(pp[32 * h + (e >> 1)]);
            // (dK/dV pass: dP already carries -D_m of its query)
            const float dl = DKV ? 0.f : my_delta;
            ds[e >> 1] = pack2<VT>(p.x * (__uint_as_float(dp[e]) - dl), p.y * (__uint_as_float(dp[e + 1]) - dl));
          }
          tc_st16(t_row + C::COL_DP + 32 * h, *reinterpret_cast<uint32_t(*)[16]>(&ds[0]));
          tc_st16(t_row + C::COL_DP + 32 * h + 16, *reinterpret_cast<uint32_t(*)[16]>(&ds[16]));
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[DS_FULL]);
        if (warp == 4 && lane == 0 && i < 250) BTR(2048 + 8 * i + 3);
      }
    }
    // ---- epilogue: accumulators -> 16-bit rows ----
    if (warp == 0 && lane == 0) BTR(8185);
    if (ok && total > 0) ok = mbar_wait(&bars[ACC_DONE], 0, a.status);
    if (warp == 0 && lane == 0) BTR(8186);
    if (ok) {
      tc_fence_after();
      const int rows_total = DKV ? a.N : a.M;
      VT* o1 = reinterpret_cast<VT*>(a.out1) + ((int64_t)fixed_bh * rows_total + grow) * D;
      VT* o2 = DKV ? reinterpret_cast<VT*>(a.out2) + ((int64_t)fixed_bh * rows_total + grow) * D : nullptr;
#pragma unroll 1
      for (int which = 0; which < (DKV ? 2 : 1); ++which) {
        const float f = (DKV && which == 0) ? 1.f : a.scale;     // dV unscaled; dK, dQ times the softmax scale
        VT* dst_row = which == 0 ? o1 : o2;
        const uint32_t t_acc = t_row + (which == 0 ? C::COL_ACC1 : C::COL_ACC2);
        if (D == 128) {
          // This warp's 32 rows x 64 channels are staged in shared memory (the B2 ring is free:
          // every MMA has completed) in the 128-byte-swizzled layout of the output tensor map --
          // 16-byte chunk j of row r at chunk j ^ (r & 7) -- and leave as one tile store; rows past
          // the end of the tensor are dropped by the copy engine.
          uint8_t* const box = smem + C::OFF_B2 + which * C::TILE_BYTES + half * C::SUB_BYTES + cw * (32 * 128);
#pragma unroll 1
          for (int c = 2 * half; c < 2 * half + 2; ++c) {
            uint32_t o[32];
            if (total > 0) {
              tc_ld32(t_acc + 32 * c, o);
              tc_wait_ld();
              tc_regs_ready(o);
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = 0u;
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack2<VT>(__uint_as_float(o[8 * v + 0]) * f, __uint_as_float(o[8 * v + 1]) * f);
              w.y = pack2<VT>(__uint_as_float(o[8 * v + 2]) * f, __uint_as_float(o[8 * v + 3]) * f);
              w.z = pack2<VT>(__uint_as_float(o[8 * v + 4]) * f, __uint_as_float(o[8 * v + 5]) * f);
              w.w = pack2<VT>(__uint_as_float(o[8 * v + 6]) * f, __uint_as_float(o[8 * v + 7]) * f);
              *reinterpret_cast<uint4*>(box + lane * 128 + ((((c & 1) * 4 + v) ^ (lane & 7)) << 4)) = w;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row_block + 32 * cw < rows_total) {
            tma_store_3d(which == 0 ? &o1_map : &o2_map, box, 64 * half, row_block + 32 * cw, fixed_bh);
            tma_store_commit();
          }
        } else {
#pragma unroll 1
          for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {   // this warp's half of the channels
            uint32_t o[32];
            if (total > 0) {
              tc_ld32(t_acc + 32 * c, o);
              tc_wait_ld();
              tc_regs_ready(o);
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = 0u;
            }
            if (grow < rows_total) {
              uint4* dst = reinterpret_cast<uint4*>(dst_row + 32 * c);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 w;
                w.x = pack2<VT>(__uint_as_float(o[8 * v + 0]) * f, __uint_as_float(o[8 * v + 1]) * f);
                w.y = pack2<VT>(__uint_as_float(o[8 * v + 2]) * f, __uint_as_float(o[8 * v + 3]) * f);
                w.z = pack2<VT>(__uint_as_float(o[8 * v + 4]) * f, __uint_as_float(o[8 * v + 5]) * f);
                w.w = pack2<VT>(__uint_as_float(o[8 * v + 6]) * f, __uint_as_float(o[8 * v + 7]) * f);
                dst[v] = w;
              }
            }
          }
        }
      }
      if (D == 128 && lane == 0) tma_store_wait_read();   // the engine has read this warp's staged tiles
      if (warp == 0 && lane == 0) BTR(8187);
    }
    tc_fence_before();
  }

  // ---- teardown: every role arrives here, on success and on a timed-out wait ----
  __syncthreads();
  if (warp == kBtMmaWarp) {
    tc_fence_after();
    tc_dealloc(tmem, 512);
  }
}

template <int D, typename VT>
int launch_bwd_tc(const sl8_bwd_params* p, float* delta, int* status, cudaStream_t stream) {
  CUtensorMap q_map, k_map, v_map, do_map;
  const uint64_t hq = (uint64_t)p->B * p->Hq, hkv = (uint64_t)p->B * p->Hkv;
  int rc = sl8_make_tmap_3d(&q_map, p->q, 2, D, p->M, hq, 64, kBT, 128);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&do_map, p->dout, 2, D, p->M, hq, 64, kBT, 128);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&k_map, p->k, 2, D, p->N, hkv, 64, kBT, 128);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&v_map, p->v, 2, D, p->N, hkv, 64, kBT, 128);
  // gradient tiles leave through the copy engine: 32 rows (one compute warp) x 64 channels per store
  CUtensorMap dq_map, dk_map, dv_map;
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&dq_map, p->dq, 2, D, p->M, hq, 64, 32, 128);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&dk_map, p->dk, 2, D, p->N, hkv, 64, 32, 128);
  if (rc == SL8_OK) rc = sl8_make_tmap_3d(&dv_map, p->dv, 2, D, p->N, hkv, 64, 32, 128);
  if (rc != SL8_OK) return rc;
  BtArgs a{};
  a.lse = p->lse; a.delta = delta; a.status = status;
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N; a.causal = p->causal; a.scale = p->softmax_scale;
  constexpr int smem_dkv = BtCfg<D, true>::SMEM, smem_dq = BtCfg<D, false>::SMEM;
  SL8_CUDA_TRY(cudaFuncSetAttribute(bwd_tc_kernel<D, VT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkv));
  SL8_CUDA_TRY(cudaFuncSetAttribute(bwd_tc_kernel<D, VT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq));
  // dQ pass: rows = queries (A1 = Q, A2 = dO), columns = keys (B1 = K, B2 = V)
  a.out1 = p->dq; a.out2 = nullptr;
  bwd_tc_kernel<D, VT, false><<<dim3((p->M + kBT - 1) / kBT, (unsigned)hq), kBtThreads, smem_dq, stream>>>(
      q_map, do_map, k_map, v_map, dq_map, dq_map, a);
  // dK/dV pass: rows = keys (A1 = K, A2 = V), columns = queries (B1 = Q, B2 = dO)
  a.out1 = p->dv; a.out2 = p->dk;
  bwd_tc_kernel<D, VT, true><<<dim3((unsigned)hkv, (p->N + kBT - 1) / kBT), kBtThreads, smem_dkv, stream>>>(
      k_map, v_map, q_map, do_map, dv_map, dk_map, a);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

}  // namespace
}  // namespace sl8

#ifdef SL8_TRACE
extern "C" int sl8_dbg_read_trace_bwd(long long* host_out, int n) {
  return (int)cudaMemcpyFromSymbol(host_out, sl8::g_trace, sizeof(long long) * n);
}
#endif

// The two tensor-memory passes of the backward (D = 64 or 128); parameters were validated and
// D_m written to `delta` by sl8_attn_bwd (bwd.cu).
int sl8_bwd_tc(const sl8_bwd_params* p, float* delta, int* status, cudaStream_t s) {
  using namespace sl8;
  if (p->D == 128)
    return p->dtype == SL8_F16 ? launch_bwd_tc<128, __half>(p, delta, status, s)
                               : launch_bwd_tc<128, __nv_bfloat16>(p, delta, status, s);
  if (p->D == 64)
    return p->dtype == SL8_F16 ? launch_bwd_tc<64, __half>(p, delta, status, s)
                               : launch_bwd_tc<64, __nv_bfloat16>(p, delta, status, s);
  return SL8_ERR_UNSUPPORTED;
}
