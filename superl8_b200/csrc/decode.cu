// Split-KV decode: one query row per sequence against an int8 K cache with
// per-token fp32 scales and an fp16 V cache.
//
// Same mathematics as the reference's flash-decoding pair
// (csrc/include/attn_decode.cuh:47-132 split kernel, :430-466 combine): split s
// owns keys [s*per, min(len, (s+1)*per)), reduces them to a partial
// (O[D], running max m in the exp2 domain, sum l), and a second kernel merges the
// partials by log-sum-exp.  logit = float(int32 q.k) * q_scale * k_scale[n].
//
// Mapping to the machine (the operation is HBM bound: D + 4 + 2D bytes per key
// and KV head):
//  * one block serves ALL query heads of a KV head (the GQA group), so K and V
//    cross HBM once per KV head, not once per query head as in the reference
//    (attn_decode.cuh:65-66 puts one warp on every query head);
//  * a producer warp streams 64-key K and V tiles with TMA into a ring of
//    128-byte-swizzled shared-memory stages (several tiles in flight per block,
//    two or three blocks per SM);
//  * four consumer warps take 16 keys of every tile each: q.k^T as
//    mma.sync m16n8k32 (int8 -> int32, heads on the M axis), the online softmax in
//    fp32 on the accumulator fragments, P.V as mma.sync m16n8k16 with P rounded to
//    fp16; each warp keeps its own (m, l, O) and the four are merged once at the end.
#include "sl8_common.cuh"
#include "sl8_mma.cuh"

#include <mutex>

namespace sl8 {
namespace {

constexpr int kDecTile = 64;          // keys per pipeline stage
constexpr int kDecConsumerWarps = 4;  // 16 keys of a tile each
constexpr int kDecThreads = 32 * (kDecConsumerWarps + 1);
constexpr int kDecHeadsPerBlock = 16; // M of the mma tile

// V8: the V cache is int8 with one fp32 scale per (batch, KV head, channel).
template <int D, bool V8>
struct DecodeCfg {
  static constexpr int K_ROW_BYTES = D < 128 ? D : 128;
  static constexpr int K_SUBS = D / K_ROW_BYTES;
  static constexpr int K_SW_BITS = K_ROW_BYTES == 128 ? 3 : (K_ROW_BYTES == 64 ? 2 : 1);
  static constexpr int V_ELEM = V8 ? 1 : 2;
  static constexpr int V_ROW_BYTES = (V_ELEM * D) < 128 ? V_ELEM * D : 128;
  static constexpr int V_SUBS = V_ELEM * D / V_ROW_BYTES;
  static constexpr int V_SW_BITS = V_ROW_BYTES == 128 ? 3 : (V_ROW_BYTES == 64 ? 2 : 1);
  static constexpr int K_BYTES = kDecTile * D;
  static constexpr int V_BYTES = kDecTile * D * V_ELEM;
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
  static constexpr int STAGES = D == 256 ? 3 : 4;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct DecodeArgs {
  const int8_t* q;
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;   // int8-V cache only: [B, Hkv, D]
  const int32_t* context_lens;
  float* o_part;
  float* m_part;
  float* l_part;
  int* status;
  int B, Hq, Hkv, N, per, n_splits;
};

// Blocks per SM the register budget must allow: two with an fp16 V (96 KB of stages each at
// D = 128; 168 registers is the most two 5-warp blocks can have), three with an int8 V (64 KB).
template <int D, bool V8>
__global__ void __launch_bounds__(kDecThreads, D > 128 ? 1 : (V8 ? 3 : 2)) decode_split_kernel(const __grid_constant__ CUtensorMap k_map,
                                                                   const __grid_constant__ CUtensorMap v_map,
                                                                   DecodeArgs a) {
  using C = DecodeCfg<D, V8>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + C::STAGES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x;
  const int bkv = blockIdx.y;              // b * Hkv + hkv
  const int hgroup = blockIdx.z;           // 16 query heads of the GQA group per block
  const int G = a.Hq / a.Hkv;
  const int b = bkv / a.Hkv, hkv = bkv % a.Hkv;
  const int len = a.context_lens ? min(max(a.context_lens[b], 0), a.N) : a.N;
  const int n0 = split * a.per;
  const int n1 = min(len, n0 + a.per);
  const int64_t BHq = (int64_t)a.B * a.Hq;
  const int64_t bhq0 = (int64_t)b * a.Hq + (int64_t)hkv * G + hgroup * kDecHeadsPerBlock;
  const int heads_here = min(kDecHeadsPerBlock, G - hgroup * kDecHeadsPerBlock);

  if (n1 <= n0) {  // empty split: sentinel only (the combine skips it)
    if (threadIdx.x < heads_here) {
      a.m_part[(int64_t)split * BHq + bhq0 + threadIdx.x] = kNegSentinel;
      a.l_part[(int64_t)split * BHq + bhq0 + threadIdx.x] = 0.f;
    }
    return;
  }
  const int ntiles = (n1 - n0 + kDecTile - 1) / kDecTile;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], kDecConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();

  bool ok = true;
  float m_run[2] = {kNegSentinel, kNegSentinel};
  float l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  if (warp == kDecConsumerWarps) {
    // ---------------- producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
      int issued = 0;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int st = i % C::STAGES;
        if (i >= C::STAGES) ok = mbar_wait(&empty_bar[st], ((i / C::STAGES) - 1) & 1, a.status);
        if (!ok) break;
        uint8_t* kd = smem + st * C::STAGE_BYTES;
        uint8_t* vd = kd + C::K_BYTES;
        mbar_expect_tx(&full_bar[st], C::STAGE_BYTES);
        const int row = n0 + i * kDecTile;
#pragma unroll
        for (int c = 0; c < C::K_SUBS; ++c)
          tma_load_3d(kd + c * (kDecTile * C::K_ROW_BYTES), &k_map, &full_bar[st], c * C::K_ROW_BYTES, row, bkv);
#pragma unroll
        for (int c = 0; c < C::V_SUBS; ++c)
          tma_load_3d(vd + c * (kDecTile * C::V_ROW_BYTES), &v_map, &full_bar[st], c * (C::V_ROW_BYTES / C::V_ELEM),
                      row, bkv);
        issued = i + 1;
      }
      if (!ok) {
        // let copies already in flight land before the block's shared memory goes away
        for (int i = max(0, issued - C::STAGES); i < issued; ++i)
          mbar_wait_quiet(&full_bar[i % C::STAGES], (i / C::STAGES) & 1, kWaitLimitNs);
      }
    }
  } else {
    // ---------------- consumers ----------------
    uint32_t qa[D / 32][4];
    float qs[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + 8 * h;
      const bool live = r < heads_here;
      qs[h] = live ? __ldg(a.q_scale + bhq0 + r) : 0.f;
      const int8_t* qrow = a.q + (bhq0 + r) * D;
#pragma unroll
      for (int s = 0; s < D / 32; ++s) {
        qa[s][h] = live ? __ldg(reinterpret_cast<const uint32_t*>(qrow + 32 * s + 4 * t)) : 0u;
        qa[s][2 + h] = live ? __ldg(reinterpret_cast<const uint32_t*>(qrow + 32 * s + 16 + 4 * t)) : 0u;
      }
    }
    const float* ks_row = a.k_scale + (int64_t)bkv * a.N;
    const int mi = lane >> 3, mr = lane & 7;
    // k_scale of this thread's four keys, fetched one tile ahead so that the global-load
    // latency is hidden behind the previous tile's work
    float ks_cur[2][2], ks_nxt[2][2];
    auto fetch_scales = [&](int tile, float (&dst)[2][2]) {
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = n0 + tile * kDecTile + 16 * warp + 8 * j + 2 * t + e;
          dst[j][e] = (key < n1) ? __ldg(ks_row + key) : 0.f;
        }
    };
    fetch_scales(0, ks_nxt);

    for (int i = 0; i < ntiles; ++i) {
      const int st = i % C::STAGES;
#pragma unroll
      for (int j = 0; j < 2; ++j) { ks_cur[j][0] = ks_nxt[j][0]; ks_cur[j][1] = ks_nxt[j][1]; }
      if (i + 1 < ntiles) fetch_scales(i + 1, ks_nxt);
      ok = mbar_wait(&full_bar[st], (i / C::STAGES) & 1, a.status);
      if (!ok) break;
      const uint32_t kbase = smem_u32(smem + st * C::STAGE_BYTES);
      const uint32_t vbase = kbase + C::K_BYTES;
      const int key0 = n0 + i * kDecTile + 16 * warp;  // first key of this warp's slice

      if (key0 < n1) {
        // ---- S = q . k^T (int32) ----
        int acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
        for (int s = 0; s < D / 32; ++s) {
          const int key_in_tile = 16 * warp + 8 * (mi >> 1) + mr;
          const int c = 2 * s + (mi & 1);  // 16-byte chunk of the K row
          constexpr int CPR = C::K_ROW_BYTES / 16;
          const uint32_t off = (c / CPR) * (kDecTile * C::K_ROW_BYTES) +
                               swizzle_offset<C::K_SW_BITS>(key_in_tile * C::K_ROW_BYTES + (c % CPR) * 16);
          uint32_t bk[4];
          ldmatrix_x4(bk, kbase + off);
          mma_s8_16832(acc[0], qa[s], bk[0], bk[1]);
          mma_s8_16832(acc[1], qa[s], bk[2], bk[3]);
        }
        // ---- logits, online softmax (exp2 domain) ----
        float sv[2][4];
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = key0 + 8 * j + 2 * t + e;
            const bool valid = key < n1;
            const float ks = ks_cur[j][e];
            sv[j][e] = valid ? (float)acc[j][e] * qs[0] * ks : -INFINITY;
            sv[j][2 + e] = valid ? (float)acc[j][2 + e] * qs[1] * ks : -INFINITY;
            tmax[0] = fmaxf(tmax[0], sv[j][e]);
            tmax[1] = fmaxf(tmax[1], sv[j][2 + e]);
          }
        }
        float resc[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
          tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
          const float m_new = fmaxf(m_run[h], tmax[h]);
          resc[h] = (m_new > m_run[h]) ? exp2f(m_run[h] - m_new) : 1.f;
          m_run[h] = m_new;
        }
        uint32_t pa[4];
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float p0 = exp2f(sv[j][0] - m_run[0]), p1 = exp2f(sv[j][1] - m_run[0]);
          const float p2 = exp2f(sv[j][2] - m_run[1]), p3 = exp2f(sv[j][3] - m_run[1]);
          psum[0] += p0 + p1;
          psum[1] += p2 + p3;
          pa[2 * j] = pack2<__half>(p0, p1);
          pa[2 * j + 1] = pack2<__half>(p2, p3);
        }
        l_run[0] = l_run[0] * resc[0] + psum[0];
        l_run[1] = l_run[1] * resc[1] + psum[1];
        if (__any_sync(0xffffffffu, resc[0] != 1.f || resc[1] != 1.f)) {
#pragma unroll
          for (int nt = 0; nt < D / 8; ++nt) {
            o[nt][0] *= resc[0];
            o[nt][1] *= resc[0];
            o[nt][2] *= resc[1];
            o[nt][3] *= resc[1];
          }
        }
        // ---- O += P . V ----
        if (V8) {
          // int8 V: one transposing ldmatrix (16-bit granularity) brings, for this warp's 16 keys,
          // 32 channels as byte pairs -- register = {v[2t][2g], v[2t][2g+1], v[2t+1][2g],
          // v[2t+1][2g+1]} -- i.e. the B fragments of an "even channels" and an "odd channels"
          // 8-wide tile.  byte -> fp16 exactly: (b ^ 0x80) | 0x6400 is 1152 + v.  The accumulator
          // tile nt = 4 q + 2 c + par therefore holds channel 32 q + 16 c + 2 n + par in column n.
          const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
          auto cvt = [&](uint32_t x, uint32_t sel) -> uint32_t {
            const uint32_t u = __byte_perm(x, 0x64646464u, sel);
            const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&u), bias);
            return *reinterpret_cast<const uint32_t*>(&h);
          };
#pragma unroll
          for (int q4 = 0; q4 < D / 32; ++q4) {
            const int key_in_tile = 16 * warp + 8 * (mi & 1) + mr;
            const int dc = 2 * q4 + (mi >> 1);  // 16-byte chunk (16 channels) of the V row
            constexpr int CPR = C::V_ROW_BYTES / 16;
            const uint32_t off = (dc / CPR) * (kDecTile * C::V_ROW_BYTES) +
                                 swizzle_offset<C::V_SW_BITS>(key_in_tile * C::V_ROW_BYTES + (dc % CPR) * 16);
            uint32_t r[4];
            ldmatrix_x4_trans(r, vbase + off);
#pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
              const uint32_t x0 = r[2 * c2] ^ 0x80808080u, x1 = r[2 * c2 + 1] ^ 0x80808080u;
              mma_f16_16816(o[4 * q4 + 2 * c2], pa, cvt(x0, 0x4240u), cvt(x1, 0x4240u));
              mma_f16_16816(o[4 * q4 + 2 * c2 + 1], pa, cvt(x0, 0x4341u), cvt(x1, 0x4341u));
            }
          }
        } else
#pragma unroll
        for (int nt = 0; nt < D / 8; nt += 2) {
          const int key_in_tile = 16 * warp + 8 * (mi & 1) + mr;
          const int dc = nt + (mi >> 1);  // 16-byte chunk (8 channels) of the V row
          constexpr int CPR = C::V_ROW_BYTES / 16;
          const uint32_t off = (dc / CPR) * (kDecTile * C::V_ROW_BYTES) +
                               swizzle_offset<C::V_SW_BITS>(key_in_tile * C::V_ROW_BYTES + (dc % CPR) * 16);
          uint32_t bv[4];
          ldmatrix_x4_trans(bv, vbase + off);
          mma_f16_16816(o[nt], pa, bv[0], bv[1]);
          mma_f16_16816(o[nt + 1], pa, bv[2], bv[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[st]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
  }

  // ---- merge the four warps' partials (stage memory is free now) ----
  ok = (__syncthreads_and(ok ? 1 : 0) != 0);
  if (!ok) return;
  float* m_w = reinterpret_cast<float*>(smem);                    // [4][16]
  float* l_w = m_w + kDecConsumerWarps * kDecHeadsPerBlock;       // [4][16]
  float* o_w = l_w + kDecConsumerWarps * kDecHeadsPerBlock;       // [4][16][D]
  if (warp < kDecConsumerWarps) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + 8 * h;
      if (t == 0) {
        m_w[warp * kDecHeadsPerBlock + r] = m_run[h];
        l_w[warp * kDecHeadsPerBlock + r] = l_run[h];
      }
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        if (V8) {   // column n of tile nt = channel 32 (nt / 4) + 16 ((nt / 2) & 1) + 2 n + (nt & 1)
          const int ch = 32 * (nt >> 2) + 16 * ((nt >> 1) & 1) + 4 * t + (nt & 1);
          o_w[(warp * kDecHeadsPerBlock + r) * D + ch] = o[nt][2 * h];
          o_w[(warp * kDecHeadsPerBlock + r) * D + ch + 2] = o[nt][2 * h + 1];
        } else {
          *reinterpret_cast<float2*>(&o_w[(warp * kDecHeadsPerBlock + r) * D + 8 * nt + 2 * t]) =
              make_float2(o[nt][2 * h], o[nt][2 * h + 1]);
        }
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < heads_here * D; idx += kDecThreads) {
    const int r = idx / D, d = idx % D;
    float gm = kNegSentinel;
#pragma unroll
    for (int w = 0; w < kDecConsumerWarps; ++w) gm = fmaxf(gm, m_w[w * kDecHeadsPerBlock + r]);
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kDecConsumerWarps; ++w) {
      const float wgt = exp2f(m_w[w * kDecHeadsPerBlock + r] - gm);
      acc += o_w[(w * kDecHeadsPerBlock + r) * D + d] * wgt;
      lsum += l_w[w * kDecHeadsPerBlock + r] * wgt;
    }
    const int64_t row = (int64_t)split * BHq + bhq0 + r;
    // the per-channel V scale factors out of the key sum (reference attn_decode.cuh:212-218)
    if (V8) acc *= __ldg(a.v_scale + (int64_t)bkv * D + d);
    a.o_part[row * D + d] = acc;
    if (d == 0) {
      a.m_part[row] = gm;
      a.l_part[row] = lsum;
    }
  }
}

// One block per query head: merge the non-empty splits of its sequence.
template <int D>
__global__ void __launch_bounds__(128) decode_combine_kernel(const float* __restrict__ o_part,
                                                             const float* __restrict__ m_part,
                                                             const float* __restrict__ l_part,
                                                             const int32_t* __restrict__ context_lens,
                                                             __half* __restrict__ out, int Hq, int N, int per,
                                                             int n_splits) {
  const int64_t bh = blockIdx.x;
  const int64_t BHq = gridDim.x;
  const int b = (int)(bh / Hq);
  const int len = context_lens ? min(max(context_lens[b], 0), N) : N;
  const int used = min(n_splits, (len + per - 1) / per);
  float gm = kNegSentinel;
  for (int s = 0; s < used; ++s) gm = fmaxf(gm, m_part[(int64_t)s * BHq + bh]);
  for (int d = threadIdx.x; d < D; d += 128) {
    float denom = 0.f, acc = 0.f;
    for (int s = 0; s < used; ++s) {
      const float ms = m_part[(int64_t)s * BHq + bh];
      if (ms == kNegSentinel) continue;
      const float w = exp2f(ms - gm);
      denom += l_part[(int64_t)s * BHq + bh] * w;
      acc += o_part[((int64_t)s * BHq + bh) * D + d] * w;
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    out[bh * D + d] = __float2half(acc * inv);
  }
}

template <int D, bool V8>
int launch_decode(const sl8_decode_params& p, const float* v_scale, int n_splits, int* status, float* o_part,
                  float* m_part, float* l_part, cudaStream_t stream) {
  using C = DecodeCfg<D, V8>;
  CUtensorMap k_map, v_map;
  const uint64_t heads = (uint64_t)p.B * p.Hkv;
  int rc = sl8_make_tmap_3d(&k_map, p.k, 1, D, p.N, heads, C::K_ROW_BYTES, kDecTile, C::K_ROW_BYTES);
  if (rc != SL8_OK) return rc;
  rc = sl8_make_tmap_3d(&v_map, p.v, C::V_ELEM, D, p.N, heads, C::V_ROW_BYTES / C::V_ELEM, kDecTile, C::V_ROW_BYTES);
  if (rc != SL8_OK) return rc;
  static bool attr_done[8] = {false};
  int dev = 0;
  SL8_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 8 && !attr_done[dev]) {
    SL8_CUDA_TRY(cudaFuncSetAttribute(decode_split_kernel<D, V8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      C::SMEM_BYTES));
    attr_done[dev] = true;
  } else if (dev >= 8) {
    SL8_CUDA_TRY(cudaFuncSetAttribute(decode_split_kernel<D, V8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      C::SMEM_BYTES));
  }
  DecodeArgs a{};
  a.q = p.q; a.q_scale = p.q_scale; a.k_scale = p.k_scale; a.v_scale = v_scale; a.context_lens = p.context_lens;
  a.o_part = o_part; a.m_part = m_part; a.l_part = l_part; a.status = status;
  a.B = p.B; a.Hq = p.Hq; a.Hkv = p.Hkv; a.N = p.N;
  a.per = (p.N + n_splits - 1) / n_splits;
  a.n_splits = n_splits;
  const int G = p.Hq / p.Hkv;
  dim3 grid(n_splits, (unsigned)heads, (G + kDecHeadsPerBlock - 1) / kDecHeadsPerBlock);
  decode_split_kernel<D, V8><<<grid, kDecThreads, C::SMEM_BYTES, stream>>>(k_map, v_map, a);
  decode_combine_kernel<D><<<(unsigned)((int64_t)p.B * p.Hq), 128, 0, stream>>>(
      o_part, m_part, l_part, p.context_lens, reinterpret_cast<__half*>(p.out), p.Hq, p.N, a.per, n_splits);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

int validate(const sl8_decode_params* p) {
  if (p == nullptr) return SL8_ERR_NULL;
  if (p->B < 0 || p->Hq < 0 || p->Hkv < 0 || p->N < 0) return SL8_ERR_BAD_SHAPE;
  if (p->D != 32 && p->D != 64 && p->D != 128 && p->D != 256) return SL8_ERR_BAD_HEAD_DIM;
  if (p->Hkv > 0 && p->Hq % p->Hkv != 0) return SL8_ERR_BAD_SHAPE;
  if (p->Hq > 0 && p->Hkv == 0) return SL8_ERR_BAD_SHAPE;
  if (p->num_splits == 0 || p->num_splits > 256 || p->num_splits < -1) return SL8_ERR_BAD_NUM_SPLITS;
  return SL8_OK;
}

// v8: the int8-V kernel moves a third fewer bytes per key, so the same time per split is twice the
// keys (4096 instead of 2048) as long as the grid still fills the GPU.
int resolve_splits(const sl8_decode_params* p, bool v8 = false) {
  if (p->num_splits > 0) return p->num_splits;
  const int64_t bhkv = (int64_t)p->B * p->Hkv;
  const int ns = sl8_choose_n_splits(p->N, bhkv);
  if (!v8 || ns < 2) return ns;
  const int half = (ns + 1) / 2;
  return (int64_t)half * bhkv >= (int64_t)kNumSms * 8 ? half : ns;
}

}  // namespace
}  // namespace sl8

using namespace sl8;

extern "C" int sl8_choose_n_splits(int64_t N, int64_t BHkv) {
  if (N <= 0 || BHkv <= 0) return 1;
  // Enough blocks for four waves of two resident blocks per SM, but never fewer
  // than 256 keys nor more than 2048 keys per split (bounded serial work keeps
  // ragged batches balanced; the floor keeps the combine negligible).
  const int64_t target_blocks = (int64_t)kNumSms * 8;
  int64_t s_occ = (target_blocks + BHkv - 1) / BHkv;
  int64_t s_lo = (N + 2047) / 2048;
  int64_t s_hi = N / 256 > 1 ? N / 256 : 1;
  int64_t s = s_occ > s_lo ? s_occ : s_lo;
  if (s > s_hi) s = s_hi;
  if (s > 256) s = 256;
  if (s < 1) s = 1;
  return (int)s;
}

extern "C" size_t sl8_attn_int8_decode_workspace(const sl8_decode_params* p) {
  if (validate(p) != SL8_OK) return 256;
  const int ns = resolve_splits(p);   // (an upper bound for the int8-V entry point)
  const size_t rows = (size_t)ns * (size_t)p->B * (size_t)p->Hq;
  return 256 + rows * (size_t)(p->D + 2) * sizeof(float);
}

namespace {
// Common body of the fp16-V and int8-V entry points (v_scale == nullptr: fp16 V).
int decode_entry(const sl8_decode_params* p, const float* v_scale, bool v8, void* workspace, size_t workspace_bytes,
                 void* stream) {
  int rc = validate(p);
  if (rc != SL8_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t BHq = (int64_t)p->B * p->Hq;
  if (BHq == 0) return SL8_OK;
  if (p->out == nullptr) return SL8_ERR_NULL;
  if (p->N == 0) {
    SL8_CUDA_TRY(cudaMemsetAsync(p->out, 0, (size_t)BHq * p->D * sizeof(__half), s));
    return SL8_OK;
  }
  if (!p->q || !p->q_scale || !p->k || !p->k_scale || !p->v || (v8 && !v_scale)) return SL8_ERR_NULL;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return SL8_ERR_MISALIGNED;
  if ((int64_t)p->B * p->Hkv > 65535) return SL8_ERR_TOO_LARGE;
  if (workspace == nullptr || workspace_bytes < sl8_attn_int8_decode_workspace(p)) return SL8_ERR_WORKSPACE;
  if (!aligned16(workspace)) return SL8_ERR_MISALIGNED;
  const int ns = resolve_splits(p, v8);
  int* status = reinterpret_cast<int*>(workspace);
  float* o_part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256);
  float* m_part = o_part + (size_t)ns * BHq * p->D;
  float* l_part = m_part + (size_t)ns * BHq;
  if (v8) {
    switch (p->D) {
      case 32: return launch_decode<32, true>(*p, v_scale, ns, status, o_part, m_part, l_part, s);
      case 64: return launch_decode<64, true>(*p, v_scale, ns, status, o_part, m_part, l_part, s);
      case 128: return launch_decode<128, true>(*p, v_scale, ns, status, o_part, m_part, l_part, s);
      case 256: return launch_decode<256, true>(*p, v_scale, ns, status, o_part, m_part, l_part, s);
    }
    return SL8_ERR_BAD_HEAD_DIM;
  }
  switch (p->D) {
    case 32: return launch_decode<32, false>(*p, nullptr, ns, status, o_part, m_part, l_part, s);
    case 64: return launch_decode<64, false>(*p, nullptr, ns, status, o_part, m_part, l_part, s);
    case 128: return launch_decode<128, false>(*p, nullptr, ns, status, o_part, m_part, l_part, s);
    case 256: return launch_decode<256, false>(*p, nullptr, ns, status, o_part, m_part, l_part, s);
  }
  return SL8_ERR_BAD_HEAD_DIM;
}
}  // namespace

extern "C" int sl8_attn_int8_decode(const sl8_decode_params* p, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  return decode_entry(p, nullptr, false, workspace, workspace_bytes, stream);
}

extern "C" int sl8_attn_int8_decode_kv8(const sl8_decode_params* p, const float* v_scale, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  return decode_entry(p, v_scale, true, workspace, workspace_bytes, stream);
}


// ---- decode without any allocation ---------------------------------------------
// Scratch for sl8_attn_int8_decode_static: lives in the library image, one copy per GPU
// that loads the library, zero-initialised at load.  First 256 bytes: status word.
static __device__ __align__(256) unsigned char g_decode_static_scratch[SL8_DECODE_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxStaticDevices = 64;
void* g_static_scratch_ptr[kMaxStaticDevices] = {nullptr};
std::mutex g_static_scratch_mutex;

// Device address of the static array on the CURRENT device.  In host code the array's name
// is only a handle, never a device address, so the address is asked for once per device
// (under a lock: two host threads may make their first call on a device together).
int static_scratch_address(void** out) {
  int dev = 0;
  SL8_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxStaticDevices) return SL8_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    SL8_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_decode_static_scratch));
    if (ptr == nullptr) return SL8_ERR_CUDA;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return SL8_OK;
}

size_t static_need(int ns, const sl8_decode_params* p) {
  return 256 + (size_t)ns * (size_t)p->B * (size_t)p->Hq * (size_t)(p->D + 2) * sizeof(float);
}
}  // namespace

extern "C" int sl8_attn_int8_decode_static(const sl8_decode_params* p, int32_t* device_status, void* stream) {
  int rc = validate(p);
  if (rc != SL8_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t BHq = (int64_t)p->B * p->Hq;
  if (BHq == 0) return SL8_OK;
  if (p->out == nullptr) return SL8_ERR_NULL;
  if (p->N == 0) {
    SL8_CUDA_TRY(cudaMemsetAsync(p->out, 0, (size_t)BHq * p->D * sizeof(__half), s));
    return SL8_OK;
  }
  if (!p->q || !p->q_scale || !p->k || !p->k_scale || !p->v) return SL8_ERR_NULL;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return SL8_ERR_MISALIGNED;
  if ((int64_t)p->B * p->Hkv > 65535) return SL8_ERR_TOO_LARGE;
  int ns = resolve_splits(p);
  if (p->num_splits < 0) {
    while (ns > 1 && static_need(ns, p) > SL8_DECODE_STATIC_SCRATCH_BYTES) --ns;  // auto: fewer splits until it fits
  }
  if (static_need(ns, p) > SL8_DECODE_STATIC_SCRATCH_BYTES) return SL8_ERR_TOO_LARGE;
  void* base = nullptr;
  rc = static_scratch_address(&base);
  if (rc != SL8_OK) return rc;
  int* status = device_status ? reinterpret_cast<int*>(device_status) : reinterpret_cast<int*>(base);
  // The built-in status word starts every call at zero (a memset allocates nothing), so an
  // expired wait of an earlier call cannot make this one bail out of its waits.
  if (device_status == nullptr) SL8_CUDA_TRY(cudaMemsetAsync(base, 0, sizeof(int), s));
  float* o_part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(base) + 256);
  float* m_part = o_part + (size_t)ns * BHq * p->D;
  float* l_part = m_part + (size_t)ns * BHq;
  switch (p->D) {
    case 32: return launch_decode<32, false>(*p, nullptr, ns, status, o_part, m_part, l_part, s);
    case 64: return launch_decode<64, false>(*p, nullptr, ns, status, o_part, m_part, l_part, s);
    case 128: return launch_decode<128, false>(*p, nullptr, ns, status, o_part, m_part, l_part, s);
    case 256: return launch_decode<256, false>(*p, nullptr, ns, status, o_part, m_part, l_part, s);
  }
  return SL8_ERR_BAD_HEAD_DIM;
}

extern "C" int sl8_decode_static_status(void* stream) {
  void* base = nullptr;
  int rc = static_scratch_address(&base);
  if (rc != SL8_OK) return rc;
  return sl8_read_device_status(base, stream);
}
