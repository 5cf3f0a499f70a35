// Full-W8A8 prefill forward: int8 Q.K^T AND int8 P.V (the reference's `int8_pv=True` route,
// csrc/include/attn_w8a8_fwd.cuh:30-235, op csrc/kernel/attn_w8a8_fwd.cu:72-160).
//
// Logits and online softmax are those of the int8-QK forward.  Per 64-key tile and query row
// P = 2^(s - m_new) is re-quantised to int8 with p_scale = max(max(P) / 127, 2e-38) -- one scale
// per row and tile, or (`per_warp`, the reference's default) one per row and 32-key half of the
// tile -- V arrives int8 with one fp32 scale per (batch, KV head, channel), the int32 product is
// de-quantised by p_scale and added to the fp32 O; the per-channel V scale factors out of the
// key sum and is applied with 1 / l in the epilogue (the reference multiplies it in per tile:
// an fp32-rounding difference).  The row sum l uses the unquantised P.
//
// Because the P scale changes with every tile, O cannot stay in an integer accumulator across
// tiles, which is what a tensor-memory (tcgen05) accumulator would need; this path therefore
// uses warp-level mma.sync m16n8k32 (int8 -> int32) for both contractions, 64 x 64 tiles as in
// the reference.  The V tile is staged channel-major in shared memory (keys contiguous, in the
// order the A fragment of P holds them), so a B fragment is one 32-bit load.
#include "sl8_common.cuh"
#include "sl8_mma.cuh"

namespace sl8 {
namespace {

constexpr int kWBM = 64, kWBN = 64, kWThreads = 128;
constexpr int kVtStride = 80;   // bytes per channel row of the transposed V tile (64 keys + pad: conflict-free)

struct W8A8Args {
  const int8_t* q;
  const float* q_scale;
  const int8_t* k;
  const float* k_scale;
  const int8_t* v;
  const float* v_scale;
  __half* out;
  int Hq, Hkv, M, N;
  int causal, causal_diag;
};

template <int D>
struct W8Cfg {
  static constexpr int DP = ((D + 31) / 32) * 32;   // contraction length of Q.K^T, padded
  static constexpr int QK_STRIDE = DP + 16;         // bytes per Q / K shared row
  static constexpr int Q_BYTES = kWBM * QK_STRIDE;
  static constexpr int K_BYTES = kWBN * QK_STRIDE;
  static constexpr int VT_BYTES = D * kVtStride;
  static constexpr int SMEM = Q_BYTES + K_BYTES + VT_BYTES + kWBN * 4;
};

// Position of local key kl (0..31) of a 32-key block in the K dimension of the P.V MMA: the
// accumulator fragment of S gives thread t the keys 8 jj + 2 t + e, and the A fragment wants four
// consecutive K positions per register, so K position = 16 (jj >> 1) + 4 t + 2 (jj & 1) + e.
__device__ __forceinline__ int pv_slot(int kl) {
  const int jj = kl >> 3, t = (kl & 7) >> 1, e = kl & 1;
  return 16 * (jj >> 1) + 4 * t + 2 * (jj & 1) + e;
}

__device__ __forceinline__ void stage_i8(uint8_t* dst, int dst_stride, const int8_t* src, int row_bytes, int rows,
                                         int valid_rows) {
  const int words = dst_stride / 8;
  for (int idx = threadIdx.x; idx < rows * words; idx += kWThreads) {
    const int r = idx / words, c = (idx % words) * 8;
    uint2 val = make_uint2(0, 0);
    if (r < valid_rows && c < row_bytes) val = __ldg(reinterpret_cast<const uint2*>(src + (int64_t)r * row_bytes + c));
    *reinterpret_cast<uint2*>(dst + r * dst_stride + c) = val;
  }
}

template <int D, bool PER_WARP>
__global__ void __launch_bounds__(kWThreads) fwd_w8a8_kernel(W8A8Args a) {
  using C = W8Cfg<D>;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* sq = smem;
  uint8_t* sk = sq + C::Q_BYTES;
  uint8_t* svt = sk + C::K_BYTES;
  float* sks = reinterpret_cast<float*>(svt + C::VT_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int mi = lane >> 3, mr = lane & 7;
  const int64_t bh = blockIdx.y;
  const int b = (int)(bh / a.Hq);
  const int G = a.Hq / a.Hkv;
  const int64_t kv_bh = (int64_t)b * a.Hkv + (bh % a.Hq) / G;
  const int m_block = (a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x) * kWBM;

  const int8_t* q_bh = a.q + bh * (int64_t)a.M * D;
  const int8_t* k_bh = a.k + kv_bh * (int64_t)a.N * D;
  const int8_t* v_bh = a.v + kv_bh * (int64_t)a.N * D;
  stage_i8(sq, C::QK_STRIDE, q_bh + (int64_t)m_block * D, D, kWBM, a.M - m_block);

  const int row0 = m_block + 16 * warp + g;   // this thread's rows: row0, row0 + 8
  int qpos[2];
  float qs[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int m = row0 + 8 * h;
    qpos[h] = m + a.causal_diag;
    qs[h] = (m < a.M) ? __ldg(a.q_scale + bh * a.M + m) : 0.f;
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  const int n_end = a.causal ? max(0, min(a.N, m_block + kWBM + a.causal_diag)) : a.N;
  const uint32_t sq_u = smem_u32(sq), sk_u = smem_u32(sk);

  for (int n_block = 0; n_block < n_end; n_block += kWBN) {
    __syncthreads();   // previous tile consumed (and Q staged on the first pass)
    stage_i8(sk, C::QK_STRIDE, k_bh + (int64_t)n_block * D, D, kWBN, a.N - n_block);
    if (threadIdx.x < kWBN) {
      const int gn = n_block + threadIdx.x;
      sks[threadIdx.x] = (gn < a.N) ? __ldg(a.k_scale + kv_bh * a.N + gn) : 0.f;
    }
    // V tile, channel-major with the keys of each 32-key block in P.V order (pv_slot): lanes walk
    // the keys (one 4-byte read of 4 channels each), so the byte stores of a warp fall in one row
    for (int idx = threadIdx.x; idx < kWBN * (D / 4); idx += kWThreads) {
      const int kl = idx % kWBN, cg = idx / kWBN;
      const int gn = n_block + kl;
      const uint32_t w = (gn < a.N) ? __ldg(reinterpret_cast<const uint32_t*>(v_bh + (int64_t)gn * D + 4 * cg)) : 0u;
      uint8_t* dst = svt + (4 * cg) * kVtStride + 32 * (kl >> 5) + pv_slot(kl & 31);
      dst[0] = (uint8_t)(w & 0xff);
      dst[kVtStride] = (uint8_t)((w >> 8) & 0xff);
      dst[2 * kVtStride] = (uint8_t)((w >> 16) & 0xff);
      dst[3 * kVtStride] = (uint8_t)(w >> 24);
    }
    __syncthreads();

    // ---- S = Q . K^T (int32) -> logits ----
    int acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;
#pragma unroll
    for (int s = 0; s < C::DP / 32; ++s) {
      uint32_t qa[4];
      ldmatrix_x4(qa, sq_u + (16 * warp + 8 * (mi & 1) + mr) * C::QK_STRIDE + 32 * s + 16 * (mi >> 1));
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t bk[4];
        ldmatrix_x4(bk, sk_u + (8 * (j + (mi >> 1)) + mr) * C::QK_STRIDE + 32 * s + 16 * (mi & 1));
        mma_s8_16832(acc[j], qa, bk[0], bk[1]);
        mma_s8_16832(acc[j + 1], qa, bk[2], bk[3]);
      }
    }
    float p[8][4];
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int gn = n_block + 8 * j + 2 * t + (e & 1);
        const bool valid = (gn < a.N) && (!a.causal || gn <= qpos[h]);
        p[j][e] = valid ? (float)acc[j][e] * qs[h] * sks[8 * j + 2 * t + (e & 1)] : -INFINITY;
        tmax[h] = fmaxf(tmax[h], p[j][e]);
      }
    // ---- online softmax; P in fp32, its row sums, its maxima per 32-key half ----
    float resc[2], psum[2] = {0.f, 0.f}, pmax[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
      const float m_new = fmaxf(m_run[h], tmax[h]);
      resc[h] = (m_run[h] == -INFINITY || m_new == -INFINITY) ? 1.f : exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const float v = (m_run[h] == -INFINITY || p[j][e] == -INFINITY) ? 0.f : exp2f(p[j][e] - m_run[h]);
        p[j][e] = v;
        psum[h] += v;
        pmax[h][j >> 2] = fmaxf(pmax[h][j >> 2], v);
      }
    float ps[2][2], inv_ps[2][2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int bk = 0; bk < 2; ++bk) {
        pmax[h][bk] = fmaxf(pmax[h][bk], __shfl_xor_sync(0xffffffffu, pmax[h][bk], 1));
        pmax[h][bk] = fmaxf(pmax[h][bk], __shfl_xor_sync(0xffffffffu, pmax[h][bk], 2));
      }
      if (!PER_WARP) pmax[h][0] = pmax[h][1] = fmaxf(pmax[h][0], pmax[h][1]);   // one scale per row and tile
#pragma unroll
      for (int bk = 0; bk < 2; ++bk) {
        ps[h][bk] = fmaxf(pmax[h][bk] * (1.f / 127.f), 2e-38f);
        inv_ps[h][bk] = __fdiv_rn(1.f, ps[h][bk]);
      }
      l_run[h] = l_run[h] * resc[h] + psum[h];
    }
    if (__any_sync(0xffffffffu, resc[0] != 1.f || resc[1] != 1.f)) {
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        o[nt][0] *= resc[0];
        o[nt][1] *= resc[0];
        o[nt][2] *= resc[1];
        o[nt][3] *= resc[1];
      }
    }
    // ---- P -> int8 A fragments (per 32-key block), O += dequant(P8 . V8) ----
    uint32_t pa[2][4];
#pragma unroll
    for (int bk = 0; bk < 2; ++bk)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int h = r & 1;             // registers 0, 2: row g; 1, 3: row g + 8
        const int j0 = 4 * bk + 2 * (r >> 1);
        uint32_t w = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float pv = p[j0 + (i >> 1)][2 * h + (i & 1)];
          w |= (uint32_t)(__float2int_rn(pv * inv_ps[h][bk]) & 0xff) << (8 * i);
        }
        pa[bk][r] = w;
      }
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      const uint8_t* vrow = svt + (8 * nt + g) * kVtStride + 4 * t;
      int acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
      mma_s8_16832(acc0, pa[0], *reinterpret_cast<const uint32_t*>(vrow), *reinterpret_cast<const uint32_t*>(vrow + 16));
      mma_s8_16832(PER_WARP ? acc1 : acc0, pa[1], *reinterpret_cast<const uint32_t*>(vrow + 32),
                   *reinterpret_cast<const uint32_t*>(vrow + 48));
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        if (PER_WARP) o[nt][e] += (float)acc0[e] * ps[h][0] + (float)acc1[e] * ps[h][1];
        else o[nt][e] += (float)acc0[e] * ps[h][0];
      }
    }
  }

  // ---- epilogue: out = O * v_scale[channel] / l ----
  const float* vsc = a.v_scale + kv_bh * D;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    const int m = row0 + 8 * h;
    if (m >= a.M) continue;
    const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
    __half* orow = a.out + bh * (int64_t)a.M * D + (int64_t)m * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      const int ch = 8 * nt + 2 * t;
      *reinterpret_cast<uint32_t*>(orow + ch) =
          pack2<__half>(o[nt][2 * h] * __ldg(vsc + ch) * inv, o[nt][2 * h + 1] * __ldg(vsc + ch + 1) * inv);
    }
  }
}

template <int D>
int launch_w8a8(const W8A8Args& a, int B, bool per_warp, cudaStream_t s) {
  using C = W8Cfg<D>;
  dim3 grid((a.M + kWBM - 1) / kWBM, (unsigned)((int64_t)B * a.Hq));
  if (per_warp) {
    SL8_CUDA_TRY(cudaFuncSetAttribute(fwd_w8a8_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    fwd_w8a8_kernel<D, true><<<grid, kWThreads, C::SMEM, s>>>(a);
  } else {
    SL8_CUDA_TRY(cudaFuncSetAttribute(fwd_w8a8_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    fwd_w8a8_kernel<D, false><<<grid, kWThreads, C::SMEM, s>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

}  // namespace
}  // namespace sl8

using namespace sl8;

extern "C" int sl8_attn_w8a8_fwd(const sl8_w8a8_params* p, void* stream) {
  if (p == nullptr) return SL8_ERR_NULL;
  if (p->B < 0 || p->Hq < 0 || p->Hkv < 0 || p->M < 0 || p->N < 0) return SL8_ERR_BAD_SHAPE;
  if (p->D != 32 && p->D != 64 && p->D != 128 && p->D != 256) return SL8_ERR_BAD_HEAD_DIM;
  if (p->Hq > 0 && (p->Hkv <= 0 || p->Hq % p->Hkv != 0)) return SL8_ERR_BAD_SHAPE;
  if ((int64_t)p->B * p->Hq * p->M == 0) return SL8_OK;   // empty output
  if (!p->q || !p->q_scale || !p->out) return SL8_ERR_NULL;
  if (p->N > 0 && (!p->k || !p->k_scale || !p->v || !p->v_scale)) return SL8_ERR_NULL;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return SL8_ERR_MISALIGNED;
  if ((int64_t)p->B * p->Hq > 65535) return SL8_ERR_TOO_LARGE;
  W8A8Args a{};
  a.q = p->q; a.q_scale = p->q_scale; a.k = p->k; a.k_scale = p->k_scale; a.v = p->v; a.v_scale = p->v_scale;
  a.out = reinterpret_cast<__half*>(p->out);
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N; a.causal = p->causal; a.causal_diag = p->causal ? p->causal_diag : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (p->D) {
    case 32: return launch_w8a8<32>(a, p->B, p->per_warp_quant != 0, s);
    case 64: return launch_w8a8<64>(a, p->B, p->per_warp_quant != 0, s);
    case 128: return launch_w8a8<128>(a, p->B, p->per_warp_quant != 0, s);
    case 256: return launch_w8a8<256>(a, p->B, p->per_warp_quant != 0, s);
  }
  return SL8_ERR_BAD_HEAD_DIM;
}
