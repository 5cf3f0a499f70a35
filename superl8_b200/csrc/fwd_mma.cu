// Prefill forward on warp-level tensor-core instructions (mma.sync): the path
// that serves EVERY head dim the reference accepts (32, 64, 72, 80, 128, 256),
// and the full-precision sibling the accuracy gate demotes to.  Head dims 64,
// 128 and 256 normally run on the tcgen05 kernel instead (fwd_tcgen05.cu).
//
// Mathematics follow the reference kernels (csrc/include/attn_int8_fwd.cuh:107-208,
// csrc/include/attn_fp16_fwd.cuh:89-230): per 64-key tile
//   s = float(int32 q.k) * q_scale[m] * k_scale[n]        (int8 mode)
//   s = (q.k) * softmax_scale * log2(e)                   (16-bit mode)
//   valid = n < N and (not causal or n <= m + N - M) and (window < 0 or n > pos - window)
// online softmax in the exp2 domain with fp32 state, O += P.V, out = O / l
// (0 when l == 0), lse = m * ln2 + ln(l).  P is rounded to V's dtype for the
// tensor-core P.V (the reference keeps P in fp32 on CUDA cores).
#include "sl8_common.cuh"
#include "sl8_mma.cuh"

namespace sl8 {
namespace {

constexpr int kBM = 64, kBN = 64, kThreads = 128;

struct FwdArgs {
  const void* q;        // int8 or VT
  const float* q_scale; // int8 mode
  const void* k;
  const float* k_scale;
  const void* v;
  void* out;
  float* lse;
  const int32_t* seqlens_q;
  const int32_t* seqlens_k;
  int Hq, Hkv, M, N;
  int causal, window_left;
  float scale_log2;     // 16-bit mode
  const void* mask;     // 16-bit mode: additive bias (natural log), element type of q, or null
  int64_t mask_sb, mask_sh, mask_sm, mask_sn;   // strides in elements, 0 on broadcast axes
  // Packed token-major tensors [tokens, heads, D] (scales [tokens, heads]) when non-null:
  // sequence b owns tokens [cu_q[b], cu_q[b+1]) of q / out and [cu_k[b], cu_k[b+1]) of k / v.
  const int32_t* cu_q;
  const int32_t* cu_k;
};

template <int D, bool I8>
struct MmaCfg {
  static constexpr int DP = I8 ? ((D + 31) / 32) * 32 : ((D + 15) / 16) * 16;  // contraction length, padded
  static constexpr int QK_ELEM = I8 ? 1 : 2;
  static constexpr int QK_STRIDE = DP * QK_ELEM + 16;   // bytes per Q/K smem row
  static constexpr int NT = ((D / 8) + 1) / 2 * 2;      // 8-channel output tiles, rounded to pairs
  static constexpr int V_STRIDE = (NT * 8 + 8) * 2;     // bytes per V smem row
  static constexpr int Q_BYTES = kBM * QK_STRIDE;
  static constexpr int K_BYTES = kBN * QK_STRIDE;
  static constexpr int V_BYTES = kBN * V_STRIDE;
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES + kBN * 4;   // K tile, V tile, k_scale tile
  static constexpr int SMEM = Q_BYTES + 2 * STAGE_BYTES;
};

// Copies `rows` x `row_bytes` from global (row pitch `pitch` bytes) into a padded
// shared tile, 8 bytes at a time; rows >= valid_rows and the pad bytes become 0.
__device__ __forceinline__ void stage_tile(uint8_t* dst, int dst_stride, int dst_row_bytes, const uint8_t* src,
                                           int row_bytes, int rows, int valid_rows, int64_t pitch) {
  const int words = dst_row_bytes / 8;
  for (int idx = threadIdx.x; idx < rows * words; idx += kThreads) {
    const int r = idx / words, c = (idx % words) * 8;
    uint2 val = make_uint2(0, 0);
    if (r < valid_rows && c < row_bytes) val = __ldg(reinterpret_cast<const uint2*>(src + (int64_t)r * pitch + c));
    *reinterpret_cast<uint2*>(dst + r * dst_stride + c) = val;
  }
}

// The same copy as asynchronous 8-byte cp.async (zero fill where the synchronous copy writes
// zeros); the caller commits the group and waits for it before the tile is read.
__device__ __forceinline__ void stage_tile_async(uint8_t* dst, int dst_stride, int dst_row_bytes, const uint8_t* src,
                                                 int row_bytes, int rows, int valid_rows, int64_t pitch) {
  const int words = dst_row_bytes / 8;
  const uint32_t dst_u = smem_u32(dst);
  for (int idx = threadIdx.x; idx < rows * words; idx += kThreads) {
    const int r = idx / words, c = (idx % words) * 8;
    const bool live = r < valid_rows && c < row_bytes;
    const uint8_t* g = live ? src + (int64_t)r * pitch + c : src;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst_u + r * dst_stride + c), "l"(g),
                 "r"(live ? 8 : 0)
                 : "memory");
  }
}

template <int D, typename VT, bool I8>
__global__ void __launch_bounds__(kThreads) fwd_mma_kernel(FwdArgs a) {
  using C = MmaCfg<D, I8>;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* sq = smem;
  uint8_t* skv = sq + C::Q_BYTES;   // two stages of {K tile, V tile, k_scale tile}

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int mi = lane >> 3, mr = lane & 7;
  const int64_t bh = blockIdx.y;
  const int b = (int)(bh / a.Hq);
  const int G = a.Hq / a.Hkv;
  const int64_t kv_bh = (int64_t)b * a.Hkv + (bh % a.Hq) / G;
  const bool packed = a.cu_q != nullptr;
  const int hq = (int)(bh % a.Hq), hkv = hq / G;
  const int q0 = packed ? a.cu_q[b] : 0, k0 = packed ? a.cu_k[b] : 0;   // first token of the sequence
  const int m_len = packed ? a.cu_q[b + 1] - q0 : (a.seqlens_q ? min(max(a.seqlens_q[b], 0), a.M) : a.M);
  const int n_len = packed ? a.cu_k[b + 1] - k0 : (a.seqlens_k ? min(max(a.seqlens_k[b], 0), a.N) : a.N);
  const int m_store = packed ? m_len : a.M;   // rows this block may write (packed: never a neighbour's)
  // rows of one head: elements between consecutive rows, and where the head's first row is
  const int64_t q_rowe = packed ? (int64_t)a.Hq * D : D, kv_rowe = packed ? (int64_t)a.Hkv * D : D;
  const int64_t q_off = packed ? ((int64_t)q0 * a.Hq + hq) * D : bh * (int64_t)a.M * D;
  const int64_t kv_off = packed ? ((int64_t)k0 * a.Hkv + hkv) * D : kv_bh * (int64_t)a.N * D;
  const int64_t qs_row = packed ? a.Hq : 1, ks_row = packed ? a.Hkv : 1;
  const float* qs_base = I8 ? a.q_scale + (packed ? (int64_t)q0 * a.Hq + hq : bh * (int64_t)a.M) : nullptr;
  const float* ks_base = I8 ? a.k_scale + (packed ? (int64_t)k0 * a.Hkv + hkv : kv_bh * (int64_t)a.N) : nullptr;
  // heavy (late) query tiles first when causal
  const int m_block = (a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x) * kBM;
  VT* out_bh = reinterpret_cast<VT*>(a.out) + q_off;

  if (m_block >= m_len) {  // padded rows of a ragged batch: zeros
    for (int idx = threadIdx.x; idx < kBM * D / 2; idx += kThreads) {
      const int r = idx / (D / 2), c = (idx % (D / 2)) * 2;
      if (m_block + r < m_store) *reinterpret_cast<uint32_t*>(out_bh + (int64_t)(m_block + r) * q_rowe + c) = 0u;
    }
    if (a.lse) for (int r = threadIdx.x; r < kBM; r += kThreads)
        if (m_block + r < m_store) a.lse[bh * a.M + m_block + r] = -INFINITY;
    return;
  }

  const uint8_t* q_bh = reinterpret_cast<const uint8_t*>(a.q) + q_off * C::QK_ELEM;
  const uint8_t* k_bh = reinterpret_cast<const uint8_t*>(a.k) + kv_off * C::QK_ELEM;
  const uint8_t* v_bh = reinterpret_cast<const uint8_t*>(a.v) + kv_off * 2;

  stage_tile(sq, C::QK_STRIDE, C::QK_STRIDE, q_bh + (int64_t)m_block * q_rowe * C::QK_ELEM, D * C::QK_ELEM, kBM,
             m_len - m_block, q_rowe * C::QK_ELEM);

  const int causal_diag = a.causal ? n_len - m_len : 0;
  const int row0 = m_block + 16 * warp + g;       // this thread's rows: row0, row0 + 8
  int qpos[2];
  float qs[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int m = row0 + 8 * h;
    qpos[h] = m + causal_diag;
    qs[h] = I8 ? ((m < m_len) ? __ldg(qs_base + m * qs_row) : 0.f) : a.scale_log2;
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[C::NT][4];
#pragma unroll
  for (int i = 0; i < C::NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  const int n_end = a.causal ? max(0, min(n_len, m_block + kBM + causal_diag)) : n_len;
  int n_begin = 0;
  if (a.window_left >= 0) n_begin = max(0, (m_block + causal_diag - a.window_left + 1)) / kBN * kBN;

  const uint32_t sq_u = smem_u32(sq);
  // tile n_block -> stage st, asynchronously (the k_scale values with plain stores: they are
  // published by the barrier at the top of the iteration that reads them)
  auto load_kv = [&](int n_block, int st) {
    uint8_t* sk_ = skv + st * C::STAGE_BYTES;
    uint8_t* sv_ = sk_ + C::K_BYTES;
    stage_tile_async(sk_, C::QK_STRIDE, C::QK_STRIDE, k_bh + (int64_t)n_block * kv_rowe * C::QK_ELEM, D * C::QK_ELEM, kBN,
                     n_len - n_block, kv_rowe * C::QK_ELEM);
    stage_tile_async(sv_, C::V_STRIDE, C::V_STRIDE, v_bh + (int64_t)n_block * kv_rowe * 2, D * 2, kBN, n_len - n_block,
                     kv_rowe * 2);
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (I8 && threadIdx.x < kBN) {
      const int gn = n_block + threadIdx.x;
      reinterpret_cast<float*>(sv_ + C::V_BYTES)[threadIdx.x] = (gn < n_len) ? __ldg(ks_base + gn * ks_row) : 0.f;
    }
  };
  if (n_begin < n_end) load_kv(n_begin, 0);

  for (int n_block = n_begin, it = 0; n_block < n_end; n_block += kBN, ++it) {
    // this tile has landed and every warp is done with the tile before it (whose stage the next
    // load overwrites); on the first pass this also publishes Q
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (n_block + kBN < n_end) load_kv(n_block + kBN, (it + 1) & 1);
    const uint32_t sk_u = smem_u32(skv + (it & 1) * C::STAGE_BYTES), sv_u = sk_u + C::K_BYTES;
    const float* sks = reinterpret_cast<const float*>(skv + (it & 1) * C::STAGE_BYTES + C::K_BYTES + C::V_BYTES);

    // ---- S = Q . K^T ----
    float sv_f[8][4];
    if (I8) {
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
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float ks = sks[8 * j + 2 * t + e];
          sv_f[j][e] = (float)acc[j][e] * qs[0] * ks;
          sv_f[j][2 + e] = (float)acc[j][2 + e] * qs[1] * ks;
        }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) sv_f[j][0] = sv_f[j][1] = sv_f[j][2] = sv_f[j][3] = 0.f;
#pragma unroll
      for (int s = 0; s < C::DP / 16; ++s) {
        uint32_t qa[4];
        ldmatrix_x4(qa, sq_u + (16 * warp + 8 * (mi & 1) + mr) * C::QK_STRIDE + 32 * s + 16 * (mi >> 1));
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          uint32_t bk[4];
          ldmatrix_x4(bk, sk_u + (8 * (j + (mi >> 1)) + mr) * C::QK_STRIDE + 32 * s + 16 * (mi & 1));
          mma_16816<VT>(sv_f[j], qa, bk[0], bk[1]);
          mma_16816<VT>(sv_f[j + 1], qa, bk[2], bk[3]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) sv_f[j][e] *= a.scale_log2;
    }

    // ---- mask + online softmax ----
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int gn = n_block + 8 * j + 2 * t + e;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const bool valid = (gn < n_len) && (!a.causal || gn <= qpos[h]) &&
                             (a.window_left < 0 || gn > qpos[h] - a.window_left);
          float& x = sv_f[j][2 * h + e];
          if (!I8 && a.mask != nullptr && valid && row0 + 8 * h < m_len) {
            // reference csrc/include/attn_fp16_fwd.cuh:176-178: natural-log bias, log2(e) folded in
            const int64_t mi_ = (int64_t)b * a.mask_sb + (bh % a.Hq) * a.mask_sh + (int64_t)(row0 + 8 * h) * a.mask_sm +
                                (int64_t)gn * a.mask_sn;
            x += to_f32<VT>(reinterpret_cast<const VT*>(a.mask)[mi_]) * 1.4426950408889634f;
          }
          x = valid ? x : -INFINITY;
          tmax[h] = fmaxf(tmax[h], x);
        }
      }
    float resc[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
      tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
      const float m_new = fmaxf(m_run[h], tmax[h]);
      resc[h] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
    }
    float psum[2] = {0.f, 0.f};
    uint32_t pa[4][4];  // A fragments of P for the four 16-key steps
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mm = m_run[e >> 1];
        p[e] = (mm == -INFINITY) ? 0.f : exp2f(sv_f[j][e] - mm);
      }
      psum[0] += p[0] + p[1];
      psum[1] += p[2] + p[3];
      pa[j >> 1][(j & 1) * 2] = pack2<VT>(p[0], p[1]);
      pa[j >> 1][(j & 1) * 2 + 1] = pack2<VT>(p[2], p[3]);
    }
    l_run[0] = l_run[0] * resc[0] + psum[0];
    l_run[1] = l_run[1] * resc[1] + psum[1];
    if (__any_sync(0xffffffffu, resc[0] != 1.f || resc[1] != 1.f)) {
#pragma unroll
      for (int nt = 0; nt < C::NT; ++nt) {
        o[nt][0] *= resc[0];
        o[nt][1] *= resc[0];
        o[nt][2] *= resc[1];
        o[nt][3] *= resc[1];
      }
    }
    // ---- O += P . V ----
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int nt = 0; nt < C::NT; nt += 2) {
        uint32_t bv[4];
        ldmatrix_x4_trans(bv, sv_u + (16 * kk + 8 * (mi & 1) + mr) * C::V_STRIDE + (nt + (mi >> 1)) * 16);
        mma_16816<VT>(o[nt], pa[kk], bv[0], bv[1]);
        mma_16816<VT>(o[nt + 1], pa[kk], bv[2], bv[3]);
      }
    }
  }

  // ---- epilogue ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    const int m = row0 + 8 * h;
    if (m >= m_store) continue;
    const bool live = m < m_len;
    const float inv = (live && l_run[h] > 0.f) ? 1.f / l_run[h] : 0.f;
    VT* orow = out_bh + (int64_t)m * q_rowe;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt)
      *reinterpret_cast<uint32_t*>(orow + 8 * nt + 2 * t) = pack2<VT>(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
    if (a.lse != nullptr && t == 0)
      a.lse[bh * a.M + m] =
          (live && l_run[h] > 0.f) ? (m_run[h] * 0.6931471805599453f + logf(l_run[h])) : -INFINITY;
  }
}

template <int D, typename VT, bool I8>
int launch(const FwdArgs& a, int B, cudaStream_t s) {
  using C = MmaCfg<D, I8>;
  SL8_CUDA_TRY(cudaFuncSetAttribute(fwd_mma_kernel<D, VT, I8>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
  dim3 grid((a.M + kBM - 1) / kBM, (unsigned)((int64_t)B * a.Hq));
  fwd_mma_kernel<D, VT, I8><<<grid, kThreads, C::SMEM, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

template <typename VT, bool I8>
int launch_d(const FwdArgs& a, int B, int D, cudaStream_t s) {
  switch (D) {
    case 32: return launch<32, VT, I8>(a, B, s);
    case 64: return launch<64, VT, I8>(a, B, s);
    case 72: return launch<72, VT, I8>(a, B, s);
    case 80: return launch<80, VT, I8>(a, B, s);
    case 128: return launch<128, VT, I8>(a, B, s);
    case 256: return launch<256, VT, I8>(a, B, s);
  }
  return SL8_ERR_BAD_HEAD_DIM;
}

}  // namespace
}  // namespace sl8

using namespace sl8;

// int8-QK forward on the mma.sync path; parameters were validated by the caller.
int sl8_fwd_mma_int8(const sl8_fwd_params* p, cudaStream_t s) {
  FwdArgs a{};
  a.q = p->q; a.q_scale = p->q_scale; a.k = p->k; a.k_scale = p->k_scale; a.v = p->v; a.out = p->out;
  a.lse = p->lse; a.seqlens_q = p->seqlens_q; a.seqlens_k = p->seqlens_k;
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N; a.causal = p->causal; a.window_left = p->window_left;
  if (p->v_dtype == SL8_F16) return launch_d<__half, true>(a, p->B, p->D, s);
  if (p->v_dtype == SL8_BF16) return launch_d<__nv_bfloat16, true>(a, p->B, p->D, s);
  return SL8_ERR_BAD_DTYPE;
}

// packed variable-length int8-QK forward on the mma.sync path; validated by the caller
int sl8_fwd_mma_int8_varlen(const sl8_varlen_params* p, cudaStream_t s) {
  FwdArgs a{};
  a.q = p->q; a.q_scale = p->q_scale; a.k = p->k; a.k_scale = p->k_scale; a.v = p->v; a.out = p->out;
  a.cu_q = p->cu_seqlens_q; a.cu_k = p->cu_seqlens_k;
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->max_seqlen_q; a.N = 0; a.causal = p->causal; a.window_left = -1;
  if (p->v_dtype == SL8_F16) return launch_d<__half, true>(a, p->B, p->D, s);
  if (p->v_dtype == SL8_BF16) return launch_d<__nv_bfloat16, true>(a, p->B, p->D, s);
  return SL8_ERR_BAD_DTYPE;
}

int sl8_fwd_tc_fp16(const sl8_fp16_fwd_params* p, int* status, cudaStream_t s);  // fwd_tcgen05.cu

extern "C" size_t sl8_attn_fp16_fwd_workspace(const sl8_fp16_fwd_params*) { return 256; }

extern "C" int sl8_attn_fp16_fwd(const sl8_fp16_fwd_params* p, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  if (p == nullptr) return SL8_ERR_NULL;
  if (p->B < 0 || p->Hq < 0 || p->Hkv < 0 || p->M < 0 || p->N < 0) return SL8_ERR_BAD_SHAPE;
  if (p->D != 32 && p->D != 64 && p->D != 72 && p->D != 80 && p->D != 128 && p->D != 256) return SL8_ERR_BAD_HEAD_DIM;
  if (p->dtype != SL8_F16 && p->dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (p->Hq > 0 && (p->Hkv <= 0 || p->Hq % p->Hkv != 0)) return SL8_ERR_BAD_SHAPE;
  if ((int64_t)p->B * p->Hq * p->M == 0) return SL8_OK;
  if (!p->q || !p->out || (p->N > 0 && (!p->k || !p->v))) return SL8_ERR_NULL;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return SL8_ERR_MISALIGNED;
  if ((int64_t)p->B * p->Hq > 65535) return SL8_ERR_TOO_LARGE;
  // the tensor-memory kernel takes the row maximum before scaling, so it wants a scale >= 0
  const bool tc_ok = (p->D == 64 || p->D == 128 || p->D == 256) && p->N > 0 && p->softmax_scale >= 0.f &&
                     (p->mask == nullptr || p->gate_flag == nullptr);
  int backend = p->backend;
  if (backend == SL8_BACKEND_AUTO) backend = tc_ok ? SL8_BACKEND_TCGEN05 : SL8_BACKEND_MMA;
  if (backend == SL8_BACKEND_TCGEN05 || backend == SL8_BACKEND_TCGEN05_2Q) {
    if (!tc_ok) return SL8_ERR_UNSUPPORTED;
    if (workspace == nullptr || workspace_bytes < 256) return SL8_ERR_WORKSPACE;
    return sl8_fwd_tc_fp16(p, reinterpret_cast<int*>(workspace), static_cast<cudaStream_t>(stream));
  }
  if (backend != SL8_BACKEND_MMA) return SL8_ERR_UNSUPPORTED;
  if (p->gate_flag != nullptr) return SL8_ERR_UNSUPPORTED;   // device-side dispatch: tensor-memory kernel only
  FwdArgs a{};
  a.q = p->q; a.k = p->k; a.v = p->v; a.out = p->out; a.lse = p->lse;
  a.seqlens_q = p->seqlens_q; a.seqlens_k = p->seqlens_k;
  a.Hq = p->Hq; a.Hkv = p->Hkv; a.M = p->M; a.N = p->N; a.causal = p->causal; a.window_left = p->window_left;
  a.scale_log2 = p->softmax_scale * 1.4426950408889634f;
  a.mask = p->mask; a.mask_sb = p->mask_stride_b; a.mask_sh = p->mask_stride_h;
  a.mask_sm = p->mask_stride_m; a.mask_sn = p->mask_stride_n;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->dtype == SL8_F16) return launch_d<__half, false>(a, p->B, p->D, s);
  return launch_d<__nv_bfloat16, false>(a, p->B, p->D, s);
}
