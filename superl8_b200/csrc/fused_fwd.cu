// attn_int8_fwd from 16-bit Q, K, V in ONE host call: accuracy gate, Q / K quantisation prologue
// and attention, queued back to back on the stream with the gate decided on the device.  It is
// the host-side sequence of the reference's Python entry (superl8/ops.py:70-175: gate ->
// quantize_qk -> _C.attn_int8_fwd, or attn_fp16_fwd when the gate fires) without its device->host
// read-back of the gate (superl8/quant/core.py:145): the int8 kernel and the full-precision
// kernel are both launched on the same output and the one whose turn it is not exits on reading
// the flag.  Everything here is calls of this library's own entry points; scratch comes from the
// caller's workspace.
#include "sl8_common.cuh"

namespace {
constexpr size_t kAlign = 256;
inline size_t up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

struct Layout {
  size_t flag, q_i8, k_i8, q_scale, k_scale, mean, mean_ws, total;
};
Layout layout(const sl8_fused_fwd_params* p) {
  Layout l{};
  const size_t qrows = (size_t)p->B * p->Hq * p->M, krows = (size_t)p->B * p->Hkv * p->N;
  size_t o = 256;                       // [0, 256): status word of the bounded device-side waits
  l.flag = o; o += 256;
  l.q_i8 = o; o += up(qrows * p->D);
  l.k_i8 = o; o += up(krows * p->D);
  l.q_scale = o; o += up(qrows * 4);
  l.k_scale = o; o += up(krows * 4);
  l.mean = o; o += up((size_t)p->B * p->Hkv * p->D * 4);
  l.mean_ws = o; o += up(sl8_k_mean_workspace((int64_t)p->B * p->Hkv, p->N, p->D));
  l.total = o;
  return l;
}
bool shape_ok(const sl8_fused_fwd_params* p) {
  return p->B >= 0 && p->Hq >= 0 && p->Hkv >= 0 && p->M >= 0 && p->N >= 0 && (p->Hq == 0 || (p->Hkv > 0 && p->Hq % p->Hkv == 0));
}
}  // namespace

extern "C" size_t sl8_attn_int8_fwd_fused_workspace(const sl8_fused_fwd_params* p) {
  if (p == nullptr || !shape_ok(p) || p->D <= 0) return 512;
  return layout(p).total;
}

extern "C" int sl8_attn_int8_fwd_fused(const sl8_fused_fwd_params* p, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  if (p == nullptr) return SL8_ERR_NULL;
  if (!shape_ok(p)) return SL8_ERR_BAD_SHAPE;
  if (p->D != 64 && p->D != 128 && p->D != 256) return SL8_ERR_UNSUPPORTED;   // the tensor-memory kernels' head dims
  if (p->dtype != SL8_F16 && p->dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (p->N == 0 || p->softmax_scale < 0.0) return SL8_ERR_UNSUPPORTED;
  if ((int64_t)p->B * p->Hq * p->M == 0) return SL8_OK;
  if (!p->q || !p->k || !p->v || !p->out) return SL8_ERR_NULL;
  const Layout l = layout(p);
  if (workspace == nullptr || workspace_bytes < l.total) return SL8_ERR_WORKSPACE;
  if (!sl8::aligned16(workspace)) return SL8_ERR_MISALIGNED;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool gate = p->ratio_threshold > 0.f;
  int32_t* flag = p->gate_flag != nullptr ? p->gate_flag : reinterpret_cast<int32_t*>(ws + l.flag);
  SL8_CUDA_TRY(cudaMemsetAsync(ws, 0, 512, s));        // status word and gate flag
  if (p->gate_flag != nullptr) SL8_CUDA_TRY(cudaMemsetAsync(p->gate_flag, 0, sizeof(int32_t), s));
  int8_t* q_i8 = reinterpret_cast<int8_t*>(ws + l.q_i8);
  int8_t* k_i8 = reinterpret_cast<int8_t*>(ws + l.k_i8);
  float* q_scale = reinterpret_cast<float*>(ws + l.q_scale);
  float* k_scale = reinterpret_cast<float*>(ws + l.k_scale);
  float* mean = reinterpret_cast<float*>(ws + l.mean);
  const int64_t bhk = (int64_t)p->B * p->Hkv;
  // the folded scale is formed in double and rounded once, like the Python layer's
  const float fold = (float)(p->softmax_scale * 1.4426950408889634);
  int rc = sl8_quant_q_prologue(p->q, p->dtype, (int64_t)p->B * p->Hq * p->M, p->D, fold,
                                gate ? p->ratio_threshold : 12.f, q_i8, q_scale, nullptr, gate ? flag : nullptr, stream);
  if (rc != SL8_OK) return rc;
  if (sl8_k_prologue_fused_ok(p->dtype, bhk, p->N, p->D)) {   // one launch, K read from HBM once
    rc = sl8_k_prologue(p->k, p->dtype, bhk, p->N, p->D, p->seqlens_k, p->Hkv, mean, k_i8, k_scale, nullptr, stream);
    if (rc != SL8_OK) return rc;
  } else {
    rc = sl8_k_mean(p->k, p->dtype, bhk, p->N, p->D, p->seqlens_k, p->Hkv, mean, ws + l.mean_ws,
                    l.total - l.mean_ws, stream);
    if (rc != SL8_OK) return rc;
    rc = sl8_smooth_quant_k(p->k, p->dtype, bhk, p->N, p->D, mean, k_i8, k_scale, nullptr, stream);
    if (rc != SL8_OK) return rc;
  }
  sl8_fwd_params f{};
  f.q = q_i8; f.q_scale = q_scale; f.k = k_i8; f.k_scale = k_scale; f.v = p->v; f.out = p->out;
  f.seqlens_q = p->seqlens_q; f.seqlens_k = p->seqlens_k;
  f.B = p->B; f.Hq = p->Hq; f.Hkv = p->Hkv; f.M = p->M; f.N = p->N; f.D = p->D; f.v_dtype = p->dtype;
  f.causal = p->causal; f.window_left = p->window_left; f.backend = SL8_BACKEND_TCGEN05;
  f.gate_flag = gate ? flag : nullptr; f.gate_want = 0;
  void* status = p->device_status != nullptr ? p->device_status : static_cast<void*>(ws);
  rc = sl8_attn_int8_fwd(&f, status, 256, stream);
  if (rc != SL8_OK || !gate) return rc;
  sl8_fp16_fwd_params h{};
  h.q = p->q; h.k = p->k; h.v = p->v; h.out = p->out; h.seqlens_q = p->seqlens_q; h.seqlens_k = p->seqlens_k;
  h.B = p->B; h.Hq = p->Hq; h.Hkv = p->Hkv; h.M = p->M; h.N = p->N; h.D = p->D; h.dtype = p->dtype;
  h.causal = p->causal; h.window_left = p->window_left; h.softmax_scale = (float)p->softmax_scale;
  h.backend = SL8_BACKEND_TCGEN05; h.gate_flag = flag; h.gate_want = 1;
  return sl8_attn_fp16_fwd(&h, status, 256, stream);
}
