// Thin torch extension over the C ABI of libsuperl8_b200.so: the operators the reference binds
// into its compiled module `superl8._C` (reference csrc/fni8_api.cpp:225-291) with the same names,
// argument lists and TORCH_CHECK key words, plus the whole prefill step from 16-bit tensors in one
// call.  torch supplies tensors, the caching allocator and the current stream; every kernel is
// the library's.  Nothing here computes, and nothing runs on the CPU.
#include <torch/extension.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cmath>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <utility>

#include "../../../include/superl8_b200.h"

namespace {

using at::Tensor;

struct PerStream {
  Tensor status;      // 256 bytes: the status word of the bounded device-side waits
  Tensor gate_flag;   // int32 [1]: the accuracy gate's device flag
  Tensor decode_ws;   // split partials of the decode, grown on demand
};
std::mutex g_mu;
std::map<std::pair<int, uintptr_t>, PerStream> g_cache;

void* stream_of(const Tensor& t) { return static_cast<void*>(at::cuda::getCurrentCUDAStream(t.get_device()).stream()); }

PerStream& per_stream(const Tensor& like) {
  const int dev = like.get_device();
  const auto key = std::make_pair(dev, reinterpret_cast<uintptr_t>(stream_of(like)));
  std::lock_guard<std::mutex> lock(g_mu);
  PerStream& ps = g_cache[key];
  if (!ps.status.defined()) {
    ps.status = at::zeros({64}, like.options().dtype(at::kInt));
    ps.gate_flag = at::zeros({1}, like.options().dtype(at::kInt));
  }
  return ps;
}

// Numbers go into messages through std::to_string: streaming an int into c10::str from this module
// crashed on a GPU box (number formatting through locale facets), strings do not.  The module also
// calls nothing of the CUDA runtime itself (flags are read and cleared through tensor methods), so
// it links torch and the library only.
void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == SL8_OK, "superl8_b200 ", what, ": ", sl8_status_string(rc), " (status ", std::to_string(rc), ")");
}

int dtype_code(const Tensor& t, const char* what) {
  if (t.scalar_type() == at::kHalf) return SL8_F16;
  if (t.scalar_type() == at::kBFloat16) return SL8_BF16;
  if (t.scalar_type() == at::kFloat) return SL8_F32;
  TORCH_CHECK(false, "superl8_b200 ", what, ": tensor must be float16, bfloat16 or float32");
  return -1;
}

struct Dims { int B, H, Hkv, M, N, D; };

Dims fwd_checks(const Tensor& q, const Tensor& q_scale, const Tensor& k, const Tensor& k_scale, const Tensor& v,
                const char* what) {
  TORCH_CHECK(q.is_cuda() && q_scale.is_cuda() && k.is_cuda() && k_scale.is_cuda() && v.is_cuda(), what,
              ": all inputs (incl. scales) must be CUDA tensors");
  TORCH_CHECK(q.get_device() == k.get_device() && q.get_device() == v.get_device() && q.get_device() == q_scale.get_device() &&
                  q.get_device() == k_scale.get_device(), what, ": all inputs must be on the same device");
  TORCH_CHECK(q.scalar_type() == at::kChar && k.scalar_type() == at::kChar, what, ": q/k must be int8");
  TORCH_CHECK(q_scale.scalar_type() == at::kFloat && k_scale.scalar_type() == at::kFloat, what, ": scales must be float32");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, what, ": expect [B,H,S,D]");
  TORCH_CHECK(q.is_contiguous() && q_scale.is_contiguous() && k.is_contiguous() && k_scale.is_contiguous() && v.is_contiguous(),
              what, ": inputs must be contiguous");
  Dims d{(int)q.size(0), (int)q.size(1), (int)k.size(1), (int)q.size(2), (int)k.size(2), (int)q.size(3)};
  TORCH_CHECK(k.size(0) == d.B && v.size(0) == d.B && v.size(1) == d.Hkv, what, ": batch/head mismatch");
  TORCH_CHECK(d.Hkv > 0 && d.H % d.Hkv == 0, what, ": H_q must be divisible by H_kv (GQA)");
  TORCH_CHECK(k.size(3) == d.D && v.size(3) == d.D && v.size(2) == d.N, what, ": K/V shape mismatch");
  TORCH_CHECK(q_scale.numel() == (int64_t)d.B * d.H * d.M && k_scale.numel() == (int64_t)d.B * d.Hkv * d.N, what,
              ": scale shape mismatch");
  return d;
}

// reference csrc/fni8_api.cpp:286-291 (op csrc/kernel/quant_rowwise.cu:84-121)
std::tuple<Tensor, Tensor> quantize_i8_rowwise(const Tensor& x_in) {
  TORCH_CHECK(x_in.is_cuda(), "superl8_b200 quantize_i8_rowwise: x must be a CUDA tensor");
  TORCH_CHECK(x_in.dim() == 2, "superl8_b200 quantize_i8_rowwise: expect [M, K]");
  const int dt = dtype_code(x_in, "quantize_i8_rowwise");
  const Tensor x = x_in.contiguous();
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor q = at::empty(x.sizes(), x.options().dtype(at::kChar));
  Tensor scale = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  check_rc(sl8_quantize_i8_rowwise(x.data_ptr(), dt, x.size(0), x.size(1), q.data_ptr<int8_t>(), scale.data_ptr<float>(),
                                   stream_of(x)), "quantize_i8_rowwise");
  return {q, scale};
}

std::tuple<Tensor, Tensor> run_fwd(const Tensor& q, const Tensor& q_scale, const Tensor& k, const Tensor& k_scale,
                                   const Tensor& v, bool causal, int64_t window_left, bool want_lse) {
  const char* what = "superl8_b200";
  const Dims d = fwd_checks(q, q_scale, k, k_scale, v, what);
  TORCH_CHECK(v.scalar_type() == at::kHalf || v.scalar_type() == at::kBFloat16, what, ": v must be float16 or bfloat16");
  TORCH_CHECK(d.D == 32 || d.D == 64 || d.D == 72 || d.D == 80 || d.D == 128 || d.D == 256, what,
              ": head dim must be 32/64/72/80/128/256, got ", std::to_string(d.D));
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty({d.B, d.H, d.M, d.D}, v.options());
  Tensor lse = want_lse ? at::empty({d.B, d.H, d.M}, q.options().dtype(at::kFloat)) : at::empty({0}, q.options().dtype(at::kFloat));
  if (d.M == 0 || d.B == 0 || d.H == 0) return {out, lse};
  sl8_fwd_params p{};
  p.q = q.data_ptr<int8_t>(); p.q_scale = q_scale.data_ptr<float>(); p.k = k.data_ptr<int8_t>();
  p.k_scale = k_scale.data_ptr<float>(); p.v = v.data_ptr(); p.out = out.data_ptr();
  p.lse = want_lse ? lse.data_ptr<float>() : nullptr;
  p.B = d.B; p.Hq = d.H; p.Hkv = d.Hkv; p.M = d.M; p.N = d.N; p.D = d.D;
  p.v_dtype = v.scalar_type() == at::kHalf ? SL8_F16 : SL8_BF16;
  p.causal = causal ? 1 : 0; p.window_left = (int32_t)window_left; p.backend = SL8_BACKEND_AUTO;
  PerStream& ps = per_stream(q);
  check_rc(sl8_attn_int8_fwd(&p, ps.status.data_ptr(), 256, stream_of(q)), "attn_int8_fwd");
  return {out, lse};
}

// reference csrc/fni8_api.cpp:225-229
Tensor attn_int8_fwd(const Tensor& q, const Tensor& q_scale, const Tensor& k, const Tensor& k_scale, const Tensor& v,
                     bool causal, int64_t window_left) {
  return std::get<0>(run_fwd(q, q_scale, k, k_scale, v, causal, window_left, false));
}

// reference csrc/fni8_api.cpp:230-233
std::tuple<Tensor, Tensor> attn_int8_fwd_train(const Tensor& q, const Tensor& q_scale, const Tensor& k,
                                               const Tensor& k_scale, const Tensor& v, bool causal) {
  return run_fwd(q, q_scale, k, k_scale, v, causal, -1, true);
}

std::tuple<Tensor, Tensor> run_fp16(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, bool causal,
                                    c10::optional<double> scale, int64_t window_left, const c10::optional<Tensor>& mask,
                                    bool want_lse) {
  const char* what = "superl8_b200 fp16 fwd";
  TORCH_CHECK(q_in.is_cuda() && k_in.is_cuda() && v_in.is_cuda(), what, ": all inputs (incl. scales) must be CUDA tensors");
  TORCH_CHECK(q_in.scalar_type() == at::kHalf || q_in.scalar_type() == at::kBFloat16, what, ": q must be float16 or bfloat16");
  TORCH_CHECK(k_in.scalar_type() == q_in.scalar_type() && v_in.scalar_type() == q_in.scalar_type(), what,
              ": q, k, v must share one dtype");
  TORCH_CHECK(q_in.dim() == 4 && k_in.dim() == 4 && v_in.dim() == 4, what, ": expect [B,H,S,D]");
  const Tensor q = q_in.contiguous(), k = k_in.contiguous(), v = v_in.contiguous();
  const int B = q.size(0), H = q.size(1), M = q.size(2), D = q.size(3), Hkv = k.size(1), N = k.size(2);
  TORCH_CHECK(k.size(0) == B && v.size(0) == B && v.size(1) == Hkv, what, ": batch/head mismatch");
  TORCH_CHECK(Hkv > 0 && H % Hkv == 0, what, ": H_q must be divisible by H_kv (GQA)");
  TORCH_CHECK(k.size(3) == D && v.size(3) == D && v.size(2) == N, what, ": K/V shape mismatch");
  TORCH_CHECK(D == 32 || D == 64 || D == 72 || D == 80 || D == 128 || D == 256, what,
              ": head dim must be 32/64/72/80/128/256, got ", std::to_string(D));
  sl8_fp16_fwd_params p{};
  if (mask.has_value() && mask->defined()) {
    const Tensor& m = *mask;
    TORCH_CHECK(m.is_cuda() && m.get_device() == q.get_device(), what, ": mask must be a CUDA tensor on q's device");
    TORCH_CHECK(m.scalar_type() == q.scalar_type(), what, ": mask dtype must match q/k/v");
    TORCH_CHECK(m.dim() == 4, what, ": mask must be 4-D [B|1, H|1, M, N]");
    TORCH_CHECK(m.size(2) == M && m.size(3) == N, what, ": mask trailing dims must be [M,N]");
    TORCH_CHECK((m.size(0) == B || m.size(0) == 1) && (m.size(1) == H || m.size(1) == 1), what,
                ": mask leading dims must broadcast to [B,H]");
    p.mask = m.data_ptr();
    p.mask_stride_b = m.size(0) == 1 ? 0 : m.stride(0);
    p.mask_stride_h = m.size(1) == 1 ? 0 : m.stride(1);
    p.mask_stride_m = m.stride(2);
    p.mask_stride_n = m.stride(3);
  }
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty({B, H, M, D}, v.options());
  Tensor lse = want_lse ? at::empty({B, H, M}, v.options().dtype(at::kFloat)) : Tensor();
  if (out.numel() == 0) return {out, lse};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.out = out.data_ptr();
  p.lse = want_lse ? lse.data_ptr<float>() : nullptr;
  p.B = B; p.Hq = H; p.Hkv = Hkv; p.M = M; p.N = N; p.D = D;
  p.dtype = q.scalar_type() == at::kHalf ? SL8_F16 : SL8_BF16;
  p.causal = causal ? 1 : 0; p.window_left = (int32_t)window_left;
  p.softmax_scale = scale.has_value() ? (float)*scale : (float)(1.0 / std::sqrt((double)D));
  p.backend = SL8_BACKEND_AUTO;
  PerStream& ps = per_stream(q);
  check_rc(sl8_attn_fp16_fwd(&p, ps.status.data_ptr(), 256, stream_of(q)), "attn_fp16_fwd");
  return {out, lse};
}

// reference csrc/fni8_api.cpp:234-244
Tensor attn_fp16_fwd(const Tensor& q, const Tensor& k, const Tensor& v, bool causal, c10::optional<double> scale,
                     int64_t window_left, const c10::optional<Tensor>& mask) {
  return std::get<0>(run_fp16(q, k, v, causal, scale, window_left, mask, false));
}
// reference csrc/fni8_api.cpp:245-248
std::tuple<Tensor, Tensor> attn_fp16_fwd_train(const Tensor& q, const Tensor& k, const Tensor& v, bool causal,
                                               c10::optional<double> scale) {
  return run_fp16(q, k, v, causal, scale, -1, c10::nullopt, true);
}

// reference csrc/fni8_api.cpp:260-263 (op csrc/kernel/attn_decode.cu:163-240)
Tensor attn_int8_decode(const Tensor& q, const Tensor& q_scale, const Tensor& k, const Tensor& k_scale, const Tensor& v,
                        int64_t num_splits) {
  const char* what = "superl8_b200 decode";
  const Dims d = fwd_checks(q, q_scale, k, k_scale, v, what);
  TORCH_CHECK(v.scalar_type() == at::kHalf, what, ": v must be float16");
  TORCH_CHECK(d.M == 1, what, ": query length M must be 1 (decode)");
  TORCH_CHECK(d.D == 32 || d.D == 64 || d.D == 128 || d.D == 256, what, ": head dim must be 32/64/128/256, got ", std::to_string(d.D));
  TORCH_CHECK(num_splits != 0, what, ": num_splits=0 is invalid; use -1 for auto or 1..256");
  if (num_splits < 0) num_splits = -1;
  TORCH_CHECK(num_splits <= 256, what, ": num_splits must be 1..256, got ", std::to_string(num_splits));
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty({d.B, d.H, 1, d.D}, v.options());
  if (out.numel() == 0) return out;
  sl8_decode_params p{};
  p.q = q.data_ptr<int8_t>(); p.q_scale = q_scale.data_ptr<float>(); p.k = k.data_ptr<int8_t>();
  p.k_scale = k_scale.data_ptr<float>(); p.v = v.data_ptr(); p.out = out.data_ptr();
  p.B = d.B; p.Hq = d.H; p.Hkv = d.Hkv; p.N = d.N; p.D = d.D; p.num_splits = (int32_t)num_splits;
  const size_t need = sl8_attn_int8_decode_workspace(&p);
  PerStream& ps = per_stream(q);
  if (!ps.decode_ws.defined() || (size_t)ps.decode_ws.numel() < need) {
    ps.decode_ws = at::empty({(int64_t)need}, q.options().dtype(at::kByte));
    ps.decode_ws.narrow(0, 0, 256).zero_();
  }
  check_rc(sl8_attn_int8_decode(&p, ps.decode_ws.data_ptr(), (size_t)ps.decode_ws.numel(), stream_of(q)), "attn_int8_decode");
  return out;
}

// reference csrc/fni8_api.cpp:256-259 (op csrc/kernel/attn_bwd.cu:62-109)
std::tuple<Tensor, Tensor, Tensor> attn_bwd(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, const Tensor& o_in,
                                            const Tensor& do_in, const Tensor& lse_in, double scale, bool causal) {
  const char* what = "superl8_b200 bwd";
  for (const Tensor* t : {&q_in, &k_in, &v_in, &o_in, &do_in, &lse_in}) {
    TORCH_CHECK(t->is_cuda(), what, ": all inputs must be CUDA");
    TORCH_CHECK(t->get_device() == q_in.get_device(), what, ": all inputs must be on the same device");
  }
  TORCH_CHECK((q_in.scalar_type() == at::kHalf || q_in.scalar_type() == at::kBFloat16) && k_in.scalar_type() == q_in.scalar_type() &&
                  v_in.scalar_type() == q_in.scalar_type() && o_in.scalar_type() == q_in.scalar_type() &&
                  do_in.scalar_type() == q_in.scalar_type(), what, ": q/k/v/o/do must be float16 (or all bfloat16)");
  TORCH_CHECK(lse_in.scalar_type() == at::kFloat, what, ": lse must be float32");
  TORCH_CHECK(q_in.dim() == 4 && k_in.dim() == 4 && v_in.dim() == 4 && o_in.dim() == 4 && do_in.dim() == 4, what, ": expect [B,H,S,D]");
  const Tensor q = q_in.contiguous(), k = k_in.contiguous(), v = v_in.contiguous(), o = o_in.contiguous(),
               dout = do_in.contiguous(), lse = lse_in.contiguous();
  const int B = q.size(0), H = q.size(1), M = q.size(2), D = q.size(3), Hkv = k.size(1), N = k.size(2);
  TORCH_CHECK(Hkv > 0 && H % Hkv == 0, what, ": H_q must be divisible by H_kv (GQA)");
  TORCH_CHECK(D == 32 || D == 64 || D == 128, what, ": head dim must be 32/64/128, got ", std::to_string(D));
  TORCH_CHECK(k.sizes() == v.sizes() && k.size(0) == B && k.size(3) == D, what, ": K/V shape mismatch");
  TORCH_CHECK(o.sizes() == q.sizes() && dout.sizes() == q.sizes(), what, ": o/do must have q's shape");
  TORCH_CHECK(lse.numel() == (int64_t)B * H * M, what, ": lse must be [B,H,M]");
  const c10::cuda::CUDAGuard guard(q.device());
  Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
  sl8_bwd_params p{};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.o = o.data_ptr(); p.dout = dout.data_ptr();
  p.lse = lse.data_ptr<float>(); p.dq = dq.data_ptr(); p.dk = dk.data_ptr(); p.dv = dv.data_ptr();
  p.B = B; p.Hq = H; p.Hkv = Hkv; p.M = M; p.N = N; p.D = D;
  p.dtype = q.scalar_type() == at::kHalf ? SL8_F16 : SL8_BF16;
  p.causal = causal ? 1 : 0; p.softmax_scale = (float)scale; p.backend = SL8_BACKEND_AUTO;
  const size_t need = sl8_attn_bwd_workspace(&p);
  Tensor ws = at::empty({(int64_t)need}, q.options().dtype(at::kByte));
  ws.narrow(0, 0, 256).zero_();
  check_rc(sl8_attn_bwd(&p, ws.data_ptr(), need, stream_of(q)), "attn_bwd");
  return {dq, dk, dv};
}

// The whole prefill step of the reference's Python entry (superl8/ops.py:70-175, default
// arguments apart from causal / scale / window_left) in one call: Q quantisation with the
// outlier statistic, the 4-byte read of the gate flag, then either the full-precision kernel
// (demoted) or K mean + K smoothing/quantisation + the int8 kernel.  gate == 0 skips the gate;
// ask_first reads Q once for the gate before quantising anything (a caller that expects a
// demotion saves the unused quantisation).  Returns (out, demoted).
std::tuple<Tensor, bool> attn_int8_prefill(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in, bool causal,
                                           double scale, int64_t window_left, bool gate, bool ask_first) {
  const char* what = "superl8_b200 prefill";
  TORCH_CHECK(q_in.is_cuda() && k_in.is_cuda() && v_in.is_cuda(), what, ": all inputs (incl. scales) must be CUDA tensors");
  TORCH_CHECK(q_in.scalar_type() == at::kHalf || q_in.scalar_type() == at::kBFloat16, what, ": q must be float16 or bfloat16");
  TORCH_CHECK(k_in.scalar_type() == q_in.scalar_type() && v_in.scalar_type() == q_in.scalar_type(), what,
              ": q, k, v must share one dtype");
  TORCH_CHECK(q_in.dim() == 4 && k_in.dim() == 4 && v_in.dim() == 4, what, ": expect [B,H,S,D]");
  const Tensor q = q_in.contiguous(), k = k_in.contiguous(), v = v_in.contiguous();
  const int B = q.size(0), H = q.size(1), M = q.size(2), D = q.size(3), Hkv = k.size(1), N = k.size(2);
  TORCH_CHECK(k.size(0) == B && v.size(0) == B && v.size(1) == Hkv, what, ": batch/head mismatch");
  TORCH_CHECK(Hkv > 0 && H % Hkv == 0, what, ": H_q must be divisible by H_kv (GQA)");
  TORCH_CHECK(k.size(3) == D && v.size(3) == D && v.size(2) == N, what, ": K/V shape mismatch");
  TORCH_CHECK(D == 32 || D == 64 || D == 72 || D == 80 || D == 128 || D == 256, what,
              ": head dim must be 32/64/72/80/128/256, got ", std::to_string(D));
  const int dt = q.scalar_type() == at::kHalf ? SL8_F16 : SL8_BF16;
  const c10::cuda::CUDAGuard guard(q.device());
  void* st = stream_of(q);
  PerStream& ps = per_stream(q);
  Tensor out = at::empty({B, H, M, D}, v.options());
  if (out.numel() == 0) return {out, false};
  const int64_t qrows = (int64_t)B * H * M;
  const float fold = (float)(scale * 1.4426950408889634);
  int32_t* flag = ps.gate_flag.data_ptr<int32_t>();
  Tensor q_i8, q_scale;
  bool demoted = false;
  auto read_flag = [&]() { return ps.gate_flag.item<int32_t>() != 0; };   // the 4-byte device->host read
  auto quantise_q = [&](bool with_gate) {
    q_i8 = at::empty(q.sizes(), q.options().dtype(at::kChar));
    q_scale = at::empty({B, H, M}, q.options().dtype(at::kFloat));
    check_rc(sl8_quant_q_prologue(q.data_ptr(), dt, qrows, D, fold, 12.f, q_i8.data_ptr<int8_t>(), q_scale.data_ptr<float>(),
                                  nullptr, with_gate ? flag : nullptr, st), "quant_q_prologue");
  };
  if (gate) ps.gate_flag.zero_();
  if (gate && ask_first) {
    check_rc(sl8_q_outlier_gate(q.data_ptr(), dt, qrows, D, 12.f, flag, st), "q_outlier_gate");
    demoted = read_flag();
    if (!demoted) quantise_q(false);
  } else {
    quantise_q(gate);
    if (gate) demoted = read_flag();
  }
  if (demoted) {
    sl8_fp16_fwd_params h{};
    h.q = q.data_ptr(); h.k = k.data_ptr(); h.v = v.data_ptr(); h.out = out.data_ptr();
    h.B = B; h.Hq = H; h.Hkv = Hkv; h.M = M; h.N = N; h.D = D; h.dtype = dt; h.causal = causal ? 1 : 0;
    h.window_left = (int32_t)window_left; h.softmax_scale = (float)scale; h.backend = SL8_BACKEND_AUTO;
    check_rc(sl8_attn_fp16_fwd(&h, ps.status.data_ptr(), 256, st), "attn_fp16_fwd");
    return {out, true};
  }
  const int64_t bhk = (int64_t)B * Hkv;
  Tensor k_i8 = at::empty(k.sizes(), k.options().dtype(at::kChar));
  Tensor k_scale = at::empty({B, Hkv, N}, k.options().dtype(at::kFloat));
  if (N > 0 && sl8_k_prologue_fused_ok(dt, bhk, N, D)) {   // one launch, K read from HBM once
    Tensor mean = at::empty({bhk * D}, k.options().dtype(at::kFloat));
    check_rc(sl8_k_prologue(k.data_ptr(), dt, bhk, N, D, nullptr, 1, mean.data_ptr<float>(), k_i8.data_ptr<int8_t>(),
                            k_scale.data_ptr<float>(), nullptr, st), "k_prologue");
  } else if (N > 0) {
    const size_t mws = sl8_k_mean_workspace(bhk, N, D);
    Tensor mean = at::empty({(int64_t)(bhk * D * 4 + mws + 256)}, k.options().dtype(at::kByte));
    float* mean_p = reinterpret_cast<float*>(mean.data_ptr());
    uint8_t* mws_p = reinterpret_cast<uint8_t*>(mean.data_ptr()) + (((size_t)bhk * D * 4 + 255) / 256) * 256;
    check_rc(sl8_k_mean(k.data_ptr(), dt, bhk, N, D, nullptr, 1, mean_p, mws_p, mws, st), "k_mean");
    check_rc(sl8_smooth_quant_k(k.data_ptr(), dt, bhk, N, D, mean_p, k_i8.data_ptr<int8_t>(), k_scale.data_ptr<float>(),
                                nullptr, st), "smooth_quant_k");
  }
  sl8_fwd_params p{};
  p.q = q_i8.data_ptr<int8_t>(); p.q_scale = q_scale.data_ptr<float>(); p.k = k_i8.data_ptr<int8_t>();
  p.k_scale = k_scale.data_ptr<float>(); p.v = v.data_ptr(); p.out = out.data_ptr();
  p.B = B; p.Hq = H; p.Hkv = Hkv; p.M = M; p.N = N; p.D = D; p.v_dtype = dt; p.causal = causal ? 1 : 0;
  p.window_left = (int32_t)window_left; p.backend = scale < 0 ? SL8_BACKEND_MMA : SL8_BACKEND_AUTO;
  check_rc(sl8_attn_int8_fwd(&p, ps.status.data_ptr(), 256, st), "attn_int8_fwd");
  return {out, false};
}

// Synchronises the current stream of `like`'s device and returns (and clears) its status word.
int64_t device_status(const Tensor& like) {
  const c10::cuda::CUDAGuard guard(like.device());
  PerStream& ps = per_stream(like);
  int rc = sl8_read_device_status(ps.status.data_ptr(), stream_of(like));
  if (rc == SL8_OK && ps.decode_ws.defined()) rc = sl8_read_device_status(ps.decode_ws.data_ptr(), stream_of(like));
  return rc;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "superl8_b200: the reference's compiled operators for the int8 attention path, over libsuperl8_b200.so";
  m.def("quantize_i8_rowwise", &quantize_i8_rowwise, py::arg("x"));
  m.def("attn_int8_fwd", &attn_int8_fwd, py::arg("q"), py::arg("q_scale"), py::arg("k"), py::arg("k_scale"), py::arg("v"),
        py::arg("causal") = false, py::arg("window_left") = -1);
  m.def("attn_int8_fwd_train", &attn_int8_fwd_train, py::arg("q"), py::arg("q_scale"), py::arg("k"), py::arg("k_scale"),
        py::arg("v"), py::arg("causal") = false);
  m.def("attn_fp16_fwd", &attn_fp16_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("causal") = false,
        py::arg("scale") = c10::nullopt, py::arg("window_left") = -1, py::arg("mask") = c10::nullopt);
  m.def("attn_fp16_fwd_train", &attn_fp16_fwd_train, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("causal") = false,
        py::arg("scale") = c10::nullopt);
  m.def("attn_bwd", &attn_bwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("o"), py::arg("do_"), py::arg("lse"),
        py::arg("scale"), py::arg("causal") = false);
  m.def("attn_int8_decode", &attn_int8_decode, py::arg("q"), py::arg("q_scale"), py::arg("k"), py::arg("k_scale"),
        py::arg("v"), py::arg("num_splits") = -1);
  m.def("attn_int8_prefill", &attn_int8_prefill, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("causal") = false,
        py::arg("scale") = 0.0, py::arg("window_left") = -1, py::arg("gate") = true, py::arg("ask_first") = false);
  m.def("device_status", &device_status, py::arg("like"));
}
