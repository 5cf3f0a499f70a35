// attn_int8_fwd for tensors that live in HOST memory: the end-to-end form of the path (the
// reference's users hand the op CUDA tensors they first copied from the host, superl8/ops.py:70-175;
// this entry owns that copy too, so that it can overlap it with the kernels).
//
// The (batch, kv-head) units of the path are independent, so the call is cut into chunks of whole
// units -- a chunk is a run of consecutive KV heads of one batch element, with their query heads:
// contiguous in q, k, v and out -- that travel through three streams:
//   copy-in stream    host -> device copies of the chunk's q, k, v into one of `slots` staging slots
//   caller's stream   sl8_attn_int8_fwd_fused on the slot (gate decided on the device per chunk,
//                     Q / K prologue, int8 kernel or its full-precision sibling): no host read-back
//   copy-out stream   device -> host copy of the chunk's output
// ordered by events only (a slot is refilled when its kernels have finished, its output buffer is
// rewritten when the copy-out has finished); the host thread never waits.  Staging slots come from
// the caller's device workspace; streams and events are created once per device and kept.
#include "sl8_common.cuh"

#include <mutex>
#include <vector>

namespace {
constexpr int kMaxDevices = 64;
constexpr int kMaxSlots = 8;
constexpr size_t kAlign = 256;
inline size_t up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

struct DeviceState {
  bool ready = false;
  std::mutex enqueue;
  cudaStream_t h2d = nullptr, d2h = nullptr;
  cudaEvent_t arrived[kMaxSlots], computed[kMaxSlots], drained[kMaxSlots], start = nullptr;
};
DeviceState g_state[kMaxDevices];
std::mutex g_state_mutex;

int device_state(DeviceState** out) {
  int dev = 0;
  SL8_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SL8_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(g_state_mutex);
  DeviceState& st = g_state[dev];
  if (!st.ready) {
    SL8_CUDA_TRY(cudaStreamCreateWithFlags(&st.h2d, cudaStreamNonBlocking));
    SL8_CUDA_TRY(cudaStreamCreateWithFlags(&st.d2h, cudaStreamNonBlocking));
    SL8_CUDA_TRY(cudaEventCreateWithFlags(&st.start, cudaEventDisableTiming));
    for (int i = 0; i < kMaxSlots; ++i) {
      SL8_CUDA_TRY(cudaEventCreateWithFlags(&st.arrived[i], cudaEventDisableTiming));
      SL8_CUDA_TRY(cudaEventCreateWithFlags(&st.computed[i], cudaEventDisableTiming));
      SL8_CUDA_TRY(cudaEventCreateWithFlags(&st.drained[i], cudaEventDisableTiming));
    }
    st.ready = true;
  }
  *out = &st;
  return SL8_OK;
}

struct Plan {
  // Chunks are kv_per_chunk KV heads wide; in the automatic plan the LAST batch element is cut into
  // narrower ones (kv_tail heads), because what follows the last host->device copy -- the last
  // chunk's kernels and its copy back -- overlaps with nothing (S = 8192, 64 heads: 2.4 ms of copy
  // behind a 134 MB chunk, 0.6 ms behind a 34 MB one).
  int kv_per_chunk, chunks_per_batch, kv_tail, tail_chunks, n_chunks, slots;
  size_t q_bytes, kv_bytes, out_bytes, fused_ws, slot_bytes, total;
  sl8_fused_fwd_params chunk;   // shape of one (full-size) chunk
};

bool shape_ok(const sl8_host_fwd_params* p) {
  return p->B >= 0 && p->Hq >= 0 && p->Hkv >= 0 && p->M >= 0 && p->N >= 0 && (p->Hq == 0 || (p->Hkv > 0 && p->Hq % p->Hkv == 0));
}

Plan plan(const sl8_host_fwd_params* p) {
  Plan pl{};
  const int G = p->Hkv > 0 ? p->Hq / p->Hkv : 1;
  int kvc = p->kv_heads_per_chunk;
  if (kvc <= 0) {
    // enough chunks to keep fill and drain of the three-stage pipeline short (about 16 per call),
    // but not so small that a chunk's kernels no longer fill the GPU -- and no smaller than that:
    // on the S = 8192, 64-head workload 16 / 32 / 64 / 128 chunks (134 ... 17 MB of Q per copy) measure
    // 58.1 / 59.0 / 63.1 / 71.9 ms per call, whatever the number of staging slots
    kvc = p->Hkv;
    while (kvc > 1 && kvc % 2 == 0 && (int64_t)p->B * (p->Hkv / kvc) < 16 && (int64_t)(kvc / 2) * G * ((p->M + 127) / 128) >= 296) kvc /= 2;
  }
  if (kvc > p->Hkv) kvc = p->Hkv;
  while (kvc > 1 && p->Hkv % kvc) --kvc;
  if (kvc < 1) kvc = 1;
  pl.kv_per_chunk = kvc;
  pl.chunks_per_batch = p->Hkv > 0 ? p->Hkv / kvc : 0;
  pl.kv_tail = kvc;
  if (p->kv_heads_per_chunk <= 0)
    while (pl.kv_tail > 1 && pl.kv_tail % 2 == 0 && pl.kv_tail * 4 > kvc && (int64_t)(pl.kv_tail / 2) * G * ((p->M + 127) / 128) >= 296)
      pl.kv_tail /= 2;
  pl.tail_chunks = p->Hkv > 0 ? p->Hkv / pl.kv_tail : 0;
  pl.n_chunks = p->B > 0 ? (p->B - 1) * pl.chunks_per_batch + pl.tail_chunks : 0;
  pl.slots = p->slots <= 0 ? 3 : (p->slots < 2 ? 2 : (p->slots > kMaxSlots ? kMaxSlots : p->slots));
  pl.q_bytes = (size_t)kvc * G * p->M * p->D * 2;
  pl.kv_bytes = (size_t)kvc * p->N * p->D * 2;
  pl.out_bytes = pl.q_bytes;
  sl8_fused_fwd_params& c = pl.chunk;
  c.B = 1; c.Hq = kvc * G; c.Hkv = kvc; c.M = p->M; c.N = p->N; c.D = p->D; c.dtype = p->dtype;
  c.causal = p->causal; c.window_left = p->window_left; c.ratio_threshold = p->ratio_threshold;
  c.softmax_scale = p->softmax_scale;
  pl.fused_ws = up(sl8_attn_int8_fwd_fused_workspace(&c));
  pl.slot_bytes = up(pl.q_bytes) + 2 * up(pl.kv_bytes) + up(pl.out_bytes) + pl.fused_ws + kAlign /*gate flag*/;
  pl.total = 256 + (size_t)pl.slots * pl.slot_bytes;
  return pl;
}
}  // namespace

extern "C" size_t sl8_attn_int8_fwd_host_workspace(const sl8_host_fwd_params* p) {
  if (p == nullptr || !shape_ok(p) || p->D <= 0) return 256;
  return plan(p).total;
}

extern "C" int sl8_attn_int8_fwd_host_chunks(const sl8_host_fwd_params* p) {
  if (p == nullptr || !shape_ok(p) || p->D <= 0) return 0;
  return plan(p).n_chunks;
}

extern "C" int sl8_attn_int8_fwd_host(const sl8_host_fwd_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  if (p == nullptr) return SL8_ERR_NULL;
  if (!shape_ok(p)) return SL8_ERR_BAD_SHAPE;
  if (p->D != 64 && p->D != 128 && p->D != 256) return SL8_ERR_UNSUPPORTED;
  if (p->dtype != SL8_F16 && p->dtype != SL8_BF16) return SL8_ERR_BAD_DTYPE;
  if (p->N == 0 || p->softmax_scale < 0.0) return SL8_ERR_UNSUPPORTED;
  if ((int64_t)p->B * p->Hq * p->M == 0) return SL8_OK;
  if (!p->q || !p->k || !p->v || !p->out) return SL8_ERR_NULL;
  const Plan pl = plan(p);
  if (workspace == nullptr || workspace_bytes < pl.total) return SL8_ERR_WORKSPACE;
  if (!sl8::aligned16(workspace)) return SL8_ERR_MISALIGNED;
  DeviceState* st = nullptr;
  int rc = device_state(&st);
  if (rc != SL8_OK) return rc;
  // The copy streams and events are shared by every call on this device: an event wait binds to
  // the record that precedes it in host order, so one call's enqueue must not interleave with another's.
  std::lock_guard<std::mutex> enqueue_lock(st->enqueue);
  cudaStream_t cur = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const int G = p->Hq / p->Hkv;
  const size_t q_batch = (size_t)p->Hq * p->M * p->D * 2, kv_batch = (size_t)p->Hkv * p->N * p->D * 2;

  // everything the caller queued before this call (it may still be writing q, k, v or reading out)
  SL8_CUDA_TRY(cudaEventRecord(st->start, cur));
  SL8_CUDA_TRY(cudaStreamWaitEvent(st->h2d, st->start, 0));
  SL8_CUDA_TRY(cudaStreamWaitEvent(st->d2h, st->start, 0));
  SL8_CUDA_TRY(cudaMemsetAsync(ws, 0, 256, cur));   // the call's status word

  auto slot_base = [&](int s) { return ws + 256 + (size_t)s * pl.slot_bytes; };
  // chunk i = KV heads [h0, h0 + kvc) of batch element b
  const int body = (p->B - 1) * pl.chunks_per_batch;
  auto chunk_of = [&](int i, int* b, int* h0, int* kvc) {
    if (i < body) { *b = i / pl.chunks_per_batch; *h0 = (i % pl.chunks_per_batch) * pl.kv_per_chunk; *kvc = pl.kv_per_chunk; }
    else { *b = p->B - 1; *h0 = (i - body) * pl.kv_tail; *kvc = pl.kv_tail; }
  };
  auto upload = [&](int i) -> int {
    const int s = i % pl.slots;
    int b, h0, kvc;
    chunk_of(i, &b, &h0, &kvc);
    const size_t qb = pl.q_bytes / pl.kv_per_chunk * kvc, kvb = pl.kv_bytes / pl.kv_per_chunk * kvc;
    uint8_t* base = slot_base(s);
    if (i >= pl.slots) SL8_CUDA_TRY(cudaStreamWaitEvent(st->h2d, st->computed[s], 0));   // the slot's previous kernels
    const uint8_t* hq = static_cast<const uint8_t*>(p->q) + (size_t)b * q_batch + (size_t)h0 * G * p->M * p->D * 2;
    const uint8_t* hk = static_cast<const uint8_t*>(p->k) + (size_t)b * kv_batch + (size_t)h0 * p->N * p->D * 2;
    const uint8_t* hv = static_cast<const uint8_t*>(p->v) + (size_t)b * kv_batch + (size_t)h0 * p->N * p->D * 2;
    SL8_CUDA_TRY(cudaMemcpyAsync(base, hq, qb, cudaMemcpyHostToDevice, st->h2d));
    SL8_CUDA_TRY(cudaMemcpyAsync(base + up(pl.q_bytes), hk, kvb, cudaMemcpyHostToDevice, st->h2d));
    SL8_CUDA_TRY(cudaMemcpyAsync(base + up(pl.q_bytes) + up(pl.kv_bytes), hv, kvb, cudaMemcpyHostToDevice, st->h2d));
    SL8_CUDA_TRY(cudaEventRecord(st->arrived[s], st->h2d));
    return SL8_OK;
  };

  const int ahead = pl.slots - 1;   // copies run this many chunks ahead of the kernels
  for (int i = 0; i < ahead && i < pl.n_chunks; ++i)
    if ((rc = upload(i)) != SL8_OK) return rc;
  for (int i = 0; i < pl.n_chunks; ++i) {
    const int s = i % pl.slots;
    int b, h0, kvc;
    chunk_of(i, &b, &h0, &kvc);
    uint8_t* base = slot_base(s);
    uint8_t* d_out = base + up(pl.q_bytes) + 2 * up(pl.kv_bytes);
    uint8_t* fused_ws = d_out + up(pl.out_bytes);
    int32_t* flag = reinterpret_cast<int32_t*>(fused_ws + pl.fused_ws);
    SL8_CUDA_TRY(cudaStreamWaitEvent(cur, st->arrived[s], 0));
    if (i >= pl.slots) SL8_CUDA_TRY(cudaStreamWaitEvent(cur, st->drained[s], 0));   // the slot's previous output has left
    sl8_fused_fwd_params c = pl.chunk;
    c.Hq = kvc * G; c.Hkv = kvc;
    c.q = base; c.k = base + up(pl.q_bytes); c.v = base + up(pl.q_bytes) + up(pl.kv_bytes); c.out = d_out;
    c.gate_flag = flag; c.device_status = ws;
    if ((rc = sl8_attn_int8_fwd_fused(&c, fused_ws, pl.fused_ws, stream)) != SL8_OK) return rc;
    SL8_CUDA_TRY(cudaEventRecord(st->computed[s], cur));
    if (i + ahead < pl.n_chunks && (rc = upload(i + ahead)) != SL8_OK) return rc;
    SL8_CUDA_TRY(cudaStreamWaitEvent(st->d2h, st->computed[s], 0));
    uint8_t* ho = static_cast<uint8_t*>(p->out) + (size_t)b * q_batch + (size_t)h0 * G * p->M * p->D * 2;
    SL8_CUDA_TRY(cudaMemcpyAsync(ho, d_out, pl.out_bytes / pl.kv_per_chunk * kvc, cudaMemcpyDeviceToHost, st->d2h));
    if (p->gate_flags != nullptr)
      SL8_CUDA_TRY(cudaMemcpyAsync(p->gate_flags + i, flag, sizeof(int32_t), cudaMemcpyDeviceToHost, st->d2h));
    SL8_CUDA_TRY(cudaEventRecord(st->drained[s], st->d2h));
  }
  // the caller's stream is ordered after the last copy-out (and after the copy-in stream's last event)
  SL8_CUDA_TRY(cudaStreamWaitEvent(cur, st->drained[(pl.n_chunks - 1) % pl.slots], 0));
  for (int s = 0; s < pl.slots && s < pl.n_chunks; ++s) SL8_CUDA_TRY(cudaStreamWaitEvent(cur, st->drained[s], 0));
  return SL8_OK;
}
