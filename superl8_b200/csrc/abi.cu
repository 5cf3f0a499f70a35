// Library-level pieces of the C ABI: version, status names, the device status
// word, and the tensor-map builder shared by the TMA kernels.
#include "sl8_common.cuh"

#include <mutex>

extern "C" int sl8_abi_version(void) { return SL8_ABI_VERSION; }

extern "C" const char* sl8_status_string(int status) {
  switch (status) {
    case SL8_OK: return "ok";
    case SL8_ERR_BAD_HEAD_DIM: return "head dim must be 32/64/72/80/128/256 (decode: 32/64/128/256)";
    case SL8_ERR_BAD_DTYPE: return "v must be float16 or bfloat16 (decode: float16)";
    case SL8_ERR_MISALIGNED: return "device pointers must be 16-byte aligned";
    case SL8_ERR_BAD_NUM_SPLITS: return "num_splits must be 1..256 (or -1 for auto)";
    case SL8_ERR_WORKSPACE: return "workspace missing or too small";
    case SL8_ERR_BAD_SHAPE: return "shape mismatch (sizes must be >= 0 and H_q divisible by H_kv)";
    case SL8_ERR_NULL: return "required pointer is null";
    case SL8_ERR_CUDA: return "CUDA call failed";
    case SL8_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
    case SL8_ERR_UNSUPPORTED: return "request not supported by the selected backend";
    case SL8_ERR_TOO_LARGE: return "request exceeds a built-in capacity";
    default: return "unknown status";
  }
}

extern "C" int sl8_read_device_status(void* workspace, void* stream) {
  if (workspace == nullptr) return SL8_ERR_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int host = 0;
  SL8_CUDA_TRY(cudaMemcpyAsync(&host, workspace, sizeof(int), cudaMemcpyDeviceToHost, s));
  SL8_CUDA_TRY(cudaStreamSynchronize(s));
  if (host != 0) SL8_CUDA_TRY(cudaMemsetAsync(workspace, 0, sizeof(int), s));
  return host == 0 ? SL8_OK : SL8_ERR_DEVICE_TIMEOUT;
}

// ---- self-test of the bounded wait ----------------------------------------------------------
// One block waits, with the kernels' own mbar_wait_limit, on a barrier that nothing ever arrives
// at; the wait runs out after limit_ns, raises the status word and the kernel returns normally.
namespace sl8 {
namespace {
__global__ void __launch_bounds__(32) wait_selftest_kernel(int* status, unsigned long long limit_ns, int* returned) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait_limit(&bar, 0, status, limit_ns);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (threadIdx.x == 0 && returned != nullptr) *returned = ok ? 1 : 2;   // 2: the wait gave up, as it must
}
}  // namespace
}  // namespace sl8

extern "C" int sl8_wait_timeout_selftest(void* workspace, size_t workspace_bytes, uint64_t limit_ns, void* stream) {
  if (workspace == nullptr || workspace_bytes < 256) return SL8_ERR_WORKSPACE;
  if (limit_ns == 0 || limit_ns > 100000000ull) return SL8_ERR_BAD_SHAPE;   // at most 0.1 s
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = reinterpret_cast<int*>(workspace);
  sl8::wait_selftest_kernel<<<1, 32, 0, s>>>(status, limit_ns, status + 1);
  return cudaGetLastError() == cudaSuccess ? SL8_OK : SL8_ERR_CUDA;
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

void resolve_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
}
}  // namespace

int sl8_make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t rows,
                     uint64_t heads, uint32_t box_inner, uint32_t box_rows, int swizzle_bytes) {
  std::call_once(g_encode_once, resolve_encode);
  if (g_encode == nullptr) return SL8_ERR_CUDA;
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                           : (elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_UINT32);
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  if (swizzle_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  cuuint64_t dims[3] = {inner, rows ? rows : 1, heads ? heads : 1};
  cuuint64_t strides[2] = {inner * elem_bytes, inner * elem_bytes * (rows ? rows : 1)};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SL8_OK : SL8_ERR_CUDA;
}

// Token-major packed tensor [tokens, heads, inner]: dimensions {inner, heads, tokens}, a box of
// box_rows tokens of one head (coordinates: inner offset, head, first token).
int sl8_make_tmap_packed(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t heads,
                         uint64_t tokens, uint32_t box_inner, uint32_t box_rows, int swizzle_bytes) {
  std::call_once(g_encode_once, resolve_encode);
  if (g_encode == nullptr) return SL8_ERR_CUDA;
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                           : (elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_UINT32);
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  if (swizzle_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  cuuint64_t dims[3] = {inner, heads ? heads : 1, tokens ? tokens : 1};
  cuuint64_t strides[2] = {inner * elem_bytes, inner * elem_bytes * (heads ? heads : 1)};
  cuuint32_t box[3] = {box_inner, 1, box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SL8_OK : SL8_ERR_CUDA;
}
