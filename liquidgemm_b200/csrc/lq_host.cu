// One W4A8 linear layer for callers whose activations and outputs live in HOST memory: a single C call
// enqueues the upload, the per-token quantiser, the fused linear and the download on one stream.
// The reference does these moves in Python around its operators (liquidgemm/ops.py:185-201 moves
// every operand with .cuda() and returns a tensor the caller copies back); doing them behind the C
// boundary removes four Python-level dispatches per layer, which is what an end-to-end measurement
// from host buffers is otherwise made of.
#include <stdint.h>

#include "lq_common.cuh"

namespace {

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }
inline size_t dtype_bytes(int dt) { return dt == LQ_DT_F32 ? 4 : 2; }

struct Scratch {
  size_t x, xq, ascale, y, total;
};

Scratch layout(int M, int N, int K, int x_dtype, int out_dtype) {
  Scratch s;
  s.x = 0;
  s.xq = align256((size_t)M * K * dtype_bytes(x_dtype));
  s.ascale = s.xq + align256((size_t)M * K);
  s.y = s.ascale + align256((size_t)M * 4);
  s.total = s.y + align256((size_t)M * N * dtype_bytes(out_dtype));
  return s;
}

}  // namespace

extern "C" {

LQ_API size_t lq_linear_host_scratch_bytes(int M, int N, int K, int x_dtype, int out_dtype) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return layout(M, N, K, x_dtype, out_dtype).total;
}

LQ_API int lq_w4a8_linear_host(const void* x_host, int x_dtype, const void* blob, const void* s1, void* y_host,
                               int out_dtype, int M, int N, int K, void* scratch, size_t scratch_bytes,
                               void* workspace, size_t workspace_bytes, void* stream) {
  if (!x_host || !blob || !s1 || !y_host || !scratch) return LQ_ERR_BAD_ARG;
  if (x_dtype < LQ_DT_BF16 || x_dtype > LQ_DT_F32 || out_dtype < LQ_DT_BF16 || out_dtype > LQ_DT_F32)
    return LQ_ERR_BAD_ARG;
  if (M <= 0 || N <= 0 || K < 128 || K % 128) return LQ_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(scratch) & 255u) return LQ_ERR_BAD_ARG;
  const Scratch s = layout(M, N, K, x_dtype, out_dtype);
  if (scratch_bytes < s.total) return LQ_ERR_WORKSPACE;
  uint8_t* base = static_cast<uint8_t*>(scratch);
  cudaStream_t st = lq::as_stream(stream);
  cudaError_t e = cudaMemcpyAsync(base + s.x, x_host, (size_t)M * K * dtype_bytes(x_dtype), cudaMemcpyHostToDevice, st);
  if (e != cudaSuccess) {
    lq::record_cuda_error(e, "lq_w4a8_linear_host upload");
    return LQ_ERR_CUDA;
  }
  int rc = lq_quant_per_token(base + s.x, x_dtype, reinterpret_cast<int8_t*>(base + s.xq),
                              reinterpret_cast<float*>(base + s.ascale), M, K, stream);
  if (rc) return rc;
  rc = lq_w4a8_gemm_fused(reinterpret_cast<const int8_t*>(base + s.xq), static_cast<const uint8_t*>(blob),
                          reinterpret_cast<const float*>(base + s.ascale), static_cast<const float*>(s1), base + s.y,
                          out_dtype, M, N, K, 0, workspace, workspace_bytes, stream);
  if (rc) return rc;
  e = cudaMemcpyAsync(y_host, base + s.y, (size_t)M * N * dtype_bytes(out_dtype), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) {
    lq::record_cuda_error(e, "lq_w4a8_linear_host download");
    return LQ_ERR_CUDA;
  }
  return LQ_OK;
}

}  // extern "C"
