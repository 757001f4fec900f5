// Shared device/host helpers for the liquidgemm_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/liquidgemm_b200.h"

namespace lq {

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
void record_cuda_error(cudaError_t e, const char* where);   // lq_api.cu
int check_launch(const char* where);                        // lq_api.cu: cudaGetLastError -> code
int sm_count();                                             // lq_api.cu: cached per device
int* status_word();                                         // lq_api.cu: device address of the status word

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Launch with programmatic stream serialisation: the kernel may start while the previous kernel
// of the stream is still draining, and must execute griddepcontrol.wait (dependency_wait()) before
// it touches anything an earlier kernel may have written or may still read-modify-write.  Switched
// off with LIQUIDGEMM_PDL=0 (then this is an ordinary launch).
bool pdl_enabled();                                         // lq_api.cu
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// ---------------------------------------------------------------------------------------------
// LQQ arithmetic
// ---------------------------------------------------------------------------------------------
// Four codes in the four byte lanes of `w` -> four int8: (code*step + a) XOR 0x80 per lane.
// code <= 15 and step <= 16 keep every product <= 240 and every sum <= 255, so no lane carries
// (reference liquidgemm/quant.py:16-22, csrc/liquid_gemm/dequant.cu:39-43).
__device__ __forceinline__ uint32_t lqq_dequant4(uint32_t codes, uint32_t step, uint32_t a_bcast) {
  return (codes * step + a_bcast) ^ 0x80808080u;
}

// The output formula of every fused epilogue: two fp32 multiplies, left to right
// (reference liquidgemm/quant.py:152, csrc/liquid_gemm/epilogue.cu:57).
__device__ __forceinline__ float lqq_scale(int acc, float a_scale, float w_scale) {
  return __fmul_rn(__fmul_rn(__int2float_rn(acc), a_scale), w_scale);
}

// Store one output element in the dtype selected by `out_dtype` (LQ_DT_*).
__device__ __forceinline__ void store_out(void* y, size_t idx, float v, int out_dtype) {
  if (out_dtype == LQ_DT_BF16) {
    reinterpret_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
  } else if (out_dtype == LQ_DT_F16) {
    reinterpret_cast<__half*>(y)[idx] = __float2half_rn(v);
  } else {
    reinterpret_cast<float*>(y)[idx] = v;
  }
}

// Bias element n of a vector stored in the output dtype, as float.
__device__ __forceinline__ float load_bias(const void* b, long n, int out_dtype) {
  if (out_dtype == LQ_DT_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[n]);
  if (out_dtype == LQ_DT_F16) return __half2float(reinterpret_cast<const __half*>(b)[n]);
  return reinterpret_cast<const float*>(b)[n];
}

// Store with an optional bias.  The product is first rounded to the output type and the bias is added to
// that rounded value in float32, then rounded again: exactly what PyTorch's `y + bias` computes on the
// operator's output (the reference adds its bias that way, liquidgemm/vllm_plugin.py:205-206).
__device__ __forceinline__ void store_out_bias(void* y, size_t idx, float v, float bias, bool has_bias, int out_dtype) {
  if (out_dtype == LQ_DT_BF16) {
    __nv_bfloat16 t = __float2bfloat16_rn(v);
    if (has_bias) t = __float2bfloat16_rn(__fadd_rn(__bfloat162float(t), bias));
    reinterpret_cast<__nv_bfloat16*>(y)[idx] = t;
  } else if (out_dtype == LQ_DT_F16) {
    __half t = __float2half_rn(v);
    if (has_bias) t = __float2half_rn(__fadd_rn(__half2float(t), bias));
    reinterpret_cast<__half*>(y)[idx] = t;
  } else {
    reinterpret_cast<float*>(y)[idx] = has_bias ? __fadd_rn(v, bias) : v;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Epilogue of the tensor-core kernels, sixteen accumulator columns (tokens) of one channel at a time.  These
// kernels are bound by instruction issue, and an epilogue that decides the output type, the bias and the
// ragged edge per element and forms every address with 64-bit arithmetic was measured to cost the CTA-pair
// kernel 16 % on layers with K = 4096: here the decisions are made once per sixteen elements and an address
// is one 32 x 32 + 64-bit multiply-add.  kEpiI32 selects raw int32 outputs.
constexpr int kEpiI32 = 3;

template <int DT, bool BIAS>
__device__ __forceinline__ uint16_t epi_bits16(int acc, float a_scale, float w_scale, float bias) {
  const float y = lqq_scale(acc, a_scale, w_scale);
  if (DT == LQ_DT_BF16) {
    __nv_bfloat16 t = __float2bfloat16_rn(y);
    if (BIAS) t = __float2bfloat16_rn(__fadd_rn(__bfloat162float(t), bias));
    return *reinterpret_cast<uint16_t*>(&t);
  }
  __half t = __float2half_rn(y);
  if (BIAS) t = __float2half_rn(__fadd_rn(__half2float(t), bias));
  return *reinterpret_cast<uint16_t*>(&t);
}

// Straight to global memory: element j goes to out + (idx0 + j * ld) elements.
template <int DT, bool BIAS, bool FULL>
__device__ __forceinline__ void epi_store_cols_t(void* out, size_t idx0, long ld, const int (&v)[16], const float (&sc)[16],
                                                 float w_scale, float bias, int valid) {
  constexpr int ES = (DT == LQ_DT_BF16 || DT == LQ_DT_F16) ? 2 : 4;
  char* p = static_cast<char*>(out) + idx0 * ES;
  const uint32_t pitch = (uint32_t)ld * ES;   // a row pitch below 4 GB
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (FULL || j < valid) {
      char* q = p + (uint64_t)pitch * (uint32_t)j;
      if (DT == kEpiI32) *reinterpret_cast<int32_t*>(q) = v[j];
      else if (DT == LQ_DT_F32) {
        const float y = lqq_scale(v[j], sc[j], w_scale);
        *reinterpret_cast<float*>(q) = BIAS ? __fadd_rn(y, bias) : y;
      } else {
        *reinterpret_cast<uint16_t*>(q) = epi_bits16<DT, BIAS>(v[j], sc[j], w_scale, bias);
      }
    }
  }
}
template <int DT>
__device__ __forceinline__ void epi_store_cols_dt(void* out, size_t idx0, long ld, const int (&v)[16], const float (&sc)[16],
                                                  float w_scale, float bias, bool has_bias, int valid) {
  if (valid >= 16) {
    if (has_bias) epi_store_cols_t<DT, true, true>(out, idx0, ld, v, sc, w_scale, bias, valid);
    else epi_store_cols_t<DT, false, true>(out, idx0, ld, v, sc, w_scale, bias, valid);
  } else {
    if (has_bias) epi_store_cols_t<DT, true, false>(out, idx0, ld, v, sc, w_scale, bias, valid);
    else epi_store_cols_t<DT, false, false>(out, idx0, ld, v, sc, w_scale, bias, valid);
  }
}
// out_mode: LQ_DT_* or kEpiI32; `valid` of the sixteen elements exist (the ragged last token chunk).
__device__ __forceinline__ void epi_store_cols(void* out, int out_mode, size_t idx0, long ld, const int (&v)[16],
                                               const float (&sc)[16], float w_scale, float bias, bool has_bias, int valid) {
  if (out_mode == LQ_DT_BF16) epi_store_cols_dt<LQ_DT_BF16>(out, idx0, ld, v, sc, w_scale, bias, has_bias, valid);
  else if (out_mode == LQ_DT_F16) epi_store_cols_dt<LQ_DT_F16>(out, idx0, ld, v, sc, w_scale, bias, has_bias, valid);
  else if (out_mode == LQ_DT_F32) epi_store_cols_dt<LQ_DT_F32>(out, idx0, ld, v, sc, w_scale, bias, has_bias, valid);
  else epi_store_cols_dt<kEpiI32>(out, idx0, ld, v, sc, w_scale, bias, false, valid);
}

// Into a shared-memory stage of 2-byte outputs: element j goes to col[j * 128] (the thread's channel column of a
// [16 tokens][128 channels] block).  out_mode: LQ_DT_BF16 or LQ_DT_F16.
template <int DT, bool BIAS>
__device__ __forceinline__ void epi_stage_cols_t(uint16_t* col, const int (&v)[16], const float (&sc)[16], float w_scale,
                                                 float bias) {
#pragma unroll
  for (int j = 0; j < 16; ++j) col[j * 128] = epi_bits16<DT, BIAS>(v[j], sc[j], w_scale, bias);
}
__device__ __forceinline__ void epi_stage_cols(uint16_t* col, int out_mode, const int (&v)[16], const float (&sc)[16],
                                               float w_scale, float bias, bool has_bias) {
  if (out_mode == LQ_DT_BF16) {
    if (has_bias) epi_stage_cols_t<LQ_DT_BF16, true>(col, v, sc, w_scale, bias);
    else epi_stage_cols_t<LQ_DT_BF16, false>(col, v, sc, w_scale, bias);
  } else {
    if (has_bias) epi_stage_cols_t<LQ_DT_F16, true>(col, v, sc, w_scale, bias);
    else epi_stage_cols_t<LQ_DT_F16, false>(col, v, sc, w_scale, bias);
  }
}

// Where a kernel's outputs go: the same [M, N] block is written into up to 8 row-major matrices with
// row stride `ld` elements at column offset `col0`.  One destination with ld = N, col0 = 0 is the
// ordinary output; several destinations (this GPU's and its peers' full-width output, mapped into this
// process) make the epilogue do the all-gather of an N-sharded layer with plain stores.
struct OutSpec {
  void* ptr[8];
  int n;
  long ld, col0;
};
inline OutSpec single_out(void* out, long N) {
  OutSpec o = {};
  o.ptr[0] = out;
  o.n = 1;
  o.ld = N;
  o.col0 = 0;
  return o;
}
// Cross-GPU ordering for the gather-by-stores epilogue.  Every CTA, after its last output store, adds 1
// to word `index` of each destination rank's flag array (release, system scope); a consumer kernel
// on rank r waits until its own word reached the number of CTAs of all ranks before it reads the
// gathered data.  The flags live in memory every rank can write (symmetric memory); the host zeroes
// them, and orders the ranks once, before the first kernel of a sequence.
struct PeerSync {
  unsigned* signal[8];     // per destination rank: its flag array (null array entries = no signalling)
  int n_signal;
  int signal_index;
  const unsigned* wait;    // this rank's flag word to wait on before reading the tokens, or null
  unsigned wait_value;
};
__device__ __forceinline__ void peer_signal(const PeerSync& p) {
#pragma unroll
  for (int r = 0; r < 8; ++r)   // constant indices: see store_out_all
    if (r < p.n_signal)
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.signal[r] + p.signal_index) : "memory");
}
// Bounded: gives up after `limit_ns` and returns false (the caller records a status code and goes on).
// Polls with relaxed loads and orders the following reads with one acquire fence at the end.
__device__ __forceinline__ bool peer_wait(const PeerSync& p, unsigned long long limit_ns) {
  if (!p.wait) return true;
  unsigned long long t0 = 0;
  bool ok = true;
  for (unsigned spins = 0;; ++spins) {
    unsigned v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait) : "memory");
    if (v >= p.wait_value) break;
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (spins == 0) t0 = now;
    else if (now - t0 > limit_ns) {
      ok = false;
      break;
    }
    __nanosleep(200);
  }
  asm volatile("fence.acquire.sys;" ::: "memory");
  return ok;
}

// Kernel parameters of the gather-by-stores variants.  They travel as a separate kernel parameter that
// only the multi-destination instantiations have: measured on B200, the programmatically serialised
// decode launches cost 0.5-1 us more once their parameters exceed 256 bytes, so the ordinary
// single-output kernels keep theirs below that.
struct MultiOut {
  OutSpec out;
  PeerSync sync;
};
struct NoMultiOut {};

__device__ __forceinline__ void store_out_all(const OutSpec& o, long m, long n, float v, int out_dtype) {
  const size_t idx = (size_t)(m * o.ld + o.col0 + n);
  // Constant indices only: a run-time index into a kernel parameter makes the compiler copy the whole
  // parameter block to local memory and read every field from there (measured: +1 us per launch).
  store_out(o.ptr[0], idx, v, out_dtype);
  if (o.n > 1) {
#pragma unroll
    for (int r = 1; r < 8; ++r)
      if (r < o.n) store_out(o.ptr[r], idx, v, out_dtype);
  }
}

__device__ __forceinline__ void store_out_all(const OutSpec& o, long m, long n, float v, float bias, bool has_bias,
                                              int out_dtype) {
  const size_t idx = (size_t)(m * o.ld + o.col0 + n);
  store_out_bias(o.ptr[0], idx, v, bias, has_bias, out_dtype);   // constant indices only, as above
  if (o.n > 1) {
#pragma unroll
    for (int r = 1; r < 8; ++r)
      if (r < o.n) store_out_bias(o.ptr[r], idx, v, bias, has_bias, out_dtype);
  }
}

// ---------------------------------------------------------------------------------------------
// memory
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Programmatic dependent launch, device side.  allow_dependents(): the next kernel of the stream may be
// scheduled once every CTA of this grid has executed it.  dependency_wait(): returns when all earlier
// kernels of the stream have completed and their writes are visible (no-op for an ordinary launch).
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

}  // namespace lq
