// Shared helpers for the blockrank_b200 kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/blockrank_b200.h"

namespace brk {

void set_error(const char* fmt, ...);

#define BRK_REQUIRE(cond, code, ...)  \
  do {                                \
    if (!(cond)) {                    \
      ::brk::set_error(__VA_ARGS__);  \
      return (code);                  \
    }                                 \
  } while (0)

#define BRK_CUDA(expr)                                                             \
  do {                                                                             \
    cudaError_t e_ = (expr);                                                       \
    if (e_ != cudaSuccess) {                                                       \
      ::brk::set_error("%s failed: %s", #expr, cudaGetErrorString(e_));            \
      return BRK_E_CUDA;                                                           \
    }                                                                              \
  } while (0)

// ---- element access helpers -------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// 4 consecutive elements -> float4 (pointer must be aligned to 4 elements)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&u.x);
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&u.y);
  float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y);
  __nv_bfloat162 b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// 8 consecutive elements <-> float[8] (pointer aligned to 8 elements)
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

struct View {
  char* ptr;
  int64_t sb, sh, ss;
};
inline View make_view(const brk_view& v) { return View{(char*)v.ptr, v.stride_b, v.stride_h, v.stride_s}; }

// Every attention call gets a 256-byte header at the start of its workspace: [0] the work counter of the
// tensor-core kernel, [1] the verdict of the span check (non-zero: malformed, the kernels write nothing).
constexpr size_t kWsHeader = 256;
// Values of the caller's status word: 10..49 name the bounded wait that gave up, 50 malformed block spans,
// 90 the self-test's wait.
constexpr int kStatusBadSpans = 50;
constexpr int kStatusSelfTest = 90;

// kernel launchers implemented in the .cu files
int attn_prologue_launch(const brk_attn_params& p, int* hdr, float2* ml, int64_t n_ml, cudaStream_t st);
int attn_simt_launch(const brk_attn_params& p, void* ws, size_t ws_bytes, cudaStream_t st);
int selftest_wait_launch(int32_t* status, uint32_t budget, cudaStream_t st);
int attn_tc_launch(const brk_attn_params& p, void* ws, size_t ws_bytes, cudaStream_t st);
size_t attn_tc_workspace(const brk_attn_params& p);
size_t attn_bwd_workspace(const brk_attn_bwd_params& p);
int attn_bwd_launch(const brk_attn_bwd_params& p, void* ws, size_t ws_bytes, cudaStream_t st);
int attn_bwd_mma_launch(const brk_attn_bwd_params& p, float* delta, float* dk32, float* dv32, float* dq32, cudaStream_t st);
int sm_count();

}  // namespace brk

namespace brk {
size_t doc_scores_workspace(const brk_score_params& p);
int doc_scores_launch(const brk_score_params& p, void* ws, size_t ws_bytes, cudaStream_t st);
int raw_scores_launch(const brk_score_params& p, void* out, cudaStream_t st);
int doc_scores_static_launch(const brk_score_params& p, cudaStream_t st);
int spans_launch(const uint8_t* mask, int B, int M, int H, int32_t* start, int32_t* len, cudaStream_t st);
int rmsnorm_launch(int dtype, const void* x, void* residual, const void* w, void* out, int64_t rows, int hidden,
                   float eps, cudaStream_t st);
int rope_launch(int dtype, void* q, int64_t q_rs, int N, void* k, int64_t k_rs, int Nk, int D, const int32_t* pos,
                const float* inv_freq, int64_t T, cudaStream_t st);
int silu_mul_launch(int dtype, const void* gu, void* out, int64_t rows, int inter, cudaStream_t st);
}  // namespace brk
