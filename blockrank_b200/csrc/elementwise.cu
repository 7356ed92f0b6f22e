// HBM-bound helpers of the early-exit runner: block spans from the collator
// mask, RMSNorm (optionally fused with the residual add), rotate-half RoPE and
// SiLU(gate) * up.  Rounding points follow what the HF Mistral modules do in
// the model dtype, so a bf16 run tracks the framework's bf16 run closely.
#include "brk_common.cuh"

namespace brk {
namespace {

// ---- spans ------------------------------------------------------------------
__global__ void spans_kernel(const uint8_t* __restrict__ mask, int total, int M, int H,
                             int32_t* __restrict__ start, int32_t* __restrict__ len) {
  // one warp per block: count valid slots; the block is left-padded so they are the last ones
  const int blk = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (blk >= total) return;
  const uint8_t* p = mask + (size_t)blk * H;
  int c = 0;
  for (int i = lane; i < H; i += 32) c += p[i] != 0;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
  if (lane == 0) {
    len[blk] = c;
    start[blk] = (blk % M) * H + (H - c);
  }
}

// ---- RMSNorm ------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const T* __restrict__ x, T* __restrict__ residual,
                                                      const T* __restrict__ w, T* __restrict__ out, int hidden,
                                                      float eps) {
  extern __shared__ __align__(16) float row[];  // [hidden] the (summed) row in fp32
  __shared__ float red[8];
  const int64_t r = blockIdx.x;
  const T* xp = x + r * hidden;
  T* rp = residual ? residual + r * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float4 v = load4(xp + i);
    if (rp) {
      const float4 h = load4(rp + i);
      // the framework adds in the model dtype: round the sum before it is normalised and stored
      v = make_float4(Elem<T>::round(v.x + h.x), Elem<T>::round(v.y + h.y), Elem<T>::round(v.z + h.z),
                      Elem<T>::round(v.w + h.w));
      store4(rp + i, v);
    }
    *reinterpret_cast<float4*>(row + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float rs = rsqrtf(tot / (float)hidden + eps);
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(row + i);
    const float4 g = load4(w + i);
    // normalised value is cast to the model dtype, then multiplied by the weight in that dtype
    store4(out + r * hidden + i,
           make_float4(g.x * Elem<T>::round(v.x * rs), g.y * Elem<T>::round(v.y * rs), g.z * Elem<T>::round(v.z * rs),
                       g.w * Elem<T>::round(v.w * rs)));
  }
}

// Register-resident variant for hidden = 16 * blockDim.x (4096 -> 256 threads): every thread keeps its 16
// elements of the row in registers between the sum of squares and the scaling, with 16-byte accesses
// and no shared-memory staging of the row.  Same arithmetic and rounding points as rmsnorm_kernel.
template <typename T>
__global__ void __launch_bounds__(1024) rmsnorm_reg_kernel(const T* __restrict__ x, T* __restrict__ residual,
                                                           const T* __restrict__ w, T* __restrict__ out, int hidden,
                                                           float eps) {
  __shared__ float red[32];
  const int64_t r = blockIdx.x;
  const int i = threadIdx.x * 16;
  const T* xp = x + r * hidden + i;
  float v[16];
  load8(xp, *reinterpret_cast<float (*)[8]>(&v[0]));
  load8(xp + 8, *reinterpret_cast<float (*)[8]>(&v[8]));
  if (residual) {
    T* rp = residual + r * hidden + i;
    float h[16];
    load8(rp, *reinterpret_cast<float (*)[8]>(&h[0]));
    load8(rp + 8, *reinterpret_cast<float (*)[8]>(&h[8]));
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = Elem<T>::round(v[j] + h[j]);
    store8(rp, *reinterpret_cast<float (*)[8]>(&v[0]));
    store8(rp + 8, *reinterpret_cast<float (*)[8]>(&v[8]));
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) ss += v[j] * v[j];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int j = 0; j < (int)(blockDim.x >> 5); ++j) tot += red[j];
  const float rs = rsqrtf(tot / (float)hidden + eps);
  float g[16];
  load8(w + i, *reinterpret_cast<float (*)[8]>(&g[0]));
  load8(w + i + 8, *reinterpret_cast<float (*)[8]>(&g[8]));
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = g[j] * Elem<T>::round(v[j] * rs);
  T* op = out + r * hidden + i;
  store8(op, *reinterpret_cast<float (*)[8]>(&v[0]));
  store8(op + 8, *reinterpret_cast<float (*)[8]>(&v[8]));
}

// ---- RoPE ---------------------------------------------------------------------
// One thread per (row, 8 rotation pairs): the 8 angles are evaluated once and applied to every
// query and key head of that row, with 16-byte loads and stores of both halves of each head.
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(T* __restrict__ q, int64_t q_rs, int N, T* __restrict__ k,
                                                   int64_t k_rs, int Nk, int D, const int32_t* __restrict__ pos,
                                                   const float* __restrict__ inv_freq, int64_t T_rows) {
  const int half = D >> 1, chunks = half >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T_rows * chunks) return;
  const int64_t t = idx / chunks;
  const int i0 = (int)(idx % chunks) * 8;
  const float p = (float)pos[t];
  float cs[8], sn[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sincosf(p * inv_freq[i0 + i], &sn[i], &cs[i]);
    cs[i] = Elem<T>::round(cs[i]);
    sn[i] = Elem<T>::round(sn[i]);
  }
  for (int h = 0; h < N + Nk; ++h) {
    T* base = (h < N ? q + t * q_rs + (int64_t)h * D : k + t * k_rs + (int64_t)(h - N) * D) + i0;
    float x1[8], x2[8], o1[8], o2[8];
    load8(base, x1);
    load8(base + half, x2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // x*cos + rotate_half(x)*sin with each product rounded in the model dtype
      o1[i] = Elem<T>::round(x1[i] * cs[i]) + Elem<T>::round(-x2[i] * sn[i]);
      o2[i] = Elem<T>::round(x2[i] * cs[i]) + Elem<T>::round(x1[i] * sn[i]);
    }
    store8(base, o1);
    store8(base + half, o2);
  }
}

// ---- SiLU(gate) * up ------------------------------------------------------------
// x / (1 + e^-x).  The bf16 path uses the hardware exponential and reciprocal (relative error about
// 2^-22, far below bf16 resolution): with expf and an IEEE division the kernel spent more time
// issuing instructions than moving its 6 bytes per element.
template <typename T>
__device__ __forceinline__ float silu(float g) {
  if constexpr (sizeof(T) == 2) return __fdividef(g, 1.f + __expf(-g));
  else return g / (1.f + expf(-g));
}

// kVec elements per thread (8 or 16): one or two 16-byte pieces of gate, up and out each.
template <typename T, int kVec>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows,
                                                       int inter) {
  const int64_t per_row = inter / kVec;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const int64_t r = idx / per_row;
  const int c = (int)(idx % per_row) * kVec;
  float g[kVec], u[kVec], o[kVec];
#pragma unroll
  for (int v = 0; v < kVec; v += 8) {
    load8(gu + r * 2 * inter + c + v, *reinterpret_cast<float (*)[8]>(&g[v]));
    load8(gu + r * 2 * inter + inter + c + v, *reinterpret_cast<float (*)[8]>(&u[v]));
  }
#pragma unroll
  for (int i = 0; i < kVec; ++i) o[i] = Elem<T>::round(silu<T>(g[i])) * u[i];
#pragma unroll
  for (int v = 0; v < kVec; v += 8) store8(out + r * inter + c + v, *reinterpret_cast<float (*)[8]>(&o[v]));
}

}  // namespace

int spans_launch(const uint8_t* mask, int B, int M, int H, int32_t* start, int32_t* len, cudaStream_t st) {
  const int total = B * M;
  const int warps = 8;
  spans_kernel<<<(total + warps - 1) / warps, warps * 32, 0, st>>>(mask, total, M, H, start, len);
  BRK_CUDA(cudaGetLastError());
  return BRK_OK;
}

int rmsnorm_launch(int dtype, const void* x, void* residual, const void* w, void* out, int64_t rows, int hidden,
                   float eps, cudaStream_t st) {
  if (hidden % 512 == 0 && hidden / 16 <= 1024) {  // whole warps of 16-element threads
    const int threads = hidden / 16;
    if (dtype == BRK_BF16)
      rmsnorm_reg_kernel<__nv_bfloat16><<<(unsigned)rows, threads, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)residual,
                                                                          (const __nv_bfloat16*)w, (__nv_bfloat16*)out, hidden, eps);
    else
      rmsnorm_reg_kernel<float><<<(unsigned)rows, threads, 0, st>>>((const float*)x, (float*)residual, (const float*)w,
                                                                  (float*)out, hidden, eps);
    BRK_CUDA(cudaGetLastError());
    return BRK_OK;
  }
  const size_t sm = (size_t)hidden * 4;
  if (dtype == BRK_BF16) {
    if (sm > 48 * 1024)
      BRK_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    rmsnorm_kernel<__nv_bfloat16><<<(unsigned)rows, 256, sm, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)residual,
                                                                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, hidden, eps);
  } else {
    if (sm > 48 * 1024)
      BRK_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    rmsnorm_kernel<float><<<(unsigned)rows, 256, sm, st>>>((const float*)x, (float*)residual, (const float*)w,
                                                          (float*)out, hidden, eps);
  }
  BRK_CUDA(cudaGetLastError());
  return BRK_OK;
}

int rope_launch(int dtype, void* q, int64_t q_rs, int N, void* k, int64_t k_rs, int Nk, int D, const int32_t* pos,
                const float* inv_freq, int64_t T, cudaStream_t st) {
  const int64_t total = T * (D / 16);
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  if (dtype == BRK_BF16)
    rope_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, st>>>((__nv_bfloat16*)q, q_rs, N, (__nv_bfloat16*)k, k_rs,
                                                                    Nk, D, pos, inv_freq, T);
  else
    rope_kernel<float><<<(unsigned)blocks, threads, 0, st>>>((float*)q, q_rs, N, (float*)k, k_rs, Nk, D, pos, inv_freq, T);
  BRK_CUDA(cudaGetLastError());
  return BRK_OK;
}

int silu_mul_launch(int dtype, const void* gu, void* out, int64_t rows, int inter, cudaStream_t st) {
  const int vec = inter % 16 == 0 ? 16 : 8;
  const int64_t total = rows * (inter / vec);
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  if (dtype == BRK_BF16) {
    auto* g = (const __nv_bfloat16*)gu;
    auto* o = (__nv_bfloat16*)out;
    if (vec == 16) silu_mul_kernel<__nv_bfloat16, 16><<<blocks, threads, 0, st>>>(g, o, rows, inter);
    else silu_mul_kernel<__nv_bfloat16, 8><<<blocks, threads, 0, st>>>(g, o, rows, inter);
  } else {
    if (vec == 16) silu_mul_kernel<float, 16><<<blocks, threads, 0, st>>>((const float*)gu, (float*)out, rows, inter);
    else silu_mul_kernel<float, 8><<<blocks, threads, 0, st>>>((const float*)gu, (float*)out, rows, inter);
  }
  BRK_CUDA(cudaGetLastError());
  return BRK_OK;
}

}  // namespace brk
