// Score extraction for BlockRank ranking: HBM-bound skinny products of a few
// signal rows of Q against every document key.
//
//   doc_partial_kernel   one CTA per (document, prompt, KV head): each thread
//                        owns whole key rows (read once per KV head, shared by
//                        the G query heads of the group) and keeps an online
//                        (max, sum-exp) per signal row; the CTA writes one
//                        (max, sum) pair per (head, row, document).  fp32 inputs.
//   doc_partial_mma_kernel  the same for bf16, a CTA walking through several documents
//                        of one (prompt, KV head): the (G*R signal rows) x (keys)
//                        products go through warp-level mma (m16n8k16), key
//                        rows straight from global memory into the B fragments,
//                        requested one group ahead across document boundaries.
//                        The product is 8-16 rows tall and bound by the K read;
//                        a tcgen05 tile (M >= 64, operands staged in shared
//                        memory, result through tensor memory) would add
//                        latency to a kernel that has no tensor-rate problem.
//   finalize (same launch) the CTA that finishes a prompt last (a counter per prompt in the
//                        scratch, bumped after each CTA's partials are globally visible)
//                        merges the per-document pairs into the softmax over all
//                        document tokens, emits the per-document probability mass and
//                        then the mean over heads and rows / temperature.
//   raw_scores_kernel    compatibility output: raw masked logits of the last R
//                        slots against every slot.
#include <algorithm>
#include <atomic>

#include "brk_common.cuh"

namespace brk {
namespace {

constexpr int kThreads = 160;  // five warps: a 160-token document is one pass
constexpr int kRowBatch = 8;  // signal rows accumulated per pass over a key
constexpr int kKeyStages = 4;   // asynchronous key-row copies a lane keeps in flight in the bf16 kernel
constexpr int kDocsPerCta = 64;  // documents one CTA of the bf16 kernel walks through, at most

struct ScoreArgs {
  View q, k;
  const int32_t* rows;
  const int32_t* blk_start;
  const int32_t* blk_len;
  float2* partial;  // [B, N, R, nd]
  unsigned* done_bg;  // [B, Nk] document CTAs of the (prompt, KV head) that have published their partials
  unsigned* done_b;   // [B] KV-head groups of the prompt whose masses are written; both wrap to 0 by themselves
  float* mass;      // [B, N, R, nd] out
  float* logits;    // [B, nd] out, optional
  float inv_count_temp;  // 1 / (N * R * temperature)
  int B, N, Nk, S, M, R;
  float scale;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void merge_ml(float& m, float& l, float m2, float l2) {
  const float mn = fmaxf(m, m2);
  const float ref = (mn == -INFINITY) ? 0.f : mn;
  l = l * exp2f(m - ref) + l2 * exp2f(m2 - ref);
  m = mn;
}

// two more logits (already in log2 units; -inf = masked) into a running (max, sum)
__device__ __forceinline__ void merge_pair(float& m, float& l, float x0, float x1) {
  const float mn = fmaxf(m, fmaxf(x0, x1));
  const float ref = (mn == -INFINITY) ? 0.f : mn;
  l = l * exp2f(m - ref) + (exp2f(x0 - ref) + exp2f(x1 - ref));
  m = mn;
}

// Called by every thread of a partial-kernel CTA after its (max, sum) pairs are written.  Two levels of
// "last one finishes the job", each a counter that atomicInc wraps back to 0 (so the scratch is ready for the
// next call): the last of the CTAs of a (prompt, KV head) to finish merges the per-document pairs of that
// group's G*R (head, signal row) rows into the softmax over all document tokens and writes their per-document
// probability masses; the last of the Nk groups of a prompt then writes the prompt's logits -- the mean over
// heads and rows of the masses, divided by the temperature, summed in a fixed order.
__device__ __forceinline__ void finalize_if_last(const ScoreArgs& a, int b, int g) {
  __shared__ int is_last;
  const int nd = a.M - 2;
  __syncthreads();  // every partial of this CTA has been issued
  if (threadIdx.x == 0) {
    __threadfence();  // ... and is visible device-wide before the counter moves
    is_last = atomicInc(a.done_bg + b * a.Nk + g, gridDim.x - 1) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int G = a.N / a.Nk, GR = G * a.R;
  constexpr int kHeld = 8;  // pairs per lane kept in registers: one round trip per row up to 256 documents
  __shared__ float gsum_w[kThreads / 32][32 * kHeld];
  float gacc[kHeld];  // this warp's rows summed per document: the group's contribution to the logits
#pragma unroll
  for (int i = 0; i < kHeld; ++i) gacc[i] = 0.f;
  const size_t w0 = ((size_t)b * a.N + (size_t)g * G) * a.R;  // the group's first (head, signal row) pair
  for (int row = warp; row < GR; row += nwarps) {
    const size_t w = w0 + row;  // (head g*G + row / R, signal row row % R)
    const float2* p = a.partial + w * nd;
    float2 held[kHeld];
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int d = lane + 32 * i;
      held[i] = d < nd ? __ldcg(&p[d]) : make_float2(-INFINITY, 0.f);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kHeld; ++i) mx = fmaxf(mx, held[i].x);
    for (int d = lane + 32 * kHeld; d < nd; d += 32) mx = fmaxf(mx, __ldcg(&p[d]).x);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float ref = (mx == -INFINITY) ? 0.f : mx;
    float z = 0.f;
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      held[i].y *= exp2f(held[i].x - ref);  // un-normalised mass of the document
      z += held[i].y;
    }
    for (int d = lane + 32 * kHeld; d < nd; d += 32) {
      const float2 x = __ldcg(&p[d]);
      z += x.y * exp2f(x.x - ref);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) z += __shfl_xor_sync(0xffffffffu, z, off);
    const float inv = z > 0.f ? 1.f / z : 0.f;
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int d = lane + 32 * i;
      if (d < nd) a.mass[w * nd + d] = held[i].y * inv;
      gacc[i] += held[i].y * inv;
    }
    for (int d = lane + 32 * kHeld; d < nd; d += 32) {
      const float2 x = __ldcg(&p[d]);
      a.mass[w * nd + d] = x.y * exp2f(x.x - ref) * inv;
    }
  }
  if (a.logits == nullptr) return;
  // The group's sum over its (head, row) pairs of every document's mass goes where the group's first row of
  // pairs was (all of them have been read by now): the prompt's last group then adds Nk numbers per document
  // instead of N*R.  The first 32*kHeld documents come from the registers of the loop above, the rest (long
  // lists) from the masses this CTA has just written.
  if (warp < kThreads / 32) {
#pragma unroll
    for (int i = 0; i < kHeld; ++i) gsum_w[warp][lane + 32 * i] = gacc[i];
  }
  __syncthreads();  // every row's pairs have been read, every warp's sums are in shared memory
  float* const gsum = reinterpret_cast<float*>(a.partial + ((size_t)b * a.N + (size_t)g * G) * a.R * nd);
  for (int d = threadIdx.x; d < min(nd, 32 * kHeld); d += blockDim.x) {
    float acc = 0.f;
    for (int wv = 0; wv < min(nwarps, kThreads / 32); ++wv) acc += gsum_w[wv][d];
    gsum[d] = acc;
  }
  for (int d = 32 * kHeld + threadIdx.x; d < nd; d += blockDim.x) {
    float acc = 0.f;
    for (int row = 0; row < GR; ++row) acc += __ldcg(&a.mass[(w0 + row) * nd + d]);
    gsum[d] = acc;
  }
  __syncthreads();  // this group's masses and sums have been issued
  if (threadIdx.x == 0) {
    __threadfence();
    is_last = atomicInc(a.done_b + b, (unsigned)a.Nk - 1) == (unsigned)a.Nk - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int d = threadIdx.x; d < nd; d += blockDim.x) {
    float acc = 0.f;
    for (int gg = 0; gg < a.Nk; ++gg)
      acc += __ldcg(reinterpret_cast<const float*>(a.partial + ((size_t)b * a.N + (size_t)gg * G) * a.R * nd) + d);
    a.logits[(size_t)b * nd + d] = acc * a.inv_count_temp;
  }
}

// dot products of one key row against kRowBatch staged query rows
template <typename T, int D>
__device__ __forceinline__ void key_dots(const T* __restrict__ kp, const float* __restrict__ qs, int nrows,
                                         float (&acc)[kRowBatch]) {
#pragma unroll
  for (int i = 0; i < kRowBatch; ++i) acc[i] = 0.f;
#pragma unroll 4
  for (int d = 0; d < D; d += 4) {
    const float4 kv = load4(kp + d);
#pragma unroll
    for (int i = 0; i < kRowBatch; ++i) {
      if (i < nrows) {
        const float4 qv = *reinterpret_cast<const float4*>(qs + i * D + d);
        acc[i] = fmaf(qv.x, kv.x, acc[i]);
        acc[i] = fmaf(qv.y, kv.y, acc[i]);
        acc[i] = fmaf(qv.z, kv.z, acc[i]);
        acc[i] = fmaf(qv.w, kv.w, acc[i]);
      }
    }
  }
}

// One CTA per (document, prompt, KV head).  Each warp stages 32 key rows at a time in shared memory
// with fully coalesced 16-byte loads (all in flight together), then every lane owns one key: its
// dot products against the G*R staged query rows read the key from shared memory (row stride padded
// by 16 bytes, conflict-free for 16-byte accesses) and the query rows as broadcasts.
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) doc_partial_kernel(ScoreArgs a) {
  constexpr int kRowBytes = D * (int)sizeof(T);
  constexpr int kPitch = kRowBytes + 16;
  constexpr int kChunks = kRowBytes / 16;  // 16-byte pieces per key row
  extern __shared__ __align__(16) float smem[];
  const int G = a.N / a.Nk;
  const int GR = G * a.R;
  float* qs = smem;                                    // [GR][D], scaled by scale*log2(e)
  float2* red = reinterpret_cast<float2*>(qs + GR * D);  // [kThreads/32][kRowBatch]
  unsigned char* ktile = reinterpret_cast<unsigned char*>(red + (kThreads / 32) * kRowBatch);  // [warps][32][kPitch]

  const int nd = a.M - 2;
  const int d = blockIdx.x;
  const int b = blockIdx.y / a.Nk, g = blockIdx.y % a.Nk;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int start = a.blk_start[(size_t)b * a.M + 1 + d];
  const int len = a.blk_len[(size_t)b * a.M + 1 + d];

  const float sl2 = a.scale * 1.4426950408889634f;
  for (int i = tid; i < GR * (D / 4); i += kThreads) {
    const int row = i / (D / 4), d4 = i % (D / 4);
    const int hl = row / a.R, r = row % a.R;
    const int slot = a.rows[b * a.R + r];
    const T* qp = reinterpret_cast<const T*>(a.q.ptr) + (int64_t)b * a.q.sb + (int64_t)(g * G + hl) * a.q.sh +
                  (int64_t)slot * a.q.ss;
    float4 x = load4(qp + d4 * 4);
    *reinterpret_cast<float4*>(qs + row * D + d4 * 4) = make_float4(x.x * sl2, x.y * sl2, x.z * sl2, x.w * sl2);
  }
  __syncthreads();

  const unsigned char* kb = reinterpret_cast<const unsigned char*>(
      reinterpret_cast<const T*>(a.k.ptr) + (int64_t)b * a.k.sb + (int64_t)g * a.k.sh);
  const int64_t row_stride = a.k.ss * (int64_t)sizeof(T);
  unsigned char* my_tile = ktile + (size_t)warp * 32 * kPitch;
  for (int r0 = 0; r0 < GR; r0 += kRowBatch) {
    const int nrows = min(kRowBatch, GR - r0);
    float m[kRowBatch], l[kRowBatch];
#pragma unroll
    for (int i = 0; i < kRowBatch; ++i) { m[i] = -INFINITY; l[i] = 0.f; }
    for (int base = warp * 32; base < len; base += kThreads) {
      const int nkeys = min(32, len - base);
      __syncwarp();
#pragma unroll
      for (int i = 0; i < kChunks; ++i) {
        const int idx = lane + 32 * i, row = idx / kChunks, ch = idx % kChunks;
        if (row < nkeys)
          *reinterpret_cast<uint4*>(my_tile + row * kPitch + ch * 16) =
              *reinterpret_cast<const uint4*>(kb + (int64_t)(start + base + row) * row_stride + ch * 16);
      }
      __syncwarp();
      if (lane < nkeys) {
        float acc[kRowBatch];
        key_dots<T, D>(reinterpret_cast<const T*>(my_tile + lane * kPitch), qs + r0 * D, nrows, acc);
#pragma unroll
        for (int i = 0; i < kRowBatch; ++i)
          if (i < nrows) merge_ml(m[i], l[i], acc[i], 1.f);
      }
    }
    // warp then CTA reduction, fixed order
#pragma unroll
    for (int i = 0; i < kRowBatch; ++i) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m[i], off);
        const float l2 = __shfl_xor_sync(0xffffffffu, l[i], off);
        merge_ml(m[i], l[i], m2, l2);
      }
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < kRowBatch; ++i) red[warp * kRowBatch + i] = make_float2(m[i], l[i]);
    }
    __syncthreads();
    if (tid < nrows) {
      float mm = -INFINITY, ll = 0.f;
      for (int w = 0; w < kThreads / 32; ++w) {
        const float2 x = red[w * kRowBatch + tid];
        merge_ml(mm, ll, x.x, x.y);
      }
      const int row = r0 + tid;
      const int n = g * G + row / a.R, r = row % a.R;
      a.partial[(((size_t)b * a.N + n) * a.R + r) * nd + d] = make_float2(mm, ll);
    }
  }
  finalize_if_last(a, b, g);
}

__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// bf16 version of doc_partial_kernel on warp-level MMA.  One CTA per (document, prompt, KV head);
// a warp takes 8 keys at a time: C[16 signal rows x 8 keys] += Q[16 x 16] K^T[16 x 8] over D/16
// steps.  Lane (q = lane/4, j = lane%4) reads 16 bytes (8 elements of d) of key q per 32 elements
// of d, which is exactly its B fragment for two consecutive k-steps when the contraction index is
// taken in the order (8j+0,1 | 8j+2,3) then (8j+4,5 | 8j+6,7); the A fragments (signal rows q and
// q+8) are read from Q with the same 16-byte pattern, so both operands come straight from global
// memory with fully used sectors and no shared-memory staging.
template <int D>
__global__ void __launch_bounds__(kThreads, 4) doc_partial_mma_kernel(ScoreArgs a) {
  constexpr int kSteps = D / 32;
  constexpr int kStride = (kThreads / 32) * 8;
  __shared__ float2 red[2][kThreads / 32][16];
  __shared__ int s_start[kDocsPerCta], s_len[kDocsPerCta];
  __shared__ uint4 ring[kKeyStages][kSteps][kThreads];  // every lane copies into and reads back its own 16-byte cells
  const int G = a.N / a.Nk;
  const int GR = G * a.R;
  const int nd = a.M - 2;
  const int b = blockIdx.y / a.Nk, g = blockIdx.y % a.Nk;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qr = lane >> 2, j = lane & 3;
  const float sl2 = a.scale * 1.4426950408889634f;
  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(a.k.ptr) + (int64_t)b * a.k.sb + (int64_t)g * a.k.sh;

  // This CTA's documents: blockIdx.x, blockIdx.x + gridDim.x, ... (the launch keeps them within kDocsPerCta).
  const int n_mine = (nd - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  for (int i = tid; i < n_mine; i += kThreads) {
    const int d = blockIdx.x + i * gridDim.x;
    s_start[i] = a.blk_start[(size_t)b * a.M + 1 + d];
    s_len[i] = a.blk_len[(size_t)b * a.M + 1 + d];
  }
  __syncthreads();

  unsigned red_par = 0;
  for (int r0 = 0; r0 < GR; r0 += 16) {
    // A warp visits the 8-key groups (document i, keys base..base+7), base = 8*warp, 8*warp + 40, ..., of
    // every document of the CTA in order.  The key rows travel through a ring of kKeyStages asynchronous
    // copies per lane (16 bytes each, global -> shared, read back by the lane that requested them), issued
    // kKeyStages - 1 groups ahead of the products and across document boundaries: the kernel is bound by the
    // latency of these loads, and this is what keeps enough of them in flight.
    const bool has_hi = r0 + 8 < GR;  // with 8 or fewer (head, signal row) pairs left, rows 8..15 of the product are padding
    int ci = -1, cbase = 0, clen = 0;  // the group requested next: keys cbase.. of the CTA's document ci (clen keys)
    const __nv_bfloat16* cptr = kbase;  // first key row of that document, this lane's 16-byte column
    auto request = [&](int stage) {
      while (ci < n_mine && cbase >= clen) {  // next document that still has a group for this warp
        ++ci;
        cbase = warp * 8;
        clen = ci < n_mine ? s_len[ci] : 0;
        if (ci < n_mine) cptr = kbase + (int64_t)s_start[ci] * a.k.ss + 8 * j;
      }
      if (ci < n_mine) {
        const int key = min(cbase + qr, clen - 1);  // rows past the end re-read the last key; their columns are dropped below
        const __nv_bfloat16* kp = cptr + (int64_t)key * a.k.ss;
#pragma unroll
        for (int st = 0; st < kSteps; ++st) cp_async16(&ring[stage][st][tid], kp + 32 * st);
        cbase += kStride;
      }
      cp_async_commit();  // (an empty group when the documents are exhausted: the count below stays uniform)
    };
#pragma unroll
    for (int s = 0; s < kKeyStages - 1; ++s) request(s);
    // (the signal rows of Q are read behind the first key requests: both latencies overlap)
    uint4 qa[kSteps], qb[kSteps];  // signal rows r0+qr and r0+qr+8
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = r0 + qr + 8 * h;
      const bool ok = row < GR;
      const int hl = ok ? row / a.R : 0, r = ok ? row % a.R : 0;
      const int slot = a.rows[b * a.R + r];
      const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(a.q.ptr) + (int64_t)b * a.q.sb +
                                (int64_t)(g * G + hl) * a.q.sh + (int64_t)slot * a.q.ss + 8 * j;
#pragma unroll
      for (int st = 0; st < kSteps; ++st) {
        const uint4 v = ok ? *reinterpret_cast<const uint4*>(qp + 32 * st) : make_uint4(0, 0, 0, 0);
        if (h == 0) qa[st] = v; else qb[st] = v;
      }
    }
    int stage_r = 0, stage_w = kKeyStages - 1;
    for (int i = 0; i < n_mine; ++i) {
      const int len = s_len[i];
      float m_lo = -INFINITY, l_lo = 0.f, m_hi = -INFINITY, l_hi = 0.f;
      for (int base = warp * 8; base < len; base += kStride) {
        request(stage_w);
        stage_w = stage_w + 1 == kKeyStages ? 0 : stage_w + 1;
        cp_async_wait<kKeyStages - 1>();  // the oldest group -- this one -- has landed
        uint4 kf[kSteps];
#pragma unroll
        for (int st = 0; st < kSteps; ++st) kf[st] = ring[stage_r][st][tid];
        stage_r = stage_r + 1 == kKeyStages ? 0 : stage_r + 1;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int st = 0; st < kSteps; ++st) {
          mma_bf16_16x8x16(c, qa[st].x, qb[st].x, qa[st].y, qb[st].y, kf[st].x, kf[st].y);
          mma_bf16_16x8x16(c, qa[st].z, qb[st].z, qa[st].w, qb[st].w, kf[st].z, kf[st].w);
        }
        // c[0], c[1]: row qr, keys base + 2j, 2j + 1; c[2], c[3]: row qr + 8, same keys
        const bool ok0 = base + 2 * j < len, ok1 = base + 2 * j + 1 < len;
        merge_pair(m_lo, l_lo, ok0 ? c[0] * sl2 : -INFINITY, ok1 ? c[1] * sl2 : -INFINITY);
        if (has_hi) merge_pair(m_hi, l_hi, ok0 ? c[2] * sl2 : -INFINITY, ok1 ? c[3] * sl2 : -INFINITY);
      }
      // the four lanes of a row, then the warps, in a fixed order
#pragma unroll
      for (int off = 1; off <= 2; off <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m_lo, off), l2 = __shfl_xor_sync(0xffffffffu, l_lo, off);
        merge_ml(m_lo, l_lo, m2, l2);
        if (has_hi) {
          const float m3 = __shfl_xor_sync(0xffffffffu, m_hi, off), l3 = __shfl_xor_sync(0xffffffffu, l_hi, off);
          merge_ml(m_hi, l_hi, m3, l3);
        }
      }
      // red[] alternates between documents: a buffer is rewritten two documents later, behind the barrier of
      // the document in between, which its readers reach only after reading it
      float2 (&rd)[kThreads / 32][16] = red[red_par];
      red_par ^= 1u;
      if (j == 0) {
        rd[warp][qr] = make_float2(m_lo, l_lo);
        rd[warp][qr + 8] = make_float2(m_hi, l_hi);
      }
      __syncthreads();
      if (tid < 16 && r0 + tid < GR) {
        float mm = -INFINITY, ll = 0.f;
        for (int w = 0; w < kThreads / 32; ++w) merge_ml(mm, ll, rd[w][tid].x, rd[w][tid].y);
        const int row = r0 + tid;
        const int n = g * G + row / a.R, r = row % a.R;
        const int d = blockIdx.x + i * gridDim.x;
        a.partial[(((size_t)b * a.N + n) * a.R + r) * nd + d] = make_float2(mm, ll);
      }
    }
  }
  finalize_if_last(a, b, g);
}

// block index of a slot, or -1 for padding (blk_start is non-decreasing)
__device__ __forceinline__ int block_of(const int32_t* bs, const int32_t* bl, int M, int s) {
  int lo = 0, hi = M;  // first index with bs > s
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (bs[mid] <= s) lo = mid + 1; else hi = mid;
  }
  const int m = lo - 1;
  return (m >= 0 && s < bs[m] + bl[m]) ? m : -1;
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) raw_scores_kernel(ScoreArgs a, T* __restrict__ out, float neg) {
  extern __shared__ __align__(16) float smem[];
  const int G = a.N / a.Nk;
  const int GR = G * a.R;
  float* qs = smem;                               // [GR][D], scaled and rounded like the reference's Q*scaling
  int* qblk = reinterpret_cast<int*>(qs + GR * D);  // [R] block index of each row (-1 = padding)
  const int b = blockIdx.y / a.Nk, g = blockIdx.y % a.Nk;
  const int tid = threadIdx.x;
  const int32_t* bs = a.blk_start + (size_t)b * a.M;
  const int32_t* bl = a.blk_len + (size_t)b * a.M;
  for (int i = tid; i < GR * D; i += kThreads) {
    const int row = i / D, dd = i % D;
    const int hl = row / a.R, r = row % a.R;
    const T* qp = reinterpret_cast<const T*>(a.q.ptr) + (int64_t)b * a.q.sb + (int64_t)(g * G + hl) * a.q.sh +
                  (int64_t)(a.S - a.R + r) * a.q.ss;
    qs[i] = Elem<T>::round(Elem<T>::load(qp + dd) * a.scale);
  }
  if (tid < a.R) qblk[tid] = block_of(bs, bl, a.M, a.S - a.R + tid);
  __syncthreads();
  const int s = blockIdx.x * kThreads + tid;
  if (s >= a.S) return;
  const int kblk = block_of(bs, bl, a.M, s);
  const T* kp = reinterpret_cast<const T*>(a.k.ptr) + (int64_t)b * a.k.sb + (int64_t)g * a.k.sh + (int64_t)s * a.k.ss;
  for (int r0 = 0; r0 < GR; r0 += kRowBatch) {
    const int nrows = min(kRowBatch, GR - r0);
    float acc[kRowBatch];
    key_dots<T, D>(kp, qs + r0 * D, nrows, acc);
#pragma unroll
    for (int i = 0; i < kRowBatch; ++i) {
      if (i < nrows) {
        const int row = r0 + i;
        const int n = g * G + row / a.R, r = row % a.R;
        const int qb = qblk[r], qslot = a.S - a.R + r;
        const bool ok = qb >= 0 && kblk >= 0 &&
                        ((kblk == qb && s <= qslot) || (qb == a.M - 1 && kblk < qb) ||
                         (qb > 0 && qb < a.M - 1 && kblk == 0));
        Elem<T>::store(out + (((size_t)b * a.N + n) * a.R + r) * a.S + s, ok ? acc[i] : neg);
      }
    }
  }
}

ScoreArgs make_args(const brk_score_params& p) {
  ScoreArgs a;
  a.q = make_view(p.q);
  a.k = make_view(p.k);
  a.rows = p.rows;
  a.blk_start = p.blk_start;
  a.blk_len = p.blk_len;
  a.partial = nullptr;
  a.done_bg = nullptr;
  a.done_b = nullptr;
  a.mass = nullptr;
  a.logits = nullptr;
  a.inv_count_temp = 0.f;
  a.B = p.B; a.N = p.N; a.Nk = p.Nk; a.S = p.S; a.M = p.M; a.R = p.R;
  a.scale = p.scale;
  return a;
}

int check(const brk_score_params& p) {
  BRK_REQUIRE(p.q.ptr && p.k.ptr && p.blk_start && p.blk_len, BRK_E_ARG, "null pointer in score params");
  BRK_REQUIRE(p.B > 0 && p.N > 0 && p.Nk > 0 && p.N % p.Nk == 0 && p.S > 0 && p.M >= 1, BRK_E_ARG,
              "bad score shape B=%d N=%d Nk=%d S=%d M=%d", p.B, p.N, p.Nk, p.S, p.M);
  BRK_REQUIRE(p.R >= 1 && p.R <= 64 && (p.N / p.Nk) * p.R <= 256, BRK_E_ARG, "R=%d out of range", p.R);
  BRK_REQUIRE(p.D == 64 || p.D == 128, BRK_E_UNSUPPORTED, "head_dim %d not supported (64 or 128)", p.D);
  BRK_REQUIRE(p.dtype == BRK_BF16 || p.dtype == BRK_F32, BRK_E_UNSUPPORTED, "dtype %d", p.dtype);
  const int al = p.dtype == BRK_BF16 ? 8 : 4;
  BRK_REQUIRE(p.q.stride_s % al == 0 && p.q.stride_h % al == 0 && p.q.stride_b % al == 0 && p.k.stride_s % al == 0 &&
                  p.k.stride_h % al == 0 && p.k.stride_b % al == 0 && ((uintptr_t)p.q.ptr % 16 == 0) &&
                  ((uintptr_t)p.k.ptr % 16 == 0),
              BRK_E_ARG, "q/k rows must be 16-byte aligned");
  BRK_REQUIRE(p.B * p.Nk <= 65535, BRK_E_UNSUPPORTED, "B*Nk too large");
  return BRK_OK;
}

}  // namespace

// scratch layout: completion counters ([B, Nk] then [B] unsigned, padded to `counter_bytes`), then the
// [B, N, R, nd] (max, sum) pairs
static size_t counter_bytes(const brk_score_params& p) {
  return (((size_t)(p.B > 0 ? p.B : 0) * (size_t)(p.Nk + 1) * sizeof(unsigned)) + 255) & ~(size_t)255;
}
static size_t partial_bytes(const brk_score_params& p) {
  const size_t nd = p.M > 2 ? p.M - 2 : 0;
  return (size_t)p.B * p.N * p.R * nd * sizeof(float2);
}

size_t doc_scores_workspace(const brk_score_params& p) { return counter_bytes(p) + partial_bytes(p); }

// counters_zero: the caller guarantees that the counters are zero (they return to zero after every completed call)
static int doc_scores_run(const brk_score_params& p, void* ws, size_t ws_bytes, size_t counter_region, bool counters_zero,
                          cudaStream_t st) {
  int rc = check(p);
  if (rc) return rc;
  BRK_REQUIRE(p.M >= 3, BRK_E_ARG, "document scores need at least one document block (M=%d)", p.M);
  BRK_REQUIRE(p.rows && p.doc_mass, BRK_E_ARG, "rows / doc_mass must be given");
  BRK_REQUIRE(ws != nullptr && ws_bytes >= counter_region + partial_bytes(p) && ((uintptr_t)ws & 7) == 0, BRK_E_WORKSPACE,
              "workspace %zu < %zu bytes (or not 8-byte aligned)", ws_bytes, counter_region + partial_bytes(p));
  BRK_REQUIRE(p.temperature > 0.f, BRK_E_ARG, "temperature must be positive");
  ScoreArgs a = make_args(p);
  a.done_bg = reinterpret_cast<unsigned*>(ws);
  a.done_b = a.done_bg + (size_t)p.B * p.Nk;
  a.partial = reinterpret_cast<float2*>(static_cast<unsigned char*>(ws) + counter_region);
  a.mass = p.doc_mass;
  a.logits = p.logits;
  a.inv_count_temp = 1.f / ((float)(p.N * p.R) * p.temperature);
  if (!counters_zero) BRK_CUDA(cudaMemsetAsync(ws, 0, (size_t)p.B * (p.Nk + 1) * sizeof(unsigned), st));
  const int nd = p.M - 2, G = p.N / p.Nk;
  dim3 grid(nd, p.B * p.Nk);
  const size_t pitch = (size_t)p.D * (p.dtype == BRK_BF16 ? 2 : 4) + 16;
  const size_t sm = (size_t)G * p.R * p.D * 4 + (kThreads / 32) * kRowBatch * sizeof(float2) + (kThreads / 32) * 32 * pitch;
  auto launch = [&](auto kern) -> int {
    // (the kernels also hold a few KB of static shared memory, which counts against the same 48 KB default)
    if (sm + 8192 > 48 * 1024) BRK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    kern<<<grid, kThreads, sm, st>>>(a);
    BRK_CUDA(cudaGetLastError());
    return BRK_OK;
  };
  if (p.dtype == BRK_BF16) {
    // A CTA walks through several documents so that its key loads overlap across document boundaries; the
    // grid is sized to be resident at once (four CTAs per SM) when there are enough documents for that.
    const int slots = 4 * std::max(1, sm_count());
    int per_bg = std::max(1, slots / (p.B * p.Nk));
    per_bg = std::min(nd, std::max(per_bg, (nd + kDocsPerCta - 1) / kDocsPerCta));
    dim3 grid_docs(per_bg, p.B * p.Nk);
    // (four CTAs with their key rings need 170 KB of shared memory per SM: ask for the large carve-out)
    if (p.D == 128) {
      BRK_CUDA(cudaFuncSetAttribute(doc_partial_mma_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    (int)cudaSharedmemCarveoutMaxShared));
      doc_partial_mma_kernel<128><<<grid_docs, kThreads, 0, st>>>(a);
    } else {
      BRK_CUDA(cudaFuncSetAttribute(doc_partial_mma_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                    (int)cudaSharedmemCarveoutMaxShared));
      doc_partial_mma_kernel<64><<<grid_docs, kThreads, 0, st>>>(a);
    }
    BRK_CUDA(cudaGetLastError());
    return BRK_OK;
  }
  return p.D == 128 ? launch(doc_partial_kernel<float, 128>) : launch(doc_partial_kernel<float, 64>);
}

int doc_scores_launch(const brk_score_params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  return doc_scores_run(p, ws, ws_bytes, counter_bytes(p), false, st);
}

// ---- allocation-free variant ----------------------------------------------------------------
// Scratch for brk_doc_scores_static: the (max, sum) pairs and the per-prompt counters live in this fixed
// array instead of a caller-provided workspace.  It is part of the library image, so every device that
// loads the library holds these bytes until the process exits.  The image initialises it to zero, and
// the counters wrap back to zero at the end of every completed call, so nothing is cleared per call.
static __device__ __align__(256) unsigned char g_static_scratch[BRK_STATIC_SCRATCH_BYTES];
constexpr size_t kStaticCounterBytes = 16384;  // room for 4096 counters: B * (Nk + 1) <= 4096

int doc_scores_static_launch(const brk_score_params& p, cudaStream_t st) {
  int rc = check(p);  // argument errors are reported as such, before the size test
  if (rc) return rc;
  BRK_REQUIRE(p.M >= 3, BRK_E_ARG, "document scores need at least one document block (M=%d)", p.M);
  // the counters keep a fixed place at the front of the array whatever the problem size, so that the zeros
  // they return to after one call are the zeros the next call starts from
  BRK_REQUIRE(counter_bytes(p) <= kStaticCounterBytes, BRK_E_WORKSPACE,
              "brk_doc_scores_static: B*(Nk+1) = %d completion counters, the built-in array reserves room for %zu",
              p.B * (p.Nk + 1), kStaticCounterBytes / sizeof(unsigned));
  const size_t need = kStaticCounterBytes + partial_bytes(p);
  BRK_REQUIRE(need <= (size_t)BRK_STATIC_SCRATCH_BYTES, BRK_E_WORKSPACE,
              "brk_doc_scores_static: 16384 + B*N*R*(M-2)*8 = %zu bytes of scratch needed, the built-in array holds %zu; "
              "use brk_doc_scores with a caller workspace for this size",
              need, (size_t)BRK_STATIC_SCRATCH_BYTES);
  // In host code the array's name is only a handle; the kernels need its device address, which
  // differs per device.  It is looked up once per device, with that device current; the cache is
  // atomic so that two host threads making their first calls at the same time both end up with
  // the (identical) address.
  static std::atomic<void*> dev_ptr[64];
  int dev = 0;
  BRK_CUDA(cudaGetDevice(&dev));
  BRK_REQUIRE(dev >= 0 && dev < 64, BRK_E_UNSUPPORTED, "device ordinal %d out of range", dev);
  void* ptr = dev_ptr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    BRK_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    BRK_REQUIRE(ptr != nullptr, BRK_E_CUDA, "cudaGetSymbolAddress returned a null scratch address");
    dev_ptr[dev].store(ptr, std::memory_order_release);
  }
  // every (prompt, head, row, document) pair is overwritten by the partial kernels before the finalizing CTA
  // reads it, and the counters are back at zero, so nothing left by an earlier call has to be cleared
  return doc_scores_run(p, ptr, (size_t)BRK_STATIC_SCRATCH_BYTES, kStaticCounterBytes, true, st);
}

int raw_scores_launch(const brk_score_params& p, void* out, cudaStream_t st) {
  int rc = check(p);
  if (rc) return rc;
  BRK_REQUIRE(out != nullptr, BRK_E_ARG, "out is null");
  BRK_REQUIRE(p.R <= p.S, BRK_E_ARG, "R=%d exceeds S=%d", p.R, p.S);
  ScoreArgs a = make_args(p);
  const int G = p.N / p.Nk;
  dim3 grid((p.S + kThreads - 1) / kThreads, p.B * p.Nk);
  const size_t sm = (size_t)G * p.R * p.D * 4 + p.R * sizeof(int);
  auto launch = [&](auto kern, auto* o, float neg) -> int {
    // (the kernels also hold a few KB of static shared memory, which counts against the same 48 KB default)
    if (sm + 8192 > 48 * 1024) BRK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    kern<<<grid, kThreads, sm, st>>>(a, o, neg);
    BRK_CUDA(cudaGetLastError());
    return BRK_OK;
  };
  // 0.7 * lowest finite value of the dtype, computed the way the reference does (python float -> dtype)
  if (p.dtype == BRK_BF16) {
    const float neg = 0.7f * -3.3895313892515355e38f;
    return p.D == 128 ? launch(raw_scores_kernel<__nv_bfloat16, 128>, (__nv_bfloat16*)out, neg)
                      : launch(raw_scores_kernel<__nv_bfloat16, 64>, (__nv_bfloat16*)out, neg);
  }
  const float neg = (float)(0.7 * -3.4028234663852886e38);
  return p.D == 128 ? launch(raw_scores_kernel<float, 128>, (float*)out, neg)
                    : launch(raw_scores_kernel<float, 64>, (float*)out, neg);
}

}  // namespace brk
