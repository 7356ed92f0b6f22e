// BlockRank attention backward on CUDA cores (fp32 accumulate), for training through the registered
// attention function: the fp32 path, and the entry point that sends bf16 to the tensor-core kernels of
// attn_bwd_mma.cu.  The reference gets these gradients from autograd over its eager / SDPA paths
// (src/blockrank/blockrank_std_attention.py:96-262, 472-650); the mathematics is that of the softmax
// attention backward restricted to each row's visible keys:
//
//   delta_i = dO_i . O_i            p_ij = exp(scale * q_i . k_j - lse_i)        dP_ij = dO_i . v_j
//   dS_ij = p_ij (dP_ij - delta_i)  dQ_i = scale * sum_j dS_ij k_j
//   dK_j = scale * sum_i dS_ij q_i  dV_j = sum_i p_ij dO_i     (i over the rows that see key j, all heads of the group)
//
// Visible keys of a row (the forward's pattern): block 0 is causal; a document block sees block 0 and
// itself causally; the last block sees every earlier block and itself causally.
//
// Two kernels.  attn_bwd_dq_kernel has the forward CUDA-core kernel's decomposition: a CTA owns
// (prompt, block, KV head, tile of query tokens) with all query heads of the group; a row is held by four
// threads (a quarter of head_dim each); K and V tiles are staged in shared memory; it also writes delta.
// attn_bwd_dkv_kernel turns this around: a CTA owns 64 keys of one block (a key row held by four threads)
// and walks through the rows that see them, Q and dO tiles staged in shared memory; block 0's keys are seen
// by every row of the prompt, so the row blocks are dealt to `nsplit` CTAs that add into fp32 accumulators
// with atomics; a last kernel converts the accumulators to the output type.
#include <algorithm>

#include "brk_common.cuh"

namespace brk {

namespace {

constexpr int kThreads = 256;
constexpr int kRows = kThreads / 4;  // rows (or keys) per CTA: four threads each
constexpr int kTile = 32;            // keys (dq kernel) or rows (dkv kernel) staged per step
// Thread `qd` (0..3) of a row owns the 4-element groups qd, qd + 4, qd + 8, ... of head_dim: for a given step the
// four threads of a row read 64 consecutive bytes of a staged row, and the eight rows of a warp read the same
// addresses (a broadcast), so shared-memory reads are conflict-free 16-byte loads.
__device__ __forceinline__ int own_dim(int qd, int i4) { return (qd + 4 * i4) * 4; }

struct BwdArgs {
  View q, k, v, o, d_o, dq, dk, dv;
  const float* lse;
  float* delta;   // [B, N, S]
  float* dk32;    // [B, Nk, S, D]
  float* dv32;
  const int32_t* blk_start;
  const int32_t* blk_len;
  int B, N, Nk, S, M, G, max_block_len, nsplit;
  float scale, scale_log2;
};

// span of block m, or len 0 when it does not lie inside [0, S) (such a block is skipped: nothing is read
// or written outside the tensors whatever the arrays hold)
__device__ __forceinline__ void span_of(const BwdArgs& a, int b, int m, int& start, int& len) {
  start = a.blk_start[(size_t)b * a.M + m];
  len = a.blk_len[(size_t)b * a.M + m];
  if (start < 0 || len < 0 || len > a.max_block_len || start > a.S - len) len = 0;
}

__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// rows [row0, row0 + kTile) of a (B, heads, S, D) tensor for head `h` -> shared memory as fp32, zero beyond `nvalid`
template <typename T, int D>
__device__ __forceinline__ void stage_rows(float (*dst)[D], const View& t, int b, int h, int row0, int nvalid) {
  const T* base = reinterpret_cast<const T*>(t.ptr) + (int64_t)b * t.sb + (int64_t)h * t.sh;
  for (int i = threadIdx.x; i < kTile * (D / 4); i += kThreads) {
    const int r = i / (D / 4), d4 = i % (D / 4);
    const float4 x = r < nvalid ? load4(base + (int64_t)(row0 + r) * t.ss + d4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(&dst[r][d4 * 4]) = x;
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) attn_bwd_dq_kernel(BwdArgs a) {
  constexpr int QD = D / 4;  // dims per thread
  __shared__ __align__(16) float Ks[kTile][D];
  __shared__ __align__(16) float Vs[kTile][D];
  const int tid = threadIdx.x, r = tid >> 2, qd = tid & 3;
  const int b = blockIdx.z / a.Nk, g = blockIdx.z % a.Nk;
  const int m = blockIdx.y, G = a.G, TQ = kRows / G;
  int start, len;
  span_of(a, b, m, start, len);

  T* dqb = reinterpret_cast<T*>(a.dq.ptr) + (int64_t)b * a.dq.sb;
  if (blockIdx.x == 0) {
    // slots in front of this block (and behind the last block) belong to no block: zero gradient
    int pstart, plen;
    if (m > 0) span_of(a, b, m - 1, pstart, plen);
    const int gap0 = (m == 0) ? 0 : max(0, min(a.S, pstart + plen));
    const int per_row = G * (D / 4);
    const int blk_lo = len > 0 ? start : gap0, blk_hi = len > 0 ? start + len : gap0;
    for (int pass = 0; pass < 2; ++pass) {
      const int lo = pass == 0 ? gap0 : blk_hi;
      const int hi = pass == 0 ? blk_lo : (m == a.M - 1 ? a.S : blk_hi);
      for (int i = tid; i < (hi - lo) * per_row; i += kThreads) {
        const int s = lo + i / per_row, rem = i % per_row;
        const int h = g * G + rem / (D / 4), d4 = rem % (D / 4);
        store4(dqb + (int64_t)s * a.dq.ss + (int64_t)h * a.dq.sh + d4 * 4, make_float4(0.f, 0.f, 0.f, 0.f));
      }
    }
  }
  const int t0 = blockIdx.x * TQ;
  if (t0 >= len) return;
  const int tok = t0 + r / G, head = g * G + r % G;
  const bool active = tok < len;
  const int slot = start + (active ? tok : 0);

  float q[QD], go[QD], acc[QD];
  float delta = 0.f;
  {
    const T* qp = reinterpret_cast<const T*>(a.q.ptr) + (int64_t)b * a.q.sb + (int64_t)head * a.q.sh + (int64_t)slot * a.q.ss;
    const T* gp = reinterpret_cast<const T*>(a.d_o.ptr) + (int64_t)b * a.d_o.sb + (int64_t)head * a.d_o.sh + (int64_t)slot * a.d_o.ss;
    const T* op = reinterpret_cast<const T*>(a.o.ptr) + (int64_t)b * a.o.sb + (int64_t)head * a.o.sh + (int64_t)slot * a.o.ss;
#pragma unroll
    for (int d = 0; d < QD; d += 4) {
      const int c = own_dim(qd, d >> 2);
      const float4 x = load4(qp + c), y = load4(gp + c), z = load4(op + c);
      q[d] = x.x; q[d + 1] = x.y; q[d + 2] = x.z; q[d + 3] = x.w;
      go[d] = y.x; go[d + 1] = y.y; go[d + 2] = y.z; go[d + 3] = y.w;
      delta += y.x * z.x + y.y * z.y + y.z * z.z + y.w * z.w;
      acc[d] = acc[d + 1] = acc[d + 2] = acc[d + 3] = 0.f;
    }
  }
  delta = quad_sum(delta);
  const size_t row_id = ((size_t)b * a.N + head) * a.S + slot;
  const float lse2 = a.lse[row_id] * 1.4426950408889634f;
  if (active && qd == 0) a.delta[row_id] = delta;

  // key segments: earlier blocks in full, then the own block causally
  const int last_tok = min(len, t0 + TQ) - 1;  // last query token of this CTA
  const int n_ctx = (m == 0) ? 0 : (m < a.M - 1 ? 1 : a.M - 1);
  for (int seg = 0; seg <= n_ctx; ++seg) {
    const bool own = seg == n_ctx;
    int ks, kl;
    if (own) { ks = start; kl = last_tok + 1; } else span_of(a, b, seg, ks, kl);
    for (int k0 = 0; k0 < kl; k0 += kTile) {
      const int nv = min(kTile, kl - k0);
      __syncthreads();
      stage_rows<T, D>(Ks, a.k, b, g, ks + k0, nv);
      stage_rows<T, D>(Vs, a.v, b, g, ks + k0, nv);
      __syncthreads();
      for (int jj = 0; jj < nv; ++jj) {
        float s = 0.f, dp = 0.f;
        float4 kq[QD / 4];
#pragma unroll
        for (int d = 0; d < QD; d += 4) {
          const int c = own_dim(qd, d >> 2);
          const float4 kx = *reinterpret_cast<const float4*>(&Ks[jj][c]), vx = *reinterpret_cast<const float4*>(&Vs[jj][c]);
          kq[d >> 2] = kx;
          s = fmaf(q[d], kx.x, fmaf(q[d + 1], kx.y, fmaf(q[d + 2], kx.z, fmaf(q[d + 3], kx.w, s))));
          dp = fmaf(go[d], vx.x, fmaf(go[d + 1], vx.y, fmaf(go[d + 2], vx.z, fmaf(go[d + 3], vx.w, dp))));
        }
        s = quad_sum(s);
        dp = quad_sum(dp);
        const bool vis = active && (!own || k0 + jj <= tok);
        const float p = vis ? exp2f(s * a.scale_log2 - lse2) : 0.f;
        const float ds = p * (dp - delta);
#pragma unroll
        for (int d = 0; d < QD; d += 4) {
          acc[d] = fmaf(ds, kq[d >> 2].x, acc[d]);
          acc[d + 1] = fmaf(ds, kq[d >> 2].y, acc[d + 1]);
          acc[d + 2] = fmaf(ds, kq[d >> 2].z, acc[d + 2]);
          acc[d + 3] = fmaf(ds, kq[d >> 2].w, acc[d + 3]);
        }
      }
    }
  }
  if (active) {
    T* dp_ = dqb + (int64_t)head * a.dq.sh + (int64_t)slot * a.dq.ss;
#pragma unroll
    for (int d = 0; d < QD; d += 4)
      store4(dp_ + own_dim(qd, d >> 2), make_float4(acc[d] * a.scale, acc[d + 1] * a.scale, acc[d + 2] * a.scale, acc[d + 3] * a.scale));
  }
}

// grid: x = 64-key tile of the block, y = key block, z = ((prompt * Nk + KV head) * nsplit + split)
template <typename T, int D>
__global__ void __launch_bounds__(kThreads) attn_bwd_dkv_kernel(BwdArgs a) {
  constexpr int QD = D / 4;
  __shared__ __align__(16) float Qs[kTile][D];
  __shared__ __align__(16) float Gs[kTile][D];
  __shared__ float lse_s[kTile], delta_s[kTile];
  const int tid = threadIdx.x, kr = tid >> 2, qd = tid & 3;
  const int split = blockIdx.z % a.nsplit, bg = blockIdx.z / a.nsplit;
  const int b = bg / a.Nk, g = bg % a.Nk;
  const int m = blockIdx.y, G = a.G;
  int start, len;
  span_of(a, b, m, start, len);
  const int j0 = blockIdx.x * kRows;
  if (j0 >= len) return;
  if (split >= ((m == 0) ? a.M : ((m < a.M - 1) ? 2 : 1))) return;  // no row block left for this split
  const int j = j0 + kr;  // key token within the block
  const bool kvalid = j < len;

  float kk[QD], vv[QD], dk[QD], dv[QD];
  {
    const int slot = start + (kvalid ? j : 0);
    const T* kp = reinterpret_cast<const T*>(a.k.ptr) + (int64_t)b * a.k.sb + (int64_t)g * a.k.sh + (int64_t)slot * a.k.ss;
    const T* vp = reinterpret_cast<const T*>(a.v.ptr) + (int64_t)b * a.v.sb + (int64_t)g * a.v.sh + (int64_t)slot * a.v.ss;
#pragma unroll
    for (int d = 0; d < QD; d += 4) {
      const int c = own_dim(qd, d >> 2);
      const float4 x = load4(kp + c), y = load4(vp + c);
      kk[d] = x.x; kk[d + 1] = x.y; kk[d + 2] = x.z; kk[d + 3] = x.w;
      vv[d] = y.x; vv[d + 1] = y.y; vv[d + 2] = y.z; vv[d + 3] = y.w;
      dk[d] = dk[d + 1] = dk[d + 2] = dk[d + 3] = 0.f;
      dv[d] = dv[d + 1] = dv[d + 2] = dv[d + 3] = 0.f;
    }
  }

  // Row blocks that see these keys: the own block (causally); every later block for block 0; the last block
  // for a document block.  Entry e of that list is handled by the CTA with split == e % nsplit.
  const int n_list = (m == 0) ? a.M : ((m < a.M - 1) ? 2 : 1);
  for (int e = split; e < n_list; e += a.nsplit) {
    const int mr = (e == 0) ? m : ((m == 0) ? e : a.M - 1);
    const bool own = e == 0;
    int rs, rl;
    span_of(a, b, mr, rs, rl);
    const int tfirst = own ? j0 : 0;  // rows before the tile's first key see none of its keys
    for (int hh = 0; hh < G; ++hh) {
      const int head = g * G + hh;
      for (int t0 = tfirst; t0 < rl; t0 += kTile) {
        const int nv = min(kTile, rl - t0);
        __syncthreads();
        stage_rows<T, D>(Qs, a.q, b, head, rs + t0, nv);
        stage_rows<T, D>(Gs, a.d_o, b, head, rs + t0, nv);
        if (tid < kTile) {
          const size_t rid = ((size_t)b * a.N + head) * a.S + rs + t0 + min(tid, nv - 1);
          lse_s[tid] = a.lse[rid] * 1.4426950408889634f;
          delta_s[tid] = a.delta[rid];
        }
        __syncthreads();
        for (int ii = 0; ii < nv; ++ii) {
          float s = 0.f, dp = 0.f;
          float4 qx[QD / 4], gx[QD / 4];
#pragma unroll
          for (int d = 0; d < QD; d += 4) {
            const int c = own_dim(qd, d >> 2);
            const float4 x = *reinterpret_cast<const float4*>(&Qs[ii][c]), y = *reinterpret_cast<const float4*>(&Gs[ii][c]);
            qx[d >> 2] = x;
            gx[d >> 2] = y;
            s = fmaf(x.x, kk[d], fmaf(x.y, kk[d + 1], fmaf(x.z, kk[d + 2], fmaf(x.w, kk[d + 3], s))));
            dp = fmaf(y.x, vv[d], fmaf(y.y, vv[d + 1], fmaf(y.z, vv[d + 2], fmaf(y.w, vv[d + 3], dp))));
          }
          s = quad_sum(s);
          dp = quad_sum(dp);
          const bool vis = kvalid && (!own || t0 + ii >= j);
          const float p = vis ? exp2f(s * a.scale_log2 - lse_s[ii]) : 0.f;
          const float ds = p * (dp - delta_s[ii]);
#pragma unroll
          for (int d = 0; d < QD; d += 4) {
            dk[d] = fmaf(ds, qx[d >> 2].x, dk[d]);
            dk[d + 1] = fmaf(ds, qx[d >> 2].y, dk[d + 1]);
            dk[d + 2] = fmaf(ds, qx[d >> 2].z, dk[d + 2]);
            dk[d + 3] = fmaf(ds, qx[d >> 2].w, dk[d + 3]);
            dv[d] = fmaf(p, gx[d >> 2].x, dv[d]);
            dv[d + 1] = fmaf(p, gx[d >> 2].y, dv[d + 1]);
            dv[d + 2] = fmaf(p, gx[d >> 2].z, dv[d + 2]);
            dv[d + 3] = fmaf(p, gx[d >> 2].w, dv[d + 3]);
          }
        }
      }
    }
  }
  if (kvalid) {
    const size_t off = (((size_t)b * a.Nk + g) * a.S + start + j) * D;
#pragma unroll
    for (int d = 0; d < QD; ++d) {
      const int c = own_dim(qd, d >> 2) + (d & 3);
      atomicAdd(a.dk32 + off + c, dk[d] * a.scale);
      atomicAdd(a.dv32 + off + c, dv[d]);
    }
  }
}

// fp32 accumulators [B, Nk, S, D] -> dk, dv in the output type (slots outside every block hold zeros)
template <typename T>
__global__ void __launch_bounds__(256) attn_bwd_store_kernel(BwdArgs a, int D) {
  const int64_t n4 = (int64_t)a.B * a.Nk * a.S * (D / 4);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const int d4 = (int)(i % (D / 4));
    const int64_t row = i / (D / 4);
    const int s = (int)(row % a.S);
    const int g = (int)((row / a.S) % a.Nk), b = (int)(row / ((int64_t)a.S * a.Nk));
    const float4 x = *reinterpret_cast<const float4*>(a.dk32 + row * D + d4 * 4);
    const float4 y = *reinterpret_cast<const float4*>(a.dv32 + row * D + d4 * 4);
    store4(reinterpret_cast<T*>(a.dk.ptr) + (int64_t)b * a.dk.sb + (int64_t)g * a.dk.sh + (int64_t)s * a.dk.ss + d4 * 4, x);
    store4(reinterpret_cast<T*>(a.dv.ptr) + (int64_t)b * a.dv.sb + (int64_t)g * a.dv.sh + (int64_t)s * a.dv.ss + d4 * 4, y);
  }
}

size_t delta_bytes(const brk_attn_bwd_params& p) {
  return (((size_t)p.B * p.N * p.S * sizeof(float)) + 255) & ~(size_t)255;
}
size_t acc_bytes(const brk_attn_bwd_params& p) { return (size_t)p.B * p.Nk * p.S * p.D * sizeof(float); }

template <typename T, int D>
int launch_all(const BwdArgs& a, cudaStream_t st) {
  const int TQ = kRows / a.G;
  dim3 g1((a.max_block_len + TQ - 1) / TQ, a.M, a.B * a.Nk);
  attn_bwd_dq_kernel<T, D><<<g1, kThreads, 0, st>>>(a);
  BRK_CUDA(cudaGetLastError());
  dim3 g2((a.max_block_len + kRows - 1) / kRows, a.M, a.B * a.Nk * a.nsplit);
  attn_bwd_dkv_kernel<T, D><<<g2, kThreads, 0, st>>>(a);
  BRK_CUDA(cudaGetLastError());
  const int64_t n4 = (int64_t)a.B * a.Nk * a.S * (D / 4);
  const int blocks = (int)std::min<int64_t>((n4 + 255) / 256, 148 * 16);
  attn_bwd_store_kernel<T><<<std::max(blocks, 1), 256, 0, st>>>(a, D);
  BRK_CUDA(cudaGetLastError());
  return BRK_OK;
}

}  // namespace

// (bf16 only) fp32 dq of the last block's rows, shared by the CTAs that split its keys
size_t dq_last_bytes(const brk_attn_bwd_params& p) {
  return p.dtype == BRK_BF16 ? (size_t)p.B * p.N * p.max_block_len * p.D * sizeof(float) : 0;
}
size_t attn_bwd_workspace(const brk_attn_bwd_params& p) { return delta_bytes(p) + 2 * acc_bytes(p) + dq_last_bytes(p); }

int attn_bwd_launch(const brk_attn_bwd_params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  BRK_REQUIRE(ws != nullptr && ws_bytes >= attn_bwd_workspace(p) && ((uintptr_t)ws & 15) == 0, BRK_E_WORKSPACE,
              "workspace %zu < %zu bytes (or not 16-byte aligned)", ws_bytes, attn_bwd_workspace(p));
  BwdArgs a;
  a.q = make_view(p.q); a.k = make_view(p.k); a.v = make_view(p.v); a.o = make_view(p.o); a.d_o = make_view(p.d_o);
  a.dq = make_view(p.dq); a.dk = make_view(p.dk); a.dv = make_view(p.dv);
  a.lse = p.lse;
  unsigned char* w = static_cast<unsigned char*>(ws);
  a.delta = reinterpret_cast<float*>(w);
  a.dk32 = reinterpret_cast<float*>(w + delta_bytes(p));
  a.dv32 = a.dk32 + (size_t)p.B * p.Nk * p.S * p.D;
  a.blk_start = p.blk_start; a.blk_len = p.blk_len;
  a.B = p.B; a.N = p.N; a.Nk = p.Nk; a.S = p.S; a.M = p.M; a.G = p.N / p.Nk; a.max_block_len = p.max_block_len;
  a.nsplit = p.M > 2 ? std::min(p.M, 64) : 1;  // block 0 is seen by every row block: its key tiles need many CTAs
  a.scale = p.scale;
  a.scale_log2 = p.scale * 1.4426950408889634f;
  BRK_CUDA(cudaMemsetAsync(w + delta_bytes(p), 0, 2 * acc_bytes(p) + dq_last_bytes(p), st));
  if (p.dtype == BRK_BF16) {
    // bf16: the tensor-core kernels compute dq and the accumulators; the conversion kernel is shared
    int rc = attn_bwd_mma_launch(p, a.delta, a.dk32, a.dv32, a.dv32 + (size_t)p.B * p.Nk * p.S * p.D, st);
    if (rc) return rc;
    const int64_t n4 = (int64_t)a.B * a.Nk * a.S * (p.D / 4);
    const int blocks = (int)std::min<int64_t>((n4 + 255) / 256, 148 * 16);
    attn_bwd_store_kernel<__nv_bfloat16><<<std::max(blocks, 1), 256, 0, st>>>(a, p.D);
    BRK_CUDA(cudaGetLastError());
    return BRK_OK;
  }
  return p.D == 128 ? launch_all<float, 128>(a, st) : launch_all<float, 64>(a, st);
}

}  // namespace brk
