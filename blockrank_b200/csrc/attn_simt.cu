// BlockRank attention forward on CUDA cores (fp32 accumulate).
//
// This is the exact-arithmetic kernel of the library: it serves fp32 models
// (tensor cores would drop to tf32) and any head_dim / group size the tcgen05
// kernel does not cover.  One CTA owns (prompt, block, KV head, tile of query
// tokens) and all query heads of that KV group, so K/V rows are staged in
// shared memory once per group (no repeat_kv).  Each query row is held by four
// threads, each owning a quarter of head_dim; keys are visited only inside the
// live segments of the row's block: [prefix block] + own block causally for a
// document, every earlier block + own block for the query block.
#include "brk_common.cuh"

namespace brk {

namespace {

constexpr int kThreads = 256;
constexpr int kRows = kThreads / 4;  // query rows (token, head) per CTA
constexpr int kKeyTile = 32;         // keys staged per step
constexpr int kChunk = 8;            // keys per softmax rescale

struct SimtArgs {
  View q, k, v, o;
  float* lse;
  const int32_t* blk_start;
  const int32_t* blk_len;
  const int* hdr;  // workspace header: hdr[1] != 0 when the prologue kernel found the block spans malformed
  int B, N, Nk, S, M;
  float scale_log2;  // scale * log2(e)
};

template <typename T, int D, int G>
__global__ void __launch_bounds__(kThreads) attn_simt_kernel(SimtArgs a) {
  constexpr int TQ = kRows / G;  // query tokens per CTA
  constexpr int F = D / 16;      // float4 groups per thread
  __shared__ __align__(16) float Ks[kKeyTile][D];
  __shared__ __align__(16) float Vs[kKeyTile][D];

  if (a.hdr[1] != 0) return;  // malformed spans: write nothing
  const int tid = threadIdx.x;
  const int b = blockIdx.z / a.Nk, g = blockIdx.z % a.Nk;
  const int m = a.M - 1 - blockIdx.y;  // the long query-block CTAs are scheduled first
  const int tile = blockIdx.x;
  const int32_t* bs = a.blk_start + (size_t)b * a.M;
  const int32_t* bl = a.blk_len + (size_t)b * a.M;
  const int start = bs[m], len = bl[m];

  T* ob = reinterpret_cast<T*>(a.o.ptr) + (int64_t)b * a.o.sb;
  {
    // Padding slots are written as zeros: the gap in front of this block by the block's first CTA, the gap behind
    // the last block (thousands of rows when a batch is padded to its longest prompt) in slices by all of the
    // last block's CTAs.
    const int per_row = G * (D / 4);
    auto zero_rows = [&](int lo, int hi) {
      for (int i = tid; i < (hi - lo) * per_row; i += kThreads) {
        const int s = lo + i / per_row, rem = i % per_row;
        const int h = g * G + rem / (D / 4), d4 = rem % (D / 4);
        store4(ob + (int64_t)s * a.o.ss + (int64_t)h * a.o.sh + d4 * 4, make_float4(0.f, 0.f, 0.f, 0.f));
      }
    };
    if (tile == 0) zero_rows((m == 0) ? 0 : bs[m - 1] + bl[m - 1], start);
    if (m == a.M - 1) {
      const int lo = start + len, rows = a.S - lo;
      const int per = (rows + (int)gridDim.x - 1) / (int)gridDim.x;
      if (rows > 0) zero_rows(lo + min(rows, tile * per), lo + min(rows, (tile + 1) * per));
    }
  }
  const int t0 = tile * TQ;
  if (t0 >= len) return;

  const int r = tid >> 2, j = tid & 3;
  const int tok = t0 + r / G;
  const int n = g * G + r % G;
  const bool active = tok < len;

  float qreg[F * 4], oacc[F * 4];
  {
    const T* qp = reinterpret_cast<const T*>(a.q.ptr) + (int64_t)b * a.q.sb + (int64_t)n * a.q.sh +
                  (int64_t)(start + (active ? tok : 0)) * a.q.ss;
#pragma unroll
    for (int f = 0; f < F; ++f) {
      float4 x = active ? load4(qp + (j + 4 * f) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      qreg[4 * f + 0] = x.x * a.scale_log2;
      qreg[4 * f + 1] = x.y * a.scale_log2;
      qreg[4 * f + 2] = x.z * a.scale_log2;
      qreg[4 * f + 3] = x.w * a.scale_log2;
      oacc[4 * f + 0] = oacc[4 * f + 1] = oacc[4 * f + 2] = oacc[4 * f + 3] = 0.f;
    }
  }
  float m_run = -INFINITY, l_run = 0.f;

  const T* kb = reinterpret_cast<const T*>(a.k.ptr) + (int64_t)b * a.k.sb + (int64_t)g * a.k.sh;
  const T* vb = reinterpret_cast<const T*>(a.v.ptr) + (int64_t)b * a.v.sb + (int64_t)g * a.v.sh;

  // context segments: none for block 0, the prefix for documents, every earlier block for the query block
  const int n_ctx = (m == 0) ? 0 : (m < a.M - 1 ? 1 : a.M - 1);
  const int own_keys = min(len, t0 + TQ);
  for (int seg = 0; seg <= n_ctx; ++seg) {
    const bool own = seg == n_ctx;
    const int seg_start = own ? start : bs[seg];
    const int seg_len = own ? own_keys : bl[seg];
    for (int kt = 0; kt < seg_len; kt += kKeyTile) {
      const int nk = min(kKeyTile, seg_len - kt);
      __syncthreads();
      for (int i = tid; i < nk * (D / 4); i += kThreads) {
        const int kk = i / (D / 4), d4 = i % (D / 4);
        const int64_t s = seg_start + kt + kk;
        *reinterpret_cast<float4*>(&Ks[kk][d4 * 4]) = load4(kb + s * a.k.ss + d4 * 4);
        *reinterpret_cast<float4*>(&Vs[kk][d4 * 4]) = load4(vb + s * a.v.ss + d4 * 4);
      }
      __syncthreads();
      for (int c = 0; c < nk; c += kChunk) {
        float sc[kChunk];
        float cmax = -INFINITY;
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
          const int kk = c + i;
          float acc = 0.f;
          if (kk < nk) {
#pragma unroll
            for (int f = 0; f < F; ++f) {
              const float4 kv = *reinterpret_cast<const float4*>(&Ks[kk][(j + 4 * f) * 4]);
              acc = fmaf(qreg[4 * f + 0], kv.x, acc);
              acc = fmaf(qreg[4 * f + 1], kv.y, acc);
              acc = fmaf(qreg[4 * f + 2], kv.z, acc);
              acc = fmaf(qreg[4 * f + 3], kv.w, acc);
            }
          }
          acc += __shfl_xor_sync(0xffffffffu, acc, 1);
          acc += __shfl_xor_sync(0xffffffffu, acc, 2);
          const bool ok = kk < nk && (!own || kt + kk <= tok);
          sc[i] = ok ? acc : -INFINITY;
          cmax = fmaxf(cmax, sc[i]);
        }
        const float m_new = fmaxf(m_run, cmax);
        // while nothing is visible to this row yet (m_new == -inf) every factor below is exp2(-inf) = 0
        const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = exp2f(m_run - m_ref);
        l_run *= corr;
#pragma unroll
        for (int x = 0; x < F * 4; ++x) oacc[x] *= corr;
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
          const int kk = c + i;
          if (kk < nk) {
            const float p = exp2f(sc[i] - m_ref);
            l_run += p;
#pragma unroll
            for (int f = 0; f < F; ++f) {
              const float4 vv = *reinterpret_cast<const float4*>(&Vs[kk][(j + 4 * f) * 4]);
              oacc[4 * f + 0] = fmaf(p, vv.x, oacc[4 * f + 0]);
              oacc[4 * f + 1] = fmaf(p, vv.y, oacc[4 * f + 1]);
              oacc[4 * f + 2] = fmaf(p, vv.z, oacc[4 * f + 2]);
              oacc[4 * f + 3] = fmaf(p, vv.w, oacc[4 * f + 3]);
            }
          }
        }
        m_run = m_new;
      }
    }
  }
  if (!active) return;
  const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
  T* op = ob + (int64_t)(start + tok) * a.o.ss + (int64_t)n * a.o.sh;
#pragma unroll
  for (int f = 0; f < F; ++f)
    store4(op + (j + 4 * f) * 4, make_float4(oacc[4 * f] * inv, oacc[4 * f + 1] * inv, oacc[4 * f + 2] * inv,
                                             oacc[4 * f + 3] * inv));
  if (a.lse != nullptr && j == 0)
    a.lse[((int64_t)b * a.N + n) * a.S + start + tok] = (m_run + log2f(l_run)) * 0.6931471805599453f;
}

template <typename T, int D>
int launch_g(const brk_attn_params& p, const SimtArgs& a, cudaStream_t st) {
  const int G = p.N / p.Nk;
  const int tq = kRows / G;
  dim3 grid((p.max_block_len + tq - 1) / tq, p.M, p.B * p.Nk);
  switch (G) {
    case 1: attn_simt_kernel<T, D, 1><<<grid, kThreads, 0, st>>>(a); break;
    case 2: attn_simt_kernel<T, D, 2><<<grid, kThreads, 0, st>>>(a); break;
    case 4: attn_simt_kernel<T, D, 4><<<grid, kThreads, 0, st>>>(a); break;
    case 8: attn_simt_kernel<T, D, 8><<<grid, kThreads, 0, st>>>(a); break;
    default:
      set_error("SIMT attention supports N/Nk in {1,2,4,8}, got %d", G);
      return BRK_E_UNSUPPORTED;
  }
  BRK_CUDA(cudaGetLastError());
  return BRK_OK;
}

}  // namespace

int attn_simt_launch(const brk_attn_params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  BRK_REQUIRE(ws != nullptr && ws_bytes >= kWsHeader && ((uintptr_t)ws & 15) == 0, BRK_E_WORKSPACE,
              "attention workspace: %zu bytes (16-byte aligned) needed, %zu given", kWsHeader, ws_bytes);
  int rc = attn_prologue_launch(p, reinterpret_cast<int*>(ws), nullptr, 0, st);
  if (rc) return rc;
  SimtArgs a;
  a.hdr = reinterpret_cast<const int*>(ws);
  a.q = make_view(p.q);
  a.k = make_view(p.k);
  a.v = make_view(p.v);
  a.o = make_view(p.o);
  a.lse = p.lse;
  a.blk_start = p.blk_start;
  a.blk_len = p.blk_len;
  a.B = p.B; a.N = p.N; a.Nk = p.Nk; a.S = p.S; a.M = p.M;
  a.scale_log2 = p.scale * 1.4426950408889634f;
  BRK_REQUIRE(p.B * p.Nk <= 65535 && p.M <= 65535, BRK_E_UNSUPPORTED, "grid too large: B*Nk=%d M=%d", p.B * p.Nk, p.M);
  if (p.dtype == BRK_F32) {
    if (p.D == 64) return launch_g<float, 64>(p, a, st);
    if (p.D == 128) return launch_g<float, 128>(p, a, st);
  } else {
    if (p.D == 64) return launch_g<__nv_bfloat16, 64>(p, a, st);
    if (p.D == 128) return launch_g<__nv_bfloat16, 128>(p, a, st);
  }
  set_error("SIMT attention supports head_dim 64 or 128, got %d", p.D);
  return BRK_E_UNSUPPORTED;
}

}  // namespace brk
