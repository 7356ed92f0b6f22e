// BlockRank attention backward for bf16 on warp-level tensor-core MMA (mma.sync m16n8k16, fp32 accumulate).
// Same mathematics and the same two-kernel split as attn_bwd.cu (which stays the fp32 path):
//
//   attn_bwd_dq_mma_kernel   a CTA owns 64 query tokens of one (prompt, head, block); each of its four warps
//                            keeps the A fragments of 16 rows of Q and dO in registers and walks through the
//                            row's visible keys, 64 staged in shared memory at a time:
//                            S = Q K^T, dP = dO V^T, dS = P (dP - delta), dQ += dS K.  Also writes delta.
//   attn_bwd_dkv_mma_kernel  a CTA owns 64 keys of one (prompt, KV head, block), K and V resident in shared
//                            memory, 16 keys per warp, and walks through the rows that see them, 64 tokens of
//                            one head staged at a time: S^T = K Q^T, dP^T = V dO^T, dV += P^T dO,
//                            dK += dS^T Q.  Row blocks are dealt to `nsplit` CTAs, which add their fp32
//                            results into the accumulators with atomics (attn_bwd.cu's layout and store kernel).
//
// Operands reach the MMAs through ldmatrix from shared-memory tiles whose rows are padded by 16 bytes
// (conflict-free); a product that is the left operand of the next MMA (P^T, dS, dS^T) goes from accumulator
// registers to A fragments without leaving the warp.
#include <algorithm>

#include "brk_common.cuh"

namespace brk {

namespace {

constexpr int kT = 64;         // tokens (rows or keys) per staged tile
constexpr int kWarps = 4;
constexpr int kThreadsM = kWarps * 32;
// Row-tile buffers of the dk/dv kernel: 2 = the next tile is requested before the current one is multiplied (104 KB
// of shared memory; the kernel runs two CTAs per SM anyway: it keeps its keys' A fragments in registers), 1 = after.
constexpr int kRowBufs = 2;

struct BwdMmaArgs {
  View q, k, v, o, d_o, dq;
  const float* lse;
  float* delta;   // [B, N, S]
  float* dk32;    // [B, Nk, S, D]
  float* dv32;
  float* dq32;    // [B, N, max_block_len, D]: dq of the last block's rows, summed over the CTAs that share its keys
  const int32_t* blk_start;
  const int32_t* blk_len;
  int B, N, Nk, S, M, G, max_block_len;
  int nsplit;   // dk/dv kernel: CTAs that share the row blocks of one key tile
  int m_base;   // first block of this launch (blockIdx.y counts from it)
  int ksplit;   // dq kernel, last block: CTAs that share the key tiles of one row tile
  float scale, scale_log2;
};

__device__ __forceinline__ void span_of(const BwdMmaArgs& a, int b, int m, int& start, int& len) {
  start = a.blk_start[(size_t)b * a.M + m];
  len = a.blk_len[(size_t)b * a.M + m];
  if (start < 0 || len < 0 || len > a.max_block_len || start > a.S - len) len = 0;  // skipped: nothing out of bounds
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float x, float y) {
  __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int D>
struct Tile {
  static constexpr int kPitch = D + 8;  // elements: 16 bytes of padding per row
  __nv_bfloat16 e[kT][kPitch];
};

// rows [row0, row0 + kT) of head `h` of a (B, heads, S, D) bf16 tensor -> tile, zero beyond `nvalid`.
// All of a thread's loads are issued before its first store, so a tile costs one memory latency.
template <int D>
__device__ __forceinline__ void stage(Tile<D>& t, const View& x, int b, int h, int row0, int nvalid) {
  constexpr int kPer = kT * (D / 8) / kThreadsM;
  const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(x.ptr) + (int64_t)b * x.sb + (int64_t)h * x.sh;
  uint4 val[kPer];
#pragma unroll
  for (int it = 0; it < kPer; ++it) {
    const int i = threadIdx.x + it * kThreadsM;
    const int r = i / (D / 8), c = i % (D / 8);
    val[it] = make_uint4(0, 0, 0, 0);
    if (r < nvalid) val[it] = *reinterpret_cast<const uint4*>(base + (int64_t)(row0 + r) * x.ss + c * 8);
  }
#pragma unroll
  for (int it = 0; it < kPer; ++it) {
    const int i = threadIdx.x + it * kThreadsM;
    *reinterpret_cast<uint4*>(&t.e[i / (D / 8)][(i % (D / 8)) * 8]) = val[it];
  }
}

__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gmem_src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// the same copy as stage(), asynchronous (completion through cp.async groups): the next tile travels while the
// current one is multiplied
template <int D>
__device__ __forceinline__ void stage_async(Tile<D>& t, const View& x, int b, int h, int row0, int nvalid) {
  constexpr int kPer = kT * (D / 8) / kThreadsM;
  const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(x.ptr) + (int64_t)b * x.sb + (int64_t)h * x.sh;
#pragma unroll
  for (int it = 0; it < kPer; ++it) {
    const int i = threadIdx.x + it * kThreadsM;
    const int r = i / (D / 8), c = i % (D / 8);
    const bool ok = r < nvalid;
    cp_async16_zfill(&t.e[r][c * 8], base + (int64_t)(row0 + (ok ? r : 0)) * x.ss + c * 8, ok);
  }
}

// A fragments (16 rows x D) of rows [r0, r0+16) of a tile: frag[ks] covers columns [16 ks, 16 ks + 16)
template <int D>
__device__ __forceinline__ void load_a(uint32_t (&frag)[D / 16][4], const Tile<D>& t, int r0, int lane) {
  const int j = lane >> 3, r = lane & 7;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) ldsm_x4(frag[ks], &t.e[r0 + r + (j & 1) * 8][ks * 16 + (j >> 1) * 8]);
}

// C[16 x 16] (two n-tiles: c[0] columns 0..7, c[1] columns 8..15) = A[16 x D] * Y[n0 .. n0+16][0 .. D)^T
template <int D>
__device__ __forceinline__ void mm_nt(float (&c)[2][4], const uint32_t (&a)[D / 16][4], const Tile<D>& y, int n0, int lane) {
  const int j = lane >> 3, r = lane & 7;
#pragma unroll
  for (int i = 0; i < 4; ++i) c[0][i] = c[1][i] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t bfr[4];
    ldsm_x4(bfr, &y.e[n0 + r + (j >> 1) * 8][ks * 16 + (j & 1) * 8]);
    mma16816(c[0], a[ks], bfr[0], bfr[1]);
    mma16816(c[1], a[ks], bfr[2], bfr[3]);
  }
}

// acc[16 x D] += A[16 x 16] * Z[k0 .. k0+16][0 .. D)   (acc[nt] covers columns [8 nt, 8 nt + 8))
template <int D>
__device__ __forceinline__ void mm_nn_acc(float (&acc)[D / 8][4], const uint32_t (&a)[4], const Tile<D>& z, int k0, int lane) {
  const int j = lane >> 3, r = lane & 7;
#pragma unroll
  for (int np = 0; np < D / 16; ++np) {
    uint32_t bfr[4];
    ldsm_x4_t(bfr, &z.e[k0 + r + (j & 1) * 8][np * 16 + (j >> 1) * 8]);
    mma16816(acc[2 * np], a, bfr[0], bfr[1]);
    mma16816(acc[2 * np + 1], a, bfr[2], bfr[3]);
  }
}

// grid: x = 64-token tile of the block, y = block, z = prompt * N + head.  kLast: the launch for the last block,
// whose rows see every key of the prompt: y = split instead, the row tile's key tiles are dealt to `ksplit` CTAs
// and the results are added into the fp32 array dq32 (converted by attn_bwd_store_dq_last_kernel).
template <int D, bool kLast>
__global__ void __launch_bounds__(kThreadsM, 3) attn_bwd_dq_mma_kernel(BwdMmaArgs a) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  Tile<D>* const tiles = reinterpret_cast<Tile<D>*>(dyn_smem);  // [0], [1]: Q / dO first, then K / V; [2], [3]: the other K / V buffer
  Tile<D>& t0s = tiles[0];
  Tile<D>& t1s = tiles[1];
  __shared__ float delta_s[kT], lse_s[kT];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int b = blockIdx.z / a.N, head = blockIdx.z % a.N, g = head / a.G;
  const int m = kLast ? a.M - 1 : (int)blockIdx.y;
  const int split = kLast ? (int)blockIdx.y : 0;
  int start, len;
  span_of(a, b, m, start, len);
  __nv_bfloat16* dqb = reinterpret_cast<__nv_bfloat16*>(a.dq.ptr) + (int64_t)b * a.dq.sb + (int64_t)head * a.dq.sh;
  if (blockIdx.x == 0 && split == 0) {
    // slots in front of this block (and behind the last block) belong to no block: zero gradient
    int pstart, plen;
    if (m > 0) span_of(a, b, m - 1, pstart, plen);
    const int gap0 = (m == 0) ? 0 : max(0, min(a.S, pstart + plen));
    const int blk_lo = len > 0 ? start : gap0, blk_hi = len > 0 ? start + len : gap0;
    for (int pass = 0; pass < 2; ++pass) {
      const int lo = pass == 0 ? gap0 : blk_hi;
      const int hi = pass == 0 ? blk_lo : (m == a.M - 1 ? a.S : blk_hi);
      for (int i = tid; i < (hi - lo) * (D / 8); i += kThreadsM)
        *reinterpret_cast<uint4*>(dqb + (int64_t)(lo + i / (D / 8)) * a.dq.ss + (i % (D / 8)) * 8) = make_uint4(0, 0, 0, 0);
    }
  }
  const int tok0 = blockIdx.x * kT;
  if (tok0 >= len) return;
  const int nrow = min(kT, len - tok0);

  // Q, dO -> A fragments; delta = rowsum(dO * O)
  stage<D>(t0s, a.q, b, head, start + tok0, nrow);
  stage<D>(t1s, a.d_o, b, head, start + tok0, nrow);
  if (tid < kT) {
    float dl = 0.f, ls = 0.f;
    if (tid < nrow) {
      const int64_t slot = start + tok0 + tid;
      const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(a.d_o.ptr) + (int64_t)b * a.d_o.sb + (int64_t)head * a.d_o.sh + slot * a.d_o.ss;
      const __nv_bfloat16* op = reinterpret_cast<const __nv_bfloat16*>(a.o.ptr) + (int64_t)b * a.o.sb + (int64_t)head * a.o.sh + slot * a.o.ss;
      for (int d = 0; d < D; d += 8) {
        float x[8], y[8];
        load8(gp + d, x);
        load8(op + d, y);
#pragma unroll
        for (int i = 0; i < 8; ++i) dl = fmaf(x[i], y[i], dl);
      }
      const size_t rid = ((size_t)b * a.N + head) * a.S + slot;
      a.delta[rid] = dl;
      ls = a.lse[rid] * 1.4426950408889634f;
    }
    delta_s[tid] = dl;
    lse_s[tid] = ls;
  }
  __syncthreads();
  uint32_t qa[D / 16][4], ga[D / 16][4];
  load_a<D>(qa, t0s, warp * 16, lane);
  load_a<D>(ga, t1s, warp * 16, lane);
  const int r_lo = warp * 16 + gq, r_hi = r_lo + 8;  // this thread's two rows of the tile
  const float lse_lo = lse_s[r_lo], lse_hi = lse_s[r_hi], dl_lo = delta_s[r_lo], dl_hi = delta_s[r_hi];
  const bool act_lo = r_lo < nrow, act_hi = r_hi < nrow;
  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  // Key tiles: the earlier blocks in full, then the own block up to this CTA's last token; tile i + 1 is
  // copied into the other pair of buffers while tile i is multiplied.
  const int n_ctx = (m == 0) ? 0 : (m < a.M - 1 ? 1 : a.M - 1);
  struct KeyIt { int seg, k0, ks, kl, no; bool own; };
  auto seg_init = [&](KeyIt& it) {
    for (; it.seg <= n_ctx; ++it.seg) {
      it.own = it.seg == n_ctx;
      if (it.own) { it.ks = start; it.kl = tok0 + nrow; } else span_of(a, b, it.seg, it.ks, it.kl);
      it.k0 = 0;
      if (it.kl > 0) return true;
    }
    return false;
  };
  auto step = [&](KeyIt& it) {
    ++it.no;
    it.k0 += kT;
    if (it.k0 < it.kl) return true;
    ++it.seg;
    return seg_init(it);
  };
  // (last block: tile number `no` belongs to the CTA with split == no % ksplit)
  auto mine = [&](const KeyIt& it) { return !kLast || it.no % a.ksplit == split; };
  auto advance = [&](KeyIt& it) {
    bool ok = step(it);
    while (ok && !mine(it)) ok = step(it);
    return ok;
  };
  auto issue = [&](const KeyIt& it, int buf) {
    const int nv = min(kT, it.kl - it.k0);
    stage_async<D>(tiles[2 * buf], a.k, b, g, it.ks + it.k0, nv);
    stage_async<D>(tiles[2 * buf + 1], a.v, b, g, it.ks + it.k0, nv);
  };
  KeyIt cur{0, 0, 0, 0, 0, false};
  bool has = seg_init(cur);
  if (has && !mine(cur)) has = advance(cur);
  __syncthreads();  // every warp holds its Q / dO fragments: buffers 0 and 1 may be overwritten
  if (has) issue(cur, 0);
  cp_async_commit();
  KeyIt nxt = cur;
  int buf = 0;
  while (has) {
    const bool has_n = advance(nxt);
    if (has_n) issue(nxt, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();  // all but the newest group: the current tile has landed
    __syncthreads();
    {
      const Tile<D>& kt = tiles[2 * buf];
      const Tile<D>& vt = tiles[2 * buf + 1];
      const bool own = cur.own;
      const int k0 = cur.k0, nv = min(kT, cur.kl - cur.k0);
      // this warp's rows see keys up to (own block) token tok0 + 16 warp + 15
      const int kmax = own ? min(nv, tok0 + warp * 16 + 16 - k0) : nv;
      for (int c0 = 0; c0 < kmax; c0 += 16) {
        float s[2][4], dp[2][4];
        mm_nt<D>(s, qa, kt, c0, lane);
        mm_nt<D>(dp, ga, vt, c0, lane);
        uint32_t dsa[4];
        float ds[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = k0 + c0 + nt * 8 + 2 * tq + (e & 1);  // token index within the key block
            const bool hi = e >= 2;
            const int tok = tok0 + (hi ? r_hi : r_lo);
            const bool vis = (hi ? act_hi : act_lo) && key < k0 + nv && (!own || key <= tok);
            const float p = vis ? exp2f(s[nt][e] * a.scale_log2 - (hi ? lse_hi : lse_lo)) : 0.f;
            ds[nt][e] = p * (dp[nt][e] - (hi ? dl_hi : dl_lo));
          }
        }
        dsa[0] = pack_bf16(ds[0][0], ds[0][1]);
        dsa[1] = pack_bf16(ds[0][2], ds[0][3]);
        dsa[2] = pack_bf16(ds[1][0], ds[1][1]);
        dsa[3] = pack_bf16(ds[1][2], ds[1][3]);
        mm_nn_acc<D>(acc, dsa, kt, c0, lane);
      }
    }
    __syncthreads();  // this pair of buffers is refilled by the next iteration's copy
    cur = nxt;
    has = has_n;
    buf ^= 1;
  }
  if (kLast) {
    float* base = a.dq32 + (((size_t)b * a.N + head) * a.max_block_len + tok0) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      const int col = nt * 8 + 2 * tq;
      if (act_lo) {
        atomicAdd(base + (size_t)r_lo * D + col, acc[nt][0] * a.scale);
        atomicAdd(base + (size_t)r_lo * D + col + 1, acc[nt][1] * a.scale);
      }
      if (act_hi) {
        atomicAdd(base + (size_t)r_hi * D + col, acc[nt][2] * a.scale);
        atomicAdd(base + (size_t)r_hi * D + col + 1, acc[nt][3] * a.scale);
      }
    }
    return;
  }
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const int col = nt * 8 + 2 * tq;
    if (act_lo)
      *reinterpret_cast<uint32_t*>(dqb + (int64_t)(start + tok0 + r_lo) * a.dq.ss + col) =
          pack_bf16(acc[nt][0] * a.scale, acc[nt][1] * a.scale);
    if (act_hi)
      *reinterpret_cast<uint32_t*>(dqb + (int64_t)(start + tok0 + r_hi) * a.dq.ss + col) =
          pack_bf16(acc[nt][2] * a.scale, acc[nt][3] * a.scale);
  }
}

// dq32 -> dq for the rows of the last block: one thread per 8 elements
template <int D>
__global__ void __launch_bounds__(256) attn_bwd_store_dq_last_kernel(BwdMmaArgs a) {
  const int64_t n8 = (int64_t)a.B * a.N * a.max_block_len * (D / 8);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % (D / 8));
    const int64_t row = i / (D / 8);
    const int tok = (int)(row % a.max_block_len);
    const int head = (int)((row / a.max_block_len) % a.N), b = (int)(row / ((int64_t)a.max_block_len * a.N));
    int start, len;
    span_of(a, b, a.M - 1, start, len);
    if (tok >= len) continue;
    float v[8];
    load8(a.dq32 + row * D + c * 8, v);
    store8(reinterpret_cast<__nv_bfloat16*>(a.dq.ptr) + (int64_t)b * a.dq.sb + (int64_t)head * a.dq.sh +
               (int64_t)(start + tok) * a.dq.ss + c * 8, v);
  }
}

// grid: x = 64-key tile of the block, y = key block, z = ((prompt * Nk + KV head) * nsplit + split)
template <int D>
__global__ void __launch_bounds__(kThreadsM, 2) attn_bwd_dkv_mma_kernel(BwdMmaArgs a) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  Tile<D>& ks_t = *reinterpret_cast<Tile<D>*>(dyn_smem);
  Tile<D>& vs_t = *reinterpret_cast<Tile<D>*>(dyn_smem + sizeof(Tile<D>));
  Tile<D>* const row_tiles = reinterpret_cast<Tile<D>*>(dyn_smem + 2 * sizeof(Tile<D>));  // [2 buf]: Q, [2 buf + 1]: dO
  float* const row_stats = reinterpret_cast<float*>(dyn_smem + (2 + 2 * kRowBufs) * sizeof(Tile<D>));  // [buf][lse: kT | delta: kT]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int split = blockIdx.z % a.nsplit, bg = blockIdx.z / a.nsplit;
  const int b = bg / a.Nk, g = bg % a.Nk;
  const int m = a.m_base + (int)blockIdx.y;
  int start, len;
  span_of(a, b, m, start, len);
  const int j0 = blockIdx.x * kT;
  if (j0 >= len) return;
  if (split >= ((m == 0) ? a.M : ((m < a.M - 1) ? 2 : 1))) return;  // no row block left for this split
  const int nkey = min(kT, len - j0);
  stage<D>(ks_t, a.k, b, g, start + j0, nkey);
  stage<D>(vs_t, a.v, b, g, start + j0, nkey);
  // (visible to every warp after the first barrier of the row loop)
  const int k_lo = j0 + warp * 16 + gq, k_hi = k_lo + 8;  // this thread's two keys (token index in the block)
  const bool kv_lo = k_lo < len, kv_hi = k_hi < len;
  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }

  // Row blocks that see these keys: the own block (causally); every later block for block 0; the last block
  // for a document block.  Entry e of that list is handled by the CTA with split == e % nsplit.
  const int n_list = (m == 0) ? a.M : ((m < a.M - 1) ? 2 : 1);
  // Row tiles in the order (list entry, head of the group, 64 tokens); tile i + 1 is copied into the other
  // pair of buffers while tile i is multiplied.
  struct RowIt { int e, hh, t0, rs, rl, tfirst; bool own; };
  auto entry_init = [&](RowIt& it) {
    for (; it.e < n_list; it.e += a.nsplit) {
      const int mr = (it.e == 0) ? m : ((m == 0) ? it.e : a.M - 1);
      it.own = it.e == 0;
      span_of(a, b, mr, it.rs, it.rl);
      it.tfirst = it.own ? j0 : 0;  // earlier rows see none of the tile's keys
      it.t0 = it.tfirst;
      it.hh = 0;
      if (it.t0 < it.rl) return true;
    }
    return false;
  };
  auto advance = [&](RowIt& it) {
    it.t0 += kT;
    if (it.t0 < it.rl) return true;
    it.t0 = it.tfirst;
    if (++it.hh < a.G) return true;
    it.e += a.nsplit;
    return entry_init(it);
  };
  auto issue = [&](const RowIt& it, int buf) {
    const int head = g * a.G + it.hh, nv = min(kT, it.rl - it.t0);
    stage_async<D>(row_tiles[2 * buf], a.q, b, head, it.rs + it.t0, nv);
    stage_async<D>(row_tiles[2 * buf + 1], a.d_o, b, head, it.rs + it.t0, nv);
    if (tid < 2 * kT) {
      const int r = tid & (kT - 1);
      const size_t rid = ((size_t)b * a.N + head) * a.S + it.rs + it.t0 + min(r, nv - 1);
      cp_async4(row_stats + buf * 2 * kT + tid, (tid < kT ? a.lse : a.delta) + rid);
    }
  };
  __syncthreads();  // K and V of this CTA's keys are in place
  uint32_t ka_k[D / 16][4], ka_v[D / 16][4];  // this warp's 16 keys as A fragments, for every row tile
  load_a<D>(ka_k, ks_t, warp * 16, lane);
  load_a<D>(ka_v, vs_t, warp * 16, lane);
  RowIt cur{split, 0, 0, 0, 0, 0, false};
  bool has = entry_init(cur);
  if (has) issue(cur, 0);
  cp_async_commit();
  RowIt nxt = cur;
  int buf = 0;
  while (has) {
    bool has_n = false;
    if (kRowBufs == 2) {
      has_n = advance(nxt);
      if (has_n) issue(nxt, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();  // all but the newest group: the current row tile has landed
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();     // (the first time also: K and V of this CTA's keys are in place)
    {
      const Tile<D>& qs_t = row_tiles[2 * buf];
      const Tile<D>& gs_t = row_tiles[2 * buf + 1];
      const float* lse_s = row_stats + buf * 2 * kT;
      const float* delta_s = lse_s + kT;
      const bool own = cur.own;
      const int t0 = cur.t0, nv = min(kT, cur.rl - cur.t0);
      // own block: this warp's keys start at token j0 + 16 warp; rows before that see none of them
      const int c_first = own ? max(0, ((j0 + warp * 16 - t0) / 16) * 16) : 0;
      for (int c0 = c_first; c0 < nv; c0 += 16) {
        float st[2][4], dpt[2][4];
        mm_nt<D>(st, ka_k, qs_t, c0, lane);   // S^T: rows = keys, columns = query tokens
        mm_nt<D>(dpt, ka_v, gs_t, c0, lane);  // dP^T
        float p[2][4], ds[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int rr = c0 + nt * 8 + 2 * tq + (x & 1);  // row of the tile
            const bool hi = x >= 2;
            const int key = hi ? k_hi : k_lo;
            const bool vis = (hi ? kv_hi : kv_lo) && rr < nv && (!own || t0 + rr >= key);
            const float pv = vis ? exp2f(st[nt][x] * a.scale_log2 - lse_s[rr] * 1.4426950408889634f) : 0.f;
            p[nt][x] = pv;
            ds[nt][x] = pv * (dpt[nt][x] - delta_s[rr]);
          }
        }
        uint32_t pa[4] = {pack_bf16(p[0][0], p[0][1]), pack_bf16(p[0][2], p[0][3]), pack_bf16(p[1][0], p[1][1]),
                          pack_bf16(p[1][2], p[1][3])};
        uint32_t da[4] = {pack_bf16(ds[0][0], ds[0][1]), pack_bf16(ds[0][2], ds[0][3]), pack_bf16(ds[1][0], ds[1][1]),
                          pack_bf16(ds[1][2], ds[1][3])};
        mm_nn_acc<D>(dv, pa, gs_t, c0, lane);
        mm_nn_acc<D>(dk, da, qs_t, c0, lane);
      }
    }
    __syncthreads();  // this pair of buffers is refilled by the next copy
    if (kRowBufs == 1) {
      has_n = advance(nxt);
      if (has_n) issue(nxt, 0);
      cp_async_commit();
    } else {
      buf ^= 1;
    }
    cur = nxt;
    has = has_n;
  }
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const int col = nt * 8 + 2 * tq;
    if (kv_lo) {
      const size_t off = (((size_t)b * a.Nk + g) * a.S + start + k_lo) * D + col;
      atomicAdd(a.dk32 + off, dk[nt][0] * a.scale);
      atomicAdd(a.dk32 + off + 1, dk[nt][1] * a.scale);
      atomicAdd(a.dv32 + off, dv[nt][0]);
      atomicAdd(a.dv32 + off + 1, dv[nt][1]);
    }
    if (kv_hi) {
      const size_t off = (((size_t)b * a.Nk + g) * a.S + start + k_hi) * D + col;
      atomicAdd(a.dk32 + off, dk[nt][2] * a.scale);
      atomicAdd(a.dk32 + off + 1, dk[nt][3] * a.scale);
      atomicAdd(a.dv32 + off, dv[nt][2]);
      atomicAdd(a.dv32 + off + 1, dv[nt][3]);
    }
  }
}

template <int D>
int launch_mma(BwdMmaArgs a, cudaStream_t st) {
  const int tiles = (a.max_block_len + kT - 1) / kT;
  const int smem_dq = 4 * (int)sizeof(Tile<D>);
  BRK_CUDA(cudaFuncSetAttribute(attn_bwd_dq_mma_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq));
  BRK_CUDA(cudaFuncSetAttribute(attn_bwd_dq_mma_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq));
  // the last block first: its CTAs are the long ones
  a.ksplit = std::max(1, std::min(32, (a.S / kT) / 8));
  attn_bwd_dq_mma_kernel<D, true><<<dim3(tiles, a.ksplit, a.B * a.N), kThreadsM, smem_dq, st>>>(a);
  BRK_CUDA(cudaGetLastError());
  if (a.M > 1) {
    attn_bwd_dq_mma_kernel<D, false><<<dim3(tiles, a.M - 1, a.B * a.N), kThreadsM, smem_dq, st>>>(a);
    BRK_CUDA(cudaGetLastError());
  }
  {
    const int64_t n8 = (int64_t)a.B * a.N * a.max_block_len * (D / 8);
    const int blocks = (int)std::min<int64_t>((n8 + 255) / 256, 148 * 8);
    attn_bwd_store_dq_last_kernel<D><<<std::max(blocks, 1), 256, 0, st>>>(a);
    BRK_CUDA(cudaGetLastError());
  }
  const int smem = (2 + 2 * kRowBufs) * (int)sizeof(Tile<D>) + 2 * kRowBufs * kT * (int)sizeof(float);
  BRK_CUDA(cudaFuncSetAttribute(attn_bwd_dkv_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  // block 0's keys are seen by every row block: many CTAs per key tile; the other blocks' keys by two at most
  a.m_base = 0;
  a.nsplit = a.M > 2 ? std::min(a.M, 64) : 1;
  attn_bwd_dkv_mma_kernel<D><<<dim3(tiles, 1, a.B * a.Nk * a.nsplit), kThreadsM, smem, st>>>(a);
  BRK_CUDA(cudaGetLastError());
  if (a.M > 1) {
    a.m_base = 1;
    a.nsplit = 2;
    attn_bwd_dkv_mma_kernel<D><<<dim3(tiles, a.M - 1, a.B * a.Nk * a.nsplit), kThreadsM, smem, st>>>(a);
    BRK_CUDA(cudaGetLastError());
  }
  return BRK_OK;
}

}  // namespace

// dq (and delta) and the fp32 dk / dv accumulators for bf16 tensors; the caller clears the accumulators
// before and converts them afterwards.
int attn_bwd_mma_launch(const brk_attn_bwd_params& p, float* delta, float* dk32, float* dv32, float* dq32,
                        cudaStream_t st) {
  BwdMmaArgs a;
  a.q = make_view(p.q); a.k = make_view(p.k); a.v = make_view(p.v); a.o = make_view(p.o); a.d_o = make_view(p.d_o);
  a.dq = make_view(p.dq);
  a.lse = p.lse; a.delta = delta; a.dk32 = dk32; a.dv32 = dv32; a.dq32 = dq32;
  a.blk_start = p.blk_start; a.blk_len = p.blk_len;
  a.B = p.B; a.N = p.N; a.Nk = p.Nk; a.S = p.S; a.M = p.M; a.G = p.N / p.Nk; a.max_block_len = p.max_block_len;
  a.nsplit = 1; a.m_base = 0; a.ksplit = 1;
  a.scale = p.scale;
  a.scale_log2 = p.scale * 1.4426950408889634f;
  return p.D == 128 ? launch_mma<128>(a, st) : launch_mma<64>(a, st);
}

}  // namespace brk
