// BlockRank attention forward on the sm_100a tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Work item = one CTA = (prompt b, block m, KV head g, tile of 128/G query
// tokens) x the G query heads that share KV head g: the 128 rows of the MMA
// tile are (token, head) pairs, so one K/V tile in shared memory serves the
// whole GQA group and the Q tile is a single 3-D TMA box of the [B,S,N,D]
// tensor.  Only live key tiles are visited:
//   block 0            : own keys, causal
//   document block     : the prefix block's keys, then own keys, causal
//   query (last) block : every slot of the earlier blocks, then own keys, causal
// Per key tile (64 keys): S = Q K^T (tcgen05.mma, both operands K-major in
// 128B-swizzled shared memory, accumulator in TMEM) -> each of the 128 threads
// owns one row: tcgen05.ld, mask, online softmax (base 2, lazy rescale), P as
// bf16 into swizzled shared memory -> O += P V (V is the MN-major B operand,
// accumulator stays in TMEM across tiles).  K and V tiles are double buffered
// and prefetched by TMA; S is double buffered in TMEM so the next QK^T runs
// under the current softmax.  Two CTAs fit per SM (112 KB smem, 256 TMEM
// columns each), which overlaps one CTA's softmax with the other's MMAs.
//
// Every mbarrier wait is bounded; on expiry the CTA records a code in the
// caller's status word, stops waiting, and still runs to its normal exit
// (TMEM is released on every path).
#include <cuda.h>

#include "brk_common.cuh"
#include "tc_ptx.cuh"

namespace brk {

// ---- host: tensor maps -----------------------------------------------------------------
EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || p == nullptr)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

int make_tmap_bf16(CUtensorMap* out, const void* ptr, int D, int heads, int S, int B, int64_t stride_h,
                   int64_t stride_s, int64_t stride_b, int box_h, int box_s) {
  EncodeTiledFn enc = get_encode_tiled();
  BRK_REQUIRE(enc != nullptr, BRK_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if (B == 1) stride_b = (int64_t)S * stride_s;  // a size-1 dim may carry any stride
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)heads, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_s * 2, (cuuint64_t)stride_b * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_h, (cuuint32_t)box_s, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BRK_REQUIRE(r == CUDA_SUCCESS, BRK_E_CUDA,
              "cuTensorMapEncodeTiled failed (%d): dims {%d,%d,%d,%d} strides {%lld,%lld,%lld} box {64,%d,%d,1}", (int)r,
              D, heads, S, B, (long long)stride_h, (long long)stride_s, (long long)stride_b, box_h, box_s);
  return BRK_OK;
}

namespace {

constexpr int BM = 128;  // query rows (token, head) per CTA
constexpr int BN = 64;   // keys per tile
constexpr int HD = 128;  // head dim
constexpr int kThreads = 128;
constexpr uint32_t kQBytes = 2 * BM * 128;   // two 64-wide halves of D
constexpr uint32_t kKVBytes = 2 * BN * 128;  // one K or V tile
constexpr uint32_t kPBytes = BM * 128;
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + kQBytes;
constexpr uint32_t kOffV = kOffK + 2 * kKVBytes;
constexpr uint32_t kOffP = kOffV + 2 * kKVBytes;
constexpr uint32_t kOffBar = kOffP + kPBytes;
constexpr uint32_t kSmemBytes = kOffBar + 256 + 512;  // barriers + slack for the 1024-byte round-up
constexpr uint32_t kTmemCols = 256;                   // S0 [0,64) S1 [64,128) O [128,256)
constexpr uint32_t kColO = 128;
constexpr float kLazy = 8.f;  // rescale O only when the running max grows by more than 2^8
constexpr uint32_t kWaitBudget = 1u << 18;

struct TcArgs {
  View o;
  float* lse;
  const int32_t* blk_start;
  const int32_t* blk_len;
  int32_t* status;
  int B, N, Nk, S, M;
  int G, g_shift;  // query heads per KV head, log2
  float scale_log2;
  int n_split;     // key chunks the query block's context is cut into (1 = no split)
  int lq_max;      // rows per (prompt, head) in the partial buffers (= max_block_len)
  float* part_o;   // [B, N, lq_max, n_split, 128] un-normalised partial outputs
  float2* part_ml; // [B, N, lq_max, n_split] (running max in log2 units, sum)
};

enum { kBarQ = 0, kBarK0 = 1, kBarK1 = 2, kBarV0 = 3, kBarV1 = 4, kBarS0 = 5, kBarS1 = 6, kBarO = 7, kNumBars = 8 };

// slot -> is it inside some block?  (blk_start is non-decreasing)
__device__ __forceinline__ bool slot_valid(const int32_t* bs, const int32_t* bl, int M, int s) {
  int lo = 0, hi = M;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (bs[mid] <= s) lo = mid + 1; else hi = mid;
  }
  const int m = lo - 1;
  return m >= 0 && s < bs[m] + bl[m];
}

__global__ void __launch_bounds__(kThreads, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const TcArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z / a.Nk, g = blockIdx.z % a.Nk;
  // grid.y: first the n_split key chunks of the query block (longest work first), then blocks M-2 .. 0
  const bool is_last = (int)blockIdx.y < a.n_split;
  const int chunk = is_last ? (int)blockIdx.y : 0;
  const int m = is_last ? a.M - 1 : a.M - 2 - ((int)blockIdx.y - a.n_split);
  const int tile = blockIdx.x;
  const int G = a.G, TOK = BM >> a.g_shift;
  const int32_t* bs = a.blk_start + (size_t)b * a.M;
  const int32_t* bl = a.blk_len + (size_t)b * a.M;
  const int start = bs[m], len = bl[m];

  __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(a.o.ptr) + (int64_t)b * a.o.sb;
  if (tile == 0 && chunk == 0) {
    // padding slots in front of this block (and behind the last one) are written as zeros
    const int gap0 = (m == 0) ? 0 : bs[m - 1] + bl[m - 1];
    const int per_row = G * (HD / 8);
    for (int pass = 0; pass < 2; ++pass) {
      const int lo = pass == 0 ? gap0 : start + len;
      const int hi = pass == 0 ? start : ((m == a.M - 1) ? a.S : start + len);
      for (int i = tid; i < (hi - lo) * per_row; i += kThreads) {
        const int s = lo + i / per_row, rem = i % per_row;
        const int h = g * G + rem / (HD / 8), d8 = rem % (HD / 8);
        *reinterpret_cast<uint4*>(ob + (int64_t)s * a.o.ss + (int64_t)h * a.o.sh + d8 * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  }
  const int t0 = tile * TOK;
  if (t0 >= len) return;  // uniform for the CTA, nothing allocated yet

  // ---- shared memory carve-up ----------------------------------------------------------------
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (sbase - raw);
  const uint32_t sQ = sbase + kOffQ, sK = sbase + kOffK, sV = sbase + kOffV, sP = sbase + kOffP;
  const uint32_t sBar = sbase + kOffBar;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBar + kNumBars * 8);
  int* red_i = reinterpret_cast<int*>(smem + kOffBar + 128);
  auto bar = [&](int i) { return sBar + (uint32_t)i * 8u; };

  // ---- key ranges ------------------------------------------------------------------------
  int ctx_lo = 0, ctx_hi = 0;
  bool ctx_check = false;  // context range may contain padding slots
  if (m > 0 && a.M > 1) {
    ctx_lo = bs[0];
    if (m < a.M - 1) {
      ctx_hi = bs[0] + bl[0];
    } else {
      ctx_hi = bs[a.M - 2] + bl[a.M - 2];
      int part = 0;
      for (int i = tid; i < a.M - 1; i += kThreads) part += bl[i];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
      if (lane == 0) red_i[warp] = part;
      __syncthreads();
      ctx_check = (red_i[0] + red_i[1] + red_i[2] + red_i[3]) != (ctx_hi - ctx_lo);
    }
  }
  const int own_n = min(len, t0 + TOK);
  const int n_ctx = (ctx_hi - ctx_lo + BN - 1) / BN;
  // this CTA's share of the tile list: everything, or one chunk of the context (+ own keys for the last chunk)
  int j0 = 0, n_tiles = n_ctx + (own_n + BN - 1) / BN;
  const bool split = is_last && a.n_split > 1;
  if (split) {
    const int per = (n_ctx + a.n_split - 1) / a.n_split;
    j0 = min(n_ctx, chunk * per);
    const int j1 = (chunk == a.n_split - 1) ? n_tiles : min(n_ctx, j0 + per);
    n_tiles = j1 - j0;
    if (n_tiles <= 0) {  // empty chunk: leave a neutral partial for the combine step
      const int rr = tid, rtok = t0 + (rr >> a.g_shift);
      if (rtok < len && rtok < a.lq_max)
        a.part_ml[(((int64_t)b * a.N + g * G + (rr & (G - 1))) * a.lq_max + rtok) * a.n_split + chunk] =
            make_float2(-INFINITY, 0.f);
      return;
    }
  }

  bool failed = (sbase - raw) > 512u;  // cannot happen with the 1024-byte aligned declaration
  if (tid == 0) {
    for (int i = 0; i < kNumBars; ++i) ptx::mbar_init(bar(i), 1);
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmQ);
    ptx::prefetch_tmap(&tmK);
    ptx::prefetch_tmap(&tmV);
  }
  __syncwarp();
  if (warp == 0) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_lane = tmem + ((uint32_t)(warp * 32) << 16);

  auto wait = [&](int i, uint32_t parity, int code) {
    if (failed) return;
    if (!ptx::mbar_wait(bar(i), parity, kWaitBudget)) {
      failed = true;
      if (a.status) atomicCAS(a.status, 0, code);
    }
  };
  auto tile_lo = [&](int jl, int& nk, bool& own) {
    const int j = jl + j0;
    own = j >= n_ctx;
    if (!own) {
      const int lo = ctx_lo + j * BN;
      nk = min(BN, ctx_hi - lo);
      return lo;
    }
    const int off = (j - n_ctx) * BN;
    nk = min(BN, own_n - off);
    return start + off;
  };
  auto load_kv = [&](const CUtensorMap* tm, uint32_t dst, int barrier, int j) {
    int nk; bool own;
    const int lo = tile_lo(j, nk, own);
    ptx::mbar_expect_tx(bar(barrier), kKVBytes);
    ptx::tma_load_4d(dst, tm, bar(barrier), 0, g, lo, b);
    ptx::tma_load_4d(dst + BN * 128, tm, bar(barrier), 64, g, lo, b);
  };
  auto issue_qk = [&](int j) {
    int nk; bool own;
    tile_lo(j, nk, own);
    const int st = j & 1;
    const uint32_t idesc = ptx::idesc_bf16(BM, (uint32_t)((nk + 15) & ~15), 0, 0);
    const uint32_t kb = sK + (uint32_t)st * kKVBytes;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      const uint64_t ad = ptx::smem_desc_sw128(sQ + (uint32_t)(ks >> 2) * (BM * 128) + (uint32_t)(ks & 3) * 32, 16, 1024);
      const uint64_t bd = ptx::smem_desc_sw128(kb + (uint32_t)(ks >> 2) * (BN * 128) + (uint32_t)(ks & 3) * 32, 16, 1024);
      ptx::mma_ss(tmem + (uint32_t)st * BN, ad, bd, idesc, ks > 0);
    }
    ptx::mma_commit(bar(kBarS0 + st));
  };
  auto issue_pv = [&](int j) {
    int nk; bool own;
    tile_lo(j, nk, own);
    const int st = j & 1;
    const uint32_t idesc = ptx::idesc_bf16(BM, HD, 0, 1);
    const uint32_t vb = sV + (uint32_t)st * kKVBytes;
    const int ksteps = (nk + 15) >> 4;
    for (int ks = 0; ks < ksteps; ++ks) {
      const uint64_t ad = ptx::smem_desc_sw128(sP + (uint32_t)ks * 32, 16, 1024);
      const uint64_t bd = ptx::smem_desc_sw128(vb + (uint32_t)ks * (16 * 128), BN * 128, 1024);
      ptx::mma_ss(tmem + kColO, ad, bd, idesc, (j > 0 || ks > 0) ? 1u : 0u);
    }
    ptx::mma_commit(bar(kBarO));
  };

  // ---- prologue: Q, the first two K/V tiles, first QK^T ----------------------------------------
  if (tid == 0) {
    ptx::mbar_expect_tx(bar(kBarQ), kQBytes);
    ptx::tma_load_4d(sQ, &tmQ, bar(kBarQ), 0, g * G, start + t0, b);
    ptx::tma_load_4d(sQ + BM * 128, &tmQ, bar(kBarQ), 64, g * G, start + t0, b);
    load_kv(&tmK, sK, kBarK0, 0);
    load_kv(&tmV, sV, kBarV0, 0);
    if (n_tiles > 1) {
      load_kv(&tmK, sK + kKVBytes, kBarK1, 1);
      load_kv(&tmV, sV + kKVBytes, kBarV1, 1);
    }
    wait(kBarQ, 0, 1);
    wait(kBarK0, 0, 2);
    ptx::tc_fence_after_sync();
    issue_qk(0);
  }
  __syncwarp();

  const int r = tid;                 // row of the tile = TMEM lane
  const int tok = t0 + (r >> a.g_shift);
  const int n = g * G + (r & (G - 1));
  const bool active = tok < len;
  float m_run = -INFINITY, l_run = 0.f;

  for (int j = 0; j < n_tiles; ++j) {
    const int st = j & 1;
    const uint32_t ph = (uint32_t)(j >> 1) & 1u;
    int nk; bool own;
    const int lo = tile_lo(j, nk, own);

    if (tid == 0 && j + 1 < n_tiles) {
      wait(kBarK0 + ((j + 1) & 1), (uint32_t)((j + 1) >> 1) & 1u, 3);
      ptx::tc_fence_after_sync();
      issue_qk(j + 1);  // runs under this tile's softmax
    }
    __syncwarp();
    wait(kBarS0 + st, ph, 4);
    ptx::tc_fence_after_sync();
    if (tid == 0 && j + 2 < n_tiles) load_kv(&tmK, sK + (uint32_t)st * kKVBytes, kBarK0 + st, j + 2);  // K stage is free
    __syncwarp();

    uint32_t sr[64];
    {
      uint32_t (&lo32)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sr[0]);
      uint32_t (&hi32)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sr[32]);
      ptx::tmem_ld32(tmem_lane + (uint32_t)st * BN, lo32);
      ptx::tmem_ld32(tmem_lane + (uint32_t)st * BN + 32, hi32);
      ptx::tmem_wait_ld();
    }
    // Tiles that lie fully inside the visible region need no per-element masking (the common case);
    // ragged tails, the causal diagonal and padded context ranges take the masked path.
    const int own_off = (j + j0 - n_ctx) * BN;
    const bool need_mask = nk < BN || (own && own_off + BN - 1 > t0) || (!own && ctx_check);
    float mx = -INFINITY;
    if (!need_mask) {
#pragma unroll
      for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(sr[c]));
    } else {
      int lim = nk;  // columns [0, lim) are visible to this row
      if (own) lim = max(0, min(nk, tok - own_off + 1));
      unsigned v0 = 0xffffffffu, v1 = 0xffffffffu;
      if (!own && ctx_check) {
        v0 = __ballot_sync(0xffffffffu, slot_valid(bs, bl, a.M, lo + lane));
        v1 = __ballot_sync(0xffffffffu, slot_valid(bs, bl, a.M, lo + 32 + lane));
      }
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const bool ok = c < lim && (((c < 32 ? v0 : v1) >> (c & 31)) & 1u);
        const float sv = ok ? __uint_as_float(sr[c]) : -INFINITY;
        sr[c] = __float_as_uint(sv);
        mx = fmaxf(mx, sv);
      }
    }
    mx *= a.scale_log2;  // scale > 0, so the max commutes with it
    float m_new = fmaxf(m_run, mx);
    if (m_run != -INFINITY && m_new - m_run <= kLazy) m_new = m_run;  // keep the old reference: p <= 2^8
    const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
    const float corr = ptx::ex2(m_run - m_ref);  // 1 when unchanged, 0 on the first visible tile
    const float neg_ref = -m_ref;
    float psum = 0.f;
    uint32_t pk[32];
#pragma unroll
    for (int c = 0; c < 64; c += 2) {
      const float p0 = ptx::ex2(fmaf(__uint_as_float(sr[c]), a.scale_log2, neg_ref));
      const float p1 = ptx::ex2(fmaf(__uint_as_float(sr[c + 1]), a.scale_log2, neg_ref));
      psum += p0 + p1;
      __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
      pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
    }
    l_run = l_run * corr + psum;
    const bool changed = m_new != m_run;
    m_run = m_new;

    if (j > 0) {
      wait(kBarO, (uint32_t)(j - 1) & 1u, 5);  // PV of the previous tile done: O stable, P and a V stage free
      ptx::tc_fence_after_sync();
      if (tid == 0 && j + 1 < n_tiles) load_kv(&tmV, sV + (uint32_t)((j + 1) & 1) * kKVBytes, kBarV0 + ((j + 1) & 1), j + 1);
      __syncwarp();
      if (__any_sync(0xffffffffu, changed)) {
#pragma unroll 1
        for (int ch = 0; ch < HD / 32; ++ch) {
          uint32_t orow[32];
          ptx::tmem_ld32(tmem_lane + kColO + (uint32_t)ch * 32, orow);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
          ptx::tmem_st32(tmem_lane + kColO + (uint32_t)ch * 32, orow);
        }
        ptx::tmem_wait_st();
      }
    }
    // P row -> shared memory in the K-major 128B-swizzled layout the MMA reads
    {
      uint8_t* prow = smem + kOffP + (uint32_t)r * 128;
#pragma unroll
      for (int c16 = 0; c16 < 8; ++c16)
        *reinterpret_cast<uint4*>(prow + ((c16 ^ (r & 7)) << 4)) =
            make_uint4(pk[c16 * 4], pk[c16 * 4 + 1], pk[c16 * 4 + 2], pk[c16 * 4 + 3]);
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      ptx::tc_fence_after_sync();
      wait(kBarV0 + st, ph, 6);
      issue_pv(j);
    }
  }

  // ---- epilogue ---------------------------------------------------------------------------------
  wait(kBarO, (uint32_t)(n_tiles - 1) & 1u, 7);
  ptx::tc_fence_after_sync();
  if (split) {
    // un-normalised partial (O, max, sum) of this key chunk; merged by attn_combine_kernel
    const int64_t prow = (((int64_t)b * a.N + n) * a.lq_max + tok) * a.n_split + chunk;
#pragma unroll 1
    for (int ch = 0; ch < HD / 32; ++ch) {
      uint32_t orow[32];
      ptx::tmem_ld32(tmem_lane + kColO + (uint32_t)ch * 32, orow);
      ptx::tmem_wait_ld();
      if (active && tok < a.lq_max) {
        float4* dst = reinterpret_cast<float4*>(a.part_o + prow * HD + ch * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[i] = make_float4(__uint_as_float(orow[4 * i]), __uint_as_float(orow[4 * i + 1]),
                               __uint_as_float(orow[4 * i + 2]), __uint_as_float(orow[4 * i + 3]));
      }
    }
    if (active && tok < a.lq_max) a.part_ml[prow] = make_float2(m_run, l_run);
    ptx::tc_fence_before_sync();
    __syncthreads();
  } else {
    // O / l -> bf16 -> staging (reusing the Q tile) -> coalesced stores
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
    for (int ch = 0; ch < HD / 32; ++ch) {
      uint32_t orow[32];
      ptx::tmem_ld32(tmem_lane + kColO + (uint32_t)ch * 32, orow);
      ptx::tmem_wait_ld();
      uint8_t* srow = smem + kOffQ + (uint32_t)(ch >> 1) * (BM * 128) + (uint32_t)r * 128;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(orow[q4 * 8 + 2 * i]) * inv,
                                                   __uint_as_float(orow[q4 * 8 + 2 * i + 1]) * inv);
          w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        const int c16 = (ch & 1) * 4 + q4;
        *reinterpret_cast<uint4*>(srow + ((c16 ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    if (active && a.lse != nullptr)
      a.lse[((int64_t)b * a.N + n) * a.S + start + tok] = (m_run + log2f(l_run)) * 0.6931471805599453f;
    ptx::tc_fence_before_sync();
    __syncthreads();
    for (int it = 0; it < 16; ++it) {
      const int rr = warp * 32 + it * 2 + (lane >> 4);
      const int piece = lane & 15;
      const int rtok = t0 + (rr >> a.g_shift);
      if (rtok < len) {
        const uint8_t* src = smem + kOffQ + (uint32_t)(piece >> 3) * (BM * 128) + (uint32_t)rr * 128 +
                             (((piece & 7) ^ (rr & 7)) << 4);
        __nv_bfloat16* dst = ob + (int64_t)(start + rtok) * a.o.ss + (int64_t)(g * G + (rr & (G - 1))) * a.o.sh + piece * 8;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
      }
    }
  }
  if (warp == 0) ptx::tmem_dealloc(tmem, kTmemCols);
}


// Merge the key-chunk partials of the query block: one warp per (prompt, head, query token).
__global__ void __launch_bounds__(128) attn_combine_kernel(TcArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int64_t total = (int64_t)a.B * a.N * a.lq_max;
  if (w >= total) return;
  const int tok = (int)(w % a.lq_max);
  const int n = (int)((w / a.lq_max) % a.N);
  const int b = (int)(w / ((int64_t)a.lq_max * a.N));
  const int start = a.blk_start[(size_t)b * a.M + a.M - 1], len = a.blk_len[(size_t)b * a.M + a.M - 1];
  if (tok >= len) return;
  const float2* ml = a.part_ml + w * a.n_split;
  float mx = -INFINITY;
  for (int c = 0; c < a.n_split; ++c) mx = fmaxf(mx, ml[c].x);
  const float ref = (mx == -INFINITY) ? 0.f : mx;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l = 0.f;
  for (int c = 0; c < a.n_split; ++c) {
    const float2 x = ml[c];
    if (x.y > 0.f) {  // chunks that saw no key carry no output
      const float wgt = exp2f(x.x - ref);
      const float4 o = *reinterpret_cast<const float4*>(a.part_o + (w * a.n_split + c) * HD + lane * 4);
      acc.x = fmaf(o.x, wgt, acc.x); acc.y = fmaf(o.y, wgt, acc.y);
      acc.z = fmaf(o.z, wgt, acc.z); acc.w = fmaf(o.w, wgt, acc.w);
      l = fmaf(x.y, wgt, l);
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.o.ptr) + (int64_t)b * a.o.sb + (int64_t)(start + tok) * a.o.ss +
                       (int64_t)n * a.o.sh + lane * 4;
  store4(dst, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
  if (a.lse != nullptr && lane == 0) a.lse[((int64_t)b * a.N + n) * a.S + start + tok] = (ref + log2f(l)) * 0.6931471805599453f;
}

}  // namespace

// Key chunks for the query block.  Its context is every earlier token of the prompt (S is the only
// bound known on the host), walked 64 keys per step by a single CTA per 128 rows; cutting it into
// chunks of about 1024 keys keeps that serial chain short and gives the SMs enough CTAs.
static int tc_splits(const brk_attn_params& p) {
  if (p.M < 2) return 1;
  int n = (p.S + 1023) / 1024;
  return n < 1 ? 1 : (n > 32 ? 32 : n);
}

size_t attn_tc_workspace(const brk_attn_params& p) {
  const int ns = tc_splits(p);
  if (ns <= 1) return 0;
  const size_t rows = (size_t)p.B * p.N * p.max_block_len * ns;
  return rows * HD * sizeof(float) + rows * sizeof(float2);
}

int attn_tc_launch(const brk_attn_params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  BRK_REQUIRE(p.dtype == BRK_BF16 && p.D == HD, BRK_E_UNSUPPORTED,
              "tcgen05 attention needs bf16 and head_dim 128 (dtype %d, head_dim %d)", p.dtype, p.D);
  const int G = p.N / p.Nk;
  BRK_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, BRK_E_UNSUPPORTED, "tcgen05 attention needs N/Nk in {1,2,4,8}, got %d", G);
  const int ns = tc_splits(p);
  BRK_REQUIRE(p.B * p.Nk <= 65535 && p.M + ns <= 65535, BRK_E_UNSUPPORTED, "grid too large: B*Nk=%d M=%d", p.B * p.Nk, p.M);
  BRK_REQUIRE(p.scale > 0.f, BRK_E_ARG, "softmax scale must be positive");
  const size_t need = attn_tc_workspace(p);
  BRK_REQUIRE(need == 0 || (ws != nullptr && ws_bytes >= need && ((uintptr_t)ws & 15) == 0), BRK_E_WORKSPACE,
              "attention workspace: %zu bytes (16-byte aligned) needed, %zu given", need, ws_bytes);
  int gs = 0;
  while ((1 << gs) < G) ++gs;
  const int TOK = BM / G;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_bf16(&tq, p.q.ptr, HD, p.N, p.S, p.B, p.q.stride_h, p.q.stride_s, p.q.stride_b, G, TOK))) return rc;
  if ((rc = make_tmap_bf16(&tk, p.k.ptr, HD, p.Nk, p.S, p.B, p.k.stride_h, p.k.stride_s, p.k.stride_b, 1, BN))) return rc;
  if ((rc = make_tmap_bf16(&tv, p.v.ptr, HD, p.Nk, p.S, p.B, p.v.stride_h, p.v.stride_s, p.v.stride_b, 1, BN))) return rc;
  static bool configured[64] = {};
  int dev = 0;
  BRK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    BRK_CUDA(cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    BRK_CUDA(cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  TcArgs a;
  a.o = make_view(p.o);
  a.lse = p.lse;
  a.blk_start = p.blk_start;
  a.blk_len = p.blk_len;
  a.status = p.status;
  a.B = p.B; a.N = p.N; a.Nk = p.Nk; a.S = p.S; a.M = p.M;
  a.G = G; a.g_shift = gs;
  a.scale_log2 = p.scale * 1.4426950408889634f;
  a.n_split = ns;
  a.lq_max = p.max_block_len;
  const size_t rows = (size_t)p.B * p.N * p.max_block_len * ns;
  a.part_o = ns > 1 ? reinterpret_cast<float*>(ws) : nullptr;
  a.part_ml = ns > 1 ? reinterpret_cast<float2*>(reinterpret_cast<float*>(ws) + rows * HD) : nullptr;
  dim3 grid((p.max_block_len + TOK - 1) / TOK, (p.M - 1) + ns, p.B * p.Nk);
  attn_tc_kernel<<<grid, kThreads, kSmemBytes, st>>>(tq, tk, tv, a);
  BRK_CUDA(cudaGetLastError());
  if (ns > 1) {
    const int64_t warps = (int64_t)p.B * p.N * p.max_block_len;
    attn_combine_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(a);
    BRK_CUDA(cudaGetLastError());
  }
  return BRK_OK;
}

}  // namespace brk
