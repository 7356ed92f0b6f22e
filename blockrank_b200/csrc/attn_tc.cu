// BlockRank attention forward on the sm_100a tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Persistent, warp-specialised kernel: one CTA per SM; the CTAs claim work items (longest first)
// from a global counter.  A work item is (prompt b, KV head g, block m, pair of row tiles[, key chunk]); a row tile is
// 128 MMA rows = 128/G consecutive query tokens x the G query heads that share KV head g, so
// one K/V tile in shared memory serves the whole GQA group and a Q tile is one 3-D TMA box of
// the [B,S,N,D] tensor.  The two row tiles of a pair ("chains") share the item's K/V tiles and
// are processed in ping-pong: while one chain's 128 softmax threads work on their S tile, the
// tensor core runs the other chain's MMAs.
//
// Only live keys are visited, in 64-key slots (one TMA box each):
//   block 0            : own keys, causal
//   document block     : the prefix block's keys, then own keys, causal
//   query (last) block : every slot of the earlier blocks, then own keys, causal; its context
//                        is cut into key chunks, each a work item that leaves an un-normalised
//                        partial (O, max, sum); attn_combine_kernel merges them.
// Two consecutive slots form one 128-key MMA tile (a document's prefix slot and its first own
// slot share a tile), which halves the barrier hops per key and runs QK^T at the full N=128 rate.
//
// Roles (320 threads):
//   warps 0-3 / 4-7  softmax + output of chain 0 / 1 (thread = row = TMEM lane)
//   warp 8           TMA producer: claims and decodes the items (the decoded item goes to the other
//                    roles through a 4-deep record ring in shared memory), loads Q tiles and a
//                    2-stage ring of 128-key K/V tiles, running ahead across items
//   warp 9           MMA issuer: S = Q K^T (both operands K-major, 128B swizzle) and O += P V
//                    (P read from tensor memory, V as the MN-major B operand)
// O stays in TMEM across the key tiles of an item; softmax is base-2, online, with a lazy
// rescale (O is only touched when the running max grows by more than 2^8).  P (bf16, two keys
// per 32-bit column) overwrites the first half of the S tile it was computed from.
//
// Shared memory 194 KB: Q 2x32 KB, K/V ring 2x64 KB, barriers, item records.  TMEM: 2 x (S 128 + O 128) columns.
// No cluster multicast anywhere.  Every mbarrier wait is bounded; on expiry the thread records
// a code in the caller's status word, stops waiting and runs to the normal exit.
#include <cuda.h>

#include <type_traits>

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

constexpr int BM = 128;  // query rows (token, head) per row tile
constexpr int BN = 64;   // keys per slot (one TMA box)
constexpr int BT = 128;  // keys per MMA tile (two slots)
constexpr int HD = 128;  // head dim
constexpr int kStages = 2;
constexpr int kThreads = 320;
constexpr uint32_t kQBytes = 2 * BM * 128;  // two 64-wide halves of D
constexpr uint32_t kSlotBytes = 2 * BN * 128;  // K (or V) of one 64-key slot
constexpr uint32_t kKBytes = 2 * BT * 128;     // one K (or V) tile: [d half][128 keys][128 B]
constexpr uint32_t kStageBytes = 2 * kKBytes;
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffKV = kOffQ + 2 * kQBytes;
constexpr uint32_t kOffBar = kOffKV + kStages * kStageBytes;
constexpr int kItemRing = 4;                        // decoded work items in flight between the producer and its consumers
constexpr uint32_t kOffItems = kOffBar + 256;       // kItemRing records of 16 ints
constexpr uint32_t kSmemBytes = kOffItems + kItemRing * 64 + 1024;  // + slack for the 1024-byte round-up
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kChainCols = 256;  // per chain: S [0,128) (P over its first 64 columns), then O [128,256)
constexpr uint32_t kColO = 128;
constexpr float kLazy = 8.f;
constexpr uint32_t kWaitBudget = 1u << 18;

enum {
  kQFull = 0,    // +chain  TMA -> MMA: Q tile landed
  kQFree = 2,    // +chain  MMA -> TMA: every QK^T of the item has read Q
  kSFull = 4,    // +chain  MMA -> softmax: S tile complete (+2, +3 unused)
  kPFull = 8,    // +chain  softmax -> MMA: P written to tensor memory, S consumed (4 warp arrivals)
  kPVDone = 10,  // +chain  MMA -> softmax: P V of a tile complete
  kOFree = 12,   // +chain  softmax -> MMA: O read out of TMEM (4 warp arrivals)
  kKVFull = 14,  // +stage  TMA -> MMA
  kKVFree = 14 + kStages,  // +stage  MMA -> TMA
  kItemFull = 14 + 2 * kStages,           // +ring slot  TMA warp -> MMA, softmax: item record written
  kItemFree = kItemFull + kItemRing,      // +ring slot  MMA + 8 softmax warps -> TMA warp: record copied (9 arrivals)
  kNumBars = kItemFree + kItemRing
};
static_assert(kNumBars * 8 + 4 <= 256, "barrier area");

// Division by a run-time constant with a host-computed reciprocal (round-up method, exact for every
// 32-bit numerator): q = umulhi(n, mul); n / d = (((n - q) >> 1) + q) >> shift.
struct FastDiv {
  uint32_t d, mul, shift;
};
inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  f.d = d; f.mul = 0; f.shift = 0;
  if (d <= 1) return f;
  uint32_t s = 0;
  while ((1u << s) < d) ++s;  // ceil(log2 d)
  f.mul = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << s) - d)) / d + 1);
  f.shift = s - 1;
  return f;
}
__device__ __forceinline__ uint32_t fdiv(uint32_t n, const FastDiv& f) {
  if (f.d <= 1) return n;
  const uint32_t q = __umulhi(n, f.mul);
  return (((n - q) >> 1) + q) >> f.shift;
}

struct TcArgs {
  View o;
  float* lse;
  const int32_t* blk_start;
  const int32_t* blk_len;
  int32_t* status;
  int B, N, Nk, S, M;
  int G, g_shift;   // query heads per KV head, log2
  float scale_log2;
  int n_split;      // key chunks of the query block's context (1 = no split)
  int lq_max;       // rows per (prompt, head) in the partial buffers (= max_block_len)
  int pairs;        // row-tile pairs per block (covers max_block_len)
  int o_align32;    // output rows are 32-byte aligned (enables 32-byte stores)
  int total_items;
  FastDiv div_sec1, div_nbg, div_sec2, div_nk;  // by nbg*n_split, nbg, nbg*(M-1), Nk
  int* work_counter;  // next unclaimed index of the work list (zeroed before the launch)
  float* part_o;    // [B, N, lq_max, n_split, 128] un-normalised partial outputs
  float2* part_ml;  // [B, N, lq_max, n_split] (running max in log2 units, sum)
};

struct Item {
  int b, g, m, chunk;
  int start, len;        // span of block m
  int t0_0, t0_1;        // first token of each chain's row tile
  int n_0, n_1;          // key tiles visible to each chain (a prefix of the item's tile list)
  // selected with a conditional move rather than an indexed array, so the item stays in registers
  __device__ __forceinline__ int t0(int x) const { return x ? t0_1 : t0_0; }
  __device__ __forceinline__ int n_x(int x) const { return x ? n_1 : n_0; }
  int ctx_lo, ctx_hi;    // context key range (slots)
  int n_ctx, j0;         // context tiles of the block, first tile of this item
  int n_tiles, own_n;
  bool split, valid;
};

// Block spans an item needs, fetched one item ahead of their use: decoding is two dependent
// global-memory round trips, which would otherwise sit on every role's critical path.
struct ItemRaw {
  int m, chunk, p, b, g;
  int start, len;      // span of block m
  int s0, l0;          // span of block 0 (the prefix)
  int s2, l2;          // span of block M-2 (end of the query block's context)
};

// Work list order: query-block chunks first (longest), then blocks M-2 .. 0.
__device__ __forceinline__ ItemRaw load_item(const TcArgs& a, int idx) {
  ItemRaw r;
  if (idx >= a.total_items) idx = a.total_items - 1;  // prefetch past the end: harmless reload
  const int nbg = a.B * a.Nk;
  const int sec1 = nbg * a.n_split * a.pairs;
  int bg;
  if (idx < sec1) {
    r.p = (int)fdiv((uint32_t)idx, a.div_sec1);
    const int q = idx - r.p * (nbg * a.n_split);
    r.chunk = (int)fdiv((uint32_t)q, a.div_nbg);
    bg = q - r.chunk * nbg;
    r.m = a.M - 1;
  } else {
    const int i2 = idx - sec1;
    r.p = (int)fdiv((uint32_t)i2, a.div_sec2);
    const int q = i2 - r.p * (nbg * (a.M - 1));
    const int mm = (int)fdiv((uint32_t)q, a.div_nbg);
    r.m = a.M - 2 - mm;
    bg = q - mm * nbg;
    r.chunk = 0;
  }
  r.b = (int)fdiv((uint32_t)bg, a.div_nk);
  r.g = bg - r.b * a.Nk;
  const int32_t* bs = a.blk_start + (size_t)r.b * a.M;
  const int32_t* bl = a.blk_len + (size_t)r.b * a.M;
  const int m2 = a.M >= 2 ? a.M - 2 : 0;
  r.start = bs[r.m];
  r.len = bl[r.m];
  r.s0 = bs[0];
  r.l0 = bl[0];
  r.s2 = bs[m2];
  r.l2 = bl[m2];
  return r;
}

__device__ __forceinline__ Item decode_item(const TcArgs& a, const ItemRaw& r) {
  Item it;
  const int TOK = BM >> a.g_shift;
  it.b = r.b; it.g = r.g; it.m = r.m; it.chunk = r.chunk;
  it.start = r.start;
  it.len = r.len;
  it.t0_0 = 2 * r.p * TOK;
  it.t0_1 = it.t0_0 + TOK;
  it.valid = it.t0_0 < it.len;
  it.split = it.m == a.M - 1 && a.n_split > 1;
  it.ctx_lo = it.ctx_hi = 0;
  it.n_ctx = it.j0 = it.n_tiles = it.own_n = 0;
  it.n_0 = it.n_1 = 0;
  if (!it.valid) return it;
  if (it.m > 0) {
    it.ctx_lo = r.s0;
    it.ctx_hi = (it.m < a.M - 1) ? r.s0 + r.l0 : r.s2 + r.l2;
  }
  const bool on1 = it.t0_1 < it.len;
  it.own_n = min(it.len, (on1 ? it.t0_1 : it.t0_0) + TOK);
  it.n_ctx = (it.ctx_hi - it.ctx_lo + BN - 1) / BN;
  const int own_tiles = (it.own_n + BN - 1) / BN;
  int j1 = it.n_ctx + own_tiles;
  if (it.split) {
    const int per = (it.n_ctx + a.n_split - 1) / a.n_split;
    it.j0 = min(it.n_ctx, it.chunk * per);
    if (it.chunk != a.n_split - 1) j1 = min(it.n_ctx, it.j0 + per);
  }
  it.n_tiles = j1 - it.j0;
  if (it.n_tiles <= 0) {  // a chunk without tiles: nothing to do (its partial stays neutral)
    it.valid = false;
    it.n_tiles = 0;
    return it;
  }
  // own tiles visible to chain x: those starting at or before its last token
  {
    const int own_x = min(own_tiles, (min(it.len, it.t0_0 + TOK) + BN - 1) / BN);
    it.n_0 = max(0, min(j1, it.n_ctx + own_x) - it.j0);
  }
  if (on1) {
    const int own_x = min(own_tiles, (min(it.len, it.t0_1 + TOK) + BN - 1) / BN);
    it.n_1 = max(0, min(j1, it.n_ctx + own_x) - it.j0);
  }
  return it;
}

// tile j of the item -> first key slot, number of keys, whether it lies in the item's own block
__device__ __forceinline__ int tile_lo(const Item& it, int j, int& nk, bool& own, int& own_off) {
  const int jg = j + it.j0;
  own = jg >= it.n_ctx;
  if (!own) {
    const int lo = it.ctx_lo + jg * BN;
    nk = min(BN, it.ctx_hi - lo);
    own_off = 0;
    return lo;
  }
  own_off = (jg - it.n_ctx) * BN;
  nk = min(BN, it.own_n - own_off);
  return it.start + own_off;
}

// Work items are decoded once, by the TMA warp, and handed to the MMA warp and the softmax warps as
// 16-int records in shared memory: decoding costs two global-memory round trips and a few hundred
// scalar instructions, which would otherwise sit on every role's critical path between two items.
constexpr int kRecSplit = 1, kRecCtxCheck = 2, kRecStop = 4;
__device__ __forceinline__ void write_record(int* rec, const Item& it, int flags) {
  reinterpret_cast<int4*>(rec)[0] = make_int4(it.b, it.g, it.m, it.chunk);
  reinterpret_cast<int4*>(rec)[1] = make_int4(it.start, it.len, it.t0_0, it.n_0);
  reinterpret_cast<int4*>(rec)[2] = make_int4(it.n_1, it.ctx_lo, it.ctx_hi, it.n_ctx);
  reinterpret_cast<int4*>(rec)[3] = make_int4(it.j0, it.n_tiles, it.own_n, flags);
}
__device__ __forceinline__ Item read_record(const int* rec, int tok_per_tile, int& flags) {
  const int4 r0 = reinterpret_cast<const int4*>(rec)[0], r1 = reinterpret_cast<const int4*>(rec)[1];
  const int4 r2 = reinterpret_cast<const int4*>(rec)[2], r3 = reinterpret_cast<const int4*>(rec)[3];
  Item it;
  it.b = r0.x; it.g = r0.y; it.m = r0.z; it.chunk = r0.w;
  it.start = r1.x; it.len = r1.y; it.t0_0 = r1.z; it.n_0 = r1.w;
  it.t0_1 = it.t0_0 + tok_per_tile;
  it.n_1 = r2.x; it.ctx_lo = r2.y; it.ctx_hi = r2.z; it.n_ctx = r2.w;
  it.j0 = r3.x; it.n_tiles = r3.y; it.own_n = r3.z;
  flags = r3.w;
  it.split = (flags & kRecSplit) != 0;
  it.valid = true;
  return it;
}

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

__global__ void __launch_bounds__(kThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const TcArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = a.G;

  // ---- padding slots of the output are written as zeros (gaps in front of / behind blocks) ----
  for (int gi = blockIdx.x; gi < a.B * (a.M + 1); gi += gridDim.x) {
    const int b = gi / (a.M + 1), m = gi % (a.M + 1);
    const int32_t* bs = a.blk_start + (size_t)b * a.M;
    const int32_t* bl = a.blk_len + (size_t)b * a.M;
    const int lo = (m == 0) ? 0 : bs[m - 1] + bl[m - 1];
    const int hi = (m == a.M) ? a.S : bs[m];
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(a.o.ptr) + (int64_t)b * a.o.sb;
    const int per_row = a.N * (HD / 8);
    for (int i = tid; i < (hi - lo) * per_row; i += kThreads) {
      const int s = lo + i / per_row, rem = i % per_row;
      *reinterpret_cast<uint4*>(ob + (int64_t)s * a.o.ss + (int64_t)(rem / (HD / 8)) * a.o.sh + (rem % (HD / 8)) * 8) =
          make_uint4(0, 0, 0, 0);
    }
  }

  // ---- shared memory carve-up, barriers, TMEM ---------------------------------------------------
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (sbase - raw);
  const uint32_t sBar = sbase + kOffBar;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBar + kNumBars * 8);
  auto bar = [&](int i) { return sBar + (uint32_t)i * 8u; };

  bool failed = false;
  if (tid == 0) {
    for (int i = 0; i < kNumBars; ++i) {
      const bool many = (i >= kPFull && i < kPFull + 2) || (i >= kOFree && i < kOFree + 2);
      const bool rec_free = i >= kItemFree && i < kItemFree + kItemRing;
      ptx::mbar_init(bar(i), rec_free ? 9u : many ? 4u : 1u);  // one arrival per softmax warp (+ the MMA warp)
    }
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

  auto wait = [&](int i, uint32_t parity, int code) {
    if (failed) return;
    if (!ptx::mbar_wait(bar(i), parity & 1u, kWaitBudget)) {
      failed = true;
      if (a.status) atomicCAS(a.status, 0, code);
    }
  };

  int* const item_ring = reinterpret_cast<int*>(smem + kOffItems);
  const int TOK = BM >> a.g_shift;
  // consumer side of the item ring: copy record number i, release its slot
  auto next_item = [&](uint32_t i, int& flags) {
    const uint32_t slot = i % kItemRing;
    wait(kItemFull + slot, i / kItemRing, 40);
    Item it = read_record(item_ring + slot * 16, TOK, flags);
    if (__any_sync(0xffffffffu, failed)) flags |= kRecStop;  // a wait gave up: the whole warp stops here
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(bar(kItemFree + slot));
    return it;
  };

  if (warp == 8) {
    // =============================== TMA producer ===============================================
    // The whole warp runs the control flow (so addresses and counters stay warp-uniform); one lane
    // issues the copies.
    {
      const bool leader = lane == 0;
      uint32_t kv_cnt = 0, q_loads[2] = {0, 0}, n_pub = 0;
      // record number n_pub -> ring; its slot must have been copied by all nine consumers
      auto publish = [&](const Item& it, int flags) {
        const uint32_t slot = n_pub % kItemRing;
        if (n_pub >= kItemRing) wait(kItemFree + slot, n_pub / kItemRing - 1, 14);
        if (leader) {
          write_record(item_ring + slot * 16, it, flags);
          ptx::mbar_arrive(bar(kItemFull + slot));  // release: the record is visible to whoever sees the phase flip
        }
        ++n_pub;
      };
      // The work list (longest items first) is handed out dynamically: whichever CTA is free claims
      // the next index.  Claims run two items ahead and the block spans of a claimed item one item
      // ahead, so neither the atomic nor the loads are waited for.
      auto claim = [&]() {
        int v = 0;
        if (leader) v = atomicAdd(a.work_counter, 1);
        return __shfl_sync(0xffffffffu, v, 0);
      };
      int idx = claim(), idx_next = claim();
      ItemRaw raw_next = load_item(a, idx);
      Item it{};
      for (; idx < a.total_items; idx = idx_next, idx_next = claim()) {
        const ItemRaw raw = raw_next;
        raw_next = load_item(a, idx_next);  // in flight while this item is processed
        it = decode_item(a, raw);
        if (!it.valid) continue;
        int flags = it.split ? kRecSplit : 0;
        if (it.m == a.M - 1 && it.m > 0) {  // the query block's context may contain padding slots
          const int32_t* bl = a.blk_len + (size_t)it.b * a.M;
          int part = 0;
          for (int i = lane; i < a.M - 1; i += 32) part += bl[i];
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
          if (part != (it.ctx_hi - it.ctx_lo)) flags |= kRecCtxCheck;
        }
        publish(it, flags);
        for (int x = 0; x < 2; ++x) {
          if (it.n_x(x) == 0) continue;
          if (q_loads[x] > 0) wait(kQFree + x, q_loads[x] - 1, 10 + x);
          const uint32_t dst = sbase + kOffQ + (uint32_t)x * kQBytes;
          if (leader) {
            ptx::mbar_expect_tx(bar(kQFull + x), kQBytes);
            ptx::tma_load_4d(dst, &tmQ, bar(kQFull + x), 0, it.g * G, it.start + it.t0(x), it.b);
            ptx::tma_load_4d(dst + BM * 128, &tmQ, bar(kQFull + x), 64, it.g * G, it.start + it.t0(x), it.b);
          }
          ++q_loads[x];
        }
        for (int t = 0; 2 * t < it.n_tiles; ++t) {
          const uint32_t st = kv_cnt % kStages, use = kv_cnt / kStages;
          if (use > 0) wait(kKVFree + st, use - 1, 12);
          const uint32_t dst = sbase + kOffKV + st * kStageBytes;
          const int nslots = min(2, it.n_tiles - 2 * t);
          if (leader) {
            ptx::mbar_expect_tx(bar(kKVFull + st), (uint32_t)nslots * 2 * kSlotBytes);
            for (int h = 0; h < nslots; ++h) {
              int nk, own_off; bool own;
              const int lo = tile_lo(it, 2 * t + h, nk, own, own_off);
              const uint32_t row = dst + (uint32_t)h * (BN * 128);  // slot h = key rows [64h, 64h+64) of the tile
              ptx::tma_load_4d(row, &tmK, bar(kKVFull + st), 0, it.g, lo, it.b);
              ptx::tma_load_4d(row + BT * 128, &tmK, bar(kKVFull + st), 64, it.g, lo, it.b);
              ptx::tma_load_4d(row + kKBytes, &tmV, bar(kKVFull + st), 0, it.g, lo, it.b);
              ptx::tma_load_4d(row + kKBytes + BT * 128, &tmV, bar(kKVFull + st), 64, it.g, lo, it.b);
            }
          }
          ++kv_cnt;
        }
      }
      publish(it, kRecStop);  // end of this CTA's work list
    }
  } else if (warp == 9) {
    // =============================== MMA issuer =================================================
    // Whole-warp control flow, one issuing lane (always the same one: tcgen05.commit tracks the
    // MMAs of the thread that executes it).
    {
      const bool leader = lane == 0;
      uint32_t kv_cnt = 0, q_uses[2] = {0, 0}, p_seen[2] = {0, 0}, items_done[2] = {0, 0};
      // Descriptors are built once: every operand buffer has a fixed address, and stepping along K
      // or to another ring stage only adds a constant to the 16-byte-unit start-address field.
      const uint32_t idesc_pv = ptx::idesc_bf16(BM, HD, 0, 1);
      const uint32_t idesc_qk0 = ptx::idesc_bf16(BM, 0, 0, 0);
      const uint64_t q_desc0 = ptx::smem_desc_sw128(sbase + kOffQ, 16, 1024);
      const uint64_t k_desc0 = ptx::smem_desc_sw128(sbase + kOffKV, 16, 1024);
      const uint64_t v_desc0 = ptx::smem_desc_sw128(sbase + kOffKV + kKBytes, BT * 128, 1024);
      // keys of tile t that chain x (seeing n_vis slots) multiplies: full first slot + the valid part of the last one
      auto tile_keys = [&](const Item& it, int t, int n_vis) {
        const int cnt = min(2, n_vis - 2 * t);
        int nk, own_off; bool own;
        tile_lo(it, 2 * t + cnt - 1, nk, own, own_off);
        return (cnt - 1) * BN + nk;
      };
      auto issue_qk = [&](int x, int keys, bool last, uint32_t st) {
        const uint32_t idesc = idesc_qk0 | ((uint32_t)((keys + 15) >> 4) << 18);  // N/8 at bit 17, N a multiple of 16
        const uint32_t a_lo = (uint32_t)q_desc0 + (uint32_t)x * (kQBytes >> 4);
        const uint32_t b_lo = (uint32_t)k_desc0 + st * (kStageBytes >> 4);
        const uint32_t a_hi = (uint32_t)(q_desc0 >> 32), b_hi = (uint32_t)(k_desc0 >> 32);
        const uint32_t d = tmem + (uint32_t)x * kChainCols;
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t aoff = (uint32_t)(ks >> 2) * ((BM * 128) >> 4) + (uint32_t)(ks & 3) * 2;
            const uint32_t boff = (uint32_t)(ks >> 2) * ((BT * 128) >> 4) + (uint32_t)(ks & 3) * 2;
            ptx::mma_ss_lohi(d, a_lo + aoff, a_hi, b_lo + boff, b_hi, idesc, ks > 0);
          }
          ptx::mma_commit(bar(kSFull + x));
          if (last) ptx::mma_commit(bar(kQFree + x));  // last read of this chain's Q tile
        }
      };
      auto issue_pv = [&](int x, int keys, bool first, uint32_t st) {
        const uint32_t pa = tmem + (uint32_t)x * kChainCols;  // P sits over the first 64 columns of S
        const uint32_t b_lo = (uint32_t)v_desc0 + st * (kStageBytes >> 4), b_hi = (uint32_t)(v_desc0 >> 32);
        const uint32_t d = tmem + (uint32_t)x * kChainCols + kColO;
        const int ksteps = (keys + 15) >> 4;
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < BT / 16; ++ks)
            if (ks < ksteps)
              ptx::mma_ts_lohi(d, pa + (uint32_t)ks * 8, b_lo + (uint32_t)ks * ((16 * 128) >> 4), b_hi, idesc_pv, (!first || ks > 0) ? 1u : 0u);
          ptx::mma_commit(bar(kPVDone + x));
        }
      };
      for (uint32_t item_no = 0;; ++item_no) {
        int flags;
        const Item it = next_item(item_no, flags);
        if (flags & kRecStop) break;
        const int n0 = it.n_0, n1 = it.n_1;
        const int T0 = (n0 + 1) >> 1, T1 = (n1 + 1) >> 1, T = (it.n_tiles + 1) >> 1;
        // Every tile but a chain's last spans 128 keys (a short context slot inside a tile is masked by
        // the softmax, not trimmed); the last one is computed once here, off the per-tile path.
        const int last_keys0 = T0 > 0 ? tile_keys(it, T0 - 1, n0) : 0, last_keys1 = T1 > 0 ? tile_keys(it, T1 - 1, n1) : 0;
        auto keys_of = [&](int x, int t) { return t + 1 < (x == 0 ? T0 : T1) ? BT : (x == 0 ? last_keys0 : last_keys1); };
#pragma unroll
        for (int x = 0; x < 2; ++x)
          if ((x == 0 ? n0 : n1) > 0) { wait(kQFull + x, q_uses[x], 20 + x); ++q_uses[x]; }
        int kv_waited = -1;
        auto need_kv = [&](int t) {
          if (kv_waited >= t) return;
          const uint32_t gidx = kv_cnt + (uint32_t)t;
          wait(kKVFull + gidx % kStages, gidx / kStages, 22);
          kv_waited = t;
        };
        need_kv(0);
        ptx::tc_fence_after_sync();
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int Tx = x == 0 ? T0 : T1;
          if (Tx > 0) issue_qk(x, keys_of(x, 0), Tx == 1, kv_cnt % kStages);
        }
        for (int t = 0; t < T; ++t) {
          const uint32_t st = (kv_cnt + (uint32_t)t) % kStages;
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int Tx = x == 0 ? T0 : T1;
            if (t >= Tx) continue;
            wait(kPFull + x, p_seen[x], 24 + x);
            ++p_seen[x];
            if (t == 0 && items_done[x] > 0) wait(kOFree + x, items_done[x] - 1, 26 + x);
            ptx::tc_fence_after_sync();
            issue_pv(x, keys_of(x, t), t == 0, st);
            if (t + 1 < Tx) {
              // the chain's next S tile: queued behind the P V that reads P out of the same columns
              need_kv(t + 1);
              ptx::tc_fence_after_sync();
              issue_qk(x, keys_of(x, t + 1), t + 2 == Tx, (kv_cnt + (uint32_t)t + 1) % kStages);
            }
          }
          if (leader) ptx::mma_commit(bar(kKVFree + st));  // both chains' MMAs on this stage are queued
        }
        kv_cnt += (uint32_t)T;
#pragma unroll
        for (int x = 0; x < 2; ++x)
          if ((x == 0 ? n0 : n1) > 0) ++items_done[x];
      }
    }
  } else {
    // =============================== softmax + output, chain x ==================================
    const int x = warp >> 2;
    const int r = tid & 127;  // row of the tile = TMEM lane
    const uint32_t tmem_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)x * kChainCols;
    uint32_t s_seen = 0, pv_seen = 0;

    for (uint32_t item_no = 0;; ++item_no) {
      int flags;
      const Item it = next_item(item_no, flags);
      if (flags & kRecStop) break;
      if (it.n_x(x) == 0) continue;
      const int32_t* bs = a.blk_start + (size_t)it.b * a.M;
      const int32_t* bl = a.blk_len + (size_t)it.b * a.M;
      const int tok = it.t0(x) + (r >> a.g_shift);
      const int n = it.g * G + (r & (G - 1));
      const bool active = tok < it.len;
      const bool ctx_check = (flags & kRecCtxCheck) != 0;  // the query block's context contains padding slots
      float m_run = -INFINITY, l_run = 0.f;
      const int n_mine = it.n_x(x);
      const int t_mine = (n_mine + 1) >> 1;

      for (int t = 0; t < t_mine; ++t) {
        const int cnt = min(2, n_mine - 2 * t);  // slots of this tile the chain sees
        wait(kSFull + x, s_seen, 30 + x);
        ++s_seen;
        ptx::tc_fence_after_sync();
        __syncwarp();
        // One pass per 64-key slot: logits -> registers, mask, row maximum, running-max update,
        // p = 2^(s*scale - m) from the same registers, P (bf16) -> columns [32h, 32h+32) of the
        // tile, which only covers logits that have already been consumed.
#pragma unroll 1
        for (int h = 0; h < cnt; ++h) {
          int nk, own_off; bool own;
          const int lo = tile_lo(it, 2 * t + h, nk, own, own_off);
          uint32_t sr[64];
          {
            uint32_t (&lo32)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sr[0]);
            uint32_t (&hi32)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sr[32]);
            ptx::tmem_ld32(tmem_lane + (uint32_t)h * BN, lo32);
            ptx::tmem_ld32(tmem_lane + (uint32_t)h * BN + 32, hi32);
            ptx::tmem_wait_ld(sr);
          }
          // Visibility.  Slots fully inside the visible region need no masking (the common case).
          // Ragged tails and the causal diagonal make columns [0, lim) of a row visible; the
          // 8-column groups below the warp's smallest lim need no masking either, the groups at or
          // above its largest lim are skipped altogether (their P is zero), and only the groups in
          // between are masked element by element.  Padded context ranges (reference layout with
          // gaps between blocks) take the general per-element path.
          int lim = BN, lim_lo = BN, lim_hi = BN;
          if (nk < BN || (own && own_off + BN - 1 > it.t0(x)) || (!own && ctx_check)) {
            lim = nk;
            if (own) lim = max(0, min(nk, tok - own_off + 1));
            if (!own && ctx_check) {
              const unsigned v0 = __ballot_sync(0xffffffffu, slot_valid(bs, bl, a.M, lo + lane));
              const unsigned v1 = __ballot_sync(0xffffffffu, slot_valid(bs, bl, a.M, lo + 32 + lane));
#pragma unroll
              for (int c = 0; c < 64; ++c) {
                const bool ok = c < lim && (((c < 32 ? v0 : v1) >> (c & 31)) & 1u);
                sr[c] = ok ? sr[c] : 0xff800000u;  // -inf
              }
            } else {
              lim_lo = __reduce_min_sync(0xffffffffu, lim);
              lim_hi = __reduce_max_sync(0xffffffffu, lim);
            }
          }
          // The slot is processed by one of two instantiations: straight-line code when nothing is
          // masked per group (one basic block: exponentials, polynomial and conversions interleave
          // freely), or the grouped form with warp-uniform branches around every 8 columns.
          auto process = [&](auto grouped_tag) {
            constexpr bool kGrouped = decltype(grouped_tag)::value;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // independent chains
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 8) {
              if (!kGrouped || c0 < lim_hi) {
                if (kGrouped && c0 + 8 > lim_lo) {
#pragma unroll
                  for (int c = c0; c < c0 + 8; ++c) sr[c] = c < lim ? sr[c] : 0xff800000u;  // -inf
                }
#pragma unroll
                for (int c = c0; c < c0 + 8; c += 2)
                  mx4[(c >> 1) & 3] = ptx::max3(mx4[(c >> 1) & 3], __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
              }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;  // scale > 0
            float m_new = fmaxf(m_run, mx);
            if (m_run != -INFINITY && m_new - m_run <= kLazy) m_new = m_run;  // keep the old reference: p <= 2^8
            const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ptx::ex2(m_run - m_ref);  // 1 when unchanged, 0 on the first visible slot
            const float neg_ref = -m_ref;
            const bool changed = m_new != m_run;
            m_run = m_new;

            if (h == 0 && t > 0) {
              // previous P V done: O is stable and the P columns (first half of S) may be overwritten
              wait(kPVDone + x, pv_seen, 32 + x);
              ++pv_seen;
              ptx::tc_fence_after_sync();
            }
            if ((t > 0 || h > 0) && __any_sync(0xffffffffu, changed)) {
              // The reference moved by more than the lazy threshold (rare): bring what was accumulated
              // against the old one in line -- O of the earlier tiles, P of this tile's first slot.
              if (t > 0) {
#pragma unroll 1
                for (int ch = 0; ch < HD / 32; ++ch) {
                  uint32_t orow[32];
                  ptx::tmem_ld32(tmem_lane + kColO + (uint32_t)ch * 32, orow);
                  ptx::tmem_wait_ld(orow);
#pragma unroll
                  for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
                  ptx::tmem_st32(tmem_lane + kColO + (uint32_t)ch * 32, orow);
                }
              }
              if (h > 0) {
                uint32_t p0[32];
                ptx::tmem_ld32(tmem_lane, p0);
                ptx::tmem_wait_ld(p0);
                const __nv_bfloat162 c2 = __float2bfloat162_rn(corr);  // corr is 1 or at most 2^-8: exact enough in bf16
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&p0[i]), c2);
                  p0[i] = *reinterpret_cast<uint32_t*>(&v);
                }
                ptx::tmem_st32(tmem_lane, p0);
              }
              ptx::tmem_wait_st();
            }
            // p with packed fp32x2 arithmetic.  Every second pair of exponentials is evaluated on the
            // FMA pipe: the special-function unit (16 results per clock per SM) would otherwise bound
            // the whole kernel.
            const ptx::f32x2 sc2 = ptx::pack2(a.scale_log2, a.scale_log2), nr2 = ptx::pack2(neg_ref, neg_ref);
            ptx::f32x2 ps2[2] = {0ull, 0ull};
            uint32_t pk[32];
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 8) {
              if (!kGrouped || c0 < lim_hi) {
#pragma unroll
                for (int c = c0; c < c0 + 8; c += 4) {
                  const ptx::f32x2 t01 = ptx::fma2(ptx::pack2(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), sc2, nr2);
                  const ptx::f32x2 t23 = ptx::fma2(ptx::pack2(__uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3])), sc2, nr2);
                  float t0, t1, p2, p3;
                  ptx::unpack2(t01, t0, t1);
                  const float p0 = ptx::ex2(t0), p1 = ptx::ex2(t1);
                  const ptx::f32x2 p23 = ptx::ex2_poly2(t23);
                  ptx::unpack2(p23, p2, p3);
                  ps2[0] = ptx::add2(ps2[0], ptx::pack2(p0, p1));
                  ps2[1] = ptx::add2(ps2[1], p23);
                  __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
                  pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h0);
                  pk[(c >> 1) + 1] = *reinterpret_cast<uint32_t*>(&h1);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) pk[(c0 >> 1) + i] = 0u;
              }
            }
            ptx::tmem_st32(tmem_lane + (uint32_t)h * 32, pk);
            float s0, s1, s2, s3;
            ptx::unpack2(ps2[0], s0, s1);
            ptx::unpack2(ps2[1], s2, s3);
            l_run = l_run * corr + ((s0 + s1) + (s2 + s3));
          };
          if (lim_hi == BN && lim_lo == BN) process(std::false_type{}); else process(std::true_type{});
        }
        ptx::tmem_wait_st();
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar(kPFull + x));
      }

      // ---- output of the item ----
      wait(kPVDone + x, pv_seen, 34 + x);  // last P V of the item
      ++pv_seen;
      ptx::tc_fence_after_sync();
      __syncwarp();
      // O leaves tensor memory in four 32-column chunks, software-pipelined: the load of the next
      // chunk is in flight while the current one is converted and stored.
      uint32_t obuf[2][32];
      ptx::tmem_ld32(tmem_lane + kColO, obuf[0]);
      if (it.split) {
        // un-normalised partial (O, max, sum) of this key chunk; merged by attn_combine_kernel
        const bool wr = active && tok < a.lq_max;
        const int64_t prow = (((int64_t)it.b * a.N + n) * a.lq_max + tok) * a.n_split + it.chunk;
#pragma unroll
        for (int ch = 0; ch < HD / 32; ++ch) {
          uint32_t (&orow)[32] = obuf[ch & 1];
          ptx::tmem_wait_ld(orow);
          if (ch + 1 < HD / 32) {
            ptx::tmem_ld32(tmem_lane + kColO + (uint32_t)(ch + 1) * 32, obuf[(ch + 1) & 1]);
          } else {  // O is out of TMEM: the next item's first P V may overwrite it
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(kOFree + x));
          }
          if (wr) {
            float4* dst = reinterpret_cast<float4*>(a.part_o + prow * HD + ch * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(orow[4 * i]), __uint_as_float(orow[4 * i + 1]),
                                   __uint_as_float(orow[4 * i + 2]), __uint_as_float(orow[4 * i + 3]));
          }
        }
        if (wr) a.part_ml[prow] = make_float2(m_run, l_run);
      } else {
        // O / l -> bf16, stored straight from registers: each thread owns one 256-byte output row
        // and writes it as eight 32-byte (full-sector) stores, or sixteen 16-byte ones if the
        // output is only 16-byte aligned.
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* out_row = reinterpret_cast<__nv_bfloat16*>(a.o.ptr) + (int64_t)it.b * a.o.sb +
                                 (int64_t)(it.start + tok) * a.o.ss + (int64_t)n * a.o.sh;
#pragma unroll
        for (int ch = 0; ch < HD / 32; ++ch) {
          uint32_t (&orow)[32] = obuf[ch & 1];
          ptx::tmem_wait_ld(orow);
          if (ch + 1 < HD / 32) {
            ptx::tmem_ld32(tmem_lane + kColO + (uint32_t)(ch + 1) * 32, obuf[(ch + 1) & 1]);
          } else {  // O is out of TMEM: the next item's first P V may overwrite it
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(kOFree + x));
          }
          if (active) {
#pragma unroll
            for (int q8 = 0; q8 < 2; ++q8) {
              uint32_t w[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(orow[q8 * 16 + 2 * i]) * inv,
                                                          __uint_as_float(orow[q8 * 16 + 2 * i + 1]) * inv);
                w[i] = *reinterpret_cast<uint32_t*>(&hh);
              }
              __nv_bfloat16* dst = out_row + ch * 32 + q8 * 16;
              if (a.o_align32) {
                ptx::st_global_v8(dst, w);
              } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
              }
            }
          }
        }
        if (active && a.lse != nullptr)
          a.lse[((int64_t)it.b * a.N + n) * a.S + it.start + tok] = (m_run + log2f(l_run)) * 0.6931471805599453f;
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------------
  ptx::tc_fence_before_sync();
  __syncthreads();
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

// neutral partials for chunks that own no tile (the combine step skips sum == 0)
__global__ void attn_clear_partials_kernel(float2* ml, int64_t n, int* work_counter) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *work_counter = 0;
  if (i < n) ml[i] = make_float2(-INFINITY, 0.f);
}

}  // namespace

// Key chunks for the query block.  Its context is every earlier token of the prompt (S is the only
// bound known on the host), walked 64 keys per step per row tile; cutting it into chunks of about
// 1024 keys keeps that serial chain short and spreads it over the SMs.
constexpr size_t kWsHeader = 256;  // workspace: [work counter, padding][partial O][partial (max, sum)]

static int tc_splits(const brk_attn_params& p) {
  if (p.M < 2) return 1;
  int n = (p.S + 1023) / 1024;
  return n < 1 ? 1 : (n > 32 ? 32 : n);
}

size_t attn_tc_workspace(const brk_attn_params& p) {
  const int ns = tc_splits(p);
  if (ns <= 1) return kWsHeader;  // the work counter
  const size_t rows = (size_t)p.B * p.N * p.max_block_len * ns;
  return kWsHeader + rows * HD * sizeof(float) + rows * sizeof(float2);
}

int attn_tc_launch(const brk_attn_params& p, void* ws, size_t ws_bytes, cudaStream_t st) {
  BRK_REQUIRE(p.dtype == BRK_BF16 && p.D == HD, BRK_E_UNSUPPORTED,
              "tcgen05 attention needs bf16 and head_dim 128 (dtype %d, head_dim %d)", p.dtype, p.D);
  const int G = p.N / p.Nk;
  BRK_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8, BRK_E_UNSUPPORTED, "tcgen05 attention needs N/Nk in {1,2,4,8}, got %d", G);
  BRK_REQUIRE(p.scale > 0.f, BRK_E_ARG, "softmax scale must be positive");
  const int ns = tc_splits(p);
  const size_t need = attn_tc_workspace(p);
  BRK_REQUIRE(ws != nullptr && ws_bytes >= need && ((uintptr_t)ws & 15) == 0, BRK_E_WORKSPACE,
              "attention workspace: %zu bytes (16-byte aligned) needed, %zu given", need, ws_bytes);
  int gs = 0;
  while ((1 << gs) < G) ++gs;
  const int TOK = BM / G;
  const int pairs = (p.max_block_len + 2 * TOK - 1) / (2 * TOK);
  const int64_t total_items = (int64_t)p.B * p.Nk * pairs * (ns + p.M - 1);
  BRK_REQUIRE(total_items < (1ll << 30), BRK_E_UNSUPPORTED, "too many work items (%lld)", (long long)total_items);
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_bf16(&tq, p.q.ptr, HD, p.N, p.S, p.B, p.q.stride_h, p.q.stride_s, p.q.stride_b, G, TOK))) return rc;
  if ((rc = make_tmap_bf16(&tk, p.k.ptr, HD, p.Nk, p.S, p.B, p.k.stride_h, p.k.stride_s, p.k.stride_b, 1, BN))) return rc;
  if ((rc = make_tmap_bf16(&tv, p.v.ptr, HD, p.Nk, p.S, p.B, p.v.stride_h, p.v.stride_s, p.v.stride_b, 1, BN))) return rc;
  static bool configured[64] = {};
  static int sms[64] = {};
  int dev = 0;
  BRK_CUDA(cudaGetDevice(&dev));
  BRK_REQUIRE(dev >= 0 && dev < 64, BRK_E_UNSUPPORTED, "device ordinal %d out of range", dev);
  if (!configured[dev]) {
    BRK_CUDA(cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    sms[dev] = sm_count();
    BRK_REQUIRE(sms[dev] > 0, BRK_E_CUDA, "could not read the SM count");
    configured[dev] = true;
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
  a.pairs = pairs;
  a.o_align32 = (((uintptr_t)p.o.ptr & 31) == 0 && p.o.stride_b % 16 == 0 && p.o.stride_h % 16 == 0 && p.o.stride_s % 16 == 0) ? 1 : 0;
  a.total_items = (int)total_items;
  a.div_sec1 = make_fastdiv((uint32_t)(p.B * p.Nk * ns));
  a.div_nbg = make_fastdiv((uint32_t)(p.B * p.Nk));
  a.div_sec2 = make_fastdiv((uint32_t)(p.B * p.Nk * (p.M > 1 ? p.M - 1 : 1)));
  a.div_nk = make_fastdiv((uint32_t)p.Nk);
  const size_t rows = (size_t)p.B * p.N * p.max_block_len * ns;
  float* const part = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + kWsHeader);
  a.work_counter = reinterpret_cast<int*>(ws);
  a.part_o = ns > 1 ? part : nullptr;
  a.part_ml = ns > 1 ? reinterpret_cast<float2*>(part + rows * HD) : nullptr;
  {
    const int64_t n_clear = ns > 1 ? (int64_t)rows : 0;  // always launched: it also resets the work counter
    attn_clear_partials_kernel<<<(unsigned)(n_clear > 0 ? (n_clear + 255) / 256 : 1), 256, 0, st>>>(a.part_ml, n_clear, a.work_counter);
    BRK_CUDA(cudaGetLastError());
  }
  const int grid = (int)(total_items < sms[dev] ? total_items : sms[dev]);
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
