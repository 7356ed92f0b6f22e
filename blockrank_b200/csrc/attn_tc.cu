// BlockRank attention forward on the sm_100a tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Persistent, warp-specialised kernel: one CTA per SM; the CTAs claim work items from a global
// counter.  Two independent "chains" run in every CTA.  A chain owns one 128-row tile at a time
// (128/G consecutive query tokens x the G query heads that share a KV head, so one K/V tile
// serves the whole GQA group and a Q tile is one 3-D TMA box of the [B,S,N,D] tensor), a
// 256-column half of tensor memory (S 128 columns, O 128 columns), a Q buffer, four softmax
// warps and its own MMA-issuing warp.  Chains are fed with "jobs" (one row tile against a list
// of 64-key slots) through per-chain record rings and never wait for one another, so one
// chain's MMAs run while the other chain's softmax threads work.
//
// Only live keys are visited:
//   block 0            : own keys, causal
//   document block     : the prefix block's keys, then own keys, causal
//   query (last) block : every slot of the earlier blocks, then own keys, causal
//
// Two kinds of work item:
//   * resident block  (blocks 0 .. M-2 whose prefix + own keys fit the five 64-key slots of
//     shared memory): the block's K/V is loaded ONCE, its row tiles are dealt to the two chains
//     largest first, and every slot is handed back as soon as the remaining (smaller) row tiles
//     of both chains no longer need it, so the next block's loads overlap the tail of this one.
//   * streamed pair   (the query block, cut into chunks of about 1024 context keys that leave
//     un-normalised partials (O, max, sum) merged by attn_combine_kernel; also any block too
//     long to be resident): the two chains take the two row tiles of a pair and walk the same
//     128-key tiles through a two-deep ring.
//
// Roles (352 threads):
//   warps 0-3 / 4-7  softmax + output of chain 0 / 1 (thread = row = TMEM lane)
//   warp 8           TMA producer: claims and decodes items, publishes jobs, loads K/V
//   warps 9 / 10     MMA issuer of chain 0 / 1: S = Q K^T (both operands K-major, 128B swizzle)
//                    and O += P V (P read from tensor memory, V as the MN-major B operand); it also
//                    requests its chain's Q tiles by TMA (it knows when the Q buffer is free)
// Softmax is base-2, online, with a lazy rescale (O is only touched when the running max grows
// by more than 2^8).  P (bf16, two keys per 32-bit column) overwrites the first half of the S
// tile it was computed from.
//
// Shared memory 226 KB: Q 2x32 KB, K pool 80 KB, V pool 80 KB, barriers, job records.
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
constexpr int kSlots = 5;        // 64-key K/V slots in shared memory
constexpr int kMaxGroup = 4;  // consecutive blocks of one (prompt, KV head) per work item, at most
constexpr int kThreads = 352;
constexpr uint32_t kQBytes = 2 * BM * 128;       // one Q tile: two 64-wide halves of D
constexpr uint32_t kSlotHalf = BN * 128;         // K (or V) of one slot, one 64-wide half of D
constexpr uint32_t kPoolHalf = kSlots * kSlotHalf;  // all slots of one half of D, contiguous: key k at k * 128 B
constexpr uint32_t kSlotBytes = 4 * kSlotHalf;   // K + V of one slot
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + 2 * kQBytes;
constexpr uint32_t kOffV = kOffK + 2 * kPoolHalf;
constexpr uint32_t kOffBar = kOffV + 2 * kPoolHalf;
constexpr int kJobRing = 4;                      // published jobs in flight per chain
constexpr uint32_t kOffJobs = kOffBar + 512;     // 2 x kJobRing records of 16 ints
constexpr uint32_t kSmemBytes = kOffJobs + 2 * kJobRing * 64 + 1024;  // + slack for the 1024-byte round-up
static_assert(kSmemBytes <= 232448, "shared memory per CTA");
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kChainCols = 256;  // per chain: S [0,128) (P over its first 64 columns), then O [128,256)
constexpr uint32_t kColO = 128;
constexpr float kLazy = 8.f;
// Exponentials per 8 evaluated as a Cody-Waite polynomial on the FMA pipe instead of the special-function unit:
// 0, 2 or 4.  Measured on the 100-document workload (4 prompts per launch): 0 -> 0.58 ms, 4 -> 0.64 ms; the
// softmax warps are bound by instruction issue, not by the special-function unit, so the default is 0.
#ifndef BRK_POLY_OF_8
#define BRK_POLY_OF_8 0
#endif
constexpr int kPolyOf8 = BRK_POLY_OF_8;
constexpr uint32_t kWaitBudget = 1u << 18;
constexpr int kTileFixedCost = 136;  // cost of a row tile beyond its keys (output drain), in keys

enum {
  kQFull = 0,    // +chain  TMA -> MMA: Q tile landed
  kQFree = 2,    // +chain  MMA -> TMA: every QK^T of the job has read Q
  kSFull = 4,    // +chain  MMA -> softmax: S tile complete
  kPFull = 6,    // +chain  softmax -> MMA: P written to tensor memory, S consumed (4 warp arrivals)
  kPVDone = 8,   // +chain  MMA -> softmax: P V of a tile complete
  kOFree = 10,   // +chain  softmax -> MMA: O read out of TMEM (4 warp arrivals)
  kKVFull = 12,              // +slot  TMA -> MMA warps: K and V of the slot (or of the tile that starts there) landed
  kKVFree = kKVFull + kSlots,  // +slot  both MMA warps -> TMA: no MMA still reads the slot (2 arrivals)
  kJobFull = kKVFree + kSlots,            // +chain*kJobRing+i  TMA warp -> MMA warp, softmax warps: record written
  kJobFree = kJobFull + 2 * kJobRing,     // +chain*kJobRing+i  MMA warp + 4 softmax warps -> TMA warp (5 arrivals)
  kNumBars = kJobFree + 2 * kJobRing
};
static_assert(kNumBars * 8 + 8 <= 512, "barrier area");  // + the TMEM base address

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
  const int* hdr;   // workspace header: [0] work counter, [1] non-zero if the block spans are malformed
  int B, N, Nk, S, M;
  int G, g_shift;   // query heads per KV head, log2
  float scale_log2;
  int n_split;      // key chunks of the query block's context (1 = no split)
  int lq_max;       // rows per (prompt, head) in the partial buffers (bound on the query block's length)
  int pairs_q;      // row-tile pairs of the query block (covers lq_max)
  int group;        // consecutive blocks 0 .. M-2 of one (prompt, KV head) per work item (their prefix stays resident)
  int n_groups;     // such groups per (prompt, KV head)
  int o_align32;    // output rows are 32-byte aligned (enables 32-byte stores)
  int sec1, total_items;
  FastDiv div_sec1, div_nbg, div_nk;  // by nbg*n_split, nbg, Nk
  int* work_counter;  // next unclaimed index of the work list (zeroed before the launch)
  float* part_o;    // [B, N, lq_max, n_split, 128] un-normalised partial outputs
  float2* part_ml;  // [B, N, lq_max, n_split] (running max in log2 units, sum)
};

// One row tile against a list of 64-key slots: what a chain works on.
constexpr int kFSplit = 1, kFCtxCheck = 2, kFStop = 4, kFDoc = 8, kFFirst = 16, kFKeep = 32;
struct Job {
  int b, g, m, chunk;
  int start, len;        // span of block m
  int t0;                // first token of the row tile
  int n;                 // key slots visible to this row tile (0: nothing to compute, only slots to hand back)
  int ctx_lo, ctx_hi;    // context key range (token slots of the prompt)
  int n_ctx, j0;         // context slots of the block, first slot of this job's list
  int own_n;             // own keys covered by the slot list
  int flags;
  int tile0;             // streamed: ring position (0/1) of the job's first 128-key tile
  int aux;               // streamed: tiles of the item; resident: rel_lo | rel_hi << 8 (slots handed back after the job)
};

// slot j of the job's list -> first key (token slot of the prompt), number of keys, whether it lies in the own block
__device__ __forceinline__ int tile_lo(const Job& it, int j, int& nk, bool& own, int& own_off) {
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

__device__ __forceinline__ void write_record(int* rec, const Job& it) {
  reinterpret_cast<int4*>(rec)[0] = make_int4(it.b, it.g, it.m, it.chunk);
  reinterpret_cast<int4*>(rec)[1] = make_int4(it.start, it.len, it.t0, it.n);
  reinterpret_cast<int4*>(rec)[2] = make_int4(it.ctx_lo, it.ctx_hi, it.n_ctx, it.j0);
  reinterpret_cast<int4*>(rec)[3] = make_int4(it.own_n, it.flags, it.tile0, it.aux);
}
__device__ __forceinline__ Job read_record(const int* rec) {
  const int4 r0 = reinterpret_cast<const int4*>(rec)[0], r1 = reinterpret_cast<const int4*>(rec)[1];
  const int4 r2 = reinterpret_cast<const int4*>(rec)[2], r3 = reinterpret_cast<const int4*>(rec)[3];
  Job it;
  it.b = r0.x; it.g = r0.y; it.m = r0.z; it.chunk = r0.w;
  it.start = r1.x; it.len = r1.y; it.t0 = r1.z; it.n = r1.w;
  it.ctx_lo = r2.x; it.ctx_hi = r2.y; it.n_ctx = r2.z; it.j0 = r2.w;
  it.own_n = r3.x; it.flags = r3.y; it.tile0 = r3.z; it.aux = r3.w;
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

// A claimed work item before decoding: the spans it needs are fetched one item ahead of their use.
//   kind 0: streamed pair p, key chunk `chunk`, of the query block (m = M-1)
//   kind 1: blocks [m, m + cnt) of (b, g); lane i of the warp holds the span of block m + i
struct ItemRaw {
  int kind, p, chunk, b, g, m, cnt;
  int start, len;      // span of block m + lane (kind 1) or of the query block (kind 0)
  int s0, l0;          // span of block 0 (the prefix)
  int s2, l2;          // span of block M-2 (end of the query block's context)
};

// Work list: streamed pairs of the query block first (the longest items), then the groups of blocks 0 .. M-2.
__device__ __forceinline__ ItemRaw load_item(const TcArgs& a, int idx, int lane) {
  ItemRaw r;
  if (idx >= a.total_items) idx = a.total_items - 1;  // prefetch past the end: harmless reload
  const int nbg = a.B * a.Nk;
  int bg;
  if (idx < a.sec1) {
    r.kind = 0;
    r.p = (int)fdiv((uint32_t)idx, a.div_sec1);
    const int q = idx - r.p * (nbg * a.n_split);
    r.chunk = (int)fdiv((uint32_t)q, a.div_nbg);
    bg = q - r.chunk * nbg;
    r.m = a.M - 1;
    r.cnt = 1;
  } else {
    r.kind = 1;
    const int i2 = idx - a.sec1;
    const int grp = (int)fdiv((uint32_t)i2, a.div_nbg);
    bg = i2 - grp * nbg;
    r.m = grp * a.group;
    r.cnt = min(a.group, a.M - 1 - r.m);
    r.p = r.chunk = 0;
  }
  r.b = (int)fdiv((uint32_t)bg, a.div_nk);
  r.g = bg - r.b * a.Nk;
  const int32_t* bs = a.blk_start + (size_t)r.b * a.M;
  const int32_t* bl = a.blk_len + (size_t)r.b * a.M;
  const int m2 = a.M >= 2 ? a.M - 2 : 0;
  const int mm = min(r.m + (r.kind ? lane : 0), a.M - 1);
  r.start = bs[mm];
  r.len = bl[mm];
  r.s0 = bs[0];
  r.l0 = bl[0];
  r.s2 = bs[m2];
  r.l2 = bl[m2];
  return r;
}

// A streamed pair: the two row tiles [2p, 2p+1] of block m against the block's slot list (or one key chunk of it).
struct Pair {
  Job job;         // fields common to both chains
  int t0_0, t0_1;  // first token of each chain's row tile
  int n_0, n_1;    // slots visible to each chain (a prefix of the item's slot list)
  int n_slots;     // slots of the item
  bool valid;
};

__device__ __forceinline__ Pair decode_pair(const TcArgs& a, int b, int g, int m, int chunk, int p, int start, int len,
                                            int s0, int l0, int s2, int l2) {
  Pair pr;
  Job& it = pr.job;
  const int TOK = BM >> a.g_shift;
  it.b = b; it.g = g; it.m = m; it.chunk = chunk;
  it.start = start;
  it.len = len;
  pr.t0_0 = 2 * p * TOK;
  pr.t0_1 = pr.t0_0 + TOK;
  pr.valid = pr.t0_0 < len;
  const bool split = m == a.M - 1 && a.n_split > 1;
  it.flags = split ? kFSplit : 0;
  it.ctx_lo = it.ctx_hi = 0;
  it.n_ctx = it.j0 = it.own_n = 0;
  it.t0 = it.n = it.tile0 = it.aux = 0;
  pr.n_0 = pr.n_1 = pr.n_slots = 0;
  if (!pr.valid) return pr;
  if (m > 0) {
    it.ctx_lo = s0;
    it.ctx_hi = (m < a.M - 1) ? s0 + l0 : s2 + l2;
  }
  const bool on1 = pr.t0_1 < len;
  it.own_n = min(len, (on1 ? pr.t0_1 : pr.t0_0) + TOK);
  it.n_ctx = (it.ctx_hi - it.ctx_lo + BN - 1) / BN;
  const int own_slots = (it.own_n + BN - 1) / BN;
  int j1 = it.n_ctx + own_slots;
  if (split) {
    const int per = (it.n_ctx + a.n_split - 1) / a.n_split;
    it.j0 = min(it.n_ctx, chunk * per);
    if (chunk != a.n_split - 1) j1 = min(it.n_ctx, it.j0 + per);
  }
  pr.n_slots = j1 - it.j0;
  if (pr.n_slots <= 0) {  // a chunk without slots: nothing to do (its partial stays neutral)
    pr.valid = false;
    pr.n_slots = 0;
    return pr;
  }
  // own slots visible to chain x: those starting at or before its last token
  {
    const int own_x = min(own_slots, (min(len, pr.t0_0 + TOK) + BN - 1) / BN);
    pr.n_0 = max(0, min(j1, it.n_ctx + own_x) - it.j0);
  }
  if (on1) {
    const int own_x = min(own_slots, (min(len, pr.t0_1 + TOK) + BN - 1) / BN);
    pr.n_1 = max(0, min(j1, it.n_ctx + own_x) - it.j0);
  }
  return pr;
}

// chain of the i-th largest row tile of a resident block when there are too many tiles to try every split
// (tiles are dealt 0,1,1,0,0,1,1,0,...)
__device__ __forceinline__ int deal_chain(int i) { return ((i & 3) == 0 || (i & 3) == 3) ? 0 : 1; }

__global__ void __launch_bounds__(kThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const TcArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (a.hdr[1] != 0) return;  // malformed block spans (found by the prologue kernel): write nothing
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = a.G;

  // ---- padding slots of the output are written as zeros (gaps in front of / behind blocks) ----
  {
    const int per_row = a.N * (HD / 8);
    auto zero_rows = [&](int b, int lo, int hi) {
      __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(a.o.ptr) + (int64_t)b * a.o.sb;
      for (int i = tid; i < (hi - lo) * per_row; i += kThreads) {
        const int s = lo + i / per_row, rem = i % per_row;
        *reinterpret_cast<uint4*>(ob + (int64_t)s * a.o.ss + (int64_t)(rem / (HD / 8)) * a.o.sh + (rem % (HD / 8)) * 8) =
            make_uint4(0, 0, 0, 0);
      }
    };
    // the gap in front of a block (at most a block's padding): one CTA each
    for (int gi = blockIdx.x; gi < a.B * a.M; gi += gridDim.x) {
      const int b = gi / a.M, m = gi % a.M;
      const int32_t* bs = a.blk_start + (size_t)b * a.M;
      const int32_t* bl = a.blk_len + (size_t)b * a.M;
      zero_rows(b, (m == 0) ? 0 : bs[m - 1] + bl[m - 1], bs[m]);
    }
    // The gap behind the last block holds thousands of rows when a batch is padded to its longest prompt (one
    // CTA writing all of it took longer than the rest of the kernel): every CTA takes a slice of it.
    for (int b = 0; b < a.B; ++b) {
      const int lo = a.blk_start[(size_t)b * a.M + a.M - 1] + a.blk_len[(size_t)b * a.M + a.M - 1];
      const int rows = a.S - lo;
      if (rows <= 0) continue;
      const int per = (rows + (int)gridDim.x - 1) / (int)gridDim.x;
      const int slot = (int)((blockIdx.x + (unsigned)b) % gridDim.x);
      zero_rows(b, lo + min(rows, slot * per), lo + min(rows, (slot + 1) * per));
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
      uint32_t cnt = 1u;
      if ((i >= kPFull && i < kPFull + 2) || (i >= kOFree && i < kOFree + 2)) cnt = 4u;  // one arrival per softmax warp
      if (i >= kKVFree && i < kKVFree + kSlots) cnt = 2u;                                 // one per MMA warp
      if (i >= kJobFree) cnt = 5u;                                                        // MMA warp + four softmax warps
      ptx::mbar_init(bar(i), cnt);
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

  int* const job_ring = reinterpret_cast<int*>(smem + kOffJobs);
  const int TOK = BM >> a.g_shift;
  // consumer side of chain x's job ring: copy record number i, release its slot
  auto next_job = [&](int x, uint32_t i) {
    const uint32_t slot = i % kJobRing;
    wait(kJobFull + x * kJobRing + slot, i / kJobRing, 40 + x);
    Job it = read_record(job_ring + (x * kJobRing + slot) * 16);
    if (__any_sync(0xffffffffu, failed)) it.flags |= kFStop;  // a wait gave up: the whole warp stops here
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(bar(kJobFree + x * kJobRing + slot));
    return it;
  };

  if (warp == 8) {
    // =============================== TMA producer ===============================================
    // The whole warp runs the control flow (so addresses and counters stay warp-uniform); one lane
    // issues the copies.
    const bool leader = lane == 0;
    uint32_t n_pub0 = 0, n_pub1 = 0;
    uint32_t out_mask = 0;    // bit s: a load signalled on barrier kKVFull+s has not been handed back yet
    uint32_t free_par = 0;    // bit s: parity of the next kKVFree+s phase
    uint32_t stream_tiles = 0;
    int mode = 0;             // 1 streamed, 2 resident: the two use the slots' barriers differently
    auto publish = [&](int x, const Job& it) {
      const uint32_t np = x ? n_pub1 : n_pub0;
      const uint32_t slot = np % kJobRing;
      if (np >= kJobRing) wait(kJobFree + x * kJobRing + slot, np / kJobRing - 1, 14 + x);
      if (leader) {
        write_record(job_ring + (x * kJobRing + slot) * 16, it);
        ptx::mbar_arrive(bar(kJobFull + x * kJobRing + slot));  // release: the record is visible to whoever sees the phase flip
      }
      if (x) ++n_pub1; else ++n_pub0;
    };
    // wait until both MMA warps have handed back the load last signalled on barrier s
    auto drain = [&](int s) {
      if ((out_mask >> s) & 1u) {
        wait(kKVFree + s, (free_par >> s) & 1u, 12);
        free_par ^= 1u << s;
        out_mask &= ~(1u << s);
      }
    };
    auto set_mode = [&](int m) {
      if (mode != m) {
#pragma unroll 1
        for (int s = 0; s < kSlots; ++s) drain(s);
        mode = m;
      }
    };
    // K and V of 64 keys starting at token slot `lo` -> pool slot s, completion on barrier `bs`
    auto load_slot = [&](int s, int bs, int g, int b, int lo) {
      const uint32_t kd = sbase + kOffK + (uint32_t)s * kSlotHalf, vd = sbase + kOffV + (uint32_t)s * kSlotHalf;
      ptx::tma_load_4d(kd, &tmK, bar(kKVFull + bs), 0, g, lo, b);
      ptx::tma_load_4d(kd + kPoolHalf, &tmK, bar(kKVFull + bs), 64, g, lo, b);
      ptx::tma_load_4d(vd, &tmV, bar(kKVFull + bs), 0, g, lo, b);
      ptx::tma_load_4d(vd + kPoolHalf, &tmV, bar(kKVFull + bs), 64, g, lo, b);
    };

    // ---- streamed pair: both chains walk the same 128-key tiles through a two-deep ring (slots 0-1, 2-3) ----
    auto run_pair = [&](int b, int g, int m, int chunk, int p, int start, int len, int s0, int l0, int s2, int l2) {
      Pair pr = decode_pair(a, b, g, m, chunk, p, start, len, s0, l0, s2, l2);
      if (!pr.valid) return;
      Job& it = pr.job;
      if (m == a.M - 1 && m > 0) {  // the query block's context may contain padding slots
        const int32_t* bl = a.blk_len + (size_t)b * a.M;
        int part = 0;
        for (int i = lane; i < a.M - 1; i += 32) part += bl[i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        if (part != (it.ctx_hi - it.ctx_lo)) it.flags |= kFCtxCheck;
      }
      set_mode(1);
      const int T = (pr.n_slots + 1) >> 1;
      it.tile0 = (int)(stream_tiles & 1u);
      it.aux = T;
      it.t0 = pr.t0_0; it.n = pr.n_0;
      publish(0, it);
      it.t0 = pr.t0_1; it.n = pr.n_1;
      publish(1, it);
      for (int t = 0; t < T; ++t) {
        const int tb = (int)((stream_tiles + (uint32_t)t) & 1u);
        drain(2 * tb);
        drain(2 * tb + 1);
        const int nslots = min(2, pr.n_slots - 2 * t);
        if (leader) {
          ptx::mbar_expect_tx(bar(kKVFull + 2 * tb), (uint32_t)nslots * kSlotBytes);
          for (int h = 0; h < nslots; ++h) {
            int nk, own_off; bool own;
            const int lo = tile_lo(it, 2 * t + h, nk, own, own_off);
            load_slot(2 * tb + h, 2 * tb, g, b, lo);
          }
        }
        out_mask |= 1u << (2 * tb);
      }
      stream_tiles += (uint32_t)T;
    };

    // ---- resident block: K/V loaded once, row tiles dealt to the chains largest first ----
    auto run_block = [&](int b, int g, int m, int start, int len, int s0, int l0, bool keep_in, bool keep_out) {
      const int ctx = m > 0 ? l0 : 0;
      const int n_ctx = (ctx + BN - 1) / BN;
      const int ns_blk = n_ctx + (len + BN - 1) / BN;
      const int R = (len + TOK - 1) / TOK;
      const int n_keep = keep_out ? (m > 0 ? n_ctx : (l0 + BN - 1) / BN) : 0;
      set_mode(2);
      // K/V slots, highest first (the previous block hands them back in that order).  The loop stops at the first
      // slot that is still in use; the block's jobs are published before the producer sleeps on it, so that the
      // chains find their records and request their Q tiles meanwhile (their MMA warps wait for the slots).
      const int s_lo = keep_in ? n_ctx : 0;
      int s_next = ns_blk - 1;
      auto load_slots = [&](bool blocking) {
        for (; s_next >= s_lo; --s_next) {
          const int s = s_next;
          if ((out_mask >> s) & 1u) {
            if (!blocking && !__all_sync(0xffffffffu, ptx::mbar_test(bar(kKVFree + s), (free_par >> s) & 1u))) return;
            drain(s);
          }
          const int lo = s < n_ctx ? s0 + s * BN : start + (s - n_ctx) * BN;
          if (leader) {
            ptx::mbar_expect_tx(bar(kKVFull + s), kSlotBytes);
            load_slot(s, s, g, b, lo);
          }
          out_mask |= 1u << s;
        }
      };
      load_slots(false);
      Job it;
      it.b = b; it.g = g; it.m = m; it.chunk = 0;
      it.start = start; it.len = len;
      it.ctx_lo = s0; it.ctx_hi = s0 + ctx; it.n_ctx = n_ctx; it.j0 = 0;
      it.tile0 = 0;
      auto slots_of = [&](int i) { return n_ctx + (min(len, (R - i) * TOK) + BN - 1) / BN; };  // i-th largest tile
      // Deal the row tiles (largest first) to the two chains so that the chains finish together: a tile costs
      // its keys plus a fixed share for writing the output.  Up to 11 tiles every split is tried (the lanes
      // share the 2^(R-1) candidates); beyond that the tiles are dealt 0,1,1,0,0,1,1,0,...
      uint32_t cmask = 0;  // bit i: chain of the i-th largest tile
      if (R <= 11) {
        const int n_cand = 1 << (R - 1);  // tile 0 (the largest) goes to chain 0
        uint32_t best = 0xffffffffu;
        for (int c = lane; c < n_cand; c += 32) {
          int load0 = 0, load1 = 0;
          for (int i = 0; i < R; ++i) {
            const int cost = ctx + min(len, (R - i) * TOK) + kTileFixedCost;
            if (((c << 1) >> i) & 1) load1 += cost; else load0 += cost;
          }
          best = min(best, ((uint32_t)max(load0, load1) << 11) | (uint32_t)(c << 1));
        }
        cmask = __reduce_min_sync(0xffffffffu, best) & 0x7ffu;
      } else {
        for (int i = 0; i < R; ++i) cmask |= (uint32_t)deal_chain(i) << i;
      }
      auto next_same = [&](int i) {  // position of the same chain's next tile, or R
        const uint32_t same = (((cmask >> i) & 1u) ? cmask : ~cmask) & ~((2u << i) - 1u) & ((1u << R) - 1u);
        return same ? __ffs((int)same) - 1 : R;
      };
      const int first1 = (cmask & ((1u << R) - 1u)) ? __ffs((int)cmask) - 1 : R;  // chain 1's first tile (R: none)
      for (int i = 0; i < R; ++i) {
        const int x = (int)((cmask >> i) & 1u), r = R - 1 - i;
        it.t0 = r * TOK;
        it.own_n = min(len, it.t0 + TOK);
        it.n = slots_of(i);
        const bool first = i == 0 || i == first1;
        const int nx = next_same(i);
        const int rel_lo = max(n_keep, nx < R ? slots_of(nx) : 0);  // slots kept for the next block are never handed back
        const int rel_hi = first ? ns_blk : it.n;
        it.flags = kFDoc | (first ? kFFirst : 0) | (keep_in ? kFKeep : 0);
        it.aux = rel_lo | (rel_hi << 8);
        publish(x, it);
        // Only the two largest tiles are published ahead of the slots that are still busy: a ring that filled
        // up with jobs whose K/V cannot be loaded (because the producer sleeps on the ring) would never drain.
        if (i == 1) load_slots(true);
      }
      if (first1 == R) {  // chain 1 has no row tile: it only hands the slots back
        it.t0 = 0; it.own_n = 0; it.n = 0;
        it.flags = kFDoc | kFFirst | (keep_in ? kFKeep : 0);
        it.aux = n_keep | (ns_blk << 8);
        publish(1, it);
      }
      load_slots(true);
    };

    // The work list is handed out dynamically: whichever CTA is free claims the next index.  Claims
    // run two items ahead and the block spans of a claimed item one item ahead, so neither the
    // atomic nor the loads are waited for.
    auto claim = [&]() {
      int v = 0;
      if (leader) v = atomicAdd(a.work_counter, 1);
      return __shfl_sync(0xffffffffu, v, 0);
    };
    int idx = claim(), idx_next = claim();
    ItemRaw raw_next = load_item(a, idx, lane);
    for (; idx < a.total_items; idx = idx_next, idx_next = claim()) {
      const ItemRaw raw = raw_next;
      raw_next = load_item(a, idx_next, lane);  // in flight while this item is processed
      if (raw.kind == 0) {
        run_pair(raw.b, raw.g, raw.m, raw.chunk, raw.p, raw.start, raw.len, raw.s0, raw.l0, raw.s2, raw.l2);
        continue;
      }
      auto fits = [&](int m, int len) {
        const int ctx = m > 0 ? raw.l0 : 0;
        return (ctx + BN - 1) / BN + (len + BN - 1) / BN <= kSlots;
      };
      bool kept = false;
      for (int i = 0; i < raw.cnt; ++i) {
        const int m = raw.m + i;
        const int start = __shfl_sync(0xffffffffu, raw.start, i), len = __shfl_sync(0xffffffffu, raw.len, i);
        const int len_nx = __shfl_sync(0xffffffffu, raw.len, (i + 1) & 31);
        if (len <= 0) continue;  // an empty block has no rows
        if (fits(m, len)) {
          const bool keep_out = i + 1 < raw.cnt && len_nx > 0 && fits(m + 1, len_nx) && raw.l0 > 0;
          run_block(raw.b, raw.g, m, start, len, raw.s0, raw.l0, kept, keep_out);
          kept = keep_out;
        } else {
          const int pairs = (len + 2 * TOK - 1) / (2 * TOK);
          for (int p = 0; p < pairs; ++p)
            run_pair(raw.b, raw.g, m, 0, p, start, len, raw.s0, raw.l0, raw.s2, raw.l2);
        }
      }
    }
    Job stop{};
    stop.flags = kFStop;
    publish(0, stop);
    publish(1, stop);
  } else if (warp == 9 || warp == 10) {
    // =============================== MMA issuer of chain x ======================================
    // Whole-warp control flow, one issuing lane (always the same one: tcgen05.commit tracks the
    // MMAs of the thread that executes it).  The two chains' issuers never wait for each other;
    // they only meet in the kKVFree barriers (two arrivals hand a slot back to the TMA warp).
    const int x = warp - 9;
    const bool leader = lane == 0;
    uint32_t q_uses = 0, p_seen = 0, jobs_done = 0;
    uint32_t full_par = 0;  // bit s: parity of the next kKVFull+s phase this warp has not consumed yet
    int blk_waited = 0;     // resident block: slots [0, blk_waited) have landed
    // Descriptors are built once: every operand buffer has a fixed address, and stepping along K
    // or to another slot only adds a constant to the 16-byte-unit start-address field.
    const uint32_t idesc_pv = ptx::idesc_bf16(BM, HD, 0, 1);
    const uint32_t idesc_qk0 = ptx::idesc_bf16(BM, 0, 0, 0);
    const uint64_t q_desc0 = ptx::smem_desc_sw128(sbase + kOffQ + (uint32_t)x * kQBytes, 16, 1024);
    const uint64_t k_desc0 = ptx::smem_desc_sw128(sbase + kOffK, 16, 1024);
    const uint64_t v_desc0 = ptx::smem_desc_sw128(sbase + kOffV, kPoolHalf, 1024);
    const uint32_t tm_s = tmem + (uint32_t)x * kChainCols, tm_o = tm_s + kColO;
    auto wait_full = [&](int s) {
      wait(kKVFull + s, (full_par >> s) & 1u, 22 + x);
      full_par ^= 1u << s;
    };
    // S = Q K^T against `keys` keys starting at pool slot `slot`
    auto issue_qk = [&](int slot, int keys, bool last) {
      const uint32_t idesc = idesc_qk0 | ((uint32_t)((keys + 15) >> 4) << 18);  // N/8 at bit 17, N a multiple of 16
      const uint32_t a_lo = (uint32_t)q_desc0, a_hi = (uint32_t)(q_desc0 >> 32);
      const uint32_t b_lo = (uint32_t)k_desc0 + (uint32_t)slot * (kSlotHalf >> 4), b_hi = (uint32_t)(k_desc0 >> 32);
      if (leader) {
#pragma unroll 1
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t aoff = (uint32_t)(ks >> 2) * ((BM * 128) >> 4) + (uint32_t)(ks & 3) * 2;
          const uint32_t boff = (uint32_t)(ks >> 2) * (kPoolHalf >> 4) + (uint32_t)(ks & 3) * 2;
          ptx::mma_ss_lohi(tm_s, a_lo + aoff, a_hi, b_lo + boff, b_hi, idesc, ks > 0);
        }
        ptx::mma_commit(bar(kSFull + x));
        if (last) ptx::mma_commit(bar(kQFree + x));  // last read of this chain's Q tile
      }
    };
    // O (+)= P V over `keys` keys starting at pool slot `slot`; P sits over the first 64 columns of S
    auto issue_pv = [&](int slot, int keys, bool first) {
      const uint32_t b_lo = (uint32_t)v_desc0 + (uint32_t)slot * (kSlotHalf >> 4), b_hi = (uint32_t)(v_desc0 >> 32);
      const int ksteps = (keys + 15) >> 4;
      if (leader) {
#pragma unroll 1
        for (int ks = 0; ks < BT / 16; ++ks)
          if (ks < ksteps)
            ptx::mma_ts_lohi(tm_o, tm_s + (uint32_t)ks * 8, b_lo + (uint32_t)ks * ((16 * 128) >> 4), b_hi, idesc_pv,
                             (!first || ks > 0) ? 1u : 0u);
        ptx::mma_commit(bar(kPVDone + x));
      }
    };
    // keys of a job's last 128-key tile (every earlier tile spans 128 keys: a short context slot inside a
    // tile is masked by the softmax, not trimmed)
    auto last_tile_keys = [&](const Job& jb) {
      const int Tj = (jb.n + 1) >> 1;
      if (Tj == 0) return 0;
      const int cnt = min(2, jb.n - 2 * (Tj - 1));
      int nk, own_off; bool own;
      tile_lo(jb, 2 * (Tj - 1) + cnt - 1, nk, own, own_off);
      return (cnt - 1) * BN + nk;
    };
    // This warp also loads its chain's Q tiles: it is the one that knows when the buffer is free (the job's last
    // Q K^T has completed) and it has nothing else to do at that moment.  q_issued counts the tiles requested;
    // the next job's tile is requested as soon as the current job's last Q K^T is in the pipe and its record
    // has been published, otherwise at the start of that job.
    uint32_t q_issued = 0;
    auto request_q = [&](const Job& jb) {
      if (q_issued > 0) wait(kQFree + x, q_issued - 1, 28 + x);  // every Q K^T of the previous job has read the buffer
      if (leader) {
        const uint32_t dst = sbase + kOffQ + (uint32_t)x * kQBytes;
        ptx::mbar_expect_tx(bar(kQFull + x), kQBytes);
        ptx::tma_load_4d(dst, &tmQ, bar(kQFull + x), 0, jb.g * G, jb.start + jb.t0, jb.b);
        ptx::tma_load_4d(dst + BM * 128, &tmQ, bar(kQFull + x), 64, jb.g * G, jb.start + jb.t0, jb.b);
      }
      ++q_issued;
    };
    // called once the current job's last Q K^T has been issued: request the next job's Q tile if its record is there
    auto request_next_q = [&](uint32_t job_no) {
      if (q_issued != q_uses) return;  // already requested
      const uint32_t nslot = (job_no + 1) % kJobRing;
      if (!__all_sync(0xffffffffu, ptx::mbar_test(bar(kJobFull + x * kJobRing + nslot), ((job_no + 1) / kJobRing) & 1u))) return;
      const Job nxt = read_record(job_ring + (x * kJobRing + nslot) * 16);
      if (!(nxt.flags & kFStop) && nxt.n > 0) request_q(nxt);
    };
    bool pre_qk = false;  // the first Q K^T of the job fetched next is already in the pipe
    for (uint32_t job_no = 0;; ++job_no) {
      const Job it = next_job(x, job_no);
      if (it.flags & kFStop) break;
      const int n = it.n, T = (n + 1) >> 1;
      const int last_keys = last_tile_keys(it);
      auto keys_of = [&](int t) { return t + 1 < T ? BT : last_keys; };
      // (a job whose first Q K^T was issued ahead has had its Q phase consumed there: by now the barrier may be
      // a phase further, and a parity wait must never fall two phases behind)
      if (T > 0 && !pre_qk) {
        if (q_issued == q_uses) request_q(it);  // not requested ahead
        wait(kQFull + x, q_uses, 20 + x);
        ++q_uses;
      }
      if (T == 1 && pre_qk) request_next_q(job_no);  // its only Q K^T went out with the previous job's last P V
      if (it.flags & kFDoc) {
        // ---- resident block: tile t = pool slots 2t, 2t+1; slots land once per block ----
        if (it.flags & kFFirst) blk_waited = (it.flags & kFKeep) ? it.n_ctx : 0;
        auto ensure = [&](int ns) {
          while (blk_waited < ns) { wait_full(blk_waited); ++blk_waited; }
        };
        if (T > 0) {
          if (!pre_qk) {
            ensure(min(n, 2));
              ptx::tc_fence_after_sync();
            issue_qk(0, keys_of(0), T == 1);
              if (T == 1) request_next_q(job_no);
          }
          pre_qk = false;
          for (int t = 0; t < T; ++t) {
            if (t + 1 < T) ensure(min(n, 2 * t + 4));
            wait(kPFull + x, p_seen, 24 + x);
            ++p_seen;
            if (t == 0 && jobs_done > 0) wait(kOFree + x, jobs_done - 1, 26 + x);
            // After the job's last tile the chain's next row tile of the same block can start at once if its
            // record and its Q tile are already here (its first key tile is resident): its first Q K^T then
            // rides behind this P V, and its S tile is waiting when the softmax warps have drained O.
            Job nxt{};
            bool chain_on = false;
            if (t + 1 == T) {
              const uint32_t nslot = (job_no + 1) % kJobRing;
              if (__all_sync(0xffffffffu, ptx::mbar_test(bar(kJobFull + x * kJobRing + nslot), ((job_no + 1) / kJobRing) & 1u))) {
                nxt = read_record(job_ring + (x * kJobRing + nslot) * 16);
                chain_on = (nxt.flags & kFDoc) && !(nxt.flags & (kFFirst | kFStop)) && nxt.n > 0 &&
                           blk_waited >= min(nxt.n, 2) && q_issued > q_uses &&
                           __all_sync(0xffffffffu, ptx::mbar_test(bar(kQFull + x), q_uses & 1u));
              }
            }
              ptx::tc_fence_after_sync();
            issue_pv(2 * t, keys_of(t), t == 0);
            // the chain's next S tile: queued behind the P V that reads P out of the same columns
            if (t + 1 < T) issue_qk(2 * t + 2, keys_of(t + 1), t + 2 == T);
            if (chain_on) {
              const int Tn = (nxt.n + 1) >> 1;
              issue_qk(0, Tn > 1 ? BT : last_tile_keys(nxt), Tn == 1);
              pre_qk = true;
              ++q_uses;  // its Q tile has landed (tested above): that phase is consumed here
            }
              if (t + 2 == T) request_next_q(job_no);  // the job's last Q K^T is in the pipe
          }
          ++jobs_done;
        }
        // hand back the slots no later job of this chain in this block needs
        // (every load of the block is consumed by both issuers, also of slots this chain never reads or
        // that stay resident for the next block: the phase parities must not fall behind)
        const int rel_lo = it.aux & 0xff, rel_hi = (it.aux >> 8) & 0xff;
        ensure(rel_hi);
        for (int s = rel_lo; s < rel_hi; ++s)
          if (leader) ptx::mma_commit(bar(kKVFree + s));
      } else {
        // ---- streamed pair: tile t sits in ring position (tile0 + t) & 1 = pool slots 0-1 or 2-3 ----
        const int Ti = it.aux;  // tiles of the item; this chain computes on the first T of them
        int kv_waited = -1;
        auto need_kv = [&](int t) {
          if (kv_waited >= t) return;
          wait_full(2 * ((it.tile0 + t) & 1));
          kv_waited = t;
        };
        if (T > 0) {
          need_kv(0);
          ptx::tc_fence_after_sync();
          issue_qk(2 * (it.tile0 & 1), keys_of(0), T == 1);
          if (T == 1) request_next_q(job_no);
        }
        for (int t = 0; t < Ti; ++t) {
          const int slot = 2 * ((it.tile0 + t) & 1);
          if (t < T) {
            if (t + 1 < T) need_kv(t + 1);  // (its ring position was handed back after P V of tile t-1)
            wait(kPFull + x, p_seen, 24 + x);
            ++p_seen;
            if (t == 0 && jobs_done > 0) wait(kOFree + x, jobs_done - 1, 26 + x);
              ptx::tc_fence_after_sync();
            issue_pv(slot, keys_of(t), t == 0);
            if (leader) ptx::mma_commit(bar(kKVFree + slot));
            if (t + 1 < T) issue_qk(2 * ((it.tile0 + t + 1) & 1), keys_of(t + 1), t + 2 == T);
              if (t + 2 == T) request_next_q(job_no);  // the job's last Q K^T is in the pipe
          } else {
            need_kv(t);  // not visible to this chain: consume the phase, then hand the tile back
            if (leader) ptx::mma_commit(bar(kKVFree + slot));
          }
        }
        if (T > 0) ++jobs_done;
      }
    }
  } else {
    // =============================== softmax + output, chain x ==================================
    const int x = warp >> 2;
    const int r = tid & 127;  // row of the tile = TMEM lane
    const uint32_t tmem_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)x * kChainCols;
    uint32_t s_seen = 0, pv_seen = 0;

    for (uint32_t job_no = 0;; ++job_no) {
      const Job it = next_job(x, job_no);
      const int flags = it.flags;
      if (flags & kFStop) break;
      if (it.n == 0) continue;
      const int32_t* bs = a.blk_start + (size_t)it.b * a.M;
      const int32_t* bl = a.blk_len + (size_t)it.b * a.M;
      const int tok = it.t0 + (r >> a.g_shift);
      const int n = it.g * G + (r & (G - 1));
      const bool active = tok < it.len;
      const bool ctx_check = (flags & kFCtxCheck) != 0;  // the query block's context contains padding slots
      float m_run = -INFINITY, l_run = 0.f;
      const int n_mine = it.n;
      const bool split = (flags & kFSplit) != 0;
      const int t_mine = (n_mine + 1) >> 1;

      for (int t = 0; t < t_mine; ++t) {
        const int cnt = min(2, n_mine - 2 * t);  // slots of this tile the chain sees
        wait(kSFull + x, s_seen, 30 + x);
        ++s_seen;
        if (t > 0) {
          // The previous tile's P V was issued before this tile's Q K^T, so it has completed too: O is stable
          // and the P columns (first half of S) may be overwritten.  Consuming that phase here keeps the pass
          // below free of calls (64 logits are live across its middle).
          wait(kPVDone + x, pv_seen, 32 + x);
          ++pv_seen;
        }
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
          // Ragged tails and the causal diagonal make columns [0, lim) of a row visible; padded
          // context ranges (reference layout with gaps between blocks) are masked column by column.
          // A masked logit becomes -inf with one select per column, so that its P is exactly 0 and the
          // pass below stays one basic block: skipping the 8-column groups that no row of the warp sees
          // with warp-uniform branches measured 5 % slower over the whole kernel than exponentiating them.
          const bool premasked = !own && ctx_check;  // padded context: columns masked one by one from the slot-validity ballots
          if (nk < BN || (own && own_off + BN - 1 > it.t0) || premasked) {  // (warp-uniform)
            int lim = nk;
            if (own) lim = max(0, min(nk, tok - own_off + 1));
            if (premasked) {
              const unsigned v0 = __ballot_sync(0xffffffffu, slot_valid(bs, bl, a.M, lo + lane));
              const unsigned v1 = __ballot_sync(0xffffffffu, slot_valid(bs, bl, a.M, lo + 32 + lane));
#pragma unroll
              for (int c = 0; c < 64; ++c) {
                const bool ok = c < lim && (((c < 32 ? v0 : v1) >> (c & 31)) & 1u);
                sr[c] = ok ? sr[c] : 0xff800000u;  // -inf
              }
            } else {
#pragma unroll
              for (int c = 0; c < 64; ++c) sr[c] = c < lim ? sr[c] : 0xff800000u;  // -inf: P = 0 exactly
            }
          }
          {
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // independent chains
#pragma unroll
            for (int c = 0; c < 64; c += 2)
              mx4[(c >> 1) & 3] = ptx::max3(mx4[(c >> 1) & 3], __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;  // scale > 0
            float m_new = fmaxf(m_run, mx);
            if (m_run != -INFINITY && m_new - m_run <= kLazy) m_new = m_run;  // keep the old reference: p <= 2^8
            const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ptx::ex2(m_run - m_ref);  // 1 when unchanged, 0 on the first visible slot
            const float neg_ref = -m_ref;
            const bool changed = m_new != m_run;
            m_run = m_new;

            // p with packed fp32x2 arithmetic; see kPolyOf8 for where the exponentials are evaluated
            const ptx::f32x2 sc2 = ptx::pack2(a.scale_log2, a.scale_log2), nr2 = ptx::pack2(neg_ref, neg_ref);
            ptx::f32x2 ps2[2] = {0ull, 0ull};
            uint32_t pk[32];
#pragma unroll
            {
              {
#pragma unroll
                for (int c = 0; c < 64; c += 4) {
                  const ptx::f32x2 t01 = ptx::fma2(ptx::pack2(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), sc2, nr2);
                  const ptx::f32x2 t23 = ptx::fma2(ptx::pack2(__uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3])), sc2, nr2);
                  float t0, t1, p2, p3;
                  ptx::unpack2(t01, t0, t1);
                  const float p0 = ptx::ex2(t0), p1 = ptx::ex2(t1);
                  // kPolyOf8 of every 8 exponentials go to the FMA pipe as a polynomial, the rest to the
                  // special-function unit (a -inf logit gives exactly 0 there)
                  if ((kPolyOf8 == 4) || (kPolyOf8 == 2 && (c & 4))) {
                    const ptx::f32x2 p23 = ptx::ex2_poly2(t23);
                    ptx::unpack2(p23, p2, p3);
                    // a masked column must contribute exactly nothing: the polynomial maps -inf to 2^-126,
                    // which times a huge (finite) value in a padding slot of V would still be visible
                    p2 = sr[c + 2] == 0xff800000u ? 0.f : p2;
                    p3 = sr[c + 3] == 0xff800000u ? 0.f : p3;
                  } else {
                    float t2, t3;
                    ptx::unpack2(t23, t2, t3);
                    p2 = ptx::ex2(t2);
                    p3 = ptx::ex2(t3);
                  }
                  ps2[1] = ptx::add2(ps2[1], ptx::pack2(p2, p3));
                  ps2[0] = ptx::add2(ps2[0], ptx::pack2(p0, p1));
                  __nv_bfloat162 h0 = __floats2bfloat162_rn(p0, p1), h1 = __floats2bfloat162_rn(p2, p3);
                  pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h0);
                  pk[(c >> 1) + 1] = *reinterpret_cast<uint32_t*>(&h1);
                }
              }
            }
            ptx::tmem_st32(tmem_lane + (uint32_t)h * 32, pk);
            if ((t > 0 || h > 0) && __any_sync(0xffffffffu, changed)) {
              // The reference moved by more than the lazy threshold (rare): bring what was accumulated
              // against the old one in line -- O of the earlier tiles, P of this tile's first slot.  (Behind the
              // exponentials, so that the common path from the row maximum to P is one basic block; all of it
              // precedes the arrival that lets the MMA warp read P and add to O.)
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
            float s0, s1, s2, s3;
            ptx::unpack2(ps2[0], s0, s1);
            ptx::unpack2(ps2[1], s2, s3);
            l_run = l_run * corr + ((s0 + s1) + (s2 + s3));
          }
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
      if (split) {
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
  if (a.hdr[1] != 0) return;
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

// The give-up path of the kernels' bounded waits, exercised without a fault: one thread waits, with a small
// budget, on an mbarrier that nothing ever arrives at; the wait runs out, the thread records kStatusSelfTest in
// the caller's status word exactly as attn_tc_kernel's waits do, and the kernel returns normally.
__global__ void selftest_wait_kernel(int32_t* status, uint32_t budget) {
  __shared__ __align__(8) uint64_t mbar;
  const uint32_t b = ptx::smem_u32(&mbar);
  ptx::mbar_init(b, 1);
  ptx::fence_barrier_init();
  if (!ptx::mbar_wait(b, 0, budget)) atomicCAS(status, 0, kStatusSelfTest);
}

int selftest_wait_launch(int32_t* status, uint32_t budget, cudaStream_t st) {
  selftest_wait_kernel<<<1, 1, 0, st>>>(status, budget);
  BRK_CUDA(cudaGetLastError());
  return BRK_OK;
}

// Launched in front of either attention kernel.  Block 0 checks the block spans (inside [0, S), no longer than
// max_block_len, ordered, not overlapping) and records the verdict in the workspace header -- a non-zero hdr[1]
// makes the attention kernels return without touching memory, and the caller's status word (if any) gets
// kStatusBadSpans.  All blocks reset the work counter and the query block's partial (max, sum) pairs to neutral.
__global__ void attn_prologue_kernel(const int32_t* __restrict__ blk_start, const int32_t* __restrict__ blk_len, int B,
                                     int M, int S, int max_block_len, int max_query_len, int* hdr, int32_t* status,
                                     float2* ml, int64_t n_ml) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_ml) ml[i] = make_float2(-INFINITY, 0.f);
  if (blockIdx.x != 0) return;
  __shared__ int bad;
  if (threadIdx.x == 0) {
    bad = 0;
    hdr[0] = 0;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < B * M; j += blockDim.x) {
    const int m = j % M;
    const int s = blk_start[j], l = blk_len[j];
    bool ok = s >= 0 && l >= 0 && l <= max_block_len && s <= S - l;
    if (ok && m > 0) ok = blk_start[j - 1] >= 0 && blk_len[j - 1] >= 0 && blk_start[j - 1] <= s - blk_len[j - 1];
    if (ok && m == M - 1 && max_query_len > 0) ok = l <= max_query_len;
    if (!ok) bad = 1;  // benign race: every writer stores the same value
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    hdr[1] = bad;
    if (bad && status) atomicCAS(status, 0, kStatusBadSpans);
  }
}

int attn_prologue_launch(const brk_attn_params& p, int* hdr, float2* ml, int64_t n_ml, cudaStream_t st) {
  const unsigned blocks = (unsigned)(n_ml > 0 ? (n_ml + 255) / 256 : 1);
  attn_prologue_kernel<<<blocks, 256, 0, st>>>(p.blk_start, p.blk_len, p.B, p.M, p.S, p.max_block_len, p.max_query_len,
                                               hdr, p.status, ml, n_ml);
  BRK_CUDA(cudaGetLastError());
  return BRK_OK;
}

// Key chunks for the query block.  Its context is every earlier token of the prompt (S is the only
// bound known on the host), walked 128 keys per step per row tile; cutting it into chunks of about
// 1024 keys keeps that serial chain short and spreads it over the SMs.
static int tc_splits(const brk_attn_params& p) {
  if (p.M < 2) return 1;
  int n = (p.S + 1023) / 1024;
  return n < 1 ? 1 : (n > 32 ? 32 : n);
}

static int query_rows(const brk_attn_params& p) {
  return (p.max_query_len > 0 && p.max_query_len < p.max_block_len) ? p.max_query_len : p.max_block_len;
}

size_t attn_tc_workspace(const brk_attn_params& p) {
  const int ns = tc_splits(p);
  if (ns <= 1) return kWsHeader;  // work counter and span verdict
  const size_t rows = (size_t)p.B * p.N * query_rows(p) * ns;
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
  const int lq = query_rows(p);
  const int pairs_q = (lq + 2 * TOK - 1) / (2 * TOK);
  const int64_t nbg = (int64_t)p.B * p.Nk;
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
  // Blocks are handed out in groups of consecutive blocks of one (prompt, KV head), so that the prefix's K/V
  // stays in shared memory from one block to the next.  Balance matters more than that reuse (measured: single
  // blocks 0.560 ms, groups of three 0.572 ms on 4 prompts of 100 documents), so groups only form when every SM
  // still gets two dozen of them.
  int group = (int)((nbg * (p.M > 1 ? p.M - 1 : 0)) / (24 * (int64_t)sms[dev]));
  group = group < 1 ? 1 : (group > kMaxGroup ? kMaxGroup : group);
  const int n_groups = p.M > 1 ? (p.M - 1 + group - 1) / group : 0;
  const int64_t sec1 = nbg * ns * pairs_q;
  const int64_t total_items = sec1 + nbg * n_groups;
  BRK_REQUIRE(total_items < (1ll << 30), BRK_E_UNSUPPORTED, "too many work items (%lld)", (long long)total_items);
  TcArgs a;
  a.o = make_view(p.o);
  a.lse = p.lse;
  a.blk_start = p.blk_start;
  a.blk_len = p.blk_len;
  a.status = p.status;
  a.hdr = reinterpret_cast<const int*>(ws);
  a.B = p.B; a.N = p.N; a.Nk = p.Nk; a.S = p.S; a.M = p.M;
  a.G = G; a.g_shift = gs;
  a.scale_log2 = p.scale * 1.4426950408889634f;
  a.n_split = ns;
  a.lq_max = lq;
  a.pairs_q = pairs_q;
  a.group = group;
  a.n_groups = n_groups;
  a.o_align32 = (((uintptr_t)p.o.ptr & 31) == 0 && p.o.stride_b % 16 == 0 && p.o.stride_h % 16 == 0 && p.o.stride_s % 16 == 0) ? 1 : 0;
  a.sec1 = (int)sec1;
  a.total_items = (int)total_items;
  a.div_sec1 = make_fastdiv((uint32_t)(nbg * ns));
  a.div_nbg = make_fastdiv((uint32_t)nbg);
  a.div_nk = make_fastdiv((uint32_t)p.Nk);
  const size_t rows = (size_t)p.B * p.N * lq * ns;
  float* const part = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + kWsHeader);
  a.work_counter = reinterpret_cast<int*>(ws);
  a.part_o = ns > 1 ? part : nullptr;
  a.part_ml = ns > 1 ? reinterpret_cast<float2*>(part + rows * HD) : nullptr;
  if ((rc = attn_prologue_launch(p, reinterpret_cast<int*>(ws), a.part_ml, ns > 1 ? (int64_t)rows : 0, st))) return rc;
  const int grid = (int)(total_items < sms[dev] ? total_items : sms[dev]);
  attn_tc_kernel<<<grid, kThreads, kSmemBytes, st>>>(tq, tk, tv, a);
  BRK_CUDA(cudaGetLastError());
  if (ns > 1) {
    const int64_t warps = (int64_t)p.B * p.N * lq;
    attn_combine_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(a);
    BRK_CUDA(cudaGetLastError());
  }
  return BRK_OK;
}

}  // namespace brk
