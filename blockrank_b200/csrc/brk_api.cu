// C ABI of libblockrank_b200: argument validation, error reporting and dispatch.
// No entry point allocates device memory; all work is enqueued on the caller's stream.
#include <stdarg.h>
#include <string.h>

#include "brk_common.cuh"

namespace brk {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

static int check_view(const brk_view& v, int dtype, const char* name) {
  const int al = dtype == BRK_BF16 ? 8 : 4;  // elements per 16 bytes
  BRK_REQUIRE(v.ptr != nullptr, BRK_E_ARG, "%s is null", name);
  BRK_REQUIRE(((uintptr_t)v.ptr & 15) == 0, BRK_E_ARG, "%s base pointer must be 16-byte aligned", name);
  BRK_REQUIRE(v.stride_b % al == 0 && v.stride_h % al == 0 && v.stride_s % al == 0, BRK_E_ARG,
              "%s strides (%lld,%lld,%lld) must keep rows 16-byte aligned", name, (long long)v.stride_b,
              (long long)v.stride_h, (long long)v.stride_s);
  return BRK_OK;
}

static int check_attn(const brk_attn_params* p) {
  BRK_REQUIRE(p != nullptr, BRK_E_ARG, "params is null");
  BRK_REQUIRE(p->dtype == BRK_BF16 || p->dtype == BRK_F32, BRK_E_UNSUPPORTED, "dtype %d not supported", p->dtype);
  BRK_REQUIRE(p->B > 0 && p->N > 0 && p->Nk > 0 && p->S > 0 && p->M > 0, BRK_E_ARG,
              "bad shape B=%d N=%d Nk=%d S=%d M=%d", p->B, p->N, p->Nk, p->S, p->M);
  BRK_REQUIRE(p->N % p->Nk == 0, BRK_E_ARG, "N=%d is not a multiple of Nk=%d", p->N, p->Nk);
  BRK_REQUIRE(p->D == 64 || p->D == 128, BRK_E_UNSUPPORTED, "head_dim %d not supported (64 or 128)", p->D);
  BRK_REQUIRE(p->max_block_len > 0 && p->max_block_len <= p->S, BRK_E_ARG, "max_block_len=%d out of range (S=%d)",
              p->max_block_len, p->S);
  BRK_REQUIRE(p->blk_start && p->blk_len, BRK_E_ARG, "block spans are null");
  BRK_REQUIRE(p->max_query_len >= 0 && p->max_query_len <= p->S, BRK_E_ARG, "max_query_len=%d out of range (S=%d)",
              p->max_query_len, p->S);
  int rc;
  if ((rc = check_view(p->q, p->dtype, "q"))) return rc;
  if ((rc = check_view(p->k, p->dtype, "k"))) return rc;
  if ((rc = check_view(p->v, p->dtype, "v"))) return rc;
  if ((rc = check_view(p->o, p->dtype, "o"))) return rc;
  return BRK_OK;
}

static int resolve_algo(const brk_attn_params* p) {
  if (p->algo == BRK_ALGO_AUTO)
    return (p->dtype == BRK_BF16 && p->D == 128 && (p->N / p->Nk) == 4) ? BRK_ALGO_TC : BRK_ALGO_SIMT;
  return p->algo;
}

}  // namespace brk

using namespace brk;

extern "C" {

int brk_version(void) { return BRK_VERSION; }

const char* brk_last_error(void) { return g_err; }

int brk_device_check(void) {
  int dev = 0, major = 0;
  BRK_CUDA(cudaGetDevice(&dev));
  BRK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  BRK_REQUIRE(major == 10, BRK_E_DEVICE, "device compute capability %d.x is not sm_100", major);
  return BRK_OK;
}

int brk_spans_from_mask(const uint8_t* mask, int32_t B, int32_t M, int32_t H, int32_t* blk_start, int32_t* blk_len,
                        void* stream) {
  BRK_REQUIRE(mask && blk_start && blk_len, BRK_E_ARG, "null pointer");
  BRK_REQUIRE(B > 0 && M > 0 && H > 0, BRK_E_ARG, "bad mask shape (%d,%d,%d)", B, M, H);
  return spans_launch(mask, B, M, H, blk_start, blk_len, (cudaStream_t)stream);
}

size_t brk_attn_fwd_workspace_bytes(const brk_attn_params* p) {
  if (p == nullptr) return 0;
  return resolve_algo(p) == BRK_ALGO_TC ? attn_tc_workspace(*p) : kWsHeader;
}

int brk_attn_fwd(const brk_attn_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_attn(p);
  if (rc) return rc;
  const int algo = resolve_algo(p);
  if (algo == BRK_ALGO_SIMT) return attn_simt_launch(*p, workspace, workspace_bytes, (cudaStream_t)stream);
  if (algo == BRK_ALGO_TC) return attn_tc_launch(*p, workspace, workspace_bytes, (cudaStream_t)stream);
  set_error("unknown attention algorithm %d", p->algo);
  return BRK_E_UNSUPPORTED;
}

static int check_attn_bwd(const brk_attn_bwd_params* p) {
  BRK_REQUIRE(p != nullptr, BRK_E_ARG, "params is null");
  BRK_REQUIRE(p->dtype == BRK_BF16 || p->dtype == BRK_F32, BRK_E_UNSUPPORTED, "dtype %d not supported", p->dtype);
  BRK_REQUIRE(p->B > 0 && p->N > 0 && p->Nk > 0 && p->S > 0 && p->M > 0, BRK_E_ARG,
              "bad shape B=%d N=%d Nk=%d S=%d M=%d", p->B, p->N, p->Nk, p->S, p->M);
  BRK_REQUIRE(p->N % p->Nk == 0, BRK_E_ARG, "N=%d is not a multiple of Nk=%d", p->N, p->Nk);
  BRK_REQUIRE(p->dtype == BRK_BF16 || 64 % (p->N / p->Nk) == 0, BRK_E_UNSUPPORTED,
              "fp32 backward: query heads per KV head (%d) must divide 64", p->N / p->Nk);
  BRK_REQUIRE(p->D == 64 || p->D == 128, BRK_E_UNSUPPORTED, "head_dim %d not supported (64 or 128)", p->D);
  BRK_REQUIRE(p->max_block_len > 0 && p->max_block_len <= p->S, BRK_E_ARG, "max_block_len=%d out of range (S=%d)",
              p->max_block_len, p->S);
  BRK_REQUIRE(p->blk_start && p->blk_len && p->lse, BRK_E_ARG, "block spans / lse are null");
  BRK_REQUIRE(p->scale > 0.f, BRK_E_ARG, "softmax scale must be positive");
  const brk_view* vs[8] = {&p->q, &p->k, &p->v, &p->o, &p->d_o, &p->dq, &p->dk, &p->dv};
  const char* names[8] = {"q", "k", "v", "o", "d_o", "dq", "dk", "dv"};
  for (int i = 0; i < 8; ++i) {
    const int rc = check_view(*vs[i], p->dtype, names[i]);
    if (rc) return rc;
  }
  return BRK_OK;
}

size_t brk_attn_bwd_workspace_bytes(const brk_attn_bwd_params* p) {
  if (p == nullptr) return 0;
  return attn_bwd_workspace(*p);
}

int brk_attn_bwd(const brk_attn_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_attn_bwd(p);
  if (rc) return rc;
  return attn_bwd_launch(*p, workspace, workspace_bytes, (cudaStream_t)stream);
}

int brk_status_poll(int32_t* status, void* stream) {
  BRK_REQUIRE(status != nullptr, BRK_E_ARG, "status is null");
  int32_t v = 0;
  BRK_CUDA(cudaMemcpyAsync(&v, status, sizeof(v), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  BRK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (v == 0) return BRK_OK;
  BRK_CUDA(cudaMemsetAsync(status, 0, sizeof(v), (cudaStream_t)stream));
  if (v == kStatusBadSpans) {
    set_error("malformed block spans (a block outside [0, S), longer than max_block_len / max_query_len, or "
              "overlapping its predecessor): the attention call wrote nothing");
    return BRK_E_ARG;
  }
  set_error("a bounded device-side wait gave up (code %d: %s); the outputs of that call are incomplete", v,
            v == kStatusSelfTest ? "self-test" : v < 20 ? "TMA warp" : v < 30 ? "MMA warp" : v < 40 ? "softmax warp" : "job ring");
  return BRK_E_TIMEOUT;
}

int brk_selftest_bounded_wait(int32_t* status, uint32_t budget, void* stream) {
  BRK_REQUIRE(status != nullptr, BRK_E_ARG, "status is null");
  BRK_REQUIRE(budget >= 1 && budget <= (1u << 16), BRK_E_ARG, "budget %u out of range [1, 65536]", budget);
  return selftest_wait_launch(status, budget, (cudaStream_t)stream);
}

size_t brk_doc_scores_workspace_bytes(const brk_score_params* p) { return p ? doc_scores_workspace(*p) : 0; }

int brk_doc_scores(const brk_score_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  BRK_REQUIRE(p != nullptr, BRK_E_ARG, "params is null");
  return doc_scores_launch(*p, workspace, workspace_bytes, (cudaStream_t)stream);
}

int brk_doc_scores_static(const brk_score_params* p, void* stream) {
  BRK_REQUIRE(p != nullptr, BRK_E_ARG, "params is null");
  return doc_scores_static_launch(*p, (cudaStream_t)stream);
}

int brk_raw_scores(const brk_score_params* p, void* out, void* stream) {
  BRK_REQUIRE(p != nullptr, BRK_E_ARG, "params is null");
  return raw_scores_launch(*p, out, (cudaStream_t)stream);
}

int brk_rmsnorm(int32_t dtype, const void* x, void* residual, const void* weight, void* out, int64_t rows,
                int32_t hidden, float eps, void* stream) {
  BRK_REQUIRE(x && weight && out, BRK_E_ARG, "null pointer");
  BRK_REQUIRE(dtype == BRK_BF16 || dtype == BRK_F32, BRK_E_UNSUPPORTED, "dtype %d", dtype);
  BRK_REQUIRE(rows > 0 && rows < (1ll << 31) && hidden > 0 && hidden % 8 == 0 && hidden <= 16384, BRK_E_ARG,
              "bad rmsnorm shape rows=%lld hidden=%d", (long long)rows, hidden);
  return rmsnorm_launch(dtype, x, residual, weight, out, rows, hidden, eps, (cudaStream_t)stream);
}

int brk_rope(int32_t dtype, void* q, int64_t q_row_stride, int32_t N, void* k, int64_t k_row_stride, int32_t Nk,
             int32_t D, const int32_t* pos, const float* inv_freq, int64_t T, void* stream) {
  BRK_REQUIRE((q || N == 0) && (k || Nk == 0) && pos && inv_freq, BRK_E_ARG, "null pointer");
  BRK_REQUIRE(dtype == BRK_BF16 || dtype == BRK_F32, BRK_E_UNSUPPORTED, "dtype %d", dtype);
  BRK_REQUIRE(T > 0 && N >= 0 && Nk >= 0 && N + Nk > 0 && D > 0 && D % 16 == 0, BRK_E_ARG, "bad rope shape (head_dim must be a multiple of 16)");
  BRK_REQUIRE((q == nullptr || (((uintptr_t)q & 15) == 0 && q_row_stride % 8 == 0)) && (k == nullptr || (((uintptr_t)k & 15) == 0 && k_row_stride % 8 == 0)), BRK_E_ARG, "rope rows must be 16-byte aligned");
  BRK_REQUIRE(T * (D / 16) / 256 < (1ll << 31), BRK_E_ARG, "rope problem too large");
  return rope_launch(dtype, q, q_row_stride, N, k, k_row_stride, Nk, D, pos, inv_freq, T, (cudaStream_t)stream);
}

int brk_silu_mul(int32_t dtype, const void* gate_up, void* out, int64_t rows, int32_t inter, void* stream) {
  BRK_REQUIRE(gate_up && out, BRK_E_ARG, "null pointer");
  BRK_REQUIRE(dtype == BRK_BF16 || dtype == BRK_F32, BRK_E_UNSUPPORTED, "dtype %d", dtype);
  BRK_REQUIRE(rows > 0 && inter > 0 && inter % 8 == 0, BRK_E_ARG, "bad silu_mul shape rows=%lld inter=%d",
              (long long)rows, inter);
  BRK_REQUIRE(rows * (inter / 8) / 256 < (1ll << 31), BRK_E_ARG, "silu_mul problem too large");
  BRK_REQUIRE((((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0, BRK_E_ARG, "silu_mul buffers must be 16-byte aligned");
  return silu_mul_launch(dtype, gate_up, out, rows, inter, (cudaStream_t)stream);
}

}  // extern "C"
