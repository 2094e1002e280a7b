// extern "C" entry points of libfgattn_b200: argument checks, TMA tensor maps, launches.
#include <cuda_runtime.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <atomic>
#include <mutex>

#include "../../include/fgattn_b200.h"
#include "dense_attn.cuh"
#include "mask_kernels.cuh"
#include "packed_mask.cuh"
#include "selftest.cuh"
#include "sparse_attn.cuh"
#include "maxq_pass.cuh"
#include "sparse_ml_persistent.cuh"
#include "sparse_token_attn.cuh"
#include "tensor_map.h"
#include "token_blocks.cuh"
#include "topk_select.cuh"

// Scratch and error word of the allocation-free entry point live in the library image.  In host code
// the names below are host-side stand-ins, not device addresses: the device addresses are looked up
// once per device with cudaGetSymbolAddress and only those are handed to kernels.
static __device__ __align__(256) unsigned char g_noalloc_scratch[FGATTN_NOALLOC_SCRATCH_BYTES];
static __device__ __align__(256) int g_noalloc_err_word;

namespace {

thread_local int g_last_cuda_error = 0;
std::mutex g_mutex;
int* g_err_word[64] = {nullptr};
struct NoAllocAddrs {
  void* scratch = nullptr;
  int* err = nullptr;
};
NoAllocAddrs g_noalloc_addrs[64];

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = int(e);
  return FGATTN_CUDA_ERROR;
}
#define FG_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e__ = (call);                           \
    if (e__ != cudaSuccess) return cuda_fail(e__);      \
  } while (0)

// 4-byte per-device error word that bounded in-kernel waits write to.
int get_err_word(int** out) {
  int dev = 0;
  FG_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FGATTN_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_err_word[dev]) {
    int* p = nullptr;
    FG_CUDA(cudaMalloc(&p, sizeof(int)));
    FG_CUDA(cudaMemset(p, 0, sizeof(int)));
    g_err_word[dev] = p;
  }
  *out = g_err_word[dev];
  return FGATTN_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tuning overrides from the environment, read once per process: FGATTN_GROUP_HEADS (units per group of
// the longest-first thread-block orders; 0 = the built-in choice), FGATTN_DENSE_PERSIST (1 / 0 forces
// the persistent / one-item form of the dense family; -1 = by key length).
// fgattn_set_tuning overrides either for the rest of the process.
constexpr int kTuningUnset = -2147483647 - 1;
std::atomic<int> g_tune_group_heads{kTuningUnset}, g_tune_dense_persist{kTuningUnset}, g_tune_token_route{kTuningUnset},
    g_tune_dense_halves{kTuningUnset}, g_tune_maxq_wide{kTuningUnset};
int env_group_heads() {
  const int t = g_tune_group_heads.load(std::memory_order_relaxed);
  if (t != kTuningUnset) return t;
  static const int v = [] { const char* e = getenv("FGATTN_GROUP_HEADS"); return e ? atoi(e) : 0; }();
  return v;
}
// FGATTN_TOKEN_BLOCK_ROUTE=1 lets the token-list operator send query blocks with well-filled lists through
// whole K/V tiles (off by default: threshold-mask lists fill only 55-60 % of the blocks they touch, and for
// them the conversion costs more than it saves)
bool env_token_block_route() {
  const int t = g_tune_token_route.load(std::memory_order_relaxed);
  if (t != kTuningUnset) return t != 0;
  static const int v = [] { const char* e = getenv("FGATTN_TOKEN_BLOCK_ROUTE"); return e ? atoi(e) : 0; }();
  return v != 0;
}
// "dense_halves" (FGATTN_DENSE_HALVES): 0 = never cut the last wave's items in two
bool env_dense_halves() {
  const int t = g_tune_dense_halves.load(std::memory_order_relaxed);
  if (t != kTuningUnset) return t != 0;
  static const int v = [] { const char* e = getenv("FGATTN_DENSE_HALVES"); return e ? atoi(e) : 1; }();
  return v != 0;
}
// "maxq_wide" (FGATTN_MAXQ_WIDE): 0 sends the max / denominator pass and the token mask over all key tiles
// through modes kML / kTokenMask of the dense family instead of the two-threads-per-row kernel (maxq_pass.cuh)
// where their one-item form runs; -1 / 1 = the default
int env_maxq_wide() {
  const int t = g_tune_maxq_wide.load(std::memory_order_relaxed);
  if (t != kTuningUnset) return t;
  static const int v = [] { const char* e = getenv("FGATTN_MAXQ_WIDE"); return e ? atoi(e) : -1; }();
  return v;
}
int env_dense_persist() {
  const int t = g_tune_dense_persist.load(std::memory_order_relaxed);
  if (t != kTuningUnset) return t;
  static const int v = [] { const char* e = getenv("FGATTN_DENSE_PERSIST"); return e ? atoi(e) : -1; }();
  return v;
}

// S = query rows, kv_rows = rows of the k / v tensors per head, kv_len = leading k / v rows that take part
int check_qk(const void* q, const void* k, int B, int H, int S, int D, int kv_rows, int kv_len) {
  if (!q || !k) return FGATTN_INVALID_ARGUMENT;
  if (B <= 0 || H <= 0 || S <= 0 || kv_rows <= 0) return FGATTN_INVALID_ARGUMENT;
  if (D != 64 && D != 128) return FGATTN_UNSUPPORTED;
  if (kv_len < 1 || kv_len > kv_rows) return FGATTN_INVALID_ARGUMENT;
  if ((long long)B * H > 65535) return FGATTN_UNSUPPORTED;
  if (!aligned16(q) || !aligned16(k)) return FGATTN_MISALIGNED;
  return FGATTN_OK;
}

float resolve_scale_log2(float scale, int D) {
  const float s = (scale > 0.f) ? scale : 1.0f / sqrtf(float(D));
  return s * 1.4426950408889634f;
}

template <typename K>
int set_smem(K kernel, int bytes) {
  FG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return FGATTN_OK;
}

// Streaming multiprocessors of the current device (looked up once per device).
int sm_count(int* out) {
  static int cached[64] = {0};
  int dev = 0;
  FG_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || cached[dev] == 0) {
    int sms = 0;
    FG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (dev < 0 || dev >= 64) { *out = sms; return FGATTN_OK; }
    cached[dev] = sms;
  }
  *out = cached[dev];
  return FGATTN_OK;
}

// One launch of the dense family over heads [bh0, bh0 + nbh).  Work item = pair of 128-row query tiles
// of one unit.  PERSIST: one CTA per SM walks the items (pays off when an item has few key tiles, so
// that the CTA prologue and the first loads would otherwise dominate); else one CTA per item.
template <int D, int MODE, bool BLOCKMAX, bool PERSIST>
int launch_dense_k(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const fg::DenseParams& p,
                   int ctas, cudaStream_t st) {
  auto kern = fg::dense_attn_kernel<D, MODE, BLOCKMAX, PERSIST>;
  int r = set_smem(kern, fg::DenseCfg<D>::kSmemBytes);
  if (r) return r;
  kern<<<dim3(ctas, 1, 1), 384, fg::DenseCfg<D>::kSmemBytes, st>>>(mq, mk, mv, p);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

constexpr int kPersistMaxKeyTiles = 8;     // persistent CTAs up to 1024 keys
// The max / denominator pass alone stays persistent up to 2048 keys: measured against its one-item kernel
// (maxq_pass.cuh) at 32768 queries x 40 heads, D = 128 / 64: 1280 keys 16 / 12 % faster, 1536 keys 13 / 6 %,
// 2048 keys 10 / 4 %, 3072 keys level / 1 % slower
constexpr int kPersistMaxKeyTilesMaxq = 16;

// The max / denominator pass with two threads per row (maxq_pass.cuh); same parameters and grid as the
// one-item form of the dense family.
template <int D, bool BLOCKMAX, bool TOKENMASK>
int launch_maxq_wide(const CUtensorMap& mq, const CUtensorMap& mk, const fg::DenseParams& p, int ctas, cudaStream_t st) {
  auto kern = fg::maxq_pass_kernel<D, BLOCKMAX, TOKENMASK>;
  int r = set_smem(kern, fg::MaxqCfg<D>::kSmemBytes);
  if (r) return r;
  kern<<<dim3(ctas, 1, 1), fg::MaxqCfg<D>::kThreads, fg::MaxqCfg<D>::kSmemBytes, st>>>(mq, mk, p);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

template <int D, int MODE, bool BLOCKMAX>
int launch_dense_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const fg::DenseParams& p,
                   int nbh, cudaStream_t st) {
  fg::DenseParams pp = p;
  pp.n_pairs = (p.S + 255) / 256;
  pp.n_items = pp.n_pairs * nbh;
  if constexpr (MODE != fg::kTokenMask && !BLOCKMAX) {
    const int persist_env = env_dense_persist();
    const bool persist = persist_env >= 0 ? persist_env != 0
                                          : p.n_kv_tiles <= (MODE == fg::kML ? kPersistMaxKeyTilesMaxq : kPersistMaxKeyTiles);
    if (persist) {
      int sms = 0;
      int r = sm_count(&sms);
      if (r) return r;
      return launch_dense_k<D, MODE, BLOCKMAX, true>(mq, mk, mv, pp, pp.n_items < sms ? pp.n_items : sms, st);
    }
  }
  // One thread block per item.  When the last wave of thread blocks would be less than half full, its items
  // are cut into their two query tiles (DenseParams::half_from), so that the wave takes about half as long.
  int ctas = pp.n_items;
  pp.half_from = pp.n_items;
  if constexpr (MODE != fg::kTokenMask) {
    int sms = 0;
    int r = sm_count(&sms);
    if (r) return r;
    const int rest = pp.n_items % sms;
    if (rest > 0 && 2 * rest <= sms && env_dense_halves()) {
      pp.half_from = pp.n_items - rest;
      ctas = pp.half_from + 2 * rest;
    }
  }
  if constexpr (MODE == fg::kML || MODE == fg::kTokenMask) {
    const int wide_env = env_maxq_wide();
    // faster at every key length of the one-item form (1536 keys and up); the token mask on listed tiles, whose
    // items are a few tiles long, stays in the dense family
    if (wide_env != 0 && !(MODE == fg::kTokenMask && p.kb_idx != nullptr))
      return launch_maxq_wide<D, BLOCKMAX, MODE == fg::kTokenMask>(mq, mk, pp, ctas, st);
  }
  return launch_dense_k<D, MODE, BLOCKMAX, false>(mq, mk, mv, pp, ctas, st);
}

template <int MODE, bool BLOCKMAX>
int launch_dense(int D, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const fg::DenseParams& p,
                 int nbh, cudaStream_t st) {
  return D == 128 ? launch_dense_t<128, MODE, BLOCKMAX>(mq, mk, mv, p, nbh, st)
                  : launch_dense_t<64, MODE, BLOCKMAX>(mq, mk, mv, p, nbh, st);
}

struct DenseSetup {
  CUtensorMap mq, mk, mv;
  fg::DenseParams p;
};

int dense_setup(DenseSetup& s, const void* q, const void* k, const void* v, int B, int H, int S, int D, int kv_rows,
                int kv_len, float scale) {
  int r = check_qk(q, k, B, H, S, D, kv_rows, kv_len);
  if (r) return r;
  if (v && !aligned16(v)) return FGATTN_MISALIGNED;
  if (fg::make_qkv_map(&s.mq, q, B * H, S, D, 128) || fg::make_qkv_map(&s.mk, k, B * H, kv_rows, D, 128) ||
      fg::make_qkv_map(&s.mv, v ? v : k, B * H, kv_rows, D, 128))
    return fg::encode_tiled_fn() ? FGATTN_INVALID_ARGUMENT : FGATTN_NO_DRIVER;
  memset(&s.p, 0, sizeof(s.p));
  s.p.S = S;
  s.p.S_pad = ((S + 127) / 128) * 128;
  s.p.kv_len = kv_len;
  s.p.n_kv_tiles = (kv_len + 127) / 128;
  s.p.nkb = (kv_len + 63) / 64;
  s.p.scale_log2 = resolve_scale_log2(scale, D);
  return get_err_word(&s.p.err);
}

// Renormalising block-sparse attention (two-slot kernel).
// `redo` (optional, [B*H * ceil(S/128)] flags): re-run pass, only the marked pairs of query blocks are computed.
int launch_sparse(void* o, const void* q, const void* k, const void* v, const int* kb_idx, const int* kb_cnt,
                  int list_stride, int B, int H, int S, int D, int kv_rows, int kv_len, float scale, void* workspace,
                  size_t workspace_bytes, cudaStream_t st, const int* redo = nullptr,
                  const unsigned long long* kb_mask = nullptr) {
  int r = check_qk(q, k, B, H, S, D, kv_rows, kv_len);
  if (r) return r;
  if (!o || !v || !kb_idx || !kb_cnt) return FGATTN_INVALID_ARGUMENT;
  if (!aligned16(o) || !aligned16(v)) return FGATTN_MISALIGNED;
  if (workspace && !aligned16(workspace)) return FGATTN_MISALIGNED;
  if (workspace && workspace_bytes < fgattn_sp_attn_workspace_bytes(B, H, S)) return FGATTN_SCRATCH_TOO_SMALL;
  fg::SparseParams p;
  memset(&p, 0, sizeof(p));
  p.o = static_cast<__nv_bfloat16*>(o);
  p.kb_idx = kb_idx;
  p.kb_cnt = kb_cnt;
  p.S = S;
  p.S_pad = ((S + 127) / 128) * 128;
  p.kv_len = kv_len;
  p.nqb = (S + 63) / 64;
  p.nkb = (kv_len + 63) / 64;
  p.list_stride = list_stride;
  p.list_cap = p.nkb + 2;
  p.scale_log2 = resolve_scale_log2(scale, D);
  if (list_stride < 1) return FGATTN_INVALID_ARGUMENT;
  r = get_err_word(&p.err);
  if (r) return r;
  CUtensorMap mq, mk, mv;
  if (fg::make_qkv_map(&mq, q, B * H, S, D, 128) || fg::make_qkv_map(&mk, k, B * H, kv_rows, D, 64) ||
      fg::make_qkv_map(&mv, v, B * H, kv_rows, D, 64))
    return fg::encode_tiled_fn() ? FGATTN_INVALID_ARGUMENT : FGATTN_NO_DRIVER;
  p.quads = (S + 255) / 256;
  p.redo = redo;
  p.kb_mask = kb_mask;                   // token-derived lists: one list (with column masks) per 128-row block
  p.npairs = (S + 127) / 128;
  const int n_units = B * H;
  if ((long long)n_units * p.quads > 2147483647LL) return FGATTN_UNSUPPORTED;
  if (workspace) {
    // CTA order: units in groups whose K/V (<= 64 MiB) stays in L2, inside a group longest lists first
    const size_t kv_bytes_per_unit = size_t(4) * kv_rows * D;
    int group = int(std::max<size_t>(1, (size_t(64) << 20) / kv_bytes_per_unit));
    if (env_group_heads() > 0) group = env_group_heads();                // tuning override
    group = std::max(1, std::min(group, n_units));
    const int n_groups = (n_units + group - 1) / group;
    group = (n_units + n_groups - 1) / n_groups;                      // groups of equal size
    int* ws = static_cast<int*>(workspace);
    fg::sparse_order_kernel<<<(n_units + group - 1) / group, 256, 0, st>>>(kb_cnt, ws + 4, ws, p.nqb, p.quads, n_units,
                                                                          group, 2, 2, 0);
    FG_CUDA(cudaGetLastError());
    p.order = ws + 4;
  }
  p.n_total = n_units * p.quads;
  int n_ctas = p.n_total;                       // one CTA per item; the re-run pass: at most one per SM
  if (redo) {
    int sms = 0;
    r = sm_count(&sms);
    if (r) return r;
    n_ctas = std::min(p.n_total, sms);
  }
  const int smem = (D == 128) ? fg::SparseCfg<128>::smem_bytes(p.list_cap, p.nkb)
                              : fg::SparseCfg<64>::smem_bytes(p.list_cap, p.nkb);
  if (smem > 232448) return FGATTN_UNSUPPORTED;
  auto go = [&](auto kern) -> int {
    int rr = set_smem(kern, smem);
    if (rr) return rr;
    kern<<<dim3(n_ctas, 1, 1), 384, smem, st>>>(mq, mk, mv, p);
    return FGATTN_OK;
  };
  if (D == 128) r = redo ? go(fg::sparse_block_attn_kernel<128, true>) : go(fg::sparse_block_attn_kernel<128, false>);
  else r = redo ? go(fg::sparse_block_attn_kernel<64, true>) : go(fg::sparse_block_attn_kernel<64, false>);
  if (r) return r;
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

}  // namespace

extern "C" {

namespace {
int launch_sparse_persistent(bool renorm, void* o, const void* q, const void* k, const void* v, const int* kb_indices,
                             const int* kb_counts, int list_stride, const float* max_q, const float* denom, int batch,
                             int heads, int seq, int D, int kv_rows, int kv_seq_len, float scale, void* workspace,
                             size_t workspace_bytes, void* stream, const unsigned long long* kb_mask = nullptr,
                             const int* route = nullptr);
}  // namespace

const char* fgattn_status_string(int status) {
  switch (status) {
    case FGATTN_OK: return "ok";
    case FGATTN_INVALID_ARGUMENT: return "invalid argument";
    case FGATTN_UNSUPPORTED: return "unsupported shape or size";
    case FGATTN_MISALIGNED: return "tensor base address is not 16-byte aligned";
    case FGATTN_CUDA_ERROR: return "CUDA error";
    case FGATTN_NO_DRIVER: return "CUDA driver tensor-map encoder not available";
    case FGATTN_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
    case FGATTN_SCRATCH_TOO_SMALL: return "scratch buffer too small";
    default: return "unknown status";
  }
}

int fgattn_last_cuda_error(void) { return g_last_cuda_error; }

int fgattn_set_tuning(const char* name, int value) {
  if (!name) return FGATTN_INVALID_ARGUMENT;
  if (!strcmp(name, "group_heads")) g_tune_group_heads.store(value < 0 ? kTuningUnset : value);
  else if (!strcmp(name, "dense_persist")) g_tune_dense_persist.store(value < -1 ? kTuningUnset : value);
  else if (!strcmp(name, "token_block_route")) g_tune_token_route.store(value < 0 ? kTuningUnset : value);
  else if (!strcmp(name, "dense_halves")) g_tune_dense_halves.store(value < 0 ? kTuningUnset : value);
  else if (!strcmp(name, "maxq_wide")) g_tune_maxq_wide.store(value < -1 ? kTuningUnset : value);
  else return FGATTN_INVALID_ARGUMENT;
  return FGATTN_OK;
}

int fgattn_check(void* stream, int* code) {
  // Two words can hold a time-out: the allocated one that most entry points use, and the one built into
  // the library that the allocation-free entry point uses while the first does not exist.  Only words that
  // some call has put to use are read, so this function itself never allocates.
  int dev = 0;
  FG_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FGATTN_UNSUPPORTED;
  int* words[2];
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    words[0] = g_err_word[dev];
    words[1] = g_noalloc_addrs[dev].err;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  FG_CUDA(cudaStreamSynchronize(st));
  int first = 0;
  for (int* w : words) {
    if (!w) continue;
    int h = 0;
    FG_CUDA(cudaMemcpy(&h, w, sizeof(int), cudaMemcpyDeviceToHost));
    if (h != 0) {
      FG_CUDA(cudaMemset(w, 0, sizeof(int)));
      if (first == 0) first = h;
    }
  }
  if (code) *code = first;
  return first != 0 ? FGATTN_DEVICE_TIMEOUT : FGATTN_OK;
}

int fgattn_full_attn(void* o, const void* q, const void* k, const void* v, int batch, int heads, int seq, int D,
                     int kv_rows, int kv_seq_len, float scale, void* stream) {
  if (!o || !v) return FGATTN_INVALID_ARGUMENT;
  if (!aligned16(o)) return FGATTN_MISALIGNED;
  DenseSetup s;
  int r = dense_setup(s, q, k, v, batch, heads, seq, D, kv_rows, kv_seq_len, scale);
  if (r) return r;
  s.p.o = static_cast<__nv_bfloat16*>(o);
  return launch_dense<fg::kFull, false>(D, s.mq, s.mk, s.mv, s.p, batch * heads, static_cast<cudaStream_t>(stream));
}

int fgattn_fullattn_maxq_denom(void* o, float* max_q, float* denom, const void* q, const void* k, const void* v,
                               int batch, int heads, int seq, int D, int kv_rows, int kv_seq_len, float scale,
                               void* stream) {
  if (!o || !v || !max_q || !denom) return FGATTN_INVALID_ARGUMENT;
  if (!aligned16(o)) return FGATTN_MISALIGNED;
  DenseSetup s;
  int r = dense_setup(s, q, k, v, batch, heads, seq, D, kv_rows, kv_seq_len, scale);
  if (r) return r;
  s.p.o = static_cast<__nv_bfloat16*>(o);
  s.p.max_q = max_q;
  s.p.denom = denom;
  return launch_dense<fg::kFullML, false>(D, s.mq, s.mk, s.mv, s.p, batch * heads, static_cast<cudaStream_t>(stream));
}

int fgattn_maxq_denom(float* max_q, float* denom, const void* q, const void* k, int batch, int heads, int seq, int D,
                      int kv_rows, int kv_seq_len, float scale, void* stream) {
  if (!max_q || !denom) return FGATTN_INVALID_ARGUMENT;
  DenseSetup s;
  int r = dense_setup(s, q, k, nullptr, batch, heads, seq, D, kv_rows, kv_seq_len, scale);
  if (r) return r;
  s.p.max_q = max_q;
  s.p.denom = denom;
  return launch_dense<fg::kML, false>(D, s.mq, s.mk, s.mv, s.p, batch * heads, static_cast<cudaStream_t>(stream));
}

namespace {
int token_mask_launch(int* booleanmask, float threshold, int mask_stride, const float* max_q, const float* denom,
                      const void* q, const void* k, const int* kb_indices, const int* kb_counts, int list_stride,
                      int batch, int heads, int seq, int D, int kv_rows, int kv_seq_len, float scale, void* workspace,
                      size_t workspace_bytes, void* stream) {
  if (!booleanmask || !max_q || !denom || !(threshold > 0.f)) return FGATTN_INVALID_ARGUMENT;
  if (mask_stride < kv_seq_len) return FGATTN_INVALID_ARGUMENT;
  if (workspace && !aligned16(workspace)) return FGATTN_MISALIGNED;
  if (workspace && workspace_bytes < fgattn_sp_attn_workspace_bytes(batch, heads, seq)) return FGATTN_SCRATCH_TOO_SMALL;
  DenseSetup s;
  int r = dense_setup(s, q, k, nullptr, batch, heads, seq, D, kv_rows, kv_seq_len, scale);
  if (r) return r;
  if (kb_indices) {
    if (!kb_counts || list_stride < 1) return FGATTN_INVALID_ARGUMENT;
    if (s.p.n_kv_tiles > fg::DenseCfg<128>::kMaxListedTiles) return FGATTN_UNSUPPORTED;
    s.p.kb_idx = kb_indices;
    s.p.kb_cnt = kb_counts;
    s.p.list_stride = list_stride;
    s.p.nqb64 = (seq + 63) / 64;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t n = size_t(batch) * heads * ((seq + 127) / 128) * mask_stride;
  FG_CUDA(cudaMemsetAsync(booleanmask, 0, n * sizeof(int), st));
  s.p.max_q = const_cast<float*>(max_q);
  s.p.denom = const_cast<float*>(denom);
  s.p.tokenmask = booleanmask;
  s.p.mask_stride = mask_stride;
  s.p.log2_tau = log2f(threshold);
  if (kb_indices && workspace) {
    // thread-block order: inside groups of units the items (four 64-row query blocks) with the longest
    // lists first.  Large groups balance better than small ones keep K in L2 (measured at
    // (1,12,32760,128): storage order 0.58 ms, 3 heads per group 0.57, 6: 0.50, all 12: 0.40).
    const int n_units = batch * heads, quads = (seq + 255) / 256;
    const size_t k_bytes_per_unit = size_t(4) * kv_rows * D;
    int group = int(std::max<size_t>(1, (size_t(256) << 20) / k_bytes_per_unit));
    if (env_group_heads() > 0) group = env_group_heads();                // tuning override
    group = std::max(1, std::min(group, n_units));
    const int n_groups = (n_units + group - 1) / group;
    group = (n_units + n_groups - 1) / n_groups;
    int shift = 0;
    while (((4 * s.p.nkb) >> shift) >= 1024) ++shift;
    int* ws = static_cast<int*>(workspace);
    fg::sparse_order_kernel<<<(n_units + group - 1) / group, 256, 0, st>>>(kb_counts, ws + 4, ws, s.p.nqb64, quads, n_units,
                                                                          group, 1, 4, shift);
    FG_CUDA(cudaGetLastError());
    s.p.order = ws + 4;
  }
  return launch_dense<fg::kTokenMask, false>(D, s.mq, s.mk, s.mv, s.p, batch * heads, st);
}
}  // namespace

int fgattn_booleanmask_128(int* booleanmask, float threshold, int mask_stride, const float* max_q, const float* denom,
                           const void* q, const void* k, int batch, int heads, int seq, int D, int kv_rows,
                           int kv_seq_len, float scale, void* stream) {
  return token_mask_launch(booleanmask, threshold, mask_stride, max_q, denom, q, k, nullptr, nullptr, 0, batch, heads,
                           seq, D, kv_rows, kv_seq_len, scale, nullptr, 0, stream);
}

int fgattn_booleanmask_128_listed(int* booleanmask, float threshold, int mask_stride, const float* max_q,
                                  const float* denom, const void* q, const void* k, const int* kb_indices,
                                  const int* kb_counts, int list_stride, int batch, int heads, int seq, int D,
                                  int kv_rows, int kv_seq_len, float scale, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  if (!kb_indices || !kb_counts) return FGATTN_INVALID_ARGUMENT;
  return token_mask_launch(booleanmask, threshold, mask_stride, max_q, denom, q, k, kb_indices, kb_counts, list_stride,
                           batch, heads, seq, D, kv_rows, kv_seq_len, scale, workspace, workspace_bytes, stream);
}

int fgattn_booleanmask_to_indexmask(int* kv_indices, int* kv_num_indices, const int* booleanmask, int batch, int heads,
                                    int seq, int seqblocks, int mask_stride, void* stream) {
  if (!kv_indices || !kv_num_indices || !booleanmask) return FGATTN_INVALID_ARGUMENT;
  if (batch <= 0 || heads <= 0 || seqblocks <= 0 || mask_stride <= 0 || seq < 0) return FGATTN_INVALID_ARGUMENT;
  const long long rows = (long long)batch * heads * seqblocks;
  if (rows > 2147483647LL) return FGATTN_UNSUPPORTED;
  fg::mask_to_index_kernel<<<unsigned(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      booleanmask, kv_indices, kv_num_indices, mask_stride, seq);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

int fgattn_all_index_mask(int* kv_indices, int* kv_num_indices, int batch, int heads, int seqblocks, int seq,
                          int index_stride, void* stream) {
  if (!kv_indices || !kv_num_indices) return FGATTN_INVALID_ARGUMENT;
  if (batch <= 0 || heads <= 0 || seqblocks <= 0 || index_stride <= 0 || seq < 0) return FGATTN_INVALID_ARGUMENT;
  const long long rows = (long long)batch * heads * seqblocks;
  if (rows > 2147483647LL) return FGATTN_UNSUPPORTED;
  fg::identity_index_kernel<<<unsigned(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(kv_indices, kv_num_indices,
                                                                                          index_stride, seq);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

int fgattn_sp_attn(void* o, const void* q, const void* k, const void* v, const int* kv_indices,
                   const int* kv_num_indices, int mask_stride, int batch, int heads, int seq, int D, int kv_rows,
                   float scale, void* workspace, size_t workspace_bytes, void* stream) {
  int r = check_qk(q, k, batch, heads, seq, D, kv_rows, kv_rows);
  if (r) return r;
  if (!o || !v || !kv_indices || !kv_num_indices || mask_stride < 1) return FGATTN_INVALID_ARGUMENT;
  if (!aligned16(o) || !aligned16(v)) return FGATTN_MISALIGNED;
  if (workspace && !aligned16(workspace)) return FGATTN_MISALIGNED;
  if (workspace && workspace_bytes < fgattn_sp_attn_workspace_bytes(batch, heads, seq)) return FGATTN_SCRATCH_TOO_SMALL;
  fg::TokenParams p;
  memset(&p, 0, sizeof(p));
  p.o = static_cast<__nv_bfloat16*>(o);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.kv_idx = kv_indices;
  p.kv_cnt = kv_num_indices;
  p.S = seq;
  p.S_kv = kv_rows;
  p.nqb = (seq + 127) / 128;
  p.mask_stride = mask_stride;
  p.scale_log2 = resolve_scale_log2(scale, D);
  r = get_err_word(&p.err);
  if (r) return r;
  CUtensorMap mq;
  if (fg::make_qkv_map(&mq, q, batch * heads, seq, D, 128))
    return fg::encode_tiled_fn() ? FGATTN_INVALID_ARGUMENT : FGATTN_NO_DRIVER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  p.pairs = (seq + 255) / 256;
  const int n_units = batch * heads;
  if ((long long)n_units * p.pairs > 2147483647LL) return FGATTN_UNSUPPORTED;
  // ---- block route: with the large workspace, query blocks whose lists nearly fill the 64-key blocks they
  // touch are computed from whole K/V tiles (TMA by block index, unlisted columns switched off) on the
  // persistent fixed-offset kernel; the others stay on the row gather below
  const int nkb = (kv_rows + 63) / 64, nqb = p.nqb, s_pad = nqb * 128;
  const size_t pre_smem = fg::token_blocks_smem_bytes(nkb, D);
  const int ml_smem = (D == 128) ? fg::SparseMLCfg<128>::smem_bytes(nkb + 2, nkb) : fg::SparseMLCfg<64>::smem_bytes(nkb + 2, nkb);
  const int two_smem = (D == 128) ? fg::SparseCfg<128>::smem_bytes(nkb + 2, nkb) : fg::SparseCfg<64>::smem_bytes(nkb + 2, nkb);
  const bool block_route = workspace && workspace_bytes >= fgattn_sp_attn_token_workspace_bytes(batch, heads, seq, kv_rows) &&
                           pre_smem <= 48 * 1024 && ml_smem <= 232448 && two_smem <= 232448 && env_token_block_route();
  if (block_route) {
    char* base = static_cast<char*>(workspace);
    const size_t small = align256(fgattn_sp_attn_workspace_bytes(batch, heads, seq));
    const size_t n_rows = size_t(n_units) * nqb;
    char* w_ml = base + small;                                   // queue / order / re-run flags of the block route
    int* kb_cnt2 = reinterpret_cast<int*>(base + 2 * small);
    int* route = reinterpret_cast<int*>(base + 2 * small + align256(n_rows * 4));
    float* hint = reinterpret_cast<float*>(base + 2 * small + 2 * align256(n_rows * 4));
    int* kb_idx2 = reinterpret_cast<int*>(reinterpret_cast<char*>(hint) + align256(size_t(n_units) * s_pad * 4));
    unsigned long long* kb_mask2 =
        reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(kb_idx2) + align256(n_rows * nkb * 4));
    fg::TokenBlocksParams tb;
    memset(&tb, 0, sizeof(tb));
    tb.kv_idx = kv_indices;
    tb.kv_cnt = kv_num_indices;
    tb.q = static_cast<const __nv_bfloat16*>(q);
    tb.k = static_cast<const __nv_bfloat16*>(k);
    tb.kb_idx = kb_idx2;
    tb.kb_mask = kb_mask2;
    tb.kb_cnt = kb_cnt2;
    tb.route = route;
    tb.hint = hint;
    tb.S = seq;
    tb.S_pad = s_pad;
    tb.S_kv = kv_rows;
    tb.nqb = nqb;
    tb.nkb = nkb;
    tb.mask_stride = mask_stride;
    tb.kb_stride = nkb;
    // whole tiles pay when the listed columns fill most of them: the block route computes every column of
    // a touched block at about 1.5 times the row gather's rate per column
    tb.fill_min = 0.75f;
    // the sampled maximum is a lower estimate of the row maximum: shift the exponent window up by 2^20
    tb.hint_margin = 20.0f / p.scale_log2;
    if (D == 128) fg::token_lists_to_blocks_kernel<128><<<dim3(nqb, n_units), 256, pre_smem, st>>>(tb);
    else fg::token_lists_to_blocks_kernel<64><<<dim3(nqb, n_units), 256, pre_smem, st>>>(tb);
    FG_CUDA(cudaGetLastError());
    r = launch_sparse_persistent(true, o, q, k, v, kb_idx2, kb_cnt2, nkb, hint, nullptr, batch, heads, seq, D, kv_rows,
                                 kv_rows, scale, w_ml, small, stream, kb_mask2, route);
    if (r) return r;
    p.route = route;
  }
  if (workspace) {
    // thread-block order: inside groups of units, longest lists first.  The row gather gains little from
    // L2 residency of K/V, and large groups balance better (measured at (1,12,32760,128): 0.90 ms in
    // storage order, 0.77 ms with 4 heads per group, 0.55 ms with all 12), so groups span up to 256 MiB of K/V.
    const size_t kv_bytes_per_unit = size_t(4) * kv_rows * D;
    int group = int(std::max<size_t>(1, (size_t(256) << 20) / kv_bytes_per_unit));
    if (env_group_heads() > 0) group = env_group_heads();                // tuning override
    group = std::max(1, std::min(group, n_units));
    const int n_groups = (n_units + group - 1) / group;
    group = (n_units + n_groups - 1) / n_groups;                      // groups of equal size
    int shift = 0;
    while ((mask_stride >> shift) >= 1024) ++shift;                   // bucketed list lengths
    int* ws = static_cast<int*>(workspace);
    fg::sparse_order_kernel<<<(n_units + group - 1) / group, 256, 0, st>>>(kv_num_indices, ws + 4, ws, p.nqb, p.pairs,
                                                                          n_units, group, 2, 1, shift);
    FG_CUDA(cudaGetLastError());
    p.order = ws + 4;
  }
  dim3 grid(n_units * p.pairs, 1, 1);
  if (D == 128) {
    auto kern = fg::sparse_token_attn_kernel<128>;
    r = set_smem(kern, fg::TokenCfg<128>::kSmemBytes);
    if (r) return r;
    kern<<<grid, fg::TokenCfg<128>::kThreads, fg::TokenCfg<128>::kSmemBytes, st>>>(mq, p);
  } else {
    auto kern = fg::sparse_token_attn_kernel<64>;
    r = set_smem(kern, fg::TokenCfg<64>::kSmemBytes);
    if (r) return r;
    kern<<<grid, fg::TokenCfg<64>::kThreads, fg::TokenCfg<64>::kSmemBytes, st>>>(mq, p);
  }
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

size_t fgattn_sp_attn_token_workspace_bytes(int batch, int heads, int seq, int kv_rows) {
  if (batch <= 0 || heads <= 0 || seq <= 0 || kv_rows <= 0) return 0;
  // two queue / order regions (block route and row gather), then per query block: touched-block count and
  // route flag; per query row: exponent hint; per (query block, key block): block index and column mask
  const size_t small = align256(fgattn_sp_attn_workspace_bytes(batch, heads, seq));
  const size_t nqb = size_t((seq + 127) / 128), nkb = size_t((kv_rows + 63) / 64), bh = size_t(batch) * heads;
  return 2 * small + 2 * align256(bh * nqb * 4) + align256(bh * nqb * 128 * 4) + align256(bh * nqb * nkb * 4) +
         align256(bh * nqb * nkb * 8);
}

size_t fgattn_block_scratch_bytes(int batch, int heads, int seq, int kv_seq_len) {
  if (batch <= 0 || heads <= 0 || seq <= 0 || kv_seq_len <= 0) return 0;
  const size_t s_pad = size_t((seq + 127) / 128) * 128, nkb = size_t((kv_seq_len + 63) / 64);
  return size_t(batch) * heads * nkb * s_pad * sizeof(float);
}

int fgattn_block_index_lists(int* kb_indices, int* kb_counts, int list_stride, float* max_q, float* denom, void* o,
                             const void* q, const void* k, const void* v, float threshold, int batch, int heads,
                             int seq, int D, int kv_rows, int kv_seq_len, float scale, void* scratch,
                             size_t scratch_bytes, void* stream) {
  if (!kb_indices || !kb_counts || !max_q || !denom || !scratch || !(threshold > 0.f)) return FGATTN_INVALID_ARGUMENT;
  if ((o == nullptr) != (v == nullptr)) return FGATTN_INVALID_ARGUMENT;
  if (o && !aligned16(o)) return FGATTN_MISALIGNED;
  DenseSetup s;
  int r = dense_setup(s, q, k, v, batch, heads, seq, D, kv_rows, kv_seq_len, scale);
  if (r) return r;
  const int nkb = s.p.nkb, nqb = (seq + 63) / 64;
  if (list_stride < nkb) return FGATTN_INVALID_ARGUMENT;
  const size_t per_head = size_t(nkb) * s.p.S_pad * sizeof(float);
  const int chunk = int(std::min<size_t>(scratch_bytes / per_head, size_t(batch) * heads));
  if (chunk < 1) return FGATTN_SCRATCH_TOO_SMALL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  s.p.o = static_cast<__nv_bfloat16*>(o);
  s.p.max_q = max_q;
  s.p.denom = denom;
  s.p.blockmax = static_cast<float*>(scratch);
  const float log2_tau = log2f(threshold);
  const int total = batch * heads;
  for (int bh0 = 0; bh0 < total; bh0 += chunk) {
    const int n = std::min(chunk, total - bh0);
    s.p.bh0 = bh0;
    r = o ? launch_dense<fg::kFullML, true>(D, s.mq, s.mk, s.mv, s.p, n, st)
          : launch_dense<fg::kML, true>(D, s.mq, s.mk, s.mv, s.p, n, st);
    if (r) return r;
    const int smem = 64 * int(sizeof(float)) + ((nkb + 15) / 16) * 16;
    fg::block_threshold_compact_kernel<<<dim3(nqb, n), 256, smem, st>>>(
        s.p.blockmax, max_q, denom, kb_indices, kb_counts, seq, s.p.S_pad, nqb, nkb, list_stride, bh0, s.p.scale_log2,
        log2_tau);
    FG_CUDA(cudaGetLastError());
  }
  return FGATTN_OK;
}

int fgattn_block_lists_from_maxima(int* kb_indices, int* kb_counts, int list_stride, const float* block_maxima,
                                   const float* max_q, const float* denom, float threshold, int batch, int heads,
                                   int seq, int D, int kv_seq_len, float scale, void* stream) {
  if (!kb_indices || !kb_counts || !block_maxima || !max_q || !denom || !(threshold > 0.f)) return FGATTN_INVALID_ARGUMENT;
  if (batch <= 0 || heads <= 0 || seq <= 0 || kv_seq_len <= 0) return FGATTN_INVALID_ARGUMENT;
  if (D != 64 && D != 128) return FGATTN_UNSUPPORTED;
  if ((long long)batch * heads > 65535) return FGATTN_UNSUPPORTED;
  const int nkb = (kv_seq_len + 63) / 64, nqb = (seq + 63) / 64, s_pad = ((seq + 127) / 128) * 128;
  if (list_stride < nkb) return FGATTN_INVALID_ARGUMENT;
  const int smem = 64 * int(sizeof(float)) + ((nkb + 15) / 16) * 16;
  fg::block_threshold_compact_kernel<<<dim3(nqb, batch * heads), 256, smem, static_cast<cudaStream_t>(stream)>>>(
      block_maxima, max_q, denom, kb_indices, kb_counts, seq, s_pad, nqb, nkb, list_stride, 0, resolve_scale_log2(scale, D),
      log2f(threshold));
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

// ---- allocation-free variant of fgattn_block_index_lists --------------------------------------
namespace {
// First use on a device: resolve the device addresses of the built-in arrays (no allocation).
int noalloc_addrs(NoAllocAddrs* out) {
  int dev = 0;
  FG_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FGATTN_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mutex);
  NoAllocAddrs& a = g_noalloc_addrs[dev];
  if (!a.scratch) {
    void* sp = nullptr;
    void* ep = nullptr;
    FG_CUDA(cudaGetSymbolAddress(&sp, g_noalloc_scratch));
    FG_CUDA(cudaGetSymbolAddress(&ep, g_noalloc_err_word));
    a.err = static_cast<int*>(ep);
    a.scratch = sp;
  }
  // prefer the word fgattn_check reads when an earlier call already created it
  out->scratch = a.scratch;
  out->err = g_err_word[dev] ? g_err_word[dev] : a.err;
  return FGATTN_OK;
}
}  // namespace

int fgattn_block_index_lists_noalloc(int* kb_indices, int* kb_counts, int list_stride, float* max_q, float* denom,
                                     void* o, const void* q, const void* k, const void* v, float threshold,
                                     int batch, int heads, int seq, int D, int kv_seq_len, float scale, void* stream) {
  if (!kb_indices || !kb_counts || !max_q || !denom || !(threshold > 0.f)) return FGATTN_INVALID_ARGUMENT;
  if ((o == nullptr) != (v == nullptr)) return FGATTN_INVALID_ARGUMENT;
  if (o && !aligned16(o)) return FGATTN_MISALIGNED;
  int r = check_qk(q, k, batch, heads, seq, D, seq, kv_seq_len);
  if (r) return r;
  if (v && !aligned16(v)) return FGATTN_MISALIGNED;
  const int nkb = (kv_seq_len + 63) / 64, nqb = (seq + 63) / 64, s_pad = ((seq + 127) / 128) * 128;
  if (list_stride < nkb) return FGATTN_INVALID_ARGUMENT;
  // reject sizes beyond the built-in maximum before anything is launched
  const size_t per_head = size_t(nkb) * s_pad * sizeof(float);
  if (per_head > size_t(FGATTN_NOALLOC_SCRATCH_BYTES)) return FGATTN_SCRATCH_TOO_SMALL;
  const int chunk = int(std::min<size_t>(size_t(FGATTN_NOALLOC_SCRATCH_BYTES) / per_head, size_t(batch) * heads));
  NoAllocAddrs addrs;
  r = noalloc_addrs(&addrs);
  if (r) return r;
  DenseSetup s;
  if (fg::make_qkv_map(&s.mq, q, batch * heads, seq, D, 128) || fg::make_qkv_map(&s.mk, k, batch * heads, seq, D, 128) ||
      fg::make_qkv_map(&s.mv, v ? v : k, batch * heads, seq, D, 128))
    return fg::encode_tiled_fn() ? FGATTN_INVALID_ARGUMENT : FGATTN_NO_DRIVER;
  memset(&s.p, 0, sizeof(s.p));
  s.p.S = seq;
  s.p.S_pad = s_pad;
  s.p.kv_len = kv_seq_len;
  s.p.n_kv_tiles = (kv_seq_len + 127) / 128;
  s.p.nkb = nkb;
  s.p.scale_log2 = resolve_scale_log2(scale, D);
  s.p.err = addrs.err;
  s.p.o = static_cast<__nv_bfloat16*>(o);
  s.p.max_q = max_q;
  s.p.denom = denom;
  s.p.blockmax = static_cast<float*>(addrs.scratch);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float log2_tau = log2f(threshold);
  const int total = batch * heads;
  for (int bh0 = 0; bh0 < total; bh0 += chunk) {
    const int n = std::min(chunk, total - bh0);
    s.p.bh0 = bh0;
    r = o ? launch_dense<fg::kFullML, true>(D, s.mq, s.mk, s.mv, s.p, n, st)
          : launch_dense<fg::kML, true>(D, s.mq, s.mk, s.mv, s.p, n, st);
    if (r) return r;
    const int smem = 64 * int(sizeof(float)) + ((nkb + 15) / 16) * 16;
    fg::block_threshold_compact_kernel<<<dim3(nqb, n), 256, smem, st>>>(
        s.p.blockmax, max_q, denom, kb_indices, kb_counts, seq, s_pad, nqb, nkb, list_stride, bh0, s.p.scale_log2,
        log2_tau);
    FG_CUDA(cudaGetLastError());
  }
  return FGATTN_OK;
}

size_t fgattn_sp_attn_workspace_bytes(int batch, int heads, int seq) {
  if (batch <= 0 || heads <= 0 || seq <= 0) return 0;
  // [0, 4): queue counter (+ padding); then the processing order of the items; then their re-run flags
  const size_t npairs = size_t((seq + 127) / 128);
  return 16 + 2 * size_t(batch) * heads * npairs * sizeof(int);
}

namespace {
// The persistent block-sparse kernel in its two forms: probabilities from the given (max_q, denom), or
// (renorm) renormalised over the kept keys with max_q as the fixed per-row exponent offset, followed by
// the re-run pass over the items that left the safe exponent range.
int launch_sparse_persistent(bool renorm, void* o, const void* q, const void* k, const void* v, const int* kb_indices,
                             const int* kb_counts, int list_stride, const float* max_q, const float* denom, int batch,
                             int heads, int seq, int D, int kv_rows, int kv_seq_len, float scale, void* workspace,
                             size_t workspace_bytes, void* stream, const unsigned long long* kb_mask,
                             const int* route) {
  int r = check_qk(q, k, batch, heads, seq, D, kv_rows, kv_seq_len);
  if (r) return r;
  if (!o || !v || !kb_indices || !kb_counts || !max_q || (!renorm && !denom) || !workspace || list_stride < 1)
    return FGATTN_INVALID_ARGUMENT;
  if (!aligned16(o) || !aligned16(v) || !aligned16(workspace)) return FGATTN_MISALIGNED;
  if (workspace_bytes < fgattn_sp_attn_workspace_bytes(batch, heads, seq)) return FGATTN_SCRATCH_TOO_SMALL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  fg::SparseMLParams p;
  memset(&p, 0, sizeof(p));
  p.o = static_cast<__nv_bfloat16*>(o);
  p.max_q = max_q;
  p.denom = denom;
  p.kb_idx = kb_indices;
  p.kb_cnt = kb_counts;
  p.kb_mask = kb_mask;
  p.route = route;
  p.S = seq;
  p.S_pad = ((seq + 127) / 128) * 128;
  p.kv_len = kv_seq_len;
  p.nqb = (seq + 63) / 64;
  p.nkb = (kv_seq_len + 63) / 64;
  p.npairs = (seq + 127) / 128;
  p.n_items = batch * heads * p.npairs;
  p.queue = static_cast<int*>(workspace);
  p.order = static_cast<int*>(workspace) + 4;
  p.redo = static_cast<int*>(workspace) + 4 + p.n_items;
  p.list_stride = list_stride;
  p.list_cap = p.nkb + 2;
  p.scale_log2 = resolve_scale_log2(scale, D);
#ifdef FG_STATS
  if (const char* dbg = getenv("FGATTN_DEBUG_SPARSE")) p.debug = atoi(dbg);
  if ((p.debug & 8) && workspace_bytes >= fgattn_sp_attn_workspace_bytes(batch, heads, seq) + 256 * 32 * 8 + 64)
    p.stats = reinterpret_cast<long long*>(static_cast<char*>(workspace) +
                                           ((fgattn_sp_attn_workspace_bytes(batch, heads, seq) + 63) / 64) * 64);
#endif
  r = get_err_word(&p.err);
  if (r) return r;
  CUtensorMap mq, mk, mv;
  if (fg::make_qkv_map(&mq, q, batch * heads, seq, D, 128) || fg::make_qkv_map(&mk, k, batch * heads, kv_rows, D, 64) ||
      fg::make_qkv_map(&mv, v, batch * heads, kv_rows, D, 64))
    return fg::encode_tiled_fn() ? FGATTN_INVALID_ARGUMENT : FGATTN_NO_DRIVER;
  int sms = 0;
  r = sm_count(&sms);
  if (r) return r;
  // Queue order: units in groups whose K/V (<= 56 MiB) stays in L2, longest items first inside a group.
  // The end of the launch is made of the last group's short items, and a small last group runs out of
  // them while long items are still going, so the last group also takes the remainder (it holds between
  // one and two groups' worth of units) and a launch with few items per SM is one single group
  // (measured on the first 16 heads of C3: 0.39 ms in groups of 6,6,4 heads, 0.34 ms as one group).
  const int n_units = batch * heads;
  const size_t kv_bytes_per_unit = size_t(4) * kv_rows * D;
  int group_heads = int(std::max<size_t>(1, (size_t(56) << 20) / kv_bytes_per_unit));
  if (p.n_items < 16 * sms) group_heads = n_units;
  if (env_group_heads() > 0) group_heads = env_group_heads();            // tuning override
  group_heads = std::max(1, std::min(group_heads, n_units));
  const int n_groups = std::max(1, n_units / group_heads);
  // an item is a pair of 64-row query blocks with one list each, or (token-derived lists) one 128-row block
  fg::sparse_order_kernel<<<n_groups, 256, 0, st>>>(
      kb_counts, static_cast<int*>(workspace) + 4, p.queue, kb_mask ? p.npairs : p.nqb, p.npairs, n_units, group_heads, 1,
      kb_mask ? 1 : 2, 0, renorm ? p.redo : nullptr);
  FG_CUDA(cudaGetLastError());
  const int grid = std::min(p.n_items, sms);
  const int smem = (D == 128) ? fg::SparseMLCfg<128>::smem_bytes(p.list_cap, p.nkb)
                              : fg::SparseMLCfg<64>::smem_bytes(p.list_cap, p.nkb);
  if (smem > 232448) return FGATTN_UNSUPPORTED;
  auto go = [&](auto kern, int threads) -> int {
    int rr = set_smem(kern, smem);
    if (rr) return rr;
    kern<<<grid, threads, smem, st>>>(mq, mk, mv, p);
    return FGATTN_OK;
  };
  if (kb_mask && !renorm) return FGATTN_INVALID_ARGUMENT;      // token-derived lists exist in the renormalising form only
  if (D == 128)
    r = kb_mask ? go(fg::sparse_ml_persistent_kernel<128, true, true>, fg::SparseMLCfg<128>::kThreads)
        : renorm ? go(fg::sparse_ml_persistent_kernel<128, true>, fg::SparseMLCfg<128>::kThreads)
                 : go(fg::sparse_ml_persistent_kernel<128, false>, fg::SparseMLCfg<128>::kThreads);
  else
    r = kb_mask ? go(fg::sparse_ml_persistent_kernel<64, true, true>, fg::SparseMLCfg<64>::kThreads)
        : renorm ? go(fg::sparse_ml_persistent_kernel<64, true>, fg::SparseMLCfg<64>::kThreads)
                 : go(fg::sparse_ml_persistent_kernel<64, false>, fg::SparseMLCfg<64>::kThreads);
  if (r) return r;
  FG_CUDA(cudaGetLastError());
  if (renorm)   // items whose rows left the safe exponent range run again with the running maximum
    return launch_sparse(o, q, k, v, kb_indices, kb_counts, list_stride, batch, heads, seq, D, kv_rows, kv_seq_len,
                         scale, nullptr, 0, st, p.redo, kb_mask);
  return FGATTN_OK;
}
}  // namespace

int fgattn_sp_attn_blocks_ml(void* o, const void* q, const void* k, const void* v, const int* kb_indices,
                             const int* kb_counts, int list_stride, const float* max_q, const float* denom, int batch,
                             int heads, int seq, int D, int kv_rows, int kv_seq_len, float scale, void* workspace,
                             size_t workspace_bytes, void* stream) {
  return launch_sparse_persistent(false, o, q, k, v, kb_indices, kb_counts, list_stride, max_q, denom, batch, heads, seq,
                                  D, kv_rows, kv_seq_len, scale, workspace, workspace_bytes, stream);
}

int fgattn_sp_attn_blocks_hint(void* o, const void* q, const void* k, const void* v, const int* kb_indices,
                               const int* kb_counts, int list_stride, const float* max_q_hint, int batch, int heads,
                               int seq, int D, int kv_rows, int kv_seq_len, float scale, void* workspace,
                               size_t workspace_bytes, void* stream) {
  return launch_sparse_persistent(true, o, q, k, v, kb_indices, kb_counts, list_stride, max_q_hint, nullptr, batch,
                                  heads, seq, D, kv_rows, kv_seq_len, scale, workspace, workspace_bytes, stream);
}

int fgattn_selftest_bounded_wait(long long budget_cycles, void* stream) {
  if (budget_cycles < 1 || budget_cycles > 100000000LL) return FGATTN_INVALID_ARGUMENT;
  int* err = nullptr;
  int r = get_err_word(&err);
  if (r) return r;
  fg::bounded_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(err, budget_cycles);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

// ---- one-bit-per-entry masks -------------------------------------------------------------------
namespace {
int byte_grid(long long n_bytes) { return int(std::min<long long>((n_bytes + 255) / 256, 148LL * 64)); }
}  // namespace

int fgattn_pack_mask(unsigned char* packed, const void* mask, int elem_size, long long rows, int width, void* stream) {
  if (!packed || !mask || rows <= 0 || width <= 0) return FGATTN_INVALID_ARGUMENT;
  if (elem_size != 1 && elem_size != 4) return FGATTN_UNSUPPORTED;
  if (width % 8) return FGATTN_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(mask) & (elem_size == 4 ? 15u : 7u)) return FGATTN_MISALIGNED;
  const long long n_bytes = rows * (width / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (elem_size == 4)
    fg::pack_mask_kernel<int><<<byte_grid(n_bytes), 256, 0, st>>>(static_cast<const int*>(mask), packed, n_bytes);
  else
    fg::pack_mask_kernel<uint8_t><<<byte_grid(n_bytes), 256, 0, st>>>(static_cast<const uint8_t*>(mask), packed, n_bytes);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

int fgattn_unpack_mask(void* mask, int elem_size, const unsigned char* packed, long long rows, int width, void* stream) {
  if (!packed || !mask || rows <= 0 || width <= 0) return FGATTN_INVALID_ARGUMENT;
  if (elem_size != 1 && elem_size != 4) return FGATTN_UNSUPPORTED;
  if (width % 8) return FGATTN_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(mask) & (elem_size == 4 ? 15u : 7u)) return FGATTN_MISALIGNED;
  const long long n_bytes = rows * (width / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (elem_size == 4)
    fg::unpack_mask_kernel<int><<<byte_grid(2 * n_bytes), 256, 0, st>>>(packed, static_cast<int*>(mask), n_bytes);
  else
    fg::unpack_mask_kernel<uint8_t><<<byte_grid(n_bytes), 256, 0, st>>>(packed, static_cast<uint8_t*>(mask), n_bytes);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

int fgattn_packedmask_to_indexmask(int* indices, int* num_indices, const unsigned char* packed, long long rows,
                                   int width, int list_stride, int n_valid, int sentinel, void* stream) {
  if (!indices || !num_indices || !packed) return FGATTN_INVALID_ARGUMENT;
  if (rows <= 0 || width <= 0 || list_stride <= 0 || n_valid < 0 || width % 8) return FGATTN_INVALID_ARGUMENT;
  if (rows > 2147483647LL) return FGATTN_UNSUPPORTED;
  fg::packed_to_index_kernel<<<unsigned(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      packed, width / 8, indices, num_indices, list_stride, std::min(n_valid, width), sentinel);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

int fgattn_indexmask_to_packedmask(unsigned char* packed, const int* indices, const int* num_indices, long long rows,
                                   int list_stride, int width, void* stream) {
  if (!indices || !num_indices || !packed) return FGATTN_INVALID_ARGUMENT;
  if (rows <= 0 || width <= 0 || list_stride <= 0 || width % 8) return FGATTN_INVALID_ARGUMENT;
  if (rows > 2147483647LL) return FGATTN_UNSUPPORTED;
  const int row_bytes = width / 8, smem = ((row_bytes + 3) / 4) * 4;
  if (smem > 48 * 1024) return FGATTN_UNSUPPORTED;        // rows of up to 393216 entries
  fg::index_to_packed_kernel<<<unsigned(rows), 256, smem, static_cast<cudaStream_t>(stream)>>>(
      indices, num_indices, list_stride, packed, row_bytes, width);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

int fgattn_sp_attn_blocks(void* o, const void* q, const void* k, const void* v, const int* kb_indices,
                          const int* kb_counts, int list_stride, int batch, int heads, int seq, int D, int kv_rows,
                          int kv_seq_len, float scale, void* workspace, size_t workspace_bytes, void* stream) {
  return launch_sparse(o, q, k, v, kb_indices, kb_counts, list_stride, batch, heads, seq, D, kv_rows, kv_seq_len, scale,
                       workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

// ---- top-k selector ------------------------------------------------------------------------------
size_t fgattn_topk_scratch_bytes(int batch, int heads, int seq, int D, int blocksz, int kv_seq_len) {
  if (batch <= 0 || heads <= 0 || seq <= 0 || D <= 0 || blocksz <= 0 || kv_seq_len <= 0) return 0;
  const size_t bh = size_t(batch) * heads, nblk = size_t((seq + blocksz - 1) / blocksz);
  const size_t s_stride = size_t((kv_seq_len + 127) / 128) * 128;
  return 2 * align256(bh * nblk * D * 2) + bh * nblk * s_stride * sizeof(float);
}

int fgattn_topk_indices(int* kv_indices, int* kv_num_indices, int list_stride, const void* q, const void* k,
                        int select_k, int batch, int heads, int seq, int D, int blocksz, int kv_rows, int kv_seq_len,
                        float scale, void* scratch, size_t scratch_bytes, void* stream) {
  int r = check_qk(q, k, batch, heads, seq, D, kv_rows, kv_seq_len);
  if (r) return r;
  if (!kv_indices || !kv_num_indices || !scratch || blocksz < 1) return FGATTN_INVALID_ARGUMENT;
  if (select_k < 1 || select_k > kv_seq_len || list_stride < select_k) return FGATTN_INVALID_ARGUMENT;
  if (select_k > 8192) return FGATTN_UNSUPPORTED;          // the selected pairs are sorted in shared memory
  if (!aligned16(scratch)) return FGATTN_MISALIGNED;
  if (scratch_bytes < fgattn_topk_scratch_bytes(batch, heads, seq, D, blocksz, kv_seq_len))
    return FGATTN_SCRATCH_TOO_SMALL;
  const int bh = batch * heads, nblk = (seq + blocksz - 1) / blocksz, s_stride = ((kv_seq_len + 127) / 128) * 128;
  if ((long long)bh * nblk > 2147483647LL || nblk > 65535 * 128) return FGATTN_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(scratch);
  const size_t mean_bytes = align256(size_t(bh) * nblk * D * 2);
  __nv_bfloat16* qm_hi = reinterpret_cast<__nv_bfloat16*>(base);
  __nv_bfloat16* qm_lo = reinterpret_cast<__nv_bfloat16*>(base + mean_bytes);
  float* scores = reinterpret_cast<float*>(base + 2 * mean_bytes);
  const float sc = (scale > 0.f) ? scale : 1.0f / sqrtf(float(D));
  fg::TopkScoreParams p;
  p.scores = scores;
  p.n_blocks = nblk;
  p.kv_len = kv_seq_len;
  p.s_stride = s_stride;
  r = get_err_word(&p.err);
  if (r) return r;
  CUtensorMap m_hi, m_lo, mk;
  if (fg::make_qkv_map(&m_hi, qm_hi, bh, nblk, D, 128) || fg::make_qkv_map(&m_lo, qm_lo, bh, nblk, D, 128) ||
      fg::make_qkv_map(&mk, k, bh, kv_rows, D, 128))
    return fg::encode_tiled_fn() ? FGATTN_INVALID_ARGUMENT : FGATTN_NO_DRIVER;
  const dim3 g_mean(nblk, bh), g_sc(s_stride / 128, (nblk + 127) / 128, bh);
  if (D == 128) {
    fg::qblock_mean_kernel<128><<<g_mean, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(q), qm_hi, qm_lo, seq, nblk,
                                                       blocksz, sc);
    auto kern = fg::topk_scores_kernel<128>;
    r = set_smem(kern, fg::TopkScoreCfg<128>::kSmemBytes);
    if (r) return r;
    kern<<<g_sc, fg::TopkScoreCfg<128>::kThreads, fg::TopkScoreCfg<128>::kSmemBytes, st>>>(m_hi, m_lo, mk, p);
  } else {
    fg::qblock_mean_kernel<64><<<g_mean, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(q), qm_hi, qm_lo, seq, nblk,
                                                      blocksz, sc);
    auto kern = fg::topk_scores_kernel<64>;
    r = set_smem(kern, fg::TopkScoreCfg<64>::kSmemBytes);
    if (r) return r;
    kern<<<g_sc, fg::TopkScoreCfg<64>::kThreads, fg::TopkScoreCfg<64>::kSmemBytes, st>>>(m_hi, m_lo, mk, p);
  }
  FG_CUDA(cudaGetLastError());
  int k_pow2 = 2;
  while (k_pow2 < select_k) k_pow2 <<= 1;
  const int smem_sel = k_pow2 * 8;
  r = set_smem(fg::topk_select_kernel, std::max(smem_sel, 1024));
  if (r) return r;
  fg::topk_select_kernel<<<unsigned(bh * nblk), fg::kSelThreads, smem_sel, st>>>(
      scores, s_stride, kv_seq_len, select_k, k_pow2, kv_indices, kv_num_indices, list_stride);
  FG_CUDA(cudaGetLastError());
  return FGATTN_OK;
}

}  // extern "C"
