// PyTorch operator boundary: registers the reference's seven `cuda_attn` operator schemas
// (python/extension.cpp:82,113,166,215,259,309,349 of sankeerth95/fgattn_tk_cuda) plus the
// block-granular additions, validates tensors and forwards raw pointers to the C ABI of
// libfgattn_b200 on the current CUDA stream.  Also a pybind module with the same names, like the
// reference's `spattn.cuda_attn` (python/extension.cpp:362-370).  No device code lives here.
//
// Every operator first checks dtypes AND shapes of all its tensors against q (the C ABI derives every
// size from q and trusts the buffers to match), so a wrong-shaped tensor is a TORCH_CHECK error and never
// an out-of-bounds access on the device.  The same checks are the operators' Meta kernels, so they also
// run on meta tensors without a GPU.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>

#include "fgattn_b200.h"

namespace {

void check_status(int st, const char* what) {
  TORCH_CHECK(st == FGATTN_OK, what, " failed: ", fgattn_status_string(st),
              st == FGATTN_CUDA_ERROR ? " (cudaError " + std::to_string(fgattn_last_cuda_error()) + ")" : "");
}

// ---- validation (device independent except for the is_cuda test, which meta tensors skip) ---------
void check_dev(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() || t.is_meta(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
void check_dtype(const torch::Tensor& t, at::ScalarType ty, const char* name) {
  check_dev(t, name);
  TORCH_CHECK(t.scalar_type() == ty, name, " has the wrong dtype");
}
void check_bf16_4d(const torch::Tensor& t, const char* name) {
  check_dev(t, name);
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
  TORCH_CHECK(t.dim() == 4, name, " must be [B, H, S, D]");
}
int64_t pad128(int64_t n) { return (n + 127) / 128 * 128; }
int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// q [B,H,S,D] and k [B,H,S_kv,D]
void check_qk(const torch::Tensor& q, const torch::Tensor& k) {
  check_bf16_4d(q, "q");
  check_bf16_4d(k, "k");
  TORCH_CHECK(q.size(3) == 64 || q.size(3) == 128, "head dimension must be 64 or 128");
  TORCH_CHECK(k.size(0) == q.size(0) && k.size(1) == q.size(1) && k.size(3) == q.size(3),
              "k must match q in batch, heads and head dimension");
  TORCH_CHECK(q.size(2) > 0 && k.size(2) > 0, "empty sequence");
}
void check_v(const torch::Tensor& v, const torch::Tensor& k) {
  check_bf16_4d(v, "v");
  TORCH_CHECK(v.sizes() == k.sizes(), "v must have the shape of k");
}
void check_o(const torch::Tensor& o, const torch::Tensor& q) {
  check_bf16_4d(o, "o");
  TORCH_CHECK(o.sizes() == q.sizes(), "o must have the shape of q");
}
// max_q / denom: fp32, at least B*H*pad128(S) elements (the kernels write the padded tail)
void check_ml(const torch::Tensor& t, const torch::Tensor& q, const char* name) {
  check_dtype(t, at::kFloat, name);
  TORCH_CHECK(t.numel() >= q.size(0) * q.size(1) * pad128(q.size(2)), name, " must hold B*H*ceil(S/128)*128 floats");
}
// key-token lists of the reference granularity: [B,H,ceil(S/128),stride] + one count per row
void check_token_lists(const torch::Tensor& idx, const torch::Tensor& cnt, const torch::Tensor& q) {
  check_dtype(idx, at::kInt, "kv_indices");
  check_dtype(cnt, at::kInt, "kv_num_indices");
  const int64_t rows = cdiv(q.size(2), 128);
  TORCH_CHECK(idx.dim() == 4 && idx.size(0) == q.size(0) && idx.size(1) == q.size(1) && idx.size(2) == rows &&
                  idx.size(3) >= 1, "kv_indices must be [B, H, ceil(S/128), stride]");
  TORCH_CHECK(cnt.numel() == q.size(0) * q.size(1) * rows, "kv_num_indices must hold B*H*ceil(S/128) counts");
}
// key-block lists: [B,H,ceil(S/64),stride >= ceil(S_kv/64)] + one count per row
void check_block_lists(const torch::Tensor& idx, const torch::Tensor& cnt, const torch::Tensor& q,
                       const torch::Tensor& k) {
  check_dtype(idx, at::kInt, "kb_indices");
  check_dtype(cnt, at::kInt, "kb_counts");
  const int64_t rows = cdiv(q.size(2), 64);
  TORCH_CHECK(idx.dim() == 4 && idx.size(0) == q.size(0) && idx.size(1) == q.size(1) && idx.size(2) == rows &&
                  idx.size(3) >= cdiv(k.size(2), 64), "kb_indices must be [B, H, ceil(S/64), >= ceil(S_kv/64)]");
  TORCH_CHECK(cnt.numel() == q.size(0) * q.size(1) * rows, "kb_counts must hold B*H*ceil(S/64) counts");
}
// token mask [B,H,ceil(S/128),stride >= S_kv]
void check_tokenmask(const torch::Tensor& m, const torch::Tensor& q, const torch::Tensor& k) {
  check_dtype(m, at::kInt, "booleanmask");
  TORCH_CHECK(m.dim() == 4 && m.size(0) == q.size(0) && m.size(1) == q.size(1) && m.size(2) == cdiv(q.size(2), 128) &&
                  m.size(3) >= k.size(2), "booleanmask must be [B, H, ceil(S/128), >= S_kv]");
}

void* stream_of(const torch::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// Work-queue / thread-block-order scratch of the sparse operators: one buffer per (device, stream),
// grown on demand and kept, so that a steady-state call allocates nothing.  Calls on one stream are
// serialised by the stream, so they can share the buffer; different streams get different buffers.
struct WorkspaceCache {
  std::mutex mu;
  std::map<std::pair<int, void*>, torch::Tensor> bufs;
  torch::Tensor get(const torch::Tensor& like, int64_t bytes) {
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_pair(int(like.get_device()), stream_of(like));
    auto it = bufs.find(key);
    if (it == bufs.end() || it->second.numel() < bytes) {
      torch::Tensor t = torch::empty({bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(like.device()));
      bufs[key] = t;
      return t;
    }
    return it->second;
  }
  void clear() {
    std::lock_guard<std::mutex> lock(mu);
    bufs.clear();
  }
};
WorkspaceCache& workspaces() {
  static WorkspaceCache* w = new WorkspaceCache;      // never destroyed: tensors must not outlive torch at exit
  return *w;
}

torch::Tensor sparse_workspace(const torch::Tensor& q) {
  return workspaces().get(q, int64_t(fgattn_sp_attn_workspace_bytes(q.size(0), q.size(1), q.size(2))));
}
void release_workspaces() { workspaces().clear(); }

// ---- the reference's seven operators: checks (also the Meta kernels) + CUDA bodies --------------
void full_attn_check(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v) {
  check_qk(q, k); check_v(v, k); check_o(o, q);
}
void full_attn(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v) {
  full_attn_check(o, q, k, v);
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_full_attn(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), q.size(0), q.size(1),
                                q.size(2), q.size(3), k.size(2), k.size(2), 0.f, stream_of(q)), "full_attn");
}

void all_index_mask_check(torch::Tensor kv_indices, torch::Tensor kv_num_indices, int64_t batch, int64_t heads,
                          int64_t seqblocks, int64_t seq) {
  check_dtype(kv_indices, at::kInt, "kv_indices"); check_dtype(kv_num_indices, at::kInt, "kv_num_indices");
  TORCH_CHECK(batch > 0 && heads > 0 && seqblocks > 0 && seq >= 0, "sizes must be positive");
  TORCH_CHECK(kv_indices.dim() == 4 && kv_indices.size(0) == batch && kv_indices.size(1) == heads &&
                  kv_indices.size(2) == seqblocks, "kv_indices must be [batch, heads, seqblocks, stride]");
  TORCH_CHECK(kv_num_indices.numel() == batch * heads * seqblocks, "kv_num_indices must hold batch*heads*seqblocks counts");
}
void all_index_mask(torch::Tensor kv_indices, torch::Tensor kv_num_indices, int64_t batch, int64_t heads,
                    int64_t seqblocks, int64_t seq) {
  all_index_mask_check(kv_indices, kv_num_indices, batch, heads, seqblocks, seq);
  c10::cuda::CUDAGuard guard(kv_indices.device());
  check_status(fgattn_all_index_mask(kv_indices.data_ptr<int>(), kv_num_indices.data_ptr<int>(), int(batch),
                                     int(heads), int(seqblocks), int(seq), int(kv_indices.size(3)),
                                     stream_of(kv_indices)), "all_index_mask");
}

void sp_attn_check(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kv_indices,
                   torch::Tensor kv_num_indices) {
  check_qk(q, k); check_v(v, k); check_o(o, q);
  check_token_lists(kv_indices, kv_num_indices, q);
}
void sp_attn(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kv_indices,
             torch::Tensor kv_num_indices) {
  sp_attn_check(o, q, k, v, kv_indices, kv_num_indices);
  c10::cuda::CUDAGuard guard(q.device());
  torch::Tensor ws = sparse_workspace(q);      // longest-first order of the thread blocks
  check_status(fgattn_sp_attn(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), kv_indices.data_ptr<int>(),
                              kv_num_indices.data_ptr<int>(), int(kv_indices.size(3)), q.size(0), q.size(1),
                              q.size(2), q.size(3), k.size(2), 0.f, ws.data_ptr(), size_t(ws.numel()), stream_of(q)),
               "sp_attn");
}

void fullattn_maxq_denom_check(torch::Tensor o, torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q,
                               torch::Tensor k, torch::Tensor v) {
  check_qk(q, k); check_v(v, k); check_o(o, q);
  check_ml(o_max_q, q, "o_max_q"); check_ml(o_denom, q, "o_denom");
}
void fullattn_maxq_denom(torch::Tensor o, torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q,
                         torch::Tensor k, torch::Tensor v) {
  fullattn_maxq_denom_check(o, o_max_q, o_denom, q, k, v);
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_fullattn_maxq_denom(o.data_ptr(), o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(),
                                          q.data_ptr(), k.data_ptr(), v.data_ptr(), q.size(0), q.size(1), q.size(2),
                                          q.size(3), k.size(2), k.size(2), 0.f, stream_of(q)), "fullattn_maxq_denom");
}

void maxq_denom_check(torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q, torch::Tensor k) {
  check_qk(q, k);
  check_ml(o_max_q, q, "o_max_q"); check_ml(o_denom, q, "o_denom");
}
void maxq_denom(torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q, torch::Tensor k) {
  maxq_denom_check(o_max_q, o_denom, q, k);
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_maxq_denom(o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(), q.data_ptr(), k.data_ptr(),
                                 q.size(0), q.size(1), q.size(2), q.size(3), k.size(2), k.size(2), 0.f, stream_of(q)),
               "maxq_denom");
}

void booleanmask_128_check(torch::Tensor booleanmask, torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q,
                           torch::Tensor k, double threshold) {
  check_qk(q, k);
  check_tokenmask(booleanmask, q, k);
  check_ml(o_max_q, q, "o_max_q"); check_ml(o_denom, q, "o_denom");
  TORCH_CHECK(threshold > 0.0, "threshold must be positive");
}
void booleanmask_128(torch::Tensor booleanmask, torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q,
                     torch::Tensor k, double threshold) {
  booleanmask_128_check(booleanmask, o_max_q, o_denom, q, k, threshold);
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_booleanmask_128(booleanmask.data_ptr<int>(), float(threshold), int(booleanmask.size(3)),
                                      o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(), q.data_ptr(),
                                      k.data_ptr(), q.size(0), q.size(1), q.size(2), q.size(3), k.size(2), k.size(2), 0.f,
                                      stream_of(q)), "booleanmask_128");
}

void booleanmask_128_listed_check(torch::Tensor booleanmask, torch::Tensor o_max_q, torch::Tensor o_denom,
                                  torch::Tensor q, torch::Tensor k, double threshold, torch::Tensor kb_indices,
                                  torch::Tensor kb_counts) {
  booleanmask_128_check(booleanmask, o_max_q, o_denom, q, k, threshold);
  check_block_lists(kb_indices, kb_counts, q, k);
}
void booleanmask_128_listed(torch::Tensor booleanmask, torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q,
                            torch::Tensor k, double threshold, torch::Tensor kb_indices, torch::Tensor kb_counts) {
  booleanmask_128_listed_check(booleanmask, o_max_q, o_denom, q, k, threshold, kb_indices, kb_counts);
  c10::cuda::CUDAGuard guard(q.device());
  torch::Tensor ws = sparse_workspace(q);      // longest-first order of the thread blocks
  check_status(fgattn_booleanmask_128_listed(booleanmask.data_ptr<int>(), float(threshold), int(booleanmask.size(3)),
                                             o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(), q.data_ptr(),
                                             k.data_ptr(), kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(),
                                             int(kb_indices.size(3)), q.size(0), q.size(1), q.size(2), q.size(3),
                                             k.size(2), k.size(2), 0.f, ws.data_ptr(), size_t(ws.numel()), stream_of(q)),
               "booleanmask_128_listed");
}

void booleanmask_to_indexmask_check(torch::Tensor kv_indices, torch::Tensor kv_numindices, torch::Tensor booleanmask,
                                    int64_t seq) {
  check_dtype(kv_indices, at::kInt, "kv_indices"); check_dtype(kv_numindices, at::kInt, "kv_numindices");
  check_dtype(booleanmask, at::kInt, "booleanmask");
  TORCH_CHECK(booleanmask.dim() == 4, "booleanmask must be [B, H, blocks, stride]");
  TORCH_CHECK(kv_indices.sizes() == booleanmask.sizes(), "kv_indices must have the shape of booleanmask");
  TORCH_CHECK(kv_numindices.numel() == booleanmask.size(0) * booleanmask.size(1) * booleanmask.size(2),
              "kv_numindices must hold one count per mask row");
  TORCH_CHECK(seq >= 0, "seq must not be negative");
}
void booleanmask_to_indexmask(torch::Tensor kv_indices, torch::Tensor kv_numindices, torch::Tensor booleanmask,
                              int64_t seq) {
  booleanmask_to_indexmask_check(kv_indices, kv_numindices, booleanmask, seq);
  c10::cuda::CUDAGuard guard(booleanmask.device());
  check_status(fgattn_booleanmask_to_indexmask(kv_indices.data_ptr<int>(), kv_numindices.data_ptr<int>(),
                                               booleanmask.data_ptr<int>(), booleanmask.size(0), booleanmask.size(1),
                                               int(seq), booleanmask.size(2), booleanmask.size(3),
                                               stream_of(booleanmask)), "booleanmask_to_indexmask");
}

// ---- 64x64 block granularity (additions) -------------------------------------------------------
void block_index_lists_check(torch::Tensor kb_indices, torch::Tensor kb_counts, torch::Tensor o_max_q,
                             torch::Tensor o_denom, c10::optional<torch::Tensor> o, torch::Tensor q, torch::Tensor k,
                             c10::optional<torch::Tensor> v, double threshold, torch::Tensor scratch) {
  check_qk(q, k);
  check_block_lists(kb_indices, kb_counts, q, k);
  check_ml(o_max_q, q, "o_max_q"); check_ml(o_denom, q, "o_denom");
  check_dev(scratch, "scratch");
  TORCH_CHECK(o.has_value() == v.has_value(), "o and v go together");
  if (o) check_o(*o, q);
  if (v) check_v(*v, k);
  TORCH_CHECK(threshold > 0.0, "threshold must be positive");
}
void block_index_lists(torch::Tensor kb_indices, torch::Tensor kb_counts, torch::Tensor o_max_q, torch::Tensor o_denom,
                       c10::optional<torch::Tensor> o, torch::Tensor q, torch::Tensor k,
                       c10::optional<torch::Tensor> v, double threshold, torch::Tensor scratch) {
  block_index_lists_check(kb_indices, kb_counts, o_max_q, o_denom, o, q, k, v, threshold, scratch);
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_block_index_lists(kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(), int(kb_indices.size(3)),
                                        o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(),
                                        o ? o->data_ptr() : nullptr, q.data_ptr(), k.data_ptr(),
                                        v ? v->data_ptr() : nullptr, float(threshold), q.size(0), q.size(1), q.size(2),
                                        q.size(3), k.size(2), k.size(2), 0.f, scratch.data_ptr(),
                                        size_t(scratch.numel()) * scratch.element_size(), stream_of(q)),
               "block_index_lists");
}

// The threshold step alone on the block maxima that block_index_lists left in a scratch sized for all units:
// key-block lists for another threshold without a new pass over the keys.  The lists give B, H and ceil(S/64).
void block_lists_from_maxima_check(torch::Tensor kb_indices, torch::Tensor kb_counts, torch::Tensor block_maxima,
                                   torch::Tensor max_q, torch::Tensor denom, int64_t seq, int64_t head_dim,
                                   int64_t kv_seq_len, double threshold) {
  check_dtype(kb_indices, at::kInt, "kb_indices"); check_dtype(kb_counts, at::kInt, "kb_counts");
  check_dtype(block_maxima, at::kFloat, "block_maxima");
  check_dtype(max_q, at::kFloat, "max_q"); check_dtype(denom, at::kFloat, "denom");
  TORCH_CHECK(seq > 0 && kv_seq_len > 0, "seq and kv_seq_len must be positive");
  TORCH_CHECK(head_dim == 64 || head_dim == 128, "head_dim must be 64 or 128");
  TORCH_CHECK(threshold > 0.0, "threshold must be positive");
  const int64_t nqb = cdiv(seq, 64), nkb = cdiv(kv_seq_len, 64);
  TORCH_CHECK(kb_indices.dim() == 4 && kb_indices.size(2) == nqb && kb_indices.size(3) >= nkb,
              "kb_indices must be [B, H, ceil(S/64), >= ceil(S_kv/64)]");
  const int64_t bh = kb_indices.size(0) * kb_indices.size(1);
  TORCH_CHECK(kb_counts.numel() == bh * nqb, "kb_counts must hold B*H*ceil(S/64) counts");
  TORCH_CHECK(max_q.numel() >= bh * pad128(seq) && denom.numel() >= bh * pad128(seq),
              "max_q and denom must hold B*H*ceil(S/128)*128 floats");
  TORCH_CHECK(block_maxima.numel() >= bh * nkb * pad128(seq),
              "block_maxima must hold B*H*ceil(S_kv/64)*ceil(S/128)*128 floats (the scratch of a list build for all units)");
}
void block_lists_from_maxima(torch::Tensor kb_indices, torch::Tensor kb_counts, torch::Tensor block_maxima,
                             torch::Tensor max_q, torch::Tensor denom, int64_t seq, int64_t head_dim,
                             int64_t kv_seq_len, double threshold) {
  block_lists_from_maxima_check(kb_indices, kb_counts, block_maxima, max_q, denom, seq, head_dim, kv_seq_len, threshold);
  c10::cuda::CUDAGuard guard(kb_indices.device());
  check_status(fgattn_block_lists_from_maxima(kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(),
                                              int(kb_indices.size(3)), block_maxima.data_ptr<float>(),
                                              max_q.data_ptr<float>(), denom.data_ptr<float>(), float(threshold),
                                              kb_indices.size(0), kb_indices.size(1), int(seq), int(head_dim),
                                              int(kv_seq_len), 0.f, stream_of(kb_indices)),
               "block_lists_from_maxima");
}

void sp_attn_blocks_ml_check(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v,
                             torch::Tensor kb_indices, torch::Tensor kb_counts, torch::Tensor max_q,
                             torch::Tensor denom) {
  check_qk(q, k); check_v(v, k); check_o(o, q);
  check_block_lists(kb_indices, kb_counts, q, k);
  check_ml(max_q, q, "max_q"); check_ml(denom, q, "denom");
}
void sp_attn_blocks_ml(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kb_indices,
                       torch::Tensor kb_counts, torch::Tensor max_q, torch::Tensor denom) {
  sp_attn_blocks_ml_check(o, q, k, v, kb_indices, kb_counts, max_q, denom);
  c10::cuda::CUDAGuard guard(q.device());
  torch::Tensor ws = sparse_workspace(q);      // work queue of the persistent kernel
  check_status(fgattn_sp_attn_blocks_ml(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                        kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(), int(kb_indices.size(3)),
                                        max_q.data_ptr<float>(), denom.data_ptr<float>(), q.size(0), q.size(1),
                                        q.size(2), q.size(3), k.size(2), k.size(2), 0.f, ws.data_ptr(),
                                        size_t(ws.numel()), stream_of(q)), "sp_attn_blocks_ml");
}

void sp_attn_blocks_hint_check(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v,
                               torch::Tensor kb_indices, torch::Tensor kb_counts, torch::Tensor max_q_hint) {
  check_qk(q, k); check_v(v, k); check_o(o, q);
  check_block_lists(kb_indices, kb_counts, q, k);
  check_ml(max_q_hint, q, "max_q_hint");
}
void sp_attn_blocks_hint(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kb_indices,
                         torch::Tensor kb_counts, torch::Tensor max_q_hint) {
  sp_attn_blocks_hint_check(o, q, k, v, kb_indices, kb_counts, max_q_hint);
  c10::cuda::CUDAGuard guard(q.device());
  torch::Tensor ws = sparse_workspace(q);      // work queue + re-run flags of the persistent kernel
  check_status(fgattn_sp_attn_blocks_hint(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                          kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(),
                                          int(kb_indices.size(3)), max_q_hint.data_ptr<float>(), q.size(0), q.size(1),
                                          q.size(2), q.size(3), k.size(2), k.size(2), 0.f, ws.data_ptr(),
                                          size_t(ws.numel()), stream_of(q)), "sp_attn_blocks_hint");
}

void sp_attn_blocks_check(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kb_indices,
                          torch::Tensor kb_counts) {
  check_qk(q, k); check_v(v, k); check_o(o, q);
  check_block_lists(kb_indices, kb_counts, q, k);
}
void sp_attn_blocks(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kb_indices,
                    torch::Tensor kb_counts) {
  sp_attn_blocks_check(o, q, k, v, kb_indices, kb_counts);
  c10::cuda::CUDAGuard guard(q.device());
  torch::Tensor ws = sparse_workspace(q);      // longest-first order of the thread blocks
  check_status(fgattn_sp_attn_blocks(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                     kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(), int(kb_indices.size(3)),
                                     q.size(0), q.size(1), q.size(2), q.size(3), k.size(2), k.size(2), 0.f,
                                     ws.data_ptr(), size_t(ws.numel()), stream_of(q)),
               "sp_attn_blocks");
}

// ---- one-bit-per-entry masks (additions) ---------------------------------------------------------
int mask_elem_size(const torch::Tensor& t, const char* name) {
  check_dev(t, name);
  if (t.scalar_type() == at::kBool || t.scalar_type() == at::kByte) return 1;
  TORCH_CHECK(t.scalar_type() == at::kInt, name, " must be bool, uint8 or int32");
  return 4;
}

void pack_mask_check(torch::Tensor packed, torch::Tensor mask) {
  check_dtype(packed, at::kByte, "packed");
  mask_elem_size(mask, "mask");
  TORCH_CHECK(mask.dim() >= 1 && mask.size(-1) % 8 == 0 && packed.numel() * 8 == mask.numel(),
              "packed must hold one bit per mask entry");
}
void pack_mask(torch::Tensor packed, torch::Tensor mask) {
  pack_mask_check(packed, mask);
  const int es = mask_elem_size(mask, "mask");
  const int64_t W = mask.size(-1);
  c10::cuda::CUDAGuard guard(mask.device());
  check_status(fgattn_pack_mask(packed.data_ptr<uint8_t>(), mask.data_ptr(), es, mask.numel() / W, int(W),
                                stream_of(mask)), "pack_mask");
}

void unpack_mask_check(torch::Tensor mask, torch::Tensor packed) { pack_mask_check(packed, mask); }
void unpack_mask(torch::Tensor mask, torch::Tensor packed) {
  unpack_mask_check(mask, packed);
  const int es = mask_elem_size(mask, "mask");
  const int64_t W = mask.size(-1);
  c10::cuda::CUDAGuard guard(mask.device());
  check_status(fgattn_unpack_mask(mask.data_ptr(), es, packed.data_ptr<uint8_t>(), mask.numel() / W, int(W),
                                  stream_of(mask)), "unpack_mask");
}

void packedmask_to_indexmask_check(torch::Tensor indices, torch::Tensor num_indices, torch::Tensor packed,
                                   int64_t n_valid, int64_t sentinel) {
  check_dtype(indices, at::kInt, "indices"); check_dtype(num_indices, at::kInt, "num_indices");
  check_dtype(packed, at::kByte, "packed");
  TORCH_CHECK(packed.dim() >= 1 && indices.dim() >= 1 && packed.size(-1) > 0 && indices.size(-1) > 0, "empty rows");
  const int64_t rows = packed.numel() / packed.size(-1);
  TORCH_CHECK(num_indices.numel() == rows && indices.numel() == rows * indices.size(-1), "row counts differ");
  TORCH_CHECK(n_valid >= 0, "n_valid must not be negative");
}
void packedmask_to_indexmask(torch::Tensor indices, torch::Tensor num_indices, torch::Tensor packed, int64_t n_valid,
                             int64_t sentinel) {
  packedmask_to_indexmask_check(indices, num_indices, packed, n_valid, sentinel);
  const int64_t rows = packed.numel() / packed.size(-1);
  c10::cuda::CUDAGuard guard(packed.device());
  check_status(fgattn_packedmask_to_indexmask(indices.data_ptr<int>(), num_indices.data_ptr<int>(),
                                              packed.data_ptr<uint8_t>(), rows, int(packed.size(-1) * 8),
                                              int(indices.size(-1)), int(n_valid), int(sentinel), stream_of(packed)),
               "packedmask_to_indexmask");
}

void indexmask_to_packedmask_check(torch::Tensor packed, torch::Tensor indices, torch::Tensor num_indices) {
  packedmask_to_indexmask_check(indices, num_indices, packed, 0, 0);
}
void indexmask_to_packedmask(torch::Tensor packed, torch::Tensor indices, torch::Tensor num_indices) {
  indexmask_to_packedmask_check(packed, indices, num_indices);
  const int64_t rows = packed.numel() / packed.size(-1);
  c10::cuda::CUDAGuard guard(packed.device());
  check_status(fgattn_indexmask_to_packedmask(packed.data_ptr<uint8_t>(), indices.data_ptr<int>(),
                                              num_indices.data_ptr<int>(), rows, int(indices.size(-1)),
                                              int(packed.size(-1) * 8), stream_of(packed)),
               "indexmask_to_packedmask");
}

// ---- top-k selector (addition) ------------------------------------------------------------------
void topk_indices_check(torch::Tensor kv_indices, torch::Tensor kv_num_indices, torch::Tensor q, torch::Tensor k,
                        int64_t select_k, int64_t blocksz) {
  check_qk(q, k);
  check_dtype(kv_indices, at::kInt, "kv_indices"); check_dtype(kv_num_indices, at::kInt, "kv_num_indices");
  TORCH_CHECK(blocksz >= 1 && select_k >= 1 && select_k <= k.size(2), "select_k must lie in [1, S_kv]");
  const int64_t rows = cdiv(q.size(2), blocksz);
  TORCH_CHECK(kv_indices.dim() == 4 && kv_indices.size(0) == q.size(0) && kv_indices.size(1) == q.size(1) &&
                  kv_indices.size(2) == rows && kv_indices.size(3) >= select_k,
              "kv_indices must be [B, H, ceil(S/blocksz), >= select_k]");
  TORCH_CHECK(kv_num_indices.numel() == q.size(0) * q.size(1) * rows, "kv_num_indices must hold one count per query block");
}
void topk_indices(torch::Tensor kv_indices, torch::Tensor kv_num_indices, torch::Tensor q, torch::Tensor k,
                  int64_t select_k, int64_t blocksz) {
  topk_indices_check(kv_indices, kv_num_indices, q, k, select_k, blocksz);
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t bytes = int64_t(fgattn_topk_scratch_bytes(q.size(0), q.size(1), q.size(2), q.size(3), int(blocksz),
                                                          int(k.size(2))));
  torch::Tensor scratch = torch::empty({bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(q.device()));
  check_status(fgattn_topk_indices(kv_indices.data_ptr<int>(), kv_num_indices.data_ptr<int>(), int(kv_indices.size(3)),
                                   q.data_ptr(), k.data_ptr(), int(select_k), q.size(0), q.size(1), q.size(2),
                                   q.size(3), int(blocksz), k.size(2), k.size(2), 0.f, scratch.data_ptr(),
                                   size_t(bytes),
                                   stream_of(q)), "topk_indices");
}

int64_t block_scratch_bytes(int64_t batch, int64_t heads, int64_t seq, int64_t kv_seq_len) {
  return int64_t(fgattn_block_scratch_bytes(int(batch), int(heads), int(seq), int(kv_seq_len)));
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(cuda_attn, m) {
  // the reference's schemas, verbatim
  m.def("full_attn(Tensor (o!) o, Tensor q, Tensor k, Tensor v) -> ()");
  m.def("all_index_mask(Tensor (kv_indices!) kv_indices, Tensor (kv_num_indices!) kv_num_indices, int batch, int heads, int seqblocks, int seq) -> ()");
  m.def("sp_attn(Tensor (o!) o, Tensor q, Tensor k, Tensor v, Tensor kv_indices, Tensor kv_num_indices) -> ()");
  m.def("fullattn_maxq_denom(Tensor (o!) o, Tensor (o_max_q!) o_max_q, Tensor (o_denom!) o_denom, Tensor q, Tensor k, Tensor v) -> ()");
  m.def("maxq_denom(Tensor (o_max_q!) o_max_q, Tensor (o_denom!) o_denom, Tensor q, Tensor k) -> ()");
  m.def("booleanmask_128(Tensor (booleanmask!) booleanmask, Tensor o_max_q, Tensor o_denom, Tensor q, Tensor k, float threshold) -> ()");
  m.def("booleanmask_to_indexmask(Tensor (kv_indices!) kv_indices, Tensor (kv_numindices!) kv_numindices, Tensor booleanmask, int seq) -> ()");
  // block-granular additions
  m.def("booleanmask_128_listed(Tensor (booleanmask!) booleanmask, Tensor o_max_q, Tensor o_denom, Tensor q, Tensor k, float threshold, Tensor kb_indices, Tensor kb_counts) -> ()");
  m.def("block_index_lists(Tensor (kb_indices!) kb_indices, Tensor (kb_counts!) kb_counts, Tensor (o_max_q!) o_max_q, Tensor (o_denom!) o_denom, Tensor(o!)? o, Tensor q, Tensor k, Tensor? v, float threshold, Tensor (scratch!) scratch) -> ()");
  m.def("block_lists_from_maxima(Tensor (kb_indices!) kb_indices, Tensor (kb_counts!) kb_counts, Tensor block_maxima, Tensor max_q, Tensor denom, int seq, int head_dim, int kv_seq_len, float threshold) -> ()");
  m.def("sp_attn_blocks_ml(Tensor (o!) o, Tensor q, Tensor k, Tensor v, Tensor kb_indices, Tensor kb_counts, Tensor max_q, Tensor denom) -> ()");
  m.def("sp_attn_blocks(Tensor (o!) o, Tensor q, Tensor k, Tensor v, Tensor kb_indices, Tensor kb_counts) -> ()");
  m.def("sp_attn_blocks_hint(Tensor (o!) o, Tensor q, Tensor k, Tensor v, Tensor kb_indices, Tensor kb_counts, Tensor max_q_hint) -> ()");
  // one-bit-per-entry masks
  m.def("pack_mask(Tensor (packed!) packed, Tensor mask) -> ()");
  m.def("unpack_mask(Tensor (mask!) mask, Tensor packed) -> ()");
  m.def("packedmask_to_indexmask(Tensor (indices!) indices, Tensor (num_indices!) num_indices, Tensor packed, int n_valid, int sentinel) -> ()");
  m.def("indexmask_to_packedmask(Tensor (packed!) packed, Tensor indices, Tensor num_indices) -> ()");
  // top-k selector
  m.def("topk_indices(Tensor (kv_indices!) kv_indices, Tensor (kv_num_indices!) kv_num_indices, Tensor q, Tensor k, int select_k, int blocksz) -> ()");
}

// Meta kernels: every operator writes into caller-allocated tensors and returns nothing, so the Meta
// kernel of an operator is its shape / dtype validation.
TORCH_LIBRARY_IMPL(cuda_attn, Meta, m) {
  m.impl("full_attn", full_attn_check);
  m.impl("all_index_mask", all_index_mask_check);
  m.impl("sp_attn", sp_attn_check);
  m.impl("fullattn_maxq_denom", fullattn_maxq_denom_check);
  m.impl("maxq_denom", maxq_denom_check);
  m.impl("booleanmask_128", booleanmask_128_check);
  m.impl("booleanmask_to_indexmask", booleanmask_to_indexmask_check);
  m.impl("booleanmask_128_listed", booleanmask_128_listed_check);
  m.impl("block_index_lists", block_index_lists_check);
  m.impl("block_lists_from_maxima", block_lists_from_maxima_check);
  m.impl("sp_attn_blocks_ml", sp_attn_blocks_ml_check);
  m.impl("sp_attn_blocks", sp_attn_blocks_check);
  m.impl("sp_attn_blocks_hint", sp_attn_blocks_hint_check);
  m.impl("pack_mask", pack_mask_check);
  m.impl("unpack_mask", unpack_mask_check);
  m.impl("packedmask_to_indexmask", packedmask_to_indexmask_check);
  m.impl("indexmask_to_packedmask", indexmask_to_packedmask_check);
  m.impl("topk_indices", topk_indices_check);
}

TORCH_LIBRARY_IMPL(cuda_attn, CUDA, m) {
  m.impl("full_attn", full_attn);
  m.impl("all_index_mask", all_index_mask);
  m.impl("sp_attn", sp_attn);
  m.impl("fullattn_maxq_denom", fullattn_maxq_denom);
  m.impl("maxq_denom", maxq_denom);
  m.impl("booleanmask_128", booleanmask_128);
  m.impl("booleanmask_to_indexmask", booleanmask_to_indexmask);
  m.impl("booleanmask_128_listed", booleanmask_128_listed);
  m.impl("block_index_lists", block_index_lists);
  m.impl("block_lists_from_maxima", block_lists_from_maxima);
  m.impl("sp_attn_blocks_ml", sp_attn_blocks_ml);
  m.impl("sp_attn_blocks", sp_attn_blocks);
  m.impl("sp_attn_blocks_hint", sp_attn_blocks_hint);
  m.impl("pack_mask", pack_mask);
  m.impl("unpack_mask", unpack_mask);
  m.impl("packedmask_to_indexmask", packedmask_to_indexmask);
  m.impl("indexmask_to_packedmask", indexmask_to_packedmask);
  m.impl("topk_indices", topk_indices);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("full_attn", &full_attn, "Full attention");
  m.def("sp_attn", &sp_attn, "Sparse attention");
  m.def("all_index_mask", &all_index_mask, "all index mask");
  m.def("maxq_denom", &maxq_denom, "maxq_denom");
  m.def("booleanmask_128", &booleanmask_128, "booleanmask_128");
  m.def("booleanmask_to_indexmask", &booleanmask_to_indexmask, "booleanmask_to_indexmask");
  m.def("fullattn_maxq_denom", &fullattn_maxq_denom, "fullattn_maxq_denom");
  m.def("booleanmask_128_listed", &booleanmask_128_listed, "token mask inside the kept 64x64 blocks");
  m.def("block_index_lists", &block_index_lists, "one-pass m/l + key-block lists");
  m.def("block_lists_from_maxima", &block_lists_from_maxima, "key-block lists for another threshold from kept block maxima");
  m.def("sp_attn_blocks_ml", &sp_attn_blocks_ml, "block-sparse attention, precomputed m/l");
  m.def("sp_attn_blocks", &sp_attn_blocks, "block-sparse attention, renormalising");
  m.def("sp_attn_blocks_hint", &sp_attn_blocks_hint, "block-sparse attention, renormalising, row-maximum hint");
  m.def("block_scratch_bytes", &block_scratch_bytes, "scratch bytes for block_index_lists");
  m.def("pack_mask", &pack_mask, "mask -> one bit per entry");
  m.def("unpack_mask", &unpack_mask, "one bit per entry -> mask");
  m.def("packedmask_to_indexmask", &packedmask_to_indexmask, "packed mask -> ascending index lists");
  m.def("indexmask_to_packedmask", &indexmask_to_packedmask, "index lists -> packed mask");
  m.def("topk_indices", &topk_indices, "top-k keys per query block");
  m.def("release_workspaces", &release_workspaces, "drop the cached per-stream scratch of the sparse operators");
}
