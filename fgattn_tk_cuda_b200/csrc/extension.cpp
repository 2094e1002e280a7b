// PyTorch operator boundary: registers the reference's seven `cuda_attn` operator schemas
// (python/extension.cpp:82,113,166,215,259,309,349 of sankeerth95/fgattn_tk_cuda) plus the
// block-granular additions, validates tensors and forwards raw pointers to the C ABI of
// libfgattn_b200 on the current CUDA stream.  Also a pybind module with the same names, like the
// reference's `spattn.cuda_attn` (python/extension.cpp:362-370).  No device code lives here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "fgattn_b200.h"

namespace {

void check_status(int st, const char* what) {
  TORCH_CHECK(st == FGATTN_OK, what, " failed: ", fgattn_status_string(st),
              st == FGATTN_CUDA_ERROR ? " (cudaError " + std::to_string(fgattn_last_cuda_error()) + ")" : "");
}

void check_bf16_4d(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
  TORCH_CHECK(t.dim() == 4 && t.is_contiguous(), name, " must be contiguous [B, H, S, D]");
}
void check_dtype(const torch::Tensor& t, at::ScalarType ty, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
  TORCH_CHECK(t.scalar_type() == ty, name, " has the wrong dtype");
}
void* stream_of(const torch::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// ---- the reference's seven operators ---------------------------------------------------------
void full_attn(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v) {
  check_bf16_4d(o, "o"); check_bf16_4d(q, "q"); check_bf16_4d(k, "k"); check_bf16_4d(v, "v");
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_full_attn(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), q.size(0), q.size(1),
                                q.size(2), q.size(3), k.size(2), k.size(2), 0.f, stream_of(q)), "full_attn");
}

void all_index_mask(torch::Tensor kv_indices, torch::Tensor kv_num_indices, int64_t batch, int64_t heads,
                    int64_t seqblocks, int64_t seq) {
  check_dtype(kv_indices, at::kInt, "kv_indices"); check_dtype(kv_num_indices, at::kInt, "kv_num_indices");
  c10::cuda::CUDAGuard guard(kv_indices.device());
  check_status(fgattn_all_index_mask(kv_indices.data_ptr<int>(), kv_num_indices.data_ptr<int>(), int(batch),
                                     int(heads), int(seqblocks), int(seq), int(kv_indices.size(3)),
                                     stream_of(kv_indices)), "all_index_mask");
}

void sp_attn(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kv_indices,
             torch::Tensor kv_num_indices) {
  check_bf16_4d(o, "o"); check_bf16_4d(q, "q"); check_bf16_4d(k, "k"); check_bf16_4d(v, "v");
  check_dtype(kv_indices, at::kInt, "kv_indices"); check_dtype(kv_num_indices, at::kInt, "kv_num_indices");
  c10::cuda::CUDAGuard guard(q.device());
  // scratch for the longest-first order of the thread blocks, from the stream-ordered caching allocator
  const int64_t ws_bytes = int64_t(fgattn_sp_attn_workspace_bytes(q.size(0), q.size(1), q.size(2)));
  torch::Tensor ws = torch::empty({ws_bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(q.device()));
  check_status(fgattn_sp_attn(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), kv_indices.data_ptr<int>(),
                              kv_num_indices.data_ptr<int>(), int(kv_indices.size(3)), q.size(0), q.size(1),
                              q.size(2), q.size(3), k.size(2), 0.f, ws.data_ptr(), size_t(ws_bytes), stream_of(q)),
               "sp_attn");
}

void fullattn_maxq_denom(torch::Tensor o, torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q,
                         torch::Tensor k, torch::Tensor v) {
  check_bf16_4d(o, "o"); check_bf16_4d(q, "q"); check_bf16_4d(k, "k"); check_bf16_4d(v, "v");
  check_dtype(o_max_q, at::kFloat, "o_max_q"); check_dtype(o_denom, at::kFloat, "o_denom");
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_fullattn_maxq_denom(o.data_ptr(), o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(),
                                          q.data_ptr(), k.data_ptr(), v.data_ptr(), q.size(0), q.size(1), q.size(2),
                                          q.size(3), k.size(2), k.size(2), 0.f, stream_of(q)), "fullattn_maxq_denom");
}

void maxq_denom(torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q, torch::Tensor k) {
  check_bf16_4d(q, "q"); check_bf16_4d(k, "k");
  check_dtype(o_max_q, at::kFloat, "o_max_q"); check_dtype(o_denom, at::kFloat, "o_denom");
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_maxq_denom(o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(), q.data_ptr(), k.data_ptr(),
                                 q.size(0), q.size(1), q.size(2), q.size(3), k.size(2), k.size(2), 0.f, stream_of(q)),
               "maxq_denom");
}

void booleanmask_128(torch::Tensor booleanmask, torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q,
                     torch::Tensor k, double threshold) {
  check_bf16_4d(q, "q"); check_bf16_4d(k, "k");
  check_dtype(booleanmask, at::kInt, "booleanmask");
  check_dtype(o_max_q, at::kFloat, "o_max_q"); check_dtype(o_denom, at::kFloat, "o_denom");
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_booleanmask_128(booleanmask.data_ptr<int>(), float(threshold), int(booleanmask.size(3)),
                                      o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(), q.data_ptr(),
                                      k.data_ptr(), q.size(0), q.size(1), q.size(2), q.size(3), k.size(2), k.size(2), 0.f,
                                      stream_of(q)), "booleanmask_128");
}

void booleanmask_128_listed(torch::Tensor booleanmask, torch::Tensor o_max_q, torch::Tensor o_denom, torch::Tensor q,
                            torch::Tensor k, double threshold, torch::Tensor kb_indices, torch::Tensor kb_counts) {
  check_bf16_4d(q, "q"); check_bf16_4d(k, "k");
  check_dtype(booleanmask, at::kInt, "booleanmask");
  check_dtype(o_max_q, at::kFloat, "o_max_q"); check_dtype(o_denom, at::kFloat, "o_denom");
  check_dtype(kb_indices, at::kInt, "kb_indices"); check_dtype(kb_counts, at::kInt, "kb_counts");
  c10::cuda::CUDAGuard guard(q.device());
  // scratch for the longest-first order of the thread blocks, from the stream-ordered caching allocator
  const int64_t ws_bytes = int64_t(fgattn_sp_attn_workspace_bytes(q.size(0), q.size(1), q.size(2)));
  torch::Tensor ws = torch::empty({ws_bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(q.device()));
  check_status(fgattn_booleanmask_128_listed(booleanmask.data_ptr<int>(), float(threshold), int(booleanmask.size(3)),
                                             o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(), q.data_ptr(),
                                             k.data_ptr(), kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(),
                                             int(kb_indices.size(3)), q.size(0), q.size(1), q.size(2), q.size(3),
                                             k.size(2), k.size(2), 0.f, ws.data_ptr(), size_t(ws_bytes), stream_of(q)),
               "booleanmask_128_listed");
}

void booleanmask_to_indexmask(torch::Tensor kv_indices, torch::Tensor kv_numindices, torch::Tensor booleanmask,
                              int64_t seq) {
  check_dtype(kv_indices, at::kInt, "kv_indices"); check_dtype(kv_numindices, at::kInt, "kv_numindices");
  check_dtype(booleanmask, at::kInt, "booleanmask");
  c10::cuda::CUDAGuard guard(booleanmask.device());
  check_status(fgattn_booleanmask_to_indexmask(kv_indices.data_ptr<int>(), kv_numindices.data_ptr<int>(),
                                               booleanmask.data_ptr<int>(), booleanmask.size(0), booleanmask.size(1),
                                               int(seq), booleanmask.size(2), booleanmask.size(3),
                                               stream_of(booleanmask)), "booleanmask_to_indexmask");
}

// ---- 64x64 block granularity (additions) -------------------------------------------------------
void block_index_lists(torch::Tensor kb_indices, torch::Tensor kb_counts, torch::Tensor o_max_q, torch::Tensor o_denom,
                       c10::optional<torch::Tensor> o, torch::Tensor q, torch::Tensor k,
                       c10::optional<torch::Tensor> v, double threshold, torch::Tensor scratch) {
  check_bf16_4d(q, "q"); check_bf16_4d(k, "k");
  check_dtype(kb_indices, at::kInt, "kb_indices"); check_dtype(kb_counts, at::kInt, "kb_counts");
  check_dtype(o_max_q, at::kFloat, "o_max_q"); check_dtype(o_denom, at::kFloat, "o_denom");
  TORCH_CHECK(scratch.is_cuda() && scratch.is_contiguous(), "scratch must be a contiguous CUDA tensor");
  if (o) check_bf16_4d(*o, "o");
  if (v) check_bf16_4d(*v, "v");
  c10::cuda::CUDAGuard guard(q.device());
  check_status(fgattn_block_index_lists(kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(), int(kb_indices.size(3)),
                                        o_max_q.data_ptr<float>(), o_denom.data_ptr<float>(),
                                        o ? o->data_ptr() : nullptr, q.data_ptr(), k.data_ptr(),
                                        v ? v->data_ptr() : nullptr, float(threshold), q.size(0), q.size(1), q.size(2),
                                        q.size(3), k.size(2), k.size(2), 0.f, scratch.data_ptr(),
                                        size_t(scratch.numel()) * scratch.element_size(), stream_of(q)),
               "block_index_lists");
}

void sp_attn_blocks_ml(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kb_indices,
                       torch::Tensor kb_counts, torch::Tensor max_q, torch::Tensor denom) {
  check_bf16_4d(o, "o"); check_bf16_4d(q, "q"); check_bf16_4d(k, "k"); check_bf16_4d(v, "v");
  check_dtype(kb_indices, at::kInt, "kb_indices"); check_dtype(kb_counts, at::kInt, "kb_counts");
  check_dtype(max_q, at::kFloat, "max_q"); check_dtype(denom, at::kFloat, "denom");
  c10::cuda::CUDAGuard guard(q.device());
  // work-queue scratch of the persistent kernel, from the stream-ordered caching allocator
  const int64_t ws_bytes = int64_t(fgattn_sp_attn_workspace_bytes(q.size(0), q.size(1), q.size(2)));
  torch::Tensor ws = torch::empty({ws_bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(q.device()));
  check_status(fgattn_sp_attn_blocks_ml(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                        kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(), int(kb_indices.size(3)),
                                        max_q.data_ptr<float>(), denom.data_ptr<float>(), q.size(0), q.size(1),
                                        q.size(2), q.size(3), k.size(2), k.size(2), 0.f, ws.data_ptr(), size_t(ws_bytes),
                                        stream_of(q)), "sp_attn_blocks_ml");
}

void sp_attn_blocks(torch::Tensor o, torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kb_indices,
                    torch::Tensor kb_counts) {
  check_bf16_4d(o, "o"); check_bf16_4d(q, "q"); check_bf16_4d(k, "k"); check_bf16_4d(v, "v");
  check_dtype(kb_indices, at::kInt, "kb_indices"); check_dtype(kb_counts, at::kInt, "kb_counts");
  c10::cuda::CUDAGuard guard(q.device());
  // scratch for the longest-first order of the thread blocks, from the stream-ordered caching allocator
  const int64_t ws_bytes = int64_t(fgattn_sp_attn_workspace_bytes(q.size(0), q.size(1), q.size(2)));
  torch::Tensor ws = torch::empty({ws_bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(q.device()));
  check_status(fgattn_sp_attn_blocks(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                     kb_indices.data_ptr<int>(), kb_counts.data_ptr<int>(), int(kb_indices.size(3)),
                                     q.size(0), q.size(1), q.size(2), q.size(3), k.size(2), k.size(2), 0.f,
                                     ws.data_ptr(), size_t(ws_bytes), stream_of(q)),
               "sp_attn_blocks");
}

// ---- one-bit-per-entry masks (additions) ---------------------------------------------------------
int mask_elem_size(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
  if (t.scalar_type() == at::kBool || t.scalar_type() == at::kByte) return 1;
  TORCH_CHECK(t.scalar_type() == at::kInt, name, " must be bool, uint8 or int32");
  return 4;
}

void pack_mask(torch::Tensor packed, torch::Tensor mask) {
  check_dtype(packed, at::kByte, "packed");
  const int es = mask_elem_size(mask, "mask");
  const int64_t W = mask.size(-1);
  TORCH_CHECK(W % 8 == 0 && packed.numel() * 8 == mask.numel(), "packed must hold one bit per mask entry");
  c10::cuda::CUDAGuard guard(mask.device());
  check_status(fgattn_pack_mask(packed.data_ptr<uint8_t>(), mask.data_ptr(), es, mask.numel() / W, int(W),
                                stream_of(mask)), "pack_mask");
}

void unpack_mask(torch::Tensor mask, torch::Tensor packed) {
  check_dtype(packed, at::kByte, "packed");
  const int es = mask_elem_size(mask, "mask");
  const int64_t W = mask.size(-1);
  TORCH_CHECK(W % 8 == 0 && packed.numel() * 8 == mask.numel(), "packed must hold one bit per mask entry");
  c10::cuda::CUDAGuard guard(mask.device());
  check_status(fgattn_unpack_mask(mask.data_ptr(), es, packed.data_ptr<uint8_t>(), mask.numel() / W, int(W),
                                  stream_of(mask)), "unpack_mask");
}

void packedmask_to_indexmask(torch::Tensor indices, torch::Tensor num_indices, torch::Tensor packed, int64_t n_valid,
                             int64_t sentinel) {
  check_dtype(indices, at::kInt, "indices"); check_dtype(num_indices, at::kInt, "num_indices");
  check_dtype(packed, at::kByte, "packed");
  const int64_t rows = packed.numel() / packed.size(-1);
  TORCH_CHECK(num_indices.numel() == rows && indices.numel() == rows * indices.size(-1), "row counts differ");
  c10::cuda::CUDAGuard guard(packed.device());
  check_status(fgattn_packedmask_to_indexmask(indices.data_ptr<int>(), num_indices.data_ptr<int>(),
                                              packed.data_ptr<uint8_t>(), rows, int(packed.size(-1) * 8),
                                              int(indices.size(-1)), int(n_valid), int(sentinel), stream_of(packed)),
               "packedmask_to_indexmask");
}

void indexmask_to_packedmask(torch::Tensor packed, torch::Tensor indices, torch::Tensor num_indices) {
  check_dtype(indices, at::kInt, "indices"); check_dtype(num_indices, at::kInt, "num_indices");
  check_dtype(packed, at::kByte, "packed");
  const int64_t rows = packed.numel() / packed.size(-1);
  TORCH_CHECK(num_indices.numel() == rows && indices.numel() == rows * indices.size(-1), "row counts differ");
  c10::cuda::CUDAGuard guard(packed.device());
  check_status(fgattn_indexmask_to_packedmask(packed.data_ptr<uint8_t>(), indices.data_ptr<int>(),
                                              num_indices.data_ptr<int>(), rows, int(indices.size(-1)),
                                              int(packed.size(-1) * 8), stream_of(packed)),
               "indexmask_to_packedmask");
}

// ---- top-k selector (addition) ------------------------------------------------------------------
void topk_indices(torch::Tensor kv_indices, torch::Tensor kv_num_indices, torch::Tensor q, torch::Tensor k,
                  int64_t select_k, int64_t blocksz) {
  check_bf16_4d(q, "q"); check_bf16_4d(k, "k");
  check_dtype(kv_indices, at::kInt, "kv_indices"); check_dtype(kv_num_indices, at::kInt, "kv_num_indices");
  TORCH_CHECK(kv_indices.dim() == 4, "kv_indices must be [B, H, blocks, stride]");
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

// Meta kernels: every operator writes into caller-allocated tensors and returns nothing.
void meta4(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor) {}
void meta_aim(torch::Tensor, torch::Tensor, int64_t, int64_t, int64_t, int64_t) {}
void meta6(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor) {}
void meta_bm(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, double) {}
void meta_b2i(torch::Tensor, torch::Tensor, torch::Tensor, int64_t) {}
void meta_bml(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, double, torch::Tensor,
              torch::Tensor) {}
void meta8(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor,
           torch::Tensor) {}
void meta_bil(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, c10::optional<torch::Tensor>, torch::Tensor,
              torch::Tensor, c10::optional<torch::Tensor>, double, torch::Tensor) {}
void meta2(torch::Tensor, torch::Tensor) {}
void meta3(torch::Tensor, torch::Tensor, torch::Tensor) {}
void meta_p2i(torch::Tensor, torch::Tensor, torch::Tensor, int64_t, int64_t) {}
void meta_topk(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, int64_t, int64_t) {}

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
  m.def("sp_attn_blocks_ml(Tensor (o!) o, Tensor q, Tensor k, Tensor v, Tensor kb_indices, Tensor kb_counts, Tensor max_q, Tensor denom) -> ()");
  m.def("sp_attn_blocks(Tensor (o!) o, Tensor q, Tensor k, Tensor v, Tensor kb_indices, Tensor kb_counts) -> ()");
  // one-bit-per-entry masks
  m.def("pack_mask(Tensor (packed!) packed, Tensor mask) -> ()");
  m.def("unpack_mask(Tensor (mask!) mask, Tensor packed) -> ()");
  m.def("packedmask_to_indexmask(Tensor (indices!) indices, Tensor (num_indices!) num_indices, Tensor packed, int n_valid, int sentinel) -> ()");
  m.def("indexmask_to_packedmask(Tensor (packed!) packed, Tensor indices, Tensor num_indices) -> ()");
  // top-k selector
  m.def("topk_indices(Tensor (kv_indices!) kv_indices, Tensor (kv_num_indices!) kv_num_indices, Tensor q, Tensor k, int select_k, int blocksz) -> ()");
}

TORCH_LIBRARY_IMPL(cuda_attn, Meta, m) {
  m.impl("full_attn", meta4);
  m.impl("all_index_mask", meta_aim);
  m.impl("sp_attn", meta6);
  m.impl("fullattn_maxq_denom", meta6);
  m.impl("maxq_denom", meta4);
  m.impl("booleanmask_128", meta_bm);
  m.impl("booleanmask_to_indexmask", meta_b2i);
  m.impl("booleanmask_128_listed", meta_bml);
  m.impl("block_index_lists", meta_bil);
  m.impl("sp_attn_blocks_ml", meta8);
  m.impl("sp_attn_blocks", meta6);
  m.impl("pack_mask", meta2);
  m.impl("unpack_mask", meta2);
  m.impl("packedmask_to_indexmask", meta_p2i);
  m.impl("indexmask_to_packedmask", meta3);
  m.impl("topk_indices", meta_topk);
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
  m.impl("sp_attn_blocks_ml", sp_attn_blocks_ml);
  m.impl("sp_attn_blocks", sp_attn_blocks);
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
  m.def("sp_attn_blocks_ml", &sp_attn_blocks_ml, "block-sparse attention, precomputed m/l");
  m.def("sp_attn_blocks", &sp_attn_blocks, "block-sparse attention, renormalising");
  m.def("block_scratch_bytes", &block_scratch_bytes, "scratch bytes for block_index_lists");
  m.def("pack_mask", &pack_mask, "mask -> one bit per entry");
  m.def("unpack_mask", &unpack_mask, "one bit per entry -> mask");
  m.def("packedmask_to_indexmask", &packedmask_to_indexmask, "packed mask -> ascending index lists");
  m.def("indexmask_to_packedmask", &indexmask_to_packedmask, "index lists -> packed mask");
  m.def("topk_indices", &topk_indices, "top-k keys per query block");
}
