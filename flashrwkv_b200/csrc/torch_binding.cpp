// PyTorch host layer of frwkv_b200: the `_C` module.
//
// It keeps the native entry names, argument order and error behaviour of the
// reference's `flashrwkv2._C` for the WKV7 time-mix path (pybind registrations in
// csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cpp:315-361 of the
// reference), checks tensors, allocates outputs/workspaces through Torch, and
// forwards raw pointers plus the current CUDA stream to the C ABI declared in
// include/frwkv_b200.h.  No kernel is defined or launched here.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cmath>
#include <limits>
#include <memory>
#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include "frwkv_b200.h"

namespace {

frwkv_stream_t current_stream(const torch::Tensor& t) {
  return reinterpret_cast<frwkv_stream_t>(at::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

void check_rc(int rc) {
  if (rc == FRWKV_OK) return;
  TORCH_CHECK(false, frwkv_last_error());
}

int io_dtype_of(const torch::Tensor& t) {
  return t.scalar_type() == torch::kBFloat16 ? FRWKV_DTYPE_BF16 : FRWKV_DTYPE_FP16;
}

void check_cuda_contiguous(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be CUDA");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

void check_same_device(const torch::Tensor& ref, const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.device() == ref.device(), name, " must be on the same device as state");
}

std::optional<uint32_t> tensor_version(const torch::Tensor& t) {
  if (t.unsafeGetTensorImpl()->is_inference()) return std::nullopt;
  return t.unsafeGetTensorImpl()->version_counter().current_version();
}

// Launches the device validation and returns {cu snapshot, idx snapshot, status[2]}.
struct PreparedMetadata {
  torch::Tensor cu, idx, status;
};

PreparedMetadata launch_validation(const torch::Tensor& cu, const torch::Tensor& idx, int64_t total_tokens,
                                   int64_t pool_size) {
  PreparedMetadata out;
  out.cu = torch::empty_like(cu);
  out.idx = torch::empty_like(idx);
  out.status = torch::empty({2}, cu.options());
  check_rc(frwkv_validate_recurrent_metadata(cu.data_ptr<int>(), idx.data_ptr<int>(),
                                             static_cast<int>(idx.numel()), static_cast<int>(total_tokens),
                                             static_cast<int>(pool_size), out.status.data_ptr<int>(),
                                             out.cu.data_ptr<int>(), out.idx.data_ptr<int>(),
                                             current_stream(cu)));
  return out;
}

// A validated-metadata ticket: binds a snapshot + status word to the identity,
// version, sizes and stream of the tensors it was prepared from, and refuses any
// later use that differs (same contract as the reference's
// RecurrentMetadataTicket, infer_recurrent_fp32io16_forward_varlen.cpp:88-201).
class MetadataTicket {
 public:
  MetadataTicket(torch::Tensor cu, torch::Tensor idx, PreparedMetadata prepared, int64_t total_tokens,
                 int64_t pool_size, int64_t max_seqlen, cudaStream_t stream)
      : cu_(std::move(cu)),
        idx_(std::move(idx)),
        prepared_(std::move(prepared)),
        cu_version_(tensor_version(cu_)),
        idx_version_(tensor_version(idx_)),
        cu_data_(cu_.data_ptr()),
        idx_data_(idx_.data_ptr()),
        cu_sizes_(cu_.sizes().vec()),
        idx_sizes_(idx_.sizes().vec()),
        total_tokens_(total_tokens),
        pool_size_(pool_size),
        max_seqlen_(max_seqlen),
        device_(cu_.device()),
        stream_(stream) {}

  void check_compatible(const torch::Tensor& cu, const torch::Tensor& idx, int64_t total_tokens,
                        int64_t pool_size, int64_t max_seqlen) const {
    TORCH_CHECK(cu.is_same(cu_), "validated_metadata query_start_loc identity mismatch");
    TORCH_CHECK(idx.is_same(idx_), "validated_metadata state_indices identity mismatch");
    TORCH_CHECK(cu.data_ptr() == cu_data_ && idx.data_ptr() == idx_data_,
                "validated_metadata metadata data_ptr mismatch");
    TORCH_CHECK(cu.sizes().vec() == cu_sizes_ && idx.sizes().vec() == idx_sizes_ && cu.is_contiguous() &&
                    idx.is_contiguous(),
                "validated_metadata metadata shape or stride mismatch");
    if (cu_version_.has_value()) {
      TORCH_CHECK(tensor_version(cu) == cu_version_, "validated_metadata query_start_loc version mismatch");
    }
    if (idx_version_.has_value()) {
      TORCH_CHECK(tensor_version(idx) == idx_version_, "validated_metadata state_indices version mismatch");
    }
    TORCH_CHECK(cu.device() == device_ && idx.device() == device_, "validated_metadata device mismatch");
    TORCH_CHECK(total_tokens == total_tokens_, "validated_metadata total_tokens mismatch");
    TORCH_CHECK(pool_size == pool_size_, "validated_metadata state_pool_size mismatch");
    if (max_seqlen > 0) {
      TORCH_CHECK(max_seqlen == max_seqlen_, "validated_metadata max_seqlen mismatch");
    }
    TORCH_CHECK(at::cuda::getCurrentCUDAStream(device_.index()).stream() == stream_,
                "validated_metadata stream mismatch; prepare and consume the ticket on the same CUDA stream");
  }

  const torch::Tensor& cu_snapshot() const { return prepared_.cu; }
  const torch::Tensor& idx_snapshot() const { return prepared_.idx; }
  const torch::Tensor& status() const { return prepared_.status; }
  int64_t max_seqlen() const { return max_seqlen_; }

 private:
  torch::Tensor cu_, idx_;
  PreparedMetadata prepared_;
  std::optional<uint32_t> cu_version_, idx_version_;
  void* cu_data_;
  void* idx_data_;
  std::vector<int64_t> cu_sizes_, idx_sizes_;
  int64_t total_tokens_, pool_size_, max_seqlen_;
  c10::Device device_;
  cudaStream_t stream_;
};

std::shared_ptr<MetadataTicket> prepare_recurrent_metadata(torch::Tensor cu, torch::Tensor idx,
                                                           int64_t total_tokens, int64_t pool_size,
                                                           int64_t max_seqlen) {
  check_cuda_contiguous(cu, "query_start_loc");
  check_cuda_contiguous(idx, "state_indices");
  check_same_device(cu, idx, "state_indices");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && idx.scalar_type() == torch::kInt32,
              "recurrent metadata must be int32");
  TORCH_CHECK(cu.dim() == 1 && idx.dim() == 1 && idx.numel() > 0 && cu.numel() == idx.numel() + 1,
              "query_start_loc must have shape [B+1] and state_indices shape [B]");
  TORCH_CHECK(idx.numel() <= 65535, "state_indices must contain at most 65535 sequences");
  TORCH_CHECK(total_tokens > 0 && total_tokens <= std::numeric_limits<int>::max(),
              "total_tokens must be positive and fit in int32");
  TORCH_CHECK(pool_size > 0 && pool_size <= std::numeric_limits<int>::max(),
              "state_pool_size must be positive and fit in int32");
  const c10::cuda::CUDAGuard guard(cu.device());
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(cu.device().index()).stream();
  auto prepared = launch_validation(cu, idx, total_tokens, pool_size);
  // One 8-byte read back: the status bits and the longest sequence.  This is the
  // only synchronisation of the path and happens once per ticket.
  int host_status[2] = {0, 0};
  C10_CUDA_CHECK(cudaMemcpyAsync(host_status, prepared.status.data_ptr<int>(), sizeof(host_status),
                                 cudaMemcpyDeviceToHost, stream));
  C10_CUDA_CHECK(cudaStreamSynchronize(stream));
  const int bits = host_status[0];
  TORCH_CHECK(!(bits & FRWKV_META_INVALID_ENDPOINT),
              "query_start_loc must start at 0 and its final offset must equal total_tokens");
  TORCH_CHECK(!(bits & FRWKV_META_INVALID_RANGE),
              "query_start_loc must be strictly increasing with non-empty sequences");
  TORCH_CHECK(!(bits & FRWKV_META_INVALID_SLOT), "state_indices entries must be within the state pool");
  TORCH_CHECK(!(bits & FRWKV_META_DUPLICATE_SLOT), "state_indices must be unique within one call");
  const int64_t inferred = host_status[1];
  if (max_seqlen <= 0) {
    max_seqlen = inferred;
  } else {
    TORCH_CHECK(max_seqlen == inferred, "max_seqlen must equal the largest packed sequence length");
  }
  return std::make_shared<MetadataTicket>(std::move(cu), std::move(idx), std::move(prepared), total_tokens,
                                          pool_size, max_seqlen, stream);
}

struct RecurrentDims {
  int64_t B, H, D;
};

RecurrentDims check_recurrent_layout(const torch::Tensor& cu, const torch::Tensor& idx,
                                     const torch::Tensor& state, const torch::Tensor& r,
                                     const torch::Tensor& w, const torch::Tensor& k, const torch::Tensor& v,
                                     const torch::Tensor& a, const torch::Tensor& b,
                                     const torch::Tensor& out, double scale) {
  const std::pair<const torch::Tensor*, const char*> all[] = {
      {&cu, "query_start_loc"}, {&idx, "state_indices"}, {&state, "state"}, {&r, "r"},
      {&w, "decay_logits"},     {&k, "k"},               {&v, "v"},         {&a, "a"},
      {&b, "b"},                {&out, "output"}};
  for (const auto& item : all) check_cuda_contiguous(*item.first, item.second);
  TORCH_CHECK(cu.scalar_type() == torch::kInt32, "query_start_loc must be int32");
  TORCH_CHECK(idx.scalar_type() == torch::kInt32, "state_indices must be int32");
  TORCH_CHECK(std::isfinite(scale), "scale must be finite");
  const int64_t B = idx.numel();
  TORCH_CHECK(B > 0 && B <= 65535, "state_indices must contain 1..65535 sequences");
  TORCH_CHECK(idx.dim() == 1, "state_indices must have shape [N]");
  TORCH_CHECK(cu.dim() == 1 && cu.size(0) == B + 1, "query_start_loc must have shape [N+1]");
  TORCH_CHECK(state.dim() == 4 && state.size(0) > 0 && state.size(1) > 0 && state.size(2) == state.size(3),
              "state must have square shape [slots,H,D,D]");
  TORCH_CHECK(state.scalar_type() == torch::kFloat32, "state must be float32");
  const int64_t D = state.size(2);
  TORCH_CHECK(D == 64 || D == 128 || D == 256, "recurrent head size must be 64, 128, or 256, got ", D);
  TORCH_CHECK(state.size(0) <= std::numeric_limits<int>::max(), "state slot count must fit in int32");
  const int64_t H = state.size(1);
  TORCH_CHECK(r.dim() == 3 && r.size(0) > 0 && r.size(1) == H && r.size(2) == D,
              "r must have shape [total_tokens,H,D] matching state");
  TORCH_CHECK(r.size(0) <= std::numeric_limits<int>::max(), "token count must fit in int32");
  TORCH_CHECK(r.sizes() == w.sizes() && r.sizes() == k.sizes() && r.sizes() == v.sizes() &&
                  r.sizes() == a.sizes() && r.sizes() == b.sizes() && r.sizes() == out.sizes(),
              "r,decay_logits,k,v,a,b,output shape mismatch");
  TORCH_CHECK(r.scalar_type() == torch::kFloat16 || r.scalar_type() == torch::kBFloat16,
              "token tensors must be float16 or bfloat16");
  const auto dt = r.scalar_type();
  TORCH_CHECK(dt == w.scalar_type() && dt == k.scalar_type() && dt == v.scalar_type() &&
                  dt == a.scalar_type() && dt == b.scalar_type() && dt == out.scalar_type(),
              "r,decay_logits,k,v,a,b,output dtype mismatch");
  for (const auto& item : all) check_same_device(state, *item.first, item.second);
  return {B, H, D};
}

void check_decay_bias(const std::optional<torch::Tensor>& bias, const torch::Tensor& state,
                      const torch::Tensor& r) {
  if (!bias.has_value()) return;
  check_cuda_contiguous(*bias, "decay_bias");
  check_same_device(state, *bias, "decay_bias");
  TORCH_CHECK(bias->scalar_type() == r.scalar_type(), "decay_bias must match the token tensor dtype");
  const int64_t H = state.size(1), D = state.size(2);
  TORCH_CHECK((bias->dim() == 1 && bias->numel() == H * D) ||
                  (bias->dim() == 2 && bias->size(0) == H && bias->size(1) == D),
              "decay_bias must have shape [H*D] or [H,D]");
}

void recurrent_fp32_from_decay_logits(torch::Tensor cu, torch::Tensor idx, torch::Tensor state,
                                      torch::Tensor r, torch::Tensor w, torch::Tensor k, torch::Tensor v,
                                      torch::Tensor a, torch::Tensor b, torch::Tensor output, double scale,
                                      std::optional<torch::Tensor> decay_bias,
                                      std::shared_ptr<MetadataTicket> ticket, int64_t max_seqlen,
                                      std::optional<torch::Tensor> output_fp32) {
  const auto dims = check_recurrent_layout(cu, idx, state, r, w, k, v, a, b, output, scale);
  check_decay_bias(decay_bias, state, r);
  if (output_fp32.has_value()) {
    check_cuda_contiguous(*output_fp32, "output_fp32");
    TORCH_CHECK(output_fp32->scalar_type() == torch::kFloat32 && output_fp32->sizes() == r.sizes() &&
                    output_fp32->device() == state.device(),
                "output_fp32 must be a float32 tensor shaped like r on the state's device");
  }
  const c10::cuda::CUDAGuard guard(state.device());
  torch::Tensor launch_cu, launch_idx, status;
  if (ticket) {
    ticket->check_compatible(cu, idx, r.size(0), state.size(0), max_seqlen);
    launch_cu = ticket->cu_snapshot();
    launch_idx = ticket->idx_snapshot();
    status = ticket->status();
    max_seqlen = ticket->max_seqlen();
  } else {
    auto prepared = launch_validation(cu, idx, r.size(0), state.size(0));
    launch_cu = std::move(prepared.cu);
    launch_idx = std::move(prepared.idx);
    status = std::move(prepared.status);
  }
  check_rc(frwkv_wkv7_recurrent_fp32io16_forward_varlen(
      launch_cu.data_ptr<int>(), launch_idx.data_ptr<int>(), status.data_ptr<int>(), state.data_ptr<float>(),
      r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
      decay_bias.has_value() ? decay_bias->data_ptr() : nullptr, output.data_ptr(),
      output_fp32.has_value() ? output_fp32->data_ptr<float>() : nullptr, static_cast<int>(r.size(0)),
      static_cast<int>(dims.B), static_cast<int>(dims.H), static_cast<int>(dims.D),
      static_cast<int>(std::min<int64_t>(std::max<int64_t>(max_seqlen, -1), std::numeric_limits<int>::max())),
      io_dtype_of(r), static_cast<float>(scale), current_stream(state)));
}

// ---- chunked forward ---------------------------------------------------------------------------------
void check_chunk_tables(const torch::Tensor& sco, const torch::Tensor& cs, const torch::Tensor& ce,
                        const torch::Tensor& ref) {
  const std::pair<const torch::Tensor*, const char*> all[] = {
      {&sco, "sequence_chunk_offsets"}, {&cs, "chunk_token_starts"}, {&ce, "chunk_token_ends"}};
  for (const auto& item : all) {
    check_cuda_contiguous(*item.first, item.second);
    TORCH_CHECK(item.first->scalar_type() == torch::kInt32, item.second, " must be int32");
    TORCH_CHECK(item.first->dim() == 1, item.second, " must be one-dimensional");
    TORCH_CHECK(item.first->device() == ref.device(), item.second, " must be on the token device");
  }
  TORCH_CHECK(sco.numel() >= 2, "sequence_chunk_offsets must have shape [B+1]");
  TORCH_CHECK(cs.numel() > 0 && cs.numel() == ce.numel(), "chunk_token_starts and chunk_token_ends must have shape [Cn]");
}

// Runs build + scan.  `state` [slots,H,64,64] fp32 is updated in place (slot = state_indices[s], or s when
// state_indices is None).  Returns the device error flag (int32[1]; non-zero = a tensor-core wait ran out).
torch::Tensor wkv7_chunk_forward(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce, torch::Tensor state,
                                 torch::Tensor r, torch::Tensor w, torch::Tensor k, torch::Tensor v, torch::Tensor a,
                                 torch::Tensor b, torch::Tensor output, double scale,
                                 std::optional<torch::Tensor> decay_bias, std::optional<torch::Tensor> state_indices,
                                 std::optional<torch::Tensor> boundary, std::optional<torch::Tensor> output_fp32,
                                 std::optional<torch::Tensor> metadata_status) {
  check_chunk_tables(sco, cs, ce, r);
  const std::pair<const torch::Tensor*, const char*> toks[] = {{&r, "r"}, {&w, "decay_logits"}, {&k, "k"},
                                                               {&v, "v"}, {&a, "a"},           {&b, "b"},
                                                               {&output, "output"}};
  for (const auto& item : toks) {
    check_cuda_contiguous(*item.first, item.second);
    TORCH_CHECK(item.first->device() == r.device(), item.second, " must share r's device");
    TORCH_CHECK(item.first->sizes() == r.sizes(), "r,decay_logits,k,v,a,b,output shape mismatch");
    TORCH_CHECK(item.first->scalar_type() == r.scalar_type(), "r,decay_logits,k,v,a,b,output dtype mismatch");
  }
  TORCH_CHECK(r.scalar_type() == torch::kFloat16 || r.scalar_type() == torch::kBFloat16,
              "token tensors must be float16 or bfloat16");
  TORCH_CHECK(r.dim() == 3 && r.size(0) > 0 && r.size(1) > 0, "token tensors must have shape [N,H,D]");
  TORCH_CHECK(r.size(2) == 64, "chunked WKV7 supports head size 64, got ", r.size(2));
  TORCH_CHECK(std::isfinite(scale), "scale must be finite");
  check_cuda_contiguous(state, "state");
  TORCH_CHECK(state.scalar_type() == torch::kFloat32, "state must be float32");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == r.size(1) && state.size(2) == 64 && state.size(3) == 64,
              "state must have shape [slots,H,D,D] matching the tokens");
  TORCH_CHECK(state.device() == r.device(), "state must share r's device");
  const int64_t B = sco.numel() - 1, Cn = cs.numel(), H = r.size(1);
  if (state_indices.has_value()) {
    check_cuda_contiguous(*state_indices, "state_indices");
    TORCH_CHECK(state_indices->scalar_type() == torch::kInt32 && state_indices->dim() == 1 &&
                    state_indices->numel() == B && state_indices->device() == r.device(),
                "state_indices must be int32 [B] on the token device");
  } else {
    TORCH_CHECK(state.size(0) >= B, "state must hold one slot per sequence");
  }
  check_decay_bias(decay_bias, state, r);
  if (boundary.has_value()) {
    check_cuda_contiguous(*boundary, "boundary");
    TORCH_CHECK(boundary->scalar_type() == torch::kFloat32 && boundary->dim() == 4 && boundary->size(0) == Cn &&
                    boundary->size(1) == H && boundary->size(2) == 64 && boundary->size(3) == 64 &&
                    boundary->device() == r.device(),
                "boundary must be float32 [Cn,H,D,D] on the token device");
  }
  if (output_fp32.has_value()) {
    check_cuda_contiguous(*output_fp32, "output_fp32");
    TORCH_CHECK(output_fp32->scalar_type() == torch::kFloat32 && output_fp32->sizes() == r.sizes() &&
                    output_fp32->device() == r.device(),
                "output_fp32 must be a float32 tensor shaped like r");
  }
  if (metadata_status.has_value()) {
    TORCH_CHECK(metadata_status->is_cuda() && metadata_status->scalar_type() == torch::kInt32 &&
                    metadata_status->numel() >= 1 && metadata_status->device() == r.device(),
                "metadata_status must be an int32 CUDA tensor");
  }
  const c10::cuda::CUDAGuard guard(r.device());
  const size_t ws_bytes = frwkv_wkv7_chunk_workspace_bytes(static_cast<int>(Cn), static_cast<int>(H));
  auto workspace = torch::empty({static_cast<int64_t>(ws_bytes)}, r.options().dtype(torch::kUInt8));
  auto error_flag = torch::zeros({1}, r.options().dtype(torch::kInt32));
  check_rc(frwkv_wkv7_chunk_fp32io16_forward(
      sco.data_ptr<int>(), cs.data_ptr<int>(), ce.data_ptr<int>(),
      state_indices.has_value() ? state_indices->data_ptr<int>() : nullptr,
      metadata_status.has_value() ? metadata_status->data_ptr<int>() : nullptr, state.data_ptr<float>(), r.data_ptr(),
      w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
      decay_bias.has_value() ? decay_bias->data_ptr() : nullptr, output.data_ptr(),
      output_fp32.has_value() ? output_fp32->data_ptr<float>() : nullptr,
      boundary.has_value() ? boundary->data_ptr<float>() : nullptr, workspace.data_ptr(), ws_bytes,
      error_flag.data_ptr<int>(), static_cast<int>(r.size(0)), static_cast<int>(B), static_cast<int>(Cn),
      static_cast<int>(H), 64, io_dtype_of(r), static_cast<float>(scale), current_stream(r)));
  return error_flag;
}

// Reference-named entry (csrc/sm90/rl_infctx/wkv7/rl_infctx_chunk_fp32io16_forward.cpp:157-241 there): the
// input state [B,H,D,D] is cloned, both strategies run the same tensor-core path.
std::tuple<torch::Tensor, torch::Tensor> rl_infctx_chunk_fp32io16_forward(
    torch::Tensor sco, torch::Tensor cs, torch::Tensor ce, torch::Tensor state, torch::Tensor r, torch::Tensor w,
    torch::Tensor k, torch::Tensor v, torch::Tensor a, torch::Tensor b, int64_t strategy, double scale,
    std::optional<torch::Tensor> decay_bias) {
  TORCH_CHECK(strategy == 0 || strategy == 1, "strategy must be 0 (materialized) or 1 (recompute)");
  check_cuda_contiguous(state, "state");
  auto working = state.clone();
  auto output = torch::empty_like(v);
  wkv7_chunk_forward(sco, cs, ce, working, r, w, k, v, a, b, output, scale, decay_bias, std::nullopt, std::nullopt,
                     std::nullopt, std::nullopt);
  return {output, working};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "frwkv_b200 host layer (WKV7 time-mix path for sm_100a)";
  m.def("abi_version", []() { return frwkv_abi_version(); });
  py::class_<MetadataTicket, std::shared_ptr<MetadataTicket>>(m, "_RecurrentMetadataTicket")
      .def("_check_compatible", &MetadataTicket::check_compatible, py::arg("query_start_loc"),
           py::arg("state_indices"), py::arg("total_tokens"), py::arg("state_pool_size"),
           py::arg("max_seqlen"))
      .def("_query_start_loc_snapshot", [](const MetadataTicket& t) { return t.cu_snapshot(); })
      .def("_state_indices_snapshot", [](const MetadataTicket& t) { return t.idx_snapshot(); })
      .def("_status", [](const MetadataTicket& t) { return t.status().narrow(0, 0, 1); })
      .def("_max_seqlen", [](const MetadataTicket& t) { return t.max_seqlen(); });
  m.def("prepare_recurrent_metadata", &prepare_recurrent_metadata, py::arg("query_start_loc"),
        py::arg("state_indices"), py::arg("total_tokens"), py::arg("state_pool_size"),
        py::arg("max_seqlen") = -1);
  m.def("recurrent_fp32_from_decay_logits", &recurrent_fp32_from_decay_logits, py::arg("query_start_loc"),
        py::arg("state_indices"), py::arg("state"), py::arg("r"), py::arg("decay_logits"), py::arg("k"),
        py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"), py::arg("scale"),
        py::arg("decay_bias") = py::none(), py::arg("validated_metadata") = py::none(),
        py::arg("max_seqlen") = -1, py::arg("output_fp32") = py::none());
  m.def("wkv7_chunk_forward", &wkv7_chunk_forward, py::arg("sequence_chunk_offsets"),
        py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("state"), py::arg("r"),
        py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"),
        py::arg("scale") = 1.0, py::arg("decay_bias") = py::none(), py::arg("state_indices") = py::none(),
        py::arg("boundary") = py::none(), py::arg("output_fp32") = py::none(),
        py::arg("metadata_status") = py::none());
  m.def("rl_infctx_chunk_fp32io16_forward", &rl_infctx_chunk_fp32io16_forward, py::arg("sequence_chunk_offsets"),
        py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("state"), py::arg("r"),
        py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("strategy") = 1,
        py::arg("scale") = 1.0, py::arg("decay_bias") = py::none());
}
