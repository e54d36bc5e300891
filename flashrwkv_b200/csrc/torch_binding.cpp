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
#include <map>
#include <mutex>
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

// ---- device error words ------------------------------------------------------------------------------------------------
// Kernels with bounded waits report a wait that ran out through an int32 word on the device (and write NaN instead of
// results).  No operator synchronises to read it; the words of the latest launches are kept here by stage name, and
// `last_error_flags()` hands them to Python, where reading them is the caller's decision.
std::mutex g_flags_mutex;
std::map<std::string, torch::Tensor> g_last_flags;
void remember_flag(const std::string& stage, const torch::Tensor& flag) {
  const std::lock_guard<std::mutex> lock(g_flags_mutex);
  g_last_flags[stage] = flag;
}
std::map<std::string, torch::Tensor> last_error_flags() {
  const std::lock_guard<std::mutex> lock(g_flags_mutex);
  return g_last_flags;
}
// one sticky word per device for the projection kernels (tensor-core GEMMs): zero until a wait runs out
torch::Tensor linear_flag(const torch::Tensor& like) {
  static std::map<int, torch::Tensor> words;
  const std::lock_guard<std::mutex> lock(g_flags_mutex);
  const int dev = static_cast<int>(like.device().index());
  auto it = words.find(dev);
  if (it == words.end()) {
    it = words.emplace(dev, torch::zeros({1}, like.options().dtype(torch::kInt32))).first;
    g_last_flags["tmix_linear"] = it->second;
  }
  return it->second;
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
                 int64_t pool_size, int64_t max_seqlen, cudaStream_t stream, bool direct_slots)
      : direct_slots_(direct_slots),
        cu_(std::move(cu)),
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

  // Number of launches made with this ticket so far; decode launches alternate their traversal order with it.
  int next_launch_parity() { return static_cast<int>(launches_++ & 1); }
  const torch::Tensor& cu_snapshot() const { return prepared_.cu; }
  const torch::Tensor& idx_snapshot() const { return prepared_.idx; }
  const torch::Tensor& status() const { return prepared_.status; }
  int64_t max_seqlen() const { return max_seqlen_; }
  // sequence i is token i and owns state slot i (checked on the device and read back when the ticket was made)
  bool direct_slots() const { return direct_slots_; }

 private:
  bool direct_slots_;
  torch::Tensor cu_, idx_;
  PreparedMetadata prepared_;
  std::optional<uint32_t> cu_version_, idx_version_;
  void* cu_data_;
  void* idx_data_;
  std::vector<int64_t> cu_sizes_, idx_sizes_;
  int64_t total_tokens_, pool_size_, max_seqlen_;
  c10::Device device_;
  cudaStream_t stream_;
  uint64_t launches_ = 0;
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
  // ... and whether every sequence is one token in the slot of its own number (decode launches are then shorter)
  auto direct_flag = torch::empty({1}, cu.options());
  check_rc(frwkv_recurrent_metadata_is_direct(prepared.cu.data_ptr<int>(), prepared.idx.data_ptr<int>(),
                                              static_cast<int>(idx.numel()), direct_flag.data_ptr<int>(), stream));
  // One read back: the status bits, the longest sequence and that flag.  This is the
  // only synchronisation of the path and happens once per ticket.
  int host_status[2] = {0, 0};
  int host_direct = 0;
  C10_CUDA_CHECK(cudaMemcpyAsync(host_status, prepared.status.data_ptr<int>(), sizeof(host_status),
                                 cudaMemcpyDeviceToHost, stream));
  C10_CUDA_CHECK(cudaMemcpyAsync(&host_direct, direct_flag.data_ptr<int>(), sizeof(host_direct),
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
                                          pool_size, max_seqlen, stream, host_direct == 1);
}

struct RecurrentDims {
  int64_t B, H, D;
};

RecurrentDims check_recurrent_layout(const torch::Tensor& cu, const torch::Tensor& idx,
                                     const torch::Tensor& state, const torch::Tensor& r,
                                     const torch::Tensor& w, const torch::Tensor& k, const torch::Tensor& v,
                                     const torch::Tensor& a, const torch::Tensor& b,
                                     const torch::Tensor& out, double scale,
                                     torch::ScalarType state_type = torch::kFloat32) {
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
  TORCH_CHECK(state.scalar_type() == state_type,
              state_type == torch::kFloat32 ? "state must be float32" : "state must be float16");
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
  int flags = 0;
  if (ticket) {
    ticket->check_compatible(cu, idx, r.size(0), state.size(0), max_seqlen);
    flags = ticket->next_launch_parity() ? FRWKV_RECURRENT_REVERSE_ORDER : 0;
    if (ticket->direct_slots()) flags |= FRWKV_RECURRENT_DIRECT_SLOTS;
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
  check_rc(frwkv_wkv7_recurrent_fp32io16_forward_varlen_ex(
      launch_cu.data_ptr<int>(), launch_idx.data_ptr<int>(), status.data_ptr<int>(), state.data_ptr<float>(),
      r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
      decay_bias.has_value() ? decay_bias->data_ptr() : nullptr, output.data_ptr(),
      output_fp32.has_value() ? output_fp32->data_ptr<float>() : nullptr, static_cast<int>(r.size(0)),
      static_cast<int>(dims.B), static_cast<int>(dims.H), static_cast<int>(dims.D),
      static_cast<int>(std::min<int64_t>(std::max<int64_t>(max_seqlen, -1), std::numeric_limits<int>::max())),
      io_dtype_of(r), static_cast<float>(scale), flags, current_stream(state)));
}

// ---- fp16-state recurrence (reference entry names and argument order:
// csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cpp:275-301) ------------------------------------------
void check_elapsed(const torch::Tensor& elapsed, const char* name) {
  check_cuda_contiguous(elapsed, name);
  TORCH_CHECK(elapsed.scalar_type() == torch::kInt32, name, " must be int32");
  TORCH_CHECK(elapsed.numel() > 0, name, " must be non-empty");
}

void recurrent_fp16_from_decay_logits(torch::Tensor cu, torch::Tensor idx, torch::Tensor elapsed, torch::Tensor state,
                                      torch::Tensor r, torch::Tensor w, torch::Tensor k, torch::Tensor v,
                                      torch::Tensor a, torch::Tensor b, torch::Tensor output, double scale,
                                      std::optional<torch::Tensor> decay_bias,
                                      std::shared_ptr<MetadataTicket> ticket, int64_t max_seqlen) {
  const auto dims = check_recurrent_layout(cu, idx, state, r, w, k, v, a, b, output, scale, torch::kFloat16);
  check_decay_bias(decay_bias, state, r);
  check_elapsed(elapsed, "elapsed_state_pool");
  check_same_device(state, elapsed, "elapsed_state_pool");
  TORCH_CHECK(elapsed.dim() == 1 && elapsed.size(0) == state.size(0),
              "elapsed_state_pool must have shape [state_pool_slots]");
  const c10::cuda::CUDAGuard guard(state.device());
  torch::Tensor launch_cu, launch_idx, status;
  int flags = 0;
  if (ticket) {
    ticket->check_compatible(cu, idx, r.size(0), state.size(0), max_seqlen);
    flags = ticket->next_launch_parity() ? FRWKV_RECURRENT_REVERSE_ORDER : 0;
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
  check_rc(frwkv_wkv7_recurrent_fp16_forward_varlen(
      launch_cu.data_ptr<int>(), launch_idx.data_ptr<int>(), status.data_ptr<int>(), elapsed.data_ptr<int>(),
      state.data_ptr(), r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
      decay_bias.has_value() ? decay_bias->data_ptr() : nullptr, output.data_ptr(), static_cast<int>(r.size(0)),
      static_cast<int>(dims.B), static_cast<int>(dims.H), static_cast<int>(dims.D),
      static_cast<int>(std::min<int64_t>(std::max<int64_t>(max_seqlen, -1), std::numeric_limits<int>::max())),
      io_dtype_of(r), static_cast<float>(scale), flags, current_stream(state)));
}

void recurrent_fp16_advance_i32(torch::Tensor elapsed, int64_t amount) {
  check_elapsed(elapsed, "elapsed_state");
  TORCH_CHECK(amount >= std::numeric_limits<int>::min() && amount <= std::numeric_limits<int>::max(),
              "amount must fit in int32");
  const c10::cuda::CUDAGuard guard(elapsed.device());
  check_rc(frwkv_recurrent_fp16_advance_i32(elapsed.data_ptr<int>(), elapsed.numel(), static_cast<int>(amount),
                                            current_stream(elapsed)));
}

void recurrent_fp16_advance_i32_varlen(torch::Tensor cu, torch::Tensor idx, torch::Tensor elapsed,
                                       int64_t total_tokens, std::shared_ptr<MetadataTicket> ticket) {
  check_elapsed(elapsed, "elapsed_state_pool");
  TORCH_CHECK(elapsed.dim() == 1, "elapsed_state_pool must have shape [slots]");
  check_cuda_contiguous(cu, "query_start_loc");
  check_cuda_contiguous(idx, "state_indices");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && idx.scalar_type() == torch::kInt32,
              "query_start_loc and state_indices must be int32");
  TORCH_CHECK(idx.dim() == 1 && idx.numel() > 0 && cu.dim() == 1 && cu.numel() == idx.numel() + 1,
              "query_start_loc must have shape [B+1] and state_indices shape [B]");
  TORCH_CHECK(total_tokens > 0, "total_tokens must be positive");
  check_same_device(elapsed, cu, "query_start_loc");
  check_same_device(elapsed, idx, "state_indices");
  const c10::cuda::CUDAGuard guard(elapsed.device());
  torch::Tensor launch_cu, launch_idx, status;
  if (ticket) {
    ticket->check_compatible(cu, idx, total_tokens, elapsed.size(0), -1);
    launch_cu = ticket->cu_snapshot();
    launch_idx = ticket->idx_snapshot();
    status = ticket->status();
  } else {
    auto prepared = launch_validation(cu, idx, total_tokens, elapsed.size(0));
    launch_cu = std::move(prepared.cu);
    launch_idx = std::move(prepared.idx);
    status = std::move(prepared.status);
  }
  check_rc(frwkv_recurrent_fp16_advance_i32_varlen(elapsed.data_ptr<int>(), launch_cu.data_ptr<int>(),
                                                   launch_idx.data_ptr<int>(), status.data_ptr<int>(),
                                                   static_cast<int>(idx.numel()), current_stream(elapsed)));
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

// The device-side verdict on caller-built chunk tables (int32[1], zero = good): kernels given it fail closed
torch::Tensor chunk_table_status(const torch::Tensor& sco, const torch::Tensor& cs, const torch::Tensor& ce,
                                 const torch::Tensor& r) {
  auto status = torch::empty({1}, r.options().dtype(torch::kInt32));
  check_rc(frwkv_validate_chunk_tables(sco.data_ptr<int>(), cs.data_ptr<int>(), ce.data_ptr<int>(),
                                       static_cast<int>(sco.numel() - 1), static_cast<int>(cs.numel()),
                                       static_cast<int>(r.size(0)), 64, status.data_ptr<int>(), current_stream(r)));
  return status;
}

// Chunked forward.  `state` [slots,H,64,64] fp32 is updated in place (slot = state_indices[s], or s when
// state_indices is None).  Returns the device error flag (int32[1]; non-zero = a tensor-core wait ran out).
// `path`: 0 = build + scan kernels with a workspace, 1 = the fused single kernel, -1 = whichever
// frwkv_wkv7_chunk_prefers_fused picks for the batch.  `state_dot_a` (fp32 [N,H,64]) is written by the fused
// kernel only, so asking for it selects that kernel.
torch::Tensor wkv7_chunk_forward(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce, torch::Tensor state,
                                 torch::Tensor r, torch::Tensor w, torch::Tensor k, torch::Tensor v, torch::Tensor a,
                                 torch::Tensor b, torch::Tensor output, double scale,
                                 std::optional<torch::Tensor> decay_bias, std::optional<torch::Tensor> state_indices,
                                 std::optional<torch::Tensor> boundary, std::optional<torch::Tensor> output_fp32,
                                 std::optional<torch::Tensor> metadata_status,
                                 std::optional<torch::Tensor> state_dot_a, int64_t path) {
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
  if (state_dot_a.has_value()) {
    check_cuda_contiguous(*state_dot_a, "state_dot_a");
    TORCH_CHECK(state_dot_a->scalar_type() == torch::kFloat32 && state_dot_a->sizes() == r.sizes() &&
                    state_dot_a->device() == r.device(),
                "state_dot_a must be a float32 tensor shaped like r");
  }
  TORCH_CHECK(path >= -1 && path <= 1, "path must be -1 (automatic), 0 (build + scan) or 1 (fused)");
  TORCH_CHECK(!(state_dot_a.has_value() && path == 0), "state_dot_a is produced by the fused kernel only");
  const c10::cuda::CUDAGuard guard(r.device());
  auto error_flag = torch::zeros({1}, r.options().dtype(torch::kInt32));
  remember_flag("wkv7_chunk_forward", error_flag);
  const bool fused = path == 1 || state_dot_a.has_value() ||
                     (path == -1 && frwkv_wkv7_chunk_prefers_fused(static_cast<int>(B), static_cast<int>(H)) != 0);
  if (fused) {
    check_rc(frwkv_wkv7_chunk_fused_fp32io16_forward(
        sco.data_ptr<int>(), cs.data_ptr<int>(), ce.data_ptr<int>(),
        state_indices.has_value() ? state_indices->data_ptr<int>() : nullptr,
        metadata_status.has_value() ? metadata_status->data_ptr<int>() : nullptr, state.data_ptr<float>(),
        r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
        decay_bias.has_value() ? decay_bias->data_ptr() : nullptr, output.data_ptr(),
        output_fp32.has_value() ? output_fp32->data_ptr<float>() : nullptr,
        boundary.has_value() ? boundary->data_ptr<float>() : nullptr,
        state_dot_a.has_value() ? state_dot_a->data_ptr<float>() : nullptr, error_flag.data_ptr<int>(),
        static_cast<int>(r.size(0)), static_cast<int>(B), static_cast<int>(Cn), static_cast<int>(H), 64,
        io_dtype_of(r), static_cast<float>(scale), current_stream(r)));
    return error_flag;
  }
  const size_t ws_bytes = frwkv_wkv7_chunk_workspace_bytes(static_cast<int>(Cn), static_cast<int>(H));
  auto workspace = torch::empty({static_cast<int64_t>(ws_bytes)}, r.options().dtype(torch::kUInt8));
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
                     std::nullopt, std::nullopt, std::nullopt, -1);
  return {output, working};
}

// ---- TMix ---------------------------------------------------------------------------------------------
void check_io16(const torch::Tensor& t, const char* name, const torch::Tensor& ref) {
  check_cuda_contiguous(t, name);
  TORCH_CHECK(t.scalar_type() == torch::kFloat16 || t.scalar_type() == torch::kBFloat16, name,
              " must be float16 or bfloat16");
  TORCH_CHECK(t.scalar_type() == ref.scalar_type(), name, " dtype mismatch");
  TORCH_CHECK(t.device() == ref.device(), name, " must share x's device");
}

std::vector<torch::Tensor> tmix_mix6_forward_varlen(torch::Tensor x, torch::Tensor shift_state_pool, torch::Tensor x_r,
                                                    torch::Tensor x_w, torch::Tensor x_k, torch::Tensor x_v,
                                                    torch::Tensor x_a, torch::Tensor x_g, torch::Tensor cu,
                                                    torch::Tensor idx, int64_t max_seqlen,
                                                    std::shared_ptr<MetadataTicket> ticket) {
  check_io16(x, "x", x);
  TORCH_CHECK(x.dim() == 2 && x.size(0) > 0 && x.size(1) > 0, "x must have packed shape [total_tokens,C]");
  TORCH_CHECK(x.size(1) % 8 == 0, "C must be a multiple of 8");
  const std::pair<const torch::Tensor*, const char*> vecs[] = {{&x_r, "x_r"}, {&x_w, "x_w"}, {&x_k, "x_k"},
                                                               {&x_v, "x_v"}, {&x_a, "x_a"}, {&x_g, "x_g"}};
  for (const auto& item : vecs) {
    check_io16(*item.first, item.second, x);
    TORCH_CHECK(item.first->dim() == 1 && item.first->size(0) == x.size(1), "all mix6 coefficients must have shape [C]");
  }
  check_io16(shift_state_pool, "shift_state_pool", x);
  TORCH_CHECK(shift_state_pool.dim() == 2 && shift_state_pool.size(1) == x.size(1),
              "shift_state_pool must have shape [slots,C]");
  check_cuda_contiguous(cu, "cu_seqlens");
  check_cuda_contiguous(idx, "state_indices");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && idx.scalar_type() == torch::kInt32, "recurrent metadata must be int32");
  TORCH_CHECK(cu.dim() == 1 && idx.dim() == 1 && idx.numel() > 0 && cu.numel() == idx.numel() + 1,
              "cu_seqlens must have shape [B+1] and state_indices shape [B]");
  const c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor launch_cu, launch_idx, status;
  if (ticket) {
    ticket->check_compatible(cu, idx, x.size(0), shift_state_pool.size(0), max_seqlen);
    launch_cu = ticket->cu_snapshot();
    launch_idx = ticket->idx_snapshot();
    status = ticket->status();
    max_seqlen = ticket->max_seqlen();
  } else {
    auto prepared = launch_validation(cu, idx, x.size(0), shift_state_pool.size(0));
    launch_cu = std::move(prepared.cu);
    launch_idx = std::move(prepared.idx);
    status = std::move(prepared.status);
  }
  auto out = torch::empty({6, x.size(0), x.size(1)}, x.options());
  check_rc(frwkv_tmix_mix6_forward_varlen(
      x.data_ptr(), shift_state_pool.data_ptr(), x_r.data_ptr(), x_w.data_ptr(), x_k.data_ptr(), x_v.data_ptr(),
      x_a.data_ptr(), x_g.data_ptr(), launch_cu.data_ptr<int>(), launch_idx.data_ptr<int>(), status.data_ptr<int>(),
      out.data_ptr(), static_cast<int>(x.size(0)), static_cast<int>(idx.numel()), static_cast<int>(x.size(1)),
      static_cast<int>(std::min<int64_t>(max_seqlen, std::numeric_limits<int>::max())), io_dtype_of(x),
      current_stream(x)));
  return out.unbind(0);
}

// ---- add + LayerNorm family (reference entry names: tmix_layer_norm_forward_varlen, tmix_add_layer_norm_forward_varlen,
// tmix_add_last_layer_norm_forward_varlen, tmix_add_forward_varlen, tmix_mix6_add_layer_norm_forward_varlen) -------------
void check_norm_inputs(const torch::Tensor& x, const torch::Tensor* residual, const torch::Tensor* weight,
                       const torch::Tensor* bias) {
  check_io16(x, "x", x);
  TORCH_CHECK(x.dim() == 2 && x.size(0) > 0 && x.size(1) > 0, "x must have packed shape [total_tokens,C]");
  TORCH_CHECK(x.size(1) % 8 == 0, "C must be a multiple of 8");
  if (residual != nullptr) {
    check_io16(*residual, "residual", x);
    TORCH_CHECK(residual->sizes() == x.sizes(), "residual must have the same shape as x");
  }
  if (weight != nullptr) {
    check_io16(*weight, "weight", x);
    check_io16(*bias, "bias", x);
    TORCH_CHECK(weight->dim() == 1 && weight->size(0) == x.size(1) && bias->sizes() == weight->sizes(),
                "weight and bias must have shape [C]");
  }
}

torch::Tensor tmix_layer_norm_forward_varlen(torch::Tensor x, torch::Tensor weight, torch::Tensor bias, double eps) {
  check_norm_inputs(x, nullptr, &weight, &bias);
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  check_rc(frwkv_tmix_add_layer_norm_forward(x.data_ptr(), nullptr, weight.data_ptr(), bias.data_ptr(), nullptr,
                                             out.data_ptr(), x.size(0), static_cast<int>(x.size(1)),
                                             static_cast<float>(eps), io_dtype_of(x), current_stream(x)));
  return out;
}

std::tuple<torch::Tensor, torch::Tensor> tmix_add_layer_norm_forward_varlen(torch::Tensor x, torch::Tensor residual,
                                                                            torch::Tensor weight, torch::Tensor bias,
                                                                            double eps, int64_t batch_size) {
  (void)batch_size;  // the reference picks between two statistics kernels with it; there is one here
  check_norm_inputs(x, &residual, &weight, &bias);
  const c10::cuda::CUDAGuard guard(x.device());
  auto sum = torch::empty_like(x), out = torch::empty_like(x);
  check_rc(frwkv_tmix_add_layer_norm_forward(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                             sum.data_ptr(), out.data_ptr(), x.size(0), static_cast<int>(x.size(1)),
                                             static_cast<float>(eps), io_dtype_of(x), current_stream(x)));
  return {sum, out};
}

torch::Tensor tmix_add_last_layer_norm_forward_varlen(torch::Tensor x, torch::Tensor residual, torch::Tensor weight,
                                                      torch::Tensor bias, double eps) {
  check_norm_inputs(x, &residual, &weight, &bias);
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  check_rc(frwkv_tmix_add_layer_norm_forward(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                             nullptr, out.data_ptr(), x.size(0), static_cast<int>(x.size(1)),
                                             static_cast<float>(eps), io_dtype_of(x), current_stream(x)));
  return out;
}

torch::Tensor tmix_add_forward_varlen(torch::Tensor x, torch::Tensor residual) {
  check_norm_inputs(x, &residual, nullptr, nullptr);
  const c10::cuda::CUDAGuard guard(x.device());
  auto sum = torch::empty_like(x);
  check_rc(frwkv_tmix_add_layer_norm_forward(x.data_ptr(), residual.data_ptr(), nullptr, nullptr, sum.data_ptr(), nullptr,
                                             x.size(0), static_cast<int>(x.size(1)), 1.0f, io_dtype_of(x),
                                             current_stream(x)));
  return sum;
}

// Fused form for batches of one-token sequences; returns (sum, x_r, x_w, x_k, x_v, x_a, x_g mixes).
std::vector<torch::Tensor> tmix_mix6_add_layer_norm_forward_varlen(
    torch::Tensor x, torch::Tensor residual, torch::Tensor weight, torch::Tensor bias, torch::Tensor shift_state_pool,
    torch::Tensor x_r, torch::Tensor x_w, torch::Tensor x_k, torch::Tensor x_v, torch::Tensor x_a, torch::Tensor x_g,
    torch::Tensor cu, torch::Tensor idx, int64_t max_seqlen, double eps, std::shared_ptr<MetadataTicket> ticket) {
  check_norm_inputs(x, &residual, &weight, &bias);
  const std::pair<const torch::Tensor*, const char*> vecs[] = {{&x_r, "x_r"}, {&x_w, "x_w"}, {&x_k, "x_k"},
                                                               {&x_v, "x_v"}, {&x_a, "x_a"}, {&x_g, "x_g"}};
  for (const auto& item : vecs) {
    check_io16(*item.first, item.second, x);
    TORCH_CHECK(item.first->dim() == 1 && item.first->size(0) == x.size(1), "all mix6 coefficients must have shape [C]");
  }
  check_io16(shift_state_pool, "shift_state_pool", x);
  TORCH_CHECK(shift_state_pool.dim() == 2 && shift_state_pool.size(1) == x.size(1),
              "shift_state_pool must have shape [slots,C]");
  check_cuda_contiguous(cu, "cu_seqlens");
  check_cuda_contiguous(idx, "state_indices");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && idx.scalar_type() == torch::kInt32, "recurrent metadata must be int32");
  TORCH_CHECK(cu.dim() == 1 && idx.dim() == 1 && idx.numel() == x.size(0) && cu.numel() == idx.numel() + 1,
              "the fused form takes one-token sequences: cu_seqlens [rows+1], state_indices [rows]");
  TORCH_CHECK(std::isfinite(eps) && eps > 0, "eps must be finite and positive");
  const c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor launch_idx, status;
  if (ticket) {
    ticket->check_compatible(cu, idx, x.size(0), shift_state_pool.size(0), max_seqlen);
    TORCH_CHECK(ticket->max_seqlen() == 1, "the fused form takes one-token sequences");
    launch_idx = ticket->idx_snapshot();
    status = ticket->status();
  } else {
    auto prepared = launch_validation(cu, idx, x.size(0), shift_state_pool.size(0));
    launch_idx = std::move(prepared.idx);
    status = std::move(prepared.status);
  }
  auto sum = torch::empty_like(x);
  auto mixes = torch::empty({6, x.size(0), x.size(1)}, x.options());
  check_rc(frwkv_tmix_mix6_add_layer_norm_forward(
      x.data_ptr(), residual.data_ptr(), weight.data_ptr(), bias.data_ptr(), x_r.data_ptr(), x_w.data_ptr(),
      x_k.data_ptr(), x_v.data_ptr(), x_a.data_ptr(), x_g.data_ptr(), shift_state_pool.data_ptr(),
      launch_idx.data_ptr<int>(), status.data_ptr<int>(), sum.data_ptr(), mixes.data_ptr(), static_cast<int>(x.size(0)),
      static_cast<int>(x.size(1)), static_cast<float>(eps), io_dtype_of(x), current_stream(x)));
  std::vector<torch::Tensor> out{sum};
  for (auto& t : mixes.unbind(0)) out.push_back(t);
  return out;
}

// Token shift fused into up to eight projections (1..8 rows): outputs[j] = mix(x, prev, mixes[j]) @ weights[j]^T;
// the shift states are updated afterwards.
std::vector<torch::Tensor> tmix_shift_project_varlen(torch::Tensor x, torch::Tensor shift_state_pool,
                                                     std::vector<torch::Tensor> mixes,
                                                     std::vector<torch::Tensor> weights, torch::Tensor cu,
                                                     torch::Tensor idx, int64_t max_seqlen,
                                                     std::shared_ptr<MetadataTicket> ticket) {
  check_io16(x, "x", x);
  TORCH_CHECK(x.dim() == 2 && x.size(0) >= 1, "x must have packed shape [M,C]");
  TORCH_CHECK(x.size(1) % 8 == 0 && x.size(1) >= 256, "C must be a multiple of 8 and at least 256");
  TORCH_CHECK(!mixes.empty() && mixes.size() <= 8 && mixes.size() == weights.size(),
              "1..8 mix vectors and as many weights are required");
  check_io16(shift_state_pool, "shift_state_pool", x);
  TORCH_CHECK(shift_state_pool.dim() == 2 && shift_state_pool.size(1) == x.size(1),
              "shift_state_pool must have shape [slots,C]");
  check_cuda_contiguous(cu, "cu_seqlens");
  check_cuda_contiguous(idx, "state_indices");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && idx.scalar_type() == torch::kInt32, "recurrent metadata must be int32");
  TORCH_CHECK(cu.dim() == 1 && idx.dim() == 1 && idx.numel() > 0 && cu.numel() == idx.numel() + 1,
              "cu_seqlens must have shape [B+1] and state_indices shape [B]");
  TORCH_CHECK(idx.numel() <= x.size(0), "more sequences than rows");
  const c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor launch_cu, launch_idx, status;
  if (ticket) {
    ticket->check_compatible(cu, idx, x.size(0), shift_state_pool.size(0), max_seqlen);
    launch_cu = ticket->cu_snapshot();
    launch_idx = ticket->idx_snapshot();
    status = ticket->status();
  } else {
    auto prepared = launch_validation(cu, idx, x.size(0), shift_state_pool.size(0));
    launch_cu = std::move(prepared.cu);
    launch_idx = std::move(prepared.idx);
    status = std::move(prepared.status);
  }
  std::vector<torch::Tensor> outs;
  std::vector<frwkv_shift_projection> proj;
  for (size_t j = 0; j < mixes.size(); ++j) {
    check_io16(mixes[j], "mix", x);
    check_io16(weights[j], "weight", x);
    TORCH_CHECK(mixes[j].dim() == 1 && mixes[j].size(0) == x.size(1), "every mix vector must have shape [C]");
    TORCH_CHECK(weights[j].dim() == 2 && weights[j].size(1) == x.size(1) && weights[j].size(0) % 8 == 0,
                "every weight must have the original layout [N,C] with N a multiple of 8");
    outs.push_back(torch::empty({x.size(0), weights[j].size(0)}, x.options()));
    proj.push_back({mixes[j].data_ptr(), weights[j].data_ptr(), outs.back().data_ptr(),
                    static_cast<int>(weights[j].size(0))});
  }
  if (x.size(0) > 8) {  // many rows: the shift happens inside the tensor-core GEMM
    auto rows = torch::empty({x.size(0)}, x.options().dtype(torch::kInt32));
    check_rc(frwkv_tmix_shift_project_gemm(x.data_ptr(), shift_state_pool.data_ptr(), launch_cu.data_ptr<int>(),
                                           launch_idx.data_ptr<int>(), status.data_ptr<int>(), proj.data(),
                                           static_cast<int>(proj.size()), static_cast<int>(x.size(0)),
                                           static_cast<int>(idx.numel()), static_cast<int>(x.size(1)), io_dtype_of(x),
                                           rows.data_ptr<int>(), linear_flag(x).data_ptr<int>(), current_stream(x)));
    return outs;
  }
  check_rc(frwkv_tmix_shift_project_varlen(x.data_ptr(), shift_state_pool.data_ptr(), launch_cu.data_ptr<int>(),
                                           launch_idx.data_ptr<int>(), status.data_ptr<int>(), proj.data(),
                                           static_cast<int>(proj.size()), static_cast<int>(x.size(0)),
                                           static_cast<int>(idx.numel()), static_cast<int>(x.size(1)), io_dtype_of(x),
                                           current_stream(x)));
  return outs;
}

// One TMix layer of a decode batch in a single cooperative launch (csrc/tmix_decode_layer.cu).  Row m is sequence m.
//   mixes = x_r, x_w, x_k, x_v, x_a, x_g [C];  big = Wr, Wk, Wv, Wo [C,C];  w1 / w2 = decay, a, gate, value-residual
//   low-rank pairs ([R,C] / [C,R]);  vecs = k_k, a0, k_a, r_k, ln_w, ln_b, v0 [C].
// Returns (out [M,C], device words: four barrier counters and the error flag at index 7).
std::tuple<torch::Tensor, torch::Tensor> tmix_decode_layer(torch::Tensor x, torch::Tensor v_first,
                                                           torch::Tensor shift_state_pool, torch::Tensor state_pool,
                                                           std::vector<torch::Tensor> mixes,
                                                           std::vector<torch::Tensor> big, std::vector<torch::Tensor> w1,
                                                           std::vector<torch::Tensor> w2, std::vector<torch::Tensor> vecs,
                                                           torch::Tensor cu, torch::Tensor idx, double eps,
                                                           std::shared_ptr<MetadataTicket> ticket) {
  check_io16(x, "x", x);
  TORCH_CHECK(x.dim() == 2 && x.size(0) >= 1 && x.size(0) <= 8, "x must have packed shape [M,C] with 1 <= M <= 8");
  const int64_t M = x.size(0), C = x.size(1);
  TORCH_CHECK(C >= 256 && C % 64 == 0, "C must be a multiple of the head size 64, at least 256");
  check_io16(v_first, "v_first", x);
  TORCH_CHECK(v_first.sizes() == x.sizes(), "v_first must have x's shape");
  check_io16(shift_state_pool, "shift_state_pool", x);
  TORCH_CHECK(shift_state_pool.dim() == 2 && shift_state_pool.size(1) == C, "shift_state_pool must have shape [slots,C]");
  check_cuda_contiguous(state_pool, "state_pool");
  TORCH_CHECK(state_pool.scalar_type() == torch::kFloat32 && state_pool.device() == x.device() && state_pool.dim() == 4 &&
                  state_pool.size(1) * 64 == C && state_pool.size(2) == 64 && state_pool.size(3) == 64,
              "state_pool must be float32 [slots,C/64,64,64] on x's device");
  TORCH_CHECK(mixes.size() == 6 && big.size() == 4 && w1.size() == 4 && w2.size() == 4 && vecs.size() == 7,
              "expected 6 mix vectors, 4 square weights, 4 + 4 low-rank weights and 7 channel vectors");
  check_cuda_contiguous(cu, "cu_seqlens");
  check_cuda_contiguous(idx, "state_indices");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && idx.scalar_type() == torch::kInt32, "recurrent metadata must be int32");
  TORCH_CHECK(cu.dim() == 1 && idx.dim() == 1 && idx.numel() == M && cu.numel() == M + 1,
              "a decode batch has one token per sequence: cu_seqlens [M+1], state_indices [M]");
  const c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor launch_idx, status;
  if (ticket) {
    TORCH_CHECK(shift_state_pool.size(0) >= state_pool.size(0),
                "with a prepared ticket the shift-state pool needs at least as many slots as the state pool");
    ticket->check_compatible(cu, idx, M, state_pool.size(0), 1);
    launch_idx = ticket->idx_snapshot();
    status = ticket->status();
  } else {
    auto prepared = launch_validation(cu, idx, M, std::min(shift_state_pool.size(0), state_pool.size(0)));
    launch_idx = std::move(prepared.idx);
    status = std::move(prepared.status);
  }
  frwkv_tmix_decode_layer_args a{};
  a.x = x.data_ptr();
  a.v_first = v_first.data_ptr();
  a.shift_state_pool = shift_state_pool.data_ptr();
  a.state_pool = state_pool.data_ptr<float>();
  for (int i = 0; i < 6; ++i) {
    check_io16(mixes[i], "mix", x);
    TORCH_CHECK(mixes[i].dim() == 1 && mixes[i].size(0) == C, "every mix vector must have shape [C]");
    a.mix[i] = mixes[i].data_ptr();
  }
  for (int i = 0; i < 4; ++i) {
    check_io16(big[i], "weight", x);
    TORCH_CHECK(big[i].dim() == 2 && big[i].size(0) == C && big[i].size(1) == C, "Wr, Wk, Wv, Wo must have shape [C,C]");
    check_io16(w1[i], "rank-in weight", x);
    check_io16(w2[i], "rank-out weight", x);
    TORCH_CHECK(w1[i].dim() == 2 && w1[i].size(1) == C && w1[i].size(0) % 8 == 0 && w1[i].size(0) >= 8 && w1[i].size(0) <= C,
                "rank-in weights must have shape [R,C], R a multiple of 8");
    TORCH_CHECK(w2[i].dim() == 2 && w2[i].size(0) == C && w2[i].size(1) == w1[i].size(0),
                "rank-out weights must have shape [C,R]");
    a.w1[i] = w1[i].data_ptr();
    a.w2[i] = w2[i].data_ptr();
    a.rank[i] = static_cast<int>(w1[i].size(0));
  }
  a.w_r = big[0].data_ptr(); a.w_k = big[1].data_ptr(); a.w_v = big[2].data_ptr(); a.w_o = big[3].data_ptr();
  for (int i = 0; i < 7; ++i) {
    check_io16(vecs[i], "channel vector", x);
    TORCH_CHECK(vecs[i].dim() == 1 && vecs[i].size(0) == C, "k_k, a0, k_a, r_k, ln_w, ln_b, v0 must have shape [C]");
  }
  a.k_k = vecs[0].data_ptr(); a.a0 = vecs[1].data_ptr(); a.k_a = vecs[2].data_ptr(); a.r_k = vecs[3].data_ptr();
  a.ln_w = vecs[4].data_ptr(); a.ln_b = vecs[5].data_ptr(); a.v0 = vecs[6].data_ptr();
  auto out = torch::empty_like(x);
  a.out = out.data_ptr();
  auto workspace = torch::empty(
      {static_cast<int64_t>(frwkv_tmix_decode_layer_workspace_bytes(static_cast<int>(M), static_cast<int>(C), a.rank))},
      x.options().dtype(torch::kUInt8));
  a.workspace = workspace.data_ptr();
  // barrier counters and the error flag: one set per (device, stream), zeroed once; the kernel leaves the counters zero
  static std::mutex words_mutex;
  static std::map<std::pair<int, void*>, torch::Tensor> words_of;
  torch::Tensor words;
  {
    const std::lock_guard<std::mutex> lock(words_mutex);
    const auto key = std::make_pair(static_cast<int>(x.device().index()), static_cast<void*>(current_stream(x)));
    auto it = words_of.find(key);
    if (it == words_of.end()) it = words_of.emplace(key, torch::zeros({8}, x.options().dtype(torch::kInt32))).first;
    words = it->second;
  }
  a.barrier = reinterpret_cast<uint32_t*>(words.data_ptr<int>());
  check_rc(frwkv_tmix_decode_layer_forward(&a, launch_idx.data_ptr<int>(), status.data_ptr<int>(), static_cast<int>(M),
                                           static_cast<int>(C), static_cast<int>(C / 64), static_cast<float>(eps),
                                           io_dtype_of(x), words.data_ptr<int>() + 7, current_stream(x)));
  remember_flag("tmix_decode_layer", words);  // index 7 is the error word
  return {out, words};
}

void check_rows_channels(const torch::Tensor& t, const char* name, const torch::Tensor& ref) {
  check_io16(t, name, ref);
  TORCH_CHECK(t.dim() == 2 && t.sizes() == ref.sizes(), name, " must have packed shape [total_tokens,C]");
}
void check_channel_vector(const torch::Tensor& t, const char* name, const torch::Tensor& ref) {
  check_io16(t, name, ref);
  TORCH_CHECK(t.dim() == 1 && t.size(0) == ref.size(1), name, " must have shape [C]");
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> tmix_kk_a_gate_forward_varlen(
    torch::Tensor k, torch::Tensor k_k, torch::Tensor a0, torch::Tensor a12, torch::Tensor k_a, int64_t head_size,
    int64_t batch_size, int64_t max_seqlen) {
  check_io16(k, "k", k);
  TORCH_CHECK(k.dim() == 2 && k.size(0) > 0 && k.size(1) > 0, "k must have packed shape [total_tokens,C]");
  TORCH_CHECK(head_size == 64 || head_size == 128 || head_size == 256, "head_size must be 64, 128, or 256");
  TORCH_CHECK(k.size(1) % head_size == 0, "C must be divisible by head_size");
  TORCH_CHECK(batch_size > 0 && max_seqlen > 0, "batch_size and max_seqlen must be positive");
  check_rows_channels(a12, "a12", k);
  check_channel_vector(k_k, "k_k", k);
  check_channel_vector(a0, "a0", k);
  check_channel_vector(k_a, "k_a", k);
  const c10::cuda::CUDAGuard guard(k.device());
  auto new_k = torch::empty_like(k), neg_kk = torch::empty_like(k), kka = torch::empty_like(k);
  check_rc(frwkv_tmix_kk_a_gate_forward_varlen(k.data_ptr(), k_k.data_ptr(), a0.data_ptr(), a12.data_ptr(),
                                               k_a.data_ptr(), new_k.data_ptr(), neg_kk.data_ptr(), kka.data_ptr(),
                                               k.size(0), static_cast<int>(k.size(1)), static_cast<int>(head_size),
                                               io_dtype_of(k), current_stream(k)));
  return {new_k, neg_kk, kka};
}

torch::Tensor tmix_lnx_rkvres_xg_forward_varlen(torch::Tensor x, torch::Tensor r, torch::Tensor k, torch::Tensor v,
                                                torch::Tensor r_k, torch::Tensor weight, torch::Tensor bias,
                                                torch::Tensor g, int64_t head_size, int64_t batch_size,
                                                int64_t max_seqlen) {
  check_io16(x, "x", x);
  TORCH_CHECK(x.dim() == 2 && x.size(0) > 0 && x.size(1) > 0, "x must have packed shape [total_tokens,C]");
  TORCH_CHECK(head_size == 64 || head_size == 128 || head_size == 256, "head_size must be 64, 128, or 256");
  TORCH_CHECK(x.size(1) % head_size == 0, "C must be divisible by head_size");
  TORCH_CHECK(batch_size > 0 && max_seqlen > 0, "batch_size and max_seqlen must be positive");
  check_rows_channels(r, "r", x);
  check_rows_channels(k, "k", x);
  check_rows_channels(v, "v", x);
  check_rows_channels(g, "g", x);
  check_channel_vector(r_k, "r_k", x);
  check_channel_vector(weight, "weight", x);
  check_channel_vector(bias, "bias", x);
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  check_rc(frwkv_tmix_lnx_rkvres_xg_forward_varlen(x.data_ptr(), r.data_ptr(), k.data_ptr(), v.data_ptr(), r_k.data_ptr(),
                                                   weight.data_ptr(), bias.data_ptr(), g.data_ptr(), out.data_ptr(),
                                                   x.size(0), static_cast<int>(x.size(1)), static_cast<int>(head_size),
                                                   64.0e-5f, io_dtype_of(x), current_stream(x)));
  return out;
}

torch::Tensor tmix_vres_gate_forward_varlen(torch::Tensor v, torch::Tensor v_first, torch::Tensor v0, torch::Tensor v12) {
  check_io16(v, "v", v);
  TORCH_CHECK(v.dim() == 2 && v.size(0) > 0 && v.size(1) > 0 && v.size(1) % 8 == 0,
              "v must have packed shape [total_tokens,C] with C a multiple of 8");
  check_rows_channels(v_first, "v_first", v);
  check_rows_channels(v12, "v12", v);
  check_channel_vector(v0, "v0", v);
  const c10::cuda::CUDAGuard guard(v.device());
  auto out = torch::empty_like(v);
  check_rc(frwkv_tmix_vres_gate_forward_varlen(v.data_ptr(), v_first.data_ptr(), v0.data_ptr(), v12.data_ptr(),
                                               out.data_ptr(), v.size(0), static_cast<int>(v.size(1)), io_dtype_of(v),
                                               current_stream(v)));
  return out;
}

torch::Tensor recurrent_add_vec_forward_varlen(torch::Tensor x, torch::Tensor vec) {
  check_io16(x, "x", x);
  check_io16(vec, "vec", x);
  TORCH_CHECK(x.dim() == 2 && x.size(0) > 0 && x.size(1) > 0 && (x.size(1) % 2) == 0,
              "x must have packed shape [total_tokens,C] with even C");
  TORCH_CHECK(vec.dim() == 1 && vec.size(0) == x.size(1), "vec must have shape [C]");
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  check_rc(frwkv_recurrent_add_vec_forward(x.data_ptr(), vec.data_ptr(), out.data_ptr(), x.size(0),
                                           static_cast<int>(x.size(1)), io_dtype_of(x), current_stream(x)));
  return out;
}

torch::Tensor tmix_act_forward(torch::Tensor x, int64_t act) {
  check_io16(x, "x", x);
  TORCH_CHECK(x.numel() > 0 && x.numel() % 8 == 0, "x must have a positive element count that is a multiple of 8");
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  check_rc(frwkv_tmix_act_forward(x.data_ptr(), out.data_ptr(), x.numel(), static_cast<int>(act), io_dtype_of(x),
                                  current_stream(x)));
  return out;
}

// y_i = act_i(x_i) @ weight_i^T for up to four projections sharing the row count; weights in the original [N,K]
// layout.  `vres` = (v, v_first, v0) applies the value-residual epilogue to the LAST projection.
std::vector<torch::Tensor> tmix_linear_grouped(std::vector<torch::Tensor> xs, std::vector<torch::Tensor> weights,
                                               std::vector<int64_t> acts,
                                               std::optional<std::tuple<torch::Tensor, torch::Tensor, torch::Tensor>> vres) {
  const size_t count = xs.size();
  TORCH_CHECK(count >= 1 && count <= 4, "between one and four projections per call");
  TORCH_CHECK(weights.size() == count && acts.size() == count, "xs, weights and acts must have the same length");
  const torch::Tensor& x0 = xs[0];
  check_io16(x0, "x", x0);
  TORCH_CHECK(x0.dim() == 2 && x0.size(0) > 0, "x must have shape [M,K]");
  const int64_t M = x0.size(0);
  TORCH_CHECK(M <= std::numeric_limits<int>::max(), "row count must fit in int32");
  std::vector<frwkv_linear_problem> problems(count);
  std::vector<torch::Tensor> outs;
  const c10::cuda::CUDAGuard guard(x0.device());
  for (size_t i = 0; i < count; ++i) {
    check_io16(xs[i], "x", x0);
    check_io16(weights[i], "weight", x0);
    TORCH_CHECK(xs[i].dim() == 2 && xs[i].size(0) == M, "all inputs must have shape [M,K]");
    TORCH_CHECK(weights[i].dim() == 2 && weights[i].size(1) == xs[i].size(1), "weight must have shape [N,K] matching x");
    TORCH_CHECK(xs[i].size(1) % 8 == 0 && weights[i].size(0) % 8 == 0, "feature counts must be multiples of 8");
    TORCH_CHECK(acts[i] >= 0 && acts[i] <= 2, "act must be 0 (none), 1 (tanh) or 2 (sigmoid)");
    outs.push_back(torch::empty({M, weights[i].size(0)}, x0.options()));
    if (M > 8 && acts[i] != 0) {
      // many rows: the TMA-fed GEMM has no activation stage, and a pass over the [M,K] input (K = a low rank) costs far
      // less than the cp.async GEMM that has one (measured at M = 512: 58 -> 43 us for the four rank-out products)
      xs[i] = tmix_act_forward(xs[i], acts[i]);
      acts[i] = 0;
    }
    problems[i] = frwkv_linear_problem{xs[i].data_ptr(), weights[i].data_ptr(), outs[i].data_ptr(),
                                       static_cast<int>(weights[i].size(0)), static_cast<int>(xs[i].size(1)),
                                       static_cast<int>(acts[i]), 0, nullptr, nullptr, nullptr};
  }
  if (vres.has_value()) {
    const auto& [v, v_first, v0] = *vres;
    const torch::Tensor& y = outs[count - 1];
    check_io16(v, "v", x0);
    check_io16(v_first, "v_first", x0);
    check_io16(v0, "v0", x0);
    TORCH_CHECK(v.sizes() == y.sizes() && v_first.sizes() == y.sizes(), "v and v_first must have shape [M,N]");
    TORCH_CHECK(v0.dim() == 1 && v0.size(0) == y.size(1), "v0 must have shape [N]");
    problems[count - 1].epilogue = 1;
    problems[count - 1].v = v.data_ptr();
    problems[count - 1].v_first = v_first.data_ptr();
    problems[count - 1].v0 = v0.data_ptr();
  }
  check_rc(frwkv_tmix_linear_grouped(problems.data(), static_cast<int>(count), static_cast<int>(M), io_dtype_of(x0),
                                     linear_flag(x0).data_ptr<int>(), current_stream(x0)));
  return outs;
}

// ---- the reference's native projection names (csrc/sm120/tmix/linear/infer_fp16_forward_varlen.cpp:399-472 there) ----
// Every one is `act(x) @ W` with W given in the original layout [N,K] (`weight`, `*_t`) and / or the runtime layout
// [K,N] (`weight_is_transposed`, the un-suffixed low-rank arguments).  The original layout is used when it is
// given; a weight given only in the runtime layout is read in place (frwkv_tmix_linear_runtime_layout).
using OptTensor = std::optional<torch::Tensor>;
using Vres = std::optional<std::tuple<torch::Tensor, torch::Tensor, torch::Tensor>>;

torch::Tensor linear_runtime_layout(torch::Tensor x, const torch::Tensor& w_kn, int64_t act, const Vres& vres) {
  check_io16(x, "x", x);
  check_io16(w_kn, "weight", x);
  TORCH_CHECK(x.dim() == 2 && x.size(0) > 0 && w_kn.dim() == 2 && w_kn.size(0) == x.size(1),
              "runtime-layout weight must have shape [K,N] matching x [M,K]");
  TORCH_CHECK(x.size(1) % 8 == 0 && w_kn.size(1) % 8 == 0, "feature counts must be multiples of 8");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t M = x.size(0);
  if (M > 8 && act != 0) {  // the many-row kernel for this layout has no activation stage
    x = tmix_act_forward(x, act);
    act = 0;
  }
  auto y = torch::empty({M, w_kn.size(1)}, x.options());
  frwkv_linear_problem p{x.data_ptr(), w_kn.data_ptr(), y.data_ptr(), static_cast<int>(w_kn.size(1)),
                         static_cast<int>(x.size(1)), static_cast<int>(act), 0, nullptr, nullptr, nullptr};
  if (vres.has_value()) {
    const auto& [v, v_first, v0] = *vres;
    check_io16(v, "v", x);
    check_io16(v_first, "v_first", x);
    check_io16(v0, "v0", x);
    TORCH_CHECK(v.sizes() == y.sizes() && v_first.sizes() == y.sizes(), "v and v_first must have shape [M,N]");
    TORCH_CHECK(v0.dim() == 1 && v0.size(0) == y.size(1), "v0 must have shape [N]");
    p.epilogue = 1;
    p.v = v.data_ptr();
    p.v_first = v_first.data_ptr();
    p.v0 = v0.data_ptr();
  }
  check_rc(frwkv_tmix_linear_runtime_layout(&p, static_cast<int>(M), io_dtype_of(x), linear_flag(x).data_ptr<int>(),
                                            current_stream(x)));
  return y;
}

// a group of projections, each with its weight in either layout: one launch when all are original-layout
std::vector<torch::Tensor> linear_any_group(std::vector<torch::Tensor> xs, const std::vector<OptTensor>& originals,
                                            const std::vector<OptTensor>& runtimes, std::vector<int64_t> acts,
                                            const Vres& vres) {
  bool all_original = true;
  for (size_t i = 0; i < xs.size(); ++i) {
    TORCH_CHECK(originals[i].has_value() || runtimes[i].has_value(), "one of weight or weight_t must be provided");
    all_original = all_original && originals[i].has_value();
  }
  if (all_original) {
    std::vector<torch::Tensor> ws;
    for (const auto& w : originals) ws.push_back(*w);
    return tmix_linear_grouped(std::move(xs), std::move(ws), std::move(acts), vres);
  }
  std::vector<torch::Tensor> outs;
  for (size_t i = 0; i < xs.size(); ++i) {
    const Vres one = (vres.has_value() && i + 1 == xs.size()) ? vres : Vres();
    if (originals[i].has_value()) outs.push_back(tmix_linear_grouped({xs[i]}, {*originals[i]}, {acts[i]}, one)[0]);
    else outs.push_back(linear_runtime_layout(xs[i], *runtimes[i], acts[i], one));
  }
  return outs;
}

torch::Tensor ref_linear_forward(torch::Tensor x, torch::Tensor weight, bool weight_is_transposed) {
  if (weight_is_transposed) return linear_runtime_layout(x, weight, 0, Vres());
  return tmix_linear_grouped({x}, {weight}, {0}, Vres())[0];
}
torch::Tensor ref_linear_c2c(torch::Tensor x, torch::Tensor weight) { return ref_linear_forward(x, weight, false); }
torch::Tensor ref_linear_t(torch::Tensor x, torch::Tensor weight_t) {
  TORCH_CHECK(x.dim() == 2 && x.size(0) <= 65535, "TMix linear_t supports at most 65535 packed rows");
  return tmix_linear_grouped({x}, {weight_t}, {0}, Vres())[0];
}
torch::Tensor ref_linear_t_tanh(torch::Tensor x, torch::Tensor weight_t) {
  TORCH_CHECK(x.dim() == 2 && x.size(0) <= 65535, "TMix linear_t supports at most 65535 packed rows");
  return tmix_linear_grouped({x}, {weight_t}, {1}, Vres())[0];
}
torch::Tensor ref_linear_t_sigmoid(torch::Tensor x, torch::Tensor weight_t) {
  TORCH_CHECK(x.dim() == 2 && x.size(0) <= 65535, "TMix linear_t supports at most 65535 packed rows");
  return tmix_linear_grouped({x}, {weight_t}, {2}, Vres())[0];
}
torch::Tensor ref_act_tanh(torch::Tensor x) { return tmix_act_forward(x, 1); }
torch::Tensor ref_act_sigmoid(torch::Tensor x) { return tmix_act_forward(x, 2); }
torch::Tensor ref_linear_t_vres(torch::Tensor x, torch::Tensor weight_t, torch::Tensor v, torch::Tensor v_first,
                                torch::Tensor v0) {
  TORCH_CHECK(x.dim() == 2 && x.size(0) <= 65535, "TMix linear_t supports at most 65535 packed rows");
  return tmix_linear_grouped({x}, {weight_t}, {0}, std::make_tuple(v, v_first, v0))[0];
}
void check_rank(const torch::Tensor& x, const OptTensor& weight, const OptTensor& weight_t, bool input_projection) {
  TORCH_CHECK(weight.has_value() || weight_t.has_value(), "one of weight or weight_t must be provided");
  const int64_t rank = weight.has_value() ? (input_projection ? weight->size(1) : weight->size(0))
                                          : (input_projection ? weight_t->size(0) : weight_t->size(1));
  TORCH_CHECK(rank <= 512, "low-rank projection requires R<=512");
  (void)x;
}
torch::Tensor ref_rank_dispatch(torch::Tensor x, OptTensor weight, OptTensor weight_t) {
  return linear_any_group({x}, {weight_t}, {weight}, {0}, Vres())[0];
}
std::vector<torch::Tensor> ref_lowrank_in(torch::Tensor x_w, torch::Tensor x_a, torch::Tensor x_g, OptTensor w1_t,
                                          OptTensor a1_t, OptTensor g1_t, OptTensor w1, OptTensor a1, OptTensor g1) {
  check_rank(x_w, w1, w1_t, true); check_rank(x_a, a1, a1_t, true); check_rank(x_g, g1, g1_t, true);
  return linear_any_group({x_w, x_a, x_g}, {w1_t, a1_t, g1_t}, {w1, a1, g1}, {0, 0, 0}, Vres());
}
std::vector<torch::Tensor> ref_lowrank_wagv_in(torch::Tensor x_w, torch::Tensor x_a, torch::Tensor x_g, torch::Tensor x_v,
                                               OptTensor w1_t, OptTensor a1_t, OptTensor g1_t, OptTensor v1_t,
                                               OptTensor w1, OptTensor a1, OptTensor g1, OptTensor v1) {
  check_rank(x_w, w1, w1_t, true); check_rank(x_a, a1, a1_t, true); check_rank(x_g, g1, g1_t, true);
  check_rank(x_v, v1, v1_t, true);
  return linear_any_group({x_w, x_a, x_g, x_v}, {w1_t, a1_t, g1_t, v1_t}, {w1, a1, g1, v1}, {0, 0, 0, 0}, Vres());
}
std::vector<torch::Tensor> ref_lowrank_out(torch::Tensor w1, torch::Tensor a1, torch::Tensor g1, OptTensor w2_t,
                                           OptTensor a2_t, OptTensor g2_t, OptTensor w2, OptTensor a2, OptTensor g2) {
  check_rank(w1, w2, w2_t, false); check_rank(a1, a2, a2_t, false); check_rank(g1, g2, g2_t, false);
  return linear_any_group({w1, a1, g1}, {w2_t, a2_t, g2_t}, {w2, a2, g2}, {1, 0, 2}, Vres());
}
std::vector<torch::Tensor> ref_lowrank_vres(torch::Tensor w1, torch::Tensor a1, torch::Tensor g1, torch::Tensor v1,
                                            OptTensor w2_t, OptTensor a2_t, OptTensor g2_t, OptTensor v2_t, OptTensor w2,
                                            OptTensor a2, OptTensor g2, OptTensor v2, torch::Tensor v,
                                            torch::Tensor v_first, torch::Tensor v0) {
  check_rank(w1, w2, w2_t, false); check_rank(a1, a2, a2_t, false); check_rank(g1, g2, g2_t, false);
  check_rank(v1, v2, v2_t, false);
  return linear_any_group({w1, a1, g1, v1}, {w2_t, a2_t, g2_t, v2_t}, {w2, a2, g2, v2}, {1, 0, 2, 0},
                          std::make_tuple(v, v_first, v0));
}

// ---- training side -------------------------------------------------------------------------------------
// state_dot_a [N,H,D] and the 16-token checkpoints [Cn,3,H,D,D] for the backward pass, from the chunk boundaries
std::tuple<torch::Tensor, torch::Tensor> wkv7_chunk_replay(torch::Tensor cs, torch::Tensor ce, torch::Tensor boundary,
                                                          torch::Tensor r, torch::Tensor w, torch::Tensor k,
                                                          torch::Tensor v, torch::Tensor a, torch::Tensor b,
                                                          std::optional<torch::Tensor> decay_bias) {
  check_cuda_contiguous(boundary, "boundary");
  TORCH_CHECK(boundary.scalar_type() == torch::kFloat32 && boundary.dim() == 4 && boundary.size(0) == cs.numel() &&
                  boundary.size(1) == r.size(1) && boundary.size(2) == 64 && boundary.size(3) == 64,
              "boundary must be float32 [Cn,H,64,64]");
  TORCH_CHECK(r.dim() == 3 && r.size(2) == 64, "token tensors must have shape [N,H,64]");
  const c10::cuda::CUDAGuard guard(r.device());
  auto sda = torch::empty(r.sizes(), r.options().dtype(torch::kFloat32));
  auto ckpt = torch::empty({cs.numel(), 3, r.size(1), 64, 64}, r.options().dtype(torch::kFloat32));
  check_rc(frwkv_wkv7_chunk_replay(cs.data_ptr<int>(), ce.data_ptr<int>(), boundary.data_ptr<float>(), r.data_ptr(),
                                   w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
                                   decay_bias.has_value() ? decay_bias->data_ptr() : nullptr, sda.data_ptr<float>(),
                                   ckpt.data_ptr<float>(), static_cast<int>(cs.numel()), static_cast<int>(r.size(1)), 64,
                                   io_dtype_of(r), current_stream(r)));
  return {sda, ckpt};
}

std::vector<torch::Tensor> wkv7_backward(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce,
                                         torch::Tensor final_state, torch::Tensor boundary, torch::Tensor checkpoints,
                                         torch::Tensor state_dot_a, torch::Tensor r, torch::Tensor w, torch::Tensor k,
                                         torch::Tensor v, torch::Tensor a, torch::Tensor b,
                                         std::optional<torch::Tensor> grad_output,
                                         std::optional<torch::Tensor> grad_final_state, double scale) {
  check_chunk_tables(sco, cs, ce, r);
  for (const torch::Tensor* t : {&final_state, &boundary, &checkpoints, &state_dot_a}) {
    check_cuda_contiguous(*t, "saved tensor");
    TORCH_CHECK(t->scalar_type() == torch::kFloat32 && t->device() == r.device(), "saved tensors must be float32 on r's device");
  }
  TORCH_CHECK(r.dim() == 3 && r.size(2) == 64, "token tensors must have shape [N,H,64]");
  const int64_t B = sco.numel() - 1, H = r.size(1);
  TORCH_CHECK(final_state.dim() == 4 && final_state.size(0) == B && final_state.size(1) == H,
              "final_state must have shape [B,H,64,64]");
  TORCH_CHECK(state_dot_a.sizes() == r.sizes(), "state_dot_a must be shaped like r");
  if (grad_output.has_value()) {
    check_cuda_contiguous(*grad_output, "grad_output");
    TORCH_CHECK(grad_output->sizes() == r.sizes() && grad_output->scalar_type() == r.scalar_type(),
                "grad_output must match r");
  }
  if (grad_final_state.has_value()) {
    check_cuda_contiguous(*grad_final_state, "grad_final_state");
    TORCH_CHECK(grad_final_state->sizes() == final_state.sizes() && grad_final_state->scalar_type() == torch::kFloat32,
                "grad_final_state must be float32 [B,H,64,64]");
  }
  const c10::cuda::CUDAGuard guard(r.device());
  std::vector<torch::Tensor> g;
  for (int i = 0; i < 6; ++i) g.push_back(torch::empty_like(r));
  g.push_back(torch::empty_like(final_state));
  check_rc(frwkv_wkv7_backward(
      sco.data_ptr<int>(), cs.data_ptr<int>(), ce.data_ptr<int>(), final_state.data_ptr<float>(),
      boundary.data_ptr<float>(), checkpoints.data_ptr<float>(), state_dot_a.data_ptr<float>(), r.data_ptr(),
      w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
      grad_output.has_value() ? grad_output->data_ptr() : nullptr,
      grad_final_state.has_value() ? grad_final_state->data_ptr<float>() : nullptr, g[0].data_ptr(), g[1].data_ptr(),
      g[2].data_ptr(), g[3].data_ptr(), g[4].data_ptr(), g[5].data_ptr(), g[6].data_ptr<float>(), static_cast<int>(B),
      static_cast<int>(H), 64, io_dtype_of(r), static_cast<float>(scale), current_stream(r)));
  return g;
}


// ---- reference-named entries of the chunk / training families ------------------------------------------------
// Same names, argument order and defaults as the reference's native module, so that its Python layer binds to this
// module unchanged.  Each is a thin arrangement of the operators above.

// csrc/sm120/tmix/wkv7/infer_chunk_bf16_forward_varlen.cpp:77-183 of the reference: bf16 state pool updated in
// place at state_indices, returns (output, state_pool).  chunk_size only has to be positive: the tensor-core
// kernels always work on 64-token tiles and the result does not depend on the split.
std::tuple<torch::Tensor, torch::Tensor> infer_chunk_bf16_forward_varlen_native(
    torch::Tensor r, torch::Tensor w, torch::Tensor k, torch::Tensor v, torch::Tensor a, torch::Tensor b,
    torch::Tensor state_pool, torch::Tensor cu, torch::Tensor idx, int64_t chunk_size, int64_t max_seqlen, double scale,
    std::optional<torch::Tensor> decay_bias) {
  TORCH_CHECK(chunk_size > 0, "chunk_size must be positive");
  check_cuda_contiguous(state_pool, "state_pool");
  TORCH_CHECK(state_pool.scalar_type() == torch::kBFloat16 && state_pool.dim() == 4 && r.dim() == 3 &&
                  state_pool.size(1) == r.size(1) && state_pool.size(2) == 64 && state_pool.size(3) == 64,
              "state_pool must be bfloat16 [slots,H,64,64]");
  TORCH_CHECK(r.scalar_type() == torch::kBFloat16, "token tensors must be bfloat16");
  check_cuda_contiguous(cu, "cu_seqlens");
  check_cuda_contiguous(idx, "state_indices");
  TORCH_CHECK(cu.scalar_type() == torch::kInt32 && idx.scalar_type() == torch::kInt32 && cu.dim() == 1 &&
                  idx.dim() == 1 && cu.numel() == idx.numel() + 1 && idx.numel() > 0,
              "cu_seqlens must be int32 [B+1] and state_indices int32 [B]");
  const c10::cuda::CUDAGuard guard(r.device());
  auto prepared = launch_validation(cu, idx, r.size(0), state_pool.size(0));
  // chunk tables from the sequence offsets (one host read, as the reference does for max_seqlen)
  auto cu_host = cu.cpu();
  const int* offs = cu_host.data_ptr<int>();
  std::vector<int> sco{0}, cs, ce;
  for (int64_t sq = 0; sq + 1 < cu_host.numel(); ++sq) {
    TORCH_CHECK(offs[sq + 1] > offs[sq] && offs[sq] >= 0 && offs[sq + 1] <= r.size(0),
                "cu_seqlens must be strictly increasing within [0, total_tokens]");
    for (int t = offs[sq]; t < offs[sq + 1]; t += 64) {
      cs.push_back(t);
      ce.push_back(std::min(t + 64, offs[sq + 1]));
    }
    sco.push_back(static_cast<int>(cs.size()));
  }
  auto to_dev = [&](const std::vector<int>& x) {
    return torch::tensor(x, torch::TensorOptions().dtype(torch::kInt32)).to(r.device());
  };
  auto slots = prepared.idx.to(torch::kInt64);
  auto working = state_pool.index_select(0, slots).to(torch::kFloat32);
  auto output = torch::empty_like(v);
  wkv7_chunk_forward(to_dev(sco), to_dev(cs), to_dev(ce), working, r, w, k, v, a, b, output, scale, decay_bias,
                     std::nullopt, std::nullopt, std::nullopt, prepared.status, std::nullopt, -1);
  // a batch that failed validation produced NaN outputs and left `working` as it was: copying it back is harmless
  state_pool.index_copy_(0, slots, working.to(torch::kBFloat16));
  (void)max_seqlen;
  return {output, state_pool};
}

// csrc/sm90/rl_infctx/wkv7/rl_infctx_chunk_fp32io16_backward.cpp:102-135 of the reference: recompute `output` and
// `state_dot_a` of every chunk from its boundary state.  Each chunk is run as a sequence of its own by the fused
// kernel on a copy of the boundaries (the kernel updates its state in place).
void rl_infctx_chunk_fp32io16_backward_replay(torch::Tensor cs, torch::Tensor ce, torch::Tensor boundary, torch::Tensor r,
                                              torch::Tensor w, torch::Tensor k, torch::Tensor v, torch::Tensor a,
                                              torch::Tensor b, torch::Tensor output, torch::Tensor state_dot_a,
                                              double scale, std::optional<torch::Tensor> decay_bias) {
  check_cuda_contiguous(boundary, "boundary");
  check_cuda_contiguous(cs, "chunk_token_starts");
  TORCH_CHECK(r.dim() == 3, "token tensors must have shape [N,H,D]");
  TORCH_CHECK(r.size(2) == 64, "this build replays head size 64 only, got ", r.size(2));
  TORCH_CHECK(boundary.scalar_type() == torch::kFloat32 && boundary.dim() == 4 && boundary.size(0) == cs.numel() &&
                  boundary.size(1) == r.size(1) && boundary.size(2) == 64 && boundary.size(3) == 64,
              "boundary must be float32 [Cn,H,D,D]");
  const c10::cuda::CUDAGuard guard(r.device());
  auto sco = torch::arange(cs.numel() + 1, cs.options());
  auto pool = boundary.clone();
  wkv7_chunk_forward(sco, cs, ce, pool, r, w, k, v, a, b, output, scale, decay_bias, std::nullopt, std::nullopt,
                     std::nullopt, std::nullopt, state_dot_a, 1);
}

// ---- head sizes 128 / 256: the plain-recurrence training kernels (csrc/wkv7_train_wide.cu) -------------------------
void check_wide_tokens(const torch::Tensor& r, const std::vector<const torch::Tensor*>& others) {
  check_cuda_contiguous(r, "r");
  TORCH_CHECK(r.dim() == 3 && (r.size(2) == 128 || r.size(2) == 256), "token tensors must have shape [N,H,128] or [N,H,256]");
  TORCH_CHECK(r.scalar_type() == torch::kBFloat16 || r.scalar_type() == torch::kFloat16,
              "token tensors must be float16 or bfloat16");
  for (const torch::Tensor* t : others) {
    check_cuda_contiguous(*t, "token tensor");
    TORCH_CHECK(t->scalar_type() == r.scalar_type() && t->device() == r.device() && t->numel() == r.numel(),
                "token tensors must match r in dtype, device and size");
  }
}

void wkv7_train_wide_forward(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce, torch::Tensor state, torch::Tensor r,
                             torch::Tensor w, torch::Tensor k, torch::Tensor v, torch::Tensor a, torch::Tensor b,
                             torch::Tensor output, std::optional<torch::Tensor> boundary,
                             std::optional<torch::Tensor> state_dot_a, double scale,
                             std::optional<torch::Tensor> dense_checkpoints) {
  check_chunk_tables(sco, cs, ce, r);
  check_wide_tokens(r, {&w, &k, &v, &a, &b, &output});
  const int64_t B = sco.numel() - 1, H = r.size(1), D = r.size(2), Cn = cs.numel();
  check_cuda_contiguous(state, "state");
  TORCH_CHECK(state.scalar_type() == torch::kFloat32 && state.device() == r.device() && state.numel() == B * H * D * D,
              "state must be float32 [B,H,D,D] on the token device");
  float* bnd = nullptr;
  float* sda = nullptr;
  float* dense = nullptr;
  int dense_groups = 0;
  if (boundary.has_value()) {
    check_cuda_contiguous(*boundary, "boundary");
    TORCH_CHECK(boundary->scalar_type() == torch::kFloat32 && boundary->numel() == Cn * H * D * D, "boundary must be float32 [Cn,H,D,D]");
    bnd = boundary->data_ptr<float>();
  }
  if (state_dot_a.has_value()) {
    check_cuda_contiguous(*state_dot_a, "state_dot_a");
    TORCH_CHECK(state_dot_a->scalar_type() == torch::kFloat32 && state_dot_a->numel() == r.numel(), "state_dot_a must be float32 [N,H,D]");
    sda = state_dot_a->data_ptr<float>();
  }
  if (dense_checkpoints.has_value()) {
    check_cuda_contiguous(*dense_checkpoints, "dense_checkpoints");
    TORCH_CHECK(dense_checkpoints->scalar_type() == torch::kFloat32 && dense_checkpoints->dim() == 5 &&
                    dense_checkpoints->size(0) == B && dense_checkpoints->size(1) == H,
                "dense_checkpoints must be float32 [B,H,T/16,D,D]");
    dense = dense_checkpoints->data_ptr<float>();
    dense_groups = static_cast<int>(dense_checkpoints->size(2));
  }
  const c10::cuda::CUDAGuard guard(r.device());
  // caller-built tables: verdict on the device; on a bad table the kernels do nothing and the output reads as NaN
  auto status = chunk_table_status(sco, cs, ce, r);
  check_rc(frwkv_wkv7_train_wide_forward(sco.data_ptr<int>(), cs.data_ptr<int>(), ce.data_ptr<int>(),
                                         state.data_ptr<float>(), r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(),
                                         a.data_ptr(), b.data_ptr(), output.data_ptr(), bnd, sda, dense, dense_groups,
                                         status.data_ptr<int>(), static_cast<int>(B), static_cast<int>(H),
                                         static_cast<int>(D), io_dtype_of(r), static_cast<float>(scale), current_stream(r)));
  output.masked_fill_(status.ne(0), std::numeric_limits<double>::quiet_NaN());
}

// returns (grad_r, grad_decay_logits, grad_k, grad_v, grad_a, grad_b, grad_initial_state)
std::vector<torch::Tensor> wkv7_train_wide_backward(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce,
                                                    torch::Tensor final_state, torch::Tensor boundary,
                                                    torch::Tensor state_dot_a, torch::Tensor r, torch::Tensor w,
                                                    torch::Tensor k, torch::Tensor v, torch::Tensor a, torch::Tensor b,
                                                    std::optional<torch::Tensor> grad_output,
                                                    std::optional<torch::Tensor> grad_final_state, double scale,
                                                    std::vector<torch::Tensor> into) {
  check_chunk_tables(sco, cs, ce, r);
  check_wide_tokens(r, {&w, &k, &v, &a, &b});
  const int64_t B = sco.numel() - 1, N = r.size(0), H = r.size(1), D = r.size(2), Cn = cs.numel();
  for (const torch::Tensor* t : {&final_state, &boundary, &state_dot_a}) {
    check_cuda_contiguous(*t, "saved tensor");
    TORCH_CHECK(t->scalar_type() == torch::kFloat32 && t->device() == r.device(), "saved tensors must be float32 on r's device");
  }
  TORCH_CHECK(final_state.numel() == B * H * D * D, "final_state must have shape [B,H,D,D]");
  TORCH_CHECK(boundary.numel() == Cn * H * D * D, "boundary must have shape [Cn,H,D,D]");
  TORCH_CHECK(state_dot_a.numel() == r.numel(), "state_dot_a must be shaped like r");
  const c10::cuda::CUDAGuard guard(r.device());
  const void* go = nullptr;
  torch::Tensor go_t, gf_t;
  if (grad_output.has_value()) {
    go_t = grad_output->contiguous();
    TORCH_CHECK(go_t.numel() == r.numel() && go_t.scalar_type() == r.scalar_type(), "grad_output must match r");
    go = go_t.data_ptr();
  }
  const float* gf = nullptr;
  if (grad_final_state.has_value()) {
    gf_t = grad_final_state->contiguous().to(torch::kFloat32);
    TORCH_CHECK(gf_t.numel() == final_state.numel(), "grad_final_state must match final_state");
    gf = gf_t.data_ptr<float>();
  }
  std::vector<torch::Tensor> g = std::move(into);
  if (g.empty())
    for (int i = 0; i < 6; ++i) g.push_back(torch::empty_like(r));
  TORCH_CHECK(g.size() == 6, "six gradient tensors are expected");
  for (const auto& t : g) {
    check_cuda_contiguous(t, "gradient tensor");
    TORCH_CHECK(t.numel() == r.numel() && t.scalar_type() == r.scalar_type(), "gradient tensors must match r");
  }
  auto dS0 = torch::empty_like(final_state);
  auto status = chunk_table_status(sco, cs, ce, r);
  const size_t floats = frwkv_wkv7_train_wide_workspace_floats(N, static_cast<int>(Cn), static_cast<int>(H), static_cast<int>(D));
  auto workspace = torch::empty({static_cast<int64_t>(floats)}, final_state.options());
  check_rc(frwkv_wkv7_train_wide_backward(
      sco.data_ptr<int>(), cs.data_ptr<int>(), ce.data_ptr<int>(), final_state.data_ptr<float>(),
      boundary.data_ptr<float>(), state_dot_a.data_ptr<float>(), r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(),
      a.data_ptr(), b.data_ptr(), go, gf, g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), g[3].data_ptr(),
      g[4].data_ptr(), g[5].data_ptr(), dS0.data_ptr<float>(), workspace.data_ptr<float>(), status.data_ptr<int>(), N,
      static_cast<int>(B), static_cast<int>(Cn), static_cast<int>(H), static_cast<int>(D), io_dtype_of(r),
      static_cast<float>(scale), current_stream(r)));
  const auto bad = status.ne(0);
  for (auto& t : g) t.masked_fill_(bad, std::numeric_limits<double>::quiet_NaN());
  dS0.masked_fill_(bad, std::numeric_limits<double>::quiet_NaN());
  g.push_back(dS0);
  return g;
}

// csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_forward.cpp:26-56 of the reference: `state` [B,H,D,D] is updated
// in place to the final state; output, boundary and state_dot_a are filled.
void statetune_recurrent_fp32io16_forward(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce, torch::Tensor state,
                                          torch::Tensor r, torch::Tensor w, torch::Tensor k, torch::Tensor v,
                                          torch::Tensor a, torch::Tensor b, torch::Tensor output, torch::Tensor boundary,
                                          torch::Tensor state_dot_a, double scale) {
  TORCH_CHECK(r.dim() == 3, "token tensors must have shape [N,H,D]");
  if (r.size(2) != 64) {  // head sizes 128 / 256: the plain-recurrence kernels
    wkv7_train_wide_forward(sco, cs, ce, state, r, w, k, v, a, b, output, boundary, state_dot_a, scale, std::nullopt);
    return;
  }
  // this entry is reached with caller-built tables (the reference's wrapper checks shapes only): verdict on the device
  wkv7_chunk_forward(sco, cs, ce, state, r, w, k, v, a, b, output, scale, std::nullopt, std::nullopt, boundary,
                     std::nullopt, chunk_table_status(sco, cs, ce, r), state_dot_a, 1);
}

std::vector<torch::Tensor> wkv7_backward_chunked(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce,
                                                 torch::Tensor final_state, torch::Tensor boundary,
                                                 torch::Tensor state_dot_a, torch::Tensor r, torch::Tensor w,
                                                 torch::Tensor k, torch::Tensor v, torch::Tensor a, torch::Tensor b,
                                                 std::optional<torch::Tensor> grad_output,
                                                 std::optional<torch::Tensor> grad_final_state, double scale,
                                                 std::vector<torch::Tensor> into = {});

// csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cpp:34-82 of the reference: gradients are written into
// the tensors the caller passes (None = not wanted).
void statetune_recurrent_fp32io16_backward(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce,
                                           torch::Tensor final_state, torch::Tensor r, torch::Tensor w, torch::Tensor k,
                                           torch::Tensor v, torch::Tensor a, torch::Tensor b, torch::Tensor state_dot_a,
                                           std::optional<torch::Tensor> grad_output,
                                           std::optional<torch::Tensor> grad_final_state, torch::Tensor boundary,
                                           std::optional<torch::Tensor> grad_r, std::optional<torch::Tensor> grad_w,
                                           std::optional<torch::Tensor> grad_k, std::optional<torch::Tensor> grad_v,
                                           std::optional<torch::Tensor> grad_a, std::optional<torch::Tensor> grad_b,
                                           std::optional<torch::Tensor> grad_initial_state, double scale) {
  TORCH_CHECK(r.dim() == 3, "token tensors must have shape [N,H,D]");
  std::optional<torch::Tensor> go, gf;
  if (grad_output.has_value()) go = grad_output->contiguous();
  if (grad_final_state.has_value()) gf = grad_final_state->contiguous().to(torch::kFloat32);
  auto g = r.size(2) == 64
               ? wkv7_backward_chunked(sco, cs, ce, final_state, boundary, state_dot_a, r, w, k, v, a, b, go, gf, scale)
               : wkv7_train_wide_backward(sco, cs, ce, final_state, boundary, state_dot_a, r, w, k, v, a, b, go, gf,
                                          scale, {});
  const std::optional<torch::Tensor>* outs[7] = {&grad_r, &grad_w, &grad_k, &grad_v, &grad_a, &grad_b,
                                                 &grad_initial_state};
  for (int i = 0; i < 7; ++i)
    if (outs[i]->has_value()) (*outs[i])->copy_(g[i]);
}

// Adjoint of the state at every chunk boundary and the gradient of the initial state (first stage of the chunked
// backward).  Returns (grad_initial_state [B,H,64,64], boundary_adjoint [Cn,H,64,64], error flag).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> wkv7_adjoint_scan(
    torch::Tensor sco, torch::Tensor cs, torch::Tensor ce, torch::Tensor r, torch::Tensor w, torch::Tensor a,
    torch::Tensor b, torch::Tensor grad_output, std::optional<torch::Tensor> grad_final_state, double scale,
    std::optional<torch::Tensor> decay_bias, std::optional<torch::Tensor> table_status) {
  check_chunk_tables(sco, cs, ce, r);
  TORCH_CHECK(r.dim() == 3 && r.size(2) == 64, "token tensors must have shape [N,H,64]");
  check_cuda_contiguous(grad_output, "grad_output");
  TORCH_CHECK(grad_output.sizes() == r.sizes() && grad_output.scalar_type() == r.scalar_type(),
              "grad_output must match r");
  const int64_t B = sco.numel() - 1, H = r.size(1), Cn = cs.numel();
  const c10::cuda::CUDAGuard guard(r.device());
  auto f32 = r.options().dtype(torch::kFloat32);
  torch::Tensor g_state = grad_final_state.has_value() ? grad_final_state->to(torch::kFloat32).contiguous().clone()
                                                       : torch::zeros({B, H, 64, 64}, f32);
  TORCH_CHECK(g_state.dim() == 4 && g_state.size(0) == B && g_state.size(1) == H, "grad_final_state must be [B,H,64,64]");
  auto boundary_adjoint = torch::empty({Cn, H, 64, 64}, f32);
  auto error_flag = torch::zeros({1}, r.options().dtype(torch::kInt32));
  remember_flag("wkv7_chunk_backward", error_flag);  // the scan and the token-gradient kernel share the word
  check_rc(frwkv_wkv7_adjoint_scan(sco.data_ptr<int>(), cs.data_ptr<int>(), ce.data_ptr<int>(), r.data_ptr(), w.data_ptr(),
                                   a.data_ptr(), b.data_ptr(), decay_bias.has_value() ? decay_bias->data_ptr() : nullptr,
                                   grad_output.data_ptr(), g_state.data_ptr<float>(), boundary_adjoint.data_ptr<float>(),
                                   error_flag.data_ptr<int>(),
                                   table_status.has_value() ? table_status->data_ptr<int>() : nullptr,
                                   static_cast<int>(r.size(0)), static_cast<int>(B), static_cast<int>(Cn),
                                   static_cast<int>(H), 64, io_dtype_of(r), static_cast<float>(scale), current_stream(r)));
  return {g_state, boundary_adjoint, error_flag};
}

// The chunked backward on the tensor cores: adjoint scan (boundary adjoints + gradient of the initial state), then
// the chunk-parallel token gradients.  Needs only what the reference's backward is given: final state, boundary,
// state_dot_a.  Returns (dr, dw, dk, dv, da, db, dS0, error flag).
std::vector<torch::Tensor> wkv7_backward_chunked(torch::Tensor sco, torch::Tensor cs, torch::Tensor ce,
                                                 torch::Tensor final_state, torch::Tensor boundary,
                                                 torch::Tensor state_dot_a, torch::Tensor r, torch::Tensor w,
                                                 torch::Tensor k, torch::Tensor v, torch::Tensor a, torch::Tensor b,
                                                 std::optional<torch::Tensor> grad_output,
                                                 std::optional<torch::Tensor> grad_final_state, double scale,
                                                 std::vector<torch::Tensor> into) {
  check_chunk_tables(sco, cs, ce, r);
  for (const torch::Tensor* t : {&final_state, &boundary, &state_dot_a}) {
    check_cuda_contiguous(*t, "saved tensor");
    TORCH_CHECK(t->scalar_type() == torch::kFloat32 && t->device() == r.device(), "saved tensors must be float32 on r's device");
  }
  TORCH_CHECK(r.dim() == 3 && r.size(2) == 64, "token tensors must have shape [N,H,64]");
  const int64_t B = sco.numel() - 1, H = r.size(1), Cn = cs.numel();
  TORCH_CHECK(final_state.dim() == 4 && final_state.size(0) == B && final_state.size(1) == H,
              "final_state must have shape [B,H,64,64]");
  TORCH_CHECK(boundary.dim() == 4 && boundary.size(0) == Cn && boundary.size(1) == H, "boundary must be [Cn,H,64,64]");
  TORCH_CHECK(state_dot_a.sizes() == r.sizes(), "state_dot_a must be shaped like r");
  const c10::cuda::CUDAGuard guard(r.device());
  torch::Tensor go = grad_output.has_value() ? grad_output->contiguous() : torch::zeros_like(r);
  TORCH_CHECK(go.sizes() == r.sizes() && go.scalar_type() == r.scalar_type(), "grad_output must match r");
  auto table_status = chunk_table_status(sco, cs, ce, r);  // bad tables: NaN gradients, no out-of-range access
  auto scanned = wkv7_adjoint_scan(sco, cs, ce, r, w, a, b, go, grad_final_state, scale, std::nullopt, table_status);
  std::vector<torch::Tensor> g = std::move(into);  // the caller's six gradient tensors, or none: allocate
  if (g.empty())
    for (int i = 0; i < 6; ++i) g.push_back(torch::empty_like(r));
  TORCH_CHECK(g.size() == 6, "six gradient tensors are expected");
  for (const auto& t : g) {
    check_cuda_contiguous(t, "gradient tensor");
    TORCH_CHECK(t.numel() == r.numel() && t.scalar_type() == r.scalar_type(), "gradient tensors must match r");
  }
  auto error_flag = std::get<2>(scanned);
  check_rc(frwkv_wkv7_chunk_backward(
      sco.data_ptr<int>(), cs.data_ptr<int>(), ce.data_ptr<int>(), final_state.data_ptr<float>(),
      boundary.data_ptr<float>(), std::get<1>(scanned).data_ptr<float>(), state_dot_a.data_ptr<float>(), r.data_ptr(),
      w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(), nullptr, go.data_ptr(), g[0].data_ptr(),
      g[1].data_ptr(), g[2].data_ptr(), g[3].data_ptr(), g[4].data_ptr(), g[5].data_ptr(), error_flag.data_ptr<int>(),
      table_status.data_ptr<int>(), static_cast<int>(r.size(0)), static_cast<int>(B), static_cast<int>(Cn),
      static_cast<int>(H), 64, io_dtype_of(r), static_cast<float>(scale), current_stream(r)));
  g.push_back(std::get<0>(scanned));
  g.push_back(error_flag);
  return g;
}

// ---- the dense pretraining operator library: torch.ops.rwkv7_clampw_v3.{forward,backward} ------------------------
// Same two schemas as csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cpp:20-53 of the reference (the Python
// wrapper flashrwkv2/tmix/wkv7/pretrain.py:50-113 calls them with tensors it allocated):
//   forward(r, w, k, v, a, b, y, s, sa, head_size):  r..b, y io16 [B,T,H,D]; s fp32 [B,H,T/16,D,D] receives the state
//     (key row, value column) after every 16 tokens; sa fp32 [B,T,H,D] receives S_{t-1}^T a_t.
//   backward(r, w, k, v, a, b, dy, s, sa, dr, dw, dk, dv, da, db, head_size): the six gradients, dw with respect to
//     the raw `w` input (the retention transform included).
// Here the forward is the fused 64-token chunk kernel (y, sa, state at every 64-token boundary) followed by the
// element-wise checkpoint kernel that fills `s`; the backward takes every fourth checkpoint as its chunk boundary.
// Unlike the reference's launches (legacy default stream) everything runs on the current Torch stream.
struct DenseTables {
  torch::Tensor sco, cs, ce;
  int64_t per;
};
DenseTables dense_tables(int64_t B, int64_t T, const torch::Tensor& like) {
  const int64_t per = (T + 63) / 64;
  auto opt = like.options().dtype(torch::kInt32);
  auto idx = torch::arange(B * per, opt);
  auto bi = torch::floor_divide(idx, per);
  auto cs = bi * T + (idx - bi * per) * 64;
  auto ce = torch::minimum(cs + 64, (bi + 1) * T);
  return {(torch::arange(B + 1, opt) * per).to(torch::kInt32).contiguous(), cs.to(torch::kInt32).contiguous(),
          ce.to(torch::kInt32).contiguous(), per};
}
torch::Tensor g_clampw_flags[2];  // device error flags of the last forward / backward (read on request only)

std::vector<torch::Tensor> clampw_error_flags() {
  std::vector<torch::Tensor> out;
  for (const auto& f : g_clampw_flags)
    if (f.defined()) out.push_back(f);
  return out;
}

void clampw_check(const torch::Tensor& r, const torch::Tensor& t, const char* name) {
  check_cuda_contiguous(t, name);
  TORCH_CHECK(t.scalar_type() == r.scalar_type() && t.device() == r.device() && t.sizes() == r.sizes(), name,
              " must match r in dtype, device and shape");
}
void clampw_check_saved(const torch::Tensor& r, const torch::Tensor& s, const torch::Tensor& sa) {
  const int64_t B = r.size(0), T = r.size(1), H = r.size(2), D = r.size(3);
  check_cuda_contiguous(s, "s");
  check_cuda_contiguous(sa, "sa");
  TORCH_CHECK(s.scalar_type() == torch::kFloat32 && sa.scalar_type() == torch::kFloat32 && s.device() == r.device() &&
                  sa.device() == r.device(),
              "s and sa must be float32 on r's device");
  TORCH_CHECK(s.numel() == B * H * (T / 16) * D * D, "s must have shape [B,H,T/16,D,D]");
  TORCH_CHECK(sa.numel() == r.numel(), "sa must have shape [B,T,H,D]");
}
void clampw_check_head(const torch::Tensor& r, int64_t head_size) {
  TORCH_CHECK(head_size == 64 || head_size == 128 || head_size == 256, "head_size must be one of 64, 128, or 256");
  TORCH_CHECK(r.dim() == 4 && r.size(3) == head_size, "input head dimension must equal head_size");
  TORCH_CHECK(r.scalar_type() == torch::kBFloat16 || r.scalar_type() == torch::kFloat16, "r must be bfloat16 or float16");
  check_cuda_contiguous(r, "r");
  TORCH_CHECK(r.numel() > 0 && r.size(1) % 16 == 0, "T must be a positive multiple of 16");
}

void clampw_forward(torch::Tensor& r, torch::Tensor& w, torch::Tensor& k, torch::Tensor& v, torch::Tensor& a,
                    torch::Tensor& b, torch::Tensor& y, torch::Tensor& s, torch::Tensor& sa, int64_t head_size) {
  clampw_check_head(r, head_size);
  const torch::Tensor* named[] = {&w, &k, &v, &a, &b, &y};
  const char* names[] = {"w", "k", "v", "a", "b", "y"};
  for (int i = 0; i < 6; ++i) clampw_check(r, *named[i], names[i]);
  clampw_check_saved(r, s, sa);
  const int64_t B = r.size(0), T = r.size(1), H = r.size(2), D = head_size;
  const c10::cuda::CUDAGuard guard(r.device());
  const DenseTables tab = dense_tables(B, T, r);
  auto state = torch::zeros({B, H, D, D}, r.options().dtype(torch::kFloat32));
  auto flat = [&](const torch::Tensor& t) { return t.view({B * T, H, D}); };
  if (D != 64) {  // head sizes 128 / 256: the plain recurrence writes the 16-token states itself
    wkv7_train_wide_forward(tab.sco, tab.cs, tab.ce, state, flat(r), flat(w), flat(k), flat(v), flat(a), flat(b), flat(y),
                            std::nullopt, flat(sa), 1.0, s.view({B, H, T / 16, D, D}));
    return;
  }
  auto boundary = torch::empty({B * tab.per, H, 64, 64}, state.options());
  g_clampw_flags[0] = wkv7_chunk_forward(tab.sco, tab.cs, tab.ce, state, flat(r), flat(w), flat(k), flat(v), flat(a),
                                         flat(b), flat(y), 1.0, std::nullopt, std::nullopt, boundary, std::nullopt,
                                         std::nullopt, flat(sa), 1);
  check_rc(frwkv_wkv7_dense_checkpoints(boundary.data_ptr<float>(), sa.data_ptr<float>(), w.data_ptr(), k.data_ptr(),
                                        v.data_ptr(), b.data_ptr(), s.data_ptr<float>(), static_cast<int>(B),
                                        static_cast<int>(T), static_cast<int>(H), 64, io_dtype_of(r), current_stream(r)));
}

void clampw_backward(torch::Tensor& r, torch::Tensor& w, torch::Tensor& k, torch::Tensor& v, torch::Tensor& a,
                     torch::Tensor& b, torch::Tensor& dy, torch::Tensor& s, torch::Tensor& sa, torch::Tensor& dr,
                     torch::Tensor& dw, torch::Tensor& dk, torch::Tensor& dv, torch::Tensor& da, torch::Tensor& db,
                     int64_t head_size) {
  clampw_check_head(r, head_size);
  const torch::Tensor* named[] = {&w, &k, &v, &a, &b, &dy, &dr, &dw, &dk, &dv, &da, &db};
  const char* names[] = {"w", "k", "v", "a", "b", "dy", "dr", "dw", "dk", "dv", "da", "db"};
  for (int i = 0; i < 12; ++i) clampw_check(r, *named[i], names[i]);
  clampw_check_saved(r, s, sa);
  const int64_t B = r.size(0), T = r.size(1), H = r.size(2), G = T / 16, D = head_size;
  const c10::cuda::CUDAGuard guard(r.device());
  const DenseTables tab = dense_tables(B, T, r);
  auto s5 = s.view({B, H, G, D, D});
  auto final_state = s5.select(2, G - 1).contiguous();
  // chunk c starts from the checkpoint after token 64 c, i.e. s[:, :, 4 c - 1]; chunk 0 from the zero state
  auto boundary = torch::zeros({B, tab.per, H, D, D}, s.options());
  if (tab.per > 1) boundary.slice(1, 1).copy_(s5.slice(2, 3, 4 * (tab.per - 1), 4).permute({0, 2, 1, 3, 4}));
  auto flat = [&](const torch::Tensor& t) { return t.view({B * T, H, D}); };
  if (D != 64) {
    wkv7_train_wide_backward(tab.sco, tab.cs, tab.ce, final_state, boundary.view({B * tab.per, H, D, D}), flat(sa),
                             flat(r), flat(w), flat(k), flat(v), flat(a), flat(b), flat(dy), std::nullopt, 1.0,
                             {flat(dr), flat(dw), flat(dk), flat(dv), flat(da), flat(db)});
    return;
  }
  auto g = wkv7_backward_chunked(tab.sco, tab.cs, tab.ce, final_state, boundary.view({B * tab.per, H, 64, 64}), flat(sa),
                                 flat(r), flat(w), flat(k), flat(v), flat(a), flat(b), flat(dy), std::nullopt, 1.0,
                                 {flat(dr), flat(dw), flat(dk), flat(dv), flat(da), flat(db)});
  g_clampw_flags[1] = g.back();
}

// ---- training-side TMix glue on dense [B,T,C] tensors (names and argument order of the reference's
// pretrain_tmix_* extension functions, flashrwkv2/tmix/{a_gate,vres_gate,mix6,kk_pre,lnx_rkvres_xg}) ----------
void check_dense(const torch::Tensor& t, const char* name, const torch::Tensor& ref) {
  check_io16(t, name, ref);
  TORCH_CHECK(t.dim() == 3 && t.sizes() == ref.sizes(), name, " must have shape [B,T,C]");
}
void check_dense_vector(const torch::Tensor& t, const char* name, const torch::Tensor& ref) {
  check_io16(t, name, ref);
  TORCH_CHECK(t.numel() == ref.size(2), name, " must have C elements");
}
void check_dense_root(const torch::Tensor& x, const char* name) {
  check_io16(x, name, x);
  TORCH_CHECK(x.dim() == 3 && x.numel() > 0, name, " must have non-empty shape [B,T,C]");
  TORCH_CHECK(x.size(2) % 8 == 0, name, ": C must be a multiple of 8");
}
torch::Tensor reduce_workspace(const torch::Tensor& ref, int vectors) {
  const int64_t rows = ref.size(0) * ref.size(1);
  return torch::empty({frwkv_pretrain_workspace_floats(rows, static_cast<int>(ref.size(2)), vectors)},
                      ref.options().dtype(torch::kFloat32));
}

torch::Tensor pretrain_tmix_a_gate_forward(torch::Tensor a0, torch::Tensor a12) {
  check_dense_root(a12, "a12");
  check_dense_vector(a0, "a0", a12);
  const c10::cuda::CUDAGuard guard(a12.device());
  auto out = torch::empty_like(a12);
  check_rc(frwkv_pretrain_a_gate_forward(a0.data_ptr(), a12.data_ptr(), out.data_ptr(), a12.size(0) * a12.size(1),
                                         static_cast<int>(a12.size(2)), io_dtype_of(a12), current_stream(a12)));
  return out;
}

std::vector<torch::Tensor> pretrain_tmix_a_gate_backward(torch::Tensor grad_output, torch::Tensor a0,
                                                         torch::Tensor a12) {
  check_dense_root(a12, "a12");
  check_dense_vector(a0, "a0", a12);
  check_dense(grad_output, "grad_output", a12);
  const c10::cuda::CUDAGuard guard(a12.device());
  auto grad_a0 = torch::empty_like(a0);
  auto grad_a12 = torch::empty_like(a12);
  auto ws = reduce_workspace(a12, 1);
  check_rc(frwkv_pretrain_a_gate_backward(grad_output.data_ptr(), a0.data_ptr(), a12.data_ptr(), grad_a0.data_ptr(),
                                          grad_a12.data_ptr(), ws.data_ptr<float>(), ws.numel(),
                                          a12.size(0) * a12.size(1), static_cast<int>(a12.size(2)), io_dtype_of(a12),
                                          current_stream(a12)));
  return {grad_a0, grad_a12};
}

torch::Tensor pretrain_tmix_vres_gate_forward(torch::Tensor v, torch::Tensor v_first, torch::Tensor v0,
                                              torch::Tensor v12) {
  check_dense_root(v, "value");
  check_dense(v_first, "first_value", v);
  check_dense(v12, "v12", v);
  check_dense_vector(v0, "v0", v);
  const c10::cuda::CUDAGuard guard(v.device());
  auto out = torch::empty_like(v);
  check_rc(frwkv_tmix_vres_gate_forward_varlen(v.data_ptr(), v_first.data_ptr(), v0.data_ptr(), v12.data_ptr(),
                                               out.data_ptr(), v.size(0) * v.size(1), static_cast<int>(v.size(2)),
                                               io_dtype_of(v), current_stream(v)));
  return out;
}

std::vector<torch::Tensor> pretrain_tmix_vres_gate_backward(torch::Tensor grad_output, torch::Tensor v,
                                                            torch::Tensor v_first, torch::Tensor v0,
                                                            torch::Tensor v12) {
  check_dense_root(v, "value");
  check_dense(v_first, "first_value", v);
  check_dense(v12, "v12", v);
  check_dense(grad_output, "grad_output", v);
  check_dense_vector(v0, "v0", v);
  const c10::cuda::CUDAGuard guard(v.device());
  auto grad_v = torch::empty_like(v), grad_vf = torch::empty_like(v), grad_v12 = torch::empty_like(v);
  auto grad_v0 = torch::empty_like(v0);
  auto ws = reduce_workspace(v, 1);
  check_rc(frwkv_pretrain_vres_gate_backward(grad_output.data_ptr(), v.data_ptr(), v_first.data_ptr(), v0.data_ptr(),
                                             v12.data_ptr(), grad_v.data_ptr(), grad_vf.data_ptr(), grad_v0.data_ptr(),
                                             grad_v12.data_ptr(), ws.data_ptr<float>(), ws.numel(),
                                             v.size(0) * v.size(1), static_cast<int>(v.size(2)), io_dtype_of(v),
                                             current_stream(v)));
  return {grad_v, grad_vf, grad_v0, grad_v12};
}

std::vector<torch::Tensor> pretrain_tmix_mix6_forward(torch::Tensor x, torch::Tensor x_r, torch::Tensor x_w,
                                                      torch::Tensor x_k, torch::Tensor x_v, torch::Tensor x_a,
                                                      torch::Tensor x_g) {
  check_dense_root(x, "x");
  const torch::Tensor mix[6] = {x_r, x_w, x_k, x_v, x_a, x_g};
  const void* mix_ptr[6];
  void* out_ptr[6];
  std::vector<torch::Tensor> outs;
  const c10::cuda::CUDAGuard guard(x.device());
  for (int j = 0; j < 6; ++j) {
    check_dense_vector(mix[j], "mix vector", x);
    outs.push_back(torch::empty_like(x));
    mix_ptr[j] = mix[j].data_ptr();
    out_ptr[j] = outs.back().data_ptr();
  }
  check_rc(frwkv_pretrain_mix6_forward(x.data_ptr(), mix_ptr, out_ptr, x.size(0), static_cast<int>(x.size(1)),
                                       static_cast<int>(x.size(2)), io_dtype_of(x), current_stream(x)));
  return outs;
}

std::vector<torch::Tensor> pretrain_tmix_mix6_backward(torch::Tensor g_r, torch::Tensor g_w, torch::Tensor g_k,
                                                       torch::Tensor g_v, torch::Tensor g_a, torch::Tensor g_g,
                                                       torch::Tensor x, torch::Tensor x_r, torch::Tensor x_w,
                                                       torch::Tensor x_k, torch::Tensor x_v, torch::Tensor x_a,
                                                       torch::Tensor x_g) {
  check_dense_root(x, "x");
  const torch::Tensor grads[6] = {g_r, g_w, g_k, g_v, g_a, g_g};
  const torch::Tensor mix[6] = {x_r, x_w, x_k, x_v, x_a, x_g};
  const void* grad_ptr[6];
  const void* mix_ptr[6];
  void* gmix_ptr[6];
  const c10::cuda::CUDAGuard guard(x.device());
  std::vector<torch::Tensor> result{torch::empty_like(x)};
  for (int j = 0; j < 6; ++j) {
    check_dense(grads[j], "grad_output", x);
    check_dense_vector(mix[j], "mix vector", x);
    result.push_back(torch::empty_like(mix[j]));
    grad_ptr[j] = grads[j].data_ptr();
    mix_ptr[j] = mix[j].data_ptr();
    gmix_ptr[j] = result.back().data_ptr();
  }
  auto ws = reduce_workspace(x, 6);
  check_rc(frwkv_pretrain_mix6_backward(grad_ptr, x.data_ptr(), mix_ptr, result[0].data_ptr(), gmix_ptr,
                                        ws.data_ptr<float>(), ws.numel(), x.size(0), static_cast<int>(x.size(1)),
                                        static_cast<int>(x.size(2)), io_dtype_of(x), current_stream(x)));
  return result;
}

void check_shift_rows(const torch::Tensor& t, const char* name, const torch::Tensor& x) {
  check_io16(t, name, x);
  TORCH_CHECK(t.dim() == 2 && t.size(0) == x.size(0) && t.size(1) == x.size(2), name, " must have shape [B,C]");
}

// returns the six mixed tensors and the final shift state x[:, -1, :]
std::vector<torch::Tensor> statetune_tmix_mix6_forward(torch::Tensor x, torch::Tensor initial_shift,
                                                       torch::Tensor x_r, torch::Tensor x_w, torch::Tensor x_k,
                                                       torch::Tensor x_v, torch::Tensor x_a, torch::Tensor x_g) {
  check_dense_root(x, "x");
  check_shift_rows(initial_shift, "initial_shift", x);
  const torch::Tensor mix[6] = {x_r, x_w, x_k, x_v, x_a, x_g};
  const void* mix_ptr[6];
  void* out_ptr[6];
  std::vector<torch::Tensor> outs;
  const c10::cuda::CUDAGuard guard(x.device());
  for (int j = 0; j < 6; ++j) {
    check_dense_vector(mix[j], "mix vector", x);
    outs.push_back(torch::empty_like(x));
    mix_ptr[j] = mix[j].data_ptr();
    out_ptr[j] = outs.back().data_ptr();
  }
  outs.push_back(torch::empty_like(initial_shift));
  check_rc(frwkv_statetune_mix6_forward(x.data_ptr(), initial_shift.data_ptr(), mix_ptr, out_ptr,
                                        outs.back().data_ptr(), x.size(0), static_cast<int>(x.size(1)),
                                        static_cast<int>(x.size(2)), io_dtype_of(x), current_stream(x)));
  return outs;
}

// gradients of (x, initial_shift, x_r, x_w, x_k, x_v, x_a, x_g)
std::vector<torch::Tensor> statetune_tmix_mix6_backward(torch::Tensor g_r, torch::Tensor g_w, torch::Tensor g_k,
                                                        torch::Tensor g_v, torch::Tensor g_a, torch::Tensor g_g,
                                                        torch::Tensor g_final, torch::Tensor x,
                                                        torch::Tensor initial_shift, torch::Tensor x_r,
                                                        torch::Tensor x_w, torch::Tensor x_k, torch::Tensor x_v,
                                                        torch::Tensor x_a, torch::Tensor x_g) {
  check_dense_root(x, "x");
  check_shift_rows(initial_shift, "initial_shift", x);
  check_shift_rows(g_final, "grad of the final shift", x);
  const torch::Tensor grads[6] = {g_r, g_w, g_k, g_v, g_a, g_g};
  const torch::Tensor mix[6] = {x_r, x_w, x_k, x_v, x_a, x_g};
  const void* grad_ptr[6];
  const void* mix_ptr[6];
  void* gmix_ptr[6];
  const c10::cuda::CUDAGuard guard(x.device());
  std::vector<torch::Tensor> result{torch::empty_like(x), torch::empty_like(initial_shift)};
  for (int j = 0; j < 6; ++j) {
    check_dense(grads[j], "grad_output", x);
    check_dense_vector(mix[j], "mix vector", x);
    result.push_back(torch::empty_like(mix[j]));
    grad_ptr[j] = grads[j].data_ptr();
    mix_ptr[j] = mix[j].data_ptr();
    gmix_ptr[j] = result.back().data_ptr();
  }
  auto ws = reduce_workspace(x, 6);
  check_rc(frwkv_statetune_mix6_backward(grad_ptr, g_final.data_ptr(), x.data_ptr(), initial_shift.data_ptr(), mix_ptr,
                                         result[0].data_ptr(), result[1].data_ptr(), gmix_ptr, ws.data_ptr<float>(),
                                         ws.numel(), x.size(0), static_cast<int>(x.size(1)),
                                         static_cast<int>(x.size(2)), io_dtype_of(x), current_stream(x)));
  return result;
}

void check_head_size(const torch::Tensor& x, int64_t head_size) {
  TORCH_CHECK(head_size == 64 || head_size == 128 || head_size == 256, "head_size must be one of 64, 128, or 256");
  TORCH_CHECK(x.size(2) % head_size == 0, "C must be divisible by head_size");
}

std::vector<torch::Tensor> pretrain_tmix_kk_pre_forward(torch::Tensor k, torch::Tensor k_k, torch::Tensor a,
                                                        torch::Tensor k_a, int64_t head_size) {
  check_dense_root(k, "key");
  check_head_size(k, head_size);
  check_dense(a, "learning_rate", k);
  check_dense_vector(k_k, "key_scale", k);
  check_dense_vector(k_a, "learning_rate_scale", k);
  const c10::cuda::CUDAGuard guard(k.device());
  auto new_k = torch::empty_like(k), neg_kk = torch::empty_like(k), kka = torch::empty_like(k);
  auto inv_norm = torch::empty({k.size(0), k.size(1), k.size(2) / head_size}, k.options().dtype(torch::kFloat32));
  check_rc(frwkv_pretrain_kk_pre_forward(k.data_ptr(), k_k.data_ptr(), a.data_ptr(), k_a.data_ptr(), new_k.data_ptr(),
                                         neg_kk.data_ptr(), kka.data_ptr(), inv_norm.data_ptr<float>(),
                                         k.size(0) * k.size(1), static_cast<int>(k.size(2)),
                                         static_cast<int>(head_size), io_dtype_of(k), current_stream(k)));
  return {new_k, neg_kk, kka, inv_norm};
}

std::vector<torch::Tensor> pretrain_tmix_kk_pre_backward(torch::Tensor g_new_k, torch::Tensor g_neg_kk,
                                                         torch::Tensor g_kka, torch::Tensor k, torch::Tensor k_k,
                                                         torch::Tensor a, torch::Tensor k_a, torch::Tensor inv_norm,
                                                         int64_t head_size) {
  check_dense_root(k, "key");
  check_head_size(k, head_size);
  check_dense(a, "learning_rate", k);
  check_dense(g_new_k, "grad_new_key", k);
  check_dense(g_neg_kk, "grad_negative_direction", k);
  check_dense(g_kka, "grad_scaled_direction", k);
  check_dense_vector(k_k, "key_scale", k);
  check_dense_vector(k_a, "learning_rate_scale", k);
  check_cuda_contiguous(inv_norm, "inverse_norm");
  TORCH_CHECK(inv_norm.scalar_type() == torch::kFloat32 &&
                  inv_norm.numel() == k.size(0) * k.size(1) * (k.size(2) / head_size),
              "inverse_norm must be float32 [B,T,C/head_size]");
  const c10::cuda::CUDAGuard guard(k.device());
  auto grad_k = torch::empty_like(k), grad_a = torch::empty_like(a);
  auto grad_k_k = torch::empty_like(k_k), grad_k_a = torch::empty_like(k_a);
  auto ws = reduce_workspace(k, 2);
  check_rc(frwkv_pretrain_kk_pre_backward(
      g_new_k.data_ptr(), g_neg_kk.data_ptr(), g_kka.data_ptr(), k.data_ptr(), k_k.data_ptr(), a.data_ptr(),
      k_a.data_ptr(), inv_norm.data_ptr<float>(), grad_k.data_ptr(), grad_k_k.data_ptr(), grad_a.data_ptr(),
      grad_k_a.data_ptr(), ws.data_ptr<float>(), ws.numel(), k.size(0) * k.size(1), static_cast<int>(k.size(2)),
      static_cast<int>(head_size), io_dtype_of(k), current_stream(k)));
  return {grad_k, grad_k_k, grad_a, grad_k_a};
}

std::vector<torch::Tensor> pretrain_tmix_lnx_rkvres_xg_forward(torch::Tensor x, torch::Tensor r, torch::Tensor k,
                                                               torch::Tensor v, torch::Tensor r_k,
                                                               torch::Tensor weight, torch::Tensor bias,
                                                               torch::Tensor g, int64_t head_size) {
  check_dense_root(x, "x");
  check_head_size(x, head_size);
  check_dense(r, "r", x);
  check_dense(k, "k", x);
  check_dense(v, "v", x);
  check_dense(g, "g", x);
  check_dense_vector(r_k, "residual_scale", x);
  check_dense_vector(weight, "weight", x);
  check_dense_vector(bias, "bias", x);
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  auto stat_opts = x.options().dtype(torch::kFloat32);
  auto mean = torch::empty({x.size(0), x.size(1), x.size(2) / head_size}, stat_opts);
  auto rstd = torch::empty_like(mean);
  check_rc(frwkv_pretrain_lnx_rkvres_xg_forward(
      x.data_ptr(), r.data_ptr(), k.data_ptr(), v.data_ptr(), r_k.data_ptr(), weight.data_ptr(), bias.data_ptr(),
      g.data_ptr(), out.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), x.size(0) * x.size(1),
      static_cast<int>(x.size(2)), static_cast<int>(head_size), io_dtype_of(x), current_stream(x)));
  return {out, mean, rstd};
}

std::vector<torch::Tensor> pretrain_tmix_lnx_rkvres_xg_backward(torch::Tensor grad_output, torch::Tensor x,
                                                                torch::Tensor r, torch::Tensor k, torch::Tensor v,
                                                                torch::Tensor r_k, torch::Tensor weight,
                                                                torch::Tensor bias, torch::Tensor g,
                                                                torch::Tensor mean, torch::Tensor rstd,
                                                                int64_t head_size) {
  check_dense_root(x, "x");
  check_head_size(x, head_size);
  check_dense(grad_output, "grad_output", x);
  check_dense(r, "r", x);
  check_dense(k, "k", x);
  check_dense(v, "v", x);
  check_dense(g, "g", x);
  check_dense_vector(r_k, "residual_scale", x);
  check_dense_vector(weight, "weight", x);
  check_dense_vector(bias, "bias", x);
  check_cuda_contiguous(mean, "mean");
  check_cuda_contiguous(rstd, "rstd");
  const int64_t stats = x.size(0) * x.size(1) * (x.size(2) / head_size);
  TORCH_CHECK(mean.scalar_type() == torch::kFloat32 && rstd.scalar_type() == torch::kFloat32 &&
                  mean.numel() == stats && rstd.numel() == stats,
              "mean and rstd must be float32 [B,T,C/head_size]");
  const c10::cuda::CUDAGuard guard(x.device());
  auto gx = torch::empty_like(x), gr = torch::empty_like(x), gk = torch::empty_like(x), gv = torch::empty_like(x),
       gg = torch::empty_like(x);
  auto grk = torch::empty_like(r_k), gw = torch::empty_like(weight), gb = torch::empty_like(bias);
  auto ws = reduce_workspace(x, 3);
  check_rc(frwkv_pretrain_lnx_rkvres_xg_backward(
      grad_output.data_ptr(), x.data_ptr(), r.data_ptr(), k.data_ptr(), v.data_ptr(), r_k.data_ptr(),
      weight.data_ptr(), bias.data_ptr(), g.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), gx.data_ptr(),
      gr.data_ptr(), gk.data_ptr(), gv.data_ptr(), grk.data_ptr(), gw.data_ptr(), gb.data_ptr(), gg.data_ptr(),
      ws.data_ptr<float>(), ws.numel(), x.size(0) * x.size(1), static_cast<int>(x.size(2)),
      static_cast<int>(head_size), io_dtype_of(x), current_stream(x)));
  return {gx, gr, gk, gv, grk, gw, gb, gg};
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
      .def("_max_seqlen", [](const MetadataTicket& t) { return t.max_seqlen(); })
      .def("_direct_slots", [](const MetadataTicket& t) { return t.direct_slots(); });
  m.def("prepare_recurrent_metadata", &prepare_recurrent_metadata, py::arg("query_start_loc"),
        py::arg("state_indices"), py::arg("total_tokens"), py::arg("state_pool_size"),
        py::arg("max_seqlen") = -1);
  m.def("recurrent_fp32_from_decay_logits", &recurrent_fp32_from_decay_logits, py::arg("query_start_loc"),
        py::arg("state_indices"), py::arg("state"), py::arg("r"), py::arg("decay_logits"), py::arg("k"),
        py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"), py::arg("scale"),
        py::arg("decay_bias") = py::none(), py::arg("validated_metadata") = py::none(),
        py::arg("max_seqlen") = -1, py::arg("output_fp32") = py::none());
  m.def("recurrent_fp16_from_decay_logits", &recurrent_fp16_from_decay_logits, py::arg("query_start_loc"),
        py::arg("state_indices"), py::arg("elapsed_state_pool"), py::arg("state"), py::arg("r"),
        py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"),
        py::arg("scale"), py::arg("decay_bias") = py::none(), py::arg("validated_metadata") = py::none(),
        py::arg("max_seqlen") = -1);
  m.def("recurrent_fp16_advance_i32", &recurrent_fp16_advance_i32, py::arg("elapsed_state"), py::arg("amount"));
  m.def("recurrent_fp16_advance_i32_varlen", &recurrent_fp16_advance_i32_varlen, py::arg("query_start_loc"),
        py::arg("state_indices"), py::arg("elapsed_state_pool"), py::arg("total_tokens"),
        py::arg("validated_metadata") = py::none());
  m.def("wkv7_chunk_forward", &wkv7_chunk_forward, py::arg("sequence_chunk_offsets"),
        py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("state"), py::arg("r"),
        py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"),
        py::arg("scale") = 1.0, py::arg("decay_bias") = py::none(), py::arg("state_indices") = py::none(),
        py::arg("boundary") = py::none(), py::arg("output_fp32") = py::none(),
        py::arg("metadata_status") = py::none(), py::arg("state_dot_a") = py::none(), py::arg("path") = -1);
  m.def("rl_infctx_chunk_fp32io16_forward", &rl_infctx_chunk_fp32io16_forward, py::arg("sequence_chunk_offsets"),
        py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("state"), py::arg("r"),
        py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("strategy") = 1,
        py::arg("scale") = 1.0, py::arg("decay_bias") = py::none());
  m.def("tmix_mix6_forward_varlen", &tmix_mix6_forward_varlen, py::arg("x"), py::arg("shift_state_pool"),
        py::arg("x_r"), py::arg("x_w"), py::arg("x_k"), py::arg("x_v"), py::arg("x_a"), py::arg("x_g"),
        py::arg("cu_seqlens"), py::arg("state_indices"), py::arg("max_seqlen") = -1,
        py::arg("validated_metadata") = py::none());
  m.def("tmix_layer_norm_forward_varlen", &tmix_layer_norm_forward_varlen, py::arg("x"), py::arg("weight"),
        py::arg("bias"), py::arg("eps") = 1e-5);
  m.def("tmix_add_layer_norm_forward_varlen", &tmix_add_layer_norm_forward_varlen, py::arg("x"), py::arg("residual"),
        py::arg("weight"), py::arg("bias"), py::arg("eps") = 1e-5, py::arg("batch_size") = -1);
  m.def("tmix_add_last_layer_norm_forward_varlen", &tmix_add_last_layer_norm_forward_varlen, py::arg("x"),
        py::arg("residual"), py::arg("weight"), py::arg("bias"), py::arg("eps") = 1e-5);
  m.def("tmix_add_forward_varlen", &tmix_add_forward_varlen, py::arg("x"), py::arg("residual"));
  m.def("tmix_mix6_add_layer_norm_forward_varlen", &tmix_mix6_add_layer_norm_forward_varlen, py::arg("x"),
        py::arg("residual"), py::arg("weight"), py::arg("bias"), py::arg("shift_state_pool"), py::arg("x_r"),
        py::arg("x_w"), py::arg("x_k"), py::arg("x_v"), py::arg("x_a"), py::arg("x_g"), py::arg("cu_seqlens"),
        py::arg("state_indices"), py::arg("max_seqlen") = -1, py::arg("eps") = 1e-5,
        py::arg("validated_metadata") = py::none());
  m.def("tmix_decode_layer", &tmix_decode_layer, py::arg("x"), py::arg("v_first"), py::arg("shift_state_pool"),
        py::arg("state_pool"), py::arg("mixes"), py::arg("square_weights"), py::arg("rank_in_weights"),
        py::arg("rank_out_weights"), py::arg("channel_vectors"), py::arg("cu_seqlens"), py::arg("state_indices"),
        py::arg("eps") = 64e-5, py::arg("validated_metadata") = py::none());
  m.def("tmix_shift_project_varlen", &tmix_shift_project_varlen, py::arg("x"), py::arg("shift_state_pool"),
        py::arg("mixes"), py::arg("weights"), py::arg("cu_seqlens"), py::arg("state_indices"),
        py::arg("max_seqlen") = -1, py::arg("validated_metadata") = py::none());
  m.def("tmix_kk_a_gate_forward_varlen", &tmix_kk_a_gate_forward_varlen, py::arg("k"), py::arg("k_k"), py::arg("a0"),
        py::arg("a12"), py::arg("k_a"), py::arg("head_size") = 64, py::arg("batch_size") = 1,
        py::arg("max_seqlen") = 1);
  m.def("tmix_lnx_rkvres_xg_forward_varlen", &tmix_lnx_rkvres_xg_forward_varlen, py::arg("x"), py::arg("r"),
        py::arg("k"), py::arg("v"), py::arg("r_k"), py::arg("weight"), py::arg("bias"), py::arg("g"),
        py::arg("head_size") = 64, py::arg("batch_size") = 1, py::arg("max_seqlen") = 1);
  m.def("tmix_vres_gate_forward_varlen", &tmix_vres_gate_forward_varlen, py::arg("v"), py::arg("v_first"),
        py::arg("v0"), py::arg("v12"));
  m.def("infer_chunk_bf16_forward_varlen", &infer_chunk_bf16_forward_varlen_native, py::arg("r"),
        py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("state_pool"),
        py::arg("cu_seqlens"), py::arg("state_indices"), py::arg("chunk_size") = 16, py::arg("max_seqlen") = -1,
        py::arg("scale") = 1.0, py::arg("decay_bias") = py::none());
  m.def("rl_infctx_chunk_fp32io16_backward_replay", &rl_infctx_chunk_fp32io16_backward_replay,
        py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("boundary"), py::arg("r"),
        py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"),
        py::arg("state_dot_a"), py::arg("scale") = 1.0, py::arg("decay_bias") = py::none());
  m.def("statetune_recurrent_fp32io16_forward", &statetune_recurrent_fp32io16_forward,
        py::arg("sequence_chunk_offsets"), py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("state"),
        py::arg("r"), py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"),
        py::arg("boundary"), py::arg("state_dot_a"), py::arg("scale") = 1.0);
  m.def("statetune_recurrent_fp32io16_backward", &statetune_recurrent_fp32io16_backward,
        py::arg("sequence_chunk_offsets"), py::arg("chunk_token_starts"), py::arg("chunk_token_ends"),
        py::arg("final_state"), py::arg("r"), py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"),
        py::arg("b"), py::arg("state_dot_a"), py::arg("grad_output"), py::arg("grad_final_state"), py::arg("boundary"),
        py::arg("grad_r"), py::arg("grad_decay_logits"), py::arg("grad_k"), py::arg("grad_v"), py::arg("grad_a"),
        py::arg("grad_b"), py::arg("grad_initial_state"), py::arg("scale") = 1.0);
  m.def("wkv7_adjoint_scan", &wkv7_adjoint_scan, py::arg("sequence_chunk_offsets"), py::arg("chunk_token_starts"),
        py::arg("chunk_token_ends"), py::arg("r"), py::arg("decay_logits"), py::arg("a"), py::arg("b"),
        py::arg("grad_output"), py::arg("grad_final_state") = py::none(), py::arg("scale") = 1.0,
        py::arg("decay_bias") = py::none(), py::arg("table_status") = py::none());
  m.def("wkv7_backward_chunked", &wkv7_backward_chunked, py::arg("sequence_chunk_offsets"),
        py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("final_state"), py::arg("boundary"),
        py::arg("state_dot_a"), py::arg("r"), py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"),
        py::arg("b"), py::arg("grad_output") = py::none(), py::arg("grad_final_state") = py::none(),
        py::arg("scale") = 1.0, py::arg("into") = std::vector<torch::Tensor>{});
  m.def("rwkv7_clampw_v3_error_flags", &clampw_error_flags);
  m.def("last_error_flags", &last_error_flags);
  m.def("wkv7_train_wide_forward", &wkv7_train_wide_forward, py::arg("sequence_chunk_offsets"),
        py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("state"), py::arg("r"),
        py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"),
        py::arg("boundary") = py::none(), py::arg("state_dot_a") = py::none(), py::arg("scale") = 1.0,
        py::arg("dense_checkpoints") = py::none());
  m.def("wkv7_train_wide_backward", &wkv7_train_wide_backward, py::arg("sequence_chunk_offsets"),
        py::arg("chunk_token_starts"), py::arg("chunk_token_ends"), py::arg("final_state"), py::arg("boundary"),
        py::arg("state_dot_a"), py::arg("r"), py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"),
        py::arg("b"), py::arg("grad_output") = py::none(), py::arg("grad_final_state") = py::none(),
        py::arg("scale") = 1.0, py::arg("into") = std::vector<torch::Tensor>{});
  m.def("wkv7_chunk_replay", &wkv7_chunk_replay, py::arg("chunk_token_starts"), py::arg("chunk_token_ends"),
        py::arg("boundary"), py::arg("r"), py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"),
        py::arg("b"), py::arg("decay_bias") = py::none());
  m.def("wkv7_backward", &wkv7_backward, py::arg("sequence_chunk_offsets"), py::arg("chunk_token_starts"),
        py::arg("chunk_token_ends"), py::arg("final_state"), py::arg("boundary"), py::arg("checkpoints"),
        py::arg("state_dot_a"), py::arg("r"), py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"),
        py::arg("b"), py::arg("grad_output") = py::none(), py::arg("grad_final_state") = py::none(),
        py::arg("scale") = 1.0);
  m.def("pretrain_tmix_a_gate_forward", &pretrain_tmix_a_gate_forward, py::arg("a0"), py::arg("a12"));
  m.def("pretrain_tmix_a_gate_backward", &pretrain_tmix_a_gate_backward, py::arg("grad_output"), py::arg("a0"),
        py::arg("a12"));
  m.def("pretrain_tmix_vres_gate_forward", &pretrain_tmix_vres_gate_forward, py::arg("value"),
        py::arg("first_value"), py::arg("v0"), py::arg("v12"));
  m.def("pretrain_tmix_vres_gate_backward", &pretrain_tmix_vres_gate_backward, py::arg("grad_output"),
        py::arg("value"), py::arg("first_value"), py::arg("v0"), py::arg("v12"));
  m.def("pretrain_tmix_mix6_forward", &pretrain_tmix_mix6_forward);
  m.def("pretrain_tmix_mix6_backward", &pretrain_tmix_mix6_backward);
  m.def("statetune_tmix_mix6_forward", &statetune_tmix_mix6_forward);
  m.def("statetune_tmix_mix6_backward", &statetune_tmix_mix6_backward);
  m.def("pretrain_tmix_kk_pre_forward", &pretrain_tmix_kk_pre_forward);
  m.def("pretrain_tmix_kk_pre_backward", &pretrain_tmix_kk_pre_backward);
  m.def("pretrain_tmix_lnx_rkvres_xg_forward", &pretrain_tmix_lnx_rkvres_xg_forward);
  m.def("pretrain_tmix_lnx_rkvres_xg_backward", &pretrain_tmix_lnx_rkvres_xg_backward);
  m.def("recurrent_add_vec_forward_varlen", &recurrent_add_vec_forward_varlen, py::arg("x"), py::arg("vec"));
  m.def("tmix_act_forward", &tmix_act_forward, py::arg("x"), py::arg("act"));
  m.def("tmix_linear_runtime_layout", &linear_runtime_layout, py::arg("x"), py::arg("weight_kn"), py::arg("act") = 0,
        py::arg("vres") = py::none());
  m.def("tmix_linear_forward_varlen", &ref_linear_forward, py::arg("x"), py::arg("weight"),
        py::arg("weight_is_transposed") = false);
  m.def("tmix_linear_attention_c2c_forward_varlen", &ref_linear_c2c, py::arg("x"), py::arg("weight"));
  m.def("tmix_linear_ffn_key_forward_varlen", &ref_linear_c2c, py::arg("x"), py::arg("weight"));
  m.def("tmix_linear_t_forward_varlen", &ref_linear_t, py::arg("x"), py::arg("weight_t"));
  m.def("tmix_linear_t_tanh_forward_varlen", &ref_linear_t_tanh, py::arg("x"), py::arg("weight_t"));
  m.def("tmix_linear_t_sigmoid_forward_varlen", &ref_linear_t_sigmoid, py::arg("x"), py::arg("weight_t"));
  m.def("tmix_linear_act_tanh_forward_varlen", &ref_act_tanh, py::arg("x"));
  m.def("tmix_linear_act_sigmoid_forward_varlen", &ref_act_sigmoid, py::arg("x"));
  m.def("tmix_linear_t_vres_forward_varlen", &ref_linear_t_vres, py::arg("x"), py::arg("weight_t"), py::arg("v"),
        py::arg("v_first"), py::arg("v0"));
  m.def("tmix_linear_rank_in_dispatch_forward_varlen", &ref_rank_dispatch, py::arg("x"), py::arg("weight") = py::none(),
        py::arg("weight_t") = py::none());
  m.def("tmix_linear_rank_out_dispatch_forward_varlen", &ref_rank_dispatch, py::arg("x"), py::arg("weight") = py::none(),
        py::arg("weight_t") = py::none());
  m.def("tmix_lowrank_in_forward_varlen", &ref_lowrank_in, py::arg("x_w"), py::arg("x_a"), py::arg("x_g"),
        py::arg("w1_t") = py::none(), py::arg("a1_t") = py::none(), py::arg("g1_t") = py::none(),
        py::arg("w1") = py::none(), py::arg("a1") = py::none(), py::arg("g1") = py::none());
  m.def("tmix_lowrank_wagv_in_forward_varlen", &ref_lowrank_wagv_in, py::arg("x_w"), py::arg("x_a"), py::arg("x_g"),
        py::arg("x_v"), py::arg("w1_t") = py::none(), py::arg("a1_t") = py::none(), py::arg("g1_t") = py::none(),
        py::arg("v1_t") = py::none(), py::arg("w1") = py::none(), py::arg("a1") = py::none(),
        py::arg("g1") = py::none(), py::arg("v1") = py::none());
  m.def("tmix_lowrank_out_forward_varlen", &ref_lowrank_out, py::arg("w1"), py::arg("a1"), py::arg("g1"),
        py::arg("w2_t") = py::none(), py::arg("a2_t") = py::none(), py::arg("g2_t") = py::none(),
        py::arg("w2") = py::none(), py::arg("a2") = py::none(), py::arg("g2") = py::none());
  m.def("tmix_lowrank_vres_forward_varlen", &ref_lowrank_vres, py::arg("w1"), py::arg("a1"), py::arg("g1"),
        py::arg("v1"), py::arg("w2_t"), py::arg("a2_t"), py::arg("g2_t"), py::arg("v2_t"), py::arg("w2"), py::arg("a2"),
        py::arg("g2"), py::arg("v2"), py::arg("v"), py::arg("v_first"), py::arg("v0"));
  m.def("tmix_linear_grouped", &tmix_linear_grouped, py::arg("xs"), py::arg("weights"), py::arg("acts"),
        py::arg("vres") = py::none());
}

TORCH_LIBRARY(rwkv7_clampw_v3, m) {
  m.def("forward", clampw_forward);
  m.def("backward", clampw_backward);
}
