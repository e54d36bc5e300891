// Device-side validation of packed-sequence metadata.
//
// Two launches on the caller's stream: the first snapshots cu_seqlens and
// state_indices and clears the status words; the second validates the SNAPSHOT
// (so a caller that mutates its tensors afterwards cannot invalidate what the
// consumers read) and ORs error bits into status[0], the longest sequence into
// status[1].  The duplicate-slot scan is quadratic like the reference's but is
// spread over many blocks instead of one.
//
// Replaces validate_recurrent_metadata_kernel of the reference
// (csrc/validation/recurrent_metadata.cu:22-97).

#include "frwkv_common.cuh"

namespace frwkv {
namespace {

__global__ void snapshot_metadata_kernel(const int* __restrict__ cu, const int* __restrict__ idx, int n,
                                         int* __restrict__ status, int* __restrict__ cu_snap,
                                         int* __restrict__ idx_snap) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) idx_snap[i] = idx[i];
  if (i <= n) cu_snap[i] = cu[i];
  if (i == 0) {
    status[0] = 0;
    status[1] = 0;
  }
}

__global__ void validate_metadata_kernel(const int* __restrict__ cu, const int* __restrict__ idx, int n,
                                         int total_tokens, int pool_size, int* __restrict__ status) {
  __shared__ int s_error;
  __shared__ int s_maxlen;
  if (threadIdx.x == 0) {
    s_error = 0;
    s_maxlen = 0;
  }
  __syncthreads();
  int error = 0, maxlen = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    if (i == 0 && (cu[0] != 0 || cu[n] != total_tokens)) error |= FRWKV_META_INVALID_ENDPOINT;
    const int t0 = cu[i], t1 = cu[i + 1];
    if (t0 < 0 || t1 <= t0 || t1 > total_tokens) {
      error |= FRWKV_META_INVALID_RANGE;
    } else {
      maxlen = max(maxlen, t1 - t0);
    }
    const int slot = idx[i];
    if (slot < 0 || slot >= pool_size) {
      error |= FRWKV_META_INVALID_SLOT;
    } else {
      for (int e = 0; e < i; ++e) {
        if (idx[e] == slot) {
          error |= FRWKV_META_DUPLICATE_SLOT;
          break;
        }
      }
    }
  }
  if (error) atomicOr(&s_error, error);
  atomicMax(&s_maxlen, maxlen);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_error) atomicOr(&status[0], s_error);
    atomicMax(&status[1], s_maxlen);
  }
}

// Chunk tables of the training operators: status[0] receives FRWKV_META_* bits when a chunk lies outside [0, N], holds
// more than max_chunk tokens, does not follow its predecessor in the same sequence, or the offsets do not rise from 0
// to the chunk count.  status[0] must be zero beforehand (the launcher clears it).
__global__ void validate_chunk_tables_kernel(const int* __restrict__ sco, const int* __restrict__ cs,
                                             const int* __restrict__ ce, int num_sequences, int num_chunks,
                                             int total_tokens, int max_chunk, int* __restrict__ status) {
  int error = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < num_chunks + num_sequences; i += gridDim.x * blockDim.x) {
    if (i < num_chunks) {
      const int a = cs[i], b = ce[i];
      if (a < 0 || b < a || b > total_tokens || b - a > max_chunk) error |= FRWKV_META_INVALID_RANGE;
    } else {
      const int s = i - num_chunks;
      const int c0 = sco[s], c1 = sco[s + 1];
      if ((s == 0 && c0 != 0) || (s == num_sequences - 1 && c1 != num_chunks) || c0 < 0 || c1 < c0 || c1 > num_chunks) {
        error |= FRWKV_META_INVALID_ENDPOINT;
      } else {
        for (int c = c0 + 1; c < c1; ++c)
          if (cs[c] != ce[c - 1]) error |= FRWKV_META_INVALID_RANGE;
      }
    }
  }
  if (error) atomicOr(&status[0], error);
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_validate_chunk_tables(const int32_t* seq_chunk_offsets, const int32_t* chunk_starts,
                                           const int32_t* chunk_ends, int num_sequences, int num_chunks,
                                           int total_tokens, int max_chunk, int32_t* status, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(seq_chunk_offsets && chunk_starts && chunk_ends && status, "validate_chunk_tables: null pointer argument");
  FRWKV_REQUIRE(num_sequences > 0 && num_chunks > 0 && total_tokens > 0 && max_chunk > 0,
                "validate_chunk_tables: sizes must be positive");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int32_t), s);
  if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "validate_chunk_tables: %s", cudaGetErrorString(e));
  const int work = num_chunks + num_sequences;
  validate_chunk_tables_kernel<<<(work + 255) / 256 < 1024 ? (work + 255) / 256 : 1024, 256, 0, s>>>(
      seq_chunk_offsets, chunk_starts, chunk_ends, num_sequences, num_chunks, total_tokens, max_chunk, status);
  return check_launch("validate_chunk_tables_kernel");
}

namespace frwkv {
namespace {
// *flag stays 1 only if sequence i is token i (cu[i] == i, i = 0..n) and owns slot i (idx[i] == i, i = 0..n-1)
__global__ void metadata_is_direct_kernel(const int* __restrict__ cu, const int* __restrict__ idx, int n,
                                          int* __restrict__ flag) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  bool bad = false;
  if (i <= n) bad = cu[i] != i;
  if (i < n) bad = bad || idx[i] != i;
  if (bad) atomicExch(flag, 0);
}
__global__ void set_flag_kernel(int* __restrict__ flag) { *flag = 1; }
}  // namespace
}  // namespace frwkv

extern "C" int frwkv_recurrent_metadata_is_direct(const int32_t* cu_seqlens, const int32_t* state_indices,
                                                  int num_sequences, int32_t* flag, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(cu_seqlens && state_indices && flag, "recurrent_metadata_is_direct: null pointer argument");
  FRWKV_REQUIRE(num_sequences > 0 && num_sequences <= 65535,
                "state_indices must contain at most 65535 sequences");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  constexpr int threads = 128;
  set_flag_kernel<<<1, 1, 0, s>>>(flag);  // the flag starts as 1, ahead of the kernel that may clear it
  int rc = check_launch("set_flag_kernel");
  if (rc != FRWKV_OK) return rc;
  metadata_is_direct_kernel<<<(num_sequences + 1 + threads - 1) / threads, threads, 0, s>>>(cu_seqlens, state_indices,
                                                                                          num_sequences, flag);
  return check_launch("metadata_is_direct_kernel");
}

extern "C" int frwkv_validate_recurrent_metadata(const int32_t* cu_seqlens, const int32_t* state_indices,
                                                 int num_sequences, int total_tokens, int state_pool_size,
                                                 int32_t* status, int32_t* cu_snapshot,
                                                 int32_t* idx_snapshot, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(cu_seqlens && state_indices && status && cu_snapshot && idx_snapshot,
                "validate_recurrent_metadata: null pointer argument");
  FRWKV_REQUIRE(num_sequences > 0 && num_sequences <= 65535,
                "state_indices must contain at most 65535 sequences");
  FRWKV_REQUIRE(total_tokens > 0, "total_tokens must be positive and fit in int32");
  FRWKV_REQUIRE(state_pool_size > 0, "state_pool_size must be positive and fit in int32");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  constexpr int threads = 128;
  const int blocks = (num_sequences + 1 + threads - 1) / threads;
  snapshot_metadata_kernel<<<blocks, threads, 0, s>>>(cu_seqlens, state_indices, num_sequences, status,
                                                      cu_snapshot, idx_snapshot);
  int rc = check_launch("snapshot_metadata_kernel");
  if (rc != FRWKV_OK) return rc;
  validate_metadata_kernel<<<(num_sequences + threads - 1) / threads, threads, 0, s>>>(
      cu_snapshot, idx_snapshot, num_sequences, total_tokens, state_pool_size, status);
  return check_launch("validate_metadata_kernel");
}
