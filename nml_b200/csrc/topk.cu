// Row-wise top-k of 16-bit logits: the per-shard half of the sampler-side reduction over a
// column-sharded vocabulary projection (the reference plans a global top-k merge for its
// column-sharded head, PRODUCT.md:673-674).  Only k (value, index) pairs per row leave a rank
// instead of its whole slice of the logits.  Larger values first; equal values go to the
// lower index, so the result does not depend on how columns are cut into chunks or shards.
//
// Pass 1: one CTA per (row, chunk of 8192 columns); every thread holds 32 logits in registers
// and the best of them; the CTA runs k rounds of arg-max over the threads' bests (warp
// shuffles, then one shared-memory step across the warps), and the winner's owner retires it
// and finds its next best.  Pass 2: one warp per row does the same k rounds over
// the chunks' candidates.  Integer/compare work on top of one read of the logits.
#include "common.cuh"

namespace nml_sm100 {
namespace {

constexpr int kThreads = 256;
constexpr int kPerThread = 32;
constexpr int kChunk = kThreads * kPerThread;  // 8192 columns
constexpr int kMaxK = 16;

struct Candidate {
  float value;
  int index;
};

__device__ __forceinline__ bool better(float value, int index, float than_value, int than_index) {
  return value > than_value || (value == than_value && index < than_index);
}

__device__ __forceinline__ Candidate warp_best(Candidate mine) {
#pragma unroll
  for (int offset = 16; offset != 0; offset >>= 1) {
    const float other_value = __shfl_xor_sync(0xffffffffu, mine.value, offset);
    const int other_index = __shfl_xor_sync(0xffffffffu, mine.index, offset);
    if (better(other_value, other_index, mine.value, mine.index)) {
      mine.value = other_value;
      mine.index = other_index;
    }
  }
  return mine;
}

constexpr int kNoIndex = 0x7fffffff;

template <typename T>
__global__ void __launch_bounds__(kThreads)
topk_chunk_kernel(const T* __restrict__ logits, Candidate* __restrict__ partial, int columns,
                  int64_t row_stride, int chunks, int k) {
  const int chunk = blockIdx.x;
  const int row = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __shared__ Candidate warp_winner[kThreads / 32];
  __shared__ Candidate winner;
  // thread t holds columns chunk * 8192 + 8 * (t + 256 j) + e, j < 4, e < 8
  float held[kPerThread];
  const T* base = logits + static_cast<int64_t>(row) * row_stride;
  const bool vector_ok = (reinterpret_cast<uintptr_t>(base) % 16 == 0);
#pragma unroll
  for (int j = 0; j < kPerThread / 8; ++j) {
    const int column0 = chunk * kChunk + 8 * (threadIdx.x + kThreads * j);
    if (vector_ok && column0 + 8 <= columns) {
      const uint4 v = *reinterpret_cast<const uint4*>(base + column0);
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        held[8 * j + 2 * e] = Elem<T>::from_bits(words[e] & 0xffffu);
        held[8 * j + 2 * e + 1] = Elem<T>::from_bits(words[e] >> 16);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        held[8 * j + e] = column0 + e < columns ? Elem<T>::load(base[column0 + e]) : -INFINITY;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    if (!(held[i] == held[i])) held[i] = -INFINITY;  // NaN never wins
  }
  // Every thread keeps the best of its own 32 values; a round reduces those over the CTA, and
  // only the thread that owned the winner retires it and looks through its values again.
  auto best_held = [&]() {
    Candidate best = {-INFINITY, kNoIndex};
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int column = chunk * kChunk + 8 * (threadIdx.x + kThreads * (i / 8)) + (i % 8);
      if (column < columns && better(held[i], column, best.value, best.index)) {
        best.value = held[i];
        best.index = column;
      }
    }
    return best;
  };
  Candidate mine = best_held();
  for (int round = 0; round < k; ++round) {
    const Candidate in_warp = warp_best(mine);
    if (lane == 0) warp_winner[warp] = in_warp;
    __syncthreads();
    if (warp == 0) {
      Candidate best = lane < kThreads / 32 ? warp_winner[lane] : Candidate{-INFINITY, kNoIndex};
      best = warp_best(best);
      if (lane == 0) {
        winner = best;
        partial[(static_cast<int64_t>(row) * chunks + chunk) * k + round] = best;
      }
    }
    __syncthreads();
    const int taken = winner.index;
    if (taken != kNoIndex && taken == mine.index) {
      // retire the winner: NaN loses every later comparison
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        const int column = chunk * kChunk + 8 * (threadIdx.x + kThreads * (i / 8)) + (i % 8);
        if (column == taken) held[i] = __int_as_float(0xffc00000);
      }
      mine = best_held();
    }
  }
}

// One warp per row: k rounds of arg-max over the chunks' candidates.
__global__ void __launch_bounds__(32)
topk_merge_kernel(const Candidate* __restrict__ partial, float* __restrict__ values,
                  int32_t* __restrict__ indices, int chunks, int k, int index_offset) {
  const int row = blockIdx.x;
  const int lane = threadIdx.x;
  const int total = chunks * k;
  const Candidate* mine = partial + static_cast<int64_t>(row) * total;
  constexpr int kHeld = 16;  // up to 512 candidates per row
  Candidate held[kHeld];
#pragma unroll
  for (int i = 0; i < kHeld; ++i) {
    const int at = lane + 32 * i;
    held[i] = at < total ? mine[at] : Candidate{-INFINITY, kNoIndex};
  }
  for (int round = 0; round < k; ++round) {
    Candidate best = {-INFINITY, kNoIndex};
    int slot = -1;
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      if (held[i].index != kNoIndex && better(held[i].value, held[i].index, best.value, best.index)) {
        best = held[i];
        slot = i;
      }
    }
    const Candidate winner = warp_best(best);
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      if (i == slot && best.index == winner.index) held[i].index = kNoIndex;  // retired
    }
    if (lane == 0) {
      values[static_cast<int64_t>(row) * k + round] = winner.value;
      indices[static_cast<int64_t>(row) * k + round] =
          winner.index == kNoIndex ? -1 : winner.index + index_offset;
    }
  }
}

// One warp per row: the k best of the parts' candidates, same order as above.
__global__ void __launch_bounds__(32)
topk_merge_parts_kernel(const float* __restrict__ values, const int32_t* __restrict__ indices,
                        float* __restrict__ out_values, int32_t* __restrict__ out_indices,
                        int parts, int rows, int64_t pitch, int k) {
  const int row = blockIdx.x;
  const int lane = threadIdx.x;
  const int total = parts * k;
  constexpr int kHeld = 16;  // up to 512 candidates per row
  Candidate held[kHeld];
#pragma unroll
  for (int i = 0; i < kHeld; ++i) {
    const int at = lane + 32 * i;
    held[i] = Candidate{-INFINITY, kNoIndex};
    if (at < total) {
      const int part = at / k, j = at - part * k;
      const int64_t from = (static_cast<int64_t>(part) * rows + row) * pitch + j;
      const int32_t index = indices[from];
      const float value = values[from];
      if (index >= 0 && value == value) held[i] = Candidate{value, index};
    }
  }
  for (int round = 0; round < k; ++round) {
    Candidate best = {-INFINITY, kNoIndex};
    int slot = -1;
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      if (held[i].index != kNoIndex && better(held[i].value, held[i].index, best.value, best.index)) {
        best = held[i];
        slot = i;
      }
    }
    const Candidate winner = warp_best(best);
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      if (i == slot && best.index == winner.index) held[i].index = kNoIndex;  // retired
    }
    if (lane == 0) {
      out_values[static_cast<int64_t>(row) * k + round] = winner.value;
      out_indices[static_cast<int64_t>(row) * k + round] =
          winner.index == kNoIndex ? -1 : winner.index;
    }
  }
}

}  // namespace
}  // namespace nml_sm100

using namespace nml_sm100;

extern "C" int32_t nml_nvfp4_sm100_topk_merge(const NmlSm100TopkMerge* request,
                                              char* error_message,
                                              size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100TopkMerge)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated top-k merge request", error_message,
                error_message_capacity);
  }
  const NmlSm100TopkMerge& r = *request;
  if (r.values == nullptr || r.indices == nullptr || r.out_values == nullptr ||
      r.out_indices == nullptr || r.stream == nullptr || r.parts <= 0 || !fits_i32(r.rows) ||
      r.rows > 0x7fffffff || r.k <= 0 || r.k > kMaxK || r.pitch < r.k || r.parts * r.k > 512) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid top-k merge request", error_message,
                error_message_capacity);
  }
  if (current_device(error_message, error_message_capacity) == nullptr) {
    return NML_SM100_LAUNCH_FAILURE;
  }
  topk_merge_parts_kernel<<<static_cast<unsigned>(r.rows), 32, 0,
                            static_cast<cudaStream_t>(r.stream)>>>(
      r.values, r.indices, r.out_values, r.out_indices, static_cast<int>(r.parts),
      static_cast<int>(r.rows), r.pitch, static_cast<int>(r.k));
  return launch_result(error_message, error_message_capacity);
}

extern "C" size_t nml_nvfp4_sm100_topk_rows_workspace_bytes(int64_t rows, int64_t columns,
                                                            int64_t k) {
  if (rows <= 0 || columns <= 0 || k <= 0) return 0;
  const int64_t chunks = (columns + kChunk - 1) / kChunk;
  return static_cast<size_t>(rows * chunks * k) * sizeof(Candidate);
}

extern "C" int32_t nml_nvfp4_sm100_topk_rows(const NmlSm100TopkRows* request, char* error_message,
                                             size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100TopkRows)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated top-k request", error_message,
                error_message_capacity);
  }
  const NmlSm100TopkRows& r = *request;
  const int64_t chunks = (r.columns + kChunk - 1) / kChunk;
  if (r.logits == nullptr || r.values == nullptr || r.indices == nullptr ||
      r.workspace == nullptr || r.stream == nullptr || !fits_i32(r.rows) || r.rows > 65535 ||
      !fits_i32(r.columns) || r.k <= 0 || r.k > kMaxK || r.k > r.columns ||
      r.row_stride < r.columns || chunks * r.k > 512 ||
      r.workspace_bytes < nml_nvfp4_sm100_topk_rows_workspace_bytes(r.rows, r.columns, r.k) ||
      reinterpret_cast<uintptr_t>(r.workspace) % 8 != 0) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid top-k request", error_message,
                error_message_capacity);
  }
  if (r.dtype != NML_SM100_F16 && r.dtype != NML_SM100_BF16) {
    return fail(NML_SM100_INVALID_ARGUMENT, "top-k supports F16 and BF16 logits only",
                error_message, error_message_capacity);
  }
  if (current_device(error_message, error_message_capacity) == nullptr) {
    return NML_SM100_LAUNCH_FAILURE;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(r.stream);
  Candidate* partial = static_cast<Candidate*>(r.workspace);
  const dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(r.rows));
  if (r.dtype == NML_SM100_F16) {
    topk_chunk_kernel<__half><<<grid, kThreads, 0, stream>>>(
        static_cast<const __half*>(r.logits), partial, static_cast<int>(r.columns), r.row_stride,
        static_cast<int>(chunks), static_cast<int>(r.k));
  } else {
    topk_chunk_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(r.logits), partial, static_cast<int>(r.columns),
        r.row_stride, static_cast<int>(chunks), static_cast<int>(r.k));
  }
  topk_merge_kernel<<<static_cast<unsigned>(r.rows), 32, 0, stream>>>(
      partial, r.values, r.indices, static_cast<int>(chunks), static_cast<int>(r.k),
      r.index_offset);
  return launch_result(error_message, error_message_capacity);
}
