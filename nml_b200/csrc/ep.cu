// Expert-parallel token exchange support: the destination plan of routed assignments, the
// row gather that builds the send buffer (token permute) and the indexed k-way sum that
// brings returned rows home (unpermute + combine).  Integer and byte work, HBM-bound.
//
// The reference shards experts by replicating every token on every device and summing
// partial outputs with one all-reduce (crates/nml-ir/src/lib.rs:9596-9728).  Here tokens stay
// sharded: each assignment travels to the device that owns its expert and back, so a device
// only computes and communicates the rows routed to it.
#include "common.cuh"

namespace nml_sm100 {
namespace {

// Single CTA.  Destination of assignment a is expert_ids[a] / experts_per_rank; assignments
// with a negative id (masked routes) have no destination.  Send slots are grouped by
// destination in rank order and keep assignment order inside a destination, so the plan is a
// pure function of the ids (deterministic, the same on every run).
__global__ void __launch_bounds__(1024)
ep_dispatch_plan_kernel(const int32_t* __restrict__ expert_ids, int32_t* __restrict__ send_order,
                        int32_t* __restrict__ slot_of_assignment,
                        int32_t* __restrict__ local_expert, int32_t* __restrict__ send_counts,
                        int assignments, int ranks, int experts_per_rank) {
  extern __shared__ int32_t ep_smem[];
  const int threads = blockDim.x;
  const int t = threadIdx.x;
  int32_t* hist = ep_smem;                  // [ranks][threads]
  int32_t* totals = hist + ranks * threads; // [ranks]
  int32_t* prefix = totals + ranks;         // [ranks + 1]
  for (int i = t; i < ranks * threads; i += threads) hist[i] = 0;
  __syncthreads();
  const int chunk = (assignments + threads - 1) / threads;
  const int begin = min(assignments, t * chunk);
  const int end = min(assignments, begin + chunk);
  for (int a = begin; a < end; ++a) {
    const int32_t id = expert_ids[a];
    const int32_t destination = id >= 0 ? id / experts_per_rank : -1;
    if (destination >= 0 && destination < ranks) hist[destination * threads + t] += 1;
  }
  __syncthreads();
  const int lane = t & 31, warp = t >> 5, warps = threads >> 5;
  for (int r = warp; r < ranks; r += warps) {
    int32_t running = 0;
    for (int base = 0; base < threads; base += 32) {
      const int32_t value = hist[r * threads + base + lane];
      int32_t inclusive = value;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const int32_t other = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (lane >= offset) inclusive += other;
      }
      hist[r * threads + base + lane] = running + inclusive - value;
      running += __shfl_sync(0xffffffffu, inclusive, 31);
    }
    if (lane == 0) totals[r] = running;
  }
  __syncthreads();
  if (t == 0) {
    int32_t start = 0;
    for (int r = 0; r < ranks; ++r) {
      prefix[r] = start;
      send_counts[r] = totals[r];
      start += totals[r];
    }
    prefix[ranks] = start;
  }
  __syncthreads();
  // Unused tail of the send arrays (masked routes shrink the total).
  for (int i = prefix[ranks] + t; i < assignments; i += threads) {
    send_order[i] = -1;
    local_expert[i] = -1;
  }
  for (int a = begin; a < end; ++a) {
    const int32_t id = expert_ids[a];
    const int32_t destination = id >= 0 ? id / experts_per_rank : -1;
    if (destination >= 0 && destination < ranks) {
      const int32_t slot = prefix[destination] + hist[destination * threads + t]++;
      send_order[slot] = a;
      local_expert[slot] = id - destination * experts_per_rank;
      slot_of_assignment[a] = slot;
    } else {
      slot_of_assignment[a] = -1;
    }
  }
}

// output[r, :] = source[row_index[r] / divisor, :]; a negative index yields a zero row.  With
// `live_blocks`, rows at or past 16 * live_blocks[0] are left untouched (schedule positions
// behind the active blocks, which no consumer reads).
template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ source, const int32_t* __restrict__ row_index,
                   T* __restrict__ output, int64_t rows, int vectors, int divisor,
                   int64_t source_rows, const int32_t* __restrict__ live_blocks) {
  const int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= rows * vectors) return;
  const int64_t row = item / vectors;
  if (live_blocks != nullptr && row >= static_cast<int64_t>(live_blocks[0]) * 16) return;
  const int vector = static_cast<int>(item - row * vectors);
  const int32_t index = row_index[row];
  uint4 value = make_uint4(0, 0, 0, 0);
  if (index >= 0) {
    const int64_t source_row = index / divisor;
    if (source_row < source_rows) {
      value = reinterpret_cast<const uint4*>(source)[source_row * vectors + vector];
    }
  }
  reinterpret_cast<uint4*>(output)[item] = value;
}

// output[t, :] = sum over routes r, in route order, of rows[row_index[t * k + r], :] (f32,
// one narrowing); routes with a negative index are skipped.
template <typename T>
__global__ void __launch_bounds__(256)
combine_rows_kernel(const T* __restrict__ rows, const int32_t* __restrict__ row_index,
                    T* __restrict__ output, int tokens, int top_k, int vectors,
                    int64_t row_count) {
  const int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= static_cast<int64_t>(tokens) * vectors) return;
  combine_rows_item<T>(rows, row_index, output, item, top_k, vectors, row_count);
}

}  // namespace

int32_t launch_ep_dispatch_plan(const int32_t* expert_ids, int32_t* send_order,
                                int32_t* slot_of_assignment, int32_t* local_expert,
                                int32_t* send_counts, int assignments, int ranks,
                                int experts_per_rank, cudaStream_t stream, char* message,
                                size_t capacity) {
  int threads = 1024;
  while (threads > 32 && static_cast<int64_t>(threads) * ranks > 8192) threads >>= 1;
  const size_t smem = (static_cast<size_t>(threads) * ranks + 2 * ranks + 2) * 4;
  ep_dispatch_plan_kernel<<<1, threads, smem, stream>>>(expert_ids, send_order,
                                                        slot_of_assignment, local_expert,
                                                        send_counts, assignments, ranks,
                                                        experts_per_rank);
  return launch_result(message, capacity);
}

int32_t launch_gather_rows(const void* source, const int32_t* row_index, void* output,
                           int64_t rows, int width, int divisor, int64_t source_rows, int dtype,
                           cudaStream_t stream, char* message, size_t capacity,
                           const int32_t* live_blocks) {
  const int vectors = width / 8;
  const int64_t grid = (rows * vectors + 255) / 256;
  if (grid > std::numeric_limits<int32_t>::max()) {
    return fail(NML_SM100_INVALID_ARGUMENT, "row gather launch extent overflows", message,
                capacity);
  }
  if (dtype == NML_SM100_F16) {
    gather_rows_kernel<__half><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<const __half*>(source), row_index, static_cast<__half*>(output), rows,
        vectors, divisor, source_rows, live_blocks);
  } else {
    gather_rows_kernel<__nv_bfloat16><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(source), row_index,
        static_cast<__nv_bfloat16*>(output), rows, vectors, divisor, source_rows, live_blocks);
  }
  return launch_result(message, capacity);
}

int32_t launch_combine_rows(const void* rows, const int32_t* row_index, void* output, int tokens,
                            int top_k, int width, int64_t row_count, int dtype,
                            cudaStream_t stream, char* message, size_t capacity) {
  const int vectors = width / 8;
  const int64_t grid = (static_cast<int64_t>(tokens) * vectors + 255) / 256;
  if (grid > std::numeric_limits<int32_t>::max()) {
    return fail(NML_SM100_INVALID_ARGUMENT, "row combine launch extent overflows", message,
                capacity);
  }
  if (dtype == NML_SM100_F16) {
    combine_rows_kernel<__half><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<const __half*>(rows), row_index, static_cast<__half*>(output), tokens, top_k,
        vectors, row_count);
  } else {
    combine_rows_kernel<__nv_bfloat16><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(rows), row_index, static_cast<__nv_bfloat16*>(output),
        tokens, top_k, vectors, row_count);
  }
  return launch_result(message, capacity);
}

}  // namespace nml_sm100
