// Expert-parallel token exchange by direct stores into peer memory over NVLink: the dispatch
// (token permute) writes every routed row straight into the receive buffer of the rank that
// owns its expert, and the return trip writes every computed row straight back to its slot
// on the token's home rank.  No kernel here waits for another rank: the only cross-rank
// ordering is a stream-ordered collective the host issues between the stages, so these are
// plain grid launches over local indices with peer pointers as store targets.
//
// The reference has no counterpart (it replicates tokens and all-reduces,
// crates/nml-ir/src/lib.rs:9596-9728); an NCCL all-to-all-v needs its split sizes on the
// host, which costs a device-to-host synchronisation per layer that this path avoids.
//
// Row placement is a pure function of the count matrix C[r][d] (rows rank r sends to rank d,
// all-gathered on the device): rank r's rows for d land at [sum_{r' < r} C[r'][d], ...) in
// d's buffer, in r's send order, so the layout is deterministic.
#include "common.cuh"

namespace nml_sm100 {
namespace {

constexpr int kMaxRanks = NML_SM100_EP_MAX_RANKS;

struct PeerTable {
  void* rows[kMaxRanks];     // receive buffers [capacity, width] (push) / return buffers (return)
  int32_t* meta[kMaxRanks];  // [capacity, 4]: local expert, weight bits, origin rank, origin slot
};

// One block per send slot.  Slots are grouped by destination in rank order (the layout of
// ep_dispatch_plan), so the destination of slot s follows from the prefix of send_counts.
template <typename T>
__global__ void __launch_bounds__(128)
ep_push_rows_kernel(const T* __restrict__ source, const int32_t* __restrict__ send_order,
                    const int32_t* __restrict__ local_expert,
                    const uint16_t* __restrict__ routing_weights,
                    const int32_t* __restrict__ send_counts,
                    const int32_t* __restrict__ count_matrix, PeerTable peers, int assignments,
                    int source_rows, int top_k, int vectors, int ranks, int rank, int capacity,
                    int* status) {
  const int slot = blockIdx.x;
  const int32_t assignment = send_order[slot];
  if (assignment < 0 || assignment >= assignments) return;  // tail of the send arrays
  int destination = -1, first = 0;
  for (int d = 0; d < ranks; ++d) {
    const int count = send_counts[d];
    if (slot < first + count) {
      destination = d;
      break;
    }
    first += count;
  }
  if (destination < 0) return;
  int base = 0;
  for (int r = 0; r < rank; ++r) base += count_matrix[r * ranks + destination];
  const int position = base + (slot - first);
  const int source_row = assignment / top_k;
  if (position < 0 || position >= capacity || source_row >= source_rows) {
    if (threadIdx.x == 0) atomicOr(status, NML_SM100_STATUS_INDEX_RANGE);
    return;
  }
  const uint4* from = reinterpret_cast<const uint4*>(source) +
                      static_cast<int64_t>(source_row) * vectors;
  uint4* to = reinterpret_cast<uint4*>(peers.rows[destination]) +
              static_cast<int64_t>(position) * vectors;
  for (int v = threadIdx.x; v < vectors; v += blockDim.x) to[v] = from[v];
  if (threadIdx.x == 0) {
    int4 meta;
    meta.x = local_expert[slot];
    meta.y = routing_weights[assignment];
    meta.z = rank;
    meta.w = slot;
    reinterpret_cast<int4*>(peers.meta[destination])[position] = meta;
  }
}

// After the exchange: expert ids and routing weights of the received rows in the form the
// routed layer takes (k = 1); rows past the received count are masked with id -1.
template <typename T>
__global__ void __launch_bounds__(256)
ep_receive_meta_kernel(const int32_t* __restrict__ meta, const int32_t* __restrict__ count_matrix,
                       int32_t* __restrict__ expert_ids, T* __restrict__ weights,
                       int32_t* __restrict__ received, int ranks, int rank, int capacity) {
  int total = 0;
  for (int r = 0; r < ranks; ++r) total += count_matrix[r * ranks + rank];
  total = min(total, capacity);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) received[0] = total;
  if (i >= capacity) return;
  if (i < total) {
    const int4 m = reinterpret_cast<const int4*>(meta)[i];
    expert_ids[i] = m.x;
    reinterpret_cast<uint16_t*>(weights)[i] = static_cast<uint16_t>(m.y);
  } else {
    expert_ids[i] = -1;
    reinterpret_cast<uint16_t*>(weights)[i] = 0;
  }
}

// One block per received row: computed[i] goes to slot meta[i].w of rank meta[i].z.
template <typename T>
__global__ void __launch_bounds__(128)
ep_return_rows_kernel(const T* __restrict__ computed, const int32_t* __restrict__ meta,
                      const int32_t* __restrict__ count_matrix, PeerTable peers, int vectors,
                      int ranks, int rank, int capacity, int return_capacity, int* status) {
  int total = 0;
  for (int r = 0; r < ranks; ++r) total += count_matrix[r * ranks + rank];
  const int i = blockIdx.x;
  if (i >= total || i >= capacity) return;
  const int4 m = reinterpret_cast<const int4*>(meta)[i];
  if (m.z < 0 || m.z >= ranks || m.w < 0 || m.w >= return_capacity) {
    if (threadIdx.x == 0) atomicOr(status, NML_SM100_STATUS_INDEX_RANGE);
    return;
  }
  const uint4* from = reinterpret_cast<const uint4*>(computed) + static_cast<int64_t>(i) * vectors;
  uint4* to = reinterpret_cast<uint4*>(peers.rows[m.z]) + static_cast<int64_t>(m.w) * vectors;
  for (int v = threadIdx.x; v < vectors; v += blockDim.x) to[v] = from[v];
}

}  // namespace

int32_t launch_ep_push_rows(const NmlSm100EpPushRows& q, const DeviceInfo& device, char* message,
                            size_t capacity) {
  PeerTable peers = {};
  for (int r = 0; r < q.ranks; ++r) {
    peers.rows[r] = q.peer_rows[r];
    peers.meta[r] = q.peer_meta[r];
  }
  const int vectors = static_cast<int>(q.width / 8);
  cudaStream_t stream = static_cast<cudaStream_t>(q.stream);
  const unsigned grid = static_cast<unsigned>(q.assignments);
  const uint16_t* weights = static_cast<const uint16_t*>(q.routing_weights);
  if (q.dtype == NML_SM100_F16) {
    ep_push_rows_kernel<__half><<<grid, 128, 0, stream>>>(
        static_cast<const __half*>(q.source), q.send_order, q.local_expert, weights, q.send_counts,
        q.count_matrix, peers, static_cast<int>(q.assignments), static_cast<int>(q.source_rows),
        static_cast<int>(q.experts_per_token), vectors, static_cast<int>(q.ranks),
        static_cast<int>(q.rank), static_cast<int>(q.capacity), device.status_word);
  } else {
    ep_push_rows_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q.source), q.send_order, q.local_expert, weights,
        q.send_counts, q.count_matrix, peers, static_cast<int>(q.assignments),
        static_cast<int>(q.source_rows), static_cast<int>(q.experts_per_token), vectors,
        static_cast<int>(q.ranks), static_cast<int>(q.rank), static_cast<int>(q.capacity),
        device.status_word);
  }
  return launch_result(message, capacity);
}

int32_t launch_ep_receive_meta(const NmlSm100EpReceiveMeta& q, char* message, size_t capacity) {
  cudaStream_t stream = static_cast<cudaStream_t>(q.stream);
  const unsigned grid = static_cast<unsigned>((q.capacity + 255) / 256);
  if (q.dtype == NML_SM100_F16) {
    ep_receive_meta_kernel<__half><<<grid, 256, 0, stream>>>(
        q.meta, q.count_matrix, q.expert_ids, static_cast<__half*>(q.routing_weights), q.received,
        static_cast<int>(q.ranks), static_cast<int>(q.rank), static_cast<int>(q.capacity));
  } else {
    ep_receive_meta_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        q.meta, q.count_matrix, q.expert_ids, static_cast<__nv_bfloat16*>(q.routing_weights),
        q.received, static_cast<int>(q.ranks), static_cast<int>(q.rank),
        static_cast<int>(q.capacity));
  }
  return launch_result(message, capacity);
}

int32_t launch_ep_return_rows(const NmlSm100EpReturnRows& q, const DeviceInfo& device,
                              char* message, size_t capacity) {
  PeerTable peers = {};
  for (int r = 0; r < q.ranks; ++r) peers.rows[r] = q.peer_return[r];
  const int vectors = static_cast<int>(q.width / 8);
  cudaStream_t stream = static_cast<cudaStream_t>(q.stream);
  const unsigned grid = static_cast<unsigned>(q.capacity);
  if (q.dtype == NML_SM100_F16) {
    ep_return_rows_kernel<__half><<<grid, 128, 0, stream>>>(
        static_cast<const __half*>(q.computed), q.meta, q.count_matrix, peers, vectors,
        static_cast<int>(q.ranks), static_cast<int>(q.rank), static_cast<int>(q.capacity),
        static_cast<int>(q.return_capacity), device.status_word);
  } else {
    ep_return_rows_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q.computed), q.meta, q.count_matrix, peers, vectors,
        static_cast<int>(q.ranks), static_cast<int>(q.rank), static_cast<int>(q.capacity),
        static_cast<int>(q.return_capacity), device.status_word);
  }
  return launch_result(message, capacity);
}

}  // namespace nml_sm100
