// Expert-parallel token exchange by direct stores into peer memory over NVLink, with the
// cross-rank ordering done on the device: the dispatch (token permute) writes every routed row
// straight into the receive buffer of the rank that owns its expert and then raises an arrival
// flag in that rank's memory; the owner's next kernel waits for the flags of all senders.  The
// return trip works the same way.  No host synchronisation and no library collective sits
// between the stages of a layer.
//
// The reference has no counterpart (it replicates tokens and all-reduces,
// crates/nml-ir/src/lib.rs:9596-9728).
//
// Placement needs no knowledge of what other ranks send: the receive buffer of every rank is
// cut into one region of `region_rows` rows per sender, and sender r writes its rows for
// destination d into region r of d's buffer in its own send order (the grouped order of
// ep_dispatch_plan).  region_rows is at least the sender's assignment count, so nothing can
// overflow whatever the routing.
//
// Ordering.  A kernel's blocks store rows into peer memory, fence at system scope and count
// themselves on a local counter; the block that counts last fences again and writes, into each
// peer's sync words, first its row count and then (st.release.sys) the epoch of this exchange.
// The receiving kernel reads the epoch with ld.acquire.sys in a bounded loop; a loop that runs
// out sets NML_SM100_STATUS_BARRIER_TIMEOUT, treats the sender as having sent nothing, and the
// kernel returns normally.  Epochs only grow (one per exchange), so flags are never reset.  A
// rank cannot overwrite a buffer another rank still reads: it starts the next exchange only
// after its own combine has seen the return flags of every owner, and an owner raises that
// flag only after its last read of the received rows.
//
// Waiting kernels wait for other GPUs, never for another launch on the same GPU: a rank's
// pushes depend on nothing remote, so every flag is eventually raised by a kernel that is
// already running or queued behind finite work.
#include "common.cuh"

namespace nml_sm100 {
namespace {

constexpr int kMaxRanks = NML_SM100_EP_MAX_RANKS;
// sync words of one rank: [0, R) rows sent by rank r in the current exchange, [R, 2R) epoch of
// rank r's completed push, [2R, 3R) epoch of rank r's completed return (R = kMaxRanks)
constexpr int kCountWords = 0;
constexpr int kArrivedWords = kMaxRanks;
constexpr int kReturnedWords = 2 * kMaxRanks;
// local state words of one rank: epoch of the last exchange this rank started, block counters
constexpr int kEpochWord = 0;
constexpr int kPushDoneWord = 1;
constexpr int kReturnDoneWord = 2;

struct Exchange {
  void* rows[kMaxRanks];
  int32_t* meta[kMaxRanks];
  void* back[kMaxRanks];
  int32_t* sync[kMaxRanks];
  int32_t* local_state;
  int ranks, rank, region_rows, vectors;
};

Exchange make_exchange(const NmlSm100EpExchange& e) {
  Exchange x = {};
  for (int r = 0; r < e.ranks; ++r) {
    x.rows[r] = e.peer_rows[r];
    x.meta[r] = e.peer_meta[r];
    x.back[r] = e.peer_back[r];
    x.sync[r] = e.peer_sync[r];
  }
  x.local_state = e.local_state;
  x.ranks = static_cast<int>(e.ranks);
  x.rank = static_cast<int>(e.rank);
  x.region_rows = static_cast<int>(e.region_rows);
  x.vectors = static_cast<int>(e.width / 8);
  return x;
}

__device__ __forceinline__ void store_release_system(int32_t* address, int32_t value) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}

__device__ __forceinline__ int32_t load_acquire_system(const int32_t* address) {
  int32_t value;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
  return value;
}

// A warp copies one row of `vectors` 16-byte words.  The loads of a pass are issued before its
// stores so that up to eight are in flight per lane: a row is a few hundred words, and a
// load-store loop would pay the memory latency once per 32 of them.
__device__ __forceinline__ void copy_row(uint4* __restrict__ to, const uint4* __restrict__ from,
                                         int vectors, int lane) {
  constexpr int kInFlight = 8;
  for (int base = lane; base < vectors; base += 32 * kInFlight) {
    uint4 held[kInFlight];
#pragma unroll
    for (int j = 0; j < kInFlight; ++j) {
      const int v = base + 32 * j;
      if (v < vectors) held[j] = from[v];
    }
#pragma unroll
    for (int j = 0; j < kInFlight; ++j) {
      const int v = base + 32 * j;
      if (v < vectors) to[v] = held[j];
    }
  }
}

// Counts this block on `counter`; true in exactly one block, the one that counted last, and
// only after every other block's earlier stores are ordered before whatever it does next.
__device__ __forceinline__ bool last_block_done(int32_t* counter) {
  __shared__ int last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int previous = atomicAdd(counter, 1);
    last = previous == static_cast<int>(gridDim.x) - 1 ? 1 : 0;
    if (last) *counter = 0;  // ready for the next launch (stream-ordered)
  }
  __syncthreads();
  if (last) __threadfence_system();
  return last != 0;
}

// Waits until word[r] has reached `epoch` for every r < ranks; threads r < ranks poll.  Sets
// bit r of the result for a sender whose flag did not arrive within `limit` polls.
__device__ __forceinline__ unsigned wait_for_epoch(const int32_t* words, int ranks, int epoch,
                                                   int64_t limit, int* status) {
  __shared__ unsigned missing;
  if (threadIdx.x == 0) missing = 0u;
  __syncthreads();
  if (threadIdx.x < ranks) {
    bool seen = false;
    for (int64_t poll = 0; poll < limit; ++poll) {
      if (load_acquire_system(words + threadIdx.x) - epoch >= 0) {
        seen = true;
        break;
      }
      __nanosleep(200);
    }
    if (!seen) {
      atomicOr(&missing, 1u << threadIdx.x);
      atomicOr(status, NML_SM100_STATUS_BARRIER_TIMEOUT | NML_SM100_STATUS_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  __threadfence_system();
  return missing;
}

constexpr int kRowsPerBlock = 8;  // one warp per row; one system-scope fence per block

// One warp per send slot.  Slots are grouped by destination in rank order (the layout of
// ep_dispatch_plan), so the destination of slot s follows from the prefix of send_counts.
template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
ep_push_rows_kernel(const T* __restrict__ source, const int32_t* __restrict__ send_order,
                    const int32_t* __restrict__ local_expert,
                    const uint16_t* __restrict__ routing_weights,
                    const int32_t* __restrict__ send_counts, Exchange x, int assignments,
                    int source_rows, int top_k, int* status) {
  const int lane = threadIdx.x & 31;
  const int slot = blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5);
  const int32_t assignment = slot < assignments ? send_order[slot] : -1;
  if (assignment >= 0 && assignment < assignments) {  // else: tail of the send arrays
    int destination = -1, first = 0;
    for (int d = 0; d < x.ranks; ++d) {
      const int count = send_counts[d];
      if (slot < first + count) {
        destination = d;
        break;
      }
      first += count;
    }
    const int position = slot - first;
    const int source_row = assignment / top_k;
    if (destination < 0 || position >= x.region_rows || source_row >= source_rows) {
      if (lane == 0) atomicOr(status, NML_SM100_STATUS_INDEX_RANGE);
    } else {
      const int64_t row = static_cast<int64_t>(x.rank) * x.region_rows + position;
      const uint4* from = reinterpret_cast<const uint4*>(source) +
                          static_cast<int64_t>(source_row) * x.vectors;
      uint4* to = reinterpret_cast<uint4*>(x.rows[destination]) + row * x.vectors;
      copy_row(to, from, x.vectors, lane);
      if (lane == 0) {
        int4 meta;
        meta.x = local_expert[slot];
        meta.y = routing_weights[assignment];
        meta.z = slot;  // row of the sender's return buffer
        meta.w = 0;
        reinterpret_cast<int4*>(x.meta[destination])[row] = meta;
      }
    }
  }
  if (last_block_done(x.local_state + kPushDoneWord)) {
    // every row of this rank is on its way: publish counts, then the epoch
    const int epoch = x.local_state[kEpochWord] + 1;
    if (threadIdx.x < x.ranks) {
      int32_t* sync = x.sync[threadIdx.x];
      sync[kCountWords + x.rank] = min(send_counts[threadIdx.x], x.region_rows);
      store_release_system(sync + kArrivedWords + x.rank, epoch);
    }
    __syncthreads();
    if (threadIdx.x == 0) x.local_state[kEpochWord] = epoch;
  }
}

// After the pushes of all ranks have arrived: expert ids and routing weights of the received
// rows in the form the routed layer takes (k = 1).  Row i of region r is live when
// i < rows sent by r; every other row is masked with id -1.
template <typename T>
__global__ void __launch_bounds__(256)
ep_receive_meta_kernel(Exchange x, int32_t* __restrict__ expert_ids, T* __restrict__ weights,
                       int32_t* __restrict__ received, void** __restrict__ row_targets,
                       int64_t wait_limit, int* status) {
  const int epoch = x.local_state[kEpochWord];
  const int32_t* sync = x.sync[x.rank];
  const unsigned missing = wait_for_epoch(sync + kArrivedWords, x.ranks, epoch, wait_limit, status);
  const int total_rows = x.ranks * x.region_rows;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) {
    int total = 0;
    for (int r = 0; r < x.ranks; ++r) {
      if (!(missing >> r & 1u)) total += min(max(sync[kCountWords + r], 0), x.region_rows);
    }
    received[0] = total;
  }
  if (i >= total_rows) return;
  const int sender = i / x.region_rows;
  const int position = i - sender * x.region_rows;
  const bool live = !(missing >> sender & 1u) && position < sync[kCountWords + sender];
  void* target = nullptr;
  if (live) {
    const int4 m = reinterpret_cast<const int4*>(x.meta[x.rank])[i];
    expert_ids[i] = m.x;
    reinterpret_cast<uint16_t*>(weights)[i] = static_cast<uint16_t>(m.y);
    if (m.z >= 0 && m.z < x.region_rows) {
      // where this row's result goes: row m.z of the sender's return buffer
      target = reinterpret_cast<uint4*>(x.back[sender]) + static_cast<int64_t>(m.z) * x.vectors;
    } else if (row_targets != nullptr) {
      atomicOr(status, NML_SM100_STATUS_INDEX_RANGE);
    }
  } else {
    expert_ids[i] = -1;
    reinterpret_cast<uint16_t*>(weights)[i] = 0;
  }
  if (row_targets != nullptr) row_targets[i] = target;
}

// One warp per received row: computed[i] of region r goes to row meta[i].z of rank r's return
// buffer.  The last block raises this rank's return flag on every rank.  With computed == null
// the rows were already stored by the kernel before this one (a down projection that wrote
// through row targets and whose writers fenced their stores at system scope): the launch is a
// single block that raises the flags.
template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
ep_return_rows_kernel(const T* __restrict__ computed, Exchange x, int* status) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5);
  const int sender = i / x.region_rows;
  const int position = i - sender * x.region_rows;
  const int32_t* sync = x.sync[x.rank];
  if (computed != nullptr && sender < x.ranks &&
      position < min(sync[kCountWords + sender], x.region_rows)) {
    const int4 m = reinterpret_cast<const int4*>(x.meta[x.rank])[i];
    if (m.z < 0 || m.z >= x.region_rows) {
      if (lane == 0) atomicOr(status, NML_SM100_STATUS_INDEX_RANGE);
    } else {
      const uint4* from = reinterpret_cast<const uint4*>(computed) +
                          static_cast<int64_t>(i) * x.vectors;
      uint4* to = reinterpret_cast<uint4*>(x.back[sender]) +
                  static_cast<int64_t>(m.z) * x.vectors;
      copy_row(to, from, x.vectors, lane);
    }
  }
  if (last_block_done(x.local_state + kReturnDoneWord)) {
    const int epoch = x.local_state[kEpochWord];
    if (threadIdx.x < x.ranks) {
      store_release_system(x.sync[threadIdx.x] + kReturnedWords + x.rank, epoch);
    }
  }
}

// Blocks until the return flags of every rank have reached this exchange's epoch (bounded).
__global__ void __launch_bounds__(32)
ep_wait_returns_kernel(Exchange x, int64_t wait_limit, int* status) {
  const int epoch = x.local_state[kEpochWord];
  wait_for_epoch(x.sync[x.rank] + kReturnedWords, x.ranks, epoch, wait_limit, status);
}

// The same wait in every block of the combine over this rank's return buffer: the k-way sum of
// a token's rows starts as soon as the owners' flags are in, without a launch in between.
template <typename T>
__global__ void __launch_bounds__(256)
ep_combine_returns_kernel(Exchange x, const int32_t* __restrict__ row_index,
                          T* __restrict__ output, int tokens, int top_k, int64_t wait_limit,
                          int* status) {
  const int epoch = x.local_state[kEpochWord];
  wait_for_epoch(x.sync[x.rank] + kReturnedWords, x.ranks, epoch, wait_limit, status);
  const int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= static_cast<int64_t>(tokens) * x.vectors) return;
  combine_rows_item<T>(static_cast<const T*>(x.back[x.rank]), row_index, output, item, top_k,
                       x.vectors, x.region_rows);
}

int64_t effective_limit(int64_t requested) {
  // polls of about a quarter microsecond each: one second by default
  return requested > 0 ? requested : (4ll << 20);
}

}  // namespace

bool valid_exchange(const NmlSm100EpExchange& e) {
  bool valid = e.ranks >= 1 && e.ranks <= kMaxRanks && e.rank >= 0 && e.rank < e.ranks &&
               fits_i32(e.region_rows) && fits_i32(e.width) && e.width % 8 == 0 &&
               e.ranks * e.region_rows <= std::numeric_limits<int32_t>::max() &&
               e.local_state != nullptr;
  for (int r = 0; valid && r < e.ranks; ++r) {
    valid = e.peer_rows[r] != nullptr && e.peer_meta[r] != nullptr && e.peer_back[r] != nullptr &&
            e.peer_sync[r] != nullptr && reinterpret_cast<uintptr_t>(e.peer_rows[r]) % 16 == 0 &&
            reinterpret_cast<uintptr_t>(e.peer_meta[r]) % 16 == 0 &&
            reinterpret_cast<uintptr_t>(e.peer_back[r]) % 16 == 0 &&
            reinterpret_cast<uintptr_t>(e.peer_sync[r]) % 4 == 0;
  }
  return valid;
}

int32_t launch_ep_push_rows(const NmlSm100EpPushRows& q, const DeviceInfo& device, char* message,
                            size_t capacity) {
  const Exchange x = make_exchange(q.exchange);
  cudaStream_t stream = static_cast<cudaStream_t>(q.stream);
  const unsigned grid =
      static_cast<unsigned>((q.assignments + kRowsPerBlock - 1) / kRowsPerBlock);
  const uint16_t* weights = static_cast<const uint16_t*>(q.routing_weights);
  constexpr int kBlock = kRowsPerBlock * 32;
  if (q.dtype == NML_SM100_F16) {
    ep_push_rows_kernel<__half><<<grid, kBlock, 0, stream>>>(
        static_cast<const __half*>(q.source), q.send_order, q.local_expert, weights, q.send_counts,
        x, static_cast<int>(q.assignments), static_cast<int>(q.source_rows),
        static_cast<int>(q.experts_per_token), device.status_word);
  } else {
    ep_push_rows_kernel<__nv_bfloat16><<<grid, kBlock, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q.source), q.send_order, q.local_expert, weights,
        q.send_counts, x, static_cast<int>(q.assignments), static_cast<int>(q.source_rows),
        static_cast<int>(q.experts_per_token), device.status_word);
  }
  return launch_result(message, capacity);
}

int32_t launch_ep_receive_meta(const NmlSm100EpReceiveMeta& q, const DeviceInfo& device,
                               char* message, size_t capacity) {
  const Exchange x = make_exchange(q.exchange);
  cudaStream_t stream = static_cast<cudaStream_t>(q.stream);
  const int64_t rows = q.exchange.ranks * q.exchange.region_rows;
  const unsigned grid = static_cast<unsigned>((rows + 255) / 256);
  const int64_t limit = effective_limit(q.wait_limit);
  void** targets = q.struct_size >= offsetof(NmlSm100EpReceiveMeta, row_targets) + sizeof(void*)
                       ? q.row_targets
                       : nullptr;
  if (q.dtype == NML_SM100_F16) {
    ep_receive_meta_kernel<__half><<<grid, 256, 0, stream>>>(
        x, q.expert_ids, static_cast<__half*>(q.routing_weights), q.received, targets, limit,
        device.status_word);
  } else {
    ep_receive_meta_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        x, q.expert_ids, static_cast<__nv_bfloat16*>(q.routing_weights), q.received, targets,
        limit, device.status_word);
  }
  return launch_result(message, capacity);
}

int32_t launch_ep_return_rows(const NmlSm100EpReturnRows& q, const DeviceInfo& device,
                              char* message, size_t capacity) {
  const Exchange x = make_exchange(q.exchange);
  cudaStream_t stream = static_cast<cudaStream_t>(q.stream);
  const unsigned grid =
      q.computed == nullptr
          ? 1u
          : static_cast<unsigned>(
                (q.exchange.ranks * q.exchange.region_rows + kRowsPerBlock - 1) / kRowsPerBlock);
  constexpr int kBlock = kRowsPerBlock * 32;
  if (q.dtype == NML_SM100_F16) {
    ep_return_rows_kernel<__half><<<grid, kBlock, 0, stream>>>(
        static_cast<const __half*>(q.computed), x, device.status_word);
  } else {
    ep_return_rows_kernel<__nv_bfloat16><<<grid, kBlock, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q.computed), x, device.status_word);
  }
  return launch_result(message, capacity);
}

int32_t launch_ep_wait_returns(const NmlSm100EpWaitReturns& q, const DeviceInfo& device,
                               char* message, size_t capacity) {
  const Exchange x = make_exchange(q.exchange);
  cudaStream_t stream = static_cast<cudaStream_t>(q.stream);
  const bool combine = q.struct_size >= offsetof(NmlSm100EpWaitReturns, dtype) + sizeof(int32_t) &&
                       q.output != nullptr;
  if (!combine) {
    ep_wait_returns_kernel<<<1, 32, 0, stream>>>(x, effective_limit(q.wait_limit),
                                                 device.status_word);
    return launch_result(message, capacity);
  }
  const int64_t items = q.tokens * x.vectors;
  const unsigned grid = static_cast<unsigned>((items + 255) / 256);
  if (q.dtype == NML_SM100_F16) {
    ep_combine_returns_kernel<__half><<<grid, 256, 0, stream>>>(
        x, q.row_index, static_cast<__half*>(q.output), static_cast<int>(q.tokens),
        static_cast<int>(q.experts_per_token), effective_limit(q.wait_limit),
        device.status_word);
  } else {
    ep_combine_returns_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        x, q.row_index, static_cast<__nv_bfloat16*>(q.output), static_cast<int>(q.tokens),
        static_cast<int>(q.experts_per_token), effective_limit(q.wait_limit),
        device.status_word);
  }
  return launch_result(message, capacity);
}

}  // namespace nml_sm100
