// Routed-expert support kernels: top-k routing, the assignment schedule, the portable SIMT
// expert projections and the k-way combine.  The tcgen05 expert projections live in
// experts_umma.cu; everything here is integer/elementwise work or the any-shape fallback.
#include <atomic>

#include "common.cuh"

namespace nml_sm100 {

// ============================================================================ routing

// Base-e exponential from correctly rounded IEEE operations only, so that it yields the
// same bits as the same sequence evaluated on a CPU; routing ties (and therefore expert
// ids) then agree exactly with a CPU evaluation of the same rule.  Valid for x <= 0.
__device__ __forceinline__ float exp_deterministic(float x) {
  if (!(x > -87.3f)) return 0.0f;
  if (x > 0.0f) x = 0.0f;
  const float n = rintf(__fmul_rn(x, 1.44269504088896341f));
  float r = __fmaf_rn(n, -0.693359375f, x);
  r = __fmaf_rn(n, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = __fmaf_rn(p, r, 1.3981999507e-3f);
  p = __fmaf_rn(p, r, 8.3334519073e-3f);
  p = __fmaf_rn(p, r, 4.1665795894e-2f);
  p = __fmaf_rn(p, r, 1.6666665459e-1f);
  p = __fmaf_rn(p, r, 5.0000001201e-1f);
  p = __fmaf_rn(p, __fmul_rn(r, r), r);
  p = __fadd_rn(p, 1.0f);
  const float scale = __uint_as_float(static_cast<uint32_t>(static_cast<int>(n) + 127) << 23);
  return __fmul_rn(p, scale);
}

namespace {

// One thread routes one token: softmax over all experts (f32, denominator summed in expert
// order), k rounds of first-maximum selection (strict >, so equal probabilities go to the
// lower expert index), renormalisation by max(sum, FLT_EPSILON)
// (crates/nml-ir/src/lib.rs:1411-1437).
template <int MAX_EXPERTS, typename T>
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, const uint8_t* __restrict__ active,
             int32_t* __restrict__ expert_ids, T* __restrict__ weights, int tokens, int experts,
             int top_k) {
  const int token = blockIdx.x * blockDim.x + threadIdx.x;
  if (token >= tokens) return;
  const float* row = logits + static_cast<int64_t>(token) * experts;
  float probability[MAX_EXPERTS];
  float maximum = -INFINITY;
#pragma unroll
  for (int e = 0; e < MAX_EXPERTS; ++e) {
    probability[e] = e < experts ? row[e] : -INFINITY;
    maximum = probability[e] > maximum ? probability[e] : maximum;
  }
  if (maximum > -INFINITY) {
    float denominator = 0.0f;
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) {
      if (e < experts) {
        probability[e] = exp_deterministic(__fsub_rn(probability[e], maximum));
        denominator = __fadd_rn(denominator, probability[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) {
      probability[e] = e < experts ? __fdiv_rn(probability[e], denominator) : -1.0f;
    }
  } else {
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) probability[e] = e < experts ? 0.0f : -1.0f;
  }
  const bool is_active = active == nullptr || active[token] != 0;
  float selected[16];
  int selected_id[16];
  float sum = 0.0f;
  for (int route = 0; route < top_k; ++route) {
    int best = 0;
    float best_value = -2.0f;  // below every probability and the -1 padding
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) {
      if (probability[e] > best_value) {
        best_value = probability[e];
        best = e;
      }
    }
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS; ++e) {
      if (e == best) probability[e] = -3.0f;  // taken
    }
    selected[route] = best_value;
    selected_id[route] = best;
    sum = __fadd_rn(sum, best_value);
  }
  const float normalizer = fmaxf(sum, 1.1920928955078125e-7f);
  for (int route = 0; route < top_k; ++route) {
    const int64_t a = static_cast<int64_t>(token) * top_k + route;
    expert_ids[a] = is_active ? selected_id[route] : -1;
    weights[a] = Elem<T>::store(is_active ? __fdiv_rn(selected[route], normalizer) : 0.0f);
  }
}

// One warp routes one token, lane e holding expert e (up to 32 experts): the same operations
// in the same order as route_kernel (maximum, exponentials, denominator summed in expert
// order, k rounds of first-maximum selection with ties to the lower index), so the bits agree;
// only the latency differs (decode-size batches spend longer in the one-thread-per-token
// kernel than in an expert projection).
template <typename T>
__global__ void __launch_bounds__(128)
route_warp_kernel(const float* __restrict__ logits, const uint8_t* __restrict__ active,
                  int32_t* __restrict__ expert_ids, T* __restrict__ weights, int tokens,
                  int experts, int top_k) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= tokens) return;
  constexpr unsigned kAll = 0xffffffffu;
  float probability = lane < experts ? logits[static_cast<int64_t>(token) * experts + lane]
                                     : -INFINITY;
  float maximum = probability;
#pragma unroll
  for (int offset = 16; offset != 0; offset >>= 1) {
    maximum = fmaxf(maximum, __shfl_xor_sync(kAll, maximum, offset));
  }
  if (maximum > -INFINITY) {
    if (lane < experts) probability = exp_deterministic(__fsub_rn(probability, maximum));
    float denominator = 0.0f;
    for (int e = 0; e < experts; ++e) {  // expert order, like the sequential kernel
      denominator = __fadd_rn(denominator, __shfl_sync(kAll, probability, e));
    }
    probability = lane < experts ? __fdiv_rn(probability, denominator) : -1.0f;
  } else {
    probability = lane < experts ? 0.0f : -1.0f;
  }
  const bool is_active = active == nullptr || active[token] != 0;
  float sum = 0.0f;
  float mine = 0.0f;  // lane r keeps the r-th selected probability and id
  int mine_id = 0;
  for (int route = 0; route < top_k; ++route) {
    // first maximum: larger value wins, equal values go to the lower lane
    float best = probability;
    int best_lane = lane;
#pragma unroll
    for (int offset = 16; offset != 0; offset >>= 1) {
      const float other = __shfl_xor_sync(kAll, best, offset);
      const int other_lane = __shfl_xor_sync(kAll, best_lane, offset);
      if (other > best || (other == best && other_lane < best_lane)) {
        best = other;
        best_lane = other_lane;
      }
    }
    if (lane == best_lane) probability = -3.0f;  // taken
    if (lane == route) {
      mine = best;
      mine_id = best_lane;
    }
    sum = __fadd_rn(sum, best);
  }
  const float normalizer = fmaxf(sum, 1.1920928955078125e-7f);
  if (lane < top_k) {
    const int64_t a = static_cast<int64_t>(token) * top_k + lane;
    expert_ids[a] = is_active ? mine_id : -1;
    weights[a] = Elem<T>::store(is_active ? __fdiv_rn(mine, normalizer) : 0.0f);
  }
}

// ====================================================================== assignment plan

// Single-CTA construction of the schedule of crates/nml-ir/src/lib.rs:5644-5779.  Thread t
// owns a contiguous chunk of assignments; hist[e][t] first counts the chunk's assignments
// to expert e, then (after a scan across threads) is the rank of the chunk's first such
// assignment inside the expert, which keeps assignments ascending inside each expert.
__global__ void __launch_bounds__(1024)
assignment_plan_kernel(const int32_t* __restrict__ expert_ids,
                       int32_t* __restrict__ sorted_assignments,
                       int32_t* __restrict__ block_experts, int32_t* __restrict__ active_blocks,
                       int assignments, int experts, int expert_offset, int positions,
                       int blocks) {
  extern __shared__ int32_t plan_smem[];
  const int threads = blockDim.x;
  const int t = threadIdx.x;
  int32_t* hist = plan_smem;                    // [experts][threads]
  int32_t* totals = hist + experts * threads;   // [experts]
  int32_t* prefix = totals + experts;           // [experts + 1] padded starts

  for (int i = t; i < positions; i += threads) sorted_assignments[i] = assignments;
  if (assignments <= experts) {
    // Sparse form: one block per route, first slot carries the assignment.
    for (int b = t; b < blocks; b += threads) {
      int32_t id = -1;
      if (b < assignments) {
        const int32_t local = expert_ids[b] - expert_offset;
        id = (expert_ids[b] >= 0 && local >= 0 && local < experts) ? local : -1;
      }
      block_experts[b] = id;
    }
    __syncthreads();
    for (int a = t; a < assignments; a += threads) sorted_assignments[a * 16] = a;
    if (t == 0) *active_blocks = assignments;
    return;
  }
  for (int b = t; b < blocks; b += threads) block_experts[b] = -1;
  for (int i = t; i < experts * threads; i += threads) hist[i] = 0;
  __syncthreads();

  const int chunk = (assignments + threads - 1) / threads;
  const int begin = min(assignments, t * chunk);
  const int end = min(assignments, begin + chunk);
  for (int a = begin; a < end; ++a) {
    const int32_t id = expert_ids[a];
    const int32_t local = id - expert_offset;
    if (id >= 0 && local >= 0 && local < experts) hist[local * threads + t] += 1;
  }
  __syncthreads();

  const int lane = t & 31;
  const int warp = t >> 5;
  const int warps = threads >> 5;
  for (int e = warp; e < experts; e += warps) {
    int32_t running = 0;
    for (int base = 0; base < threads; base += 32) {
      const int32_t value = hist[e * threads + base + lane];
      int32_t inclusive = value;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const int32_t other = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (lane >= offset) inclusive += other;
      }
      hist[e * threads + base + lane] = running + inclusive - value;
      running += __shfl_sync(0xffffffffu, inclusive, 31);
    }
    if (lane == 0) totals[e] = running;
  }
  __syncthreads();
  if (t == 0) {
    int32_t start = 0;
    for (int e = 0; e < experts; ++e) {
      prefix[e] = start;
      start += (totals[e] + 15) / 16 * 16;
    }
    prefix[experts] = start;
    *active_blocks = start / 16;
  }
  __syncthreads();
  for (int e = warp; e < experts; e += warps) {
    for (int b = prefix[e] / 16 + lane; b < prefix[e + 1] / 16; b += 32) block_experts[b] = e;
  }
  for (int a = begin; a < end; ++a) {
    const int32_t id = expert_ids[a];
    const int32_t local = id - expert_offset;
    if (id >= 0 && local >= 0 && local < experts) {
      const int32_t rank = hist[local * threads + t]++;
      sorted_assignments[prefix[local] + rank] = a;
    }
  }
}

// ============================================================================= combine

template <typename T>
__global__ void __launch_bounds__(256)
combine_kernel(const T* __restrict__ weighted, const int32_t* __restrict__ expert_ids,
               T* __restrict__ output, int tokens, int top_k, int hidden, int experts,
               int expert_offset) {
  const int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int vectors = hidden / 8;
  if (item >= static_cast<int64_t>(tokens) * vectors) return;
  const int token = static_cast<int>(item / vectors);
  const int column = static_cast<int>(item - static_cast<int64_t>(token) * vectors) * 8;
  float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int route = 0; route < top_k; ++route) {
    const int64_t a = static_cast<int64_t>(token) * top_k + route;
    if (expert_ids != nullptr) {
      const int32_t id = expert_ids[a];
      const int32_t local = id - expert_offset;
      if (id < 0 || local < 0 || local >= experts) continue;
    }
    const uint4 v = *reinterpret_cast<const uint4*>(weighted + a * hidden + column);
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sum[2 * i] += Elem<T>::from_bits(words[i] & 0xffffu);
      sum[2 * i + 1] += Elem<T>::from_bits(words[i] >> 16);
    }
  }
  uint4 out;
  out.x = Elem<T>::pack2(sum[0], sum[1]);
  out.y = Elem<T>::pack2(sum[2], sum[3]);
  out.z = Elem<T>::pack2(sum[4], sum[5]);
  out.w = Elem<T>::pack2(sum[6], sum[7]);
  *reinterpret_cast<uint4*>(output + static_cast<int64_t>(token) * hidden + column) = out;
}

template <typename T>
__global__ void __launch_bounds__(256)
combine_scalar_kernel(const T* __restrict__ weighted, const int32_t* __restrict__ expert_ids,
                      T* __restrict__ output, int tokens, int top_k, int hidden, int experts,
                      int expert_offset) {
  const int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= static_cast<int64_t>(tokens) * hidden) return;
  const int token = static_cast<int>(item / hidden);
  const int column = static_cast<int>(item - static_cast<int64_t>(token) * hidden);
  float sum = 0.0f;
  for (int route = 0; route < top_k; ++route) {
    const int64_t a = static_cast<int64_t>(token) * top_k + route;
    if (expert_ids != nullptr) {
      const int32_t id = expert_ids[a];
      const int32_t local = id - expert_offset;
      if (id < 0 || local < 0 || local >= experts) continue;
    }
    sum += Elem<T>::load(weighted[a * hidden + column]);
  }
  output[item] = Elem<T>::store(sum);
}

// ================================================================= SIMT expert kernels

constexpr int kExpertWarps = 4;

// Any-shape grouped projection over the 16-slot block schedule.  One warp owns one output
// column of one schedule block: for gate/up that is intermediate column i (weight rows 2i
// and 2i+1 of the block's expert, SwiGLU epilogue), for down it is hidden column h (bias
// and routing-weight epilogue).  Blocks at or past *active_blocks, and blocks whose expert
// is -1 or not held locally, leave before touching weights
// (crates/nml-kernel-nvfp4/src/turing_adapter.cu:270-275, crates/nml-kernel-triton/src/nvfp4.rs:867-937).
template <typename T, bool GATE_UP>
__global__ void __launch_bounds__(kExpertWarps * 32)
experts_simt_kernel(const T* __restrict__ input, const int32_t* __restrict__ sorted_assignments,
                    const int32_t* __restrict__ block_experts,
                    const uint8_t* __restrict__ payload, const uint8_t* __restrict__ block_scales,
                    const float* __restrict__ global_scale, const T* __restrict__ bias,
                    const T* __restrict__ routing_weights, T* __restrict__ output,
                    void* const* __restrict__ row_targets,
                    const int32_t* __restrict__ active_blocks,
                    const int32_t* __restrict__ expert_offset, int assignments, int inputs,
                    int outputs, int experts, int top_k) {
  const int block = blockIdx.y;
  if (active_blocks != nullptr && block >= active_blocks[0]) return;
  const int offset = expert_offset != nullptr ? expert_offset[0] : 0;
  const int32_t expert_id = block_experts[block];
  const int32_t expert = expert_id - offset;
  if (expert_id < 0 || expert < 0 || expert >= experts) return;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int column = blockIdx.x * kExpertWarps + warp;
  if (column >= outputs) return;

  constexpr int kRowsPerColumn = GATE_UP ? 2 : 1;
  const int packed_width = (inputs + 1) / 2;
  const int scale_width = (inputs + 15) / 16;
  const int64_t weight_row0 =
      (static_cast<int64_t>(expert) * outputs + column) * kRowsPerColumn;
  const float g = global_scale[0];

  int32_t slot_assignment[16];
#pragma unroll
  for (int s = 0; s < 16; ++s) {
    const int32_t a = sorted_assignments[block * 16 + s];
    slot_assignment[s] = (a >= 0 && a < assignments) ? a : -1;
  }
  float acc[kRowsPerColumn][16];
#pragma unroll
  for (int r = 0; r < kRowsPerColumn; ++r) {
#pragma unroll
    for (int s = 0; s < 16; ++s) acc[r][s] = 0.0f;
  }
  for (int kb = lane; kb < scale_width; kb += 32) {
    const int start = kb * 16;
    const int count = min(16, inputs - start);
    float w[kRowsPerColumn][16];
#pragma unroll
    for (int r = 0; r < kRowsPerColumn; ++r) {
      const uint8_t* row_payload = payload + (weight_row0 + r) * packed_width;
      const float effective =
          __fmul_rn(e4m3_scale_to_f32(block_scales[(weight_row0 + r) * scale_width + kb]), g);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float value = 0.0f;
        if (i < count) {
          const uint32_t byte = row_payload[(start + i) >> 1];
          const uint32_t code = ((start + i) & 1) ? (byte >> 4) : (byte & 0xfu);
          value = __fmul_rn(e2m1_to_f32(code), effective);
        }
        w[r][i] = value;
      }
    }
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      const int32_t a = slot_assignment[s];
      if (a < 0) continue;
      const int64_t source_row = GATE_UP ? a / top_k : a;
      const T* x = input + source_row * inputs + start;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (i < count) {
          const float xv = Elem<T>::load(x[i]);
#pragma unroll
          for (int r = 0; r < kRowsPerColumn; ++r) acc[r][s] = fmaf(xv, w[r][i], acc[r][s]);
        }
      }
    }
  }
#pragma unroll
  for (int s = 0; s < 16; ++s) {
    float sums[kRowsPerColumn];
#pragma unroll
    for (int r = 0; r < kRowsPerColumn; ++r) {
      float v = acc[r][s];
#pragma unroll
      for (int o = 16; o != 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      sums[r] = v;
    }
    const int32_t a = slot_assignment[s];
    if (lane == 0 && a >= 0) {
      if constexpr (GATE_UP) {
        const int64_t bias_base = (static_cast<int64_t>(expert) * outputs + column) * 2;
        const float gate = sums[0] + Elem<T>::load(bias[bias_base]);
        const float up = sums[1] + Elem<T>::load(bias[bias_base + 1]);
        output[static_cast<int64_t>(a) * outputs + column] =
            Elem<T>::store(clamped_swiglu(gate, up));
      } else {
        const float value =
            (sums[0] + Elem<T>::load(bias[static_cast<int64_t>(expert) * outputs + column])) *
            Elem<T>::load(routing_weights[a]);
        T* destination = row_targets != nullptr
                             ? static_cast<T*>(row_targets[a])
                             : output + static_cast<int64_t>(a) * outputs;
        if (destination != nullptr) destination[column] = Elem<T>::store(value);
        // a destination in another GPU's memory is announced by a later launch: the writer
        // orders its own store at system scope
        if (row_targets != nullptr) __threadfence_system();
      }
    }
  }
}

template <typename T>
int32_t launch_experts_simt_typed(const ExpertArgs& args, char* message, size_t capacity) {
  const dim3 grid(static_cast<unsigned>((args.outputs + kExpertWarps - 1) / kExpertWarps),
                  static_cast<unsigned>(args.schedule_blocks));
  if (args.schedule_blocks > 65535) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "NVFP4 expert schedule has too many blocks for the portable kernel", message,
                capacity);
  }
  if (args.gate_up) {
    experts_simt_kernel<T, true><<<grid, kExpertWarps * 32, 0, args.stream>>>(
        static_cast<const T*>(args.input), args.sorted_assignments, args.block_experts,
        args.payload, args.block_scales, args.global_scale, static_cast<const T*>(args.bias),
        nullptr, static_cast<T*>(args.output), nullptr, args.active_blocks, args.expert_offset,
        args.assignments, args.inputs, args.outputs, args.experts, args.experts_per_token);
  } else {
    experts_simt_kernel<T, false><<<grid, kExpertWarps * 32, 0, args.stream>>>(
        static_cast<const T*>(args.input), args.sorted_assignments, args.block_experts,
        args.payload, args.block_scales, args.global_scale, static_cast<const T*>(args.bias),
        static_cast<const T*>(args.routing_weights), static_cast<T*>(args.output),
        args.row_targets, args.active_blocks, args.expert_offset, args.assignments, args.inputs,
        args.outputs,
        args.experts, args.experts_per_token);
  }
  return launch_result(message, capacity);
}

}  // namespace

int32_t launch_experts_simt(const ExpertArgs& args, const DeviceInfo&, char* message,
                            size_t capacity) {
  return args.dtype == NML_SM100_F16
             ? launch_experts_simt_typed<__half>(args, message, capacity)
             : launch_experts_simt_typed<__nv_bfloat16>(args, message, capacity);
}

int32_t launch_route(const NmlSm100Route& r, char* message, size_t capacity) {
  const int tokens = static_cast<int>(r.tokens);
  const int experts = static_cast<int>(r.experts);
  const int top_k = static_cast<int>(r.experts_per_token);
  const unsigned grid = static_cast<unsigned>((tokens + 127) / 128);
  cudaStream_t stream = static_cast<cudaStream_t>(r.stream);
  if (experts <= 32 && top_k <= 32 && tokens <= 4096) {
    // few tokens: one warp per token
    const unsigned warp_grid = static_cast<unsigned>((tokens + 3) / 4);
    if (r.dtype == NML_SM100_F16) {
      route_warp_kernel<__half><<<warp_grid, 128, 0, stream>>>(
          r.logits, r.active_tokens, r.expert_ids, static_cast<__half*>(r.routing_weights),
          tokens, experts, top_k);
    } else {
      route_warp_kernel<__nv_bfloat16><<<warp_grid, 128, 0, stream>>>(
          r.logits, r.active_tokens, r.expert_ids,
          static_cast<__nv_bfloat16*>(r.routing_weights), tokens, experts, top_k);
    }
    return launch_result(message, capacity);
  }
#define NML_ROUTE(MAXE, T)                                                                  \
  route_kernel<MAXE, T><<<grid, 128, 0, stream>>>(r.logits, r.active_tokens, r.expert_ids,   \
                                                  static_cast<T*>(r.routing_weights), tokens, \
                                                  experts, top_k)
#define NML_ROUTE_BY_EXPERTS(T) \
  if (experts <= 32) {          \
    NML_ROUTE(32, T);           \
  } else if (experts <= 64) {   \
    NML_ROUTE(64, T);           \
  } else if (experts <= 128) {  \
    NML_ROUTE(128, T);          \
  } else {                      \
    NML_ROUTE(256, T);          \
  }
  if (r.dtype == NML_SM100_F16) {
    NML_ROUTE_BY_EXPERTS(__half)
  } else {
    NML_ROUTE_BY_EXPERTS(__nv_bfloat16)
  }
#undef NML_ROUTE_BY_EXPERTS
#undef NML_ROUTE
  return launch_result(message, capacity);
}

int32_t launch_assignment_plan(const int32_t* expert_ids, int32_t* sorted_assignments,
                               int32_t* block_experts, int32_t* active_blocks, int assignments,
                               int experts, int expert_offset, int positions, int blocks,
                               int device, cudaStream_t stream, char* message, size_t capacity) {
  // threads * experts histogram words must fit the shared memory requested below.
  // one thread per couple of assignments for small batches (the per-thread histograms make
  // the kernel's fixed cost grow with the thread count), up to 1024
  int threads = 32;
  while (threads < 1024 && threads * 2 < assignments) threads <<= 1;
  while (threads > 32 && static_cast<int64_t>(threads) * experts > 32768) threads >>= 1;
  const size_t smem = (static_cast<size_t>(threads) * experts + 2 * experts + 2) * 4;
  static std::atomic<int> configured[64];
  const bool known = device >= 0 && device < 64;
  if (!known || !configured[device].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(assignment_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             144 * 1024) != cudaSuccess) {
      return fail(NML_SM100_LAUNCH_FAILURE, "cannot reserve shared memory for the plan kernel",
                  message, capacity);
    }
    if (known) configured[device].store(1, std::memory_order_release);
  }
  assignment_plan_kernel<<<1, threads, smem, stream>>>(expert_ids, sorted_assignments,
                                                       block_experts, active_blocks, assignments,
                                                       experts, expert_offset, positions, blocks);
  return launch_result(message, capacity);
}

int32_t launch_combine(const void* weighted, const int32_t* expert_ids, void* output, int tokens,
                       int top_k, int hidden, int experts, int expert_offset, int dtype,
                       cudaStream_t stream, char* message, size_t capacity) {
  const bool vector_ok = hidden % 8 == 0 && reinterpret_cast<uintptr_t>(weighted) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(output) % 16 == 0;
  const int64_t items = static_cast<int64_t>(tokens) * (vector_ok ? hidden / 8 : hidden);
  const int64_t grid = (items + 255) / 256;
  if (grid > std::numeric_limits<int32_t>::max()) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 combine launch extent overflows", message,
                capacity);
  }
#define NML_COMBINE(KERNEL, T)                                                                \
  KERNEL<T><<<static_cast<unsigned>(grid), 256, 0, stream>>>(                                 \
      static_cast<const T*>(weighted), expert_ids, static_cast<T*>(output), tokens, top_k,    \
      hidden, experts, expert_offset)
  if (dtype == NML_SM100_F16) {
    if (vector_ok) NML_COMBINE(combine_kernel, __half);
    else NML_COMBINE(combine_scalar_kernel, __half);
  } else {
    if (vector_ok) NML_COMBINE(combine_kernel, __nv_bfloat16);
    else NML_COMBINE(combine_scalar_kernel, __nv_bfloat16);
  }
#undef NML_COMBINE
  return launch_result(message, capacity);
}

}  // namespace nml_sm100
