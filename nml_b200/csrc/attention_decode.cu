// Paged-attention decode (one query token per sequence) for grouped-query models: the largest
// byte mover of a GPT-OSS-shaped decode step after the expert weights.  Semantics follow the
// reference's graph operator (crates/nml-ir/src/lib.rs:4717-4730): K/V storage
// [physical_pages, page_size, kv_heads, head_dim], page table [batch, logical_pages], sequence
// lengths [batch]; causal (the query is the last token of its sequence), optional sliding
// window, optional learned per-head sinks (one extra softmax column without a value, i.e.
// out * sigmoid(lse - sink), crates/nml-ir/src/attention_sink.rs:1-8).  The reference runs
// this on GPUs through Triton kernels (crates/nml-kernel-triton/src/unified_attention.rs:82,
// 189,755: a split-K "3D" kernel with a segment reduction); this is their sm_100a
// counterpart, HBM-bound: every K and V byte of the visible tokens is read once.
//
// Shape of the work: one CTA per (sequence, kv head, split of the visible pages), four warps
// that take pages round-robin.  A page of 16 tokens is one mma.sync row block: scores
// [16 tokens x 8 query heads of the group] = K_page [16 x 64] . Q_group^T, four
// mma.sync.m16n8k16 with the page's keys loaded straight into A fragments (16-byte loads; the
// K index order inside an instruction is free as long as Q uses the same order).  Softmax is
// online per warp (running maximum and sum per head), probabilities pass through a 512-byte
// shared-memory tile, and P.V runs on FMA lanes: lane l owns dimensions 2l and 2l + 1 of all
// eight heads.  Warps merge in shared memory, splits through a caller-provided f32 scratch
// that a second small kernel reduces (applying the sink) into the 16-bit output.
#include <type_traits>

#include "common.cuh"

namespace nml_sm100 {
namespace {

constexpr int kPage = 16;
constexpr int kHeadDim = 64;
constexpr int kGroup = 8;    // query heads per kv head
constexpr int kWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct DecodeParams {
  const void* query;         // [batch, query_heads, 64]
  const void* key_cache;     // [pages, 16, kv_heads, 64]
  const void* value_cache;
  const int32_t* page_table; // [batch, table_width]
  const int32_t* lengths;    // [batch] visible tokens (the query token included)
  const float* sinks;        // [query_heads] or null
  float* partial;            // [batch, kv_heads, splits, 8, 66]: out[64], max, sum
  void* output;              // [batch, query_heads, 64]
  int batch, kv_heads, table_width, physical_pages, splits, window;
  float scale_log2;          // softmax scale * log2(e)
  int* status;
};

// partial layout per (batch, kv head, split, head of the group)
constexpr int kPartialWidth = kHeadDim + 2;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attention_decode_kernel(const DecodeParams p) {
  const int head = blockIdx.x;   // kv head
  const int b = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  __shared__ float probability[kWarps][kPage][kGroup];          // per warp: one page of P
  __shared__ float merged[kWarps][kGroup][kPartialWidth];       // per warp results

  const int length = p.lengths[b];
  const int first_token = p.window > 0 ? max(0, length - p.window) : 0;
  const int first_page = first_token / kPage;
  const int pages = max(0, (length + kPage - 1) / kPage - first_page);
  // this split's share of the visible pages
  const int per_split = (pages + p.splits - 1) / p.splits;
  const int page_begin = first_page + split * per_split;
  const int page_end = min(first_page + pages, page_begin + per_split);

  // Q of the group as B fragments: head g, dimensions 16 c + 4 i + {0..3} for instruction i
  uint32_t q[4][2];
  {
    const T* row = static_cast<const T*>(p.query) +
                   (static_cast<int64_t>(b) * p.kv_heads * kGroup + head * kGroup + g) * kHeadDim +
                   16 * c;
    const uint4 lo = *reinterpret_cast<const uint4*>(row);
    const uint4 hi = *reinterpret_cast<const uint4*>(row + 8);
    q[0][0] = lo.x; q[0][1] = lo.y; q[1][0] = lo.z; q[1][1] = lo.w;
    q[2][0] = hi.x; q[2][1] = hi.y; q[3][0] = hi.z; q[3][1] = hi.w;
  }
  // running state: this lane keeps heads 2 c and 2 c + 1 statistics (replicated over g) and
  // the output of dimensions 2 lane, 2 lane + 1 for all eight heads
  float running_max[2] = {-INFINITY, -INFINITY};
  float running_sum[2] = {0.0f, 0.0f};
  float out[kGroup][2];
#pragma unroll
  for (int h = 0; h < kGroup; ++h) out[h][0] = out[h][1] = 0.0f;

  const int64_t token_stride = static_cast<int64_t>(p.kv_heads) * kHeadDim;  // elements
  for (int page = page_begin + warp; page < page_end; page += kWarps) {
    int32_t physical = p.page_table[static_cast<int64_t>(b) * p.table_width + page];
    if (physical < 0 || physical >= p.physical_pages) {
      if (lane == 0) atomicOr(p.status, NML_SM100_STATUS_INDEX_RANGE);
      physical = 0;  // the page still reads valid memory; its scores are masked below
    }
    const int64_t page_base = (static_cast<int64_t>(physical) * kPage) * token_stride +
                              static_cast<int64_t>(head) * kHeadDim;
    // keys of tokens g and g + 8, dimensions 16 c .. 16 c + 15
    const T* key = static_cast<const T*>(p.key_cache) + page_base + 16 * c;
    const uint4 k_lo_g = *reinterpret_cast<const uint4*>(key + g * token_stride);
    const uint4 k_hi_g = *reinterpret_cast<const uint4*>(key + g * token_stride + 8);
    const uint4 k_lo_h = *reinterpret_cast<const uint4*>(key + (g + 8) * token_stride);
    const uint4 k_hi_h = *reinterpret_cast<const uint4*>(key + (g + 8) * token_stride + 8);
    // values: lane owns dimensions 2 lane, 2 lane + 1 of every token of the page
    const T* value = static_cast<const T*>(p.value_cache) + page_base + 2 * lane;
    uint32_t v[kPage];
#pragma unroll
    for (int t = 0; t < kPage; ++t) {
      v[t] = *reinterpret_cast<const uint32_t*>(value + t * token_stride);
    }
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // tokens g (s0, s1) and g + 8 (s2, s3), heads 2c, 2c+1
    if constexpr (std::is_same<T, __half>::value) {
      mma_f16(s, k_lo_g.x, k_lo_h.x, k_lo_g.y, k_lo_h.y, q[0][0], q[0][1]);
      mma_f16(s, k_lo_g.z, k_lo_h.z, k_lo_g.w, k_lo_h.w, q[1][0], q[1][1]);
      mma_f16(s, k_hi_g.x, k_hi_h.x, k_hi_g.y, k_hi_h.y, q[2][0], q[2][1]);
      mma_f16(s, k_hi_g.z, k_hi_h.z, k_hi_g.w, k_hi_h.w, q[3][0], q[3][1]);
    } else {
      mma_bf16(s, k_lo_g.x, k_lo_h.x, k_lo_g.y, k_lo_h.y, q[0][0], q[0][1]);
      mma_bf16(s, k_lo_g.z, k_lo_h.z, k_lo_g.w, k_lo_h.w, q[1][0], q[1][1]);
      mma_bf16(s, k_hi_g.x, k_hi_h.x, k_hi_g.y, k_hi_h.y, q[2][0], q[2][1]);
      mma_bf16(s, k_hi_g.z, k_hi_h.z, k_hi_g.w, k_hi_h.w, q[3][0], q[3][1]);
    }
    // mask tokens outside [first_token, length), scale into the exp2 domain
    const int token_g = page * kPage + g;
    const bool seen_g = token_g >= first_token && token_g < length;
    const bool seen_h = token_g + 8 >= first_token && token_g + 8 < length;
    s[0] = seen_g ? s[0] * p.scale_log2 : -INFINITY;
    s[1] = seen_g ? s[1] * p.scale_log2 : -INFINITY;
    s[2] = seen_h ? s[2] * p.scale_log2 : -INFINITY;
    s[3] = seen_h ? s[3] * p.scale_log2 : -INFINITY;
    // page maximum per head over the 16 tokens (lanes with the same c)
    float page_max[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#pragma unroll
    for (int offset = 4; offset < 32; offset <<= 1) {
      page_max[0] = fmaxf(page_max[0], __shfl_xor_sync(0xffffffffu, page_max[0], offset));
      page_max[1] = fmaxf(page_max[1], __shfl_xor_sync(0xffffffffu, page_max[1], offset));
    }
    float rescale[2], new_max[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      new_max[i] = fmaxf(running_max[i], page_max[i]);
      // a page with no visible token leaves the state unchanged (both maxima -inf)
      rescale[i] = new_max[i] == -INFINITY ? 1.0f : exp2f(running_max[i] - new_max[i]);
    }
    const float base0 = new_max[0] == -INFINITY ? 0.0f : new_max[0];
    const float base1 = new_max[1] == -INFINITY ? 0.0f : new_max[1];
    const float p0 = exp2f(s[0] - base0), p1 = exp2f(s[1] - base1);
    const float p2 = exp2f(s[2] - base0), p3 = exp2f(s[3] - base1);
    float page_sum[2] = {p0 + p2, p1 + p3};
#pragma unroll
    for (int offset = 4; offset < 32; offset <<= 1) {
      page_sum[0] += __shfl_xor_sync(0xffffffffu, page_sum[0], offset);
      page_sum[1] += __shfl_xor_sync(0xffffffffu, page_sum[1], offset);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      running_sum[i] = running_sum[i] * rescale[i] + page_sum[i];
      running_max[i] = new_max[i];
    }
    __syncwarp();
    probability[warp][g][2 * c] = p0;
    probability[warp][g][2 * c + 1] = p1;
    probability[warp][g + 8][2 * c] = p2;
    probability[warp][g + 8][2 * c + 1] = p3;
    // every lane needs the rescale factors of all eight heads: head h lives in lanes c = h / 2
    float factor[kGroup];
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
      factor[h] = __shfl_sync(0xffffffffu, rescale[h & 1], h >> 1);
    }
    __syncwarp();
#pragma unroll
    for (int h = 0; h < kGroup; ++h) {
      out[h][0] *= factor[h];
      out[h][1] *= factor[h];
    }
#pragma unroll
    for (int t = 0; t < kPage; ++t) {
      const float v0 = Elem<T>::from_bits(v[t] & 0xffffu);
      const float v1 = Elem<T>::from_bits(v[t] >> 16);
      const float4 pa = *reinterpret_cast<const float4*>(&probability[warp][t][0]);
      const float4 pb = *reinterpret_cast<const float4*>(&probability[warp][t][4]);
      const float weights[kGroup] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        out[h][0] = fmaf(weights[h], v0, out[h][0]);
        out[h][1] = fmaf(weights[h], v1, out[h][1]);
      }
    }
  }

  // ---- merge the four warps, then write this split's partial result -----------------------
#pragma unroll
  for (int h = 0; h < kGroup; ++h) {
    merged[warp][h][2 * lane] = out[h][0];
    merged[warp][h][2 * lane + 1] = out[h][1];
  }
  if (g == 0) {  // lanes 0..3 hold the statistics of heads 2 c, 2 c + 1
    merged[warp][2 * c][kHeadDim] = running_max[0];
    merged[warp][2 * c][kHeadDim + 1] = running_sum[0];
    merged[warp][2 * c + 1][kHeadDim] = running_max[1];
    merged[warp][2 * c + 1][kHeadDim + 1] = running_sum[1];
  }
  __syncthreads();
  // thread t: head t / 16, dimensions 4 (t % 16) .. + 3
  const int h = threadIdx.x >> 4;
  const int d0 = (threadIdx.x & 15) * 4;
  float total_max = -INFINITY;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) total_max = fmaxf(total_max, merged[w][h][kHeadDim]);
  float total_sum = 0.0f;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const float m = merged[w][h][kHeadDim];
    const float weight = m == -INFINITY ? 0.0f : exp2f(m - total_max);
    total_sum += merged[w][h][kHeadDim + 1] * weight;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fmaf(merged[w][h][d0 + i], weight, acc[i]);
  }
  float* destination = p.partial +
      ((((static_cast<int64_t>(b) * p.kv_heads + head) * p.splits + split) * kGroup) + h) *
          kPartialWidth;
  *reinterpret_cast<float2*>(destination + d0) = make_float2(acc[0], acc[1]);
  *reinterpret_cast<float2*>(destination + d0 + 2) = make_float2(acc[2], acc[3]);
  if ((threadIdx.x & 15) == 0) {
    destination[kHeadDim] = total_max;
    destination[kHeadDim + 1] = total_sum;
  }
}

// One warp per query head: merges the splits, applies the sink, narrows.
template <typename T>
__global__ void __launch_bounds__(128)
attention_reduce_kernel(const DecodeParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t query_head = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  const int64_t heads_total = static_cast<int64_t>(p.batch) * p.kv_heads * kGroup;
  if (query_head >= heads_total) return;
  const int64_t pair = query_head / kGroup;  // (batch, kv head)
  const int h = static_cast<int>(query_head - pair * kGroup);
  const float* base = p.partial + ((pair * p.splits) * kGroup + h) * kPartialWidth;
  const int64_t split_stride = static_cast<int64_t>(kGroup) * kPartialWidth;
  float total_max = -INFINITY;
  for (int s = 0; s < p.splits; ++s) total_max = fmaxf(total_max, base[s * split_stride + kHeadDim]);
  float total_sum = 0.0f, a0 = 0.0f, a1 = 0.0f;
  for (int s = 0; s < p.splits; ++s) {
    const float* part = base + s * split_stride;
    const float m = part[kHeadDim];
    const float weight = m == -INFINITY ? 0.0f : exp2f(m - total_max);
    total_sum += part[kHeadDim + 1] * weight;
    const float2 v = *reinterpret_cast<const float2*>(part + 2 * lane);
    a0 = fmaf(v.x, weight, a0);
    a1 = fmaf(v.y, weight, a1);
  }
  float denominator = total_sum;
  if (p.sinks != nullptr) {
    // the sink is one more column of the softmax with no value: add exp(sink - max)
    const int head_index = static_cast<int>(query_head % (p.kv_heads * kGroup));
    const float sink2 = p.sinks[head_index] * kLog2e;
    if (total_max == -INFINITY) {
      denominator = 1.0f;  // nothing visible: the sink takes all the weight, the output is 0
    } else {
      denominator += exp2f(sink2 - total_max);
    }
  }
  const float inverse = denominator > 0.0f ? 1.0f / denominator : 0.0f;
  T* out = static_cast<T*>(p.output) + query_head * kHeadDim + 2 * lane;
  *reinterpret_cast<uint32_t*>(out) = Elem<T>::pack2(a0 * inverse, a1 * inverse);
}

}  // namespace
}  // namespace nml_sm100

using namespace nml_sm100;

extern "C" size_t nml_sm100_paged_attention_decode_workspace_bytes(int64_t batch,
                                                                   int64_t query_heads,
                                                                   int64_t splits) {
  if (batch <= 0 || query_heads <= 0 || splits <= 0) return 0;
  return static_cast<size_t>(batch) * query_heads * splits * kPartialWidth * sizeof(float);
}

extern "C" int32_t nml_sm100_paged_attention_decode(const NmlSm100PagedAttentionDecode* request,
                                                    char* error_message,
                                                    size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100PagedAttentionDecode)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated paged attention request", error_message,
                error_message_capacity);
  }
  const NmlSm100PagedAttentionDecode& r = *request;
  if (r.query == nullptr || r.key_cache == nullptr || r.value_cache == nullptr ||
      r.page_table == nullptr || r.sequence_lengths == nullptr || r.output == nullptr ||
      r.workspace == nullptr || r.stream == nullptr || !fits_i32(r.batch) ||
      !fits_i32(r.kv_heads) || !fits_i32(r.physical_pages) || !fits_i32(r.table_width) ||
      r.splits <= 0 || r.splits > 64 || r.sliding_window < 0 || r.batch > 65535 ||
      r.kv_heads * static_cast<int64_t>(kGroup) != r.query_heads || r.head_dim != kHeadDim ||
      r.page_size != kPage || !(r.scale > 0.0f) ||
      reinterpret_cast<uintptr_t>(r.query) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(r.key_cache) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(r.value_cache) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(r.workspace) % 16 != 0) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "invalid paged attention request (this kernel takes head_dim 64, page size 16 "
                "and 8 query heads per kv head)",
                error_message, error_message_capacity);
  }
  if (r.workspace_bytes <
      nml_sm100_paged_attention_decode_workspace_bytes(r.batch, r.query_heads, r.splits)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "paged attention workspace is too small",
                error_message, error_message_capacity);
  }
  if (r.dtype != NML_SM100_F16 && r.dtype != NML_SM100_BF16) {
    return fail(NML_SM100_INVALID_ARGUMENT, "paged attention supports F16 and BF16 only",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  DecodeParams p = {};
  p.query = r.query;
  p.key_cache = r.key_cache;
  p.value_cache = r.value_cache;
  p.page_table = r.page_table;
  p.lengths = r.sequence_lengths;
  p.sinks = r.sinks;
  p.partial = static_cast<float*>(r.workspace);
  p.output = r.output;
  p.batch = static_cast<int>(r.batch);
  p.kv_heads = static_cast<int>(r.kv_heads);
  p.table_width = static_cast<int>(r.table_width);
  p.physical_pages = static_cast<int>(r.physical_pages);
  p.splits = static_cast<int>(r.splits);
  p.window = static_cast<int>(r.sliding_window);
  p.scale_log2 = r.scale * kLog2e;
  p.status = device->status_word;
  cudaStream_t stream = static_cast<cudaStream_t>(r.stream);
  const dim3 grid(static_cast<unsigned>(r.kv_heads), static_cast<unsigned>(r.batch),
                  static_cast<unsigned>(r.splits));
  const unsigned reduce_grid = static_cast<unsigned>((r.batch * r.query_heads + 3) / 4);
  if (r.dtype == NML_SM100_F16) {
    attention_decode_kernel<__half><<<grid, kWarps * 32, 0, stream>>>(p);
    attention_reduce_kernel<__half><<<reduce_grid, 128, 0, stream>>>(p);
  } else {
    attention_decode_kernel<__nv_bfloat16><<<grid, kWarps * 32, 0, stream>>>(p);
    attention_reduce_kernel<__nv_bfloat16><<<reduce_grid, 128, 0, stream>>>(p);
  }
  return launch_result(error_message, error_message_capacity);
}
