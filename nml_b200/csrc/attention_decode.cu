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
// online per warp (running maximum and sum per head); the probabilities, narrowed to the
// cache's 16-bit type, pass through a small shared-memory tile into B fragments, and P.V is
// four more mma.sync: out^T [64 dimensions x 8 heads] += V_page^T [64 x 16] . P [16 x 8], the
// value page staged in shared memory by cp.async one page ahead and read transposed with
// ldmatrix.  Warps merge in shared memory, splits through a caller-provided f32 scratch that a
// second small kernel reduces (applying the sink) into the 16-bit output.
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

// Four 8x8 16-bit matrices from shared memory, transposed: with the rows of a value tile
// [token][dimension] as matrix rows, lane (g, c) receives (V[2c][g], V[2c + 1][g]) of each
// matrix, which is the A fragment of mma.sync for a [dimension x token] operand.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row_address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(row_address))));
}

// 16-byte asynchronous copy into shared memory; zeros instead when `valid` is false.
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const uint32_t size = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                   static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
               "l"(src), "r"(size)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kValueStride = kHeadDim + 8;  // elements per token row of a staged value page
constexpr int kProbabilityStride = 24;      // 16 tokens + padding: conflict-free fragment reads

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attention_decode_kernel(const DecodeParams p) {
  constexpr bool kHalf = std::is_same<T, __half>::value;
  const int head = blockIdx.x;   // kv head
  const int b = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  // per warp: two staged value pages and one page of probabilities [head][token] (16 bit)
  __shared__ __align__(16) T values[kWarps][2][kPage][kValueStride];
  __shared__ __align__(16) T probability[kWarps][kGroup][kProbabilityStride];
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
  // Running state of this lane: statistics of heads 2 c and 2 c + 1 (replicated over g), and
  // the output as mma.sync accumulators [dimension x head]: block i holds dimensions
  // 16 i + g (registers 0, 1) and 16 i + g + 8 (registers 2, 3) of heads 2 c and 2 c + 1.
  float running_max[2] = {-INFINITY, -INFINITY};
  float running_sum[2] = {0.0f, 0.0f};
  float out[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i][0] = out[i][1] = out[i][2] = out[i][3] = 0.0f;

  const int64_t token_stride = static_cast<int64_t>(p.kv_heads) * kHeadDim;  // elements
  // physical page of a logical one; a bad entry is reported and replaced by page 0, whose
  // scores are then computed like any other (the table is the caller's to keep valid)
  auto page_base_of = [&](int page) -> int64_t {
    int32_t physical = p.page_table[static_cast<int64_t>(b) * p.table_width + page];
    if (physical < 0 || physical >= p.physical_pages) {
      if (lane == 0) atomicOr(p.status, NML_SM100_STATUS_INDEX_RANGE);
      physical = 0;
    }
    return (static_cast<int64_t>(physical) * kPage) * token_stride +
           static_cast<int64_t>(head) * kHeadDim;
  };
  // Stage the values of a page: 16 token rows of 128 bytes, four 16-byte pieces per lane.
  // Rows of tokens outside the visible range become zeros: their probabilities are zero, but
  // whatever an unwritten cache slot holds (a NaN pattern, say) must not meet the product.
  auto stage_values = [&](int buffer, int logical_page, int64_t page_base) {
    const T* value = static_cast<const T*>(p.value_cache) + page_base;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int piece = lane + 32 * i;
      const int token = piece >> 3, part = piece & 7;
      const int position = logical_page * kPage + token;
      cp_async_16(&values[warp][buffer][token][8 * part], value + token * token_stride + 8 * part,
                  position >= first_token && position < length);
    }
    cp_async_commit();
  };

  int buffer = 0;
  int page = page_begin + warp;
  int64_t page_base = 0;
  if (page < page_end) {
    page_base = page_base_of(page);
    stage_values(0, page, page_base);
  }
  for (; page < page_end; page += kWarps, buffer ^= 1) {
    // keys of tokens g and g + 8, dimensions 16 c .. 16 c + 15
    const T* key = static_cast<const T*>(p.key_cache) + page_base + 16 * c;
    const uint4 k_lo_g = *reinterpret_cast<const uint4*>(key + g * token_stride);
    const uint4 k_hi_g = *reinterpret_cast<const uint4*>(key + g * token_stride + 8);
    const uint4 k_lo_h = *reinterpret_cast<const uint4*>(key + (g + 8) * token_stride);
    const uint4 k_hi_h = *reinterpret_cast<const uint4*>(key + (g + 8) * token_stride + 8);
    // the next page's values start moving before this page is worked on
    const int next = page + kWarps;
    int64_t next_base = 0;
    if (next < page_end) {
      next_base = page_base_of(next);
      stage_values(buffer ^ 1, next, next_base);
    }
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // tokens g (s0, s1) and g + 8 (s2, s3), heads 2c, 2c+1
    if constexpr (kHalf) {
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
    // probabilities are narrowed to the cache's 16-bit type for the second product; the
    // running sum adds the narrowed values, so numerator and denominator stay consistent
    const T n0 = Elem<T>::store(exp2f(s[0] - base0)), n1 = Elem<T>::store(exp2f(s[1] - base1));
    const T n2 = Elem<T>::store(exp2f(s[2] - base0)), n3 = Elem<T>::store(exp2f(s[3] - base1));
    float page_sum[2] = {Elem<T>::load(n0) + Elem<T>::load(n2),
                         Elem<T>::load(n1) + Elem<T>::load(n3)};
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
    __syncwarp();  // the previous page's fragment reads are done
    probability[warp][2 * c][g] = n0;
    probability[warp][2 * c + 1][g] = n1;
    probability[warp][2 * c][g + 8] = n2;
    probability[warp][2 * c + 1][g + 8] = n3;
    // this page's values have landed (the next page's copy may still be in flight)
    if (next < page_end) {
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    // out[dimension, head] = rescale * out + V^T [dimension x token] . P [token x head]
    const uint32_t p_lo = *reinterpret_cast<const uint32_t*>(&probability[warp][g][2 * c]);
    const uint32_t p_hi = *reinterpret_cast<const uint32_t*>(&probability[warp][g][2 * c + 8]);
    const int matrix = lane >> 3, matrix_row = lane & 7;
    const T* tile_row = &values[warp][buffer][(matrix >> 1) * 8 + matrix_row][(matrix & 1) * 8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[i][0] *= rescale[0];
      out[i][1] *= rescale[1];
      out[i][2] *= rescale[0];
      out[i][3] *= rescale[1];
      uint32_t a[4];
      ldmatrix_x4_trans(a, tile_row + 16 * i);
      if constexpr (kHalf) {
        mma_f16(out[i], a[0], a[1], a[2], a[3], p_lo, p_hi);
      } else {
        mma_bf16(out[i], a[0], a[1], a[2], a[3], p_lo, p_hi);
      }
    }
    page_base = next_base;
  }

  // ---- merge the four warps, then write this split's partial result -----------------------
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    merged[warp][2 * c][16 * i + g] = out[i][0];
    merged[warp][2 * c + 1][16 * i + g] = out[i][1];
    merged[warp][2 * c][16 * i + g + 8] = out[i][2];
    merged[warp][2 * c + 1][16 * i + g + 8] = out[i][3];
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
