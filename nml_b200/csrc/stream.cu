// Host-side selection and launch of the weight-streaming kernel (stream_gemm.cuh): the dense
// linear at up to 64 activation rows (more than 16 only for weights that stay in L2, which
// are then streamed once per group of 16 rows) and the routed-expert projections of decode-size
// batches (at most 16 slots per schedule block).
#include <atomic>

#include "stream_gemm.cuh"

namespace nml_sm100 {
namespace {

using namespace stream;

// Opts one kernel instantiation into its dynamic shared memory once per device.
template <typename Kernel>
bool reserve(Kernel kernel, int device, std::atomic<int> (&configured)[64]) {
  if (device >= 0 && device < 64 && configured[device].load(std::memory_order_acquire)) {
    return true;
  }
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) !=
      cudaSuccess) {
    return false;
  }
  if (device >= 0 && device < 64) configured[device].store(1, std::memory_order_release);
  return true;
}

template <int NT, int UT, int RT, typename T, int MODE, bool FULL>
int32_t launch_variant(const Params& p, int smem_bytes, int64_t units_bound,
                       const DeviceInfo& device, cudaStream_t stream, char* message,
                       size_t capacity) {
  auto kernel = stream_kernel<NT, UT, RT, T, MODE, FULL>;
  static std::atomic<int> configured[64];
  if (!reserve(kernel, device.device, configured)) {
    return fail(NML_SM100_LAUNCH_FAILURE,
                "cannot reserve shared memory for the weight-streaming kernel", message,
                capacity);
  }
  const unsigned grid =
      static_cast<unsigned>(units_bound < device.sm_count ? units_bound : device.sm_count);
  const unsigned threads = static_cast<unsigned>((p.compute_warps + NT + 1) * 32);
  kernel<<<grid, threads, smem_bytes, stream>>>(p);
  return launch_result(message, capacity);
}

template <typename T, int MODE>
int32_t launch_for_shape(const Params& p, int nt, int rt, int smem_bytes, int64_t units_bound,
                         const DeviceInfo& device, cudaStream_t stream, char* message,
                         size_t capacity) {
#define NML_STREAM_VARIANT(NT, UT, RT, FULL)                                                  \
  launch_variant<NT, UT, RT, T, MODE, FULL>(p, smem_bytes, units_bound, device, stream,       \
                                            message, capacity)
#define NML_STREAM_TILE(UT, FULL)                                                             \
  (nt == 2 ? (rt == 2 ? NML_STREAM_VARIANT(2, UT, 2, FULL) : NML_STREAM_VARIANT(2, UT, 1, FULL)) \
           : (rt == 2 ? NML_STREAM_VARIANT(1, UT, 2, FULL) : NML_STREAM_VARIANT(1, UT, 1, FULL)))
  // Three variants: K units that split evenly into 3 per warp (K = 2880), evenly into 4 per
  // warp (K = 4096), and the guarded form for every other width; each for one or two
  // activation-row tiles and 16- or 32-row weight tiles.
  const bool even = p.compute_warps * p.units_per_warp == p.k_units;
  if (even && p.units_per_warp == 3) return NML_STREAM_TILE(3, true);
  if (even && p.units_per_warp == 4) return NML_STREAM_TILE(4, true);
  return NML_STREAM_TILE(4, false);
#undef NML_STREAM_TILE
#undef NML_STREAM_VARIANT
}

// 32-row tiles once every CTA walks at least this many 16-row tiles: the launch is then long
// enough for the per-tile bookkeeping to matter and coarse enough tiles still balance.
constexpr int64_t kLargeTileWalk = 6;

int tile_fragments(int64_t fragments, const DeviceInfo& device) {
  return fragments >= kLargeTileWalk * device.sm_count ? 2 : 1;
}

// The layout for the preferred tile height, or for 16-row tiles when the larger one does not
// leave two stages of shared memory (wide K with two activation-row tiles).
bool plan_tiles(int K, int nt, int* rt, Params* p, int* smem_bytes) {
  if (*rt == 2 && plan_layout(K, nt, 2, p, smem_bytes)) return true;
  *rt = 1;
  return plan_layout(K, nt, 1, p, smem_bytes);
}

bool aligned16(const void* pointer) { return reinterpret_cast<uintptr_t>(pointer) % 16 == 0; }

// Weights up to this many packed bytes stay in L2 between the passes of a launch that
// streams them once per group of 16 activation rows.
constexpr int64_t kResidentWeightBytes = 32ll << 20;
constexpr int kMaxStreamRows = 64;

}  // namespace

bool linear_stream_supported(const LinearArgs& args) {
  if (args.rows > kMaxStreamRows || args.inputs % kUnitK != 0 || args.inputs > 4 * 16 * kUnitK) {
    return false;
  }
  bool ok = aligned16(args.activation) && aligned16(args.payload) &&
            aligned16(args.block_scales) && args.outputs % 4 == 0;
  int64_t weight_bytes = static_cast<int64_t>(args.outputs) * (args.inputs / 2);
  for (int i = 0; i < args.extra_projections; ++i) {
    ok = ok && aligned16(args.extra[i].payload) && aligned16(args.extra[i].block_scales) &&
         args.extra[i].outputs % 4 == 0;
    weight_bytes += static_cast<int64_t>(args.extra[i].outputs) * (args.inputs / 2);
  }
  return ok && (args.rows <= 16 || weight_bytes <= kResidentWeightBytes);
}

int32_t launch_linear_stream(const LinearArgs& args, const DeviceInfo& device, char* message,
                             size_t capacity) {
  Params p = {};
  const int nt = args.rows <= 8 ? 1 : 2;
  int64_t fragments = (args.outputs + kFragmentRows - 1) / kFragmentRows;
  for (int i = 0; i < args.extra_projections; ++i) {
    fragments += (args.extra[i].outputs + kFragmentRows - 1) / kFragmentRows;
  }
  int rt = tile_fragments(fragments * ((args.rows + 15) / 16), device);
  int smem_bytes = 0;
  if (!plan_tiles(args.inputs, nt, &rt, &p, &smem_bytes)) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "the weight-streaming linear does not support this input width", message,
                capacity);
  }
  const int kTileRows = kFragmentRows * rt;
  p.x = args.activation;
  p.M = args.rows;
  p.segments = 1 + args.extra_projections;
  p.segment[0] = {args.payload, args.block_scales, args.global_scale, args.bias, args.output,
                  args.outputs, 0, args.residual};
  int tiles = (args.outputs + kTileRows - 1) / kTileRows;
  for (int i = 0; i < args.extra_projections; ++i) {
    const LinearArgs::Projection& e = args.extra[i];
    p.segment[1 + i] = {e.payload, e.block_scales, e.global_scale, e.bias, e.output, e.outputs,
                        tiles, nullptr};
    tiles += (e.outputs + kTileRows - 1) / kTileRows;
  }
  p.groups = (args.rows + 15) / 16;
  p.tiles_per_group = tiles;
  p.status = device.status_word;
  const int64_t units = static_cast<int64_t>(p.groups) * tiles;
  note_linear_kernel("stream", 16);
  if (args.dtype == NML_SM100_F16) {
    return launch_for_shape<__half, kDense>(p, nt, rt, smem_bytes, units, device, args.stream,
                                            message, capacity);
  }
  return launch_for_shape<__nv_bfloat16, kDense>(p, nt, rt, smem_bytes, units, device,
                                                 args.stream, message, capacity);
}

bool experts_stream_supported(const ExpertArgs& args) {
  const int64_t rows_per_expert = args.gate_up ? 2ll * args.outputs : args.outputs;
  return !args.slot_input && args.inputs % kUnitK == 0 && args.inputs <= 4 * 16 * kUnitK &&
         rows_per_expert % kFragmentRows == 0 &&
         args.experts * rows_per_expert <= std::numeric_limits<int32_t>::max() &&
         aligned16(args.payload) && aligned16(args.block_scales) && aligned16(args.input) &&
         // decode-size batches: at most one full schedule block per expert on average
         static_cast<int64_t>(args.live_routes > 0 ? args.live_routes : args.assignments) <=
             16ll * args.experts;
}

int32_t launch_experts_stream(const ExpertArgs& args, const DeviceInfo& device, char* message,
                              size_t capacity) {
  Params p = {};
  // sparse schedule form (one route per block, nml-ir/src/lib.rs:5696-5721): slot 0 only
  const int nt = args.assignments <= args.experts ? 1 : 2;  // (the plan's form follows all routes)
  const int rows_per_expert = args.gate_up ? 2 * args.outputs : args.outputs;
  // blocks with work: at most one per live route and at most ceil(routes / 16) + experts
  const int64_t live = args.live_routes > 0 ? args.live_routes : args.assignments;
  int64_t busy_blocks = nt == 1 ? live : live / 16 + args.experts;
  if (busy_blocks > args.schedule_blocks) busy_blocks = args.schedule_blocks;
  int rt = tile_fragments(busy_blocks * (rows_per_expert / kFragmentRows), device);
  int smem_bytes = 0;
  if (!plan_tiles(args.inputs, nt, &rt, &p, &smem_bytes)) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "the weight-streaming expert kernel does not support this input width", message,
                capacity);
  }
  const int kTileRows = kFragmentRows * rt;
  p.input = args.input;
  p.sorted_assignments = args.sorted_assignments;
  p.block_experts = args.block_experts;
  p.active_blocks = args.active_blocks;
  p.expert_offset = args.expert_offset;
  p.routing_weights = args.routing_weights;
  p.row_targets = args.row_targets;
  p.payload = args.payload;
  p.block_scales = args.block_scales;
  p.global_scale = args.global_scale;
  p.bias = args.bias;
  p.output = args.output;
  p.assignments = args.assignments;
  p.schedule_blocks = args.schedule_blocks;
  p.experts = args.experts;
  p.top_k = args.experts_per_token;
  p.rows_per_expert = rows_per_expert;
  p.N = args.outputs;
  p.groups = args.schedule_blocks;
  p.tiles_per_group = (p.rows_per_expert + kTileRows - 1) / kTileRows;
  p.status = device.status_word;
  const int64_t units = static_cast<int64_t>(p.groups) * p.tiles_per_group;
#define NML_STREAM_EXPERTS(T)                                                                  \
  (args.gate_up ? launch_for_shape<T, kGateUp>(p, nt, rt, smem_bytes, units, device,          \
                                               args.stream, message, capacity)                 \
                : launch_for_shape<T, kDown>(p, nt, rt, smem_bytes, units, device, args.stream, \
                                             message, capacity))
  if (args.dtype == NML_SM100_F16) return NML_STREAM_EXPERTS(__half);
  return NML_STREAM_EXPERTS(__nv_bfloat16);
#undef NML_STREAM_EXPERTS
}

}  // namespace nml_sm100
