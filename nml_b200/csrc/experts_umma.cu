// Grouped (routed-expert) NVFP4 projections on tcgen05: host-side launch of
// umma::gemm_kernel in gate/up and down mode.
//
// The schedule (16-slot blocks sorted by expert) is read on the device: each CTA derives the
// runs of blocks that share an expert and cuts them into units of BM slots x 128 weight
// rows, so the launch shape never depends on routing.  Activation rows are gathered by
// assignment (hidden[a / k] for gate/up, activated[a] for down) straight into the swizzled
// UMMA operand tile with 16-byte cp.async; there is no permuted copy of the tokens in HBM.
// Gate/up keeps the checkpoint's interleaved rows (2i = gate, 2i+1 = up): lane pairs of the
// epilogue exchange accumulators and write swiglu(gate, up) for intermediate column i.
#include <cstdlib>

#include "umma_gemm.cuh"

namespace nml_sm100 {
namespace {

using namespace umma;

constexpr int32_t kDoesNotFit = -1000;  // internal: the variant's shared memory exceeds the SM's

template <int BM, int KS, int PS, int XS, int WB, int DG, int MI, int PA, bool WT, int AFMT,
          typename T, int MODE, bool XTMA, bool SB = false>
int32_t launch_config(const ExpertArgs& args, const DeviceInfo& device, char* message,
                      size_t capacity) {
  using L = KernelLayout<BM, KS, PS, XS, WB, WT, AFMT, MODE, SB>;
  const int scale_buffer_bytes = (WT || SB) ? bulk_scale_buffer_bytes(args.inputs / 16) : 0;
  const int scale_buffers = L::kSmemBytes + 2 * scale_buffer_bytes > kSmemBudget ? 1 : 2;
  const int smem_bytes = L::kSmemBytes + scale_buffers * scale_buffer_bytes;
  if (smem_bytes > kSmemBudget) return kDoesNotFit;
  const int rows_per_expert = args.gate_up ? 2 * args.outputs : args.outputs;
  const int64_t weight_rows = static_cast<int64_t>(args.experts) * rows_per_expert;
  CUtensorMap tmap_payload, tmap_x;
  if (!encode_payload_map<KS>(&tmap_payload, args.payload, weight_rows, args.inputs)) {
    return fail(NML_SM100_LAUNCH_FAILURE, "tensor map encoding failed", message, capacity);
  }
  if constexpr (XTMA) {
    // rows of the input are schedule slots
    if (!encode_activation_map<T>(&tmap_x, args.input,
                                  static_cast<int64_t>(args.schedule_blocks) * 16, args.inputs,
                                  BM, KS)) {
      return fail(NML_SM100_LAUNCH_FAILURE, "tensor map encoding failed", message, capacity);
    }
  } else {
    tmap_x = tmap_payload;  // unused
  }
  Params p = {};
  p.block_scales = args.block_scales;
  p.global_scale = args.global_scale;
  p.bias = args.bias;
  p.scale_width = args.inputs / 16;
  p.weight_rows_total = static_cast<int>(weight_rows);
  p.rows_per_expert = rows_per_expert;
  p.M = 0;
  p.N = args.outputs;
  p.K = args.inputs;
  p.n_tiles = (rows_per_expert + kTileN - 1) / kTileN;
  p.m_tiles = 0;
  p.k_steps = args.inputs / kTileK;
  p.n_fastest = 1;
  p.output = args.output;
  p.input = args.input;
  p.sorted_assignments = args.sorted_assignments;
  p.block_experts = args.block_experts;
  p.active_blocks = args.active_blocks;
  p.expert_offset = args.expert_offset;
  p.routing_weights = args.routing_weights;
  p.row_targets = args.row_targets;
  p.assignments = args.assignments;
  p.schedule_blocks = args.schedule_blocks;
  p.experts = args.experts;
  p.top_k = args.experts_per_token;
  p.status = device.status_word;
  p.scale_buffer_bytes = scale_buffer_bytes;
  p.scale_stride = bulk_scale_stride(static_cast<int>(args.inputs / 16));
  p.scale_buffers = scale_buffers;
  p.split_k = 1;

  auto kernel = gemm_kernel<BM, KS, PS, XS, WB, DG, MI, PA, WT, AFMT, T, MODE, XTMA, SB>;
  static std::atomic<int> configured[64];
  if (!reserve_smem(kernel, (WT || SB) ? kSmemBudget : L::kSmemBytes, device.device,
                    configured)) {
    return fail(NML_SM100_LAUNCH_FAILURE, "cannot reserve shared memory for the tcgen05 experts",
                message, capacity);
  }
  // Upper bound of units: every block could open its own slot tile.
  const int64_t slot_tiles = args.schedule_blocks;
  const int64_t max_units = slot_tiles * p.n_tiles;
  const unsigned grid =
      static_cast<unsigned>(max_units < device.sm_count ? max_units : device.sm_count);
  kernel<<<grid, launch_threads<DG, MI, XTMA>(), smem_bytes, args.stream>>>(
      tmap_payload, tmap_x, p, tmap_payload, tmap_payload);
  return launch_result(message, capacity);
}

template <int AFMT, typename T, int MODE, bool XTMA>
int32_t launch_for_load(const ExpertArgs& args, const DeviceInfo& device, char* message,
                        size_t capacity) {
  // Expected slots per expert under balanced routing decide the slot-tile height.
  const int64_t routes = args.live_routes > 0 && args.live_routes < args.assignments
                             ? args.live_routes
                             : args.assignments;
  const int64_t average = routes <= args.experts ? 1 : (routes + args.experts - 1) / args.experts;
  // Decoded weights in tensor memory: every tile's block scales (128 rows x K/16 bytes) must
  // form a legal bulk copy and two such buffers must fit beside the rings.
  const int rows_per_expert = args.gate_up ? 2 * args.outputs : args.outputs;
  const bool tmem_weights = get_kernel_policy() != NML_SM100_POLICY_UMMA_SMEM &&
                            rows_per_expert % 4 == 0 &&
                            reinterpret_cast<uintptr_t>(args.block_scales) % 16 == 0;
  if (tmem_weights && average <= 160 && AFMT == kAbf16) {
    // bf16 operands through the byte table (32 KB of shared memory; slightly shallower rings)
    int32_t rc;
    if (average <= 16) {
      rc = launch_config<16, 4, 6, 4, 8, 2, 2, 8, true, kAbf16Lut, T, MODE, XTMA>(
          args, device, message, capacity);
    } else if (average <= 32) {
      rc = launch_config<32, 4, 4, 4, 8, 2, 1, 4, true, kAbf16Lut, T, MODE, XTMA>(
          args, device, message, capacity);
    } else if (average <= 64) {
      rc = launch_config<64, 4, 3, 2, 8, 2, 1, 2, true, kAbf16Lut, T, MODE, XTMA>(
          args, device, message, capacity);
    } else {
      rc = launch_config<128, 1, 8, 6, 6, 2, 1, 1, true, kAbf16Lut, T, MODE, XTMA>(
          args, device, message, capacity);
    }
    if (rc != kDoesNotFit) return rc;
  }
  if (tmem_weights && average <= 160) {
    int32_t rc;
    if (average <= 16) {
      rc = launch_config<16, 4, 6, 4, 8, 2, 2, 8, true, AFMT, T, MODE, XTMA>(args, device, message,
                                                                            capacity);
    } else if (average <= 32) {
      rc = launch_config<32, 4, 5, 4, 8, 2, 1, 4, true, AFMT, T, MODE, XTMA>(args, device, message,
                                                                            capacity);
    } else if (average <= 64) {
      rc = launch_config<64, 4, 3, 3, 8, 2, 1, 2, true, AFMT, T, MODE, XTMA>(args, device, message,
                                                                            capacity);
    } else {
      rc = launch_config<128, 1, 8, 8, 8, 2, 1, 1, true, AFMT, T, MODE, XTMA>(args, device,
                                                                             message, capacity);
    }
    if (rc != kDoesNotFit) return rc;
  }
  if (average <= 16) {
    return launch_config<16, 4, 5, 4, 4, 2, 2, 8, false, AFMT, T, MODE, XTMA>(args, device, message,
                                                                             capacity);
  }
  if (average <= 32) {
    return launch_config<32, 4, 4, 3, 4, 2, 2, 8, false, AFMT, T, MODE, XTMA>(args, device, message,
                                                                             capacity);
  }
  if (average <= 64) {
    return launch_config<64, 4, 3, 3, 4, 2, 1, 4, false, AFMT, T, MODE, XTMA>(args, device, message,
                                                                             capacity);
  }
  if (average <= 160) {
    return launch_config<128, 1, 6, 5, 5, 2, 1, 1, false, AFMT, T, MODE, XTMA>(args, device,
                                                                              message, capacity);
  }
  if constexpr (XTMA) {
    // slot-ordered input by TMA: no gather warps, so a third decode group fits, and the unit's
    // block scales come by bulk copy (the form the dense 256-row tile runs in)
    if (tmem_weights) {
      const int32_t rc = launch_config<256, 1, 4, 3, 4, 3, 1, 1, false, AFMT, T, MODE, XTMA, true>(
          args, device, message, capacity);
      if (rc != kDoesNotFit) return rc;
    }
  }
  return launch_config<256, 1, 4, 4, 4, 2, 1, 1, false, AFMT, T, MODE, XTMA>(args, device, message,
                                                                            capacity);
}

template <int MODE>
int32_t launch_mode(const ExpertArgs& args, const DeviceInfo& device, char* message,
                    size_t capacity) {
  if (args.slot_input) {
    if (args.dtype == NML_SM100_F16) {
      return launch_for_load<kAf16, __half, MODE, true>(args, device, message, capacity);
    }
    return launch_for_load<kAbf16, __nv_bfloat16, MODE, true>(args, device, message, capacity);
  }
  if (args.dtype == NML_SM100_F16) {
    return launch_for_load<kAf16, __half, MODE, false>(args, device, message, capacity);
  }
  return launch_for_load<kAbf16, __nv_bfloat16, MODE, false>(args, device, message, capacity);
}

}  // namespace

bool experts_umma_supported(const ExpertArgs& args) {
  const int64_t rows_per_expert = args.gate_up ? 2ll * args.outputs : args.outputs;
  return args.inputs % kTileK == 0 && args.experts <= kMaxGroups &&
         args.experts * rows_per_expert <= std::numeric_limits<int32_t>::max() &&
         reinterpret_cast<uintptr_t>(args.payload) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(args.input) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(args.block_scales) % 4 == 0;
}

int32_t launch_experts_umma(const ExpertArgs& args, const DeviceInfo& device, char* message,
                            size_t capacity) {
  return args.gate_up ? launch_mode<kGateUp>(args, device, message, capacity)
                      : launch_mode<kDown>(args, device, message, capacity);
}

}  // namespace nml_sm100
