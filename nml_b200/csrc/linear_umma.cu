// Dense NVFP4 linear on tcgen05: host-side tile selection and launch of umma::gemm_kernel
// in dense mode.  Y[M, N] = X[M, K] . W[N, K]^T * g (+ bias).
//
// Tile height BM (activation rows per tile = UMMA N) follows M; for M > 64 the choice
// between 64, 128 and 256 minimises waves x per-tile time on the device's SM count.  Small
// tiles (decode shapes, HBM-bound) use raw stages of four K steps so that ~100 KB of packed
// weight bytes are in flight per SM; large tiles are MMA-bound and use one K step per stage.
#include "umma_gemm.cuh"

namespace nml_sm100 {
namespace {

using namespace umma;


constexpr int32_t kDoesNotFit = -1000;  // internal: the variant's shared memory exceeds the SM's

template <int BM, int KS, int PS, int XS, int WB, int DG, int MI, int PA, bool WT, int AFMT,
          typename T, bool SB = false>
int32_t launch_config(const LinearArgs& args, const DeviceInfo& device, char* message,
                      size_t capacity) {
  using L = KernelLayout<BM, KS, PS, XS, WB, WT, AFMT, kDense, SB>;
  const int scale_buffer_bytes = (WT || SB) ? bulk_scale_buffer_bytes(args.inputs / 16) : 0;
  // Few tiles and few rows (decode shapes of the 2880-class weights): cut K over a cluster so
  // that more SMs stream the weights.  One unit per cluster, at least 8 K steps per CTA.
  int total_tiles = (args.outputs + kTileN - 1) / kTileN;
  for (int i = 0; i < args.extra_projections; ++i) {
    total_tiles += (args.extra[i].outputs + kTileN - 1) / kTileN;
  }
  int split_k = 1;
  if (BM <= 32 && args.rows <= BM && get_kernel_policy() != NML_SM100_POLICY_NO_SPLIT_K) {
    const int k_steps = args.inputs / kTileK;
    while (split_k < 4 && total_tiles * (split_k + 1) <= device.sm_count &&
           k_steps / (split_k + 1) >= 8) {
      ++split_k;
    }
  }
  // Two scale buffers let the next unit's scales land while this one is decoded; when they do
  // not fit (K = 4096) one buffer does: the decode of a unit's first K step then waits for the
  // copy, once per unit, which costs far less than giving up an activation stage.
  int scale_buffers = 2;
  if (L::kSmemBytes + 2 * scale_buffer_bytes > kSmemBudget) scale_buffers = 1;
  int smem_bytes = L::kSmemBytes + scale_buffers * scale_buffer_bytes;
  // rank 0 keeps the f32 partial tiles of the other ranks behind the scale buffers: step the
  // split down until they fit instead of giving it up
  while (split_k > 1 && smem_bytes + (split_k - 1) * kTileN * BM * 4 > kSmemBudget) --split_k;
  if (split_k > 1) smem_bytes += (split_k - 1) * kTileN * BM * 4;
  if (smem_bytes > kSmemBudget) return kDoesNotFit;
  CUtensorMap tmap_payload, tmap_x, tmap_extra[2];
  if (!encode_payload_map<KS>(&tmap_payload, args.payload, args.outputs, args.inputs) ||
      !encode_activation_map<T>(&tmap_x, args.activation, args.rows, args.inputs, BM, KS)) {
    return fail(NML_SM100_LAUNCH_FAILURE, "tensor map encoding failed", message, capacity);
  }
  tmap_extra[0] = tmap_extra[1] = tmap_payload;
  for (int i = 0; i < args.extra_projections; ++i) {
    if (!encode_payload_map<KS>(&tmap_extra[i], args.extra[i].payload, args.extra[i].outputs,
                                args.inputs)) {
      return fail(NML_SM100_LAUNCH_FAILURE, "tensor map encoding failed", message, capacity);
    }
  }
  Params p = {};
  p.block_scales = args.block_scales;
  p.global_scale = args.global_scale;
  p.bias = args.bias;
  p.scale_width = args.inputs / 16;
  p.weight_rows_total = args.outputs;
  p.rows_per_expert = args.outputs;
  p.M = args.rows;
  p.N = args.outputs;
  p.K = args.inputs;
  p.split_k = split_k;
  p.tile_scale = args.tile_scale;
  p.gate = args.gate;
  p.gate_when = args.gate_when;
  p.segments = 1 + args.extra_projections;
  p.segment[0] = {args.block_scales, args.global_scale, args.bias, args.output, args.outputs, 0,
                  args.residual};
  p.n_tiles = (args.outputs + kTileN - 1) / kTileN;
  int64_t weight_bytes = static_cast<int64_t>(args.outputs) * (args.inputs / 2);
  for (int i = 0; i < args.extra_projections; ++i) {
    const LinearArgs::Projection& e = args.extra[i];
    p.segment[1 + i] = {e.block_scales, e.global_scale, e.bias, e.output, e.outputs, p.n_tiles,
                        nullptr};
    p.n_tiles += (e.outputs + kTileN - 1) / kTileN;
    weight_bytes += static_cast<int64_t>(e.outputs) * (args.inputs / 2);
  }
  p.m_tiles = (args.rows + BM - 1) / BM;
  p.k_steps = args.inputs / kTileK;
  // Walk n fastest when the packed weights stay L2-resident (activations stream once);
  // otherwise walk m fastest so the large weight tensor streams once.
  p.n_fastest = weight_bytes <= (32ll << 20) ? 1 : 0;
  // m fastest over more activations than stay in L2 beside the weight stream: walk them in
  // blocks; the weights then stream once per block, which costs little (0.33 GB per block
  // against 16 ms of arithmetic at M = 16384).  Measured on the vocabulary projection: up to
  // 24 MB of activations (M = 4096) one block is fastest (1271-1339 TFLOP/s against 1235-1263
  // in blocks of 12 MB); at 94 MB (M = 16384) blocks of 12 MB give 1232-1324, of 24 MB
  // 1145-1262, of 6 MB 1203-1315, of 3 MB 1194-1256, one block about 1085.
  const int64_t tile_bytes = static_cast<int64_t>(BM) * args.inputs * 2;
  int m_block = 1;  // the largest power of two of row tiles within 12 MB
  while (2 * m_block * tile_bytes <= (12ll << 20)) m_block *= 2;
  p.m_block = (!p.n_fastest && p.m_tiles * tile_bytes > (24ll << 20) && split_k == 1) ? m_block : 0;
  p.output = args.output;
  p.status = device.status_word;
  p.scale_buffer_bytes = scale_buffer_bytes;
  p.scale_stride = bulk_scale_stride(static_cast<int>(args.inputs / 16));
  p.scale_buffers = scale_buffers;

  auto kernel = gemm_kernel<BM, KS, PS, XS, WB, DG, MI, PA, WT, AFMT, T, kDense, true, SB>;
  static std::atomic<int> configured[64];
  if (!reserve_smem(kernel, kSmemBudget, device.device, configured)) {
    return fail(NML_SM100_LAUNCH_FAILURE, "cannot reserve shared memory for the tcgen05 linear",
                message, capacity);
  }
  const int64_t tiles = static_cast<int64_t>(p.n_tiles) * p.m_tiles;
  const unsigned grid = static_cast<unsigned>(tiles < device.sm_count ? tiles : device.sm_count);
  if (split_k > 1) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(tiles) * split_k);
    config.blockDim = dim3(launch_threads<DG, MI, true>());
    config.dynamicSmemBytes = smem_bytes;
    config.stream = args.stream;
    cudaLaunchAttribute cluster;
    cluster.id = cudaLaunchAttributeClusterDimension;
    cluster.val.clusterDim.x = split_k;
    cluster.val.clusterDim.y = 1;
    cluster.val.clusterDim.z = 1;
    config.attrs = &cluster;
    config.numAttrs = 1;
    if (cudaLaunchKernelEx(&config, kernel, tmap_payload, tmap_x, p, tmap_extra[0],
                           tmap_extra[1]) != cudaSuccess) {
      return launch_result(message, capacity);
    }
  } else {
    kernel<<<grid, launch_threads<DG, MI, true>(), smem_bytes, args.stream>>>(
        tmap_payload, tmap_x, p, tmap_extra[0], tmap_extra[1]);
  }
  if (args.gate != nullptr && args.gate_when != 0) return launch_result(message, capacity);
  note_linear_kernel(WT ? (AFMT == kAf16      ? "umma_tmem_weights_af16"
                           : AFMT == kAbf16Lut ? "umma_tmem_weights_abf16_lut"
                                               : "umma_tmem_weights_abf16")
                        : args.tile_scale != nullptr ? "umma_swapab_narrowed_af16"
                        : (AFMT == kAf16 ? "umma_swapab_af16" : "umma_swapab_abf16"), BM);
  return launch_result(message, capacity);
}

// `wide` allows the 192-row tile (decoded weights in tensor memory leave room for two
// 192-column accumulators, not for two of 256).
int choose_tile_rows(int rows, int outputs, int sm_count, bool wide) {
  if (rows <= 16) return 16;
  if (rows <= 32) return 32;
  if (rows <= 64) return 64;
  const int n_tiles = (outputs + kTileN - 1) / kTileN;
  // relative time of one K step of a tile: decode-bound for few rows, MMA-bound beyond
  // measured time of one K step of a tile (2880 -> 5760 at M = 16384, relative units)
  const int candidates[4] = {64, 128, 192, 256};
  const int step_cost[4] = {137, wide ? 156 : 190, 180, 228};
  int best = 256;
  int64_t best_cost = -1;
  for (int i = 0; i < 4; ++i) {
    const int bm = candidates[i];
    if (bm == 192 && !wide) continue;
    if (bm > 64 && rows <= bm / 2) continue;
    const int64_t tiles = static_cast<int64_t>(n_tiles) * ((rows + bm - 1) / bm);
    const int64_t waves = (tiles + sm_count - 1) / sm_count;
    const int64_t cost = waves * step_cost[i];
    if (best_cost < 0 || cost < best_cost || (cost == best_cost && bm > best)) {
      best = bm;
      best_cost = cost;
    }
  }
  return best;
}

// BF16 activations of a wide weight, narrowed once per call to F16 so that the weights decode
// with cvt.rn.f16x2.e2m1x2 / e4m3x2 instead of the integer sequences of the BF16 decode (the
// decode warps bound the 256-row tile).  Every tile of 256 rows is multiplied by one power of
// two that puts its largest magnitude into [2^14, 2^15); the inverse power multiplies the
// tile's f32 sums.  F16 then holds every element down to 2^-28 of the tile's largest exactly
// and rounds smaller ones at 2^-39 of it.  The narrowed kernel is used only when that is far
// below the rounding of the f32 sums for every row: each row's largest magnitude must lie
// within 2^8 of its tile's (rows of zeros aside), the tile must be finite and not tiny.  If
// any row fails, the verdict word is raised and the BF16-operand kernel, launched behind the
// narrowed one, produces the output instead; each of the two returns at once when the word
// names the other.
constexpr int kNarrowTileRows = 256;

// largest 15-bit magnitude of every row; block 0 clears the verdict
__global__ void __launch_bounds__(256)
row_magnitude_kernel(const __nv_bfloat16* __restrict__ x, uint32_t* __restrict__ row_magnitude,
                     uint32_t* __restrict__ verdict, int inputs) {
  const int64_t row = blockIdx.x;
  const uint4* source = reinterpret_cast<const uint4*>(x + row * inputs);
  __shared__ uint32_t warp_max[8];
  uint32_t magnitude = 0;
  for (int i = threadIdx.x; i < inputs / 8; i += blockDim.x) {
    const uint4 q = __ldg(source + i);
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      magnitude = max(magnitude, max(words[w] & 0x7fffu, (words[w] >> 16) & 0x7fffu));
    }
  }
#pragma unroll
  for (int offset = 16; offset != 0; offset >>= 1) {
    magnitude = max(magnitude, __shfl_xor_sync(0xffffffffu, magnitude, offset));
  }
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = magnitude;
  __syncthreads();
  if (threadIdx.x == 0) {
    magnitude = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) magnitude = max(magnitude, warp_max[w]);
    row_magnitude[row] = magnitude;
    if (row == 0) *verdict = 0u;
  }
}

__global__ void __launch_bounds__(256)
narrow_rows_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ row_magnitude,
                   __half* __restrict__ narrowed, float* __restrict__ tile_scale,
                   uint32_t* __restrict__ verdict, int rows, int inputs) {
  const int row = blockIdx.x;
  const int tile = row / kNarrowTileRows;
  __shared__ uint32_t warp_max[8];
  const int peer = tile * kNarrowTileRows + static_cast<int>(threadIdx.x);
  uint32_t magnitude = peer < rows ? row_magnitude[peer] : 0u;
#pragma unroll
  for (int offset = 16; offset != 0; offset >>= 1) {
    magnitude = max(magnitude, __shfl_xor_sync(0xffffffffu, magnitude, offset));
  }
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = magnitude;
  __syncthreads();
  magnitude = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) magnitude = max(magnitude, warp_max[w]);
  const int tile_exponent = static_cast<int>(magnitude >> 7);  // biased, 0..255
  const int shift = tile_exponent - 127 - 14;                  // tile's largest -> [2^14, 2^15)
  if (threadIdx.x == 0) {
    const uint32_t own = row_magnitude[row];
    const int own_exponent = static_cast<int>(own >> 7);
    const bool tile_ok = magnitude == 0u || (tile_exponent != 255 && tile_exponent >= 16);
    const bool row_ok = own == 0u || own_exponent >= tile_exponent - 8;
    if (!tile_ok || !row_ok) atomicOr(verdict, 1u);
    if (row % kNarrowTileRows == 0) {
      tile_scale[tile] = magnitude == 0u || !tile_ok
                             ? 1.0f
                             : __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);
    }
  }
  if (magnitude != 0u && (tile_exponent == 255 || tile_exponent < 16)) return;  // verdict raised
  // (a tile of zeros is written as zeros)
  const float down =
      magnitude == 0u ? 1.0f : __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
  const uint4* source = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * inputs);
  uint4* target = reinterpret_cast<uint4*>(narrowed + static_cast<int64_t>(row) * inputs);
  for (int i = threadIdx.x; i < inputs / 8; i += blockDim.x) {
    const uint4 q = __ldg(source + i);
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
    uint32_t packed[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const __half2 h = __floats2half2_rn(__uint_as_float(words[w] << 16) * down,
                                          __uint_as_float(words[w] & 0xffff0000u) * down);
      packed[w] = *reinterpret_cast<const uint32_t*>(&h);
    }
    target[i] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

// Rows and outputs from which the narrowing passes pay: they move 6 bytes per activation
// element, the projection 2 * outputs flops.
constexpr int64_t kNarrowMinRows = 512;
constexpr int64_t kNarrowMinOutputs = 16384;

struct NarrowWorkspace {
  size_t magnitudes, tile_scales, verdict, total;
};

NarrowWorkspace narrow_workspace(int64_t rows, int64_t inputs) {
  auto align = [](size_t v) { return (v + 255) / 256 * 256; };
  NarrowWorkspace w;
  w.magnitudes = align(static_cast<size_t>(rows) * inputs * 2);
  w.tile_scales = w.magnitudes + align(static_cast<size_t>(rows) * 4);
  w.verdict = w.tile_scales +
              align(static_cast<size_t>((rows + kNarrowTileRows - 1) / kNarrowTileRows) * 4);
  w.total = w.verdict + 256;
  return w;
}

template <int AFMT, typename T>
int32_t launch_for_rows(const LinearArgs& args, const DeviceInfo& device, char* message,
                        size_t capacity) {
  // Decoded weights in tensor memory: the unit's block scales (128 rows x K/16 bytes) must
  // form a legal bulk copy and two such buffers must fit beside the rings.
  const int policy = get_kernel_policy();
  bool bulk_scales_legal = args.outputs % 4 == 0 &&
                           reinterpret_cast<uintptr_t>(args.block_scales) % 16 == 0;
  int total_outputs = args.outputs;
  for (int i = 0; i < args.extra_projections; ++i) {
    bulk_scales_legal = bulk_scales_legal && args.extra[i].outputs % 4 == 0 &&
                        reinterpret_cast<uintptr_t>(args.extra[i].block_scales) % 16 == 0;
    total_outputs += args.extra[i].outputs;
  }
  const bool tmem_weights = policy != NML_SM100_POLICY_UMMA_SMEM && bulk_scales_legal;
  if (tmem_weights && AFMT == kAbf16) {
    // bf16 operands through the byte table (32 KB of shared memory; slightly shallower rings)
    int32_t rc = kDoesNotFit;
    switch (choose_tile_rows(args.rows, total_outputs, device.sm_count, true)) {
      case 16:
        rc = launch_config<16, 4, 6, 4, 8, 3, 2, 8, true, kAbf16Lut, T>(args, device, message,
                                                                        capacity);
        break;
      case 32:
        rc = launch_config<32, 4, 5, 4, 8, 3, 2, 4, true, kAbf16Lut, T>(args, device, message,
                                                                        capacity);
        break;
      case 64:
        rc = launch_config<64, 4, 3, 2, 8, 3, 2, 2, true, kAbf16Lut, T>(args, device, message,
                                                                        capacity);
        break;
      case 128:
        rc = launch_config<128, 1, 8, 6, 6, 4, 1, 1, true, kAbf16Lut, T>(args, device, message,
                                                                         capacity);
        break;
      case 192:
        rc = launch_config<192, 1, 6, 4, 4, 3, 1, 1, true, kAbf16Lut, T>(args, device, message,
                                                                         capacity);
        break;
      default:
        break;
    }
    if (rc != kDoesNotFit) return rc;
  }
  if (tmem_weights) {
    int32_t rc = kDoesNotFit;
    switch (choose_tile_rows(args.rows, total_outputs, device.sm_count, true)) {
      case 16:
        rc = launch_config<16, 4, 6, 4, 8, 3, 2, 8, true, AFMT, T>(args, device, message, capacity);
        break;
      case 32:
        rc = launch_config<32, 4, 5, 4, 8, 3, 1, 4, true, AFMT, T>(args, device, message, capacity);
        break;
      case 64:
        rc = launch_config<64, 4, 3, 3, 8, 3, 1, 2, true, AFMT, T>(args, device, message, capacity);
        break;
      case 128:
        rc = launch_config<128, 1, 8, 8, 8, 4, 1, 1, true, AFMT, T>(args, device, message,
                                                                    capacity);
        break;
      case 192:
        rc = launch_config<192, 1, 6, 6, 4, 3, 1, 1, true, AFMT, T>(args, device, message,
                                                                    capacity);
        break;
      default:
        break;
    }
    if (rc != kDoesNotFit) return rc;
  }
  switch (choose_tile_rows(args.rows, total_outputs, device.sm_count, false)) {
    case 16:
      return launch_config<16, 4, 5, 4, 4, 3, 1, 8, false, AFMT, T>(args, device, message,
                                                                    capacity);
    case 32:
      return launch_config<32, 4, 4, 3, 4, 3, 1, 8, false, AFMT, T>(args, device, message,
                                                                    capacity);
    case 64:
      return launch_config<64, 4, 3, 3, 4, 3, 1, 4, false, AFMT, T>(args, device, message,
                                                                    capacity);
    case 128:
      return launch_config<128, 1, 8, 5, 5, 3, 1, 1, false, AFMT, T>(args, device, message,
                                                                     capacity);
    default: {
      LinearArgs plain = args;
      if constexpr (AFMT == kAbf16) {
        // wide weight, many rows, scratch given: F16 operands, with the BF16-operand kernel
        // behind it for inputs the narrowing does not hold (see narrow_rows_kernel)
        const size_t wanted = linear_umma_workspace_bytes(args.rows, args.outputs, args.inputs,
                                                          args.dtype);
        if (wanted != 0 && args.workspace_bytes >= wanted && bulk_scales_legal &&
            policy == NML_SM100_POLICY_AUTO && args.extra_projections == 0 &&
            reinterpret_cast<uintptr_t>(args.workspace) % 256 == 0 &&
            KernelLayout<256, 1, 4, 3, 4, false, kAf16, kDense, true>::kSmemBytes +
                    2 * bulk_scale_buffer_bytes(args.inputs / 16) <= kSmemBudget) {
          const NarrowWorkspace w = narrow_workspace(args.rows, args.inputs);
          uint8_t* base = static_cast<uint8_t*>(args.workspace);
          __half* narrowed = reinterpret_cast<__half*>(base);
          uint32_t* magnitudes = reinterpret_cast<uint32_t*>(base + w.magnitudes);
          float* tile_scales = reinterpret_cast<float*>(base + w.tile_scales);
          uint32_t* verdict = reinterpret_cast<uint32_t*>(base + w.verdict);
          const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(args.activation);
          row_magnitude_kernel<<<static_cast<unsigned>(args.rows), 256, 0, args.stream>>>(
              x, magnitudes, verdict, args.inputs);
          narrow_rows_kernel<<<static_cast<unsigned>(args.rows), 256, 0, args.stream>>>(
              x, magnitudes, narrowed, tile_scales, verdict, args.rows, args.inputs);
          LinearArgs narrowed_args = args;
          narrowed_args.activation = narrowed;
          narrowed_args.tile_scale = tile_scales;
          narrowed_args.gate = verdict;
          narrowed_args.gate_when = 0;
          const int32_t rc = launch_config<256, 1, 4, 3, 4, 3, 1, 1, false, kAf16, T, true>(
              narrowed_args, device, message, capacity);
          if (rc != NML_SM100_OK && rc != kDoesNotFit) return rc;
          if (rc == NML_SM100_OK) {
            plain.gate = verdict;
            plain.gate_when = 1;
          }
        }
      }
      // Wide K (4096): the shared-memory ring variant has room for one scale buffer only; the
      // tensor-memory variant (one accumulator set beside eight W' tiles, byte-table decode)
      // measured 9 % faster there, and equal or slower at K = 2880.
      if constexpr (AFMT == kAbf16) {
        using Ring = KernelLayout<256, 1, 4, 3, 4, false, AFMT, kDense, true>;
        if (bulk_scales_legal && policy != NML_SM100_POLICY_UMMA_SMEM &&
            Ring::kSmemBytes + 2 * bulk_scale_buffer_bytes(args.inputs / 16) > kSmemBudget) {
          const int32_t rc = launch_config<256, 1, 4, 4, 8, 3, 1, 1, true, kAbf16Lut, T>(
              plain, device, message, capacity);
          if (rc != kDoesNotFit) return rc;
        }
      }
      // 256-row tiles: scales by bulk copy when the copy is legal and a buffer (two up to
      // K ~ 2900) fits beside three activation stages; else per-stage 4-byte copies
      if (bulk_scales_legal) {
        int32_t rc = launch_config<256, 1, 4, 3, 4, 3, 1, 1, false, AFMT, T, true>(
            plain, device, message, capacity);
        if (rc != kDoesNotFit) return rc;
      }
      return launch_config<256, 1, 6, 4, 4, 3, 1, 1, false, AFMT, T>(plain, device, message,
                                                                     capacity);
    }
  }
}

}  // namespace

bool linear_umma_supported(const LinearArgs& args) {
  bool ok = args.inputs % kTileK == 0 && reinterpret_cast<uintptr_t>(args.payload) % 16 == 0 &&
            reinterpret_cast<uintptr_t>(args.activation) % 16 == 0 &&
            reinterpret_cast<uintptr_t>(args.block_scales) % 4 == 0;
  for (int i = 0; i < args.extra_projections; ++i) {
    ok = ok && reinterpret_cast<uintptr_t>(args.extra[i].payload) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(args.extra[i].block_scales) % 4 == 0;
  }
  return ok;
}

size_t linear_umma_workspace_bytes(int64_t rows, int64_t outputs, int64_t inputs,
                                   int32_t dtype) {
  if (dtype != NML_SM100_BF16 || rows < kNarrowMinRows || outputs < kNarrowMinOutputs ||
      inputs % kTileK != 0) {
    return 0;
  }
  return narrow_workspace(rows, inputs).total;
}

size_t linear_umma_workspace_verdict_offset(int64_t rows, int64_t inputs) {
  return narrow_workspace(rows, inputs).verdict;
}

int32_t launch_linear_umma(const LinearArgs& args, const DeviceInfo& device, char* message,
                           size_t capacity) {
  // The decoded operand shares the activation format: tcgen05.mma kind::f16 with A = f16 and
  // B = bf16 raises an illegal instruction on sm_100a.
  if (args.dtype == NML_SM100_F16) {
    return launch_for_rows<kAf16, __half>(args, device, message, capacity);
  }
  return launch_for_rows<kAbf16, __nv_bfloat16>(args, device, message, capacity);
}

}  // namespace nml_sm100
