// NVFP4 linear on the 5th-generation tensor cores (tcgen05 + TMEM), weights stationary.
//
//   Y[M, N] = X[M, K] . W[N, K]^T * g (+ bias)
//
// The MMA is issued "swapped": the 128-row UMMA M dimension carries a tile of weight rows
// (n), the UMMA N dimension (16..256) carries activation rows (m).  A tile of packed
// weights is therefore decoded exactly once per K step whatever M is, and small M (decode)
// costs no padding of the 128-wide dimension.
//
// Per K step of 64 (one pipeline stage):
//   warp 0      producer   TMA: payload tile [128 x 32 B] and X tile [BM x 64] (128B swizzle);
//                          cp.async: the tile's 128 x 4 block-scale bytes
//   warps 6-13  decode     e2m1 * e4m3 -> exact 16-bit operand tile W' [128 x 64], written in
//                          the UMMA K-major 128B-swizzled layout, then fence.proxy.async
//   warp 1      MMA        4 x tcgen05.mma (K=16 each) D[128 x BM] += W' . X^T, f32 in TMEM;
//                          tcgen05.commit frees the stage
//   warps 2-5   epilogue   tcgen05.ld -> * g (+ bias[n]) -> narrow -> global (lanes span n, so a
//                          warp writes 64 contiguous bytes per activation row)
// Accumulators are double-buffered in TMEM so the epilogue of one tile overlaps the main
// loop of the next; the kernel is persistent over tiles.
//
// W' = e2m1 * e4m3 has at most 6 significant bits and magnitude in [2^-10, 2688], so it is
// exact in f16 and in bf16: the only rounding left is the f32 accumulation order.  The f32
// global scale is applied in the epilogue.
//
// Operand-format variants of the decode, both exact; the variant follows the activation
// dtype because tcgen05.mma kind::f16 with A = f16 and B = bf16 raises an illegal
// instruction on sm_100a (observed), so both operands always share one format:
//   kAf16   (f16 activations) W' in f16 by the hardware converts cvt.rn.f16x2.e2m1x2 /
//           .e4m3x2 and one half2 multiply.
//   kAbf16  (bf16 activations) W' in bf16 by bit placement: the code's magnitude bits at
//           bf16 bits 8:6 read as value * 2^-126 (0.5 is the bf16 subnormal); one bf16x2
//           multiply by scale * 2^119 gives value * scale * 2^-7, and the epilogue
//           multiplies by g * 128.
#include <type_traits>

#include "common.cuh"
#include "sm100_primitives.cuh"

namespace nml_sm100 {
namespace {

constexpr int kTileN = 128;  // weight rows per tile (UMMA M)
constexpr int kTileK = 64;   // K per stage: one 128-byte swizzled row of 16-bit operands
constexpr int kUmmaK = 16;
constexpr int kProducerWarp = 0;
constexpr int kMmaWarp = 1;
constexpr int kEpilogueWarps = 4;
constexpr int kDecodeWarp0 = 6;
constexpr int kDecodeWarps = 8;
constexpr int kThreads = (kDecodeWarp0 + kDecodeWarps) * 32;  // 448
constexpr int kDecodeThreads = kDecodeWarps * 32;             // 256: two threads per weight row

constexpr int kWBytes = kTileN * 128;         // decoded operand tile
constexpr int kPayloadBytes = kTileN * 32;    // 64 codes per row
constexpr int kScaleBytes = 1024;             // 128 x 4 used, padded to keep 1024-byte alignment
constexpr int kSmemBudget = 227 * 1024;
constexpr int kBarrierBytes = 512;

enum AFormat : int { kAf16 = 0, kAbf16 = 1 };

template <int BM>
struct Tiling {
  static constexpr int kXBytes = BM * 128;
  static constexpr int kStageBytes = kWBytes + kXBytes + kPayloadBytes + kScaleBytes;
  static constexpr int kStagesFit = (kSmemBudget - 1024 - kBarrierBytes) / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + kBarrierBytes;
  static constexpr int kAccColumns = 2 * BM;  // two accumulators
  static constexpr int kTmemColumns = kAccColumns < 32 ? 32 : kAccColumns;
  static_assert(kStages >= 3, "pipeline too shallow");
  static_assert((kTmemColumns & (kTmemColumns - 1)) == 0 && kTmemColumns <= 512, "TMEM columns");
};

struct Params {
  const uint8_t* block_scales;
  const float* global_scale;
  const void* bias;
  void* output;
  int M, N, K;
  int n_tiles, m_tiles, k_steps;
  int scale_width;
  int n_fastest;  // tile order: 1 = consecutive tiles walk n, 0 = walk m
  int* status;
};

__device__ __forceinline__ void decode_tile_coords(const Params& p, int tile, int& n_tile,
                                                   int& m_tile) {
  if (p.n_fastest) {
    m_tile = tile / p.n_tiles;
    n_tile = tile - m_tile * p.n_tiles;
  } else {
    n_tile = tile / p.m_tiles;
    m_tile = tile - n_tile * p.m_tiles;
  }
}

// 8 codes (one 32-bit payload word) -> 8 exact f16 products with the block scale,
// as four f16x2 words in K order.
__device__ __forceinline__ void decode8_f16(uint32_t word, uint32_t scale2, uint32_t (&out)[4]) {
  uint32_t h0, h1, h2, h3;
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3)
      : "r"(word));
  asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(h0) : "r"(scale2));
  asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(h1) : "r"(scale2));
  asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(h2) : "r"(scale2));
  asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(h3) : "r"(scale2));
  out[0] = h0;
  out[1] = h1;
  out[2] = h2;
  out[3] = h3;
}

// Two E4M3 scale bytes -> two duplicated f16x2 scale words.
__device__ __forceinline__ void scales2_f16(uint32_t two_bytes, uint32_t& first, uint32_t& second) {
  uint32_t pair;
  asm("{\n"
      ".reg .b16 s;\n"
      "cvt.u16.u32 s, %1;\n"
      "cvt.rn.f16x2.e4m3x2 %0, s;\n"
      "}\n"
      : "=r"(pair)
      : "r"(two_bytes));
  first = __byte_perm(pair, pair, 0x1010);
  second = __byte_perm(pair, pair, 0x3232);
}

// 8 codes -> 8 exact bf16 values value * scale * 2^-7 as four bf16x2 words in K order.
// scale2 holds bf16(scale * 2^119) in both halves.
__device__ __forceinline__ void decode8_bf16(uint32_t word, uint32_t scale2, uint32_t (&out)[4]) {
  uint32_t t[4];
  uint32_t q = word;
#pragma unroll
  for (int i = 3; i >= 0; --i) {
    // halves hold codes i and i+4 at their top nibble: sign stays at bit 15, the three
    // magnitude bits move from 14:12 to 8:6.
    t[i] = (q & 0x80008000u) | ((q & 0x70007000u) >> 6);
    q <<= 4;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(t[i]) : "r"(scale2));
  }
  out[0] = __byte_perm(t[0], t[1], 0x5410);  // codes 0, 1
  out[1] = __byte_perm(t[2], t[3], 0x5410);  // codes 2, 3
  out[2] = __byte_perm(t[0], t[1], 0x7632);  // codes 4, 5
  out[3] = __byte_perm(t[2], t[3], 0x7632);  // codes 6, 7
}

// One E4M3 scale byte -> bf16(scale * 2^119) duplicated in both halves.  The byte's value
// bits at bf16 bits 10:4 read as scale * 2^-120; two exact bf16 multiplies rescale.
__device__ __forceinline__ uint32_t scale_bf16_dup(uint32_t byte) {
  uint32_t s = (byte & 0x7fu) << 4;
  s |= s << 16;
  const uint32_t two_p120 = 0x7b807b80u;  // bf16 2^120 in both halves
  const uint32_t two_p119 = 0x7b007b00u;  // bf16 2^119
  asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(s) : "r"(two_p120));
  asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(s) : "r"(two_p119));
  return s;
}

template <int BM, int AFMT, typename T>
__global__ void __launch_bounds__(kThreads, 1)
linear_umma_kernel(const __grid_constant__ CUtensorMap tmap_payload,
                   const __grid_constant__ CUtensorMap tmap_x, const Params p) {
  using Tile = Tiling<BM>;
  constexpr int kStages = Tile::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_address = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_address & 1023u)) & 1023u);

  auto w_tile = [&](int s) { return smem + s * Tile::kStageBytes; };
  auto x_tile = [&](int s) { return smem + s * Tile::kStageBytes + kWBytes; };
  auto payload_tile = [&](int s) { return smem + s * Tile::kStageBytes + kWBytes + Tile::kXBytes; };
  auto scale_tile = [&](int s) {
    return smem + s * Tile::kStageBytes + kWBytes + Tile::kXBytes + kPayloadBytes;
  };
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * Tile::kStageBytes);
  uint64_t* full_raw = bars;                 // [kStages] TMA bytes + scale copies landed
  uint64_t* full_w = bars + kStages;         // [kStages] decoded operand tile written
  uint64_t* empty = bars + 2 * kStages;      // [kStages] MMAs of the stage retired
  uint64_t* tmem_full = bars + 3 * kStages;  // [2] accumulator complete
  uint64_t* tmem_empty = tmem_full + 2;      // [2] accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_raw[s], 1 + 32);
      mbar_init(&full_w[s], kDecodeThreads);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], kEpilogueWarps * 32);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_descriptor(&tmap_payload);
    tma_prefetch_descriptor(&tmap_x);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, Tile::kTmemColumns);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.n_tiles * p.m_tiles;

  auto give_up = [&]() {
    *abort_flag = 1;
    atomicOr(p.status, NML_SM100_STATUS_BARRIER_TIMEOUT);
  };

  if (warp == kProducerWarp) {
    // ---------------------------------------------------------------- producer
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int n_tile, m_tile;
      decode_tile_coords(p, tile, n_tile, m_tile);
      const int n0 = n_tile * kTileN;
      for (int k_step = 0; k_step < p.k_steps; ++k_step) {
        if (*abort_flag || !mbar_wait(&empty[stage], phase ^ 1u)) {
          if (!*abort_flag) give_up();
          ok = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&full_raw[stage], kPayloadBytes + Tile::kXBytes);
          tma_load_2d(payload_tile(stage), &tmap_payload, &full_raw[stage], k_step * 32, n0);
          tma_load_2d(x_tile(stage), &tmap_x, &full_raw[stage], k_step * kTileK, m_tile * BM);
        }
#pragma unroll
        for (int i = 0; i < kTileN / 32; ++i) {
          const int row = lane + 32 * i;
          const int n = min(n0 + row, p.N - 1);
          cp_async_4(scale_tile(stage) + row * 4,
                     p.block_scales + static_cast<int64_t>(n) * p.scale_width + k_step * 4);
        }
        cp_async_mbar_arrive_noinc(&full_raw[stage]);
        ++issued;
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    // Do not leave while copies this warp started may still be landing in shared memory.
    const int pending = issued < kStages ? issued : kStages;
    for (int i = 0; i < pending; ++i) {
      stage = stage == 0 ? kStages - 1 : stage - 1;
      if (stage == kStages - 1) phase ^= 1u;
      if (!mbar_wait(&full_raw[stage], phase)) give_up();
    }
  } else if (warp == kMmaWarp) {
    // --------------------------------------------------------------------- MMA
    if (lane == 0) {
      constexpr uint32_t a_format = AFMT == kAf16 ? kUmmaF16 : kUmmaBF16;
      constexpr uint32_t b_format = sizeof(T) == 2 && std::is_same<T, __half>::value
                                        ? kUmmaF16
                                        : kUmmaBF16;
      constexpr uint32_t idesc = umma_idesc_f16(a_format, b_format, kTileN, BM);
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (*abort_flag || !mbar_wait(&tmem_empty[acc], acc_phase ^ 1u)) {
          if (!*abort_flag) give_up();
          break;
        }
        tcgen05_fence_after_sync();
        const uint32_t d_address = tmem_base + acc * BM;
        for (int k_step = 0; k_step < p.k_steps; ++k_step) {
          if (*abort_flag || !mbar_wait(&full_w[stage], phase) ||
              !mbar_wait(&full_raw[stage], phase)) {
            if (!*abort_flag) give_up();
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(w_tile(stage)));
          const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(x_tile(stage)));
#pragma unroll
          for (int j = 0; j < kTileK / kUmmaK; ++j) {
            // each K=16 slice is 32 bytes further along the swizzled 128-byte rows
            umma_f16(d_address, a_desc + 2 * j, b_desc + 2 * j, idesc, (k_step | j) != 0);
          }
          umma_commit(&empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
    __syncwarp();
  } else if (warp < kDecodeWarp0) {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes a warp may read: 32 * (warp % 4)
    const float g = __ldg(p.global_scale) * (AFMT == kAbf16 ? 128.0f : 1.0f);
    T* out = static_cast<T*>(p.output);
    const T* bias = static_cast<const T*>(p.bias);
    int local_tile = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      int n_tile, m_tile;
      decode_tile_coords(p, tile, n_tile, m_tile);
      const int acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      if (*abort_flag || !mbar_wait(&tmem_full[acc], acc_phase)) {
        if (!*abort_flag) give_up();
        break;
      }
      tcgen05_fence_after_sync();
      const int n = n_tile * kTileN + quarter * 32 + lane;
      const bool n_ok = n < p.N;
      const float bias_value = (bias != nullptr && n_ok) ? Elem<T>::load(bias[n]) : 0.0f;
      const int m0 = m_tile * BM;
      constexpr int kChunk = BM >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < BM; c += kChunk) {
        const uint32_t address =
            tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BM + c;
        uint32_t v[kChunk];
        if constexpr (kChunk == 32) {
          tmem_load_32x32(address, v);
        } else {
          tmem_load_32x16(address, v);
        }
        tmem_load_wait();
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < kChunk; ++j) {
            const int m = m0 + c + j;
            if (m < p.M) {
              out[static_cast<int64_t>(m) * p.N + n] =
                  Elem<T>::store(fmaf(__uint_as_float(v[j]), g, bias_value));
            }
          }
        }
      }
      tcgen05_fence_before_sync();
      mbar_arrive(&tmem_empty[acc]);
    }
  } else {
    // ------------------------------------------------------------------ decode
    const int t = threadIdx.x - kDecodeWarp0 * 32;  // 0..255
    const int row = t >> 1;
    const int half = t & 1;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      for (int k_step = 0; k_step < p.k_steps; ++k_step) {
        if (*abort_flag || !mbar_wait(&full_raw[stage], phase)) {
          if (!*abort_flag) give_up();
          ok = false;
          break;
        }
        const uint4 codes = *reinterpret_cast<const uint4*>(payload_tile(stage) + t * 16);
        const uint32_t two_scales =
            *reinterpret_cast<const uint16_t*>(scale_tile(stage) + row * 4 + half * 2);
        uint32_t scale_a, scale_b;
        if constexpr (AFMT == kAf16) {
          scales2_f16(two_scales, scale_a, scale_b);
        } else {
          scale_a = scale_bf16_dup(two_scales & 0xffu);
          scale_b = scale_bf16_dup(two_scales >> 8);
        }
        uint8_t* w_row = w_tile(stage) + row * 128;
        const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t out[4];
          if constexpr (AFMT == kAf16) {
            decode8_f16(words[j], j < 2 ? scale_a : scale_b, out);
          } else {
            decode8_bf16(words[j], j < 2 ? scale_a : scale_b, out);
          }
          const int chunk = (half * 4 + j) ^ (row & 7);
          *reinterpret_cast<uint4*>(w_row + chunk * 16) = make_uint4(out[0], out[1], out[2], out[3]);
        }
        fence_proxy_async_smem();
        mbar_arrive(&full_w[stage]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, Tile::kTmemColumns);
  }
}

// ---- host side ------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* symbol = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      symbol = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(symbol);
  }();
  return fn;
}

template <int BM, int AFMT, typename T>
int32_t launch_variant(const LinearArgs& args, const DeviceInfo& device, char* message,
                       size_t capacity) {
  using Tile = Tiling<BM>;
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) {
    return fail(NML_SM100_LAUNCH_FAILURE, "cuTensorMapEncodeTiled is unavailable", message,
                capacity);
  }
  CUtensorMap tmap_payload, tmap_x;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(args.inputs / 2),
                                static_cast<cuuint64_t>(args.outputs)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(args.inputs / 2)};
    const cuuint32_t box[2] = {32, kTileN};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&tmap_payload, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
               const_cast<uint8_t*>(args.payload), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return fail(NML_SM100_LAUNCH_FAILURE, "payload tensor map encoding failed", message,
                  capacity);
    }
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(args.inputs),
                                static_cast<cuuint64_t>(args.rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(args.inputs) * 2};
    const cuuint32_t box[2] = {kTileK, BM};
    const cuuint32_t elem[2] = {1, 1};
    const CUtensorMapDataType type = std::is_same<T, __half>::value
                                         ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                         : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (encode(&tmap_x, type, 2, const_cast<void*>(args.activation), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return fail(NML_SM100_LAUNCH_FAILURE, "activation tensor map encoding failed", message,
                  capacity);
    }
  }
  Params p;
  p.block_scales = args.block_scales;
  p.global_scale = args.global_scale;
  p.bias = args.bias;
  p.output = args.output;
  p.M = args.rows;
  p.N = args.outputs;
  p.K = args.inputs;
  p.n_tiles = (args.outputs + kTileN - 1) / kTileN;
  p.m_tiles = (args.rows + BM - 1) / BM;
  p.k_steps = args.inputs / kTileK;
  p.scale_width = args.inputs / 16;
  const int64_t weight_bytes = static_cast<int64_t>(args.outputs) * (args.inputs / 2);
  p.n_fastest = weight_bytes <= (32ll << 20) ? 1 : 0;
  p.status = device.status_word;

  auto kernel = linear_umma_kernel<BM, AFMT, T>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Tile::kSmemBytes) != cudaSuccess) {
      return fail(NML_SM100_LAUNCH_FAILURE, "cannot reserve shared memory for the tcgen05 linear",
                  message, capacity);
    }
    configured = true;
  }
  const int64_t tiles = static_cast<int64_t>(p.n_tiles) * p.m_tiles;
  const unsigned grid = static_cast<unsigned>(tiles < device.sm_count ? tiles : device.sm_count);
  kernel<<<grid, kThreads, Tile::kSmemBytes, args.stream>>>(tmap_payload, tmap_x, p);
  note_linear_kernel(AFMT == kAf16 ? "umma_swapab_af16" : "umma_swapab_abf16");
  return launch_result(message, capacity);
}

template <int AFMT, typename T>
int32_t launch_for_rows(const LinearArgs& args, const DeviceInfo& device, char* message,
                        size_t capacity) {
  const int rows = args.rows;
  if (rows <= 16) return launch_variant<16, AFMT, T>(args, device, message, capacity);
  if (rows <= 32) return launch_variant<32, AFMT, T>(args, device, message, capacity);
  if (rows <= 64) return launch_variant<64, AFMT, T>(args, device, message, capacity);
  if (rows <= 128) return launch_variant<128, AFMT, T>(args, device, message, capacity);
  return launch_variant<256, AFMT, T>(args, device, message, capacity);
}

}  // namespace

bool linear_umma_supported(const LinearArgs& args) {
  return args.inputs % kTileK == 0 && reinterpret_cast<uintptr_t>(args.payload) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(args.activation) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(args.block_scales) % 4 == 0;
}

int32_t launch_linear_umma(const LinearArgs& args, const DeviceInfo& device, char* message,
                           size_t capacity) {
  if (args.dtype == NML_SM100_F16) {
    return launch_for_rows<kAf16, __half>(args, device, message, capacity);
  }
  return launch_for_rows<kAbf16, __nv_bfloat16>(args, device, message, capacity);
}

}  // namespace nml_sm100
