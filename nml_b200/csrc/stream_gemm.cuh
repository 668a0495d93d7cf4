// Weight-streaming NVFP4 contraction for few activation rows (decode shapes): the packed
// weights are read from HBM exactly once, at the rate the memory system delivers them, and
// nothing but the weights moves per K step.
//
//   D[n, m] = sum_k W'[n, k] * X[m, k]        W' = e2m1 code * e4m3 block scale (exact in f16)
//
// The reference serves these shapes with dedicated GEMV bodies
// (crates/nml-kernel-nvfp4/src/turing_adapter.cu:156-200 and :458-631,
// crates/nml-kernel-triton/src/nvfp4.rs:523-731 and :1421-1970); this is their sm_100a
// counterpart, for 1..16 activation rows (or schedule slots) per group.
//
// Work unit: a tile of 16 or 32 weight rows (RT = 1 or 2 fragments of 16; the larger tile
// halves the per-tile bookkeeping and is used when every CTA walks many tiles) over the whole
// K range.  The rows of a tile are
// contiguous in the payload tensor, so the producer warp brings a tile (payload and block
// scales) into a shared-memory ring with untiled bulk copies (cp.async.bulk); no tensor map
// is involved.  The K range is cut into units of 64 and dealt to the W <= 16 compute
// warps, `units_per_warp` consecutive units each: the activations of a warp's K slice stay in
// its registers for the whole launch (as mma.sync B fragments), so per tile a warp reads only
// its slice of the packed weights from shared memory, decodes it in registers
// (cvt.rn.f16x2.e2m1x2, cvt.rn.f16x2.e4m3x2, one mul.f16x2) and issues mma.sync.m16n8k16 with
// the decoded weights as the A operand: 16 weight rows x 8 activation rows per instruction,
// f32 accumulation.  No tensor memory, no decoded tile in shared memory, no per-K-step
// hand-off between warps.  Per tile every compute warp leaves its 16 x 8 (x NT) partial sums
// in a ring of shared-memory slots; the reducer warp adds them in warp order (ascending K, so
// the result is deterministic), applies the global scale and the mode's epilogue, and stores
// (one reducer warp per tile of 8 activation rows).
//
// bf16 activations: mma.sync wants both operands in one format and the decoded weights are
// f16, so every warp rescales its slice of each activation row by a power of two that puts
// the slice's largest magnitude into [2^14, 2^15) and narrows to f16.  bf16 has 8 significant
// bits and f16 has 11, so the narrowing is exact for every element within 2^29 of the slice
// maximum; smaller elements round at 2^-25 relative to that maximum, far below the f32
// accumulation error.  The warp multiplies its partial sums by the inverse power of two.
//
// Scale bytes that the format does not define (sign bit set, 0x7f) poison the affected output
// rows with NaN, as the reference device kernels do (turing_adapter.cu:35-40).
//
// Every mbarrier wait is bounded; a wait that runs out sets the barrier-timeout bit of the
// device status word, raises the CTA's abort flag, and every role leaves through the common
// end of the kernel.
#pragma once

#include <type_traits>

#include "common.cuh"
#include "sm100_primitives.cuh"

namespace nml_sm100 {
namespace stream {

enum Mode : int { kDense = 0, kGateUp = 1, kDown = 2 };

constexpr int kFragmentRows = 16;     // weight rows of one mma.sync A fragment
constexpr int kUnitK = 64;            // K values of one unit: a quad of lanes reads 32 bytes per row
constexpr int kMaxComputeWarps = 16;
constexpr int kMaxThreads = (kMaxComputeWarps + 3) * 32;  // + reducer warp(s) + producer warp
constexpr int kMaxStages = 4;         // weight tiles in flight per CTA (more were measured to add nothing)
constexpr int kMaxSlots = 4;          // partial-sum slots between compute warps and reducer
constexpr int kSmemBudget = 227 * 1024;

// One dense weight (fused Q/K/V: up to three that share the activations).
struct Segment {
  const uint8_t* payload;
  const uint8_t* block_scales;
  const float* global_scale;
  const void* bias;
  void* output;
  int outputs;     // rows of this weight = output columns
  int tile_begin;  // first tile of the segment in the launch's tile list
  const void* residual;  // [M, outputs] added to the narrowed result, or null
};

struct Params {
  // dense: activations [M, K], groups of 16 rows
  const void* x;
  Segment segment[3];
  int segments;
  int M;
  // grouped (routed experts): one group per 16-slot schedule block
  const void* input;                  // hidden [tokens, K] (gate/up) or activated [A, K] (down)
  const int32_t* sorted_assignments;  // [schedule_blocks * 16]
  const int32_t* block_experts;       // [schedule_blocks]
  const int32_t* active_blocks;       // may be null
  const int32_t* expert_offset;       // may be null
  const void* routing_weights;        // down: [A]
  void* const* row_targets;           // down: optional [A] destinations of the result rows
  const uint8_t* payload;
  const uint8_t* block_scales;
  const float* global_scale;
  const void* bias;                   // [experts, rows_per_expert]
  void* output;                       // activated [A, N] or weighted [A, N]
  int assignments, schedule_blocks, experts, top_k;
  int rows_per_expert;                // 2 * intermediate (gate/up) or hidden (down)
  int N;                              // output columns per assignment row
  // common
  int K;
  int groups;            // dense: ceil(M / 16); grouped: schedule_blocks (upper bound)
  int tiles_per_group;   // weight tiles every group walks
  int compute_warps;     // W
  int units_per_warp;    // consecutive 64-wide K units per compute warp (<= UT)
  int k_units;           // K / 64
  int row_bytes;         // K / 2
  int scale_width;       // K / 16
  int row_stride;        // shared-memory stride of a payload row (bank-conflict-free)
  int scale_stride;      // shared-memory stride of a scale row
  int scale_offset;      // offset of the scale rows inside a stage
  int stage_bytes;
  int stages;
  int slots;             // partial-sum slots in the ring (<= kMaxSlots)
  int second_offset;     // NT = 2: the compute warps' copies of the second activation-row tile
  int partial_offset;    // offset of the partial-sum slots
  int barrier_offset;
  int* status;
};

// D (16 x 8, f32) += A (16 x 16, f16, row) * B (16 x 8, f16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8 codes (one payload word, K order) -> 8 exact f16 products with the block scale.
__device__ __forceinline__ void decode8(uint32_t word, uint32_t scale2, uint32_t (&out)[4]) {
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3])
      : "r"(word));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(out[i]) : "r"(scale2));
  }
}

// One E4M3 scale byte -> the f16 scale in both halves of a word.
__device__ __forceinline__ uint32_t scale_pair(uint32_t byte) {
  uint32_t pair;
  const uint32_t twice = byte * 0x0101u;
  asm("{\n"
      ".reg .b16 s;\n"
      "cvt.u16.u32 s, %1;\n"
      "cvt.rn.f16x2.e4m3x2 %0, s;\n"
      "}\n"
      : "=r"(pair)
      : "r"(twice));
  return pair;
}

struct Ring {
  int index = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int depth) {
    if (++index == depth) {
      index = 0;
      phase ^= 1u;
    }
  }
};

// Which bounded wait ran out: bit (8 + site) of the device status word.
enum WaitSite : int {
  kSiteProducer = 12,
  kSiteCompute = 13,
  kSiteSlot = 14,
  kSiteReducer = 15,
  kSiteDrain = 16,
};

// NT: activation-row tiles of 8 per group (1: up to 8 rows, 2: up to 16).
// RT: 16-row fragments of weight rows per tile.
// UT: K units a compute warp can hold activations for (registers: 8 * NT * UT).
// FULL: every compute warp holds exactly UT units (no per-unit guards).
template <int UT>
constexpr int max_threads() {
  return kMaxThreads;
}

template <int NT, int UT, int RT, typename T, int MODE, bool FULL>
__global__ void __launch_bounds__(max_threads<UT>(), 1) stream_kernel(const Params p) {
  constexpr bool kGrouped = MODE != kDense;
  constexpr int kTileRows = kFragmentRows * RT;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  extern __shared__ uint8_t stream_smem_raw[];
  uint8_t* smem = stream_smem_raw + ((128u - (smem_u32(stream_smem_raw) & 127u)) & 127u);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int W = p.compute_warps;
  const int g = lane >> 2;  // fragment row: weight rows g and g + 8, activation row g
  const int c = lane & 3;   // position in the quad: 16 K values of every unit

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.barrier_offset);
  uint64_t* full_p = bars;                       // [kMaxStages] tile landed
  uint64_t* empty_p = full_p + kMaxStages;       // [kMaxStages] every compute warp has read it
  uint64_t* full_s = empty_p + kMaxStages;       // [kSlots] every compute warp has written
  uint64_t* empty_s = full_s + kMaxSlots;        // [kSlots] the reducer has read
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_s + kMaxSlots);
  // [slot][W][NT][RT][32]
  float4* partials = reinterpret_cast<float4*>(smem + p.partial_offset);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&full_p[s], 1);
      mbar_init(&empty_p[s], W);
    }
    for (int s = 0; s < kMaxSlots; ++s) {
      mbar_init(&full_s[s], W);
      mbar_init(&empty_s[s], NT);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }

  // ---- the walk every role makes: units [first, last) of (group, tile) pairs -------------
  int groups = p.groups;
  if constexpr (kGrouped) {
    if (p.active_blocks != nullptr) groups = max(0, min(groups, p.active_blocks[0]));
  }
  const int tiles = p.tiles_per_group;
  const int64_t total = static_cast<int64_t>(groups) * tiles;
  const int expert_base = (kGrouped && p.expert_offset != nullptr) ? p.expert_offset[0] : 0;
  // grouped: local expert of a schedule block, -1 when the block has no work here
  auto group_expert = [&](int group) -> int {
    if constexpr (kGrouped) {
      const int id = p.block_experts[group];
      const int local = id - expert_base;
      return (id >= 0 && local >= 0 && local < p.experts) ? local : -1;
    } else {
      return 0;
    }
  };
  // The units are dealt to the CTAs in contiguous ranges.  Grouped launches weigh them first:
  // a block without work here costs nothing, a block with routes in its second eight slots
  // costs about a third more than one without (its tiles issue twice the mma.sync), and equal
  // shares of units would leave the CTAs that drew the heavy blocks running long after the
  // others.  Warp 0 weighs the blocks (lane l takes a contiguous chunk), scans, and finds the
  // two units where this CTA's share of the weight begins and ends.
  constexpr int kWeighedGroups = 256;
  // behind the barriers and the abort flag in the launch's shared memory (plan_layout)
  int* range = reinterpret_cast<int*>(smem + p.barrier_offset + 136);
  uint8_t* group_weight = smem + p.barrier_offset + 256;
  bool weighed = false;
  if constexpr (kGrouped) {
    weighed = NT == 2 && groups <= kWeighedGroups && groups > 0;  // NT = 1: all blocks alike
    if (weighed && warp == 0) {
      const int chunk = (groups + 31) / 32;
      const int begin = min(groups, lane * chunk), end = min(groups, begin + chunk);
      int mine = 0;
      for (int group = begin; group < end; ++group) {
        int weight = 0;
        if (group_expert(group) >= 0) {
          weight = 3;
          if constexpr (NT == 2) {
            // slots fill in order, so the ninth slot tells whether the second tile is live
            const int32_t ninth = p.sorted_assignments[group * 16 + 8];
            if (ninth >= 0 && ninth < p.assignments) weight = 4;
          }
        }
        group_weight[group] = static_cast<uint8_t>(weight);
        mine += weight;
      }
      int before = mine;  // inclusive scan over the lanes' chunk sums
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, before, offset);
        if (lane >= offset) before += other;
      }
      const int64_t all = static_cast<int64_t>(__shfl_sync(0xffffffffu, before, 31)) * tiles;
      before -= mine;  // weight of the groups before this lane's chunk
      if (lane == 0 && all == 0) range[0] = range[1] = 0;
      if (all > 0) {
#pragma unroll
        for (int side = 0; side < 2; ++side) {
          // the unit at which the weight all * (block + side) / grid is reached
          const int64_t target = all * (blockIdx.x + side) / gridDim.x;
          if (side == 1 && blockIdx.x + 1 == gridDim.x) {
            if (lane == 0) range[1] = static_cast<int>(total);
            continue;
          }
          int64_t reached = static_cast<int64_t>(before) * tiles;
          if (target >= reached && target < reached + static_cast<int64_t>(mine) * tiles) {
            for (int group = begin; group < end; ++group) {
              const int64_t span = static_cast<int64_t>(group_weight[group]) * tiles;
              if (target < reached + span) {
                range[side] = group * tiles +
                              static_cast<int>((target - reached) / group_weight[group]);
                break;
              }
              reached += span;
            }
          }
        }
      }
    }
  }
  __syncthreads();
  const int first = weighed ? range[0] : static_cast<int>(total * blockIdx.x / gridDim.x);
  const int last = weighed ? range[1] : static_cast<int>(total * (blockIdx.x + 1) / gridDim.x);
  // A position of the walk; always at a unit with work, or at `last`.
  struct Walk {
    int unit, group, tile, expert;
  };
  auto settle = [&](Walk& w) {  // skips groups without work
    while (w.unit < last && w.expert < 0) {
      w.unit += tiles - w.tile;
      w.tile = 0;
      ++w.group;
      w.expert = (w.unit < last && w.group < groups) ? group_expert(w.group) : -1;
    }
    if (w.unit > last) w.unit = last;
  };
  auto walk_begin = [&]() {
    Walk w;
    w.unit = first;
    w.group = first / tiles;
    w.tile = first - w.group * tiles;
    w.expert = (first < last && w.group < groups) ? group_expert(w.group) : -1;
    settle(w);
    return w;
  };
  auto walk_next = [&](Walk& w) {
    ++w.unit;
    if (++w.tile == tiles) {
      w.tile = 0;
      ++w.group;
      w.expert = (w.unit < last && w.group < groups) ? group_expert(w.group) : -1;
    }
    settle(w);
  };

  auto give_up = [&](int site) {
    *abort_flag = 1;
    atomicOr(p.status, NML_SM100_STATUS_BARRIER_TIMEOUT | (0x100 << site));
  };
  auto wait = [&](uint64_t* bar, uint32_t parity, int site) -> bool {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t poll = 0; poll < kWaitPolls; ++poll) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((poll & 63u) == 63u && *abort_flag) return false;
    }
    give_up(site);
    return false;
  };

  if (warp < W) {
    // ------------------------------------------------------------------- compute
    const int units = max(0, min(p.units_per_warp, p.k_units - warp * p.units_per_warp));
    const int unit0 = warp * p.units_per_warp;  // first K unit of this warp
    // Activations of the slice as mma.sync B fragments: row 8 jn + g, K = 64 unit + 16 c + 2 r.
    // The first activation-row tile stays in registers; the second one (NT = 2) would push the
    // kernel into spills, so it lives in this warp's corner of shared memory, one 16-byte
    // read per lane and half unit.
    uint32_t b[UT][8];
    uint4* b_second = reinterpret_cast<uint4*>(smem + p.second_offset) + warp * (UT * 2 * 32) + lane;
    float back[NT][2];       // inverse rescale of activation rows 8 jn + 2 c and 8 jn + 2 c + 1
    bool second_live = false;  // NT = 2: the group has a row (slot) among its second eight
    // Loads the slice of the group's activation rows and narrows it to f16.
    auto load_activations = [&](int group) {
#pragma unroll
      for (int jn = 0; jn < NT; ++jn) {
        const int slot = 8 * jn + g;
        const uint8_t* row = nullptr;
        if constexpr (kGrouped) {
          const int32_t a = p.sorted_assignments[group * 16 + slot];
          if (a >= 0 && a < p.assignments) {
            const int64_t source = MODE == kGateUp ? a / p.top_k : a;
            row = static_cast<const uint8_t*>(p.input) + source * p.K * 2;
          }
        } else {
          const int m = group * 16 + slot;
          if (m < p.M) row = static_cast<const uint8_t*>(p.x) + static_cast<int64_t>(m) * p.K * 2;
        }
        if (jn == 1) second_live = __any_sync(0xffffffffu, row != nullptr);
        uint32_t magnitude = 0;
        uint32_t fresh[UT][8];
#pragma unroll
        for (int u = 0; u < UT; ++u) {
          uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
          if (row != nullptr && (FULL || u < units)) {
            const uint4* source =
                reinterpret_cast<const uint4*>(row + ((unit0 + u) * kUnitK + 16 * c) * 2);
            lo = __ldg(source);
            hi = __ldg(source + 1);
          }
          fresh[u][0] = lo.x; fresh[u][1] = lo.y; fresh[u][2] = lo.z; fresh[u][3] = lo.w;
          fresh[u][4] = hi.x; fresh[u][5] = hi.y; fresh[u][6] = hi.z; fresh[u][7] = hi.w;
          if constexpr (kBf16) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              magnitude = max(magnitude, fresh[u][r] & 0x7fffu);
              magnitude = max(magnitude, (fresh[u][r] >> 16) & 0x7fffu);
            }
          }
        }
        int shift = 0;  // the row slice is multiplied by 2^-shift before narrowing
        if constexpr (kBf16) {
          magnitude = max(magnitude, __shfl_xor_sync(0xffffffffu, magnitude, 1));
          magnitude = max(magnitude, __shfl_xor_sync(0xffffffffu, magnitude, 2));
          const int exponent = static_cast<int>(magnitude >> 7);  // biased, 0..255
          if (exponent != 0 && exponent != 255) {
            // largest magnitude lands in [2^14, 2^15); both powers of two stay normal f32
            shift = min(max(exponent - 127 - 14, -126), 126);
          }
          const float down = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
#pragma unroll
          for (int u = 0; u < UT; ++u) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              const uint32_t word = fresh[u][r];
              const float low = __uint_as_float(word << 16) * down;
              const float high = __uint_as_float(word & 0xffff0000u) * down;
              const __half2 narrowed = __floats2half2_rn(low, high);
              fresh[u][r] = *reinterpret_cast<const uint32_t*>(&narrowed);
            }
          }
        }
        if (jn == 0) {
#pragma unroll
          for (int u = 0; u < UT; ++u) {
#pragma unroll
            for (int r = 0; r < 8; ++r) b[u][r] = fresh[u][r];
          }
        } else {
#pragma unroll
          for (int u = 0; u < UT; ++u) {
            b_second[(2 * u) * 32] = make_uint4(fresh[u][0], fresh[u][1], fresh[u][2], fresh[u][3]);
            b_second[(2 * u + 1) * 32] =
                make_uint4(fresh[u][4], fresh[u][5], fresh[u][6], fresh[u][7]);
          }
        }
        // the accumulator columns of this lane are activation rows 8 jn + 2 c and + 1, whose
        // shifts live in the lanes with g = 2 c and g = 2 c + 1
        const int shift0 = __shfl_sync(0xffffffffu, shift, (2 * c) * 4);
        const int shift1 = __shfl_sync(0xffffffffu, shift, (2 * c + 1) * 4);
        back[jn][0] = __uint_as_float(static_cast<uint32_t>(127 + shift0) << 23);
        back[jn][1] = __uint_as_float(static_cast<uint32_t>(127 + shift1) << 23);
      }
    };

    Ring ring, slots;
    int loaded_group = -1;
    // per-lane offsets inside a stage
    const int payload_offset = g * p.row_stride + unit0 * 32 + 8 * c;
    const int scale_offset = p.scale_offset + g * p.scale_stride + unit0 * 4 + c;
    for (Walk w = walk_begin(); w.unit < last; walk_next(w)) {
      if (loaded_group != w.group) {
        load_activations(w.group);
        loaded_group = w.group;
      }
      if (!wait(&full_p[ring.index], ring.phase, kSiteCompute)) break;
      const uint8_t* stage = smem + ring.index * p.stage_bytes;
      // With one activation-row tile the mma.sync instructions of a fragment alternate over
      // two accumulators (added in index order below); with two tiles each has one, which
      // leaves registers for the 32-row tile.  The count depends on nothing but NT, so a
      // weight row's sum is formed in the same order whatever the tile height: a fused launch
      // equals separate launches bit for bit.
      constexpr int kChains = NT == 1 ? 2 : 1;
      float acc[RT][NT][kChains][4];
      uint32_t seen[RT][2];  // OR of the scale bytes of rows g and g + 8: bit 7 marks an invalid one
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        seen[rt][0] = seen[rt][1] = 0;
#pragma unroll
        for (int jn = 0; jn < NT; ++jn) {
#pragma unroll
          for (int q = 0; q < kChains; ++q) {
            acc[rt][jn][q][0] = acc[rt][jn][q][1] = acc[rt][jn][q][2] = acc[rt][jn][q][3] = 0.0f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UT; ++u) {
        if (FULL || u < units) {
#pragma unroll
          for (int rt = 0; rt < RT; ++rt) {
            const uint8_t* payload_g = stage + payload_offset + rt * 16 * p.row_stride + u * 32;
            const uint8_t* scale_g = stage + scale_offset + rt * 16 * p.scale_stride + u * 4;
            const uint2 words_g = *reinterpret_cast<const uint2*>(payload_g);
            const uint2 words_h = *reinterpret_cast<const uint2*>(payload_g + 8 * p.row_stride);
            const uint32_t byte_g = scale_g[0];
            const uint32_t byte_h = scale_g[8 * p.scale_stride];
            seen[rt][0] |= byte_g;
            seen[rt][1] |= byte_h;
            const uint32_t pair_g = scale_pair(byte_g);
            const uint32_t pair_h = scale_pair(byte_h);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t dg[4], dh[4];
              decode8(half == 0 ? words_g.x : words_g.y, pair_g, dg);
              decode8(half == 0 ? words_h.x : words_h.y, pair_h, dh);
              mma_16816(acc[rt][0][0], dg[0], dh[0], dg[1], dh[1], b[u][4 * half],
                        b[u][4 * half + 1]);
              mma_16816(acc[rt][0][kChains - 1], dg[2], dh[2], dg[3], dh[3], b[u][4 * half + 2],
                        b[u][4 * half + 3]);
              if (NT == 2 && (!kGrouped || second_live)) {  // skipped for blocks of <= 8 routes
                const uint4 second = b_second[(2 * u + half) * 32];
                mma_16816(acc[rt][NT - 1][0], dg[0], dh[0], dg[1], dh[1], second.x, second.y);
                mma_16816(acc[rt][NT - 1][kChains - 1], dg[2], dh[2], dg[3], dh[3], second.z,
                          second.w);
              }
            }
          }
        }
      }
      // this warp has read its last byte of the stage
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_p[ring.index]);
      ring.advance(p.stages);
      // invalid scale bytes seen by any lane of the quad poison the two rows (rare: one vote
      // per tile keeps the common path free of shuffles)
      float poison[RT][2];
      uint32_t any_seen = 0;
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        poison[rt][0] = poison[rt][1] = 0.0f;
        any_seen |= seen[rt][0] | seen[rt][1];
      }
      if (__any_sync(0xffffffffu, (any_seen & 0x80u) != 0u)) {
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t bits = seen[rt][h];
            bits |= __shfl_xor_sync(0xffffffffu, bits, 1);
            bits |= __shfl_xor_sync(0xffffffffu, bits, 2);
            if (bits & 0x80u) poison[rt][h] = __uint_as_float(0x7fc00000u);
          }
        }
      }
      if (!wait(&empty_s[slots.index], slots.phase ^ 1u, kSiteSlot)) break;
      float4* mine = partials + ((slots.index * W + warp) * NT * RT) * 32 + lane;
#pragma unroll
      for (int jn = 0; jn < NT; ++jn) {
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
          float total[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            total[i] = acc[rt][jn][0][i];
#pragma unroll
            for (int q = 1; q < kChains; ++q) total[i] = __fadd_rn(total[i], acc[rt][jn][q][i]);
          }
          mine[(jn * RT + rt) * 32] = make_float4(total[0] * back[jn][0] + poison[rt][0],
                                                  total[1] * back[jn][1] + poison[rt][0],
                                                  total[2] * back[jn][0] + poison[rt][1],
                                                  total[3] * back[jn][1] + poison[rt][1]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_s[slots.index]);
      slots.advance(p.slots);
    }
  } else if (warp == W + NT) {
    // ------------------------------------------------------------------ producer
    // Lane 0 owns the ring (waits, transaction counts); when rows are padded in shared memory
    // and have to be copied one by one, lane r issues payload row r and lane 16 + r scale
    // row r (lane r both, when the tile has 32 rows).
    Ring ring;
    int issued = 0;
    auto produce = [&](const Walk& w) -> bool {
      const uint8_t* payload;
      const uint8_t* scales;
      int row0, rows;
      if constexpr (kGrouped) {
        row0 = w.tile * kTileRows;
        rows = p.rows_per_expert;
        const int64_t base = static_cast<int64_t>(w.expert) * p.rows_per_expert;
        payload = p.payload + base * p.row_bytes;
        scales = p.block_scales + base * p.scale_width;
      } else {
        int s = 0;
        if (p.segments > 1 && w.tile >= p.segment[1].tile_begin) s = 1;
        if (p.segments > 2 && w.tile >= p.segment[2].tile_begin) s = 2;
        row0 = (w.tile - p.segment[s].tile_begin) * kTileRows;
        rows = p.segment[s].outputs;
        payload = p.segment[s].payload;
        scales = p.segment[s].block_scales;
      }
      const int valid = min(kTileRows, rows - row0);
      int ok = 1;
      if (lane == 0) {
        ok = wait(&empty_p[ring.index], ring.phase ^ 1u, kSiteProducer) ? 1 : 0;
        if (ok) {
          mbar_arrive_expect_tx(&full_p[ring.index],
                                static_cast<uint32_t>(valid) * (p.row_bytes + p.scale_width));
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return false;
      uint8_t* stage = smem + ring.index * p.stage_bytes;
      const uint8_t* from = payload + static_cast<int64_t>(row0) * p.row_bytes;
      const uint8_t* scale_from = scales + static_cast<int64_t>(row0) * p.scale_width;
      if (p.row_stride == p.row_bytes) {
        if (lane == 0) {
          bulk_load(stage, from, static_cast<uint32_t>(valid * p.row_bytes), &full_p[ring.index]);
        }
      } else if (lane < valid) {
        bulk_load(stage + lane * p.row_stride, from + static_cast<int64_t>(lane) * p.row_bytes,
                  static_cast<uint32_t>(p.row_bytes), &full_p[ring.index]);
      }
      const int scale_row = RT == 1 ? lane - 16 : lane;
      if (p.scale_stride == p.scale_width) {
        if (lane == 16) {
          bulk_load(stage + p.scale_offset, scale_from,
                    static_cast<uint32_t>(valid * p.scale_width), &full_p[ring.index]);
        }
      } else if (scale_row >= 0 && scale_row < valid) {
        const int r = scale_row;
        bulk_load(stage + p.scale_offset + r * p.scale_stride,
                  scale_from + static_cast<int64_t>(r) * p.scale_width,
                  static_cast<uint32_t>(p.scale_width), &full_p[ring.index]);
      }
      __syncwarp();
      ++issued;
      ring.advance(p.stages);
      return true;
    };

    for (Walk w = walk_begin(); w.unit < last; walk_next(w)) {
      if (!produce(w)) break;
    }
    // Do not leave while copies this warp started may still be landing.
    if (lane == 0) {
      const int pending = issued < p.stages ? issued : p.stages;
      for (int i = 0; i < pending; ++i) {
        ring.index = ring.index == 0 ? p.stages - 1 : ring.index - 1;
        if (ring.index == p.stages - 1) ring.phase ^= 1u;
        if (!mbar_wait(&full_p[ring.index], ring.phase)) give_up(kSiteDrain);
      }
    }
  } else {
    // -------------------------------------------------------------------- reducer
    // One reducer warp per activation-row tile of 8: warp W + jn sums and finishes tile jn.
    const int jn = warp - W;
    Ring slots;
    int loaded_group = -1;
    // grouped: the assignment (output row) and routing weight of this lane's columns
    int32_t target[2];
    float route_weight[2];
    T* down_row[2] = {nullptr, nullptr};  // down: where this lane's two result rows go
    for (Walk w = walk_begin(); w.unit < last; walk_next(w)) {
      if constexpr (kGrouped) {
        if (loaded_group != w.group) {
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int32_t a = p.sorted_assignments[w.group * 16 + 8 * jn + 2 * c + i];
            const bool valid = a >= 0 && a < p.assignments;
            target[i] = valid ? a : -1;
            route_weight[i] = 0.0f;
            if (MODE == kDown) {
              down_row[i] = nullptr;
              if (valid) {
                route_weight[i] = Elem<T>::load(static_cast<const T*>(p.routing_weights)[a]);
                // row a of the output, or wherever the caller's table sends it (an
                // expert-parallel owner: the sender's return buffer, over NVLink)
                down_row[i] = p.row_targets != nullptr
                                  ? static_cast<T*>(p.row_targets[a])
                                  : static_cast<T*>(p.output) + static_cast<int64_t>(a) * p.N;
              }
            }
          }
          loaded_group = w.group;
        }
      }
      if (!wait(&full_s[slots.index], slots.phase, kSiteReducer)) break;
      const float4* slot = partials + ((slots.index * W) * NT + jn) * RT * 32 + lane;
      float4 sums[RT];
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) sums[rt] = slot[rt * 32];
#pragma unroll 4
      for (int cw = 1; cw < W; ++cw) {  // ascending K
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
          const float4 v = slot[(cw * NT * RT + rt) * 32];
          sums[rt].x = __fadd_rn(sums[rt].x, v.x);
          sums[rt].y = __fadd_rn(sums[rt].y, v.y);
          sums[rt].z = __fadd_rn(sums[rt].z, v.z);
          sums[rt].w = __fadd_rn(sums[rt].w, v.w);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_s[slots.index]);
      slots.advance(p.slots);
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
      const float4 sum = sums[rt];

      if constexpr (MODE == kDense) {
        int s = 0;
        if (p.segments > 1 && w.tile >= p.segment[1].tile_begin) s = 1;
        if (p.segments > 2 && w.tile >= p.segment[2].tile_begin) s = 2;
        const Segment& segment = p.segment[s];
        const float scale = __ldg(segment.global_scale);
        T* out = static_cast<T*>(segment.output);
        const T* bias = static_cast<const T*>(segment.bias);
        const T* residual = static_cast<const T*>(segment.residual);
        const int n0 = (w.tile - segment.tile_begin) * kTileRows + 16 * rt + g;
#pragma unroll
        for (int half = 0; half < 2; ++half) {  // weight rows g and g + 8
          const int n = n0 + 8 * half;
          if (n < segment.outputs) {
            const float bias_value = bias != nullptr ? Elem<T>::load(bias[n]) : 0.0f;
            const float v0 = half == 0 ? sum.x : sum.z;
            const float v1 = half == 0 ? sum.y : sum.w;
            const int m = w.group * 16 + 8 * jn + 2 * c;
            if (residual == nullptr) {  // the plain form keeps its own, shorter store sequence
              if (m < p.M) {
                out[static_cast<int64_t>(m) * segment.outputs + n] =
                    Elem<T>::store(fmaf(v0, scale, bias_value));
              }
              if (m + 1 < p.M) {
                out[static_cast<int64_t>(m + 1) * segment.outputs + n] =
                    Elem<T>::store(fmaf(v1, scale, bias_value));
              }
            } else {
              if (m < p.M) {
                const int64_t index = static_cast<int64_t>(m) * segment.outputs + n;
                out[index] =
                    narrow_with_residual<T>(fmaf(v0, scale, bias_value), residual, index);
              }
              if (m + 1 < p.M) {
                const int64_t index = static_cast<int64_t>(m + 1) * segment.outputs + n;
                out[index] =
                    narrow_with_residual<T>(fmaf(v1, scale, bias_value), residual, index);
              }
            }
          }
        }
      } else {
        const float scale = __ldg(p.global_scale);
        T* out = static_cast<T*>(p.output);
        const T* bias = static_cast<const T*>(p.bias) +
                        static_cast<int64_t>(w.expert) * p.rows_per_expert;
        const int n0 = w.tile * kTileRows + 16 * rt + g;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int n = n0 + 8 * half;  // weight row inside the expert
          const bool n_ok = n < p.rows_per_expert;
          const float bias_value = n_ok ? Elem<T>::load(bias[n]) : 0.0f;
          const float v[2] = {fmaf(half == 0 ? sum.x : sum.z, scale, bias_value),
                              fmaf(half == 0 ? sum.y : sum.w, scale, bias_value)};
          if constexpr (MODE == kGateUp) {
            // Even weight rows carry gate, odd rows up of the same intermediate column, and
            // the lane four further on holds the partner row.  The even lane finishes
            // activation row 2 c, the odd lane row 2 c + 1, so both halves of the warp share
            // the SwiGLU evaluations.
            const bool odd = (g & 1) != 0;
            const float received0 = __shfl_xor_sync(0xffffffffu, v[0], 4);
            const float received1 = __shfl_xor_sync(0xffffffffu, v[1], 4);
            const float gate = odd ? received1 : v[0];
            const float up = odd ? v[1] : received0;
            const int32_t row = odd ? target[1] : target[0];
            if (n_ok && row >= 0) {
              out[static_cast<int64_t>(row) * p.N + (n >> 1)] =
                  Elem<T>::store(clamped_swiglu(gate, up));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              if (n_ok && down_row[i] != nullptr) {
                down_row[i][n] = Elem<T>::store(v[i] * route_weight[i]);
              }
            }
          }
        }
      }
      }  // rt
    }
    if constexpr (MODE == kDown) {
      // stores through the caller's table may go to another GPU, whose flag a later launch
      // raises: each writer orders its own stores at system scope before the kernel ends
      if (p.row_targets != nullptr) __threadfence_system();
    }
  }
  __syncthreads();
}

// ---- host side ------------------------------------------------------------------------------

// Shared-memory layout and warp split of a launch; false when the shape does not fit.
inline bool plan_layout(int K, int nt, int rt, Params* p, int* smem_bytes) {
  const int tile_rows = kFragmentRows * rt;
  if (K <= 0 || K % kUnitK != 0) return false;
  p->K = K;
  p->k_units = K / kUnitK;
  p->row_bytes = K / 2;
  p->scale_width = K / 16;
  // compute warps: as many as divide the K units evenly, else the least padded split
  int best_w = 1, best_u = p->k_units;
  for (int w = kMaxComputeWarps; w >= 1; --w) {
    const int u = (p->k_units + w - 1) / w;
    if (u < best_u || (u == best_u && w * u < best_w * best_u)) {
      best_w = w;
      best_u = u;
    }
  }
  // drop warps that would hold no unit at all
  while (best_w > 1 && (best_w - 1) * best_u >= p->k_units) --best_w;
  if (best_u > 4) return false;
  p->compute_warps = best_w;
  p->units_per_warp = best_u;
  // A half-warp's 8-byte reads of rows g = 0..3 are conflict-free when the row stride is 32
  // or 96 modulo 128 bytes; byte reads of rows g = 0..7 when the stride is not a multiple of
  // 32 bytes.  Padded rows are copied one by one.
  const int r = p->row_bytes % 128;
  p->row_stride = p->row_bytes + ((r == 32 || r == 96) ? 0 : (32 + 128 - r) % 128);
  p->scale_stride = p->scale_width + (p->scale_width % 32 == 0 ? 16 : 0);
  p->scale_offset = (tile_rows * p->row_stride + 127) / 128 * 128;
  p->stage_bytes = p->scale_offset + (tile_rows * p->scale_stride + 127) / 128 * 128;
  p->slots = rt == 1 ? kMaxSlots : 2;
  const int partial_bytes = p->slots * p->compute_warps * nt * rt * 32 * 16;
  // the kernel variant that serves this split holds 3 units per warp when that divides K
  // evenly, else 4 (see launch_for_shape)
  const int held_units = (best_w * best_u == p->k_units && best_u == 3) ? 3 : 4;
  const int second_bytes = nt == 2 ? p->compute_warps * held_units * 2 * 32 * 16 : 0;
  const int fixed = partial_bytes + second_bytes +
                    512 /* barriers, unit range, block weights */ + 128 /* alignment slack */;
  int stages = kMaxStages;
  while (stages > 1 && stages * p->stage_bytes + fixed > kSmemBudget) --stages;
  if (stages < 2) return false;
  p->stages = stages;
  p->partial_offset = stages * p->stage_bytes;
  p->second_offset = p->partial_offset + partial_bytes;
  p->barrier_offset = p->second_offset + second_bytes;
  *smem_bytes = stages * p->stage_bytes + fixed;
  return true;
}

}  // namespace stream
}  // namespace nml_sm100
