// The weights-stationary tcgen05 NVFP4 GEMM, shared by the dense linear and the grouped
// (routed-expert) projections.
//
//   D[n, m] = sum_k W'[n, k] * X[m, k]        W' = e2m1 code * e4m3 block scale (exact 16-bit)
//
// A tile of 128 weight rows is the UMMA M dimension; BM in {16..256} activation rows (dense)
// or schedule slots (grouped) are the UMMA N dimension, so packed weights are decoded once
// per K step whatever the number of rows.
//
// Three rings, each with its own producer and consumer, so that no stage waits for a
// consumer it does not need:
//   P ring   (PS stages of KS K-steps of 64): packed payload tile [128 x 32*KS B] by TMA, and,
//            when the decoded tiles live in shared memory, the stage's block-scale bytes by
//            4-byte cp.async.  Producer warp -> decode warps, which free a stage themselves.
//   X ring   (XS stages of KS K-steps): activation tiles [BM x 64], 128B-swizzled, by TMA
//            (dense, slot-ordered grouped) or by 16-byte cp.async gathers of scheduled rows.
//            X warp(s) -> MMA, freed by tcgen05.commit.
//   W' ring  (WB decoded operand tiles [128 x 64]): decode warps -> MMA, freed by commit.
//            Either in tensor memory (the MMA reads its A operand there; block scales of a
//            whole unit then arrive with one bulk copy into one of two buffers) or in shared
//            memory as UMMA K-major 128B-swizzled tiles.
// The packed weights are the only HBM stream; decoupling lets decode run WB tiles ahead of
// the MMA while the X ring alone sets how far the MMA's operands are prefetched.
// Warp roles: 0 payload producer, 1 MMA issuer + TMEM owner, 2-5 epilogue, then DG decode
// groups of four warps, then the X side (one TMA warp, or four row-gather warps), then the
// second MMA issuer if any.  Accumulators are double-buffered in TMEM; the kernel is persistent.
//
// Every mbarrier wait is bounded; a wait that runs out sets the barrier-timeout bit of the
// device status word and all roles leave through the common teardown.
//
// Parity waits cannot tell "phase k done" from "phase k - 1 not yet done": every waiter below
// either gates the reuse of what it waits on (its own arrival is needed before the barrier
// can advance again) or has itself consumed the previous phase.
#pragma once

#include <atomic>
#include <type_traits>

#include "common.cuh"
#include "sm100_primitives.cuh"

namespace nml_sm100 {
namespace umma {

enum Mode : int { kDense = 0, kGateUp = 1, kDown = 2 };
// kAbf16Lut: bf16 operands decoded through a byte -> two-bf16 table in shared memory instead
// of integer bit placement (a third of the integer-pipe work; needs 32 KB for the table).
enum AFormat : int { kAf16 = 0, kAbf16 = 1, kAbf16Lut = 2 };
constexpr int kLutBytes = 256 * 32 * 4;  // 256 entries, one copy per lane (bank)

constexpr int kTileN = 128;
constexpr int kTileK = 64;
constexpr int kUmmaK = 16;
constexpr int kProducerWarp = 0;
constexpr int kMmaWarp = 1;
constexpr int kEpilogueWarps = 4;
constexpr int kDecodeWarp0 = 6;
constexpr int kGroupThreads = 128;  // one decode group: one thread per weight row of the tile
constexpr int kGatherWarps = 4;
constexpr int kGatherThreads = kGatherWarps * 32;

// Thread budget of a launch with DG decode groups.  Group g decodes the K steps whose
// sequence number is congruent to g modulo DG, so DG K steps are in decode at once: the
// decode of one K step is a long dependent instruction chain, and it is the number of
// chains in flight, not the instruction count, that keeps the tensor pipe fed.
// Threads of a launch: the roles above, the X side (one warp issuing TMA loads, or the four
// gather warps), and one more warp when a second MMA issuer is used.
template <int DG, int MI, bool XTMA>
constexpr int launch_threads();

template <int DG>
struct Roles {
  static constexpr int kDecodeWarps = 4 * DG;
  static constexpr int kGatherWarp0 = kDecodeWarp0 + kDecodeWarps;
  static constexpr int kThreadsDense = (kGatherWarp0 + 1) * 32;
  static constexpr int kThreadsGrouped = (kGatherWarp0 + kGatherWarps) * 32;
};
template <int DG, int MI, bool XTMA>
constexpr int launch_threads() {
  return (XTMA ? Roles<DG>::kThreadsDense : Roles<DG>::kThreadsGrouped) + (MI == 2 ? 32 : 0);
}
constexpr int kWBytes = kTileN * 128;
constexpr int kSmemBudget = 227 * 1024;
constexpr int kMaxGroups = 256;

// WT: the decoded weight tiles live in tensor memory (the MMA reads its A operand there) and
// the block scales of a whole unit arrive with one bulk copy into one of two buffers;
// otherwise the decoded tiles form a shared-memory ring and every P stage carries its own
// scale bytes.
// BULK (always with WT, optional without): block scales by one bulk copy per unit.
template <int BM, int KS, int PS, int XS, int WB, bool GROUPED, bool WT, bool BULK = WT,
          bool LUT = false>
struct Layout {
  static_assert(BULK || !WT, "tensor-memory weight tiles take their scales by bulk copy");
  static constexpr int kPayloadBytes = kTileN * 32 * KS;
  static constexpr int kScaleBytes = BULK ? 0 : (kTileN * 4 * KS < 1024 ? 1024 : kTileN * 4 * KS);
  static constexpr int kPBytes = kPayloadBytes + kScaleBytes;  // one P stage
  static constexpr int kXBytes = BM * 128;                     // one K step of X
  static constexpr int kXStageBytes = KS * kXBytes;
  static constexpr int kXOffset = WT ? 0 : WB * kWBytes;       // the W' ring comes first
  static constexpr int kPOffset = kXOffset + XS * kXStageBytes;
  static constexpr int kLutOffset = kPOffset + PS * kPBytes;
  static constexpr int kBarrierOffset = kLutOffset + (LUT ? kLutBytes : 0);
  static constexpr int kBarrierBytes = 2048;
  // grouped: group table + one slot table (assignment id, routing weight) per epilogue warp
  static constexpr int kSlotTableBytes = GROUPED ? kEpilogueWarps * BM * 6 : 0;
  static constexpr int kGroupBytes =
      GROUPED ? ((kMaxGroups * 16 + 64 + kSlotTableBytes + 127) / 128) * 128 : 0;
  // BULK: two scale buffers of Params::scale_buffer_bytes each follow (sized at launch)
  static constexpr int kScaleBufferOffset = kBarrierOffset + kBarrierBytes + kGroupBytes;
  static constexpr int kSmemBytes = kScaleBufferOffset + 1024;  // + alignment slack
  static constexpr int kTmemColumns = 2 * BM < 32 ? 32 : 2 * BM;
  static_assert(kSmemBytes <= kSmemBudget, "shared memory budget exceeded");
  static_assert(kPBytes % 1024 == 0 && kXBytes % 1024 == 0, "stages keep 1024-byte alignment");
  static_assert(KS == 1 || KS == 2 || KS == 4, "K steps per stage");
};

// The one place that maps a kernel instantiation to its shared-memory layout; the kernel and
// its launchers both use it, so the launch can never reserve less than the kernel addresses.
template <int BM, int KS, int PS, int XS, int WB, bool WT, int AFMT, int MODE, bool SB>
using KernelLayout =
    Layout<BM, KS, PS, XS, WB, MODE != kDense, WT, WT || SB, AFMT == kAbf16Lut>;

struct Params {
  // weights
  const uint8_t* block_scales;
  const float* global_scale;
  const void* bias;
  int scale_width;        // K / 16
  int weight_rows_total;  // rows of the payload tensor (N, or experts * rows_per_expert)
  int rows_per_expert;    // grouped: 2I (gate/up) or H (down)
  // problem
  int M, N, K;            // dense: rows, outputs, inputs; grouped: N = output columns per expert
  int n_tiles, m_tiles, k_steps, n_fastest;
  int m_block;            // dense, m fastest: row tiles per block (0: all row tiles in one)
  void* output;
  // grouped
  const void* input;  // hidden [tokens, K] (gate/up) or activated [assignments, K] (down)
  const int32_t* sorted_assignments;
  const int32_t* block_experts;
  const int32_t* active_blocks;
  const int32_t* expert_offset;
  void* const* row_targets;       // down: optional destination of each assignment's row
  const float* tile_scale;        // dense: optional factor of the sums of every BM-row tile
  const uint32_t* gate;           // optional: the launch does nothing unless (*gate != 0) == gate_when
  int gate_when;
  const void* routing_weights;
  int assignments, schedule_blocks, experts, top_k;
  // dense: up to three weights that share the activation operand (fused Q/K/V); a plain
  // linear is one segment.  Weight tile t belongs to the last segment with tile_begin <= t.
  struct Segment {
    const uint8_t* block_scales;
    const float* global_scale;
    const void* bias;
    void* output;
    int outputs;     // rows of this weight = output columns
    int tile_begin;  // first weight tile of the segment
    const void* residual;  // dense: [M, outputs] added to the narrowed result, or null
  };
  Segment segment[3];
  int segments;
  // dense, few tiles: the K range of a unit is cut over the `split_k` CTAs of a cluster (one
  // unit per cluster); ranks > 0 hand their f32 partial tile to rank 0 through distributed
  // shared memory, rank 0 adds them in rank order (ascending K) and finishes the unit.
  int split_k;  // 1: no split
  int* status;
  int scale_buffer_bytes;  // BULK: bytes of one scale buffer (128 rows x scale_stride, 128-aligned)
  int scale_stride;        // BULK: bytes between the scale rows of a buffer (bulk_scale_stride)
  int scale_buffers;       // BULK: 2, or 1 when a second buffer would cost an activation stage
};

// One unit of work: a 128-row weight tile against BM activation rows / schedule slots.
struct Unit {
  int weight_row0;  // first row of the tile in the payload tensor
  int n0;           // first output column (dense) / first weight row inside the expert (grouped)
  int m0;           // dense: first activation row; grouped: first schedule slot
  int rows;         // grouped: valid slots in this unit (<= BM)
  int expert;       // grouped: local expert index
};

// Group table in shared memory (grouped mode): runs of schedule blocks with one expert.
struct Groups {
  int count;
  int total_units;
  int expert[kMaxGroups];
  int first_block[kMaxGroups];
  int blocks[kMaxGroups];
  int unit_prefix[kMaxGroups];
};

// ---- operand decode -------------------------------------------------------------------

// 8 codes (one payload word) -> 8 exact f16 products with the block scale, K order.
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
__device__ __forceinline__ void scales2_f16(uint32_t two_bytes, uint32_t& first,
                                            uint32_t& second) {
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

// 8 codes -> 8 exact bf16 values code * scale * 2^-7, K order.  scale2 holds
// bf16(scale * 2^119) in both halves.  The code's magnitude bits placed at bf16 bits 8:6
// read as value * 2^-126 (0.5 is the bf16 subnormal); the sign goes to bit 15.  Nibble i of
// each 16-bit half (codes i and i + 4) needs its own pair of shifts; all come from the one
// payload word, so there is no dependent shift chain.
__device__ __forceinline__ void decode8_bf16(uint32_t q, uint32_t scale2, uint32_t (&out)[4]) {
  constexpr uint32_t kSign = 0x80008000u, kMagnitude = 0x01c001c0u;
  uint32_t t[4];
  t[3] = (q & kSign) | ((q >> 6) & kMagnitude);
  t[2] = ((q << 4) & kSign) | ((q >> 2) & kMagnitude);
  t[1] = ((q << 8) & kSign) | ((q << 2) & kMagnitude);
  t[0] = ((q << 12) & kSign) | ((q << 6) & kMagnitude);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(t[i]) : "r"(scale2));
  }
  out[0] = __byte_perm(t[0], t[1], 0x5410);
  out[1] = __byte_perm(t[2], t[3], 0x5410);
  out[2] = __byte_perm(t[0], t[1], 0x7632);
  out[3] = __byte_perm(t[2], t[3], 0x7632);
}

// 8 codes -> 8 exact bf16 values code * scale through the byte table: entry stride 128 bytes,
// this lane's copy at `lut_lane`.  Four shift+mask pairs, four loads, four multiplies; the
// table already holds the two values of a byte in K order.
__device__ __forceinline__ void decode8_bf16_lut(uint32_t q, uint32_t scale2, uint32_t (&out)[4],
                                                 const uint8_t* lut_lane) {
  const uint32_t offset[4] = {(q << 7) & 0x7f80u, (q >> 1) & 0x7f80u, (q >> 9) & 0x7f80u,
                              (q >> 17) & 0x7f80u};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[i] = *reinterpret_cast<const uint32_t*>(lut_lane + offset[i]);
    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(out[i]) : "r"(scale2));
  }
}

// Four E4M3 scale bytes -> four words holding the exact bf16 scale in both halves (a byte's
// value bits at bf16 bits 10:4 read as scale * 2^-120).
__device__ __forceinline__ void scales4_bf16_true(uint32_t four_bytes, uint32_t (&scale)[4]) {
  const uint32_t two_p120 = 0x7b807b80u;
  uint32_t pair[2];
  pair[0] = __byte_perm(four_bytes, 0u, 0x4140);
  pair[1] = __byte_perm(four_bytes, 0u, 0x4342);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    pair[i] = (pair[i] & 0x007f007fu) << 4;
    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(pair[i]) : "r"(two_p120));
    scale[2 * i] = __byte_perm(pair[i], pair[i], 0x1010);
    scale[2 * i + 1] = __byte_perm(pair[i], pair[i], 0x3232);
  }
}

// Four E4M3 scale bytes -> four words holding bf16(scale * 2^119) in both halves: a byte's
// value bits at bf16 bits 10:4 read as scale * 2^-120; two exact bf16 multiplies rescale.
__device__ __forceinline__ void scales4_bf16(uint32_t four_bytes, uint32_t (&scale)[4]) {
  const uint32_t two_p120 = 0x7b807b80u;
  const uint32_t two_p119 = 0x7b007b00u;
  uint32_t pair[2];
  pair[0] = __byte_perm(four_bytes, 0u, 0x4140);  // byte 0 -> low half, byte 1 -> high half
  pair[1] = __byte_perm(four_bytes, 0u, 0x4342);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    pair[i] = (pair[i] & 0x007f007fu) << 4;
    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(pair[i]) : "r"(two_p120));
    asm("mul.rn.bf16x2 %0, %0, %1;" : "+r"(pair[i]) : "r"(two_p119));
    scale[2 * i] = __byte_perm(pair[i], pair[i], 0x1010);
    scale[2 * i + 1] = __byte_perm(pair[i], pair[i], 0x3232);
  }
}

// ---- unit enumeration -------------------------------------------------------------------

// Built by one warp: consecutive schedule blocks with the same (valid, local) expert form a
// group; a group is cut into slot tiles of BM and weight tiles of 128 rows.
__device__ __forceinline__ void build_groups(Groups* groups, const Params& p, int BM, int lane) {
  int blocks = p.schedule_blocks;
  if (p.active_blocks != nullptr) blocks = max(0, min(blocks, p.active_blocks[0]));
  const int offset = p.expert_offset != nullptr ? p.expert_offset[0] : 0;
  auto local_expert = [&](int b) -> int {
    if (b < 0 || b >= blocks) return -1;
    const int id = p.block_experts[b];
    const int local = id - offset;
    return (id >= 0 && local >= 0 && local < p.experts) ? local : -1;
  };
  int starts = 0, ends = 0;
  for (int base = 0; base < blocks; base += 32) {
    const int b = base + lane;
    const int e = local_expert(b);
    const bool is_start = e >= 0 && local_expert(b - 1) != e;
    const bool is_end = e >= 0 && local_expert(b + 1) != e;
    const unsigned start_mask = __ballot_sync(0xffffffffu, is_start);
    const unsigned end_mask = __ballot_sync(0xffffffffu, is_end);
    const unsigned below = (1u << lane) - 1u;
    const int start_index = starts + __popc(start_mask & below);
    const int end_index = ends + __popc(end_mask & below);
    if (is_start && start_index < kMaxGroups) {
      groups->expert[start_index] = e;
      groups->first_block[start_index] = b;
    }
    if (is_end && end_index < kMaxGroups) groups->blocks[end_index] = b + 1;  // end for now
    starts += __popc(start_mask);
    ends += __popc(end_mask);
  }
  __syncwarp();
  const int count = min(starts, kMaxGroups);
  // A schedule with more runs of equal experts than the table holds (blocks not sorted by
  // expert) cannot be walked completely: report it instead of dropping the tail silently.
  if (lane == 0 && starts > kMaxGroups) atomicOr(p.status, NML_SM100_STATUS_INDEX_RANGE);
  if (lane == 0) {
    int prefix = 0;
    for (int g = 0; g < count; ++g) {
      const int n_blocks = groups->blocks[g] - groups->first_block[g];
      groups->blocks[g] = n_blocks;
      groups->unit_prefix[g] = prefix;
      prefix += ((n_blocks * 16 + BM - 1) / BM) * p.n_tiles;
    }
    groups->count = count;
    groups->total_units = prefix;
  }
  __syncwarp();
}

template <int BM, bool GROUPED>
__device__ __forceinline__ int total_units(const Params& p, const Groups* groups) {
  if constexpr (GROUPED) {
    return groups->total_units;
  } else {
    return p.n_tiles * p.m_tiles;
  }
}

template <int BM, bool GROUPED>
__device__ __forceinline__ Unit get_unit(const Params& p, const Groups* groups, int index) {
  Unit u;
  if constexpr (GROUPED) {
    int lo = 0, hi = groups->count - 1;
    while (lo < hi) {  // last group whose prefix <= index
      const int mid = (lo + hi + 1) >> 1;
      if (groups->unit_prefix[mid] <= index) {
        lo = mid;
      } else {
        hi = mid - 1;
      }
    }
    const int local = index - groups->unit_prefix[lo];
    const int slot_tile = local / p.n_tiles;
    const int n_tile = local - slot_tile * p.n_tiles;
    u.expert = groups->expert[lo];
    u.n0 = n_tile * kTileN;
    u.weight_row0 = u.expert * p.rows_per_expert + u.n0;
    u.m0 = groups->first_block[lo] * 16 + slot_tile * BM;
    u.rows = min(BM, groups->blocks[lo] * 16 - slot_tile * BM);
  } else {
    int n_tile, m_tile;
    if (p.n_fastest) {
      m_tile = index / p.n_tiles;
      n_tile = index - m_tile * p.n_tiles;
    } else if (p.m_block > 0) {
      // m fastest inside blocks of m_block row tiles: the block's activations stay in L2 while
      // every weight tile passes over them; the weights stream once per block
      const int block_units = p.m_block * p.n_tiles;
      const int block = min(index / block_units, (p.m_tiles - 1) / p.m_block);
      const int block_tiles = min(p.m_block, p.m_tiles - block * p.m_block);
      const int inside = index - block * block_units;
      n_tile = inside / block_tiles;
      m_tile = block * p.m_block + (inside - n_tile * block_tiles);
    } else {
      n_tile = index / p.m_tiles;
      m_tile = index - n_tile * p.m_tiles;
    }
    int segment = 0;
    if (p.segments > 1 && n_tile >= p.segment[1].tile_begin) segment = 1;
    if (p.segments > 2 && n_tile >= p.segment[2].tile_begin) segment = 2;
    u.expert = segment;  // dense: index of the weight the tile belongs to
    u.n0 = (n_tile - p.segment[segment].tile_begin) * kTileN;
    u.weight_row0 = u.n0;
    u.m0 = m_tile * BM;
    u.rows = min(BM, p.M - u.m0);
  }
  return u;
}

// Which bounded wait ran out: bit (8 + site) of the device status word.
enum WaitSite : int {
  kSiteProducerRaw = 0,
  kSiteProducerScale = 1,
  kSiteProducerDrain = 2,
  kSiteMmaAccumulator = 3,
  kSiteMmaRaw = 4,
  kSiteMmaWeights = 5,
  kSiteEpilogue = 6,
  kSiteDecodeRaw = 7,
  kSiteDecodeWeights = 8,
  kSiteDecodeScale = 9,
  kSiteGather = 10,
};


struct RingState {
  int index = 0;
  uint32_t phase = 0;
  template <int N>
  __device__ __forceinline__ void advance() {
    if (++index == N) {
      index = 0;
      phase ^= 1u;
    }
  }
};

// ---- the kernel ---------------------------------------------------------------------------

// XTMA: the activation operand arrives by TMA from a row-contiguous tensor (always for
// dense; for grouped modes when the caller permuted the rows into schedule-slot order, in
// which case gate/up also writes its result in slot order).  Otherwise (grouped only) rows
// are gathered by assignment with cp.async.
// PA: partial accumulators per tile.  Consecutive tcgen05.mma into one accumulator form a
// dependent chain whose per-instruction latency (not its throughput) bounds tiles with few
// activation rows, so the K=16 slices rotate over PA accumulators (instruction i of a unit
// goes to accumulator i % PA) and the epilogue adds them in index order.
template <int BM, int KS, int PS, int XS, int WB, int DG, int MI, int PA, bool WT, int AFMT,
          typename T, int MODE, bool XTMA, bool SB = false>
__global__ void __launch_bounds__(launch_threads<DG, MI, XTMA>(), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_payload,
            const __grid_constant__ CUtensorMap tmap_x, const Params p,
            const __grid_constant__ CUtensorMap tmap_payload1,
            const __grid_constant__ CUtensorMap tmap_payload2) {
  // Two launches share one decision made on the device (see narrow_rows_kernel): each reads
  // the word and the one it does not name returns before it touches anything.
  if (p.gate != nullptr && (__ldg(p.gate) != 0u) != (p.gate_when != 0)) return;
  constexpr bool GROUPED = MODE != kDense;
  constexpr int kGatherWarp0 = Roles<DG>::kGatherWarp0;  // first warp of the X side
  constexpr int kMmaWarpB = XTMA ? kGatherWarp0 + 1 : kGatherWarp0 + kGatherWarps;
  static_assert(2 * PA * BM <= 512, "partial accumulators exceed tensor memory");
  static_assert(MI == 1 || (PA >= 2 && PA % 2 == 0),
                "two issuers need disjoint sets of partial accumulators");
  static_assert(WB > DG, "the W' ring must hold one tile per decode group plus one");
  static_assert(GROUPED || XTMA, "the dense mode always loads activations by TMA");
  constexpr bool kBulk = WT || SB;  // block scales of a unit by one bulk copy
  constexpr bool kLut = AFMT == kAbf16Lut;
  using L = KernelLayout<BM, KS, PS, XS, WB, WT, AFMT, MODE, SB>;
  constexpr int kWColumns = kTileK / 2;                // one decoded K step: 64 x 16 bit per row
  // Two accumulator sets of PA partials overlap a unit's epilogue with the next unit's MMAs.
  // Where they do not fit beside the W' tiles in tensor memory (256 activation rows) there is
  // one set: the MMA warp then waits for the epilogue, while the decode warps run ahead into
  // the W' ring.
  constexpr int kAccSets = (WT && PA * L::kTmemColumns + WB * kWColumns > 512) ? 1 : 2;
  constexpr int kAccColumns = kAccSets * PA * (L::kTmemColumns / 2);
  constexpr int kTmemNeeded = kAccColumns + (WT ? WB * kWColumns : 0);
  constexpr int kTmemColumns = kTmemNeeded <= 32    ? 32
                               : kTmemNeeded <= 64  ? 64
                               : kTmemNeeded <= 128 ? 128
                               : kTmemNeeded <= 256 ? 256
                                                    : 512;
  static_assert(kTmemNeeded <= 512, "tensor memory budget exceeded");
  // With one K step per stage and equally deep X and W' rings the two advance in lockstep, so
  // the commit that frees a W' tile also frees the X stage of the same index.
  constexpr bool kSharedEmpty = KS == 1 && XS == WB && MI == 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  auto w_tile = [&](int w) { return smem + w * kWBytes; };
  auto x_tile = [&](int r, int j) { return smem + L::kXOffset + r * L::kXStageBytes + j * L::kXBytes; };
  auto payload_tile = [&](int r) { return smem + L::kPOffset + r * L::kPBytes; };
  auto scale_tile = [&](int r) { return payload_tile(r) + L::kPayloadBytes; };
  auto scale_buffer = [&](int b) { return smem + L::kScaleBufferOffset + b * p.scale_buffer_bytes; };
  // split K, rank 0: f32 partial tiles [128 x BM] of ranks 1.. behind the scale buffers
  auto partial_tile = [&](int i) {
    return reinterpret_cast<float*>(smem + L::kScaleBufferOffset +
                                    p.scale_buffers * p.scale_buffer_bytes +
                                    i * (kTileN * BM * 4));
  };
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarrierOffset);
  uint64_t* full_p = bars;                 // [PS]
  uint64_t* empty_p = full_p + PS;         // [PS]
  uint64_t* full_x = empty_p + PS;         // [XS]
  uint64_t* empty_x = full_x + XS;         // [XS]
  uint64_t* full_w = empty_x + XS;         // [WB]
  uint64_t* empty_w = full_w + WB;         // [WB]
  uint64_t* tmem_full = empty_w + WB;      // [2]
  uint64_t* tmem_empty = tmem_full + 2;    // [2]
  uint64_t* full_scale = tmem_empty + 2;   // [2] (WT)
  uint64_t* empty_scale = full_scale + 2;  // [2] (WT)
  uint64_t* partial_full = empty_scale + 2;  // [1] (split K, rank 0: partial tiles have landed)
  uint64_t* mma_drained = partial_full + 1;  // [1] every MMA of this CTA has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_drained + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((2 * PS + 2 * XS + 2 * WB + 10) * 8 + 8 <= L::kBarrierBytes, "barrier area");
  Groups* groups = reinterpret_cast<Groups*>(smem + L::kBarrierOffset + L::kBarrierBytes);
  uint64_t* x_free = kSharedEmpty ? empty_w : empty_x;
  // Per-unit weight operands: in dense mode they come from the unit's segment.
  // the scale buffer and barrier phase of the CTA's `local`-th unit
  auto scale_slot = [&](int local) { return p.scale_buffers == 2 ? (local & 1) : 0; };
  auto scale_phase = [&](int local) -> uint32_t {
    return p.scale_buffers == 2 ? ((local >> 1) & 1) : (local & 1);
  };
  auto scale_base = [&](const Unit& u) -> const uint8_t* {
    return GROUPED ? p.block_scales : p.segment[u.expert].block_scales;
  };
  auto weight_rows = [&](const Unit& u) -> int {
    return GROUPED ? p.weight_rows_total : p.segment[u.expert].outputs;
  };
  auto payload_map = [&](const Unit& u) -> const CUtensorMap* {
    if constexpr (!GROUPED) {
      if (u.expert == 1) return &tmap_payload1;
      if (u.expert == 2) return &tmap_payload2;
    }
    return &tmap_payload;
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int r = 0; r < PS; ++r) {
      mbar_init(&full_p[r], 1 + (kBulk ? 0 : 32));  // expect_tx arrival (+ the lanes' scale copies)
      mbar_init(&empty_p[r], 4 * DG);            // every decode warp
    }
    for (int r = 0; r < XS; ++r) {
      mbar_init(&full_x[r], XTMA ? 1 : kGatherWarps);
      mbar_init(&empty_x[r], MI);
    }
    for (int w = 0; w < WB; ++w) {
      mbar_init(&full_w[w], kGroupThreads / 32);
      mbar_init(&empty_w[w], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], MI);
      mbar_init(&tmem_empty[a], kEpilogueWarps);
      mbar_init(&full_scale[a], 1);
      mbar_init(&empty_scale[a], 4 * DG);
    }
    mbar_init(partial_full, p.split_k > 1 ? (p.split_k - 1) * kEpilogueWarps : 1);
    mbar_init(mma_drained, MI);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kProducerWarp) {
    if (lane == 0) {
      tma_prefetch_descriptor(&tmap_payload);
      if (!GROUPED && p.segments > 1) tma_prefetch_descriptor(&tmap_payload1);
      if (!GROUPED && p.segments > 2) tma_prefetch_descriptor(&tmap_payload2);
    }
    if constexpr (GROUPED) build_groups(groups, p, BM, lane);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemColumns);
    tmem_relinquish_alloc_permit();
  }
  if constexpr (kLut) {
    // entry b = bf16 values of the two codes of byte b (low nibble in the low half); copy
    // `lane` of an entry sits in bank `lane`, so a warp's 32 lookups never conflict
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem + L::kLutOffset);
    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
      const uint32_t byte = static_cast<uint32_t>(i) >> 5;
      uint32_t entry = 0;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t code = (byte >> (4 * half)) & 0xfu;
        const uint32_t m = code & 0x7u;
        uint32_t bits = m == 0 ? 0u : m == 1 ? 0x3f00u : ((126u + (m >> 1)) << 7) | ((m & 1u) << 6);
        bits |= (code & 0x8u) << 12;
        entry |= bits << (16 * half);
      }
      lut[i] = entry;
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int units = total_units<BM, GROUPED>(p, groups);
  // K range of this CTA and the units it walks (split K: one unit per cluster, a K slice per
  // CTA; otherwise every K step and a persistent walk over the units)
  int k_begin = 0, k_count = p.k_steps;
  int first_unit = blockIdx.x, unit_stride = gridDim.x;
  uint32_t split_rank = 0;
  const bool split = !GROUPED && p.split_k > 1;
  if (split) {
    split_rank = cluster_cta_rank();
    const int share = p.k_steps / p.split_k, extra = p.k_steps % p.split_k;
    k_count = share + (static_cast<int>(split_rank) < extra ? 1 : 0);
    k_begin = static_cast<int>(split_rank) * share + min(static_cast<int>(split_rank), extra);
    first_unit = blockIdx.x / p.split_k;
    unit_stride = gridDim.x / p.split_k;
    // remote arrivals must find initialised barriers
    cluster_sync_all();
  }
  const int stages = (k_count + KS - 1) / KS;  // per unit, of the P ring and of the X ring

  // `site` says which wait ran out (diagnostic bits 8.. of the status word).
  auto give_up = [&](int site) {
    *abort_flag = 1;
    atomicOr(p.status, NML_SM100_STATUS_BARRIER_TIMEOUT | (0x100 << site));
  };
  // Bounded wait that also honours an abort raised by another role.
  auto wait = [&](uint64_t* bar, uint32_t parity, int site) -> bool {
    if (mbar_try_wait(bar, parity)) return true;  // fast path: no shared-memory flag read
    for (uint32_t poll = 0; poll < kWaitPolls; ++poll) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((poll & 63u) == 63u && *abort_flag) {
        return false;
      }
    }
    give_up(site);
    return false;
  };
  if (warp == kProducerWarp) {
    // ---------------------------------------------------------- payload producer
    RingState ps;
    int issued = 0;
    int local = 0;
    bool ok = true;
    for (int index = first_unit; index < units && ok; index += unit_stride, ++local) {
      const Unit u = get_unit<BM, GROUPED>(p, groups, index);
      // All block scales of the unit's weight rows: one contiguous range of the tensor, copied
      // at once, or row by row when the rows are padded apart in shared memory.  With two
      // buffers the copy goes first; with one it has to wait for the previous unit's decode to
      // end, so the first payload stages of this unit are put in flight before it (it must
      // still precede the wait for a stage that only this unit's decode can free).
      auto issue_scales = [&]() -> bool {
        const int b = scale_slot(local);
        if (!wait(&empty_scale[b], scale_phase(local) ^ 1u, kSiteProducerScale)) return false;
        const int rows = min(kTileN, weight_rows(u) - u.weight_row0);
        const uint8_t* from =
            scale_base(u) + static_cast<int64_t>(u.weight_row0) * p.scale_width;
        if (lane == 0) {
          mbar_arrive_expect_tx(&full_scale[b], static_cast<uint32_t>(rows * p.scale_width));
          if (p.scale_stride == p.scale_width) {
            bulk_load(scale_buffer(b), from, static_cast<uint32_t>(rows * p.scale_width),
                      &full_scale[b]);
          }
        }
        if (p.scale_stride != p.scale_width) {
          __syncwarp();
          for (int r = lane; r < rows; r += 32) {
            bulk_load(scale_buffer(b) + r * p.scale_stride, from + r * p.scale_width,
                      static_cast<uint32_t>(p.scale_width), &full_scale[b]);
          }
          __syncwarp();
        }
        return true;
      };
      const int scales_at = p.scale_buffers == 2 ? 0 : min(PS, stages) - 1;
      for (int rs = 0; rs < stages; ++rs) {
        if constexpr (kBulk) {
          if (rs == scales_at && !issue_scales()) {
            ok = false;
            break;
          }
        }
        if (!wait(&empty_p[ps.index], ps.phase ^ 1u, kSiteProducerRaw)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&full_p[ps.index], L::kPayloadBytes);
          tma_load_2d(payload_tile(ps.index), payload_map(u), &full_p[ps.index],
                      (k_begin + rs * KS) * 32, u.weight_row0);
        }
        if constexpr (!kBulk) {
          // block scales: 4 bytes per row and K step (scale rows are not TMA-legal)
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            const int k_step = k_begin + rs * KS + j;
            if (rs * KS + j < k_count) {
#pragma unroll
              for (int i = 0; i < kTileN / 32; ++i) {
                const int row = lane + 32 * i;
                const int n = min(u.weight_row0 + row, weight_rows(u) - 1);
                cp_async_4(scale_tile(ps.index) + row * (4 * KS) + j * 4,
                           scale_base(u) + static_cast<int64_t>(n) * p.scale_width + k_step * 4);
              }
            }
          }
          cp_async_mbar_arrive_noinc(&full_p[ps.index]);
        } else {
          __syncwarp();
        }
        ++issued;
        ps.advance<PS>();
      }
    }
    // Do not leave while copies this warp started may still be landing in shared memory.
    const int pending = issued < PS ? issued : PS;
    for (int i = 0; i < pending; ++i) {
      ps.index = ps.index == 0 ? PS - 1 : ps.index - 1;
      if (ps.index == PS - 1) ps.phase ^= 1u;
      if (!mbar_wait(&full_p[ps.index], ps.phase)) give_up(kSiteProducerDrain);
    }
    if constexpr (kBulk) {
      for (int back = 1; back <= p.scale_buffers && back <= local; ++back) {
        const int unit = local - back;
        if (!mbar_wait(&full_scale[scale_slot(unit)], scale_phase(unit))) {
          give_up(kSiteProducerDrain);
        }
      }
    }
  } else if (XTMA && warp == kGatherWarp0) {
    // ------------------------------------------------------- activation producer
    if constexpr (XTMA) {
      RingState xs;
      int issued = 0;
      bool ok = true;
      if (lane == 0) tma_prefetch_descriptor(&tmap_x);
      for (int index = first_unit; index < units && ok; index += unit_stride) {
        const Unit u = get_unit<BM, GROUPED>(p, groups, index);
        for (int rs = 0; rs < stages; ++rs) {
          if (!wait(&x_free[xs.index], xs.phase ^ 1u, kSiteGather)) {
            ok = false;
            break;
          }
          if (lane == 0) {
            // the box always covers KS K steps; columns past K read as zeros
            mbar_arrive_expect_tx(&full_x[xs.index], L::kXStageBytes);
            if constexpr (KS == 1) {
              tma_load_2d(x_tile(xs.index, 0), &tmap_x, &full_x[xs.index],
                          (k_begin + rs) * kTileK, u.m0);
            } else {
              // the activation map is a 3-D view [K/64][rows][64]: one box carries KS K steps
              tma_load_3d(x_tile(xs.index, 0), &tmap_x, &full_x[xs.index], 0, u.m0,
                          k_begin + rs * KS);
            }
          }
          __syncwarp();
          ++issued;
          xs.advance<XS>();
        }
      }
      const int pending = issued < XS ? issued : XS;
      for (int i = 0; i < pending; ++i) {
        xs.index = xs.index == 0 ? XS - 1 : xs.index - 1;
        if (xs.index == XS - 1) xs.phase ^= 1u;
        if (!mbar_wait(&full_x[xs.index], xs.phase)) give_up(kSiteProducerDrain);
      }
    }
  } else if (warp == kMmaWarp || (MI == 2 && warp == kMmaWarpB)) {
    // ----------------------------------------------------------------------- MMA
    // With MI == 2 two warps issue alternate K steps into disjoint partial accumulators that
    // the epilogue adds in a fixed order, so the split stays deterministic.  Ownership
    // follows the parity of the K step's position in the CTA's whole sequence (not inside
    // the unit): with an even ring depth every W' slot then has one consumer for good.  A
    // parity wait cannot tell "phase k done" from "phase k - 1 not yet done", so a consumer
    // may only wait on a slot whose previous use it has consumed itself; an issuer that took
    // over a slot at a unit boundary (odd K steps per unit) could run ahead of the other
    // issuer and pass that wait a whole phase early.
    const int issuer = warp == kMmaWarp ? 0 : 1;
    static_assert(MI == 1 || WB % 2 == 0, "two issuers need an even W' ring depth");
    // The decode side has the mirror-image rule: group g may wait for the consumption of
    // position Q - WB only when Q - 2 WB is known consumed.  Its own history gives
    // Q - i DG - WB consumed; with one in-order issuer i = 1 suffices (WB >= DG), with two
    // the position must also share Q's parity, i.e. i DG even.
    static_assert(MI == 1 || (DG % 2 == 0 ? DG : 2 * DG) <= WB,
                  "W' ring too shallow for two issuers");
    // Every lane runs this loop and one elected lane issues: the loop then is uniform to the
    // compiler, which keeps descriptors and addresses in uniform registers.  The waits return
    // nothing (see mbar_wait_or_abort), so a timeout does not make the control flow divergent.
    {
      constexpr uint32_t a_format = AFMT == kAf16 ? kUmmaF16 : kUmmaBF16;
      // the activation tile holds F16 also when a BF16 call narrowed its rows beforehand
      constexpr uint32_t b_format =
          (std::is_same<T, __half>::value || AFMT == kAf16) ? kUmmaF16 : kUmmaBF16;
      // Tall tiles issue only as many activation rows (the MMA's N) as the unit has, rounded
      // up to 16: an expert's last slot tile, or the last rows of a dense operand, then costs
      // its share of the tensor pipe and of the operand reads instead of a full tile's.
      constexpr bool kDynamicRows = BM >= 64;
      constexpr uint64_t desc_hi = static_cast<uint64_t>(kUmmaDescHiSw128) << 32;
      RingState xs, wb;
      int local = 0;
      int sequence = 0;  // K steps seen so far by this CTA, over all units
      const uint64_t w_desc = desc_hi | (WT ? 0u : umma_desc_lo(smem_u32(w_tile(0))));
      const uint64_t x_desc = desc_hi | umma_desc_lo(smem_u32(x_tile(0, 0)));
      for (int index = first_unit; index < units; index += unit_stride, ++local) {
        // After a timeout anywhere in the CTA nothing further is issued: the waits below have
        // become no-ops and the operands would not be ready.
        if (__shfl_sync(0xffffffffu, *abort_flag, 0) != 0) break;
        const int acc = kAccSets == 2 ? (local & 1) : 0;
        const uint32_t acc_phase = kAccSets == 2 ? ((local >> 1) & 1) : (local & 1);
        mbar_wait_or_abort(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, p.status,
                           kSiteMmaAccumulator);
        tcgen05_fence_after_sync();
        uint32_t issued_rows = BM;
        if constexpr (kDynamicRows) {
          const Unit u = get_unit<BM, GROUPED>(p, groups, index);
          issued_rows = static_cast<uint32_t>(min(BM, max(16, (u.rows + 15) & ~15)));
        }
        const uint32_t idesc = umma_idesc_f16(a_format, b_format, kTileN, issued_rows);
        const uint32_t d_base = tmem_base + acc * PA * BM;
        int step = 0;  // K step inside the unit
        for (int rs = 0; rs < stages; ++rs) {
          mbar_wait_or_abort(&full_x[xs.index], xs.phase, abort_flag, p.status,
                             kSiteMmaRaw);
          const int sub_steps = min(KS, k_count - rs * KS);
          for (int j = 0; j < sub_steps; ++j, ++step, ++sequence, wb.advance<WB>()) {
            if (MI == 2 && (sequence & 1) != issuer) continue;
            mbar_wait_or_abort(&full_w[wb.index], wb.phase, abort_flag, p.status,
                               kSiteMmaWeights);
            // Orders the MMAs after the decode threads' tensor-memory stores.  A decoded tile
            // in shared memory needs no such fence: its writers fenced the async proxy before
            // they arrived on the barrier.
            if constexpr (WT) tcgen05_fence_after_sync();
            // Descriptors differ only in the start-address field (16-byte units); each
            // K=16 slice is 32 bytes further along the swizzled 128-byte rows.
            const uint32_t a_tmem = tmem_base + kAccColumns + wb.index * kWColumns;
            const uint64_t a_desc = w_desc + wb.index * (kWBytes >> 4);
            const uint64_t b_desc =
                x_desc + xs.index * (L::kXStageBytes >> 4) + j * (L::kXBytes >> 4);
#pragma unroll
            for (int q = 0; q < kTileK / kUmmaK; ++q) {
              const int instruction = step * (kTileK / kUmmaK) + q;
              // One issuer: slice i of the unit goes to partial accumulator i % PA.  Two
              // issuers: the K step's parity picks a half of the accumulators (a K step has
              // one issuer, so the halves never share a writer), q walks inside the half.
              constexpr int kHalf = PA / 2;
              const int partial = MI == 2 ? (step & 1) * kHalf + q % (kHalf > 0 ? kHalf : 1)
                                          : instruction % PA;
              const bool first = MI == 2 ? (step < 2 && q < kHalf) : instruction < PA;
              const uint32_t d = d_base + partial * BM;
              const uint32_t accumulate = first ? 0u : 1u;
              if constexpr (WT) {
                umma_f16_tmem_a_elect(d, a_tmem + q * (kUmmaK / 2), b_desc + 2 * q, idesc,
                                      accumulate);
              } else {
                umma_f16_elect(d, a_desc + 2 * q, b_desc + 2 * q, idesc, accumulate);
              }
            }
            umma_commit_elect(&empty_w[wb.index]);
          }
          if constexpr (!kSharedEmpty) {
            umma_commit_elect(&empty_x[xs.index]);
          }
          xs.advance<XS>();
        }
        umma_commit_elect(&tmem_full[acc]);
      }
      // Tensor memory and the barriers may only be released once every MMA this warp issued
      // (and the arrival of its commits) has completed, also on the abort path.
      umma_commit_elect(mma_drained);
      if (!mbar_wait(mma_drained, 0)) give_up(kSiteMmaAccumulator);
    }
    __syncwarp();
  } else if (warp < kDecodeWarp0) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes a warp may read: 32 * (warp % 4)
    constexpr float kDecodeFactor = AFMT == kAbf16 ? 128.0f : 1.0f;
    float g = GROUPED ? __ldg(p.global_scale) * kDecodeFactor : 0.0f;
    T* out = static_cast<T*>(p.output);
    const T* bias = static_cast<const T*>(p.bias);
    const T* residual = nullptr;  // dense: the segment's residual operand
    int out_columns = p.N;
    const int row = quarter * 32 + lane;  // row of the weight tile this thread reads
    int local = 0;
    for (int index = first_unit; index < units; index += unit_stride, ++local) {
      const Unit u = get_unit<BM, GROUPED>(p, groups, index);
      const int acc = kAccSets == 2 ? (local & 1) : 0;
      const uint32_t acc_phase = kAccSets == 2 ? ((local >> 1) & 1) : (local & 1);
      if (!wait(&tmem_full[acc], acc_phase, kSiteEpilogue)) break;
      tcgen05_fence_after_sync();
      // Grouped modes that address the output by assignment keep the unit's slot -> (assignment,
      // routing weight) map in a table private to this warp, filled with coalesced loads.
      constexpr bool kSlotOutput = MODE == kGateUp && XTMA;  // result rows in slot order
      constexpr bool kNeedsTable = GROUPED && !kSlotOutput;
      int32_t* slot_assignment = nullptr;
      uint16_t* slot_weight = nullptr;
      uint32_t chunk_valid = 0;  // bit i: the slots 32 i .. 32 i + 31 all carry an assignment
      if constexpr (kNeedsTable) {
        uint8_t* table = reinterpret_cast<uint8_t*>(groups) + (kMaxGroups * 16 + 64) +
                         (warp & 3) * (BM * 6);
        slot_assignment = reinterpret_cast<int32_t*>(table);
        slot_weight = reinterpret_cast<uint16_t*>(table + BM * 4);
        __syncwarp();
        for (int r = lane; r < BM; r += 32) {
          int32_t a = -1;
          uint16_t weight_bits = 0;
          if (r < u.rows) {
            const int32_t candidate = p.sorted_assignments[u.m0 + r];
            if (candidate >= 0 && candidate < p.assignments) {
              a = candidate;
              if constexpr (MODE == kDown) {
                weight_bits = static_cast<const uint16_t*>(p.routing_weights)[a];
              }
            }
          }
          slot_assignment[r] = a;
          slot_weight[r] = weight_bits;
          if constexpr (BM >= 32) {  // every lane runs every iteration
            if (__all_sync(0xffffffffu, a >= 0)) chunk_valid |= 1u << (r >> 5);
          }
        }
        __syncwarp();
      }
      if constexpr (!GROUPED) {
        const Params::Segment& segment = p.segment[u.expert];
        g = __ldg(segment.global_scale) * kDecodeFactor;
        if (p.tile_scale != nullptr) g *= __ldg(p.tile_scale + u.m0 / BM);  // a power of two
        out = static_cast<T*>(segment.output);
        bias = static_cast<const T*>(segment.bias);
        residual = static_cast<const T*>(segment.residual);
        out_columns = segment.outputs;
      }
      const int n = u.n0 + row;  // output column (dense, down) or weight row in the expert
      const bool n_ok = n < (MODE == kGateUp ? p.rows_per_expert : out_columns);
      float bias_value = 0.0f;
      if (bias != nullptr && n_ok) {
        bias_value = Elem<T>::load(
            bias[(GROUPED ? static_cast<int64_t>(u.expert) * p.rows_per_expert : 0) + n]);
      }
      constexpr int kChunk = BM >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c = 0; c < BM; c += kChunk) {
        if (BM >= 64 && c >= u.rows) break;  // columns the MMAs of this unit did not write
        const uint32_t address =
            tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * PA * BM + c;
        uint32_t v[kChunk];
        if constexpr (kChunk == 32) {
          tmem_load_32x32(address, v);
        } else {
          tmem_load_32x16(address, v);
        }
        tmem_load_wait();
        if constexpr (PA > 1) {
          // add the other partial accumulators in index order; a unit with few K steps has
          // touched only the first 4 * k_steps of them
          const int used = MI == 2 ? (k_count > 1 ? PA : min(PA / 2, kTileK / kUmmaK))
                                   : min(PA, k_count * (kTileK / kUmmaK));
#pragma unroll 1
          for (int partial = 1; partial < used; ++partial) {
            uint32_t extra[kChunk];
            if constexpr (kChunk == 32) {
              tmem_load_32x32(address + partial * BM, extra);
            } else {
              tmem_load_32x16(address + partial * BM, extra);
            }
            tmem_load_wait();
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), __uint_as_float(extra[j])));
            }
          }
        }
        if (c >= u.rows) continue;  // uniform: nothing valid left in this chunk
        if constexpr (MODE == kDense) {
          if (split) {
            if (split_rank != 0) {
              // hand this K slice's partial sums to rank 0 and skip the store
              const uint32_t local = smem_u32(partial_tile(static_cast<int>(split_rank) - 1)) +
                                     static_cast<uint32_t>(row * BM + c) * 4u;
              const uint32_t remote = cluster_map_shared(local, 0);
#pragma unroll
              for (int j = 0; j < kChunk; j += 4) {
                cluster_store_f32x4(remote + j * 4, __uint_as_float(v[j]),
                                    __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                    __uint_as_float(v[j + 3]));
              }
              continue;
            }
            if (c == 0) {
              bool landed = false;
              for (uint32_t poll = 0; poll < kWaitPolls && !landed; ++poll) {
                landed = mbar_try_wait_cluster(partial_full, 0);
              }
              if (!landed) give_up(kSiteEpilogue);
            }
            for (int other = 1; other < p.split_k; ++other) {  // ascending K
              const float* partial = partial_tile(other - 1) + row * BM + c;
#pragma unroll
              for (int j = 0; j < kChunk; j += 4) {
                const float4 add = *reinterpret_cast<const float4*>(partial + j);
                v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), add.x));
                v[j + 1] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 1]), add.y));
                v[j + 2] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 2]), add.z));
                v[j + 3] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 3]), add.w));
              }
            }
          }
          // two copies of the store loop: the residual form costs the plain one nothing
          if (n_ok && residual == nullptr) {
            T* target = out + static_cast<int64_t>(u.m0 + c) * out_columns + n;
            if (c + kChunk <= u.rows) {  // a full chunk: no test per row (measured +5..9 %)
#pragma unroll
              for (int j = 0; j < kChunk; ++j) {
                target[static_cast<int64_t>(j) * out_columns] =
                    Elem<T>::store(fmaf(__uint_as_float(v[j]), g, bias_value));
              }
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j) {
                if (c + j < u.rows) {
                  target[static_cast<int64_t>(j) * out_columns] =
                      Elem<T>::store(fmaf(__uint_as_float(v[j]), g, bias_value));
                }
              }
            }
          } else if (n_ok && c + kChunk <= u.rows) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int64_t index = static_cast<int64_t>(u.m0 + c + j) * out_columns + n;
              out[index] = narrow_with_residual<T>(fmaf(__uint_as_float(v[j]), g, bias_value),
                                                   residual, index);
            }
          } else if (n_ok) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int m = u.m0 + c + j;
              if (c + j < u.rows) {
                const int64_t index = static_cast<int64_t>(m) * out_columns + n;
                out[index] = narrow_with_residual<T>(
                    fmaf(__uint_as_float(v[j]), g, bias_value), residual, index);
              }
            }
          }
        } else if constexpr (MODE == kDown) {
          if (p.row_targets == nullptr && n_ok && ((chunk_valid >> (c / kChunk)) & 1u) != 0) {
            // every slot of the chunk carries an assignment: no test per row
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int a = slot_assignment[c + j];
              const float weight = Elem<T>::from_bits(slot_weight[c + j]);
              out[static_cast<int64_t>(a) * p.N + n] =
                  Elem<T>::store(fmaf(__uint_as_float(v[j]), g, bias_value) * weight);
            }
          } else if (p.row_targets == nullptr) {
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int a = slot_assignment[c + j];
              if (n_ok && a >= 0) {
                const float weight = Elem<T>::from_bits(slot_weight[c + j]);
                out[static_cast<int64_t>(a) * p.N + n] =
                    Elem<T>::store(fmaf(__uint_as_float(v[j]), g, bias_value) * weight);
              }
            }
          } else {
            // the caller's table says where each assignment's row goes (an expert-parallel
            // owner: straight into the sender's return buffer, over NVLink)
#pragma unroll
            for (int j = 0; j < kChunk; ++j) {
              const int a = slot_assignment[c + j];
              if (n_ok && a >= 0) {
                T* destination = static_cast<T*>(p.row_targets[a]);
                if (destination != nullptr) {
                  const float weight = Elem<T>::from_bits(slot_weight[c + j]);
                  destination[n] =
                      Elem<T>::store(fmaf(__uint_as_float(v[j]), g, bias_value) * weight);
                }
              }
            }
          }
        } else {
          // gate/up: even tile rows carry gate, odd rows carry up of the same intermediate
          // column.  Lane pairs swap one value per column pair, so the even lane finishes
          // column c+2q and the odd lane column c+2q+1.
          const bool odd = (lane & 1) != 0;
          const int column = n >> 1;  // intermediate column inside the expert
          // full chunks (slot order: all rows exist; by assignment: all slots carry one) store
          // without a test per row
          const bool full_chunk = kSlotOutput ? c + kChunk <= u.rows
                                              : ((chunk_valid >> (c / kChunk)) & 1u) != 0;
          if (full_chunk) {
#pragma unroll
            for (int q = 0; q < kChunk / 2; ++q) {
              const float mine_even = fmaf(__uint_as_float(v[2 * q]), g, bias_value);
              const float mine_odd = fmaf(__uint_as_float(v[2 * q + 1]), g, bias_value);
              const float received =
                  __shfl_xor_sync(0xffffffffu, odd ? mine_even : mine_odd, 1);
              const int j = 2 * q + (odd ? 1 : 0);
              const float gate = odd ? received : mine_even;
              const float up = odd ? mine_odd : received;
              int64_t target_row;
              if constexpr (kSlotOutput) {
                target_row = u.m0 + c + j;
              } else {
                target_row = slot_assignment[c + j];
              }
              if (n_ok) out[target_row * p.N + column] = Elem<T>::store(clamped_swiglu(gate, up));
            }
            continue;
          }
#pragma unroll
          for (int q = 0; q < kChunk / 2; ++q) {
            const float mine_even = fmaf(__uint_as_float(v[2 * q]), g, bias_value);
            const float mine_odd = fmaf(__uint_as_float(v[2 * q + 1]), g, bias_value);
            const float received =
                __shfl_xor_sync(0xffffffffu, odd ? mine_even : mine_odd, 1);
            const int j = 2 * q + (odd ? 1 : 0);
            const float gate = odd ? received : mine_even;
            const float up = odd ? mine_odd : received;
            if constexpr (kSlotOutput) {
              if (n_ok && c + j < u.rows) {
                out[static_cast<int64_t>(u.m0 + c + j) * p.N + column] =
                    Elem<T>::store(clamped_swiglu(gate, up));
              }
            } else {
              const int a = slot_assignment[c + j];
              if (n_ok && a >= 0) {
                out[static_cast<int64_t>(a) * p.N + column] =
                    Elem<T>::store(clamped_swiglu(gate, up));
              }
            }
          }
        }
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if constexpr (MODE == kDense) {
        if (split && split_rank != 0 && lane == 0) {
          // this warp's share of the partial tile is written: tell rank 0
          cluster_mbar_arrive(cluster_map_shared(smem_u32(partial_full), 0));
        }
      }
    }
    if constexpr (MODE == kDown) {
      // Rows stored through the caller's table may sit in another GPU's memory, and the flag
      // that announces them is raised by a later launch: every writer orders its own stores
      // at system scope before the kernel ends (a fence by another thread, or the end of the
      // grid, does not wait for posted peer writes).
      if (p.row_targets != nullptr) __threadfence_system();
    }
  } else if (warp < kGatherWarp0) {
    // -------------------------------------------------------------------- decode
    const int dt = threadIdx.x - kDecodeWarp0 * 32;
    const int group = dt / kGroupThreads;
    // Weight row of the tile this thread decodes.  A warp may only touch the tensor-memory
    // lanes 32 * (warp % 4) + lane, and with the weights in tensor memory row = lane.
    const int row = ((warp & 3) << 5) | lane;
    RingState ps, wb;
    int sequence = 0;  // K steps seen so far by this CTA, over all units
    int turn = 0;      // the decode group whose K step `sequence` is
    bool ok = true;
    int local = 0;
    const uint8_t* lut_lane = smem + L::kLutOffset + lane * 4;  // this lane's copy of the table
    for (int index = first_unit; index < units && ok; index += unit_stride, ++local) {
      const uint8_t* unit_scales = nullptr;
      if constexpr (kBulk) {
        if (!wait(&full_scale[scale_slot(local)], scale_phase(local), kSiteDecodeScale)) break;
        unit_scales = scale_buffer(scale_slot(local)) + row * p.scale_stride;
      }
      for (int rs = 0; rs < stages && ok; ++rs) {
        if (!wait(&full_p[ps.index], ps.phase, kSiteDecodeRaw)) {
          ok = false;
          break;
        }
        const int sub_steps = min(KS, k_count - rs * KS);
        for (int j = 0; j < sub_steps;
             ++j, ++sequence, turn = turn + 1 == DG ? 0 : turn + 1, wb.advance<WB>()) {
          if (turn != group) continue;  // turn == sequence % DG
          if constexpr (!WT) {
            // the decoded tile is written as it is computed: the slot must be free first
            if (!wait(&empty_w[wb.index], wb.phase ^ 1u, kSiteDecodeWeights)) {
              ok = false;
              break;
            }
          }
          uint4 codes[2];
          if constexpr (KS == 1) {
            // rows of 32 bytes, 32-byte swizzled by the TMA load (16-byte halves of rows 4..7
            // of every 8 swapped), which spreads a quarter-warp's 16-byte reads over all banks
            const uint8_t* source = payload_tile(ps.index) + row * 32;
            const int swap = (row >> 2) & 1;
            codes[0] = *reinterpret_cast<const uint4*>(source + (swap * 16));
            codes[1] = *reinterpret_cast<const uint4*>(source + ((swap ^ 1) * 16));
          } else {
            // rows of 32*KS bytes, 128-byte swizzled by the TMA load
            const uint8_t* source = payload_tile(ps.index) + row * (32 * KS);
            codes[0] = *reinterpret_cast<const uint4*>(source + (((2 * j) ^ (row & 7)) * 16));
            codes[1] = *reinterpret_cast<const uint4*>(source + (((2 * j + 1) ^ (row & 7)) * 16));
          }
          const uint32_t four_scales =
              kBulk ? *reinterpret_cast<const uint32_t*>(unit_scales + (k_begin + rs * KS + j) * 4)
                 : *reinterpret_cast<const uint32_t*>(scale_tile(ps.index) + row * (4 * KS) +
                                                      j * 4);
          uint32_t scale[4];
          if constexpr (AFMT == kAf16) {
            scales2_f16(four_scales & 0xffffu, scale[0], scale[1]);
            scales2_f16(four_scales >> 16, scale[2], scale[3]);
          } else if constexpr (kLut) {
            scales4_bf16_true(four_scales, scale);
          } else {
            scales4_bf16(four_scales, scale);
          }
          // Scale bytes the format does not define (sign bit set, 0x7f) poison their block
          // with NaN like the reference device kernels (turing_adapter.cu:35-40); 0x7fff is a
          // NaN in f16 and in bf16, and NaN times any code, zero included, stays NaN.
          const uint32_t invalid =
              (four_scales | ((four_scales & 0x7f7f7f7fu) + 0x01010101u)) & 0x80808080u;
          if (invalid != 0u) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (invalid & (0x80u << (8 * i))) scale[i] = 0x7fff7fffu;
            }
          }
          const uint32_t words[8] = {codes[0].x, codes[0].y, codes[0].z, codes[0].w,
                                     codes[1].x, codes[1].y, codes[1].z, codes[1].w};
          if constexpr (WT) {
            // The row is decoded into registers before the warp waits for a free W' tile.
            uint32_t o[4][8];
#pragma unroll
            for (int pair = 0; pair < 4; ++pair) {
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                uint32_t q4[4];
                if constexpr (AFMT == kAf16) {
                  decode8_f16(words[2 * pair + half], scale[pair], q4);
                } else if constexpr (kLut) {
                  decode8_bf16_lut(words[2 * pair + half], scale[pair], q4, lut_lane);
                } else {
                  decode8_bf16(words[2 * pair + half], scale[pair], q4);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) o[pair][4 * half + i] = q4[i];
              }
            }
            if (!wait(&empty_w[wb.index], wb.phase ^ 1u, kSiteDecodeWeights)) {
              ok = false;
              break;
            }
            // 32-bit column c of this thread's lane holds elements 2c and 2c + 1 of the row
            const uint32_t w_address = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) +
                                       kAccColumns + wb.index * kWColumns;
            __syncwarp();
#pragma unroll
            for (int pair = 0; pair < 4; ++pair) tmem_store_32x8(w_address + pair * 8, o[pair]);
            // Announcing the tile one own K step later, so that the stores overlap the next
            // row's arithmetic, was measured 1-3 % slower; so was freeing tiles in groups of
            // KS with one commit per group.
            tmem_store_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_w[wb.index]);
            continue;
          } else {
            uint8_t* w_row = w_tile(wb.index) + row * 128;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              uint32_t o[4];
              if constexpr (AFMT == kAf16) {
                decode8_f16(words[jj], scale[jj >> 1], o);
              } else if constexpr (kLut) {
                decode8_bf16_lut(words[jj], scale[jj >> 1], o, lut_lane);
              } else {
                decode8_bf16(words[jj], scale[jj >> 1], o);
              }
              const int chunk = jj ^ (row & 7);
              *reinterpret_cast<uint4*>(w_row + chunk * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            fence_proxy_async_smem();
          }
          // one arrival per warp: 128 arrivals on one barrier word serialise
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_w[wb.index]);
        }
        // this warp has read its last byte of the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_p[ps.index]);
        ps.advance<PS>();
      }
      if constexpr (kBulk) {
        // this warp has read its last scale of the unit: the buffer may be refilled
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_scale[scale_slot(local)]);
      }
    }
  } else {
    // -------------------------------------------------------------------- gather
    if constexpr (!XTMA) {
      // Thread t copies 16-byte chunk (t & 7) of rows (t >> 3) + 16 i.  All its rows share
      // (row & 7), so the swizzled chunk position is a per-thread constant, and the source
      // byte offsets of its rows live in registers for the whole unit.
      constexpr int kRowsPerThread = BM / 16;
      const int t = threadIdx.x - kGatherWarp0 * 32;  // 0..127
      const int chunk = t & 7;
      const int row0 = t >> 3;
      const int position = (chunk ^ (row0 & 7)) * 16;
      const uint8_t* input = static_cast<const uint8_t*>(p.input);
      constexpr int kLag = XS > 2 ? 2 : XS - 1;  // stages whose copies may still be landing
      RingState xs, arrive;
      int in_flight = 0;
      bool ok = true;
      auto retire = [&](int keep) {
        while (in_flight > keep) {
          if (in_flight - 1 >= 2) {
            asm volatile("cp.async.wait_group 2;" ::: "memory");
          } else if (in_flight - 1 == 1) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");
          } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_x[arrive.index]);
          arrive.advance<XS>();
          --in_flight;
        }
      };
      for (int index = first_unit; index < units && ok; index += unit_stride) {
        const Unit u = get_unit<BM, GROUPED>(p, groups, index);
        int64_t source_offset[kRowsPerThread];  // byte offset of the source row, -1 = zero row
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) {
          const int r = row0 + 16 * i;
          int64_t offset = -1;
          if (r < u.rows) {
            const int a = p.sorted_assignments[u.m0 + r];
            if (a >= 0 && a < p.assignments) {
              offset = static_cast<int64_t>(MODE == kGateUp ? a / p.top_k : a) * p.K * 2;
            }
          }
          source_offset[i] = offset;
        }
        for (int rs = 0; rs < stages; ++rs) {
          if (!wait(&x_free[xs.index], xs.phase ^ 1u, kSiteGather)) {
            ok = false;
            break;
          }
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            const int k_step = rs * KS + j;
            if (k_step < p.k_steps) {
              const uint8_t* column = input + (static_cast<int64_t>(k_step) * kTileK + chunk * 8) * 2;
              uint8_t* tile = x_tile(xs.index, j) + position + row0 * 128;
#pragma unroll
              for (int i = 0; i < kRowsPerThread; ++i) {
                const bool valid = source_offset[i] >= 0;
                cp_async_16_zfill(tile + i * (16 * 128),
                                  column + (valid ? source_offset[i] : 0), valid);
              }
            }
          }
          asm volatile("cp.async.commit_group;" ::: "memory");
          ++in_flight;
          xs.advance<XS>();
          retire(kLag);
        }
      }
      retire(0);
    }
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
  // No CTA of a cluster leaves while another may still write into its shared memory.
  if (split) cluster_sync_all();
}

}  // namespace umma
}  // namespace nml_sm100

// ---- host helpers -------------------------------------------------------------------------


namespace nml_sm100 {
namespace umma {

// Bytes between the scale rows of a unit's shared-memory scale buffer.  Thread r of a decode
// warp reads the 4-byte word (row r, K step s), so a row pitch of an even number of words maps
// several lanes to one bank (all 32 at K = 4096, 256-byte rows).  Such rows are copied one by
// one and padded apart to a pitch of 4 (mod 8) words: eight distinct banks, the best a 16-byte
// aligned bulk-copy destination allows.  Odd word pitches (K = 2880: 45 words) stay contiguous.
inline int bulk_scale_stride(int scale_width) {
  if (scale_width % 16 != 0) return scale_width;
  int stride = scale_width + 16;
  while ((stride / 4) % 8 != 4) stride += 16;
  return stride;
}

inline int bulk_scale_buffer_bytes(int scale_width) {
  return (bulk_scale_stride(scale_width) * kTileN + 127) / 128 * 128;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, resolved through the runtime so the library has no link-time
// dependency on the driver.
inline EncodeTiledFn encode_tiled() {
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

// Payload tensor [rows, K/2] bytes; one box is 128 rows x 32*KS bytes (128B-swizzled when a
// row of the box is 128 bytes).
template <int KS>
inline bool encode_payload_map(CUtensorMap* map, const uint8_t* payload, int64_t rows, int K) {
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K / 2), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K / 2)};
  const cuuint32_t box[2] = {32 * KS, kTileN};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(payload), dims,
                strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                KS == 4   ? CU_TENSOR_MAP_SWIZZLE_128B
                : KS == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                          : CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Activation tensor [M, K] of 16-bit elements; one box is BM rows x 64 columns, 128B swizzle.
template <typename T>
inline bool encode_activation_map(CUtensorMap* map, const void* x, int64_t rows, int K, int BM,
                                  int KS = 1) {
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) return false;
  if (KS > 1) {
    // 3-D view [K/64][rows][64] of the same row-major tensor: one box is KS consecutive
    // 64-column slabs of BM rows, each slab a 128B-swizzled UMMA operand tile.
    const cuuint64_t dims3[3] = {kTileK, static_cast<cuuint64_t>(rows),
                                 static_cast<cuuint64_t>(K / kTileK)};
    const cuuint64_t strides3[2] = {static_cast<cuuint64_t>(K) * 2, kTileK * 2};
    const cuuint32_t box3[3] = {kTileK, static_cast<cuuint32_t>(BM), static_cast<cuuint32_t>(KS)};
    const cuuint32_t elem3[3] = {1, 1, 1};
    const CUtensorMapDataType type3 = std::is_same<T, __half>::value
                                          ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                          : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    return encode(map, type3, 3, const_cast<void*>(x), dims3, strides3, box3, elem3,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {kTileK, static_cast<cuuint32_t>(BM)};
  const cuuint32_t elem[2] = {1, 1};
  const CUtensorMapDataType type = std::is_same<T, __half>::value
                                       ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                       : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return encode(map, type, 2, const_cast<void*>(x), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Opts a kernel into its dynamic shared memory once per device.  `configured` is the
// caller's per-kernel table (one static array per kernel instantiation); concurrent first
// calls may both set the attribute, which is harmless, and later calls see the flag.
template <typename Kernel>
inline bool reserve_smem(Kernel kernel, int bytes, int device,
                         std::atomic<int> (&configured)[64]) {
  if (device >= 0 && device < 64 && configured[device].load(std::memory_order_acquire)) {
    return true;
  }
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) !=
      cudaSuccess) {
    return false;
  }
  if (device >= 0 && device < 64) configured[device].store(1, std::memory_order_release);
  return true;
}

}  // namespace umma
}  // namespace nml_sm100
