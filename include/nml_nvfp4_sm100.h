/*
 * C ABI of the sm_100a (B200) NVFP4 packed-weight kernels.
 *
 * This is the boundary a host runtime binds.  It is a drop-in for the
 * reference's SM75 adapter ABI (crates/nml-kernel-nvfp4/include/nml_nvfp4.h):
 * the four request structs below begin with exactly the reference's fields in
 * the reference's order, so the `#[repr(C)]` mirrors in
 * crates/nml-kernel-nvfp4/src/cuda.rs:39-117 can be passed unchanged.  Fields
 * added here sit after the reference's last field and are read only when
 * `struct_size` says they are present.
 *
 * Conventions (same as the reference, nml_nvfp4.h:16-17,
 * turing_adapter.cu:13-22): every pointer is a borrowed device address; the
 * library only enqueues work on `stream`, never synchronises, and never
 * allocates or retains memory.  Every entry point returns 0 on success,
 * 1 for an invalid argument, 2 for a launch failure, and writes a
 * NUL-terminated message into `error_message` (when capacity > 0) on failure.
 * All extents must be positive and fit in int32.
 *
 * Weight representation (NVFP4 recipe v2, crates/nml-parameter/src/lib.rs:393-597):
 *   payload      u8 [rows, ceil(K/2)]  two E2M1 codes per byte, even column in the low nibble
 *   block_scales u8 [rows, ceil(K/16)] unsigned E4M3FN, one per 16 consecutive K
 *   global_scale f32 scalar in device memory
 *   value(r, k) = e2m1(code) * (e4m3(scale) * global)
 */
#ifndef NML_NVFP4_SM100_H_
#define NML_NVFP4_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same codes as NmlNvFp4DType (nml_nvfp4.h:11-14). */
typedef enum NmlSm100DType {
  NML_SM100_F16 = 1,
  NML_SM100_BF16 = 2,
} NmlSm100DType;

#define NML_SM100_OK 0
#define NML_SM100_INVALID_ARGUMENT 1
#define NML_SM100_LAUNCH_FAILURE 2

/* Y[rows, outputs] = X[rows, inputs] * W[outputs, inputs]^T (+ bias), f32 accumulate.
 * Field-for-field NmlNvFp4Linear (nml_nvfp4.h:18-31), plus one optional trailing field that is
 * read only when struct_size covers it: `residual` [rows, outputs] is added to the narrowed
 * result, Y = narrow(narrow(X W^T + bias) + residual), which is what the reference graph
 * computes with a separate add after the attention output projection
 * (products/serve/src/gpt_oss/graph.rs:534-543); `residual` may alias `output`. */
typedef struct NmlSm100Linear {
  size_t struct_size;
  const void *activation;      /* [rows, inputs] dtype */
  const uint8_t *payload;      /* [outputs, ceil(inputs/2)] */
  const uint8_t *block_scales; /* [outputs, ceil(inputs/16)] */
  const float *global_scale;   /* device scalar */
  const void *bias;            /* [outputs] dtype, may be NULL */
  void *output;                /* [rows, outputs] dtype */
  void *stream;                /* cudaStream_t, must not be NULL */
  int64_t rows;
  int64_t outputs;
  int64_t inputs;
  int32_t dtype; /* NmlSm100DType */
  const void *residual; /* optional: [rows, outputs] dtype, or NULL */
  /* Optional scratch (read when struct_size covers both fields), 256-byte aligned: with at
   * least nml_nvfp4_sm100_linear_workspace_bytes(...) bytes, a BF16 call on a wide weight
   * first narrows the activations to F16, every tile of 256 rows times one power of two that
   * puts the tile's largest magnitude into [2^14, 2^15), so that the weights decode with the
   * hardware FP4/FP8 conversions; the inverse power multiplies the tile's f32 sums.  Elements
   * down to 2^-28 of the tile's largest stay exact, smaller ones round at 2^-39 of it.  The
   * device checks the input first: when a row's largest magnitude is more than 2^8 below its
   * tile's, or a tile holds an infinity, a NaN or nothing above 2^-111, the BF16-operand
   * kernel produces the output instead (it is launched behind the narrowed one; each of the
   * two returns at once when the other is meant) and the word at
   * nml_nvfp4_sm100_linear_workspace_verdict_offset(...) of the scratch reads nonzero.
   * Without scratch the call decodes to BF16, several per cent slower. */
  void *workspace;
  size_t workspace_bytes;
} NmlSm100Linear;

/* Scratch bytes nml_nvfp4_sm100_linear can use for this call; 0 when it would not use any. */
size_t nml_nvfp4_sm100_linear_workspace_bytes(int64_t rows, int64_t outputs, int64_t inputs,
                                              int32_t dtype);
/* Byte offset, in that scratch, of the uint32 the call leaves at 0 when the F16-operand kernel
 * produced the output and at 1 when the BF16-operand kernel did. */
size_t nml_nvfp4_sm100_linear_workspace_verdict_offset(int64_t rows, int64_t outputs,
                                                       int64_t inputs, int32_t dtype);

/* Three linears that share one activation (the Q, K and V projections), in one launch:
 * output[i][rows, outputs[i]] = X * W_i^T (+ bias[i]).  The reference fuses them only for
 * rows <= 8 on its Triton path (crates/nml-ir/src/nvfp4_backend.rs:221-380, config
 * NvFp4QkvConfig) and lowers three custom calls otherwise; here one launch serves every row
 * count the tcgen05 kernel takes (inputs a multiple of 64), else the call is answered by three
 * linear launches.  Same dtype and inputs for all three; each weight has its own global scale
 * and optional bias.  Results equal those of three nml_nvfp4_sm100_linear calls bit for bit
 * when both select the same kernel variant and K split (always for at most 16 rows), and to
 * GEMM tolerance otherwise: the tile height and the split follow the launch's total tile
 * count, so the f32 summation order can differ. */
typedef struct NmlSm100LinearQkv {
  size_t struct_size;
  const void *activation;         /* [rows, inputs] dtype */
  const uint8_t *payload[3];      /* [outputs[i], ceil(inputs/2)] */
  const uint8_t *block_scales[3]; /* [outputs[i], ceil(inputs/16)] */
  const float *global_scale[3];   /* device scalars */
  const void *bias[3];            /* [outputs[i]] dtype, each may be NULL */
  void *output[3];                /* [rows, outputs[i]] dtype */
  void *stream;
  int64_t rows;
  int64_t outputs[3];
  int64_t inputs;
  int32_t dtype;
} NmlSm100LinearQkv;

/* out[r, :] = decode(W[indices[r], :]); an index outside [0, vocabulary) yields a row of
 * zeros and raises the device status bit NML_SM100_STATUS_INDEX_RANGE.
 * Field-for-field NmlNvFp4Embedding (nml_nvfp4.h:33-46). */
typedef struct NmlSm100Embedding {
  size_t struct_size;
  const void *indices; /* [rows] i32 or i64 */
  const uint8_t *payload;
  const uint8_t *block_scales;
  const float *global_scale;
  void *output; /* [rows, width] dtype */
  void *stream;
  int64_t rows;
  int64_t vocabulary;
  int64_t width;
  int32_t dtype;
  uint8_t indices_are_i64;
} NmlSm100Embedding;

/* activated[a, i] = swiglu(hidden[a / k, :] . W[e, 2i, :] + b[e, 2i],
 *                          hidden[a / k, :] . W[e, 2i+1, :] + b[e, 2i+1])
 * for every assignment a listed in the schedule; e = block_experts[slot / 16].
 * The first 20 fields are NmlNvFp4ExpertGateUp (nml_nvfp4.h:48-69).  The two
 * trailing pointers are the operands the reference's Triton grouped ABI also
 * carries (crates/nml-ir/src/nvfp4_backend.rs:633-651); both may be NULL or
 * absent (struct_size of the reference struct):
 *   active_blocks  device i32 scalar: blocks at or past it are skipped
 *   expert_offset  device i32 scalar: payload/scales/bias hold experts
 *                  [offset, offset + experts); other blocks are skipped. */
typedef struct NmlSm100ExpertGateUp {
  size_t struct_size;
  const void *hidden;                /* [tokens, hidden_size] dtype */
  const int32_t *sorted_assignments; /* [schedule_positions], sentinel >= assignments */
  const int32_t *block_experts;      /* [schedule_blocks], -1 = padding block */
  const uint8_t *payload;            /* [experts, 2*intermediate, ceil(hidden/2)] */
  const uint8_t *block_scales;       /* [experts, 2*intermediate, ceil(hidden/16)] */
  const float *global_scale;
  const void *bias;  /* [experts, 2*intermediate] dtype */
  void *activated;   /* [assignments, intermediate] dtype */
  void *stream;
  int64_t tokens;
  int64_t assignments;
  int64_t schedule_positions;
  int64_t schedule_blocks;
  int64_t hidden_size;
  int64_t intermediate_size;
  int64_t experts;
  int64_t experts_per_token;
  int32_t block_size; /* must be 16 */
  int32_t dtype;
  const int32_t *active_blocks;
  const int32_t *expert_offset;
} NmlSm100ExpertGateUp;

/* weighted[a, h] = (activated[a, :] . W[e, h, :] + b[e, h]) * routing_weights[a].
 * The first 20 fields are NmlNvFp4ExpertDown (nml_nvfp4.h:71-92). */
typedef struct NmlSm100ExpertDown {
  size_t struct_size;
  const void *activated; /* [assignments, intermediate] dtype */
  const int32_t *sorted_assignments;
  const int32_t *block_experts;
  const uint8_t *payload;      /* [experts, hidden, ceil(intermediate/2)] */
  const uint8_t *block_scales; /* [experts, hidden, ceil(intermediate/16)] */
  const float *global_scale;
  const void *bias;            /* [experts, hidden] dtype */
  const void *routing_weights; /* [assignments] dtype */
  void *weighted_output;       /* [assignments, hidden] dtype */
  void *stream;
  int64_t assignments;
  int64_t schedule_positions;
  int64_t schedule_blocks;
  int64_t intermediate_size;
  int64_t hidden_size;
  int64_t experts;
  int64_t experts_per_token;
  int32_t block_size;
  int32_t dtype;
  const int32_t *active_blocks;
  const int32_t *expert_offset;
  /* Optional (read when struct_size covers it): [assignments] device pointers; when set, the
   * result row of assignment a is stored at row_targets[a] (hidden_size values) instead of
   * weighted + a * hidden_size.  An expert-parallel owner points them into the senders'
   * return buffers (nml_nvfp4_sm100_ep_receive_meta fills the table), so the projection's
   * epilogue is also the return trip.  NULL entries are skipped. */
  void *const *row_targets;
} NmlSm100ExpertDown;

/* Top-k routing from f32 router logits: softmax over all experts, top-k by
 * descending probability with ties to the lower expert index, renormalise by
 * max(sum, FLT_EPSILON), masked tokens get expert -1 / weight 0, weights
 * narrowed to dtype.  Replaces the StableHLO subgraph authored by
 * routed_clamped_swiglu_impl (crates/nml-ir/src/lib.rs:1411-1437, softmax
 * :4109-4137, top_k :3581-3605). */
typedef struct NmlSm100Route {
  size_t struct_size;
  const float *logits;          /* [tokens, experts] */
  const uint8_t *active_tokens; /* [tokens] bool, may be NULL (all active) */
  int32_t *expert_ids;          /* [tokens, experts_per_token] */
  void *routing_weights;        /* [tokens, experts_per_token] dtype */
  void *stream;
  int64_t tokens;
  int64_t experts;           /* at most 256 */
  int64_t experts_per_token; /* at most 16 */
  int32_t dtype;
} NmlSm100Route;

/* The assignment schedule of moe_assignment_plan (crates/nml-ir/src/lib.rs:5644-5779),
 * block size 16, same capacity rule:
 *   schedule_blocks = ceil((A + min(A, E) * 15) / 16), positions = 16 * blocks.
 * Expert-parallel use: ids are global, this device holds experts
 * [expert_offset, expert_offset + experts); other ids are left out of the schedule like
 * masked routes, and block_experts holds local indices (id - expert_offset). */
typedef struct NmlSm100AssignmentPlan {
  size_t struct_size;
  const int32_t *expert_ids;   /* [assignments], -1 = masked */
  int32_t *sorted_assignments; /* [schedule_positions] */
  int32_t *block_experts;      /* [schedule_blocks] */
  int32_t *active_blocks;      /* device scalar */
  void *stream;
  int64_t assignments;
  int64_t experts;             /* at most 1024 */
  int64_t schedule_positions;
  int64_t schedule_blocks;
  int32_t block_size;          /* must be 16 */
  int32_t expert_offset;
} NmlSm100AssignmentPlan;

/* out[t, h] = sum over routes r (in route order) of weighted[t * k + r, h], f32
 * accumulation, one narrowing.  When expert_ids is given, routes whose id is negative or
 * outside [expert_offset, expert_offset + experts) are skipped (their rows were never
 * written).
 * Replaces the reshape + stablehlo.reduce of lower_routed_swiglu
 * (crates/nml-ir/src/nvfp4_backend.rs:486-508). */
typedef struct NmlSm100Combine {
  size_t struct_size;
  const void *weighted;      /* [tokens * k, hidden] dtype */
  const int32_t *expert_ids; /* [tokens * k] or NULL (every route contributes) */
  void *output;              /* [tokens, hidden] dtype */
  void *stream;
  int64_t tokens;
  int64_t experts_per_token;
  int64_t hidden_size;
  int64_t experts;           /* used with expert_ids */
  int32_t expert_offset;     /* used with expert_ids */
  int32_t dtype;
} NmlSm100Combine;

/* The whole routed clamped-SwiGLU layer, the unit the reference's CPU target
 * "nml.nvfp4.routed_swiglu" computes in one call
 * (crates/nml-kernel-nvfp4/src/ffi.rs:228-428, lib.rs:333-448): plan, gate/up
 * with the SwiGLU epilogue, down with bias and routing weight, k-way sum.
 * `workspace` is caller-provided scratch of at least
 * nml_nvfp4_sm100_routed_swiglu_workspace_bytes(...) bytes, 256-byte aligned. */
typedef struct NmlSm100RoutedSwiglu {
  size_t struct_size;
  const void *hidden;           /* [tokens, hidden_size] dtype */
  const int32_t *expert_ids;    /* [tokens, k], -1 = masked */
  const void *routing_weights;  /* [tokens, k] dtype */
  const uint8_t *gate_payload;  /* [experts, 2I, ceil(H/2)] */
  const uint8_t *gate_scales;
  const float *gate_global;
  const void *gate_bias;        /* [experts, 2I] dtype */
  const uint8_t *down_payload;  /* [experts, H, ceil(I/2)] */
  const uint8_t *down_scales;
  const float *down_global;
  const void *down_bias;        /* [experts, H] dtype */
  void *output;                 /* [tokens, hidden_size] dtype */
  void *workspace;
  size_t workspace_bytes;
  void *stream;
  int64_t tokens;
  int64_t hidden_size;
  int64_t intermediate_size;
  int64_t experts;              /* experts held by payload/scales/bias */
  int64_t experts_per_token;
  int32_t expert_offset;        /* first expert id held locally (expert parallel), else 0 */
  int32_t dtype;
  /* Optional (read when struct_size covers it): how many of the tokens * k routes the caller
   * expects to be live (not masked, expert held locally); 0 = all.  A hint for kernel
   * selection only: an expert-parallel owner passes rows of which most are masked. */
  int64_t live_routes_hint;
  /* Optional: NML_SM100_ROUTED_LEAVE_MASKED_ROWS with experts_per_token == 1 lets the down
   * projection write each token's one result row straight into `output` (no k-way sum pass);
   * rows of masked tokens are then left untouched instead of being zeroed.  For callers that
   * never read those rows (an expert-parallel owner returning rows to their senders). */
  int32_t flags;
  /* Optional, with NML_SM100_ROUTED_LEAVE_MASKED_ROWS and experts_per_token == 1:
   * [tokens] device pointers, the destination of every token's result row (see
   * NmlSm100ExpertDown::row_targets); `output` is then not written. */
  void *const *row_targets;
} NmlSm100RoutedSwiglu;
#define NML_SM100_ROUTED_LEAVE_MASKED_ROWS 1

/* Expert-parallel dispatch plan.  The reference shards experts by replicating all tokens on
 * every device and all-reducing partial outputs (crates/nml-ir/src/lib.rs:9596-9728); these
 * three entry points support the token exchange that replaces it: assignments are grouped by
 * the rank that owns their expert (rank = id / experts_per_rank, the contiguous placement of
 * crates/nml-sharding/src/lib.rs:180-213), in rank order and assignment order inside a rank.
 *   send_order[slot]          assignment index carried by send slot `slot` (-1 past the total)
 *   local_expert[slot]        expert index on the destination rank
 *   slot_of_assignment[a]     send slot of assignment a, -1 for masked routes
 *   send_counts[rank]         rows sent to each rank */
typedef struct NmlSm100EpDispatchPlan {
  size_t struct_size;
  const int32_t *expert_ids;   /* [assignments] global ids, -1 = masked */
  int32_t *send_order;         /* [assignments] */
  int32_t *local_expert;       /* [assignments] */
  int32_t *slot_of_assignment; /* [assignments] */
  int32_t *send_counts;        /* [ranks] */
  void *stream;
  int64_t assignments;
  int64_t ranks;               /* at most 64 */
  int64_t experts_per_rank;
} NmlSm100EpDispatchPlan;

/* Token permute: output[r, :] = source[row_index[r] / index_divisor, :]; a negative index gives
 * a zero row.  width must be a multiple of 8 and both buffers 16-byte aligned. */
typedef struct NmlSm100GatherRows {
  size_t struct_size;
  const void *source;        /* [source_rows, width] dtype */
  const int32_t *row_index;  /* [rows] */
  void *output;              /* [rows, width] dtype */
  void *stream;
  int64_t rows;
  int64_t source_rows;
  int64_t width;
  int32_t index_divisor;     /* experts_per_token when indices are assignment ids, else 1 */
  int32_t dtype;
} NmlSm100GatherRows;

/* Token unpermute + k-way sum: output[t, :] = sum over routes r (route order, f32, one
 * narrowing) of rows[row_index[t * k + r], :]; negative indices are skipped. */
typedef struct NmlSm100CombineRows {
  size_t struct_size;
  const void *rows;          /* [row_count, hidden] dtype */
  const int32_t *row_index;  /* [tokens * k] */
  void *output;              /* [tokens, hidden] dtype */
  void *stream;
  int64_t tokens;
  int64_t experts_per_token;
  int64_t hidden_size;
  int64_t row_count;
  int32_t dtype;
} NmlSm100CombineRows;

/* Replaces nml_nvfp4_turing_linear (nml_nvfp4.h:94-96, turing_adapter.cu:669-733). */
int32_t nml_nvfp4_sm100_linear(const NmlSm100Linear *request, char *error_message,
                               size_t error_message_capacity);

/* Replaces the three linears of lower_qkv and its fused small-batch kernel
 * (crates/nml-ir/src/nvfp4_backend.rs:221-380). */
int32_t nml_nvfp4_sm100_linear_qkv(const NmlSm100LinearQkv *request, char *error_message,
                                   size_t error_message_capacity);

/* Replaces nml_nvfp4_turing_embedding (nml_nvfp4.h:98-100, turing_adapter.cu:735-783). */
int32_t nml_nvfp4_sm100_embedding(const NmlSm100Embedding *request, char *error_message,
                                  size_t error_message_capacity);

/* Replaces nml_nvfp4_turing_expert_gate_up (nml_nvfp4.h:102-104, turing_adapter.cu:785-864)
 * and the Triton grouped gate/up kernels (crates/nml-kernel-triton/src/nvfp4.rs:1007-1227). */
int32_t nml_nvfp4_sm100_expert_gate_up(const NmlSm100ExpertGateUp *request, char *error_message,
                                       size_t error_message_capacity);

/* Replaces nml_nvfp4_turing_expert_down (nml_nvfp4.h:106-108, turing_adapter.cu:866-942)
 * and the Triton grouped down kernels (crates/nml-kernel-triton/src/nvfp4.rs:1229-1420). */
int32_t nml_nvfp4_sm100_expert_down(const NmlSm100ExpertDown *request, char *error_message,
                                    size_t error_message_capacity);

/* Replaces the routing subgraph (crates/nml-ir/src/lib.rs:1411-1437). */
int32_t nml_nvfp4_sm100_route(const NmlSm100Route *request, char *error_message,
                              size_t error_message_capacity);

/* Replaces moe_assignment_plan (crates/nml-ir/src/lib.rs:5644-5779). */
int32_t nml_nvfp4_sm100_assignment_plan(const NmlSm100AssignmentPlan *request,
                                        char *error_message, size_t error_message_capacity);

/* Replaces the k-way reduce of lower_routed_swiglu (crates/nml-ir/src/nvfp4_backend.rs:486-508). */
int32_t nml_nvfp4_sm100_combine(const NmlSm100Combine *request, char *error_message,
                                size_t error_message_capacity);

/* Replaces the CPU target "nml.nvfp4.routed_swiglu" (crates/nml-kernel-nvfp4/src/ffi.rs:228-428). */
int32_t nml_nvfp4_sm100_routed_swiglu(const NmlSm100RoutedSwiglu *request, char *error_message,
                                      size_t error_message_capacity);

/* Expert-parallel token exchange support; together they replace lower_expert_parallel's
 * replicate-and-all-reduce scheme (crates/nml-ir/src/lib.rs:9596-9728). */
/* Token exchange by direct stores into peer memory (NVLink), for ranks that have mapped each
 * other's buffers into their own address space (symmetric memory).  No counterpart in the
 * reference.  Cross-rank ordering is done on the device with flags in peer memory; there is
 * no host synchronisation and no collective between the stages.  Stage order per layer, all
 * on the caller's stream: ep_dispatch_plan; ep_push_rows (stores rows and meta into the
 * owners' buffers, then raises this rank's arrival flag on every rank); ep_receive_meta
 * (waits for every rank's arrival flag, then writes the expert ids and routing weights of the
 * received rows); the routed layer over the receive buffer (k = 1); ep_return_rows (stores
 * result rows into the senders' return buffers, then raises the return flag);
 * ep_wait_returns; combine_rows over the return buffer.  Optional fusions: with the
 * row_targets that ep_receive_meta fills, the routed layer's down projection stores its rows
 * into the senders' return buffers itself (its writers fence at system scope) and
 * ep_return_rows without `computed` only raises the flag; ep_wait_returns with its combine
 * fields does the k-way sum in the same launch.
 *
 * Every rank's receive buffer holds one region of `region_rows` rows per sender; sender r
 * writes its rows for a destination into region r in its send order, so placement needs no
 * counts from other ranks and cannot overflow when region_rows >= the sender's assignments.
 * Waits are bounded (`wait_limit` polls of about a quarter microsecond, 0 = one second); a
 * wait that runs out sets NML_SM100_STATUS_BARRIER_TIMEOUT | NML_SM100_STATUS_PEER_TIMEOUT,
 * the missing sender counts as having sent nothing, and the kernel returns.  All ranks must
 * run the same sequence of exchanges on the same buffers; buffers start zeroed. */
#define NML_SM100_EP_MAX_RANKS 16
#define NML_SM100_EP_SYNC_WORDS (3 * NML_SM100_EP_MAX_RANKS) /* i32 words per rank */
#define NML_SM100_EP_STATE_WORDS 4                           /* i32 words, local */
typedef struct NmlSm100EpExchange {
  void *peer_rows[NML_SM100_EP_MAX_RANKS];    /* receive rows [ranks * region_rows, width] */
  int32_t *peer_meta[NML_SM100_EP_MAX_RANKS]; /* receive meta [ranks * region_rows, 4] i32 */
  void *peer_back[NML_SM100_EP_MAX_RANKS];    /* return rows [region_rows, width] */
  int32_t *peer_sync[NML_SM100_EP_MAX_RANKS]; /* sync words [NML_SM100_EP_SYNC_WORDS] */
  int32_t *local_state; /* [NML_SM100_EP_STATE_WORDS], this rank's own memory, starts zeroed */
  int64_t ranks;
  int64_t rank;
  int64_t region_rows;
  int64_t width;        /* multiple of 8 */
} NmlSm100EpExchange;

typedef struct NmlSm100EpPushRows {
  size_t struct_size;
  const void *source;              /* [source_rows, width] dtype: this rank's tokens */
  const int32_t *send_order;       /* [assignments] from ep_dispatch_plan (-1 in the tail) */
  const int32_t *local_expert;     /* [assignments] from ep_dispatch_plan */
  const void *routing_weights;     /* [assignments] dtype */
  const int32_t *send_counts;      /* [ranks] from ep_dispatch_plan */
  NmlSm100EpExchange exchange;
  void *stream;
  int64_t assignments;             /* <= exchange.region_rows */
  int64_t source_rows;
  int64_t experts_per_token;
  int32_t dtype;
} NmlSm100EpPushRows;

typedef struct NmlSm100EpReceiveMeta {
  size_t struct_size;
  NmlSm100EpExchange exchange;
  int32_t *expert_ids;             /* [ranks * region_rows] local expert, -1 where no row arrived */
  void *routing_weights;           /* [ranks * region_rows] dtype */
  int32_t *received;               /* device scalar: rows received */
  void *stream;
  int64_t wait_limit;
  int32_t dtype;
  /* Optional (read when struct_size covers it): [ranks * region_rows] device pointers, set to
   * where row i's result goes in its sender's return buffer (NULL where no row arrived). */
  void **row_targets;
} NmlSm100EpReceiveMeta;

typedef struct NmlSm100EpReturnRows {
  size_t struct_size;
  const void *computed;            /* [ranks * region_rows, width] dtype: results in receive order;
                                      NULL when the projection stored them through row_targets:
                                      the call then only publishes the return flags */
  NmlSm100EpExchange exchange;
  void *stream;
  int32_t dtype;
} NmlSm100EpReturnRows;

typedef struct NmlSm100EpWaitReturns {
  size_t struct_size;
  NmlSm100EpExchange exchange;
  void *stream;
  int64_t wait_limit;
  /* Optional (read when struct_size covers them; output != NULL): do the combine over this
   * rank's return buffer in the same launch, every block after its own wait:
   * output[t, :] = sum over routes of back[row_index[t * experts_per_token + route], :]. */
  const int32_t *row_index;        /* [tokens * experts_per_token], -1 = no row */
  void *output;                    /* [tokens, width] dtype */
  int64_t tokens;
  int64_t experts_per_token;
  int32_t dtype;
} NmlSm100EpWaitReturns;

int32_t nml_nvfp4_sm100_ep_push_rows(const NmlSm100EpPushRows *request, char *error_message,
                                     size_t error_message_capacity);
int32_t nml_nvfp4_sm100_ep_receive_meta(const NmlSm100EpReceiveMeta *request,
                                        char *error_message, size_t error_message_capacity);
int32_t nml_nvfp4_sm100_ep_return_rows(const NmlSm100EpReturnRows *request, char *error_message,
                                       size_t error_message_capacity);
int32_t nml_nvfp4_sm100_ep_wait_returns(const NmlSm100EpWaitReturns *request,
                                        char *error_message, size_t error_message_capacity);
int32_t nml_nvfp4_sm100_ep_dispatch_plan(const NmlSm100EpDispatchPlan *request,
                                         char *error_message, size_t error_message_capacity);
int32_t nml_nvfp4_sm100_gather_rows(const NmlSm100GatherRows *request, char *error_message,
                                    size_t error_message_capacity);
int32_t nml_nvfp4_sm100_combine_rows(const NmlSm100CombineRows *request, char *error_message,
                                     size_t error_message_capacity);

/* Row-wise top-k of 16-bit logits, the per-shard half of a sampler's reduction over the
 * column-sharded vocabulary projection (the reference plans a global top-k merge for its
 * column-sharded head, PRODUCT.md:673-674; it has no kernel for it).  values[r, :] are the k
 * largest logits of row r in descending order, indices[r, :] their columns plus
 * `index_offset` (the shard's first vocabulary index); equal values go to the lower index.
 * k <= 16 and ceil(columns / 8192) * k <= 512. */
typedef struct NmlSm100TopkRows {
  size_t struct_size;
  const void *logits;      /* [rows, columns] dtype, rows `row_stride` elements apart */
  float *values;           /* [rows, k] f32 */
  int32_t *indices;        /* [rows, k] */
  void *workspace;         /* nml_nvfp4_sm100_topk_rows_workspace_bytes(rows, columns, k) */
  size_t workspace_bytes;
  void *stream;
  int64_t rows;
  int64_t columns;
  int64_t row_stride;
  int64_t k;
  int32_t index_offset;
  int32_t dtype;
} NmlSm100TopkRows;
int32_t nml_nvfp4_sm100_topk_rows(const NmlSm100TopkRows *request, char *error_message,
                                  size_t error_message_capacity);
size_t nml_nvfp4_sm100_topk_rows_workspace_bytes(int64_t rows, int64_t columns, int64_t k);

/* The other half: merges the candidates of `parts` shards (or ranks) into the k best of every
 * row, with the same order as nml_nvfp4_sm100_topk_rows (larger value first, equal values to
 * the lower index), so the result equals a top-k over the unsharded row.  Candidate j of part p
 * and row r is values[(p * rows + r) * pitch + j] / indices[(p * rows + r) * pitch + j] for
 * j < k (an all-gather of every rank's [rows, pitch] block gives exactly this layout);
 * indices < 0 mark empty candidates.  parts * k <= 512. */
typedef struct NmlSm100TopkMerge {
  size_t struct_size;
  const float *values;     /* [parts, rows, pitch] */
  const int32_t *indices;  /* [parts, rows, pitch] */
  float *out_values;       /* [rows, k] */
  int32_t *out_indices;    /* [rows, k] */
  void *stream;
  int64_t parts;
  int64_t rows;
  int64_t pitch;
  int64_t k;
} NmlSm100TopkMerge;
int32_t nml_nvfp4_sm100_topk_merge(const NmlSm100TopkMerge *request, char *error_message,
                                   size_t error_message_capacity);

/* Paged-attention decode: one query token per sequence over a paged K/V cache, grouped-query
 * heads, causal, optional sliding window and learned per-head sinks.  Not part of the
 * reference's NVFP4 kernel ABI: it is the operator next to it in the product graph
 * (Graph::paged_attention, crates/nml-ir/src/lib.rs:4717-4730, lowered on GPUs to the Triton
 * kernels of crates/nml-kernel-triton/src/unified_attention.rs:82,189,755), provided because it
 * moves the most bytes of a decode step after the expert weights.  Same argument meaning as
 * the graph operator for a query length of one; the query is the last visible token.
 * This kernel takes head_dim 64, page_size 16 and 8 query heads per kv head. */
typedef struct NmlSm100PagedAttentionDecode {
  size_t struct_size;
  const void *query;               /* [batch, query_heads, head_dim] dtype */
  const void *key_cache;           /* [physical_pages, page_size, kv_heads, head_dim] dtype */
  const void *value_cache;         /* same shape */
  const int32_t *page_table;       /* [batch, table_width] physical page of every logical page */
  const int32_t *sequence_lengths; /* [batch] visible tokens, the query token included */
  const float *sinks;              /* [query_heads] f32 or NULL */
  void *output;                    /* [batch, query_heads, head_dim] dtype */
  void *workspace;                 /* f32 scratch, ..._workspace_bytes(batch, query_heads, splits) */
  size_t workspace_bytes;
  void *stream;
  int64_t batch;
  int64_t query_heads;
  int64_t kv_heads;
  int64_t head_dim;
  int64_t page_size;
  int64_t physical_pages;
  int64_t table_width;
  int64_t sliding_window;          /* 0: none; else only the last `sliding_window` tokens */
  int64_t splits;                  /* CTAs per (sequence, kv head) along the sequence, 1..64 */
  float scale;                     /* softmax scale, usually head_dim^-0.5 */
  int32_t dtype;
} NmlSm100PagedAttentionDecode;
int32_t nml_sm100_paged_attention_decode(const NmlSm100PagedAttentionDecode *request,
                                         char *error_message, size_t error_message_capacity);
size_t nml_sm100_paged_attention_decode_workspace_bytes(int64_t batch, int64_t query_heads,
                                                        int64_t splits);

/* Routed clamped-SwiGLU layer for callers that cannot hand over scratch memory.
 *
 * This entry point has no counterpart in the reference.  Some hosts of this library have
 * no way to obtain device memory for the layer's intermediates at call time: a custom-call
 * handler that only receives the operand and result buffers the compiler planned, or a
 * runtime that forbids cudaMalloc once serving has started.  For them the intermediates
 * (schedule, activated rows, weighted rows) live in a fixed array inside the library's
 * device image instead of in `workspace`.
 *
 * Same request struct and same result as nml_nvfp4_sm100_routed_swiglu; `workspace` and
 * `workspace_bytes` are ignored.  Limits and rules:
 *   - the array is NML_SM100_STATIC_SCRATCH_BYTES (8 MiB) and every GPU that loads the
 *     library holds it until the process exits; a request whose
 *     nml_nvfp4_sm100_routed_swiglu_workspace_bytes(...) exceeds it is rejected with
 *     status 1 and a message naming both sizes (at GPT-OSS widths, hidden = intermediate =
 *     2880 and 4 routes per token, that is about 180 tokens);
 *   - the first call on a device looks up the array's device address (one runtime query,
 *     no allocation); make that first call before starting any stream capture;
 *   - nothing is allocated or freed, here or in anything it calls;
 *   - all calls on a device share the one array and it keeps whatever the previous call
 *     left.  That is harmless for a single call, because every word the layer reads it
 *     has written earlier in the same call, but two calls that overlap on the GPU (different
 *     streams, or one stream captured twice and replayed concurrently) race on it: keep
 *     calls on one device ordered. */
#define NML_SM100_STATIC_SCRATCH_BYTES (8u << 20)
int32_t nml_nvfp4_sm100_routed_swiglu_static(const NmlSm100RoutedSwiglu *request,
                                             char *error_message,
                                             size_t error_message_capacity);

/* Scratch bytes nml_nvfp4_sm100_routed_swiglu needs for the given extents (0 on overflow). */
size_t nml_nvfp4_sm100_routed_swiglu_workspace_bytes(int64_t tokens, int64_t hidden_size,
                                                     int64_t intermediate_size, int64_t experts,
                                                     int64_t experts_per_token);

/* Where nml_nvfp4_sm100_routed_swiglu keeps its intermediates inside the caller's workspace
 * (byte offsets), so that a test or a diagnostic tool can read the schedule and the
 * per-stage results of a call after it has run.  `slot_ordered` is 1 when a batch of this
 * size takes the large-batch path (rows permuted into schedule-slot order once, gate/up
 * result kept in slot order in `slot_activated`, `activated` unused) given a workspace of
 * nml_nvfp4_sm100_routed_swiglu_workspace_bytes(...) bytes.  Returns 1 on extents the layer
 * rejects.  No counterpart in the reference (its intermediates are XLA-owned buffers). */
typedef struct NmlSm100RoutedWorkspaceLayout {
  size_t sorted_assignments; /* i32 [schedule_positions] */
  size_t block_experts;      /* i32 [schedule_blocks] */
  size_t active_blocks;      /* i32 scalar */
  size_t activated;          /* dtype [assignments, intermediate] */
  size_t weighted;           /* dtype [assignments, hidden] */
  size_t permuted_hidden;    /* dtype [schedule_positions, hidden], slot-ordered path only */
  size_t slot_activated;     /* dtype [schedule_positions, intermediate], slot-ordered path only */
  int64_t schedule_blocks;
  int64_t schedule_positions;
  int32_t slot_ordered;
} NmlSm100RoutedWorkspaceLayout;
int32_t nml_nvfp4_sm100_routed_swiglu_workspace_layout(int64_t tokens, int64_t hidden_size,
                                                       int64_t intermediate_size,
                                                       int64_t experts,
                                                       int64_t experts_per_token,
                                                       NmlSm100RoutedWorkspaceLayout *layout);

/* Schedule capacity of the assignment plan: writes blocks and positions, returns 0,
 * or 1 when the schedule would not be addressable by int32
 * (crates/nml-ir/src/lib.rs:5662-5688). */
int32_t nml_nvfp4_sm100_plan_capacity(int64_t assignments, int64_t experts, int64_t *blocks,
                                      int64_t *positions);

/* Device status word of the current device: 0 when healthy, else an OR of the bits below.
 * Kernels never trap; a bounded wait that runs out or an out-of-range index records a
 * bit here and the kernel returns.  Bits 8 and up say which wait of the tcgen05 kernel ran
 * out (diagnostic only).  Reading synchronises `stream`; `clear` resets it. */
#define NML_SM100_STATUS_BARRIER_TIMEOUT 1
#define NML_SM100_STATUS_TMEM_ALLOC 2
#define NML_SM100_STATUS_INDEX_RANGE 4
#define NML_SM100_STATUS_PEER_TIMEOUT 8 /* an expert-parallel wait for another rank ran out */
int32_t nml_nvfp4_sm100_device_status(void *stream, int32_t clear, int32_t *status);

/* Kernel selection override for tests: every shape has one automatic choice, and each kernel
 * family must also be testable on shapes where it is not that choice.  The value belongs to
 * the calling thread (calls on other threads are not affected); returns the previous value.
 * A forced family that does not support the shape makes the call fail with
 * NML_SM100_INVALID_ARGUMENT. */
#define NML_SM100_POLICY_AUTO 0
#define NML_SM100_POLICY_SIMT 1        /* the portable any-shape kernels */
#define NML_SM100_POLICY_UMMA 2        /* the tcgen05 kernels */
#define NML_SM100_POLICY_UMMA_SMEM 3   /* tcgen05 with the decoded weight tiles in shared memory */
#define NML_SM100_POLICY_NO_SPLIT_K 5  /* tcgen05, never cut K over a cluster */
#define NML_SM100_POLICY_STREAM 6      /* the weight-streaming kernels for few rows */
int32_t nml_nvfp4_sm100_set_kernel_policy(int32_t policy);

/* Name of the kernel family the last nml_nvfp4_sm100_linear call on this thread selected
 * ("stream", "umma_tmem_weights_af16", "umma_tmem_weights_abf16",
 * "umma_tmem_weights_abf16_lut", "umma_swapab_af16", "umma_swapab_abf16", "simt"), for tests
 * and benchmark records; the fused Q/K/V call records its one launch the same way. */
const char *nml_nvfp4_sm100_last_linear_kernel(void);
/* Activation rows per tile of that launch (0 for the SIMT kernel). */
int32_t nml_nvfp4_sm100_last_linear_tile_rows(void);

/* ABI version of this header. */
#define NML_NVFP4_SM100_ABI_VERSION 2
int32_t nml_nvfp4_sm100_abi_version(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* NML_NVFP4_SM100_H_ */
