// extern "C" entry points of the sm_100a NVFP4 library: argument validation in the manner of
// the reference adapter (crates/nml-kernel-nvfp4/src/turing_adapter.cu:669-942), kernel
// selection, and the routed-layer orchestration.  Nothing here allocates device memory or
// synchronises a stream except nml_nvfp4_sm100_device_status, which exists to read a result.
#include <atomic>
#include <cstddef>
#include <cstring>

#include "common.cuh"

namespace nml_sm100 {

__device__ int g_status_word = 0;

// Scratch for nml_nvfp4_sm100_routed_swiglu_static: lives in the device image, so no call
// ever allocates it.  In host code this name is only a handle for cudaGetSymbolAddress, not
// a device pointer; kernels receive the address looked up by static_scratch_address().
static __device__ __align__(256) unsigned char g_static_scratch[NML_SM100_STATIC_SCRATCH_BYTES];

namespace {
thread_local int t_kernel_policy = NML_SM100_POLICY_AUTO;
thread_local const char* t_last_linear_kernel = "none";
thread_local int t_last_linear_tile_rows = 0;
constexpr int kMaxDevices = 64;
DeviceInfo g_devices[kMaxDevices];
std::atomic<int> g_device_ready[kMaxDevices];
}  // namespace

int get_kernel_policy() { return t_kernel_policy; }
static bool policy_forces_tensor_cores(int policy) {
  return policy == NML_SM100_POLICY_UMMA || policy == NML_SM100_POLICY_UMMA_SMEM;
}
static bool policy_allows_stream(int policy) {
  return policy == NML_SM100_POLICY_AUTO || policy == NML_SM100_POLICY_STREAM;
}
void note_linear_kernel(const char* name, int tile_rows) {
  t_last_linear_kernel = name;
  t_last_linear_tile_rows = tile_rows;
}

const DeviceInfo* current_device(char* message, size_t capacity) {
  int device = 0;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) {
    fail(NML_SM100_LAUNCH_FAILURE, cudaGetErrorString(status), message, capacity);
    return nullptr;
  }
  if (device < 0 || device >= kMaxDevices) {
    fail(NML_SM100_LAUNCH_FAILURE, "device ordinal out of range", message, capacity);
    return nullptr;
  }
  if (g_device_ready[device].load(std::memory_order_acquire) == 2) return &g_devices[device];
  // First use on this device: racing threads compute identical values.
  DeviceInfo info;
  info.device = device;
  if ((status = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device)) !=
          cudaSuccess ||
      (status = cudaDeviceGetAttribute(&info.major, cudaDevAttrComputeCapabilityMajor, device)) !=
          cudaSuccess ||
      (status = cudaDeviceGetAttribute(&info.minor, cudaDevAttrComputeCapabilityMinor, device)) !=
          cudaSuccess) {
    fail(NML_SM100_LAUNCH_FAILURE, cudaGetErrorString(status), message, capacity);
    return nullptr;
  }
  if (info.major != 10) {
    fail(NML_SM100_INVALID_ARGUMENT,
         "the NVFP4 sm_100a library requires compute capability 10.x", message, capacity);
    return nullptr;
  }
  void* address = nullptr;
  if ((status = cudaGetSymbolAddress(&address, g_status_word)) != cudaSuccess) {
    fail(NML_SM100_LAUNCH_FAILURE, cudaGetErrorString(status), message, capacity);
    return nullptr;
  }
  info.status_word = static_cast<int*>(address);
  int expected = 0;
  if (g_device_ready[device].compare_exchange_strong(expected, 1)) {
    g_devices[device] = info;
    g_device_ready[device].store(2, std::memory_order_release);
    return &g_devices[device];
  }
  while (g_device_ready[device].load(std::memory_order_acquire) != 2) {
  }
  return &g_devices[device];
}

int32_t launch_route(const NmlSm100Route& r, char* message, size_t capacity);
int32_t launch_assignment_plan(const int32_t* expert_ids, int32_t* sorted_assignments,
                               int32_t* block_experts, int32_t* active_blocks, int assignments,
                               int experts, int expert_offset, int positions, int blocks,
                               int device, cudaStream_t stream, char* message, size_t capacity);
int32_t launch_combine(const void* weighted, const int32_t* expert_ids, void* output, int tokens,
                       int top_k, int hidden, int experts, int expert_offset, int dtype,
                       cudaStream_t stream, char* message, size_t capacity);

int32_t launch_ep_dispatch_plan(const int32_t* expert_ids, int32_t* send_order,
                                int32_t* slot_of_assignment, int32_t* local_expert,
                                int32_t* send_counts, int assignments, int ranks,
                                int experts_per_rank, cudaStream_t stream, char* message,
                                size_t capacity);
int32_t launch_gather_rows(const void* source, const int32_t* row_index, void* output,
                           int64_t rows, int width, int divisor, int64_t source_rows, int dtype,
                           cudaStream_t stream, char* message, size_t capacity,
                           const int32_t* live_blocks = nullptr);
int32_t launch_combine_rows(const void* rows, const int32_t* row_index, void* output, int tokens,
                            int top_k, int width, int64_t row_count, int dtype,
                            cudaStream_t stream, char* message, size_t capacity);

namespace {

bool valid_dtype(int32_t dtype) { return dtype == NML_SM100_F16 || dtype == NML_SM100_BF16; }

bool plan_capacity(int64_t assignments, int64_t experts, int64_t* blocks, int64_t* positions) {
  if (assignments <= 0 || experts <= 0) return false;
  const int64_t nonempty = assignments < experts ? assignments : experts;
  const int64_t padded = assignments + nonempty * 15;
  const int64_t b = (padded + 15) / 16;
  const int64_t p = b * 16;
  if (assignments > std::numeric_limits<int32_t>::max() ||
      p > std::numeric_limits<int32_t>::max()) {
    return false;
  }
  *blocks = b;
  *positions = p;
  return true;
}

// One linear launch (one to three projections over one activation) on the kernel family the
// shape and the thread's policy select.  Returns kNoSingleLaunch when no family takes the
// projections in one launch.
constexpr int32_t kNoSingleLaunch = -1001;

int32_t dispatch_linear(const LinearArgs& args, const DeviceInfo& device, char* message,
                        size_t capacity) {
  const int policy = get_kernel_policy();
  if (policy_allows_stream(policy) && linear_stream_supported(args)) {
    return launch_linear_stream(args, device, message, capacity);
  }
  if (policy == NML_SM100_POLICY_STREAM) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "the weight-streaming kernel was forced but does not support this shape", message,
                capacity);
  }
  if (policy != NML_SM100_POLICY_SIMT && linear_umma_supported(args)) {
    return launch_linear_umma(args, device, message, capacity);
  }
  if (policy_forces_tensor_cores(policy)) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "the tcgen05 linear kernel was forced but does not support this shape", message,
                capacity);
  }
  if (args.extra_projections != 0) return kNoSingleLaunch;
  return launch_linear_simt(args, device, message, capacity);
}

int32_t dispatch_experts(const ExpertArgs& args, const DeviceInfo& device, char* message,
                         size_t capacity) {
  const int policy = get_kernel_policy();
  if (policy_allows_stream(policy) && experts_stream_supported(args)) {
    return launch_experts_stream(args, device, message, capacity);
  }
  if (policy == NML_SM100_POLICY_STREAM) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "the weight-streaming kernel was forced but does not support this shape", message,
                capacity);
  }
  if (policy != NML_SM100_POLICY_SIMT && experts_umma_supported(args)) {
    return launch_experts_umma(args, device, message, capacity);
  }
  if (policy_forces_tensor_cores(policy)) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "the tcgen05 expert kernel was forced but does not support this shape", message,
                capacity);
  }
  return launch_experts_simt(args, device, message, capacity);
}

size_t align_up(size_t value, size_t alignment) {
  return (value + alignment - 1) / alignment * alignment;
}

struct RoutedWorkspace {
  size_t sorted_offset, block_experts_offset, active_offset, activated_offset, weighted_offset;
  size_t total;           // bytes of the assignment-ordered layout (gathered rows)
  // Slot-ordered layout used for large batches: hidden rows permuted into schedule-slot order
  // and the activations kept in slot order, so both projections read contiguous rows by TMA.
  size_t permuted_offset, slot_activated_offset;
  size_t total_permuted;  // bytes including the two slot-ordered regions
  int64_t blocks, positions;
};

bool routed_workspace(int64_t tokens, int64_t hidden, int64_t intermediate, int64_t experts,
                      int64_t top_k, RoutedWorkspace* w) {
  if (tokens <= 0 || hidden <= 0 || intermediate <= 0 || experts <= 0 || top_k <= 0) return false;
  if (tokens > std::numeric_limits<int32_t>::max() / top_k) return false;
  const int64_t assignments = tokens * top_k;
  if (!plan_capacity(assignments, experts, &w->blocks, &w->positions)) return false;
  size_t offset = 0;
  w->sorted_offset = offset;
  offset = align_up(offset + static_cast<size_t>(w->positions) * 4, 256);
  w->block_experts_offset = offset;
  offset = align_up(offset + static_cast<size_t>(w->blocks) * 4, 256);
  w->active_offset = offset;
  offset = align_up(offset + 4, 256);
  w->activated_offset = offset;
  offset = align_up(offset + static_cast<size_t>(assignments) * intermediate * 2, 256);
  w->weighted_offset = offset;
  offset = align_up(offset + static_cast<size_t>(assignments) * hidden * 2, 256);
  w->total = offset;
  w->permuted_offset = offset;
  offset = align_up(offset + static_cast<size_t>(w->positions) * hidden * 2, 256);
  w->slot_activated_offset = offset;
  offset = align_up(offset + static_cast<size_t>(w->positions) * intermediate * 2, 256);
  w->total_permuted = offset;
  return true;
}

// Batches with more than this many expected slots per expert use the slot-ordered layout
// when the workspace has room for it.
constexpr int64_t kPermuteThreshold = 64;

template <typename Request>
bool has_field(const Request* request, size_t offset, size_t size) {
  return request->struct_size >= offset + size;
}

}  // namespace
}  // namespace nml_sm100

using namespace nml_sm100;

extern "C" int32_t nml_nvfp4_sm100_abi_version(void) { return NML_NVFP4_SM100_ABI_VERSION; }

extern "C" int32_t nml_nvfp4_sm100_set_kernel_policy(int32_t policy) {
  const int previous = t_kernel_policy;
  t_kernel_policy = policy;
  return previous;
}

extern "C" const char* nml_nvfp4_sm100_last_linear_kernel(void) { return t_last_linear_kernel; }
extern "C" int32_t nml_nvfp4_sm100_last_linear_tile_rows(void) { return t_last_linear_tile_rows; }

extern "C" int32_t nml_nvfp4_sm100_plan_capacity(int64_t assignments, int64_t experts,
                                                 int64_t* blocks, int64_t* positions) {
  if (blocks == nullptr || positions == nullptr) return NML_SM100_INVALID_ARGUMENT;
  return plan_capacity(assignments, experts, blocks, positions) ? NML_SM100_OK
                                                                : NML_SM100_INVALID_ARGUMENT;
}

extern "C" int32_t nml_nvfp4_sm100_device_status(void* stream, int32_t clear, int32_t* status) {
  if (status == nullptr) return NML_SM100_INVALID_ARGUMENT;
  const DeviceInfo* device = current_device(nullptr, 0);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int value = 0;
  if (cudaMemcpyAsync(&value, device->status_word, sizeof(int), cudaMemcpyDeviceToHost, s) !=
          cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    return NML_SM100_LAUNCH_FAILURE;
  }
  *status = value;
  if (clear && value != 0) {
    if (cudaMemsetAsync(device->status_word, 0, sizeof(int), s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
      return NML_SM100_LAUNCH_FAILURE;
    }
  }
  return NML_SM100_OK;
}

extern "C" int32_t nml_nvfp4_sm100_linear(const NmlSm100Linear* request, char* error_message,
                                          size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < offsetof(NmlSm100Linear, residual)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 linear request", error_message,
                error_message_capacity);
  }
  if (request->activation == nullptr || request->payload == nullptr ||
      request->block_scales == nullptr || request->global_scale == nullptr ||
      request->output == nullptr || request->stream == nullptr || !fits_i32(request->rows) ||
      !fits_i32(request->outputs) || !fits_i32(request->inputs)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 linear request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 linear supports F16 and BF16 only",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  LinearArgs args;
  args.activation = request->activation;
  args.payload = request->payload;
  args.block_scales = request->block_scales;
  args.global_scale = request->global_scale;
  args.bias = request->bias;
  args.output = request->output;
  args.stream = static_cast<cudaStream_t>(request->stream);
  args.rows = static_cast<int>(request->rows);
  args.outputs = static_cast<int>(request->outputs);
  args.inputs = static_cast<int>(request->inputs);
  args.dtype = request->dtype;
  args.residual = has_field(request, offsetof(NmlSm100Linear, residual), sizeof(void*))
                      ? request->residual
                      : nullptr;
  if (has_field(request, offsetof(NmlSm100Linear, workspace_bytes), sizeof(size_t))) {
    args.workspace = request->workspace;
    args.workspace_bytes = request->workspace != nullptr ? request->workspace_bytes : 0;
  }
  return dispatch_linear(args, *device, error_message, error_message_capacity);
}

extern "C" size_t nml_nvfp4_sm100_linear_workspace_bytes(int64_t rows, int64_t outputs,
                                                         int64_t inputs, int32_t dtype) {
  if (rows <= 0 || outputs <= 0 || inputs <= 0 || !fits_i32(rows) || !fits_i32(outputs) ||
      !fits_i32(inputs) || !valid_dtype(dtype)) {
    return 0;
  }
  return linear_umma_workspace_bytes(rows, outputs, inputs, dtype);
}

extern "C" size_t nml_nvfp4_sm100_linear_workspace_verdict_offset(int64_t rows, int64_t outputs,
                                                                  int64_t inputs,
                                                                  int32_t dtype) {
  if (nml_nvfp4_sm100_linear_workspace_bytes(rows, outputs, inputs, dtype) == 0) return 0;
  return linear_umma_workspace_verdict_offset(rows, inputs);
}

extern "C" int32_t nml_nvfp4_sm100_linear_qkv(const NmlSm100LinearQkv* request,
                                              char* error_message,
                                              size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100LinearQkv)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 QKV request", error_message,
                error_message_capacity);
  }
  bool valid = request->activation != nullptr && request->stream != nullptr &&
               fits_i32(request->rows) && fits_i32(request->inputs);
  int64_t total_outputs = 0;
  for (int i = 0; i < 3; ++i) {
    valid = valid && request->payload[i] != nullptr && request->block_scales[i] != nullptr &&
            request->global_scale[i] != nullptr && request->output[i] != nullptr &&
            fits_i32(request->outputs[i]);
    total_outputs += request->outputs[i];
  }
  if (!valid || !fits_i32(total_outputs)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 QKV request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 QKV supports F16 and BF16 only", error_message,
                error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  LinearArgs args;
  args.activation = request->activation;
  args.payload = request->payload[0];
  args.block_scales = request->block_scales[0];
  args.global_scale = request->global_scale[0];
  args.bias = request->bias[0];
  args.output = request->output[0];
  args.stream = static_cast<cudaStream_t>(request->stream);
  args.rows = static_cast<int>(request->rows);
  args.outputs = static_cast<int>(request->outputs[0]);
  args.inputs = static_cast<int>(request->inputs);
  args.dtype = request->dtype;
  args.extra_projections = 2;
  for (int i = 0; i < 2; ++i) {
    args.extra[i] = {request->payload[i + 1], request->block_scales[i + 1],
                     request->global_scale[i + 1], request->bias[i + 1], request->output[i + 1],
                     static_cast<int>(request->outputs[i + 1])};
  }
  const int32_t fused = dispatch_linear(args, *device, error_message, error_message_capacity);
  if (fused != kNoSingleLaunch) return fused;
  // one launch per projection
  for (int i = 0; i < 3; ++i) {
    LinearArgs one;
    one.activation = request->activation;
    one.payload = request->payload[i];
    one.block_scales = request->block_scales[i];
    one.global_scale = request->global_scale[i];
    one.bias = request->bias[i];
    one.output = request->output[i];
    one.stream = args.stream;
    one.rows = args.rows;
    one.outputs = static_cast<int>(request->outputs[i]);
    one.inputs = args.inputs;
    one.dtype = args.dtype;
    const int32_t rc = dispatch_linear(one, *device, error_message, error_message_capacity);
    if (rc != NML_SM100_OK) return rc;
  }
  return NML_SM100_OK;
}

extern "C" int32_t nml_nvfp4_sm100_embedding(const NmlSm100Embedding* request,
                                             char* error_message,
                                             size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100Embedding)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 embedding request", error_message,
                error_message_capacity);
  }
  if (request->indices == nullptr || request->payload == nullptr ||
      request->block_scales == nullptr || request->global_scale == nullptr ||
      request->output == nullptr || request->stream == nullptr || !fits_i32(request->rows) ||
      !fits_i32(request->vocabulary) || !fits_i32(request->width)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 embedding request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 embedding supports F16 and BF16 only",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  EmbeddingArgs args;
  args.indices = request->indices;
  args.payload = request->payload;
  args.block_scales = request->block_scales;
  args.global_scale = request->global_scale;
  args.output = request->output;
  args.stream = static_cast<cudaStream_t>(request->stream);
  args.rows = request->rows;
  args.vocabulary = static_cast<int>(request->vocabulary);
  args.width = static_cast<int>(request->width);
  args.dtype = request->dtype;
  args.indices_are_i64 = request->indices_are_i64 != 0;
  return launch_embedding(args, *device, error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_expert_gate_up(const NmlSm100ExpertGateUp* request,
                                                  char* error_message,
                                                  size_t error_message_capacity) {
  constexpr size_t kReferenceSize = offsetof(NmlSm100ExpertGateUp, active_blocks);
  if (request == nullptr || request->struct_size < kReferenceSize ||
      request->hidden == nullptr || request->sorted_assignments == nullptr ||
      request->block_experts == nullptr || request->payload == nullptr ||
      request->block_scales == nullptr || request->global_scale == nullptr ||
      request->bias == nullptr || request->activated == nullptr || request->stream == nullptr ||
      request->block_size != 16 || !fits_i32(request->assignments) ||
      !fits_i32(request->hidden_size) || !fits_i32(request->intermediate_size) ||
      request->intermediate_size > std::numeric_limits<int32_t>::max() / 2 ||
      request->tokens <= 0 || !fits_i32(request->experts) || request->experts_per_token <= 0 ||
      request->tokens > std::numeric_limits<int64_t>::max() / request->experts_per_token ||
      request->assignments != request->tokens * request->experts_per_token ||
      !fits_i32(request->schedule_blocks) ||
      request->schedule_blocks > std::numeric_limits<int32_t>::max() / 16 ||
      request->schedule_positions != request->schedule_blocks * 16) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 expert gate/up request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 experts support F16 and BF16 only",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  ExpertArgs args;
  args.input = request->hidden;
  args.sorted_assignments = request->sorted_assignments;
  args.block_experts = request->block_experts;
  args.payload = request->payload;
  args.block_scales = request->block_scales;
  args.global_scale = request->global_scale;
  args.bias = request->bias;
  args.routing_weights = nullptr;
  args.output = request->activated;
  args.active_blocks =
      has_field(request, offsetof(NmlSm100ExpertGateUp, active_blocks), sizeof(void*))
          ? request->active_blocks
          : nullptr;
  args.expert_offset =
      has_field(request, offsetof(NmlSm100ExpertGateUp, expert_offset), sizeof(void*))
          ? request->expert_offset
          : nullptr;
  args.stream = static_cast<cudaStream_t>(request->stream);
  args.assignments = static_cast<int>(request->assignments);
  args.schedule_blocks = static_cast<int>(request->schedule_blocks);
  args.inputs = static_cast<int>(request->hidden_size);
  args.outputs = static_cast<int>(request->intermediate_size);
  args.experts = static_cast<int>(request->experts);
  args.experts_per_token = static_cast<int>(request->experts_per_token);
  args.dtype = request->dtype;
  args.gate_up = true;
  return dispatch_experts(args, *device, error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_expert_down(const NmlSm100ExpertDown* request,
                                               char* error_message,
                                               size_t error_message_capacity) {
  constexpr size_t kReferenceSize = offsetof(NmlSm100ExpertDown, active_blocks);
  if (request == nullptr || request->struct_size < kReferenceSize ||
      request->activated == nullptr || request->sorted_assignments == nullptr ||
      request->block_experts == nullptr || request->payload == nullptr ||
      request->block_scales == nullptr || request->global_scale == nullptr ||
      request->bias == nullptr || request->routing_weights == nullptr ||
      request->weighted_output == nullptr || request->stream == nullptr ||
      request->block_size != 16 || !fits_i32(request->assignments) ||
      !fits_i32(request->intermediate_size) || !fits_i32(request->hidden_size) ||
      !fits_i32(request->experts) || request->experts_per_token <= 0 ||
      !fits_i32(request->schedule_blocks) ||
      request->schedule_blocks > std::numeric_limits<int32_t>::max() / 16 ||
      request->schedule_positions != request->schedule_blocks * 16) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 expert down request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 experts support F16 and BF16 only",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  ExpertArgs args;
  args.input = request->activated;
  args.sorted_assignments = request->sorted_assignments;
  args.block_experts = request->block_experts;
  args.payload = request->payload;
  args.block_scales = request->block_scales;
  args.global_scale = request->global_scale;
  args.bias = request->bias;
  args.routing_weights = request->routing_weights;
  args.output = request->weighted_output;
  args.active_blocks =
      has_field(request, offsetof(NmlSm100ExpertDown, active_blocks), sizeof(void*))
          ? request->active_blocks
          : nullptr;
  args.expert_offset =
      has_field(request, offsetof(NmlSm100ExpertDown, expert_offset), sizeof(void*))
          ? request->expert_offset
          : nullptr;
  args.row_targets = has_field(request, offsetof(NmlSm100ExpertDown, row_targets), sizeof(void*))
                         ? request->row_targets
                         : nullptr;
  args.stream = static_cast<cudaStream_t>(request->stream);
  args.assignments = static_cast<int>(request->assignments);
  args.schedule_blocks = static_cast<int>(request->schedule_blocks);
  args.inputs = static_cast<int>(request->intermediate_size);
  args.outputs = static_cast<int>(request->hidden_size);
  args.experts = static_cast<int>(request->experts);
  args.experts_per_token = static_cast<int>(request->experts_per_token);
  args.dtype = request->dtype;
  args.gate_up = false;
  return dispatch_experts(args, *device, error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_route(const NmlSm100Route* request, char* error_message,
                                         size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100Route)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 route request", error_message,
                error_message_capacity);
  }
  if (request->logits == nullptr || request->expert_ids == nullptr ||
      request->routing_weights == nullptr || request->stream == nullptr ||
      !fits_i32(request->tokens) || request->experts <= 0 || request->experts > 256 ||
      request->experts_per_token <= 0 || request->experts_per_token > 16 ||
      request->experts_per_token > request->experts ||
      request->tokens > std::numeric_limits<int32_t>::max() / request->experts_per_token) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 route request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 routing weights support F16 and BF16 only",
                error_message, error_message_capacity);
  }
  if (current_device(error_message, error_message_capacity) == nullptr) {
    return NML_SM100_LAUNCH_FAILURE;
  }
  return launch_route(*request, error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_assignment_plan(const NmlSm100AssignmentPlan* request,
                                                   char* error_message,
                                                   size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100AssignmentPlan)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 assignment plan request",
                error_message, error_message_capacity);
  }
  int64_t blocks = 0, positions = 0;
  if (request->expert_ids == nullptr || request->sorted_assignments == nullptr ||
      request->block_experts == nullptr || request->active_blocks == nullptr ||
      request->stream == nullptr || request->block_size != 16 || request->experts > 1024 ||
      request->expert_offset < 0 ||
      !plan_capacity(request->assignments, request->experts, &blocks, &positions) ||
      request->schedule_blocks != blocks || request->schedule_positions != positions) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 assignment plan request",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  return launch_assignment_plan(request->expert_ids, request->sorted_assignments,
                                request->block_experts, request->active_blocks,
                                static_cast<int>(request->assignments),
                                static_cast<int>(request->experts), request->expert_offset,
                                static_cast<int>(positions), static_cast<int>(blocks),
                                device->device, static_cast<cudaStream_t>(request->stream),
                                error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_combine(const NmlSm100Combine* request, char* error_message,
                                           size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100Combine)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 combine request", error_message,
                error_message_capacity);
  }
  if (request->weighted == nullptr || request->output == nullptr || request->stream == nullptr ||
      !fits_i32(request->tokens) || !fits_i32(request->hidden_size) ||
      request->experts_per_token <= 0 ||
      request->tokens > std::numeric_limits<int32_t>::max() / request->experts_per_token ||
      (request->expert_ids != nullptr && (!fits_i32(request->experts) ||
                                          request->expert_offset < 0))) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 combine request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 combine supports F16 and BF16 only",
                error_message, error_message_capacity);
  }
  if (current_device(error_message, error_message_capacity) == nullptr) {
    return NML_SM100_LAUNCH_FAILURE;
  }
  return launch_combine(request->weighted, request->expert_ids, request->output,
                        static_cast<int>(request->tokens),
                        static_cast<int>(request->experts_per_token),
                        static_cast<int>(request->hidden_size),
                        static_cast<int>(request->experts), request->expert_offset,
                        request->dtype, static_cast<cudaStream_t>(request->stream), error_message,
                        error_message_capacity);
}

extern "C" size_t nml_nvfp4_sm100_routed_swiglu_workspace_bytes(int64_t tokens,
                                                                int64_t hidden_size,
                                                                int64_t intermediate_size,
                                                                int64_t experts,
                                                                int64_t experts_per_token) {
  RoutedWorkspace w;
  if (!routed_workspace(tokens, hidden_size, intermediate_size, experts, experts_per_token, &w)) {
    return 0;
  }
  return tokens * experts_per_token > kPermuteThreshold * experts ? w.total_permuted : w.total;
}

extern "C" int32_t nml_nvfp4_sm100_routed_swiglu_workspace_layout(
    int64_t tokens, int64_t hidden_size, int64_t intermediate_size, int64_t experts,
    int64_t experts_per_token, NmlSm100RoutedWorkspaceLayout* layout) {
  RoutedWorkspace w;
  if (layout == nullptr || !routed_workspace(tokens, hidden_size, intermediate_size, experts,
                                             experts_per_token, &w)) {
    return NML_SM100_INVALID_ARGUMENT;
  }
  layout->sorted_assignments = w.sorted_offset;
  layout->block_experts = w.block_experts_offset;
  layout->active_blocks = w.active_offset;
  layout->activated = w.activated_offset;
  layout->weighted = w.weighted_offset;
  layout->permuted_hidden = w.permuted_offset;
  layout->slot_activated = w.slot_activated_offset;
  layout->schedule_blocks = w.blocks;
  layout->schedule_positions = w.positions;
  layout->slot_ordered = tokens * experts_per_token > kPermuteThreshold * experts ? 1 : 0;
  return NML_SM100_OK;
}

extern "C" int32_t nml_nvfp4_sm100_routed_swiglu(const NmlSm100RoutedSwiglu* request,
                                                 char* error_message,
                                                 size_t error_message_capacity) {
  if (request == nullptr ||
      request->struct_size < offsetof(NmlSm100RoutedSwiglu, live_routes_hint)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 routed SwiGLU request",
                error_message, error_message_capacity);
  }
  RoutedWorkspace w;
  if (request->hidden == nullptr || request->expert_ids == nullptr ||
      request->routing_weights == nullptr || request->gate_payload == nullptr ||
      request->gate_scales == nullptr || request->gate_global == nullptr ||
      request->gate_bias == nullptr || request->down_payload == nullptr ||
      request->down_scales == nullptr || request->down_global == nullptr ||
      request->down_bias == nullptr || request->output == nullptr ||
      request->workspace == nullptr || request->stream == nullptr ||
      request->expert_offset < 0 || !fits_i32(request->tokens) ||
      !fits_i32(request->hidden_size) || !fits_i32(request->intermediate_size) ||
      request->intermediate_size > std::numeric_limits<int32_t>::max() / 2 ||
      !fits_i32(request->experts) || request->experts > 1024 ||
      !routed_workspace(request->tokens, request->hidden_size, request->intermediate_size,
                        request->experts, request->experts_per_token, &w)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 routed SwiGLU request", error_message,
                error_message_capacity);
  }
  if (request->workspace_bytes < w.total ||
      reinterpret_cast<uintptr_t>(request->workspace) % 256 != 0) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "NVFP4 routed SwiGLU workspace is too small or not 256-byte aligned",
                error_message, error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 experts support F16 and BF16 only",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;

  uint8_t* base = static_cast<uint8_t*>(request->workspace);
  int32_t* sorted = reinterpret_cast<int32_t*>(base + w.sorted_offset);
  int32_t* block_experts = reinterpret_cast<int32_t*>(base + w.block_experts_offset);
  int32_t* active = reinterpret_cast<int32_t*>(base + w.active_offset);
  void* activated = base + w.activated_offset;
  void* weighted = base + w.weighted_offset;
  cudaStream_t stream = static_cast<cudaStream_t>(request->stream);
  const int assignments = static_cast<int>(request->tokens * request->experts_per_token);

  int32_t status = launch_assignment_plan(
      request->expert_ids, sorted, block_experts, active, assignments,
      static_cast<int>(request->experts), request->expert_offset, static_cast<int>(w.positions),
      static_cast<int>(w.blocks), device->device, stream, error_message, error_message_capacity);
  if (status != NML_SM100_OK) return status;

  ExpertArgs args;
  args.sorted_assignments = sorted;
  args.block_experts = block_experts;
  args.active_blocks = active;
  args.expert_offset = nullptr;  // the plan already stores local expert indices
  args.stream = stream;
  args.assignments = assignments;
  args.schedule_blocks = static_cast<int>(w.blocks);
  args.experts = static_cast<int>(request->experts);
  args.experts_per_token = static_cast<int>(request->experts_per_token);
  args.dtype = request->dtype;
  if (has_field(request, offsetof(NmlSm100RoutedSwiglu, live_routes_hint), sizeof(int64_t)) &&
      request->live_routes_hint > 0 && request->live_routes_hint < assignments) {
    args.live_routes = static_cast<int>(request->live_routes_hint);
  }

  args.inputs = static_cast<int>(request->hidden_size);
  args.outputs = static_cast<int>(request->intermediate_size);
  args.gate_up = true;
  args.input = request->hidden;
  args.payload = request->gate_payload;
  args.block_scales = request->gate_scales;
  args.global_scale = request->gate_global;
  args.bias = request->gate_bias;
  args.routing_weights = nullptr;
  args.output = activated;
  // Large batches: permute the hidden rows into slot order once (token permute) so that both
  // projections stream contiguous rows by TMA instead of gathering through the load/store
  // unit; the result rows go back to assignment order in the down epilogue (unpermute).
  const int64_t live = args.live_routes > 0 ? args.live_routes : assignments;
  const bool slot_ordered =
      live > kPermuteThreshold * request->experts &&
      request->workspace_bytes >= w.total_permuted &&
      get_kernel_policy() != NML_SM100_POLICY_SIMT &&
      experts_umma_supported(args) && request->hidden_size % 8 == 0 &&
      request->intermediate_size % 64 == 0 &&
      reinterpret_cast<uintptr_t>(request->hidden) % 16 == 0;
  if (slot_ordered) {
    void* permuted = base + w.permuted_offset;
    void* slot_activated = base + w.slot_activated_offset;
    status = launch_gather_rows(request->hidden, sorted, permuted, w.positions,
                                static_cast<int>(request->hidden_size),
                                static_cast<int>(request->experts_per_token), request->tokens,
                                request->dtype, stream, error_message, error_message_capacity,
                                active);
    if (status != NML_SM100_OK) return status;
    args.input = permuted;
    args.output = slot_activated;
    args.slot_input = true;
    status = launch_experts_umma(args, *device, error_message, error_message_capacity);
    if (status != NML_SM100_OK) return status;
    args.input = slot_activated;
  } else {
    status = dispatch_experts(args, *device, error_message, error_message_capacity);
    if (status != NML_SM100_OK) return status;
    args.input = activated;
  }

  args.payload = request->down_payload;
  args.block_scales = request->down_scales;
  args.global_scale = request->down_global;
  args.bias = request->down_bias;
  args.routing_weights = request->routing_weights;
  args.output = weighted;
  args.inputs = static_cast<int>(request->intermediate_size);
  args.outputs = static_cast<int>(request->hidden_size);
  args.gate_up = false;
  if (slot_ordered && !experts_umma_supported(args)) {
    return fail(NML_SM100_INVALID_ARGUMENT,
                "NVFP4 routed SwiGLU: the down projection cannot read slot-ordered rows",
                error_message, error_message_capacity);
  }
  const bool rows_are_routes =
      request->experts_per_token == 1 &&
      has_field(request, offsetof(NmlSm100RoutedSwiglu, flags), sizeof(int32_t)) &&
      (request->flags & NML_SM100_ROUTED_LEAVE_MASKED_ROWS) != 0;
  if (rows_are_routes) {
    args.output = request->output;  // assignment a is token a
    if (has_field(request, offsetof(NmlSm100RoutedSwiglu, row_targets), sizeof(void*))) {
      args.row_targets = request->row_targets;
    }
  }
  status = dispatch_experts(args, *device, error_message, error_message_capacity);
  if (status != NML_SM100_OK || rows_are_routes) return status;

  return launch_combine(weighted, request->expert_ids, request->output,
                        static_cast<int>(request->tokens),
                        static_cast<int>(request->experts_per_token),
                        static_cast<int>(request->hidden_size),
                        static_cast<int>(request->experts), request->expert_offset,
                        request->dtype, stream, error_message, error_message_capacity);
}


namespace nml_sm100 {
namespace {

uint8_t* g_static_scratch_address[kMaxDevices];
std::atomic<int> g_static_scratch_ready[kMaxDevices];

// Device address of g_static_scratch on the current device, looked up once per device with
// that device current.  Returns nullptr and fills the message when the lookup fails.
uint8_t* static_scratch_address(int device, char* message, size_t capacity) {
  if (g_static_scratch_ready[device].load(std::memory_order_acquire) == 2) {
    return g_static_scratch_address[device];
  }
  void* address = nullptr;
  const cudaError_t status = cudaGetSymbolAddress(&address, g_static_scratch);
  if (status != cudaSuccess || address == nullptr) {
    fail(NML_SM100_LAUNCH_FAILURE,
         status != cudaSuccess ? cudaGetErrorString(status)
                               : "the static scratch array has no device address",
         message, capacity);
    return nullptr;
  }
  int expected = 0;
  if (g_static_scratch_ready[device].compare_exchange_strong(expected, 1)) {
    g_static_scratch_address[device] = static_cast<uint8_t*>(address);
    g_static_scratch_ready[device].store(2, std::memory_order_release);
  } else {
    while (g_static_scratch_ready[device].load(std::memory_order_acquire) != 2) {
    }
  }
  return g_static_scratch_address[device];
}

}  // namespace
}  // namespace nml_sm100

extern "C" int32_t nml_nvfp4_sm100_routed_swiglu_static(const NmlSm100RoutedSwiglu* request,
                                                        char* error_message,
                                                        size_t error_message_capacity) {
  if (request == nullptr ||
      request->struct_size < offsetof(NmlSm100RoutedSwiglu, live_routes_hint)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 routed SwiGLU request",
                error_message, error_message_capacity);
  }
  RoutedWorkspace w;
  if (request->hidden == nullptr || request->expert_ids == nullptr ||
      request->routing_weights == nullptr || request->gate_payload == nullptr ||
      request->gate_scales == nullptr || request->gate_global == nullptr ||
      request->gate_bias == nullptr || request->down_payload == nullptr ||
      request->down_scales == nullptr || request->down_global == nullptr ||
      request->down_bias == nullptr || request->output == nullptr ||
      request->stream == nullptr || request->expert_offset < 0 || !fits_i32(request->tokens) ||
      !fits_i32(request->hidden_size) || !fits_i32(request->intermediate_size) ||
      request->intermediate_size > std::numeric_limits<int32_t>::max() / 2 ||
      !fits_i32(request->experts) || request->experts > 1024 ||
      !routed_workspace(request->tokens, request->hidden_size, request->intermediate_size,
                        request->experts, request->experts_per_token, &w)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 routed SwiGLU request", error_message,
                error_message_capacity);
  }
  if (w.total > NML_SM100_STATIC_SCRATCH_BYTES) {
    char text[160];
    std::snprintf(text, sizeof(text),
                  "NVFP4 routed SwiGLU needs %zu scratch bytes, the static scratch holds %u",
                  w.total, static_cast<unsigned>(NML_SM100_STATIC_SCRATCH_BYTES));
    return fail(NML_SM100_INVALID_ARGUMENT, text, error_message, error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 experts support F16 and BF16 only",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  uint8_t* base =
      static_scratch_address(device->device, error_message, error_message_capacity);
  if (base == nullptr) return NML_SM100_LAUNCH_FAILURE;

  int32_t* sorted = reinterpret_cast<int32_t*>(base + w.sorted_offset);
  int32_t* block_experts = reinterpret_cast<int32_t*>(base + w.block_experts_offset);
  int32_t* active = reinterpret_cast<int32_t*>(base + w.active_offset);
  void* activated = base + w.activated_offset;
  void* weighted = base + w.weighted_offset;
  cudaStream_t stream = static_cast<cudaStream_t>(request->stream);
  const int assignments = static_cast<int>(request->tokens * request->experts_per_token);

  // The schedule is rewritten in full (sentinels included) and the combine reads only rows
  // of routes the schedule covered, so nothing has to be cleared between calls.
  int32_t status = launch_assignment_plan(
      request->expert_ids, sorted, block_experts, active, assignments,
      static_cast<int>(request->experts), request->expert_offset, static_cast<int>(w.positions),
      static_cast<int>(w.blocks), device->device, stream, error_message, error_message_capacity);
  if (status != NML_SM100_OK) return status;

  ExpertArgs args;
  args.sorted_assignments = sorted;
  args.block_experts = block_experts;
  args.active_blocks = active;
  args.expert_offset = nullptr;
  args.stream = stream;
  args.assignments = assignments;
  args.schedule_blocks = static_cast<int>(w.blocks);
  args.experts = static_cast<int>(request->experts);
  args.experts_per_token = static_cast<int>(request->experts_per_token);
  args.dtype = request->dtype;

  args.input = request->hidden;
  args.payload = request->gate_payload;
  args.block_scales = request->gate_scales;
  args.global_scale = request->gate_global;
  args.bias = request->gate_bias;
  args.routing_weights = nullptr;
  args.output = activated;
  args.inputs = static_cast<int>(request->hidden_size);
  args.outputs = static_cast<int>(request->intermediate_size);
  args.gate_up = true;
  status = dispatch_experts(args, *device, error_message, error_message_capacity);
  if (status != NML_SM100_OK) return status;

  args.input = activated;
  args.payload = request->down_payload;
  args.block_scales = request->down_scales;
  args.global_scale = request->down_global;
  args.bias = request->down_bias;
  args.routing_weights = request->routing_weights;
  args.output = weighted;
  args.inputs = static_cast<int>(request->intermediate_size);
  args.outputs = static_cast<int>(request->hidden_size);
  args.gate_up = false;
  status = dispatch_experts(args, *device, error_message, error_message_capacity);
  if (status != NML_SM100_OK) return status;

  return launch_combine(weighted, request->expert_ids, request->output,
                        static_cast<int>(request->tokens),
                        static_cast<int>(request->experts_per_token),
                        static_cast<int>(request->hidden_size),
                        static_cast<int>(request->experts), request->expert_offset,
                        request->dtype, stream, error_message, error_message_capacity);
}


extern "C" int32_t nml_nvfp4_sm100_ep_dispatch_plan(const NmlSm100EpDispatchPlan* request,
                                                    char* error_message,
                                                    size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100EpDispatchPlan)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 dispatch plan request",
                error_message, error_message_capacity);
  }
  if (request->expert_ids == nullptr || request->send_order == nullptr ||
      request->local_expert == nullptr || request->slot_of_assignment == nullptr ||
      request->send_counts == nullptr || request->stream == nullptr ||
      !fits_i32(request->assignments) || request->ranks <= 0 || request->ranks > 64 ||
      !fits_i32(request->experts_per_rank)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 dispatch plan request", error_message,
                error_message_capacity);
  }
  if (current_device(error_message, error_message_capacity) == nullptr) {
    return NML_SM100_LAUNCH_FAILURE;
  }
  return launch_ep_dispatch_plan(request->expert_ids, request->send_order,
                                 request->slot_of_assignment, request->local_expert,
                                 request->send_counts, static_cast<int>(request->assignments),
                                 static_cast<int>(request->ranks),
                                 static_cast<int>(request->experts_per_rank),
                                 static_cast<cudaStream_t>(request->stream), error_message,
                                 error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_gather_rows(const NmlSm100GatherRows* request,
                                               char* error_message,
                                               size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100GatherRows)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 row gather request", error_message,
                error_message_capacity);
  }
  if (request->source == nullptr || request->row_index == nullptr ||
      request->output == nullptr || request->stream == nullptr || !fits_i32(request->rows) ||
      !fits_i32(request->source_rows) || !fits_i32(request->width) || request->width % 8 != 0 ||
      request->index_divisor <= 0 || reinterpret_cast<uintptr_t>(request->source) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(request->output) % 16 != 0) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 row gather request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 row gather supports F16 and BF16 only",
                error_message, error_message_capacity);
  }
  if (current_device(error_message, error_message_capacity) == nullptr) {
    return NML_SM100_LAUNCH_FAILURE;
  }
  return launch_gather_rows(request->source, request->row_index, request->output, request->rows,
                            static_cast<int>(request->width), request->index_divisor,
                            request->source_rows, request->dtype,
                            static_cast<cudaStream_t>(request->stream), error_message,
                            error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_ep_push_rows(const NmlSm100EpPushRows* request,
                                                char* error_message,
                                                size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100EpPushRows)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 row push request", error_message,
                error_message_capacity);
  }
  const bool valid = request->source != nullptr && request->send_order != nullptr &&
                     request->local_expert != nullptr && request->routing_weights != nullptr &&
                     request->send_counts != nullptr && request->stream != nullptr &&
                     fits_i32(request->assignments) && fits_i32(request->source_rows) &&
                     request->experts_per_token > 0 && valid_exchange(request->exchange) &&
                     request->assignments <= request->exchange.region_rows &&
                     reinterpret_cast<uintptr_t>(request->source) % 16 == 0;
  if (!valid || !valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 row push request", error_message,
                error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  return launch_ep_push_rows(*request, *device, error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_ep_receive_meta(const NmlSm100EpReceiveMeta* request,
                                                   char* error_message,
                                                   size_t error_message_capacity) {
  if (request == nullptr ||
      request->struct_size < offsetof(NmlSm100EpReceiveMeta, row_targets)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 receive meta request", error_message,
                error_message_capacity);
  }
  if (request->expert_ids == nullptr || request->routing_weights == nullptr ||
      request->received == nullptr || request->stream == nullptr || request->wait_limit < 0 ||
      !valid_exchange(request->exchange) || !valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 receive meta request", error_message,
                error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  return launch_ep_receive_meta(*request, *device, error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_ep_return_rows(const NmlSm100EpReturnRows* request,
                                                  char* error_message,
                                                  size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100EpReturnRows)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 row return request", error_message,
                error_message_capacity);
  }
  if (request->stream == nullptr || !valid_exchange(request->exchange) ||
      !valid_dtype(request->dtype) ||
      reinterpret_cast<uintptr_t>(request->computed) % 16 != 0) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 row return request", error_message,
                error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  return launch_ep_return_rows(*request, *device, error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_ep_wait_returns(const NmlSm100EpWaitReturns* request,
                                                   char* error_message,
                                                   size_t error_message_capacity) {
  if (request == nullptr ||
      request->struct_size < offsetof(NmlSm100EpWaitReturns, row_index)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 return wait request", error_message,
                error_message_capacity);
  }
  if (request->stream == nullptr || request->wait_limit < 0 ||
      !valid_exchange(request->exchange)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 return wait request", error_message,
                error_message_capacity);
  }
  if (request->struct_size >= sizeof(NmlSm100EpWaitReturns) && request->output != nullptr &&
      (request->row_index == nullptr || request->tokens <= 0 || !fits_i32(request->tokens) ||
       request->experts_per_token <= 0 || !fits_i32(request->experts_per_token) ||
       !valid_dtype(request->dtype) ||
       reinterpret_cast<uintptr_t>(request->output) % 16 != 0)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 return combine request",
                error_message, error_message_capacity);
  }
  const DeviceInfo* device = current_device(error_message, error_message_capacity);
  if (device == nullptr) return NML_SM100_LAUNCH_FAILURE;
  return launch_ep_wait_returns(*request, *device, error_message, error_message_capacity);
}

extern "C" int32_t nml_nvfp4_sm100_combine_rows(const NmlSm100CombineRows* request,
                                                char* error_message,
                                                size_t error_message_capacity) {
  if (request == nullptr || request->struct_size < sizeof(NmlSm100CombineRows)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "truncated NVFP4 row combine request", error_message,
                error_message_capacity);
  }
  if (request->rows == nullptr || request->row_index == nullptr || request->output == nullptr ||
      request->stream == nullptr || !fits_i32(request->tokens) ||
      !fits_i32(request->hidden_size) || request->hidden_size % 8 != 0 ||
      request->experts_per_token <= 0 || request->row_count < 0 ||
      request->row_count > std::numeric_limits<int32_t>::max() ||
      request->tokens > std::numeric_limits<int32_t>::max() / request->experts_per_token ||
      reinterpret_cast<uintptr_t>(request->rows) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(request->output) % 16 != 0) {
    return fail(NML_SM100_INVALID_ARGUMENT, "invalid NVFP4 row combine request", error_message,
                error_message_capacity);
  }
  if (!valid_dtype(request->dtype)) {
    return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 row combine supports F16 and BF16 only",
                error_message, error_message_capacity);
  }
  if (current_device(error_message, error_message_capacity) == nullptr) {
    return NML_SM100_LAUNCH_FAILURE;
  }
  return launch_combine_rows(request->rows, request->row_index, request->output,
                             static_cast<int>(request->tokens),
                             static_cast<int>(request->experts_per_token),
                             static_cast<int>(request->hidden_size), request->row_count,
                             request->dtype, static_cast<cudaStream_t>(request->stream),
                             error_message, error_message_capacity);
}
