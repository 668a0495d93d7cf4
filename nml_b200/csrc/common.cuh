// Shared host/device helpers of the sm_100a NVFP4 library: error reporting in the
// reference adapter's convention, exact NVFP4 decode arithmetic, 16-bit dtype traits.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <limits>

#include "../../include/nml_nvfp4_sm100.h"

namespace nml_sm100 {

// ---- host-side error convention (crates/nml-kernel-nvfp4/src/turing_adapter.cu:13-22) ----
inline int32_t fail(int32_t code, const char* message, char* output, size_t capacity) {
  if (output != nullptr && capacity != 0) {
    std::snprintf(output, capacity, "%s", message);
  }
  return code;
}

inline int32_t launch_result(char* message, size_t capacity) {
  const cudaError_t status = cudaPeekAtLastError();
  return status == cudaSuccess
             ? NML_SM100_OK
             : fail(NML_SM100_LAUNCH_FAILURE, cudaGetErrorString(status), message, capacity);
}

inline bool fits_i32(int64_t value) {
  return value > 0 && value <= std::numeric_limits<int32_t>::max();
}

// Properties of the current device, looked up once per device and cached.
struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int major = 0;
  int minor = 0;
  int* status_word = nullptr;  // device address of the status word on this device
};

// Returns nullptr and fills the message when the device cannot be queried.
const DeviceInfo* current_device(char* message, size_t capacity);

// ---- exact decode arithmetic --------------------------------------------------
// E2M1 code -> f32.  The three magnitude bits placed at f32 bits 24:22 read as
// value * 2^-126 (0.5 is the f32 subnormal), so one exact multiply by 2^126 gives
// {0, .5, 1, 1.5, 2, 3, 4, 6}; bit 3 is the sign and -0 is preserved.
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  const float magnitude = __fmul_rn(__uint_as_float((code & 0x7u) << 22), 0x1p126f);
  return __uint_as_float(__float_as_uint(magnitude) | ((code & 0x8u) << 28));
}

// Unsigned E4M3FN scale byte -> f32.  The seven value bits placed at f32 bits
// 26:20 read as scale * 2^-120 for normal and subnormal codes alike.  Bytes the
// format does not define for a scale (sign bit set, or 0x7f) decode to NaN, the
// same poison the reference device kernels produce (turing_adapter.cu:35-40).
__device__ __forceinline__ float e4m3_scale_to_f32(uint32_t bits) {
  if ((bits & 0x80u) != 0u || (bits & 0x7fu) == 0x7fu) return __uint_as_float(0x7fc00000u);
  return __fmul_rn(__uint_as_float((bits & 0x7fu) << 20), 0x1p120f);
}

// ---- 16-bit element traits ------------------------------------------------------
template <typename T>
struct Elem;

template <>
struct Elem<__half> {
  static __device__ __forceinline__ float load(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half store(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float from_bits(uint32_t bits16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
  }
};

template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 store(float v) {
    return __float2bfloat16_rn(v);
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float from_bits(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
  }
};

// Narrows a finished linear output; with a residual operand the narrowed value and the
// residual are added and narrowed again, as a separate elementwise add on 16-bit tensors would.
template <typename T>
__device__ __forceinline__ T narrow_with_residual(float value, const T* residual, int64_t index) {
  const T narrowed = Elem<T>::store(value);
  if (residual == nullptr) return narrowed;
  return Elem<T>::store(Elem<T>::load(narrowed) + Elem<T>::load(residual[index]));
}

// One 16-byte item of an indexed k-way sum: output[token, vector] = sum over routes, in route
// order, of rows[row_index[token * k + route], vector] (f32, one narrowing); routes with an
// index outside [0, row_count) are skipped.
template <typename T>
__device__ __forceinline__ void combine_rows_item(const T* __restrict__ rows,
                                                  const int32_t* __restrict__ row_index,
                                                  T* __restrict__ output, int64_t item,
                                                  int top_k, int vectors, int64_t row_count) {
  const int token = static_cast<int>(item / vectors);
  const int vector = static_cast<int>(item - static_cast<int64_t>(token) * vectors);
  float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int route = 0; route < top_k; ++route) {
    const int32_t index = row_index[static_cast<int64_t>(token) * top_k + route];
    if (index < 0 || index >= row_count) continue;
    const uint4 v =
        reinterpret_cast<const uint4*>(rows)[static_cast<int64_t>(index) * vectors + vector];
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sum[2 * i] += Elem<T>::from_bits(words[i] & 0xffffu);
      sum[2 * i + 1] += Elem<T>::from_bits(words[i] >> 16);
    }
  }
  uint4 out;
  out.x = Elem<T>::pack2(sum[0], sum[1]);
  out.y = Elem<T>::pack2(sum[2], sum[3]);
  out.z = Elem<T>::pack2(sum[4], sum[5]);
  out.w = Elem<T>::pack2(sum[6], sum[7]);
  reinterpret_cast<uint4*>(output)[item] = out;
}

// Clamped residual SwiGLU of the routed experts (crates/nml-kernel-nvfp4/src/lib.rs:424-429):
// gate clamps above 7, up clamps to [-7, 7], result (up + 1) * gate * sigmoid(1.702 * gate).
__device__ __forceinline__ float clamped_swiglu(float gate, float up) {
  gate = fminf(gate, 7.0f);
  up = fminf(fmaxf(up, -7.0f), 7.0f);
  const float swish = gate * (1.0f / (1.0f + expf(-1.702f * gate)));
  return (up + 1.0f) * swish;
}

// ---- launchers implemented in the kernel translation units --------------------
struct LinearArgs {
  const void* activation;
  const uint8_t* payload;
  const uint8_t* block_scales;
  const float* global_scale;
  const void* bias;
  void* output;
  cudaStream_t stream;
  int rows, outputs, inputs;
  int dtype;
  const void* residual = nullptr;  // [rows, outputs], added to the narrowed result
  void* workspace = nullptr;       // optional scratch of the caller
  size_t workspace_bytes = 0;
  // internal (the narrowed-operand form of the tcgen05 linear)
  const float* tile_scale = nullptr;  // factor of the f32 sums of every 256-row tile
  const uint32_t* gate = nullptr;     // the launch runs only if (*gate != 0) == gate_when
  int gate_when = 0;
  // Fused projections that share the activation (Q/K/V): further weights after the first.
  struct Projection {
    const uint8_t* payload;
    const uint8_t* block_scales;
    const float* global_scale;
    const void* bias;
    void* output;
    int outputs;
  };
  int extra_projections = 0;  // 0..2
  Projection extra[2] = {};
};

int32_t launch_linear_simt(const LinearArgs& args, const DeviceInfo& device, char* message,
                           size_t capacity);
// Returns true when the tcgen05 path supports this shape and alignment.
bool linear_umma_supported(const LinearArgs& args);
int32_t launch_linear_umma(const LinearArgs& args, const DeviceInfo& device, char* message,
                           size_t capacity);
// Scratch the tcgen05 linear can use (F16 copy of BF16 activations for wide weights), else 0.
size_t linear_umma_workspace_bytes(int64_t rows, int64_t outputs, int64_t inputs, int32_t dtype);
size_t linear_umma_workspace_verdict_offset(int64_t rows, int64_t inputs);
// The weight-streaming kernel: few activation rows, K a multiple of 64 up to 4096.
bool linear_stream_supported(const LinearArgs& args);
int32_t launch_linear_stream(const LinearArgs& args, const DeviceInfo& device, char* message,
                             size_t capacity);

struct EmbeddingArgs {
  const void* indices;
  const uint8_t* payload;
  const uint8_t* block_scales;
  const float* global_scale;
  void* output;
  cudaStream_t stream;
  int64_t rows;
  int vocabulary, width;
  int dtype;
  bool indices_are_i64;
};

int32_t launch_embedding(const EmbeddingArgs& args, const DeviceInfo& device, char* message,
                         size_t capacity);

struct ExpertArgs {
  const void* input;  // hidden [tokens, K] (gate/up) or activated [assignments, K] (down)
  const int32_t* sorted_assignments;
  const int32_t* block_experts;
  const uint8_t* payload;
  const uint8_t* block_scales;
  const float* global_scale;
  const void* bias;
  const void* routing_weights;  // down only
  void* output;                 // activated [A, I] or weighted [A, H]
  const int32_t* active_blocks; // may be null
  const int32_t* expert_offset; // may be null
  cudaStream_t stream;
  int assignments, schedule_blocks;
  int inputs;        // K: hidden (gate/up) or intermediate (down)
  int outputs;       // output columns: intermediate (gate/up) or hidden (down)
  int experts, experts_per_token;
  int dtype;
  bool gate_up;      // true: two weight rows per output column + SwiGLU; false: down
  // Orchestrated layer only: `input` holds one row per schedule slot (rows permuted into slot
  // order); gate/up then also writes its result rows in slot order.
  bool slot_input = false;
  // Routes expected to be live (kernel selection only); 0: all of `assignments`.
  int live_routes = 0;
  // Down only: where each assignment's result row goes instead of output + a * outputs (null
  // entries are skipped); null table: the plain layout.
  void* const* row_targets = nullptr;
};

int32_t launch_experts_simt(const ExpertArgs& args, const DeviceInfo& device, char* message,
                            size_t capacity);
bool experts_umma_supported(const ExpertArgs& args);
int32_t launch_experts_umma(const ExpertArgs& args, const DeviceInfo& device, char* message,
                            size_t capacity);
// The weight-streaming kernel for decode-size batches (at most 16 slots per expert on average).
bool experts_stream_supported(const ExpertArgs& args);
int32_t launch_experts_stream(const ExpertArgs& args, const DeviceInfo& device, char* message,
                              size_t capacity);

int32_t launch_ep_push_rows(const NmlSm100EpPushRows& request, const DeviceInfo& device,
                            char* message, size_t capacity);
int32_t launch_ep_receive_meta(const NmlSm100EpReceiveMeta& request, const DeviceInfo& device,
                               char* message, size_t capacity);
int32_t launch_ep_wait_returns(const NmlSm100EpWaitReturns& request, const DeviceInfo& device,
                               char* message, size_t capacity);
bool valid_exchange(const NmlSm100EpExchange& exchange);
int32_t launch_ep_return_rows(const NmlSm100EpReturnRows& request, const DeviceInfo& device,
                              char* message, size_t capacity);

int get_kernel_policy();
void note_linear_kernel(const char* name, int tile_rows);

}  // namespace nml_sm100
