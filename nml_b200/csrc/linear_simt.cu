// Portable SIMT NVFP4 linear: correct for every shape and alignment (odd K, K not a
// multiple of 16, any N, any M).  It is the path for shapes the tcgen05 kernel does not
// take; it is not tuned for bandwidth.
//
// One warp owns one weight row n and up to kRowsPerPass activation rows at a time; lanes
// stride over 16-value blocks of K, decode the block once (value * fl(scale * global), the
// reference CPU association, crates/nml-kernel-nvfp4/src/lib.rs:193-200) and accumulate in
// f32; a shuffle tree finishes the dot products and lane 0 adds the bias and narrows.
#include "common.cuh"

namespace nml_sm100 {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kRowsPerPass = 8;

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
linear_simt_kernel(const T* __restrict__ activation, const uint8_t* __restrict__ payload,
                   const uint8_t* __restrict__ block_scales,
                   const float* __restrict__ global_scale, const T* __restrict__ bias,
                   const T* residual, T* output, int rows, int outputs, int inputs) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t n = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp;
  if (n >= outputs) return;
  const int packed_width = (inputs + 1) / 2;
  const int scale_width = (inputs + 15) / 16;
  const float g = global_scale[0];
  const uint8_t* row_payload = payload + n * packed_width;
  const uint8_t* row_scales = block_scales + n * scale_width;
  const float bias_value = bias == nullptr ? 0.0f : Elem<T>::load(bias[n]);

  for (int row_base = 0; row_base < rows; row_base += kRowsPerPass) {
    float acc[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) acc[r] = 0.0f;
    for (int block = lane; block < scale_width; block += 32) {
      const int start = block * 16;
      const int count = min(16, inputs - start);
      const float effective = __fmul_rn(e4m3_scale_to_f32(row_scales[block]), g);
      float w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float value = 0.0f;
        if (i < count) {
          const uint32_t byte = row_payload[(start + i) >> 1];
          const uint32_t code = ((start + i) & 1) ? (byte >> 4) : (byte & 0xfu);
          value = __fmul_rn(e2m1_to_f32(code), effective);
        }
        w[i] = value;
      }
#pragma unroll
      for (int r = 0; r < kRowsPerPass; ++r) {
        const int row = row_base + r;
        if (row < rows) {
          const T* x = activation + static_cast<int64_t>(row) * inputs + start;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (i < count) acc[r] = fmaf(Elem<T>::load(x[i]), w[i], acc[r]);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) {
      float sum = acc[r];
#pragma unroll
      for (int offset = 16; offset != 0; offset >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      }
      const int row = row_base + r;
      if (lane == 0 && row < rows) {
        const int64_t index = static_cast<int64_t>(row) * outputs + n;
        output[index] = narrow_with_residual<T>(sum + bias_value, residual, index);
      }
    }
  }
}

}  // namespace

int32_t launch_linear_simt(const LinearArgs& args, const DeviceInfo&, char* message,
                           size_t capacity) {
  const unsigned grid = static_cast<unsigned>((args.outputs + kWarpsPerBlock - 1) /
                                              kWarpsPerBlock);
  if (args.dtype == NML_SM100_F16) {
    linear_simt_kernel<__half><<<grid, kWarpsPerBlock * 32, 0, args.stream>>>(
        static_cast<const __half*>(args.activation), args.payload, args.block_scales,
        args.global_scale, static_cast<const __half*>(args.bias),
        static_cast<const __half*>(args.residual), static_cast<__half*>(args.output), args.rows,
        args.outputs, args.inputs);
  } else {
    linear_simt_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, args.stream>>>(
        static_cast<const __nv_bfloat16*>(args.activation), args.payload, args.block_scales,
        args.global_scale, static_cast<const __nv_bfloat16*>(args.bias),
        static_cast<const __nv_bfloat16*>(args.residual),
        static_cast<__nv_bfloat16*>(args.output), args.rows, args.outputs, args.inputs);
  }
  note_linear_kernel("simt", 0);
  return launch_result(message, capacity);
}

}  // namespace nml_sm100
