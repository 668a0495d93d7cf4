// Packed NVFP4 embedding gather + decode.
//
// out[r, c] = narrow(e2m1(code) * fl(e4m3(scale) * global)) for row indices[r]:
// the association of the reference CPU path (crates/nml-kernel-nvfp4/src/lib.rs:193-200,
// x86.rs:48-53), evaluated with explicitly rounded f32 multiplies so the result is
// bit-identical to it.  Pure HBM traffic: per gathered row K/2 payload bytes, K/16
// scale bytes and 2K output bytes.
#include "common.cuh"

namespace nml_sm100 {
namespace {

// One thread decodes one 16-value block: one 8-byte payload load, one scale byte,
// two 16-byte stores.  Requires width % 16 == 0 and aligned bases.
template <typename Index, typename T>
__global__ void __launch_bounds__(256)
embedding_block_kernel(const Index* __restrict__ indices, const uint8_t* __restrict__ payload,
                       const uint8_t* __restrict__ block_scales,
                       const float* __restrict__ global_scale, T* __restrict__ output,
                       int64_t rows, int vocabulary, int blocks_per_row, int* status) {
  const int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= rows * blocks_per_row) return;
  const int64_t row = item / blocks_per_row;
  const int block = static_cast<int>(item - row * blocks_per_row);
  const int64_t token = static_cast<int64_t>(indices[row]);
  uint4* destination =
      reinterpret_cast<uint4*>(output + (row * blocks_per_row + block) * 16);
  if (token < 0 || token >= vocabulary) {
    // Indices live in device memory, so the host cannot reject them; the row
    // reads as zeros and the status word records the event.
    destination[0] = make_uint4(0, 0, 0, 0);
    destination[1] = make_uint4(0, 0, 0, 0);
    if (block == 0) atomicOr(status, NML_SM100_STATUS_INDEX_RANGE);
    return;
  }
  const uint2 packed = __ldg(reinterpret_cast<const uint2*>(
      payload + (token * blocks_per_row + block) * 8));
  const float effective = __fmul_rn(
      e4m3_scale_to_f32(__ldg(block_scales + token * blocks_per_row + block)),
      __ldg(global_scale));
  uint32_t words[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t source = i < 4 ? packed.x : packed.y;
    const uint32_t byte = (source >> ((i & 3) * 8)) & 0xffu;
    const float lo = __fmul_rn(e2m1_to_f32(byte & 0xfu), effective);
    const float hi = __fmul_rn(e2m1_to_f32(byte >> 4), effective);
    words[i] = Elem<T>::pack2(lo, hi);
  }
  destination[0] = make_uint4(words[0], words[1], words[2], words[3]);
  destination[1] = make_uint4(words[4], words[5], words[6], words[7]);
}

// Any width, any alignment: one thread per output element.
template <typename Index, typename T>
__global__ void __launch_bounds__(256)
embedding_element_kernel(const Index* __restrict__ indices, const uint8_t* __restrict__ payload,
                         const uint8_t* __restrict__ block_scales,
                         const float* __restrict__ global_scale, T* __restrict__ output,
                         int64_t rows, int vocabulary, int width, int* status) {
  const int64_t element = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (element >= rows * width) return;
  const int64_t row = element / width;
  const int column = static_cast<int>(element - row * width);
  const int64_t token = static_cast<int64_t>(indices[row]);
  if (token < 0 || token >= vocabulary) {
    output[element] = Elem<T>::store(0.0f);
    if (column == 0) atomicOr(status, NML_SM100_STATUS_INDEX_RANGE);
    return;
  }
  const int packed_width = (width + 1) / 2;
  const int scale_width = (width + 15) / 16;
  const uint32_t byte = payload[token * packed_width + column / 2];
  const uint32_t code = (column & 1) ? (byte >> 4) : (byte & 0xfu);
  const float effective = __fmul_rn(
      e4m3_scale_to_f32(block_scales[token * scale_width + column / 16]), global_scale[0]);
  output[element] = Elem<T>::store(__fmul_rn(e2m1_to_f32(code), effective));
}

template <typename Index, typename T>
int32_t launch_typed(const EmbeddingArgs& args, const DeviceInfo& device, char* message,
                     size_t capacity) {
  const bool vector_ok = args.width % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(args.payload) % 8 == 0 &&
                         reinterpret_cast<uintptr_t>(args.output) % 16 == 0;
  if (vector_ok) {
    const int blocks_per_row = args.width / 16;
    const int64_t items = args.rows * blocks_per_row;
    const int64_t grid = (items + 255) / 256;
    if (grid > std::numeric_limits<int32_t>::max()) {
      return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 embedding launch extent overflows",
                  message, capacity);
    }
    embedding_block_kernel<Index, T><<<static_cast<unsigned>(grid), 256, 0, args.stream>>>(
        static_cast<const Index*>(args.indices), args.payload, args.block_scales,
        args.global_scale, static_cast<T*>(args.output), args.rows, args.vocabulary,
        blocks_per_row, device.status_word);
  } else {
    const int64_t extent = args.rows * args.width;
    const int64_t grid = (extent + 255) / 256;
    if (grid > std::numeric_limits<int32_t>::max()) {
      return fail(NML_SM100_INVALID_ARGUMENT, "NVFP4 embedding launch extent overflows",
                  message, capacity);
    }
    embedding_element_kernel<Index, T><<<static_cast<unsigned>(grid), 256, 0, args.stream>>>(
        static_cast<const Index*>(args.indices), args.payload, args.block_scales,
        args.global_scale, static_cast<T*>(args.output), args.rows, args.vocabulary, args.width,
        device.status_word);
  }
  return launch_result(message, capacity);
}

}  // namespace

int32_t launch_embedding(const EmbeddingArgs& args, const DeviceInfo& device, char* message,
                         size_t capacity) {
  if (args.dtype == NML_SM100_F16) {
    return args.indices_are_i64
               ? launch_typed<int64_t, __half>(args, device, message, capacity)
               : launch_typed<int32_t, __half>(args, device, message, capacity);
  }
  return args.indices_are_i64
             ? launch_typed<int64_t, __nv_bfloat16>(args, device, message, capacity)
             : launch_typed<int32_t, __nv_bfloat16>(args, device, message, capacity);
}

}  // namespace nml_sm100
