// Shared device/host helpers for the qengine_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace qb {

using bf16 = __nv_bfloat16;

// ---- bf16 helpers -----------------------------------------------------------------------------
__device__ __forceinline__ float tofloat(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 tobf16(float v) { return __float2bfloat16_rn(v); }
// One torch bf16 op: round an fp32 intermediate to bf16 (nearest even) and widen again.
__device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// 8 bf16 packed in a uint4 -> 8 floats (bf16 -> fp32 is a 16-bit shift).
__device__ __forceinline__ void widen8(const uint4& p, float (&f)[8]) {
  const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint4 narrow8(const float (&f)[8]) {
  return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}
// eight floats -> eight fp16 (round to nearest), one 16-byte packet
__device__ __forceinline__ uint4 half8(const float (&f)[8]) {
  const __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]);
  const __half2 c = __floats2half2_rn(f[4], f[5]), d = __floats2half2_rn(f[6], f[7]);
  return make_uint4(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b),
                    *reinterpret_cast<const uint32_t*>(&c), *reinterpret_cast<const uint32_t*>(&d));
}

// torch-accurate activations (expf, not the fast intrinsic).
__device__ __forceinline__ float silu_acc(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float sigmoid_acc(float v) { return 1.0f / (1.0f + expf(-v)); }

// ---- reductions ---------------------------------------------------------------------------------
__device__ __forceinline__ float warp_allsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Block-wide sum, every thread gets the result. `scratch` holds >= 32 floats. The order of the
// additions is fixed by the thread layout, so the result is reproducible run to run.
__device__ __forceinline__ float block_allsum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_allsum(v);
  __syncthreads();
  if (lane == 0) scratch[w] = v;
  __syncthreads();
  float t = lane < nw ? scratch[lane] : 0.f;
  return warp_allsum(t);
}

// ---- programmatic dependent launch ------------------------------------------------------------
// Producer side: let the next kernel of the stream start its prologue (it still waits in
// dep_wait() for this whole grid to finish before touching anything this grid writes).
__device__ __forceinline__ void dep_release() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Consumer side: block until the preceding grid has completed and its writes are visible.
// A no-op for a kernel launched without the programmatic-serialization attribute.
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Host-side switches shared by every translation unit (defined in capi.cu).
bool& pdl_launch_enabled();
int pdl_trigger_enabled();

// Launch helper: optional programmatic stream serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t s, bool pdl, Args... args) {
  cudaLaunchConfig_t c = {};
  c.gridDim = grid;
  c.blockDim = block;
  c.dynamicSmemBytes = smem;
  c.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  c.attrs = at;
  c.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&c, kern, static_cast<KArgs>(args)...);
}

}  // namespace qb
