// Feed-forward layers whose experts are chosen per token from a table indexed by the token id.
//
//   table_experts_kernel   one block per token: for each of the token's `top` experts,
//                          act = relu(W_up[e] h)^2 and sum += W_down[e] act, the sum over the
//                          experts divided by `top` and added to the float32 residual stream.
//                          The experts' matrices are stacked: up [experts * ff, width],
//                          down [experts * width, ff].
//
// A token id of -1 - r stands for row r of `fed` (the tokens drawn in the step before), as for
// the embedding.  Products are float32 sums of products of the stored operands, in an order that
// depends on the sizes only.
#include "common.cuh"

namespace vx {

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ v, int n, int lane);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ w, const float* __restrict__ v, int n,
                                                int lane) {
  float acc = 0.f;
  for (int i = lane; i < n; i += 32) acc = fmaf(w[i], v[i], acc);
  return warp_sum(acc);
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w,
                                                        const float* __restrict__ v, int n, int lane) {
  float acc = 0.f;
  if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(pairs[k]);
        acc = fmaf(f.x, v[i + 2 * k], acc);
        acc = fmaf(f.y, v[i + 2 * k + 1], acc);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) acc = fmaf(__bfloat162float(w[i]), v[i], acc);
  }
  return warp_sum(acc);
}

template <typename T>
__global__ void table_experts_kernel(const T* __restrict__ h, long long h_stride, const int* __restrict__ ids,
                                     const int* __restrict__ fed, int num_fed, const int* __restrict__ table,
                                     int vocab, int top, int experts, const T* __restrict__ w_up,
                                     const T* __restrict__ w_down, int width, int ff, float* __restrict__ resid,
                                     int* status) {
  extern __shared__ float moe_s[];
  float* h_s = moe_s;           // [width]
  float* act_s = h_s + width;   // [ff]
  float* sum_s = act_s + ff;    // [width]
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  int id = ids[t];
  if (id < 0 && fed != nullptr && -1 - id < num_fed) id = fed[-1 - id];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_TOKEN_ID);
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    h_s[i] = to_float(h[(size_t)t * h_stride + i]);
    sum_s[i] = 0.f;
  }
  for (int k = 0; k < top; ++k) {
    const int e = table[(size_t)id * top + k];
    if (e < 0 || e >= experts) {
      if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_TOKEN_ID);
      continue;
    }
    __syncthreads();
    const T* up = w_up + (size_t)e * ff * width;
    for (int j = warp; j < ff; j += warps) {
      const float v = dot_row<T>(up + (size_t)j * width, h_s, width, lane);
      if (lane == 0) {
        const float r = fmaxf(v, 0.f);
        act_s[j] = r * r;
      }
    }
    __syncthreads();
    const T* down = w_down + (size_t)e * width * ff;
    for (int o = warp; o < width; o += warps) {
      const float v = dot_row<T>(down + (size_t)o * ff, act_s, ff, lane);
      if (lane == 0) sum_s[o] += v;
    }
  }
  __syncthreads();
  const float scale = 1.0f / (float)top;
  for (int i = threadIdx.x; i < width; i += blockDim.x) resid[(size_t)t * width + i] += sum_s[i] * scale;
}

}  // namespace vx

using namespace vx;

VX_API int vx_table_experts(const void* h, int dtype, long long h_stride, const int* ids, const int* fed,
                            int num_fed, const int* table, int vocab, int top, int experts, const void* w_up,
                            const void* w_down, int width, int ff, float* resid, int num_tokens, int* status,
                            cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const size_t smem = sizeof(float) * ((size_t)2 * width + ff);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == VX_DTYPE_F32) {
    static size_t configured = 48 * 1024;
    if (smem > configured) {
      cudaError_t e = cudaFuncSetAttribute(table_experts_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = smem;
    }
    launch_pdl(table_experts_kernel<float>, dim3(num_tokens), dim3(256), smem, stream, (const float*)h, h_stride, ids,
               fed, num_fed, table, vocab, top, experts, (const float*)w_up, (const float*)w_down, width, ff, resid,
               status);
  } else {
    static size_t configured = 48 * 1024;
    if (smem > configured) {
      cudaError_t e = cudaFuncSetAttribute(table_experts_kernel<__nv_bfloat16>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      configured = smem;
    }
    launch_pdl(table_experts_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(256), smem, stream,
               (const __nv_bfloat16*)h, h_stride, ids, fed, num_fed, table, vocab, top, experts,
               (const __nv_bfloat16*)w_up, (const __nv_bfloat16*)w_down, width, ff, resid, status);
  }
  return (int)cudaGetLastError();
}
