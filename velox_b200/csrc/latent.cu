// Kernels around attention over a cached low-rank latent.
//
// The mixer caches, per token, one row [c | k_rot | 0-pad]: the normalised latent c (kv_rank
// values) and one rotated key part shared by all heads (rot_dim values).  A head's unrotated
// key is W_uk c and its value W_uv c, so with
//     q_abs[h] = W_uk[h]^T q_unrot[h]                       (kv_rank values per head)
// the score is  (q_abs[h] . c + q_rot[h] . k_rot) * scale, and the head's output is
//     W_uv[h] (sum_n p_n c_n).
// Attention itself is then multi-query attention whose single "KV head" is the cached row, with
// the same rows serving as keys and as values, and runs on the paged attention kernels.  This
// file has what comes before and after it:
//
//   latent_prepare_kernel   per token: RMS norm of the latent and interleaved-pair rotation of
//                           the shared key part, both written to the token's cache slot; the
//                           rotation of every head's q_rot into the query row [q_abs | q_rot | 0]
//   headwise_linear_kernel  out[t, h, :] = W[h] x[t, h, :] for every head, optionally times
//                           sigmoid(gate[t, h]): the absorption of W_uk into the queries and
//                           the expansion of the attention result by W_uv
//
// Rotation: dims 2i and 2i + 1 of the first 2 * rot_pairs dims are a pair (u, v) ->
// (u cos a - v sin a, v cos a + u sin a), a = position * base^(-2i / (2 rot_pairs)); cos and sin
// come from float32 tables [max_pos, rot_pairs].  Norm, rotation, sigmoid and all sums are
// float32.
#include "common.cuh"

namespace vx {

template <typename T>
__device__ __forceinline__ float rotated_interleaved(const T* __restrict__ x, int j, int rot_pairs,
                                                     const float* __restrict__ cos_row,
                                                     const float* __restrict__ sin_row) {
  if (j >= 2 * rot_pairs) return to_float(x[j]);
  const int i = j >> 1;
  const float u = to_float(x[2 * i]), v = to_float(x[2 * i + 1]);
  const float c = cos_row[i], s = sin_row[i];
  return (j & 1) ? fmaf(v, c, u * s) : fmaf(u, c, -(v * s));
}

// proj [T, proj_ld]: q head h at q_off + h * (dim + R), its last R dims rotate; the token's own
// latent (kr values, then R values of the shared key part) at dkv_off, or dkv_off < 0 for a layer
// that reads another layer's cache.  qa [T, H, Dp]: [kr absorbed dims (written elsewhere) | R
// rotated dims | zero pad].  cache [slots, Dp].
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, long long proj_ld, int q_off, int dkv_off,
                                      const int* __restrict__ positions, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int max_pos, int rot_pairs,
                                      const float* __restrict__ latent_w, float eps,
                                      const int* __restrict__ slots, T* __restrict__ cache, long long num_slots,
                                      T* __restrict__ qa, int H, int dim, int R, int kr, int Dp, int* status) {
  __shared__ float scratch[32];
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_POSITION);
    pos = 0;
  }
  const float* cos_row = cos_t + (size_t)pos * rot_pairs;
  const float* sin_row = sin_t + (size_t)pos * rot_pairs;
  const T* row = proj + (size_t)t * proj_ld;
  const int tail = Dp - kr;
  for (int idx = threadIdx.x; idx < H * tail; idx += blockDim.x) {
    const int h = idx / tail, j = idx - h * tail;
    float v = 0.f;
    if (j < R) v = rotated_interleaved(row + q_off + (size_t)h * (dim + R) + dim, j, rot_pairs, cos_row, sin_row);
    qa[((size_t)t * H + h) * Dp + kr + j] = from_float<T>(v);
  }
  if (dkv_off < 0) return;
  const T* lat = row + dkv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < kr; i += blockDim.x) {
    const float v = to_float(lat[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const long long slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, VX_STATUS_BAD_SLOT);
    return;
  }
  const float inv = 1.0f / sqrtf(ss / (float)kr + eps);
  T* dst = cache + (size_t)slot * Dp;
  for (int i = threadIdx.x; i < Dp; i += blockDim.x) {
    float v = 0.f;
    if (i < kr) v = to_float(lat[i]) * inv * latent_w[i];
    else if (i < kr + R) v = rotated_interleaved(lat + kr, i - kr, rot_pairs, cos_row, sin_row);
    dst[i] = from_float<T>(v);
  }
}

// out[t * out_ld + h * out_hs + n] = sum_k x[t * x_ld + h * x_hs + k] * w[(h * N + n) * K + k]
//                                    (* sigmoid(gate[t * gate_ld + h]) with a gate)
// One block per (tile of HL_TOKENS tokens, head); the tile's inputs are staged in shared memory
// as float32, a warp takes output n and its lanes split k, so a weight row is read once per
// block, coalesced.  Every output is summed in an order that depends on K only.
constexpr int HL_TOKENS = 8;

template <typename T>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const T* __restrict__ x, long long x_ld, int x_hs, const T* __restrict__ w,
                       T* __restrict__ out, long long out_ld, int out_hs, const T* __restrict__ gate,
                       long long gate_ld, int num_tokens, int N, int K) {
  extern __shared__ float xs[];  // [HL_TOKENS][K]
  allow_dependents();
  grid_dependency_wait();
  const int t0 = blockIdx.x * HL_TOKENS, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, num_warps = blockDim.x >> 5;
  for (int idx = threadIdx.x; idx < HL_TOKENS * K; idx += blockDim.x) {
    const int r = idx / K, k = idx - r * K;
    const int t = t0 + r;
    xs[idx] = t < num_tokens ? to_float(x[(size_t)t * x_ld + (size_t)h * x_hs + k]) : 0.f;
  }
  __syncthreads();
  float g[HL_TOKENS];
#pragma unroll
  for (int r = 0; r < HL_TOKENS; ++r) {
    const int t = t0 + r;
    g[r] = (gate != nullptr && t < num_tokens) ? 1.0f / (1.0f + expf(-to_float(gate[(size_t)t * gate_ld + h]))) : 1.0f;
  }
  for (int n = warp; n < N; n += num_warps) {
    const T* wr = w + ((size_t)h * N + n) * K;
    float acc[HL_TOKENS];
#pragma unroll
    for (int r = 0; r < HL_TOKENS; ++r) acc[r] = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float wv = to_float(wr[k]);
#pragma unroll
      for (int r = 0; r < HL_TOKENS; ++r) acc[r] = fmaf(xs[r * K + k], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < HL_TOKENS; ++r) acc[r] = warp_sum(acc[r]);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < HL_TOKENS; ++r) {
        const int t = t0 + r;
        if (t < num_tokens) out[(size_t)t * out_ld + (size_t)h * out_hs + n] = from_float<T>(acc[r] * g[r]);
      }
    }
  }
}

}  // namespace vx

using namespace vx;

VX_API int vx_latent_prepare(const void* proj, long long proj_ld, int q_off, int dkv_off, int dtype,
                             const int* positions, const float* cos_t, const float* sin_t, int max_pos,
                             int rot_pairs, const float* latent_w, float eps, const int* slots, void* cache,
                             long long num_slots, void* qa, int num_tokens, int H, int dim, int R, int kr, int Dp,
                             int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || dim < 0 || R < 0 || kr <= 0 || Dp < kr + R || 2 * rot_pairs > R) return (int)cudaErrorInvalidValue;
  if (dkv_off >= 0 && (cache == nullptr || slots == nullptr || latent_w == nullptr)) return (int)cudaErrorInvalidValue;
  const int threads = 128;
  if (dtype == VX_DTYPE_F32)
    launch_pdl(latent_prepare_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)proj, proj_ld,
               q_off, dkv_off, positions, cos_t, sin_t, max_pos, rot_pairs, latent_w, eps, slots, (float*)cache,
               num_slots, (float*)qa, H, dim, R, kr, Dp, status);
  else
    launch_pdl(latent_prepare_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream,
               (const __nv_bfloat16*)proj, proj_ld, q_off, dkv_off, positions, cos_t, sin_t, max_pos, rot_pairs,
               latent_w, eps, slots, (__nv_bfloat16*)cache, num_slots, (__nv_bfloat16*)qa, H, dim, R, kr, Dp, status);
  return (int)cudaGetLastError();
}

VX_API int vx_headwise_linear(const void* x, long long x_ld, int x_hs, const void* w, void* out, long long out_ld,
                              int out_hs, const void* gate, long long gate_ld, int dtype, int num_tokens, int H,
                              int N, int K, cudaStream_t stream) {
  if (num_tokens <= 0 || H <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * HL_TOKENS * (size_t)K;
  if (smem > 96 * 1024) return -1;
  const dim3 grid((num_tokens + HL_TOKENS - 1) / HL_TOKENS, H);
  if (dtype == VX_DTYPE_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(headwise_linear_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(headwise_linear_kernel<float>, grid, dim3(256), smem, stream, (const float*)x, x_ld, x_hs,
               (const float*)w, (float*)out, out_ld, out_hs, (const float*)gate, gate_ld, num_tokens, N, K);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(headwise_linear_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem);
    launch_pdl(headwise_linear_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)x, x_ld,
               x_hs, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_ld, out_hs, (const __nv_bfloat16*)gate,
               gate_ld, num_tokens, N, K);
  }
  return (int)cudaGetLastError();
}
