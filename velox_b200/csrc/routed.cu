// Feed-forward layers whose experts are chosen per token from a table indexed by the token id.
//
//   table_experts_kernel   one block per token: for each of the token's `top` experts,
//                          act = relu(W_up[e] h)^2 and sum += W_down[e] act, the sum over the
//                          experts divided by `top` and added to the float32 residual stream.
//                          The experts' matrices are stacked: up [experts * ff, width],
//                          down [experts * width, ff].  (The plain form: any size.)
//   expert_up_rows_kernel, expert_down_rows_kernel
//                          the same as matrix-vector products spread over the grid (small steps
//                          and the float32 path)
//   route_pairs_kernel, grouped_gemm_kernel, gather_pairs_kernel
//                          the same as tiled tensor-core products over the pairs ordered by
//                          expert (long bfloat16 steps)
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
  if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(v) & 15) == 0) {
    // Four 16-byte loads of a lane are under way before the first is used.
    for (int i0 = lane * 8; i0 < n; i0 += 1024) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * 256;
        raw[u] = i < n ? __ldg(reinterpret_cast<const uint4*>(w + i)) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * 256;
        if (i < n) {
          const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
          const float4 v0 = *reinterpret_cast<const float4*>(v + i), v1 = *reinterpret_cast<const float4*>(v + i + 4);
          const float2 f0 = __bfloat1622float2(pairs[0]), f1 = __bfloat1622float2(pairs[1]);
          const float2 f2 = __bfloat1622float2(pairs[2]), f3 = __bfloat1622float2(pairs[3]);
          acc = fmaf(f0.x, v0.x, acc); acc = fmaf(f0.y, v0.y, acc);
          acc = fmaf(f1.x, v0.z, acc); acc = fmaf(f1.y, v0.w, acc);
          acc = fmaf(f2.x, v1.x, acc); acc = fmaf(f2.y, v1.y, acc);
          acc = fmaf(f3.x, v1.z, acc); acc = fmaf(f3.y, v1.w, acc);
        }
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
  extern __shared__ __align__(16) float moe_s[];
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


// ---------------------------------------------------------------------------------------------
// Small steps: the two projections of every (token, expert) pair as matrix-vector products
// spread over the grid.  act [tokens, top, ff] float32.
template <typename T>
__global__ void expert_up_rows_kernel(const T* __restrict__ h, long long h_stride, const int* __restrict__ ids,
                                      const int* __restrict__ fed, int num_fed, const int* __restrict__ table,
                                      int vocab, int top, int experts, const T* __restrict__ w_up, int width, int ff,
                                      int rows_per_block, float* __restrict__ act, int* status) {
  extern __shared__ __align__(16) float moe_s[];  // [width]
  allow_dependents();
  grid_dependency_wait();
  const int pair = blockIdx.y, t = pair / top, k = pair - t * top;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  int id = ids[t];
  if (id < 0 && fed != nullptr && -1 - id < num_fed) id = fed[-1 - id];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, VX_STATUS_BAD_TOKEN_ID);
    return;
  }
  const int e = table[(size_t)id * top + k];
  if (e < 0 || e >= experts) {
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, VX_STATUS_BAD_TOKEN_ID);
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) moe_s[i] = to_float(h[(size_t)t * h_stride + i]);
  __syncthreads();
  const T* up = w_up + (size_t)e * ff * width;
  const int j0 = blockIdx.x * rows_per_block;
  for (int j = j0 + warp; j < min(ff, j0 + rows_per_block); j += warps) {
    const float v = dot_row<T>(up + (size_t)j * width, moe_s, width, lane);
    if (lane == 0) {
      const float r = fmaxf(v, 0.f);
      act[(size_t)pair * ff + j] = r * r;
    }
  }
}

template <typename T>
__global__ void expert_down_rows_kernel(const float* __restrict__ act, const int* __restrict__ ids,
                                        const int* __restrict__ fed, int num_fed, const int* __restrict__ table,
                                        int vocab, int top, int experts, const T* __restrict__ w_down, int width,
                                        int ff, int rows_per_block, float* __restrict__ resid) {
  extern __shared__ __align__(16) float moe_s[];  // [top][ff]
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  int id = ids[t];
  if (id < 0 && fed != nullptr && -1 - id < num_fed) id = fed[-1 - id];
  if (id < 0 || id >= vocab) return;
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) moe_s[i] = act[(size_t)t * top * ff + i];
  __syncthreads();
  const int o0 = blockIdx.x * rows_per_block;
  const float scale = 1.0f / (float)top;
  for (int o = o0 + warp; o < min(width, o0 + rows_per_block); o += warps) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = table[(size_t)id * top + k];
      if (e < 0 || e >= experts) continue;
      sum += dot_row<T>(w_down + ((size_t)e * width + o) * ff, moe_s + (size_t)k * ff, ff, lane);
    }
    if (lane == 0) resid[(size_t)t * width + o] += sum * scale;
  }
}

// ---------------------------------------------------------------------------------------------
// Long steps (bfloat16): the (token, expert) pairs are ordered by expert, every expert's run
// padded to whole tiles of GG_M rows, and the two projections run as tiled tensor-core products
// whose tiles each belong to one expert.
//
//   route_pairs_kernel    one block: counts per expert, the runs' (padded) starts, for every tile
//                         its expert, for every place its token (-1: padding), for every pair
//                         its place
//   grouped_gemm_kernel   out[place, n] = sum_k A[row(place), k] * W[expert(tile)][n, k]; the rows
//                         of A are gathered by token (up) or are the places themselves (down);
//                         the up form squares the positive part and writes bfloat16
//   gather_pairs_kernel   resid[t] += (sum over the token's pairs, in their order) / top
constexpr int GG_M = 64, GG_N = 128, GG_K = 64, GG_LD = GG_K + 8, GG_STAGES = 2;
constexpr int GG_STAGE_ELEMS = (GG_M + GG_N) * GG_LD;
constexpr size_t GG_SMEM_BYTES = (size_t)GG_STAGES * GG_STAGE_ELEMS * sizeof(__nv_bfloat16);

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;  // 0: the sixteen bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int LEFT>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(LEFT) : "memory"); }

__global__ void route_pairs_kernel(const int* __restrict__ ids, const int* __restrict__ fed, int num_fed,
                                   const int* __restrict__ table, int vocab, int top, int experts, int num_tokens,
                                   int capacity, int max_tiles, int* __restrict__ tile_expert,
                                   int* __restrict__ place_token, int* __restrict__ pair_place, int* status,
                                   int* __restrict__ run_ends) {
  extern __shared__ int route_s[];  // counts [experts], starts [experts], cursor [experts]
  int* counts = route_s;
  int* starts = counts + experts;
  int* cursor = starts + experts;
  allow_dependents();
  grid_dependency_wait();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
  for (int i = threadIdx.x; i < capacity; i += blockDim.x) place_token[i] = -1;
  for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
  __syncthreads();
  const int pairs = num_tokens * top;
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int t = p / top;
    int id = ids[t];
    if (id < 0 && fed != nullptr && -1 - id < num_fed) id = fed[-1 - id];
    int e = -1;
    if (id >= 0 && id < vocab) e = table[(size_t)id * top + (p - t * top)];
    if (e < 0 || e >= experts) {
      atomicOr(status, VX_STATUS_BAD_TOKEN_ID);
      continue;
    }
    atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      starts[e] = at;
      const int tiles = (counts[e] + GG_M - 1) / GG_M;
      for (int i = 0; i < tiles; ++i) tile_expert[at / GG_M + i] = e;
      at += tiles * GG_M;
      if (run_ends != nullptr) run_ends[e] = at;  // where the expert's (padded) run ends
    }
  }
  __syncthreads();
  // Which place of its expert's run a pair gets depends on the timing; its result does not (a
  // product's rows are independent of one another, and a token's pairs are summed in their order).
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) pair_place[p] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int t = p / top;
    int id = ids[t];
    if (id < 0 && fed != nullptr && -1 - id < num_fed) id = fed[-1 - id];
    if (id < 0 || id >= vocab) continue;
    const int e = table[(size_t)id * top + (p - t * top)];
    if (e < 0 || e >= experts) continue;
    const int place = starts[e] + atomicAdd(&cursor[e], 1);
    place_token[place] = t;
    pair_place[p] = place;
  }
}

// A block of four warps (two by two) makes a tile of GG_M places by GG_N outputs; a warp's share is
// 32 x 64.  Slabs of GG_K inner values of both operands come into shared memory by asynchronous
// 16-byte copies, the next slab while this one is multiplied (two stages).
template <bool UP>
__global__ void __launch_bounds__(128) grouped_gemm_kernel(
    const __nv_bfloat16* __restrict__ a, long long a_stride, const int* __restrict__ place_token,
    const int* __restrict__ tile_expert, const __nv_bfloat16* __restrict__ w, int N, int K,
    __nv_bfloat16* __restrict__ out_lowp, float* __restrict__ out_f32, long long out_stride) {
  extern __shared__ __align__(16) __nv_bfloat16 gg_s[];
  __shared__ int row_of[GG_M];
  allow_dependents();
  grid_dependency_wait();
  const int tile = blockIdx.x;
  const int e = tile_expert[tile];
  if (e < 0) return;
  const int n0 = blockIdx.y * GG_N;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;
  if (tid < GG_M) {
    const int place = tile * GG_M + tid;
    const int token = place_token[place];
    row_of[tid] = token < 0 ? -1 : (UP ? token : place);
  }
  __syncthreads();
  const __nv_bfloat16* wb = w + (size_t)e * N * K;
  float acc[2][8][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m][j][i] = 0.f;
  // Rows of a slab are eight 16-byte chunks; a thread copies chunk tid % 8 of rows tid / 8 + 16 u.
  const int chunk = (tid & 7) * 8, row0 = tid >> 3;
  auto fetch = [&](int k0, int stage) {
    __nv_bfloat16* a_s = gg_s + stage * GG_STAGE_ELEMS;
    __nv_bfloat16* b_s = a_s + GG_M * GG_LD;
    const bool k_ok = k0 + chunk < K;
#pragma unroll
    for (int u = 0; u < GG_M / 16; ++u) {
      const int r = row0 + 16 * u;
      const int row = row_of[r];
      const bool ok = k_ok && row >= 0;
      cp_async_16(a_s + r * GG_LD + chunk, ok ? a + (size_t)row * a_stride + k0 + chunk : a, ok);
    }
#pragma unroll
    for (int u = 0; u < GG_N / 16; ++u) {
      const int r = row0 + 16 * u;
      const bool ok = k_ok && n0 + r < N;
      cp_async_16(b_s + r * GG_LD + chunk, ok ? wb + (size_t)(n0 + r) * K + k0 + chunk : wb, ok);
    }
    cp_async_commit();
  };
  const int slabs = (K + GG_K - 1) / GG_K;
  fetch(0, 0);
  for (int slab = 0; slab < slabs; ++slab) {
    const int stage = slab & 1;
    if (slab + 1 < slabs) {
      fetch((slab + 1) * GG_K, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const __nv_bfloat16* a_s = gg_s + stage * GG_STAGE_ELEMS;
    const __nv_bfloat16* b_s = a_s + GG_M * GG_LD;
#pragma unroll
    for (int kk = 0; kk < GG_K; kk += 16) {
      uint32_t fa[2][4];
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const __nv_bfloat16* p = a_s + (wm * 32 + m * 16 + (lane & 15)) * GG_LD + kk + (lane >> 4) * 8;
        const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(fa[m][0]), "=r"(fa[m][1]), "=r"(fa[m][2]), "=r"(fa[m][3]) : "r"(addr));
      }
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t fb[4];
        const __nv_bfloat16* p = b_s + (wn * 64 + j * 8 + (lane & 7) + ((lane >> 4) << 3)) * GG_LD + kk + ((lane >> 3) & 1) * 8;
        const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(fb[0]), "=r"(fb[1]), "=r"(fb[2]), "=r"(fb[3]) : "r"(addr));
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                       : "+f"(acc[m][j][0]), "+f"(acc[m][j][1]), "+f"(acc[m][j][2]), "+f"(acc[m][j][3])
                       : "r"(fa[m][0]), "r"(fa[m][1]), "r"(fa[m][2]), "r"(fa[m][3]), "r"(fb[0]), "r"(fb[1]));
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                       : "+f"(acc[m][j + 1][0]), "+f"(acc[m][j + 1][1]), "+f"(acc[m][j + 1][2]), "+f"(acc[m][j + 1][3])
                       : "r"(fa[m][0]), "r"(fa[m][1]), "r"(fa[m][2]), "r"(fa[m][3]), "r"(fb[2]), "r"(fb[3]));
        }
      }
    }
    __syncthreads();  // the stage may be overwritten by the copy after next
  }
  // A thread holds rows g and g + 8 of each of its two sixteens, columns 2 * (lane % 4) + {0, 1} of every n8.
  const int g = lane >> 2, c2 = 2 * (lane & 3);
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + m * 16 + g + 8 * half;
      if (row_of[r] < 0) continue;
      const size_t place = (size_t)tile * GG_M + r;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int n = n0 + wn * 64 + j * 8 + c2;
        float v0 = acc[m][j][2 * half], v1 = acc[m][j][2 * half + 1];
        if (UP) {
          v0 = fmaxf(v0, 0.f); v0 *= v0;
          v1 = fmaxf(v1, 0.f); v1 *= v1;
          if (n + 1 < N) *reinterpret_cast<__nv_bfloat162*>(out_lowp + place * out_stride + n) = __floats2bfloat162_rn(v0, v1);
          else if (n < N) out_lowp[place * out_stride + n] = __float2bfloat16_rn(v0);
        } else {
          if (n + 1 < N) *reinterpret_cast<float2*>(out_f32 + place * out_stride + n) = make_float2(v0, v1);
          else if (n < N) out_f32[place * out_stride + n] = v0;
        }
      }
    }
}

// rows[place, :] = h[token of the place, :], zeros for padding places (16-byte chunks).
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ h, long long h_stride,
                                   const int* __restrict__ place_token, int chunks, long long total,
                                   __nv_bfloat16* __restrict__ rows) {
  allow_dependents();
  grid_dependency_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long place = idx / chunks;
    const int c = (int)(idx - place * chunks) * 8;
    const int token = place_token[place];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (token >= 0) v = *reinterpret_cast<const uint4*>(h + (size_t)token * h_stride + c);
    *reinterpret_cast<uint4*>(rows + (size_t)place * chunks * 8 + c) = v;
  }
}

template <typename R>
__global__ void gather_pairs_kernel(const R* __restrict__ rows, long long row_stride,
                                    const int* __restrict__ pair_place, int top, int width,
                                    float* __restrict__ resid) {
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const float scale = 1.0f / (float)top;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const int place = pair_place[t * top + k];
      if (place >= 0) sum += to_float(rows[(size_t)place * row_stride + i]);
    }
    resid[(size_t)t * width + i] += sum * scale;
  }
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

// The two-kernel form for small steps; act: float32 [tokens * top * ff].
VX_API int vx_table_experts_rows(const void* h, int dtype, long long h_stride, const int* ids, const int* fed,
                                 int num_fed, const int* table, int vocab, int top, int experts, const void* w_up,
                                 const void* w_down, int width, int ff, float* act, float* resid, int num_tokens,
                                 int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const size_t smem_up = sizeof(float) * (size_t)width, smem_down = sizeof(float) * (size_t)top * ff;
  if (smem_up > 48 * 1024 || smem_down > 48 * 1024) return (int)cudaErrorInvalidValue;
  // Eight warps a block: four rows a warp of the first product, two of the second (whose rows are
  // `top` dot products each), so that both grids have several blocks for every SM.
  const int rows_up = 32, rows_down = 16;
  const dim3 grid_up((ff + rows_up - 1) / rows_up, num_tokens * top);
  const dim3 grid_down((width + rows_down - 1) / rows_down, num_tokens);
  if (dtype == VX_DTYPE_F32) {
    launch_pdl(expert_up_rows_kernel<float>, grid_up, dim3(256), smem_up, stream, (const float*)h, h_stride, ids, fed,
               num_fed, table, vocab, top, experts, (const float*)w_up, width, ff, rows_up, act, status);
    launch_pdl(expert_down_rows_kernel<float>, grid_down, dim3(256), smem_down, stream, (const float*)act, ids, fed,
               num_fed, table, vocab, top, experts, (const float*)w_down, width, ff, rows_down, resid);
  } else {
    launch_pdl(expert_up_rows_kernel<__nv_bfloat16>, grid_up, dim3(256), smem_up, stream, (const __nv_bfloat16*)h,
               h_stride, ids, fed, num_fed, table, vocab, top, experts, (const __nv_bfloat16*)w_up, width, ff, rows_up,
               act, status);
    launch_pdl(expert_down_rows_kernel<__nv_bfloat16>, grid_down, dim3(256), smem_down, stream, (const float*)act, ids,
               fed, num_fed, table, vocab, top, experts, (const __nv_bfloat16*)w_down, width, ff, rows_down, resid);
  }
  return (int)cudaGetLastError();
}

VX_API int vx_grouped_tile_rows() { return GG_M; }

// The grouped tensor-core form for long bfloat16 steps.  capacity: places (a multiple of the
// tile height, at least tokens * top + experts * (tile height - 1)); route: int32 scratch of
// capacity / tile + capacity + tokens * top entries; act: bfloat16 [capacity, act_stride];
// rows: float32 [capacity, width].
VX_API int vx_table_experts_grouped(const void* h, long long h_stride, const int* ids, const int* fed, int num_fed,
                                    const int* table, int vocab, int top, int experts, const void* w_up,
                                    const void* w_down, int width, int ff, int* route, int capacity, void* act,
                                    long long act_stride, float* rows, float* resid, int num_tokens, int* status,
                                    cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (capacity % GG_M != 0 || capacity < num_tokens * top + experts * (GG_M - 1)) return (int)cudaErrorInvalidValue;
  if ((width & 7) != 0 || (ff & 7) != 0 || (h_stride & 7) != 0 || (act_stride & 7) != 0)
    return (int)cudaErrorInvalidValue;
  const int max_tiles = capacity / GG_M;
  int* tile_expert = route;
  int* place_token = route + max_tiles;
  int* pair_place = place_token + capacity;
  const size_t smem = sizeof(int) * 3 * (size_t)experts;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  launch_pdl(route_pairs_kernel, dim3(1), dim3(1024), smem, stream, ids, fed, num_fed, table, vocab, top, experts,
             num_tokens, capacity, max_tiles, tile_expert, place_token, pair_place, status, (int*)nullptr);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)GG_SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(grouped_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)GG_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  launch_pdl(grouped_gemm_kernel<true>, dim3(max_tiles, (ff + GG_N - 1) / GG_N), dim3(128), GG_SMEM_BYTES, stream,
             (const __nv_bfloat16*)h, h_stride, (const int*)place_token, (const int*)tile_expert,
             (const __nv_bfloat16*)w_up, ff, width, (__nv_bfloat16*)act, (float*)nullptr, act_stride);
  launch_pdl(grouped_gemm_kernel<false>, dim3(max_tiles, (width + GG_N - 1) / GG_N), dim3(128), GG_SMEM_BYTES, stream,
             (const __nv_bfloat16*)act, act_stride, (const int*)place_token, (const int*)tile_expert,
             (const __nv_bfloat16*)w_down, width, ff, (__nv_bfloat16*)nullptr, rows, (long long)width);
  launch_pdl(gather_pairs_kernel<float>, dim3(num_tokens), dim3(256), 0, stream, (const float*)rows, (long long)width,
             (const int*)pair_place, top, width, resid);
  return (int)cudaGetLastError();
}

// The same for bfloat16 rows of whole 16-byte chunks: eight values a thread.
__global__ void gather_pairs_vec_kernel(const __nv_bfloat16* __restrict__ rows, long long row_stride,
                                        const int* __restrict__ pair_place, int top, int width,
                                        float* __restrict__ resid) {
  allow_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const float scale = 1.0f / (float)top;
  for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top; ++k) {
      const int place = pair_place[t * top + k];
      if (place < 0) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(rows + (size_t)place * row_stride + i);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(pairs[q]);
        sum[2 * q] += f.x;
        sum[2 * q + 1] += f.y;
      }
    }
    float4* out = reinterpret_cast<float4*>(resid + (size_t)t * width + i);
    float4 a = out[0], b = out[1];
    a.x += sum[0] * scale; a.y += sum[1] * scale; a.z += sum[2] * scale; a.w += sum[3] * scale;
    b.x += sum[4] * scale; b.y += sum[5] * scale; b.z += sum[6] * scale; b.w += sum[7] * scale;
    out[0] = a;
    out[1] = b;
  }
}

// The routing alone, for a caller that runs the two products as a library's grouped product: the
// places as above, run_ends [experts] (where each expert's padded run ends), and the rows of h
// gathered by place into a_rows [capacity, width] (bfloat16).
VX_API int vx_route_and_gather(const void* h, long long h_stride, const int* ids, const int* fed, int num_fed,
                               const int* table, int vocab, int top, int experts, int width, int* route,
                               int capacity, int* run_ends, void* a_rows, int num_tokens, int* status,
                               cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (capacity % GG_M != 0 || capacity < num_tokens * top + experts * (GG_M - 1)) return (int)cudaErrorInvalidValue;
  if ((width & 7) != 0 || (h_stride & 7) != 0) return (int)cudaErrorInvalidValue;
  const int max_tiles = capacity / GG_M;
  int* tile_expert = route;
  int* place_token = route + max_tiles;
  int* pair_place = place_token + capacity;
  const size_t smem = sizeof(int) * 3 * (size_t)experts;
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  launch_pdl(route_pairs_kernel, dim3(1), dim3(1024), smem, stream, ids, fed, num_fed, table, vocab, top, experts,
             num_tokens, capacity, max_tiles, tile_expert, place_token, pair_place, status, run_ends);
  const long long total = (long long)capacity * (width / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_pdl(gather_rows_kernel, dim3((int)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)h, h_stride,
             (const int*)place_token, width / 8, total, (__nv_bfloat16*)a_rows);
  return (int)cudaGetLastError();
}

// resid[t] += (sum over the token's pairs, in their order, of rows[place of the pair]) / top;
// rows bfloat16 [capacity, width]; route as written by vx_route_and_gather.
VX_API int vx_gather_pairs(const void* rows, const int* route, int capacity, int top, int width, float* resid,
                           int num_tokens, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int* pair_place = route + capacity / GG_M + capacity;
  if ((width & 7) == 0 && (reinterpret_cast<uintptr_t>(rows) & 15) == 0 && (reinterpret_cast<uintptr_t>(resid) & 15) == 0) {
    const int threads = width / 8 >= 256 ? 256 : (width / 8 + 31) / 32 * 32;
    launch_pdl(gather_pairs_vec_kernel, dim3(num_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)rows,
               (long long)width, pair_place, top, width, resid);
    return (int)cudaGetLastError();
  }
  launch_pdl(gather_pairs_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(256), 0, stream, (const __nv_bfloat16*)rows,
             (long long)width, pair_place, top, width, resid);
  return (int)cudaGetLastError();
}
